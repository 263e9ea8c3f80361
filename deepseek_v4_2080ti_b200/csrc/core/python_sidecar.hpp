// Child process speaking JSON lines over pipes: the native server delegates chat templating, tokenisation and
// completion parsing to `python -m pocketllm.sidecar`.  One request at a time (guarded by a mutex); a reply that does
// not arrive within the timeout, or a dead child, is reported as an error and the child is restarted on the next call.
// (Role of cpp_engine/include/python_sidecar.hpp:38-62, core/python_sidecar.cpp.)
#pragma once
#include <mutex>
#include <string>
#include <vector>

#include "json_lite.hpp"

namespace pocket {

class PythonSidecar {
 public:
  // argv of the child, e.g. {"python", "-m", "pocketllm.sidecar", "--gguf", path}.
  explicit PythonSidecar(std::vector<std::string> argv, int timeout_ms = 30000);
  ~PythonSidecar();
  PythonSidecar(const PythonSidecar&) = delete;
  PythonSidecar& operator=(const PythonSidecar&) = delete;

  // Sends one request object, returns the reply object.  Throws std::runtime_error on timeout / dead child / bad JSON.
  Json call(const Json& request);
  bool ping();
  void shutdown();
  bool running() const { return pid_ > 0; }

 private:
  void start();
  void stop(bool graceful);
  std::vector<std::string> argv_;
  int timeout_ms_;
  int pid_ = -1, in_fd_ = -1, out_fd_ = -1;   // we write to in_fd_, read from out_fd_
  std::string pending_;
  std::mutex mu_;
};

}  // namespace pocket
