// OpenAI-compatible HTTP front end of the native engine: a small blocking HTTP/1.1 server (one thread per connection,
// generation serialised through the batch scheduler), JSON and server-sent-event responses.
//   GET  /health  /v1/models
//   POST /v1/chat/completions   {"messages": [...]} (templated and tokenised by the sidecar) or {"prompt_token_ids": [...]}
//   POST /v1/completions        {"prompt_token_ids": [...]} or {"prompt": "..."} (needs a tokenizer in the sidecar)
// Options: "max_tokens", "stream".  Replies carry "token_ids" always and text when the sidecar can detokenise.
// (Role of cpp_engine/include/openai_server.hpp:12-35, core/openai_server.cpp:1-466; the reference uses httplib.)
#pragma once
#include <atomic>
#include <condition_variable>
#include <mutex>
#include <set>
#include <memory>
#include <string>
#include <thread>
#include <vector>

#include "batch_scheduler.hpp"
#include "python_sidecar.hpp"

namespace pocket {

struct OpenAIServerOptions {
  std::string host = "127.0.0.1";
  int port = 8000;                       // 0 = pick a free port (see port())
  std::string model_name = "pocketllm";
  std::string chat_family = "deepseek_v4";
  int default_max_tokens = 256;
  std::vector<std::string> sidecar_argv; // empty = no sidecar: only token-id requests are accepted
};

class OpenAIServer {
 public:
  OpenAIServer(InferenceEngine& engine, OpenAIServerOptions opt, SchedulerOptions sched = SchedulerOptions());
  ~OpenAIServer();
  void start();                          // binds, listens, serves on a background thread
  void stop();
  int port() const { return port_; }
  uint64_t requests_served() const { return served_.load(); }

  // Exposed for tests: handle one parsed request, returns (status, content type, body).
  struct Reply { int status; std::string content_type; std::string body; };
  Reply handle(const std::string& method, const std::string& path, const std::string& body);

 private:
  void accept_loop();
  void serve_connection(int fd);
  Reply completion(const Json& body, bool chat, int fd_for_stream);
  InferenceEngine& eng_;
  OpenAIServerOptions opt_;
  std::unique_ptr<BatchScheduler> sched_;
  std::unique_ptr<PythonSidecar> sidecar_;
  int listen_fd_ = -1, port_ = 0;
  std::atomic<bool> stop_{false};
  std::atomic<uint64_t> served_{0}, next_id_{1};
  std::thread thread_;
  // connection threads run detached but are counted: stop() closes their sockets, wakes the requests that wait on
  // the scheduler and leaves only when the last of them has returned, so none can touch a destroyed server
  std::mutex conn_mu_;
  std::condition_variable conn_cv_;
  std::set<int> conn_fds_;
  int live_connections_ = 0;
};

}  // namespace pocket
