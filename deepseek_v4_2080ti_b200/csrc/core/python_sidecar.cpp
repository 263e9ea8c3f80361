#include "python_sidecar.hpp"

#include <cerrno>
#include <csignal>
#include <cstring>
#include <poll.h>
#include <stdexcept>
#include <sys/wait.h>
#include <unistd.h>

namespace pocket {

PythonSidecar::PythonSidecar(std::vector<std::string> argv, int timeout_ms) : argv_(std::move(argv)), timeout_ms_(timeout_ms) {
  if (argv_.empty()) throw std::runtime_error("sidecar: empty command");
}

PythonSidecar::~PythonSidecar() { stop(true); }

void PythonSidecar::start() {
  int to_child[2], from_child[2];
  if (pipe(to_child) != 0 || pipe(from_child) != 0) throw std::runtime_error(std::string("sidecar: pipe: ") + strerror(errno));
  const pid_t pid = fork();
  if (pid < 0) throw std::runtime_error(std::string("sidecar: fork: ") + strerror(errno));
  if (pid == 0) {
    dup2(to_child[0], STDIN_FILENO);
    dup2(from_child[1], STDOUT_FILENO);
    close(to_child[0]); close(to_child[1]); close(from_child[0]); close(from_child[1]);
    std::vector<char*> args;
    for (auto& a : argv_) args.push_back(const_cast<char*>(a.c_str()));
    args.push_back(nullptr);
    execvp(args[0], args.data());
    _exit(127);
  }
  close(to_child[0]);
  close(from_child[1]);
  pid_ = pid;
  in_fd_ = to_child[1];
  out_fd_ = from_child[0];
  pending_.clear();
}

void PythonSidecar::stop(bool graceful) {
  if (pid_ <= 0) return;
  if (graceful && in_fd_ >= 0) {
    const char* bye = "{\"op\": \"shutdown\"}\n";
    (void)!write(in_fd_, bye, strlen(bye));
  }
  if (in_fd_ >= 0) close(in_fd_);
  if (out_fd_ >= 0) close(out_fd_);
  in_fd_ = out_fd_ = -1;
  int status = 0;
  for (int i = 0; i < 50; ++i) {                 // up to ~1 s for a clean exit, then terminate
    if (waitpid(pid_, &status, WNOHANG) == pid_) { pid_ = -1; return; }
    usleep(20000);
  }
  kill(pid_, SIGTERM);
  waitpid(pid_, &status, 0);
  pid_ = -1;
}

Json PythonSidecar::call(const Json& request) {
  std::lock_guard<std::mutex> lk(mu_);
  if (pid_ <= 0) start();
  const std::string line = request.dump() + "\n";
  size_t off = 0;
  while (off < line.size()) {
    const ssize_t n = write(in_fd_, line.data() + off, line.size() - off);
    if (n <= 0) {
      if (errno == EINTR) continue;
      stop(false);
      throw std::runtime_error("sidecar: the helper process is gone");
    }
    off += size_t(n);
  }
  int waited = 0;
  for (;;) {
    const size_t nl = pending_.find('\n');
    if (nl != std::string::npos) {
      const std::string reply = pending_.substr(0, nl);
      pending_.erase(0, nl + 1);
      return Json::parse(reply);
    }
    pollfd pfd{out_fd_, POLLIN, 0};
    const int rc = poll(&pfd, 1, 100);
    if (rc < 0 && errno != EINTR) { stop(false); throw std::runtime_error("sidecar: poll failed"); }
    if (rc == 0) {
      waited += 100;
      if (waited >= timeout_ms_) { stop(false); throw std::runtime_error("sidecar: no reply within the timeout"); }
      continue;
    }
    char buf[65536];
    const ssize_t n = read(out_fd_, buf, sizeof buf);
    if (n <= 0) { stop(false); throw std::runtime_error("sidecar: the helper process closed its output"); }
    pending_.append(buf, size_t(n));
  }
}

bool PythonSidecar::ping() {
  try {
    Json r = Json::object();
    r.set("op", "ping");
    return call(r)["ok"].as_bool(false);
  } catch (const std::exception&) {
    return false;
  }
}

void PythonSidecar::shutdown() {
  std::lock_guard<std::mutex> lk(mu_);
  stop(true);
}

}  // namespace pocket
