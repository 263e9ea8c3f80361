#include "cmd_channel.hpp"

#include <cerrno>
#include <chrono>
#include <cstring>
#include <thread>

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

namespace pocket {
namespace {

bool write_all(int fd, const void* buf, size_t n) {
  const char* p = static_cast<const char*>(buf);
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) { if (errno == EINTR) continue; return false; }
    p += w;
    n -= static_cast<size_t>(w);
  }
  return true;
}

bool read_all(int fd, void* buf, size_t n, int timeout_ms) {
  char* p = static_cast<char*>(buf);
  while (n) {
    if (timeout_ms >= 0) {
      pollfd pf{fd, POLLIN, 0};
      int r = ::poll(&pf, 1, timeout_ms);
      if (r == 0) return false;
      if (r < 0) { if (errno == EINTR) continue; return false; }
    }
    ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) return false;
    if (r < 0) { if (errno == EINTR) continue; return false; }
    p += r;
    n -= static_cast<size_t>(r);
  }
  return true;
}

bool fill_addr(sockaddr_un& a, const std::string& path) {
  std::memset(&a, 0, sizeof a);
  a.sun_family = AF_UNIX;
  if (path.size() >= sizeof a.sun_path) return false;
  std::memcpy(a.sun_path, path.c_str(), path.size() + 1);
  return true;
}

}  // namespace

CmdChannel::~CmdChannel() { close(); }

void CmdChannel::close() {
  for (int fd : peers_) if (fd >= 0) ::close(fd);
  peers_.clear();
  if (listen_fd_ >= 0) { ::close(listen_fd_); listen_fd_ = -1; if (!path_.empty()) ::unlink(path_.c_str()); }
  open_ = false;
}

bool CmdChannel::open(const std::string& base_path, int rank, int world, int timeout_ms, int retry_ms) {
  close();
  rank_ = rank;
  world_ = world;
  if (world <= 1) { open_ = true; return true; }
  path_ = base_path + ".cmdsock";
  sockaddr_un addr;
  if (!fill_addr(addr, path_)) return false;
  using clock = std::chrono::steady_clock;
  const auto deadline = clock::now() + std::chrono::milliseconds(timeout_ms);
  if (rank == 0) {
    ::unlink(path_.c_str());
    listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
    if (listen_fd_ < 0) return false;
    if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), sizeof addr) != 0 || ::listen(listen_fd_, world) != 0) { close(); return false; }
    peers_.assign(world - 1, -1);
    int connected = 0;
    while (connected < world - 1) {
      const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - clock::now()).count();
      if (left <= 0) { close(); return false; }
      pollfd pf{listen_fd_, POLLIN, 0};
      int r = ::poll(&pf, 1, static_cast<int>(std::min<long long>(left, 1000)));
      if (r <= 0) continue;
      int fd = ::accept(listen_fd_, nullptr, nullptr);
      if (fd < 0) continue;
      int32_t who = -1;
      if (!read_all(fd, &who, sizeof who, 5000) || who < 1 || who >= world || peers_[who - 1] >= 0) { ::close(fd); continue; }
      peers_[who - 1] = fd;
      ++connected;
    }
  } else {
    int fd = -1;
    for (;;) {
      fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
      if (fd < 0) return false;
      if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof addr) == 0) break;
      ::close(fd);
      fd = -1;
      if (clock::now() >= deadline) return false;
      std::this_thread::sleep_for(std::chrono::milliseconds(retry_ms));
    }
    int32_t who = rank;
    if (!write_all(fd, &who, sizeof who)) { ::close(fd); return false; }
    peers_.assign(1, fd);
    path_.clear();   // only rank 0 owns (and unlinks) the socket path
  }
  open_ = true;
  return true;
}

bool CmdChannel::broadcast(const std::vector<int32_t>& words) {
  if (!open_ || rank_ != 0) return false;
  if (world_ <= 1) return true;
  std::vector<int32_t> msg;
  msg.reserve(words.size() + 1);
  msg.push_back(static_cast<int32_t>(words.size()));
  msg.insert(msg.end(), words.begin(), words.end());
  bool ok = true;
  for (int fd : peers_) ok = write_all(fd, msg.data(), msg.size() * sizeof(int32_t)) && ok;
  return ok;
}

bool CmdChannel::receive(std::vector<int32_t>& words, int timeout_ms) {
  if (!open_ || rank_ == 0 || peers_.empty()) return false;
  int32_t n = 0;
  if (!read_all(peers_[0], &n, sizeof n, timeout_ms)) return false;
  if (n < 0 || n > (1 << 26)) return false;
  words.resize(static_cast<size_t>(n));
  return n == 0 || read_all(peers_[0], words.data(), words.size() * sizeof(int32_t), timeout_ms < 0 ? -1 : timeout_ms);
}

}  // namespace pocket
