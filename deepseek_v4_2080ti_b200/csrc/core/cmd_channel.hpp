// Rank 0 -> worker ranks command fan-out over a unix-domain socket (int32 words), so workers
// block on a socket instead of a device collective while idle.  Rank 0 listens on
// "<base_path>.cmdsock"; each worker connects (retrying while rank 0 starts up) and introduces
// itself with its rank.  (Role of cpp_engine/include/cmd_channel.hpp:17-40, core/cmd_channel.cpp.)
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace pocket {

class CmdChannel {
 public:
  CmdChannel() = default;
  ~CmdChannel();
  CmdChannel(const CmdChannel&) = delete;
  CmdChannel& operator=(const CmdChannel&) = delete;

  // Rank 0: bind + listen, then accept world-1 workers (timeout_ms total). Workers: connect with retries.
  bool open(const std::string& base_path, int rank, int world, int timeout_ms = 600000, int retry_ms = 50);
  void close();
  bool is_open() const { return open_; }
  int world() const { return world_; }
  int rank() const { return rank_; }

  // Rank 0: one message = [n_words, words...] sent to every worker. False if any peer is gone.
  bool broadcast(const std::vector<int32_t>& words);
  // Worker: blocking receive of one message. False on EOF / error / timeout (timeout_ms < 0: wait forever).
  bool receive(std::vector<int32_t>& words, int timeout_ms = -1);

 private:
  bool open_ = false;
  int rank_ = 0, world_ = 1;
  int listen_fd_ = -1;
  std::vector<int> peers_;   // rank 0: one fd per worker (index rank-1); worker: single fd at [0]
  std::string path_;
};

}  // namespace pocket
