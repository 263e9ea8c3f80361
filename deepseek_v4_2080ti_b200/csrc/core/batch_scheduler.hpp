// Continuous-batching scheduler: one background thread runs
//   admit (worst-case KV-block reservation, FIFO with head-of-line blocking)
//   -> prefill batch (bounded by a token budget, chunked)
//   -> decode batch (every running sequence advances one token)
//   -> completions / cancellations.
// (Role of cpp_engine/include/batch_scheduler.hpp:75-193 and engine/batch_scheduler.cpp:169-518.)
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstdint>
#include <deque>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "inference_engine.hpp"

namespace pocket {

struct SchedulerOptions {
  int max_batch = 32;                 // sequences decoding together
  int prefill_token_budget = 8192;    // prompt tokens processed per scheduling round
  int prefill_chunk_tokens = 8192;    // largest single prefill call per sequence
  bool decode_first = true;           // run the decode batch before admitting more prefill work
};

struct SchedulerRequest {
  uint64_t id = 0;
  std::vector<int32_t> prompt;
  int max_new_tokens = 256;
  bool stop_on_eos = true;
};

struct SchedulerResult {
  uint64_t id = 0;
  std::vector<int32_t> tokens;
  std::string finish_reason;          // stop | length | cancelled | error
  std::string error;
  double queue_seconds = 0, prefill_seconds = 0, decode_seconds = 0;
};

struct SchedulerStats {
  int queued = 0, prefilling = 0, decoding = 0;
  uint64_t completed = 0, cancelled = 0, failed = 0;
  int kv_blocks_total = 0, kv_blocks_reserved = 0;
  uint64_t prefill_tokens = 0, decode_tokens = 0, rounds = 0;
};

class BatchScheduler {
 public:
  BatchScheduler(InferenceEngine& engine, SchedulerOptions options);
  ~BatchScheduler();
  BatchScheduler(const BatchScheduler&) = delete;
  BatchScheduler& operator=(const BatchScheduler&) = delete;

  uint64_t submit(std::vector<int32_t> prompt, int max_new_tokens, bool stop_on_eos = true);  // throws on invalid input
  bool cancel(uint64_t id);
  // Non-blocking: moves a finished result out. Blocking variant waits up to timeout_ms (<0: forever).
  bool poll(uint64_t id, SchedulerResult& out);
  bool wait(uint64_t id, SchedulerResult& out, int timeout_ms = -1);
  SchedulerStats stats() const;
  void stop();                        // drains nothing: running requests finish as "cancelled"
  // Runs one scheduling round on the caller's thread (tests; requires start_thread = false).
  bool step();
  static std::unique_ptr<BatchScheduler> make_manual(InferenceEngine& engine, SchedulerOptions options);

 private:
  struct Seq {
    SchedulerRequest req;
    int slot = -1;
    int64_t prefilled = 0;            // prompt tokens already in the KV cache
    int reserved_blocks = 0;
    std::vector<int32_t> out;
    int32_t last_token = -1;
    bool cancelled = false;
    double t_submit = 0, t_admit = 0, t_first = 0;
  };
  BatchScheduler(InferenceEngine& engine, SchedulerOptions options, bool start_thread);
  void loop();
  bool round();                       // returns false when there was nothing to do
  int worst_case_blocks(const Seq& s) const;
  void admit();
  void run_prefill();
  void run_decode();
  void finish(std::unique_ptr<Seq> s, const char* reason, const std::string& error = "");
  static double now();

  InferenceEngine& eng_;
  SchedulerOptions opt_;
  mutable std::mutex mu_;
  std::condition_variable cv_work_, cv_done_;
  std::deque<std::unique_ptr<Seq>> queue_;
  std::vector<std::unique_ptr<Seq>> prefilling_, decoding_;
  std::map<uint64_t, SchedulerResult> done_;
  std::atomic<bool> stop_{false};
  uint64_t next_id_ = 1;
  int reserved_blocks_ = 0;
  SchedulerStats stats_;
  std::thread thread_;
};

}  // namespace pocket
