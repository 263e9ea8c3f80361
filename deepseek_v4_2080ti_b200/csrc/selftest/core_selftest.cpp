// Host-only self-test of the C++ runtime core, meant to be built with -fsanitize=address,undefined or
// -fsanitize=thread (build.py build_selftest): block pool / table invariants, the batch scheduler driven by several
// submitting threads against a deterministic fake engine (with cancellation and KV exhaustion), the command channel
// between threads, the JSON parser on hostile input, the host sampler.  Exit code 0 = every check held.
// (The reference ships no sanitizer builds; its counterparts are the plain unit executables under cpp_engine/tests.)
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <string>
#include <thread>
#include <unistd.h>
#include <vector>

#include "../core/batch_scheduler.hpp"
#include "../core/block_pool.hpp"
#include "../core/block_table.hpp"
#include "../core/cmd_channel.hpp"
#include "../core/json_lite.hpp"
#include "../core/sampler.hpp"

using namespace pocket;

static int g_fail = 0;
#define CHECK(cond)                                                              \
  do {                                                                           \
    if (!(cond)) { std::fprintf(stderr, "CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #cond); ++g_fail; } \
  } while (0)

// next token = (sum of the slot's tokens + position) % 97; EOS = 96.
class FakeEngine : public InferenceEngine {
 public:
  FakeEngine(int slots, int blocks, int block_tokens) : pool_(blocks + 1, block_tokens), table_(pool_, slots, 64), sum_(slots, 0), len_(slots, 0), used_(slots, 0) {}
  int max_slots() const override { return int(used_.size()); }
  int block_tokens() const override { return pool_.block_tokens(); }
  int total_blocks() const override { return pool_.total_blocks(); }
  int64_t max_context() const override { return 64LL * pool_.block_tokens(); }
  int allocate_slot() override {
    for (size_t s = 0; s < used_.size(); ++s)
      if (!used_[s]) { used_[s] = 1; sum_[s] = 0; len_[s] = 0; return int(s); }
    return -1;
  }
  void free_slot(int s) override { table_.free_slot(s); used_[s] = 0; }
  bool reserve(int s, int64_t tokens) override { return table_.ensure_capacity(s, tokens); }
  StepResult batch_prefill(const std::vector<PrefillItem>& items) override {
    StepResult r;
    for (const auto& it : items) {
      CHECK(it.position == len_[it.slot]);
      CHECK(reserve(it.slot, it.position + int64_t(it.tokens.size())));
      for (int32_t t : it.tokens) sum_[it.slot] += t;
      len_[it.slot] += int64_t(it.tokens.size());
      r.next_tokens.push_back(it.last_chunk ? next(it.slot) : -1);
    }
    return r;
  }
  StepResult batch_decode(const std::vector<int>& slots, const std::vector<int32_t>& tokens) override {
    StepResult r;
    for (size_t i = 0; i < slots.size(); ++i) {
      CHECK(reserve(slots[i], len_[slots[i]] + 1));
      sum_[slots[i]] += tokens[i];
      len_[slots[i]] += 1;
      r.next_tokens.push_back(next(slots[i]));
    }
    ++decode_calls;
    max_batch = std::max<int>(max_batch, int(slots.size()));
    return r;
  }
  bool is_eos(int32_t t) const override { return t == 96; }
  static std::vector<int32_t> expected(const std::vector<int32_t>& prompt, int max_new) {
    int64_t sum = 0, len = int64_t(prompt.size());
    for (int32_t t : prompt) sum += t;
    std::vector<int32_t> out;
    while (int(out.size()) < max_new) {
      const int32_t t = int32_t((sum + len) % 97);
      out.push_back(t);
      if (t == 96) break;
      sum += t;
      len += 1;
    }
    return out;
  }
  int decode_calls = 0, max_batch = 0;

 private:
  int32_t next(int s) const { return int32_t((sum_[s] + len_[s]) % 97); }
  BlockPool pool_;
  BlockTable table_;
  std::vector<int64_t> sum_, len_;
  std::vector<uint8_t> used_;
};

static void test_blocks() {
  BlockPool pool(9, 16);
  CHECK(pool.total_blocks() == 8 && pool.free_blocks() == 8);
  std::vector<int32_t> a, b;
  CHECK(pool.allocate(5, a) && a.size() == 5);
  CHECK(!pool.allocate(4, b) && b.empty() && pool.free_blocks() == 3);      // all-or-nothing
  for (int32_t x : a) CHECK(x != 0);                                         // block 0 is never handed out
  pool.retain(a[0]);
  pool.release_all(a);
  CHECK(pool.free_blocks() == 7 && pool.refcount(a[0]) == 1);
  pool.release(a[0]);
  CHECK(pool.free_blocks() == 8);
  BlockTable table(pool, 2, 4);
  CHECK(table.ensure_capacity(0, 40) && table.blocks_in(0) == 3);
  CHECK(!table.ensure_capacity(0, 16 * 4 + 1));                              // beyond max_blocks_per_seq
  CHECK(table.share_prefix(1, 0, 2) && table.block_at(1, 1) == table.block_at(0, 1));
  CHECK(table.element_offset(0, 17) == int64_t(table.block_at(0, 1)) * 16 + 1);
  table.free_slot(0);
  CHECK(pool.refcount(table.block_at(1, 0)) == 1);
  table.free_slot(1);
  CHECK(pool.free_blocks() == 8);
}

static void test_scheduler() {
  FakeEngine eng(4, 64, 16);
  SchedulerOptions so;
  so.max_batch = 4;
  so.prefill_token_budget = 48;
  so.prefill_chunk_tokens = 32;
  BatchScheduler sched(eng, so);
  constexpr int kThreads = 4, kPer = 12;
  std::vector<std::vector<std::pair<uint64_t, std::vector<int32_t>>>> submitted(kThreads);
  std::vector<std::thread> ts;
  std::atomic<int> cancelled{0};
  for (int t = 0; t < kThreads; ++t)
    ts.emplace_back([&, t] {
      std::mt19937 rng(100 + t);
      for (int i = 0; i < kPer; ++i) {
        std::vector<int32_t> prompt(1 + rng() % 70);
        for (auto& x : prompt) x = int32_t(rng() % 90);
        const uint64_t id = sched.submit(prompt, 10);
        if (i % 5 == 4 && sched.cancel(id)) { ++cancelled; continue; }
        submitted[t].emplace_back(id, prompt);
      }
    });
  for (auto& t : ts) t.join();
  int done = 0;
  for (auto& per : submitted)
    for (auto& [id, prompt] : per) {
      SchedulerResult r;
      CHECK(sched.wait(id, r, 30000));
      if (r.finish_reason == "cancelled") continue;
      CHECK(r.finish_reason == "stop" || r.finish_reason == "length");
      CHECK(r.tokens == FakeEngine::expected(prompt, 10));
      ++done;
    }
  CHECK(done > 0 && eng.max_batch > 1);                                      // requests really shared decode batches
  const SchedulerStats st = sched.stats();
  CHECK(st.queued == 0 && st.decoding == 0 && st.prefilling == 0 && st.kv_blocks_reserved == 0);
  bool threw = false;
  try { sched.submit({}, 4); } catch (const std::exception&) { threw = true; }
  CHECK(threw);
  sched.stop();
}

static void test_cmd_channel() {
  const std::string base = "/tmp/b200_selftest_" + std::to_string(::getpid());
  constexpr int kWorld = 3;
  std::vector<std::thread> workers;
  std::atomic<int> got{0};
  for (int r = 1; r < kWorld; ++r)
    workers.emplace_back([&, r] {
      CmdChannel ch;
      if (!ch.open(base, r, kWorld, 10000, 10)) return;
      std::vector<int32_t> w;
      while (ch.receive(w, 5000)) {
        if (w.size() == 1 && w[0] == 0) break;
        if (w.size() == 4 && w[0] == 3 && w[3] == w[1] + w[2]) ++got;
      }
    });
  CmdChannel root;
  CHECK(root.open(base, 0, kWorld, 10000, 10));
  for (int i = 0; i < 50; ++i) CHECK(root.broadcast({3, i, 2 * i, 3 * i}));
  CHECK(root.broadcast({0}));
  for (auto& t : workers) t.join();
  CHECK(got == 50 * (kWorld - 1));
  root.close();
}

static void test_json_and_sampler() {
  const Json j = Json::parse(R"({"a": [1, 2.5, "x\né", true, null], "b": {"c": -3}})");
  CHECK(j.is_object());
  for (const char* bad : {"{", "[1,", "{\"a\":}", "\"\\u12", "tru", "[1 2]", "{\"a\":1,}", ""}) {
    bool threw = false;
    try { Json::parse(bad); } catch (const std::exception&) { threw = true; }
    CHECK(threw);
  }
  std::string deep(5000, '[');
  bool threw = false;
  try { Json::parse(deep); } catch (const std::exception&) { threw = true; }
  CHECK(threw);
  std::vector<float> logits = {0.1f, 3.0f, -1.0f, 2.9f};
  CHECK(argmax(logits.data(), 4) == 1);
  std::mt19937_64 rng(7);
  HostSamplingParams p;
  p.temperature = 0.8f;
  p.top_k = 2;
  for (int i = 0; i < 200; ++i) {
    const int32_t t = sample(logits.data(), 4, p, rng);
    CHECK(t == 1 || t == 3);
  }
}

int main() {
  test_blocks();
  test_scheduler();
  test_cmd_channel();
  test_json_and_sampler();
  if (g_fail) { std::fprintf(stderr, "%d check(s) failed\n", g_fail); return 1; }
  std::puts("CORE_SELFTEST_OK");
  return 0;
}
