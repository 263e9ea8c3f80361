// Host-only self-test of the C++ runtime core, meant to be built with -fsanitize=address,undefined or
// -fsanitize=thread (build.py build_selftest): block pool / table invariants (prefix sharing and adoption), the batch
// scheduler driven by several submitting threads against a deterministic fake engine (with cancellation and KV
// exhaustion), the command channel between threads, the JSON parser on hostile input, the host sampler, the HTTP server
// under hostile and concurrent requests over the loopback, and the GGUF / safetensors readers and the model
// configuration on damaged files.  Exit code 0 = every check held.
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
#include "../core/gguf_reader.hpp"
#include "../core/json_lite.hpp"
#include "../core/model_config.hpp"
#include "../core/openai_server.hpp"
#include "../core/safetensors_reader.hpp"
#include "../core/sampler.hpp"
#include "../core/tokenizer.hpp"

#include <arpa/inet.h>
#include <cstring>
#include <fstream>
#include <netinet/in.h>
#include <sys/socket.h>

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

// ---- block adoption: blocks held by a cache enter an empty row, every holder gives its reference back
static void test_adopt() {
  BlockPool pool(9, 4);                                      // 8 usable blocks of 4 tokens
  BlockTable table(pool, 3, 8);
  CHECK(table.ensure_capacity(0, 10));                       // 3 blocks
  int32_t held[2] = {table.block_at(0, 0), table.block_at(0, 1)};
  for (int32_t b : held) pool.retain(b);                     // the cache's own references
  CHECK(pool.free_blocks() == 5);
  CHECK(table.adopt(1, held, 2) && table.blocks_in(1) == 2 && table.block_at(1, 1) == held[1]);
  CHECK(pool.refcount(held[0]) == 3);
  CHECK(!table.adopt(1, held, 2));                           // the row is no longer empty
  CHECK(!table.adopt(2, held, 9));                           // more blocks than a row holds
  int32_t mixed[2] = {held[0], 1000};
  CHECK(!table.adopt(2, mixed, 2) && table.blocks_in(2) == 0 && pool.refcount(held[0]) == 3);   // nothing kept of a bad list
  CHECK(table.ensure_capacity(1, 12) && table.blocks_in(1) == 3 && pool.free_blocks() == 4);
  table.free_slot(0);
  table.free_slot(1);
  CHECK(pool.free_blocks() == 6 && pool.refcount(held[1]) == 1);          // the cache still holds its two blocks
  for (int32_t b : held) pool.release(b);
  CHECK(pool.free_blocks() == 8);
  int32_t stale[1] = {held[0]};
  CHECK(!table.adopt(2, stale, 1));                          // a block that went back to the pool cannot be adopted
}

// ---- hostile HTTP: the same request bytes a socket would deliver, against a live server on the loopback
static std::string http_exchange(int port, const std::string& raw) {
  const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons(uint16_t(port));
  a.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  std::string out;
  if (::connect(fd, reinterpret_cast<sockaddr*>(&a), sizeof a) == 0) {
    size_t off = 0;
    while (off < raw.size()) {
      const ssize_t n = ::send(fd, raw.data() + off, raw.size() - off, MSG_NOSIGNAL);
      if (n <= 0) break;
      off += size_t(n);
    }
    ::shutdown(fd, SHUT_WR);
    timeval tv{3, 0};
    ::setsockopt(fd, SOL_SOCKET, SO_RCVTIMEO, &tv, sizeof tv);
    char buf[4096];
    for (;;) {
      const ssize_t n = ::recv(fd, buf, sizeof buf, 0);
      if (n <= 0) break;
      out.append(buf, size_t(n));
    }
  }
  ::close(fd);
  return out;
}

static int status_of(const std::string& reply) { return reply.rfind("HTTP/1.1 ", 0) == 0 ? std::atoi(reply.c_str() + 9) : 0; }

class VocabEngine : public FakeEngine {
 public:
  using FakeEngine::FakeEngine;
  int64_t vocab_size() const override { return 97; }
};

static void test_http_server() {
  VocabEngine eng(4, 64, 16);
  OpenAIServerOptions opt;
  opt.port = 0;
  OpenAIServer srv(eng, opt);
  srv.start();
  const int port = srv.port();
  CHECK(port > 0);
  auto post = [](const std::string& body, const std::string& len = "") {
    return "POST /v1/completions HTTP/1.1\r\nContent-Type: application/json\r\nContent-Length: " +
           (len.empty() ? std::to_string(body.size()) : len) + "\r\n\r\n" + body;
  };
  const std::string good = post(R"({"prompt_token_ids": [1, 2, 3], "max_tokens": 3})");
  CHECK(status_of(http_exchange(port, good)) == 200);
  for (const char* len : {"-5", "abc", "12x"}) CHECK(status_of(http_exchange(port, post("{}", len))) == 400);
  CHECK(status_of(http_exchange(port, post("{}", "99999999999999999999"))) == 413);
  CHECK(status_of(http_exchange(port, "GET /health HTTP/1.1\r\nX: " + std::string(2000000, 'a') + "\r\n\r\n")) == 413);
  CHECK(http_exchange(port, post("{}", "100000")).empty());               // the announced body never arrives
  for (const char* ids : {"[1.5]", "[-3]", "[1e30]", "[\"7\"]", "[null]", "[97]", "[2147483648]", "\"12\"", "{}"})
    CHECK(status_of(http_exchange(port, post(std::string("{\"prompt_token_ids\": ") + ids + ", \"max_tokens\": 2}"))) == 400);
  for (const char* body : {"{{{{", "{\"prompt_token_ids\": [1], \"max_tokens\": 1e18}", "{\"prompt_token_ids\": [1], \"max_tokens\": \"y\"}"})
    CHECK(status_of(http_exchange(port, post(body))) == 400);
  CHECK(status_of(http_exchange(port, post(std::string(100001, '[') + std::string(100001, ']')))) == 400);
  std::mt19937 rng(5);
  for (int i = 0; i < 150; ++i) {                                          // random byte damage to a valid request
    std::string b = good;
    for (int k = 0, n = 1 + int(rng() % 7); k < n; ++k) b[rng() % b.size()] = char(rng() & 0xFF);
    (void)http_exchange(port, b);
  }
  std::vector<std::thread> clients;                                        // concurrent clients while damage continues
  std::atomic<int> ok{0};
  for (int t = 0; t < 6; ++t)
    clients.emplace_back([&] { for (int i = 0; i < 5; ++i) ok += status_of(http_exchange(port, good)) == 200; });
  for (auto& t : clients) t.join();
  CHECK(ok.load() == 30);
  srv.stop();
}

// ---- damaged model files: the readers throw, they do not read outside the mapping
static std::string write_tmp(const std::string& name, const std::string& bytes) {
  const std::string path = std::string("/tmp/core_selftest_") + std::to_string(::getpid()) + "_" + name;
  std::ofstream f(path, std::ios::binary);
  f.write(bytes.data(), std::streamsize(bytes.size()));
  return path;
}

template <class T> static void put(std::string& s, T v) { s.append(reinterpret_cast<const char*>(&v), sizeof v); }
static void put_str(std::string& s, const std::string& v) { put<uint64_t>(s, v.size()); s += v; }

static void test_file_readers() {
  // a small GGUF v3: two metadata entries, one F32 tensor of 8 values
  std::string g;
  put<uint32_t>(g, 0x46554747u); put<uint32_t>(g, 3); put<uint64_t>(g, 1); put<uint64_t>(g, 2);
  put_str(g, "general.architecture"); put<uint32_t>(g, 8); put_str(g, "glm-dsa");
  put_str(g, "glm-dsa.block_count"); put<uint32_t>(g, 4); put<uint32_t>(g, 2);
  put_str(g, "t.weight"); put<uint32_t>(g, 1); put<uint64_t>(g, 8); put<uint32_t>(g, 0); put<uint64_t>(g, 0);
  while (g.size() % 32) g.push_back('\0');
  for (int i = 0; i < 8; ++i) put<float>(g, float(i));
  {
    const std::string p = write_tmp("ok.gguf", g);
    GGUFReader r(p);
    CHECK(r.get_string("general.architecture") == "glm-dsa" && r.tensors().size() == 1);
    const GGUFTensorInfo* t = r.tensor("t.weight");
    CHECK(t != nullptr && reinterpret_cast<const float*>(r.tensor_data(*t))[7] == 7.0f);
    ::unlink(p.c_str());
  }
  // safetensors: header + 16 bytes
  const std::string hdr = R"({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}})";
  std::string st;
  put<uint64_t>(st, hdr.size());
  st += hdr;
  st.append(16, '\1');
  {
    const std::string p = write_tmp("ok.safetensors", st);
    SafetensorsFile f(p);
    CHECK(f.tensors().size() == 1 && f.find("a") != nullptr && f.find("a")->nbytes() == 16);
    ::unlink(p.c_str());
  }
  std::mt19937 rng(11);
  int threw = 0, read_ok = 0;
  for (int i = 0; i < 400; ++i) {
    const bool gguf = i & 1;
    std::string b = gguf ? g : st;
    switch (rng() % 4) {
      case 0: b.resize(rng() % b.size()); break;
      case 1: for (int k = 0, n = 1 + int(rng() % 5); k < n; ++k) b[rng() % b.size()] ^= char(1u << (rng() % 8)); break;
      case 2: { const uint64_t big[] = {1ull << 63, ~0ull, 1ull << 40, (1ull << 32) + 5}; const uint64_t v = big[rng() % 4];
                std::memcpy(&b[rng() % (b.size() - 8)], &v, 8); break; }
      default: std::memset(&b[rng() % (b.size() - 8)], 0, 8); break;
    }
    const std::string p = write_tmp(gguf ? "bad.gguf" : "bad.safetensors", b);
    try {
      if (gguf) {
        GGUFReader r(p);
        for (const auto& t : r.tensors()) { const uint8_t* d = r.tensor_data(t); volatile uint8_t x = d[0]; (void)x; }
        try { (void)MoeModelConfig::from_gguf(r).problems(8, 8); } catch (const std::exception&) {}
      } else {
        SafetensorsFile f(p);
        for (const auto& t : f.tensors()) if (t.nbytes()) { volatile uint8_t x = f.data(t)[t.nbytes() - 1]; (void)x; }
      }
      ++read_ok;
    } catch (const std::exception&) {
      ++threw;
    }
    ::unlink(p.c_str());
  }
  CHECK(threw > 50 && read_ok > 20);
  // model configuration from hostile JSON: wrong types and absurd values produce problems or exceptions, not crashes
  for (const char* js : {R"({"model_type": "deepseek_v4", "dim": "x"})", R"({"n_routed_experts": -4, "n_layers": 1e30})",
                         R"({"dim": 0, "n_heads": 0, "n_routed_experts": 0})", R"([1, 2])", R"({})"}) {
    try { (void)MoeModelConfig::from_hf_json(Json::parse(js)).problems(8, 8); } catch (const std::exception&) {}
  }
}

// ---- tokenizer: arbitrary bytes in, arbitrary ids back; merges that name unknown pieces are ignored
static void test_tokenizer() {
  std::vector<std::string> toks;
  for (int c = 33; c < 127; ++c) toks.emplace_back(1, char(c));
  toks.insert(toks.end(), {"\xC4\xA0", "hi", "th", "the", "<eos>"});
  const std::vector<std::string> merges = {"h i", "t h", "th e", "zz qq", "", "a", "a b c"};
  const Tokenizer t = Tokenizer::from_vocab(toks, merges, -1, int32_t(toks.size()) - 1);
  CHECK(t.find("the") >= 0 && t.find("nope") == -1);
  const std::vector<int32_t> ids = t.encode_basic("hi the");
  CHECK(!ids.empty() && t.decode(ids).find("hi") != std::string::npos);
  std::mt19937 rng(3);
  for (int i = 0; i < 300; ++i) {
    std::string text(rng() % 64, '\0');
    for (char& c : text) c = char(rng() & 0xFF);
    const std::vector<int32_t> e = t.encode_basic(text, i & 1);
    for (int32_t id : e) CHECK(id >= 0 && id < int32_t(toks.size()));
    (void)t.decode(e);
    std::vector<int32_t> wild(rng() % 16);
    for (int32_t& id : wild) id = int32_t(rng());
    (void)t.decode(wild);                                    // ids outside the vocabulary decode to nothing
  }
}

int main() {
  test_tokenizer();
  test_blocks();
  test_scheduler();
  test_cmd_channel();
  test_json_and_sampler();
  test_adopt();
  test_http_server();
  test_file_readers();
  if (g_fail) { std::fprintf(stderr, "%d check(s) failed\n", g_fail); return 1; }
  std::puts("CORE_SELFTEST_OK");
  return 0;
}
