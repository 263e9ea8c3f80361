// pocketllm_engine: command-line front end of the native engine.
//
//   --ckpt DIR                 checkpoint directory (config.json + *.safetensors)
//   --dump-config              print the parsed model configuration and exit
//   --inspect [--grep S]       list checkpoint tensors (name, dtype, shape, bytes)
//   --inspect-tensor NAME      print one tensor's header and its first values
//   --model-config PATH        describe a sparse-attention MoE checkpoint (PATH = a .gguf file or a directory with
//                              config.json): every field that is set, then the problems of the shape on
//                              --tp-world x --ep-world ranks; needs no --ckpt
//   --qwen-audit [--qwen-audit-strict] [--tp-world N]   check the checkpoint against the weight map (no GPU needed):
//                              missing / unexpected tensors, shapes, dtypes, tensor-parallel divisibility
//   --kv-cache-dtype auto|bf16|fp16   accepted; the 8-bit cache layouts are refused with a pointer to the Python runtime
//   --context-info             bytes of KV cache / recurrent state per token and per slot
//   --smoke-forward            run the prompt, generate --max-new-tokens tokens, print tokens and timings
//   --resident-bench           load once, then time --bench-runs generations of the same prompt
//   --qwen-persistent-stdin    stay resident; each stdin line "<max_new_tokens> tok tok ..." is one request
//   --serve-batch              read every stdin line as a request and run them through the continuous-batching
//                              scheduler together (--max-slots sequences share the decode batch)
//   --serve [--host H --port P] OpenAI-compatible HTTP server (/health, /v1/models, /v1/chat/completions, /v1/completions)
//                              over the continuous-batching scheduler; text prompts go through the Python helper
//                              (--python EXE, --sidecar-gguf FILE for its tokenizer, --chat-family NAME), token-id
//                              requests need no helper
//   --token-ids a,b,c | --token-ids-file F | --tokens N (synthetic ids)   the prompt
//   --max-new-tokens N --max-context C --prefill-chunk-tokens T --smoke-layers L --max-slots S --device D
//   --prefix-cache-interval N [--prefix-cache-entries M]   keep KV blocks + recurrent state every N prompt tokens and
//                              resume later prompts that share the prefix (--qwen-no-prefix-cache: off, the default)
//   --qwen-temperature F --qwen-top-k K --qwen-top-p P --qwen-seed S     host-side sampling (default greedy)
//   --eos a,b                  stop tokens;  --json  machine-readable result line
// (Role of cpp_engine/engine/main.cpp.)
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>

#include <csignal>
#include <unistd.h>

#include "../core/batch_scheduler.hpp"
#include "../core/cmd_channel.hpp"
#include "../core/gguf_reader.hpp"
#include "../core/model_config.hpp"
#include "../core/openai_server.hpp"
#include "../core/qwen_weight_map.hpp"
#include "../core/safetensors_reader.hpp"
#include "qwen_engine.hpp"

using namespace pocket;

namespace {

struct Args {
  std::string ckpt, model_config, grep, tensor, token_ids, token_file, eos, host = "127.0.0.1", python = "python", sidecar_gguf,
      chat_family = "deepseek_v4", served_name = "pocketllm";
  int port = 8000, tp_world = 1, tp_rank = 0, ep_world = 1, prefix_interval = 0, prefix_entries = 4;
  std::string nccl_id_path;
  bool serve = false, audit = false, audit_strict = false;
  bool dump_config = false, inspect = false, context_info = false, smoke = false, bench = false, persistent = false,
       serve_batch = false, json = false, verbose = false;
  int max_new = 16, chunk = 8192, layers = 0, device = 0, synthetic = 0, slots = 1, bench_runs = 3, topk_print = 0;
  long long max_context = 8192 + 512;
  HostSamplingParams sampling;
  unsigned long long seed = 0;
};

// Whole numbers separated by commas or blanks.  Anything else ("abc", "1.5", a value that does not fit 32 bits) makes the
// line invalid as a whole: `err` says which field, nothing is guessed.
bool parse_ids_checked(const std::string& s, std::vector<int32_t>& out, std::string& err) {
  out.clear();
  std::string cur;
  for (char c : s + ",") {
    if (c == ',' || c == ' ' || c == '\n' || c == '\t' || c == '\r') {
      if (!cur.empty()) {
        errno = 0;
        char* end = nullptr;
        const long long v = std::strtoll(cur.c_str(), &end, 10);
        if (end == cur.c_str() || *end != '\0' || errno != 0 || v < -2147483648ll || v > 2147483647ll) {
          err = "not a whole 32-bit number: " + cur.substr(0, 32);
          return false;
        }
        out.push_back(int32_t(v));
      }
      cur.clear();
    } else {
      cur.push_back(c);
    }
  }
  return true;
}

std::vector<int32_t> parse_ids(const std::string& s) {
  std::vector<int32_t> out;
  std::string err;
  if (!parse_ids_checked(s, out, err)) throw std::runtime_error(err);
  return out;
}

// Empty when every id is a row of the model's tables (0 .. vocab - 1), else what is wrong.  Kernels index the embedding
// with these ids, so a foreign one is refused here.
std::string bad_token(const std::vector<int32_t>& ids, int64_t vocab) {
  for (int32_t t : ids)
    if (t < 0 || (vocab > 0 && int64_t(t) >= vocab))
      return "token id " + std::to_string(t) + " is outside the vocabulary (" + std::to_string(vocab) + ")";
  return "";
}

std::string join(const std::vector<int32_t>& v) {
  std::string s;
  for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + std::to_string(v[i]);
  return s;
}

void usage() {
  std::fprintf(stderr,
               "usage: pocketllm_engine --ckpt DIR [--dump-config | --inspect [--grep S] | --inspect-tensor NAME |\n"
               "         --context-info | --smoke-forward | --resident-bench | --qwen-persistent-stdin | --serve-batch]\n"
               "       [--token-ids a,b,c | --token-ids-file F | --tokens N] [--max-new-tokens N] [--max-context C]\n"
               "       [--prefill-chunk-tokens T] [--smoke-layers L] [--max-slots S] [--device D] [--eos a,b] [--json]\n"
               "       [--qwen-temperature F] [--qwen-top-k K] [--qwen-top-p P] [--qwen-seed S] [--bench-runs R]\n");
}

bool parse(int argc, char** argv, Args& a) {
  for (int i = 1; i < argc; ++i) {
    const std::string arg = argv[i];
    auto val = [&](const char* name) -> const char* {
      if (i + 1 >= argc) throw std::runtime_error(std::string("missing value for ") + name);
      return argv[++i];
    };
    if (arg == "--ckpt" || arg == "--model") a.ckpt = val("--ckpt");
    else if (arg == "--dump-config") a.dump_config = true;
    else if (arg == "--inspect") a.inspect = true;
    else if (arg == "--model-config") a.model_config = val("--model-config");
    else if (arg == "--ep-world") a.ep_world = std::atoi(val("--ep-world"));
    else if (arg == "--grep") a.grep = val("--grep");
    else if (arg == "--inspect-tensor" || arg == "--tensor") a.tensor = val("--inspect-tensor");
    else if (arg == "--context-info") a.context_info = true;
    else if (arg == "--smoke-forward") a.smoke = true;
    else if (arg == "--resident-bench") a.bench = true;
    else if (arg == "--bench-runs") a.bench_runs = std::atoi(val("--bench-runs"));
    else if (arg == "--qwen-persistent-stdin") a.persistent = true;
    else if (arg == "--serve-batch") a.serve_batch = true;
    else if (arg == "--serve") a.serve = true;
    else if (arg == "--qwen-audit") a.audit = true;
    else if (arg == "--qwen-audit-strict") a.audit = a.audit_strict = true;
    else if (arg == "--tp-world") a.tp_world = std::atoi(val("--tp-world"));
    else if (arg == "--tp-rank") a.tp_rank = std::atoi(val("--tp-rank"));
    else if (arg == "--nccl-id-path") a.nccl_id_path = val("--nccl-id-path");
    else if (arg == "--host") a.host = val("--host");
    else if (arg == "--port") a.port = std::atoi(val("--port"));
    else if (arg == "--python") a.python = val("--python");
    else if (arg == "--sidecar-gguf" || arg == "--sidecar") a.sidecar_gguf = val("--sidecar-gguf");
    else if (arg == "--chat-family") a.chat_family = val("--chat-family");
    else if (arg == "--served-model-name") a.served_name = val("--served-model-name");
    else if (arg == "--token-ids" || arg == "--ids") a.token_ids = val("--token-ids");
    else if (arg == "--token-ids-file") a.token_file = val("--token-ids-file");
    else if (arg == "--tokens") a.synthetic = std::atoi(val("--tokens"));
    else if (arg == "--max-new-tokens") a.max_new = std::atoi(val("--max-new-tokens"));
    else if (arg == "--max-context") a.max_context = std::atoll(val("--max-context"));
    else if (arg == "--kv-cache-dtype") {
      // the executable keeps the paged cache in bf16; the 8-bit layouts (fp8, int8_per_token_head, turboquant_k8v4)
      // are served by the Python runtime (pocketllm serve --kv-cache-dtype ...)
      const std::string v = val("--kv-cache-dtype");
      if (v == "fp8" || v == "int8_per_token_head" || v == "turboquant_k8v4")
        throw std::invalid_argument("--kv-cache-dtype " + v + " is not available in this executable (bf16 cache only); use pocketllm serve");
      if (v != "auto" && v != "bf16" && v != "fp16") throw std::invalid_argument("unknown kv cache dtype: " + v);
    }
    else if (arg == "--prefill-chunk-tokens") a.chunk = std::atoi(val("--prefill-chunk-tokens"));
    else if (arg == "--smoke-layers") a.layers = std::atoi(val("--smoke-layers"));
    else if (arg == "--max-slots") a.slots = std::atoi(val("--max-slots"));
    else if (arg == "--device") a.device = std::atoi(val("--device"));
    else if (arg == "--eos") a.eos = val("--eos");
    else if (arg == "--json") a.json = true;
    else if (arg == "--verbose") a.verbose = true;
    else if (arg == "--print-topk") a.topk_print = std::atoi(val("--print-topk"));
    else if (arg == "--qwen-temperature") a.sampling.temperature = float(std::atof(val("--qwen-temperature")));
    else if (arg == "--qwen-top-k") a.sampling.top_k = std::atoi(val("--qwen-top-k"));
    else if (arg == "--qwen-top-p") a.sampling.top_p = float(std::atof(val("--qwen-top-p")));
    else if (arg == "--qwen-seed") a.seed = std::strtoull(val("--qwen-seed"), nullptr, 10);
    else if (arg == "--qwen-no-prefix-cache") a.prefix_interval = 0;
    else if (arg == "--prefix-cache-interval" || arg == "--qwen-snapshot-interval") a.prefix_interval = std::atoi(val(arg.c_str()));
    else if (arg == "--prefix-cache-entries" || arg == "--qwen-max-snapshots") a.prefix_entries = std::atoi(val(arg.c_str()));
    else if (arg == "--qwen-mtp" || arg == "--qwen-mtp-adaptive" || arg == "--qwen-dspark" || arg == "--qwen-dflash2" ||
             arg == "--qwen-mtp-tokens" || arg == "--qwen-attention-window" || arg == "--qwen-attention-sink-tokens")
      // options of the reference executable that this one leaves to the Python runtime: say where they live
      throw std::invalid_argument(arg + " is not available in this executable: speculative decoding and windowed attention are "
                                  "served by `pocketllm serve --speculative-method mtp|ngram|dspark|dflash2 --speculative-tokens N "
                                  "--attention-window W --attention-sink-tokens S`");
    else if (arg == "-h" || arg == "--help") return false;
    else throw std::runtime_error("unknown argument " + arg);
  }
  return !a.ckpt.empty() || !a.model_config.empty();
}

std::vector<int32_t> prompt_of(const Args& a, int64_t vocab) {
  if (!a.token_ids.empty() || !a.token_file.empty()) {
    std::vector<int32_t> p = parse_ids(a.token_ids.empty() ? read_text_file(a.token_file) : a.token_ids);
    const std::string why = bad_token(p, vocab);
    if (!why.empty()) throw std::runtime_error(why);
    return p;
  }
  std::vector<int32_t> p;
  uint64_t x = 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < std::max(1, a.synthetic); ++i) {
    x ^= x << 13; x ^= x >> 7; x ^= x << 17;
    p.push_back(int32_t(x % uint64_t(vocab)));
  }
  return p;
}

int describe_model(const Args& a) {
  const std::string& p = a.model_config;
  const bool gguf = p.size() > 5 && p.compare(p.size() - 5, 5, ".gguf") == 0;
  MoeModelConfig c;
  if (gguf) {
    GGUFReader file(p);
    c = MoeModelConfig::from_gguf(file);
  } else {
    c = MoeModelConfig::from_hf_dir(p);
  }
  std::printf("%s\n", c.describe().c_str());
  std::printf("kv_bytes_per_token_layer=%llu mla=%d indexer=%d\n", (unsigned long long)c.kv_bytes_per_token_layer(),
              int(c.is_mla()), int(c.has_indexer()));
  const auto probs = c.problems(std::max(1, a.tp_world), std::max(1, a.ep_world));
  for (const auto& q : probs) std::printf("problem: %s\n", q.c_str());
  std::printf("model_config_ok=%d\n", int(probs.empty()));
  return probs.empty() ? 0 : 3;
}

int inspect(const Args& a) {
  SafetensorsModel model(a.ckpt);
  if (!a.tensor.empty()) {
    const uint8_t* base = nullptr;
    const SafeTensorInfo* info = model.find(a.tensor, &base);
    if (!info) { std::fprintf(stderr, "no tensor %s\n", a.tensor.c_str()); return 2; }
    std::printf("name=%s dtype=%s shape=[", a.tensor.c_str(), info->dtype.c_str());
    for (size_t i = 0; i < info->shape.size(); ++i) std::printf("%s%llu", i ? "," : "", (unsigned long long)info->shape[i]);
    std::printf("] bytes=%llu first_bytes=", (unsigned long long)info->nbytes());
    for (size_t i = 0; i < std::min<size_t>(16, info->nbytes()); ++i) std::printf("%02x", base[i]);
    std::printf("\n");
    return 0;
  }
  size_t total = 0, shown = 0;
  for (const std::string& n : model.names()) {
    if (!a.grep.empty() && n.find(a.grep) == std::string::npos) continue;
    const uint8_t* base = nullptr;
    const SafeTensorInfo* info = model.find(n, &base);
    std::printf("%s %s [", n.c_str(), info->dtype.c_str());
    for (size_t i = 0; i < info->shape.size(); ++i) std::printf("%s%llu", i ? "," : "", (unsigned long long)info->shape[i]);
    std::printf("] %llu\n", (unsigned long long)info->nbytes());
    total += info->nbytes();
    ++shown;
  }
  std::printf("tensors=%zu bytes=%zu shards=%zu\n", shown, total, model.shard_count());
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  Args a;
  try {
    if (!parse(argc, argv, a)) { usage(); return 2; }
    if (!a.model_config.empty()) return describe_model(a);
    if (a.inspect || !a.tensor.empty()) return inspect(a);
    QwenConfig cfg = QwenConfig::from_file(a.ckpt + "/config.json");
    if (a.dump_config) {
      std::printf("vocab_size=%lld hidden_size=%lld intermediate_size=%lld layers=%lld full_layers=%lld linear_layers=%lld\n"
                  "attention_heads=%lld kv_heads=%lld head_dim=%lld rotary_dim=%lld rope_theta=%g output_gate=%d\n"
                  "linear_key_heads=%lld linear_value_heads=%lld conv_kernel=%lld quant=%s block=%lld\n",
                  (long long)cfg.vocab_size, (long long)cfg.hidden_size, (long long)cfg.intermediate_size,
                  (long long)cfg.num_hidden_layers, (long long)cfg.num_full_layers(), (long long)cfg.num_linear_layers(),
                  (long long)cfg.num_attention_heads, (long long)cfg.num_key_value_heads, (long long)cfg.head_dim,
                  (long long)cfg.rotary_dim(), cfg.rope_theta, int(cfg.attn_output_gate), (long long)cfg.linear_num_key_heads,
                  (long long)cfg.linear_num_value_heads, (long long)cfg.linear_conv_kernel_dim, cfg.quant_method.c_str(),
                  (long long)cfg.quant_block);
      return 0;
    }
    if (a.audit) {
      SafetensorsModel model(a.ckpt);
      const QwenAuditReport r = qwen_audit(model, cfg, a.tp_world);
      auto dump = [](const char* what, const std::vector<std::string>& v) {
        for (const auto& n : v) std::printf("qwen_audit_%s=%s\n", what, n.c_str());
      };
      dump("missing", r.missing); dump("unexpected", r.unexpected); dump("wrong_shape", r.wrong_shape);
      dump("wrong_dtype", r.wrong_dtype); dump("not_divisible", r.not_divisible);
      std::printf("qwen_audit=1 ok=%d expected=%zu found=%zu bytes=%llu tp_world=%d missing=%zu unexpected=%zu mtp=%d\n",
                  int(r.ok(a.audit_strict)), r.expected, r.found, (unsigned long long)r.bytes, a.tp_world, r.missing.size(),
                  r.unexpected.size(), int(r.has_mtp));
      return r.ok(a.audit_strict) ? 0 : 3;
    }
    if (a.context_info) {
      const long long kv_token = 2LL * cfg.num_full_layers() * cfg.num_key_value_heads * cfg.head_dim * 2;
      const long long state_slot = cfg.num_linear_layers() * cfg.linear_num_value_heads * cfg.linear_key_head_dim *
                                   cfg.linear_value_head_dim * 4;
      size_t free_b = 0, total_b = 0;
      int ndev = 0;
      if (cudaGetDeviceCount(&ndev) == cudaSuccess && ndev > 0) { cudaSetDevice(a.device); cudaMemGetInfo(&free_b, &total_b); }
      std::printf("kv_bytes_per_token=%lld recurrent_state_bytes_per_slot=%lld device_free_bytes=%zu device_total_bytes=%zu\n",
                  kv_token, state_slot, free_b, total_b);
      return 0;
    }

    std::unique_ptr<WeightSource> ws = WeightSource::open(a.ckpt);
    QwenEngineOptions opt;
    opt.max_slots = std::max(1, a.slots);
    opt.prefix_cache_interval = std::max(0, a.prefix_interval);
    opt.prefix_cache_entries = std::max(1, a.prefix_entries);
    opt.max_context = a.max_context;
    opt.prefill_chunk = std::max(1, a.chunk);
    opt.layers = a.layers;
    opt.device = a.device;
    opt.eos_tokens = parse_ids(a.eos);
    opt.sampling = a.sampling;
    opt.seed = a.seed;
    opt.tp_world = std::max(1, a.tp_world);
    opt.tp_rank = a.tp_rank;
    opt.nccl_id_path = a.nccl_id_path;
    // Multi-rank runs: one process per GPU, every rank started with the same arguments plus its --tp-rank.  Rank 0 owns
    // stdin / HTTP and hands each request to the others over the command channel (a unix socket beside the id file),
    // so idle workers block on a socket, not on a device collective (cpp_engine/engine/main.cpp:100-216, 640-764).
    const bool multi = opt.tp_world > 1;
    if (multi && (a.serve || a.serve_batch))
      throw std::invalid_argument("--serve / --serve-batch run on one rank; multi-rank serving goes through pocketllm serve");
    CmdChannel channel;
    if (multi && a.persistent) {
      if (!channel.open(a.nccl_id_path, a.tp_rank, opt.tp_world))
        throw std::runtime_error("command channel could not be opened beside " + a.nccl_id_path);
    }
    QwenNativeEngine eng(cfg, *ws, opt);
    if (a.verbose)
      std::fprintf(stderr, "loaded %.2f GB of weights in %.2f s; cache/state %.2f GB\n", eng.stats().weight_bytes / 1e9,
                   eng.stats().load_seconds, eng.stats().state_bytes / 1e9);

    auto report = [&](const std::vector<int32_t>& prompt, const std::vector<int32_t>& out, double ps, double ds,
                      const char* tag) {
      const double ptok = prompt.size() / std::max(ps, 1e-9);
      const double dtok = out.size() > 1 ? (out.size() - 1) / std::max(ds, 1e-9) : 0.0;
      if (a.json)
        std::printf("{\"%s\": 1, \"prompt_tokens\": %zu, \"tokens\": [%s], \"prefill_seconds\": %.6f, \"decode_seconds\": %.6f, "
                    "\"prefill_tok_s\": %.2f, \"decode_tok_s\": %.2f}\n", tag, prompt.size(), join(out).c_str(), ps, ds, ptok, dtok);
      else
        std::printf("%s=1 prompt_tokens=%zu tokens=%s prefill_seconds=%.6f decode_seconds=%.6f prefill_tok_s=%.2f decode_tok_s=%.2f\n",
                    tag, prompt.size(), join(out).c_str(), ps, ds, ptok, dtok);
      std::fflush(stdout);
    };

    if (a.persistent && multi && a.tp_rank > 0) {
      // worker rank: mirror rank 0's requests ([1, max_new, tokens...] = generate, [0] = stop)
      std::vector<int32_t> msg;
      while (channel.receive(msg, -1)) {
        if (msg.empty() || msg[0] == 0) break;
        if (msg[0] == 1 && msg.size() >= 3) {
          std::vector<int32_t> prompt(msg.begin() + 2, msg.end());
          try {
            eng.generate(prompt, msg[1]);
          } catch (const std::exception& e) {
            std::fprintf(stderr, "[rank %d] generate failed: %s\n", a.tp_rank, e.what());
          }
        }
      }
      return 0;
    }
    if (a.persistent) {
      std::printf("qwen_persistent_ready=1 max_context=%lld tp_world=%d\n", a.max_context, opt.tp_world);
      std::fflush(stdout);
      std::string line;
      while (std::getline(std::cin, line)) {
        if (line == "quit" || line == "exit") break;
        std::vector<int32_t> f;
        std::string why;
        if (!parse_ids_checked(line, f, why)) { std::printf("qwen_persistent_error=1 message=%s\n", why.c_str()); std::fflush(stdout); continue; }
        if (f.size() < 2 || f[0] < 1) { std::printf("qwen_persistent_error=1 message=expected <max_new_tokens> tok...\n"); std::fflush(stdout); continue; }
        const int max_new = f[0];
        std::vector<int32_t> prompt(f.begin() + 1, f.end());
        why = bad_token(prompt, cfg.vocab_size);
        if (!why.empty()) { std::printf("qwen_persistent_error=1 message=%s\n", why.c_str()); std::fflush(stdout); continue; }
        try {
          double ps = 0, ds = 0;
          if (multi) {
            std::vector<int32_t> msg{1, max_new};
            msg.insert(msg.end(), prompt.begin(), prompt.end());
            if (!channel.broadcast(msg)) throw std::runtime_error("a worker rank closed its command channel");
          }
          std::vector<int32_t> out = eng.generate(prompt, max_new, &ps, &ds);
          report(prompt, out, ps, ds, "qwen_persistent_result");
        } catch (const std::exception& e) {
          std::printf("qwen_persistent_error=1 message=%s\n", e.what());
          std::fflush(stdout);
        }
      }
      if (multi) channel.broadcast({0});
      return 0;
    }

    if (a.serve) {
      OpenAIServerOptions so;
      so.host = a.host;
      so.port = a.port;
      so.model_name = a.served_name;
      so.chat_family = a.chat_family;
      so.default_max_tokens = a.max_new;
      if (!a.sidecar_gguf.empty()) so.sidecar_argv = {a.python, "-m", "pocketllm.sidecar", "--gguf", a.sidecar_gguf};
      SchedulerOptions sched;
      sched.max_batch = opt.max_slots;
      sched.prefill_chunk_tokens = opt.prefill_chunk;
      sched.prefill_token_budget = opt.prefill_chunk;
      OpenAIServer server(eng, so, sched);
      server.start();
      std::printf("pocketllm_engine_serving=1 host=%s port=%d model=%s\n", a.host.c_str(), server.port(), a.served_name.c_str());
      std::fflush(stdout);
      static volatile std::sig_atomic_t stop_flag = 0;
      std::signal(SIGINT, [](int) { stop_flag = 1; });
      std::signal(SIGTERM, [](int) { stop_flag = 1; });
      while (!stop_flag) ::usleep(100000);
      server.stop();
      std::printf("pocketllm_engine_stopped=1 requests=%llu\n", (unsigned long long)server.requests_served());
      return 0;
    }

    if (a.serve_batch) {
      SchedulerOptions so;
      so.max_batch = opt.max_slots;
      so.prefill_chunk_tokens = opt.prefill_chunk;
      so.prefill_token_budget = opt.prefill_chunk;
      BatchScheduler sched(eng, so);
      std::vector<std::pair<uint64_t, size_t>> ids;
      std::string line;
      while (std::getline(std::cin, line)) {
        std::vector<int32_t> f;
        std::string why;
        if (!parse_ids_checked(line, f, why) || f.size() < 2 || f[0] < 1 ||
            !(why = bad_token(std::vector<int32_t>(f.begin() + 1, f.end()), cfg.vocab_size)).empty()) {
          std::fprintf(stderr, "skipped a request line: %s\n", why.empty() ? "expected <max_new_tokens> tok..." : why.c_str());
          continue;
        }
        ids.emplace_back(sched.submit(std::vector<int32_t>(f.begin() + 1, f.end()), f[0]), f.size() - 1);
      }
      for (auto& [id, n_prompt] : ids) {
        SchedulerResult r;
        sched.wait(id, r);
        std::printf("request=%llu finish=%s prompt_tokens=%zu tokens=%s queue_seconds=%.6f prefill_seconds=%.6f decode_seconds=%.6f%s%s\n",
                    (unsigned long long)id, r.finish_reason.c_str(), n_prompt, join(r.tokens).c_str(), r.queue_seconds,
                    r.prefill_seconds, r.decode_seconds, r.error.empty() ? "" : " error=", r.error.c_str());
      }
      SchedulerStats st = sched.stats();
      std::printf("scheduler completed=%llu failed=%llu prefill_tokens=%llu decode_tokens=%llu rounds=%llu\n",
                  (unsigned long long)st.completed, (unsigned long long)st.failed, (unsigned long long)st.prefill_tokens,
                  (unsigned long long)st.decode_tokens, (unsigned long long)st.rounds);
      sched.stop();
      return 0;
    }

    const std::vector<int32_t> prompt = prompt_of(a, cfg.vocab_size);
    if (a.bench) {
      double best_p = 1e30, best_d = 1e30;
      std::vector<int32_t> out;
      for (int r = 0; r < std::max(1, a.bench_runs) + 1; ++r) {     // first run is the warm-up
        double ps = 0, ds = 0;
        out = eng.generate(prompt, a.max_new, &ps, &ds);
        if (r == 0) continue;
        best_p = std::min(best_p, ps);
        best_d = std::min(best_d, ds);
      }
      report(prompt, out, best_p, best_d, "resident_bench");
      return 0;
    }
    // default and --smoke-forward: one generation
    double ps = 0, ds = 0;
    std::vector<int32_t> out = eng.generate(prompt, a.max_new, &ps, &ds);
    report(prompt, out, ps, ds, "smoke_forward");
    if (a.topk_print > 0)
      for (auto& [tok, logit] : eng.last_topk(a.topk_print)) std::printf("topk token=%d logit=%.6f\n", tok, logit);
    std::printf("kernel_launches=%llu\n", (unsigned long long)eng.stats().kernel_launches);
    return 0;
  } catch (const std::exception& e) {
    std::fprintf(stderr, "pocketllm_engine: %s\n", e.what());
    return 1;
  }
}
