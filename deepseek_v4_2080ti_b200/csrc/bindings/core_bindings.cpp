// pybind11 module `pocketllm_cpp`: the C++ runtime exposed to Python - block pool/table,
// continuous-batching scheduler (driving a Python-implemented engine through a trampoline),
// command channel, GGUF / safetensors readers, weight source, tokenizer, configs, host sampler.
// The GIL is released around every blocking call.
// (Role of cpp_engine/python/bindings.cpp:1-494.)
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "core/batch_scheduler.hpp"
#include "core/openai_server.hpp"
#include "core/python_sidecar.hpp"
#include "core/block_pool.hpp"
#include "core/block_table.hpp"
#include "core/cmd_channel.hpp"
#include "core/gguf_reader.hpp"
#include "core/json_lite.hpp"
#include "core/model_config.hpp"
#include "core/qwen_config.hpp"
#include "core/qwen_weight_map.hpp"
#include "core/safetensors_reader.hpp"
#include "core/sampler.hpp"
#include "core/tokenizer.hpp"
#include "core/weight_source.hpp"

namespace py = pybind11;
using namespace pocket;

namespace {

// Python subclass implements the engine; every override takes the GIL.
class PyEngine : public InferenceEngine {
 public:
  using InferenceEngine::InferenceEngine;
  int max_slots() const override { PYBIND11_OVERRIDE_PURE(int, InferenceEngine, max_slots); }
  int block_tokens() const override { PYBIND11_OVERRIDE_PURE(int, InferenceEngine, block_tokens); }
  int total_blocks() const override { PYBIND11_OVERRIDE_PURE(int, InferenceEngine, total_blocks); }
  int64_t max_context() const override { PYBIND11_OVERRIDE_PURE(int64_t, InferenceEngine, max_context); }
  int allocate_slot() override { PYBIND11_OVERRIDE_PURE(int, InferenceEngine, allocate_slot); }
  void free_slot(int slot) override { PYBIND11_OVERRIDE_PURE(void, InferenceEngine, free_slot, slot); }
  bool reserve(int slot, int64_t tokens) override { PYBIND11_OVERRIDE_PURE(bool, InferenceEngine, reserve, slot, tokens); }
  StepResult batch_prefill(const std::vector<PrefillItem>& items) override {
    PYBIND11_OVERRIDE_PURE(StepResult, InferenceEngine, batch_prefill, items);
  }
  StepResult batch_decode(const std::vector<int>& slots, const std::vector<int32_t>& tokens) override {
    PYBIND11_OVERRIDE_PURE(StepResult, InferenceEngine, batch_decode, slots, tokens);
  }
  bool is_eos(int32_t token) const override { PYBIND11_OVERRIDE_PURE(bool, InferenceEngine, is_eos, token); }
  int64_t vocab_size() const override { PYBIND11_OVERRIDE(int64_t, InferenceEngine, vocab_size); }
};

py::object value_to_py(const GGUFValue& v) {
  switch (v.kind) {
    case GGUFValue::Kind::UInt: return py::int_(v.u);
    case GGUFValue::Kind::Int: return py::int_(v.i);
    case GGUFValue::Kind::Float: return py::float_(v.f);
    case GGUFValue::Kind::Bool: return py::bool_(v.b);
    case GGUFValue::Kind::String: return py::str(v.s);
    case GGUFValue::Kind::Array: {
      py::list l;
      for (const auto& i : v.items) l.append(value_to_py(i));
      return std::move(l);
    }
    default: return py::none();
  }
}

py::dict view_to_py(const TensorView& t, py::object keepalive) {
  py::dict d;
  d["name"] = t.name;
  d["dtype"] = t.dtype;
  d["ggml_type"] = t.ggml_type == 0xffffffffu ? py::object(py::none()) : py::object(py::int_(t.ggml_type));
  d["shape"] = t.shape;
  d["nbytes"] = t.nbytes;
  d["data"] = py::memoryview::from_memory(t.data, static_cast<py::ssize_t>(t.nbytes));
  d["_owner"] = keepalive;
  return d;
}

}  // namespace

PYBIND11_MODULE(pocketllm_cpp, m) {
  m.doc() = "C++ runtime of the B200-native PocketLLM engine";
  m.attr("backend") = "b200";

  py::class_<BlockPool>(m, "BlockPool")
      .def(py::init<int, int>(), py::arg("num_blocks"), py::arg("block_tokens"))
      .def_property_readonly("block_tokens", &BlockPool::block_tokens)
      .def_property_readonly("total_blocks", &BlockPool::total_blocks)
      .def_property_readonly("free_blocks", &BlockPool::free_blocks)
      .def("blocks_for_tokens", &BlockPool::blocks_for_tokens)
      .def("allocate", [](BlockPool& p, int n) -> py::object {
        std::vector<int32_t> out;
        if (!p.allocate(n, out)) return py::none();
        return py::cast(out);
      })
      .def("retain", &BlockPool::retain)
      .def("release", &BlockPool::release)
      .def("release_all", &BlockPool::release_all)
      .def("refcount", &BlockPool::refcount);

  py::class_<BlockTable>(m, "BlockTable")
      .def(py::init<BlockPool&, int, int>(), py::arg("pool"), py::arg("max_slots"), py::arg("max_blocks_per_seq"),
           py::keep_alive<1, 2>())
      .def_property_readonly("max_slots", &BlockTable::max_slots)
      .def_property_readonly("max_blocks_per_seq", &BlockTable::max_blocks_per_seq)
      .def("ensure_capacity", &BlockTable::ensure_capacity)
      .def("share_prefix", &BlockTable::share_prefix)
      .def("adopt", [](BlockTable& t, int dst, const std::vector<int32_t>& blocks) { return t.adopt(dst, blocks.data(), int(blocks.size())); })
      .def("free_slot", &BlockTable::free_slot)
      .def("blocks_in", &BlockTable::blocks_in)
      .def("block_at", &BlockTable::block_at)
      .def("element_offset", &BlockTable::element_offset)
      .def("row", [](const BlockTable& t, int slot) {
        return std::vector<int32_t>(t.row(slot), t.row(slot) + t.max_blocks_per_seq());
      })
      .def("take_dirty_rows", &BlockTable::take_dirty_rows);

  py::class_<PrefillItem>(m, "PrefillItem")
      .def(py::init<>())
      .def_readwrite("slot", &PrefillItem::slot)
      .def_readwrite("tokens", &PrefillItem::tokens)
      .def_readwrite("position", &PrefillItem::position)
      .def_readwrite("last_chunk", &PrefillItem::last_chunk);
  py::class_<StepResult>(m, "StepResult")
      .def(py::init<>())
      .def(py::init([](std::vector<int32_t> t) { StepResult r; r.next_tokens = std::move(t); return r; }))
      .def_readwrite("next_tokens", &StepResult::next_tokens);
  py::class_<InferenceEngine, PyEngine>(m, "InferenceEngine")
      .def(py::init<>())
      .def("vocab_size", [](const InferenceEngine& e) { return e.InferenceEngine::vocab_size(); },
           "0: the engine does not say how many token ids it knows (override to let front ends refuse foreign ids)");

  py::class_<SchedulerOptions>(m, "SchedulerOptions")
      .def(py::init<>())
      .def_readwrite("max_batch", &SchedulerOptions::max_batch)
      .def_readwrite("prefill_token_budget", &SchedulerOptions::prefill_token_budget)
      .def_readwrite("prefill_chunk_tokens", &SchedulerOptions::prefill_chunk_tokens)
      .def_readwrite("decode_first", &SchedulerOptions::decode_first);
  py::class_<SchedulerResult>(m, "SchedulerGenerationResult")
      .def_readonly("id", &SchedulerResult::id)
      .def_readonly("tokens", &SchedulerResult::tokens)
      .def_readonly("finish_reason", &SchedulerResult::finish_reason)
      .def_readonly("error", &SchedulerResult::error)
      .def_readonly("queue_seconds", &SchedulerResult::queue_seconds)
      .def_readonly("prefill_seconds", &SchedulerResult::prefill_seconds)
      .def_readonly("decode_seconds", &SchedulerResult::decode_seconds);
  py::class_<SchedulerStats>(m, "BatchSchedulerStats")
      .def_readonly("queued", &SchedulerStats::queued)
      .def_readonly("prefilling", &SchedulerStats::prefilling)
      .def_readonly("decoding", &SchedulerStats::decoding)
      .def_readonly("completed", &SchedulerStats::completed)
      .def_readonly("cancelled", &SchedulerStats::cancelled)
      .def_readonly("failed", &SchedulerStats::failed)
      .def_readonly("kv_blocks_total", &SchedulerStats::kv_blocks_total)
      .def_readonly("kv_blocks_reserved", &SchedulerStats::kv_blocks_reserved)
      .def_readonly("prefill_tokens", &SchedulerStats::prefill_tokens)
      .def_readonly("decode_tokens", &SchedulerStats::decode_tokens)
      .def_readonly("rounds", &SchedulerStats::rounds);
  py::class_<BatchScheduler>(m, "BatchScheduler")
      .def(py::init<InferenceEngine&, SchedulerOptions>(), py::arg("engine"), py::arg("options") = SchedulerOptions(),
           py::keep_alive<1, 2>())
      .def_static("make_manual", &BatchScheduler::make_manual, py::arg("engine"), py::arg("options") = SchedulerOptions(),
                  py::keep_alive<0, 1>())
      // Every call that takes the scheduler's mutex drops the GIL first: the scheduler thread may hold that mutex while
      // it calls into a Python engine, which needs the GIL - holding both ends in different order would deadlock.
      .def("submit", [](BatchScheduler& s, std::vector<int32_t> prompt, int max_new_tokens, bool stop_on_eos) {
        py::gil_scoped_release rel;
        return s.submit(std::move(prompt), max_new_tokens, stop_on_eos);
      }, py::arg("prompt"), py::arg("max_new_tokens"), py::arg("stop_on_eos") = true)
      .def("cancel", [](BatchScheduler& s, uint64_t id) { py::gil_scoped_release rel; return s.cancel(id); })
      .def("poll", [](BatchScheduler& s, uint64_t id) -> py::object {
        SchedulerResult r;
        bool ok;
        { py::gil_scoped_release rel; ok = s.poll(id, r); }
        if (!ok) return py::none();
        return py::cast(std::move(r));
      })
      .def("wait", [](BatchScheduler& s, uint64_t id, int timeout_ms) -> py::object {
        SchedulerResult r;
        bool ok;
        { py::gil_scoped_release rel; ok = s.wait(id, r, timeout_ms); }
        if (!ok) return py::none();
        return py::cast(std::move(r));
      }, py::arg("id"), py::arg("timeout_ms") = -1)
      .def("step", [](BatchScheduler& s) { py::gil_scoped_release rel; return s.step(); })
      .def("get_stats", [](BatchScheduler& s) { py::gil_scoped_release rel; return s.stats(); })
      .def("stop", [](BatchScheduler& s) { py::gil_scoped_release rel; s.stop(); });

  py::class_<CmdChannel>(m, "CmdChannel")
      .def(py::init<>())
      .def("open", [](CmdChannel& c, const std::string& base, int rank, int world, int timeout_ms, int retry_ms) {
        py::gil_scoped_release rel;
        return c.open(base, rank, world, timeout_ms, retry_ms);
      }, py::arg("base_path"), py::arg("rank"), py::arg("world"), py::arg("timeout_ms") = 600000, py::arg("retry_ms") = 50)
      .def("close", &CmdChannel::close)
      .def_property_readonly("is_open", &CmdChannel::is_open)
      .def_property_readonly("world", &CmdChannel::world)
      .def_property_readonly("rank", &CmdChannel::rank)
      .def("broadcast", [](CmdChannel& c, const std::vector<int32_t>& w) { py::gil_scoped_release rel; return c.broadcast(w); })
      .def("receive", [](CmdChannel& c, int timeout_ms) -> py::object {
        std::vector<int32_t> w;
        bool ok;
        { py::gil_scoped_release rel; ok = c.receive(w, timeout_ms); }
        if (!ok) return py::none();
        return py::cast(w);
      }, py::arg("timeout_ms") = -1);

  py::class_<GGUFReader, std::shared_ptr<GGUFReader>>(m, "GGUFReader")
      .def(py::init<const std::string&>())
      .def_property_readonly("version", &GGUFReader::version)
      .def_property_readonly("alignment", &GGUFReader::alignment)
      .def_property_readonly("data_offset", &GGUFReader::data_offset)
      .def("metadata", [](const GGUFReader& g) {
        py::dict d;
        for (const auto& kv : g.metadata()) d[py::str(kv.first)] = value_to_py(kv.second);
        return d;
      })
      .def("tensor_names", [](const GGUFReader& g) {
        std::vector<std::string> n;
        for (const auto& t : g.tensors()) n.push_back(t.name);
        return n;
      })
      .def("tensor_info", [](const GGUFReader& g, const std::string& name) -> py::object {
        const GGUFTensorInfo* t = g.tensor(name);
        if (!t) return py::none();
        py::dict d;
        d["name"] = t->name;
        d["shape"] = t->shape;
        d["type"] = t->type;
        const GGMLTypeInfo* ti = ggml_type_info(t->type);
        d["type_name"] = ti ? ti->name : "unknown";
        d["offset"] = t->offset;
        d["nbytes"] = t->nbytes;
        return std::move(d);
      })
      .def("tensor_bytes", [](std::shared_ptr<GGUFReader> g, const std::string& name) -> py::object {
        const GGUFTensorInfo* t = g->tensor(name);
        if (!t) return py::none();
        return py::memoryview::from_memory(g->tensor_data(*t), static_cast<py::ssize_t>(t->nbytes));
      }, py::keep_alive<0, 1>());
  m.def("gguf_shard_paths", &gguf_shard_paths);
  m.def("ggml_type_info", [](uint32_t type) -> py::object {
    const GGMLTypeInfo* ti = ggml_type_info(type);
    if (!ti) return py::none();
    return py::make_tuple(ti->name, ti->block_elems, ti->block_bytes);
  });

  py::class_<WeightSource, std::shared_ptr<WeightSource>>(m, "WeightSource")
      .def_static("open", [](const std::string& p) { return std::shared_ptr<WeightSource>(WeightSource::open(p)); })
      .def_property_readonly("format", &WeightSource::format)
      .def("names", &WeightSource::names)
      .def("get", [](std::shared_ptr<WeightSource> w, const std::string& name) -> py::object {
        TensorView t;
        if (!w->get(name, t)) return py::none();
        return view_to_py(t, py::cast(w));
      })
      .def("get_expert", [](std::shared_ptr<WeightSource> w, const std::string& name, int e) -> py::object {
        TensorView t;
        if (!w->get_expert(name, e, t)) return py::none();
        return view_to_py(t, py::cast(w));
      })
      .def("set_name_map", [](WeightSource& w, std::function<std::string(const std::string&)> f) { w.set_name_map(std::move(f)); });

  py::class_<Tokenizer>(m, "Tokenizer")
      .def_static("from_gguf", [](const GGUFReader& g) { return Tokenizer::from_gguf(g); })
      .def_static("from_vocab", &Tokenizer::from_vocab, py::arg("tokens"), py::arg("merges"), py::arg("bos") = -1, py::arg("eos") = -1)
      .def_property_readonly("vocab_size", &Tokenizer::vocab_size)
      .def_property_readonly("bos_id", &Tokenizer::bos_id)
      .def_property_readonly("eos_id", &Tokenizer::eos_id)
      .def("encode_basic", &Tokenizer::encode_basic, py::arg("text"), py::arg("add_bos") = false)
      .def("decode", [](const Tokenizer& t, const std::vector<int32_t>& ids) { return py::bytes(t.decode(ids)); })
      .def("find", &Tokenizer::find);

  py::class_<QwenConfig>(m, "QwenConfig")
      .def_static("from_file", &QwenConfig::from_file)
      .def_static("from_json_text", [](const std::string& s) { return QwenConfig::from_json(Json::parse(s)); })
      .def("validate", &QwenConfig::validate, py::arg("tp_world") = 1)
      .def_readonly("vocab_size", &QwenConfig::vocab_size)
      .def_readonly("hidden_size", &QwenConfig::hidden_size)
      .def_readonly("intermediate_size", &QwenConfig::intermediate_size)
      .def_readonly("num_hidden_layers", &QwenConfig::num_hidden_layers)
      .def_readonly("num_attention_heads", &QwenConfig::num_attention_heads)
      .def_readonly("num_key_value_heads", &QwenConfig::num_key_value_heads)
      .def_readonly("head_dim", &QwenConfig::head_dim)
      .def_readonly("layer_types", &QwenConfig::layer_types)
      .def_readonly("rope_theta", &QwenConfig::rope_theta)
      .def_readonly("partial_rotary_factor", &QwenConfig::partial_rotary_factor)
      .def_property_readonly("num_full_layers", &QwenConfig::num_full_layers)
      .def_property_readonly("num_linear_layers", &QwenConfig::num_linear_layers);
  py::class_<MoeModelConfig>(m, "MoeModelConfig")
      .def_static("from_gguf", [](const GGUFReader& g) { return MoeModelConfig::from_gguf(g); })
      .def_static("from_gguf_file", [](const std::string& path) { GGUFReader g(path); return MoeModelConfig::from_gguf(g); })
      .def_static("from_hf_json_text", [](const std::string& s) { return MoeModelConfig::from_hf_json(Json::parse(s)); })
      .def_static("from_hf_dir", &MoeModelConfig::from_hf_dir)
      .def("describe", &MoeModelConfig::describe)
      .def("to_json_text", [](const MoeModelConfig& c) { return c.to_json().dump(); })
      .def("problems", &MoeModelConfig::problems, py::arg("tp_world") = 1, py::arg("ep_world") = 1)
      .def_property_readonly("is_mla", &MoeModelConfig::is_mla)
      .def_property_readonly("has_indexer", &MoeModelConfig::has_indexer)
      .def_property_readonly("kv_bytes_per_token_layer", &MoeModelConfig::kv_bytes_per_token_layer)
      .def_readonly("architecture", &MoeModelConfig::architecture)
      .def_readonly("compress_ratios", &MoeModelConfig::compress_ratios)
      .def_readonly("swiglu_clamp_exp", &MoeModelConfig::swiglu_clamp_exp);
  m.def("is_qwen3_5_checkpoint", [](const std::string& dir) {
    try {
      return QwenConfig::is_qwen3_5(Json::parse(read_text_file(dir + "/config.json")));
    } catch (const std::exception&) {
      return false;
    }
  });
  m.def("json_roundtrip", [](const std::string& s) { return Json::parse(s).dump(); });

  py::class_<HostSamplingParams>(m, "SamplingParams")
      .def(py::init<>())
      .def_readwrite("temperature", &HostSamplingParams::temperature)
      .def_readwrite("top_k", &HostSamplingParams::top_k)
      .def_readwrite("top_p", &HostSamplingParams::top_p)
      .def_readwrite("min_p", &HostSamplingParams::min_p)
      .def_readwrite("repetition_penalty", &HostSamplingParams::repetition_penalty)
      .def_readwrite("frequency_penalty", &HostSamplingParams::frequency_penalty)
      .def_readwrite("presence_penalty", &HostSamplingParams::presence_penalty);
  m.def("sample", [](const std::vector<float>& logits, const HostSamplingParams& p, uint64_t seed, const std::vector<int32_t>& hist) {
    std::mt19937_64 rng(seed);
    return sample(logits.data(), static_cast<int>(logits.size()), p, rng, hist);
  }, py::arg("logits"), py::arg("params"), py::arg("seed") = 0, py::arg("history") = std::vector<int32_t>{});
  py::class_<PythonSidecar>(m, "PythonSidecar")
      .def(py::init<std::vector<std::string>, int>(), py::arg("argv"), py::arg("timeout_ms") = 30000)
      .def("call", [](PythonSidecar& s, const std::string& request_json) {
        std::string out;
        { py::gil_scoped_release rel; out = s.call(Json::parse(request_json)).dump(); }
        return out;
      })
      .def("ping", [](PythonSidecar& s) { py::gil_scoped_release rel; return s.ping(); })
      .def("shutdown", [](PythonSidecar& s) { py::gil_scoped_release rel; s.shutdown(); })
      .def_property_readonly("running", &PythonSidecar::running);

  py::class_<OpenAIServerOptions>(m, "OpenAIServerOptions")
      .def(py::init<>())
      .def_readwrite("host", &OpenAIServerOptions::host)
      .def_readwrite("port", &OpenAIServerOptions::port)
      .def_readwrite("model_name", &OpenAIServerOptions::model_name)
      .def_readwrite("chat_family", &OpenAIServerOptions::chat_family)
      .def_readwrite("default_max_tokens", &OpenAIServerOptions::default_max_tokens)
      .def_readwrite("sidecar_argv", &OpenAIServerOptions::sidecar_argv);
  py::class_<OpenAIServer>(m, "OpenAIServer")
      .def(py::init<InferenceEngine&, OpenAIServerOptions, SchedulerOptions>(), py::arg("engine"), py::arg("options"),
           py::arg("scheduler_options") = SchedulerOptions(), py::keep_alive<1, 2>())
      .def("start", [](OpenAIServer& s) { py::gil_scoped_release rel; s.start(); })
      .def("stop", [](OpenAIServer& s) { py::gil_scoped_release rel; s.stop(); })
      .def_property_readonly("port", &OpenAIServer::port)
      .def_property_readonly("requests_served", &OpenAIServer::requests_served)
      .def("handle", [](OpenAIServer& s, const std::string& method, const std::string& path, const std::string& body) {
        OpenAIServer::Reply r;
        { py::gil_scoped_release rel; r = s.handle(method, path, body); }
        return py::make_tuple(r.status, r.content_type, r.body);
      });

  m.def("qwen_expected_tensors", [](const QwenConfig& cfg, bool mtp) {
    py::list out;
    for (const QwenTensorSpec& s : mtp ? qwen_mtp_tensors(cfg) : qwen_expected_tensors(cfg)) {
      py::dict d;
      d["name"] = s.name; d["shape"] = s.shape; d["dtype"] = s.dtype; d["rule"] = to_string(s.rule); d["group"] = s.group;
      out.append(d);
    }
    return out;
  }, py::arg("config"), py::arg("mtp") = false);
  m.def("qwen_audit", [](const std::string& dir, int tp_world) {
    SafetensorsModel model(dir);
    const QwenConfig cfg = QwenConfig::from_file(dir + "/config.json");
    const QwenAuditReport r = qwen_audit(model, cfg, tp_world);
    py::dict d;
    d["expected"] = r.expected; d["found"] = r.found; d["bytes"] = r.bytes; d["missing"] = r.missing;
    d["unexpected"] = r.unexpected; d["wrong_shape"] = r.wrong_shape; d["wrong_dtype"] = r.wrong_dtype;
    d["not_divisible"] = r.not_divisible; d["ok"] = r.ok(false); d["ok_strict"] = r.ok(true); d["has_mtp"] = r.has_mtp;
    return d;
  }, py::arg("checkpoint"), py::arg("tp_world") = 1);

  m.def("parse_kv_cache_dtype", [](const std::string& s) {
    if (s == "auto" || s == "bf16" || s == "fp16") return 0;
    if (s == "fp8") return 1;
    if (s == "turboquant_k8v4") return 2;
    if (s == "int8_per_token_head") return 3;
    throw std::invalid_argument("unknown kv cache dtype: " + s);
  });
}
