// pybind module `pocketllm_engine_cpp`: the native Qwen hybrid engine and a batch scheduler bound to it.
// Kept apart from `pocketllm_cpp` so that the host-only module imports on machines without the CUDA libraries.
// The GIL is released around every call that launches device work or waits.
// (Role of cpp_engine/python/bindings.cpp: QwenEngineOptions, QwenEngine, QwenBatchScheduler, stats structs.)
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "../core/batch_scheduler.hpp"
#include "../core/safetensors_reader.hpp"
#include "../engine/qwen_engine.hpp"

namespace py = pybind11;
using namespace pocket;

namespace {

struct EngineHolder {
  std::unique_ptr<WeightSource> ws;
  std::unique_ptr<QwenNativeEngine> eng;
  std::unique_ptr<BatchScheduler> sched;
};

}  // namespace

PYBIND11_MODULE(pocketllm_engine_cpp, m) {
  m.doc() = "Native sm_100a Qwen hybrid engine";
  m.attr("backend") = "b200";

  py::class_<HostSamplingParams>(m, "SamplingParams", py::module_local())
      .def(py::init<>())
      .def_readwrite("temperature", &HostSamplingParams::temperature)
      .def_readwrite("top_k", &HostSamplingParams::top_k)
      .def_readwrite("top_p", &HostSamplingParams::top_p)
      .def_readwrite("min_p", &HostSamplingParams::min_p);

  py::class_<QwenEngineOptions>(m, "QwenEngineOptions")
      .def(py::init<>())
      .def_readwrite("max_slots", &QwenEngineOptions::max_slots)
      .def_readwrite("prefix_cache_interval", &QwenEngineOptions::prefix_cache_interval)
      .def_readwrite("prefix_cache_entries", &QwenEngineOptions::prefix_cache_entries)
      .def_readwrite("max_context", &QwenEngineOptions::max_context)
      .def_readwrite("block_tokens", &QwenEngineOptions::block_tokens)
      .def_readwrite("prefill_chunk", &QwenEngineOptions::prefill_chunk)
      .def_readwrite("layers", &QwenEngineOptions::layers)
      .def_readwrite("device", &QwenEngineOptions::device)
      .def_readwrite("eos_tokens", &QwenEngineOptions::eos_tokens)
      .def_readwrite("sampling", &QwenEngineOptions::sampling)
      .def_readwrite("seed", &QwenEngineOptions::seed);

  py::class_<QwenEngineStats>(m, "QwenEngineStats")
      .def_readonly("kernel_launches", &QwenEngineStats::kernel_launches)
      .def_readonly("prefix_hits", &QwenEngineStats::prefix_hits)
      .def_readonly("prefix_tokens_reused", &QwenEngineStats::prefix_tokens_reused)
      .def_readonly("prefix_snapshots", &QwenEngineStats::prefix_snapshots)
      .def_readonly("prefix_evictions", &QwenEngineStats::prefix_evictions)
      .def_readonly("load_seconds", &QwenEngineStats::load_seconds)
      .def_readonly("weight_bytes", &QwenEngineStats::weight_bytes)
      .def_readonly("state_bytes", &QwenEngineStats::state_bytes);

  py::class_<SchedulerResult>(m, "SchedulerGenerationResult", py::module_local())
      .def_readonly("id", &SchedulerResult::id)
      .def_readonly("tokens", &SchedulerResult::tokens)
      .def_readonly("finish_reason", &SchedulerResult::finish_reason)
      .def_readonly("error", &SchedulerResult::error)
      .def_readonly("queue_seconds", &SchedulerResult::queue_seconds)
      .def_readonly("prefill_seconds", &SchedulerResult::prefill_seconds)
      .def_readonly("decode_seconds", &SchedulerResult::decode_seconds);

  py::class_<EngineHolder>(m, "QwenEngine")
      .def(py::init([](const std::string& ckpt, const QwenEngineOptions& opt) {
             auto h = std::make_unique<EngineHolder>();
             py::gil_scoped_release rel;
             QwenConfig cfg = QwenConfig::from_file(ckpt + "/config.json");
             h->ws = WeightSource::open(ckpt);
             h->eng = std::make_unique<QwenNativeEngine>(cfg, *h->ws, opt);
             return h;
           }),
           py::arg("checkpoint"), py::arg("options") = QwenEngineOptions())
      .def_property_readonly("max_slots", [](EngineHolder& h) { return h.eng->max_slots(); })
      .def_property_readonly("max_context", [](EngineHolder& h) { return h.eng->max_context(); })
      .def_property_readonly("total_blocks", [](EngineHolder& h) { return h.eng->total_blocks(); })
      .def_property_readonly("vocab_size", [](EngineHolder& h) { return h.eng->vocab_size(); })
      .def("allocate_slot", [](EngineHolder& h) { return h.eng->allocate_slot(); })
      .def("free_slot", [](EngineHolder& h, int s) { h.eng->free_slot(s); })
      .def("slot_length", [](EngineHolder& h, int s) { return h.eng->slot_length(s); })
      .def("prefill", [](EngineHolder& h, int slot, std::vector<int32_t> tokens, bool last_chunk) {
             PrefillItem it;
             it.slot = slot; it.tokens = std::move(tokens); it.position = h.eng->slot_length(slot); it.last_chunk = last_chunk;
             py::gil_scoped_release rel;
             return h.eng->batch_prefill({it}).next_tokens.at(0);
           }, py::arg("slot"), py::arg("tokens"), py::arg("last_chunk") = true)
      .def("decode_step", [](EngineHolder& h, std::vector<int> slots, std::vector<int32_t> tokens) {
             py::gil_scoped_release rel;
             return h.eng->batch_decode(slots, tokens).next_tokens;
           })
      .def("generate", [](EngineHolder& h, std::vector<int32_t> prompt, int max_new) {
             double ps = 0, ds = 0;
             std::vector<int32_t> out;
             { py::gil_scoped_release rel; out = h.eng->generate(prompt, max_new, &ps, &ds); }
             return py::make_tuple(out, ps, ds);
           }, py::arg("prompt"), py::arg("max_new_tokens"))
      .def("prefix_entries", [](EngineHolder& h) { return h.eng->prefix_entries(); })
      .def("last_topk", [](EngineHolder& h, int k) { return h.eng->last_topk(k); })
      // the target's output head as drafters see it: shard geometry, and a host-to-host projection for tests
      .def("target_head_info", [](EngineHolder& h) {
             const QwenTargetHead t = h.eng->target_head();
             py::dict d;
             d["wfmt"] = t.wfmt; d["local_vocab"] = t.local_vocab; d["hidden"] = t.hidden;
             d["vocab_start"] = t.vocab_start; d["valid"] = t.valid();
             return d;
           })
      .def("target_head_project", [](EngineHolder& h, const std::vector<uint16_t>& hidden_bf16_bits, int rows) {
             const QwenTargetHead t = h.eng->target_head();
             if (rows <= 0 || hidden_bf16_bits.size() != size_t(rows) * t.hidden) throw std::runtime_error("hidden must hold rows x hidden bf16 values");
             std::vector<float> out(size_t(rows) * t.local_vocab);
             {
               py::gil_scoped_release rel;
               void* dx = nullptr; float* dl = nullptr;
               cudaStream_t st = h.eng->stream();
               if (cudaMalloc(&dx, hidden_bf16_bits.size() * 2) != cudaSuccess || cudaMalloc(&dl, out.size() * 4) != cudaSuccess) {
                 cudaFree(dx);
                 throw std::runtime_error("target_head_project: out of device memory");
               }
               cudaMemcpyAsync(dx, hidden_bf16_bits.data(), hidden_bf16_bits.size() * 2, cudaMemcpyHostToDevice, st);
               const int rc = t.project(dx, dl, rows, st);
               cudaMemcpyAsync(out.data(), dl, out.size() * 4, cudaMemcpyDeviceToHost, st);
               const cudaError_t e = cudaStreamSynchronize(st);
               cudaFree(dx); cudaFree(dl);
               if (rc != 0 || e != cudaSuccess) throw std::runtime_error("target_head_project failed: rc " + std::to_string(rc));
             }
             return out;
           }, py::arg("hidden_bf16_bits"), py::arg("rows"))
      .def("stats", [](EngineHolder& h) { return h.eng->stats(); })
      // continuous batching over this engine
      .def("start_scheduler", [](EngineHolder& h, int max_batch, int prefill_token_budget) {
             SchedulerOptions so;
             so.max_batch = max_batch;
             so.prefill_token_budget = prefill_token_budget;
             so.prefill_chunk_tokens = prefill_token_budget;
             h.sched = std::make_unique<BatchScheduler>(*h.eng, so);
           }, py::arg("max_batch") = 8, py::arg("prefill_token_budget") = 8192)
      .def("submit", [](EngineHolder& h, std::vector<int32_t> prompt, int max_new, bool stop_on_eos) {
             if (!h.sched) throw std::runtime_error("start_scheduler() first");
             return h.sched->submit(std::move(prompt), max_new, stop_on_eos);
           }, py::arg("prompt"), py::arg("max_new_tokens"), py::arg("stop_on_eos") = true)
      .def("cancel", [](EngineHolder& h, uint64_t id) { return h.sched ? h.sched->cancel(id) : false; })
      .def("wait", [](EngineHolder& h, uint64_t id, int timeout_ms) -> py::object {
             if (!h.sched) throw std::runtime_error("start_scheduler() first");
             SchedulerResult r;
             bool ok;
             { py::gil_scoped_release rel; ok = h.sched->wait(id, r, timeout_ms); }
             if (!ok) return py::none();
             return py::cast(std::move(r));
           }, py::arg("id"), py::arg("timeout_ms") = -1)
      .def("stop_scheduler", [](EngineHolder& h) {
             if (h.sched) { py::gil_scoped_release rel; h.sched->stop(); }
             h.sched.reset();
           });

  m.def("is_qwen3_5_checkpoint", [](const std::string& ckpt) {
    try {
      return QwenConfig::is_qwen3_5(Json::parse(read_text_file(ckpt + "/config.json")));
    } catch (const std::exception&) {
      return false;
    }
  });
}
