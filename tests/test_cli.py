import pytest

from pocketllm.cli import _args, _backend_options, build_parser


def test_serve_flags_map_to_engine_args():
    ns = build_parser().parse_args(["serve", "/ckpt", "--tensor-parallel-size", "4", "--kv-cache-dtype", "fp8",
                                    "--prefill-chunk-tokens", "4096", "--no-enable-prefix-caching", "--max-batch-size", "8",
                                    "--speculative-method", "mtp", "--speculative-tokens", "3", "--engine-kind", "qwen_hybrid",
                                    "--attention-window", "2048", "--attention-sink-tokens", "4", "--port", "9000"])
    a = _args(ns, 2)
    assert (a.model, a.tensor_parallel_size, a.tensor_parallel_rank, a.kv_cache_dtype) == ("/ckpt", 4, 2, "fp8")
    assert a.prefill_chunk_tokens == 4096 and a.enable_prefix_caching is False and a.max_batch_size == 8
    assert a.speculative_method == "mtp" and a.speculative_tokens == 3 and a.attention_window == 2048
    assert _backend_options(ns)["engine_kind"] == "qwen_hybrid" and ns.port == 9000


def test_model_is_required():
    ns = build_parser().parse_args(["serve"])
    with pytest.raises(SystemExit):
        _args(ns, 0)
