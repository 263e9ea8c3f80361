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


def test_backend_options_and_supervisor_flags():
    from pocketllm import cli
    ns = cli.build_parser().parse_args(["serve", "/m", "-tp", "2", "--backend-option", "window=512", "--backend-option",
                                        'mix={"attn": "Q8_0"}', "--backend-option", "name=plain text",
                                        "--tensor-parallel-startup-timeout", "90", "--tensor-parallel-shutdown-timeout", "3",
                                        "--no-tensor-parallel-supervisor"])
    a = cli._args(ns, 0)
    assert a.backend_options["window"] == 512 and a.backend_options["mix"] == {"attn": "Q8_0"}
    assert a.backend_options["name"] == "plain text" and a.backend_options["pd_mode"] == "serial"
    assert ns.tensor_parallel_startup_timeout == 90.0 and ns.tensor_parallel_shutdown_timeout == 3.0
    assert ns.tensor_parallel_supervisor is False and ns.supervised_child is False
    import pytest
    with pytest.raises(SystemExit):
        cli.parse_backend_options(["novalue"])
    # several ranks without the supervisor and without a rank: refused before anything is loaded
    with pytest.raises(SystemExit, match="needs --tensor-parallel-rank"):
        cli.main(["serve", "/m", "-tp", "2", "--no-tensor-parallel-supervisor"])
