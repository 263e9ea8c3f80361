"""The native executable (csrc/engine): inspection modes on CPU; on a GPU, greedy tokens of the C++ engine against
the Python runtime on the same tiny checkpoint, for one-shot, persistent-stdin and continuous-batching modes."""
import os
import re
import subprocess
import tempfile

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "deepseek_v4_2080ti_b200", "bin", "pocketllm_engine")
needs_exe = pytest.mark.skipif(not os.path.isfile(EXE), reason="native executable not built")


def _write_tiny(d, device="cpu", layers=4):
    from deepseek_v4_2080ti_b200.formats import safetensors_io
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=layers)
    state = list(qh.synth_state(cfg, 0, device, std=0.05))
    safetensors_io.write_checkpoint(d, iter(state), config_json=cfg.to_json())
    return cfg, state


def _run(args, stdin=None, timeout=300):
    return subprocess.run([EXE] + args, input=stdin, capture_output=True, text=True, timeout=timeout)


@needs_exe
def test_dump_config_inspect_and_context_info_need_no_gpu():
    with tempfile.TemporaryDirectory() as d:
        cfg, state = _write_tiny(d)
        r = _run(["--ckpt", d, "--dump-config"])
        assert r.returncode == 0, r.stderr
        assert f"hidden_size={cfg.hidden_size}" in r.stdout and f"layers={cfg.num_hidden_layers}" in r.stdout
        r = _run(["--ckpt", d, "--inspect", "--grep", "layers.0."])
        assert r.returncode == 0, r.stderr
        names = [n for n, _ in state if "layers.0." in n]
        assert f"tensors={len(names)}" in r.stdout
        assert "model.language_model.layers.0.input_layernorm.weight BF16" in r.stdout
        r = _run(["--ckpt", d, "--inspect-tensor", "model.language_model.norm.weight"])
        assert r.returncode == 0 and f"shape=[{cfg.hidden_size}]" in r.stdout
        r = _run(["--ckpt", d, "--context-info"])
        n_full = sum(t == "full_attention" for t in cfg.layer_types)
        assert r.returncode == 0
        assert f"kv_bytes_per_token={2 * n_full * cfg.num_key_value_heads * cfg.head_dim * 2}" in r.stdout


@needs_exe
def test_weight_map_audit_finds_missing_misshaped_and_indivisible_tensors():
    from deepseek_v4_2080ti_b200 import pocketllm_cpp as core
    from deepseek_v4_2080ti_b200.formats import safetensors_io
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    with tempfile.TemporaryDirectory() as d:
        cfg, state = _write_tiny(d)
        rep = core.qwen_audit(d, 1)
        assert rep["ok"] and rep["ok_strict"], rep
        assert rep["found"] == len(state) and rep["bytes"] > 0
        specs = {s["name"]: s for s in core.qwen_expected_tensors(core.QwenConfig.from_file(os.path.join(d, "config.json")))}
        assert set(specs) >= {n for n, _ in state}
        assert specs["model.language_model.layers.0.mlp.down_proj.weight"]["rule"] == "row_parallel"
        r = _run(["--ckpt", d, "--qwen-audit"])
        assert r.returncode == 0 and "qwen_audit=1 ok=1" in r.stdout, (r.stdout[-400:], r.stderr[-400:])
        # two ranks would split the 384-wide MLP inside a 128-row scale block (the loader refuses the same shard);
        # the attention and DeltaNet projections divide cleanly
        rep2 = core.qwen_audit(d, 2)
        assert not rep2["ok"] and all(".mlp." in n for n in rep2["not_divisible"]), rep2["not_divisible"]
        r = _run(["--ckpt", d, "--qwen-audit", "--tp-world", "3"])
        assert r.returncode == 3 and "qwen_audit_not_divisible=" in r.stdout and "self_attn" in r.stdout
    with tempfile.TemporaryDirectory() as d:
        cfg = qh.QwenHybridConfig.tiny(layers=4)
        state = list(qh.synth_state(cfg, 0, "cpu", std=0.05))
        victim = "model.language_model.layers.1.mlp.up_proj.weight"
        bad = [(n, t) for n, t in state if n != victim]
        bad = [(n, t[:-1] if n.endswith("layers.0.input_layernorm.weight") else t) for n, t in bad]
        bad.append(("model.language_model.layers.0.extra.bias", torch.zeros(4, dtype=torch.bfloat16)))
        safetensors_io.write_checkpoint(d, iter(bad), config_json=cfg.to_json())
        rep = core.qwen_audit(d, 1)
        assert rep["missing"] == [victim] and not rep["ok"]
        assert rep["wrong_shape"] == ["model.language_model.layers.0.input_layernorm.weight"]
        assert rep["unexpected"] == ["model.language_model.layers.0.extra.bias"]
        r = _run(["--ckpt", d, "--qwen-audit"])
        assert r.returncode == 3 and f"qwen_audit_missing={victim}" in r.stdout


@needs_exe
def test_weight_map_audit_requires_a_whole_mtp_head_when_one_is_present():
    from deepseek_v4_2080ti_b200 import pocketllm_cpp as core
    from deepseek_v4_2080ti_b200.formats import safetensors_io
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import synth_mtp_state
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    trunk = list(qh.synth_state(cfg, 0, "cpu", std=0.05))
    for fp8 in (False, True):
        with tempfile.TemporaryDirectory() as d:
            mtp = synth_mtp_state(cfg, 0, fp8_linears=fp8)
            safetensors_io.write_checkpoint(d, iter(trunk + mtp), config_json=cfg.to_json())
            rep = core.qwen_audit(d, 1)
            assert rep["ok"] and rep["ok_strict"] and rep["has_mtp"], rep
            assert rep["found"] == rep["expected"] == len(trunk) + len(mtp)
            names = {s["name"] for s in core.qwen_expected_tensors(core.QwenConfig.from_file(os.path.join(d, "config.json")), mtp=True)}
            assert {n for n, _ in mtp} <= names and "mtp.fc.weight" in names
            r = _run(["--ckpt", d, "--qwen-audit", "--qwen-audit-strict"])
            assert r.returncode == 0 and "mtp=1" in r.stdout
    with tempfile.TemporaryDirectory() as d:                      # half a head is an error, not an extra
        mtp = [(n, t) for n, t in synth_mtp_state(cfg, 0) if n != "mtp.norm.weight"]
        mtp = [(n, t[:, :-8].contiguous() if n == "mtp.fc.weight" else t) for n, t in mtp]
        safetensors_io.write_checkpoint(d, iter(trunk + mtp), config_json=cfg.to_json())
        rep = core.qwen_audit(d, 1)
        assert rep["missing"] == ["mtp.norm.weight"] and rep["wrong_shape"] == ["mtp.fc.weight"] and not rep["unexpected"]
    with tempfile.TemporaryDirectory() as d:
        safetensors_io.write_checkpoint(d, iter(trunk), config_json=cfg.to_json())
        assert not core.qwen_audit(d, 1)["has_mtp"]


@needs_exe
def test_bad_arguments_exit_non_zero():
    assert _run(["--nonsense"]).returncode != 0
    r = _run(["--ckpt", "x", "--kv-cache-dtype", "fp8", "--dump-config"])
    assert r.returncode != 0 and "bf16 cache only" in r.stderr
    assert "unknown kv cache dtype" in _run(["--ckpt", "x", "--kv-cache-dtype", "fp3"]).stderr
    assert _run([]).returncode == 2
    for flag in ("--qwen-dspark", "--qwen-mtp", "--qwen-attention-window"):      # options the reference executable has
        r = _run(["--ckpt", "x", flag])
        assert r.returncode != 0 and "pocketllm serve --speculative-method" in r.stderr, flag
    with tempfile.TemporaryDirectory() as d:
        # the reference's names for the snapshot settings are accepted
        assert "unknown argument" not in _run(["--ckpt", d, "--qwen-snapshot-interval", "64", "--qwen-max-snapshots", "4", "--dump-config"]).stderr
    with tempfile.TemporaryDirectory() as d:
        r = _run(["--ckpt", d, "--dump-config"])
        assert r.returncode == 1 and "pocketllm_engine:" in r.stderr


def _tokens(line):
    m = re.search(r"(?<![a-z_])tokens=([0-9,]+)", line)
    assert m, line
    return [int(t) for t in m.group(1).split(",")]


@pytest.mark.gpu
@needs_exe
def test_native_engine_tokens_match_python_runtime():
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    gen = torch.Generator().manual_seed(11)
    n_new = 10
    with tempfile.TemporaryDirectory() as d:
        cfg, state = _write_tiny(d, "cuda")
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen, dtype=torch.int32) for n in (70, 33, 5)]
        w = qh.QwenHybridWeights(cfg, iter(state), "cuda")
        rt = qh.QwenHybridRuntime(cfg, w, max_slots=1, max_context=256)
        want = [rt.generate(p, n_new) for p in prompts]

        ids = ",".join(map(str, prompts[0].tolist()))
        r = _run(["--ckpt", d, "--smoke-forward", "--token-ids", ids, "--max-new-tokens", str(n_new), "--max-context", "256",
                  "--print-topk", "3"])
        assert r.returncode == 0, (r.stdout[-500:], r.stderr[-500:])
        assert _tokens(r.stdout.splitlines()[0]) == want[0]
        assert "topk token=" in r.stdout and "kernel_launches=" in r.stdout

        # chunked prefill (chunk smaller than the prompt) gives the same stream
        r = _run(["--ckpt", d, "--token-ids", ids, "--max-new-tokens", str(n_new), "--max-context", "256",
                  "--prefill-chunk-tokens", "32"])
        assert r.returncode == 0, r.stderr[-500:]
        got = _tokens(r.stdout.splitlines()[0])
        assert got[:4] == want[0][:4]

        # persistent mode: several requests on one resident engine
        lines = "".join(f"{n_new} " + " ".join(map(str, p.tolist())) + "\n" for p in prompts) + "quit\n"
        r = _run(["--ckpt", d, "--qwen-persistent-stdin", "--max-context", "256"], stdin=lines)
        assert r.returncode == 0, r.stderr[-500:]
        res = [l for l in r.stdout.splitlines() if l.startswith("qwen_persistent_result=1")]
        assert [_tokens(l) for l in res] == want

        # continuous batching: the three requests share the decode batch; greedy streams stay per-request
        r = _run(["--ckpt", d, "--serve-batch", "--max-slots", "3", "--max-context", "256"], stdin=lines.replace("quit\n", ""))
        assert r.returncode == 0, r.stderr[-500:]
        res = [l for l in r.stdout.splitlines() if l.startswith("request=")]
        assert len(res) == 3 and all("finish=length" in l for l in res)
        for l, wnt in zip(res, want):
            assert _tokens(l)[:4] == wnt[:4]
        assert "scheduler completed=3" in r.stdout


@pytest.mark.gpu
def test_device_prepack_matches_host_prepack():
    import ctypes
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    for n, k in ((256, 512), (300, 192), (128, 64)):
        w = torch.randint(0, 256, (n, k), dtype=torch.uint8, device="cuda")
        want = gemm.prepack_fp8(w.view(torch.float8_e4m3fn))
        L = _lib.lib()
        L.b200_prepack_fp8_bytes.restype = ctypes.c_ulonglong
        out = torch.zeros(int(L.b200_prepack_fp8_bytes(n, k)), dtype=torch.uint8, device="cuda")
        assert L.b200_prepack_fp8(_lib.ptr(w), _lib.ptr(out), n, k, _lib.stream()) == 0
        torch.cuda.synchronize()
        assert torch.equal(out, want.view(torch.uint8).reshape(-1))


@pytest.mark.gpu
def test_pybind_engine_and_cpp_backend_match_python_runtime():
    """``pocketllm_engine_cpp.QwenEngine`` directly, and through ``pocketllm.LLM(backend="cpp")``."""
    from deepseek_v4_2080ti_b200 import pocketllm_engine_cpp as cpp
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    gen = torch.Generator().manual_seed(13)
    with tempfile.TemporaryDirectory() as d:
        cfg, state = _write_tiny(d, "cuda")
        assert cpp.is_qwen3_5_checkpoint(d) in (True, False)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=gen, dtype=torch.int32).tolist() for n in (50, 21)]
        w = qh.QwenHybridWeights(cfg, iter(state), "cuda")
        rt = qh.QwenHybridRuntime(cfg, w, max_slots=1, max_context=256)
        want = [rt.generate(torch.tensor(p, dtype=torch.int32), 6) for p in prompts]
        opt = cpp.QwenEngineOptions()
        opt.max_slots, opt.max_context = 2, 256
        eng = cpp.QwenEngine(d, opt)
        toks, ps, ds = eng.generate(prompts[0], 6)
        assert list(toks) == want[0] and ps > 0 and eng.stats().kernel_launches > 0
        s = eng.allocate_slot()
        t0 = eng.prefill(s, prompts[1])
        assert t0 == want[1][0] and eng.slot_length(s) == len(prompts[1])
        assert eng.decode_step([s], [t0])[0] == want[1][1]
        eng.free_slot(s)
        # the target head view: shard geometry, and the projection drafters use equals the plain matrix product
        info = eng.target_head_info()
        assert info["valid"] and info["local_vocab"] == cfg.vocab_size and info["hidden"] == cfg.hidden_size and info["vocab_start"] == 0
        head = dict(state).get("lm_head.weight")
        if head is None:
            head = dict(state)["model.language_model.embed_tokens.weight"]
        hid = (torch.randn(3, cfg.hidden_size, generator=gen) * 0.5).to(torch.bfloat16)
        bits = hid.view(torch.int16).to(torch.int32).bitwise_and(0xFFFF).flatten().tolist()
        got = torch.tensor(eng.target_head_project(bits, 3)).view(3, -1)
        ref = hid.float() @ head.detach().to("cpu", torch.bfloat16).float().t()
        assert ((got - ref).norm() / ref.norm()) < 2e-3
        eng.start_scheduler(2, 64)
        ids = [eng.submit(p, 6) for p in prompts]
        res = [eng.wait(i, 60000) for i in ids]
        assert [list(r.tokens)[:3] for r in res] == [x[:3] for x in want] and all(r.finish_reason == "length" for r in res)
        eng.stop_scheduler()
        del eng
        from pocketllm import LLM, EngineArgs, SamplingParams
        llm = LLM(EngineArgs(model=d, backend="cpp", max_model_len=256))
        out = llm.generate([{"prompt_token_ids": prompts[0]}], SamplingParams(max_tokens=6))
        assert list(out[0].token_ids) == want[0]
        llm.close()


@pytest.mark.gpu
def test_native_prefix_cache_resumes_from_shared_blocks_and_state():
    """Prompts that share their first tokens: the second one adopts the cached KV blocks and the recurrent-state
    snapshot of the longest common multiple of the interval and computes only the rest - same tokens as an engine
    without the cache (reference: the Qwen engine's snapshot ring, cpp_engine/engine/qwen_engine.cpp:5369-5563)."""
    from deepseek_v4_2080ti_b200 import pocketllm_engine_cpp as cpp
    gen = torch.Generator().manual_seed(21)
    with tempfile.TemporaryDirectory() as d:
        cfg, _ = _write_tiny(d, "cuda")
        base = torch.randint(0, cfg.vocab_size, (200,), generator=gen, dtype=torch.int32).tolist()
        other = torch.randint(0, cfg.vocab_size, (60,), generator=gen, dtype=torch.int32).tolist()
        prompts = [base, base[:150] + other, base[:70] + other, other + base[:100], base]
        plain_opt = cpp.QwenEngineOptions()
        plain_opt.max_slots, plain_opt.max_context = 2, 512
        plain = cpp.QwenEngine(d, plain_opt)
        want = [list(plain.generate(p, 5)[0]) for p in prompts]
        del plain
        opt = cpp.QwenEngineOptions()
        opt.max_slots, opt.max_context, opt.prefix_cache_interval, opt.prefix_cache_entries = 2, 512, 64, 8
        eng = cpp.QwenEngine(d, opt)
        got, reused = [], []
        for p in prompts:
            before = eng.stats().prefix_tokens_reused
            got.append(list(eng.generate(p, 5)[0]))
            reused.append(eng.stats().prefix_tokens_reused - before)
        assert got == want
        # 200 tokens: snapshots at 64, 128, 192.  150 shared -> resumes at 128; 70 shared -> 64; a prompt that starts
        # differently -> nothing; the first prompt again -> 192, the longest entry shorter than the prompt
        assert reused == [0, 128, 64, 0, 192]
        st = eng.stats()
        assert st.prefix_hits == 3 and st.prefix_snapshots >= 6 and st.prefix_evictions == 0 and eng.prefix_entries() <= 8
        # more distinct prompts than entries: the oldest snapshots go, results stay right
        for k in range(3):
            p = torch.randint(0, cfg.vocab_size, (200,), generator=gen, dtype=torch.int32).tolist()
            assert len(eng.generate(p, 2)[0]) == 2
        assert eng.stats().prefix_evictions > 0 and eng.prefix_entries() == 8
        assert list(eng.generate(prompts[1], 5)[0]) == want[1]
        with pytest.raises(Exception):
            bad = cpp.QwenEngineOptions()
            bad.prefix_cache_interval = 50                       # not a multiple of the block size
            cpp.QwenEngine(d, bad)
