"""GQA + routed-expert GGUF family (MiniMax-M2.7-shaped): synthetic GGUF round trip and the fp32 oracle on CPU; on a
GPU, the runtime (GGUF blocks decoded inside the tensor-core GEMMs) against that oracle."""
import os
import tempfile

import pytest
import torch

from deepseek_v4_2080ti_b200.formats import gguf as G
from deepseek_v4_2080ti_b200.models import gqa_moe as gm


def test_synthetic_gguf_round_trip_and_oracle_runs_on_cpu():
    cfg = gm.GqaMoeConfig.tiny(layers=1, experts=8)
    cfg.gate_up_type, cfg.down_type = "Q2_K", "Q2_K"          # the IQ quantisers are slow on CPU; covered on the GPU
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "tiny.gguf")
        gm.write_synthetic_gguf(path, cfg, seed=3)
        b = G.read_bundle(path)
        assert b.architecture == "minimax-m2"
        got = gm.GqaMoeConfig.from_metadata(b.metadata, b.tensors)
        got.norm_eps = cfg.norm_eps                      # stored as float32 in the file
        assert got == cfg
        store = gm.TensorStore(b)
        mem = gm.TensorStore(gm.synth_tensors(cfg, seed=3))
        for n in ("blk.0.attn_q.weight", "blk.0.ffn_down_exps.weight", "blk.0.exp_probs_b.bias", "output.weight"):
            a, ta, sa = store.get(n)
            m, tm, sm = mem.get(n)
            assert ta == tm and sa == sm and torch.equal(a.reshape(-1), m.reshape(-1)), n
        ref = gm.GqaMoeReference(cfg, store.dequantized())
        prompt = torch.randint(0, cfg.vocab, (12,), generator=torch.Generator().manual_seed(1))
        logits = ref.forward(prompt)
        assert logits.shape == (12, cfg.vocab) and torch.isfinite(logits).all()
        # incremental decoding continues the same context: one more token equals a longer one-shot pass
        nxt = torch.tensor([int(logits[-1].argmax())])
        step = ref.forward(nxt)
        full = gm.GqaMoeReference(cfg, store.dequantized()).forward(torch.cat([prompt, nxt]))
        assert torch.allclose(step[-1], full[-1], atol=1e-4, rtol=1e-4)


@pytest.mark.gpu
@pytest.mark.parametrize("types", [("Q5_K", "Q4_K", "IQ1_M", "IQ2_XXS"), ("Q8_0", "Q8_0", "Q2_K", "IQ3_XXS")])
def test_gpu_runtime_follows_fp32_oracle(types):
    from deepseek_v4_2080ti_b200.ops import _lib
    cfg = gm.GqaMoeConfig.tiny(layers=2, experts=16)
    cfg.attn_type, cfg.dense_type, cfg.gate_up_type, cfg.down_type = types
    tensors = list(gm.synth_tensors(cfg, seed=5, device="cuda", std=0.05))
    store = gm.TensorStore(tensors)
    ref = gm.GqaMoeReference(cfg, {k: v.cpu() for k, v in store.dequantized().items()})
    prompt = torch.randint(0, cfg.vocab, (40,), generator=torch.Generator().manual_seed(2))
    want_logits = ref.forward(prompt)[-1]
    w = gm.GqaMoeGpuWeights(cfg, store, "cuda")
    rt = gm.GqaMoeRuntime(cfg, w, max_slots=2, max_context=256)
    slot = rt.allocate()
    ids = prompt.to("cuda", torch.int32)
    st = rt.seqs[slot]
    rt._ensure(st, 40)
    pos = torch.arange(40, dtype=torch.int32, device="cuda")
    kv_slots = (rt.block_table[slot][(pos // 64).long()] * 64 + pos % 64).to(torch.int32)
    i32 = lambda v: torch.tensor([v], dtype=torch.int32, device="cuda")
    meta = {"mode": "prefill", "block_table": rt.block_table[slot:slot + 1], "q_start": i32(0), "q_len": i32(40),
            "kv_len": i32(40), "max_q_len": 40}
    got = rt._forward(ids, pos, kv_slots, meta, torch.tensor([39], device="cuda"))[0].float().cpu()
    torch.cuda.synchronize()
    _lib.check_status()
    rt.free(slot)
    rel = ((got - want_logits).norm() / want_logits.norm()).item()
    assert rel < 0.05, rel
    # greedy streams: chunked prefill + graph-replayed decode against the oracle (bf16 activations may flip a near-tie late)
    want = gm.GqaMoeReference(cfg, {k: v.cpu() for k, v in store.dequantized().items()}).generate(prompt, 8)
    ours = rt.generate(prompt, 8, chunk=16)
    eager = rt.generate(prompt, 8, chunk=64, use_graph=False)
    _lib.check_status()
    assert ours[:3] == want[:3], (ours, want)
    assert eager[:3] == want[:3], (eager, want)


@pytest.mark.gpu
def test_public_api_serves_a_gguf_checkpoint():
    """``pocketllm.LLM`` on a MiniMax-style GGUF file: the loader routes it through the family registry; greedy tokens
    equal the runtime driven directly."""
    import os
    import tempfile
    from deepseek_v4_2080ti_b200.formats import gguf as G
    from deepseek_v4_2080ti_b200.models import gqa_moe as gm
    from deepseek_v4_2080ti_b200.models import registry
    from pocketllm import LLM, EngineArgs, SamplingParams
    cfg = gm.GqaMoeConfig.tiny()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "m.gguf")
        gm.write_synthetic_gguf(path, cfg, seed=3)
        b = G.read_bundle(path)
        _, rt = registry.detect(b).build_runtime(b, "cuda", 0, 1, None, max_slots=2, max_context=256)
        prompts = [[5, 9, 17, 3, 8], [1, 2, 3]]
        want = []
        for p in prompts:
            s = rt.allocate()
            t = rt.prefill(s, torch.tensor(p, dtype=torch.int32, device="cuda"), 64)
            out = [int(t.item())]
            for _ in range(4):
                t = rt.decode([s], t.to(torch.int32))
                out.append(int(t.item()))
            rt.free(s)
            want.append(out)
        del rt
        llm = LLM(EngineArgs(model=path, max_model_len=256, max_batch_size=2))
        outs = llm.generate([{"prompt_token_ids": p} for p in prompts], SamplingParams(max_tokens=5))
        assert [list(o.token_ids) for o in outs] == want
        llm.close()
