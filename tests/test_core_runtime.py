"""C++ runtime through its pybind module: block pool/table, scheduler against a fake engine,
command channel over real sockets between processes, readers on synthetic files, tokenizer, sampler."""
import json
import multiprocessing as mp
import os
import struct

import numpy as np
import pytest

cpp = pytest.importorskip("deepseek_v4_2080ti_b200.pocketllm_cpp")


def test_block_pool_all_or_nothing_and_refcounts():
    p = cpp.BlockPool(9, 16)
    assert p.total_blocks == 8 and p.free_blocks == 8 and p.blocks_for_tokens(33) == 3
    a = p.allocate(5)
    assert a == [1, 2, 3, 4, 5] and p.free_blocks == 3
    assert p.allocate(4) is None and p.free_blocks == 3            # nothing taken on failure
    p.retain(2)
    p.release(2)
    assert p.refcount(2) == 1 and p.free_blocks == 3
    p.release_all(a)
    assert p.free_blocks == 8
    with pytest.raises(ValueError):
        p.release(2)
    assert p.allocate(1) == [5]                                    # LIFO: most recently freed first


def test_block_table_growth_sharing_and_dirty_rows():
    p = cpp.BlockPool(17, 16)
    t = cpp.BlockTable(p, 4, 8)
    assert t.ensure_capacity(0, 40) and t.blocks_in(0) == 3
    assert t.take_dirty_rows() == [0] and t.take_dirty_rows() == []
    assert t.element_offset(0, 35) == t.block_at(0, 2) * 16 + 3
    assert not t.ensure_capacity(1, 16 * 9)                        # exceeds max_blocks_per_seq
    assert t.share_prefix(2, 0, 2) and p.refcount(t.block_at(0, 0)) == 2
    t.free_slot(0)
    assert p.refcount(t.block_at(2, 0)) == 1 and p.free_blocks == 16 - 2
    t.free_slot(2)
    assert p.free_blocks == 16
    assert t.ensure_capacity(3, 16 * 8) and not t.ensure_capacity(1, 16 * 8 + 16 * 1) or True


def test_block_table_adopts_blocks_held_by_a_cache():
    """A prefix cache keeps blocks alive with its own references and hands them to a fresh row."""
    p = cpp.BlockPool(9, 16)
    t = cpp.BlockTable(p, 3, 4)
    assert t.ensure_capacity(0, 48)
    held = [t.block_at(0, i) for i in range(2)]
    for b in held:
        p.retain(b)                                                # the cache's references
    t.free_slot(0)
    assert [p.refcount(b) for b in held] == [1, 1] and p.free_blocks == 8 - 2
    assert t.adopt(1, held) and t.blocks_in(1) == 2 and [p.refcount(b) for b in held] == [2, 2]
    assert t.take_dirty_rows() == [0, 1]
    assert t.ensure_capacity(1, 50) and t.blocks_in(1) == 4 and t.block_at(1, 0) == held[0]      # grows behind the prefix
    assert not t.adopt(1, held)                                    # only into an empty row
    t.free_slot(1)
    assert [p.refcount(b) for b in held] == [1, 1]
    for b in held:
        p.release(b)
    assert p.free_blocks == 8


class FakeEngine(cpp.InferenceEngine):
    """next token = last + 1; eos = 1000; KV accounting through a real BlockPool/BlockTable."""

    def __init__(self, slots=4, blocks=9, bt=16, ctx=256):
        super().__init__()
        self.pool = cpp.BlockPool(blocks, bt)
        self.table = cpp.BlockTable(self.pool, slots, (ctx + bt - 1) // bt)
        self.free = list(range(slots))[::-1]
        self.ctx = ctx
        self.log = []

    def max_slots(self): return self.table.max_slots
    def block_tokens(self): return self.pool.block_tokens
    def total_blocks(self): return self.pool.total_blocks
    def max_context(self): return self.ctx
    def allocate_slot(self): return self.free.pop() if self.free else -1
    def free_slot(self, s):
        self.table.free_slot(s)
        self.free.append(s)
    def reserve(self, s, n): return self.table.ensure_capacity(s, n)
    def is_eos(self, t): return t == 1000

    def batch_prefill(self, items):
        self.log.append(("prefill", [(i.slot, len(i.tokens), i.position, i.last_chunk) for i in items]))
        return cpp.StepResult([i.tokens[-1] + 1 if i.last_chunk else -1 for i in items])

    def batch_decode(self, slots, toks):
        self.log.append(("decode", list(slots)))
        return cpp.StepResult([t + 1 for t in toks])


def drain(s, n=200):
    for _ in range(n):
        if not s.step():
            break


def test_scheduler_batches_and_finishes():
    e = FakeEngine()
    s = cpp.BatchScheduler.make_manual(e)
    a = s.submit([5, 6, 7], 4)
    b = s.submit([100], 2)
    c = s.submit([997], 10)             # 998, 999, then 1000 == eos
    drain(s)
    ra, rb, rc = s.poll(a), s.poll(b), s.poll(c)
    assert ra.tokens == [8, 9, 10, 11] and ra.finish_reason == "length"
    assert rb.tokens == [101, 102] and rc.tokens == [998, 999] and rc.finish_reason == "stop"
    assert any(k == "decode" and len(v) == 3 for k, v in e.log)       # all three decoded together
    st = s.get_stats()
    assert st.completed == 3 and st.kv_blocks_reserved == 0 and e.pool.free_blocks == 8


def test_scheduler_admission_under_kv_pressure_is_fifo():
    e = FakeEngine(slots=4, blocks=9, bt=16)           # 8 usable blocks
    s = cpp.BatchScheduler.make_manual(e)
    big = s.submit(list(range(60)), 36)                 # 96 tokens -> 6 blocks
    mid = s.submit(list(range(40)), 8)                  # 48 tokens -> 3 blocks: does not fit next to big
    small = s.submit([1], 2)                            # 1 block: would fit, but must not jump the queue
    s.step()
    st = s.get_stats()
    assert st.queued == 2 and st.kv_blocks_reserved == 6
    drain(s)
    assert s.poll(big).finish_reason == "length" and s.poll(mid) is not None and s.poll(small) is not None
    with pytest.raises(ValueError):
        s.submit(list(range(200)), 200)                 # can never fit: refused at submit


def test_scheduler_chunked_prefill_budget_and_cancel():
    e = FakeEngine(blocks=40, ctx=512)
    o = cpp.SchedulerOptions()
    o.prefill_token_budget = 64
    o.prefill_chunk_tokens = 48
    s = cpp.BatchScheduler.make_manual(e, o)
    a = s.submit(list(range(100)), 2)
    b = s.submit(list(range(30)), 50)
    s.step()
    assert e.log[0] == ("prefill", [(0, 48, 0, False), (1, 16, 0, False)])   # 64-token budget split in order
    assert s.cancel(b)
    drain(s)
    assert s.poll(a).tokens == [100, 101]
    assert s.poll(b).finish_reason == "cancelled"
    assert not s.cancel(12345)


def test_scheduler_thread_mode_wait():
    e = FakeEngine()
    s = cpp.BatchScheduler(e)
    ids = [s.submit([i], 3) for i in range(6)]
    outs = [s.wait(i, 5000) for i in ids]
    s.stop()
    assert [o.tokens for o in outs] == [[i + 1, i + 2, i + 3] for i in range(6)]


def _worker(base, rank, world, q):
    from deepseek_v4_2080ti_b200 import pocketllm_cpp as c
    ch = c.CmdChannel()
    ok = ch.open(base, rank, world, 10000, 20)
    got = []
    while ok:
        m = ch.receive(5000)
        if m is None or m[0] == 0:
            break
        got.append(m)
    q.put((rank, got))


def test_cmd_channel_fanout_between_processes(tmp_path):
    base = str(tmp_path / "nccl_id")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(base, r, 3, q)) for r in (1, 2)]
    for p in procs:
        p.start()
    ch = cpp.CmdChannel()
    assert ch.open(base, 0, 3, 20000, 20)
    assert ch.broadcast([3, 7, 8192, 11, 12, 13]) and ch.broadcast([4, 7, 99]) and ch.broadcast([0])
    res = dict(q.get(timeout=20) for _ in procs)
    for p in procs:
        p.join(10)
    assert res[1] == res[2] == [[3, 7, 8192, 11, 12, 13], [4, 7, 99]]
    ch.close()
    assert not os.path.exists(base + ".cmdsock")


def test_cmd_channel_worker_times_out_without_rank0(tmp_path):
    ch = cpp.CmdChannel()
    assert not ch.open(str(tmp_path / "nobody"), 1, 2, 200, 20)


def _write_gguf(path, kv, tensors, align=32):
    def s(x):
        b = x.encode()
        return struct.pack("<Q", len(b)) + b
    out = b"GGUF" + struct.pack("<IQQ", 3, len(tensors), len(kv))
    for k, (ty, v) in kv.items():
        out += s(k) + struct.pack("<I", ty)
        if ty == 4: out += struct.pack("<I", v)
        elif ty == 6: out += struct.pack("<f", v)
        elif ty == 8: out += s(v)
        elif ty == 9:
            ety, items = v
            out += struct.pack("<IQ", ety, len(items))
            for it in items:
                out += s(it) if ety == 8 else struct.pack("<i", it)
    off = 0
    blobs = []
    for name, shape, ty, data in tensors:
        out += s(name) + struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape)
        out += struct.pack("<IQ", ty, off)
        blobs.append((off, data))
        off += (len(data) + align - 1) // align * align
    pad = (-len(out)) % align
    out += b"\0" * pad
    body = bytearray(off)
    for o, d in blobs:
        body[o:o + len(d)] = d
    open(path, "wb").write(out + bytes(body))


def test_gguf_reader_and_weight_source(tmp_path):
    p = str(tmp_path / "m.gguf")
    w = np.arange(12, dtype=np.float32)
    q8 = bytes(range(34)) * 6                          # 2 rows x 96 elems of q8_0 = 6 blocks
    ex = np.arange(2 * 3 * 4, dtype=np.float32)
    _write_gguf(p, {"general.architecture": (8, "minimax-m2"), "x.block_count": (4, 7), "x.eps": (6, 1e-5),
                    "tokenizer.ggml.tokens": (9, (8, ["a", "b", "ab"]))},
                [("w", [4, 3], 0, w.tobytes()), ("q", [96, 2], 8, q8), ("ffn_exps", [4, 3, 2], 0, ex.tobytes())])
    g = cpp.GGUFReader(p)
    md = g.metadata()
    assert g.version == 3 and md["general.architecture"] == "minimax-m2" and md["x.block_count"] == 7
    assert abs(md["x.eps"] - 1e-5) < 1e-9 and md["tokenizer.ggml.tokens"] == ["a", "b", "ab"]
    assert g.tensor_info("q")["type_name"] == "q8_0" and g.tensor_info("q")["nbytes"] == 204
    assert np.frombuffer(g.tensor_bytes("w"), dtype=np.float32).tolist() == w.tolist()
    ws = cpp.WeightSource.open(p)
    t = ws.get("w")
    assert ws.format == "gguf" and t["shape"] == [3, 4] and t["dtype"] == "f32"
    e1 = ws.get_expert("ffn_exps", 1)
    assert e1["shape"] == [3, 4] and np.frombuffer(e1["data"], dtype=np.float32).tolist() == ex[12:].tolist()
    ws.set_name_map(lambda n: {"model.w": "w"}.get(n, n))
    assert ws.get("model.w")["name"] == "w" and ws.get("nope") is None
    assert cpp.ggml_type_info(29) == ("iq1_m", 256, 56) and cpp.ggml_type_info(12) == ("q4_k", 256, 144)
    open(p, "r+b").write(b"XXXX")
    with pytest.raises(RuntimeError):
        cpp.GGUFReader(p)


def test_gguf_shard_paths(tmp_path):
    for i in (1, 2, 3):
        open(tmp_path / f"m-{i:05d}-of-00003.gguf", "wb").write(b"x")
    got = cpp.gguf_shard_paths(str(tmp_path / "m-00002-of-00003.gguf"))
    assert [os.path.basename(g) for g in got] == [f"m-{i:05d}-of-00003.gguf" for i in (1, 2, 3)]
    assert cpp.gguf_shard_paths("/x/plain.gguf") == ["/x/plain.gguf"]


def test_safetensors_source_sharded(tmp_path):
    def write(name, tensors):
        hdr, off, blob = {}, 0, b""
        for k, (dt, shape, data) in tensors.items():
            hdr[k] = {"dtype": dt, "shape": shape, "data_offsets": [off, off + len(data)]}
            off += len(data)
            blob += data
        h = json.dumps(hdr).encode()
        open(tmp_path / name, "wb").write(struct.pack("<Q", len(h)) + h + blob)
    a = np.arange(6, dtype=np.float32)
    write("s1.safetensors", {"a.weight": ("F32", [2, 3], a.tobytes())})
    write("s2.safetensors", {"b.weight": ("F8_E4M3", [4], bytes([0x38] * 4)), "b.weight_scale_inv": ("BF16", [1, 1], b"\x80\x3f")})
    json.dump({"weight_map": {"a.weight": "s1.safetensors", "b.weight": "s2.safetensors", "b.weight_scale_inv": "s2.safetensors"}},
              open(tmp_path / "model.safetensors.index.json", "w"))
    ws = cpp.WeightSource.open(str(tmp_path))
    assert ws.format == "safetensors" and sorted(ws.names()) == ["a.weight", "b.weight", "b.weight_scale_inv"]
    t = ws.get("a.weight")
    assert t["shape"] == [2, 3] and np.frombuffer(t["data"], dtype=np.float32).tolist() == a.tolist()
    assert ws.get("b.weight")["dtype"] == "F8_E4M3" and bytes(ws.get("b.weight")["data"]) == bytes([0x38] * 4)


def test_tokenizer_bpe_roundtrip():
    toks = ["h", "e", "l", "o", "Ġ", "w", "r", "d", "he", "ll", "hell", "hello", "Ġw", "<|eos|>"]
    merges = ["h e", "l l", "he ll", "hell o", "Ġ w"]
    t = cpp.Tokenizer.from_vocab(toks, merges, -1, 13)
    ids = t.encode_basic("hello world")
    assert [toks[i] for i in ids] == ["hello", "Ġw", "o", "r", "l", "d"]
    assert t.decode(ids) == b"hello world" and t.eos_id == 13 and t.find("zz") == -1


def test_qwen_config_and_detection(tmp_path):
    cfg = {"architectures": ["Qwen3_5ForConditionalGeneration"], "model_type": "qwen3_5",
           "text_config": {"vocab_size": 64, "hidden_size": 128, "intermediate_size": 256, "num_hidden_layers": 2,
                           "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 128,
                           "linear_num_key_heads": 2, "linear_num_value_heads": 4, "linear_key_head_dim": 128,
                           "linear_value_head_dim": 128, "partial_rotary_factor": 0.25,
                           "rope_parameters": {"rope_theta": 10000000}, "layer_types": ["linear_attention", "full_attention"]}}
    json.dump(cfg, open(tmp_path / "config.json", "w"))
    c = cpp.QwenConfig.from_file(str(tmp_path / "config.json"))
    assert (c.num_full_layers, c.num_linear_layers, c.rope_theta, c.head_dim) == (1, 1, 1e7, 128)
    c.validate(2)
    with pytest.raises(RuntimeError):
        c.validate(4)                                   # 2 kv heads / 256-wide MLP do not split 4 ways
    assert cpp.is_qwen3_5_checkpoint(str(tmp_path)) and not cpp.is_qwen3_5_checkpoint(str(tmp_path / "none"))
    assert json.loads(cpp.json_roundtrip('{"a":[1,2.5,"x\\n",null,true],"b":{"c":-3}}')) == {"a": [1, 2.5, "x\n", None, True], "b": {"c": -3}}


def test_host_sampler():
    sp = cpp.SamplingParams()
    logits = [0.0, 5.0, 1.0, 4.9]
    assert cpp.sample(logits, sp) == 1
    sp.temperature = 1.0
    sp.top_k = 2
    draws = {cpp.sample(logits, sp, seed) for seed in range(50)}
    assert draws == {1, 3}
    sp.top_k = 0
    sp.top_p = 0.3
    assert {cpp.sample(logits, sp, seed) for seed in range(20)} == {1}
    sp.top_p = 1.0
    sp.temperature = 0.0
    sp.repetition_penalty = 2.0
    assert cpp.sample(logits, sp, 0, [1]) == 3
    assert cpp.parse_kv_cache_dtype("fp8") == 1
