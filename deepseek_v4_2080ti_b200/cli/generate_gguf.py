"""Greedy generation from a GGUF checkpoint (one process per GPU under torchrun for tensor / expert parallelism):

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m deepseek_v4_2080ti_b200.cli.generate_gguf \\
        --gguf model.gguf --token-ids 1,2,3 --max-new-tokens 64

Prints the token ids and a ``RESULT prefill_tps=... decode_tps=...`` line (prompt tokens / prefill seconds, generated
tokens after the first / decode seconds), the format of the reference's GGUF drivers
(src/runtime/generation.py:168-276, src/cli/generate_gguf.py, generate_glm.py)."""
from __future__ import annotations

import argparse
import sys
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="generate_gguf")
    ap.add_argument("--gguf", required=True)
    ap.add_argument("--token-ids", default="")
    ap.add_argument("--runtime-option", action="append", default=[], metavar="KEY=VALUE",
                    help="family-specific runtime option, repeatable (deepseek4: dspark=PATH|synthetic, dspark_block=N, "
                         "spec_gate=1, flashmemory=CKPT, flashmemory_ensemble=max|mean, kv_swap_chunks=N, kv_swap_chunk_entries=G)")
    ap.add_argument("--prompt", default="", help="text, encoded with the checkpoint's own BPE tokenizer")
    ap.add_argument("--max-new-tokens", type=int, default=32)
    ap.add_argument("--max-context", type=int, default=4096)
    ap.add_argument("--prefill-chunk-tokens", type=int, default=4096)
    ap.add_argument("--nccl", action="store_true", help="library collectives instead of the peer-memory kernels")
    ap.add_argument("--prewarm", action="store_true", help="stream the checkpoint through the page cache first")
    a = ap.parse_args(argv)
    from ..formats.gguf import read_bundle
    from ..models import registry
    from ..parallel import tp
    rank, world, local = tp.init_distributed()
    on_gpu = torch.cuda.is_available()
    dev = torch.device("cuda", local) if on_gpu else torch.device("cpu")     # host-only families run without a GPU
    if on_gpu:
        torch.cuda.set_device(dev)
    b = read_bundle(a.gguf)
    if a.prewarm:
        from ..formats.gguf.prewarm import prewarm_bundle
        prewarm_bundle(b)
    spec = registry.detect(b)
    if a.token_ids:
        ids = [int(x) for x in a.token_ids.replace(" ", ",").split(",") if x]
    else:
        from ..encoding.gguf_tokenizer import GGUFTokenizer
        ids = GGUFTokenizer.from_metadata(b.metadata).encode(a.prompt or "Hello")
    comm = None
    if world > 1:
        comm = tp.TPComm() if a.nccl else tp.PeerComm(slot_elems=max(1 << 20, a.prefill_chunk_tokens * 8192))
    t0 = time.time()
    extra = {}
    for item in a.runtime_option:
        if "=" not in item:
            raise SystemExit(f"--runtime-option {item!r}: expected KEY=VALUE")
        k, v = item.split("=", 1)
        extra[k.strip()] = v.strip()
    cfg, rt = spec.build_runtime(b, dev, rank, world, comm, max_slots=1, max_context=a.max_context, **extra)
    load_s = time.time() - t0
    vocab = int(getattr(cfg, "vocab_size", 0) or getattr(cfg, "vocab", 0) or 0)
    bad = [t for t in ids if t < 0 or (vocab and t >= vocab)]
    if bad or not ids:                                    # kernels index tables with the ids: refuse before the device sees them
        raise SystemExit(f"--token-ids: {bad[:4] if bad else 'empty'} is not a token id of this model"
                         + (f" (vocabulary {vocab})" if vocab else ""))
    prompt = torch.tensor(ids, dtype=torch.int32, device=dev)
    slot = rt.allocate()
    sync = torch.cuda.synchronize if on_gpu else (lambda: None)
    sync()
    t0 = time.time()
    tok = rt.prefill(slot, prompt, a.prefill_chunk_tokens)
    out = [int(tok.item())]
    t1 = time.time()
    while len(out) < a.max_new_tokens:
        tok = rt.decode([slot], tok.to(torch.int32))
        out.append(int(tok.item()))
    sync()
    t2 = time.time()
    rt.free(slot)
    if rank == 0:
        print("tokens=" + ",".join(map(str, out)))
        if hasattr(rt, "stats"):
            print("runtime_stats " + " ".join(f"{k}={v}" for k, v in rt.stats().items()))
        print(f"RESULT family={spec.architecture} world={world} load_seconds={load_s:.2f} prompt_tokens={len(ids)} "
              f"prefill_tps={len(ids) / max(t1 - t0, 1e-9):.2f} decode_tps={(len(out) - 1) / max(t2 - t1, 1e-9):.2f}", flush=True)
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
