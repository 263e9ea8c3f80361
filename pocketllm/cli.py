"""``pocketllm serve``: parse flags, then run either as the supervising parent of a tensor-parallel
group or as one rank (rank 0 serves HTTP, the others run the worker loop).
Flag names follow the reference (pocketllm/cli.py:16-81)."""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Sequence

from .api.errors import PocketLLMError
from .api.types import EngineArgs

CHILD_ENV = "POCKETLLM_IS_TP_CHILD"


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="pocketllm", description="B200-native PocketLLM engine")
    sub = p.add_subparsers(dest="command", required=True)
    s = sub.add_parser("serve", help="start the OpenAI-compatible server")
    s.add_argument("model", nargs="?", default=None)
    s.add_argument("--model", dest="model_flag", default=None)
    s.add_argument("--backend", default="auto")
    s.add_argument("--tokenizer-path")
    s.add_argument("--config-path")
    s.add_argument("--model-format", default="auto")
    s.add_argument("--tensor-parallel-size", "-tp", type=int, default=1)
    s.add_argument("--tensor-parallel-rank", type=int, default=None)
    s.add_argument("--tensor-parallel-master-addr", default="127.0.0.1")
    s.add_argument("--tensor-parallel-master-port", type=int, default=0)
    s.add_argument("--tensor-parallel-rendezvous-dir")
    s.add_argument("--device", help="cuda index or 'cuda:N'; 'cpu' serves small models from the fp32 host runtimes")
    s.add_argument("--max-model-len", type=int)
    s.add_argument("--dtype")
    s.add_argument("--kv-cache-dtype", default="auto")
    s.add_argument("--prefill-chunk-tokens", type=int, default=0)
    s.add_argument("--enable-prefix-caching", action=argparse.BooleanOptionalAction, default=True)
    s.add_argument("--max-batch-size", type=int, default=1)
    s.add_argument("--host", default="127.0.0.1")
    s.add_argument("--port", type=int, default=8000)
    s.add_argument("--engine-kind", default=None, help="model family override: qwen_hybrid | gqa_moe | mla_moe")
    s.add_argument("--routed-experts-device", default="cuda", help="kept for compatibility; experts are GPU-resident")
    s.add_argument("--pd-mode", default="serial", choices=["serial", "interleave"])
    s.add_argument("--attention-window", type=int, default=0)
    s.add_argument("--attention-sink-tokens", type=int, default=0)
    s.add_argument("--speculative-method", default=None,
                   help="mtp | ngram on the GPU; the host path (--device cpu) also serves dspark | dflash2 "
                        "(--backend-option drafter=DIR)")
    s.add_argument("--speculative-tokens", type=int, default=1)
    s.add_argument("--served-model-name", default=None)
    s.add_argument("--tensor-parallel-supervisor", action=argparse.BooleanOptionalAction, default=True,
                   help="spawn and supervise the local ranks of a tensor-parallel group (default); with "
                        "--no-tensor-parallel-supervisor this process is one rank (--tensor-parallel-rank)")
    s.add_argument("--tensor-parallel-startup-timeout", type=float, default=1800.0, metavar="SECONDS",
                   help="how long the supervisor waits for every rank to report ready")
    s.add_argument("--tensor-parallel-shutdown-timeout", type=float, default=10.0, metavar="SECONDS",
                   help="grace period between TERM and KILL when the group is taken down")
    s.add_argument("--backend-option", action="append", default=[], metavar="KEY=VALUE",
                   help="backend-specific option, repeatable; the value is parsed as JSON when it parses, else kept as text")
    s.add_argument("--supervised-child", action="store_true", help=argparse.SUPPRESS)   # set by the supervisor on its ranks
    return p


def parse_backend_options(items: Sequence[str]) -> dict:
    """``KEY=VALUE`` pairs -> dict; JSON keeps numbers, booleans and nested values typed, a bare word stays a string
    (reference: pocketllm/cli.py:84-104)."""
    out: dict = {}
    for item in items:
        key, sep, raw = item.partition("=")
        if not sep or not key:
            raise SystemExit(f"--backend-option expects KEY=VALUE, got {item!r}")
        try:
            out[key] = json.loads(raw)
        except ValueError:
            out[key] = raw
    return out


def _backend_options(ns: argparse.Namespace) -> dict:
    opts = {}
    if ns.engine_kind:
        opts["engine_kind"] = ns.engine_kind
    if ns.routed_experts_device != "cuda":
        opts["routed_experts_device"] = ns.routed_experts_device
    opts["pd_mode"] = ns.pd_mode
    opts.update(parse_backend_options(ns.backend_option))
    return opts


def _args(ns: argparse.Namespace, rank: int) -> EngineArgs:
    model = ns.model or ns.model_flag
    if not model:
        raise SystemExit("pocketllm serve: a model path is required")
    return EngineArgs(model=model, backend=ns.backend, tokenizer_path=ns.tokenizer_path, config_path=ns.config_path,
                      model_format=ns.model_format, tensor_parallel_size=ns.tensor_parallel_size,
                      tensor_parallel_rank=rank, device=ns.device, max_model_len=ns.max_model_len, dtype=ns.dtype,
                      kv_cache_dtype=ns.kv_cache_dtype, prefill_chunk_tokens=ns.prefill_chunk_tokens,
                      enable_prefix_caching=ns.enable_prefix_caching, attention_window=ns.attention_window,
                      attention_sink_tokens=ns.attention_sink_tokens, speculative_method=ns.speculative_method,
                      speculative_tokens=ns.speculative_tokens, max_batch_size=ns.max_batch_size,
                      backend_options=_backend_options(ns))


def _emit_readiness(rank: int) -> None:
    print(f"POCKETLLM_RANK_READY rank={rank}", flush=True)


def _serve_rank(ns: argparse.Namespace, rank: int) -> int:
    from .backends.factory import create_backend
    from .server.openai import serve
    args = _args(ns, rank)
    backend = create_backend(args, supervise=False)
    backend.prepare()
    _emit_readiness(rank)
    if rank == 0:
        name = ns.served_model_name or os.path.basename(os.path.normpath(args.model)) or "pocketllm"
        print(f"pocketllm: serving {name} on http://{ns.host}:{ns.port}", file=sys.stderr, flush=True)
        serve(backend, ns.host, ns.port, name)
    else:
        backend.run_worker()
    return 0


def main(argv: Sequence[str] | None = None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    ns = build_parser().parse_args(argv)
    try:
        if ns.command != "serve":
            raise SystemExit(2)
        tp = ns.tensor_parallel_size
        is_child = os.environ.get(CHILD_ENV) == "1" or ns.tensor_parallel_rank is not None or ns.supervised_child
        if tp > 1 and not is_child and not ns.tensor_parallel_supervisor:
            raise SystemExit("pocketllm serve: --no-tensor-parallel-supervisor needs --tensor-parallel-rank (one process per rank)")
        if tp > 1 and not is_child:
            from .supervisor import TensorParallelConfig, TensorParallelSupervisor
            _args(ns, 0)  # validate before spawning anything
            cmd = [sys.executable, "-m", "pocketllm", *argv]
            cfg = TensorParallelConfig(world_size=tp, command=cmd, master_addr=ns.tensor_parallel_master_addr,
                                       master_port=ns.tensor_parallel_master_port,
                                       rendezvous_dir=ns.tensor_parallel_rendezvous_dir, extra_env={CHILD_ENV: "1"},
                                       ready_timeout=ns.tensor_parallel_startup_timeout,
                                       shutdown_grace=ns.tensor_parallel_shutdown_timeout)
            return TensorParallelSupervisor(cfg).run()
        rank = ns.tensor_parallel_rank if ns.tensor_parallel_rank is not None else int(os.environ.get("TP_RANK", os.environ.get("RANK", "0")))
        return _serve_rank(ns, rank)
    except PocketLLMError as exc:
        print(f"pocketllm: {type(exc).__name__}: {exc}", file=sys.stderr)
        return 1


if __name__ == "__main__":
    raise SystemExit(main())
