"""Backend selection and construction (reference surface: pocketllm/backends/factory.py:101-227).

There is one engine, so ``auto``, ``b200``, ``torch`` and ``cpp`` all resolve to ``NativeBackend``;
the old names are accepted so existing launch scripts keep working.  For tensor-parallel use from
plain Python (``LLM(model, tensor_parallel_size=N)`` outside ``pocketllm serve``), the factory starts
the hidden worker ranks through the supervisor and returns the rank-0 backend.
"""
from __future__ import annotations

import json
import os
import sys
from typing import Any

from ..api.errors import ConfigurationError
from ..api.types import EngineArgs
from .native_backend import NativeBackend

_WORKER_ENV = "POCKETLLM_IS_TP_CHILD"


def detect_model_format(args: EngineArgs) -> str:
    if args.model_format != "auto":
        return args.model_format
    m = os.path.expanduser(args.model)
    if m.startswith("synthetic:"):
        return "synthetic"
    if m.endswith(".gguf") or (os.path.isdir(m) and any(f.endswith(".gguf") for f in os.listdir(m))):
        return "gguf"
    if os.path.isdir(m) and (os.path.exists(os.path.join(m, "model.safetensors.index.json"))
                             or any(f.endswith(".safetensors") for f in os.listdir(m))):
        return "safetensors"
    raise ConfigurationError(f"cannot detect the checkpoint format of {args.model!r}")


def select_backend(args: EngineArgs) -> str:
    if args.backend in ("auto", "b200", "torch", "cpp"):
        return "b200"
    raise ConfigurationError(f"unknown backend {args.backend!r}")


def _worker_script() -> str:
    return ("import sys\n"
            "from pocketllm.api.types import EngineArgs\n"
            "from pocketllm.backends.factory import create_backend\n"
            "args = EngineArgs.from_env()\n"
            "b = create_backend(args, supervise=False)\n"
            "b.prepare()\n"
            "print(f'POCKETLLM_RANK_READY rank={args.tensor_parallel_rank}', flush=True)\n"
            "b.run_worker()\n")


def create_backend(args: EngineArgs, supervise: bool | None = None, **inject: Any) -> NativeBackend:
    select_backend(args)
    is_child = os.environ.get(_WORKER_ENV) == "1"
    if supervise is None:
        supervise = args.tensor_parallel_size > 1 and not is_child and not inject
    if supervise and args.tensor_parallel_size > 1 and args.tensor_parallel_rank == 0:
        from ..supervisor import TensorParallelConfig, TensorParallelSupervisor
        env = {"POCKETLLM_CHECKPOINT": args.model, "POCKETLLM_TP_SIZE": str(args.tensor_parallel_size),
               "POCKETLLM_BACKEND_OPTIONS": json.dumps(args.backend_options), _WORKER_ENV: "1",
               "POCKETLLM_MODEL_FORMAT": args.model_format, "POCKETLLM_MAX_BATCH_SIZE": str(args.max_batch_size)}
        if args.max_model_len:
            env["POCKETLLM_MAX_MODEL_LEN"] = str(args.max_model_len)
        cfg = TensorParallelConfig(world_size=args.tensor_parallel_size, command=[sys.executable, "-c", _worker_script()],
                                   extra_env=env, ranks=list(range(1, args.tensor_parallel_size)))
        sup = TensorParallelSupervisor(cfg)
        sup.start()
        for k, v in sup.rank_env(0).items():      # rank 0 lives in this process
            os.environ[k] = v
        backend = NativeBackend(args, **inject)
        backend._supervisor = sup                  # kept alive with the backend
        orig_release = backend._release

        def release() -> None:
            orig_release()
            sup.cleanup()

        backend._release = release                 # type: ignore[method-assign]
        backend.prepare()
        sup.wait_ready()
        return backend
    return NativeBackend(args, **inject)
