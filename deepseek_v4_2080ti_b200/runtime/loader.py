"""Build a model runtime from ``EngineArgs``: pick the model family from the checkpoint, shard it
for this rank, open the rank-0 -> workers command channel.

Model strings:
  ``synthetic:qwen-tiny`` / ``synthetic:qwen-27b``  random-init models generated on the device
  a directory with ``config.json`` + safetensors      Qwen-style hybrid FP8 checkpoints
  a ``.gguf`` file or bundle                          MoE families (routed by ``general.architecture``)
"""
from __future__ import annotations

import os
from typing import Any

import torch

from ..models import qwen_hybrid as qh
from ..parallel import tp


class Channel:
    """Rank 0 -> workers command fan-out over the C++ ``CmdChannel`` (unix socket, int32 words)."""

    def __init__(self, base_path: str, rank: int, world: int, timeout_ms: int = 600000):
        from .. import pocketllm_cpp as cpp
        self.world, self.rank = world, rank
        self._ch = cpp.CmdChannel()
        if not self._ch.open(base_path, rank, world, timeout_ms, 50):
            raise RuntimeError(f"command channel could not be opened at {base_path}.cmdsock (rank {rank}/{world})")

    def send(self, op: int, *payload) -> None:
        words = [int(op)]
        for p in payload:
            if isinstance(p, (list, tuple)):
                words.append(len(p))
                words.extend(int(x) for x in p)
            else:
                words.append(int(p))
        if not self._ch.broadcast(words):
            from pocketllm.api.errors import BackendUnavailableError     # 503 to the client: the group is going down
            raise BackendUnavailableError("a worker rank closed its command channel")

    def recv(self):
        w = self._ch.receive(-1)
        if w is None:
            return (0,)                          # rank 0 went away: stop
        op = w[0]
        if op == 3:                              # prefill: slot, chunk, n, tokens...
            return (op, w[1], w[2], list(w[4:4 + w[3]]))
        return tuple(w)



def logprobs_of_row(logits_row: torch.Tensor, token: int, top_n: int) -> dict:
    """fp32 logits [vocab] of one step -> {"logprob": of ``token``, "top": [(id, logprob)] best ``top_n``} under the
    soft-max of the raw logits (before temperature and penalties, as the OpenAI API defines them)."""
    lp = torch.log_softmax(logits_row.float(), -1)
    out = {"logprob": float(lp[int(token)].item()), "top": []}
    if top_n > 0:
        v, i = lp.topk(min(int(top_n), lp.numel()))
        out["top"] = [(int(a), float(b)) for a, b in zip(i.tolist(), v.tolist())]
    return out


class RuntimeAdapter:
    """The surface ``NativeBackend`` drives, over a ``QwenHybridRuntime``."""
    supports_sampling = True
    supports_prefix_cache = True
    speculative_methods: tuple[str, ...] = ()

    def __init__(self, rt: qh.QwenHybridRuntime, max_context: int, eos_token_ids=()):
        self.rt, self.max_context, self.eos_token_ids = rt, max_context, tuple(eos_token_ids)
        # log-probabilities need the whole vocabulary in one place: single-rank runs (a rank of a tensor-parallel group
        # holds a vocabulary shard of the head)
        self.supports_logprobs = getattr(getattr(rt, "comm", None), "world", 1) == 1
        self.vocab_size = int(rt.cfg.vocab_size)
        self.last_cached_tokens = 0
        self._rng: dict[int, torch.Generator] = {}      # per slot: the request's seeded generator
        self._counts: dict[int, torch.Tensor] = {}      # per slot: occurrences of each local vocabulary id
        self._seed_counter = 0

    # ---- sampling state of a slot
    def _sampling(self, slot: int, sp: Any, prompt: list[int] | None):
        from ..ops.sampling import DeviceSampling
        ds = DeviceSampling.from_params(sp)
        if ds is None:
            return None
        if slot not in self._rng:
            g = torch.Generator()
            seed = getattr(sp, "seed", None)
            if seed is None:
                self._seed_counter += 1
                seed = 0x5EED0000 + self._seed_counter
            g.manual_seed(int(seed))
            self._rng[slot] = g
        if ds.has_penalties and slot not in self._counts:
            w = self.rt.w
            n_local = w.lm_head.n
            c = torch.zeros(n_local, dtype=torch.int32, device=self.rt.device)
            if prompt:
                self._count(c, prompt)
            self._counts[slot] = c
        return ds

    def _count(self, c: torch.Tensor, tokens: list[int]) -> None:
        lo = self.rt.w.head_lo
        ids = torch.tensor([t - lo for t in tokens if lo <= t < lo + c.numel()], dtype=torch.int64, device=c.device)
        if ids.numel():
            c.index_add_(0, ids, torch.ones_like(ids, dtype=torch.int32))

    def _draws(self, slots: list[int]) -> torch.Tensor:
        return torch.cat([torch.rand(1, generator=self._rng[s]) for s in slots])

    def allocate(self) -> int:
        return self.rt.allocate()

    def free(self, slot: int) -> None:
        self.rt.free(slot)
        self._rng.pop(slot, None)
        self._counts.pop(slot, None)

    def token_logprobs(self, slot: int, token: int, top_n: int) -> dict:
        """Of the token just produced for ``slot`` (after ``prefill_tokens`` or a single-slot ``decode_tokens``)."""
        return logprobs_of_row(self.rt.last_logits[-1], token, top_n)

    def _check_collectives(self) -> None:
        """Multi-rank only: the step's tokens are on the host, so the kernels have finished - read the error word.
        A bounded wait that expired surfaces here as ``CollectiveTimeoutError`` (see ``recover``)."""
        chk = getattr(self.rt.comm, "check", None)
        if chk is not None and self.rt.comm.world > 1:
            chk()

    def recover(self) -> None:
        """Collective: every rank calls it after any rank saw ``CollectiveTimeoutError``; afterwards the collectives
        run on the library path and the slots must be filled again (their state may hold half a step)."""
        self.rt.recover_collectives()

    def prefill_tokens(self, slot: int, prompt: list[int], chunk: int, sp: Any) -> int:
        tok = self._prefill_tokens(slot, prompt, chunk, sp)
        self._check_collectives()
        return tok

    def decode_tokens(self, slots: list[int], toks: list[int], sp: Any) -> list[int]:
        """``sp``: one SamplingParams for the whole batch, a list with one per slot, or None (greedy)."""
        out = self._decode_tokens(slots, toks, sp)
        self._check_collectives()
        return out

    def _prefill_tokens(self, slot: int, prompt: list[int], chunk: int, sp: Any) -> int:
        ids = torch.tensor(prompt, dtype=torch.int32).pin_memory().to(self.rt.device, non_blocking=True)
        ds = self._sampling(slot, sp, prompt)
        before = self.rt.prefill_tokens_computed
        if ds is None:
            tok = int(self.rt.prefill(slot, ids, chunk, host_tokens=prompt).item())
        else:
            counts = self._counts[slot][None] if slot in self._counts else None
            tok = int(self.rt.prefill(slot, ids, chunk, host_tokens=prompt, sampling=ds, u=self._draws([slot]),
                                      counts=counts).item())
            if slot in self._counts:
                self._count(self._counts[slot], [tok])
        self.last_cached_tokens = len(prompt) - (self.rt.prefill_tokens_computed - before)
        return tok

    def _decode_tokens(self, slots: list[int], toks: list[int], sp: Any) -> list[int]:
        t = torch.tensor(toks, dtype=torch.int32, device=self.rt.device)
        sps = sp if isinstance(sp, (list, tuple)) else [sp] * len(slots)
        dss = [self._sampling(s, p, None) for s, p in zip(slots, sps)]
        if all(d is None for d in dss):
            return [int(x) for x in self.rt.decode(slots, t).tolist()]
        if all(d == dss[0] for d in dss):
            counts = torch.stack([self._counts[s] for s in slots]) if all(s in self._counts for s in slots) and dss[0].has_penalties else None
            out = [int(x) for x in self.rt.decode(slots, t, sampling=dss[0], u=self._draws(slots), counts=counts).tolist()]
        else:
            # mixed settings in one batch: one forward pass, then one draw per row from the step's logits
            greedy = self.rt.decode(slots, t).tolist()
            logits = next(e for e in self.rt._graphs.values() if e["buf"]["ids"].numel() == len(slots))["buf"]["logits"]
            out = []
            for r, (s, d) in enumerate(zip(slots, dss)):
                if d is None:
                    out.append(int(greedy[r]))
                else:
                    c = self._counts[s][None] if s in self._counts else None
                    out.append(int(self.rt._next_tokens(logits[r:r + 1], d, self._draws([s]), c).item()))
        for s, tok in zip(slots, out):
            if s in self._counts:
                self._count(self._counts[s], [tok])
        return out

    def generate_batch(self, prompts, max_new, eos_ids, max_batch):
        """Greedy continuous batching: admit up to ``max_batch`` sequences, decode them together."""
        import time
        results: list[Any] = [None] * len(prompts)
        pending = list(range(len(prompts)))[::-1]
        active: dict[int, dict] = {}
        while pending or active:
            while pending and len(active) < min(max_batch, self.rt.max_slots):
                i = pending.pop()
                t0 = time.perf_counter()
                slot = self.rt.allocate()
                first = self.prefill_tokens(slot, prompts[i], 8192, None)
                active[i] = {"slot": slot, "out": [first], "t0": t0, "t1": time.perf_counter()}
            done = [i for i, a in active.items() if a["out"][-1] in eos_ids or len(a["out"]) >= max_new[i]]
            for i in done:
                a = active.pop(i)
                self.rt.free(a["slot"])
                eos = a["out"][-1] in eos_ids
                ids = a["out"][:-1] if eos else a["out"]
                now = time.perf_counter()
                results[i] = (ids, "stop" if eos else "length",
                              {"prefill_seconds": a["t1"] - a["t0"], "decode_seconds": now - a["t1"],
                               "total_seconds": now - a["t0"], "ttft_seconds": a["t1"] - a["t0"]})
            if active:
                order = list(active)
                nxt = self.decode_tokens([active[i]["slot"] for i in order], [active[i]["out"][-1] for i in order], None)
                for i, t in zip(order, nxt):
                    active[i]["out"].append(t)
        return results

    def stats(self) -> dict:
        return {"kv_blocks_free": len(self.rt.free_blocks), "kv_blocks_total": self.rt.num_blocks - 1,
                "slots_free": len(self.rt.free_slots)}


class SpecRuntimeAdapter(RuntimeAdapter):
    """Greedy speculative decoding behind the same surface: a decode call hands out the next token of the last
    verified block and runs a new draft / verify round only when that block is used up.  Worker ranks mirror the same
    calls, so their rounds stay in step with rank 0's."""
    supports_sampling = False
    supports_prefix_cache = False

    def __init__(self, rt, spec, max_context: int, eos_token_ids=()):
        super().__init__(rt, max_context, eos_token_ids)
        self.spec = spec
        self.speculative_methods = (spec.method,)

    def allocate(self) -> int:
        return self.spec.allocate()

    def free(self, slot: int) -> None:
        self.spec.free(slot)

    def prefill_tokens(self, slot: int, prompt: list[int], chunk: int, sp) -> int:
        ids = torch.tensor(prompt, dtype=torch.int32).pin_memory().to(self.rt.device, non_blocking=True)
        tok = self.spec.prefill(slot, ids, chunk, host_tokens=prompt)
        self.spec.seqs[slot].queue = []
        self.last_cached_tokens = 0
        self._check_collectives()
        return tok

    def decode_tokens(self, slots: list[int], toks: list[int], sp) -> list[int]:
        out = []
        for s in slots:
            q = self.spec.seqs[s].queue
            if not q:
                q.extend(self.spec.step(s))
                self._check_collectives()
            out.append(q.pop(0))
        return out

    def stats(self) -> dict:
        c = self.spec.stats
        return {"spec_rounds": c.rounds, "spec_drafted": c.drafted, "spec_accepted": c.accepted,
                "spec_accept_rate": round(c.accept_rate, 4), "spec_tokens_per_pass": round(c.tokens_per_pass, 3)}


class CppRuntimeAdapter:
    """The same surface over the native C++ engine (``pocketllm_engine_cpp.QwenEngine``): safetensors checkpoints,
    one GPU, greedy decoding; batches go through the C++ continuous-batching scheduler."""
    supports_sampling = False
    supports_prefix_cache = False
    speculative_methods: tuple[str, ...] = ()

    def __init__(self, checkpoint_dir: str, device_index: int, max_context: int, max_slots: int, chunk: int = 8192,
                 eos_token_ids=()):
        from .. import pocketllm_engine_cpp as cpp
        opt = cpp.QwenEngineOptions()
        opt.max_slots, opt.max_context, opt.prefill_chunk, opt.device = max_slots, max_context, chunk, device_index
        opt.eos_tokens = list(eos_token_ids)
        self.eng = cpp.QwenEngine(checkpoint_dir, opt)
        self.max_context, self.eos_token_ids = max_context, tuple(eos_token_ids)
        self.vocab_size = int(getattr(self.eng, "vocab_size", 0) or 0)
        self.last_cached_tokens = 0
        self._sched_batch = 0

    def allocate(self) -> int:
        s = self.eng.allocate_slot()
        if s < 0:
            raise RuntimeError("no free slot")
        return s

    def free(self, slot: int) -> None:
        self.eng.free_slot(slot)

    def prefill_tokens(self, slot: int, prompt: list[int], chunk: int, sp: Any) -> int:
        return int(self.eng.prefill(slot, [int(t) for t in prompt]))

    def decode_tokens(self, slots: list[int], toks: list[int], sp: Any) -> list[int]:
        return [int(t) for t in self.eng.decode_step(list(slots), [int(t) for t in toks])]

    def generate_batch(self, prompts, max_new, eos_ids, max_batch):
        if self._sched_batch != max_batch:
            self.eng.stop_scheduler()
            self.eng.start_scheduler(max(1, min(max_batch, self.eng.max_slots)), 8192)
            self._sched_batch = max_batch
        ids = [self.eng.submit([int(t) for t in p], int(n), True) for p, n in zip(prompts, max_new)]
        out = []
        for i in ids:
            r = self.eng.wait(i, -1)
            toks = list(r.tokens)
            eos = bool(toks) and toks[-1] in eos_ids
            out.append((toks[:-1] if eos else toks, "stop" if eos else r.finish_reason,
                        {"prefill_seconds": r.prefill_seconds, "decode_seconds": r.decode_seconds,
                         "total_seconds": r.queue_seconds + r.prefill_seconds + r.decode_seconds,
                         "ttft_seconds": r.queue_seconds + r.prefill_seconds}))
        return out

    def stats(self) -> dict:
        st = self.eng.stats()
        return {"kv_blocks_total": self.eng.total_blocks, "kernel_launches": st.kernel_launches, "weight_bytes": st.weight_bytes}


class GgufRuntimeAdapter:
    """The same surface over a GGUF family runtime (``models.registry`` builds it: GQA-MoE with paged slots, or the
    one-sequence MLA runtime): greedy decoding, sequences admitted up to the runtime's slot count."""
    supports_sampling = False
    supports_prefix_cache = False
    speculative_methods: tuple[str, ...] = ()

    def __init__(self, rt, max_context: int, max_slots: int, device, eos_token_ids=()):
        self.rt, self.max_context, self.device = rt, max_context, device
        self.max_slots = 1 if getattr(rt, "single_sequence", False) else max(1, int(max_slots))
        self.eos_token_ids = tuple(eos_token_ids)
        self.last_cached_tokens = 0
        self._active: set[int] = set()
        # runtimes that leave the step's full-vocabulary logits in ``last_logits`` ([rows, vocab] fp32, one row per
        # sequence of the step) can be sampled from: temperature / top-k / top-p / min-p / penalties on the device
        self.supports_sampling = bool(getattr(rt, "exposes_logits", False))
        self.supports_logprobs = self.supports_sampling
        cfg = getattr(rt, "cfg", None)
        self.vocab_size = int(getattr(cfg, "vocab_size", 0) or getattr(cfg, "vocab", 0) or 0)
        self._rng: dict[int, torch.Generator] = {}
        self._counts: dict[int, torch.Tensor] = {}
        self._seed_counter = 0

    def allocate(self) -> int:
        if len(self._active) >= self.max_slots:
            raise RuntimeError("no free slot")
        slot = int(self.rt.allocate())
        self._active.add(slot)
        return slot

    def free(self, slot: int) -> None:
        self._active.discard(slot)
        self._rng.pop(slot, None)
        self._counts.pop(slot, None)
        self.rt.free(slot)

    def token_logprobs(self, slot: int, token: int, top_n: int) -> dict:
        """Of the token just produced for ``slot`` (after ``prefill_tokens`` or a single-slot ``decode_tokens``)."""
        return logprobs_of_row(self.rt.last_logits[-1], token, top_n)

    # ---- sampling from the step's logits
    def _sampling(self, slot: int, sp: Any, prompt: list[int] | None):
        from ..ops.sampling import DeviceSampling
        ds = DeviceSampling.from_params(sp) if sp is not None else None
        if ds is None or not self.supports_sampling:
            return None
        if slot not in self._rng:
            g = torch.Generator()
            seed = getattr(sp, "seed", None)
            if seed is None:
                self._seed_counter += 1
                seed = 0x5EED0000 + self._seed_counter
            g.manual_seed(int(seed))
            self._rng[slot] = g
        if ds.has_penalties and slot not in self._counts:
            c = torch.zeros(self.rt.last_logits.shape[-1], dtype=torch.int32, device=self.device)
            self._counts[slot] = c
            if prompt:
                self._count(slot, prompt)
        return ds

    def _count(self, slot: int, tokens: list[int]) -> None:
        c = self._counts[slot]
        ids = torch.tensor([t for t in tokens if 0 <= t < c.numel()], dtype=torch.int64, device=c.device)
        if ids.numel():
            c.index_add_(0, ids, torch.ones_like(ids, dtype=torch.int32))

    def _draw_row(self, slot: int, row: int, ds) -> int:
        from ..ops import sampling
        u = torch.rand(1, generator=self._rng[slot]).to(self.device)
        counts = self._counts[slot][None] if slot in self._counts else None
        tok = int(sampling.sample(self.rt.last_logits[row:row + 1].contiguous(), ds, u, counts=counts).item())
        if slot in self._counts:
            self._count(slot, [tok])
        return tok

    def prefill_tokens(self, slot: int, prompt: list[int], chunk: int, sp: Any) -> int:
        ids = torch.tensor([int(t) for t in prompt], dtype=torch.int32).to(self.device)
        greedy = int(self.rt.prefill(slot, ids, int(chunk) if chunk else 4096).item())
        ds = self._sampling(slot, sp, prompt)
        return greedy if ds is None else self._draw_row(slot, self.rt.last_logits.shape[0] - 1, ds)

    def decode_tokens(self, slots: list[int], toks: list[int], sp: Any) -> list[int]:
        if getattr(self.rt, "single_sequence", False):
            assert len(slots) == 1
        t = torch.tensor([int(x) for x in toks], dtype=torch.int32).to(self.device)
        greedy = [int(x) for x in self.rt.decode(list(slots), t).reshape(-1).tolist()]
        sps = sp if isinstance(sp, (list, tuple)) else [sp] * len(slots)
        out = []
        for row, (s, p) in enumerate(zip(slots, sps)):
            ds = self._sampling(s, p, None)
            out.append(greedy[row] if ds is None else self._draw_row(s, row, ds))
        return out

    def generate_batch(self, prompts, max_new, eos_ids, max_batch):
        import time
        results: list[Any] = [None] * len(prompts)
        pending = list(range(len(prompts)))[::-1]
        active: dict[int, dict] = {}
        width = max(1, min(int(max_batch), self.max_slots))
        while pending or active:
            while pending and len(active) < width:
                i = pending.pop()
                t0 = time.perf_counter()
                slot = self.allocate()
                first = self.prefill_tokens(slot, prompts[i], 4096, None)
                active[i] = {"slot": slot, "out": [first], "t0": t0, "t1": time.perf_counter()}
            for i in [i for i, a in active.items() if a["out"][-1] in eos_ids or len(a["out"]) >= max_new[i]]:
                a = active.pop(i)
                self.free(a["slot"])
                eos = a["out"][-1] in eos_ids
                now = time.perf_counter()
                results[i] = (a["out"][:-1] if eos else a["out"], "stop" if eos else "length",
                              {"prefill_seconds": a["t1"] - a["t0"], "decode_seconds": now - a["t1"],
                               "total_seconds": now - a["t0"], "ttft_seconds": a["t1"] - a["t0"]})
            if active:
                order = list(active)
                if getattr(self.rt, "single_sequence", False) or len(order) == 1:
                    nxt = [self.decode_tokens([active[i]["slot"]], [active[i]["out"][-1]], None)[0] for i in order]
                else:
                    nxt = self.decode_tokens([active[i]["slot"] for i in order], [active[i]["out"][-1] for i in order], None)
                for i, t in zip(order, nxt):
                    active[i]["out"].append(t)
        return results

    def stats(self) -> dict:
        out = {"slots_free": self.max_slots - len(self._active), "slots_total": self.max_slots}
        inner = getattr(self.rt, "stats", None)
        if callable(inner):                                  # speculation / swap counters of runtimes that keep them
            try:
                got = inner()
            except Exception:
                got = None
            if isinstance(got, dict):
                out.update({k: v for k, v in got.items() if isinstance(v, (int, float))})
        return out


def _is_gguf(model: str) -> bool:
    return model.endswith(".gguf") or (os.path.isdir(model) and any(f.endswith(".gguf") for f in os.listdir(model)))


def _device(args) -> torch.device:
    if args.device is not None:
        return torch.device(args.device if isinstance(args.device, str) else f"cuda:{args.device}")
    return torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))


def _load_host(args):
    """The Qwen-style hybrid on the host (``device="cpu"``): fp32 oracle, one rank, every drafter
    (``runtime/host_runtime.py``)."""
    from pocketllm.api.errors import ConfigurationError
    from pocketllm.backends.native_backend import NullChannel
    from .host_runtime import build_host_adapter
    world, rank = args.tensor_parallel_size, args.tensor_parallel_rank
    channel = None
    if world > 1:
        # replicated ranks: every rank holds the whole (small) model and mirrors rank 0's commands over the command
        # channel - no collective is needed, but the supervisor, the fan-out and the worker loop run as on the GPUs
        base = os.environ.get("POCKETLLM_NCCL_ID_PATH") or f"/tmp/pocketllm-{os.environ.get('MASTER_PORT', '0')}"
        channel = Channel(base, rank, world)
    model = args.model
    if model.startswith("synthetic:"):
        if "tiny" not in model:
            raise ConfigurationError("the host path generates only the tiny synthetic model")
        cfg = qh.QwenHybridConfig.tiny()
        state = qh.synth_state(cfg, 0, "cpu", std=0.05)
    else:
        from ..formats import safetensors_io
        cfg = qh.QwenHybridConfig.from_json(args.config_path or os.path.join(args.checkpoint_dir, "config.json"))
        state = safetensors_io.read_checkpoint(args.checkpoint_dir)
    max_ctx = args.max_model_len or 2048
    return build_host_adapter(args, cfg, state, max_ctx, max(1, args.max_batch_size)), None, channel or NullChannel()


def load_runtime(args):
    """Returns (adapter, chat-template family or None, command channel)."""
    world, rank = args.tensor_parallel_size, args.tensor_parallel_rank
    spec_method = getattr(args, "speculative_method", None)
    if str(args.device or "") == "cpu" and not _is_gguf(args.model):
        return _load_host(args)
    if spec_method and spec_method not in ("mtp", "ngram"):
        # refuse rather than decode without it: the learned block drafters run on the host path only (device="cpu")
        from pocketllm.api.errors import ConfigurationError
        raise ConfigurationError(f"speculative_method={spec_method!r} is not implemented on the GPU (available there: "
                                 "'mtp' with a checkpoint that carries the head, 'ngram' prompt lookup; device='cpu' "
                                 "serves 'dspark' and 'dflash2' from the host statements)")
    if spec_method and (_is_gguf(args.model) or getattr(args, "backend", "auto") == "cpp"):
        from pocketllm.api.errors import ConfigurationError
        raise ConfigurationError("speculative_method is served by the Qwen-style hybrid runtime only")
    dev = _device(args)
    if dev.type == "cuda":
        torch.cuda.set_device(dev)
    elif not _is_gguf(args.model):
        from pocketllm.api.errors import ConfigurationError
        raise ConfigurationError(f"device {dev} cannot run this model")
    comm = None
    channel = None
    if world > 1:
        os.environ.setdefault("RANK", str(rank))
        os.environ.setdefault("WORLD_SIZE", str(world))
        os.environ.setdefault("LOCAL_RANK", str(dev.index or 0))
        tp.init_distributed("nccl")
        base = os.environ.get("POCKETLLM_NCCL_ID_PATH") or f"/tmp/pocketllm-{os.environ.get('MASTER_PORT', '0')}"
        channel = Channel(base, rank, world)
    model = args.model
    max_ctx = args.max_model_len or 8192 + 512
    slots = max(1, args.max_batch_size)
    chunk = int(args.prefill_chunk_tokens or 8192)

    def make_comm(hidden: int):
        """Peer-memory communicator (fused GEMM + collective kernels over NVLink) sized for one prefill chunk of hidden
        states; POCKETLLM_TP_COMM=nccl selects the library baseline."""
        if world <= 1:
            return None
        if os.environ.get("POCKETLLM_TP_COMM", "peer") == "nccl":
            return tp.TPComm()
        return tp.PeerComm(slot_elems=max(1 << 20, min(chunk, max_ctx) * int(hidden)))
    if _is_gguf(model):
        # MoE families from GGUF: the family registry reads the metadata, validates the tensor inventory and builds the
        # runtime (attention heads and experts sharded over the ranks); greedy decoding through the slot interface
        from ..encoding import family_from_architecture
        from ..formats.gguf import read_bundle
        from ..models import registry
        from pocketllm.backends.native_backend import NullChannel
        bundle = read_bundle(model)
        spec = registry.detect(bundle)
        comm = make_comm(int(bundle.metadata.get(f"{spec.architecture}.embedding_length", 8192)))
        report = spec.validate(bundle)
        if not report.ok:
            raise ValueError(f"{model}: missing {report.missing[:4]} unsupported {list(report.unsupported)[:4]}")
        if dev.type != "cuda" and spec.architecture != "deepseek4":
            from pocketllm.api.errors import ConfigurationError
            raise ConfigurationError(f"the {spec.architecture} family needs a GPU; only deepseek4 files run on the host")
        # family-specific runtime options travel as backend options (deepseek4: dspark=..., flashmemory=..., kv_swap_chunks=...)
        extra = {k: v for k, v in (getattr(args, "backend_options", None) or {}).items()
                 if k in ("dspark", "dspark_block", "dspark_target_layers", "spec_gate", "flashmemory", "flashmemory_ensemble",
                          "kv_swap_chunks", "kv_swap_chunk_entries")} if spec.architecture == "deepseek4" else {}
        _, rt = spec.build_runtime(bundle, dev, rank, world, comm, max_slots=slots, max_context=max_ctx, **extra)
        try:
            family = family_from_architecture(spec.architecture)
        except ValueError:
            family = None
        return GgufRuntimeAdapter(rt, max_ctx, slots, dev), family, channel or NullChannel()
    if getattr(args, "backend", "auto") == "cpp" and world == 1 and not model.startswith("synthetic:"):
        from pocketllm.backends.native_backend import NullChannel
        return CppRuntimeAdapter(args.checkpoint_dir, dev.index or 0, max_ctx, slots,
                                 args.prefill_chunk_tokens or 8192), None, NullChannel()
    if not model.startswith("synthetic:"):
        # MLA + routed-expert checkpoints (DeepSeek inference layout: FP8 block-128 or bf16 dense matrices, FP4 or
        # bf16 experts, config.json in the dim / n_layers / n_routed_experts spelling) as safetensors shards
        import json as _json
        from ..models.mla_moe import MlaMoeConfig
        cfg_path = args.config_path or os.path.join(args.checkpoint_dir, "config.json")
        try:
            with open(cfg_path) as f:
                raw_cfg = _json.load(f)
        except (OSError, ValueError):
            raw_cfg = None
        if MlaMoeConfig.is_mla_moe_json(raw_cfg):
            from ..formats import safetensors_io
            from ..models import mla_moe_gpu as mg
            from ..models.registry import _MlaSlotAdapter
            from pocketllm.backends.native_backend import NullChannel
            mcfg = MlaMoeConfig.from_json(raw_cfg)
            comm = make_comm(mcfg.hidden_size)
            w = mg.MlaMoeGpuWeights(mcfg, safetensors_io.read_checkpoint(args.checkpoint_dir), dev, rank, world,
                                    dense_fp8=str(raw_cfg.get("dtype", "bf16")).lower() == "fp8")
            if slots > 1:
                rt = mg.MlaMoeBatchRuntime(mcfg, w, max_slots=slots, max_context=max_ctx, comm=comm)
            else:
                rt = _MlaSlotAdapter(mg.MlaMoeGpuRuntime(mcfg, w, max_context=max_ctx, comm=comm))
            return GgufRuntimeAdapter(rt, max_ctx, slots, dev), "deepseek_v4", channel or NullChannel()
    if model.startswith("synthetic:"):
        name = model.split(":", 1)[1]
        cfg = qh.QwenHybridConfig.tiny() if name in ("qwen-tiny", "tiny") else qh.QwenHybridConfig.config2()
        state = qh.synth_state(cfg, 0, dev, std=0.05 if "tiny" in name else 0.02)
    else:
        cfg_path = args.config_path or os.path.join(args.checkpoint_dir, "config.json")
        cfg = qh.QwenHybridConfig.from_json(cfg_path)
        from ..formats import safetensors_io
        state = safetensors_io.read_checkpoint(args.checkpoint_dir)
    weights = qh.QwenHybridWeights(cfg, state, dev, rank, world)
    comm = make_comm(cfg.hidden_size)
    spec_k = int(getattr(args, "speculative_tokens", 1) or 1) if spec_method else 0
    rt = qh.QwenHybridRuntime(cfg, weights, max_slots=slots, max_context=max_ctx + (spec_k + 1 if spec_k else 0), comm=comm,
                              attention_window=int(getattr(args, "attention_window", 0) or 0),
                              attention_sink_tokens=int(getattr(args, "attention_sink_tokens", 0) or 0),
                              kv_cache_dtype=getattr(args, "kv_cache_dtype", "auto") or "auto")
    if getattr(args, "enable_prefix_caching", False):
        # snapshot points every 2048 tokens: a snapshot copies the recurrent state of every Gated-DeltaNet layer
        # (~100 MB at the 27B shape), and chunks of 2048 keep the prefill GEMMs at full efficiency
        rt.enable_prefix_cache(interval=2048, max_entries=4)
    from pocketllm.backends.native_backend import NullChannel
    if spec_method:
        if getattr(args, "enable_prefix_caching", False):
            from pocketllm.api.errors import ConfigurationError
            raise ConfigurationError("speculative decoding and prefix caching cannot be combined")
        from ..models.qwen_spec import QwenSpeculator
        try:
            spec = QwenSpeculator(rt, k=spec_k, method=spec_method)
        except ValueError as exc:
            from pocketllm.api.errors import ConfigurationError
            raise ConfigurationError(str(exc)) from exc
        return SpecRuntimeAdapter(rt, spec, max_ctx), None, channel or NullChannel()
    return RuntimeAdapter(rt, max_ctx), None, channel or NullChannel()
