"""The single engine backend: drives the sm_100a runtimes in ``deepseek_v4_2080ti_b200``.

Replaces both of the reference's adapters (``TorchBackend`` pocketllm/backends/torch_backend.py:33-397
and ``CppBackend`` pocketllm/backends/cpp_backend.py:147-844).  The contract kept from them:
rank 0 owns the request loop and, before every local prefill/decode, fans the same command out
to the worker ranks so all ranks enter the same collectives in the same order.
A ``runtime`` / ``tokenizer`` / ``channel`` can be injected, which is how the CPU tests exercise
this file with fakes.
"""
from __future__ import annotations

import time
from typing import Any, Iterable, Iterator

from ..api.errors import BackendUnavailableError, ConfigurationError, UnsupportedFeatureError
from ..api.types import (BackendCapabilities, EngineArgs, GenerationRequest, GenerationResult, TimingMetrics,
                         TokenEvent, Usage)
from ..protocol.chat import held_back_suffix, truncate_at_stop
from ..protocol.prompt import TokenizerHandle
from .base import BackendBase

OP_STOP, OP_ALLOC, OP_FREE, OP_PREFILL, OP_DECODE, OP_SAMPLING, OP_RECOVER = 0, 1, 2, 3, 4, 5, 6


def _is_collective_timeout(exc: BaseException) -> bool:
    # by name: this module must stay importable without torch / the kernel package
    return type(exc).__name__ == "CollectiveTimeoutError"


class NullChannel:
    """Command fan-out for a single-rank engine: nothing to send."""
    world = 1

    def send(self, op: int, *payload) -> None:
        pass

    def recv(self):  # pragma: no cover - never called at world 1
        raise BackendUnavailableError("no command channel")


_Q = 1_000_000          # sampling settings travel as int32 words: fixed point, 6 decimals


def _with_seed(sp):
    import dataclasses
    import random
    seed = random.getrandbits(31) if sp.seed is None else int(sp.seed) & 0x7FFFFFFF    # what fits one channel word
    return dataclasses.replace(sp, seed=seed)


def _encode_sampling(sp) -> list[int]:
    q = lambda x: int(round(float(x or 0.0) * _Q))
    return [q(sp.temperature), int(sp.top_k or 0), q(sp.top_p if sp.top_p is not None else 1.0), q(sp.min_p),
            q(sp.repetition_penalty), q(sp.presence_penalty), q(sp.frequency_penalty), int(sp.seed) & 0x7FFFFFFF]


def _decode_sampling(w) -> Any:
    from types import SimpleNamespace
    return SimpleNamespace(temperature=w[0] / _Q, top_k=int(w[1]), top_p=w[2] / _Q, min_p=w[3] / _Q,
                           repetition_penalty=w[4] / _Q, presence_penalty=w[5] / _Q, frequency_penalty=w[6] / _Q,
                           seed=int(w[7]))


class NativeBackend(BackendBase):
    name = "b200"

    def __init__(self, args: EngineArgs, runtime: Any = None, tokenizer: TokenizerHandle | None = None,
                 channel: Any = None):
        super().__init__(args)
        self.runtime = runtime
        self.tokenizer = tokenizer
        self.channel = channel or NullChannel()
        self.family: str | None = None
        self._stats = {"requests": 0, "prompt_tokens": 0, "completion_tokens": 0}
        if runtime is not None:
            self._ready = True
            if self.tokenizer is None:
                self.tokenizer = TokenizerHandle(None, "bytes")

    # ---- loading
    def _load(self) -> None:
        if self.runtime is not None:
            return
        try:
            from deepseek_v4_2080ti_b200.runtime import loader
        except Exception as exc:
            raise BackendUnavailableError(f"native engine cannot be imported: {exc}") from exc
        self.runtime, self.family, self.channel = loader.load_runtime(self.args)
        if self.tokenizer is None:
            self.tokenizer = TokenizerHandle.load(self.args.tokenizer_path or self.args.checkpoint_dir)

    def _release(self) -> None:
        try:
            if self.channel.world > 1 and self.args.tensor_parallel_rank == 0:
                self.channel.send(OP_STOP)
        except Exception:
            pass
        self.runtime = None

    def capabilities(self) -> BackendCapabilities:
        rt = self.runtime
        return BackendCapabilities(
            name=self.name, models=("qwen3_5", "minimax_m2", "deepseek_v4", "glm_dsa"),
            model_formats=("safetensors", "gguf", "synthetic"), devices=("cuda:sm_100a",),
            supports_batch=True, supports_streaming=True, supports_cancellation=True,
            supports_prefix_caching=bool(getattr(rt, "supports_prefix_cache", False)),
            supports_logprobs=bool(getattr(rt, "supports_logprobs", False)), supports_structured_outputs=False,
            supports_speculative_decoding=tuple(getattr(rt, "speculative_methods", ())),
            details={"tensor_parallel_size": self.args.tensor_parallel_size})

    def _health_details(self) -> dict:
        d = dict(self._stats)
        stats = getattr(self.runtime, "stats", None)
        if callable(stats):
            d.update(stats())
        return d

    # ---- helpers
    def _tokens(self, req: GenerationRequest) -> list[int]:
        if req.prompt_tokens is not None:
            return req.prompt_tokens
        return self.tokenizer.encode(req.prompt or "")

    def _check_features(self, req: GenerationRequest) -> None:
        sp = req.sampling_params
        if (sp.logprobs or sp.top_logprobs) and not getattr(self.runtime, "supports_logprobs", False):
            raise UnsupportedFeatureError("this runtime does not report log-probabilities")
        if sp.response_format and sp.response_format.get("type") not in (None, "text") \
                and not req.metadata.get("response_format_in_prompt"):
            # chat requests carry the schema as an instruction in the prompt; a raw completion has nowhere to put it
            raise UnsupportedFeatureError("response_format needs a chat request: the schema is given to the model as an instruction")
        if not sp.greedy and not getattr(self.runtime, "supports_sampling", False):
            raise UnsupportedFeatureError("this runtime only supports greedy decoding (temperature 0)")
        limit = self.args.max_model_len or getattr(self.runtime, "max_context", None)
        toks = self._tokens(req)
        n = len(toks)
        # token ids index embedding and count tables on the device: refuse anything the model has no row for
        vocab = int(getattr(self.runtime, "vocab_size", 0) or 0)
        try:
            lo, hi = (min(toks), max(toks)) if toks else (0, 0)          # two C-speed passes, also for 64K-token prompts
        except TypeError:
            lo, hi = -1, -1
        if not isinstance(lo, int) or not isinstance(hi, int) or lo < 0 or hi > 0x7FFFFFFF or (vocab and hi >= vocab):
            bad = next((t for t in toks if not isinstance(t, int) or t < 0 or t > 0x7FFFFFFF or (vocab and t >= vocab)), lo)
            raise ConfigurationError(f"prompt holds {bad!r}, which is not a token id of this model"
                                     + (f" (vocabulary {vocab})" if vocab else ""))
        if limit and n + 1 > limit:
            raise ConfigurationError(f"prompt of {n} tokens does not fit max_model_len {limit}")

    def _eos_ids(self) -> set[int]:
        ids = set(getattr(self.runtime, "eos_token_ids", ()) or ())
        if self.tokenizer is not None and self.tokenizer.eos_token_id is not None:
            ids.add(int(self.tokenizer.eos_token_id))
        return ids

    # ---- the serial request loop (rank 0)
    def _run_one(self, req: GenerationRequest, on_token=None) -> GenerationResult:
        self._require_open()
        self.prepare()
        self._check_features(req)
        sp = req.sampling_params
        prompt = self._tokens(req)
        limit = self.args.max_model_len or getattr(self.runtime, "max_context", None)
        max_new = sp.max_tokens if not limit else max(1, min(sp.max_tokens, limit - len(prompt)))
        eos = self._eos_ids()
        chunk = self.args.prefill_chunk_tokens or 8192
        rt, ch = self.runtime, self.channel
        self._begin(req.request_id)
        t0 = time.perf_counter()
        with self._lock:
            ch.send(OP_ALLOC)
            slot = rt.allocate()
            try:
                if not sp.greedy:
                    # worker ranks take part in the sampled draw (candidate gather over the vocabulary shards) and
                    # must use the same settings and the same random stream: the seed is fixed here
                    sp = _with_seed(sp)
                    ch.send(OP_SAMPLING, slot, *_encode_sampling(sp))
                out: list[int] = []
                recovered = False
                want_lp = bool(sp.logprobs or sp.top_logprobs)
                top_n = int(sp.top_logprobs or 0)
                lps: list[dict] = []

                def step(fn):
                    """Run one prefill / decode; if a peer-memory collective timed out, re-synchronise the ranks on
                    the library path and rebuild the sequence (prompt + tokens so far) there, once per request."""
                    nonlocal slot, recovered
                    try:
                        return fn()
                    except Exception as exc:
                        if recovered or not _is_collective_timeout(exc) or not hasattr(rt, "recover"):
                            raise
                    recovered = True
                    self._stats["collective_recoveries"] = self._stats.get("collective_recoveries", 0) + 1
                    ch.send(OP_RECOVER)
                    rt.recover()
                    ch.send(OP_FREE, slot)
                    rt.free(slot)
                    ch.send(OP_ALLOC)
                    slot = rt.allocate()
                    if not sp.greedy:
                        ch.send(OP_SAMPLING, slot, *_encode_sampling(sp))
                    history = prompt + out
                    ch.send(OP_PREFILL, slot, chunk, history)
                    return rt.prefill_tokens(slot, history, chunk, sp)

                def first():
                    ch.send(OP_PREFILL, slot, chunk, prompt)
                    return rt.prefill_tokens(slot, prompt, chunk, sp)

                tok = step(first)
                if want_lp:
                    lps.append(rt.token_logprobs(slot, tok, top_n))
                t1 = time.perf_counter()
                text_done = ""
                finish = "length"
                while True:
                    out.append(tok)
                    if tok in eos:
                        out.pop()
                        finish = "stop"
                        break
                    if sp.stop:
                        text = self.tokenizer.decode(out)
                        cut, hit = truncate_at_stop(text, sp.stop)
                        if hit:
                            text_done = cut
                            finish = "stop"
                            break
                    if on_token is not None:
                        on_token(tok, out)
                    if len(out) >= max_new:
                        break
                    self._check_cancel(req.request_id)
                    def nxt(tok=tok):
                        ch.send(OP_DECODE, slot, tok)
                        return rt.decode_tokens([slot], [tok], sp)[0]

                    tok = step(nxt)
                    if want_lp:
                        lps.append(rt.token_logprobs(slot, tok, top_n))
                t2 = time.perf_counter()
            finally:
                ch.send(OP_FREE, slot)
                rt.free(slot)
                self._end(req.request_id)
        text = text_done if (finish == "stop" and sp.stop and text_done) else self.tokenizer.decode(out)
        if sp.stop and not text_done:
            text, _ = truncate_at_stop(text, sp.stop)
        usage = Usage(len(prompt), len(out), int(getattr(rt, "last_cached_tokens", 0) or 0))
        n_dec = max(1, len(out) - 1)
        timings = TimingMetrics(prefill_seconds=t1 - t0, decode_seconds=t2 - t1, total_seconds=t2 - t0,
                                ttft_seconds=t1 - t0, tpot_seconds=(t2 - t1) / n_dec)
        self._stats["requests"] += 1
        self._stats["prompt_tokens"] += usage.prompt_tokens
        self._stats["completion_tokens"] += usage.completion_tokens
        logprobs = None
        if want_lp:
            # one entry per kept token (an end-of-sequence token that was cut has none)
            logprobs = [dict(e, token_id=t, token=self.tokenizer.decode([t])) for t, e in zip(out, lps)]
            for e in logprobs:
                e["top_logprobs"] = [{"token_id": i, "token": self.tokenizer.decode([i]), "logprob": v} for i, v in e.pop("top", [])]
        return GenerationResult(req.request_id, out, text, finish, usage, timings, logprobs=logprobs,
                                metadata={"throughput": timings.throughput(usage)})

    def generate(self, requests: Iterable[GenerationRequest]) -> list[GenerationResult]:
        from ..protocol.requests import expand_choices, merge_choices
        asked = list(requests)
        groups = [expand_choices(r) for r in asked]              # n > 1: n single-completion requests each
        reqs = [r for g in groups for r in g]
        if len(reqs) > 1 and self.args.max_batch_size > 1 and hasattr(self.runtime, "generate_batch") \
                and all(r.sampling_params.greedy for r in reqs):
            flat = self._generate_batched(reqs)
        else:
            flat = [self._run_one(r) for r in reqs]
        out, at = [], 0
        for r, g in zip(asked, groups):
            out.append(merge_choices(r, flat[at:at + len(g)]))
            at += len(g)
        return out

    def _generate_batched(self, reqs: list[GenerationRequest]) -> list[GenerationResult]:
        """Continuous batching through the runtime's scheduler (greedy requests only)."""
        self.prepare()
        for r in reqs:
            self._check_features(r)
        t0 = time.perf_counter()
        with self._lock:
            outs = self.runtime.generate_batch([self._tokens(r) for r in reqs],
                                               [r.sampling_params.max_tokens for r in reqs],
                                               self._eos_ids(), self.args.max_batch_size)
        dt = time.perf_counter() - t0
        results = []
        for r, (ids, finish, timing) in zip(reqs, outs):
            text = self.tokenizer.decode(ids)
            if r.sampling_params.stop:
                text, hit = truncate_at_stop(text, r.sampling_params.stop)
                finish = "stop" if hit else finish
            usage = Usage(len(self._tokens(r)), len(ids))
            tm = TimingMetrics.from_mapping(timing) if timing else TimingMetrics(total_seconds=dt)
            results.append(GenerationResult(r.request_id, ids, text, finish, usage, tm))
            self._stats["requests"] += 1
        return results

    def stream(self, request: GenerationRequest) -> Iterator[TokenEvent]:
        """Yields one event per token as it is produced, then a final event with finish_reason and usage."""
        import queue
        import threading

        if request.sampling_params.n != 1:
            raise UnsupportedFeatureError("streaming returns one completion: n must be 1")
        q: "queue.Queue[Any]" = queue.Queue()
        stops = request.sampling_params.stop
        sent = {"n": 0}

        def on_token(tok: int, out: list[int]) -> None:
            text = self.tokenizer.decode(out)
            safe = len(text) - held_back_suffix(text, stops)
            piece = text[sent["n"]:safe] if safe > sent["n"] else ""
            if "�" in piece:          # incomplete UTF-8 sequence: wait for the next token
                piece = ""
            else:
                sent["n"] = max(sent["n"], safe)
            q.put(TokenEvent(request.request_id, tok, piece))

        def work() -> None:
            try:
                q.put(self._run_one(request, on_token))
            except BaseException as exc:  # delivered to the consumer thread
                q.put(exc)

        threading.Thread(target=work, daemon=True, name=f"stream-{request.request_id}").start()
        while True:
            item = q.get()
            if isinstance(item, TokenEvent):
                yield item
            elif isinstance(item, GenerationResult):
                tail = item.text[sent["n"]:] if len(item.text) > sent["n"] else ""
                meta = {"timings": item.timings.as_dict()}
                if item.logprobs:
                    meta["logprobs"] = item.logprobs          # a stream delivers them with its last event
                yield TokenEvent(request.request_id, None, tail, item.finish_reason, item.usage, meta)
                return
            else:
                raise item

    # ---- worker ranks
    def run_worker(self) -> None:
        """Ranks > 0: mirror every command rank 0 issues until OP_STOP. A failing command is reported and
        the loop keeps serving (as the reference's persistent worker loop does,
        cpp_engine/engine/deepseek_v4_engine.cpp:11143-11239)."""
        self.prepare()
        rt, ch = self.runtime, self.channel
        slot_sp: dict[int, Any] = {}
        # After a collective timed out on THIS rank it has already joined the group's recovery on its own; commands
        # that rank 0 sent before it noticed the failure are stale and are dropped until its OP_RECOVER arrives.
        skipping = False
        while True:
            op, *payload = ch.recv()
            try:
                if op == OP_STOP:
                    return
                if op == OP_RECOVER:
                    if not skipping and hasattr(rt, "recover"):
                        rt.recover()
                    skipping = False
                    continue
                if skipping:
                    continue
                if op == OP_ALLOC:
                    rt.allocate()
                elif op == OP_FREE:
                    slot_sp.pop(payload[0], None)
                    rt.free(payload[0])
                elif op == OP_SAMPLING:
                    slot_sp[payload[0]] = _decode_sampling(payload[1:])
                elif op == OP_PREFILL:
                    slot, chunk, prompt = payload
                    rt.prefill_tokens(slot, prompt, chunk, slot_sp.get(slot))
                elif op == OP_DECODE:
                    slot, tok = payload
                    rt.decode_tokens([slot], [tok], slot_sp.get(slot))
                else:
                    raise BackendUnavailableError(f"unknown worker opcode {op}")
            except BackendUnavailableError:
                raise
            except Exception as exc:  # keep the group alive; rank 0 sees the failure through its own call
                if _is_collective_timeout(exc) and hasattr(rt, "recover"):
                    rt.recover()
                    skipping = True
                import sys
                print(f"[pocketllm worker rank {self.args.tensor_parallel_rank}] command {op} failed: {exc}",
                      file=sys.stderr, flush=True)
