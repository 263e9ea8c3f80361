"""Resident engine: a loaded multi-sequence runtime behind a command loop that survives a failing command.

The loop reads one JSON object per line and answers with one JSON object per line:

    {"op": "alloc"}                                   -> {"ok": true, "slot": 0}
    {"op": "prefill", "slot": 0, "tokens": [..]}      -> {"ok": true, "token": 17, "length": 42}
    {"op": "decode", "slots": [0, 1], "tokens": [..]} -> {"ok": true, "tokens": [3, 9]}
    {"op": "verify", "slot": 0, "tokens": [t0, d1..]} -> {"ok": true, "accepted": 2, "token": 5, "length": 45}
    {"op": "free", "slot": 0} | {"op": "reset"} | {"op": "stats"} | {"op": "stop"}

A command that raises (bad slot, no free page, a kernel error) is answered with ``{"ok": false, "error": ...}`` and the
loop goes on with the next line: the weights stay loaded and the other sequences keep their caches.  On ranks other
than 0 of a tensor-parallel group the same loop is fed from the rank-0 command channel, so every rank executes the
same commands in the same order.  Reference: PersistentEngine (cpp_engine/include/persistent_engine.hpp:24-208;
worker loop cpp_engine/engine/deepseek_v4_engine.cpp:11143-11239: prefill / decode / verify / batch_verify /
speculative_step, per-command exceptions reported and survived).
"""
from __future__ import annotations

import json
import sys
import time
from typing import Any, Callable, Iterable, TextIO


class ResidentEngine:
    """``runtime``: allocate() / free(slot) / prefill(slot, ids, chunk) / decode(slots, ids) / verify(slot, ids) and
    ``lengths`` (``models.mla_moe_gpu.MlaMoeBatchRuntime`` is one).  ``to_ids``: token list -> what the runtime takes."""

    def __init__(self, runtime: Any, to_ids: Callable[[list[int]], Any] | None = None, chunk: int = 2048):
        self.rt, self.chunk = runtime, int(chunk)
        self.to_ids = to_ids or (lambda toks: toks)
        self.stats = {"commands": 0, "errors": 0, "prefill_tokens": 0, "decode_tokens": 0, "drafted": 0, "accepted": 0,
                      "busy_seconds": 0.0}
        self._live: set[int] = set()
        cfg = getattr(runtime, "cfg", None)
        self.vocab = int(getattr(runtime, "vocab_size", 0) or getattr(cfg, "vocab_size", 0) or getattr(cfg, "vocab", 0) or 0)

    def _tokens(self, cmd: dict) -> list[int]:
        """The command's token ids, each a whole number the model has a row for: kernels index tables with them."""
        out = []
        for t in cmd["tokens"]:
            if isinstance(t, bool) or not isinstance(t, (int, float)) or t != int(t) or t < 0 or t > 0x7FFFFFFF \
                    or (self.vocab and t >= self.vocab):
                raise ValueError(f"{t!r} is not a token id of this model" + (f" (vocabulary {self.vocab})" if self.vocab else ""))
            out.append(int(t))
        return out

    # ---- one command
    def _scalar(self, t: Any) -> int:
        return int(t.item()) if hasattr(t, "item") else int(t)

    def _list(self, t: Any) -> list[int]:
        return [int(x) for x in (t.reshape(-1).tolist() if hasattr(t, "reshape") else t)]

    def _slot(self, cmd: dict) -> int:
        s = int(cmd["slot"])
        if s not in self._live:
            raise KeyError(f"slot {s} is not allocated")
        return s

    def execute(self, cmd: dict) -> dict:
        op = cmd.get("op")
        rt = self.rt
        if op == "alloc":
            s = int(rt.allocate())
            self._live.add(s)
            return {"slot": s}
        if op == "free":
            s = self._slot(cmd)
            rt.free(s)
            self._live.discard(s)
            return {}
        if op == "reset":
            for s in sorted(self._live):
                rt.free(s)
            self._live.clear()
            return {}
        if op == "prefill":
            s, toks = self._slot(cmd), self._tokens(cmd)
            if not toks:
                raise ValueError("prefill needs at least one token")
            chunk = cmd.get("chunk", self.chunk)
            if isinstance(chunk, bool) or not isinstance(chunk, int) or not 1 <= chunk <= 1 << 20:
                raise ValueError("chunk must be a whole number of tokens in [1, 1048576]")
            tok = self._scalar(rt.prefill(s, self.to_ids(toks), chunk))
            self.stats["prefill_tokens"] += len(toks)
            return {"token": tok, "length": int(rt.lengths[s])}
        if op == "decode":
            slots, toks = [int(s) for s in cmd["slots"]], self._tokens(cmd)
            if len(slots) != len(toks) or not slots or len(set(slots)) != len(slots):
                raise ValueError("decode takes one token for each of a set of distinct slots")
            for s in slots:
                self._slot({"slot": s})
            out = self._list(rt.decode(slots, self.to_ids(toks)))
            self.stats["decode_tokens"] += len(slots)
            return {"tokens": out}
        if op == "verify":
            s, toks = self._slot(cmd), self._tokens(cmd)
            if not toks:
                raise ValueError("verify needs the last accepted token and the drafts")
            accepted, tok = rt.verify(s, self.to_ids(toks))
            self.stats["drafted"] += len(toks) - 1
            self.stats["accepted"] += int(accepted)
            self.stats["decode_tokens"] += int(accepted) + 1
            return {"accepted": int(accepted), "token": int(tok), "length": int(rt.lengths[s])}
        if op == "stats":
            return {"stats": dict(self.stats), "live_slots": sorted(self._live)}
        raise ValueError(f"unknown op {op!r}")

    # ---- the loop
    def serve(self, lines: Iterable[str], out: TextIO = sys.stdout, after_command: Callable[[], None] | None = None) -> int:
        """Run until ``{"op": "stop"}`` or the end of ``lines``; returns the number of commands that failed."""
        for line in lines:
            line = line.strip()
            if not line:
                continue
            t0 = time.perf_counter()
            self.stats["commands"] += 1
            cmd = None
            try:
                cmd = json.loads(line)
                if not isinstance(cmd, dict):
                    raise ValueError("a command is a JSON object")
                if cmd.get("op") == "stop":
                    out.write(json.dumps({"ok": True, "stopped": True}) + "\n")
                    out.flush()
                    break
                reply = {"ok": True, **self.execute(cmd)}
                if after_command is not None:
                    after_command()             # e.g. the check of the device error word
            except Exception as exc:            # the loop survives: report and take the next command
                self.stats["errors"] += 1
                reply = {"ok": False, "error": f"{type(exc).__name__}: {exc}"}
            self.stats["busy_seconds"] += time.perf_counter() - t0
            if isinstance(cmd, dict) and "id" in cmd:
                reply["id"] = cmd["id"]
            out.write(json.dumps(reply) + "\n")
            out.flush()
        return self.stats["errors"]
