"""Greedy speculative decoding for the Qwen-style hybrid runtime: multi-token-prediction head or prompt-lookup drafts,
multi-row verification in one target pass, recurrent-state transaction with per-row checkpoints.

What the reference's native engine does for ``--qwen-mtp`` (cpp_engine/engine/qwen_engine.cpp:402-447 options and
stats, :1444-1540 verify rows with recurrent-state snapshots, :3680-3730 the head: normalised embedding and hidden
concatenated -> ``mtp.fc`` -> one full-attention layer -> ``mtp.norm`` -> shared output head; verify attention
cpp_engine/backends/cuda/kernels/qwen_gqa_optimized.cu:2119-2457), rebuilt on this package's decode kernels:

* verify pass: the committed token and the K drafts run as K+1 rows through the weight-streaming decode path.  Rows of
  one sequence are K+1 entries of a decode batch that share the block table and differ in context length, so the
  split-KV decode attention kernel gives each row exactly its causal view.  The Gated-DeltaNet layers run their fused
  one-token mixer row after row and copy the layer's recurrent state and conv tail aside after every row but the last
  (2 MB per layer and row at the 27B shape), so a rejected tail is undone by copying one checkpoint back: no replay
  pass and no whole-model snapshot.
* the head runs on the same K+1 rows right after (row i: embedding of the target's own prediction for position i+1 and
  the target's hidden state of row i), which both catches the head's cache up on every accepted position and yields the
  next round's first draft at the row of the last accepted token; deeper drafts apply the head to its own hidden state.
* one host read per round (predictions and drafts together).

The output is token for token the greedy output of the target; drafts only change how many target passes it takes.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..components.speculative import PromptLookupDrafter
from ..ops import basic, gdn, gemm
from . import qwen_hybrid as qh


@dataclass
class SpecCounters:
    rounds: int = 0
    drafted: int = 0
    accepted: int = 0
    plain_steps: int = 0
    rollbacks: int = 0

    @property
    def accept_rate(self) -> float:
        return self.accepted / max(1, self.drafted)

    @property
    def tokens_per_pass(self) -> float:
        return (self.accepted + self.rounds + self.plain_steps) / max(1, self.rounds + self.plain_steps)


@dataclass
class _Seq:
    committed: int = -1                                  # token at position ``length`` (predicted, not yet run)
    drafts: torch.Tensor | None = None                   # int32 [K] on the device (mtp) - tokens after ``committed``
    history: list[int] = field(default_factory=list)    # prompt + generated tokens (prompt-lookup drafter)
    queue: list[int] = field(default_factory=list)      # tokens produced by the last round, not yet handed out


class QwenSpeculator:
    """Wraps a ``QwenHybridRuntime``.  ``method``: "mtp" (needs a checkpoint with the head) or "ngram"."""

    def __init__(self, rt: qh.QwenHybridRuntime, k: int = 1, method: str = "mtp"):
        if method not in ("mtp", "ngram"):
            raise ValueError(f"unknown speculative method {method!r}")
        if method == "mtp" and rt.mtp is None:
            raise ValueError("speculative_method='mtp' needs a checkpoint with a multi-token-prediction head (mtp.* tensors)")
        if not rt.fused_decode:
            raise ValueError("speculative decoding runs on the FP8 weight-streaming decode path")
        if not 1 <= k <= 7:
            raise ValueError("1 <= speculative tokens <= 7")
        self.rt, self.k, self.method = rt, int(k), method
        self.stats = SpecCounters()
        self.seqs: dict[int, _Seq] = {}
        self.lookup = PromptLookupDrafter(max_ngram=4)
        dev, nl = rt.device, len(rt.lin_layers)
        cw = 2 * rt.kd + rt.vd
        # per-row checkpoints of one sequence's recurrent state and conv tails (rows 0..K-1 of a verify pass)
        self.ck_states = torch.empty(self.k, nl, rt.hv_lin, 128, 128, dtype=torch.float32, device=dev)
        self.ck_tails = torch.empty(self.k, nl, rt.cfg.linear_conv_kernel_dim - 1, cw, dtype=torch.bfloat16, device=dev)
        if rt.prefix_cache is not None:
            raise ValueError("speculative decoding and the prefix cache are not combined: a resumed prefix would leave "
                             "holes in the draft head's cache")
        if method == "mtp":
            rt.keep_hidden = True
        self.mtp_cache_layer = len(rt.full_layers)       # index of the head's layer in the KV cache

    # ------------------------------------------------------------------ helpers
    def _rows_meta(self, st: qh.SeqState, n: int):
        """Positions, cache slots and decode-attention metadata of ``n`` consecutive rows starting at the sequence's
        current length: the rows are entries of a decode batch over one block table."""
        rt, dev = self.rt, self.rt.device
        rt._ensure_blocks(st, st.length + n)
        pos = torch.arange(st.length, st.length + n, dtype=torch.int32, device=dev)
        bt_row = rt.block_table[st.slot]
        kv_slots = (bt_row[(pos // rt.block_size).long()] * rt.block_size + pos % rt.block_size).to(torch.int32)
        max_len = st.length + n
        meta = {"mode": "decode", "block_table": bt_row[None].expand(n, -1).contiguous(),
                "kv_len": (pos + 1).contiguous(), "max_kv_len": 1 << max(10, (max_len - 1).bit_length())}
        return pos, kv_slots, meta

    # ------------------------------------------------------------------ target: K+1 rows of one sequence
    @torch.no_grad()
    def _verify_forward(self, st: qh.SeqState, ids: torch.Tensor):
        """ids int32 [R] on the device: the committed token followed by R-1 drafts.  Appends all R rows to the caches
        and the recurrent state; checkpoints the state after each of the first R-1 rows.  Returns (next-token
        prediction per row int32 [R], final-normed hidden [R, H])."""
        rt = self.rt
        cfg, w, comm = rt.cfg, rt.w, rt.comm
        r_rows = ids.numel()
        pos, kv_slots, meta = self._rows_meta(st, r_rows)
        slot1 = torch.tensor([st.slot], dtype=torch.int32, device=rt.device)
        _, terms = gemm.stream_layout(r_rows)
        eps = cfg.rms_norm_eps
        h = rt._embed(ids)
        delta = None
        for i, lw in enumerate(w.layers):
            x, xs = basic.rmsnorm_split(h, delta, lw.in_ln, terms, eps, True, want_bf16=lw.kind == "linear")
            proj = gemm.linear_stream(None, lw.proj, xsplit=xs)
            if lw.kind == "linear":
                idx = rt.lin_layers.index(i)
                ys = []
                for r in range(r_rows):
                    ys.append(gdn.decode_fused(proj[r:r + 1], x[r:r + 1], lw.ab.weight, lw.a_log, lw.dt_bias, lw.conv_w,
                                               rt.tails[:, idx], rt.states[:, idx], slot1, lw.gdn_norm, rt.hv_lin,
                                               rt.hk_lin, eps))
                    if r < r_rows - 1:
                        self.ck_states[r, idx].copy_(rt.states[st.slot, idx])
                        self.ck_tails[r, idx].copy_(rt.tails[st.slot, idx])
                y = torch.cat(ys) if r_rows > 1 else ys[0]
                d_attn = rt._stream_row_parallel(y, lw.out)
            else:
                o = rt._attend(rt.full_layers.index(i), lw, proj, r_rows, pos, kv_slots, meta, eps)
                d_attn = rt._stream_row_parallel(o.view(r_rows, rt.hq * 128), lw.out)
            _, xs2 = basic.rmsnorm_split(h, d_attn, lw.post_ln, terms, eps, True, want_bf16=False)
            gu = gemm.linear_stream(None, lw.gate_up, xsplit=xs2)
            delta = rt._stream_row_parallel(None, lw.down, basic.silu_mul_split(gu, terms))
        x = basic.add_rmsnorm(h, delta, w.final_norm, eps, True)
        logits = gemm.linear(x, w.lm_head, out_f32=True)
        return rt._next_tokens(logits), x

    def _rollback(self, st: qh.SeqState, row: int) -> None:
        """Put the recurrent state back to what it was after verify row ``row`` (the caches need nothing: rows past
        the new length are overwritten by the next pass)."""
        self.rt.states[st.slot].copy_(self.ck_states[row])
        self.rt.tails[st.slot].copy_(self.ck_tails[row])
        self.stats.rollbacks += 1

    # ------------------------------------------------------------------ the head
    @torch.no_grad()
    def _mtp_rows(self, st_len: int, slot: int, next_ids: torch.Tensor, hidden: torch.Tensor, prefill: bool):
        """The head on R rows at positions st_len .. st_len+R-1 of slot ``slot``: row i fuses the embedding of
        ``next_ids[i]`` with ``hidden[i]``.  Appends the rows to the head's own cache layer.  Returns (predicted token
        per row int32 [R], the head's normalised hidden [R, H])."""
        rt, m = self.rt, self.rt.mtp
        cfg, eps = rt.cfg, rt.cfg.rms_norm_eps
        n = next_ids.numel()
        dev = rt.device
        rt._ensure_blocks(rt.seqs[slot], st_len + n)
        e = basic.rmsnorm(rt._embed(next_ids), m.norm_embed, eps, True)
        hn = basic.rmsnorm(hidden.contiguous(), m.norm_hidden, eps, True)
        h = gemm.linear(torch.cat([e, hn], -1).contiguous(), m.fc)
        pos = torch.arange(st_len, st_len + n, dtype=torch.int32, device=dev)
        bt_row = rt.block_table[slot]
        kv_slots = (bt_row[(pos // rt.block_size).long()] * rt.block_size + pos % rt.block_size).to(torch.int32)
        if prefill:
            i32 = lambda v: torch.tensor([v], dtype=torch.int32, device=dev)
            meta = {"mode": "prefill", "block_table": rt.block_table[slot:slot + 1], "q_start": i32(0), "q_len": i32(n),
                    "kv_len": i32(st_len + n), "max_q_len": n, "past": st_len}
        else:
            meta = {"mode": "decode", "block_table": bt_row[None].expand(n, -1).contiguous(),
                    "kv_len": (pos + 1).contiguous(), "max_kv_len": 1 << max(10, (st_len + n - 1).bit_length())}
        lw = m.layer
        x = basic.rmsnorm(h, lw.in_ln, eps, True)
        proj = gemm.linear(x, lw.proj)
        o = rt._attend(self.mtp_cache_layer, lw, proj, n, pos, kv_slots, meta, eps)
        d_attn = rt._row_parallel(o.view(n, rt.hq * 128), lw.out)
        x2 = basic.add_rmsnorm(h, d_attn, lw.post_ln, eps, True)
        act = basic.silu_mul(gemm.linear(x2, lw.gate_up))
        delta = rt._row_parallel(act, lw.down)
        out = basic.add_rmsnorm(h, delta, m.norm_out, eps, True)
        rows = out if not prefill else out[-1:]
        logits = gemm.linear(rows.contiguous(), rt.w.lm_head, out_f32=True)
        return rt._next_tokens(logits), out

    def _draft_from(self, st: qh.SeqState, first: torch.Tensor, hidden_row: torch.Tensor) -> torch.Tensor:
        """K drafts: ``first`` (the head's prediction at the last accepted row) and K-1 recursive steps of the head
        on its own hidden state, at the positions that follow."""
        drafts = [first.reshape(1).to(torch.int32)]
        hid = hidden_row
        for j in range(1, self.k):
            tok, hid_all = self._mtp_rows(st.length - 1 + j, st.slot, drafts[-1], hid, prefill=False)
            drafts.append(tok.reshape(1).to(torch.int32))
            hid = hid_all[-1:]
        return torch.cat(drafts)

    # ------------------------------------------------------------------ public
    def allocate(self) -> int:
        slot = self.rt.allocate()
        self.seqs[slot] = _Seq()
        return slot

    def free(self, slot: int) -> None:
        self.seqs.pop(slot, None)
        self.rt.free(slot)

    @torch.no_grad()
    def prefill(self, slot: int, token_ids: torch.Tensor, chunk: int = 8192, host_tokens: list[int] | None = None) -> int:
        """Prefill through the target (chunked); with the head, every chunk's rows also pass through it so its cache
        covers the prompt.  Returns the first generated token."""
        rt = self.rt
        st, sq = rt.seqs[slot], self.seqs[slot]
        total = token_ids.numel()
        sq.history = list(host_tokens) if host_tokens is not None else [int(t) for t in token_ids.tolist()]
        tok = None
        last_out = None
        for s in range(0, total, chunk):
            e = min(total, s + chunk)
            start_len = st.length
            tok = rt.prefill(slot, token_ids[s:e], chunk)
            if self.method == "mtp":
                nxt = token_ids[s + 1:e + 1] if e < total else torch.cat([token_ids[s + 1:e], tok.reshape(1).to(torch.int32)])
                t_last, out = self._mtp_rows(start_len, slot, nxt.to(torch.int32).contiguous(), rt.hidden_rows, prefill=True)
                last_out = (t_last, out[-1:])
        first = int(tok.item())
        sq.committed = first
        sq.history.append(first)
        if self.method == "mtp":
            sq.drafts = self._draft_from(st, last_out[0], last_out[1])
        return first

    def _propose(self, slot: int) -> torch.Tensor | None:
        """Drafts for the tokens after the committed one: int32 [<= K] on the device, or None for a plain step."""
        sq = self.seqs[slot]
        if self.method == "mtp":
            return sq.drafts
        prop, _ = self.lookup.propose(sq.history, self.k)
        return torch.tensor(prop, dtype=torch.int32, device=self.rt.device) if prop else None

    @torch.no_grad()
    def step(self, slot: int) -> list[int]:
        """One round: verify the committed token + drafts, commit the accepted prefix and the target's own next
        token.  Returns the newly produced tokens (1 .. K+1)."""
        rt = self.rt
        st, sq = rt.seqs[slot], self.seqs[slot]
        dev = rt.device
        drafts = self._propose(slot)
        if drafts is None or drafts.numel() == 0:
            tok = rt.decode([slot], torch.tensor([sq.committed], dtype=torch.int32, device=dev))
            sq.committed = int(tok.item())
            sq.history.append(sq.committed)
            self.stats.plain_steps += 1
            return [sq.committed]
        n = drafts.numel()
        ids = torch.cat([torch.tensor([sq.committed], dtype=torch.int32, device=dev), drafts])
        pred, x = self._verify_forward(st, ids)
        both = torch.cat([pred.to(torch.int32), drafts]).tolist()          # the round's one host read
        p, d = both[:n + 1], both[n + 1:]
        a = 0
        while a < n and p[a] == d[a]:
            a += 1
        self.stats.rounds += 1
        self.stats.drafted += n
        self.stats.accepted += a
        if a < n:
            self._rollback(st, a)
        start_len = st.length
        st.length += a + 1
        new = d[:a] + [p[a]]
        sq.committed = p[a]
        sq.history.extend(new)
        if self.method == "mtp":
            # the head on every verified row: catches its cache up on the accepted positions; its prediction at row a
            # is the next round's first draft (rows past a are scratch that later rows overwrite)
            m_pred, m_hid = self._mtp_rows(start_len, slot, pred.to(torch.int32), x, prefill=False)
            sq.drafts = self._draft_from(st, m_pred[a:a + 1], m_hid[a:a + 1])
        return new

    @torch.no_grad()
    def generate(self, prompt: torch.Tensor, max_new_tokens: int, chunk: int = 8192, eos: int | None = None) -> list[int]:
        slot = self.allocate()
        try:
            out = [self.prefill(slot, prompt.to(self.rt.device, torch.int32), chunk)]
            while len(out) < max_new_tokens and (eos is None or eos not in out):
                out.extend(self.step(slot))
            if eos is not None and eos in out:
                out = out[:out.index(eos) + 1]
            return out[:max_new_tokens]
        finally:
            self.free(slot)
