"""DSpark-style block drafter for the DeepSeek-V4 CPU runtime, fp32: from one committed token it proposes ``block``
tokens in a single pass of a few draft stages, with a confidence score per token.

* The stages are V4 blocks (hyper-connections, window attention, routed experts) whose attention takes its *keys and
  values for the committed context from the target model*: the mean over streams of a few target layers' hidden states,
  concatenated, projected and normalised (``main_proj`` / ``main_norm``), goes through each stage's own ``wkv`` into a
  window ring.  Only queries (and the block's own keys) come from the draft input.
* The draft input is the committed token followed by ``block - 1`` noise tokens; every draft position sees the whole
  ring and the whole block (no causal mask inside the block).
* The last stage ends in the hyper-connection head and the target's vocabulary head; position ``i`` then gets a
  low-rank bigram bias from the token chosen at position ``i - 1`` (``markov_w1`` row -> ``markov_w2``), which is what
  makes the block sequentially consistent, and the confidence is a linear read-out of [hidden, bigram embedding].

``DSparkLoop`` is the greedy draft / verify / commit loop with the adaptive gate.  The CPU target advances one token at
a time, so verification stops at the first mismatch instead of running the whole block and rolling back; the committed
tokens are the same.

Reference behaviour: src/models/deepseek_v4/dspark.py:40-275 (attention over main-model KV, Markov and confidence
heads, forward_embed / forward_head) and dspark_loop.py:97-244 (hidden capture, ring priming, rounds).
"""
from __future__ import annotations

import torch

from ..components.spec_gate import SpecGate
from . import v4_components as V
from .v4_block_ref import V4BlockRef, V4Config, _Layer, _layer_weights, _rms, sparse_attention_ref


def synth_dspark_weights(cfg: V4Config, n_stages: int = 3, n_target: int = 2, markov_rank: int = 8, seed: int = 0) -> dict:
    g = torch.Generator().manual_seed(seed + 77)
    r = lambda *s, sd=0.05: torch.randn(*s, generator=g) * sd
    one = lambda *s: 1.0 + r(*s, sd=0.05)
    d, hc = cfg.dim, cfg.hc_mult
    w = {}
    for s in range(n_stages):
        w.update(_layer_weights(cfg, r, one, f"dspark.{s}.", 0, False))
    w["dspark.main_proj"], w["dspark.main_norm"] = r(d, d * n_target, sd=0.1), one(d)
    w["dspark.norm"] = one(d)
    w["dspark.hc_head_fn"], w["dspark.hc_head_scale"], w["dspark.hc_head_base"] = r(hc, hc * d), one(1), r(hc, sd=0.3)
    w["dspark.markov_w1"], w["dspark.markov_w2"] = r(cfg.vocab_size, markov_rank, sd=0.5), r(cfg.vocab_size, markov_rank, sd=0.5)
    w["dspark.confidence"] = r(1, d + markov_rank, sd=0.5)
    return w


def save_dspark_weights(path: str, weights: dict, target_layer_ids) -> int:
    """One safetensors file of the ``dspark.*`` tensors; the target layers whose hidden states feed the drafter travel
    in the file's metadata (``target_layer_ids``: "1,2")."""
    from ..formats import safetensors_io
    ids = ",".join(str(int(i)) for i in target_layer_ids)
    return safetensors_io.write_file(path, {k: v for k, v in weights.items() if k.startswith("dspark.")},
                                     metadata={"target_layer_ids": ids})


def load_dspark_weights(path: str, cfg: V4Config, target_layer_ids=None) -> tuple[dict, tuple[int, ...]]:
    """(weights, target layer ids) of a drafter file, checked against the target's shape."""
    from ..formats.safetensors_io import SafetensorsFile
    f = SafetensorsFile(path)
    w = {k: f.get(k) for k in f.keys()}
    raw = target_layer_ids if target_layer_ids is not None else f.metadata.get("target_layer_ids", "")
    ids = tuple(int(x) for x in (raw if not isinstance(raw, str) else raw.replace(" ", "").split(",")) if str(x) != "")
    if not ids or max(ids) >= cfg.n_layers or min(ids) < 0 or "dspark.main_proj" not in w \
            or tuple(w["dspark.main_proj"].shape) != (cfg.dim, cfg.dim * len(ids)):
        raise ValueError("the DSpark drafter file does not match this model (target_layer_ids / dspark.main_proj)")
    return w, ids


class _DraftStage(_Layer):
    """A V4 block whose attention reads the committed context from target-model hidden states."""

    def write_main_kv(self, main_x: torch.Tensor, start: int) -> None:
        """Ring entries for positions start .. start + S - 1 from ``main_x`` [S, D]; no attention."""
        cfg, w, a, win, rd = self.cfg, self.w, self.p + "attn.", self.cfg.window, self.cfg.rope_head_dim
        s = main_x.shape[0]
        if s > win:                                             # only the last ``win`` positions survive
            main_x, start, s = main_x[-win:], start + s - win, win
        kv = _rms(main_x @ w[a + "wkv"].t(), w[a + "kv_norm"], cfg.norm_eps)[None]
        kv = torch.cat([kv[..., :-rd], V.apply_rotary(kv[..., -rd:].contiguous(), self.table[start:start + s])], -1)[0]
        self.kv[(torch.arange(s) + start) % win] = kv

    def draft_attention(self, x: torch.Tensor, start: int, main_x: torch.Tensor) -> torch.Tensor:
        """x [block, D] draft inputs at positions start + 1 ..; main_x [1, D] enters the ring at position ``start``."""
        cfg, w, a, win, rd = self.cfg, self.w, self.p + "attn.", self.cfg.window, self.cfg.rope_head_dim
        assert start > 0 and main_x.shape[0] == 1
        blk = x.shape[0]
        tab = self.table[start + 1:start + 1 + blk]
        self.write_main_kv(main_x, start)
        qr = _rms(x @ w[a + "wq_a"].t(), w[a + "q_norm"], cfg.norm_eps)
        q = _rms((qr @ w[a + "wq_b"].t()).view(1, blk, cfg.n_heads, cfg.head_dim), None, cfg.norm_eps)
        q = torch.cat([q[..., :-rd], V.apply_rotary(q[..., -rd:].contiguous(), tab)], -1)[0]
        kv = _rms(x @ w[a + "wkv"].t(), w[a + "kv_norm"], cfg.norm_eps)[None]
        kv = torch.cat([kv[..., :-rd], V.apply_rotary(kv[..., -rd:].contiguous(), tab)], -1)[0]
        idx = torch.cat([torch.arange(min(win, start + 1)), win + torch.arange(blk)]).expand(blk, -1)
        o = sparse_attention_ref(q, torch.cat([self.kv[:win], kv]), w[a + "attn_sink"], idx, cfg.head_dim ** -0.5)
        o = torch.cat([o[..., :-rd], V.apply_rotary(o[None, ..., -rd:].contiguous(), tab, inverse=True)[0]], -1)
        o = torch.einsum("sgd,grd->sgr", o.reshape(blk, cfg.o_groups, -1), w[a + "wo_a"].view(cfg.o_groups, cfg.o_lora_rank, -1))
        return o.flatten(1) @ w[a + "wo_b"].t()

    def draft_forward(self, streams: torch.Tensor, start: int, ids: torch.Tensor, main_x: torch.Tensor) -> torch.Tensor:
        cfg, w, p = self.cfg, self.w, self.p
        for blk, fn in (("attn", lambda t: self.draft_attention(t, start, main_x)), ("ffn", lambda t: self.ffn(t, ids))):
            y, post, comb = V.hc_pre(streams[None], w[p + f"hc_{blk}_fn"], w[p + f"hc_{blk}_scale"], w[p + f"hc_{blk}_base"],
                                     cfg.norm_eps, cfg.hc_iters, cfg.hc_eps)
            y = fn(_rms(y[0], w[p + f"{blk}_norm"], cfg.norm_eps))
            streams = V.hc_post(y[None], streams[None], post, comb)[0]
        return streams


class DSparkRef:
    def __init__(self, target: V4BlockRef, weights: dict, target_layer_ids: tuple[int, ...], block: int = 4,
                 noise_token_id: int = 0):
        self.t, self.cfg, self.block, self.noise, self.layer_ids = target, target.cfg, block, noise_token_id, tuple(target_layer_ids)
        self.w = dict(target.w)
        self.w.update({k: (v.float() if v.is_floating_point() else v) for k, v in weights.items()})
        assert self.w["dspark.main_proj"].shape[1] == self.cfg.dim * len(self.layer_ids)
        n = 1 + max(int(k.split(".")[1]) for k in weights if k.split(".")[1].isdigit())
        self.stages = [_DraftStage(self.cfg, self.w, f"dspark.{s}.", 0, False) for s in range(n)]

    def reset(self) -> None:
        for s in self.stages:
            s.reset()

    def target_hidden(self) -> torch.Tensor:
        """[S, D * n_target] from the target's last forward."""
        return torch.cat([self.t.layer_hidden[i] for i in self.layer_ids], -1)

    def _main_x(self, hidden: torch.Tensor) -> torch.Tensor:
        return _rms(hidden @ self.w["dspark.main_proj"].t(), self.w["dspark.main_norm"], self.cfg.norm_eps)

    def write_kv(self, hidden: torch.Tensor, start: int) -> None:
        mx = self._main_x(hidden)
        for s in self.stages:
            s.write_main_kv(mx, start)

    @torch.no_grad()
    def draft(self, hidden_last: torch.Tensor, committed: int, start: int) -> tuple[list[int], torch.Tensor, torch.Tensor]:
        """(tokens [block], logits [block, vocab] with the bigram bias applied, confidence [block])."""
        cfg, w = self.cfg, self.w
        ids = torch.full((self.block,), self.noise, dtype=torch.long)
        ids[0] = committed
        streams = w["embed"][ids][:, None, :].repeat(1, cfg.hc_mult, 1)
        mx = self._main_x(hidden_last.reshape(1, -1))
        for s in self.stages:
            streams = s.draft_forward(streams, start, ids, mx)
        flat = streams.flatten(1)
        mixes = (flat @ w["dspark.hc_head_fn"].t()) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + cfg.norm_eps)
        pre = torch.sigmoid(mixes * w["dspark.hc_head_scale"] + w["dspark.hc_head_base"]) + cfg.hc_eps
        x = (pre[..., None] * streams).sum(1)                                              # [block, D]
        logits = _rms(x, w["dspark.norm"], cfg.norm_eps) @ w["head"].t()
        toks, prev, embeds = [], committed, []
        for i in range(self.block):                             # each position is biased by the token before it
            e = w["dspark.markov_w1"][prev]
            logits[i] += w["dspark.markov_w2"] @ e
            embeds.append(e)
            prev = int(logits[i].argmax())
            toks.append(prev)
        conf = (torch.cat([x, torch.stack(embeds)], -1) @ w["dspark.confidence"].t()).squeeze(-1)
        return toks, logits, conf


class DSparkLoop:
    """prefill / step rounds over a ``V4BlockRef`` target; greedy, one sequence."""

    def __init__(self, drafter: DSparkRef, gate: SpecGate | None = None):
        self.d, self.t = drafter, drafter.t
        self.gate = gate if gate is not None else SpecGate(drafter.block, enabled=False)
        self.rounds = self.drafted = self.accepted = self.target_steps = 0

    def _advance(self, tok: int) -> int:
        """Feed one token to the target, enter its hidden state into the draft rings, return the greedy next token."""
        pos = self.t.length
        self.logits = self.t.forward(torch.tensor([tok]))[-1]
        self.hidden = self.d.target_hidden()[-1:]
        self.d.write_kv(self.hidden, pos)
        self.target_steps += 1
        return int(self.logits.argmax())

    def prefill(self, prompt: torch.Tensor) -> int:
        self.t.reset(); self.d.reset()
        self.logits = self.t.forward(prompt)[-1]
        h = self.d.target_hidden()
        self.d.write_kv(h, 0)
        self.hidden = h[-1:]
        self.committed = int(self.logits.argmax())
        return self.committed

    def step(self) -> tuple[list[int], int]:
        """One round: (tokens committed by it - the pending token and the accepted drafts, number of drafts verified)."""
        self.rounds += 1
        n, draft, conf = 0, [], []
        if not self.gate.should_draft(self.logits.topk(2).values.tolist()):
            self.gate.note_skipped(by_margin=True)
        else:
            draft, _, conf = self.d.draft(self.hidden, self.committed, self.t.length)
            n = min(self.gate.choose(conf.tolist()), len(draft))
            if n == 0:
                self.gate.note_skipped()
        out = [self.committed]
        nxt = self._advance(self.committed)
        ok = 0
        while ok < n and draft[ok] == nxt:                      # draft i stands iff the target predicts it
            out.append(nxt)
            nxt = self._advance(nxt)
            ok += 1
        if n:
            self.gate.observe(conf.tolist(), ok, n)
            self.drafted += n
            self.accepted += ok
        self.committed = nxt
        return out, n

    def generate(self, prompt: torch.Tensor, max_new_tokens: int) -> list[int]:
        self.prefill(prompt)
        out: list[int] = []
        while len(out) < max_new_tokens:
            toks, _ = self.step()
            out.extend(toks)
        return out[:max_new_tokens]
