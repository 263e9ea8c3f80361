"""The Qwen-style hybrid served from the host: the fp32 oracle behind the slot interface of the serving backend, with
every drafter of the speculative loop (``mtp``, ``ngram``, ``dspark``, ``dflash2``).

This is the path ``device="cpu"`` takes (``runtime/loader.py``).  It exists so that the whole public surface - typed
API, OpenAI server, log-probabilities, the learned block drafters - can be driven end to end on a machine without a
GPU, on small models: the oracle keeps no caches and re-runs the whole sequence for every target pass.

A decode call hands out the next token of the last verified block and runs a new draft / verify round only when the
block is used up (the same contract as the GPU speculative adapter); greedy acceptance, so the tokens are exactly the
oracle's greedy tokens.  ``backend_options["spec_gate"]`` puts the adaptive draft-length gate in front of every round.
The learned drafters come from ``backend_options["drafter"]`` (a checkpoint directory, read by
``load_dspark`` / ``load_dflash2``); a ``synthetic:`` model without that option gets a seeded random drafter of a small
shape, which proposes poorly but exercises the same code.

Reference behaviour: the speculative step of the native engine (cpp_engine/engine/qwen_engine.cpp:3904-3995 for DSpark,
:3790-3900 for DFlash2: propose from the committed token, verify ``[committed] + drafts`` in one pass, keep the
agreeing prefix and the target's own next token, append the kept rows' taps to the drafter).
"""
from __future__ import annotations

from typing import Any

import torch

from ..components.speculative import MtpDrafter, PromptLookupDrafter, WholeSequenceTarget
from ..models import qwen_hybrid as qh
from ..models.reference_cpu.qwen_hybrid_ref import QwenHybridRef, synth_mtp_state
from .loader import logprobs_of_row

METHODS = ("mtp", "ngram", "dspark", "dflash2")


class _Seq:
    def __init__(self, target: WholeSequenceTarget, drafter):
        self.target, self.drafter = target, drafter
        self.context: list[int] = []           # every committed token, the last one not yet run through the target
        self.queue: list[tuple[int, torch.Tensor]] = []      # verified tokens not handed out yet, with their logits rows
        self.last_row: torch.Tensor | None = None


class HostQwenAdapter:
    supports_sampling = False
    supports_logprobs = True
    supports_prefix_cache = False

    def __init__(self, oracle: QwenHybridRef, max_context: int, max_slots: int = 1, method: str | None = None,
                 block: int = 4, make_drafter=None, eos_token_ids=(), gate=None):
        self.oracle, self.max_context, self.max_slots = oracle, int(max_context), int(max_slots)
        self.method, self.block, self._make_drafter = method, max(1, int(block)), make_drafter
        self.gate = gate                       # SpecGate: how much of each block to verify, learnt from acceptance
        self.eos_token_ids = tuple(eos_token_ids)
        self.vocab_size = int(oracle.cfg.vocab_size)
        self.speculative_methods = (method,) if method else ()
        self.seqs: dict[int, _Seq] = {}
        self.last_cached_tokens = 0
        self.rounds = self.drafted = self.accepted = self.passes = 0

    # ---- slots
    def allocate(self) -> int:
        if len(self.seqs) >= self.max_slots:
            raise RuntimeError("no free sequence slot")
        slot = next(i for i in range(self.max_slots) if i not in self.seqs)
        tgt = WholeSequenceTarget(self.oracle)
        self.seqs[slot] = _Seq(tgt, self._make_drafter(tgt) if self._make_drafter else None)
        return slot

    def free(self, slot: int) -> None:
        self.seqs.pop(slot, None)

    def token_logprobs(self, slot: int, token: int, top_n: int) -> dict:
        return logprobs_of_row(self.seqs[slot].last_row, token, top_n)

    # ---- steps
    def _forward(self, st: _Seq, ids: list[int]) -> torch.Tensor:
        self.passes += 1
        return st.target.forward(torch.tensor(ids))

    def prefill_tokens(self, slot: int, prompt: list[int], chunk: int, sp: Any) -> int:
        st = self.seqs[slot]
        if len(prompt) + 1 > self.max_context:
            raise RuntimeError("prompt does not fit the context")
        st.target.reset()
        logits = self._forward(st, list(prompt))
        tok = int(logits[-1].argmax())
        st.context, st.queue, st.last_row = list(prompt) + [tok], [], logits[-1]
        return tok

    def _round(self, st: _Seq) -> None:
        """One draft / verify round after the committed token ``st.context[-1]``: fills ``st.queue``."""
        committed = st.context[-1]
        room = self.max_context - len(st.context) - 1
        draft: list[int] = []
        conf: list[float] = []
        gate = self.gate
        if st.drafter is not None and room > 1:
            if gate is not None and st.last_row is not None and not gate.should_draft(st.last_row.float().topk(2).values.tolist()):
                gate.note_skipped(by_margin=True)               # the target itself is unsure: a plain step
            else:
                draft, conf = st.drafter.propose(st.context, min(self.block, room - 1))
                if gate is not None and draft:
                    pad = list(conf) + [conf[-1]] * (gate.block - len(draft))
                    n = min(gate.choose(pad), len(draft))
                    if n == 0:
                        gate.note_skipped()
                    draft, conf = draft[:n], list(conf)[:n]
        if not draft:
            logits = self._forward(st, [committed])
            st.queue.append((int(logits[-1].argmax()), logits[-1]))
            return
        snap = st.target.snapshot()
        ver = self._forward(st, [committed] + draft)
        pred = ver.argmax(-1).tolist()
        a = 0
        while a < len(draft) and pred[a] == draft[a]:
            a += 1
        self.rounds += 1
        self.drafted += len(draft)
        self.accepted += a
        if gate is not None:
            gate.observe(conf, a, len(draft))
        st.queue.extend((t, ver[i]) for i, t in enumerate(draft[:a] + [pred[a]]))
        if a < len(draft):                                   # undo the rejected tail: the oracle's state is its token list
            st.target.restore(snap)
            self._forward(st, [committed] + draft[:a])

    def decode_tokens(self, slots: list[int], toks: list[int], sp: Any) -> list[int]:
        out = []
        for s in slots:
            st = self.seqs[s]
            if not st.queue:
                self._round(st)
            tok, row = st.queue.pop(0)
            st.context.append(tok)
            st.last_row = row
            out.append(tok)
        return out

    def stats(self) -> dict:
        out = {"target_passes": self.passes, "spec_rounds": self.rounds, "spec_drafted": self.drafted,
               "spec_accepted": self.accepted,
               "spec_accept_rate": round(self.accepted / self.drafted, 4) if self.drafted else 0.0}
        if self.gate is not None:
            out.update({"spec_gate_" + k: v for k, v in self.gate.stats().items() if isinstance(v, (int, float))})
        return out


def _tap_layers(cfg: qh.QwenHybridConfig, n: int = 2) -> list[int]:
    L = cfg.num_hidden_layers
    return sorted({min(L - 1, max(0, round((i + 1) * L / (n + 1)))) for i in range(n)})


def build_host_adapter(args, cfg: qh.QwenHybridConfig, state, max_context: int, max_slots: int) -> HostQwenAdapter:
    """``state``: (name, tensor) pairs of the target checkpoint.  Chooses the drafter from ``args.speculative_method``."""
    from pocketllm.api.errors import ConfigurationError
    method = getattr(args, "speculative_method", None)
    if method and method not in METHODS:
        raise ConfigurationError(f"speculative_method={method!r} is not one of {METHODS}")
    opts = dict(getattr(args, "backend_options", None) or {})
    block = int(getattr(args, "speculative_tokens", 1) or 1)
    synthetic = str(args.model).startswith("synthetic:")
    state = dict(state)
    if method == "mtp" and not any(k.startswith("mtp.") for k in state):
        if not synthetic:
            raise ConfigurationError("speculative_method='mtp' needs a checkpoint that carries the mtp.* tensors")
        state.update(synth_mtp_state(cfg, 0))
    oracle = QwenHybridRef(cfg, state)
    emb, head = oracle.p["model.language_model.embed_tokens.weight"], oracle.p["lm_head.weight"]
    make = None
    if method == "ngram":
        make = lambda tgt: PromptLookupDrafter()
    elif method == "mtp":
        make = lambda tgt: MtpDrafter(tgt)
    elif method in ("dspark", "dflash2"):
        from ..models import qwen_dflash2_ref as df
        from ..models import qwen_dspark_ref as ds
        path = opts.get("drafter")
        if path:
            dcfg, w = (ds.load_dspark if method == "dspark" else df.load_dflash2)(path)
        elif not synthetic:
            raise ConfigurationError(f"speculative_method={method!r} needs backend option drafter=<checkpoint directory>")
        elif method == "dspark":
            dcfg = ds.QwenDSparkConfig(hidden_size=cfg.hidden_size, intermediate_size=2 * cfg.hidden_size, vocab_size=cfg.vocab_size,
                                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                       block_size=max(block, 2), mask_token_id=cfg.vocab_size - 1, markov_rank=16,
                                       target_layer_ids=_tap_layers(cfg), original_max_position_embeddings=max_context)
            w = ds.synth_dspark_weights(dcfg, 0)
        else:
            dcfg = df.QwenDFlash2Config(hidden_size=cfg.hidden_size, intermediate_size=2 * cfg.hidden_size, vocab_size=cfg.vocab_size,
                                        num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                        block_size=max(block, 2) + 1, conv_group_size=16, conv_kernel_size=2,
                                        mask_token_id=cfg.vocab_size - 1, selector_rank=8, selector_top_k=4,
                                        sliding_window=max_context, target_layer_ids=_tap_layers(cfg))
            w = df.synth_dflash2_weights(dcfg, 0)
        if dcfg.hidden_size != cfg.hidden_size or dcfg.vocab_size != cfg.vocab_size \
                or max(dcfg.target_layer_ids) >= cfg.num_hidden_layers:
            raise ConfigurationError("the drafter checkpoint does not match the target model")
        oracle.capture_layers = tuple(dcfg.target_layer_ids)
        if method == "dspark":
            block = min(block, dcfg.block_size)
            make = lambda tgt: ds.QwenDSparkDrafter(tgt, ds.QwenDSparkRef(dcfg, w, emb, head, max_context=max_context))
        else:
            block = min(block, dcfg.draft_tokens)
            viterbi = str(opts.get("viterbi", "0")).lower() in ("1", "true", "yes")
            make = lambda tgt: df.QwenDFlash2Drafter(tgt, df.QwenDFlash2Ref(dcfg, w, emb, head, max_context=max_context,
                                                                              viterbi=viterbi))
    gate = None
    if method and str(opts.get("spec_gate", "0")).lower() in ("1", "true", "yes", "on"):
        from ..components.spec_gate import SpecGate
        gate = SpecGate.from_env(block)                      # constants from POCKETLLM_SPEC_GATE_* when set
    return HostQwenAdapter(oracle, max_context, max_slots, method, block, make, gate=gate)
