"""Byte-level BPE tokenizer built from GGUF metadata (``tokenizer.ggml.tokens`` / ``merges`` / ``token_type`` /
``*_token_id`` / ``pre``), the tokenizer the GGUF model families ship with
(reference: src/encoding/gguf_tokenizer.py, cpp_engine/core/tokenizer.cpp)."""
from __future__ import annotations

from functools import lru_cache
from typing import Any, Iterable

try:
    import regex as _re
except Exception:  # pragma: no cover
    import re as _re

# pre-tokenizer patterns by ``tokenizer.ggml.pre`` name; the default is the GPT-2 / llama-bpe style split
_PRE = {
    "default": r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""",
    "deepseek-v3": r"""\p{N}{1,3}|[一-龥぀-ゟ゠-ヿ]+|[!"#$%&'()*+,\-./:;<=>?@\[\\\]^_`{|}~][A-Za-z]+|[^\r\n\p{L}\p{P}\p{S}]?[\p{L}\p{M}]+| ?[\p{P}\p{S}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""",
    "glm4": r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}{1,3}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""",
    "minimax-m2": r"""(?i:'s|'t|'re|'ve|'m|'ll|'d)|[^\r\n\p{L}\p{N}]?\p{L}+|\p{N}| ?[^\s\p{L}\p{N}]+[\r\n]*|\s*[\r\n]+|\s+(?!\S)|\s+""",
}
TOKEN_NORMAL, TOKEN_UNKNOWN, TOKEN_CONTROL, TOKEN_USER_DEFINED, TOKEN_UNUSED, TOKEN_BYTE = 1, 2, 3, 4, 5, 6


@lru_cache(maxsize=1)
def _byte_maps() -> tuple[dict[int, str], dict[str, int]]:
    """GPT-2 byte <-> printable-unicode mapping."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs = bs[:]
    n = 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    enc = {b: chr(c) for b, c in zip(bs, cs)}
    return enc, {v: k for k, v in enc.items()}


class GGUFTokenizer:
    def __init__(self, tokens: list[str], merges: list[str], token_types: list[int] | None = None, pre: str = "default",
                 bos_id: int | None = None, eos_id: int | None = None, eot_ids: Iterable[int] = (), add_bos: bool = False):
        self.tokens = list(tokens)
        self.vocab = {t: i for i, t in enumerate(self.tokens)}
        self.ranks = {tuple(m.split(" ", 1)): i for i, m in enumerate(merges)}
        self.types = list(token_types) if token_types else [TOKEN_NORMAL] * len(self.tokens)
        self.pre = pre if pre in _PRE else "default"
        self._split = _re.compile(_PRE[self.pre])
        self.bos_id, self.eos_id, self.add_bos = bos_id, eos_id, add_bos
        self.eot_ids = set(eot_ids)
        special = [t for t, ty in zip(self.tokens, self.types) if ty in (TOKEN_CONTROL, TOKEN_USER_DEFINED) and t]
        special.sort(key=len, reverse=True)
        self._special = _re.compile("|".join(_re.escape(s) for s in special)) if special else None
        self._cache: dict[str, list[int]] = {}

    @classmethod
    def from_metadata(cls, md: dict[str, Any]) -> "GGUFTokenizer":
        model = md.get("tokenizer.ggml.model", "gpt2")
        if model not in ("gpt2", "bpe"):
            raise ValueError(f"unsupported GGUF tokenizer model {model!r} (byte-level BPE only)")
        eot = [md[k] for k in ("tokenizer.ggml.eot_token_id", "tokenizer.ggml.eom_token_id") if k in md]
        return cls(md["tokenizer.ggml.tokens"], md.get("tokenizer.ggml.merges", []), md.get("tokenizer.ggml.token_type"),
                   md.get("tokenizer.ggml.pre", "default"), md.get("tokenizer.ggml.bos_token_id"),
                   md.get("tokenizer.ggml.eos_token_id"), eot, bool(md.get("tokenizer.ggml.add_bos_token", False)))

    @classmethod
    def from_gguf(cls, path: str) -> "GGUFTokenizer":
        from ..formats.gguf import read_bundle
        return cls.from_metadata(read_bundle(path).metadata)

    @property
    def eos_ids(self) -> set[int]:
        return ({self.eos_id} if self.eos_id is not None else set()) | self.eot_ids

    # ---- encode
    def _bpe(self, word: str) -> list[int]:
        hit = self._cache.get(word)
        if hit is not None:
            return hit
        parts = list(word)
        while len(parts) > 1:
            best, bi = None, -1
            for i in range(len(parts) - 1):
                r = self.ranks.get((parts[i], parts[i + 1]))
                if r is not None and (best is None or r < best):
                    best, bi = r, i
            if best is None:
                break
            parts[bi:bi + 2] = [parts[bi] + parts[bi + 1]]
        ids = []
        for p in parts:
            i = self.vocab.get(p)
            if i is not None:
                ids.append(i)
            else:                       # unknown piece: fall back to its bytes' single-character tokens
                ids.extend(self.vocab[c] for c in p if c in self.vocab)
        if len(self._cache) < 65536:
            self._cache[word] = ids
        return ids

    def _encode_plain(self, text: str) -> list[int]:
        enc, _ = _byte_maps()
        out: list[int] = []
        for piece in self._split.findall(text):
            out.extend(self._bpe("".join(enc[b] for b in piece.encode("utf-8"))))
        return out

    def encode(self, text: str, add_special: bool | None = None, parse_special: bool = True) -> list[int]:
        out: list[int] = []
        if (self.add_bos if add_special is None else add_special) and self.bos_id is not None:
            out.append(self.bos_id)
        if not parse_special or self._special is None:
            return out + self._encode_plain(text)
        pos = 0
        for m in self._special.finditer(text):
            if m.start() > pos:
                out.extend(self._encode_plain(text[pos:m.start()]))
            out.append(self.vocab[m.group(0)])
            pos = m.end()
        if pos < len(text):
            out.extend(self._encode_plain(text[pos:]))
        return out

    # ---- decode
    def decode(self, ids: Iterable[int], skip_special: bool = True) -> str:
        _, dec = _byte_maps()
        buf = bytearray()
        for i in ids:
            if not (0 <= i < len(self.tokens)):
                continue
            ty = self.types[i]
            if ty == TOKEN_CONTROL and skip_special:
                continue
            t = self.tokens[i]
            if ty in (TOKEN_CONTROL, TOKEN_USER_DEFINED):
                buf.extend(t.encode("utf-8"))
            elif ty == TOKEN_BYTE and len(t) == 6 and t.startswith("<0x"):
                buf.append(int(t[3:5], 16))
            else:
                buf.extend(dec[c] if c in dec else ord("?") for c in t)
        return buf.decode("utf-8", errors="replace")
