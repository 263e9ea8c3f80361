"""JSON-lines helper process for native front ends that do not embed a chat-template engine: reads one request per
line on stdin, answers one line on stdout.

    {"op": "ping"}                                              -> {"ok": true}
    {"op": "encode", "family": "deepseek_v4", "messages": [...], "tools": [...], "thinking": false,
     "reasoning_effort": null}                                  -> {"ok": true, "prompt": "...", "token_ids": [...]?}
    {"op": "parse", "family": "deepseek_v4", "text": "...", "thinking": false}
                                                                -> {"ok": true, "message": {...}}
    {"op": "decode", "family": "...", "token_ids": [...]}       -> {"ok": true, "text": "...", "message": {...}?}
    {"op": "shutdown"}                                          -> {"ok": true} and exit

``token_ids`` are returned when a tokenizer was given (``--gguf`` with embedded BPE vocabulary).  Errors come back as
``{"ok": false, "error": "..."}``; the process keeps serving.
Reference behaviour: src/server/cpp_sidecar.py:59-137 (encode / parse / ping / shutdown over pipes)."""
from __future__ import annotations

import argparse
import json
import sys


def handle(req: dict, tokenizer=None) -> dict:
    op = req.get("op")
    if op == "ping":
        return {"ok": True}
    if op == "shutdown":
        return {"ok": True, "shutdown": True}
    family = req.get("family", "deepseek_v4")
    from deepseek_v4_2080ti_b200 import encoding
    enc = {"deepseek_v4": encoding.deepseek_v4, "glm_dsa": encoding.glm_dsa, "minimax_m2": encoding.minimax_m2}.get(family)
    if enc is None:
        return {"ok": False, "error": f"unknown chat family {family!r}"}
    if op == "encode":
        kw = {}
        if family == "deepseek_v4":
            kw = {"tools": req.get("tools"), "thinking": bool(req.get("thinking", False)),
                  "reasoning_effort": req.get("reasoning_effort")}
        prompt = enc.render(req.get("messages", []), **kw)
        out = {"ok": True, "prompt": prompt}
        if tokenizer is not None:
            out["token_ids"] = tokenizer.encode(prompt)
        return out
    if op == "decode":
        if tokenizer is None:
            return {"ok": False, "error": "no tokenizer: start the sidecar with --gguf"}
        text = tokenizer.decode([int(t) for t in req.get("token_ids", [])])
        out = {"ok": True, "text": text}
        if hasattr(enc, "parse_completion"):
            out["message"] = enc.parse_completion(text, thinking=bool(req.get("thinking", False)))
        return out
    if op == "parse":
        if not hasattr(enc, "parse_completion"):
            return {"ok": True, "message": {"role": "assistant", "content": req.get("text", "")}}
        return {"ok": True, "message": enc.parse_completion(req.get("text", ""), thinking=bool(req.get("thinking", False)))}
    return {"ok": False, "error": f"unknown op {op!r}"}


def main(argv=None, stdin=None, stdout=None) -> int:
    ap = argparse.ArgumentParser(prog="pocketllm-sidecar")
    ap.add_argument("--gguf", default="", help="take the tokenizer from this GGUF file's metadata")
    a = ap.parse_args(argv)
    stdin, stdout = stdin or sys.stdin, stdout or sys.stdout
    tok = None
    if a.gguf:
        from deepseek_v4_2080ti_b200.encoding.gguf_tokenizer import GGUFTokenizer
        tok = GGUFTokenizer.from_gguf(a.gguf)
    # bytes in, bytes out: a line that is not UTF-8 is answered with an error like any other bad request, whatever the
    # locale's error handler for the standard streams is; exactly one answer per line that holds anything
    raw_in = getattr(stdin, "buffer", stdin)
    raw_out = getattr(stdout, "buffer", None)
    for raw in raw_in:
        line = (raw.decode("utf-8", errors="replace") if isinstance(raw, bytes) else raw).strip()
        if not line:
            continue
        try:
            resp = handle(json.loads(line), tok)
        except Exception as exc:                       # a bad request must not end the helper
            resp = {"ok": False, "error": f"{type(exc).__name__}: {exc}"[:500]}
        text = json.dumps(resp, ensure_ascii=False) + "\n"
        if raw_out is not None:
            raw_out.write(text.encode("utf-8", errors="replace"))
            raw_out.flush()
        else:
            stdout.write(text)
            stdout.flush()
        if resp.get("shutdown"):
            break
    return 0


if __name__ == "__main__":
    sys.exit(main())
