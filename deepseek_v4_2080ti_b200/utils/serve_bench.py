"""Load generator for a running OpenAI-compatible server: fixed-size token-id prompts from N concurrent clients, streamed
so that time-to-first-token is seen, one JSON line per concurrency level.

    python -m deepseek_v4_2080ti_b200.utils.serve_bench --url http://127.0.0.1:8000 --concurrency 1,2,4,8 \\
        --requests 16 --prompt-tokens 512 --max-tokens 64 [--vocab 150000] [--seed 0] [--no-stream]

Per level: requests per second, generated tokens per second (whole server), time-to-first-token and end-to-end latency
(median and p90), errors.  Counterpart of the reference's concurrent-throughput and single-request-latency harnesses
(scripts/bench_concurrent_throughput.py, bench_single_request_latency.py: 2 / 4 / 8 concurrent 16 + 32-token requests).
Uses only the standard library; token-id prompts avoid any dependence on the server's tokenizer."""
from __future__ import annotations

import argparse
import http.client
import json
import random
import sys
import threading
import time
import urllib.parse


def _quantile(xs: list[float], q: float) -> float:
    if not xs:
        return 0.0
    s = sorted(xs)
    return s[min(len(s) - 1, int(q * (len(s) - 1) + 0.5))]


def one_request(host: str, port: int, prompt: list[int], max_tokens: int, stream: bool, timeout: float,
                route: str = "/v1/completions") -> dict:
    """Returns {"ok", "ttft", "latency", "tokens", "error"}; ``ttft`` is measured at the first streamed text (or token
    ids, for a server that has no tokenizer).  The prompt travels under both spellings servers use for token ids."""
    body = json.dumps({"prompt": prompt, "prompt_token_ids": prompt, "max_tokens": max_tokens, "stream": stream, "temperature": 0})
    t0 = time.perf_counter()
    out = {"ok": False, "ttft": 0.0, "latency": 0.0, "tokens": 0, "error": ""}
    try:
        c = http.client.HTTPConnection(host, port, timeout=timeout)
        c.request("POST", route, body=body, headers={"Content-Type": "application/json"})
        r = c.getresponse()
        if r.status != 200:
            out["error"] = f"HTTP {r.status}: {r.read()[:200].decode(errors='replace')}"
            return out
        if not stream:
            data = json.loads(r.read())
            n_tok = data.get("usage", {}).get("completion_tokens")
            if n_tok is None:
                n_tok = len(data["choices"][0].get("token_ids", []))
            out.update(ok=True, tokens=int(n_tok))
            out["ttft"] = float(data.get("timings", {}).get("ttft_seconds", 0.0) or 0.0)
        else:
            first = None
            for raw in r:
                line = raw.strip()
                if not line.startswith(b"data: ") or line == b"data: [DONE]":
                    continue
                ev = json.loads(line[6:])
                if "error" in ev:
                    out["error"] = str(ev["error"].get("message", ev["error"]))[:200]
                    return out
                ch = ev["choices"][0]
                delta = ch.get("delta") or {}
                if first is None and (ch.get("text") or delta.get("content") or ch.get("token_ids")):
                    first = time.perf_counter() - t0
                if ev.get("usage"):
                    out["tokens"] = int(ev["usage"]["completion_tokens"])
                elif ch.get("token_ids") and not out["tokens"]:
                    out["tokens"] = len(ch["token_ids"])
            out.update(ok=True, ttft=first if first is not None else time.perf_counter() - t0)
        c.close()
    except (OSError, ValueError, KeyError) as exc:
        out["error"] = f"{type(exc).__name__}: {exc}"
    finally:
        out["latency"] = time.perf_counter() - t0
    return out


def run_level(host: str, port: int, concurrency: int, requests: int, prompt_tokens: int, max_tokens: int, vocab: int,
              seed: int, stream: bool = True, timeout: float = 600.0, route: str = "/v1/completions") -> dict:
    rng = random.Random(seed)
    prompts = [[rng.randrange(1, vocab) for _ in range(prompt_tokens)] for _ in range(requests)]
    results: list[dict] = []
    lock = threading.Lock()
    todo = list(range(requests))

    def worker() -> None:
        while True:
            with lock:
                if not todo:
                    return
                i = todo.pop()
            res = one_request(host, port, prompts[i], max_tokens, stream, timeout, route)
            with lock:
                results.append(res)

    t0 = time.perf_counter()
    threads = [threading.Thread(target=worker, daemon=True) for _ in range(concurrency)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    wall = time.perf_counter() - t0
    good = [r for r in results if r["ok"]]
    return {"concurrency": concurrency, "requests": requests, "ok": len(good), "errors": len(results) - len(good),
            "first_error": next((r["error"] for r in results if not r["ok"]), ""), "wall_seconds": round(wall, 4),
            "requests_per_second": round(len(good) / wall, 4) if wall > 0 else 0.0,
            "generated_tokens_per_second": round(sum(r["tokens"] for r in good) / wall, 2) if wall > 0 else 0.0,
            "ttft_median_s": round(_quantile([r["ttft"] for r in good], 0.5), 5),
            "ttft_p90_s": round(_quantile([r["ttft"] for r in good], 0.9), 5),
            "latency_median_s": round(_quantile([r["latency"] for r in good], 0.5), 5),
            "latency_p90_s": round(_quantile([r["latency"] for r in good], 0.9), 5),
            "prompt_tokens": prompt_tokens, "max_tokens": max_tokens, "stream": stream}


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--url", default="http://127.0.0.1:8000")
    ap.add_argument("--concurrency", default="1,2,4,8")
    ap.add_argument("--requests", type=int, default=16)
    ap.add_argument("--prompt-tokens", type=int, default=16)
    ap.add_argument("--max-tokens", type=int, default=32)
    ap.add_argument("--vocab", type=int, default=1000, help="token ids are drawn from [1, vocab)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-stream", action="store_true")
    ap.add_argument("--timeout", type=float, default=600.0)
    ap.add_argument("--route", default="/v1/completions", help="/v1/completions or /v1/chat/completions")
    a = ap.parse_args(argv)
    u = urllib.parse.urlparse(a.url)
    host, port = u.hostname or "127.0.0.1", u.port or 80
    base = None
    for c in [int(x) for x in a.concurrency.split(",") if x]:
        row = run_level(host, port, c, a.requests, a.prompt_tokens, a.max_tokens, a.vocab, a.seed, not a.no_stream, a.timeout,
                        a.route)
        if base is None and row["requests_per_second"]:
            base = row["requests_per_second"]
        row["speedup_vs_first_level"] = round(row["requests_per_second"] / base, 3) if base else 0.0
        print(json.dumps(row), flush=True)
        if row["errors"] == row["requests"]:
            return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
