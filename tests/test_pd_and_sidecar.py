"""Prefill/decode phase scheduler (decode first, per-phase resources, server pause) and the JSON-lines chat sidecar."""
import io
import json
import signal

from deepseek_v4_2080ti_b200.runtime import pd_scheduler as pd
from pocketllm import sidecar


def test_decode_first_and_phase_resources():
    calls = []
    s = pd.PDScheduler({"prefill": pd.PhaseResources(cpus=(0, 1), host_threads=8, pause_server=True),
                        "decode": pd.PhaseResources(host_threads=2)}, server_pid=4242,
                       set_host_threads=lambda n: calls.append(("threads", n)),
                       set_affinity=lambda c: calls.append(("cpus", tuple(sorted(c)))),
                       send_signal=lambda pid, sig: calls.append(("sig", pid, sig)))
    a, b = s.submit([1, 2, 3], 3), s.submit([4], 2)
    order = []
    done = list(s.run(lambda r: order.append(("p", r.request_id)) or 10 + r.request_id,
                      lambda r: order.append(("d", r.request_id)) or 20 + len(r.output)))
    # request 0 prefills, then decodes to completion before request 1 is prefilled (decode queue goes first)
    assert order == [("p", 0), ("d", 0), ("d", 0), ("p", 1), ("d", 1)]
    assert [r.request_id for r in done] == [0, 1] and a.output == [10, 21, 22] and b.output == [11, 21]
    assert not s.has_work() and s.phase_switches == 4
    assert calls[:3] == [("cpus", (0, 1)), ("threads", 8), ("sig", 4242, signal.SIGSTOP)]
    assert ("sig", 4242, signal.SIGCONT) in calls and not s.server_paused
    assert pd.parse_cpu_list("0-2, 8,10-11") == (0, 1, 2, 8, 10, 11)


def test_eos_ends_a_request_early():
    s = pd.PDScheduler()
    r = s.submit([1], 10)
    done = list(s.run(lambda r: 5, lambda r: 99 if len(r.output) == 2 else 6, is_eos=lambda t: t == 99))
    assert done == [r] and r.output == [5, 6, 99] and r.phase == "done"


def test_sidecar_protocol():
    reqs = [{"op": "ping"},
            {"op": "encode", "family": "deepseek_v4", "messages": [{"role": "user", "content": "hi"}], "thinking": True},
            {"op": "parse", "family": "deepseek_v4", "text": "plan</think>answer", "thinking": True},
            {"op": "encode", "family": "glm_dsa", "messages": [{"role": "user", "content": "hi"}]},
            {"op": "nonsense"}, {"op": "encode", "family": "zzz"},
            {"op": "shutdown"}, {"op": "ping"}]
    out = io.StringIO()
    bad = "this is not json\n"
    assert sidecar.main([], stdin=io.StringIO(bad + "\n".join(json.dumps(r) for r in reqs) + "\n"), stdout=out) == 0
    lines = [json.loads(l) for l in out.getvalue().splitlines()]
    assert len(lines) == 8                                   # the request after shutdown is never read
    assert lines[0]["ok"] is False and "JSONDecodeError" in lines[0]["error"]
    assert lines[1] == {"ok": True}
    assert lines[2]["ok"] and lines[2]["prompt"].endswith("<think>") and "hi" in lines[2]["prompt"]
    assert lines[3]["message"]["reasoning_content"] == "plan" and lines[3]["message"]["content"] == "answer"
    assert lines[4]["ok"] and "[gMASK]" in lines[4]["prompt"]
    assert not lines[5]["ok"] and not lines[6]["ok"] and lines[7].get("shutdown")


def test_sidecar_answers_every_line_whatever_bytes_it_holds():
    """One answer per non-empty line, errors included: invalid UTF-8, random bytes, JSON that is not an object, nesting
    that exhausts the parser; the helper stays alive and still answers a ping afterwards."""
    import os
    import random
    import select
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    p = subprocess.Popen([sys.executable, "-m", "pocketllm.sidecar"], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                         stderr=subprocess.PIPE, env=dict(os.environ, PYTHONPATH=root))
    try:
        rng = random.Random(1)
        lines = [b'{"op":"ping"}', b"garbage", b"[1,2]", b'{"op":"encode"}', b'{"op":"encode","family":"zzz","messages":[]}',
                 b'{"op":"decode","token_ids":"abc"}', b"\xff\xfe\x00", b'{"op":' + b"[" * 50000]
        for _ in range(40):
            lines.append(bytes(rng.randrange(256) for _ in range(rng.randrange(1, 80))).replace(b"\n", b" ").replace(b"\r", b" "))
        lines.append(b'{"op":"ping"}')
        answers = []
        for l in lines:
            p.stdin.write(l + b"\n")
            p.stdin.flush()
            if not l.decode("utf-8", "replace").strip():
                continue
            ready, _, _ = select.select([p.stdout], [], [], 20)
            assert ready, f"no answer for {l[:40]!r}"
            answers.append(json.loads(p.stdout.readline()))
        assert answers[0] == {"ok": True} and answers[-1] == {"ok": True}
        assert answers[3]["ok"] is True                      # an encode request without messages renders the bare prefix
        assert all(a["ok"] is False and a["error"] for i, a in enumerate(answers[1:-1], 1) if i != 3)
        assert p.poll() is None
    finally:
        p.stdin.close()
        try:
            p.wait(timeout=10)
        except subprocess.TimeoutExpired:
            p.kill()
