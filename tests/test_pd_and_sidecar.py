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
