"""The reference arm's request driver against a fake engine (a script that answers like
``pocketllm_engine --qwen-persistent-stdin``): budget cut-off, partial results, engine death."""
import os
import sys
import textwrap
import time

from baseline import reference_arm as ra

FAKE = textwrap.dedent("""
    import sys, time
    load, per, die_after = float(sys.argv[1]), float(sys.argv[2]), int(sys.argv[3])
    time.sleep(load)
    n = 0
    for line in sys.stdin:
        if not line.strip():
            continue
        time.sleep(per)
        n += 1
        print(f"qwen_persistent_result=1 prompt_tokens=4 generated_tokens=2 tokens=1,2 wall={per} "
              f"prefill_seconds={per / 2} decode_seconds={per / 2}", flush=True)
        if die_after and n >= die_after:
            sys.exit(3)
""")


def _drive(tmp_path, load, per, die_after, warmup, steps, budget):
    script = tmp_path / "fake_engine.py"
    script.write_text(FAKE)
    cmd = [sys.executable, str(script), str(load), str(per), str(die_after)]
    return ra.drive_engine(cmd, dict(os.environ), "2 1 2 3 4\n", leader=True, warmup=warmup, steps=steps,
                           budget=budget, t_arm0=time.time())


def test_all_requests_fit(tmp_path):
    r = _drive(tmp_path, 0.1, 0.02, 0, warmup=3, steps=4, budget=30)
    assert r["warm_done"] == 3 and len(r["results"]) == 7 and r["why_short"] == "" and r["rc"] == 0


def test_budget_cuts_warmup_to_one_then_steps(tmp_path):
    r = _drive(tmp_path, 0.1, 0.3, 0, warmup=5, steps=20, budget=2.0)
    assert r["warm_done"] == 1
    timed = r["results"][1:]
    assert 2 <= len(timed) < 20 and "budget" in r["why_short"]
    assert r["t_done"] - r["t_arm0"] < 2.5          # stopped between requests, inside the budget
    assert ra._field(timed[0], "prefill_seconds") == 0.15


def test_engine_death_keeps_completed_results(tmp_path):
    r = _drive(tmp_path, 0.0, 0.02, 3, warmup=1, steps=10, budget=30)
    assert len(r["results"]) == 3 and r["why_short"] in ("engine exited", "engine closed its input") and r["rc"] == 3


def test_follower_is_bounded(tmp_path):
    script = tmp_path / "fake_engine.py"
    script.write_text(FAKE)
    cmd = [sys.executable, str(script), "0", "0", "0"]
    t0 = time.time()
    r = ra.drive_engine(cmd, dict(os.environ), "", leader=False, warmup=1, steps=1, budget=-89.0, t_arm0=time.time())
    assert time.time() - t0 < 20 and "rc" in r
