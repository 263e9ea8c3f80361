"""Phase profiler: off by default (null scope), timed accumulation per site, NVTX-only mode does not record."""
import time

import pytest

from deepseek_v4_2080ti_b200.utils.phase_profile import PROFILER, PhaseProfiler


def test_modes_and_accumulation():
    assert not PROFILER.enabled and PROFILER.scope("x") is PROFILER.scope("y")      # one shared null context when off
    p = PhaseProfiler("timed")
    for _ in range(3):
        with p.scope("lin.qkv"):
            time.sleep(0.002)
    with p.scope("ar.mlp"):
        pass
    rep = p.report()
    assert list(rep)[0] == "lin.qkv" and rep["lin.qkv"]["calls"] == 3 and rep["ar.mlp"]["calls"] == 1
    assert rep["lin.qkv"]["ms"] >= 5.0 and abs(sum(v["share"] for v in rep.values()) - 1.0) < 1e-6
    assert "phase site=lin.qkv calls=3" in p.format()
    p.reset()
    assert p.report() == {}
    p.set_mode("range")
    with p.scope("z"):
        pass
    assert p.report() == {}
    with pytest.raises(ValueError):
        p.set_mode("loud")
