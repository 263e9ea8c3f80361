"""The collective protocol on CPU ranks (processes over shared memory): correctness over many epochs, a late peer, a
peer that never raises its flag (bounded wait -> CollectiveTimeoutError on the waiting ranks only), stale epochs."""
import multiprocessing as mp
import os

import numpy as np
import pytest

from deepseek_v4_2080ti_b200.parallel.shm_comm import ShmPeerComm
from deepseek_v4_2080ti_b200.parallel.tp import CollectiveTimeoutError


def _rank(name, rank, world, scenario, q):
    try:
        c = ShmPeerComm(name, rank, world, slot_elems=1024, budget_s=2.5 if scenario == "missing" else 60.0)    # generous: a loaded machine starts ranks seconds apart
        c.connect(timeout_s=180.0)                              # a loaded machine starts the ranks many seconds apart
        out = []
        for it in range(6):
            x = np.full(300 + it, float(rank + 1) * (it + 1), dtype=np.float32)
            kw = {}
            if scenario == "late" and rank == 1 and it == 2:
                kw["delay_s"] = 0.3
            if scenario == "missing" and rank == 2 and it == 3:
                kw["skip_push_to"] = {0, 1}                   # rank 2's data never becomes visible to the others
            try:
                y = c.all_reduce(x, **kw)
                out.append(("ok", float(y[0]), y.tobytes()[:16]))
            except CollectiveTimeoutError:
                out.append(("timeout", 0.0, b""))
                break
        q.put((rank, out))
        c.close()
    except Exception as exc:                                   # pragma: no cover - reported through the queue
        q.put((rank, [("error", 0.0, repr(exc).encode())]))
    q.close()
    q.join_thread()                                            # flush the feeder thread before leaving
    os._exit(0)


def _run(scenario, world=3):
    ctx = mp.get_context("spawn")      # fork from a threaded pytest process can deadlock the child
    q = ctx.Queue()
    name = f"b200_shmcomm_{os.getpid()}_{scenario}"
    ps = [ctx.Process(target=_rank, args=(name, r, world, scenario, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = dict(q.get(timeout=240) for _ in range(world))
    for p in ps:
        p.join(30)
    return res


@pytest.mark.parametrize("scenario", ["normal", "late"])
def test_all_reduce_over_epochs_is_correct_and_identical(scenario):
    res = _run(scenario)
    for it in range(6):
        want = sum((r + 1) * (it + 1) for r in range(3))
        vals = [res[r][it] for r in range(3)]
        assert all(v[0] == "ok" and v[1] == want for v in vals), (it, vals)
        assert len({v[2] for v in vals}) == 1                  # same bits on every rank


def test_missing_peer_times_out_on_the_waiting_ranks():
    res = _run("missing")
    # epochs 1..3 complete everywhere; at the 4th, ranks 0 and 1 never see rank 2's flag and give up after the budget,
    # while rank 2 (which did receive theirs) completes that epoch and then waits in vain for the next one
    for r in (0, 1):
        assert [x[0] for x in res[r]] == ["ok", "ok", "ok", "timeout"]
    assert [x[0] for x in res[2]][:4] == ["ok", "ok", "ok", "ok"] and res[2][-1][0] == "timeout"


def test_stale_flag_from_an_older_epoch_is_not_accepted():
    name = f"b200_shmcomm_{os.getpid()}_stale"
    a, b = ShmPeerComm(name, 0, 2, 64, budget_s=0.2), ShmPeerComm(name, 1, 2, 64, budget_s=0.2)
    a.connect(); b.connect()
    try:
        import struct
        # a flag left behind by epoch 1 (same parity as epoch 3) must not satisfy a wait for epoch 3
        a.epoch = b.epoch = 2
        struct.pack_into("q", a.bufs[0].buf, a._flag_off(1, 1), 1)
        with pytest.raises(CollectiveTimeoutError):
            a.all_reduce(np.ones(4, dtype=np.float32))
        with pytest.raises(ValueError):
            a.all_reduce(np.ones(65, dtype=np.float32))
    finally:
        a.close(); b.close()
