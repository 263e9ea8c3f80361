"""The serving-side batching queue: compatible requests share a batch, budgets and queue limits reject early, a failing
batch does not kill the worker."""
import threading
import time

import pytest

from pocketllm.api.errors import BackendUnavailableError, ConfigurationError
from pocketllm.api.types import GenerationRequest, SamplingParams
from pocketllm.server.batching import BatchingQueue, request_tokens


def _req(n=4, **sp):
    return GenerationRequest(prompt_tokens=list(range(1, n + 1)), sampling_params=SamplingParams(**sp))


def _submit_all(q, reqs):
    out = [None] * len(reqs)

    def go(i):
        try:
            out[i] = q.submit(reqs[i], timeout=20)
        except Exception as e:  # noqa: BLE001
            out[i] = e
    ts = [threading.Thread(target=go, args=(i,)) for i in range(len(reqs))]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    return out


def test_compatible_requests_share_a_batch_and_others_wait_their_turn():
    seen = []
    gate = threading.Event()

    def run(reqs, emit):
        gate.wait(5)
        seen.append([r.request_id for r in reqs])
        return [f"done:{r.request_id}" for r in reqs]

    q = BatchingQueue(run, max_batch=4, batch_wait_ms=200)
    a = [_req(max_tokens=8) for _ in range(3)]
    b = [_req(max_tokens=8, temperature=0.7) for _ in range(2)]
    t = threading.Thread(target=lambda: gate.set() if time.sleep(0.3) is None else None)
    t.start()
    res = _submit_all(q, a + b)
    t.join()
    assert res == [f"done:{r.request_id}" for r in a + b]
    assert sorted(map(len, seen)) == [2, 3]                     # one batch per sampling setting
    for batch in seen:
        assert set(batch) <= {r.request_id for r in a} or set(batch) <= {r.request_id for r in b}
    assert q.stats.batches == 2 and q.stats.batched_requests == 5 and q.stats.max_batch_seen == 3
    q.close()


def test_token_budget_splits_batches_and_rejects_oversized_requests():
    sizes = []
    q = BatchingQueue(lambda reqs, emit: [sizes.append(len(reqs)) or "ok" for _ in reqs], max_batch=8, batch_wait_ms=150,
                      max_total_tokens=40)
    assert request_tokens(_req(4, max_tokens=12)) == 16
    res = _submit_all(q, [_req(4, max_tokens=12) for _ in range(4)])       # 16 tokens each: two fit in 40
    assert res == ["ok"] * 4 and max(sizes) <= 2
    with pytest.raises(ConfigurationError):
        q.submit(_req(30, max_tokens=20))
    assert q.stats.rejected == 1
    q.close()
    with pytest.raises(BackendUnavailableError):
        q.submit(_req(max_tokens=4))


def test_full_queue_is_refused_and_a_failing_batch_leaves_the_worker_alive():
    hold = threading.Event()
    calls = {"n": 0}

    def run(reqs, emit):
        calls["n"] += 1
        if calls["n"] == 1:
            hold.wait(5)
            raise RuntimeError("device fell over")
        return ["ok"] * len(reqs)

    q = BatchingQueue(run, max_queue=1, max_batch=1, batch_wait_ms=0)
    first = {}
    t1 = threading.Thread(target=lambda: first.setdefault("r", _try(q, _req())))
    t1.start()
    while calls["n"] == 0:
        time.sleep(0.01)                                        # the first request is running, the queue is empty
    second = {}
    t2 = threading.Thread(target=lambda: second.setdefault("r", _try(q, _req())))
    t2.start()
    while q.stats.submitted < 2:
        time.sleep(0.01)
    with pytest.raises(BackendUnavailableError):                # one waiting already
        q.submit(_req())
    hold.set()
    t1.join(); t2.join()
    assert isinstance(first["r"], RuntimeError) and second["r"] == "ok" and q.stats.failed_batches == 1
    q.close()


def _try(q, r):
    try:
        return q.submit(r, timeout=20)
    except Exception as e:  # noqa: BLE001
        return e


def test_streaming_events_reach_only_their_request_and_env_constructor(monkeypatch):
    def run(reqs, emit):
        for step in range(3):
            for i, r in enumerate(reqs):
                emit(i, (r.request_id, step))
        return ["fin"] * len(reqs)

    q = BatchingQueue(run, max_batch=4, batch_wait_ms=100)
    r1, r2 = _req(max_tokens=4), _req(max_tokens=4)
    got = {}

    def consume(r):
        evs = []
        it = q.submit_stream(r)
        try:
            while True:
                evs.append(next(it))
        except StopIteration as stop:
            got[r.request_id] = (evs, stop.value)
    ts = [threading.Thread(target=consume, args=(r,)) for r in (r1, r2)]
    for t in ts:
        t.start()
    for t in ts:
        t.join()
    for r in (r1, r2):
        assert got[r.request_id] == ([(r.request_id, s) for s in range(3)], "fin")
    assert q.stats.batches == 1                                 # both streamed requests rode one batch
    q.close()
    monkeypatch.setenv("POCKETLLM_SERVING_MAX_BATCH", "3")
    monkeypatch.setenv("POCKETLLM_SERVING_BATCH_WAIT_MS", "7.5")
    e = BatchingQueue.from_env(lambda reqs, emit: ["x"] * len(reqs))
    assert e.max_batch == 3 and abs(e.batch_wait_s - 0.0075) < 1e-9 and e.max_queue == 32
    e.close()
