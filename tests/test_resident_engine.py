"""Resident engine command loop (runtime/resident_engine.py) against a scripted runtime: every op, and the loop
surviving commands that fail (reference: PersistentEngine's worker loop, deepseek_v4_engine.cpp:11143-11239)."""
import io
import json

from deepseek_v4_2080ti_b200.runtime.resident_engine import ResidentEngine


class FakeRuntime:
    """Next token = (sum of the sequence so far) % 97; two slots; verify accepts drafts that equal that rule."""

    def __init__(self):
        self.seqs, self.lengths = {}, [0, 0]

    def allocate(self):
        for s in (0, 1):
            if s not in self.seqs:
                self.seqs[s] = []
                self.lengths[s] = 0
                return s
        raise RuntimeError("no free slot")

    def free(self, s):
        del self.seqs[s]
        self.lengths[s] = 0

    def _next(self, s):
        return sum(self.seqs[s]) % 97

    def prefill(self, s, toks, chunk):
        if any(t < 0 for t in toks):
            raise ValueError("negative token")
        self.seqs[s] += list(toks)
        self.lengths[s] = len(self.seqs[s])
        return self._next(s)

    def decode(self, slots, toks):
        out = []
        for s, t in zip(slots, toks):
            self.seqs[s].append(t)
            self.lengths[s] += 1
            out.append(self._next(s))
        return out

    def verify(self, s, toks):
        self.seqs[s].append(toks[0])
        acc = 0
        for d in toks[1:]:
            if d != self._next(s):
                break
            self.seqs[s].append(d)
            acc += 1
        self.lengths[s] = len(self.seqs[s])
        return acc, self._next(s)


def _run(cmds):
    eng = ResidentEngine(FakeRuntime())
    out = io.StringIO()
    failed = eng.serve([json.dumps(c) if not isinstance(c, str) else c for c in cmds], out)
    return eng, failed, [json.loads(l) for l in out.getvalue().splitlines()]


def test_ops_round_trip():
    eng, failed, r = _run([{"op": "alloc"}, {"op": "alloc"}, {"op": "prefill", "slot": 0, "tokens": [1, 2, 3], "id": "a"},
                           {"op": "prefill", "slot": 1, "tokens": [10]}, {"op": "decode", "slots": [0, 1], "tokens": [6, 10]},
                           {"op": "verify", "slot": 0, "tokens": [12, 24, 48, 5]}, {"op": "stats"}, {"op": "free", "slot": 1},
                           {"op": "stop"}, {"op": "alloc"}])
    assert failed == 0 and all(x["ok"] for x in r) and len(r) == 9            # nothing after stop
    assert r[0]["slot"] == 0 and r[1]["slot"] == 1
    assert r[2] == {"ok": True, "token": 6, "length": 3, "id": "a"} and r[3]["token"] == 10
    assert r[4]["tokens"] == [12, 20]
    # sequence 0 is [1,2,3,6]; verify feeds 12 (sum 24), drafts 24 (ok -> sum 48), 48 (ok -> sum 96), 5 (wrong)
    assert r[5] == {"ok": True, "accepted": 2, "token": 96, "length": 7}
    st = r[6]["stats"]
    assert st["prefill_tokens"] == 4 and st["decode_tokens"] == 2 + 3 and st["drafted"] == 3 and st["accepted"] == 2
    assert r[6]["live_slots"] == [0, 1] and r[8] == {"ok": True, "stopped": True}


def test_loop_survives_failing_commands():
    eng, failed, r = _run([{"op": "prefill", "slot": 0, "tokens": [1]},           # not allocated
                           "this is not json", [1, 2], {"op": "launch"},
                           {"op": "alloc"}, {"op": "alloc"}, {"op": "alloc"},        # third: no free slot
                           {"op": "prefill", "slot": 0, "tokens": [-1]},            # refused before the runtime sees it
                           {"op": "decode", "slots": [0, 0], "tokens": [1, 2]},      # duplicate slot
                           {"op": "prefill", "slot": 0, "tokens": [5, 6]},           # and the engine still works
                           {"op": "reset"}, {"op": "stats"}])
    oks = [x["ok"] for x in r]
    assert oks == [False, False, False, False, True, True, False, False, False, True, True, True]
    assert failed == 7 and "not allocated" in r[0]["error"] and "JSONDecodeError" in r[1]["error"]
    assert "unknown op" in r[3]["error"] and "no free slot" in r[6]["error"] and "not a token id" in r[7]["error"]
    assert r[9]["token"] == 11 and r[11]["live_slots"] == [] and r[11]["stats"]["errors"] == 7


def test_token_ids_are_checked_against_the_vocabulary():
    class Rt(FakeRuntime):
        vocab_size = 100
    from deepseek_v4_2080ti_b200.runtime.resident_engine import ResidentEngine
    eng = ResidentEngine(Rt())
    s = eng.execute({"op": "alloc"})["slot"]
    for bad in ([100], [3, 1.5], ["7"], [True], [2 ** 31], [-2]):
        with __import__("pytest").raises(ValueError, match="not a token id"):
            eng.execute({"op": "prefill", "slot": s, "tokens": bad})
    assert eng.execute({"op": "prefill", "slot": s, "tokens": [99, 7.0]})["length"] >= 2
    with __import__("pytest").raises(ValueError, match="not a token id"):
        eng.execute({"op": "decode", "slots": [s], "tokens": [100]})
