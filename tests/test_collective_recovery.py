"""Recovery protocol after a peer-memory collective timed out (host side, fake runtime, no GPU): rank 0 tells the
workers, every rank re-synchronises once, the sequence is rebuilt on the library path and generation continues; a
worker that saw the failure first drops the commands rank 0 sent before it noticed."""
from pocketllm import EngineArgs, GenerationRequest, SamplingParams
from pocketllm.backends.native_backend import (NativeBackend, OP_ALLOC, OP_DECODE, OP_FREE, OP_PREFILL, OP_RECOVER,
                                               OP_STOP)


class CollectiveTimeoutError(RuntimeError):
    """Stand-in with the name the backend recognises (the real one lives next to the kernels)."""


class FlakyRuntime:
    """Echo model (next = last + 1) whose ``fail_at``-th prefill/decode call raises a collective timeout."""
    eos_token_ids = ()
    max_context = 64
    supports_sampling = False

    def __init__(self, fail_at):
        self.fail_at, self.n, self.calls, self.recovered, self.next_slot = fail_at, 0, [], 0, 0

    def _maybe_fail(self):
        self.n += 1
        if self.n == self.fail_at:
            raise CollectiveTimeoutError("device kernel reported error 4: peer flag wait expired")

    def allocate(self):
        self.next_slot += 1
        self.calls.append(("allocate", self.next_slot))
        return self.next_slot

    def free(self, slot):
        self.calls.append(("free", slot))

    def recover(self):
        self.recovered += 1
        self.calls.append(("recover",))

    def prefill_tokens(self, slot, prompt, chunk, sp):
        self.calls.append(("prefill", slot, tuple(prompt)))
        self._maybe_fail()
        return prompt[-1] + 1

    def decode_tokens(self, slots, toks, sp):
        self.calls.append(("decode", tuple(slots), tuple(toks)))
        self._maybe_fail()
        return [t + 1 for t in toks]


class Chan:
    world = 2

    def __init__(self, msgs=()):
        self.sent, self.msgs = [], list(msgs)

    def send(self, op, *payload):
        self.sent.append((op, *payload))

    def recv(self):
        return self.msgs.pop(0)


def _generate(fail_at, n=5):
    rt, ch = FlakyRuntime(fail_at), Chan()
    b = NativeBackend(EngineArgs(model="fake", tensor_parallel_size=2), runtime=rt, channel=ch)
    res = b.generate([GenerationRequest(prompt_tokens=[10, 11], sampling_params=SamplingParams(max_tokens=n))])[0]
    return res, rt, ch, b


def test_decode_timeout_rebuilds_the_sequence_and_continues():
    res, rt, ch, b = _generate(fail_at=3)           # prefill ok, decode ok, second decode fails
    assert res.token_ids == [12, 13, 14, 15, 16]      # what an undisturbed run produces
    assert rt.recovered == 1 and b._stats["collective_recoveries"] == 1
    ops = [m[0] for m in ch.sent]
    i = ops.index(OP_RECOVER)
    assert ops[i:i + 4] == [OP_RECOVER, OP_FREE, OP_ALLOC, OP_PREFILL]
    # the re-prefill carries the prompt plus everything generated before the failed step, on a fresh slot
    assert ch.sent[i + 3][1] == 2 and ch.sent[i + 3][3] == [10, 11, 12, 13]
    names = [c[0] for c in rt.calls]
    assert names[names.index("recover"):names.index("recover") + 4] == ["recover", "free", "allocate", "prefill"]


def test_prefill_timeout_recovers_too_and_a_second_failure_propagates():
    res, rt, _, _ = _generate(fail_at=1)
    assert res.token_ids == [12, 13, 14, 15, 16] and rt.recovered == 1

    class TwiceFlaky(FlakyRuntime):
        def _maybe_fail(self):
            self.n += 1
            if self.n in (2, 3):
                raise CollectiveTimeoutError("peer flag wait expired")

    rt, ch = TwiceFlaky(0), Chan()
    b = NativeBackend(EngineArgs(model="fake", tensor_parallel_size=2), runtime=rt, channel=ch)
    try:
        b.generate([GenerationRequest(prompt_tokens=[1], sampling_params=SamplingParams(max_tokens=4))])
    except CollectiveTimeoutError:
        pass
    else:
        raise AssertionError("the second timeout of one request must surface")
    assert rt.recovered == 1


def test_worker_that_fails_first_recovers_alone_and_drops_stale_commands():
    rt = FlakyRuntime(fail_at=2)                      # its first decode times out
    msgs = [(OP_ALLOC,), (OP_PREFILL, 1, 8192, [1, 2]), (OP_DECODE, 1, 3),
            (OP_DECODE, 1, 4),                        # sent by rank 0 before it noticed: stale
            (OP_RECOVER,), (OP_FREE, 1), (OP_ALLOC,), (OP_PREFILL, 2, 8192, [1, 2, 3]), (OP_DECODE, 2, 4), (OP_STOP,)]
    b = NativeBackend(EngineArgs(model="fake", tensor_parallel_size=2, tensor_parallel_rank=1), runtime=rt,
                      channel=Chan(msgs))
    b.run_worker()
    assert rt.recovered == 1                          # joined the recovery once, not again on OP_RECOVER
    assert [c[0] for c in rt.calls] == ["allocate", "prefill", "decode", "recover", "free", "allocate", "prefill",
                                        "decode"]


def test_worker_recovers_on_command_when_it_saw_no_failure():
    rt = FlakyRuntime(fail_at=0)
    msgs = [(OP_ALLOC,), (OP_PREFILL, 1, 8192, [1]), (OP_RECOVER,), (OP_FREE, 1), (OP_STOP,)]
    b = NativeBackend(EngineArgs(model="fake", tensor_parallel_size=2, tensor_parallel_rank=1), runtime=rt,
                      channel=Chan(msgs))
    b.run_worker()
    assert rt.recovered == 1 and [c[0] for c in rt.calls] == ["allocate", "prefill", "recover", "free"]
