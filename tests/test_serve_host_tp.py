"""The whole multi-rank serving stack on the host: ``pocketllm serve ... --device cpu -tp 2`` starts the supervisor, which
starts two rank processes; rank 0 serves HTTP and fans its commands out over the command channel, rank 1 mirrors them
in its worker loop.  The ranks are replicas (the host path needs no collective), so the tokens must be the single-rank
greedy tokens, and a signal to the supervisor must end every process."""
import json
import os
import signal
import socket
import subprocess
import sys
import time
import urllib.request

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PROMPT = [3, 17, 99, 4, 250, 31, 8, 77, 12, 5]


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _post(port, body, timeout=60):
    req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", data=json.dumps(body).encode(),
                                 headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def _children(pid):
    """Direct children of ``pid`` from /proc (no dependence on a ``ps`` binary)."""
    out = []
    for d in os.listdir("/proc"):
        if d.isdigit():
            try:
                stat = open(f"/proc/{d}/stat").read()
                if int(stat.rsplit(")", 1)[1].split()[1]) == pid:
                    out.append(int(d))
            except (OSError, ValueError, IndexError):
                pass
    return sorted(out)


def _alive(pid):
    try:
        os.kill(pid, 0)
        return True
    except OSError:
        return False


@pytest.mark.timeout(300)
def test_two_host_ranks_under_the_supervisor_serve_and_stop(tmp_path):
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import QwenHybridRef
    cfg = qh.QwenHybridConfig.tiny()
    ref = QwenHybridRef(cfg, dict(qh.synth_state(cfg, 0, "cpu", std=0.05)))
    ids, want = list(PROMPT), []
    for _ in range(6):
        want.append(int(ref.forward(torch.tensor(ids))[-1].argmax()))
        ids.append(want[-1])
    port = _free_port()
    log = open(tmp_path / "serve.log", "wb")
    proc = subprocess.Popen([sys.executable, "-m", "pocketllm", "serve", "synthetic:qwen-tiny", "--device", "cpu", "-tp", "2",
                             "--port", str(port), "--max-model-len", "128", "--speculative-method", "ngram",
                             "--tensor-parallel-rendezvous-dir", str(tmp_path), "--tensor-parallel-startup-timeout", "120"],
                            stdout=log, stderr=subprocess.STDOUT, env=dict(os.environ, PYTHONPATH=ROOT), start_new_session=True)
    try:
        deadline = time.time() + 150
        while time.time() < deadline:
            assert proc.poll() is None, (tmp_path / "serve.log").read_text()[-2000:]
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/ready", timeout=2) as r:
                    if r.status == 200:
                        break
            except OSError:
                time.sleep(0.5)
        else:
            pytest.fail("the server did not become ready:\n" + (tmp_path / "serve.log").read_text()[-2000:])
        out = _post(port, {"prompt": PROMPT, "max_tokens": 6})
        assert out["usage"]["completion_tokens"] == 6
        out2 = _post(port, {"prompt": PROMPT, "max_tokens": 6, "n": 2})        # two more sequences through both ranks
        assert len(out2["choices"]) == 2 and out2["choices"][0]["text"] == out["choices"][0]["text"]
        text = (tmp_path / "serve.log").read_text()
        assert "[rank 0] pocketllm: serving" in text                        # the supervisor relays its ranks' output
        # the ranks are children of the supervisor: find them, stop the supervisor, and see them all leave
        kids = _children(proc.pid)
        assert len(kids) == 2
        proc.send_signal(signal.SIGTERM)
        proc.wait(timeout=60)
        t0 = time.time()
        while any(_alive(k) for k in kids) and time.time() - t0 < 30:
            time.sleep(0.2)
        assert not any(_alive(k) for k in kids)
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGKILL)
        log.close()
    # the tokens: decode the byte-level text back through the same fallback tokenizer the server used
    from pocketllm.protocol.prompt import TokenizerHandle
    assert TokenizerHandle.load(None).decode(want) == out["choices"][0]["text"]


@pytest.mark.timeout(300)
def test_a_rank_that_dies_takes_the_service_down(tmp_path):
    """Failure made on the host: one rank process is killed between requests; the supervisor notices, ends the other
    rank and exits non-zero, so whatever restarts services sees the failure."""
    port = _free_port()
    log = open(tmp_path / "serve.log", "wb")
    proc = subprocess.Popen([sys.executable, "-m", "pocketllm", "serve", "synthetic:qwen-tiny", "--device", "cpu", "-tp", "2",
                             "--port", str(port), "--max-model-len", "64", "--tensor-parallel-rendezvous-dir", str(tmp_path),
                             "--tensor-parallel-startup-timeout", "120", "--tensor-parallel-shutdown-timeout", "5"],
                            stdout=log, stderr=subprocess.STDOUT, env=dict(os.environ, PYTHONPATH=ROOT), start_new_session=True)
    try:
        deadline = time.time() + 150
        while time.time() < deadline:
            assert proc.poll() is None, (tmp_path / "serve.log").read_text()[-2000:]
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/ready", timeout=2) as r:
                    if r.status == 200:
                        break
            except OSError:
                time.sleep(0.5)
        assert _post(port, {"prompt": PROMPT, "max_tokens": 2})["usage"]["completion_tokens"] == 2
        kids = _children(proc.pid)
        assert len(kids) == 2
        # the worker rank is the one that does not listen on the port: kill the child whose command line says rank 1,
        # or simply the younger one (rank 1 is started after rank 0)
        os.kill(max(kids), signal.SIGKILL)
        code = proc.wait(timeout=60)
        assert code != 0
        t0 = time.time()
        while any(_alive(k) for k in kids) and time.time() - t0 < 30:
            time.sleep(0.2)
        assert not any(_alive(k) for k in kids)
        with pytest.raises(OSError):
            urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2)
    finally:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGKILL)
        log.close()
