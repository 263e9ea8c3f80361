"""Shared-memory expert mailbox (two processes), shared weight arena, TQ4NC quantiser."""
import multiprocessing as mp
import os

import pytest
import torch

from deepseek_v4_2080ti_b200.components import moe_ipc, tq4nc


def _server(name, dim, topk, n):
    box = moe_ipc.MoEMailbox(name, dim, topk, max_tokens=4)
    served = moe_ipc.serve_experts(box, lambda layer, x, ids, w: x * w.sum(-1, keepdim=True) + layer + ids.sum(-1, keepdim=True).float(),
                                   readers=[0], max_requests=n)
    box.close()
    os._exit(0 if served == n else 3)


def test_mailbox_round_trips_between_processes_and_times_out():
    name = f"b200_moe_test_{os.getpid()}"
    box = moe_ipc.MoEMailbox(name, 8, 2, max_tokens=4, create=True)
    try:
        p = mp.get_context("spawn").Process(target=_server, args=(name, 8, 2, 6))
        p.start()
        for i in range(6):
            t = 1 + i % 4
            x, ids, w = torch.randn(t, 8), torch.randint(0, 16, (t, 2)), torch.rand(t, 2)
            seq = box.submit(3 + i, x, ids, w)
            out = box.wait_response(seq, timeout_s=30).clone()
            box.ack(0, seq)
            assert torch.allclose(out, x * w.sum(-1, keepdim=True) + 3 + i + ids.sum(-1, keepdim=True).float(), atol=1e-6)
        p.join(30)
        assert p.exitcode == 0
        with pytest.raises(TimeoutError):
            box.wait_response(box.submit(0, torch.zeros(1, 8), torch.zeros(1, 2), torch.zeros(1, 2)), timeout_s=0.2)
        with pytest.raises(ValueError):
            box.submit(0, torch.zeros(5, 8), torch.zeros(5, 2), torch.zeros(5, 2))
        box.stop()
        with pytest.raises(RuntimeError):
            box.wait_response(99, timeout_s=1)
        assert box.wait_request(0) is None
    finally:
        box.close(unlink=True)


def test_shared_weight_arena():
    name = f"b200_arena_test_{os.getpid()}"
    layout = [("w13", (4, 6), torch.uint8), ("scale", (4, 3), torch.float32)]
    a = moe_ipc.SharedWeightArena(name, layout, create=True)
    try:
        b = moe_ipc.SharedWeightArena(name, layout)
        with pytest.raises(TimeoutError):
            b.wait_ready(timeout_s=0.05)
        w = {"w13": torch.arange(24, dtype=torch.uint8).view(4, 6), "scale": torch.rand(4, 3)}
        a.publish(w)
        b.wait_ready(timeout_s=5)
        assert torch.equal(b.view("w13"), w["w13"]) and torch.equal(b.view("scale"), w["scale"])
        b.close()
    finally:
        a.close(unlink=True)


def test_tq4nc_round_trip_error_and_outlier_robustness():
    torch.manual_seed(0)
    x = torch.randn(64, 128)
    codes, scale = tq4nc.quantize(x)
    assert codes.shape == (64, 64) and codes.dtype == torch.uint8 and scale.dtype == torch.float16
    y = tq4nc.dequantize(codes, scale)
    rel = ((y - x).norm() / x.norm()).item()
    assert rel < 0.12, rel                                   # 16 Lloyd levels on a Gaussian: ~0.1 relative RMS error
    x2 = x.clone()
    x2[:, 5] *= 30                                          # one outlier channel
    r2 = ((tq4nc.dequantize(*tq4nc.quantize(x2)) - x2).norm() / x2.norm()).item()
    assert r2 < 0.2, r2                                      # the rotation spreads it over all components
    cb = tq4nc.codebook()
    assert cb.shape == (16,) and torch.allclose(cb, -cb.flip(0), atol=1e-5) and (cb[1:] > cb[:-1]).all()
