"""GPU: failure detection without faulting the GPU.  Every cross-CTA wait in the time loops is bounded (~1 s); when
a message never arrives the waiting CTAs record it in the status block, stop waiting and let the kernel finish.  The
test hook `frnn_plan.test_drop_exchange` makes CTA 0 of every cluster withhold exactly one message; nothing traps,
hangs or reads out of bounds, and the CUDA context stays usable."""
import ctypes
import time

import pytest
import torch

from flashrnn_b200 import FlashRNNConfig, _native as nv, flashrnn
from tests.util import make_inputs

pytestmark = pytest.mark.gpu


def _inputs(device):
    return [t.to(device, torch.bfloat16) for t in make_inputs("lstm", 8, 6, 1, 128, seed=31)]


def test_forward_wait_expiry_is_reported_and_context_survives(cuda_device):
    Wx, R, b, s0 = _inputs(cuda_device)
    cfg = FlashRNNConfig(function="lstm", head_dim=128, num_heads=1, batch_size=8, check_device_status=True,
                         _test_drop_exchange=True)
    t0 = time.time()
    with pytest.raises(RuntimeError, match="device-side wait expired in the forward"):
        with torch.no_grad():
            flashrnn(Wx, R, b, s0, function="lstm", config=cfg)
    assert time.time() - t0 < 20.0  # bounded: about one second per expired wait, not a hang
    # the same problem without the hook runs clean right afterwards, in the same context
    ok = FlashRNNConfig(function="lstm", head_dim=128, num_heads=1, batch_size=8, check_device_status=True)
    with torch.no_grad():
        states, _ = flashrnn(Wx, R, b, s0, function="lstm", config=ok)
    assert torch.isfinite(states.float()).all()


def test_backward_wait_expiry_sets_the_status_word(cuda_device):
    Wx, R, b, s0 = _inputs(cuda_device)
    B, T, _, N, D = Wx.shape
    plan = nv.query(nv.make_problem("lstm", B, T, N, D, False, True))
    assert plan.cluster_size > 1
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    states = torch.zeros(2, B, T, N, D, device=cuda_device, dtype=torch.bfloat16)
    cache = torch.zeros(int(plan.cache_bytes), device=cuda_device, dtype=torch.uint8)
    ws = torch.zeros(int(plan.workspace_bytes), device=cuda_device, dtype=torch.uint8)
    L = nv.lib()
    fa = nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), P(cache), P(ws))
    nv.check("frnn_forward", L.frnn_forward(ctypes.byref(plan), ctypes.byref(fa), stream))
    st = nv.FrnnDevStatus()
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 0
    dst = torch.ones_like(states)
    dWx, ds0 = torch.zeros_like(Wx), torch.zeros_like(s0)
    ba = nv.FrnnBwdArgs(P(R), P(s0), P(states), P(cache), P(dst), P(dWx), P(ds0), P(ws))
    plan.test_drop_exchange = 1
    nv.check("frnn_backward", L.frnn_backward(ctypes.byref(plan), ctypes.byref(ba), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 1 and st.cta < plan.cluster_size * N
    plan.test_drop_exchange = 0
    nv.check("frnn_backward", L.frnn_backward(ctypes.byref(plan), ctypes.byref(ba), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 0 and torch.isfinite(dWx.float()).all()


def test_wide_loops_report_a_copy_that_never_lands(cuda_device):
    """128-row tensor-core loops: one tile copy is announced to its barrier and never issued; the issuing thread and
    the row threads give up after their bounded waits, drain what is in flight and report it."""
    Wx, R, b, s0 = [t.to(cuda_device, torch.bfloat16) for t in make_inputs("elman", 128, 8, 2, 64, seed=5)]
    bad = FlashRNNConfig(function="elman", head_dim=64, num_heads=2, batch_size=128, batch_tile=128,
                         check_device_status=True, _test_drop_exchange=True)
    t0 = time.time()
    with pytest.raises(RuntimeError, match="device-side wait expired in the forward"):
        with torch.no_grad():
            flashrnn(Wx, R, b, s0, function="elman", config=bad)
    assert time.time() - t0 < 20.0
    # backward through the C ABI: clean forward first, then the reverse loop with the hook
    B, T, _, N, D = Wx.shape
    plan = nv.query(nv.make_problem("elman", B, T, N, D, False, True), 0, 128)
    assert plan.batch_tile == 128
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    states = torch.zeros(1, B, T, N, D, device=cuda_device, dtype=torch.bfloat16)
    cache = torch.zeros(256, device=cuda_device, dtype=torch.uint8)
    ws = torch.zeros(int(plan.workspace_bytes), device=cuda_device, dtype=torch.uint8)
    L = nv.lib()
    fa = nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), P(cache), P(ws))
    nv.check("frnn_forward", L.frnn_forward(ctypes.byref(plan), ctypes.byref(fa), stream))
    st = nv.FrnnDevStatus()
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 0 and torch.isfinite(states.float()).all()
    dst = torch.ones_like(states)
    dWx, ds0 = torch.zeros_like(Wx), torch.zeros_like(s0)
    ba = nv.FrnnBwdArgs(P(R), P(s0), P(states), P(cache), P(dst), P(dWx), P(ds0), P(ws))
    plan.test_drop_exchange = 1
    nv.check("frnn_backward", L.frnn_backward(ctypes.byref(plan), ctypes.byref(ba), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 1
    plan.test_drop_exchange = 0
    nv.check("frnn_backward", L.frnn_backward(ctypes.byref(plan), ctypes.byref(ba), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 0 and torch.isfinite(dWx.float()).all()


def test_float32_cluster_loops_report_a_withheld_message(cuda_device):
    """The float32 cluster loops use the same exchange protocol: forward (h slices) and reverse loop (partial sums of dh)
    each report the message CTA 0 withholds, the kernels end, and a clean run follows in the same context."""
    Wx, R, b, s0 = [t.to(cuda_device, torch.float32) for t in make_inputs("lstm", 8, 6, 1, 128, seed=33, dtype=torch.float32)]
    B, T, _, N, D = Wx.shape
    plan = nv.query(nv.make_problem("lstm", B, T, N, D, True, True, f32=True))
    assert plan.cluster_size > 1
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(cuda_device).cuda_stream)
    states = torch.zeros(2, B, T, N, D, device=cuda_device, dtype=torch.float32)
    cache = torch.zeros(int(plan.cache_bytes), device=cuda_device, dtype=torch.uint8)
    ws = torch.zeros(int(plan.workspace_bytes), device=cuda_device, dtype=torch.uint8)
    L = nv.lib()
    fa = nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), P(cache), P(ws))
    st = nv.FrnnDevStatus()
    t0 = time.time()
    plan.test_drop_exchange = 1
    nv.check("frnn_forward", L.frnn_forward(ctypes.byref(plan), ctypes.byref(fa), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 1 and st.cta < plan.cluster_size * N * ((B + plan.batch_tile - 1) // plan.batch_tile)
    plan.test_drop_exchange = 0
    nv.check("frnn_forward", L.frnn_forward(ctypes.byref(plan), ctypes.byref(fa), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 0 and torch.isfinite(states).all()
    dst = torch.ones_like(states)
    dWx, ds0 = torch.zeros_like(Wx), torch.zeros_like(s0)
    ba = nv.FrnnBwdArgs(P(R), P(s0), P(states), P(cache), P(dst), P(dWx), P(ds0), P(ws))
    plan.test_drop_exchange = 1
    nv.check("frnn_backward", L.frnn_backward(ctypes.byref(plan), ctypes.byref(ba), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 1
    assert time.time() - t0 < 30.0  # bounded: about a second per expired wait
    plan.test_drop_exchange = 0
    nv.check("frnn_backward", L.frnn_backward(ctypes.byref(plan), ctypes.byref(ba), stream))
    nv.check("status", L.frnn_read_device_status(P(ws), stream, ctypes.byref(st)))
    assert st.code == 0 and torch.isfinite(dWx).all()


def test_wide_lstm_forward_reports_a_copy_that_never_lands(cuda_device):
    """128-row LSTM forward loop: the copy of one Wx box is announced and never issued; the issuing thread and the row
    threads give up after their bounded waits and report it; a clean run follows in the same context."""
    Wx, R, b, s0 = [t.to(cuda_device, torch.bfloat16) for t in make_inputs("lstm", 128, 8, 2, 64, seed=7)]
    bad = FlashRNNConfig(function="lstm", head_dim=64, num_heads=2, batch_size=128, batch_tile=128,
                         check_device_status=True, _test_drop_exchange=True)
    t0 = time.time()
    with pytest.raises(RuntimeError, match="device-side wait expired in the forward"):
        with torch.no_grad():
            flashrnn(Wx, R, b, s0, function="lstm", config=bad)
    assert time.time() - t0 < 20.0
    ok = FlashRNNConfig(function="lstm", head_dim=64, num_heads=2, batch_size=128, batch_tile=128, check_device_status=True)
    with torch.no_grad():
        states, _ = flashrnn(Wx, R, b, s0, function="lstm", config=ok)
    assert torch.isfinite(states.float()).all()
