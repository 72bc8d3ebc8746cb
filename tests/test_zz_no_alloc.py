"""GPU: frnn_forward_noalloc, the forward entry point for callers that cannot allocate device memory where they
call the library (a fixed arena sized at start-up, a latency-critical loop that must not hit cudaMalloc's device
synchronisation).  Its scratch is a fixed array inside the library, shared by all calls on a device, so the test
makes different calls in a row and compares each with the regular entry point on a caller-provided workspace and
with the oracle's states.
Collected last on purpose (file name), and self-contained so that it also passes alone in a fresh process."""
import ctypes

import pytest
import torch

from flashrnn_b200 import _native as nv
from tests.util import H_MAX_ABS, make_inputs, max_abs

pytestmark = pytest.mark.gpu


def _forward_both(function, shape, training, device, dt=torch.bfloat16):
    B, T, N, D = shape
    Wx, R, b, s0 = (t.to(device, dt).contiguous() for t in make_inputs(function, B, T, N, D, seed=B + D, dtype=dt))
    S = s0.shape[0]
    prob = nv.make_problem(function, B, T, N, D, False, training, f32=dt == torch.float32)
    plan = nv.query(prob)
    P = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)
    L = nv.lib()
    out = []
    for use_noalloc in (False, True):
        states = torch.zeros(S, B, T, N, D, device=device, dtype=dt)
        cache = torch.zeros(max(16, int(plan.cache_bytes)), device=device, dtype=torch.uint8) if training else None
        if use_noalloc:
            args = nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), P(cache), None)
            nv.check("frnn_forward_noalloc", L.frnn_forward_noalloc(ctypes.byref(prob), ctypes.byref(args), stream))
        else:
            ws = torch.zeros(int(plan.workspace_bytes), device=device, dtype=torch.uint8)
            args = nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), P(cache), P(ws))
            nv.check("frnn_forward", L.frnn_forward(ctypes.byref(plan), ctypes.byref(args), stream))
        torch.cuda.synchronize(device)
        out.append((states, cache))
    from oracle import oracle_forward

    f = lambda x: x.to(torch.float64).cpu().numpy()
    ref, _ = oracle_forward(function, f(Wx), f(R), f(b), f(s0), slstm_global_rule=False)
    return out, ref


def test_noalloc_forward_matches_workspace_forward_twice(cuda_device):
    # two calls in a row on the shared scratch: different cell, shape and R each time
    # (the float32 problem keeps a transposed fp32 copy of R in the scratch: twice the bytes of the 16-bit fragments)
    for function, shape, training, dt in (("lstm", (16, 12, 2, 256), True, torch.bfloat16), ("gru", (5, 9, 3, 64), False, torch.bfloat16),
                                          ("lstm", (6, 7, 2, 128), True, torch.float32), ("lstm", (16, 12, 2, 256), True, torch.bfloat16)):
        ((ref_states, ref_cache), (got_states, got_cache)), oracle = _forward_both(function, shape, training, cuda_device, dt)
        got = got_states.to(torch.float64).cpu().numpy()
        tol = 1e-4 if dt == torch.float32 else H_MAX_ABS
        assert max_abs(got[0], oracle[0]) <= tol  # h against the oracle
        for s in range(1, oracle.shape[0]):
            assert max_abs(got[s], oracle[s]) <= tol * max(1.0, float(abs(oracle[s]).max()))
        assert float((got_states.float() - ref_states.float()).abs().max()) <= tol
        assert torch.equal(got_states, ref_states)  # same kernels, same inputs: in fact bit-identical
        if training:
            assert torch.equal(got_cache, ref_cache)


def test_noalloc_rejects_oversized_and_null(cuda_device):
    L = nv.lib()
    big = nv.make_problem("lstm", 2, 2, 64, 256, False, False)  # 4*64*256*256*2 B = 32 MiB of fragments > 8 MiB
    args = nv.FrnnFwdArgs()
    assert L.frnn_forward_noalloc(ctypes.byref(big), ctypes.byref(args), None) == -9
    assert b"limit" in L.frnn_status_string(-9)
    assert L.frnn_forward_noalloc(None, ctypes.byref(args), None) == -1
    ok = nv.make_problem("elman", 2, 2, 1, 32, False, False)
    assert L.frnn_forward_noalloc(ctypes.byref(ok), ctypes.byref(args), None) == -1  # NULL tensors: nothing launched
