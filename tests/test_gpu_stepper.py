"""GPU: step-by-step decoding through FlashRNNStepper against the oracle's states (every cell, one-step and multi-step
chunks) and against the full-sequence forward of the same inputs, also when the step is replayed from a CUDA graph.  Inside one launch the
cell states that do not feed the matrix product (c, n, m) are carried in fp32 registers and only their stored copy is
rounded; across launches they pass through the state tensor.  So with float32 states the comparison is bit-exact, and
with bfloat16 states it holds to bfloat16 rounding."""
import pytest
import torch

from flashrnn_b200 import FlashRNNStepper, flashrnn
from tests.util import H_MAX_ABS, make_inputs, max_abs, run_oracle

pytestmark = pytest.mark.gpu


def _inputs(function, B, T, N, D, dev, seed):
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=seed, random_init=True)
    to = lambda x: x.to(torch.bfloat16).to(dev).contiguous()
    return to(Wx), to(R), to(b), to(s0)


def _oracle_states(function, Wx, R, b, s0):
    """fp64 oracle forward on the very values the device tensors hold."""
    from oracle import oracle_forward

    f = lambda x: x.detach().to(torch.float64).cpu().numpy()
    states, _ = oracle_forward(function, f(Wx), f(R), f(b), f(s0), slstm_global_rule=False)
    return states


def _assert_states_match_oracle(got, ref, tag):
    """the tolerance rule of tests/util.py: h to 2e-2, unbounded states relative to their size"""
    import numpy as np

    got = got.detach().to(torch.float64).cpu().numpy()
    assert max_abs(got[0], ref[0]) <= H_MAX_ABS, tag
    for s in range(1, ref.shape[0]):
        assert max_abs(got[s], ref[s]) <= H_MAX_ABS * max(1.0, float(np.abs(ref[s]).max())), (tag, s)


@pytest.mark.parametrize("function", ["lstm", "gru", "elman", "slstm"])
@pytest.mark.parametrize("chunk", [1, 4])
@pytest.mark.parametrize("dtype_s", ["float32", "bfloat16"])
def test_stepper_equals_full_sequence(cuda_device, function, chunk, dtype_s):
    B, T, N, D = 16, 12, 3, 64
    Wx, R, b, s0 = _inputs(function, B, T, N, D, cuda_device, seed=11)
    exact = dtype_s == "float32"
    if exact:
        s0 = s0.float()
    with torch.no_grad():
        full, last = flashrnn(Wx, R, b, states=s0, function=function)
    assert full.dtype == s0.dtype
    oracle = _oracle_states(function, Wx, R, b, s0)
    st = FlashRNNStepper(R, b, function=function, batch_size=B, chunk=chunk, dtype_s=dtype_s, states=s0)
    for t in range(0, T, chunk):
        out = st.step(Wx[:, t:t + chunk].contiguous())
        _assert_states_match_oracle(out, oracle[:, :, t:t + chunk], (function, chunk, t))
        ref = full[:, :, t:t + chunk]
        if exact:
            assert torch.equal(out, ref), (function, chunk, t)
        else:
            torch.testing.assert_close(out.float(), ref.float(), atol=3e-2, rtol=3e-2)
    if exact:
        assert torch.equal(st.states, last)
    st.reset()
    assert float(st.states.abs().max()) == 0.0


def test_stepper_replays_from_a_cuda_graph(cuda_device):
    B, T, N, D = 8, 10, 4, 128
    Wx, R, b, s0 = _inputs("lstm", B, T, N, D, cuda_device, seed=5)
    s0 = s0.float()
    with torch.no_grad():
        full, _ = flashrnn(Wx, R, b, states=s0, function="lstm")
    st = FlashRNNStepper(R, b, function="lstm", batch_size=B, dtype_s="float32", states=s0)
    x = torch.empty_like(Wx[:, :1]).contiguous()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):       # first call packs R; done outside the graph
        x.copy_(Wx[:, :1])
        st.step(x)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = st.step(x)
    st.reset(s0)
    for t in range(T):
        x.copy_(Wx[:, t:t + 1])
        graph.replay()
        assert torch.equal(out, full[:, :, t:t + 1]), t


@pytest.mark.parametrize("function,B,N,D,tile", [("lstm", 12, 2, 128, 0), ("slstm", 8, 1, 64, 0), ("gru", 40, 3, 64, 0),
                                                 ("elman", 136, 2, 64, 128)])
def test_last_states_output_of_the_c_abi(cuda_device, function, B, N, D, tile):
    """frnn_fwd_args.last receives states[:, :, T-1], into a separate buffer and in place over s0 (cluster kernels and
    the 128-row loops, which serve it with a strided copy)."""
    import ctypes
    from flashrnn_b200 import _native as nv
    T = 5
    Wx, R, b, s0 = _inputs(function, B, T, N, D, cuda_device, seed=9)
    S = s0.shape[0]
    plan = nv.query(nv.make_problem(function, B, T, N, D, False, False), 0, tile)
    assert plan.batch_tile == (tile or plan.batch_tile)
    states = torch.empty(S, B, T, N, D, dtype=torch.bfloat16, device=cuda_device)
    ws = torch.empty(int(plan.workspace_bytes), dtype=torch.uint8, device=cuda_device)
    last = torch.full((S, B, 1, N, D), 7.0, dtype=torch.bfloat16, device=cuda_device)
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    L = nv.lib()
    nv.check("fwd", L.frnn_forward(ctypes.byref(plan), ctypes.byref(nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(s0), P(states), None, P(ws), P(last))), stream))
    assert torch.equal(last, states[:, :, -1:])
    ref = states.clone()
    carried = s0.clone()
    nv.check("fwd", L.frnn_forward(ctypes.byref(plan), ctypes.byref(nv.FrnnFwdArgs(P(Wx), P(R), P(b), P(carried), P(states), None, P(ws), P(carried))), stream))
    assert torch.equal(states, ref) and torch.equal(carried, ref[:, :, -1:])


def test_stepper_refuses_wrong_shapes(cuda_device):
    _, R, b, _ = _inputs("gru", 4, 1, 2, 64, cuda_device, seed=1)
    st = FlashRNNStepper(R, b, function="gru", batch_size=4)
    with pytest.raises(ValueError):
        st.step(torch.zeros(4, 2, 3, 2, 64, dtype=torch.bfloat16, device=cuda_device))
    with pytest.raises(ValueError):
        FlashRNNStepper(R, b, function="lstm", batch_size=4)
