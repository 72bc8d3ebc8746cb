"""GPU: the benchmark configurations at FULL size.

C1-C4 are compared with the oracle outright, every output and every gradient of the whole batch (the oracle works
through the batch a few rows at a time; C3 and C4 take it some tens of seconds on the host cores).  C5 (1024 rows) is
too much for the CPU: there the oracle checks (i) a few rows of the full run (rows are independent, so states, dWx
and ds0 of those rows must match) and (ii) everything, dR and db included, of a 128-row full-length sub-batch forced
onto the same 128-row tensor-core loops the full configuration takes.  Size-independent properties cover the rest:
dR/db of the full batch equal the sum over batch shards (what the multi-GPU path relies on), and permuting the batch
permutes the outputs.  Inputs follow the distributions the configurations name (tests/util.py, bench.py)."""
import numpy as np
import pytest
import torch

from tests.util import GRAD_REL_L2, H_MAX_ABS, assert_parity, max_abs, rel_l2, run_oracle, run_oracle_sliced

pytestmark = pytest.mark.gpu

DIMS = {"lstm": (4, 4, 4, 2), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1), "slstm": (4, 4, 4, 4)}
#        name  cell     B     T     N   D    f32 states
CONFIGS = {
    "C1": ("lstm", 4, 256, 2, 64, False),
    "C2": ("lstm", 16, 1024, 4, 256, False),
    "C3": ("gru", 32, 2048, 8, 128, False),
    "C4": ("slstm", 8, 4096, 4, 192, True),
    "C5": ("elman", 1024, 2048, 16, 64, False),
}


def config_inputs(name, device="cuda"):
    function, B, T, N, D, f32 = CONFIGS[name]
    Gr, Gw, Gt, S = DIMS[function]
    g = torch.Generator().manual_seed(0)
    Wx = torch.randn(B, T, Gw, N, D, generator=g).to(torch.bfloat16)
    R = (torch.randn(Gr, N, D, D, generator=g) / D ** 0.5).to(torch.bfloat16)
    b = 0.1 * torch.randn(Gt, N, D, generator=g)
    if name == "C3":
        b.zero_()
    if name == "C4":
        b.zero_()
        b[1] = 3.0 + 3.0 * torch.rand(N, D, generator=g)
    b = b.to(torch.bfloat16)
    sdt = torch.float32 if f32 else torch.bfloat16
    s0 = (0.1 * torch.randn(S, B, 1, N, D, generator=g) if name == "C2" else torch.zeros(S, B, 1, N, D)).to(sdt)
    return function, [t.to(device) for t in (Wx, R, b, s0)]


def run_full(function, tensors, **cfg_kw):
    """fwd + bwd (loss = sum(h)) through the public API; tensors stay on the GPU."""
    from flashrnn_b200 import FlashRNNConfig, flashrnn

    Wx, R, b, s0 = (t.detach().clone().requires_grad_(True) for t in tensors)
    cfg = None
    if cfg_kw:
        cfg = FlashRNNConfig(function=function, head_dim=Wx.shape[4], num_heads=Wx.shape[3], batch_size=Wx.shape[0],
                             dtype_s="float32" if s0.dtype == torch.float32 else "bfloat16", **cfg_kw)
    states, last = flashrnn(Wx, R, b, s0, function=function, config=cfg)
    states[0].float().sum().backward()
    torch.cuda.synchronize()
    return dict(states=states.detach(), last=last.detach(), dWx=Wx.grad, dR=R.grad, db=b.grad, ds0=s0.grad)


def to_np(d, rows=None):
    f = lambda t: t.to(torch.float64).cpu().numpy()
    out = {k: f(v) for k, v in d.items()}
    if rows is not None:
        out["states"], out["last"], out["dWx"], out["ds0"] = (out["states"][:, rows], out["last"][:, rows], out["dWx"][rows],
                                                            out["ds0"][:, rows])
    return out


@pytest.mark.parametrize("name", ["C1", "C2", "C3", "C4"])
def test_full_size_against_oracle(cuda_device, name):
    """states, dWx, ds0 of every row and dR, db summed over the whole batch and all T steps."""
    function, tensors = config_inputs(name)
    got = to_np(run_full(function, tensors))
    ref = run_oracle_sliced(function, *tensors)
    errs = assert_parity(function, got, ref, tag=name, zero_init=(name != "C2"))
    print(name, {k: f"{v:.2e}" for k, v in errs.items()})


def test_full_length_128_row_loops_against_oracle(cuda_device):
    """C5's 128-row tensor-core loops over all 2048 steps on a 128-row sub-batch (dR accumulated in tensor memory over
    the whole sequence): every output and gradient against the oracle."""
    function, tensors = config_inputs("C5")
    Wx, R, b, s0 = tensors
    rows = 128
    sub = (Wx[:rows].contiguous(), R, b, s0[:, :rows].contiguous())
    del Wx, tensors
    got = to_np(run_full(function, sub, batch_tile=128))
    ref = run_oracle_sliced(function, *sub, rows_per_slice=32)
    errs = assert_parity(function, got, ref, tag="C5/128 rows")
    print("C5 sub-batch", {k: f"{v:.2e}" for k, v in errs.items()})


@pytest.mark.parametrize("name,rows", [("C5", 4)])
def test_full_size_batch_slice_against_oracle(cuda_device, name, rows):
    function, tensors = config_inputs(name)
    full = run_full(function, tensors)
    sl = slice(0, rows)
    got = to_np(full, rows=sl)
    Wx, R, b, s0 = (t.to(torch.float64).cpu() for t in tensors)
    ref = run_oracle(function, Wx[sl], R, b, s0[:, sl])
    S = ref["states"].shape[0]
    assert max_abs(got["states"][0], ref["states"][0]) <= H_MAX_ABS
    for s in range(1, S):
        assert max_abs(got["states"][s], ref["states"][s]) <= H_MAX_ABS * max(1.0, float(np.abs(ref["states"][s]).max()))
    assert rel_l2(got["dWx"], ref["dWx"]) <= GRAD_REL_L2
    assert rel_l2(got["ds0"][:1], ref["ds0"][:1]) <= GRAD_REL_L2


@pytest.mark.parametrize("name", ["C3", "C4", "C5"])
def test_full_size_properties(cuda_device, name):
    """(i) dR/db of the whole batch = sum over two batch shards; (ii) reversing the batch order reverses the outputs."""
    function, tensors = config_inputs(name)
    Wx, R, b, s0 = tensors
    B = Wx.shape[0]
    full = run_full(function, tensors)
    h = B // 2
    a = run_full(function, (Wx[:h], R, b, s0[:, :h]))
    c = run_full(function, (Wx[h:], R, b, s0[:, h:]))
    for k in ("dR", "db"):
        summed = a[k].float() + c[k].float()
        err = float((summed - full[k].float()).norm() / full[k].float().norm())
        assert err <= GRAD_REL_L2, (k, err)
    assert torch.equal(torch.cat([a["states"], c["states"]], dim=1), full["states"])
    del a, c
    idx = torch.arange(B - 1, -1, -1, device=Wx.device)
    rev = run_full(function, (Wx[idx].contiguous(), R, b, s0[:, idx].contiguous()))
    assert torch.equal(rev["states"][:, idx], full["states"])
    assert torch.equal(rev["dWx"][idx], full["dWx"])
