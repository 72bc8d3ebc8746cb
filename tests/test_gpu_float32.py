"""GPU: dtype="float32" -- the float32 loops (fp32 products on the CUDA cores, exp-based nonlinearities) against the
reference's own float32 results and against the fp64 oracle, to the tolerance the task states for fp32: 1e-4
(max-abs on the states, rel-L2 on the gradients).  The reference tests float32 on every cell
(tests/test_lstm.py:48-60); the golden files hold what its `vanilla` backend returned for float32 inputs."""
import glob
from pathlib import Path

import numpy as np
import pytest
import torch

from tests.util import make_inputs, max_abs, rel_l2, run_native, run_oracle

pytestmark = pytest.mark.gpu
TOL = 1e-4
GOLDEN32 = sorted(glob.glob(str(Path(__file__).parent / "golden" / "*_float32.npz")))


def _check(function, got, ref, tag, n_ds0=None):
    S = ref["states"].shape[0]
    for s in range(S):
        scale = max(1.0, float(np.abs(ref["states"][s]).max()))
        assert max_abs(got["states"][s], ref["states"][s]) <= TOL * scale, (tag, "state", s)
    for k in ("dWx", "dR", "db"):
        assert rel_l2(got[k], ref[k]) <= TOL, (tag, k, rel_l2(got[k], ref[k]))
    n = (1 if function == "slstm" else S) if n_ds0 is None else n_ds0
    assert rel_l2(got["ds0"][:n], ref["ds0"][:n]) <= TOL, (tag, "ds0")


@pytest.mark.parametrize("path", GOLDEN32, ids=lambda p: Path(p).stem)
def test_float32_matches_the_reference_float32_results(cuda_device, path):
    from flashrnn_b200 import flashrnn

    z = np.load(path)
    function = Path(path).stem.split("_")[0]
    t = lambda k: torch.from_numpy(z[k]).to(cuda_device)
    Wx, R, b, s0 = (t(k).requires_grad_(True) for k in ("Wx", "R", "b", "s0"))
    states, last = flashrnn(Wx, R, b, s0, function=function, dtype="float32")
    assert states.dtype == torch.float32
    ((states * t("cot")).sum() + (last * t("cot_last")).sum()).backward()
    f = lambda x: x.detach().double().cpu().numpy()
    got = dict(states=f(states), dWx=f(Wx.grad), dR=f(R.grad), db=f(b.grad), ds0=f(s0.grad))
    assert max_abs(f(last), z["last"]) <= TOL
    _check(function, got, {k: z[k].astype(np.float64) for k in ("states", "dWx", "dR", "db", "ds0")}, Path(path).stem)


@pytest.mark.parametrize("function", ["lstm", "gru", "elman", "slstm"])
@pytest.mark.parametrize("shape", [(2, 1, 1, 32), (11, 9, 3, 64), (5, 6, 2, 20), (16, 12, 2, 256), (3, 4, 1, 512), (8, 3, 1, 1024)],
                         ids=lambda s: "B%dT%dN%dD%d" % s)
def test_float32_against_the_fp64_oracle(cuda_device, function, shape):
    """Ragged batches, head dims that are no multiple of 16, heads whose R no longer fits shared memory (streamed from L2)."""
    B, T, N, D = shape
    Wx, R, b, s0 = (x.float().double() for x in make_inputs(function, B, T, N, D, seed=61 + D, random_init=(function != "slstm"),
                                                            dtype=torch.float32))
    S = s0.shape[0]
    g = torch.Generator().manual_seed(3)
    cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64).float().double()
    if function == "slstm":
        cot[1:] = 0
    got = run_native(function, Wx, R, b, s0, cot=cot, dtype=torch.float32)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot)
    _check(function, got, ref, f"{function}{shape}", n_ds0=1 if function == "slstm" else None)


def test_float32_options_layouts_and_stepper(cuda_device):
    """Clip options and gradient cut, a time-major input layout, and token-by-token decoding in float32."""
    from flashrnn_b200 import FlashRNNConfig, FlashRNNStepper, flashrnn

    B, T, N, D = 6, 8, 2, 64
    Wx, R, b, s0 = (x.float().double() for x in make_inputs("lstm", B, T, N, D, seed=71, random_init=True, dtype=torch.float32))
    got = run_native("lstm", Wx, R, b, s0, dtype=torch.float32, forward_clipval=0.5, gradient_recurrent_clipval=0.05)
    ref = run_oracle("lstm", Wx, R, b, s0, forward_clip=0.5, clip=0.05)
    _check("lstm", got, ref, "clip")
    got = run_native("lstm", Wx, R, b, s0, dtype=torch.float32, gradient_recurrent_cut=True)
    ref = run_oracle("lstm", Wx, R, b, s0, cut=True)
    _check("lstm", got, ref, "cut")
    # time-major Wx: read through strides
    dev = [x.to(cuda_device, torch.float32) for x in (Wx, R, b, s0)]
    cfg = FlashRNNConfig(function="lstm", head_dim=D, num_heads=N, batch_size=B, dtype="float32", input_shape="TBGHD")
    with torch.no_grad():
        base, _ = flashrnn(*dev, function="lstm", dtype="float32")
        alt, _ = flashrnn(dev[0].permute(1, 0, 2, 3, 4).contiguous(), dev[1], dev[2], dev[3], function="lstm", config=cfg)
    assert torch.equal(base, alt)
    ref = run_oracle("lstm", Wx, R, b, s0)
    st = FlashRNNStepper(dev[1], dev[2], function="lstm", batch_size=B, dtype="float32", states=dev[3])
    for t in range(T):
        out = st.step(dev[0][:, t:t + 1].contiguous())
        assert max_abs(out.double().cpu().numpy(), ref["states"][:, :, t:t + 1]) <= 4 * TOL


def test_float32_first_benchmark_configuration(cuda_device):
    """LSTM float32 B4 T256 N2 D64, zero initial states, seed 0, loss = sum(h): the configuration the reference runs on
    its CPU backend in float32, here in float32 on the GPU over all 256 steps."""
    B, T, N, D = 4, 256, 2, 64
    g = torch.Generator().manual_seed(0)
    Wx = torch.randn(B, T, 4, N, D, generator=g).double()
    R = (torch.randn(4, N, D, D, generator=g) / D ** 0.5).double()
    b = (0.1 * torch.randn(4, N, D, generator=g)).double()
    s0 = torch.zeros(2, B, 1, N, D, dtype=torch.float64)
    got = run_native("lstm", Wx, R, b, s0, dtype=torch.float32)
    ref = run_oracle("lstm", Wx, R, b, s0)
    _check("lstm", got, ref, "C1")


@pytest.mark.parametrize("function,D,cs,bt", [("lstm", 64, 1, 8), ("lstm", 64, 2, 4), ("lstm", 64, 4, 2), ("lstm", 64, 8, 8),
                                              ("gru", 96, 3, 0), ("gru", 128, 0, 8), ("slstm", 192, 0, 4), ("elman", 128, 0, 0),
                                              ("elman", 512, 0, 8), ("lstm", 128, 2, 8), ("slstm", 128, 4, 0), ("gru", 256, 0, 2),
                                              ("lstm", 48, 1, 0), ("lstm", 256, 0, 8), ("lstm", 256, 0, 4), ("slstm", 64, 1, 8)])
def test_float32_cluster_sizes(cuda_device, function, D, cs, bt):
    """The cluster loops at every cluster size and batch tile (0 = the preferred one): exchange of h slices forward, of
    partial sums of dh in the reverse loop; ragged batch (11 rows: the last tile is partial for every tile size)."""
    from flashrnn_b200 import _native

    B, T, N = 11, 10, 2
    plan = _native.query(_native.make_problem(function, B, T, N, D, True, True, f32=True), cs, bt)
    assert plan.cluster_size * plan.units_per_cta == D and (cs == 0 or plan.cluster_size == cs) and (bt == 0 or plan.batch_tile == bt)
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=5 + D + cs, random_init=(function != "slstm"), dtype=torch.float32)
    g = torch.Generator().manual_seed(9)
    cot = torch.randn(s0.shape[0], B, T, N, D, generator=g, dtype=torch.float64).float().double()
    if function == "slstm":
        cot[1:] = 0
    got = run_native(function, Wx, R, b, s0, cot=cot, dtype=torch.float32, cluster_size=cs, batch_tile=bt)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot)
    _check(function, got, ref, f"{function} D{D} cs{cs} bt{bt}", n_ds0=1 if function == "slstm" else None)


@pytest.mark.parametrize("function", ["lstm", "gru", "elman", "slstm"])
def test_float32_odd_head_dims(cuda_device, function):
    """Head dims on both sides of every switch of the tile table (one CTA, clusters of 2..8, R streamed from L2)."""
    for D in (4, 12, 36, 68, 100, 132, 196, 260, 324, 516):
        B, T, N = 3, 5, 2
        Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=D, random_init=(function != "slstm"), dtype=torch.float32)
        got = run_native(function, Wx, R, b, s0, dtype=torch.float32)
        ref = run_oracle(function, Wx, R, b, s0)
        _check(function, got, ref, f"{function} D{D}", n_ds0=1 if function == "slstm" else None)
