"""GPU parity of the 128-row tensor-core time loops (Elman, head dim 64; tcgen05 + tensor memory, tensor-map bulk
copies, dR/db accumulated inside the reverse loop) against the fp64 oracle, through the public API.

The tile is forced with ``batch_tile=128`` so that small batches exercise it; ragged batches cover the rows a
tensor-map copy clips (zero-filled loads, dropped stores); batches that are a multiple of 8 take the copies of two time
steps per box, the others one step per box."""
import numpy as np
import pytest
import torch

from flashrnn_b200 import _native as nv
from tests.util import assert_parity, make_inputs, run_native, run_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("B,T,N", [(128, 5, 1), (128, 1, 2), (128, 2, 1), (130, 9, 2), (37, 12, 3), (300, 33, 2), (136, 7, 2), (264, 34, 3), (8, 3, 1)])
def test_wide_elman_matches_oracle(cuda_device, B, T, N):
    Wx, R, b, s0 = make_inputs("elman", B, T, N, 64, seed=B + T, random_init=True)
    g = torch.Generator().manual_seed(7)
    cot = torch.randn(1, B, T, N, 64, generator=g, dtype=torch.float64).to(torch.bfloat16).to(torch.float64)
    got = run_native("elman", Wx, R, b, s0, cot=cot, batch_tile=128)
    ref = run_oracle("elman", Wx, R, b, s0, cot=cot)
    errs = assert_parity("elman", got, ref, tag=f"wide B{B} T{T} N{N}")
    assert errs["h"] < 1.5e-2


def test_wide_matches_small_tile_kernels(cuda_device):
    """Same problem through the 8-row warp-MMA loops and through the 128-row tcgen05 loops."""
    Wx, R, b, s0 = make_inputs("elman", 256, 64, 4, 64, seed=3)
    a = run_native("elman", Wx, R, b, s0, batch_tile=128)
    c = run_native("elman", Wx, R, b, s0, batch_tile=8)
    assert np.abs(a["states"] - c["states"]).max() < 2e-2
    for k in ("dWx", "dR", "db"):
        den = np.linalg.norm(c[k].ravel())
        assert np.linalg.norm((a[k] - c[k]).ravel()) / den < 1e-2, k


def test_wide_is_the_default_for_large_batches():
    big = nv.query(nv.make_problem("elman", 1024, 16, 16, 64, False, True))
    assert (big.batch_tile, big.cluster_size, big.threads) == (128, 1, 160)
    small = nv.query(nv.make_problem("elman", 64, 16, 16, 64, False, True))
    assert small.batch_tile == 8
    # cells / options the 128-row loops do not cover keep the warp-MMA loops (16-row tiles for large multi-gate batches)
    assert nv.query(nv.make_problem("lstm", 1024, 16, 16, 64, False, True)).batch_tile == 16
    assert nv.query(nv.make_problem("elman", 1024, 16, 16, 64, True, True)).batch_tile == 8


@pytest.mark.parametrize("function", ["lstm", "gru"])
@pytest.mark.parametrize("B,T,N", [(128, 5, 1), (128, 1, 2), (128, 2, 1), (130, 9, 2), (37, 12, 3), (300, 33, 2), (264, 34, 3), (8, 3, 1)])
def test_wide_lstm_forward_matches_oracle(cuda_device, function, B, T, N):
    """LSTM and GRU, head dim 64: the forward loop on the 128-row tensor-core kernel (forced with batch_tile=128), the
    reverse loop on 16-row tiles that read the cache the forward loop wrote: states and every gradient against the oracle."""
    plan = nv.query(nv.make_problem(function, B, T, N, 64, False, True), 0, 128)
    assert (plan.wide_forward, plan.cluster_size, plan.batch_tile) == (1, 1, 16)
    Wx, R, b, s0 = make_inputs(function, B, T, N, 64, seed=B + T, random_init=True)
    S = s0.shape[0]
    g = torch.Generator().manual_seed(11)
    cot = torch.randn(S, B, T, N, 64, generator=g, dtype=torch.float64).to(torch.bfloat16).to(torch.float64)
    got = run_native(function, Wx, R, b, s0, cot=cot, batch_tile=128)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot)
    errs = assert_parity(function, got, ref, tag=f"wide {function} B{B} T{T} N{N}", zero_init=False)
    assert errs["h"] < 1.5e-2


def test_wide_lstm_forward_variants(cuda_device):
    """Inference (no cache), a time-major Wx read through strides, float16, and the same problem on the 16-row tiles."""
    from flashrnn_b200 import FlashRNNConfig, flashrnn

    B, T, N, D = 136, 11, 2, 64
    Wx, R, b, s0 = make_inputs("lstm", B, T, N, D, seed=17, random_init=True)
    ref = run_oracle("lstm", Wx, R, b, s0)
    a = run_native("lstm", Wx, R, b, s0, batch_tile=128)
    c = run_native("lstm", Wx, R, b, s0, batch_tile=16)
    assert np.abs(a["states"] - c["states"]).max() < 2e-2
    for k in ("dWx", "dR", "db"):
        assert np.linalg.norm((a[k] - c[k]).ravel()) / np.linalg.norm(c[k].ravel()) < 1e-2, k
    dev = [x.to(cuda_device, torch.bfloat16) for x in (Wx, R, b, s0)]
    cfg = FlashRNNConfig(function="lstm", head_dim=D, num_heads=N, batch_size=B, batch_tile=128)
    with torch.no_grad():
        inf, last = flashrnn(*dev, function="lstm", config=cfg)
    assert np.abs(inf.double().cpu().numpy() - ref["states"]).max() < 2e-2 * max(1.0, float(np.abs(ref["states"]).max()))
    assert np.abs(last.double().cpu().numpy() - ref["last"]).max() < 2e-2 * max(1.0, float(np.abs(ref["last"]).max()))
    cfg_t = FlashRNNConfig(function="lstm", head_dim=D, num_heads=N, batch_size=B, batch_tile=128, input_shape="TBGHD")
    with torch.no_grad():
        alt, _ = flashrnn(dev[0].permute(1, 0, 2, 3, 4).contiguous(), dev[1], dev[2], dev[3], function="lstm", config=cfg_t)
    assert torch.equal(inf, alt)
    for function in ("lstm", "gru"):  # forward clamp and the gradient options (the reverse loop's) on top of the 128-row forward
        Wc, Rc, bc, sc = make_inputs(function, B, T, N, D, seed=19, random_init=True)
        gotc = run_native(function, Wc, Rc, bc, sc, batch_tile=128, forward_clipval=0.4, gradient_recurrent_clipval=0.05)
        assert np.abs(gotc["states"][0]).max() <= 0.4 * (1 + 2.0 ** -8)  # the clamp value as rounded to bfloat16
        assert_parity(function, gotc, run_oracle(function, Wc, Rc, bc, sc, forward_clip=0.4, clip=0.05), tag=f"wide {function} clip",
                      zero_init=False)
    Wx16, R16, b16, s16 = make_inputs("lstm", B, T, N, D, seed=17, random_init=True, dtype=torch.float16)
    got16 = run_native("lstm", Wx16, R16, b16, s16, dtype=torch.float16, batch_tile=128)
    assert_parity("lstm", got16, run_oracle("lstm", Wx16, R16, b16, s16), tag="wide lstm f16", zero_init=False)


def test_wide_lstm_forward_is_the_default_for_large_batches():
    big = nv.query(nv.make_problem("lstm", 1024, 16, 16, 64, False, True))
    assert (big.wide_forward, big.batch_tile, big.cluster_size) == (1, 16, 1)
    assert nv.query(nv.make_problem("lstm", 64, 16, 16, 64, False, True)).wide_forward == 0
    assert nv.query(nv.make_problem("lstm", 512, 16, 16, 64, False, True)).wide_forward == 0  # 64 CTAs of 128 rows: too few
    assert nv.query(nv.make_problem("lstm", 1024, 16, 16, 64, True, True)).wide_forward == 0  # fp32 states
    assert nv.query(nv.make_problem("lstm", 1024, 16, 16, 128, False, True)).wide_forward == 0
    assert nv.query(nv.make_problem("lstm", 1024, 16, 16, 64, False, True), 1, 16).wide_forward == 0  # a forced tile
    assert nv.query(nv.make_problem("gru", 1024, 16, 16, 64, False, True)).wide_forward == 1
    assert nv.query(nv.make_problem("slstm", 1024, 16, 16, 64, False, True)).wide_forward == 0
