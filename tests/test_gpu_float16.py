"""GPU parity of the float16 build of the kernels (``dtype="float16"``; every CUDA source is compiled once per 16-bit
element type) against the fp64 oracle on inputs rounded to float16 values: the four cells, 16-bit and fp32 states,
head dims that reach each dR kernel (warp MMA, tcgen05 fed by cp.async, tcgen05 fed by tensor-map copies), the
streamed kernels (D = 512), the 128-row tcgen05 loops, and the stepper.  The reference tests the same dtype list
(tests/test_lstm.py:51-139)."""
import numpy as np
import pytest
import torch

from tests.util import assert_parity, make_inputs, run_native, run_oracle

pytestmark = pytest.mark.gpu
F16 = torch.float16


@pytest.mark.parametrize("function,B,T,N,D,f32", [
    ("lstm", 16, 24, 2, 64, False), ("lstm", 8, 16, 2, 256, False), ("lstm", 5, 9, 1, 128, True),
    ("gru", 16, 20, 2, 128, False), ("gru", 9, 12, 3, 64, True),
    ("elman", 16, 32, 4, 64, False), ("elman", 7, 8, 2, 32, False),
    ("slstm", 8, 24, 2, 192, True), ("slstm", 16, 16, 2, 64, False),
    ("lstm", 4, 6, 1, 512, False),
])
def test_float16_matches_oracle(cuda_device, function, B, T, N, D, f32):
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=B + T + D, random_init=True, state_f32=f32, dtype=F16)
    S = s0.shape[0]
    g = torch.Generator().manual_seed(3)
    cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64).to(F16).to(torch.float64)
    if function == "slstm":
        cot[1:] = 0
    got = run_native(function, Wx, R, b, s0, cot=cot, state_f32=f32, dtype=F16)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot)
    assert_parity(function, got, ref, tag=f"f16 {function} B{B} T{T} N{N} D{D}", zero_init=False)


@pytest.mark.parametrize("B,T,N", [(128, 6, 2), (136, 7, 1), (37, 5, 2)])
def test_float16_wide_elman(cuda_device, B, T, N):
    Wx, R, b, s0 = make_inputs("elman", B, T, N, 64, seed=B + T, random_init=True, dtype=F16)
    g = torch.Generator().manual_seed(7)
    cot = torch.randn(1, B, T, N, 64, generator=g, dtype=torch.float64).to(F16).to(torch.float64)
    got = run_native("elman", Wx, R, b, s0, cot=cot, batch_tile=128, dtype=F16)
    ref = run_oracle("elman", Wx, R, b, s0, cot=cot)
    assert_parity("elman", got, ref, tag=f"f16 wide B{B} T{T} N{N}")


def test_float16_is_closer_than_bfloat16(cuda_device):
    """Same fp64 inputs (exactly representable in both types): the float16 run has the smaller state error."""
    Wx, R, b, s0 = make_inputs("lstm", 8, 32, 2, 128, seed=1, random_init=True)
    Wx, R, b, s0 = (x.to(torch.float16).to(torch.bfloat16).to(torch.float64) for x in (Wx, R, b, s0))
    ref = run_oracle("lstm", Wx, R, b, s0)
    e16 = np.abs(run_native("lstm", Wx, R, b, s0, dtype=F16)["states"] - ref["states"]).max()
    ebf = np.abs(run_native("lstm", Wx, R, b, s0)["states"] - ref["states"]).max()
    assert e16 < ebf


def test_float16_stepper(cuda_device):
    from flashrnn_b200 import FlashRNNStepper, flashrnn
    Wx, R, b, s0 = make_inputs("gru", 8, 6, 2, 64, seed=2, random_init=True, dtype=F16)
    to = lambda x: x.to(F16).to(cuda_device).contiguous()
    Wx, R, b, s0 = to(Wx), to(R), to(b), s0.float().to(cuda_device)
    with torch.no_grad():
        full, _ = flashrnn(Wx, R, b, states=s0, function="gru", dtype="float16")
    st = FlashRNNStepper(R, b, function="gru", batch_size=8, dtype="float16", dtype_s="float32", states=s0)
    for t in range(6):
        assert torch.equal(st.step(Wx[:, t:t + 1].contiguous()), full[:, :, t:t + 1])
