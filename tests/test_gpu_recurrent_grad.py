"""GPU parity of the parameter gradients at the edges of the tensor-map-fed dR kernel (bf16 states, head dims 128 / 192 /
256): sequences shorter than, equal to and just beyond the 64-step chunks of its copies, non-zero initial states (the
h_{-1} term that is added outside the MMA), batches that do not fill a split evenly, and the GRU whose first gate's
deltas come from a side buffer."""
import pytest
import torch

from tests.util import assert_parity, make_inputs, run_native, run_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("function,B,T,N,D", [
    ("lstm", 3, 1, 2, 128), ("lstm", 5, 64, 1, 256), ("lstm", 2, 65, 2, 128), ("lstm", 9, 130, 1, 192),
    ("gru", 4, 1, 3, 128), ("gru", 7, 63, 1, 192), ("gru", 3, 129, 2, 256),
    ("slstm", 6, 66, 1, 128), ("elman", 5, 70, 2, 256), ("elman", 11, 2, 1, 128),
])
def test_parameter_gradients_at_chunk_edges(cuda_device, function, B, T, N, D):
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=B * T + D, random_init=True)
    S = s0.shape[0]
    g = torch.Generator().manual_seed(11)
    cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64).to(torch.bfloat16).to(torch.float64)
    if function == "slstm":
        cot[3] = 0.0  # the stabiliser state has no cotangent in the closed-form backward
    got = run_native(function, Wx, R, b, s0, cot=cot)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot)
    assert_parity(function, got, ref, tag=f"{function} B{B} T{T} N{N} D{D}", zero_init=False)
