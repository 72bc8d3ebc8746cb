"""CPU: pins the oracle against golden vectors produced by the unmodified reference
(tests/golden/make_golden.py) and against torch.nn.LSTM, the reference's own external anchor
(reference tests/test_lstm.py:62-115)."""
import glob
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import cell_dims, oracle_forward, oracle_fwbw
from oracle.vanilla_port import vanilla_forward, vanilla_fwbw

GOLDEN = sorted(glob.glob(str(Path(__file__).parent / "golden" / "*.npz")))


def test_golden_files_present():
    assert len(GOLDEN) >= 16


@pytest.mark.parametrize("path", GOLDEN, ids=[Path(p).stem for p in GOLDEN])
def test_c_oracle_matches_reference_golden(path):
    z = np.load(path)
    function = Path(path).stem.split("_")[0]
    f64 = "float64" in path
    dt = np.float64 if f64 else np.float32
    tol = 1e-12 if f64 else 2e-5
    o = oracle_fwbw(function, z["Wx"], z["R"], z["b"], z["s0"], dstates=z["cot"], dlast=z["cot_last"], dtype=dt)
    for k in ("states", "last", "dWx", "dR", "db"):
        err = np.abs(o[k] - z[k]).max() / max(1e-30, np.abs(z[k]).max())
        assert err <= tol, (k, err)
    # cotangent of the initial states: the sLSTM stabiliser m is excluded (the closed form treats it as a
    # constant; the reference's own tests mask the initial-state gradient, tests/utils.py:328-333)
    n_chk = 1 if function == "slstm" else z["ds0"].shape[0]
    err = np.abs(o["ds0"][:n_chk] - z["ds0"][:n_chk]).max() / max(1e-30, np.abs(z["ds0"][:n_chk]).max())
    assert err <= tol, ("ds0", err)


@pytest.mark.parametrize("path", [p for p in GOLDEN if "float64" in p], ids=lambda p: Path(p).stem)
def test_torch_port_matches_reference_golden(path):
    z = np.load(path)
    function = Path(path).stem.split("_")[0]
    t = lambda k: torch.from_numpy(z[k])
    states, last = vanilla_forward(t("Wx"), t("R"), t("b"), t("s0"), function)
    assert np.abs(states.numpy() - z["states"]).max() <= 1e-12
    assert np.abs(last.numpy() - z["last"]).max() <= 1e-12


@pytest.mark.parametrize("function", ["lstm", "gru", "elman", "slstm"])
def test_c_oracle_matches_torch_port_autograd(function):
    Gr, Gw, Gt, S = cell_dims(function)
    g = torch.Generator().manual_seed(5)
    B, T, N, D = 3, 11, 2, 16
    Wx = torch.randn(B, T, Gw, N, D, generator=g, dtype=torch.float64)
    R = torch.randn(Gr, N, D, D, generator=g, dtype=torch.float64) / D ** 0.5
    b = 0.1 * torch.randn(Gt, N, D, generator=g, dtype=torch.float64)
    states, dWx, dR, db = vanilla_fwbw(Wx, R, b, None, function)
    o = oracle_fwbw(function, Wx.numpy(), R.numpy(), b.numpy())
    assert np.abs(o["states"] - states.numpy()).max() <= 1e-12
    for got, ref in ((o["dWx"], dWx), (o["dR"], dR), (o["db"], db)):
        assert np.abs(got - ref.numpy()).max() <= 1e-10 * max(1.0, float(ref.abs().max()))


def test_oracle_lstm_matches_torch_nn_lstm():
    """FlashRNN's LSTM gate order i,f,z,o and R[g,n,d_out,d_in] equal torch.nn.LSTM's weight_hh packing."""
    torch.manual_seed(0)
    B, T, D, I = 3, 6, 8, 5
    lstm = torch.nn.LSTM(I, D, batch_first=True).double()
    x = torch.randn(B, T, I, dtype=torch.float64)
    ref, _ = lstm(x)
    Wx = (x @ lstm.weight_ih_l0.T).reshape(B, T, 4, 1, D)
    R = lstm.weight_hh_l0.reshape(4, 1, D, D)
    b = (lstm.bias_ih_l0 + lstm.bias_hh_l0).reshape(4, 1, D)
    states, _ = oracle_forward("lstm", Wx.detach().numpy(), R.detach().numpy(), b.detach().numpy())
    assert np.abs(states[0][:, :, 0] - ref.detach().numpy()).max() <= 1e-10


def test_slstm_rules_agree_for_zero_initial_state():
    g = torch.Generator().manual_seed(2)
    Wx = torch.randn(2, 6, 4, 1, 16, generator=g, dtype=torch.float64).numpy()
    R = (torch.randn(4, 1, 16, 16, generator=g, dtype=torch.float64) / 4).numpy()
    b = np.zeros((4, 1, 16))
    a, _ = oracle_forward("slstm", Wx, R, b, slstm_global_rule=True)
    c, _ = oracle_forward("slstm", Wx, R, b, slstm_global_rule=False)
    assert np.array_equal(a, c)
