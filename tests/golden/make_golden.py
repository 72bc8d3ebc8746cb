"""Generates the golden vectors under tests/golden/ by importing the UNMODIFIED reference.

Run where the reference checkout is available (it is not needed to run the tests):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py --reference <path to the reference checkout>

For every cell it calls the reference's public entry point ``flashrnn(Wx, R, b, states, function,
backend="vanilla", dtype=...)`` on CPU (reference flashrnn/flashrnn/flashrnn.py:1114-1135) with seeded
inputs, back-propagates a seeded random cotangent through autograd and stores inputs, outputs and
gradients in ``<cell>_<tag>.npz`` (float64 and float32 variants).  The LSTM/GRU/Elman cotangent covers
every state; the sLSTM cotangent reaches the loss through ``h`` only (the reference's own tests do the
same, tests/utils.py:318-327) because the closed-form backward treats the stabiliser ``m`` as constant.

``<cell>_fwbw_float32.npz`` (lstm, slstm) come from the reference's second CPU backend, ``backend="vanilla_fwbw"``: the
same loop with the hand-written closed-form backward (flashrnn/flashrnn/vanilla_fwbw/bw.py:19-189) instead of autograd.
That backend takes ``gradient_recurrent_clipval`` (flashrnn.py:1005-1024) but cannot run with one: its autograd
function hands the float to ``save_for_backward`` (vanilla_fwbw/fwbw.py:52-54), which raises TypeError, and
``backward_sequence`` never reads the value (bw.py:19-97).  So no CPU path of the reference applies the clip options;
the vectors here are generated without them.
"""
import argparse
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
DIMS = {"lstm": (4, 4, 4, 2), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1), "slstm": (4, 4, 4, 4)}
# (tag, B, T, N, D, random initial states?)
CASES = [("small", 3, 7, 2, 16, False), ("init", 2, 5, 3, 32, True), ("long", 2, 32, 1, 32, False)]


def make_inputs(function, B, T, N, D, random_init, dtype, seed):
    Gr, Gw, Gt, S = DIMS[function]
    g = torch.Generator().manual_seed(seed)
    Wx = torch.randn(B, T, Gw, N, D, generator=g, dtype=torch.float64)
    R = torch.randn(Gr, N, D, D, generator=g, dtype=torch.float64) / D ** 0.5
    b = 0.1 * torch.randn(Gt, N, D, generator=g, dtype=torch.float64)
    if function == "slstm":
        b[1] = 3.0 + 3.0 * torch.rand(N, D, generator=g, dtype=torch.float64)
    s0 = torch.zeros(S, B, 1, N, D, dtype=torch.float64)
    if random_init:
        s0 = 0.1 * torch.randn(S, B, 1, N, D, generator=g, dtype=torch.float64)
        if function == "slstm":
            s0[2] = s0[2].abs() + 1.0  # n >= 1 for a running sLSTM
    cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64)
    cot_last = torch.randn(S, B, 1, N, D, generator=g, dtype=torch.float64)
    if function == "slstm":
        cot[1:] = 0
        cot_last[1:] = 0
    return [x.to(dtype) for x in (Wx, R, b, s0, cot, cot_last)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the reference project (the directory that holds flashrnn/)")
    ap.add_argument("--only-fwbw", action="store_true", help="write only the vanilla_fwbw vectors")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    sys.dont_write_bytecode = True
    from flashrnn import flashrnn  # the reference, unmodified

    for function in ("lstm", "slstm"):  # closed-form backward of the reference's manual PyTorch path
        B, T, N, D = 3, 9, 2, 16
        Wx, R, b, s0, cot, cot_last = make_inputs(function, B, T, N, D, True, torch.float32, seed=2000)
        Wx.requires_grad_(True), R.requires_grad_(True), b.requires_grad_(True), s0.requires_grad_(True)
        states, last = flashrnn(Wx, R, b, s0, function=function, backend="vanilla_fwbw", dtype="float32")
        loss = (states * cot).sum() + (last * cot_last).sum()
        loss.backward()
        out = dict(Wx=Wx, R=R, b=b, s0=s0, cot=cot, cot_last=cot_last, states=states, last=last,
                   dWx=Wx.grad, dR=R.grad, db=b.grad, ds0=s0.grad)
        np.savez_compressed(HERE / f"{function}_fwbw_float32.npz", **{k: v.detach().numpy() for k, v in out.items()})
        print(function, "fwbw", tuple(states.shape), float(loss))
    if args.only_fwbw:
        return
    for function in DIMS:
        for ci, (tag, B, T, N, D, rinit) in enumerate(CASES):
            for dt, dname in ((torch.float64, "float64"), (torch.float32, "float32")):
                if dname == "float32" and tag != "small":
                    continue  # keep the fixture set small
                Wx, R, b, s0, cot, cot_last = make_inputs(function, B, T, N, D, rinit, dt, seed=1000 + 17 * ci)
                Wx.requires_grad_(True), R.requires_grad_(True), b.requires_grad_(True), s0.requires_grad_(True)
                states, last = flashrnn(Wx, R, b, s0, function=function, backend="vanilla", dtype=dname)
                loss = (states * cot).sum() + (last * cot_last).sum()
                loss.backward()
                out = dict(Wx=Wx, R=R, b=b, s0=s0, cot=cot, cot_last=cot_last, states=states, last=last,
                           dWx=Wx.grad, dR=R.grad, db=b.grad, ds0=s0.grad)
                np.savez_compressed(HERE / f"{function}_{tag}_{dname}.npz",
                                    **{k: v.detach().numpy() for k, v in out.items()})
                print(function, tag, dname, tuple(states.shape), float(loss))


if __name__ == "__main__":
    main()
