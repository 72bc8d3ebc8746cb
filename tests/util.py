"""Shared helpers of the parity tests: seeded inputs in the distributions the benchmark configs name,
bf16 rounding policy and the tolerance rules.

Tolerances (bf16 kernels vs the fp64 oracle run on the SAME bf16-rounded inputs):
  * h (= states[0], bounded by 1):            max-abs <= 2e-2
  * other states (c, n, m; unbounded):        max-abs <= 2e-2 * max(1, max|state|)
  * gradients dWx, dR, db, ds0:               rel-L2  <= 1e-2
"""
from __future__ import annotations

import numpy as np
import torch

from oracle import cell_dims, oracle_fwbw

H_MAX_ABS = 2e-2
GRAD_REL_L2 = 1e-2


def bf16_round(x: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    return x.to(dtype).to(torch.float64)


def make_inputs(function, B, T, N, D, seed=0, random_init=False, bias_scale=0.1, state_f32=False, dtype=torch.bfloat16):
    """fp64 tensors already rounded to values of ``dtype`` (bfloat16 or float16; states too unless ``state_f32``)."""
    rnd = lambda x: bf16_round(x, dtype)
    Gr, Gw, Gt, S = cell_dims(function)
    g = torch.Generator().manual_seed(seed)
    Wx = rnd(torch.randn(B, T, Gw, N, D, generator=g, dtype=torch.float64))
    R = rnd(torch.randn(Gr, N, D, D, generator=g, dtype=torch.float64) / D ** 0.5)
    b = bias_scale * torch.randn(Gt, N, D, generator=g, dtype=torch.float64)
    if function == "slstm":
        b[1] = 3.0 + 3.0 * torch.rand(N, D, generator=g, dtype=torch.float64)
    b = rnd(b)
    s0 = torch.zeros(S, B, 1, N, D, dtype=torch.float64)
    if random_init:
        s0 = 0.1 * torch.randn(S, B, 1, N, D, generator=g, dtype=torch.float64)
        if function == "slstm":
            s0[2] = s0[2].abs() + 1.0
        s0 = s0.to(torch.float32).to(torch.float64) if state_f32 else rnd(s0)
    return Wx, R, b, s0


def rel_l2(a, ref) -> float:
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    den = np.linalg.norm(ref.ravel())
    return float(np.linalg.norm((a - ref).ravel()) / (den if den > 0 else 1.0))


def max_abs(a, ref) -> float:
    return float(np.max(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(ref, dtype=np.float64)))) if np.size(ref) else 0.0


def run_native(function, Wx, R, b, s0, cot=None, state_f32=False, device="cuda", dtype=torch.bfloat16, **cfg_kw):
    """Runs the CUDA path through the public API; returns numpy float64 dict like oracle_fwbw."""
    from flashrnn_b200 import FlashRNNConfig, flashrnn

    name = {torch.bfloat16: "bfloat16", torch.float16: "float16", torch.float32: "float32"}[dtype]
    state_f32 = state_f32 or dtype == torch.float32
    sdt = torch.float32 if state_f32 else dtype
    Wx_d = Wx.to(device=device, dtype=dtype).requires_grad_(True)
    R_d = R.to(device=device, dtype=dtype).requires_grad_(True)
    b_d = b.to(device=device, dtype=dtype).requires_grad_(True)
    s_d = s0.to(device=device, dtype=sdt).requires_grad_(True)
    B, T, _, N, D = Wx.shape
    cfg = FlashRNNConfig(function=function, head_dim=D, num_heads=N, batch_size=B, dtype=name,
                         dtype_s="float32" if state_f32 else name, **cfg_kw)
    states, last = flashrnn(Wx_d, R_d, b_d, s_d, function=function, config=cfg)
    if cot is None:
        loss = states[0].float().sum()
    else:
        loss = (states.float() * cot.to(device=device, dtype=torch.float32)).sum()
    loss.backward()
    torch.cuda.synchronize()
    f = lambda t: t.detach().to(torch.float64).cpu().numpy()
    return dict(states=f(states), last=f(last), dWx=f(Wx_d.grad), dR=f(R_d.grad), db=f(b_d.grad), ds0=f(s_d.grad))


def run_oracle(function, Wx, R, b, s0, cot=None, clip=0.0, forward_clip=0.0, cut=False):
    return oracle_fwbw(function, Wx.numpy(), R.numpy(), b.numpy(), s0.numpy(),
                       dstates=None if cot is None else cot.numpy(), dtype=np.float64, clip=clip,
                       slstm_global_rule=False, forward_clip=forward_clip, cut=cut)


def run_oracle_sliced(function, Wx, R, b, s0, rows_per_slice=8):
    """The oracle over the whole batch, ``rows_per_slice`` batch rows at a time (rows are independent: states, dWx and
    ds0 are concatenated, dR and db summed).  Takes tensors of any dtype; each slice is widened to fp64 on its own so
    that the full-size configurations stay within a few GB of host memory."""
    B = Wx.shape[0]
    R64, b64 = R.to(torch.float64).cpu(), b.to(torch.float64).cpu()
    parts = []
    for r0 in range(0, B, rows_per_slice):
        sl = slice(r0, min(B, r0 + rows_per_slice))
        parts.append(run_oracle(function, Wx[sl].to(torch.float64).cpu(), R64, b64, s0[:, sl].to(torch.float64).cpu()))
    out = {k: np.concatenate([p[k] for p in parts], axis=1) for k in ("states", "last", "ds0")}
    out["dWx"] = np.concatenate([p["dWx"] for p in parts], axis=0)
    out["dR"] = sum(p["dR"] for p in parts)
    out["db"] = sum(p["db"] for p in parts)
    return out


def assert_parity(function, got, ref, check_ds0=True, tag="", zero_init=True):
    S = ref["states"].shape[0]
    errs = {}
    errs["h"] = max_abs(got["states"][0], ref["states"][0])
    assert errs["h"] <= H_MAX_ABS, f"{tag} h max-abs {errs['h']:.3e} > {H_MAX_ABS}"
    for s in range(1, S):
        scale = max(1.0, float(np.abs(ref["states"][s]).max()))
        e = max_abs(got["states"][s], ref["states"][s])
        errs[f"s{s}"] = e
        assert e <= H_MAX_ABS * scale, f"{tag} state {s} max-abs {e:.3e} > {H_MAX_ABS * scale:.3e}"
    for k in ("dWx", "dR", "db"):
        errs[k] = rel_l2(got[k], ref[k])
        assert errs[k] <= GRAD_REL_L2, f"{tag} {k} rel-L2 {errs[k]:.3e} > {GRAD_REL_L2}"
    if check_ds0:
        # sLSTM: the stabiliser m has no closed-form cotangent; from an all-zero initial state the first step has
        # m' = i~ and the kernels clamp f = min(1, exp(..)) like the reference's CUDA code while the PyTorch loop
        # does not, which only shows in the cotangents of the (zero) initial c and n -- the reference's own tests
        # mask the initial-state gradient for the same reason (tests/utils.py:328-333)
        n_chk = (1 if zero_init else 3) if function == "slstm" else S
        e = rel_l2(got["ds0"][:n_chk], ref["ds0"][:n_chk])
        errs["ds0"] = e
        assert e <= GRAD_REL_L2, f"{tag} ds0 rel-L2 {e:.3e} > {GRAD_REL_L2}"
    return errs
