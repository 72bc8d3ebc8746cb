"""PyTorch restatement of the reference's ``vanilla`` CPU backend.  TEST INFRASTRUCTURE ONLY.

The reference's CPU path is a Python loop over time in which every step is one batched matmul of the
previous ``h`` with the head's recurrent matrix, followed by an elementwise cell; the backward is plain
autograd through the unrolled loop (reference flashrnn/flashrnn/vanilla/__init__.py:20-70, cells in
vanilla/{lstm,gru,elman,slstm}.py).  This module states the same computation directly in the user
layouts so that it can (a) be timed on the host cores as the CPU baseline and (b) cross-check the C
oracle with an independent autograd backward.  It is never used by the CUDA product path.
"""
from __future__ import annotations

import torch

_DIMS = {"lstm": (4, 4, 4, 2), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1), "slstm": (4, 4, 4, 4)}


def _step(function, wx, ry, b, st):
    """One cell update.  wx[B,Gw,N,D], ry[B,Gr,N,D], b[Gt,N,D], st: tuple of S tensors [B,N,D]."""
    if function == "lstm":  # vanilla/lstm.py:16-27
        pre = wx + ry + b
        i, f, o = torch.sigmoid(pre[:, 0]), torch.sigmoid(pre[:, 1]), torch.sigmoid(pre[:, 3])
        c = f * st[1] + i * torch.tanh(pre[:, 2])
        return (o * torch.tanh(c), c)
    if function == "gru":  # vanilla/gru.py:16-29
        g = ry[:, 0] + b[0]
        r = torch.sigmoid(wx[:, 0] + ry[:, 1] + b[1])
        z = torch.sigmoid(wx[:, 1] + ry[:, 2] + b[2])
        n = torch.tanh(wx[:, 2] + b[3] + r * g)
        return (z * st[0] + (1 - z) * n,)
    if function == "elman":  # vanilla/elman.py:16-20
        return (torch.tanh(wx[:, 0] + ry[:, 0] + b[0]),)
    if function == "slstm":  # vanilla/slstm.py:14-31
        pre = wx + ry + b
        _, c, n, m = st
        lfm = torch.nn.functional.logsigmoid(pre[:, 1]) + m
        m_new = pre[:, 0] if bool(torch.all(n == 0.0)) else torch.maximum(pre[:, 0], lfm)
        i = torch.exp(pre[:, 0] - m_new)
        f = torch.exp(lfm - m_new)
        c_new = f * c + i * torch.tanh(pre[:, 2])
        n_new = torch.maximum(f * n + i, torch.ones_like(n))
        return (torch.sigmoid(pre[:, 3]) * c_new / n_new, c_new, n_new, m_new)
    raise ValueError(function)


def vanilla_forward(Wx, R, b, states=None, function="lstm"):
    """Wx[B,T,Gw,N,D], R[Gr,N,D,D], b[Gt,N,D], states[S,B,1,N,D] -> (states[S,B,T,N,D], last[S,B,1,N,D])."""
    Gr, Gw, Gt, S = _DIMS[function]
    B, T, _, N, D = Wx.shape
    if states is None:
        states = torch.zeros(S, B, 1, N, D, dtype=Wx.dtype, device=Wx.device)
    st = tuple(states[s, :, 0] for s in range(S))
    # per head: [D_in, Gr*D_out] so that h[B,N,1,D] @ Rm[N,D,Gr*D] gives all gates at once
    Rm = R.permute(1, 3, 0, 2).reshape(N, D, Gr * D)
    outs = []
    for t in range(T):
        ry = torch.matmul(st[0].unsqueeze(2), Rm).reshape(B, N, Gr, D).transpose(1, 2)
        st = _step(function, Wx[:, t], ry, b, st)
        outs.append(torch.stack(st, dim=0))
    all_states = torch.stack(outs, dim=2)  # [S,B,T,N,D]
    return all_states, all_states[:, :, -1:]


def vanilla_fwbw(Wx, R, b, states=None, function="lstm"):
    """Forward + autograd backward with loss = sum(h); returns (states, dWx, dR, db)."""
    Wx = Wx.detach().requires_grad_(True)
    R = R.detach().requires_grad_(True)
    b = b.detach().requires_grad_(True)
    out, _ = vanilla_forward(Wx, R, b, states, function)
    out[0].sum().backward()
    return out.detach(), Wx.grad, R.grad, b.grad
