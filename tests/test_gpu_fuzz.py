"""GPU: seeded random problems (cell, shape, dtypes, options, forced or default tile) against the fp64 oracle.  Every case
is small enough for the oracle to finish in a fraction of a second; together they walk through combinations the
hand-written cases do not pair up (e.g. float16 + fp32 states + gradient clip on a ragged batch at head dim 96)."""
import os
import random

import numpy as np
import pytest
import torch

from flashrnn_b200 import _native as nv
from tests.util import assert_parity, make_inputs, max_abs, rel_l2, run_native, run_oracle

pytestmark = pytest.mark.gpu

HEAD_DIMS_16BIT = [16, 32, 64, 96, 128, 192, 256, 320]


def _case(seed):
    rnd = random.Random(seed)
    function = rnd.choice(["lstm", "gru", "elman", "slstm"])
    kind = rnd.choice(["bfloat16", "bfloat16", "float16", "float32"])
    D = rnd.choice(HEAD_DIMS_16BIT + [64, 64, 64] if kind != "float32" else [8, 20, 64, 100, 128, 192])
    B = rnd.choice([1, 3, 8, 17, 33]) if D <= 128 else rnd.choice([1, 5, 12])
    T = rnd.choice([1, 2, 5, 9, 14])
    N = rnd.choice([1, 2, 3])
    opts = {}
    if rnd.random() < 0.3:
        opts["forward_clipval"] = 0.6
    if rnd.random() < 0.3:
        opts["gradient_recurrent_clipval"] = 0.04
    if rnd.random() < 0.2:
        opts["gradient_recurrent_cut"] = True
    state_f32 = kind != "float32" and rnd.random() < 0.4
    big_tile = kind != "float32" and D == 64 and function in ("lstm", "gru", "elman") and not state_f32 and rnd.random() < 0.7
    if big_tile and function == "elman" and opts:
        big_tile = False  # the 128-row Elman loops take no clip / cut options
    return function, kind, B, T, N, D, state_f32, opts, big_tile


@pytest.mark.parametrize("seed", range(int(os.environ.get("FRNN_FUZZ_CASES", "48"))))  # more seeds: set FRNN_FUZZ_CASES
def test_random_problem_against_oracle(cuda_device, seed):
    function, kind, B, T, N, D, state_f32, opts, big_tile = _case(seed)
    dt = getattr(torch, kind)
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=1000 + seed, random_init=(function != "slstm"), state_f32=state_f32, dtype=dt)
    S = s0.shape[0]
    g = torch.Generator().manual_seed(seed)
    cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64).to(dt).to(torch.float64)
    if function == "slstm":
        cot[1:] = 0
    kw = dict(opts)
    if big_tile:
        kw["batch_tile"] = 128
    got = run_native(function, Wx, R, b, s0, cot=cot, state_f32=state_f32, dtype=dt, **kw)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot, clip=opts.get("gradient_recurrent_clipval", 0.0),
                     forward_clip=opts.get("forward_clipval", 0.0), cut=opts.get("gradient_recurrent_cut", False))
    tag = f"seed {seed}: {function} {kind} B{B} T{T} N{N} D{D} f32s={state_f32} {opts} big={big_tile}"
    if kind == "float32":
        for s in range(S):
            assert max_abs(got["states"][s], ref["states"][s]) <= 1e-4 * max(1.0, float(np.abs(ref["states"][s]).max())), tag
        for k in ("dWx", "dR", "db"):
            assert rel_l2(got[k], ref[k]) <= 1e-4, (tag, k)
    else:
        assert_parity(function, got, ref, tag=tag, zero_init=(function == "slstm"))
