"""CPU: host-side logic -- the C-ABI library loads and exports every symbol include/frnn.h declares, the
planner validates problems and picks tiles, the front end mirrors the reference's config/API.  No kernel runs."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

from flashrnn_b200 import FlashRNNConfig, _native, flashrnn
from flashrnn_b200.flashrnn import _zero_state, rnn_function_registry

ROOT = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "frnn.h").read_text()
    declared = set(re.findall(r"\b(frnn_[a-z_]+)\s*\(", header))
    assert declared == set(_native.EXPORTS), declared ^ set(_native.EXPORTS)
    L = _native.lib()
    for sym in declared:
        assert getattr(L, sym) is not None
    assert L.frnn_abi_version() == _native.ABI_VERSION


def test_struct_sizes_match_header():
    # int32 x 8 + float x 2; plan = 4 + 40 + 6*4 + 6*4 (reserved) padded to 8 + 4 * 8
    assert ctypes.sizeof(_native.FrnnProblem) == 44
    assert ctypes.sizeof(_native.FrnnPlan) == 128
    assert ctypes.sizeof(_native.FrnnFwdArgs) == 8 * 8 and ctypes.sizeof(_native.FrnnBwdArgs) == 8 * 8


@pytest.mark.parametrize("function,B,T,N,D,f32", [
    ("lstm", 4, 256, 2, 64, False), ("lstm", 16, 1024, 4, 256, False), ("gru", 32, 2048, 8, 128, False),
    ("slstm", 8, 4096, 4, 192, True), ("elman", 1024, 2048, 16, 64, False)])
def test_plan_for_benchmark_configs(function, B, T, N, D, f32):
    Gr, Gw, Gi, Gt, S = rnn_function_registry[function]["gates_states"]
    plan = _native.query(_native.make_problem(function, B, T, N, D, f32, True))
    assert plan.cluster_size * plan.units_per_cta == D
    if plan.batch_tile == 128:  # 128-row tensor-core loops: 4 row warps + 1 issuing warp, whole head in one CTA
        assert function == "elman" and (plan.cluster_size, plan.threads) == (1, 160)
    else:
        assert plan.units_per_cta % 16 == 0 and plan.threads == 2 * Gr * plan.units_per_cta
        assert plan.batch_tile in (8, 16, 32) and 1 <= plan.cluster_size <= 8
    assert plan.grads_count == Gr * N * D * D + Gt * N * D
    assert plan.workspace_bytes >= plan.grads_offset + 4 * plan.grads_count
    rows = -(-B // plan.batch_tile) * plan.batch_tile
    assert plan.cache_bytes == rows * T * plan.cache_slots * N * D * 2


def test_large_head_dims_take_the_streamed_geometry():
    for D, cs in ((512, 8), (768, 12), (1024, 16), (320, 5)):
        plan = _native.query(_native.make_problem("lstm", 8, 16, 1, D, False, True))
        assert (plan.cluster_size, plan.units_per_cta, plan.threads) == (cs, 64, 512)
    plan = _native.query(_native.make_problem("elman", 8, 16, 2, 1024, False, True))
    assert (plan.cluster_size, plan.units_per_cta, plan.threads) == (16, 64, 128)


def test_small_batch_spreads_head_large_batch_does_not():
    small = _native.query(_native.make_problem("lstm", 16, 64, 4, 256, False, True))
    large = _native.query(_native.make_problem("elman", 1024, 64, 16, 64, False, True))
    assert small.cluster_size == 8 and large.cluster_size == 1


def test_query_rejects_bad_problems():
    mk = _native.make_problem
    for prob, code in [(mk("lstm", 2, 3, 1, 40, False, True), -3), (mk("lstm", 0, 3, 1, 32, False, True), -3),
                       (mk("lstm", 2, 3, 1, 1088, False, True), -3), (mk("lstm", 2, 3, 1, 288, False, True), -3)]:
        with pytest.raises(_native.FrnnError) as e:
            _native.query(prob)
        assert e.value.code == code
    bad = mk("lstm", 2, 3, 1, 32, False, True)
    bad.cell = 9
    with pytest.raises(_native.FrnnError) as e:
        _native.query(bad)
    assert e.value.code == -2
    with pytest.raises(_native.FrnnError) as e:  # tile that does not exist: 4 gates x 256 units in one CTA
        _native.query(mk("lstm", 16, 8, 1, 256, False, True), cluster_size=1, batch_tile=16)
    assert e.value.code == -6


def test_null_and_alignment_checks_happen_before_any_launch():
    L = _native.lib()
    plan = _native.query(_native.make_problem("elman", 2, 3, 1, 32, False, True))
    args = _native.FrnnFwdArgs()  # all NULL
    assert L.frnn_forward(ctypes.byref(plan), ctypes.byref(args), None) == -1
    for i, name in enumerate(("Wx", "R", "b", "s0", "states", "cache", "workspace")):
        setattr(args, name, 4096 + 8 if name == "Wx" else 4096)
    assert L.frnn_forward(ctypes.byref(plan), ctypes.byref(args), None) == -5
    inf = _native.query(_native.make_problem("elman", 2, 3, 1, 32, False, False))
    assert L.frnn_backward(ctypes.byref(inf), ctypes.byref(_native.FrnnBwdArgs()), None) == -7
    plan.abi_version = 99
    assert L.frnn_forward(ctypes.byref(plan), ctypes.byref(args), None) == -6
    assert b"16-byte" in L.frnn_status_string(-5)


def test_config_mirrors_reference_registry():
    for fn, ref in {"lstm": (4, 4, 4, 4, 2), "slstm": (4, 4, 4, 4, 4), "gru": (3, 3, 4, 4, 1), "elman": (1, 1, 1, 1, 1)}.items():
        c = FlashRNNConfig(function=fn, head_dim=64, num_heads=2, batch_size=3)
        assert (c.num_gates_r, c.num_gates_w, c.num_gates_i, c.num_gates_t, c.num_states) == ref
        assert c.hidden_dim == 128 and c.dtype_s == "bfloat16"
    with pytest.raises(AssertionError):
        FlashRNNConfig(function="mgu")
    c = FlashRNNConfig(function="slstm", head_dim=8, num_heads=2)
    z = _zero_state(c, torch.zeros(3, 5, 4, 2, 8, dtype=torch.bfloat16))
    assert z.shape == (4, 3, 1, 2, 8) and z.dtype == torch.bfloat16 and float(z.abs().sum()) == 0.0


def test_no_cpu_fallback_and_removed_backends():
    Wx, R, b = torch.zeros(2, 3, 4, 1, 32), torch.zeros(4, 1, 32, 32), torch.zeros(4, 1, 32)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        flashrnn(Wx.bfloat16(), R.bfloat16(), b.bfloat16(), function="lstm")
    for backend in ("cuda", "triton_fused", "vanilla", "vanilla_fwbw"):
        with pytest.raises(NotImplementedError):
            flashrnn(Wx, R, b, function="lstm", backend=backend)
    with pytest.raises(ValueError):
        flashrnn(Wx, R, b, function="lstm", backend="tpu")
    with pytest.raises(NotImplementedError):
        flashrnn(Wx, R, b, function="lstm", dtype="float32")
    with pytest.raises(RuntimeError, match="no CPU fallback"):  # float16 is a kernel dtype; still no CPU path
        flashrnn(Wx.half(), R.half(), b.half(), function="lstm", dtype="float16")


def test_stepper_has_no_cpu_path_and_checks_shapes():
    from flashrnn_b200 import FlashRNNStepper
    R, b = torch.zeros(4, 1, 32, 32, dtype=torch.bfloat16), torch.zeros(4, 1, 32, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        FlashRNNStepper(R, b, function="lstm", batch_size=2)
    with pytest.raises(AssertionError):
        FlashRNNStepper(R, b, function="rnn", batch_size=2)
    plan = _native.query(_native.make_problem("lstm", 2, 1, 1, 32, False, False))
    assert plan.keep_packed_r == 0  # frnn_forward repacks R unless the caller says the workspace still holds it


def test_float16_problems_reach_the_float16_build():
    """Same tile table for both 16-bit element types; states must be of the same type or float32."""
    for fn, B, T, N, D in [("lstm", 16, 1024, 4, 256), ("elman", 1024, 2048, 16, 64), ("gru", 32, 64, 8, 128)]:
        a = _native.query(_native.make_problem(fn, B, T, N, D, False, True))
        h = _native.query(_native.make_problem(fn, B, T, N, D, False, True, f16=True))
        assert h.prob.dtype_io == _native.DTYPE_F16 and h.prob.dtype_state == _native.DTYPE_F16
        assert (a.cluster_size, a.batch_tile, a.threads, a.workspace_bytes, a.cache_bytes) == \
               (h.cluster_size, h.batch_tile, h.threads, h.workspace_bytes, h.cache_bytes)
    mixed = _native.make_problem("lstm", 8, 4, 1, 64, False, True, f16=True)
    mixed.dtype_state = _native.DTYPE_BF16
    with pytest.raises(_native.FrnnError) as e:
        _native.query(mixed)
    assert e.value.code == -4
    mixed.dtype_io, mixed.dtype_state = _native.DTYPE_BF16, _native.DTYPE_F16
    with pytest.raises(_native.FrnnError) as e:
        _native.query(mixed)
    assert e.value.code == -4


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", tmp_path / "nope.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _native.lib()
