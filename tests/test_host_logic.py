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
    # 8 pointers + 4 int64 strides each
    assert ctypes.sizeof(_native.FrnnFwdArgs) == 12 * 8 and ctypes.sizeof(_native.FrnnBwdArgs) == 12 * 8


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
        flashrnn(Wx, R, b, function="lstm", dtype="float64")
    with pytest.raises(RuntimeError, match="no CPU fallback"):  # float32 is a kernel dtype; still no CPU path
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


def _c_layout():
    """sizeof / offsetof of the structs in include/frnn.h as the C compiler sees them."""
    import subprocess
    import tempfile
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    src = r'''
#include <stdio.h>
#include <stddef.h>
#include "frnn.h"
#define S(t) printf(#t " %zu\n", sizeof(t))
#define O(t, f) printf(#t "." #f " %zu\n", offsetof(t, f))
int main(void) {
  S(frnn_problem); O(frnn_problem, grad_cut);
  S(frnn_plan); O(frnn_plan, prob); O(frnn_plan, probe_noop_cell); O(frnn_plan, cache_bytes); O(frnn_plan, grads_count);
  S(frnn_fwd_args); O(frnn_fwd_args, last); O(frnn_fwd_args, wx_stride);
  S(frnn_bwd_args); O(frnn_bwd_args, workspace); O(frnn_bwd_args, dstates_stride);
  S(frnn_dev_status);
  printf("abi %d\n", FRNN_ABI_VERSION);
  return 0;
}'''
    with tempfile.TemporaryDirectory() as d:
        (Path(d) / "layout.c").write_text(src)
        subprocess.run(["gcc", "-I", str(root / "include"), str(Path(d) / "layout.c"), "-o", str(Path(d) / "layout")], check=True)
        out = subprocess.run([str(Path(d) / "layout")], check=True, capture_output=True, text=True).stdout
    return {k: int(v) for k, v in (line.rsplit(" ", 1) for line in out.strip().splitlines())}


def test_ctypes_structs_mirror_the_c_header():
    c = _c_layout()
    n = _native
    assert c["abi"] == n.ABI_VERSION == n.lib().frnn_abi_version()
    for cname, cls in (("frnn_problem", n.FrnnProblem), ("frnn_plan", n.FrnnPlan), ("frnn_fwd_args", n.FrnnFwdArgs),
                       ("frnn_bwd_args", n.FrnnBwdArgs), ("frnn_dev_status", n.FrnnDevStatus)):
        assert ctypes.sizeof(cls) == c[cname], cname
    assert n.FrnnProblem.grad_cut.offset == c["frnn_problem.grad_cut"]
    assert n.FrnnPlan.prob.offset == c["frnn_plan.prob"]
    assert n.FrnnPlan.probe_noop_cell.offset == c["frnn_plan.probe_noop_cell"]
    assert n.FrnnPlan.cache_bytes.offset == c["frnn_plan.cache_bytes"]
    assert n.FrnnPlan.grads_count.offset == c["frnn_plan.grads_count"]
    assert n.FrnnFwdArgs.last.offset == c["frnn_fwd_args.last"]
    assert n.FrnnFwdArgs.wx_stride.offset == c["frnn_fwd_args.wx_stride"]
    assert n.FrnnBwdArgs.dstates_stride.offset == c["frnn_bwd_args.dstates_stride"]


def test_integration_stub_structs_have_the_header_sizes():
    """The binding INTEGRATION.md shows a maintainer (its ``class Problem`` ... lines) must describe the same bytes."""
    import re
    from pathlib import Path

    text = (Path(__file__).resolve().parent.parent / "INTEGRATION.md").read_text()
    block = re.search(r"    import ctypes, torch\n(.*?)\n\n", text, re.S)
    assert block, "stub not found in INTEGRATION.md"
    code = "import ctypes\n" + "\n".join(l[4:] for l in block.group(1).splitlines() if not l.strip().startswith("L ="))
    ns = {}
    exec(code, ns)
    c = _c_layout()
    assert ctypes.sizeof(ns["Problem"]) == c["frnn_problem"] == ctypes.sizeof(_native.FrnnProblem)
    assert ctypes.sizeof(ns["Plan"]) == c["frnn_plan"]
    assert ctypes.sizeof(ns["FwdArgs"]) == c["frnn_fwd_args"]
    assert ctypes.sizeof(ns["BwdArgs"]) == c["frnn_bwd_args"]


def test_strided_views_are_passed_through_and_everything_else_is_densified():
    ks = _native.kernel_strides
    x = torch.zeros(6, 4, 3, 2, 64, dtype=torch.bfloat16)          # stored as [T,B,G,N,D]
    v = x.permute(1, 0, 2, 3, 4)                                    # seen as [B,T,G,N,D]
    t, st = ks(v, torch.bfloat16)
    assert t.data_ptr() == x.data_ptr() and tuple(st) == (3 * 2 * 64, 4 * 3 * 2 * 64, 2 * 64, 64)
    t, st = ks(v.contiguous(), torch.bfloat16)
    assert tuple(st) == (0, 0, 0, 0)
    t, st = ks(v.float(), torch.bfloat16)                           # wrong dtype: cast + dense
    assert t.dtype == torch.bfloat16 and t.is_contiguous() and tuple(st) == (0, 0, 0, 0)
    odd = torch.zeros(4, 6, 3, 2, 36, dtype=torch.bfloat16)[..., :32]  # strides not multiples of 8 elements
    t, st = ks(odd, torch.bfloat16)
    assert t.is_contiguous() and tuple(st) == (0, 0, 0, 0)
    t, st = ks(torch.zeros(1).to(torch.bfloat16).expand(4, 6, 3, 2, 64), torch.bfloat16)  # broadcast: last stride 0
    assert t.is_contiguous() and tuple(st) == (0, 0, 0, 0)


def test_stride_validation_happens_before_any_launch():
    L = _native.lib()
    plan = _native.query(_native.make_problem("elman", 2, 3, 1, 32, False, True))
    args = _native.FrnnFwdArgs()
    for name in ("Wx", "R", "b", "s0", "states", "cache", "workspace"):
        setattr(args, name, 4096)
    args.wx_stride[0] = 100  # not a multiple of 8 elements
    assert L.frnn_forward(ctypes.byref(plan), ctypes.byref(args), None) == -5
    args.wx_stride[0] = -64
    assert L.frnn_forward(ctypes.byref(plan), ctypes.byref(args), None) == -5


def test_floor_probe_exists_for_the_benchmark_tiles_only():
    """probe_noop_cell is a measurement hook of three tiles; any other plan refuses it before launching."""
    L = _native.lib()
    plan = _native.query(_native.make_problem("elman", 2, 3, 1, 32, False, True))
    plan.probe_noop_cell = 1
    args = _native.FrnnFwdArgs()
    for name in ("Wx", "R", "b", "s0", "states", "cache", "workspace"):
        setattr(args, name, 4096)
    assert L.frnn_forward(ctypes.byref(plan), ctypes.byref(args), None) != 0


def test_float32_problems_take_the_float32_loops():
    """dtype_io = float32: clusters of CTAs with fp32 slices of R in shared memory (batch tiles of 8, 4 or 2 rows: the
    smallest whose grid still fits one wave of SMs), fp32 cache and workspace, any head_dim % 4."""
    Gr, Gt, GC = 4, 4, 4
    B, T, N, D = 5, 7, 3, 20
    plan = _native.query(_native.make_problem("lstm", B, T, N, D, True, True, f32=True))
    assert (plan.cluster_size, plan.units_per_cta, plan.batch_tile, plan.threads) == (1, D, 2, 256)
    for name, shape, tile in [("lstm", (16, 1024, 4, 256), (8, 32, 8)), ("gru", (32, 2048, 8, 128), (4, 32, 8)),
                              ("slstm", (8, 4096, 4, 192), (6, 32, 2)), ("elman", (1024, 64, 16, 64), (1, 64, 8)),
                              ("lstm", (4, 8, 1, 512), (1, 512, 8))]:  # the last one: R streamed from L2, one CTA per head
        pl = _native.query(_native.make_problem(name, *shape, True, True, f32=True))
        assert (pl.cluster_size, pl.units_per_cta, pl.batch_tile) == tile, (name, shape)
    forced = _native.query(_native.make_problem("lstm", 16, 8, 2, 64, True, True, f32=True), 4, 8)
    assert (forced.cluster_size, forced.units_per_cta, forced.batch_tile) == (4, 16, 8)
    assert plan.prob.dtype_io == _native.DTYPE_F32 and plan.prob.dtype_state == _native.DTYPE_F32
    assert plan.cache_bytes == B * T * GC * N * D * 4
    assert plan.grads_count == Gr * N * D * D + Gt * N * D and plan.workspace_bytes >= plan.grads_offset + 4 * plan.grads_count
    with pytest.raises(_native.FrnnError) as e:  # no other tile exists
        _native.query(_native.make_problem("lstm", B, T, N, D, True, True, f32=True), 2, 8)
    assert e.value.code == -6
    with pytest.raises(_native.FrnnError) as e:  # batch tiles are 8, 4 or 2 rows
        _native.query(_native.make_problem("lstm", B, T, N, D, True, True, f32=True), 1, 16)
    assert e.value.code == -6
    with pytest.raises(_native.FrnnError) as e:
        _native.query(_native.make_problem("lstm", B, T, N, 1030, True, True, f32=True))
    assert e.value.code == -3
    bad = _native.make_problem("lstm", B, T, N, D, True, True, f32=True)
    bad.dtype_state = _native.DTYPE_BF16  # fp32 inputs need fp32 states
    with pytest.raises(_native.FrnnError) as e:
        _native.query(bad)
    assert e.value.code == -4


def test_float32_tile_table_covers_every_head_dim():
    """Every head dim the float32 loops accept gets a tile whose units add up to the head, for every cell."""
    for function in ("lstm", "gru", "elman", "slstm"):
        for D in range(4, 1025, 4):
            for B in (1, 8, 100):
                plan = _native.query(_native.make_problem(function, B, 3, 2, D, True, True, f32=True))
                assert plan.cluster_size * plan.units_per_cta == D and plan.batch_tile in (2, 4, 8), (function, D, B)
                assert plan.units_per_cta <= 64 or plan.cluster_size == 1
