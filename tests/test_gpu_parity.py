"""GPU: the CUDA path (through the public API -> C ABI) against the fp64 oracle on identical seeded,
bf16-rounded inputs.  Shapes follow the reference's test grids (tests/test_lstm.py:9-46: small B, T in
{1,3}, several heads, plus a longer sequence) reduced to what the oracle finishes in seconds."""
import numpy as np
import pytest
import torch

from tests.util import assert_parity, make_inputs, run_native, run_oracle

pytestmark = pytest.mark.gpu

CELLS = ["lstm", "gru", "elman", "slstm"]
# (B, T, N, D)
SHAPES = [(2, 1, 1, 32), (2, 3, 2, 32), (8, 3, 4, 64), (16, 5, 2, 128), (3, 7, 2, 96), (5, 4, 1, 192), (16, 6, 2, 256),
          (64, 3, 2, 64), (19, 33, 3, 64)]


@pytest.mark.parametrize("function", CELLS)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "B%dT%dN%dD%d" % s)
def test_parity_default_tile(cuda_device, function, shape):
    B, T, N, D = shape
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=B * 131 + T * 17 + D)
    got = run_native(function, Wx, R, b, s0)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=f"{function}{shape}")


# head dim 128: tiles that do not exist -- one CTA would need more than 512 threads (a whole 3- or 4-gate head, 2 x Gr x 128)
# or, with 32-row batch tiles, more than the 227 KB of shared memory.  Named here so that no case is skipped silently.
NO_SUCH_TILE = {("lstm", 1, 8), ("lstm", 1, 32), ("lstm", 2, 32), ("gru", 1, 8), ("gru", 1, 32), ("slstm", 1, 8), ("slstm", 1, 32),
                ("slstm", 2, 32)}


@pytest.mark.parametrize("function", CELLS)
@pytest.mark.parametrize("cs,bt", [(1, 8), (2, 16), (4, 8), (8, 16), (1, 32), (2, 32)])
def test_parity_every_cluster_size(cuda_device, function, cs, bt):
    """Same answer whatever tile the plan uses (cluster exchange through DSMEM vs single CTA); a tile that cannot exist
    is refused with FRNN_ERR_PLAN before anything is launched."""
    B, T, N, D = 20, 12, 2, 128
    from flashrnn_b200 import _native

    if (function, cs, bt) in NO_SUCH_TILE:
        with pytest.raises(_native.FrnnError) as e:
            _native.query(_native.make_problem(function, B, T, N, D, False, True), cs, bt)
        assert e.value.code == -6
        return
    _native.query(_native.make_problem(function, B, T, N, D, False, True), cs, bt)
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=7, random_init=True)
    got = run_native(function, Wx, R, b, s0, cluster_size=cs, batch_tile=bt)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=f"{function} cs{cs} bt{bt}", zero_init=False)


@pytest.mark.parametrize("function", ["lstm", "gru", "slstm"])
@pytest.mark.parametrize("D,T,state_f32", [(128, 1, False), (128, 2, True), (192, 3, False), (192, 9, True), (256, 8, False),
                                           (256, 11, True)])
def test_parity_32_unit_tiles(cuda_device, function, D, T, state_f32):
    """The tile of the benchmark configurations (32 units per CTA, 8-row batch tiles, clusters of 4 / 6 / 8) with odd and
    even sequence lengths, a ragged batch, two batch tiles per head and 16-bit or fp32 states."""
    B, N, cs = 11, 2, D // 32
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=47 + T, random_init=(function != "slstm"), state_f32=state_f32)
    got = run_native(function, Wx, R, b, s0, state_f32=state_f32, cluster_size=cs, batch_tile=8)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=f"{function} D{D} T{T}", zero_init=(function == "slstm"))


@pytest.mark.parametrize("function,D", [("lstm", 64), ("gru", 64), ("slstm", 64), ("lstm", 128)])
def test_parity_large_batch_16_row_tiles(cuda_device, function, D):
    """Enough (head, batch tile) pairs to fill the GPU: the table switches the cells with three or four gates to 16-row
    batch tiles (one CTA per head up to head dim 64, clusters of 32-unit CTAs above)."""
    from flashrnn_b200 import _native

    B, T, N = 168, 5, 13  # ragged: 10.5 tiles of 16 rows
    plan = _native.query(_native.make_problem(function, B, T, N, D, False, True))
    assert plan.batch_tile == 16 and plan.units_per_cta == (64 if D == 64 else 32)
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=53, random_init=(function != "slstm"))
    got = run_native(function, Wx, R, b, s0)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=f"{function} D{D} large batch", zero_init=(function == "slstm"))


@pytest.mark.parametrize("function", CELLS)
def test_parity_16_cta_cluster(cuda_device, function):
    """Head dim 256 spread over 16 CTAs of 16 units (a non-portable cluster size; reduce-scatter backward for the
    four-gate cells)."""
    B, T, N, D = 12, 10, 2, 256
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=43, random_init=True)
    got = run_native(function, Wx, R, b, s0, cluster_size=16, batch_tile=8)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=f"{function} cs16", zero_init=False)


@pytest.mark.parametrize("function", CELLS)
def test_parity_random_cotangent_and_initial_state(cuda_device, function):
    """Random cotangent on the states (h only for sLSTM, as the reference's tests do) + random initial states."""
    B, T, N, D = 6, 9, 2, 64
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=11, random_init=True)
    S = s0.shape[0]
    g = torch.Generator().manual_seed(3)
    cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64)
    if function == "slstm":
        cot[1:] = 0
    got = run_native(function, Wx, R, b, s0, cot=cot)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot)
    assert_parity(function, got, ref, tag=function, zero_init=False)


@pytest.mark.parametrize("function", ["lstm", "slstm", "gru"])
def test_parity_fp32_states(cuda_device, function):
    """bf16 Wx/R/b with float32 states (the sLSTM benchmark configuration's dtype mix)."""
    B, T, N, D = 8, 40, 2, 192 if function == "slstm" else 64
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=13, random_init=(function != "slstm"), state_f32=True)
    got = run_native(function, Wx, R, b, s0, state_f32=True)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=function, zero_init=(function == "slstm"))


@pytest.mark.parametrize("function", CELLS)
def test_long_sequence_drift(cuda_device, function):
    """Error stays inside the tolerance over a long sequence (the recurrence runs in fp32 on chip)."""
    B, T, N, D = 4, 512, 1, 64
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=21)
    got = run_native(function, Wx, R, b, s0)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=function)


@pytest.mark.parametrize("function", CELLS)
@pytest.mark.parametrize("shape", [(8, 5, 1, 512), (2, 3, 2, 1024), (16, 4, 1, 384), (8, 3, 1, 768)],
                         ids=lambda s: "B%dT%dN%dD%d" % s)
def test_parity_large_head_dim(cuda_device, function, shape):
    """Head dims above 256 (the reference's grids go to 1024, tests/test_lstm.py:9-14): R no longer fits the registers
    of a cluster and is partly streamed from L2 every step; clusters of up to 16 CTAs."""
    B, T, N, D = shape
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=29 + D, random_init=True)
    got = run_native(function, Wx, R, b, s0)
    ref = run_oracle(function, Wx, R, b, s0)
    assert_parity(function, got, ref, tag=f"{function}{shape}", zero_init=False)


@pytest.mark.parametrize("function", CELLS)
def test_clip_options(cuda_device, function):
    """forward_clipval clamps the new h; gradient_recurrent_clipval clamps the recurrent cotangent
    (reference flashrnn.py:131-136).  The bounds are chosen so that both clamps bite."""
    B, T, N, D = 8, 12, 2, 64
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=17)
    got = run_native(function, Wx, R, b, s0, forward_clipval=0.5, gradient_recurrent_clipval=0.05)
    ref = run_oracle(function, Wx, R, b, s0, forward_clip=0.5, clip=0.05)
    unclipped = run_oracle(function, Wx, R, b, s0, forward_clip=0.5)
    assert np.abs(ref["dWx"] - unclipped["dWx"]).max() > 1e-4  # the gradient clamp is active too
    assert float(np.abs(got["states"][0]).max()) <= 0.5 + 1e-6
    assert float(np.abs(ref["states"][0]).max()) == pytest.approx(0.5)  # the clamp is active in this case
    assert_parity(function, got, ref, tag=function)


@pytest.mark.parametrize("function", CELLS)
def test_gradient_recurrent_cut(cuda_device, function):
    """gradient_recurrent_cut drops the R^T delta term of the backward recurrence (truncated BPTT of depth 1,
    reference fused/flashrnn_fused_backward_cut.cu:89-178); dR/db are still formed from the deltas."""
    B, T, N, D = 8, 10, 2, 64
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=19, random_init=True)
    got = run_native(function, Wx, R, b, s0, gradient_recurrent_cut=True)
    ref = run_oracle(function, Wx, R, b, s0, cut=True)
    full = run_oracle(function, Wx, R, b, s0)
    assert np.abs(ref["dWx"] - full["dWx"]).max() > 1e-3  # the option changes the gradients
    assert_parity(function, got, ref, tag=function, zero_init=False)


def test_alternative_user_layouts(cuda_device):
    """input_shape / recurrent_shape / bias_shape / output_shape other than the defaults (reference flashrnn.py:165-173)
    give the same numbers, delivered in the requested layouts, gradients included."""
    from flashrnn_b200 import FlashRNNConfig, flashrnn

    B, T, N, D = 4, 6, 2, 64
    cpu_inputs = make_inputs("lstm", B, T, N, D, seed=23, random_init=True)
    oracle = run_oracle("lstm", *cpu_inputs)
    Wx, R, b, s0 = (t.to("cuda", torch.bfloat16) for t in cpu_inputs)
    base = [t.clone().requires_grad_(True) for t in (Wx, R, b, s0)]
    ref_states, ref_last = flashrnn(*base[:3], base[3], function="lstm")
    ref_states[0].float().sum().backward()
    cfg = FlashRNNConfig(function="lstm", head_dim=D, num_heads=N, batch_size=B, input_shape="TBGHD",
                         recurrent_shape="HGDP", bias_shape="HGD", output_shape="STBHD")
    alt = [Wx.permute(1, 0, 2, 3, 4).contiguous().requires_grad_(True), R.permute(1, 0, 2, 3).contiguous().requires_grad_(True),
           b.permute(1, 0, 2).contiguous().requires_grad_(True), s0.permute(0, 2, 1, 3, 4).contiguous().requires_grad_(True)]
    states, last = flashrnn(alt[0], alt[1], alt[2], alt[3], function="lstm", config=cfg)
    assert states.shape == (2, T, B, N, D) and last.shape == (2, 1, B, N, D)
    assert torch.equal(states.permute(0, 2, 1, 3, 4), ref_states) and torch.equal(last.permute(0, 2, 1, 3, 4), ref_last)
    states[0].float().sum().backward()
    assert torch.equal(alt[0].grad.permute(1, 0, 2, 3, 4), base[0].grad)
    assert torch.allclose(alt[1].grad.permute(1, 0, 2, 3).float(), base[1].grad.float(), atol=1e-2, rtol=1e-2)
    assert torch.allclose(alt[2].grad.permute(1, 0, 2).float(), base[2].grad.float(), atol=1e-2, rtol=1e-2)
    # and against the oracle, after mapping the alternative layouts back
    f = lambda x: x.detach().to(torch.float64).cpu().numpy()
    got = dict(states=f(states.permute(0, 2, 1, 3, 4)), last=f(last.permute(0, 2, 1, 3, 4)), dWx=f(alt[0].grad.permute(1, 0, 2, 3, 4)),
               dR=f(alt[1].grad.permute(1, 0, 2, 3)), db=f(alt[2].grad.permute(1, 0, 2)), ds0=f(alt[3].grad.permute(0, 2, 1, 3, 4)))
    assert_parity("lstm", got, oracle, tag="alternative layouts", zero_init=False)


def test_strided_inputs_through_the_c_abi(cuda_device):
    """Wx stored time-major and the cotangent stored state-time-batch-major reach the kernels through
    frnn_fwd_args.wx_stride / frnn_bwd_args.dstates_stride (no dense copy) and give the oracle's numbers: the
    cluster kernels (lstm) and the 128-row tensor-core loops (elman, with and without two-step copies)."""
    import ctypes
    from flashrnn_b200 import _native as nv

    for function, (B, T, N, D), tile in (("lstm", (10, 7, 2, 128), 0), ("elman", (136, 6, 2, 64), 128), ("elman", (131, 5, 2, 64), 128)):
        cpu = make_inputs(function, B, T, N, D, seed=31, random_init=True)
        S = cpu[3].shape[0]
        g = torch.Generator().manual_seed(5)
        cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64).to(torch.bfloat16).to(torch.float64)
        ref = run_oracle(function, *cpu, cot=cot)
        Wx, R, b, s0 = (t.to("cuda", torch.bfloat16).contiguous() for t in cpu)
        Wx_tm = Wx.permute(1, 0, 2, 3, 4).contiguous()                        # memory order [T,B,G,N,D]
        cot_tm = cot.to("cuda", torch.bfloat16).permute(0, 2, 1, 3, 4).contiguous()  # memory order [S,T,B,N,D]
        wx_view, ds_view = Wx_tm.permute(1, 0, 2, 3, 4), cot_tm.permute(0, 2, 1, 3, 4)
        plan = nv.query(nv.make_problem(function, B, T, N, D, False, True), 0, tile)
        states = torch.empty(S, B, T, N, D, device="cuda", dtype=torch.bfloat16)
        cache = torch.empty(max(16, int(plan.cache_bytes)), device="cuda", dtype=torch.uint8)
        ws = torch.empty(int(plan.workspace_bytes), device="cuda", dtype=torch.uint8)
        dWx, ds0, dR, db = torch.empty_like(Wx), torch.empty_like(s0), torch.empty_like(R), torch.empty_like(b)
        P = lambda t: ctypes.c_void_p(t.data_ptr())
        strides = lambda t: (ctypes.c_int64 * 4)(*t.stride()[:4])
        sp = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        L = nv.lib()
        fa = nv.FrnnFwdArgs(P(wx_view), P(R), P(b), P(s0), P(states), P(cache), P(ws), None, strides(wx_view))
        ba = nv.FrnnBwdArgs(P(R), P(s0), P(states), P(cache), P(ds_view), P(dWx), P(ds0), P(ws), strides(ds_view))
        nv.check("fwd", L.frnn_forward(ctypes.byref(plan), ctypes.byref(fa), sp))
        nv.check("bwd", L.frnn_backward(ctypes.byref(plan), ctypes.byref(ba), sp))
        off, cnt = int(plan.grads_offset), int(plan.grads_count)
        nv.check("cast", L.frnn_finalize_grads(ctypes.byref(plan), P(ws[off:off + 4 * cnt]), P(dR), P(db), sp))
        torch.cuda.synchronize()
        f = lambda x: x.to(torch.float64).cpu().numpy()
        got = dict(states=f(states), last=f(states[:, :, -1:]), dWx=f(dWx), dR=f(dR), db=f(db), ds0=f(ds0))
        assert_parity(function, got, ref, tag=f"strided {function} B{B}", zero_init=False)


def test_autocast_behaves_like_the_reference_decorators(cuda_device):
    """Under torch.autocast float32 inputs are computed in the kernel dtype (what the reference's
    custom_fwd(cast_inputs=...) does, flashrnn.py:690-695) and the gradients come back as float32."""
    from flashrnn_b200 import flashrnn

    cpu = make_inputs("lstm", 4, 6, 2, 64, seed=37)
    a32 = [t.to("cuda", torch.float32).requires_grad_(True) for t in cpu[:3]]
    a16 = [t.to("cuda", torch.bfloat16).requires_grad_(True) for t in cpu[:3]]
    with torch.autocast("cuda", dtype=torch.bfloat16):
        s32, _ = flashrnn(*a32, function="lstm")
        s32[0].float().sum().backward()
    # float32 Wx makes the states float32 (dtype_s follows dtype_w, as in the reference's config); same thing spelled out:
    s16, _ = flashrnn(*a16, states=torch.zeros(2, 4, 1, 2, 64, device="cuda"), function="lstm")
    s16[0].float().sum().backward()
    assert s32.dtype == torch.float32 and torch.equal(s32, s16)
    for x32, x16 in zip(a32, a16):
        assert x32.grad.dtype == torch.float32 and torch.equal(x32.grad, x16.grad.float())


def test_deterministic_forward(cuda_device):
    """Two runs give bit-identical states (no race in the h exchange)."""
    from flashrnn_b200 import flashrnn

    Wx, R, b, s0 = make_inputs("lstm", 16, 64, 4, 256, seed=1)
    a = [t.to("cuda", torch.bfloat16) for t in (Wx, R, b, s0)]
    with torch.no_grad():
        s1, _ = flashrnn(a[0], a[1], a[2], a[3], function="lstm")
        s2, _ = flashrnn(a[0], a[1], a[2], a[3], function="lstm")
    assert torch.equal(s1, s2)


def test_inference_matches_training_forward(cuda_device):
    from flashrnn_b200 import flashrnn

    Wx, R, b, s0 = make_inputs("gru", 8, 16, 2, 64, seed=4)
    a = [t.to("cuda", torch.bfloat16) for t in (Wx, R, b, s0)]
    with torch.no_grad():
        s_inf, last_inf = flashrnn(*a[:3], a[3], function="gru")
    a[0].requires_grad_(True)
    s_tr, _ = flashrnn(*a[:3], a[3], function="gru")
    assert torch.equal(s_inf, s_tr.detach())
    assert torch.equal(last_inf, s_inf[:, :, -1:])
    ref = run_oracle("gru", Wx, R, b, s0)  # the no-cache (inference) plan against the oracle
    assert np.abs(s_inf.to(torch.float64).cpu().numpy()[0] - ref["states"][0]).max() <= 2e-2


def test_chunked_sequence_equals_whole(cuda_device):
    """Feeding `last` back as `states` continues the sequence (the reference's only long-T mechanism)."""
    from flashrnn_b200 import flashrnn

    Wx, R, b, s0 = make_inputs("lstm", 4, 32, 2, 64, seed=9)
    Wx_d, R_d, b_d = (t.to("cuda", torch.bfloat16) for t in (Wx, R, b))
    s_d = s0.to("cuda", torch.float32)
    with torch.no_grad():
        whole, _ = flashrnn(Wx_d, R_d, b_d, s_d, function="lstm")
        first, last = flashrnn(Wx_d[:, :16], R_d, b_d, s_d, function="lstm")
        second, _ = flashrnn(Wx_d[:, 16:].contiguous(), R_d, b_d, last, function="lstm")
    assert torch.allclose(torch.cat([first, second], dim=2), whole, atol=2e-2)


def test_error_paths(cuda_device):
    from flashrnn_b200 import flashrnn

    Wx = torch.zeros(2, 3, 4, 1, 32, device="cuda", dtype=torch.bfloat16)
    R = torch.zeros(4, 1, 32, 32, device="cuda", dtype=torch.bfloat16)
    b = torch.zeros(4, 1, 32, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(NotImplementedError):
        flashrnn(Wx, R, b, function="lstm", backend="triton_fused")
    with pytest.raises(ValueError):
        flashrnn(Wx, R, b, function="lstm", backend="nope")
    with pytest.raises(AssertionError):
        flashrnn(Wx, R, b, function="mgu")
    with pytest.raises(ValueError):
        flashrnn(Wx, R[:3], b, function="lstm")
    out, last = flashrnn(Wx[:, :0], R, b, function="lstm")
    assert out.shape == (2, 2, 0, 1, 32) and last.shape == (2, 2, 1, 1, 32)


@pytest.mark.parametrize("function", CELLS)
@pytest.mark.parametrize("B,T,N,state_f32", [(3, 7, 2, False), (16, 12, 48, False), (9, 5, 3, True), (300, 6, 4, False), (40, 9, 5, False)])
def test_parity_head_dim_16(cuda_device, function, B, T, N, state_f32):
    """Head dim 16, the smallest of the reference's head-dim sweep (16 x 48 heads): one 16-unit tile per gate and CTA,
    8-row and (large batches of the multi-gate cells) 16-row batch tiles, random cotangent and initial states."""
    D = 16
    Wx, R, b, s0 = make_inputs(function, B, T, N, D, seed=B + T + N, random_init=(function != "slstm"), state_f32=state_f32)
    S = s0.shape[0]
    g = torch.Generator().manual_seed(5)
    cot = torch.randn(S, B, T, N, D, generator=g, dtype=torch.float64).to(torch.bfloat16).to(torch.float64)
    if function == "slstm":
        cot[1:] = 0
    got = run_native(function, Wx, R, b, s0, cot=cot, state_f32=state_f32)
    ref = run_oracle(function, Wx, R, b, s0, cot=cot)
    assert_parity(function, got, ref, tag=f"{function} D16 B{B} T{T} N{N}", zero_init=(function == "slstm"))
