"""Functional front end with the reference's signature, on top of the C ABI of libfrnn_b200.so.

Mirrors ``flashrnn(Wx, R, b, states, function, config, backend, dtype)`` and ``FlashRNNConfig`` of the
reference (flashrnn/flashrnn/flashrnn.py:124-207, 1093-1135).  What changed on purpose:

* one native backend (``"cuda_fused"``, alias ``"b200"``); Triton, the alternating cuBLAS backend and the
  PyTorch loops are gone and there is no CPU fallback -- other backend names raise;
* tensors are consumed and produced in the user layouts directly (no permute + ``.contiguous()`` copies,
  reference flashrnn.py:1049-1057, 1130-1135); the other layout strings (``input_shape="TBGHD"`` ...) reach the
  kernels as strided views of Wx and of the incoming cotangent, and leave as permuted views of the outputs;
* under ``torch.autocast`` the call behaves like the reference's ``custom_fwd(cast_inputs=dtype)`` / ``custom_bwd``
  pair (flashrnn.py:690-695, 735-738): inputs of any floating dtype are cast to the kernel dtype by hand, gradients
  come back in the inputs' dtypes, and since forward and backward consist of library calls only (no torch op that
  autocast could re-type), there is nothing for the decorators to switch off;
* GRU runs fused (the reference silently switches it to the alternating backend, flashrnn.py:280-284);
* states may be kept in float32 while Wx/R/b are bfloat16 / float16 (``dtype_s="float32"`` or by passing float32
  ``states``), which the reference's fused kernel cannot express;
* ``dtype`` is ``"bfloat16"`` or ``"float16"`` (the MMA operand type; accumulation and gate math are fp32 for both,
  where the reference accumulates float16 in float16, fused/flashrnn_fused_forward.cu), or ``"float32"``: everything in
  fp32 on the CUDA cores -- accurate to ~1e-5 against the fp32 ``vanilla`` loop (the reference multiplies in tf32
  there, fused/flashrnn_fused_forward.cu:108-112), 4-5 x slower than the 16-bit tensor-core loops.
"""
from __future__ import annotations

import ctypes
import logging
from dataclasses import dataclass
from typing import Optional, Sequence, Union

import torch

from . import _native

LOGGER = logging.getLogger(__name__)

DTYPE_DICT = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32, "float64": torch.float64}
DTYPE_DICT_REV = {v: k for k, v in DTYPE_DICT.items()}

# (num_gates_r, num_gates_w, num_gates_i, num_gates_t, num_states) -- reference flashrnn.py:49-71
rnn_function_registry = {
    "slstm": {"gates_states": (4, 4, 4, 4, 4), "constants": {}, "simple_agg": True},
    "lstm": {"gates_states": (4, 4, 4, 4, 2), "constants": {}, "simple_agg": True},
    "gru": {"gates_states": (3, 3, 4, 4, 1), "constants": {}, "simple_agg": False},
    "elman": {"gates_states": (1, 1, 1, 1, 1), "constants": {}, "simple_agg": True},
}

_NATIVE_BACKENDS = ("cuda_fused", "b200")
_REMOVED_BACKENDS = ("cuda", "triton_fused", "vanilla", "vanilla_fwbw")


@dataclass
class FlashRNNConfig:
    """Result-affecting subset of the reference's FlashRNNConfig (flashrnn.py:124-207), same field names."""

    backend: str = "cuda_fused"
    function: str = "lstm"
    gradient_recurrent_cut: bool = False
    gradient_recurrent_clipval: Optional[float] = None
    forward_clipval: Optional[float] = None
    constants: Optional[dict] = None
    simple_agg: bool = True
    hidden_dim: int = -1
    num_heads: int = -1
    head_dim: int = -1
    num_states: int = 4
    num_gates_r: int = 4
    num_gates_w: int = 4
    num_gates_i: int = 4
    num_gates_t: int = 4
    batch_size: int = 8
    input_shape: str = "BTGHD"
    output_shape: str = "SBTHD"
    recurrent_shape: str = "GHDP"
    bias_shape: str = "GHD"
    dtype: str = "bfloat16"
    dtype_acc: Optional[str] = "float32"
    dtype_b: Optional[str] = None
    dtype_r: Optional[str] = None
    dtype_w: Optional[str] = None
    dtype_g: Optional[str] = None
    dtype_s: Optional[str] = None
    dtype_a: Optional[str] = None
    enable_automatic_mixed_precision: bool = True
    initial_val: Union[float, Sequence[float]] = 0.0
    # sm_100a tile override for measurements: 0 = take the library's table
    cluster_size: int = 0
    batch_tile: int = 0
    # synchronise after each launch and raise if a bounded device-side wait expired (a CTA of a cluster never
    # delivered its part); off by default because it costs a host synchronisation per call
    check_device_status: bool = False
    _test_drop_exchange: bool = False  # test hook: make one CTA per cluster withhold a message (see include/frnn.h)

    def __post_init__(self):
        if self.num_heads <= 0 and self.head_dim <= 0:
            self.num_heads = 1
        if self.num_heads <= 0:
            self.num_heads = self.hidden_dim // self.head_dim
        elif self.head_dim <= 0:
            self.head_dim = self.hidden_dim // self.num_heads
        if self.hidden_dim <= 0:
            self.hidden_dim = self.num_heads * self.head_dim
        for name in ("dtype_b", "dtype_r", "dtype_w"):
            if getattr(self, name) is None:
                setattr(self, name, self.dtype)
        if self.dtype_a is None:
            self.dtype_a = "float32"  # gate math always runs in fp32 here
        if self.dtype_s is None:
            self.dtype_s = self.dtype_w
        if self.dtype_g is None:
            self.dtype_g = self.dtype_r
        assert self.function in rnn_function_registry, f"RNN function {self.function} not in registry"
        (self.num_gates_r, self.num_gates_w, self.num_gates_i, self.num_gates_t, self.num_states) = \
            rnn_function_registry[self.function]["gates_states"]
        if self.constants is None:
            self.constants = rnn_function_registry[self.function]["constants"]
        self.simple_agg = rnn_function_registry[self.function]["simple_agg"]

    @property
    def torch_dtype(self) -> torch.dtype:
        return DTYPE_DICT[self.dtype]

    @property
    def torch_dtype_s(self) -> torch.dtype:
        return DTYPE_DICT[self.dtype_s]


def _to_layout(x: torch.Tensor, src: str, dst: str) -> torch.Tensor:
    """View of ``x`` with its dimensions reordered from layout string ``src`` to ``dst`` (e.g. "TBGHD" -> "BTGHD")."""
    if src == dst:
        return x
    if sorted(src) != sorted(dst) or len(set(src)) != len(src):
        raise ValueError(f"layout '{src}' is not a permutation of '{dst}'")
    return x.permute(tuple(src.index(c) for c in dst))


def _zero_state(config: FlashRNNConfig, inp: torch.Tensor, batch: Optional[int] = None) -> torch.Tensor:
    """Initial states filled with ``initial_val`` in the dtype/device of ``inp``: [S,B,1,N,D] reordered to
    ``config.output_shape`` (reference flashrnn.py:927-954).  ``inp`` is in ``config.input_shape`` unless ``batch``
    is given."""
    B = batch if batch is not None else inp.shape[config.input_shape.index("B")]
    state = torch.zeros((config.num_states, B, 1, config.num_heads, config.head_dim), dtype=inp.dtype, device=inp.device)
    if isinstance(config.initial_val, (int, float)):
        if config.initial_val != 0.0:
            state += config.initial_val
    else:
        for i in range(config.num_states):
            state[i] += config.initial_val[i]
    return _to_layout(state, "SBTHD", config.output_shape)


def _get_config(Wx, R, b, function, backend, dtype) -> FlashRNNConfig:
    return FlashRNNConfig(
        head_dim=Wx.shape[4], num_heads=Wx.shape[3], batch_size=Wx.shape[0], function=function, backend=backend,
        dtype=dtype if dtype is not None else "bfloat16",
        dtype_w=DTYPE_DICT_REV[Wx.dtype], dtype_r=DTYPE_DICT_REV[R.dtype], dtype_b=DTYPE_DICT_REV[b.dtype])


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def _raise_on_device_status(ws: torch.Tensor, device, what: str) -> None:
    """Reads the status block of a workspace (synchronises the stream) and raises if a bounded wait expired."""
    st = _native.FrnnDevStatus()
    _native.check("frnn_read_device_status",
                  _native.lib().frnn_read_device_status(_ptr(ws), _stream_ptr(device), ctypes.byref(st)))
    if st.code != 0:
        raise RuntimeError(f"flashrnn_b200: a device-side wait expired in the {what} time loop "
                           f"(time step {st.where}, CTA {st.cta}); the results of this call are invalid")


class _FrnnFunction(torch.autograd.Function):
    """autograd bridge: one frnn_forward, one frnn_backward (+ optional all-reduce) + frnn_finalize_grads.
    Takes the place of FlashRNNFunctionFused (reference flashrnn.py:688-801)."""

    @staticmethod
    def forward(ctx, Wx, R, b, s0, cfg: FlashRNNConfig, training: bool, grad_group):
        B, T, _, N, D = Wx.shape
        state_dtype = cfg.torch_dtype_s
        kdt = cfg.torch_dtype  # element type the kernels compute in: bfloat16 or float16
        in_dtypes = (Wx.dtype, R.dtype, b.dtype, s0.dtype)
        Wx_k, wx_strides = _native.kernel_strides(Wx, kdt)  # a strided view (other input_shape) is read in place
        R_k = R.to(kdt).contiguous()
        b_k = b.to(kdt).contiguous()
        s0_k = s0.to(state_dtype).contiguous()
        prob = _native.make_problem(cfg.function, B, T, N, D, state_dtype == torch.float32, training,
                                    cfg.forward_clipval, cfg.gradient_recurrent_clipval, cfg.gradient_recurrent_cut,
                                    f16=kdt == torch.float16, f32=kdt == torch.float32)
        plan = _native.query(prob, cfg.cluster_size, cfg.batch_tile)
        plan.test_drop_exchange = 1 if cfg._test_drop_exchange else 0
        dev = Wx.device
        states = torch.empty((cfg.num_states, B, T, N, D), dtype=state_dtype, device=dev)
        cache = torch.empty(max(int(plan.cache_bytes), 16), dtype=torch.uint8, device=dev) if training else None
        ws = torch.empty(int(plan.workspace_bytes), dtype=torch.uint8, device=dev)
        args = _native.FrnnFwdArgs(_ptr(Wx_k), _ptr(R_k), _ptr(b_k), _ptr(s0_k), _ptr(states), _ptr(cache), _ptr(ws), None,
                                   wx_strides)
        with torch.cuda.device(dev):
            _native.check("frnn_forward", _native.lib().frnn_forward(ctypes.byref(plan), ctypes.byref(args), _stream_ptr(dev)))
            if cfg.check_device_status:
                _raise_on_device_status(ws, dev, "forward")
        if training:
            ctx.save_for_backward(R_k, s0_k, states, cache)
            ctx.plan, ctx.ws, ctx.in_dtypes, ctx.wx_shape, ctx.grad_group = plan, ws, in_dtypes, Wx.shape, grad_group
            ctx.b_shape = b.shape
            ctx.check_status = cfg.check_device_status
        ctx.training = training
        return states

    @staticmethod
    def backward(ctx, dstates):
        if not ctx.training:
            raise RuntimeError("FLASHRNN backward can only be called in training mode")
        R_k, s0_k, states, cache = ctx.saved_tensors
        plan, ws = ctx.plan, ctx.ws
        dev = states.device
        dstates, ds_strides = _native.kernel_strides(dstates, states.dtype)  # e.g. the cotangent of a permuted output view
        dWx = torch.empty(ctx.wx_shape, dtype=R_k.dtype, device=dev)
        ds0 = torch.empty_like(s0_k)
        args = _native.FrnnBwdArgs(_ptr(R_k), _ptr(s0_k), _ptr(states), _ptr(cache), _ptr(dstates), _ptr(dWx), _ptr(ds0), _ptr(ws),
                                   ds_strides)
        L = _native.lib()
        with torch.cuda.device(dev):
            _native.check("frnn_backward", L.frnn_backward(ctypes.byref(plan), ctypes.byref(args), _stream_ptr(dev)))
            if ctx.check_status:
                _raise_on_device_status(ws, dev, "backward")
            off, cnt = int(plan.grads_offset), int(plan.grads_count)
            grads = ws[off:off + 4 * cnt].view(torch.float32)
            if ctx.grad_group is not None:
                # batch sharding: every rank holds the gradient of its batch slice; sum them (fp32, one packed buffer)
                torch.distributed.all_reduce(grads, group=ctx.grad_group if ctx.grad_group is not True else None)
            dR = torch.empty_like(R_k)
            db = torch.empty(ctx.b_shape, dtype=R_k.dtype, device=dev)
            _native.check("frnn_finalize_grads",
                          L.frnn_finalize_grads(ctypes.byref(plan), _ptr(grads), _ptr(dR), _ptr(db), _stream_ptr(dev)))
        dt = ctx.in_dtypes
        return dWx.to(dt[0]), dR.to(dt[1]), db.to(dt[2]), ds0.to(dt[3]), None, None, None


def flashrnn(
    Wx: torch.Tensor,
    R: torch.Tensor,
    b: torch.Tensor,
    states: Optional[torch.Tensor] = None,
    function: str = "lstm",
    config: Optional[FlashRNNConfig] = None,
    backend: str = "cuda_fused",
    dtype: str = "bfloat16",
    grad_allreduce_group=None,
):
    """Wx[B,T,Gw,N,D], R[Gr,N,D,D], b[Gt,N,D], states[S,B,1,N,D] -> (states[S,B,T,N,D], last[S,B,1,N,D]).

    Same call as the reference's ``flashrnn`` (flashrnn.py:1114-1135).  ``grad_allreduce_group`` is the one
    addition: a ``torch.distributed`` process group (or ``True`` for the default group) over which dR/db are
    summed in backward when the batch is sharded across GPUs.
    """
    if config is None:
        config = _get_config(Wx, R, b, function, backend, dtype=dtype)
        if states is not None and states.dtype == torch.float32 and Wx.dtype != torch.float32:
            config.dtype_s = "float32"
    if config.backend in _REMOVED_BACKENDS:
        raise NotImplementedError(
            f"backend '{config.backend}' does not exist in flashrnn_b200: only the native sm_100a path "
            f"{_NATIVE_BACKENDS} is provided (no Triton, no alternating cuBLAS backend, no CPU/PyTorch path)")
    if config.backend not in _NATIVE_BACKENDS:
        raise ValueError(f"Unknown backend {config.backend}")
    if config.dtype not in ("bfloat16", "float16", "float32"):
        raise NotImplementedError(f"dtype '{config.dtype}': the sm_100a kernels compute in bfloat16, float16 or float32")
    if config.dtype == "float32":
        config.dtype_s = "float32"  # the float32 loops keep everything in fp32
    elif config.dtype_s in ("bfloat16", "float16"):
        config.dtype_s = config.dtype  # 16-bit states live in the kernel dtype (inputs of the other 16-bit type are cast)
    elif config.dtype_s != "float32":
        raise NotImplementedError(f"states in '{config.dtype_s}': states are kept in the kernel dtype or in float32")
    if not Wx.is_cuda:
        raise RuntimeError("flashrnn_b200 runs on CUDA tensors only; there is no CPU fallback")
    if Wx.dim() != 5 or R.dim() != 4 or b.dim() != 3:
        raise ValueError("expected Wx[B,T,G,N,D], R[G,N,D,D], b[G,N,D]")
    # other user layouts (reference flashrnn.py:165-173) are views of the native one: Wx and the cotangent of the states
    # reach the kernels through their strides, the outputs leave as permuted views; only R, b and the initial states
    # (small) are copied into GHDP / GHD / SBTHD order
    Wx = _to_layout(Wx, config.input_shape, "BTGHD")
    R = _to_layout(R, config.recurrent_shape, "GHDP")
    b = _to_layout(b, config.bias_shape, "GHD")
    if states is not None:
        if states.dim() != 5:
            raise ValueError("states must have 5 dimensions (S, B, 1, N, D in the order of output_shape)")
        states = _to_layout(states, config.output_shape, "SBTHD")
    B, T, Gw, N, D = Wx.shape
    if Gw != config.num_gates_w or tuple(R.shape) != (config.num_gates_r, N, D, D) or tuple(b.shape) != (config.num_gates_t, N, D):
        raise ValueError(f"shape mismatch for function '{config.function}': Wx{tuple(Wx.shape)} R{tuple(R.shape)} b{tuple(b.shape)}")
    if states is None:
        states = _to_layout(_zero_state(config, Wx, batch=B), config.output_shape, "SBTHD").to(config.torch_dtype_s)
    if tuple(states.shape) != (config.num_states, B, 1, N, D):
        raise ValueError(f"states must be [S,B,1,N,D] = {(config.num_states, B, 1, N, D)}, got {tuple(states.shape)}")
    if T == 0:
        out = torch.empty((config.num_states, B, 0, N, D), dtype=config.torch_dtype_s, device=Wx.device)
        return (_to_layout(out, "SBTHD", config.output_shape),
                _to_layout(states.to(config.torch_dtype_s), "SBTHD", config.output_shape))
    training = torch.is_grad_enabled() and any(t.requires_grad for t in (Wx, R, b, states))
    all_states = _FrnnFunction.apply(Wx, R, b, states, config, training, grad_allreduce_group)
    return (_to_layout(all_states, "SBTHD", config.output_shape),
            _to_layout(all_states[:, :, -1:], "SBTHD", config.output_shape))
