"""Step-by-step (decoding) use of the forward loop.

``FlashRNNStepper`` keeps R, b, the carried states and every scratch buffer on the device and advances the recurrence
by one chunk of time steps (default: one) per call: no allocation and no repacking of R per call -- the time loop and
one strided copy that carries the last states in place, on the caller's current stream, so a step can be captured in a CUDA graph.  It is the
counterpart of the reference's per-step kernel selection (``_get_kernel_step``, flashrnn/flashrnn/flashrnn.py:957-983;
``flashrnn_forward_step``, flashrnn/flashrnn/vanilla/__init__.py:73-121): same cells, same state layout, forward only.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _native
from .flashrnn import DTYPE_DICT, rnn_function_registry


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


class FlashRNNStepper:
    """R[Gr,N,D,D], b[Gt,N,D] fixed; ``step(Wx[B,chunk,Gw,N,D])`` returns ``states[S,B,chunk,N,D]`` (a view of an
    internal buffer, overwritten by the next call) and carries the last state into the next call."""

    def __init__(self, R: torch.Tensor, b: torch.Tensor, function: str = "lstm", batch_size: int = 1, chunk: int = 1,
                 dtype_s: Optional[str] = None, states: Optional[torch.Tensor] = None, dtype: str = "bfloat16"):
        if function not in rnn_function_registry:
            raise AssertionError(f"unknown function {function}")
        if not R.is_cuda:
            raise RuntimeError("flashrnn_b200 runs on CUDA tensors only; there is no CPU fallback")
        Gr, Gw, Gi, Gt, S = rnn_function_registry[function]["gates_states"]
        _, N, D, _ = R.shape
        if tuple(R.shape) != (Gr, N, D, D) or tuple(b.shape) != (Gt, N, D):
            raise ValueError(f"shape mismatch for function '{function}': R{tuple(R.shape)} b{tuple(b.shape)}")
        self.function, self.B, self.chunk, self.N, self.D, self.S, self.Gw = function, batch_size, chunk, N, D, S, Gw
        dev = R.device
        if dtype not in ("bfloat16", "float16", "float32"):
            raise NotImplementedError(f"dtype '{dtype}': the sm_100a kernels compute in bfloat16, float16 or float32")
        self._kdt = DTYPE_DICT[dtype]
        sdt = DTYPE_DICT["float32" if dtype == "float32" else (dtype_s or dtype)]
        if sdt not in (self._kdt, torch.float32):
            raise NotImplementedError("states are kept in the kernel dtype or in float32")
        self._R = R.detach().to(self._kdt).contiguous()
        self._b = b.detach().to(self._kdt).contiguous()
        prob = _native.make_problem(function, batch_size, chunk, N, D, sdt == torch.float32, False, f16=self._kdt == torch.float16,
                                    f32=self._kdt == torch.float32)
        self._plan = _native.query(prob)
        self._s0 = torch.zeros((S, batch_size, 1, N, D), dtype=sdt, device=dev)
        self._out = torch.empty((S, batch_size, chunk, N, D), dtype=sdt, device=dev)
        self._ws = torch.empty(int(self._plan.workspace_bytes), dtype=torch.uint8, device=dev)
        self._packed = False
        if states is not None:
            self.reset(states)

    def reset(self, states: Optional[torch.Tensor] = None) -> None:
        """Carried states back to zero, or to ``states[S,B,1,N,D]``."""
        if states is None:
            self._s0.zero_()
        else:
            self._s0.copy_(states.reshape(self._s0.shape))

    @property
    def states(self) -> torch.Tensor:
        """The carried states [S,B,1,N,D] (after the last step)."""
        return self._s0

    def step(self, Wx: torch.Tensor) -> torch.Tensor:
        if tuple(Wx.shape) != (self.B, self.chunk, self.Gw, self.N, self.D) or Wx.dtype != self._kdt or not Wx.is_contiguous():
            raise ValueError(f"expected contiguous {self._kdt} Wx{(self.B, self.chunk, self.Gw, self.N, self.D)}")
        dev = Wx.device
        self._plan.keep_packed_r = 1 if self._packed else 0
        # `last` = the s0 buffer itself: the carried states are updated in place by the library call
        args = _native.FrnnFwdArgs(_ptr(Wx), _ptr(self._R), _ptr(self._b), _ptr(self._s0), _ptr(self._out), None, _ptr(self._ws),
                                   _ptr(self._s0))
        stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        with torch.cuda.device(dev):
            _native.check("frnn_forward", _native.lib().frnn_forward(ctypes.byref(self._plan), ctypes.byref(args), stream))
        self._packed = True
        return self._out
