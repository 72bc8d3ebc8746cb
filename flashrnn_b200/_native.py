"""ctypes binding of libfrnn_b200.so (the C ABI declared in include/frnn.h).

The library is loaded from the package directory (built in-tree by ``flashrnn_b200.build``).  There is no
fallback of any kind: a missing library or a failing call raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import os

PKG = Path(__file__).resolve().parent
# FRNN_B200_LIB points the binding at another build of the same library (development variants)
LIB_PATH = Path(os.environ.get("FRNN_B200_LIB") or PKG / "libfrnn_b200.so")

ABI_VERSION = 3
NOALLOC_MAX_SCRATCH_BYTES = 8 << 20  # FRNN_NOALLOC_MAX_SCRATCH_BYTES
CELL_IDS = {"lstm": 0, "gru": 1, "elman": 2, "slstm": 3}
DTYPE_BF16, DTYPE_F32, DTYPE_F16 = 0, 1, 2

# every symbol include/frnn.h declares
EXPORTS = (
    "frnn_abi_version", "frnn_query", "frnn_query_tile", "frnn_forward", "frnn_backward", "frnn_backward_parts",
    "frnn_forward_noalloc",
    "frnn_finalize_grads", "frnn_read_device_status", "frnn_status_string",
)


class FrnnProblem(ctypes.Structure):
    _fields_ = [
        ("cell", ctypes.c_int32), ("B", ctypes.c_int32), ("T", ctypes.c_int32), ("N", ctypes.c_int32),
        ("D", ctypes.c_int32), ("dtype_io", ctypes.c_int32), ("dtype_state", ctypes.c_int32),
        ("training", ctypes.c_int32), ("forward_clip", ctypes.c_float), ("grad_clip", ctypes.c_float),
        ("grad_cut", ctypes.c_int32),
    ]


class FrnnPlan(ctypes.Structure):
    _fields_ = [
        ("abi_version", ctypes.c_int32), ("prob", FrnnProblem), ("cluster_size", ctypes.c_int32),
        ("units_per_cta", ctypes.c_int32), ("batch_tile", ctypes.c_int32), ("threads", ctypes.c_int32),
        ("wx_stages", ctypes.c_int32), ("cache_slots", ctypes.c_int32), ("test_drop_exchange", ctypes.c_int32),
        ("keep_packed_r", ctypes.c_int32), ("probe_noop_cell", ctypes.c_int32), ("wide_forward", ctypes.c_int32),
        ("reserved", ctypes.c_int32 * 2),
        ("cache_bytes", ctypes.c_uint64), ("workspace_bytes", ctypes.c_uint64), ("grads_offset", ctypes.c_uint64),
        ("grads_count", ctypes.c_uint64),
    ]


class FrnnFwdArgs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("Wx", "R", "b", "s0", "states", "cache", "workspace", "last")] + \
               [("wx_stride", ctypes.c_int64 * 4)]


class FrnnBwdArgs(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("R", "s0", "states", "cache", "dstates", "dWx", "ds0", "workspace")] + \
               [("dstates_stride", ctypes.c_int64 * 4)]


def kernel_strides(t, kernel_dtype):
    """``(tensor, strides)`` for a 5-d tensor the kernels may read through strides: the element strides of its four
    outer dimensions when the innermost one is contiguous, the dtype is the kernels' own and every stride is a
    non-negative multiple of 8 (16 bytes) and the first element is 16-byte aligned; otherwise a dense copy and
    ``(0, 0, 0, 0)`` (= dense)."""
    if (t.dtype == kernel_dtype and t.dim() == 5 and t.stride(4) == 1 and not t.is_contiguous()
            and (t.data_ptr() - 0) % 16 == 0):
        st = tuple(int(s) for s in t.stride()[:4])
        if all(s >= 0 and s % 8 == 0 for s in st) and any(st):
            return t, (ctypes.c_int64 * 4)(*st)
    return t.to(kernel_dtype).contiguous(), (ctypes.c_int64 * 4)(0, 0, 0, 0)


class FrnnDevStatus(ctypes.Structure):
    _fields_ = [("code", ctypes.c_uint32), ("where", ctypes.c_uint32), ("cta", ctypes.c_uint32), ("pad", ctypes.c_uint32)]


class FrnnError(RuntimeError):
    """A call into libfrnn_b200.so returned a non-zero status."""

    def __init__(self, what: str, code: int, text: str):
        super().__init__(f"{what} failed with status {code}: {text}")
        self.code = code


_lib = None


def lib() -> ctypes.CDLL:
    """The loaded library.  Raises if it has not been built; nothing else can stand in for it."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m flashrnn_b200.build` "
                "(nvcc, sm_100a).  flashrnn_b200 has no CPU or PyTorch fallback.")
        L = ctypes.CDLL(str(LIB_PATH))
        L.frnn_abi_version.restype = ctypes.c_int
        L.frnn_query.argtypes = [ctypes.POINTER(FrnnProblem), ctypes.POINTER(FrnnPlan)]
        L.frnn_query_tile.argtypes = [ctypes.POINTER(FrnnProblem), ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                      ctypes.POINTER(FrnnPlan)]
        L.frnn_forward.argtypes = [ctypes.POINTER(FrnnPlan), ctypes.POINTER(FrnnFwdArgs), ctypes.c_void_p]
        L.frnn_backward.argtypes = [ctypes.POINTER(FrnnPlan), ctypes.POINTER(FrnnBwdArgs), ctypes.c_void_p]
        L.frnn_backward_parts.argtypes = [ctypes.POINTER(FrnnPlan), ctypes.POINTER(FrnnBwdArgs), ctypes.c_void_p, ctypes.c_int]
        L.frnn_backward_parts.restype = ctypes.c_int
        L.frnn_forward_noalloc.argtypes = [ctypes.POINTER(FrnnProblem), ctypes.POINTER(FrnnFwdArgs), ctypes.c_void_p]
        L.frnn_forward_noalloc.restype = ctypes.c_int
        L.frnn_finalize_grads.argtypes = [ctypes.POINTER(FrnnPlan), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                                          ctypes.c_void_p]
        L.frnn_read_device_status.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(FrnnDevStatus)]
        L.frnn_status_string.argtypes = [ctypes.c_int]
        L.frnn_status_string.restype = ctypes.c_char_p
        for fn in ("frnn_query", "frnn_query_tile", "frnn_forward", "frnn_backward", "frnn_finalize_grads",
                   "frnn_read_device_status"):
            getattr(L, fn).restype = ctypes.c_int
        if L.frnn_abi_version() != ABI_VERSION:
            raise RuntimeError(f"libfrnn_b200.so has ABI {L.frnn_abi_version()}, the binding expects {ABI_VERSION}")
        _lib = L
    return _lib


def status_string(code: int) -> str:
    return lib().frnn_status_string(int(code)).decode()


def check(what: str, code: int) -> None:
    if code != 0:
        raise FrnnError(what, code, status_string(code))


def make_problem(function: str, B: int, T: int, N: int, D: int, state_f32: bool, training: bool,
                 forward_clip: float | None = None, grad_clip: float | None = None, grad_cut: bool = False,
                 f16: bool = False, f32: bool = False) -> FrnnProblem:
    """``f16``: Wx, R, b, the gradients and (unless ``state_f32``) the states are float16 instead of bfloat16.
    ``f32``: everything, states included, is float32 (the float32 loops)."""
    if function not in CELL_IDS:
        raise AssertionError(f"RNN function {function} not in registry")
    io = DTYPE_F32 if f32 else (DTYPE_F16 if f16 else DTYPE_BF16)
    state_f32 = state_f32 or f32
    return FrnnProblem(CELL_IDS[function], B, T, N, D, io, DTYPE_F32 if state_f32 else io,
                       1 if training else 0, float(forward_clip or 0.0), float(grad_clip or 0.0), 1 if grad_cut else 0)


def query(problem: FrnnProblem, cluster_size: int = 0, batch_tile: int = 0) -> FrnnPlan:
    plan = FrnnPlan()
    if cluster_size or batch_tile:
        check("frnn_query_tile", lib().frnn_query_tile(ctypes.byref(problem), cluster_size, batch_tile, 0, ctypes.byref(plan)))
    else:
        check("frnn_query", lib().frnn_query(ctypes.byref(problem), ctypes.byref(plan)))
    return plan
