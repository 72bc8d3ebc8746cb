"""ctypes front end of the C oracle (``frnn_oracle.c``).  TEST INFRASTRUCTURE ONLY.

All arrays are numpy, dense, in the reference's user-facing layouts
(reference flashrnn/flashrnn/flashrnn.py:165-173, 1114-1135):

    Wx[B,T,Gw,N,D]  R[Gr,N,D,D]  b[Gt,N,D]  s0[S,B,1,N,D]  ->  states[S,B,T,N,D], last[S,B,1,N,D]
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "libfrnn_oracle.so"
_lib = None

CELLS = {"lstm": 0, "gru": 1, "elman": 2, "slstm": 3}
# (Gr, Gw, Gt, S) per cell -- reference flashrnn/flashrnn/flashrnn.py:49-71
_DIMS = {"lstm": (4, 4, 4, 2), "gru": (3, 3, 4, 1), "elman": (1, 1, 1, 1), "slstm": (4, 4, 4, 4)}


def cell_dims(function: str) -> tuple[int, int, int, int]:
    """(num_gates_r, num_gates_w, num_gates_t, num_states) of a cell."""
    return _DIMS[function]


def build_oracle(force: bool = False) -> Path:
    """Compile the C oracle with the Makefile next to it (idempotent)."""
    src = _HERE / "frnn_oracle.c"
    if force or not _LIB_PATH.exists() or _LIB_PATH.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_HERE), "-s"] + (["-B"] if force else []), check=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        build_oracle()
        _lib = ctypes.CDLL(str(_LIB_PATH))
        for sfx in ("f64", "f32"):
            getattr(_lib, f"frnn_oracle_forward_{sfx}").restype = ctypes.c_int
            getattr(_lib, f"frnn_oracle_backward_{sfx}").restype = ctypes.c_int
    return _lib


def _ptr(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _prep(a, dtype):
    return np.ascontiguousarray(np.asarray(a, dtype=dtype))


def oracle_forward(function, Wx, R, b, s0=None, dtype=np.float64, with_cache=False, slstm_global_rule=True,
                   forward_clip=0.0):
    """Forward of the reference's ``vanilla`` loop.  Returns (states[S,B,T,N,D], last[S,B,1,N,D][, cache])."""
    lib = _load()
    Gr, Gw, Gt, S = _DIMS[function]
    Wx = _prep(Wx, dtype)
    R = _prep(R, dtype)
    b = _prep(b, dtype)
    B, T, gw, N, D = Wx.shape
    assert gw == Gw and R.shape == (Gr, N, D, D) and b.shape == (Gt, N, D), (Wx.shape, R.shape, b.shape)
    if s0 is None:
        s0 = np.zeros((S, B, 1, N, D), dtype=dtype)
    s0 = _prep(s0, dtype).reshape(S, B, N, D)
    states = np.empty((S, B, T, N, D), dtype=dtype)
    cache = np.empty((B, T, 5, N, D), dtype=dtype) if with_cache else None
    sfx = "f64" if dtype == np.float64 else "f32"
    fwd = getattr(lib, f"frnn_oracle_forward_{sfx}")
    fwd.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_double]
    rc = fwd(
        CELLS[function], B, T, N, D, _ptr(Wx), _ptr(R), _ptr(b), _ptr(s0), _ptr(states), _ptr(cache),
        1 if slstm_global_rule else 0, float(forward_clip))
    if rc != 0:
        raise RuntimeError(f"frnn_oracle_forward failed: {rc}")
    last = states[:, :, T - 1:T].copy() if T > 0 else s0.reshape(S, B, 1, N, D).copy()
    return (states, last, cache) if with_cache else (states, last)


def oracle_fwbw(function, Wx, R, b, s0=None, dstates=None, dlast=None, dtype=np.float64, clip=0.0,
                slstm_global_rule=True, forward_clip=0.0, cut=False):
    """Forward + closed-form backward.

    ``dstates`` is the cotangent of ``states`` ([S,B,T,N,D]; default: ones on states[0], i.e. loss = sum(h));
    ``dlast`` ([S,B,1,N,D], optional) is the cotangent of ``last`` and is added into the t = T-1 slot, as the
    reference does because ``last`` is a slice of ``states`` (flashrnn.py:1058).
    Returns dict(states, last, dWx, dR, db, ds0[S,B,1,N,D]).
    """
    lib = _load()
    Gr, Gw, Gt, S = _DIMS[function]
    states, last, cache = oracle_forward(function, Wx, R, b, s0, dtype, with_cache=True,
                                         slstm_global_rule=slstm_global_rule, forward_clip=forward_clip)
    _, B, T, N, D = states.shape
    R = _prep(R, dtype)
    if s0 is None:
        s0 = np.zeros((S, B, 1, N, D), dtype=dtype)
    s0 = _prep(s0, dtype).reshape(S, B, N, D)
    if dstates is None:
        dstates = np.zeros((S, B, T, N, D), dtype=dtype)
        dstates[0] = 1.0
    dstates = _prep(dstates, dtype).copy()
    if dlast is not None:
        dstates[:, :, T - 1:T] += np.asarray(dlast, dtype=dtype)
    dWx = np.empty((B, T, Gw, N, D), dtype=dtype)
    dR = np.empty((Gr, N, D, D), dtype=dtype)
    db = np.empty((Gt, N, D), dtype=dtype)
    ds0 = np.empty((S, B, N, D), dtype=dtype)
    sfx = "f64" if dtype == np.float64 else "f32"
    fn = getattr(lib, f"frnn_oracle_backward_{sfx}")
    fn.argtypes = [ctypes.c_int] * 5 + [ctypes.c_void_p] * 9 + [ctypes.c_double, ctypes.c_int]
    rc = fn(CELLS[function], B, T, N, D, _ptr(R), _ptr(s0), _ptr(states), _ptr(cache), _ptr(dstates),
            _ptr(dWx), _ptr(dR), _ptr(db), _ptr(ds0), float(clip), 1 if cut else 0)
    if rc != 0:
        raise RuntimeError(f"frnn_oracle_backward failed: {rc}")
    return dict(states=states, last=last, dWx=dWx, dR=dR, db=db, ds0=ds0.reshape(S, B, 1, N, D))


def set_threads(n: int) -> None:
    """Number of OpenMP threads the oracle uses (defaults to all cores)."""
    os.environ["OMP_NUM_THREADS"] = str(n)
