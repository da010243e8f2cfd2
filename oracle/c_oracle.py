"""ctypes view of oracle/omni_oracle.c (test infrastructure only)."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_SO = _DIR / "_build" / "libomni_oracle.so"


def build(force: bool = False) -> Path:
    src = _DIR / "omni_oracle.c"
    if force or not _SO.exists() or _SO.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["make", "-C", str(_DIR), "-s"], check=True)
    return _SO


def _lib():
    lib = C.CDLL(str(build()))
    lib.oracle_route.restype = C.c_uint32
    return lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t))


def assign_padded(ids, n_expert=128, top=8, pad=32):
    ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
    live = ids.size
    padded = live + min(live, n_expert) * (pad - 1)
    counts = np.zeros(n_expert, np.int32)
    offsets = np.zeros(n_expert + 1, np.int32)
    rowmap = np.zeros(padded, np.int32)
    slots = np.zeros(live, np.int32)
    r = _lib().oracle_assign_padded(_p(ids, C.c_int32), live, n_expert, top, pad, _p(counts, C.c_int32),
                                    _p(offsets, C.c_int32), _p(rowmap, C.c_int32), _p(slots, C.c_int32))
    if r < 0:
        raise ValueError("invalid ids")
    return counts, offsets, rowmap, slots


def assign_canonical(ids, n_expert=128, top=8):
    ids = np.ascontiguousarray(ids, dtype=np.int32).reshape(-1)
    live = ids.size
    counts = np.zeros(n_expert, np.int32)
    offsets = np.zeros(n_expert + 1, np.int32)
    rowmap = np.zeros(live, np.int32)
    slots = np.zeros(live, np.int32)
    r = _lib().oracle_assign_canonical(_p(ids, C.c_int32), live, n_expert, top, _p(counts, C.c_int32),
                                       _p(offsets, C.c_int32), _p(rowmap, C.c_int32), _p(slots, C.c_int32))
    if r < 0:
        raise ValueError("invalid ids")
    return counts, offsets, rowmap, slots


def route(hi, lo=None, top=8):
    hi = np.ascontiguousarray(hi, dtype=np.float32)
    rows, n_expert = hi.shape
    lo_p = None
    if lo is not None:
        lo = np.ascontiguousarray(lo, dtype=np.float32)
        lo_p = _p(lo, C.c_float)
    ids = np.zeros((rows, top), np.int32)
    w = np.zeros((rows, top), np.float64)
    status = _lib().oracle_route(_p(hi, C.c_float), lo_p, rows, n_expert, top, _p(ids, C.c_int32), _p(w, C.c_double))
    return ids, w, int(status)


def router_dot(x, w_bf16_bits):
    x = np.ascontiguousarray(x, dtype=np.float32)
    w = np.ascontiguousarray(w_bf16_bits, dtype=np.uint16)
    out = np.zeros((x.shape[0], w.shape[0]), np.float64)
    _lib().oracle_router_dot(_p(x, C.c_float), _p(w, C.c_uint16), x.shape[0], w.shape[0], x.shape[1], _p(out, C.c_double))
    return out


def rmsnorm(x, w, eps=1e-6):
    x = np.ascontiguousarray(x, dtype=np.float64)
    w = np.ascontiguousarray(w, dtype=np.float64)
    out = np.zeros_like(x)
    _lib().oracle_rmsnorm(_p(x, C.c_double), _p(w, C.c_double), C.c_double(eps), x.shape[0], x.shape[1], _p(out, C.c_double))
    return out


def moe_rows(x, residual, ids, weights, gate_up_bits, down_bits, top=8):
    x = np.ascontiguousarray(x, dtype=np.float32)
    rows, hn = x.shape
    gu = np.ascontiguousarray(gate_up_bits, dtype=np.uint16)
    dn = np.ascontiguousarray(down_bits, dtype=np.uint16)
    fn = gu.shape[1] // 2
    ids = np.ascontiguousarray(ids, dtype=np.int32)
    weights = np.ascontiguousarray(weights, dtype=np.float64)
    res_p = None
    if residual is not None:
        residual = np.ascontiguousarray(residual, dtype=np.float32)
        res_p = _p(residual, C.c_float)
    y = np.zeros((rows, hn), np.float64)
    _lib().oracle_moe_rows(_p(x, C.c_float), res_p, _p(ids, C.c_int32), _p(weights, C.c_double),
                           _p(gu, C.c_uint16), _p(dn, C.c_uint16), rows, hn, fn, top, _p(y, C.c_double))
    return y
