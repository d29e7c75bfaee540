"""TEST INFRASTRUCTURE — ctypes front-end of the C oracle (oracle/wkv7_oracle.c).

numpy arrays in, numpy arrays out.  dtype float32 or float64 selects the
instantiation.  Layouts follow the reference's internal op layout
(wind_rwkv/rwkv7/rwkv7_attn.py:53-59): r,w,k,v,a,b,g : [B,T,H,N];
states [B,H,N,N]; params [3,H*N].
"""
import ctypes
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import build as _build  # noqa: E402

_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(_build.build())
    return _lib


def _p(x):
    return None if x is None else x.ctypes.data_as(ctypes.c_void_p)


def _prep(dtype, *xs):
    return [None if x is None else np.ascontiguousarray(x, dtype=dtype) for x in xs]


def _sfx(dtype):
    dtype = np.dtype(dtype)
    assert dtype in (np.dtype(np.float32), np.dtype(np.float64))
    return "_f32" if dtype == np.dtype(np.float32) else "_f64"


def wkv7_fwd(r, w, k, v, a, b, s0=None, dtype=np.float64):
    """Returns (y [B,T,H,N], sT [B,H,N,N])."""
    r, w, k, v, a, b, s0 = _prep(dtype, r, w, k, v, a, b, s0)
    B, T, H, N = r.shape
    y = np.empty_like(r)
    sT = np.empty((B, H, N, N), dtype=dtype)
    f = getattr(lib(), "wkv7_oracle_fwd" + _sfx(dtype))
    f(ctypes.c_long(B), ctypes.c_long(T), ctypes.c_long(H), ctypes.c_int(N),
      _p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(s0), _p(y), _p(sT))
    return y, sT


def wkv7_bwd(r, w, k, v, a, b, dy, s0=None, dsT=None, dtype=np.float64):
    """Returns (dr, dw, dk, dv, da, db, ds0)."""
    r, w, k, v, a, b, dy, s0, dsT = _prep(dtype, r, w, k, v, a, b, dy, s0, dsT)
    B, T, H, N = r.shape
    outs = [np.empty_like(r) for _ in range(6)]
    ds0 = np.empty((B, H, N, N), dtype=dtype)
    f = getattr(lib(), "wkv7_oracle_bwd" + _sfx(dtype))
    f(ctypes.c_long(B), ctypes.c_long(T), ctypes.c_long(H), ctypes.c_int(N),
      _p(r), _p(w), _p(k), _p(v), _p(a), _p(b), _p(s0), _p(dy), _p(dsT),
      *[_p(o) for o in outs], _p(ds0))
    return (*outs, ds0)


def _real(dtype, x):
    return (ctypes.c_float if np.dtype(dtype) == np.dtype(np.float32) else ctypes.c_double)(x)


def attn_ln_fwd(r, w, k, v, a, b, g, params, s0=None, eps=64e-5, dtype=np.float64):
    """Returns (out, y_pre, sT): fused output, recurrence output before the norm, final state."""
    y, sT = wkv7_fwd(r, w, k, v, a, b, s0, dtype)
    r, k, v, g, params = _prep(dtype, r, k, v, g, params)
    B, T, H, N = r.shape
    out = np.empty_like(y)
    f = getattr(lib(), "attn_ln_post_fwd" + _sfx(dtype))
    f(ctypes.c_long(B), ctypes.c_long(T), ctypes.c_long(H), ctypes.c_int(N),
      _p(r), _p(k), _p(v), _p(g), _p(params), _real(dtype, eps), _p(y), _p(out))
    return out, y, sT


def attn_ln_bwd(r, w, k, v, a, b, g, params, dout, s0=None, dsT=None, eps=64e-5, dtype=np.float64):
    """Returns (dr, dw, dk, dv, da, db, dg, dparams, ds0)."""
    y, _ = wkv7_fwd(r, w, k, v, a, b, s0, dtype)
    r_, k_, v_, g_, params_, dout_ = _prep(dtype, r, k, v, g, params, dout)
    B, T, H, N = r_.shape
    dy = np.empty_like(y)
    dg = np.empty_like(y)
    dr_add, dk_add, dv_add = (np.zeros_like(y) for _ in range(3))
    dparams = np.zeros((3, H * N), dtype=dtype)
    f = getattr(lib(), "attn_ln_post_bwd" + _sfx(dtype))
    f(ctypes.c_long(B), ctypes.c_long(T), ctypes.c_long(H), ctypes.c_int(N),
      _p(r_), _p(k_), _p(v_), _p(g_), _p(params_), _real(dtype, eps), _p(y), _p(dout_),
      _p(dy), _p(dg), _p(dr_add), _p(dk_add), _p(dv_add), _p(dparams))
    dr, dw, dk, dv, da, db, ds0 = wkv7_bwd(r, w, k, v, a, b, dy, s0, dsT, dtype)
    return dr + dr_add, dw, dk + dk_add, dv + dv_add, da, db, dg, dparams, ds0
