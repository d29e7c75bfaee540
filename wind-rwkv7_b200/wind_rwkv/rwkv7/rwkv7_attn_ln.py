"""WKV7 + fused per-head GroupNorm, bonus term and output gate: drop-in for
wind_rwkv/rwkv7/rwkv7_attn_ln.py (`load_attn_ln`, `attn_ln(r,w,k,v,a,b,g,params,HEAD_SIZE)`).

    y = (GroupNorm_head(WKV7(r,w,k,v,a,b); eps=64e-5, params[0], params[1])
         + (r*k*params[2]).sum_head * v) * g
"""
import torch as th

from . import _lib
from .rwkv7_attn import _check_inputs, _same_layout

EPS = 64e-5


def fw_attn_ln(w, q, k, v, a, b, g, params, s0):
    """Forward launcher (upstream: rwkv7_attn_ln.py:5-11)."""
    B, T, H, C = w.shape
    _lib.require_cuda(w, q, k, v, a, b, g, params, s0)
    if not _same_layout([w, q, k, v, a, b, g]):
        w, q, k, v, a, b, g = [i.contiguous() for i in (w, q, k, v, a, b, g)]
    y = th.empty_strided(v.shape, v.stride(), dtype=v.dtype, device=v.device)
    sT = th.empty(B, H, C, C, dtype=th.float32, device=w.device)
    s = th.empty(B, H, T // _lib.CHUNK, C, C, dtype=th.float32, device=w.device)
    sb, st, sh = _lib.strides4(w)
    rc = _lib.lib().wkv7_attn_ln_fwd(q.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                     b.data_ptr(), g.data_ptr(), params.data_ptr(), _lib.ptr(s0), y.data_ptr(),
                                     sT.data_ptr(), s.data_ptr(), EPS, B, T, H, C, sb, st, sh,
                                     _lib.io_dtype(w), _lib.stream_of(w))
    _lib.check(rc, 'wkv7_attn_ln_fwd')
    return y, sT, s


def load_attn_ln(HEAD_SIZE):
    if HEAD_SIZE != _lib.HEAD_SIZE:
        raise ValueError(f'only HEAD_SIZE == {_lib.HEAD_SIZE} is built, got {HEAD_SIZE}')
    _lib.lib()
