"""WKV7 + fused per-head GroupNorm, bonus term and output gate: drop-in for
wind_rwkv/rwkv7/rwkv7_attn_ln.py (`load_attn_ln`, `attn_ln(r,w,k,v,a,b,g,params,HEAD_SIZE)`).

    y = (GroupNorm_head(WKV7(r,w,k,v,a,b); eps=64e-5, params[0], params[1])
         + (r*k*params[2]).sum_head * v) * g
"""
import torch as th

from . import _lib
from .rwkv7_attn import _check_inputs, _same_layout

EPS = 64e-5


def fw_attn_ln(w, q, k, v, a, b, g, params, s0, save_checkpoints=True):
    """Forward launcher (upstream: rwkv7_attn_ln.py:5-11); save_checkpoints as in rwkv7_attn.fw_attn."""
    B, T, H, C = w.shape
    _lib.require_cuda(w, q, k, v, a, b, g, params, s0)
    if not _same_layout([w, q, k, v, a, b, g]):
        w, q, k, v, a, b, g = [i.contiguous() for i in (w, q, k, v, a, b, g)]
    y = th.empty_strided(v.shape, v.stride(), dtype=v.dtype, device=v.device)
    sT = th.empty(B, H, C, C, dtype=th.float32, device=w.device)
    s = th.empty(B, H, _lib.chunks(T) if save_checkpoints else 0, _lib.CKPT_FLOATS, dtype=th.float32, device=w.device)
    sb, st, sh = _lib.strides4(w)
    with _lib.on_device(w, q, k, v, a, b, g, params, s0):
        rc = _lib.lib().wkv7_attn_ln_fwd(q.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(),
                                         b.data_ptr(), g.data_ptr(), params.data_ptr(), _lib.ptr(s0), y.data_ptr(),
                                         sT.data_ptr(), s.data_ptr() if save_checkpoints else None, EPS, B, T, H, C, sb, st, sh,
                                         _lib.io_dtype(w), _lib.stream_of(w))
    _lib.check(rc, 'wkv7_attn_ln_fwd')
    return y, sT, s


def bw_attn_ln(w, q, k, v, a, b, g, params, s, dy, dsT, sT):
    """Backward launcher (upstream: rwkv7_attn_ln.py:13-17). dparams is fp32 [3, H*C], deterministic."""
    B, T, H, C = w.shape
    if not _same_layout([w, q, k, v, a, b, g, dy]):
        w, q, k, v, a, b, g, dy = [i.contiguous() for i in (w, q, k, v, a, b, g, dy)]
    dw, dq, dk, dv, da, db, dg = [th.empty_strided(w.shape, w.stride(), dtype=w.dtype, device=w.device) for _ in range(7)]
    dparams = th.empty(3, H * C, dtype=th.float32, device=w.device)
    ws = th.empty(B, 3, H * C, dtype=th.float32, device=w.device)
    ds0 = th.empty(B, H, C, C, dtype=th.float32, device=w.device)
    sb, st, sh = _lib.strides4(w)
    with _lib.on_device(w, q, k, v, a, b, g, params, s, dy, dsT):
        rc = _lib.lib().wkv7_attn_ln_bwd(
            q.data_ptr(), w.data_ptr(), k.data_ptr(), v.data_ptr(), a.data_ptr(), b.data_ptr(), g.data_ptr(),
            params.data_ptr(), dy.data_ptr(), s.data_ptr(), _lib.ptr(dsT), _lib.ptr(sT if dsT is not None else None),
            dq.data_ptr(), dw.data_ptr(), dk.data_ptr(), dv.data_ptr(), da.data_ptr(), db.data_ptr(), dg.data_ptr(),
            dparams.data_ptr(), ws.data_ptr(), ds0.data_ptr(), EPS, B, T, H, C, sb, st, sh,
            _lib.io_dtype(w), _lib.stream_of(w))
    _lib.check(rc, 'wkv7_attn_ln_bwd')
    return dw, dq, dk, dv, da, db, dg, dparams, ds0


def _fake_fw(w, q, k, v, a, b, g, params, s0, save_checkpoints=True):
    B, T, H, C = w.shape
    return (th.empty_like(v), w.new_empty((B, H, C, C), dtype=th.float32),
            w.new_empty((B, H, _lib.chunks(T) if save_checkpoints else 0, _lib.CKPT_FLOATS), dtype=th.float32))


def _fake_bw(w, q, k, v, a, b, g, params, s, dy, dsT, sT):
    B, T, H, C = w.shape
    return tuple(th.empty_like(w) for _ in range(7)) + (th.empty_like(params), w.new_empty((B, H, C, C), dtype=th.float32))


_fw_op = _lib.opaque_op('attn_ln_fwd', fw_attn_ln, _fake_fw,
                        '(Tensor w, Tensor q, Tensor k, Tensor v, Tensor a, Tensor b, Tensor g, Tensor params, Tensor? s0, bool save_checkpoints=True) -> (Tensor, Tensor, Tensor)')
_bw_op = _lib.opaque_op('attn_ln_bwd', bw_attn_ln, _fake_bw,
                        '(Tensor w, Tensor q, Tensor k, Tensor v, Tensor a, Tensor b, Tensor g, Tensor params, Tensor s, Tensor dy, Tensor? dsT, Tensor sT) -> (Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)')


class WindRWKV7(th.autograd.Function):
    """(w,q,k,v,a,b,g,params,s0) -> (y, sT, s), as upstream's autograd function (rwkv7_attn_ln.py:19-47)."""

    @staticmethod
    def forward(ctx, w, q, k, v, a, b, g, params, s0):
        if not th.compiler.is_compiling():  # as upstream, checks are skipped while tracing
            _check_inputs(w, q, k, v, a, b, s0)
            B, T, H, C = w.shape
            assert g.shape == w.shape and g.dtype == w.dtype
            assert params.dtype == th.float32 and list(params.shape) == [3, H * C]
        params = params.contiguous()
        s0f = None if s0 is None else s0.float().contiguous()
        save = True if th.compiler.is_compiling() else any(ctx.needs_input_grad)
        y, sT, s = _lib.call(_fw_op, fw_attn_ln, w, q, k, v, a, b, g, params, s0f, save)
        ctx.save_for_backward(w, q, k, v, a, b, g, params, s, sT)
        ctx.s0_dtype = None if s0 is None else s0.dtype
        ctx.mark_non_differentiable(s)
        ctx.set_materialize_grads(False)
        if s0 is not None and s0.dtype != th.float32:
            return y, sT.to(s0.dtype), s
        return y, sT, s

    @staticmethod
    def backward(ctx, dy, dsT, ds):
        w, q, k, v, a, b, g, params, s, sT = ctx.saved_tensors
        if not th.compiler.is_compiling():
            assert ds is None
        if dy is None:
            dy = th.zeros_like(v)
        if dsT is not None:
            dsT = dsT.float().contiguous()
        dw, dq, dk, dv, da, db, dg, dparams, ds0 = _lib.call(_bw_op, bw_attn_ln, w, q, k, v, a, b, g, params, s, dy, dsT, sT)
        if ctx.s0_dtype is None:
            ds0 = None
        elif ctx.s0_dtype != th.float32:
            ds0 = ds0.to(ctx.s0_dtype)
        return dw, dq, dk, dv, da, db, dg, dparams, ds0


def load_attn_ln(HEAD_SIZE):
    if HEAD_SIZE != _lib.HEAD_SIZE:
        raise ValueError(f'only HEAD_SIZE == {_lib.HEAD_SIZE} is built, got {HEAD_SIZE}')
    _lib.lib()


def attn_ln(r, w, k, v, a, b, g, params, HEAD_SIZE, *, s0=None, return_state=False):
    """Fused WKV7 + GroupNorm + bonus + gate for [B,T,H*HEAD_SIZE] tensors (upstream: rwkv7_attn_ln.py:56-62)."""
    B, T, HC = w.shape
    C = HEAD_SIZE
    H = HC // C
    r, w, k, v, a, b, g = [i.view(B, T, H, C) for i in [r, w, k, v, a, b, g]]
    y, sT, _ = WindRWKV7.apply(w, r, k, v, a, b, g, params, s0)
    y = y.view(B, T, HC)
    return (y, sT) if return_state else y
