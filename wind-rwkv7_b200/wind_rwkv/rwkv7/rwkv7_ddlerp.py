"""ddlerp: drop-in for wind_rwkv/rwkv7/rwkv7_ddlerp.py (`ddlerp(x, alpha, L, R, beta) -> (xrg, xwa, xk, xv)`).

    xx = shift(x) - x ;  m = tanh((x + xx*alpha) @ L^T) ;  y_k = x + xx*(m_k @ R_k^T + beta_k)

As upstream (rwkv7_ddlerp.py:309) the parameters are cast to bf16 for the kernels; their gradients
come back in fp32 and autograd casts them to the parameter dtype.
"""
import torch as th

from . import _lib


def fw_ddlerp(x, ab, Lb, Rb, bb):
    """Forward launcher (upstream fw1_triton + fw2_triton, rwkv7_ddlerp.py:51-84). Returns (m, y)."""
    B, T, C = x.shape
    D = Rb.shape[2]
    m = th.empty(B, T, 4 * D, dtype=th.bfloat16, device=x.device)
    y = th.empty(4, B, T, C, dtype=th.bfloat16, device=x.device)
    # tcgen05 + TMA form; its scratch (shifted-weight form of L, rearranged R) comes from torch's allocator
    ws = th.empty(_lib.lib().wkv7_ddlerp_fwd_tc_workspace_bytes(C, D), dtype=th.uint8, device=x.device)
    with _lib.on_device(x, ab, Lb, Rb, bb):
        rc = _lib.lib().wkv7_ddlerp_fwd_tc(x.data_ptr(), ab.data_ptr(), Lb.data_ptr(), Rb.data_ptr(), bb.data_ptr(),
                                           m.data_ptr(), y.data_ptr(), ws.data_ptr(), B, T, C, D, _lib.stream_of(x))
    _lib.check(rc, 'wkv7_ddlerp_fwd_tc')
    return m, y


def bw_ddlerp(x, ab, Lb, Rb, bb, m, dy0, dy1, dy2, dy3):
    """Backward launcher (upstream bw1..bw4_triton, rwkv7_ddlerp.py:323-334). Parameter gradients fp32."""
    B, T, C = x.shape
    D = Rb.shape[2]
    dev = x.device
    dpre = th.empty(B, T, 4 * D, dtype=th.bfloat16, device=dev)
    dx = th.empty_like(x)
    dalpha = th.empty(C, dtype=th.float32, device=dev)
    dL = th.empty(4 * D, C, dtype=th.float32, device=dev)
    dR = th.empty(4, C, D, dtype=th.float32, device=dev)
    dbeta = th.empty(4, 1, 1, C, dtype=th.float32, device=dev)
    ws = th.empty(_lib.lib().wkv7_ddlerp_bwd_tc_workspace_bytes(C, D), dtype=th.uint8, device=dev)
    with _lib.on_device(x, ab, Lb, Rb, bb, m, dy0, dy1, dy2, dy3):
        rc = _lib.lib().wkv7_ddlerp_bwd_tc(x.data_ptr(), ab.data_ptr(), Lb.data_ptr(), Rb.data_ptr(), bb.data_ptr(),
                                           m.data_ptr(), dy0.data_ptr(), dy1.data_ptr(), dy2.data_ptr(), dy3.data_ptr(),
                                           dpre.data_ptr(), dx.data_ptr(), dalpha.data_ptr(), dL.data_ptr(), dR.data_ptr(),
                                           dbeta.data_ptr(), ws.data_ptr(), B, T, C, D, _lib.stream_of(x))
    _lib.check(rc, 'wkv7_ddlerp_bwd_tc')
    return dx, dalpha, dL, dR, dbeta


def _fake_fw(x, ab, Lb, Rb, bb):
    B, T, C = x.shape
    return x.new_empty((B, T, 4 * Rb.shape[2])), x.new_empty((4, B, T, C))


def _fake_bw(x, ab, Lb, Rb, bb, m, dy0, dy1, dy2, dy3):
    C, D = x.shape[2], Rb.shape[2]
    f32 = dict(dtype=th.float32)
    return th.empty_like(x), x.new_empty((C,), **f32), x.new_empty((4 * D, C), **f32), x.new_empty((4, C, D), **f32), x.new_empty((4, 1, 1, C), **f32)


_fw_op = _lib.opaque_op('ddlerp_fwd', fw_ddlerp, _fake_fw, '(Tensor x, Tensor alpha, Tensor L, Tensor R, Tensor beta) -> (Tensor, Tensor)')
_bw_op = _lib.opaque_op('ddlerp_bwd', bw_ddlerp, _fake_bw,
                        '(Tensor x, Tensor alpha, Tensor L, Tensor R, Tensor beta, Tensor m, Tensor dy0, Tensor dy1, Tensor dy2, Tensor dy3) -> (Tensor, Tensor, Tensor, Tensor, Tensor)')


class DDLerp(th.autograd.Function):
    @staticmethod
    def forward(ctx, x, alpha, L, R, beta):
        if not th.compiler.is_compiling():
            _lib.require_cuda(x, alpha, L, R, beta)
            assert x.dtype == th.bfloat16, 'x must be bfloat16'
            B, T, C = x.shape
            D = R.shape[2]
            assert list(alpha.shape) == [C] and list(beta.shape) == [4, 1, 1, C]
            assert list(L.shape) == [4 * D, C] and list(R.shape) == [4, C, D]
            assert C % 64 == 0, 'ddlerp needs C % 64 == 0'
        x = x.contiguous()
        Lb, Rb, ab, bb = [i.detach().to(th.bfloat16).contiguous() for i in [L, R, alpha, beta]]
        m, y = _lib.call(_fw_op, fw_ddlerp, x, ab, Lb, Rb, bb)
        ctx.save_for_backward(x, ab, Lb, Rb, bb, m)
        ctx.param_dtypes = (alpha.dtype, L.dtype, R.dtype, beta.dtype)
        return y.unbind(dim=0)

    @staticmethod
    def backward(ctx, dy0, dy1, dy2, dy3):
        x, ab, Lb, Rb, bb, m = ctx.saved_tensors
        dys = [th.zeros_like(x) if d is None else d.to(th.bfloat16).contiguous() for d in (dy0, dy1, dy2, dy3)]
        dx, dalpha, dL, dR, dbeta = _lib.call(_bw_op, bw_ddlerp, x, ab, Lb, Rb, bb, m, *dys)
        ta, tL, tR, tb = ctx.param_dtypes
        return dx, dalpha.to(ta), dL.to(tL), dR.to(tR), dbeta.to(tb)


ddlerp = DDLerp.apply
