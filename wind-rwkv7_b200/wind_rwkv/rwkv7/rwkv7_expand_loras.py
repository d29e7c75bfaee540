"""expand_loras: drop-in for wind_rwkv/rwkv7/rwkv7_expand_loras.py
(`expand_loras(w_in,k_in,z_in,a_in,ma_in,mk_in, Wz,Wa,Wma,Wmk, w_bias,a_bias,ma_bias,mk_bias, HEAD_SIZE)
 -> (w, k, kk, b)`).  As upstream (:217-218) the rank-D inputs are made contiguous and the weights and
biases are cast to bf16; their gradients come back in fp32 and autograd casts them to the parameter dtype.
"""
import torch as th

from . import _lib


class ExpandLoras(th.autograd.Function):
    @staticmethod
    def forward(ctx, w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias, HEAD_SIZE):
        _lib.require_cuda(w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias)
        if HEAD_SIZE != _lib.HEAD_SIZE:
            raise ValueError(f'only HEAD_SIZE == {_lib.HEAD_SIZE} is built, got {HEAD_SIZE}')
        acts = [i.contiguous() for i in [w_in, k_in, z_in, a_in, ma_in, mk_in]]
        assert all(i.dtype == th.bfloat16 for i in acts), 'activations must be bfloat16'
        params = [Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias]
        pb = [i.detach().to(th.bfloat16).contiguous() for i in params]
        B, T, C = w_in.shape
        D = z_in.shape[2]
        assert all(list(i.shape) == [B, T, C] for i in acts[:2]) and all(list(i.shape) == [B, T, D] for i in acts[2:])
        assert all(list(i.shape) == [C, D] for i in pb[:4]) and all(list(i.shape) == [C] for i in pb[4:])
        assert T % 16 == 0 and C % HEAD_SIZE == 0
        outs = [th.empty_like(acts[0]) for _ in range(4)]
        rc = _lib.lib().wkv7_expand_loras_fwd(*[i.data_ptr() for i in acts + pb + outs], B, T, C, D, _lib.stream_of(w_in))
        _lib.check(rc, 'wkv7_expand_loras_fwd')
        ctx.save_for_backward(*acts, *pb)
        ctx.param_dtypes = [i.dtype for i in params]
        return tuple(outs)

    @staticmethod
    def backward(ctx, dw_out, dk_out, dz_out, db_out):
        saved = ctx.saved_tensors
        acts, pb = list(saved[:6]), list(saved[6:])
        B, T, C = acts[0].shape
        D = acts[2].shape[2]
        dev = acts[0].device
        douts = [th.zeros_like(acts[0]) if d is None else d.to(th.bfloat16).contiguous() for d in (dw_out, dk_out, dz_out, db_out)]
        dact = [th.empty_like(i) for i in acts]
        dW = [th.empty(C, D, dtype=th.float32, device=dev) for _ in range(4)]
        dbias = [th.empty(C, dtype=th.float32, device=dev) for _ in range(4)]
        ws = th.empty(_lib.lib().wkv7_expand_loras_bwd_workspace_bytes(B, T, C, D), dtype=th.uint8, device=dev)
        rc = _lib.lib().wkv7_expand_loras_bwd(*[i.data_ptr() for i in acts + pb + douts + dact + dW + dbias], ws.data_ptr(),
                                              B, T, C, D, _lib.stream_of(acts[0]))
        _lib.check(rc, 'wkv7_expand_loras_bwd')
        grads = dact + [g.to(t) for g, t in zip(dW + dbias, ctx.param_dtypes)]
        return (*grads, None)


expand_loras = ExpandLoras.apply
