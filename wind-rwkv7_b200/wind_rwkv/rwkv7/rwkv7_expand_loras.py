"""expand_loras: drop-in for wind_rwkv/rwkv7/rwkv7_expand_loras.py
(`expand_loras(w_in,k_in,z_in,a_in,ma_in,mk_in, Wz,Wa,Wma,Wmk, w_bias,a_bias,ma_bias,mk_bias, HEAD_SIZE)
 -> (w, k, kk, b)`).  As upstream (:217-218) the rank-D inputs are made contiguous and the weights and
biases are cast to bf16; their gradients come back in fp32 and autograd casts them to the parameter dtype.
Any sequence length: the kernels take whole 16-token groups, other lengths are zero-padded here (upstream's kernel
walks 16-token tiles as well, rwkv7_expand_loras.py:75-76, and is only ever called with T % 16 == 0).
"""
import torch as th

from . import _lib


def fw_loras(w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias):
    """Forward launcher (upstream fw_triton, rwkv7_expand_loras.py:81-89); all arguments bf16, contiguous."""
    B, T, C = w_in.shape
    D = z_in.shape[2]
    ins = [w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias]
    outs = [th.empty_like(w_in) for _ in range(4)]
    with _lib.on_device(*ins):
        rc = _lib.lib().wkv7_expand_loras_fwd(*[i.data_ptr() for i in ins + outs], B, T, C, D, _lib.stream_of(w_in))
    _lib.check(rc, 'wkv7_expand_loras_fwd')
    return tuple(outs)


def bw_loras(w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias, dw, dk, dkk, db):
    """Backward launcher (upstream bw_triton, rwkv7_expand_loras.py:193-211): 6 bf16 input gradients,
    4 fp32 weight gradients, 4 fp32 bias gradients."""
    B, T, C = w_in.shape
    D = z_in.shape[2]
    dev = w_in.device
    acts = [w_in, k_in, z_in, a_in, ma_in, mk_in]
    pb = [Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias]
    dact = [th.empty_like(i) for i in acts]
    dW = [th.empty(C, D, dtype=th.float32, device=dev) for _ in range(4)]
    dbias = [th.empty(C, dtype=th.float32, device=dev) for _ in range(4)]
    ws = th.empty(_lib.lib().wkv7_expand_loras_bwd_workspace_bytes(B, T, C, D), dtype=th.uint8, device=dev)
    with _lib.on_device(*acts, *pb, dw, dk, dkk, db):
        rc = _lib.lib().wkv7_expand_loras_bwd(*[i.data_ptr() for i in acts + pb + [dw, dk, dkk, db] + dact + dW + dbias],
                                              ws.data_ptr(), B, T, C, D, _lib.stream_of(w_in))
    _lib.check(rc, 'wkv7_expand_loras_bwd')
    return tuple(dact + dW + dbias)


def _fake_fw(w_in, *rest):
    return tuple(th.empty_like(w_in) for _ in range(4))


def _fake_bw(w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias, dw, dk, dkk, db):
    f32 = dict(dtype=th.float32)
    return tuple([th.empty_like(i) for i in (w_in, k_in, z_in, a_in, ma_in, mk_in)] +
                 [Wz.new_empty(Wz.shape, **f32) for _ in range(4)] + [w_bias.new_empty(w_bias.shape, **f32) for _ in range(4)])


_T14 = ', '.join(f'Tensor {n}' for n in ['w_in', 'k_in', 'z_in', 'a_in', 'ma_in', 'mk_in', 'Wz', 'Wa', 'Wma', 'Wmk', 'w_bias', 'a_bias', 'ma_bias', 'mk_bias'])
_fw_op = _lib.opaque_op('expand_loras_fwd', fw_loras, _fake_fw, f'({_T14}) -> (Tensor, Tensor, Tensor, Tensor)')
_bw_op = _lib.opaque_op('expand_loras_bwd', bw_loras, _fake_bw,
                        f'({_T14}, Tensor dw, Tensor dk, Tensor dkk, Tensor db) -> (' + ', '.join(['Tensor'] * 14) + ')')


class ExpandLoras(th.autograd.Function):
    @staticmethod
    def forward(ctx, w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias, HEAD_SIZE):
        if HEAD_SIZE != _lib.HEAD_SIZE:
            raise ValueError(f'only HEAD_SIZE == {_lib.HEAD_SIZE} is built, got {HEAD_SIZE}')
        T = w_in.shape[1]
        pad = (-T) % 16
        acts = [i.contiguous() for i in [w_in, k_in, z_in, a_in, ma_in, mk_in]]
        if pad:  # the kernels work on whole 16-token groups of a sequence: zero rows are appended (one copy) and cut again
            acts = [th.nn.functional.pad(i, (0, 0, 0, pad)) for i in acts]
        params = [Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias]
        pb = [i.detach().to(th.bfloat16).contiguous() for i in params]
        if not th.compiler.is_compiling():
            _lib.require_cuda(*acts, *pb)
            assert all(i.dtype == th.bfloat16 for i in acts), 'activations must be bfloat16'
            B, _, C = w_in.shape
            D = z_in.shape[2]
            assert all(list(i.shape) == [B, T + pad, C] for i in acts[:2]) and all(list(i.shape) == [B, T + pad, D] for i in acts[2:])
            assert all(list(i.shape) == [C, D] for i in pb[:4]) and all(list(i.shape) == [C] for i in pb[4:])
            assert C % HEAD_SIZE == 0
        outs = _lib.call(_fw_op, fw_loras, *acts, *pb)
        ctx.save_for_backward(*acts, *pb)
        ctx.param_dtypes = [i.dtype for i in params]
        ctx.seq_len, ctx.pad = T, pad
        return tuple(o[:, :T] for o in outs) if pad else tuple(outs)

    @staticmethod
    def backward(ctx, dw_out, dk_out, dz_out, db_out):
        saved = ctx.saved_tensors
        douts = [None if d is None else d.to(th.bfloat16) for d in (dw_out, dk_out, dz_out, db_out)]
        if ctx.pad:
            douts = [None if d is None else th.nn.functional.pad(d, (0, 0, 0, ctx.pad)) for d in douts]
        douts = [th.zeros_like(saved[0]) if d is None else d.contiguous() for d in douts]
        grads = _lib.call(_bw_op, bw_loras, *saved, *douts)
        acts_g = [g[:, :ctx.seq_len] for g in grads[:6]] if ctx.pad else list(grads[:6])
        grads = acts_g + [g.to(t) for g, t in zip(grads[6:], ctx.param_dtypes)]
        return (*grads, None)


expand_loras = ExpandLoras.apply
