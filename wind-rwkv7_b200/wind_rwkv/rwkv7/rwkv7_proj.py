"""Narrow projections of the time mixer with the activation fused: `proj(x, W, tanh_cols)` = act(x @ W^T).

Upstream computes the first stages of its LoRAs as `x @ W.bfloat16().mT` followed, where the second stage wants it,
by a separate `torch.tanh` pass (time_mixer.py:120-131).  Here the product runs on the tcgen05 kernel of
csrc/proj_gemm.cu (bf16 operands, fp32 accumulation in tensor memory, operands by bulk tensor loads) and tanh is applied
to the chosen output columns before they are stored.  For the narrow outputs of the LoRA first stages (32 to 128
columns) this is faster than the library GEMM plus the extra pass; the square projections stay library calls.
The backward uses library matmuls (d tanh = 1 - tanh^2 from the stored output).
"""
import torch as th

from . import _lib


def fw_proj(x, w, tanh_from, tanh_to):
    """Launcher: x [..., K] bf16 contiguous, w [N, K] bf16 contiguous -> [..., N] bf16."""
    K = x.shape[-1]
    N = w.shape[0]
    M = x.numel() // K
    out = th.empty(*x.shape[:-1], N, dtype=th.bfloat16, device=x.device)
    with _lib.on_device(x, w):
        rc = _lib.lib().wkv7_proj_gemm(x.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K, tanh_from, tanh_to, _lib.stream_of(x))
    _lib.check(rc, 'wkv7_proj_gemm')
    return out


def _fake_fw(x, w, tanh_from, tanh_to):
    return x.new_empty((*x.shape[:-1], w.shape[0]), dtype=th.bfloat16)


_fw_op = _lib.opaque_op('proj_gemm', fw_proj, _fake_fw, '(Tensor x, Tensor w, int tanh_from, int tanh_to) -> Tensor')


class Proj(th.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, tanh_from, tanh_to):
        if not th.compiler.is_compiling():
            _lib.require_cuda(x, w)
            assert x.dtype == th.bfloat16 and w.dtype == th.bfloat16, 'proj takes bfloat16 tensors'
            assert w.dim() == 2 and w.shape[1] == x.shape[-1] and 0 <= tanh_from <= tanh_to <= w.shape[0]
        x, w = x.contiguous(), w.contiguous()
        out = _lib.call(_fw_op, fw_proj, x, w, tanh_from, tanh_to)
        ctx.save_for_backward(x, w, out)
        ctx.cols = (tanh_from, tanh_to)
        return out

    @staticmethod
    def backward(ctx, dout):
        x, w, out = ctx.saved_tensors
        f, t = ctx.cols
        dpre = dout.to(th.bfloat16)
        if t > f:  # d tanh = 1 - tanh^2, from the stored output: g - (g y) y
            if f == 0 and t == out.shape[-1]:
                dpre = th.addcmul(dpre, dpre * out, out, value=-1)
            else:
                dpre = dpre.clone()
                g, y = dpre[..., f:t], out[..., f:t]
                g.copy_(th.addcmul(g, g * y, y, value=-1))
        dx = dpre @ w
        dw = dpre.reshape(-1, dpre.shape[-1]).mT @ x.reshape(-1, x.shape[-1])
        return dx, dw, None, None


def proj(x, w, tanh_cols=None):
    """act(x @ w^T): x [..., K] bf16, w [N, K] bf16; tanh on output columns tanh_cols = (from, to), identity elsewhere."""
    f, t = tanh_cols if tanh_cols is not None else (0, 0)
    return Proj.apply(x, w, int(f), int(t))
