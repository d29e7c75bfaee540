"""The tcgen05 projection kernel (C = act(A W^T), tanh on a column range) against torch in fp32 on the same bf16
values.  bf16 outputs: within the bf16 rounding of the result (half an ulp of the largest element) plus the error of
the hardware tanh (2^-11 relative); gradients against autograd through the fp32 formula, relative L2 <= 1e-2 (upstream's
tolerance, tests/utils.py:18)."""
import pytest
import torch as th

from test_attn_gpu import floor_of, maxabs_rms, rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('M,N,K,cols', [(128, 128, 64, None), (300, 96, 768, (0, 64)), (1000, 800, 768, (768, 800)),
                                        (4096, 32, 768, None), (77, 128, 128, (0, 128)), (5, 8, 8, (0, 8))])
def test_forward_and_backward(M, N, K, cols):
    from wind_rwkv.rwkv7 import proj
    gen = th.Generator().manual_seed(M + N + K)
    x = th.randn(M, K, generator=gen).bfloat16()
    w = (th.randn(N, K, generator=gen) / K ** 0.5).bfloat16()
    dy = th.randn(M, N, generator=gen).bfloat16()
    xr, wr = x.double().requires_grad_(), w.double().requires_grad_()
    ref = xr @ wr.T
    if cols:
        ref = th.cat([ref[:, :cols[0]], th.tanh(ref[:, cols[0]:cols[1]]), ref[:, cols[1]:]], 1)
    ref.backward(dy.double())
    xd, wd = x.cuda().requires_grad_(), w.cuda().requires_grad_()
    out = proj(xd, wd, cols)
    out.backward(dy.cuda())
    e, fl = maxabs_rms(out, ref.detach().numpy()), floor_of(ref.detach().numpy(), th.bfloat16)
    assert e <= fl + 2e-3, f'output: {e:.2e} vs bf16 rounding floor {fl:.2e}'
    assert rel_l2(xd.grad, xr.grad.numpy()) <= 1e-2 and rel_l2(wd.grad, wr.grad.numpy()) <= 1e-2


def test_batched_shape_and_rejections():
    from wind_rwkv.rwkv7 import _lib, proj
    x = th.randn(2, 48, 64, device='cuda').bfloat16()
    w = th.randn(16, 64, device='cuda').bfloat16()
    assert proj(x, w).shape == (2, 48, 16)
    L = _lib.lib()
    p = x.data_ptr()
    assert L.wkv7_proj_gemm(p, p, p, 8, 12, 64, 0, 0, None) == -4      # N not a multiple of 8
    assert L.wkv7_proj_gemm(p, p, p, 8, 16, 64, 4, 20, None) == -1     # tanh range outside the columns
    assert L.wkv7_proj_gemm(None, p, p, 8, 16, 64, 0, 0, None) == -6
    assert L.wkv7_proj_gemm(None, None, None, 0, 16, 64, 0, 0, None) == 0
