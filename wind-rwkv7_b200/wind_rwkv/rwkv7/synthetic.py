"""Seeded synthetic inputs with the shapes and value distributions of the WKV7 workloads.

Distributions: r,k,v ~ N(0,1); raw decay input w ~ N(-0.6, 0.5^2) (the op applies
exp(-exp(w)) itself); kappa = unit-L2-normalised N(0,1) per head; a = -kappa;
b = kappa * sigmoid(N(0,1)); upstream gradient dy ~ N(0,1).  The upstream test
scripts draw from slightly different distributions (tests/test_attn.py:25-30:
w = -softplus(N(0,1)) - 0.5, a = kappa, b = -a*sigmoid(.)); `dist='upstream'`
selects those.

Values are generated in fp32, rounded once to `dtype`, so that a checker can
upcast the very same rounded values.
"""
import torch as th

F = th.nn.functional


def wkv7_inputs(B, T, H, N=64, seed=0, dtype=th.bfloat16, device='cpu', dist='baseline', s0_std=None):
    """Returns dict with r,w,k,v,a,b,dy of shape [B,T,H*N] (dtype) and optional fp32 s0 [B,H,N,N]."""
    gen = th.Generator(device=device)
    gen.manual_seed(seed)

    def rn(*shape):
        return th.randn(*shape, generator=gen, device=device, dtype=th.float32)

    r, k, v, dy = rn(B, T, H, N), rn(B, T, H, N), rn(B, T, H, N), rn(B, T, H, N)
    if dist == 'baseline':
        w = rn(B, T, H, N) * 0.5 - 0.6
        kappa = F.normalize(rn(B, T, H, N), dim=-1)
        a = -kappa
        b = kappa * th.sigmoid(rn(B, T, H, N))
    elif dist == 'upstream':
        w = -F.softplus(rn(B, T, H, N)) - 0.5
        a = F.normalize(rn(B, T, H, N), dim=-1)
        b = -a * th.sigmoid(rn(B, T, H, N))
    else:
        raise ValueError(dist)
    out = {n: x.to(dtype).view(B, T, H * N) for n, x in dict(r=r, w=w, k=k, v=v, a=a, b=b, dy=dy).items()}
    if s0_std is not None:
        out['s0'] = rn(B, H, N, N) * s0_std
    return out


def attn_ln_extras(B, T, H, N=64, seed=0, dtype=th.bfloat16, device='cpu'):
    """g = sigmoid(N(0,1)) [B,T,H*N]; params fp32 [3,H*N] = (ln_w ~ 1+N(0,0.1), ln_b = 0, bonus ~ N(0,0.1))."""
    gen = th.Generator(device=device)
    gen.manual_seed(seed + 7919)
    g = th.sigmoid(th.randn(B, T, H * N, generator=gen, device=device)).to(dtype)
    ln_w = 1 + 0.1 * th.randn(H * N, generator=gen, device=device)
    ln_b = th.zeros(H * N, device=device)
    bonus = 0.1 * th.randn(H * N, generator=gen, device=device)
    return g, th.stack([ln_w, ln_b, bonus]).float()
