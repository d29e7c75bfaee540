"""Parity of the fused attn_ln op (WKV7 + per-head GroupNorm + bonus + gate) with the oracle.
Tolerances as in test_attn_gpu.py; dparams is an fp32 output and is held to 2e-2 (bf16 path) /
1e-4 (fp32 path) of its RMS."""
import numpy as np
import pytest
import torch as th

from test_attn_gpu import N, NAMES, check, maxabs_rms, rel_l2

pytestmark = pytest.mark.gpu


@pytest.fixture(params=[4, 0], ids=['tcgen05', 'mma'], autouse=True)
def fwd_impl(request):
    """Every test of this file runs with both bf16 forward kernels (the fp32 paths ignore the switch)."""
    from wind_rwkv.rwkv7 import _lib
    old = _lib.set_fwd_impl(request.param)
    yield request.param
    _lib.set_fwd_impl(old)


def run_case(B, T, H, dtype, seed=0, upstream_params=False, s0=False):
    import c_oracle
    from wind_rwkv.rwkv7 import _lib, attn_ln, synthetic
    d = synthetic.wkv7_inputs(B, T, H, N, seed=seed, dtype=dtype, dist='upstream' if upstream_params else 'baseline',
                              s0_std=0.1 if s0 else None)
    if upstream_params:  # tests/test_attn_ln.py:33-39: g ~ N(0,1), params ~ N(0,1)
        gen = th.Generator().manual_seed(seed + 3)
        g = th.randn(B, T, H * N, generator=gen).to(dtype)
        params = th.randn(3, H * N, generator=gen)
    else:
        g, params = synthetic.attn_ln_extras(B, T, H, N, seed=seed, dtype=dtype)
    cpu = {n: d[n].double().numpy().reshape(B, T, H, N) for n in list(NAMES) + ['dy']}
    g4 = g.double().numpy().reshape(B, T, H, N)
    s0n = d['s0'].numpy() if s0 else None
    dev = [d[n].cuda().requires_grad_() for n in NAMES]
    gd, pd = g.cuda().requires_grad_(), params.cuda().requires_grad_()
    s0d = th.from_numpy(s0n).cuda().requires_grad_() if s0 else None
    y = attn_ln(*dev, gd, pd, N, s0=s0d)
    y.backward(d['dy'].cuda())
    out, _, _ = c_oracle.attn_ln_fwd(*[cpu[n] for n in NAMES], g4, params.double().numpy(), s0=s0n)
    go = c_oracle.attn_ln_bwd(*[cpu[n] for n in NAMES], g4, params.double().numpy(), cpu['dy'], s0=s0n)
    check('y', y, out, dtype)
    for n, x, ref in zip(NAMES, dev, go[:6]):
        check('d' + n, x.grad, ref, dtype, through_groupnorm=True)
    check('dg', gd.grad, go[6], dtype)
    e = maxabs_rms(pd.grad, go[7])
    assert e <= (1e-4 if dtype == th.float32 else 2e-2), f'dparams: {e:.2e}'
    if s0:
        e = maxabs_rms(s0d.grad, go[8])
        assert e <= (1e-4 if dtype == th.float32 else 2e-2), f'ds0: {e:.2e}'
    assert _lib.device_status() == 0


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_small(dtype):
    run_case(1, 32, 2, dtype)


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_upstream_test_distribution(dtype):
    run_case(2, 256, 3, dtype, seed=2, upstream_params=True)


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_with_initial_state(dtype):
    run_case(2, 128, 2, dtype, seed=4, s0=True)


def test_golden(golden):
    """The committed output and gradients of upstream's ref_attn_ln (tests/test_attn_ln.py:6-21)."""
    from wind_rwkv.rwkv7 import attn_ln
    g = golden('attn_ln_small.npz')
    names = list(NAMES) + ['g', 'params']
    dev = [th.from_numpy(g[n]).cuda().requires_grad_() for n in names]
    y = attn_ln(*dev, N)
    y.backward(th.from_numpy(g['dy']).cuda())
    assert maxabs_rms(y, g['y']) <= 1e-4
    for n, x in zip(names, dev):
        assert maxabs_rms(x.grad, g['d' + n]) <= 1e-4, n


def test_dparams_is_deterministic():
    from wind_rwkv.rwkv7 import attn_ln, synthetic
    B, T, H = 8, 128, 4
    d = synthetic.wkv7_inputs(B, T, H, N, seed=6, dtype=th.bfloat16, device='cuda')
    g, params = synthetic.attn_ln_extras(B, T, H, N, seed=6, dtype=th.bfloat16, device='cuda')
    res = []
    for _ in range(2):
        p = params.clone().requires_grad_()
        attn_ln(*[d[n] for n in NAMES], g, p, N).backward(d['dy'])
        res.append(p.grad.clone())
    assert th.equal(res[0], res[1])


def test_config2_full_batch():
    """1.5B shape at its real batch (B16 T4096 H32): finite everywhere; batch entry 11, heads 5-6 against the oracle.

    y and dparams meet the usual bounds.  For the gradients the per-element bound of check() (rounding floor + 2e-2)
    is exceeded at a handful of time steps: over 4096 steps there are steps where the recurrence output of a head has
    a spread far below its RMS, GroupNorm divides by that spread and amplifies the TF32-level error of y in that step's
    gradients (the fp32 path shows the same amplification at its own level).  That explanation is tested, not assumed:
    no step exceeds 3 x floor, at most 0.2 % of the steps exceed floor + 2e-2 (measured: 0 to 6 of 8192), and at least
    half of those lie in the lowest decile of spread / RMS of the oracle's recurrence output."""
    import c_oracle
    from wind_rwkv.rwkv7 import _lib, attn_ln, synthetic
    B, T, H = 16, 4096, 32
    d = synthetic.wkv7_inputs(B, T, H, N, seed=7, dtype=th.bfloat16, device='cuda')
    g, params = synthetic.attn_ln_extras(B, T, H, N, seed=7, dtype=th.bfloat16, device='cuda')
    dev = [d[n].requires_grad_() for n in NAMES]
    gd, pd = g.requires_grad_(), params.requires_grad_()
    y = attn_ln(*dev, gd, pd, N)
    y.backward(d['dy'])
    assert bool(th.isfinite(y).all()) and all(bool(th.isfinite(x.grad).all()) for x in dev + [gd, pd])
    bsel, hs = 11, slice(5 * N, 7 * N)
    cut = lambda x: x.detach()[bsel:bsel + 1, :, hs].double().cpu().numpy().reshape(1, T, 2, N)
    ins = [cut(x) for x in dev]
    prm = params.detach()[:, hs].double().cpu().numpy()
    out, _, _ = c_oracle.attn_ln_fwd(*ins, cut(gd), prm)
    go = c_oracle.attn_ln_bwd(*ins, cut(gd), prm, cut(d['dy']))
    check('y', y[bsel:bsel + 1, :, hs], out, th.bfloat16)
    yrec, _ = c_oracle.wkv7_fwd(*ins)                     # the recurrence output the GroupNorm sees
    spread = yrec.std(axis=-1) / np.sqrt(np.mean(yrec ** 2))   # [1, T, 2]
    low = np.quantile(spread, 0.1)
    for n, x, ref in zip(list(NAMES) + ['g'], dev + [gd], go[:7]):
        got = x.grad[bsel:bsel + 1, :, hs].double().cpu().numpy().reshape(1, T, 2, N)
        rms = np.sqrt(np.mean(ref ** 2))
        fl = np.abs(th.from_numpy(ref).to(th.bfloat16).double().numpy() - ref).max() / rms
        per_step = np.abs(got - ref).max(axis=-1) / rms
        over = per_step > fl + 2e-2
        print(f'd{n}: max {per_step.max():.2e}, floor {fl:.2e}, steps over floor + 2e-2: {int(over.sum())} of {over.size}, '
              f'of which in the lowest decile of spread: {int((spread[over] <= low).sum())}')
        assert rel_l2(x.grad[bsel:bsel + 1, :, hs], ref) <= 4e-3, n
        assert per_step.max() <= 3 * fl, f'd{n}: {per_step.max():.2e} vs floor {fl:.2e}'
        assert over.sum() <= 0.002 * over.size, f'd{n}: {int(over.sum())} steps over floor + 2e-2'
        assert over.sum() < 2 or (spread[over] <= low).sum() * 2 >= over.sum(), f'd{n}: the outliers are not at low-spread steps'
    # dparams sums over the whole batch: the oracle on this slice cannot check it; it is checked at B = 1 below
    assert _lib.device_status() == 0


def test_config2_dparams_slice():
    """dparams at the config-2 sequence length (B1 T4096, 2 of 32 heads against the oracle)."""
    import c_oracle
    from wind_rwkv.rwkv7 import attn_ln, synthetic
    B, T, H = 1, 4096, 32
    d = synthetic.wkv7_inputs(B, T, H, N, seed=7, dtype=th.bfloat16, device='cuda')
    g, params = synthetic.attn_ln_extras(B, T, H, N, seed=7, dtype=th.bfloat16, device='cuda')
    dev = [d[n] for n in NAMES]
    pd = params.requires_grad_()
    attn_ln(*dev, g, pd, N).backward(d['dy'])
    hs = slice(5 * N, 7 * N)
    cut = lambda x: x.detach()[:, :, hs].double().cpu().numpy().reshape(B, T, 2, N)
    go = c_oracle.attn_ln_bwd(*[cut(x) for x in dev], cut(g), params.detach()[:, hs].double().cpu().numpy(), cut(d['dy']))
    assert maxabs_rms(pd.grad[:, hs], go[7]) <= 2e-2
