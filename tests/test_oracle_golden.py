"""Pins the oracle (torch restatement and C restatement) against the committed golden vectors,
which were produced by upstream's own reference functions (tests/golden/make_golden.py)."""
import numpy as np
import torch as th

import c_oracle
import wkv7_ref

NAMES = 'rwkvab'


def t(x):
    return th.from_numpy(np.asarray(x))


def rel(a, b):
    a, b = np.asarray(a, dtype=np.float64), np.asarray(b, dtype=np.float64)
    return np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-30)


def test_attn_cfg0_torch_restatement_is_bit_exact(golden):
    g = golden('attn_cfg0.npz')
    ins = [t(g[n]).requires_grad_() for n in NAMES]
    y = wkv7_ref.ref_attn(*ins, 64)
    assert th.equal(y, t(g['y']))
    y.backward(t(g['dy']))
    for n, x in zip(NAMES, ins):
        assert th.equal(x.grad, t(g['d' + n])), n


def test_attn_cfg0_c_oracle(golden):
    g = golden('attn_cfg0.npz')
    B, T, H, N = 1, 64, 2, 64
    ins = [g[n].reshape(B, T, H, N) for n in NAMES]
    for dtype, tol in ((np.float32, 2e-6), (np.float64, 2e-6)):  # golden itself is fp32
        y, sT = c_oracle.wkv7_fwd(*ins, dtype=dtype)
        assert rel(y.reshape(B, T, -1), g['y']) < tol
        grads = c_oracle.wkv7_bwd(*ins, g['dy'].reshape(B, T, H, N), dtype=dtype)
        for n, x in zip(NAMES, grads):
            assert rel(x.reshape(B, T, -1), g['d' + n]) < tol, n


def test_state_carry_matches_one_long_call(golden):
    g = golden('attn_carry.npz')
    B, T, H, N = 2, 128, 1, 64
    ins = [g[n].reshape(B, T, H, N) for n in NAMES]
    y_full, sT_full = c_oracle.wkv7_fwd(*ins, dtype=np.float64)
    assert rel(y_full.reshape(B, T, -1), g['y']) < 2e-6
    y1, s1 = c_oracle.wkv7_fwd(*[x[:, :64] for x in ins], dtype=np.float64)
    y2, s2 = c_oracle.wkv7_fwd(*[x[:, 64:] for x in ins], s0=s1, dtype=np.float64)
    assert rel(np.concatenate([y1, y2], 1).reshape(B, T, -1), g['y']) < 2e-6
    assert rel(s2, sT_full) < 1e-12
    # torch restatement, same property
    tin = [t(g[n]) for n in NAMES]
    ya, sa = wkv7_ref.ref_attn(*[x[:, :64] for x in tin], 64, return_state=True)
    yb, sb = wkv7_ref.ref_attn(*[x[:, 64:] for x in tin], 64, s0=sa, return_state=True)
    assert rel(th.cat([ya, yb], 1).numpy(), g['y']) < 1e-6
    assert rel(sb.numpy(), sT_full) < 1e-5


def test_c_oracle_state_gradients_match_autograd():
    th.manual_seed(3)
    B, T, H, N = 1, 48, 2, 64
    from wind_rwkv.rwkv7 import synthetic
    d = synthetic.wkv7_inputs(B, T, H, N, seed=11, dtype=th.float64, s0_std=0.1)
    ins = [d[n].double().requires_grad_() for n in NAMES]
    s0 = d['s0'].double().requires_grad_()
    y, sT = wkv7_ref.ref_attn(*ins, N, s0=s0, return_state=True, compute_dtype=th.float64)
    dy, dsT = th.randn_like(y), th.randn_like(sT)
    th.autograd.backward([y, sT], [dy, dsT])
    to4 = lambda x: x.detach().numpy().reshape(B, T, H, N)
    yc, sTc = c_oracle.wkv7_fwd(*[to4(x) for x in ins], s0=s0.detach().numpy())
    assert rel(yc, to4(y)) < 1e-12 and rel(sTc, sT.detach().numpy()) < 1e-12
    gr = c_oracle.wkv7_bwd(*[to4(x) for x in ins], to4(dy), s0=s0.detach().numpy(), dsT=dsT.numpy())
    for n, x, ref in zip(NAMES, gr[:6], ins):
        assert rel(x, to4(ref.grad)) < 1e-11, n
    assert rel(gr[6], s0.grad.numpy()) < 1e-11


def test_attn_ln_golden(golden):
    g = golden('attn_ln_small.npz')
    B, T, H, N = 1, 32, 2, 64
    names = list(NAMES) + ['g', 'params']
    ins = [t(g[n]).requires_grad_() for n in names]
    y = wkv7_ref.ref_attn_ln(*ins, N)
    assert rel(y.detach().numpy(), g['y']) < 1e-6
    y.backward(t(g['dy']))
    for n, x in zip(names, ins):
        assert rel(x.grad.numpy(), g['d' + n]) < 1e-5, n
    # C oracle
    ins4 = [g[n].reshape(B, T, H, N) for n in list(NAMES) + ['g']]
    out, _, _ = c_oracle.attn_ln_fwd(*ins4, g['params'])
    assert rel(out.reshape(B, T, -1), g['y']) < 2e-6
    gr = c_oracle.attn_ln_bwd(*ins4, g['params'], g['dy'].reshape(B, T, H, N))
    for n, x in zip(['r', 'w', 'k', 'v', 'a', 'b', 'g'], gr[:7]):
        assert rel(x.reshape(B, T, -1), g['d' + n]) < 5e-6, n
    assert rel(gr[7], g['dparams']) < 5e-6


def test_ddlerp_golden(golden):
    g = golden('ddlerp_small.npz')
    names = ['x', 'alpha', 'L', 'R', 'beta']
    ins = [t(g[n]).requires_grad_() for n in names]
    ys = wkv7_ref.ref_ddlerp(*ins)
    for i, y in enumerate(ys):
        assert th.equal(y, t(g[f'y{i}']))
    th.autograd.backward(ys, [t(g[f'dy{i}']) for i in range(4)])
    for n, x in zip(names, ins):
        assert rel(x.grad.numpy(), g['d' + n]) < 1e-6, n


def test_expand_loras_golden(golden):
    g = golden('loras_small.npz')
    names = ['w_in', 'k_in', 'z_in', 'a_in', 'ma_in', 'mk_in', 'Wz', 'Wa', 'Wma', 'Wmk', 'w_bias', 'a_bias', 'ma_bias', 'mk_bias']
    ins = [t(g[n]).requires_grad_() for n in names]
    ys = wkv7_ref.ref_expand_loras(*ins, 64)
    for i, y in enumerate(ys):
        assert th.equal(y.float(), t(g[f'y{i}']))
    th.autograd.backward(ys, [t(g[f'dy{i}']).bfloat16() for i in range(4)])
    for n, x in zip(names, ins):
        assert rel(x.grad.numpy(), g['d' + n]) < 1e-6, n


def test_time_mixer_golden(golden):
    g = golden('mixer_small.npz')
    p = {k[2:]: t(v).requires_grad_() for k, v in g.items() if k.startswith('p.')}
    x = t(g['x']).requires_grad_()
    y = wkv7_ref.ref_time_mixer(p, x, int(g['n_head']))
    assert rel(y.detach().numpy(), g['y']) < 1e-6
    y.backward(t(g['dy']))
    assert rel(x.grad.numpy(), g['dx']) < 1e-5
    for n, v in p.items():
        ref = g['dp.' + n]
        if np.linalg.norm(ref) > 0:
            assert rel(v.grad.numpy(), ref) < 1e-4, n
