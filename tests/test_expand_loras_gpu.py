"""Parity of the expand_loras kernels with upstream's fp32 reference (tests/test_expand_loras.py:6-19),
restated in oracle/wkv7_ref.py and pinned by tests/golden/loras_small.npz.  All inputs are bf16 (as
upstream's test feeds them), so kernels and oracle see identical values.

Tolerances: bf16 outputs and input gradients within 3x the bf16 rounding floor of the same tensor
and relative L2 <= 1e-2 (upstream's tolerance); fp32 weight and bias gradients within 2e-2 of their
RMS (max-abs)."""
import pytest
import torch as th

from test_attn_gpu import floor_of, maxabs_rms, rel_l2

pytestmark = pytest.mark.gpu
NAMES = ['w_in', 'k_in', 'z_in', 'a_in', 'ma_in', 'mk_in', 'Wz', 'Wa', 'Wma', 'Wmk', 'w_bias', 'a_bias', 'ma_bias', 'mk_bias']


def data(B, T, C, D, seed, scale=1.0):
    gen = th.Generator().manual_seed(seed)  # tests/test_expand_loras.py:37-45: all randn, bf16
    shapes = [(B, T, C)] * 2 + [(B, T, D)] * 4 + [(C, D)] * 4 + [(C,)] * 4
    t = [th.randn(*s, generator=gen) for s in shapes]
    return [x.bfloat16() for x in t[:6]] + [(x * scale).bfloat16() for x in t[6:]]


def run_case(B, T, C, D, seed=0, scale=1.0):
    import wkv7_ref
    from wind_rwkv.rwkv7 import expand_loras
    ins = data(B, T, C, D, seed, scale)
    ref_in = [i.double().requires_grad_() for i in ins]
    ys_ref = wkv7_ref.ref_expand_loras(*ref_in, 64, compute_dtype=th.float64, out_dtype=th.float64)
    gen = th.Generator().manual_seed(seed + 1)
    dys = [th.randn(B, T, C, generator=gen).bfloat16() for _ in range(4)]
    th.autograd.backward(ys_ref, [d.double() for d in dys])
    dev = [i.cuda().requires_grad_() for i in ins[:6]] + [i.float().cuda().requires_grad_() for i in ins[6:]]
    ys = expand_loras(*dev, 64)
    th.autograd.backward(ys, [d.cuda() for d in dys])
    checks = [(n, y, yr.detach().numpy()) for n, y, yr in zip(['w', 'k', 'kk', 'b'], ys, ys_ref)]
    checks += [('d' + n, a.grad, b.grad.numpy()) for n, a, b in zip(NAMES[:6], dev[:6], ref_in[:6])]
    for n, got, ref in checks:
        e, fl, r = maxabs_rms(got, ref), floor_of(ref, th.bfloat16), rel_l2(got, ref)
        assert e <= 3 * fl and r <= 1e-2, f'{n}: {e:.2e} (floor {fl:.2e}), rel {r:.2e}'
    for n, a, b in zip(NAMES[6:], dev[6:], ref_in[6:]):
        e = maxabs_rms(a.grad, b.grad.numpy())
        assert e <= 2e-2, f'd{n}: {e:.2e}'


def test_small():
    run_case(2, 32, 128, 16)


def test_rank32_ragged_tile():
    run_case(2, 80, 128, 32, seed=2)   # T = 80: the last 64-token tile is partly empty


def test_rank64():
    run_case(1, 64, 128, 64, seed=3)


def test_rank128():
    run_case(1, 64, 128, 128, seed=5)


def test_sequence_length_not_a_multiple_of_16():
    """T = 40: padded to 48 inside the wrapper; outputs, input gradients and weight gradients as for any other length."""
    run_case(2, 40, 128, 16, seed=6)


def test_mixer_shape():
    """C = 768, D = 16 as in the time mixer (tests/test_expand_loras.py:48-52), batch 2."""
    run_case(2, 1024, 768, 16, seed=4)


def test_mixer_shape_small_weights():
    run_case(2, 1024, 768, 16, seed=5, scale=0.1)


def test_golden(golden):
    from wind_rwkv.rwkv7 import expand_loras
    g = golden('loras_small.npz')
    dev = [th.from_numpy(g[n]).bfloat16().cuda().requires_grad_() for n in NAMES[:6]] + \
          [th.from_numpy(g[n]).cuda().requires_grad_() for n in NAMES[6:]]
    ys = expand_loras(*dev, 64)
    th.autograd.backward(ys, [th.from_numpy(g[f'dy{i}']).bfloat16().cuda() for i in range(4)])
    for i, y in enumerate(ys):
        assert rel_l2(y, g[f'y{i}']) <= 1e-2      # the fixture's outputs are already bf16-rounded
    for n, t in zip(NAMES, dev):
        assert rel_l2(t.grad, g['d' + n]) <= 1e-2, n


def test_rejects_other_head_sizes():
    from wind_rwkv.rwkv7 import expand_loras
    ins = [i.cuda() for i in data(1, 16, 128, 16, 0)]
    with pytest.raises(ValueError):
        expand_loras(*ins, 32)
