"""Generates the golden vectors under tests/golden/ by running the UPSTREAM reference code.

Run where a checkout of upstream (johanwind/wind-rwkv7) is available and name it in
WIND_RWKV_REFERENCE or as the first argument; the produced .npz files are
committed, so the tests themselves never need the checkout:

    WIND_RWKV_REFERENCE=<path to the upstream checkout> python tests/golden/make_golden.py

Every fixture stores the seeded inputs and what upstream's own fp32 reference
functions return for them (outputs, and gradients from autograd through them):

  attn_cfg0.npz      time_mixer.ref_attn and tests/test_attn.ref_attn, B1 T64 H2 N64 (fp32)
  attn_carry.npz     the same function on T=128: pins the s0 -> sT carry (two
                     chained 64-step calls must reproduce one 128-step call)
  attn_ln_small.npz  tests/test_attn_ln.ref_attn_ln
  ddlerp_small.npz   tests/test_ddlerp.ref_ddlerp
  loras_small.npz    tests/test_expand_loras.ref_expand_loras
  mixer_small.npz    tests/test_time_mixer.RefTimeMixer (class body executed from
                     the script's source; the script itself needs a GPU at import)
"""
import os
import sys
import types

import numpy as np
import torch as th

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get('WIND_RWKV_REFERENCE')
if not REF or not os.path.isdir(REF):
    sys.exit('make_golden.py: give the upstream checkout in WIND_RWKV_REFERENCE or as the first argument')
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, 'tests'))
sys.path.insert(0, os.path.join(HERE, '..', '..', 'wind-rwkv7_b200', 'wind_rwkv', 'rwkv7'))

import synthetic  # noqa: E402  (our seeded input generator; a plain module import, not the package)
import wind_rwkv.rwkv7.time_mixer as up_tm  # noqa: E402  upstream
import test_attn as up_attn  # noqa: E402
import test_attn_ln as up_attn_ln  # noqa: E402
import test_ddlerp as up_ddlerp  # noqa: E402
import test_expand_loras as up_loras  # noqa: E402

assert up_tm.__file__.startswith(REF), up_tm.__file__
F = th.nn.functional


def grads(f, inputs, dys_seed):
    xs = [x.clone().requires_grad_() for x in inputs]
    ys = f(*xs)
    if not isinstance(ys, tuple):
        ys = (ys,)
    gen = th.Generator().manual_seed(dys_seed)
    dys = tuple(th.randn(y.shape, generator=gen).to(y.dtype) for y in ys)
    th.autograd.backward(ys, dys)
    return ys, dys, [x.grad if x.grad is not None else th.zeros_like(x) for x in xs]


def save(name, **kw):
    out = {}
    for k, v in kw.items():
        out[k] = v.detach().float().numpy() if isinstance(v, th.Tensor) else np.asarray(v)
    path = os.path.join(HERE, name)
    np.savez_compressed(path, **out)
    print(name, os.path.getsize(path) // 1024, 'KiB')


def attn_cfg0():
    d = synthetic.wkv7_inputs(1, 64, 2, 64, seed=0, dtype=th.float32)
    ins = [d[n] for n in 'rwkvab']
    (y,), (dy,), g = grads(lambda *x: up_tm.ref_attn(*x, 64), ins, 100)
    y2 = up_attn.ref_attn(*ins, 64)
    assert th.equal(y, y2), 'the two upstream copies of ref_attn disagree'
    save('attn_cfg0.npz', **{n: d[n] for n in 'rwkvab'}, y=y, dy=dy,
         **{'d' + n: gi for n, gi in zip('rwkvab', g)})


def attn_carry():
    d = synthetic.wkv7_inputs(2, 128, 1, 64, seed=1, dtype=th.float32)
    ins = [d[n] for n in 'rwkvab']
    y = up_attn.ref_attn(*ins, 64)
    save('attn_carry.npz', **{n: d[n] for n in 'rwkvab'}, y=y)


def attn_ln_small():
    B, T, H, N = 1, 32, 2, 64
    d = synthetic.wkv7_inputs(B, T, H, N, seed=2, dtype=th.float32, dist='upstream')
    gen = th.Generator().manual_seed(5)
    g = th.randn(B, T, H * N, generator=gen)
    params = th.randn(3, H * N, generator=gen)
    ins = [d[n] for n in 'rwkvab'] + [g, params]
    (y,), (dy,), gr = grads(lambda *x: up_attn_ln.ref_attn_ln(*x, N), ins, 101)
    save('attn_ln_small.npz', **{n: d[n] for n in 'rwkvab'}, g=g, params=params, y=y, dy=dy,
         **{'d' + n: gi for n, gi in zip(['r', 'w', 'k', 'v', 'a', 'b', 'g', 'params'], gr)})


def ddlerp_small():
    B, T, C, D = 2, 64, 128, 16
    gen = th.Generator().manual_seed(6)
    x, mix, W1, W2, bias = [th.randn(*s, generator=gen) / 2 for s in [(B, T, C), (C,), (D * 4, C), (4, C, D), (4, 1, 1, C)]]
    ins = [x, mix, W1, W2, bias]
    ys, dys, gr = grads(up_ddlerp.ref_ddlerp, ins, 102)
    save('ddlerp_small.npz', x=x, alpha=mix, L=W1, R=W2, beta=bias,
         **{f'y{i}': y for i, y in enumerate(ys)}, **{f'dy{i}': y for i, y in enumerate(dys)},
         **{'d' + n: gi for n, gi in zip(['x', 'alpha', 'L', 'R', 'beta'], gr)})


def loras_small():
    B, T, C, D, N = 2, 32, 128, 16, 64
    up_loras.B, up_loras.T, up_loras.C = B, T, C  # upstream's reference reads these module globals
    gen = th.Generator().manual_seed(7)
    shapes = [(B, T, C)] * 2 + [(B, T, D)] * 4 + [(C, D)] * 4 + [(C,)] * 4
    ins = [th.randn(*s, generator=gen).bfloat16().float() for s in shapes]
    names = ['w_in', 'k_in', 'z_in', 'a_in', 'ma_in', 'mk_in', 'Wz', 'Wa', 'Wma', 'Wmk', 'w_bias', 'a_bias', 'ma_bias', 'mk_bias']
    ys, dys, gr = grads(lambda *x: up_loras.ref_expand_loras(*x, N), ins, 103)
    save('loras_small.npz', **dict(zip(names, ins)),
         **{f'y{i}': y for i, y in enumerate(ys)}, **{f'dy{i}': y for i, y in enumerate(dys)},
         **{'d' + n: gi for n, gi in zip(names, gr)})


def mixer_small():
    from collections import namedtuple
    src = open(os.path.join(REF, 'tests', 'test_time_mixer.py')).read()
    head = src.split('\nB1 = ')[0]  # imports + the RefTimeMixer class, nothing that touches a GPU
    mod = types.ModuleType('up_test_time_mixer')
    import wind_rwkv.rwkv7 as up_pkg
    up_pkg.load_attn_ln = lambda *a, **k: None  # constructing TimeMixer would JIT-build a CUDA extension
    exec(compile(head, 'test_time_mixer.py', 'exec'), mod.__dict__)
    HC, N, B, T = 128, 64, 1, 32
    th.manual_seed(8)
    cfg = namedtuple('Config', ['n_layer', 'n_head', 'n_embd'])(12, HC // N, HC)
    model = mod.RefTimeMixer(cfg, 6)
    params = dict(model.named_parameters())
    gen = th.Generator().manual_seed(9)
    vals = [th.randn(p.shape, generator=gen) * 0.1 for p in params.values()]
    x = th.randn(B, T, HC, generator=gen)

    def f(*ins):
        return th.func.functional_call(model, dict(zip(params.keys(), ins[:-1])), (ins[-1],))
    (y,), (dy,), gr = grads(f, vals + [x], 104)
    save('mixer_small.npz', x=x, y=y, dy=dy, dx=gr[-1], n_head=HC // N,
         **{'p.' + n: v for n, v in zip(params.keys(), vals)},
         **{'dp.' + n: gi for n, gi in zip(params.keys(), gr[:-1])})


if __name__ == '__main__':
    th.set_grad_enabled(True)
    attn_cfg0()
    attn_carry()
    attn_ln_small()
    ddlerp_small()
    loras_small()
    mixer_small()
