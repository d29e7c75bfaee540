"""wkv7_attn_ln_bwd_static: the attn_ln backward for callers that cannot supply a workspace (a
runtime whose pool already owns all device memory, a plugin inside a host application, a thread
that must not trigger cudaMalloc's device-wide synchronisation).  It keeps the scratch for the
per-batch partial parameter gradients in an array built into the library.

Checked here through the C ABI: on two calls in a row, with different inputs, it must return
what wkv7_attn_ln_bwd returns with a caller-allocated workspace (the same kernels run in the same
order, so the comparison is exact), and it must refuse a problem that does not fit its array.
This file sorts last on purpose: a run that stops at the first failure has then already run every
other test.  It passes alone in a fresh process and after the other tests.
"""
import pytest
import torch as th

pytestmark = pytest.mark.gpu

N = 64
NAMES = 'rwkvab'
EPS = 64e-5


def _backward_both_ways(B, T, H, seed):
    from wind_rwkv.rwkv7 import _lib, synthetic
    from wind_rwkv.rwkv7.rwkv7_attn_ln import fw_attn_ln
    L = _lib.lib()
    d = synthetic.wkv7_inputs(B, T, H, N, seed=seed, dtype=th.bfloat16, device='cuda')
    g, params = synthetic.attn_ln_extras(B, T, H, N, seed=seed, dtype=th.bfloat16, device='cuda')
    x = {n: d[n].view(B, T, H, N) for n in list(NAMES) + ['dy']}
    g4 = g.view(B, T, H, N)
    _, sT, ck = fw_attn_ln(x['w'], x['r'], x['k'], x['v'], x['a'], x['b'], g4, params, None)
    st = (T * H * N, H * N, N)

    def outputs():
        return [th.full_like(g4, float('nan')) for _ in range(7)] + [th.full((3, H * N), float('nan'), device='cuda')]

    ins = [x[n].data_ptr() for n in NAMES] + [g4.data_ptr(), params.data_ptr(), x['dy'].data_ptr(), ck.data_ptr(), None, None]
    ref = outputs()
    ws = th.empty(B, 3, H * N, device='cuda')
    rc = L.wkv7_attn_ln_bwd(*ins, *[o.data_ptr() for o in ref], ws.data_ptr(), None, EPS, B, T, H, N, *st, 0, None)
    assert rc == 0
    got = outputs()
    before = th.cuda.memory_allocated()
    rc = L.wkv7_attn_ln_bwd_static(*ins, *[o.data_ptr() for o in got], None, EPS, B, T, H, N, *st, 0, None)
    assert rc == 0
    th.cuda.synchronize()
    assert th.cuda.memory_allocated() == before
    return ref, got


def test_static_scratch_matches_workspace_variant_twice():
    for seed, (B, T, H) in enumerate([(3, 64, 2), (5, 32, 4)]):
        ref, got = _backward_both_ways(B, T, H, seed=20 + seed)
        for i, (a, b) in enumerate(zip(ref, got)):
            assert bool(th.isfinite(b.float()).all()), f'output {i} not written'
            assert th.equal(a, b), f'output {i} differs on call {seed + 1}'


def test_static_scratch_rejects_oversized_problem():
    from wind_rwkv.rwkv7 import _lib
    L = _lib.lib()
    p = 0x1000
    big_B = (4 << 20) // (3 * 64 * 4) + 1  # one batch entry more than the array holds at H=1
    rc = L.wkv7_attn_ln_bwd_static(*([p] * 20), None, EPS, big_B, 16, 1, N, 16 * N, N, N, 0, None)
    assert rc == -10
    assert b'WKV7_STATIC_SCRATCH_BYTES' in L.wkv7_status_string(rc)
