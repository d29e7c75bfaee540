"""Parity of the sm_100a WKV7 kernels with the oracle (the reference's naive recurrence), through
the reference-shaped Python entry points, which call the C ABI of libwkv7_sm100.so.

Tolerances (max-abs error relative to the RMS of the oracle tensor, the metric of the task):
  fp32 path (3xTF32 products)                       <= 1e-4
  bf16 path arithmetic (single-TF32 products),
  observed on fp32 outputs                          <= 2e-2   (measured: y, sT, dr, dk, dv <= 7e-3; da, db <= 1.5e-2;
                                                               dw <= 1.9e-2)
  bf16 outputs: rounding the exact result to bf16 already costs about 2.5e-2 of RMS (half an ulp
  of the largest elements; 3e-2 to 7e-2 for the heavy-tailed da, db, dw), above the 2e-2 bound, so the
  literal metric cannot hold for any bf16 output.  A bf16 output is the rounding of a value that the
  arithmetic bound allows to lie 2e-2 of RMS from the oracle, so it is held to (rounding floor measured
  on the same tensor) + 2e-2 (measured: 1.0 to 1.25 times the floor; 1.6 to 1.7 times on 3 of about 150 tensors), and to a
  relative L2 error <= 4e-3 (bf16 rounding alone gives 1.7e-3; upstream's own tolerance is 1e-2,
  tests/utils.py:18).
"""
import ctypes

import numpy as np
import pytest
import torch as th

pytestmark = pytest.mark.gpu

N = 64
NAMES = 'rwkvab'


@pytest.fixture(params=[4, 0], ids=['tcgen05', 'mma'], autouse=True)
def fwd_impl(request):
    """Every test of this file runs with both bf16 forward kernels: the tcgen05 kernel (state in tensor
    memory, 4 preparation groups: the default) and the warp-MMA kernel.  The fp32 paths ignore it."""
    from wind_rwkv.rwkv7 import _lib
    old = _lib.set_fwd_impl(request.param)
    yield request.param
    _lib.set_fwd_impl(old)


def _mods():
    import c_oracle
    from wind_rwkv.rwkv7 import _lib, attn, synthetic
    from wind_rwkv.rwkv7.rwkv7_attn import WindRWKV7
    return c_oracle, _lib, attn, synthetic, WindRWKV7


def maxabs_rms(x, ref):
    x = x.detach().double().cpu().numpy().reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.abs(x - ref).max() / (np.sqrt(np.mean(ref ** 2)) + 1e-300))


def rel_l2(x, ref):
    x = x.detach().double().cpu().numpy().reshape(-1)
    ref = np.asarray(ref, np.float64).reshape(-1)
    return float(np.linalg.norm(x - ref) / (np.linalg.norm(ref) + 1e-300))


def floor_of(ref, dtype):
    return maxabs_rms(th.from_numpy(np.asarray(ref, np.float64)).to(dtype), ref)


def check(name, x, ref, dtype, through_groupnorm=False):
    """through_groupnorm: gradients of the fused attn_ln op.  At a time step where the recurrence output of a head has
    a small spread, GroupNorm divides by that spread and amplifies the arithmetic error of that step's gradients (the
    fp32 path shows the same amplification at its own level); the per-element bound there is 3 x the rounding floor,
    and tests/test_attn_ln_gpu.py::test_config2_full_batch checks where the excess sits."""
    if dtype == th.float32:
        e = maxabs_rms(x, ref)
        assert e <= 1e-4, f'{name}: {e:.2e} > 1e-4'
    else:
        e, fl, r = maxabs_rms(x, ref), floor_of(ref, dtype), rel_l2(x, ref)
        if through_groupnorm:
            assert e <= 3 * fl, f'{name}: {e:.2e} vs 3 x bf16 rounding floor {fl:.2e}'
        else:
            assert e <= fl + 2e-2, f'{name}: {e:.2e} vs bf16 rounding floor {fl:.2e} + 2e-2'
        assert r <= 4e-3, f'{name}: rel L2 {r:.2e}'


def run_case(B, T, H, dtype, dist='baseline', s0=False, dsT=False, seed=0):
    c_oracle, _lib, attn, synthetic, WindRWKV7 = _mods()
    d = synthetic.wkv7_inputs(B, T, H, N, seed=seed, dtype=dtype, dist=dist, s0_std=0.1 if s0 else None)
    cpu = {n: d[n].double().numpy().reshape(B, T, H, N) for n in list(NAMES) + ['dy']}
    s0n = d['s0'].numpy() if s0 else None
    dsTn = th.randn(B, H, N, N, generator=th.Generator().manual_seed(seed + 1)).numpy() if dsT else None
    dev = {n: d[n].cuda().requires_grad_() for n in NAMES}
    s0d = th.from_numpy(s0n).cuda().requires_grad_() if s0 else None
    y, sT = attn(*[dev[n] for n in NAMES], N, s0=s0d, return_state=True)
    outs, gr = [y], [d['dy'].cuda()]
    if dsT:
        outs.append(sT)
        gr.append(th.from_numpy(dsTn).cuda())
    th.autograd.backward(outs, gr)
    yo, sTo = c_oracle.wkv7_fwd(*[cpu[n] for n in NAMES], s0=s0n)
    go = c_oracle.wkv7_bwd(*[cpu[n] for n in NAMES], cpu['dy'], s0=s0n, dsT=dsTn)
    check('y', y, yo, dtype)
    e = maxabs_rms(sT, sTo)
    assert e <= (1e-4 if dtype == th.float32 else 2e-2), f'sT: {e:.2e}'
    for n, gx in zip(NAMES, go[:6]):
        check('d' + n, dev[n].grad, gx, dtype)
    if s0:
        e = maxabs_rms(s0d.grad, go[6])
        assert e <= (1e-4 if dtype == th.float32 else 2e-2), f'ds0: {e:.2e}'
    assert _lib.device_status() == 0


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_config0_shape(dtype):
    """B1 T64 H2 N64, s0 = 0 (the reference's CPU-runnable configuration)."""
    run_case(1, 64, 2, dtype)


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_single_chunk(dtype):
    run_case(1, 16, 1, dtype, s0=True, dsT=True)


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_state_in_and_state_gradient(dtype):
    run_case(2, 256, 3, dtype, s0=True, dsT=True, seed=3)


@pytest.mark.parametrize('impl', [2, 3, -2, -3, -4])
def test_tcgen05_variants(impl):
    """The other builds of the tcgen05 forward: 2 and 3 preparation groups, and operands left for the tensor
    core to truncate (negative) instead of rounded to TF32 by their producer."""
    from wind_rwkv.rwkv7 import _lib
    old = _lib.set_fwd_impl(impl)
    try:
        run_case(2, 256, 3, th.bfloat16, s0=True, dsT=True, seed=4)
        run_case(1, 16, 1, th.bfloat16, seed=6)   # fewer chunks than groups
        run_case(1, 48, 2, th.bfloat16, s0=True, seed=7)
    finally:
        _lib.set_fwd_impl(old)


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_upstream_test_distribution(dtype):
    """Value distributions of tests/test_attn.py:25-30 at its check shape (B2 T1024 C64), 4 of 12 heads."""
    run_case(2, 1024, 4, dtype, dist='upstream', seed=5)


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
@pytest.mark.parametrize('T', [1000, 5, 17])
def test_sequence_length_not_a_multiple_of_16(T, dtype):
    """The reference asserts T % 16 == 0 (rwkv7_attn.py:22); here the last chunk may be partial.  Forward, final
    state and all gradients against the oracle; the output buffers are poisoned beyond nothing (they have exactly
    T rows), so a store past row T-1 would corrupt a neighbouring tensor and show up in its comparison."""
    run_case(2, T, 2, dtype, s0=True, dsT=True, seed=21)


def test_golden_config0(golden):
    """The committed output of upstream's own ref_attn on config 0 (fp32 inputs)."""
    _, _, attn, _, _ = _mods()
    g = golden('attn_cfg0.npz')
    dev = [th.from_numpy(g[n]).cuda().requires_grad_() for n in NAMES]
    y = attn(*dev, N)
    y.backward(th.from_numpy(g['dy']).cuda())
    assert maxabs_rms(y, g['y']) <= 1e-4
    for n, x in zip(NAMES, dev):
        assert maxabs_rms(x.grad, g['d' + n]) <= 1e-4, n


def _single_tf32_on_fp32_outputs(B, T, H, seed, dist, w=None):
    """Runs forward + backward of the WKV7_F32_TF32 class (fp32 tensors, single-TF32 products: the bf16 path's
    arithmetic without bf16 output rounding) through the C ABI and returns max-abs/RMS errors against the oracle."""
    c_oracle, _lib, _, synthetic, _ = _mods()
    d = synthetic.wkv7_inputs(B, T, H, N, seed=seed, dtype=th.bfloat16, dist=dist)  # bf16-representable values
    if w is not None:
        d['w'] = w.to(th.bfloat16)
    dev = {n: d[n].float().cuda().view(B, T, H, N).contiguous() for n in list(NAMES) + ['dy']}
    y = th.empty_like(dev['r'])
    sT = th.empty(B, H, N, N, device='cuda')
    L = _lib.lib()
    ck = th.empty(L.wkv7_checkpoint_bytes(B, T, H, N) // 4, device='cuda')
    st = (T * H * N, H * N, N)
    rc = L.wkv7_fwd(*[dev[n].data_ptr() for n in NAMES], None, y.data_ptr(), sT.data_ptr(), ck.data_ptr(),
                    B, T, H, N, *st, 2, None)
    assert rc == 0
    grads = [th.empty_like(y) for _ in range(6)]
    rc = L.wkv7_bwd(*[dev[n].data_ptr() for n in NAMES], dev['dy'].data_ptr(), ck.data_ptr(), None, None,
                    *[x.data_ptr() for x in grads], None, B, T, H, N, *st, 2, None)
    assert rc == 0
    th.cuda.synchronize()
    cpu = {n: dev[n].double().cpu().numpy() for n in dev}
    yo, sTo = c_oracle.wkv7_fwd(*[cpu[n] for n in NAMES])
    go = c_oracle.wkv7_bwd(*[cpu[n] for n in NAMES], cpu['dy'])
    errs = {'y': maxabs_rms(y, yo), 'sT': maxabs_rms(sT, sTo)}
    errs.update({'d' + n: maxabs_rms(x, ref) for n, x, ref in zip(NAMES, grads, go)})
    print({k: f'{v:.2e}' for k, v in errs.items()})
    assert _lib.device_status() == 0
    return errs


@pytest.mark.parametrize('dist', ['baseline', 'upstream'])
def test_bf16_arithmetic_on_fp32_outputs(dist, fwd_impl):
    """The bf16 path's arithmetic meets the stated 2e-2 bound on all eight tensors at T = 1024, both input
    distributions, when bf16 output rounding is taken out of the picture."""
    if fwd_impl == 0:
        pytest.skip('fp32 tensors always run the warp-MMA forward: one run is enough')
    errs = _single_tf32_on_fp32_outputs(2, 1024, 2, 9, dist)
    for k, v in errs.items():
        assert v <= 2e-2, f'{k}: {v:.2e}'


def test_strong_decay(fwd_impl):
    """Decays far stronger than the workload's.  Inside a chunk the kernels work with the running decay product and its
    reciprocal; they keep both inside fp32's range by a power-of-two shift of the product (exact) and a floor of -7.75
    on the per-step log-decay -exp(w).  (a) w ~ N(0.5, 1) cut at 2.0 (per-step decays down to e^-7.4, chunk products
    down to e^-110): no floor acts, normal tolerances except for dw, whose large cancelling terms leave it near 6e-2.
    (b) w ~ N(1, 1), uncut: 15 % of the steps are at the floor (they multiply the state by e^-7.75 = 4e-4 instead of
    less); the stated 2e-2 still holds for everything but dw.  RWKV-7 itself cannot produce either: w <= -0.5."""
    if fwd_impl == 0:
        pytest.skip('one run is enough')
    gen = th.Generator().manual_seed(13)
    B, T, H = 2, 256, 2
    w = (th.randn(B, T, H * N, generator=gen) + 0.5).clamp(max=2.0)
    errs = _single_tf32_on_fp32_outputs(B, T, H, 13, 'baseline', w=w)
    for k, v in errs.items():
        assert v <= (0.1 if k == 'dw' else 2e-2), f'{k}: {v:.2e}'
    w = th.randn(B, T, H * N, generator=gen) + 1.0
    errs = _single_tf32_on_fp32_outputs(B, T, H, 13, 'baseline', w=w)
    for k, v in errs.items():
        assert v <= (0.5 if k == 'dw' else 2e-2), f'{k}: {v:.2e}'
    # the same inputs through the bf16 kernels (tcgen05 forward) and the fp32 kernels
    c_oracle, _lib, attn, synthetic, _ = _mods()
    for dtype in (th.bfloat16, th.float32):
        d = synthetic.wkv7_inputs(B, T, H, N, seed=13, dtype=dtype, device='cuda')
        ins = [d[n].requires_grad_() for n in NAMES]
        ins[1] = w.to(dtype).cuda().requires_grad_()
        y, sT = attn(*ins, N, return_state=True)
        y.backward(d['dy'])
        assert bool(th.isfinite(y).all()) and all(bool(th.isfinite(x.grad).all()) for x in ins)
        yo, sTo = c_oracle.wkv7_fwd(*[x.detach().double().cpu().numpy().reshape(B, T, H, N) for x in ins])
        if dtype == th.bfloat16:
            check('y', y.view(B, T, H, N), yo, dtype)
            assert maxabs_rms(sT, sTo) <= 2e-2
        else:  # the floor's own effect: e^-7.75 of a channel's content per floored step
            assert maxabs_rms(y.view(B, T, H, N), yo) <= 5e-3 and maxabs_rms(sT, sTo) <= 5e-3   # measured 2e-3


def test_bounded_wait_gives_up_and_reports(fwd_impl):
    """A device-side wait that can never be satisfied runs out after its limit, raises the CTA's abort
    flag (later waits return at once), leaves WKV7_ERR_DEVICE_TIMEOUT in the status word and the
    context usable: the next forward runs and reports no error."""
    if fwd_impl == 0:
        pytest.skip('one run is enough')
    _, _lib, attn, synthetic, _ = _mods()
    limit = 400_000  # cycles, about 0.2 ms
    cyc = (ctypes.c_int64 * 4)()
    rc = _lib.lib().wkv7_selftest_bounded_wait(limit, cyc, None)
    assert rc == -9, rc                                # WKV7_ERR_DEVICE_TIMEOUT
    assert limit <= cyc[0] < 100 * limit and limit <= cyc[1] < 100 * limit, list(cyc)
    assert cyc[2] < limit and cyc[3] < limit, list(cyc)  # aborted CTA: no second wait
    assert _lib.device_status() == 0                   # the status word was cleared by the read
    d = synthetic.wkv7_inputs(1, 64, 2, N, seed=2, dtype=th.bfloat16, device='cuda')
    with th.no_grad():
        y = attn(*[d[n] for n in NAMES], N)
    assert th.isfinite(y.float()).all() and _lib.device_status() == 0


def test_split_sequence_is_bit_identical():
    """State carry: two calls over the halves of T reproduce one call bit for bit (same chunking)."""
    _, _, attn, synthetic, _ = _mods()
    B, T, H = 3, 512, 2
    d = synthetic.wkv7_inputs(B, T, H, N, seed=12, dtype=th.bfloat16, device='cuda')
    ins = [d[n] for n in NAMES]
    with th.no_grad():
        y, sT = attn(*ins, N, return_state=True)
        y1, s1 = attn(*[x[:, :256].contiguous() for x in ins], N, return_state=True)
        y2, s2 = attn(*[x[:, 256:].contiguous() for x in ins], N, s0=s1, return_state=True)
    assert th.equal(th.cat([y1, y2], 1), y) and th.equal(s2, sT)


def test_strided_head_shard_matches_contiguous():
    """A head-sharded view (stride_t = H_total*N) gives what the contiguous copy gives."""
    _, _, _, synthetic, WindRWKV7 = _mods()
    B, T, H = 2, 64, 4
    d = synthetic.wkv7_inputs(B, T, H, N, seed=13, dtype=th.bfloat16, device='cuda')
    full = [d[n].view(B, T, H, N) for n in 'wrkvab']
    with th.no_grad():
        y_view, sT_view, _ = WindRWKV7.apply(*[x[:, :, 1:3] for x in full], None)
        y_cont, sT_cont, _ = WindRWKV7.apply(*[x[:, :, 1:3].contiguous() for x in full], None)
    assert th.equal(y_view, y_cont) and th.equal(sT_view, sT_cont)


def test_strided_head_shard_backward_matches_contiguous():
    """Backward through head-sharded views: inputs and the gradient tensors all carry stride_t = H_total*N, which is
    what the tensor maps of the bulk output stores are encoded with."""
    _, _, attn, synthetic, _ = _mods()
    B, T, H = 2, 128, 4
    d = synthetic.wkv7_inputs(B, T, H, N, seed=17, dtype=th.bfloat16, device='cuda')
    hs = slice(N, 3 * N)   # heads 1..2 of 4

    def grads(make):
        ins = [make(d[n]).detach().requires_grad_() for n in 'rwkvab']
        y = attn(*ins, N)
        y.backward(make(d['dy']))
        return [y.detach()] + [x.grad for x in ins]

    g_cont = grads(lambda x: x[:, :, hs].contiguous())
    g_view = grads(lambda x: x[:, :, hs])
    for a, b in zip(g_view, g_cont):
        assert th.equal(a.contiguous(), b)


def test_empty_and_rejected_inputs():
    _, _, attn, _, _ = _mods()
    z = th.zeros(0, 16, N, dtype=th.bfloat16, device='cuda')
    assert attn(z, z, z, z, z, z, N).shape == (0, 16, N)
    z = th.zeros(2, 0, 2 * N, dtype=th.bfloat16, device='cuda')
    s0 = th.randn(2, 2, N, N, device='cuda')
    y, sT = attn(z, z, z, z, z, z, N, s0=s0, return_state=True)
    assert y.shape == (2, 0, 2 * N) and th.equal(sT, s0)
    bad = th.zeros(1, 16, 32, dtype=th.bfloat16, device='cuda')
    with pytest.raises(AssertionError):
        attn(bad, bad, bad, bad, bad, bad, 32)   # head size 32 is not built
    with pytest.raises(TypeError):
        h = th.zeros(1, 16, N, dtype=th.float16, device='cuda')
        attn(h, h, h, h, h, h, N)


def test_config1_full_size_properties():
    """B64 T1024 H12 bf16 (the benchmark shape): a 2-of-64 batch slice against the oracle, the
    whole batch against the slice-independent property that every chain is computed alone."""
    c_oracle, _lib, attn, synthetic, _ = _mods()
    B, T, H = 64, 1024, 12
    d = synthetic.wkv7_inputs(B, T, H, N, seed=1, dtype=th.bfloat16, device='cuda')
    dev = [d[n].requires_grad_() for n in NAMES]
    y = attn(*dev, N)
    y.backward(d['dy'])
    assert bool(th.isfinite(y).all()) and all(bool(th.isfinite(x.grad).all()) for x in dev)
    sl = slice(31, 33)
    sub = [d[n][sl].detach().clone().requires_grad_() for n in NAMES]
    ys = attn(*sub, N)
    ys.backward(d['dy'][sl])
    assert th.equal(ys, y[sl]) and all(th.equal(a.grad, b.grad[sl]) for a, b in zip(sub, dev))
    cpu = [d[n][sl].detach().double().cpu().numpy().reshape(2, T, H, N) for n in list(NAMES) + ['dy']]
    yo, _ = c_oracle.wkv7_fwd(*cpu[:6])
    go = c_oracle.wkv7_bwd(*cpu[:6], cpu[6])
    check('y', ys, yo, th.bfloat16)
    for n, x, ref in zip(NAMES, sub, go):
        check('d' + n, x.grad, ref, th.bfloat16)
    assert _lib.device_status() == 0


def test_config4_long_context_prefill():
    """The 2.9B prefill shape at its real batch: B8 T65536 H40, non-zero fp32 initial state, forward only, no
    checkpoints.  The whole batch for the chained property (two 32768-step calls reproduce one call bit for bit),
    batch entry 5, heads 0-3 for y and the final state against the oracle."""
    c_oracle, _lib, attn, synthetic, _ = _mods()
    B, T, H = 8, 65536, 40
    d = synthetic.wkv7_inputs(B, T, H, N, seed=4, dtype=th.bfloat16, device='cuda', s0_std=0.1)
    ins = [d[n] for n in NAMES]
    with th.no_grad():
        y, sT = attn(*ins, N, s0=d['s0'], return_state=True)
        y1, s1 = attn(*[x[:, :T // 2] for x in ins], N, s0=d['s0'], return_state=True)   # strided views, no copies
        assert th.equal(y1, y[:, :T // 2])
        del y1
        y2, s2 = attn(*[x[:, T // 2:] for x in ins], N, s0=s1, return_state=True)
    assert th.equal(y2, y[:, T // 2:]) and th.equal(s2, sT)
    del y2
    bsel, hs = 5, slice(0, 4 * N)  # four heads of one batch entry through the oracle
    cpu = [x[bsel:bsel + 1, :, hs].double().cpu().numpy().reshape(1, T, 4, N) for x in ins]
    yo, sTo = c_oracle.wkv7_fwd(*cpu, s0=d['s0'][bsel:bsel + 1, :4].double().cpu().numpy())
    check('y', y[bsel:bsel + 1, :, hs], yo, th.bfloat16)
    assert maxabs_rms(sT[bsel:bsel + 1, :4], sTo) <= 2e-2
    assert _lib.device_status() == 0


@pytest.mark.parametrize('nseg', [2, 8])
def test_time_split_forward(nseg):
    """attn(..., time_split=n): the sequence as n parallel segments joined by the affine form S_end = S_start M + R.
    y and the final state against the oracle with the usual bounds, and against the unsplit call (the two differ by the
    rounding of M, not bit for bit)."""
    c_oracle, _lib, attn, synthetic, _ = _mods()
    B, T, H = 1, 2048, 3
    d = synthetic.wkv7_inputs(B, T, H, N, seed=31, dtype=th.bfloat16, device='cuda', s0_std=0.1)
    ins = [d[n] for n in NAMES]
    with th.no_grad():
        y, sT = attn(*ins, N, s0=d['s0'], return_state=True, time_split=nseg)
        y1, sT1 = attn(*ins, N, s0=d['s0'], return_state=True)
    cpu = [x.double().cpu().numpy().reshape(B, T, H, N) for x in ins]
    yo, sTo = c_oracle.wkv7_fwd(*cpu, s0=d['s0'].double().cpu().numpy())
    check('y', y.view(B, T, H, N), yo, th.bfloat16)
    assert maxabs_rms(sT, sTo) <= 2e-2
    assert maxabs_rms(sT, sT1.double().cpu().numpy()) <= 2e-2
    # fp32 tensors: the split is exact to the fp32 path's tolerance
    d = synthetic.wkv7_inputs(B, 512, H, N, seed=32, dtype=th.float32, device='cuda')
    ins = [d[n] for n in NAMES]
    with th.no_grad():
        y, sT = attn(*ins, N, return_state=True, time_split=nseg)
    cpu = [x.double().cpu().numpy().reshape(B, 512, H, N) for x in ins]
    yo, sTo = c_oracle.wkv7_fwd(*cpu)
    assert maxabs_rms(y.view(B, 512, H, N), yo) <= 1e-4 and maxabs_rms(sT, sTo) <= 1e-4
    assert _lib.device_status() == 0


def test_tail_split_forward():
    """attn(..., time_split='tail'): the chains of the last, partly filled round of SMs are cut in time, the others run
    as usual, all into views of one output.  Against the unsplit call on every chain (they differ only on the split
    chains, by the rounding of M) and against the oracle on the last batch entry (which holds the split heads and,
    next to them, plainly run ones).  Without such a tail the call is the plain forward."""
    c_oracle, _lib, attn, synthetic, _ = _mods()
    from wind_rwkv.rwkv7.rwkv7_attn import tail_split_plan
    sms = th.cuda.get_device_properties(0).multi_processor_count
    H, T = 40, 8192                        # (the split only pays for long sequences: tail_split_plan declines T = 1024)
    B = sms // H + 1                       # one round of SMs and a few heads of the last batch entry
    plan = tail_split_plan(B, T, H, sms)
    assert plan is not None and plan[0] == B * H - sms
    d = synthetic.wkv7_inputs(B, T, H, N, seed=41, dtype=th.bfloat16, device='cuda', s0_std=0.1)
    ins = [d[n] for n in NAMES]
    with th.no_grad():
        y, sT = attn(*ins, N, s0=d['s0'], return_state=True, time_split='tail')
        y1, sT1 = attn(*ins, N, s0=d['s0'], return_state=True)
    th.cuda.synchronize()
    h0 = H - plan[0]
    y4, y14 = y.view(B, T, H, N), y1.view(B, T, H, N)
    assert th.equal(y4[:B - 1], y14[:B - 1]) and th.equal(y4[B - 1, :, :h0], y14[B - 1, :, :h0])   # plainly run chains: same kernel, same inputs
    assert th.equal(sT[:B - 1], sT1[:B - 1]) and th.equal(sT[B - 1, :h0], sT1[B - 1, :h0])
    hs = slice(h0 - 2, H)                  # two plainly run heads and the split ones
    cpu = [x.view(B, T, H, N)[B - 1:, :, hs].double().cpu().numpy() for x in ins]
    yo, sTo = c_oracle.wkv7_fwd(*cpu, s0=d['s0'][B - 1:, hs].double().cpu().numpy())
    check('y', y4[B - 1:, :, hs], yo, th.bfloat16)
    assert maxabs_rms(sT[B - 1:, hs], sTo) <= 2e-2
    assert maxabs_rms(sT[B - 1:, h0:], sT1[B - 1:, h0:].double().cpu().numpy()) <= 2e-2
    # no tail: plain forward, bit for bit
    d = synthetic.wkv7_inputs(2, 256, 3, N, seed=42, dtype=th.bfloat16, device='cuda')
    ins = [d[n] for n in NAMES]
    with th.no_grad():
        assert th.equal(attn(*ins, N, time_split='tail'), attn(*ins, N))
    assert _lib.device_status() == 0
