"""wkv7_step (decode): the recurrence one time step at a time, sharing the fp32 state format of wkv7_fwd.
Checked against the oracle (the reference's naive recurrence, time_mixer.py:13-15, with s0 in / sT out)
and against the chunked forward."""
import numpy as np
import pytest
import torch as th

from test_attn_gpu import N, NAMES, check, maxabs_rms

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, dtype, seed):
    from wind_rwkv.rwkv7 import synthetic
    return synthetic.wkv7_inputs(B, T, H, N, seed=seed, dtype=dtype, device='cuda', s0_std=0.1)


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
@pytest.mark.parametrize('T', [1, 3, 15])
def test_short_calls_against_the_oracle(T, dtype):
    import c_oracle
    from wind_rwkv.rwkv7 import attn_step
    B, H = 3, 5
    d = _inputs(B, T, H, dtype, seed=30 + T)
    y, sT = attn_step(*[d[n] for n in NAMES], N, d['s0'])
    cpu = [d[n].double().cpu().numpy().reshape(B, T, H, N) for n in NAMES]
    yo, sTo = c_oracle.wkv7_fwd(*cpu, s0=d['s0'].double().cpu().numpy())
    check('y', y.view(B, T, H, N), yo, dtype)
    assert maxabs_rms(sT, sTo) <= 1e-5   # fp32 arithmetic for every tensor dtype


@pytest.mark.parametrize('dtype', [th.float32, th.bfloat16])
def test_64_single_steps_equal_one_chunked_call(dtype):
    """Prefill + decode consistency: 64 chained T = 1 calls (state updated in place) against one T = 64 call of
    the chunked forward.  fp32 tensors: both are exact to about 1e-5 of RMS; bf16 tensors: the chunked kernel
    uses single-TF32 products, so y agrees to bf16 rounding and the fp32 state to 2e-2 of RMS."""
    from wind_rwkv.rwkv7 import attn, attn_step
    B, T, H = 2, 64, 3
    d = _inputs(B, T, H, dtype, seed=41)
    ins = [d[n] for n in NAMES]
    with th.no_grad():
        y_ref, sT_ref = attn(*ins, N, s0=d['s0'], return_state=True)
    state = d['s0'].clone()
    ys = []
    for t in range(T):
        y, s = attn_step(*[x[:, t:t + 1] for x in ins], N, state, inplace=True)
        assert s.data_ptr() == state.data_ptr()
        ys.append(y)
    y = th.cat(ys, 1)
    tol_state = 1e-4 if dtype == th.float32 else 2e-2
    assert maxabs_rms(state, sT_ref.double().cpu().numpy()) <= tol_state
    if dtype == th.float32:
        assert maxabs_rms(y, y_ref.double().cpu().numpy()) <= 1e-4
    else:
        # two correctly rounded bf16 results of nearly equal fp32 values differ by at most one bf16 ulp
        ulp = th.maximum(y_ref.float().abs(), th.tensor(1e-30, device='cuda')) * 2 ** -7
        assert bool(((y.float() - y_ref.float()).abs() <= ulp + 2e-2 * y_ref.float().pow(2).mean().sqrt()).all())


def test_one_call_of_T_steps_equals_T_calls_bit_for_bit():
    from wind_rwkv.rwkv7 import attn_step
    B, T, H = 2, 7, 2
    d = _inputs(B, T, H, th.bfloat16, seed=43)
    ins = [d[n] for n in NAMES]
    y_all, s_all = attn_step(*ins, N, d['s0'])
    state, ys = d['s0'], []
    for t in range(T):
        y, state = attn_step(*[x[:, t:t + 1] for x in ins], N, state)
        ys.append(y)
    assert th.equal(th.cat(ys, 1), y_all) and th.equal(state, s_all)


def test_zero_state_and_empty_sequence():
    from wind_rwkv.rwkv7 import attn, attn_step
    d = _inputs(1, 2, 1, th.float32, seed=44)
    ins = [d[n] for n in NAMES]
    y, s = attn_step(*ins, N)            # state None = zeros
    y0, s0 = attn_step(*ins, N, th.zeros(1, 1, N, N, device='cuda'))
    assert th.equal(y, y0) and th.equal(s, s0)
    e = [x[:, :0] for x in ins]
    y, s = attn_step(*e, N, d['s0'])
    assert y.shape == (1, 0, N) and th.equal(s, d['s0'])
