"""The chunked formulation the CUDA kernels implement, written out in float64 torch and checked
against autograd through the naive recurrence (the oracle).  This pins the algebra — including
the decay gradient obtained from the running log-decay and the carried chunk-boundary term —
independently of any GPU."""
import torch as th

import wkv7_ref

dt = th.float64


def chunk_fwd(q, w, k, v, a, b, S0):
    Lc = q.shape[0]
    lw = -th.exp(w)
    c = th.cumsum(lw, 0)
    incl, inv, non, fw = th.exp(c), th.exp(-c), th.exp(c - lw), th.exp(c[-1])
    wq, wa, kwi, bwi = q * incl, a * non, k * inv, b * inv
    QK, QB = th.tril(wq @ kwi.T), th.tril(wq @ bwi.T)
    AK, AB = th.tril(wa @ kwi.T, -1), th.tril(wa @ bwi.T, -1)
    AI = th.linalg.inv(th.eye(Lc, dtype=dt) - AB)
    U = AI @ (AK @ v + wa @ S0.T)
    Y = QK @ v + QB @ U + wq @ S0.T
    S1 = (S0 + v.T @ kwi + U.T @ bwi) * fw[None, :]
    return Y, S1, dict(lw=lw, incl=incl, inv=inv, non=non, fw=fw, wq=wq, wa=wa, kwi=kwi, bwi=bwi,
                       QK=QK, QB=QB, AK=AK, AB=AB, AI=AI, U=U)


def chunk_bwd(q, w, k, v, a, b, S0, dY, dS, G):
    _, _, m = chunk_fwd(q, w, k, v, a, b, S0)
    wq, wa, kwi, bwi, U = m['wq'], m['wa'], m['kwi'], m['bwi'], m['U']
    dSf = dS * m['fw'][None, :]
    du = m['QB'].T @ dY + bwi @ dSf.T
    dabu = m['AI'].T @ du
    dV = m['QK'].T @ dY + kwi @ dSf.T + m['AK'].T @ dabu
    dAB, dAK = th.tril(dabu @ U.T, -1), th.tril(dabu @ v.T, -1)
    dQB, dQK = th.tril(dY @ U.T), th.tril(dY @ v.T)
    DA = dAB @ bwi + dAK @ kwi + dabu @ S0
    DQ = dQB @ bwi + dQK @ kwi + dY @ S0
    DB = dAB.T @ wa + dQB.T @ wq + U @ dSf
    DK = dAK.T @ wa + dQK.T @ wq + v @ dSf
    dS0 = dSf + dY.T @ wq + dabu.T @ wa
    e2 = wa * DA
    x = wq * DQ - kwi * DK - bwi * DB + e2
    sfx = th.flip(th.cumsum(th.flip(x, [0]), 0), [0])
    dw = (sfx - e2 + G[None, :]) * m['lw']
    return dw, m['incl'] * DQ, m['inv'] * DK, dV, m['non'] * DA, m['inv'] * DB, dS0, (dS0 * S0).sum(0)


def test_chunked_forward_backward_equals_autograd_of_the_recurrence():
    from wind_rwkv.rwkv7 import synthetic
    T, N, Lc = 96, 64, 16
    d = synthetic.wkv7_inputs(1, T, 1, N, seed=4, dtype=dt, s0_std=0.1)
    ins = [d[n][0].double().requires_grad_() for n in 'rwkvab']
    s0 = d['s0'][0, 0].double().requires_grad_()
    y, sT = wkv7_ref.ref_attn(*[x[None] for x in ins], N, s0=s0[None, None], return_state=True, compute_dtype=dt)
    th.manual_seed(0)
    dy, dsT = th.randn(T, N, dtype=dt), th.randn(N, N, dtype=dt)
    th.autograd.backward([y[0], sT[0, 0]], [dy, dsT])
    r, w, k, v, a, b = [x.detach() for x in ins]
    S, cks, ys = s0.detach(), [], []
    for c in range(T // Lc):
        sl = slice(c * Lc, (c + 1) * Lc)
        cks.append(S)
        Y, S, _ = chunk_fwd(r[sl], w[sl], k[sl], v[sl], a[sl], b[sl], S)
        ys.append(Y)
    assert (th.cat(ys) - y[0]).abs().max() < 1e-11 and (S - sT[0, 0]).abs().max() < 1e-11
    dS, G = dsT.clone(), (dsT * S).sum(0)
    out = {n: [] for n in 'wqkvab'}
    for c in reversed(range(T // Lc)):
        sl = slice(c * Lc, (c + 1) * Lc)
        *gr, dS, G = chunk_bwd(r[sl], w[sl], k[sl], v[sl], a[sl], b[sl], cks[c], dy[sl], dS, G)
        for n, x in zip('wqkvab', gr):
            out[n].insert(0, x)
    for n, ref in zip('qwkvab', ins):
        got = th.cat(out[n])
        assert (got - ref.grad).abs().max() <= 1e-10 * ref.grad.abs().max().clamp(min=1), n
    assert (dS - s0.grad).abs().max() < 1e-11
