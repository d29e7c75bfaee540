/*
 * TEST INFRASTRUCTURE — not part of the shipped library.
 *
 * CPU restatement of the reference's naive WKV7 recurrence, included twice by
 * wkv7_oracle.c with REAL = float and REAL = double.  Only the test-suite, the
 * smoke check and the CPU-baseline leg of the benchmark may call it.
 *
 * Recurrence (reference: wind_rwkv/rwkv7/time_mixer.py:6-16 and the fp32
 * upcasting copy tests/test_attn.py:6-18), per (batch, head), S[i][j] with
 * i = value index, j = key index:
 *     wd_t = exp(-exp(w_t))
 *     S_t  = S_{t-1} * wd_t[None,:] + (S_{t-1} a_t) b_t^T + v_t k_t^T
 *     y_t  = S_t r_t
 * The reference hard-codes S_0 = 0 and drops S_T; here S_0 may be supplied and
 * S_T is returned (same loop body).
 *
 * attn_ln post-processing (reference: tests/test_attn_ln.py:17-20):
 *     y <- group_norm(y over the head's N channels, eps = 64e-5, affine)
 *     y <- y + (sum_j r_j k_j bonus_j) * v ;   y <- y * g
 *
 * Gradients are exact reverse-mode sweeps of the same loop (what autograd does
 * through the reference loop), with states re-materialised segment by segment.
 *
 * Tensor layout: r,w,k,v,a,b,g,y,dy : [B,T,H,N] contiguous; states [B,H,N,N];
 * params [3,H*N] = (ln_weight, ln_bias, bonus).
 */

#define CAT_(a, b) a##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

static void FN(step_fwd)(int N, REAL *S, const REAL *r, const REAL *w, const REAL *k, const REAL *v,
                         const REAL *a, const REAL *b, REAL *y, REAL *sa_out, REAL *wd_out) {
    REAL wd[MAXN], sa[MAXN];
    for (int j = 0; j < N; j++) wd[j] = (REAL)exp(-exp((double)w[j]));
    for (int i = 0; i < N; i++) {
        REAL *Si = S + (size_t)i * N;
        REAL acc = 0;
        for (int j = 0; j < N; j++) acc += Si[j] * a[j];
        sa[i] = acc;
    }
    for (int i = 0; i < N; i++) {
        REAL *Si = S + (size_t)i * N;
        REAL acc = 0, sai = sa[i], vi = v[i];
        for (int j = 0; j < N; j++) {
            REAL s = Si[j] * wd[j] + sai * b[j] + vi * k[j];
            Si[j] = s;
            acc += s * r[j];
        }
        if (y) y[i] = acc;
    }
    if (sa_out) for (int i = 0; i < N; i++) sa_out[i] = sa[i];
    if (wd_out) for (int j = 0; j < N; j++) wd_out[j] = wd[j];
}

/* Forward for all chains. s0/sT may be NULL. */
void FN(wkv7_oracle_fwd)(long B, long T, long H, int N, const REAL *r, const REAL *w, const REAL *k,
                         const REAL *v, const REAL *a, const REAL *b, const REAL *s0, REAL *y, REAL *sT) {
    long BH = B * H;
#pragma omp parallel for schedule(dynamic, 1)
    for (long bh = 0; bh < BH; bh++) {
        long bi = bh / H, hi = bh % H;
        REAL *S = (REAL *)malloc(sizeof(REAL) * N * N);
        if (s0) memcpy(S, s0 + (size_t)bh * N * N, sizeof(REAL) * N * N);
        else memset(S, 0, sizeof(REAL) * N * N);
        for (long t = 0; t < T; t++) {
            size_t off = (((size_t)bi * T + t) * H + hi) * N;
            FN(step_fwd)(N, S, r + off, w + off, k + off, v + off, a + off, b + off, y + off, NULL, NULL);
        }
        if (sT) memcpy(sT + (size_t)bh * N * N, S, sizeof(REAL) * N * N);
        free(S);
    }
}

/* Backward for all chains.  dsT/ds0 may be NULL. dy is the gradient of y. */
void FN(wkv7_oracle_bwd)(long B, long T, long H, int N, const REAL *r, const REAL *w, const REAL *k,
                         const REAL *v, const REAL *a, const REAL *b, const REAL *s0, const REAL *dy,
                         const REAL *dsT, REAL *dr, REAL *dw, REAL *dk, REAL *dv, REAL *da, REAL *db,
                         REAL *ds0) {
    long BH = B * H;
    const long SEG = 128;
    long nseg = (T + SEG - 1) / SEG;
    size_t NN = (size_t)N * N;
#pragma omp parallel for schedule(dynamic, 1)
    for (long bh = 0; bh < BH; bh++) {
        long bi = bh / H, hi = bh % H;
        REAL *seg0 = (REAL *)malloc(sizeof(REAL) * NN * (nseg + 1)); /* state at each segment start */
        REAL *hist = (REAL *)malloc(sizeof(REAL) * NN * (SEG + 1));  /* states inside one segment  */
        REAL *dS = (REAL *)malloc(sizeof(REAL) * NN);
        REAL *S = (REAL *)malloc(sizeof(REAL) * NN);
        if (s0) memcpy(S, s0 + (size_t)bh * NN, sizeof(REAL) * NN);
        else memset(S, 0, sizeof(REAL) * NN);
        for (long t = 0; t < T; t++) {
            if (t % SEG == 0) memcpy(seg0 + (t / SEG) * NN, S, sizeof(REAL) * NN);
            size_t off = (((size_t)bi * T + t) * H + hi) * N;
            FN(step_fwd)(N, S, r + off, w + off, k + off, v + off, a + off, b + off, NULL, NULL, NULL);
        }
        if (dsT) memcpy(dS, dsT + (size_t)bh * NN, sizeof(REAL) * NN);
        else memset(dS, 0, sizeof(REAL) * NN);
        for (long sg = nseg - 1; sg >= 0; sg--) {
            long t0 = sg * SEG, t1 = t0 + SEG < T ? t0 + SEG : T;
            memcpy(hist, seg0 + sg * NN, sizeof(REAL) * NN);
            for (long t = t0; t < t1; t++) {
                size_t off = (((size_t)bi * T + t) * H + hi) * N;
                REAL *nxt = hist + (t - t0 + 1) * NN;
                memcpy(nxt, hist + (t - t0) * NN, sizeof(REAL) * NN);
                FN(step_fwd)(N, nxt, r + off, w + off, k + off, v + off, a + off, b + off, NULL, NULL, NULL);
            }
            for (long t = t1 - 1; t >= t0; t--) {
                size_t off = (((size_t)bi * T + t) * H + hi) * N;
                const REAL *P = hist + (t - t0) * NN, *St = hist + (t - t0 + 1) * NN;
                const REAL *rt = r + off, *wt = w + off, *kt = k + off, *vt = v + off, *at = a + off,
                           *bt = b + off, *dyt = dy + off;
                REAL wd[MAXN], ew[MAXN], sa[MAXN], dsa[MAXN], acc_r[MAXN], acc_k[MAXN], acc_b[MAXN],
                    acc_w[MAXN], acc_a[MAXN];
                for (int j = 0; j < N; j++) {
                    ew[j] = (REAL)exp((double)wt[j]);
                    wd[j] = (REAL)exp(-(double)ew[j]);
                    acc_r[j] = acc_k[j] = acc_b[j] = acc_w[j] = acc_a[j] = 0;
                }
                for (int i = 0; i < N; i++) {
                    REAL s = 0;
                    for (int j = 0; j < N; j++) s += P[i * N + j] * at[j];
                    sa[i] = s;
                }
                for (int i = 0; i < N; i++) {
                    REAL *dSi = dS + (size_t)i * N;
                    const REAL *Sti = St + (size_t)i * N, *Pi = P + (size_t)i * N;
                    REAL dyi = dyt[i], vi = vt[i], sai = sa[i], dvi = 0, dsai = 0;
                    for (int j = 0; j < N; j++) {
                        REAL g = dSi[j] + dyi * rt[j]; /* total gradient wrt S_t[i][j] */
                        dSi[j] = g;
                        acc_r[j] += Sti[j] * dyi;
                        dvi += g * kt[j];
                        acc_k[j] += g * vi;
                        dsai += g * bt[j];
                        acc_b[j] += g * sai;
                        acc_w[j] += g * Pi[j];
                    }
                    dv[off + i] = dvi;
                    dsa[i] = dsai;
                }
                for (int i = 0; i < N; i++) {
                    REAL *dSi = dS + (size_t)i * N;
                    const REAL *Pi = P + (size_t)i * N;
                    REAL dsai = dsa[i];
                    for (int j = 0; j < N; j++) {
                        acc_a[j] += Pi[j] * dsai;
                        dSi[j] = dSi[j] * wd[j] + dsai * at[j]; /* gradient wrt S_{t-1} */
                    }
                }
                for (int j = 0; j < N; j++) {
                    dr[off + j] = acc_r[j];
                    dk[off + j] = acc_k[j];
                    db[off + j] = acc_b[j];
                    da[off + j] = acc_a[j];
                    dw[off + j] = acc_w[j] * wd[j] * (-ew[j]);
                }
            }
        }
        if (ds0) memcpy(ds0 + (size_t)bh * NN, dS, sizeof(REAL) * NN);
        free(seg0); free(hist); free(dS); free(S);
    }
}

/* attn_ln post-processing, forward: y (in place) from the recurrence output. */
void FN(attn_ln_post_fwd)(long B, long T, long H, int N, const REAL *r, const REAL *k, const REAL *v,
                          const REAL *g, const REAL *params, REAL eps, const REAL *y_in, REAL *out) {
    long HC = H * N, BT = B * T;
#pragma omp parallel for schedule(static)
    for (long bt = 0; bt < BT; bt++)
        for (long h = 0; h < H; h++) {
            size_t off = ((size_t)bt * H + h) * N;
            const REAL *lw = params + h * N, *lb = params + HC + h * N, *bo = params + 2 * HC + h * N;
            REAL mu = 0, var = 0, s = 0;
            for (int i = 0; i < N; i++) mu += y_in[off + i];
            mu /= N;
            for (int i = 0; i < N; i++) var += (y_in[off + i] - mu) * (y_in[off + i] - mu);
            var /= N;
            REAL rstd = (REAL)(1.0 / sqrt((double)(var + eps)));
            for (int j = 0; j < N; j++) s += r[off + j] * k[off + j] * bo[j];
            for (int i = 0; i < N; i++) {
                REAL z = (y_in[off + i] - mu) * rstd * lw[i] + lb[i] + s * v[off + i];
                out[off + i] = z * g[off + i];
            }
        }
}

/* attn_ln post-processing, backward.  Given dout, produces dy (gradient of the
 * recurrence output), dg, the bonus-term contributions ADDED into dr/dk/dv
 * (which must already hold zeros or the recurrence gradients) and dparams
 * [3,H*N] (accumulated; caller zero-fills). */
void FN(attn_ln_post_bwd)(long B, long T, long H, int N, const REAL *r, const REAL *k, const REAL *v,
                          const REAL *g, const REAL *params, REAL eps, const REAL *y_in, const REAL *dout,
                          REAL *dy, REAL *dg, REAL *dr_add, REAL *dk_add, REAL *dv_add, REAL *dparams) {
    long HC = H * N, BT = B * T;
    for (long bt = 0; bt < BT; bt++) /* serial: dparams accumulates in a fixed order */
        for (long h = 0; h < H; h++) {
            size_t off = ((size_t)bt * H + h) * N;
            const REAL *lw = params + h * N, *lb = params + HC + h * N, *bo = params + 2 * HC + h * N;
            REAL *dlw = dparams + h * N, *dlb = dparams + HC + h * N, *dbo = dparams + 2 * HC + h * N;
            REAL mu = 0, var = 0, s = 0, ds = 0, m1 = 0, m2 = 0;
            REAL xh[MAXN], dxh[MAXN];
            for (int i = 0; i < N; i++) mu += y_in[off + i];
            mu /= N;
            for (int i = 0; i < N; i++) var += (y_in[off + i] - mu) * (y_in[off + i] - mu);
            var /= N;
            REAL rstd = (REAL)(1.0 / sqrt((double)(var + eps)));
            for (int j = 0; j < N; j++) s += r[off + j] * k[off + j] * bo[j];
            for (int i = 0; i < N; i++) {
                xh[i] = (y_in[off + i] - mu) * rstd;
                REAL z = xh[i] * lw[i] + lb[i] + s * v[off + i];
                REAL dz = dout[off + i] * g[off + i];
                dg[off + i] = dout[off + i] * z;
                dlw[i] += dz * xh[i];
                dlb[i] += dz;
                ds += dz * v[off + i];
                dv_add[off + i] += dz * s;
                dxh[i] = dz * lw[i];
                m1 += dxh[i];
                m2 += dxh[i] * xh[i];
            }
            m1 /= N; m2 /= N;
            for (int i = 0; i < N; i++) dy[off + i] = rstd * (dxh[i] - m1 - xh[i] * m2);
            for (int j = 0; j < N; j++) {
                dr_add[off + j] += ds * k[off + j] * bo[j];
                dk_add[off + j] += ds * r[off + j] * bo[j];
                dbo[j] += ds * r[off + j] * k[off + j];
            }
        }
}

#undef FN
#undef CAT
#undef CAT_
