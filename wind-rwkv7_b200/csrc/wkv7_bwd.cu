// WKV7 backward for sm_100a: one CTA per (batch, head) chain, 4 warps, chunks of 16 time steps
// walked in reverse; the gradient dS of the state stays in registers across chunks.
//
// Replaces the reference's backward_kernel (wind_rwkv/rwkv7/attn.cu:131-326).  The forward
// intermediates of a chunk are rebuilt from the fp32 chunk-start state S0 the forward wrote.
// With the forward's notation (wq, wa, kwi, bwi, fw, QK, QB, AK, AB, AI = (I-AB)^-1, U) and
// dSf = dS * fw[None,:]:
//     du   = QB^T dY + bwi dSf^T          dabu = AI^T du
//     dV   = QK^T dY + kwi dSf^T + AK^T dabu
//     dAB = stril(dabu U^T)  dAK = stril(dabu V^T)  dQB = tril(dY U^T)  dQK = tril(dY V^T)
//     DA = dAB bwi + dAK kwi + dabu S0     DQ = dQB bwi + dQK kwi + dY S0
//     DB = dAB^T wa + dQB^T wq + U dSf     DK = dAK^T wa + dQK^T wq + V dSf
//     da = P_{t-1} DA   dq = P_t DQ   db = DB / P_t   dk = DK / P_t
//     dS0 = dSf + dY^T wq + dabu^T wa
// The decay gradient uses that w enters only through the running log-decay c_t = sum_{s<=t}
// -exp(w_s): every scaled operand is (input * exp(+-c)), so
//     d/dc_t = wq.DQ - kwi.DK - bwi.DB (row t) + wa.DA (row t+1),   d/dc_L += sum_i dS[i,:] S'[i,:]
// and dlogdecay_k = sum_{t>=k} d/dc_t; dw = dlogdecay * (-exp(w)).  The last term for chunk c-1
// equals sum_i dS0_c[i,:] S0_c[i,:], which is formed while chunk c is processed and carried.
//
// Stage B (rows = value index, per warp, no cross-warp traffic): U^T, du^T, dabu^T, dV^T, dS0.
// Stage C (contractions over the value index, warp owns 16 key columns): the four score
// gradients and DA, DQ, DB, DK with S0 and dSf read from shared memory.
#include "wkv7_kernels.h"

namespace wkv7 {

constexpr int SS = N + 4;  // row stride (floats) of the [value][key] state buffers

template <typename IoT> struct BwdLayout {
    static constexpr int ROWB = N * (int)sizeof(IoT) + 16;
    static constexpr int TILEB = L * ROWB;
    static constexpr int YS = (sizeof(IoT) == 2) ? 24 : 20;
};

template <typename IoT> struct BwdSmem {
    using Lay = BwdLayout<IoT>;
    alignas(16) unsigned char st_in[5][Lay::TILEB];  // q, w, k, a, b (dead after the scan)
    alignas(16) unsigned char st_v[2][Lay::TILEB];
    alignas(16) unsigned char st_dy[2][Lay::TILEB];
    alignas(16) float wq[L * OPS], wa[L * OPS], kwi[L * OPS], bwi[L * OPS];
    alignas(16) float cum[L * OPS], lw[L * OPS];
    alignas(16) float QK[L * SCS], QB[L * SCS], AK[L * SCS], AB[L * SCS], AI[L * SCS];
    alignas(16) float dQK[L * SCS], dQB[L * SCS], dAK[L * SCS], dAB[L * SCS];
    alignas(16) float Ut[L * OPS], Dt[L * OPS];  // U and dabu as [time][value]
    alignas(16) float S0s[N * SS], dSs[N * SS];  // chunk-start state and dSf as [value][key]
    alignas(16) float fw[N];
    alignas(16) float Gp[2][WARPS][N];
    alignas(16) IoT dvsc[WARPS][L * Lay::YS];
    alignas(8) uint64_t bar_in, bar_vdy[2], bar_s0;
};

template <typename IoT> __device__ __forceinline__ float bst_elem(const unsigned char* tile, int row, int col) {
    return to_f32<IoT>(*reinterpret_cast<const IoT*>(tile + row * BwdLayout<IoT>::ROWB + col * (int)sizeof(IoT)));
}
// two adjacent elements (col even) of a staging tile
template <typename IoT> __device__ __forceinline__ float2 bst_pair(const unsigned char* tile, int row, int col);
template <> __device__ __forceinline__ float2 bst_pair<float>(const unsigned char* tile, int row, int col) {
    return *reinterpret_cast<const float2*>(tile + row * BwdLayout<float>::ROWB + col * 4);
}
template <> __device__ __forceinline__ float2 bst_pair<__nv_bfloat16>(const unsigned char* tile, int row, int col) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(tile + row * BwdLayout<__nv_bfloat16>::ROWB + col * 2));
}
// A operand [m = time][k = value] straight from a staging tile laid out [time][value]
template <typename IoT, int PREC>
__device__ __forceinline__ FragA<PREC> fragA_mk_st(const unsigned char* tile, int k0, int g, int t4) {
    FragA<PREC> f;
    float2 lo = bst_pair<IoT>(tile, g, k0 + 2 * t4), hi = bst_pair<IoT>(tile, g + 8, k0 + 2 * t4);
    f.x[0].set(lo.x); f.x[1].set(hi.x); f.x[2].set(lo.y); f.x[3].set(hi.y);
    return f;
}
// B operand [k = value][n = time] from a staging tile laid out [time][value]
template <typename IoT, int PREC>
__device__ __forceinline__ FragB<PREC> fragB_nk_st(const unsigned char* tile, int n0, int k0, int g, int t4) {
    FragB<PREC> f;
    float2 v = bst_pair<IoT>(tile, n0 + g, k0 + 2 * t4);
    f.x[0].set(v.x); f.x[1].set(v.y);
    return f;
}
// A operand [m = value][k = time] (the transpose) from a staging tile laid out [time][value]
template <typename IoT, int PREC>
__device__ __forceinline__ FragA<PREC> fragA_km_st(const unsigned char* tile, int m0, int k0, int g, int t4) {
    FragA<PREC> f;
    const int tr = k0 + 2 * t4, vc = m0 + g;
    f.x[0].set(bst_elem<IoT>(tile, tr, vc));
    f.x[1].set(bst_elem<IoT>(tile, tr, vc + 8));
    f.x[2].set(bst_elem<IoT>(tile, tr + 1, vc));
    f.x[3].set(bst_elem<IoT>(tile, tr + 1, vc + 8));
    return f;
}

template <typename IoT> __device__ __forceinline__ void store_pair(IoT* p, float x, float y);
template <> __device__ __forceinline__ void store_pair<float>(float* p, float x, float y) {
    *reinterpret_cast<float2*>(p) = make_float2(x, y);
}
template <> __device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* p, float x, float y) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
}

template <typename IoT, int PREC>
__global__ void __launch_bounds__(THREADS) wkv7_bwd_kernel(BwdParams p) {
    using Lay = BwdLayout<IoT>;
    using Smem = BwdSmem<IoT>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const long long bh = blockIdx.x;
    const long long bi = bh / p.H, hi = bh % p.H;
    const long long base = bi * p.st.b + hi * p.st.h;
    const int nchunks = (int)(p.T / L);
    const IoT* gin[5] = {(const IoT*)p.r + base, (const IoT*)p.w + base, (const IoT*)p.k + base,
                         (const IoT*)p.a + base, (const IoT*)p.b + base};
    const IoT* gv = (const IoT*)p.v + base;
    const IoT* gdy = (const IoT*)p.dy + base;
    IoT* gout[5] = {(IoT*)p.dr + base, (IoT*)p.dw + base, (IoT*)p.dk + base, (IoT*)p.da + base, (IoT*)p.db + base};
    IoT* gdv = (IoT*)p.dv + base;
    const float* ckpt = p.ckpt + bh * nchunks * (long long)(N * N);
    constexpr uint32_t ROW_BYTES = N * sizeof(IoT);

    if (tid == 0) {
        mbar_init(&sm.bar_in, 1);
        mbar_init(&sm.bar_vdy[0], 1);
        mbar_init(&sm.bar_vdy[1], 1);
        mbar_init(&sm.bar_s0, 1);
        mbar_fence_init();
    }
    // Carried decay term for the last chunk: sum_i dsT[i,:] * sT[i,:] (zero without dsT).
    for (int i = tid; i < WARPS * N; i += THREADS) sm.Gp[1][i / N][i % N] = 0.f;
    __syncthreads();
    if (p.dsT && p.sT && tid < N) {
        const float* d = p.dsT + bh * N * N;
        const float* s = p.sT + bh * N * N;
        float acc = 0.f;
        for (int i = 0; i < N; ++i) acc += d[i * N + tid] * s[i * N + tid];
        sm.Gp[1][0][tid] = acc;
    }

    // iteration `it` handles chunk c = nchunks-1-it
    auto issue_in = [&](int c) {
        if (lane == 0) mbar_arrive_expect_tx(&sm.bar_in, 5 * L * ROW_BYTES);
        __syncwarp();
        for (int i = lane; i < 5 * L; i += 32) {
            int ten = i / L, row = i % L;
            bulk_g2s(sm.st_in[ten] + row * Lay::ROWB, gin[ten] + ((long long)c * L + row) * p.st.t, ROW_BYTES, &sm.bar_in);
        }
    };
    auto issue_vdy = [&](int c, int s) {
        if (lane == 0) mbar_arrive_expect_tx(&sm.bar_vdy[s], 2 * L * ROW_BYTES);
        __syncwarp();
        {
            int ten = lane / L, row = lane % L;
            const IoT* src = (ten == 0 ? gv : gdy) + ((long long)c * L + row) * p.st.t;
            unsigned char* dst = (ten == 0 ? sm.st_v[s] : sm.st_dy[s]) + row * Lay::ROWB;
            bulk_g2s(dst, src, ROW_BYTES, &sm.bar_vdy[s]);
        }
    };
    auto issue_s0 = [&](int c) {
        if (lane == 0) mbar_arrive_expect_tx(&sm.bar_s0, N * N * 4);
        __syncwarp();
        for (int i = lane; i < N; i += 32) bulk_g2s(sm.S0s + i * SS, ckpt + (long long)c * N * N + i * N, N * 4, &sm.bar_s0);
    };
    if (warp == 0 && nchunks > 0) {
        issue_in(nchunks - 1);
        issue_vdy(nchunks - 1, 0);
        issue_s0(nchunks - 1);
    }

    // dS: warp owns value rows 16*warp + {g, g+8}; tile nt covers key columns 8nt..8nt+7.
    float dS[8][4];
    {
        const float* d = p.dsT ? p.dsT + bh * N * N : nullptr;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            if (d) {
                float2 lo = *reinterpret_cast<const float2*>(d + (16 * warp + g) * N + 8 * nt + 2 * t4);
                float2 hi2 = *reinterpret_cast<const float2*>(d + (16 * warp + g + 8) * N + 8 * nt + 2 * t4);
                dS[nt][0] = lo.x; dS[nt][1] = lo.y; dS[nt][2] = hi2.x; dS[nt][3] = hi2.y;
            } else {
                dS[nt][0] = dS[nt][1] = dS[nt][2] = dS[nt][3] = 0.f;
            }
        }
    }

    bool failed = false;
    for (int it = 0; it < nchunks; ++it) {
        const int c = nchunks - 1 - it;
        const int vs = it & 1;
        // ---------------- P1: decay scan and scaled operands -------------------------------------
        bool ok = mbar_wait(&sm.bar_in, it & 1);
        {
            const int j = tid & 63, half = tid >> 6;
            float cum = 0.f;
            if (half)
#pragma unroll
                for (int r = 0; r < 8; ++r) cum -= exp_p<PREC>(bst_elem<IoT>(sm.st_in[1], r, j));
            float prev = half ? exp_p<PREC>(cum) : 1.f;
#pragma unroll
            for (int r8 = 0; r8 < 8; ++r8) {
                const int r = half * 8 + r8;
                const float lw = -exp_p<PREC>(bst_elem<IoT>(sm.st_in[1], r, j));
                cum += lw;
                const float incl = exp_p<PREC>(cum), inv = exp_p<PREC>(-cum);
                sm.wq[r * OPS + j] = bst_elem<IoT>(sm.st_in[0], r, j) * incl;
                sm.wa[r * OPS + j] = bst_elem<IoT>(sm.st_in[3], r, j) * prev;
                sm.kwi[r * OPS + j] = bst_elem<IoT>(sm.st_in[2], r, j) * inv;
                sm.bwi[r * OPS + j] = bst_elem<IoT>(sm.st_in[4], r, j) * inv;
                sm.cum[r * OPS + j] = cum;
                sm.lw[r * OPS + j] = lw;
                prev = incl;
            }
            if (half) sm.fw[j] = prev;
        }
        if (__syncthreads_or(!ok)) { failed = true; break; }  // (A)

        if (warp == 0 && c > 0) {
            issue_in(c - 1);
            issue_vdy(c - 1, vs ^ 1);
        }

        // ---------------- P2: masked score matrices, one per warp ------------------------------
        {
            const float* Am = (warp & 1) ? sm.wa : sm.wq;
            const float* Bm = (warp >> 1) ? sm.bwi : sm.kwi;
            float* dst = warp == 0 ? sm.QK : warp == 1 ? sm.AK : warp == 2 ? sm.QB : sm.AB;
            const bool strict = warp & 1;
            float d[2][4] = {};
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                FragA<PREC> a = fragA_mk<PREC>(Am, OPS, 0, 8 * kk, g, t4);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) mma<PREC>(d[nt], a, fragB_nk<PREC>(Bm, OPS, 8 * nt, 8 * kk, g, t4));
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int s = 8 * nt + 2 * t4;
                auto keep = [&](int tq, int ss) { return strict ? ss < tq : ss <= tq; };
                *reinterpret_cast<float2*>(dst + g * SCS + s) =
                    make_float2(keep(g, s) ? d[nt][0] : 0.f, keep(g, s + 1) ? d[nt][1] : 0.f);
                *reinterpret_cast<float2*>(dst + (g + 8) * SCS + s) =
                    make_float2(keep(g + 8, s) ? d[nt][2] : 0.f, keep(g + 8, s + 1) ? d[nt][3] : 0.f);
            }
        }
        if (warp == 3) {  // AI = (I - AB)^-1
            __syncwarp();
            if (lane < L) {
                float m[L];
#pragma unroll
                for (int tq = 0; tq < L; ++tq) {
                    float acc = (tq == lane) ? 1.f : 0.f;
#pragma unroll
                    for (int s = 0; s < tq; ++s) acc = fmaf(sm.AB[tq * SCS + s], m[s], acc);
                    m[tq] = acc;
                    sm.AI[tq * SCS + lane] = acc;
                }
            }
        }

        bool ok2 = mbar_wait(&sm.bar_s0, it & 1);
        ok2 = mbar_wait(&sm.bar_vdy[vs], (it >> 1) & 1) && ok2;
        if (__syncthreads_or(!ok2)) { failed = true; break; }  // (B)

        // ---------------- stage B: rows = value index -----------------------------------------
        const unsigned char* vt = sm.st_v[vs];
        const unsigned char* dyt = sm.st_dy[vs];
        FragA<PREC> vf[2], dyf[2];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            vf[kk] = fragA_km_st<IoT, PREC>(vt, 16 * warp, 8 * kk, g, t4);
            dyf[kk] = fragA_km_st<IoT, PREC>(dyt, 16 * warp, 8 * kk, g, t4);
        }
        float U[2][4] = {};
        {
            float X[2][4] = {};
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                FragA<PREC> a = fragA_mk<PREC>(sm.S0s, SS, 16 * warp, 8 * kk, g, t4);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) mma<PREC>(X[nt], a, fragB_nk<PREC>(sm.wa, OPS, 8 * nt, 8 * kk, g, t4));
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int kk = 0; kk <= nt; ++kk) mma<PREC>(X[nt], vf[kk], fragB_nk<PREC>(sm.AK, SCS, 8 * nt, 8 * kk, g, t4));
            FragA<PREC> xa[2] = {fragA_from_acc<PREC>(X[0]), fragA_from_acc<PREC>(X[1])};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int kk = 0; kk <= nt; ++kk) mma<PREC>(U[nt], xa[kk], fragB_nk<PREC>(sm.AI, SCS, 8 * nt, 8 * kk, g, t4));
        }
        // dS <- dSf = dS * fw
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            const float2 f = *reinterpret_cast<const float2*>(sm.fw + 8 * nt + 2 * t4);
            dS[nt][0] *= f.x; dS[nt][1] *= f.y; dS[nt][2] *= f.x; dS[nt][3] *= f.y;
        }
        float du[2][4] = {}, dV[2][4] = {};
#pragma unroll
        for (int sb = 0; sb < 2; ++sb)
#pragma unroll
            for (int tb = sb; tb < 2; ++tb) {
                mma<PREC>(du[sb], dyf[tb], fragB_kn<PREC>(sm.QB, SCS, 8 * sb, 8 * tb, g, t4));
                mma<PREC>(dV[sb], dyf[tb], fragB_kn<PREC>(sm.QK, SCS, 8 * sb, 8 * tb, g, t4));
            }
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            FragA<PREC> a = fragA_from_acc<PREC>(dS[kk]);
#pragma unroll
            for (int sb = 0; sb < 2; ++sb) {
                mma<PREC>(du[sb], a, fragB_nk<PREC>(sm.bwi, OPS, 8 * sb, 8 * kk, g, t4));
                mma<PREC>(dV[sb], a, fragB_nk<PREC>(sm.kwi, OPS, 8 * sb, 8 * kk, g, t4));
            }
        }
        float dabu[2][4] = {};
        {
            FragA<PREC> da2[2] = {fragA_from_acc<PREC>(du[0]), fragA_from_acc<PREC>(du[1])};
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                for (int kb = nb; kb < 2; ++kb) mma<PREC>(dabu[nb], da2[kb], fragB_kn<PREC>(sm.AI, SCS, 8 * nb, 8 * kb, g, t4));
        }
        FragA<PREC> dbf[2] = {fragA_from_acc<PREC>(dabu[0]), fragA_from_acc<PREC>(dabu[1])};
#pragma unroll
        for (int sb = 0; sb < 2; ++sb)
#pragma unroll
            for (int tb = sb; tb < 2; ++tb) mma<PREC>(dV[sb], dbf[tb], fragB_kn<PREC>(sm.AK, SCS, 8 * sb, 8 * tb, g, t4));

        // dv out (transposed through a per-warp scratch tile for 16-byte stores)
        {
            IoT* sc = sm.dvsc[warp];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int tq = 8 * nt + 2 * t4;
                sc[tq * Lay::YS + g] = from_f32<IoT>(dV[nt][0]);
                sc[(tq + 1) * Lay::YS + g] = from_f32<IoT>(dV[nt][1]);
                sc[tq * Lay::YS + g + 8] = from_f32<IoT>(dV[nt][2]);
                sc[(tq + 1) * Lay::YS + g + 8] = from_f32<IoT>(dV[nt][3]);
            }
            __syncwarp();
            const int row = lane >> 1, hf = lane & 1;
            const uint4* src = reinterpret_cast<const uint4*>(sc + row * Lay::YS + 8 * hf);
            uint4* dst = reinterpret_cast<uint4*>(gdv + ((long long)c * L + row) * p.st.t + 16 * warp + 8 * hf);
            dst[0] = src[0];
            if (sizeof(IoT) == 4) dst[1] = src[1];
        }
        // dSf, U, dabu to shared memory for stage C
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(sm.dSs + (16 * warp + g) * SS + 8 * nt + 2 * t4) = make_float2(dS[nt][0], dS[nt][1]);
            *reinterpret_cast<float2*>(sm.dSs + (16 * warp + g + 8) * SS + 8 * nt + 2 * t4) = make_float2(dS[nt][2], dS[nt][3]);
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int tq = 8 * nt + 2 * t4, vc = 16 * warp + g;
            sm.Ut[tq * OPS + vc] = U[nt][0]; sm.Ut[(tq + 1) * OPS + vc] = U[nt][1];
            sm.Ut[tq * OPS + vc + 8] = U[nt][2]; sm.Ut[(tq + 1) * OPS + vc + 8] = U[nt][3];
            sm.Dt[tq * OPS + vc] = dabu[nt][0]; sm.Dt[(tq + 1) * OPS + vc] = dabu[nt][1];
            sm.Dt[tq * OPS + vc + 8] = dabu[nt][2]; sm.Dt[(tq + 1) * OPS + vc + 8] = dabu[nt][3];
        }
        // dS0 = dSf + dY^T wq + dabu^T wa ; carried decay term sum_i dS0[i,:] S0[i,:]
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                mma<PREC>(dS[nt], dyf[kk], fragB_kn<PREC>(sm.wq, OPS, 8 * nt, 8 * kk, g, t4));
                mma<PREC>(dS[nt], dbf[kk], fragB_kn<PREC>(sm.wa, OPS, 8 * nt, 8 * kk, g, t4));
            }
            const float2 lo = *reinterpret_cast<const float2*>(sm.S0s + (16 * warp + g) * SS + 8 * nt + 2 * t4);
            const float2 hi2 = *reinterpret_cast<const float2*>(sm.S0s + (16 * warp + g + 8) * SS + 8 * nt + 2 * t4);
            float gx = dS[nt][0] * lo.x + dS[nt][2] * hi2.x, gy2 = dS[nt][1] * lo.y + dS[nt][3] * hi2.y;
#pragma unroll
            for (int m = 4; m <= 16; m <<= 1) {
                gx += __shfl_xor_sync(0xffffffffu, gx, m);
                gy2 += __shfl_xor_sync(0xffffffffu, gy2, m);
            }
            if (g == 0) *reinterpret_cast<float2*>(&sm.Gp[it & 1][warp][8 * nt + 2 * t4]) = make_float2(gx, gy2);
        }
        __syncthreads();  // (C1)

        // ---------------- stage C: contractions over the value index --------------------------
        float DA[2][4] = {}, DQ[2][4] = {}, DB[2][4] = {}, DK[2][4] = {};
        {
            // one score gradient per warp: 0 dQK = tril(dY V^T), 1 dAK = stril(dabu V^T),
            // 2 dQB = tril(dY U^T), 3 dAB = stril(dabu U^T)
            float d[2][4] = {};
            const bool strict = warp & 1;
            float* dst = warp == 0 ? sm.dQK : warp == 1 ? sm.dAK : warp == 2 ? sm.dQB : sm.dAB;
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                FragA<PREC> aD = fragA_mk<PREC>(sm.Dt, OPS, 0, 8 * kk, g, t4);
                FragA<PREC> aY = fragA_mk_st<IoT, PREC>(dyt, 8 * kk, g, t4);
                FragA<PREC> aU = fragA_mk<PREC>(sm.Ut, OPS, 0, 8 * kk, g, t4);
                FragA<PREC> aV = fragA_mk_st<IoT, PREC>(vt, 8 * kk, g, t4);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    FragB<PREC> bsc = (warp >> 1) ? fragB_nk<PREC>(sm.Ut, OPS, 8 * nt, 8 * kk, g, t4)
                                                  : fragB_nk_st<IoT, PREC>(vt, 8 * nt, 8 * kk, g, t4);
                    mma<PREC>(d[nt], strict ? aD : aY, bsc);
                    FragB<PREC> bS = fragB_kn<PREC>(sm.S0s, SS, 16 * warp + 8 * nt, 8 * kk, g, t4);
                    FragB<PREC> bD = fragB_kn<PREC>(sm.dSs, SS, 16 * warp + 8 * nt, 8 * kk, g, t4);
                    mma<PREC>(DA[nt], aD, bS);
                    mma<PREC>(DQ[nt], aY, bS);
                    mma<PREC>(DB[nt], aU, bD);
                    mma<PREC>(DK[nt], aV, bD);
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int s = 8 * nt + 2 * t4;
                auto keep = [&](int tq, int ss) { return strict ? ss < tq : ss <= tq; };
                *reinterpret_cast<float2*>(dst + g * SCS + s) =
                    make_float2(keep(g, s) ? d[nt][0] : 0.f, keep(g, s + 1) ? d[nt][1] : 0.f);
                *reinterpret_cast<float2*>(dst + (g + 8) * SCS + s) =
                    make_float2(keep(g + 8, s) ? d[nt][2] : 0.f, keep(g + 8, s + 1) ? d[nt][3] : 0.f);
            }
        }
        __syncthreads();  // (C2) score gradients visible; S0s free
        if (warp == 0 && c > 0) issue_s0(c - 1);

#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            FragA<PREC> aAB = fragA_mk<PREC>(sm.dAB, SCS, 0, 8 * kk, g, t4), aAK = fragA_mk<PREC>(sm.dAK, SCS, 0, 8 * kk, g, t4);
            FragA<PREC> aQB = fragA_mk<PREC>(sm.dQB, SCS, 0, 8 * kk, g, t4), aQK = fragA_mk<PREC>(sm.dQK, SCS, 0, 8 * kk, g, t4);
            FragA<PREC> tAB = fragA_km<PREC>(sm.dAB, SCS, 0, 8 * kk, g, t4), tAK = fragA_km<PREC>(sm.dAK, SCS, 0, 8 * kk, g, t4);
            FragA<PREC> tQB = fragA_km<PREC>(sm.dQB, SCS, 0, 8 * kk, g, t4), tQK = fragA_km<PREC>(sm.dQK, SCS, 0, 8 * kk, g, t4);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int n0 = 16 * warp + 8 * nt;
                FragB<PREC> bb = fragB_kn<PREC>(sm.bwi, OPS, n0, 8 * kk, g, t4), bk = fragB_kn<PREC>(sm.kwi, OPS, n0, 8 * kk, g, t4);
                FragB<PREC> ba = fragB_kn<PREC>(sm.wa, OPS, n0, 8 * kk, g, t4), bq = fragB_kn<PREC>(sm.wq, OPS, n0, 8 * kk, g, t4);
                mma<PREC>(DA[nt], aAB, bb); mma<PREC>(DA[nt], aAK, bk);
                mma<PREC>(DQ[nt], aQB, bb); mma<PREC>(DQ[nt], aQK, bk);
                mma<PREC>(DB[nt], tAB, ba); mma<PREC>(DB[nt], tQB, bq);
                mma<PREC>(DK[nt], tAK, ba); mma<PREC>(DK[nt], tQK, bq);
            }
        }

        // ---------------- epilogue: thread holds rows g, g+8 x key columns n0+2*t4, +1 ---------
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int key = 16 * warp + 8 * nt + 2 * t4;
            float x[2][2], e2[2][2], lwv[2][2];  // [row half][column]
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int tq = g + 8 * hrow;
                const float2 cu = *reinterpret_cast<const float2*>(sm.cum + tq * OPS + key);
                const float2 lwp = *reinterpret_cast<const float2*>(sm.lw + tq * OPS + key);
                const float2 oq = *reinterpret_cast<const float2*>(sm.wq + tq * OPS + key);
                const float2 oa = *reinterpret_cast<const float2*>(sm.wa + tq * OPS + key);
                const float2 okw = *reinterpret_cast<const float2*>(sm.kwi + tq * OPS + key);
                const float2 ob = *reinterpret_cast<const float2*>(sm.bwi + tq * OPS + key);
                const float cuv[2] = {cu.x, cu.y}, lwa[2] = {lwp.x, lwp.y};
                const float wqv[2] = {oq.x, oq.y}, wav[2] = {oa.x, oa.y}, kwv[2] = {okw.x, okw.y}, bwv[2] = {ob.x, ob.y};
                float o_q[2], o_k[2], o_a[2], o_b[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int i = e + 2 * hrow;
                    const float incl = exp_p<PREC>(cuv[e]), inv = exp_p<PREC>(-cuv[e]), non = exp_p<PREC>(cuv[e] - lwa[e]);
                    o_a[e] = non * DA[nt][i];
                    o_q[e] = incl * DQ[nt][i];
                    o_b[e] = inv * DB[nt][i];
                    o_k[e] = inv * DK[nt][i];
                    e2[hrow][e] = wav[e] * DA[nt][i];
                    x[hrow][e] = wqv[e] * DQ[nt][i] - kwv[e] * DK[nt][i] - bwv[e] * DB[nt][i] + e2[hrow][e];
                    lwv[hrow][e] = lwa[e];
                }
                const long long off = ((long long)c * L + tq) * p.st.t + key;
                store_pair<IoT>(gout[0] + off, o_q[0], o_q[1]);
                store_pair<IoT>(gout[2] + off, o_k[0], o_k[1]);
                store_pair<IoT>(gout[3] + off, o_a[0], o_a[1]);
                store_pair<IoT>(gout[4] + off, o_b[0], o_b[1]);
            }
            // inclusive suffix sum over the 16 time rows (rows live in lanes g = 0..7, two halves)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
#pragma unroll
                for (int d = 1; d < 8; d <<= 1) {
                    const float yl = __shfl_down_sync(0xffffffffu, x[0][e], 4 * d);
                    const float yh = __shfl_down_sync(0xffffffffu, x[1][e], 4 * d);
                    if (g + d < 8) { x[0][e] += yl; x[1][e] += yh; }
                }
                const float tot_hi = __shfl_sync(0xffffffffu, x[1][e], t4);
                x[0][e] += tot_hi;
            }
            const float2 Gc = make_float2(
                sm.Gp[(it & 1) ^ 1][0][key] + sm.Gp[(it & 1) ^ 1][1][key] + sm.Gp[(it & 1) ^ 1][2][key] + sm.Gp[(it & 1) ^ 1][3][key],
                sm.Gp[(it & 1) ^ 1][0][key + 1] + sm.Gp[(it & 1) ^ 1][1][key + 1] + sm.Gp[(it & 1) ^ 1][2][key + 1] + sm.Gp[(it & 1) ^ 1][3][key + 1]);
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int tq = g + 8 * hrow;
                const float d0 = (x[hrow][0] - e2[hrow][0] + Gc.x) * lwv[hrow][0];
                const float d1 = (x[hrow][1] - e2[hrow][1] + Gc.y) * lwv[hrow][1];
                store_pair<IoT>(gout[1] + ((long long)c * L + tq) * p.st.t + key, d0, d1);
            }
        }
        __syncthreads();  // (E)
    }

    if (failed) {
        if (tid == 0) atomicExch(p.status, (int)kDeviceTimeout);
        return;
    }
    if (p.ds0) {
        float* o = p.ds0 + bh * N * N;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(o + (16 * warp + g) * N + 8 * nt + 2 * t4) = make_float2(dS[nt][0], dS[nt][1]);
            *reinterpret_cast<float2*>(o + (16 * warp + g + 8) * N + 8 * nt + 2 * t4) = make_float2(dS[nt][2], dS[nt][3]);
        }
    }
}

template <typename IoT, int PREC> static int launch_bwd_t(const BwdParams& p, cudaStream_t stream) {
    using Smem = BwdSmem<IoT>;
    auto kern = wkv7_bwd_kernel<IoT, PREC>;
    const int smem = (int)sizeof(Smem);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return kLaunchFailed;
    kern<<<(unsigned)(p.B * p.H), THREADS, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int launch_bwd(const BwdParams& p, int io_dtype, cudaStream_t stream) {
    if (io_dtype == 0) return launch_bwd_t<__nv_bfloat16, 1>(p, stream);
    if (io_dtype == 2) return launch_bwd_t<float, 1>(p, stream);
    return launch_bwd_t<float, 3>(p, stream);
}

}  // namespace wkv7
