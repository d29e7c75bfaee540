// WKV7 forward for sm_100a: one CTA per (batch, head) chain, 4 warps, chunks of 16 time steps.
//
// Replaces the reference's forward_kernel (wind_rwkv/rwkv7/attn.cu:11-106) and, with LN = true,
// the fused variant (wind_rwkv/rwkv7/attn_ln.cu:106-212).  Not a translation: the whole
// state-dependent part of a chunk is computed TRANSPOSED (rows = value index), so that warp w
// owns value rows 16w..16w+15 of the state S, of X^T, U^T and Y^T, keeps S in registers across
// chunks as MMA accumulators, feeds accumulators straight back as A operands, and needs no
// cross-warp reduction.  Only the state-independent chunk preparation (decay scan, scaled
// operands, the four masked 16x16 score matrices and the triangular inverse) is shared through
// shared memory.
//
// Per chunk (rows = time, P_t = prod_{s<=t} exp(-exp(w_s)) per key channel, S0 = state at the
// chunk start, S[value][key]):
//     wq = q*P_t     wa = a*P_{t-1}     kwi = k/P_t     bwi = b/P_t     fw = P_L
// (in the code P_t is kept as 2^64 P_t and the state as 2^-64 S, which leaves every formula as it is: see ANCHOR_LN)
//     QK = tril(wq kwi^T)  QB = tril(wq bwi^T)  AK = stril(wa kwi^T)  AB = stril(wa bwi^T)
//     X = AK V + wa S0^T ;  U = (I-AB)^-1 X ;  Y = QK V + QB U + wq S0^T
//     S' = (S0 + V^T kwi + U^T bwi) * fw[None,:]
// Inputs are fetched one chunk ahead with 16-byte cp.async copies issued by all threads.
#include "wkv7_kernels.h"

namespace wkv7 {

template <typename IoT> struct FwdLayout {
    static constexpr int ROWB = N * (int)sizeof(IoT) + 16;  // padded staging row (bytes)
    static constexpr int TILEB = L * ROWB;
    static constexpr int YS = (sizeof(IoT) == 2) ? 24 : 20;  // y scratch row stride (elements)
};

template <typename IoT, bool LN> struct FwdSmem {
    using Lay = FwdLayout<IoT>;
    alignas(16) unsigned char st_in[5][Lay::TILEB];  // q, w, k, a, b of the current chunk
    alignas(16) unsigned char st_v[2][Lay::TILEB];   // v, double buffered (read late in the chunk)
    alignas(16) unsigned char st_g[LN ? 2 : 1][LN ? Lay::TILEB : 16];
    alignas(16) float wq[L * OPS], wa[L * OPS], kwi[L * OPS], bwi[L * OPS];
    alignas(16) float QK[L * SCS], QB[L * SCS], AK[L * SCS], AB[L * SCS], AI[L * SCS];
    alignas(16) float fw[N];
    alignas(16) float lnp[LN ? 3 * N : 4];
    float bdot[L];
    float red[WARPS][L][2];
    alignas(16) IoT ysc[WARPS][L * Lay::YS];
};

template <typename IoT> __device__ __forceinline__ float st_elem(const unsigned char* tile, int row, int col) {
    return to_f32<IoT>(*reinterpret_cast<const IoT*>(tile + row * FwdLayout<IoT>::ROWB + col * (int)sizeof(IoT)));
}

template <typename IoT, int PREC, bool LN>
__global__ void __launch_bounds__(THREADS) wkv7_fwd_kernel(FwdParams p) {
    using Lay = FwdLayout<IoT>;
    using Smem = FwdSmem<IoT, LN>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const long long bh = blockIdx.x;
    const long long bi = bh / p.H, hi = bh % p.H;
    const long long base = bi * p.st.b + hi * p.st.h;
    const int nchunks = (int)((p.T + L - 1) / L);  // the last chunk may be partial: its missing rows read as zeros
    const bool has_tail = (p.T % L) != 0;
    const IoT* gin[5] = {(const IoT*)p.r + base, (const IoT*)p.w + base, (const IoT*)p.k + base,
                         (const IoT*)p.a + base, (const IoT*)p.b + base};
    const IoT* gv = (const IoT*)p.v + base;
    const IoT* gg = LN ? (const IoT*)p.g + base : nullptr;
    IoT* gy = (IoT*)p.y + base;
    constexpr uint32_t ROW_BYTES = N * sizeof(IoT);

    if (LN) {
        for (int i = tid; i < 3 * N; i += THREADS) sm.lnp[i] = p.params[(long long)(i / N) * p.H * N + hi * N + (i % N)];
    }
    __syncthreads();

    // q, w, k, a, b are dead once the scan has run, so the next chunk's copies are issued right
    // after the first barrier of the iteration; v (and g) are read late and double buffered.
    constexpr int CH = ROW_BYTES / 16;
    auto issue_in = [&](int c) {
        for (int i = tid; i < 5 * L * CH; i += THREADS) {
            int ten = i / (L * CH), row = (i / CH) % L, ch = i % CH;
            const long long tt = (long long)c * L + row;
            if (has_tail) cp_async16_zfill(sm.st_in[ten] + row * Lay::ROWB + ch * 16,
                             reinterpret_cast<const unsigned char*>(gin[ten] + (tt < p.T ? tt : p.T - 1) * p.st.t) + ch * 16, tt < p.T);
            else cp_async16(sm.st_in[ten] + row * Lay::ROWB + ch * 16, reinterpret_cast<const unsigned char*>(gin[ten] + tt * p.st.t) + ch * 16);
        }
    };
    auto issue_v = [&](int c) {
        int s = c & 1;
        for (int i = tid; i < (LN ? 2 : 1) * L * CH; i += THREADS) {
            int ten = i / (L * CH), row = (i / CH) % L, ch = i % CH;
            const long long tt = (long long)c * L + row;
            const IoT* src = (ten == 0 ? gv : gg) + (tt < p.T ? tt : p.T - 1) * p.st.t;
            unsigned char* dst = (ten == 0 ? sm.st_v[s] : sm.st_g[LN ? s : 0]) + row * Lay::ROWB;
            if (has_tail) cp_async16_zfill(dst + ch * 16, reinterpret_cast<const unsigned char*>(src) + ch * 16, tt < p.T);
            else cp_async16(dst + ch * 16, reinterpret_cast<const unsigned char*>(src) + ch * 16);
        }
    };
    if (nchunks > 0) {
        issue_in(0);
        issue_v(0);
        cp_async_commit();
        cp_async_wait<0>();
    }
    __syncthreads();

    // State: warp owns value rows 16*warp + {g, g+8}; tile nt covers key columns 8nt..8nt+7,
    // thread holds columns 8nt+2*t4, +1.
    float S[8][4];
    {
        const float* s0 = p.s0 ? p.s0 + bh * N * N : nullptr;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            if (s0) {
                float2 lo = *reinterpret_cast<const float2*>(s0 + (16 * warp + g) * N + 8 * nt + 2 * t4);
                float2 hi2 = *reinterpret_cast<const float2*>(s0 + (16 * warp + g + 8) * N + 8 * nt + 2 * t4);
                // the state is carried as S~ = 2^-64 S (see ANCHOR_LN)
                S[nt][0] = lo.x * STATE_SCALE; S[nt][1] = lo.y * STATE_SCALE; S[nt][2] = hi2.x * STATE_SCALE; S[nt][3] = hi2.y * STATE_SCALE;
            } else {
                S[nt][0] = S[nt][1] = S[nt][2] = S[nt][3] = 0.f;
            }
        }
    }

    for (int c = 0; c < nchunks; ++c) {
        // ---------------- P1: decay scan and scaled operands ------------------------------------
        {
            decay_scan<IoT, PREC>(sm.st_in[0], sm.st_in[1], sm.st_in[2], sm.st_in[3], sm.st_in[4], Lay::ROWB, sm.wq, sm.wa,
                                  sm.kwi, sm.bwi, sm.fw, nullptr, nullptr, warp, lane, (int)min((long long)L, p.T - (long long)c * L));
            if (LN) {  // bonus dot  sum_j r_j k_j bonus_j  per time step: 8 threads per row
                const int row = tid >> 3, part = tid & 7;
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int ch = part * 8 + i;
                    acc += st_elem<IoT>(sm.st_in[0], row, ch) * st_elem<IoT>(sm.st_in[2], row, ch) * sm.lnp[2 * N + ch];
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                acc += __shfl_xor_sync(0xffffffffu, acc, 4);
                if (part == 0) sm.bdot[row] = acc;
            }
        }
        __syncthreads();  // (A)
        if (c + 1 < nchunks) {
            issue_in(c + 1);
            issue_v(c + 1);
        }
        cp_async_commit();
        // ---------------- P2: masked score matrices, one per warp ------------------------------
        {
            const float* Am = (warp & 1) ? sm.wa : sm.wq;
            const float* Bm = (warp >> 1) ? sm.bwi : sm.kwi;
            float* dst = warp == 0 ? sm.QK : warp == 1 ? sm.AK : warp == 2 ? sm.QB : sm.AB;
            const bool strict = warp & 1;
            float d[2][4] = {};
#pragma unroll 2
            for (int kk = 0; kk < 8; ++kk) {
                FragA<PREC> a = fragA_mk<PREC, true>(Am, OPS, 0, 8 * kk, g, t4);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) mma<PREC>(d[nt], a, fragB_nk<PREC, true>(Bm, OPS, 8 * nt, 8 * kk, g, t4));
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int s = 8 * nt + 2 * t4;
                auto keep = [&](int tq, int ss) { return strict ? ss < tq : ss <= tq; };
                // AB only feeds the inverse and stays unrounded; the other three are MMA operands
                auto val = [&](float x) { return warp == 3 ? x : pre<PREC>(x); };
                float2 lo = make_float2(keep(g, s) ? val(d[nt][0]) : 0.f, keep(g, s + 1) ? val(d[nt][1]) : 0.f);
                float2 hi2 = make_float2(keep(g + 8, s) ? val(d[nt][2]) : 0.f, keep(g + 8, s + 1) ? val(d[nt][3]) : 0.f);
                if (warp == 3) {  // AB is kept transposed for the inverse
                    dst[s * SCS + g] = lo.x; dst[(s + 1) * SCS + g] = lo.y;
                    dst[s * SCS + g + 8] = hi2.x; dst[(s + 1) * SCS + g + 8] = hi2.y;
                } else {
                    *reinterpret_cast<float2*>(dst + g * SCS + s) = lo;
                    *reinterpret_cast<float2*>(dst + (g + 8) * SCS + s) = hi2;
                }
            }
        }
        // ---------------- P3: AI = (I - AB)^-1 by forward substitution (the warp that made AB) --
        if (warp == 3) {
            __syncwarp();
            if (lane < L) tri_inverse_column<PREC>(sm.AB, sm.AI, lane);
        }
        // ---------------- chain, part 1: needs only S and the scaled operands ------------------
        if (p.ckpt) {
            float* ck = p.ckpt + (bh * nchunks + c) * (long long)CK_FLOATS;
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                // exact fp32: in the single-TF32 class the backward's tensor-core products read the upper 19 bits without a
                // conversion, and its carried decay term uses the full value
                *reinterpret_cast<float2*>(ck + (16 * warp + g) * N + 8 * nt + 2 * t4) = make_float2(S[nt][0], S[nt][1]);
                *reinterpret_cast<float2*>(ck + (16 * warp + g + 8) * N + 8 * nt + 2 * t4) = make_float2(S[nt][2], S[nt][3]);
            }
        }
        float XY[4][4] = {};  // [0..1] X^T (time blocks 0,1), [2..3] Y^T
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
            FragA<PREC> a = fragA_from_acc<PREC>(S[kk]);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
                mma<PREC>(XY[nt], a, fragB_nk<PREC, true>(nt < 2 ? sm.wa : sm.wq, OPS, 8 * (nt & 1), 8 * kk, g, t4));
        }
        __syncthreads();  // (B) scores and AI visible
        if (p.ckpt) {  // the chunk's four 16x16 matrices go into the checkpoint record: 8 floats per thread
            float* ck = p.ckpt + (bh * nchunks + c) * (long long)CK_FLOATS;
            const int m = tid >> 5, r = (tid & 31) >> 1, hf = tid & 1;
            const float* src = (m == 0 ? sm.QK : m == 1 ? sm.QB : m == 2 ? sm.AK : sm.AI) + r * SCS + 8 * hf;
            float* dst = ck + (m == 0 ? CK_SC + ck_tile_at(16 + r, 2 * hf) : m == 1 ? CK_QB + ck_tile_at(r, 2 * hf)
                                                                            : m == 2 ? CK_SC + ck_tile_at(r, 2 * hf) : CK_AI + ck_tile_at(r, 2 * hf));
            *reinterpret_cast<float4*>(dst) = *reinterpret_cast<const float4*>(src);
            *reinterpret_cast<float4*>(dst + 32) = *reinterpret_cast<const float4*>(src + 4);
        }

        // ---------------- chain, part 2 ----------------------------------------------------------
        const unsigned char* vt = sm.st_v[c & 1];
        FragA<PREC> vf[2];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const int tr = 8 * kk + 2 * t4, vc = 16 * warp + g;
            constexpr bool EXACT = sizeof(IoT) == 2;  // a bf16 value is a TF32 value
            vf[kk].x[0].template put<EXACT>(st_elem<IoT>(vt, tr, vc));
            vf[kk].x[1].template put<EXACT>(st_elem<IoT>(vt, tr, vc + 8));
            vf[kk].x[2].template put<EXACT>(st_elem<IoT>(vt, tr + 1, vc));
            vf[kk].x[3].template put<EXACT>(st_elem<IoT>(vt, tr + 1, vc + 8));
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int kk = 0; kk <= nt; ++kk) {
                mma<PREC>(XY[nt], vf[kk], fragB_nk<PREC, true>(sm.AK, SCS, 8 * nt, 8 * kk, g, t4));
                mma<PREC>(XY[2 + nt], vf[kk], fragB_nk<PREC, true>(sm.QK, SCS, 8 * nt, 8 * kk, g, t4));
            }
        float U[2][4] = {};
        {
            FragA<PREC> xa[2] = {fragA_from_acc<PREC>(XY[0]), fragA_from_acc<PREC>(XY[1])};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int kk = 0; kk <= nt; ++kk) mma<PREC>(U[nt], xa[kk], fragB_nk<PREC, true>(sm.AI, SCS, 8 * nt, 8 * kk, g, t4));
        }
        FragA<PREC> ua[2] = {fragA_from_acc<PREC>(U[0]), fragA_from_acc<PREC>(U[1])};
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int kk = 0; kk <= nt; ++kk) mma<PREC>(XY[2 + nt], ua[kk], fragB_nk<PREC, true>(sm.QB, SCS, 8 * nt, 8 * kk, g, t4));

        // ---------------- output -----------------------------------------------------------------
        if (LN) {
            // GroupNorm over the head's 64 value channels of each time step: per-warp mean and
            // centred sum of squares over 16 rows, merged across warps (Chan's formula).
            float mean_w[4], m2_w[4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    float s = XY[2 + nt][e] + XY[2 + nt][e + 2];
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    s += __shfl_xor_sync(0xffffffffu, s, 8);
                    s += __shfl_xor_sync(0xffffffffu, s, 16);
                    const float mu = s * (1.f / 16.f);
                    const float d0 = XY[2 + nt][e] - mu, d1 = XY[2 + nt][e + 2] - mu;
                    float q = d0 * d0 + d1 * d1;
                    q += __shfl_xor_sync(0xffffffffu, q, 4);
                    q += __shfl_xor_sync(0xffffffffu, q, 8);
                    q += __shfl_xor_sync(0xffffffffu, q, 16);
                    mean_w[2 * nt + e] = mu;
                    m2_w[2 * nt + e] = q;
                }
            if (g == 0)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tq = 8 * (i >> 1) + 2 * t4 + (i & 1);
                    sm.red[warp][tq][0] = mean_w[i];
                    sm.red[warp][tq][1] = m2_w[i];
                }
            __syncthreads();  // (D)
            const unsigned char* gt = sm.st_g[c & 1];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int nt = i >> 1, e = i & 1, tq = 8 * nt + 2 * t4 + e;
                float mu = 0.f, m2 = 0.f;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; ++w2) mu += sm.red[w2][tq][0];
                mu *= 0.25f;
#pragma unroll
                for (int w2 = 0; w2 < WARPS; ++w2) {
                    const float dm = sm.red[w2][tq][0] - mu;
                    m2 += sm.red[w2][tq][1] + 16.f * dm * dm;
                }
                const float rstd = 1.f / sqrtf(m2 * (1.f / N) + p.eps);
                const float bd = sm.bdot[tq];
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int vc = 16 * warp + g + 8 * hrow;
                    float y = XY[2 + nt][e + 2 * hrow];
                    y = (y - mu) * rstd * sm.lnp[vc] + sm.lnp[N + vc] + bd * st_elem<IoT>(vt, tq, vc);
                    XY[2 + nt][e + 2 * hrow] = y * st_elem<IoT>(gt, tq, vc);
                }
            }
        }
        {
            IoT* sc = sm.ysc[warp];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int tq = 8 * nt + 2 * t4;
                sc[tq * Lay::YS + g] = from_f32<IoT>(XY[2 + nt][0]);
                sc[(tq + 1) * Lay::YS + g] = from_f32<IoT>(XY[2 + nt][1]);
                sc[tq * Lay::YS + g + 8] = from_f32<IoT>(XY[2 + nt][2]);
                sc[(tq + 1) * Lay::YS + g + 8] = from_f32<IoT>(XY[2 + nt][3]);
            }
            __syncwarp();
            const int row = lane >> 1, hf = lane & 1;
            const uint4* src = reinterpret_cast<const uint4*>(sc + row * Lay::YS + 8 * hf);
            uint4* dst = reinterpret_cast<uint4*>(gy + ((long long)c * L + row) * p.st.t + 16 * warp + 8 * hf);
            if ((long long)c * L + row < p.T) {
                dst[0] = src[0];
                if (sizeof(IoT) == 4) dst[1] = src[1];
            }
        }
        // ---------------- state update -----------------------------------------------------------
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
            for (int kk = 0; kk < 2; ++kk) {
                mma<PREC>(S[nt], vf[kk], fragB_kn<PREC, true>(sm.kwi, OPS, 8 * nt, 8 * kk, g, t4));
                mma<PREC>(S[nt], ua[kk], fragB_kn<PREC, true>(sm.bwi, OPS, 8 * nt, 8 * kk, g, t4));
            }
            const float2 f = *reinterpret_cast<const float2*>(sm.fw + 8 * nt + 2 * t4);  // P~_L = 2^64 P_L
            S[nt][0] = S[nt][0] * f.x * STATE_SCALE; S[nt][1] = S[nt][1] * f.y * STATE_SCALE;
            S[nt][2] = S[nt][2] * f.x * STATE_SCALE; S[nt][3] = S[nt][3] * f.y * STATE_SCALE;
        }
        cp_async_wait<0>();
        __syncthreads();  // (E) operand and score buffers are free again
    }

    if (p.sT) {
        float* sT = p.sT + bh * N * N;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(sT + (16 * warp + g) * N + 8 * nt + 2 * t4) = make_float2(S[nt][0] * STATE_UNSCALE, S[nt][1] * STATE_UNSCALE);
            *reinterpret_cast<float2*>(sT + (16 * warp + g + 8) * N + 8 * nt + 2 * t4) = make_float2(S[nt][2] * STATE_UNSCALE, S[nt][3] * STATE_UNSCALE);
        }
    }
}

template <typename IoT, int PREC, bool LN> static int launch_fwd_t(const FwdParams& p, cudaStream_t stream) {
    using Smem = FwdSmem<IoT, LN>;
    auto kern = wkv7_fwd_kernel<IoT, PREC, LN>;
    const int smem = (int)sizeof(Smem);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return kLaunchFailed;
    kern<<<(unsigned)(p.B * p.H), THREADS, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int launch_fwd(const FwdParams& p, int io_dtype, bool ln, cudaStream_t stream) {
    if (io_dtype == 0) return ln ? launch_fwd_t<__nv_bfloat16, 1, true>(p, stream) : launch_fwd_t<__nv_bfloat16, 1, false>(p, stream);
    if (io_dtype == 2) return ln ? launch_fwd_t<float, 1, true>(p, stream) : launch_fwd_t<float, 1, false>(p, stream);
    return ln ? launch_fwd_t<float, 3, true>(p, stream) : launch_fwd_t<float, 3, false>(p, stream);
}

}  // namespace wkv7
