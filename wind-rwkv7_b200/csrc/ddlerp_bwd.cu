// ddlerp backward for sm_100a.  Replaces bw1..bw4_triton_ of the reference
// (wind_rwkv/rwkv7/rwkv7_ddlerp.py:92-303) with three kernels:
//
//   dpre  (token tiles, all channels)   dm_k = (dy_k * xx) @ R_k ;  dpre = dm * (1 - m^2)      -> [rows,4D]
//   main  (channel block x batch, walks the sequence backwards in 32-token tiles)
//         du = dpre @ L[:,cb] ; z_k = m_k @ R_k[cb]^T + beta_k
//         X = sum_k dy_k z_k + du alpha   (gradient of xx)      Dd = sum_k dy_k + du
//         dx_t = Dd_t - X_t + X_{t+1}     (X_{t+1} of the following tile is carried in shared memory)
//         dR_k[cb] += (dy_k xx)^T m_k ;  dalpha += colsum(du xx) ;  dbeta_k += colsum(dy_k xx)
//   dL    (channel block x row segment)  dL[:,cb] += dpre^T (x + xx alpha)
//
// with xx = x_{t-1} - x_t.  Weight gradients are accumulated in registers over a CTA's whole row
// range and flushed once with fp32 atomics.  Operands whose contraction index is the row index of
// their shared-memory tile are fetched with transposing ldmatrix.
#include "ddlerp.h"
#include "mma_bf16.cuh"

namespace wkv7 {

constexpr int BLD = 64 + 8;  // row stride (bf16) of 64-channel tiles

// ------------------------------------------------------------------------------------------------
// dpre kernel: 32-token tiles, 8 warps = 2 m-tiles x 4 streams.
template <int D> struct DpreSmem {
    bf16 dz[2][4][32][BLD];
    bf16 RB[2][4][64][D + 8];
};

template <int D>
__global__ void __launch_bounds__(256) ddlerp_bwd_dpre_kernel(DdlerpBwdParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sm = *reinterpret_cast<DpreSmem<D>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const long long row0 = (long long)blockIdx.x * 32;
    const int C = (int)p.C, nkb = C / 64;
    const int erow = tid >> 3, eseg = tid & 7;  // 8 threads per row, 8 channels each
    const long long grow = row0 + erow;
    const bool live = grow < p.rows;
    const bool first = (grow % p.T) == 0;
    const bf16* x = (const bf16*)p.x;

    uint4 rx, rp, rdy[4];
    auto load_in = [&](int cb) {
        if (!live) {
            rx = rp = rdy[0] = rdy[1] = rdy[2] = rdy[3] = make_uint4(0, 0, 0, 0);
            return;
        }
        const long long off = grow * C + cb * 64 + eseg * 8;
        rx = *reinterpret_cast<const uint4*>(x + off);
        rp = first ? make_uint4(0, 0, 0, 0) : *reinterpret_cast<const uint4*>(x + off - C);
#pragma unroll
        for (int k = 0; k < 4; ++k) rdy[k] = *reinterpret_cast<const uint4*>((const bf16*)p.dy[k] + off);
    };
    auto issue_R = [&](int cb, int buf) {
        constexpr int CH = D / 8;
        for (int i = tid; i < 4 * 64 * CH; i += 256) {
            const int k = i / (64 * CH), r = (i / CH) % 64, ch = i % CH;
            cp_async16(&sm.RB[buf][k][r][ch * 8], (const bf16*)p.R + ((long long)k * C + cb * 64 + r) * D + ch * 8);
        }
        cp_async_commit();
    };

    const int wmt = warp & 1, wk = warp >> 1;  // m-tile, stream
    float acc[D / 8][4] = {};
    load_in(0);
    issue_R(0, 0);
    for (int cb = 0; cb < nkb; ++cb) {
        const int buf = cb & 1;
        {
            float xv[8], pv[8];
            unpack8(rx, xv); unpack8(rp, pv);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float dv[8], o[8];
                unpack8(rdy[k], dv);
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = dv[i] * (pv[i] - xv[i]);
                *reinterpret_cast<uint4*>(&sm.dz[buf][k][erow][eseg * 8]) = pack8(o);
            }
        }
        if (cb + 1 < nkb) {
            load_in(cb + 1);
            issue_R(cb + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t a[4];
            ldA_mk(a, &sm.dz[buf][wk][0][0], BLD, 16 * wmt, 16 * ks, g, t4);
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                uint32_t b[2];
                ldB_kn_trans(b, &sm.RB[buf][wk][0][0], D + 8, 8 * j, 16 * ks, lane);
                mma_bf16(acc[j], a, b);
            }
        }
    }
    const bf16* m = (const bf16*)p.m;
    bf16* dp = (bf16*)p.dpre;
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            if (row0 + 16 * wmt + g + 8 * hrow >= p.rows) continue;
            const long long off = (row0 + 16 * wmt + g + 8 * hrow) * (4 * D) + wk * D + 8 * j + 2 * t4;
            const float2 mv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(m + off));
            *reinterpret_cast<uint32_t*>(dp + off) =
                pack_bf16x2(acc[j][2 * hrow] * (1.f - mv.x * mv.x), acc[j][2 * hrow + 1] * (1.f - mv.y * mv.y));
        }
}

// ------------------------------------------------------------------------------------------------
// main kernel: grid (C/64, B); 32-token tiles walked backwards; 8 warps = 2 m-tiles x 4 column groups.
template <int D> struct MainSmem {
    bf16 Lb[4 * D][BLD];        // L[:, cb]   [4D][64]
    bf16 RB[4][64][D + 8];      // R_k[cb]    [64][D]
    float alpha[64], beta[4][64];
    bf16 xS[33][BLD];           // row 0 = token before the tile
    bf16 dyS[4][32][BLD];       // dy_k, overwritten in place by dy_k * xx
    bf16 mS[32][4 * D + 8], dpS[32][4 * D + 8];
    float XS[33][68];           // row 32 = first row of the following tile (carry)
    bf16 dxS[32][BLD];
};

template <int D>
__global__ void __launch_bounds__(256) ddlerp_bwd_main_kernel(DdlerpBwdParams p, int segs, int tiles_per_seg) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sm = *reinterpret_cast<MainSmem<D>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int cb = blockIdx.x;
    // blockIdx.y = sequence * segs + segment: a sequence is cut into `segs` runs of tiles_per_seg 32-token tiles, each walked
    // backwards by its own CTA.  A run that is not the sequence's last first processes the tile that follows it, only to
    // obtain the carried row X of that tile's first token (its accumulators are reset afterwards, nothing is stored).
    const int seg = (int)(blockIdx.y % segs);
    const long long b0 = (long long)(blockIdx.y / segs) * p.T;  // first row of this sequence
    const int C = (int)p.C, T = (int)p.T;
    const bf16* x = (const bf16*)p.x;

    // resident operands
    for (int i = tid; i < 4 * D * 8; i += 256) {
        const int r = i / 8, ch = i % 8;
        cp_async16(&sm.Lb[r][ch * 8], (const bf16*)p.L + (long long)r * C + cb * 64 + ch * 8);
    }
    {
        constexpr int CH = D / 8;
        for (int i = tid; i < 4 * 64 * CH; i += 256) {
            const int k = i / (64 * CH), r = (i / CH) % 64, ch = i % CH;
            cp_async16(&sm.RB[k][r][ch * 8], (const bf16*)p.R + ((long long)k * C + cb * 64 + r) * D + ch * 8);
        }
    }
    cp_async_commit();
    if (tid < 64) {
        sm.alpha[tid] = __bfloat162float(((const bf16*)p.alpha)[cb * 64 + tid]);
        sm.XS[32][tid] = 0.f;  // nothing follows the last token
    }
    sm.beta[tid >> 6][tid & 63] = __bfloat162float(((const bf16*)p.beta)[(long long)(tid >> 6) * C + cb * 64 + (tid & 63)]);

    const int wmt = warp & 1, wn = warp >> 1;  // m-tile (16 tokens), column group (16 channels = 2 n-tiles)
    float dR[D / 8][4] = {};                   // stream k = warp >> 1, channel m-tiles 2*(warp&1) + {0,1} ... see MMA-3
    float dR2[D / 8][4] = {};
    float dal[2][2] = {}, dbe[4][2][2] = {};

    const int t_last = ((T - 1) / 32) * 32;                       // first token of the sequence's last tile
    const int t_lo = seg * tiles_per_seg * 32;                    // first token of this run
    const int t_next = t_lo + tiles_per_seg * 32;                 // first token of the following run
    bool warm = t_next <= t_last;                                 // a run follows: start with its first tile
    for (int t0 = warm ? t_next : t_last; t0 >= t_lo; t0 -= 32) {
        const long long r0 = b0 + t0;
        const int nrow = T - t0 < 32 ? T - t0 : 32;  // live rows of this tile (the last one may be short)
        // ---- loads -----------------------------------------------------------------------------
        for (int i = tid; i < 33 * 8; i += 256) {
            const int r = i / 8, ch = i % 8;
            if ((t0 == 0 && r == 0) || r > nrow) *reinterpret_cast<uint4*>(&sm.xS[r][ch * 8]) = make_uint4(0, 0, 0, 0);
            else cp_async16(&sm.xS[r][ch * 8], x + (r0 + r - 1) * C + cb * 64 + ch * 8);
        }
        for (int i = tid; i < 4 * 32 * 8; i += 256) {
            const int k = i / 256, r = (i / 8) % 32, ch = i % 8;
            if (r >= nrow) *reinterpret_cast<uint4*>(&sm.dyS[k][r][ch * 8]) = make_uint4(0, 0, 0, 0);
            else cp_async16(&sm.dyS[k][r][ch * 8], (const bf16*)p.dy[k] + (r0 + r) * C + cb * 64 + ch * 8);
        }
        for (int i = tid; i < 32 * (4 * D / 8); i += 256) {
            const int r = i / (4 * D / 8), ch = i % (4 * D / 8);
            if (r >= nrow) {
                *reinterpret_cast<uint4*>(&sm.mS[r][ch * 8]) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(&sm.dpS[r][ch * 8]) = make_uint4(0, 0, 0, 0);
            } else {
                cp_async16(&sm.mS[r][ch * 8], (const bf16*)p.m + (r0 + r) * (4 * D) + ch * 8);
                cp_async16(&sm.dpS[r][ch * 8], (const bf16*)p.dpre + (r0 + r) * (4 * D) + ch * 8);
            }
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();

        // ---- du = dpre @ L[:,cb],  z_k = m_k @ R_k[cb]^T -----------------------------------------
        float du[2][4] = {}, z[4][2][4] = {};
#pragma unroll
        for (int ks = 0; ks < 4 * D / 16; ++ks) {
            uint32_t a[4];
            ldA_mk(a, &sm.dpS[0][0], 4 * D + 8, 16 * wmt, 16 * ks, g, t4);
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                uint32_t b[2];
                ldB_kn_trans(b, &sm.Lb[0][0], BLD, 16 * wn + 8 * j, 16 * ks, lane);
                mma_bf16(du[j], a, b);
            }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a[4];
                ldA_mk(a, &sm.mS[0][0], 4 * D + 8, 16 * wmt, k * D + 16 * ks, g, t4);
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    uint32_t b[2];
                    ldB_nk(b, &sm.RB[k][0][0], D + 8, 16 * wn + 8 * j, 16 * ks, g, t4);
                    mma_bf16(z[k][j], a, b);
                }
            }
        // ---- elementwise at the accumulator positions ---------------------------------------------
        float dd[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int r = 16 * wmt + g + 8 * hrow, cc = 16 * wn + 8 * j + 2 * t4;
                const float2 xv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.xS[r + 1][cc]));
                const float2 pv = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.xS[r][cc]));
                const float xx0 = pv.x - xv.x, xx1 = pv.y - xv.y;
                const float du0 = du[j][2 * hrow], du1 = du[j][2 * hrow + 1];
                float X0 = du0 * sm.alpha[cc], X1 = du1 * sm.alpha[cc + 1];
                float D0 = du0, D1 = du1;
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 dy = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.dyS[k][r][cc]));
                    X0 += dy.x * (z[k][j][2 * hrow] + sm.beta[k][cc]);
                    X1 += dy.y * (z[k][j][2 * hrow + 1] + sm.beta[k][cc + 1]);
                    D0 += dy.x; D1 += dy.y;
                    const float dz0 = dy.x * xx0, dz1 = dy.y * xx1;
                    dbe[k][j][0] += dz0; dbe[k][j][1] += dz1;
                    *reinterpret_cast<uint32_t*>(&sm.dyS[k][r][cc]) = pack_bf16x2(dz0, dz1);
                }
                dal[j][0] += du0 * xx0; dal[j][1] += du1 * xx1;
                *reinterpret_cast<float2*>(&sm.XS[r][cc]) = make_float2(X0, X1);
                dd[j][2 * hrow] = D0; dd[j][2 * hrow + 1] = D1;
            }
        __syncthreads();
        // ---- dx_t = Dd_t - X_t + X_{t+1} ---------------------------------------------------------------
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int r = 16 * wmt + g + 8 * hrow, cc = 16 * wn + 8 * j + 2 * t4;
                const float2 Xc = *reinterpret_cast<const float2*>(&sm.XS[r][cc]);
                const float2 Xn = *reinterpret_cast<const float2*>(&sm.XS[r + 1][cc]);
                *reinterpret_cast<uint32_t*>(&sm.dxS[r][cc]) =
                    pack_bf16x2(dd[j][2 * hrow] - Xc.x + Xn.x, dd[j][2 * hrow + 1] - Xc.y + Xn.y);
            }
        // ---- dR_k[cb] += (dy_k xx)^T m_k : warp = (stream pair, channel m-tile pair) ------------------
        {
            const int k = warp >> 1, mp = warp & 1;  // stream, channel half (2 m-tiles of 16 channels)
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
                uint32_t a0[4], a1[4];
                ldA_km_trans(a0, &sm.dyS[k][0][0], BLD, 32 * mp, 16 * ks, lane);
                ldA_km_trans(a1, &sm.dyS[k][0][0], BLD, 32 * mp + 16, 16 * ks, lane);
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    uint32_t b[2];
                    ldB_kn_trans(b, &sm.mS[0][0], 4 * D + 8, k * D + 8 * j, 16 * ks, lane);
                    mma_bf16(dR[j], a0, b);
                    mma_bf16(dR2[j], a1, b);
                }
            }
        }
        __syncthreads();
        // ---- dx out (coalesced), carry X_{t0} for the previous tile ----------------------------------
        {
            const int r = tid >> 3, ch = tid & 7;
            if (r < nrow && !warm)
                *reinterpret_cast<uint4*>((bf16*)p.dx + (r0 + r) * C + cb * 64 + ch * 8) = *reinterpret_cast<const uint4*>(&sm.dxS[r][ch * 8]);
        }
        if (tid < 64) sm.XS[32][tid] = sm.XS[0][tid];
        if (warm) {  // the following run's tile only supplied the carry
            warm = false;
#pragma unroll
            for (int j = 0; j < D / 8; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) dR[j][i] = dR2[j][i] = 0.f;
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    dal[j][e] = 0.f;
#pragma unroll
                    for (int k = 0; k < 4; ++k) dbe[k][j][e] = 0.f;
                }
        }
        __syncthreads();
    }

    // ---- flush weight gradients -------------------------------------------------------------------
    {
        const int k = warp >> 1, mp = warp & 1;
#pragma unroll
        for (int j = 0; j < D / 8; ++j)
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                float* o = p.dR + ((long long)k * C + cb * 64 + 32 * mp + g + 8 * hrow) * D + 8 * j + 2 * t4;
                atomicAdd(o, dR[j][2 * hrow]); atomicAdd(o + 1, dR[j][2 * hrow + 1]);
                atomicAdd(o + 16 * D, dR2[j][2 * hrow]); atomicAdd(o + 16 * D + 1, dR2[j][2 * hrow + 1]);
            }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            float a = dal[j][e];
            a += __shfl_xor_sync(0xffffffffu, a, 4); a += __shfl_xor_sync(0xffffffffu, a, 8); a += __shfl_xor_sync(0xffffffffu, a, 16);
            if (g == 0) atomicAdd(p.dalpha + cb * 64 + 16 * wn + 8 * j + 2 * t4 + e, a);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float bsum = dbe[k][j][e];
                bsum += __shfl_xor_sync(0xffffffffu, bsum, 4); bsum += __shfl_xor_sync(0xffffffffu, bsum, 8); bsum += __shfl_xor_sync(0xffffffffu, bsum, 16);
                if (g == 0) atomicAdd(p.dbeta + (long long)k * C + cb * 64 + 16 * wn + 8 * j + 2 * t4 + e, bsum);
            }
        }
}

// ------------------------------------------------------------------------------------------------
// dL kernel: grid (C/64, segments); dL[:,cb] += dpre^T u over the segment's rows, 64-row tiles.
template <int D> struct DLSmem {
    bf16 uS[64][BLD];
    bf16 dpS[64][4 * D + 8];
};

template <int D>
__global__ void __launch_bounds__(256) ddlerp_bwd_dL_kernel(DdlerpBwdParams p, long long rows_per_seg) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sm = *reinterpret_cast<DLSmem<D>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int cb = blockIdx.x, C = (int)p.C;
    const long long rbeg = (long long)blockIdx.y * rows_per_seg;
    const long long rend = rbeg + rows_per_seg < p.rows ? rbeg + rows_per_seg : p.rows;
    const bf16* x = (const bf16*)p.x;
    const int erow = tid >> 2, eseg = tid & 3;  // 4 threads per row, 16 channels each
    float alv[16];
    {
        const uint4* al = reinterpret_cast<const uint4*>((const bf16*)p.alpha + cb * 64 + eseg * 16);
        float t0[8], t1[8];
        unpack8(al[0], t0); unpack8(al[1], t1);
#pragma unroll
        for (int i = 0; i < 8; ++i) { alv[i] = t0[i]; alv[8 + i] = t1[i]; }
    }
    // warp owns m-tiles {warp, warp+8, ...} of the 4D rows (4D/16 m-tiles), all 8 channel n-tiles
    constexpr int MT = 4 * D / 16;
    constexpr int MPW = (MT + 7) / 8;
    float acc[MPW][8][4] = {};
    for (long long r0 = rbeg; r0 < rend; r0 += 64) {
        const long long grow = r0 + erow;
        {
            const bool live = grow < p.rows;
            const bool first = (grow % p.T) == 0;
            const uint4* a = reinterpret_cast<const uint4*>(x + grow * C + cb * 64 + eseg * 16);
            const uint4* b = reinterpret_cast<const uint4*>(x + (grow - 1) * C + cb * 64 + eseg * 16);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float xv[8], pv[8], uv[8];
                if (live) {
                    unpack8(a[h], xv);
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) xv[i] = 0.f;
                }
                if (first || !live) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) pv[i] = 0.f;
                } else {
                    unpack8(b[h], pv);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) uv[i] = xv[i] + (pv[i] - xv[i]) * alv[h * 8 + i];
                *reinterpret_cast<uint4*>(&sm.uS[erow][eseg * 16 + h * 8]) = pack8(uv);
            }
        }
        for (int i = tid; i < 64 * (4 * D / 8); i += 256) {
            const int r = i / (4 * D / 8), ch = i % (4 * D / 8);
            if (r0 + r >= p.rows) *reinterpret_cast<uint4*>(&sm.dpS[r][ch * 8]) = make_uint4(0, 0, 0, 0);
            else cp_async16(&sm.dpS[r][ch * 8], (const bf16*)p.dpre + (r0 + r) * (4 * D) + ch * 8);
        }
        cp_async_commit();
        cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t b[8][2];
#pragma unroll
            for (int j = 0; j < 8; ++j) ldB_kn_trans(b[j], &sm.uS[0][0], BLD, 8 * j, 16 * ks, lane);
#pragma unroll
            for (int i = 0; i < MPW; ++i) {
                const int mt = warp + 8 * i;
                if (mt < MT) {
                    uint32_t a[4];
                    ldA_km_trans(a, &sm.dpS[0][0], 4 * D + 8, 16 * mt, 16 * ks, lane);
#pragma unroll
                    for (int j = 0; j < 8; ++j) mma_bf16(acc[i][j], a, b[j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < MPW; ++i) {
        const int mt = warp + 8 * i;
        if (mt < MT)
#pragma unroll
            for (int j = 0; j < 8; ++j)
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    float* o = p.dL + (long long)(16 * mt + g + 8 * hrow) * C + cb * 64 + 8 * j + 2 * t4;
                    atomicAdd(o, acc[i][j][2 * hrow]);
                    atomicAdd(o + 1, acc[i][j][2 * hrow + 1]);
                }
    }
}

template <int D> static int launch_ddlerp_bwd_t(const DdlerpBwdParams& p, cudaStream_t stream, void* ws = nullptr, int* status = nullptr) {
    const long long B = p.rows / p.T;
    const int C = (int)p.C;
    if (cudaMemsetAsync(p.dalpha, 0, sizeof(float) * C, stream) != cudaSuccess) return kLaunchFailed;
    if (cudaMemsetAsync(p.dbeta, 0, sizeof(float) * 4 * C, stream) != cudaSuccess) return kLaunchFailed;
    if (cudaMemsetAsync(p.dR, 0, sizeof(float) * 4 * C * D, stream) != cudaSuccess) return kLaunchFailed;
    if (cudaMemsetAsync(p.dL, 0, sizeof(float) * 4 * D * C, stream) != cudaSuccess) return kLaunchFailed;
    if (ws && (D == 16 || D == 32) && launch_ddlerp_prep_bwd(p, ws, stream) != kOk) return kLaunchFailed;
    int dpre_rc = ws ? launch_ddlerp_dpre_tc(p, ws, status, stream) : kBadShape;  // tcgen05 form where it covers the rank
    if (dpre_rc != kOk && dpre_rc != kBadShape) return dpre_rc;
    if (dpre_rc == kBadShape) {
        auto kern = ddlerp_bwd_dpre_kernel<D>;
        const int smem = (int)sizeof(DpreSmem<D>);
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
        kern<<<(unsigned)((p.rows + 31) / 32), 256, smem, stream>>>(p);
        if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    }
    int main_rc = ws ? launch_ddlerp_main_tc(p, ws, status, stream) : kBadShape;  // tcgen05 form where it covers the rank
    if (main_rc != kOk && main_rc != kBadShape) return main_rc;
    if (main_rc == kBadShape) {
        auto kern = ddlerp_bwd_main_kernel<D>;
        const int smem = (int)sizeof(MainSmem<D>);
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
        // Runs per sequence: the count (up to 8) that minimises rounds of resident CTAs x tiles walked per CTA, the
        // extra tile of a run that has a successor included (two CTAs per SM fit).
        static const int slots = [] {
            int dev = 0, sms = 148;
            if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            return 2 * sms;
        }();
        const long long tiles = (p.T + 31) / 32;
        int segs = 1;
        long long best = -1;
        for (int s = 1; s <= 8 && s <= tiles; ++s) {
            const long long tps = (tiles + s - 1) / s;
            if ((s - 1) * tps >= tiles) continue;  // the last run would be empty
            const long long cost = (((long long)(C / 64) * B * s + slots - 1) / slots) * (tps + (s > 1 ? 1 : 0));
            if (best < 0 || cost < best) { best = cost; segs = s; }
        }
        const int tiles_per_seg = (int)((tiles + segs - 1) / segs);
        if (B * segs > 65535) return kTooLarge;
        kern<<<dim3((unsigned)(C / 64), (unsigned)(B * segs)), 256, smem, stream>>>(p, segs, tiles_per_seg);
        if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    }
    if (ws) {  // dL on the tensor cores
        const int rc = launch_ddlerp_dL_tc(p, ws, status, stream, main_rc == kOk);  // the tcgen05 main kernel leaves dalpha to this step
        if (rc != kOk) return rc;
    } else {
        auto kern = ddlerp_bwd_dL_kernel<D>;
        const int smem = (int)sizeof(DLSmem<D>);
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
        // about two CTAs per SM in total; segments are whole 64-row tiles
        long long segs = (2 * 148 + C / 64 - 1) / (C / 64);
        long long tiles = (p.rows + 63) / 64;
        if (segs > tiles) segs = tiles;
        const long long rows_per_seg = ((tiles + segs - 1) / segs) * 64;
        segs = (p.rows + rows_per_seg - 1) / rows_per_seg;
        kern<<<dim3((unsigned)(C / 64), (unsigned)segs), 256, smem, stream>>>(p, rows_per_seg);
        if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    }
    return kOk;
}

int launch_ddlerp_bwd_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream) {
    switch (p.D) {
        case 16: return launch_ddlerp_bwd_t<16>(p, stream, ws, status);
        case 32: return launch_ddlerp_bwd_t<32>(p, stream, ws, status);
        case 64: return launch_ddlerp_bwd_t<64>(p, stream, ws, status);
        default: return kBadShape;
    }
}

int launch_ddlerp_bwd(const DdlerpBwdParams& p, cudaStream_t stream) {
    switch (p.D) {
        case 16: return launch_ddlerp_bwd_t<16>(p, stream);
        case 32: return launch_ddlerp_bwd_t<32>(p, stream);
        case 64: return launch_ddlerp_bwd_t<64>(p, stream);
        default: return kBadShape;
    }
}

}  // namespace wkv7
