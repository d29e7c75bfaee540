// ddlerp forward for sm_100a: data-dependent token-shift interpolation feeding the RWKV-7 time mixer.
//
// Replaces fw1_triton_ + fw2_triton_ of the reference (wind_rwkv/rwkv7/rwkv7_ddlerp.py:19-84) with ONE
// kernel, so x is read from HBM once:
//     xx = x_{t-1} - x_t  (x_{-1} = 0)          u = x + xx * alpha
//     m  = tanh(u @ L^T)                [rows, 4D]   (stored: the backward needs it)
//     y_k = x + xx * (m_k @ R_k^T + beta_k),  k = 0..3   [4, rows, C]
// One CTA per tile of 64 tokens, 8 warps.  Phase 1 runs the K = C contraction in blocks of 64
// channels (u built in fp32 from coalesced 16-byte loads, rounded to bf16 into shared memory; L
// blocks arrive by cp.async, double buffered).  Phase 2 walks the channel blocks again: the small
// K = D products go to shared memory as fp32, and a coalesced elementwise pass (16 channels per
// thread, 16-byte loads and stores) forms the four outputs.  The second pass over x hits L2.
// HBM-bound: 10*C bytes per token (x in, four y out) plus 8*D for m.
#include "ddlerp.h"
#include "mma_bf16.cuh"

namespace wkv7 {

constexpr int DT = 64;        // tokens per tile
constexpr int DKB = 64;       // channels per block
constexpr int DLD = DKB + 8;  // shared-memory row stride (bf16) of 64-wide tiles
constexpr int ZLD = DKB + 4;  // row stride (floats) of the fp32 staging tile

template <int D> struct DdlerpFwdSmem {
    union {
        struct {
            bf16 uA[2][DT][DLD];
            bf16 LB[2][4 * D][DLD];
        } p1;
        struct {
            bf16 RB[2][2][DKB][D + 8];
            float zS[2][DT][ZLD];
        } p2;
    };
    bf16 mT[DT][4 * D + 8];
};

template <int D>
__global__ void __launch_bounds__(256) ddlerp_fwd_kernel(DdlerpFwdParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sm = *reinterpret_cast<DdlerpFwdSmem<D>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const long long row0 = (long long)blockIdx.x * DT;
    const int C = (int)p.C, nkb = C / DKB;
    const bf16* x = (const bf16*)p.x;

    // elementwise mapping: 4 threads per token row, 16 channels each
    const int erow = tid >> 2, eseg = tid & 3;
    const long long grow = row0 + erow;
    const bool live = grow < p.rows;       // the last tile may be partly empty
    const bool first = (grow % p.T) == 0;  // first token of a sequence: previous token is zero
    const bf16* xrow = x + grow * C + eseg * 16;

    auto load_x = [&](int kb, uint4 (&xr)[2], uint4 (&xp)[2]) {
        if (!live) {
            xr[0] = xr[1] = xp[0] = xp[1] = make_uint4(0, 0, 0, 0);
            return;
        }
        const uint4* a = reinterpret_cast<const uint4*>(xrow + kb * DKB);
        xr[0] = a[0]; xr[1] = a[1];
        if (first) {
            xp[0] = xp[1] = make_uint4(0, 0, 0, 0);
        } else {
            const uint4* b = reinterpret_cast<const uint4*>(xrow - C + kb * DKB);
            xp[0] = b[0]; xp[1] = b[1];
        }
    };
    auto issue_L = [&](int kb, int buf) {
        for (int i = tid; i < 4 * D * (DKB / 8); i += 256) {
            const int r = i / (DKB / 8), ch = i % (DKB / 8);
            cp_async16(&sm.p1.LB[buf][r][ch * 8], (const bf16*)p.L + (long long)r * C + kb * DKB + ch * 8);
        }
        cp_async_commit();
    };

    // ---------------- phase 1: m = tanh(u @ L^T) --------------------------------------------------
    const int wm = warp & 1, wn = warp >> 1;  // 32-row half, stream index
    float acc[2][D / 8][4] = {};
    uint4 xr[2], xp[2];
    load_x(0, xr, xp);
    issue_L(0, 0);
    for (int kb = 0; kb < nkb; ++kb) {
        const int buf = kb & 1;
        {
            const uint4* al = reinterpret_cast<const uint4*>((const bf16*)p.alpha + kb * DKB + eseg * 16);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float xv[8], pv[8], av[8], uv[8];
                unpack8(xr[h], xv); unpack8(xp[h], pv); unpack8(al[h], av);
#pragma unroll
                for (int i = 0; i < 8; ++i) uv[i] = xv[i] + (pv[i] - xv[i]) * av[i];
                *reinterpret_cast<uint4*>(&sm.p1.uA[buf][erow][eseg * 16 + h * 8]) = pack8(uv);
            }
        }
        if (kb + 1 < nkb) {
            load_x(kb + 1, xr, xp);
            issue_L(kb + 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < DKB / 16; ++ks) {
            uint32_t a[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) ldA_mk(a[i], &sm.p1.uA[buf][0][0], DLD, 16 * (2 * wm + i), 16 * ks, g, t4);
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                uint32_t b[2];
                ldB_nk(b, &sm.p1.LB[buf][0][0], DLD, wn * D + 8 * j, 16 * ks, g, t4);
#pragma unroll
                for (int i = 0; i < 2; ++i) mma_bf16(acc[i][j], a[i], b);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            const int r = 16 * (2 * wm + i) + g, col = wn * D + 8 * j + 2 * t4;
            *reinterpret_cast<uint32_t*>(&sm.mT[r][col]) = pack_bf16x2(tanh_f(acc[i][j][0]), tanh_f(acc[i][j][1]));
            *reinterpret_cast<uint32_t*>(&sm.mT[r + 8][col]) = pack_bf16x2(tanh_f(acc[i][j][2]), tanh_f(acc[i][j][3]));
        }
    __syncthreads();  // mT complete; phase-1 buffers free
    if (live) {
        bf16* mo = (bf16*)p.m + grow * (4 * D) + eseg * D;
#pragma unroll
        for (int i = 0; i < D / 8; ++i)
            *reinterpret_cast<uint4*>(mo + 8 * i) = *reinterpret_cast<const uint4*>(&sm.mT[erow][eseg * D + 8 * i]);
    }

    // ---------------- phase 2: y_k = x + xx * (m_k @ R_k^T + beta_k) ------------------------------
    auto issue_R = [&](int cb, int kp, int buf) {
        constexpr int CH = D / 8;  // 16-byte chunks per row
        for (int i = tid; i < 2 * DKB * CH; i += 256) {
            const int kk = i / (DKB * CH), r = (i / CH) % DKB, ch = i % CH;
            cp_async16(&sm.p2.RB[buf][kk][r][ch * 8],
                       (const bf16*)p.R + ((long long)(2 * kp + kk) * C + cb * DKB + r) * D + ch * 8);
        }
        cp_async_commit();
    };
    const int wmt = warp & 3, wkk = warp >> 2;  // m-tile, which stream of the pair
    issue_R(0, 0, 0);
    float xf[16], xxf[16];
    for (int it = 0; it < 2 * nkb; ++it) {
        const int cb = it >> 1, kp = it & 1, buf = it & 1;
        if (kp == 0) {
            load_x(cb, xr, xp);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float xv[8], pv[8];
                unpack8(xr[h], xv); unpack8(xp[h], pv);
#pragma unroll
                for (int i = 0; i < 8; ++i) { xf[h * 8 + i] = xv[i]; xxf[h * 8 + i] = pv[i] - xv[i]; }
            }
        }
        if (it + 1 < 2 * nkb) {
            issue_R((it + 1) >> 1, (it + 1) & 1, buf ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();  // R block landed; previous elementwise pass done with zS
        {
            const int k = 2 * kp + wkk;
            float z[8][4] = {};
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                uint32_t a[4];
                ldA_mk(a, &sm.mT[0][0], 4 * D + 8, 16 * wmt, k * D + 16 * ks, g, t4);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    uint32_t b[2];
                    ldB_nk(b, &sm.p2.RB[buf][wkk][0][0], D + 8, 8 * j, 16 * ks, g, t4);
                    mma_bf16(z[j], a, b);
                }
            }
            const bf16* be = (const bf16*)p.beta + (long long)k * C + cb * DKB;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float2 bt = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(be + 8 * j + 2 * t4));
                *reinterpret_cast<float2*>(&sm.p2.zS[wkk][16 * wmt + g][8 * j + 2 * t4]) = make_float2(z[j][0] + bt.x, z[j][1] + bt.y);
                *reinterpret_cast<float2*>(&sm.p2.zS[wkk][16 * wmt + g + 8][8 * j + 2 * t4]) = make_float2(z[j][2] + bt.x, z[j][3] + bt.y);
            }
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 2 && live; ++kk) {
            bf16* yo = (bf16*)p.y + ((long long)(2 * kp + kk) * p.rows + grow) * C + cb * DKB + eseg * 16;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float4 z0 = *reinterpret_cast<const float4*>(&sm.p2.zS[kk][erow][eseg * 16 + h * 8]);
                const float4 z1 = *reinterpret_cast<const float4*>(&sm.p2.zS[kk][erow][eseg * 16 + h * 8 + 4]);
                const float zz[8] = {z0.x, z0.y, z0.z, z0.w, z1.x, z1.y, z1.z, z1.w};
                float yv[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) yv[i] = xf[h * 8 + i] + xxf[h * 8 + i] * zz[i];
                *reinterpret_cast<uint4*>(yo + h * 8) = pack8(yv);
            }
        }
    }
}

template <int D> static int launch_ddlerp_fwd_t(const DdlerpFwdParams& p, cudaStream_t stream) {
    auto kern = ddlerp_fwd_kernel<D>;
    const int smem = (int)sizeof(DdlerpFwdSmem<D>);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    kern<<<(unsigned)((p.rows + DT - 1) / DT), 256, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int launch_ddlerp_fwd(const DdlerpFwdParams& p, cudaStream_t stream) {
    switch (p.D) {
        case 16: return launch_ddlerp_fwd_t<16>(p, stream);
        case 32: return launch_ddlerp_fwd_t<32>(p, stream);
        case 64: return launch_ddlerp_fwd_t<64>(p, stream);
        default: return kBadShape;
    }
}

}  // namespace wkv7
