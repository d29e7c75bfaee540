// ddlerp forward on the 5th-generation tensor cores (tcgen05 + TMA), bf16.
//
// Replaces fw1_triton_ + fw2_triton_ of the reference (wind_rwkv/rwkv7/rwkv7_ddlerp.py:19-84).  With xx = x_{t-1} - x_t:
//     u   = x + xx * alpha                         m = tanh(u L^T)                y_i = x + xx * (m_i R_i^T + beta_i)
// The token shift is linear, so it moves into the weights and into the coordinates of the tile copies:
//     u L^T = x_t (L (1 - alpha))^T + x_{t-1} (L alpha)^T  =  [x_t | x_{t-1}] [L1 | L2]^T,      y_i = x_t + (x_{t-1} - x_t) z_i.
// Three launches:
//   prep      W12 = [L (1 - alpha) | L alpha]  ([4D, 2C] bf16)  and  R' = R as [C, 4D] (column i D + d = R[i][c][d]): 0.6 MB.
//   gemm1     m = tanh([x_t | x_{t-1}] W12^T): one CTA per 128 tokens of one sequence x 128 columns; the K = 2C loop takes
//             its A blocks from x through ONE 3-D tensor map (channel, time, batch): the second half of the loop reads the
//             same tiles one time step earlier, and the row before a sequence's first token is out of range for the map,
//             i.e. zero.  TMA ring of 3 stages, tcgen05.mma kind::f16 into tensor memory, tanh + bf16 epilogue, bulk stores.
//   lerp      one CTA per 128 tokens x 64 channels: bulk tensor loads of the m tile, the R' tile, the x tile and the x tile
//             one step earlier; four K = D products z_i (tensor-memory columns 64 i ...); the epilogue reads z_i one token row
//             per thread, forms y_i from the two x rows in shared memory and stores four [128 x 64] tiles by bulk tensor
//             stores.  HBM traffic = x once (its re-reads hit L2) + m + the four outputs.
// Every wait on an mbarrier is bounded (mbar_wait_bounded): a wait that runs out sets the CTA's abort flag, reports
// kDeviceTimeout, and the CTA leaves without storing; tensor memory is released in every case.
#include <cuda.h>
#include <cstring>

#include "ddlerp.h"
#include "wkv7_kernels.h"

namespace wkv7 {
namespace dtc {

constexpr int BM = 128, BK = 64;

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t p;
    asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}\n" : "=r"(p));
    return p;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int x, int y, int z) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
                 ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// K-major operand block with 128-byte rows and the 128-byte swizzle: 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// fp32 accumulate, bf16 operands, both K-major, M = 128
__host__ __device__ constexpr uint32_t idesc(int n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24); }
__device__ __forceinline__ void mma_f16(uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d), "l"(a), "l"(b), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t ta, uint32_t* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]),"=r"(v[1]),"=r"(v[2]),"=r"(v[3]),"=r"(v[4]),"=r"(v[5]),"=r"(v[6]),"=r"(v[7]),"=r"(v[8]),"=r"(v[9]),"=r"(v[10]),"=r"(v[11]),"=r"(v[12]),"=r"(v[13]),"=r"(v[14]),"=r"(v[15]) : "r"(ta));
}
__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

// ---- prep: W12 = [L (1 - alpha) | L alpha]  [4D, 2C],  R' [C, 4D] -------------------------------------------------------
__global__ void ddlerp_prep_kernel(const __nv_bfloat16* __restrict__ L, const __nv_bfloat16* __restrict__ alpha, const __nv_bfloat16* __restrict__ R,
                                   __nv_bfloat16* __restrict__ W12, __nv_bfloat16* __restrict__ Rp, int C, int D) {
    const int n4 = 4 * D;
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    const long long nW = (long long)n4 * 2 * C, nR = (long long)C * n4;
    if (i < nW) {
        const int n = (int)(i / (2 * C)), k = (int)(i % (2 * C)), c = k < C ? k : k - C;
        const float l = __bfloat162float(L[(long long)n * C + c]), a = __bfloat162float(alpha[c]);
        W12[i] = __float2bfloat16_rn(k < C ? l * (1.f - a) : l * a);
    } else if (i < nW + nR) {
        const long long j = i - nW;
        const int c = (int)(j / n4), q = (int)(j % n4), s = q / D, d = q % D;
        Rp[j] = R[((long long)s * C + c) * D + d];
    }
}

// ---- gemm1: m = tanh([x_t | x_{t-1}] W12^T) -----------------------------------------------------------------------------
namespace g1 {
constexpr int BN = 128, STAGES = 3;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;  // warps 0-3: epilogue (tensor-memory lane quarters 0-3), warp 4: TMA, warp 5: MMA
struct Ctrl {
    uint64_t full[STAGES], empty[STAGES], accum;
    uint32_t tmem_base;
    volatile int abort;
};
}  // namespace g1

// mapX: x as (channel, time, batch), box 64 x 128 x 1;  mapW: W12 as (k, row), box 64 x 128;  mapM: m as (column, time, batch), box 64 x 32 x 1
__global__ void __launch_bounds__(g1::THREADS) ddlerp_gemm1_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapW,
                                                                  const __grid_constant__ CUtensorMap mapM, int C, int n4, int T, int* status) {
    using namespace g1;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(sm + STAGES * STAGE_BYTES);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int n0 = blockIdx.x * BN, t0 = blockIdx.y * BM, bi = blockIdx.z;
    const int nkh = C / BK, nkb = 2 * nkh;  // the second half of the K loop reads x one time step earlier

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&ctrl->full[s], 1); mbar_init(&ctrl->empty[s], 1); }
        mbar_init(&ctrl->accum, 1);
        ctrl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctrl->tmem_base;

    if (warp == 4) {
        if (elect_one()) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES, round = kb / STAGES;
                if (round > 0) mbar_wait_bounded<true>(&ctrl->empty[s], (round - 1) & 1, &ctrl->abort, status);
                const uint32_t dst = smem_u32(sm + s * STAGE_BYTES);
                mbar_expect(&ctrl->full[s], (uint32_t)STAGE_BYTES);
                const bool prev = kb >= nkh;
                tma_load_3d(dst, &mapX, &ctrl->full[s], (prev ? kb - nkh : kb) * BK, prev ? t0 - 1 : t0, bi);
                tma_load_2d(dst + A_BYTES, &mapW, &ctrl->full[s], kb * BK, n0);
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        if (elect_one()) {
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES, round = kb / STAGES;
                mbar_wait_bounded<false>(&ctrl->full[s], round & 1, &ctrl->abort, status);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = desc_sw128(smem_u32(sm + s * STAGE_BYTES)), db = desc_sw128(smem_u32(sm + s * STAGE_BYTES + A_BYTES));
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks) mma_f16(tmem, da + (uint64_t)(2 * ks), db + (uint64_t)(2 * ks), idesc(BN), (kb > 0 || ks > 0) ? 1u : 0u);
                tc_commit(&ctrl->empty[s]);  // the stage may be refilled once these products have read it
            }
            tc_commit(&ctrl->accum);
        }
        __syncwarp();
    } else {
        // epilogue: warp q owns tensor-memory lanes 32q..32q+31 = tokens t0 + 32q + lane.  The tile leaves through shared
        // memory (the operand stages are free now) as two [128 rows][64 columns] bf16 halves in the 128-byte-swizzled layout.
        mbar_wait_bounded<true>(&ctrl->accum, 0, &ctrl->abort, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool ok = !ctrl->abort;
        const int r = 32 * warp + lane;
#pragma unroll 1
        for (int cb = 0; cb < BN; cb += 16) {
            uint32_t v[16];
            tmem_ld16(tmem + ((uint32_t)(32 * warp) << 16) + cb, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            unsigned char* half = sm + (cb >> 6) * (BM * 128);
#pragma unroll
            for (int c8 = 0; c8 < 16; c8 += 8) {
                uint4 pk;
                pk.x = pack2(tanh_approx(__uint_as_float(v[c8 + 0])), tanh_approx(__uint_as_float(v[c8 + 1])));
                pk.y = pack2(tanh_approx(__uint_as_float(v[c8 + 2])), tanh_approx(__uint_as_float(v[c8 + 3])));
                pk.z = pack2(tanh_approx(__uint_as_float(v[c8 + 4])), tanh_approx(__uint_as_float(v[c8 + 5])));
                pk.w = pack2(tanh_approx(__uint_as_float(v[c8 + 6])), tanh_approx(__uint_as_float(v[c8 + 7])));
                const int piece = ((cb & 63) + c8) >> 3;
                *reinterpret_cast<uint4*>(half + r * 128 + ((piece ^ (r & 7)) << 4)) = pk;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (ok && lane == 0 && t0 + 32 * warp < T) {
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
                if (n0 + 64 * h2 < n4)
                    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                                 ::"l"(&mapM), "r"(n0 + 64 * h2), "r"(t0 + 32 * warp), "r"(bi), "r"(smem_u32(sm + h2 * (BM * 128) + 32 * warp * 128)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory must outlive the stores' reads
        }
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BN) : "memory");
}

// ---- lerp: y_i = x_t + (x_{t-1} - x_t) (m_i R_i^T + beta_i) --------------------------------------------------------------
namespace g2 {
constexpr int BN = 64;            // channels per CTA
constexpr int THREADS = 160;      // warps 0-3: epilogue, warp 4: bulk loads and the products
constexpr int X_BYTES = BM * BN * 2, OUT_BYTES = BM * BN * 2;
struct Ctrl {
    uint64_t ops, xs, accum;      // m and R' tiles landed; the two x tiles landed; products complete
    uint32_t tmem_base;
    volatile int abort;
    float beta[4][BN];
};
// shared memory: [m tile: (4D/64) blocks of 128 rows x 128 B][R' tile: (4D/64) blocks of 64 rows x 128 B] -- reused, once the
// products are complete, by the four output tiles --, then x_t, x_{t-1} (64 channels = 128-byte rows), then Ctrl
__host__ __device__ constexpr int ops_bytes(int D) { return (4 * D / 64) * (BM * 128 + BN * 128); }
__host__ __device__ constexpr int out_region(int D) { return ops_bytes(D) > 4 * OUT_BYTES ? ops_bytes(D) : 4 * OUT_BYTES; }
}  // namespace g2

// mapM: m as (column, time, batch), box 64 x 128 x 1;  mapR: R' as (column, channel), box 64 x 64;
// mapX: x as (channel, time, batch), box 64 x 128 x 1;  mapY: y as (channel, time, batch, stream), box 64 x 32 x 1 x 1
template <int D>
__global__ void __launch_bounds__(g2::THREADS) ddlerp_lerp_kernel(const __grid_constant__ CUtensorMap mapM, const __grid_constant__ CUtensorMap mapR,
                                                                 const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY,
                                                                 const __nv_bfloat16* __restrict__ beta, int C, int T, int* status) {
    using namespace g2;
    constexpr int KB = 4 * D / 64;             // 64-column blocks of the m and R' tiles
    constexpr int NCOLS = 256;                 // tensor-memory columns: z_i at 64 i
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char* smM = sm;
    unsigned char* smR = sm + KB * (BM * 128);
    unsigned char* smX = sm + out_region(D);
    unsigned char* smP = smX + X_BYTES;
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smP + X_BYTES);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int c0 = blockIdx.x * BN, t0 = blockIdx.y * BM, bi = blockIdx.z;

    if (tid == 0) {
        mbar_init(&ctrl->ops, 1); mbar_init(&ctrl->xs, 1); mbar_init(&ctrl->accum, 1);
        ctrl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < 4 * BN; i += THREADS) ctrl->beta[i / BN][i % BN] = __bfloat162float(beta[(long long)(i / BN) * C + c0 + (i % BN)]);
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(NCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctrl->tmem_base;

    if (warp == 4) {
        if (elect_one()) {
            mbar_expect(&ctrl->ops, (uint32_t)ops_bytes(D));
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                tma_load_3d(smem_u32(smM + kb * (BM * 128)), &mapM, &ctrl->ops, kb * 64, t0, bi);
                tma_load_2d(smem_u32(smR + kb * (BN * 128)), &mapR, &ctrl->ops, kb * 64, c0);
            }
            mbar_expect(&ctrl->xs, (uint32_t)(2 * X_BYTES));
            tma_load_3d(smem_u32(smX), &mapX, &ctrl->xs, c0, t0, bi);
            tma_load_3d(smem_u32(smP), &mapX, &ctrl->xs, c0, t0 - 1, bi);  // the row before the sequence's first token is out of range: zeros
            mbar_wait_bounded<false>(&ctrl->ops, 0, &ctrl->abort, status);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // columns i D .. i D + D - 1 of the tiles: block (i D) / 64, byte offset ((i D) % 64) * 2 inside the 128-byte rows
                const int blk = (i * D) / 64, off = ((i * D) % 64) * 2;
                const uint64_t da = desc_sw128(smem_u32(smM + blk * (BM * 128))) + (uint64_t)(off >> 4);
                const uint64_t db = desc_sw128(smem_u32(smR + blk * (BN * 128))) + (uint64_t)(off >> 4);
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) mma_f16(tmem + 64 * i, da + (uint64_t)(2 * ks), db + (uint64_t)(2 * ks), idesc(BN), ks > 0 ? 1u : 0u);
            }
            tc_commit(&ctrl->accum);
        }
        __syncwarp();
    } else {
        // epilogue: thread = token row r of the tile (tensor-memory lane r), 16 channels at a time for all four streams
        const int r = 32 * warp + lane;
        mbar_wait_bounded<true>(&ctrl->xs, 0, &ctrl->abort, status);
        mbar_wait_bounded<true>(&ctrl->accum, 0, &ctrl->abort, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool ok = !ctrl->abort;
#pragma unroll 1
        for (int cc = 0; cc < BN / 16; ++cc) {
            float xv[16], xx[16];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int at = r * 128 + (((2 * cc + h) ^ (r & 7)) << 4);
                float pv[8];
                unpack8(*reinterpret_cast<const uint4*>(smX + at), xv + 8 * h);
                unpack8(*reinterpret_cast<const uint4*>(smP + at), pv);
#pragma unroll
                for (int j = 0; j < 8; ++j) xx[8 * h + j] = pv[j] - xv[8 * h + j];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint32_t v[16];
                tmem_ld16(tmem + ((uint32_t)(32 * warp) << 16) + 64 * i + 16 * cc, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float y[16];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 b = *reinterpret_cast<const float4*>(&ctrl->beta[i][16 * cc + 4 * q]);
                    y[4 * q + 0] = xv[4 * q + 0] + xx[4 * q + 0] * (__uint_as_float(v[4 * q + 0]) + b.x);
                    y[4 * q + 1] = xv[4 * q + 1] + xx[4 * q + 1] * (__uint_as_float(v[4 * q + 1]) + b.y);
                    y[4 * q + 2] = xv[4 * q + 2] + xx[4 * q + 2] * (__uint_as_float(v[4 * q + 2]) + b.z);
                    y[4 * q + 3] = xv[4 * q + 3] + xx[4 * q + 3] * (__uint_as_float(v[4 * q + 3]) + b.w);
                }
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint4 pk;
                    pk.x = pack2(y[8 * h + 0], y[8 * h + 1]); pk.y = pack2(y[8 * h + 2], y[8 * h + 3]);
                    pk.z = pack2(y[8 * h + 4], y[8 * h + 5]); pk.w = pack2(y[8 * h + 6], y[8 * h + 7]);
                    *reinterpret_cast<uint4*>(sm + i * OUT_BYTES + r * 128 + (((2 * cc + h) ^ (r & 7)) << 4)) = pk;
                }
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (ok && lane == 0 && t0 + 32 * warp < T) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
                asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
                             ::"l"(&mapY), "r"(c0), "r"(t0 + 32 * warp), "r"(bi), "r"(i), "r"(smem_u32(sm + i * OUT_BYTES + 32 * warp * 128)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NCOLS) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}
// bf16 tensor of `rank` dimensions (innermost first: extents d[], element strides of dimensions 1.. in st[]), box b[],
// 128-byte swizzle; out-of-range parts of a box read as zeros and are not written
static bool encode(CUtensorMap* m, const void* base, int rank, const long long* d, const long long* st, const int* b) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[4], strides[3];
    cuuint32_t box[4], es[4] = {1, 1, 1, 1};
    for (int i = 0; i < rank; ++i) { dims[i] = (cuuint64_t)d[i]; box[i] = (cuuint32_t)b[i]; }
    for (int i = 0; i + 1 < rank; ++i) strides[i] = (cuuint64_t)st[i] * 2;
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t)rank, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D> static int launch_lerp(const CUtensorMap& mM, const CUtensorMap& mR, const CUtensorMap& mX, const CUtensorMap& mY,
                                       const DdlerpFwdParams& p, long long B, int* status, cudaStream_t stream) {
    auto kern = ddlerp_lerp_kernel<D>;
    const int smem = g2::out_region(D) + 2 * g2::X_BYTES + (int)sizeof(g2::Ctrl) + 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    dim3 grid((unsigned)(p.C / g2::BN), (unsigned)((p.T + BM - 1) / BM), (unsigned)B);
    kern<<<grid, g2::THREADS, smem, stream>>>(mM, mR, mX, mY, (const __nv_bfloat16*)p.beta, (int)p.C, (int)p.T, status);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace dtc

size_t ddlerp_fwd_tc_workspace_bytes(long long C, int D) { return (size_t)(4 * D) * (size_t)(3 * C) * 2; }

int launch_ddlerp_fwd_tc(const DdlerpFwdParams& p, void* ws, int* status, cudaStream_t stream) {
    using namespace dtc;
    if (p.rows == 0) return kOk;
    const long long B = p.rows / p.T, C = p.C, T = p.T;
    const int D = p.D, n4 = 4 * D;
    if (D != 16 && D != 32 && D != 64) return kBadShape;
    if (B > 65535 || (T + BM - 1) / BM > 65535) return kTooLarge;
    __nv_bfloat16* W12 = (__nv_bfloat16*)ws;
    __nv_bfloat16* Rp = W12 + (long long)n4 * 2 * C;
    {
        const long long n = (long long)n4 * 3 * C;
        ddlerp_prep_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)p.L, (const __nv_bfloat16*)p.alpha, (const __nv_bfloat16*)p.R,
                                                                          W12, Rp, (int)C, D);
        if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    }
    alignas(64) CUtensorMap mX, mW, mMs, mMl, mR, mY;
    {
        const long long dx[3] = {C, T, B}, sx[2] = {C, T * C};
        const int bx[3] = {BK, BM, 1};
        const long long dw[2] = {2 * C, n4}, sw[1] = {2 * C};
        const int bw[2] = {BK, g1::BN};
        const long long dm[3] = {n4, T, B}, sm_[2] = {n4, T * n4};
        const int bms[3] = {64, 32, 1}, bml[3] = {64, BM, 1};
        const long long dr[2] = {n4, C}, sr[1] = {n4};
        const int br[2] = {64, g2::BN};
        const long long dy[4] = {C, T, B, 4}, sy[3] = {C, T * C, B * T * C};
        const int by[4] = {g2::BN, 32, 1, 1};
        if (!(encode(&mX, p.x, 3, dx, sx, bx) && encode(&mW, W12, 2, dw, sw, bw) && encode(&mMs, p.m, 3, dm, sm_, bms) &&
              encode(&mMl, p.m, 3, dm, sm_, bml) && encode(&mR, Rp, 2, dr, sr, br) && encode(&mY, p.y, 4, dy, sy, by)))
            return kLaunchFailed;
    }
    {
        const int smem = g1::STAGES * g1::STAGE_BYTES + (int)sizeof(g1::Ctrl) + 1024;
        if (cudaFuncSetAttribute(ddlerp_gemm1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
        dim3 grid((unsigned)((n4 + g1::BN - 1) / g1::BN), (unsigned)((T + BM - 1) / BM), (unsigned)B);
        ddlerp_gemm1_kernel<<<grid, g1::THREADS, smem, stream>>>(mX, mW, mMs, (int)C, n4, (int)T, status);
        if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    }
    switch (D) {
        case 16: return launch_lerp<16>(mMl, mR, mX, mY, p, B, status, stream);
        case 32: return launch_lerp<32>(mMl, mR, mX, mY, p, B, status, stream);
        default: return launch_lerp<64>(mMl, mR, mX, mY, p, B, status, stream);
    }
}

}  // namespace wkv7
