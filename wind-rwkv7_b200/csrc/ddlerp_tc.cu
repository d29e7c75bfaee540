// ddlerp forward and backward on the 5th-generation tensor cores (tcgen05 + TMA), bf16.
//
// Forward: replaces fw1_triton_ + fw2_triton_ of the reference (wind_rwkv/rwkv7/rwkv7_ddlerp.py:19-84).  With xx = x_{t-1} - x_t:
//     u   = x + xx * alpha                         m = tanh(u L^T)                y_i = x + xx * (m_i R_i^T + beta_i)
// The token shift is linear, so it moves into the weights and into the coordinates of the tile copies:
//     u L^T = x_t (L (1 - alpha))^T + x_{t-1} (L alpha)^T  =  [x_t | x_{t-1}] [L1 | L2]^T,      y_i = x_t + (x_{t-1} - x_t) z_i.
// Three launches:
//   prep      W12 = [L (1 - alpha) | L alpha]  ([4D, 2C] bf16)  and  R' = R as [C, 4D] (column i D + d = R[i][c][d]): 0.6 MB.
//   gemm1     m = tanh([x_t | x_{t-1}] W12^T): one CTA per 128 tokens of one sequence x 128 columns; the K = 2C loop takes
//             its A blocks from x through ONE 3-D tensor map (channel, time, batch): the second half of the loop reads the
//             same tiles one time step earlier, and the row before a sequence's first token is out of range for the map,
//             i.e. zero.  TMA ring of 3 stages, tcgen05.mma kind::f16 into tensor memory, tanh + bf16 epilogue, bulk stores.
//   lerp      persistent, one CTA per SM over units of 128 tokens x 64 channels: bulk tensor loads of the m tile, the R' tile
//             and a 129-row x tile that starts one token early (two stages: the next unit's loads run under this unit's
//             epilogue); four K = D products z_i into one of two sets of 4 x 64 tensor-memory columns; eight epilogue
//             warps read z_i one token row per thread, form y_i from rows r and r + 1 of the x tile and store [32 x 64]
//             pieces of the four output tiles by bulk tensor stores.  HBM traffic = x once (re-reads hit L2) + m + outputs.
//             Rank 64 (two stages would not fit shared memory) runs the mma.sync forward of ddlerp_fwd.cu instead.
// Backward (replaces bw1..bw4_triton_, rwkv7_ddlerp.py:92-303; ranks 16 and 32, rank 64 runs ddlerp_bwd.cu's kernels), further
// down in this file, each with its own description: the rearranged weights (one small launch), dpre (ddlerp_dpre_tc_kernel),
// the main step dx / dR / dbeta (ddlerp_main_tc_kernel), dW12 = dpre^T [x_t | x_{t-1}] (ddlerp_dw12_kernel) and the step
// that turns it into dL and dalpha (ddlerp_dl_finish_kernel).
// Every wait on an mbarrier is bounded (mbar_wait_bounded): a wait that runs out sets the CTA's abort flag, reports
// kDeviceTimeout, and the CTA leaves without storing; tensor memory is released in every case.
#include <cuda.h>
#include <cstddef>
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
// Abort path: a bounded wait gave up, later waits fall through.  The thread that issued tensor-core products commits them
// to a barrier of its own and waits for it, bounded and regardless of the abort flag, before tensor memory is released.
__device__ __forceinline__ void drain_products(uint64_t* bar, volatile int* never_set, int* status) {
    tc_commit(bar);
    mbar_wait_bounded<false>(bar, 0, never_set, status);
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
    uint64_t full[STAGES], empty[STAGES], accum, drain;
    uint32_t tmem_base;
    volatile int abort, zero;
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
        mbar_init(&ctrl->accum, 1); mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0; ctrl->zero = 0;
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
            if (ctrl->abort) drain_products(&ctrl->drain, &ctrl->zero, status);
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
// Persistent: one CTA per SM walks work units (128 tokens of one sequence) x (64 channels), consecutive CTAs taking the
// channel blocks of the same token tile (its m tile then comes out of L2).  Warp 8 issues the bulk loads of the NEXT unit
// into the other of two shared-memory stages and the current unit's four products into the other of two accumulator
// sets; warps 0-7 are the epilogue (warp w: token rows 32 (w % 4) ..., streams SPW (w / 4) ... SPW (w / 4) + SPW - 1).
namespace g2 {
constexpr int BN = 64;            // channels per unit
constexpr int SPW = 2;           // streams per epilogue warp (1: sixteen epilogue warps; measured equal)
constexpr int EPI_WARPS = 4 * (4 / SPW), THREADS = 32 * (EPI_WARPS + 1);
constexpr int XROWS = BM + 1;     // the x tile starts one token early: row r holds x_{t0 + r - 1}
constexpr int X_BYTES = ((XROWS * 128 + 1023) / 1024) * 1024, OUT_BYTES = BM * BN * 2;
struct Ctrl {
    uint64_t ops[2], xs[2], accum[2];   // per stage: R' tile landed; x tile landed; per accumulator set: products complete
    uint64_t mfull[2];                  // per m buffer: tile landed
    uint64_t stage_free[2], acc_free[2];  // the epilogue warps are done with the stage's x tile / the accumulator set
    uint64_t drain;                     // abort path only
    uint32_t tmem_base;
    volatile int abort, zero;
    alignas(16) float beta[2][4][BN];   // read as float4
};
static_assert(offsetof(Ctrl, beta) % 16 == 0, "beta is read with 16-byte loads");
// shared memory: two m tiles ((4D/64) blocks of 128 rows x 128 B; a token tile's m is loaded once for all of its channel
// blocks that this CTA handles), two stages of [R' tile: (4D/64) blocks of 64 rows x 128 B][x tile], the four output tiles, Ctrl
__host__ __device__ constexpr int m_bytes(int D) { return (4 * D / 64) * (BM * 128); }
__host__ __device__ constexpr int r_bytes(int D) { return (4 * D / 64) * (BN * 128); }
__host__ __device__ constexpr int stage_bytes(int D) { return r_bytes(D) + X_BYTES; }
__host__ __device__ constexpr int smem_bytes(int D) { return 2 * m_bytes(D) + 2 * stage_bytes(D) + 4 * OUT_BYTES + (int)sizeof(Ctrl) + 1024; }
}  // namespace g2

// mapM: m as (column, time, batch), box 64 x 128 x 1;  mapR: R' as (column, channel), box 64 x 64;
// mapX: x as (channel, time, batch), box 64 x 129 x 1;  mapY: y as (channel, time, batch, stream), box 64 x 32 x 1 x 1
template <int D>
__global__ void __launch_bounds__(g2::THREADS, 1) ddlerp_lerp_kernel(const __grid_constant__ CUtensorMap mapM, const __grid_constant__ CUtensorMap mapR,
                                                                    const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY,
                                                                    const __nv_bfloat16* __restrict__ beta, int C, int T, int tiles_per_seq, int units, int* status) {
    using namespace g2;
    constexpr int KB = 4 * D / 64;             // 64-column blocks of the m and R' tiles
    constexpr int NCOLS = 512;                 // two accumulator sets of 4 x 64 columns: z_i at 256 set + 64 i
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    unsigned char* smSt = sm + 2 * m_bytes(D);
    unsigned char* smOut = smSt + 2 * stage_bytes(D);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(smOut + 4 * OUT_BYTES);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int ncb = C / BN;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&ctrl->ops[s], 1); mbar_init(&ctrl->xs[s], 1); mbar_init(&ctrl->accum[s], 1);
            mbar_init(&ctrl->stage_free[s], EPI_WARPS); mbar_init(&ctrl->acc_free[s], EPI_WARPS);
            mbar_init(&ctrl->mfull[s], 1);
        }
        mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0; ctrl->zero = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(NCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctrl->tmem_base;
    // this CTA's units: a contiguous range of the (token tile, channel block) list, channel blocks running fastest
    const int u_lo = (int)((long long)units * blockIdx.x / gridDim.x), nmine = (int)((long long)units * (blockIdx.x + 1) / gridDim.x) - u_lo;

    if (warp == EPI_WARPS) {
        if (elect_one()) {
            int mslot = 1, mtile = -1;   // m buffer and token tile of the unit whose loads were issued last
            auto issue_loads = [&](int n) {
                const int u = u_lo + n, s = n & 1;
                const int cb = u % ncb, tile = u / ncb, t0 = (tile % tiles_per_seq) * BM, bi = tile / tiles_per_seq;
                unsigned char* st = smSt + s * stage_bytes(D);
                if (tile != mtile) {  // the buffer's previous tile was read by products that completed before the stage_free wait
                    mtile = tile; mslot ^= 1;
                    mbar_expect(&ctrl->mfull[mslot], (uint32_t)m_bytes(D));
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb) tma_load_3d(smem_u32(sm + mslot * m_bytes(D) + kb * (BM * 128)), &mapM, &ctrl->mfull[mslot], kb * 64, t0, bi);
                }
                mbar_expect(&ctrl->ops[s], (uint32_t)r_bytes(D));
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) tma_load_2d(smem_u32(st + kb * (BN * 128)), &mapR, &ctrl->ops[s], kb * 64, cb * BN);
                mbar_expect(&ctrl->xs[s], (uint32_t)(XROWS * 128));
                tma_load_3d(smem_u32(st + r_bytes(D)), &mapX, &ctrl->xs[s], cb * BN, t0 - 1, bi);  // the row before the sequence's first token is out of range: zeros
            };
            int cur_slot = 1, waited[2] = {0, 0};  // m buffer of the unit whose products are issued; completed waits per buffer
            if (nmine > 0) issue_loads(0);
            for (int n = 0; n < nmine; ++n) {
                const int s = n & 1;
                const bool tile_first = n == 0 || (u_lo + n - 1) / ncb != (u_lo + n) / ncb;  // buffers alternate from tile to tile, as in issue_loads
                if (tile_first) cur_slot ^= 1;
                if (n + 1 < nmine) {  // the other stage was last used by unit n - 1
                    if (n >= 1) mbar_wait_bounded<true>(&ctrl->stage_free[s ^ 1], ((n - 1) >> 1) & 1, &ctrl->abort, status);
                    issue_loads(n + 1);
                }
                if (tile_first) {  // its m tile must have landed: load number waited + 1 of this buffer
                    mbar_wait_bounded<false>(&ctrl->mfull[cur_slot], waited[cur_slot] & 1, &ctrl->abort, status);
                    ++waited[cur_slot];
                }
                mbar_wait_bounded<false>(&ctrl->ops[s], (n >> 1) & 1, &ctrl->abort, status);
                if (n >= 2) mbar_wait_bounded<true>(&ctrl->acc_free[s], ((n - 2) >> 1) & 1, &ctrl->abort, status);  // set s was last read for unit n - 2
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char* st = smSt + s * stage_bytes(D);
                unsigned char* mt = sm + cur_slot * m_bytes(D);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    // columns i D .. i D + D - 1 of the tiles: block (i D) / 64, byte offset ((i D) % 64) * 2 inside the 128-byte rows
                    const int blk = (i * D) / 64, off = ((i * D) % 64) * 2;
                    const uint64_t da = desc_sw128(smem_u32(mt + blk * (BM * 128))) + (uint64_t)(off >> 4);
                    const uint64_t db = desc_sw128(smem_u32(st + blk * (BN * 128))) + (uint64_t)(off >> 4);
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) mma_f16(tmem + 256 * s + 64 * i, da + (uint64_t)(2 * ks), db + (uint64_t)(2 * ks), idesc(BN), ks > 0 ? 1u : 0u);
                }
                tc_commit(&ctrl->accum[s]);
            }
            if (ctrl->abort) drain_products(&ctrl->drain, &ctrl->zero, status);
        }
        __syncwarp();
    } else {
        const int q = warp & 3, h = warp >> 2;       // lane quarter of tensor memory, stream group
        const int r = 32 * q + lane;                 // token row of the tile
        for (int n = 0; n < nmine; ++n) {
            const int u = u_lo + n, s = n & 1;
            const int cb = u % ncb, tile = u / ncb, t0 = (tile % tiles_per_seq) * BM, bi = tile / tiles_per_seq;
            const unsigned char* smX = smSt + s * stage_bytes(D) + r_bytes(D);
            // this unit's beta values (buffer s): the first warp of a stream group loads the group's SPW x 64 values; the named barrier
            // below publishes them to the pair's four warps.  Buffer s is written again two units later, after every warp of
            // the pair has passed the next unit's barrier, i.e. has finished this unit.
            if (q == 0) {
                for (int i = lane; i < SPW * BN; i += 32)
                    ctrl->beta[s][SPW * h + i / BN][i % BN] = __bfloat162float(beta[(long long)(SPW * h + i / BN) * C + cb * BN + (i % BN)]);
            }
            mbar_wait_bounded<true>(&ctrl->xs[s], (n >> 1) & 1, &ctrl->abort, status);
            mbar_wait_bounded<true>(&ctrl->accum[s], (n >> 1) & 1, &ctrl->abort, status);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the previous unit's stores out of this warp's staging rows must have been read
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            switch (h) {  // the four warps of a stream group: beta visible
                case 0: asm volatile("bar.sync 1, 128;" ::: "memory"); break;
                case 1: asm volatile("bar.sync 2, 128;" ::: "memory"); break;
                case 2: asm volatile("bar.sync 3, 128;" ::: "memory"); break;
                default: asm volatile("bar.sync 4, 128;" ::: "memory"); break;
            }
            const bool ok = !ctrl->abort;
            // both streams' accumulator columns of all four 16-channel groups are requested before the first is used, so
            // that the tensor-memory read latency is paid once per unit
            uint32_t v[SPW][BN / 16][16];
#pragma unroll
            for (int ii = 0; ii < SPW; ++ii)
#pragma unroll
                for (int cc = 0; cc < BN / 16; ++cc) tmem_ld16(tmem + ((uint32_t)(32 * q) << 16) + 256 * s + 64 * (SPW * h + ii) + 16 * cc, v[ii][cc]);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int cc = 0; cc < BN / 16; ++cc) {
                float xv[16], xx[16];
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    float pv[8];
                    unpack8(*reinterpret_cast<const uint4*>(smX + (r + 1) * 128 + (((2 * cc + hh) ^ ((r + 1) & 7)) << 4)), xv + 8 * hh);
                    unpack8(*reinterpret_cast<const uint4*>(smX + r * 128 + (((2 * cc + hh) ^ (r & 7)) << 4)), pv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) xx[8 * hh + j] = pv[j] - xv[8 * hh + j];
                }
#pragma unroll
                for (int ii = 0; ii < SPW; ++ii) {
                    const int i = SPW * h + ii;
                    float y[16];
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) {
                        const float4 b = *reinterpret_cast<const float4*>(&ctrl->beta[s][i][16 * cc + 4 * k4]);
                        y[4 * k4 + 0] = xv[4 * k4 + 0] + xx[4 * k4 + 0] * (__uint_as_float(v[ii][cc][4 * k4 + 0]) + b.x);
                        y[4 * k4 + 1] = xv[4 * k4 + 1] + xx[4 * k4 + 1] * (__uint_as_float(v[ii][cc][4 * k4 + 1]) + b.y);
                        y[4 * k4 + 2] = xv[4 * k4 + 2] + xx[4 * k4 + 2] * (__uint_as_float(v[ii][cc][4 * k4 + 2]) + b.z);
                        y[4 * k4 + 3] = xv[4 * k4 + 3] + xx[4 * k4 + 3] * (__uint_as_float(v[ii][cc][4 * k4 + 3]) + b.w);
                    }
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint4 pk;
                        pk.x = pack2(y[8 * hh + 0], y[8 * hh + 1]); pk.y = pack2(y[8 * hh + 2], y[8 * hh + 3]);
                        pk.z = pack2(y[8 * hh + 4], y[8 * hh + 5]); pk.w = pack2(y[8 * hh + 6], y[8 * hh + 7]);
                        *reinterpret_cast<uint4*>(smOut + i * OUT_BYTES + r * 128 + (((2 * cc + hh) ^ (r & 7)) << 4)) = pk;
                    }
                }
            }
            // the stage's x tile and the accumulator set are free; the staged rows leave by bulk tensor stores
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ctrl->stage_free[s])) : "memory");
                asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ctrl->acc_free[s])) : "memory");
                if (ok && t0 + 32 * q < T) {
#pragma unroll
                    for (int ii = 0; ii < SPW; ++ii)
                        asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
                                     ::"l"(&mapY), "r"(cb * BN), "r"(t0 + 32 * q), "r"(bi), "r"(SPW * h + ii), "r"(smem_u32(smOut + (SPW * h + ii) * OUT_BYTES + 32 * q * 128)) : "memory");
                }
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            __syncwarp();
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory must outlive the stores' reads
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NCOLS) : "memory");
}

// ------------------------------------------------------------------------------------------------------------------------
// dL of the backward on the tensor cores.  With W12 = [L (1 - alpha) | L alpha] (see the forward):
//     dW12 = dpre^T [x_t | x_{t-1}]   ([4D, 2C], contraction over all tokens),      dL = dW1 (1 - alpha) + dW2 alpha.
// Both operands are read as they lie in memory, token-major, i.e. MN-major for a product that contracts over tokens:
// A = dpre^T from [128 tokens][64 columns] boxes of dpre, B = x from [128 tokens][64 channels] boxes of x (the second half
// of the columns one time step earlier, by the copy's coordinate).  One CTA owns 128 rows x 256 columns of dW12 and a
// contiguous range of token tiles; its fp32 accumulator stays in tensor memory over the whole range and is added to global
// memory once (vector reductions): dW1 straight into dL, dW2 into a scratch array; a small kernel then forms dL in place.
namespace g3 {
constexpr int BN = 256, STAGES = 2;
constexpr int A_BYTES = 2 * BM * 128, B_BYTES = (BN / 64) * BM * 128, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;  // warps 0-3: epilogue, warp 4: TMA, warp 5: MMA
struct Ctrl {
    uint64_t full[STAGES], empty[STAGES], accum, drain;
    uint32_t tmem_base;
    volatile int abort, zero;
};
// MN-major operand: [k = token][64 columns] boxes with the 128-byte swizzle; 8 token rows = 1024 bytes (SBO), next 64
// columns = next box of 128 tokens = 16384 bytes (LBO)
__device__ __forceinline__ uint64_t desc_mn(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)(16384 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// fp32 accumulate, bf16 operands, both MN-major, M = 128, N = 256
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}  // namespace g3

// mapD: dpre as (column, time, batch), box 64 x 128 x 1;  mapX: x as (channel, time, batch), box 64 x 128 x 1.
// grid: (column tiles of 256: first the x_t half, then the x_{t-1} half; token splits; row tiles of 128 of the 4D rows)
__global__ void __launch_bounds__(g3::THREADS) ddlerp_dw12_kernel(const __grid_constant__ CUtensorMap mapD, const __grid_constant__ CUtensorMap mapX,
                                                                 float* __restrict__ dW1, float* __restrict__ dW2, int C, int n4, int tiles_per_seq,
                                                                 int total_tiles, int* status) {
    using namespace g3;
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(sm + STAGES * STAGE_BYTES);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int tiles_per_half = (C + BN - 1) / BN;
    const int half = blockIdx.x / tiles_per_half, c0 = (blockIdx.x % tiles_per_half) * BN, m0 = blockIdx.z * BM;
    const int lo = (int)((long long)total_tiles * blockIdx.y / gridDim.y), hi = (int)((long long)total_tiles * (blockIdx.y + 1) / gridDim.y);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&ctrl->full[s], 1); mbar_init(&ctrl->empty[s], 1); }
        mbar_init(&ctrl->accum, 1); mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0; ctrl->zero = 0;
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
            for (int i = lo; i < hi; ++i) {
                const int n = i - lo, s = n % STAGES, round = n / STAGES;
                const int t0 = (i % tiles_per_seq) * BM, bi = i / tiles_per_seq;
                if (round > 0) mbar_wait_bounded<true>(&ctrl->empty[s], (round - 1) & 1, &ctrl->abort, status);
                const uint32_t dst = smem_u32(sm + s * STAGE_BYTES);
                mbar_expect(&ctrl->full[s], (uint32_t)STAGE_BYTES);
#pragma unroll
                for (int b = 0; b < 2; ++b) tma_load_3d(dst + b * (BM * 128), &mapD, &ctrl->full[s], m0 + 64 * b, t0, bi);  // columns beyond 4D: zeros
#pragma unroll
                for (int b = 0; b < BN / 64; ++b) tma_load_3d(dst + A_BYTES + b * (BM * 128), &mapX, &ctrl->full[s], c0 + 64 * b, t0 - half, bi);
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        if (elect_one()) {
            for (int i = lo; i < hi; ++i) {
                const int n = i - lo, s = n % STAGES, round = n / STAGES;
                mbar_wait_bounded<false>(&ctrl->full[s], round & 1, &ctrl->abort, status);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = desc_mn(smem_u32(sm + s * STAGE_BYTES)), db = desc_mn(smem_u32(sm + s * STAGE_BYTES + A_BYTES));
#pragma unroll
                for (int ks = 0; ks < BM / 16; ++ks)  // 16 tokens = two groups of 8 rows = 2048 bytes per step
                    mma_f16(tmem, da + (uint64_t)(ks * (2048 >> 4)), db + (uint64_t)(ks * (2048 >> 4)), IDESC, (n > 0 || ks > 0) ? 1u : 0u);
                tc_commit(&ctrl->empty[s]);
            }
            tc_commit(&ctrl->accum);
            if (ctrl->abort) drain_products(&ctrl->drain, &ctrl->zero, status);
        }
        __syncwarp();
    } else if (hi > lo) {
        // epilogue: lane = row m0 + 32 warp + lane of dW12, 256 columns; added to global memory with 16-byte reductions
        mbar_wait_bounded<true>(&ctrl->accum, 0, &ctrl->abort, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int row = m0 + 32 * warp + lane;
        float* out = (half ? dW2 : dW1) + (long long)row * C + c0;
        const bool ok = !ctrl->abort && row < n4;
#pragma unroll 1
        for (int cb = 0; cb < BN; cb += 16) {
            uint32_t v[16];
            tmem_ld16(tmem + ((uint32_t)(32 * warp) << 16) + cb, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (ok) {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (c0 + cb + 4 * q < C)
                        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(out + cb + 4 * q), "f"(__uint_as_float(v[4 * q])),
                                     "f"(__uint_as_float(v[4 * q + 1])), "f"(__uint_as_float(v[4 * q + 2])), "f"(__uint_as_float(v[4 * q + 3])) : "memory");
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BN) : "memory");
}

// dL = dW1 (1 - alpha) + dW2 alpha, in place (dL holds dW1 on entry); a thread takes 8 rows of one channel.  With dalpha !=
// nullptr (zero on entry) also dalpha[c] += sum_n L[n, c] (dW2 - dW1)[n, c]  ( = sum_t (dpre L)[t, c] (x_{t-1} - x_t)[c] ).
__global__ void ddlerp_dl_finish_kernel(float* __restrict__ dL, const float* __restrict__ dW2, const __nv_bfloat16* __restrict__ alpha,
                                        const __nv_bfloat16* __restrict__ L, float* __restrict__ dalpha, int C, int n4) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x, n0 = blockIdx.y * 8;
    if (c >= C) return;
    const float a = __bfloat162float(alpha[c]);
    // (4D is a multiple of 8: every thread has its 8 rows; all loads are issued before the first use)
    float w1[8], w2[8], lv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const long long i = (long long)(n0 + j) * C + c;
        w1[j] = dL[i]; w2[j] = dW2[i]; lv[j] = __bfloat162float(L[i]);
    }
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        dL[(long long)(n0 + j) * C + c] = w1[j] * (1.f - a) + w2[j] * a;
        acc += lv[j] * (w2[j] - w1[j]);
    }
    if (dalpha) atomicAdd(dalpha + c, acc);
}

// ------------------------------------------------------------------------------------------------------------------------
// dpre of the backward on the tensor cores:  dm_k = (dy_k * (x_{t-1} - x_t)) R_k  (contraction over all C channels),
// dpre = dm * (1 - m^2).  One CTA per 128 tokens of one sequence, 64 channels per step through two stages: bulk tensor
// loads bring the four dy tiles, a 129-row x tile and the block of R^T; four warps turn the dy tiles into dz = dy * xx IN
// PLACE (eight warps: one token row per thread and two streams per warp; the tiles keep the swizzled K-major layout the copy
// gave them, so they are the A operands as they stand); one thread issues, per stream k, the K = 64 products into
// tensor-memory columns k D ...; at the end the same warps read dm, apply the tanh derivative from m and store dpre.
namespace g4 {
constexpr int STAGES = 2, THREADS = 320;  // warps 0-7: transform + epilogue (row quarter w % 4, stream pair w / 4), warp 8: TMA, warp 9: MMA
constexpr int X_BYTES = ((BM + 1) * 128 + 1023) / 1024 * 1024, DY_BYTES = BM * 128;
struct Ctrl {
    uint64_t full[STAGES], ready[STAGES], empty[STAGES], accum, drain;
    uint32_t tmem_base;
    volatile int abort, zero;
};
__host__ __device__ constexpr int rt_bytes(int D) { return 4 * D * 128; }           // [4D rows][64 channels] bf16
__host__ __device__ constexpr int stage_bytes(int D) { return 4 * DY_BYTES + X_BYTES + (rt_bytes(D) + 1023) / 1024 * 1024; }
}  // namespace g4

// The backward's rearranged weights, one launch: R^T as [4D, C] (row k D + d = R[k][:, d]), L^T as [C, 4D], and R' as [C, 4D]
// (column k D + d = R[k][c][d])
__global__ void ddlerp_prep_bwd_kernel(const __nv_bfloat16* __restrict__ L, const __nv_bfloat16* __restrict__ R, __nv_bfloat16* __restrict__ Rt,
                                       __nv_bfloat16* __restrict__ Lt, __nv_bfloat16* __restrict__ Rp, int C, int D) {
    const int n4 = 4 * D;
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= (long long)C * n4) return;
    {
        const int n = (int)(i / C), c = (int)(i % C);
        Rt[i] = R[((long long)(n / D) * C + c) * D + (n % D)];
    }
    {
        const int c = (int)(i / n4), n = (int)(i % n4);
        Lt[i] = L[(long long)n * C + c];
        Rp[i] = R[((long long)(n / D) * C + c) * D + (n % D)];
    }
}

// mapY: the four dy as (channel, time, batch) each (four maps), box 64 x 128 x 1;  mapX: x, box 64 x 129 x 1;
// mapRt: R^T as (channel, row), box 64 x 4D;  mapP: dpre as (column, time, batch), box 64 x 32 x 1
struct DyMaps { CUtensorMap m[4]; };
template <int D>
__global__ void __launch_bounds__(g4::THREADS, 1) ddlerp_dpre_tc_kernel(const __grid_constant__ DyMaps mapY, const __grid_constant__ CUtensorMap mapX,
                                                                       const __grid_constant__ CUtensorMap mapRt, const __grid_constant__ CUtensorMap mapP,
                                                                       const __nv_bfloat16* __restrict__ m, int C, int T, int* status) {
    using namespace g4;
    constexpr int N4 = 4 * D;
    static_assert(N4 <= 128, "one accumulator of 4D columns and one 128-row block of R^T per stage");
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(sm + STAGES * stage_bytes(D));
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int t0 = blockIdx.x * BM, bi = blockIdx.y;
    const int ncb = C / 64;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&ctrl->full[s], 1); mbar_init(&ctrl->ready[s], 8); mbar_init(&ctrl->empty[s], 1); }
        mbar_init(&ctrl->accum, 1); mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0; ctrl->zero = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(128) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctrl->tmem_base;

    if (warp == 8) {
        if (elect_one()) {
            for (int cb = 0; cb < ncb; ++cb) {
                const int s = cb % STAGES, round = cb / STAGES;
                if (round > 0) mbar_wait_bounded<true>(&ctrl->empty[s], (round - 1) & 1, &ctrl->abort, status);
                const uint32_t dst = smem_u32(sm + s * stage_bytes(D));
                mbar_expect(&ctrl->full[s], (uint32_t)(4 * DY_BYTES + (BM + 1) * 128 + rt_bytes(D)));
#pragma unroll
                for (int k = 0; k < 4; ++k) tma_load_3d(dst + k * DY_BYTES, &mapY.m[k], &ctrl->full[s], cb * 64, t0, bi);
                tma_load_3d(dst + 4 * DY_BYTES, &mapX, &ctrl->full[s], cb * 64, t0 - 1, bi);   // row r: x_{t0 + r - 1}; before the sequence: zeros
                tma_load_2d(dst + 4 * DY_BYTES + X_BYTES, &mapRt, &ctrl->full[s], cb * 64, 0);
            }
        }
        __syncwarp();
    } else if (warp == 9) {
        if (elect_one()) {
            for (int cb = 0; cb < ncb; ++cb) {
                const int s = cb % STAGES, round = cb / STAGES;
                mbar_wait_bounded<false>(&ctrl->ready[s], round & 1, &ctrl->abort, status);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t st = smem_u32(sm + s * stage_bytes(D));
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint64_t da = desc_sw128(st + k * DY_BYTES), db = desc_sw128(st + 4 * DY_BYTES + X_BYTES + k * D * 128);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) mma_f16(tmem + k * D, da + (uint64_t)(2 * ks), db + (uint64_t)(2 * ks), idesc(D), (cb > 0 || ks > 0) ? 1u : 0u);
                }
                tc_commit(&ctrl->empty[s]);
            }
            tc_commit(&ctrl->accum);
            if (ctrl->abort) drain_products(&ctrl->drain, &ctrl->zero, status);
        }
        __syncwarp();
    } else {
        const int q = warp & 3, g = warp >> 2;  // row quarter (= tensor-memory lane quarter), stream pair
        const int r = 32 * q + lane;     // token row of the tile = tensor-memory lane
        for (int cb = 0; cb < ncb; ++cb) {
            const int s = cb % STAGES, round = cb / STAGES;
            mbar_wait_bounded<true>(&ctrl->full[s], round & 1, &ctrl->abort, status);
            unsigned char* st = sm + s * stage_bytes(D);
            const unsigned char* xs = st + 4 * DY_BYTES;
#pragma unroll 2
            for (int pc = 0; pc < 8; ++pc) {  // 16-byte pieces of the 64-channel rows
                float xv[8], pv[8];
                unpack8(*reinterpret_cast<const uint4*>(xs + (r + 1) * 128 + ((pc ^ ((r + 1) & 7)) << 4)), xv);
                unpack8(*reinterpret_cast<const uint4*>(xs + r * 128 + ((pc ^ (r & 7)) << 4)), pv);
#pragma unroll
                for (int j = 0; j < 8; ++j) pv[j] -= xv[j];
#pragma unroll
                for (int k = 2 * g; k < 2 * g + 2; ++k) {
                    uint4* cell = reinterpret_cast<uint4*>(st + k * DY_BYTES + r * 128 + ((pc ^ (r & 7)) << 4));
                    float dv[8];
                    unpack8(*cell, dv);
                    uint4 o;
                    o.x = pack2(dv[0] * pv[0], dv[1] * pv[1]); o.y = pack2(dv[2] * pv[2], dv[3] * pv[3]);
                    o.z = pack2(dv[4] * pv[4], dv[5] * pv[5]); o.w = pack2(dv[6] * pv[6], dv[7] * pv[7]);
                    *cell = o;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads what these threads wrote
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ctrl->ready[s])) : "memory");
        }
        // epilogue: dpre = dm (1 - m^2), staged as [128 rows][64 columns] bf16 blocks (swizzled) in stage 0, stored by bulk tensor stores
        mbar_wait_bounded<true>(&ctrl->accum, 0, &ctrl->abort, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const bool ok = !ctrl->abort;
        const bool live = t0 + r < T;
        const __nv_bfloat16* mrow = m + ((long long)bi * T + (live ? t0 + r : 0)) * N4;
        // columns of this warp: with 4D = 128 the stream pair's 64; with 4D = 64 the first group takes all, the second none
        const int col0 = N4 == 128 ? 64 * g : 0, col1 = N4 == 128 ? 64 * g + 64 : (g == 0 ? N4 : 0);
#pragma unroll 1
        for (int cbk = col0; cbk < col1; cbk += 16) {
            uint32_t v[16];
            tmem_ld16(tmem + ((uint32_t)(32 * q) << 16) + cbk, v);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float mv[8];
                unpack8(live ? *reinterpret_cast<const uint4*>(mrow + cbk + 8 * h) : make_uint4(0, 0, 0, 0), mv);
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) o[j] = __uint_as_float(v[8 * h + j]) * (1.f - mv[j] * mv[j]);
                uint4 pk;
                pk.x = pack2(o[0], o[1]); pk.y = pack2(o[2], o[3]); pk.z = pack2(o[4], o[5]); pk.w = pack2(o[6], o[7]);
                const int piece = ((cbk & 63) >> 3) + h;
                *reinterpret_cast<uint4*>(sm + (cbk >> 6) * (BM * 128) + r * 128 + ((piece ^ (r & 7)) << 4)) = pk;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (ok && lane == 0 && t0 + 32 * q < T && col1 > col0) {
            const int h2 = col0 >> 6;
            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                         ::"l"(&mapP), "r"(64 * h2), "r"(t0 + 32 * q), "r"(bi), "r"(smem_u32(sm + h2 * (BM * 128) + 32 * q * 128)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(128) : "memory");
}

// ------------------------------------------------------------------------------------------------------------------------
// The rest of the backward on the tensor cores, per (128 tokens of one sequence) x (64 channels):
//     du  = dpre L[:, cb]                 z_k = m_k R_k[cb]^T                      (products 1: contraction over 4D / D)
//     X   = du alpha + sum_k dy_k (z_k + beta_k)        Dd = du + sum_k dy_k        dz_k = dy_k (x_{t-1} - x_t)
//     dx_t = Dd_t - X_t + X_{t+1}
//     dR_k[cb] += dz_k^T m_k              dbeta_k[cb] += dz_k^T 1                  (products 2: contraction over tokens)
// Persistent: one CTA per SM walks a contiguous range of the unit list (channel blocks slowest), so the token-contracted
// accumulators stay in tensor memory until the channel block changes.  Per unit: bulk tensor loads of the dpre, m, dy_k and
// x tiles (and, when the channel block changes, of its blocks of L^T and R'); products 1 into tensor-memory columns 0..319;
// sixteen epilogue warps (row quarter x channel quarter) read them one token row per thread, form X, Dd, write dz_k IN PLACE into
// the dy tiles (which then are, as they lie, the MN-major A operands of products 2) and dx into a staging tile for a bulk
// tensor store; X_{t+1} comes from the next lane, across warps through shared memory, and for the tile's last row from a
// halo row computed on the CUDA cores out of the weight tiles in shared memory (one row of du and z_k: 16K multiply-adds),
// so units are independent of each other.
namespace g5 {
constexpr int EPI_WARPS = 16, THREADS = 32 * (EPI_WARPS + 2);  // warps 0-15: epilogue (row quarter w % 4, channel quarter w / 4), warp 16: TMA, warp 17: MMA
constexpr int CPT = 64 / (EPI_WARPS / 4);   // channels per epilogue thread
constexpr int TILE = BM * 128;                               // a [128 rows][64 columns] bf16 block
constexpr int X_BYTES = ((BM + 1) * 128 + 1023) / 1024 * 1024;
struct Ctrl {
    uint64_t full, full_a, full_x, wfull, acc1, dz_ready, unit_free, flushed, drain;   // full: m and dy tiles; full_a: dpre tile; full_x: x tile
    uint32_t tmem_base;
    volatile int abort, zero;
    alignas(16) float alpha[64], beta[4][64], halo[64], edge[4][64];
};
// shared memory: dpre tile, m tile (KB blocks each), four dy tiles, x tile, L^T block, R' block (KB blocks of 64 rows each),
// a tile of ones, the dx staging tile, Ctrl
__host__ __device__ constexpr int kb_of(int D) { return 4 * D / 64; }
__host__ __device__ constexpr int off_m(int D) { return kb_of(D) * TILE; }
__host__ __device__ constexpr int off_dy(int D) { return 2 * kb_of(D) * TILE; }
__host__ __device__ constexpr int off_x(int D) { return off_dy(D) + 4 * TILE; }
__host__ __device__ constexpr int off_lt(int D) { return off_x(D) + X_BYTES; }
__host__ __device__ constexpr int off_rp(int D) { return off_lt(D) + kb_of(D) * 64 * 128; }
__host__ __device__ constexpr int off_ones(int D) { return off_rp(D) + kb_of(D) * 64 * 128; }
__host__ __device__ constexpr int off_dx(int D) { return off_ones(D) + TILE; }
__host__ __device__ constexpr int off_ctrl(int D) { return off_dx(D) + TILE; }
// tensor-memory columns: du 0..63, z_k 64 + 64 k, dR_k 320 + D k, dbeta_k 320 + 4D + 8 k
constexpr int C_DU = 0, C_Z = 64, C_DR = 320;
// MN-major operand out of [token][64 columns] tiles with the 128-byte swizzle (see g3::desc_mn); M = 64
__device__ __forceinline__ uint64_t desc_mn(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)(16384 >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__host__ __device__ constexpr uint32_t idesc_mn64(int n) {  // fp32 accumulate, bf16 operands, both MN-major, M = 64
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t)(n >> 3) << 17) | (4u << 24);
}
}  // namespace g5

struct MainMaps { CUtensorMap dy[4], x, dpre, m, lt, rp, dx; };
// maps: dy_k, x as (channel, time, batch), boxes 64 x 128 x 1 and 64 x 129 x 1; dpre, m as (column, time, batch), box 64 x 128 x 1;
// lt, rp as (column, channel), box 64 x 64; dx as (channel, time, batch), box 64 x 32 x 1
template <int D>
__global__ void __launch_bounds__(g5::THREADS, 1) ddlerp_main_tc_kernel(const __grid_constant__ MainMaps maps, const __nv_bfloat16* __restrict__ dyp0,
                                                                       const __nv_bfloat16* __restrict__ dyp1, const __nv_bfloat16* __restrict__ dyp2,
                                                                       const __nv_bfloat16* __restrict__ dyp3, const __nv_bfloat16* __restrict__ dpre,
                                                                       const __nv_bfloat16* __restrict__ mten, const __nv_bfloat16* __restrict__ alpha,
                                                                       const __nv_bfloat16* __restrict__ beta, float* __restrict__ dR,
                                                                       float* __restrict__ dbeta, int C, int T, int tiles_per_seq, int tiles, int units,
                                                                       int* status) {
    using namespace g5;
    constexpr int KB = 4 * D / 64, N4 = 4 * D;
    constexpr int C_DB = C_DR + N4;
    static_assert(C_DB + 32 <= 512, "tensor-memory columns");
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(sm + off_ctrl(D));
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int u_lo = (int)((long long)units * blockIdx.x / gridDim.x), nmine = (int)((long long)units * (blockIdx.x + 1) / gridDim.x) - u_lo;
    // unit u: channel block u / tiles, token tile u % tiles (tile -> sequence tile / tiles_per_seq, first token (tile % tiles_per_seq) * 128)

    if (tid == 0) {
        mbar_init(&ctrl->full, 1); mbar_init(&ctrl->full_a, 1); mbar_init(&ctrl->full_x, 1); mbar_init(&ctrl->wfull, 1); mbar_init(&ctrl->acc1, 1); mbar_init(&ctrl->dz_ready, EPI_WARPS);
        mbar_init(&ctrl->unit_free, 1); mbar_init(&ctrl->flushed, EPI_WARPS); mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0; ctrl->zero = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = tid; i < TILE / 4; i += THREADS) reinterpret_cast<uint32_t*>(sm + off_ones(D))[i] = 0x3f803f80u;  // bf16 1.0 pairs
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) {
        __syncwarp();
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctrl->tmem_base;
    const uint32_t sb = smem_u32(sm);

    if (warp == EPI_WARPS) {
        if (elect_one()) {
            int cb_prev = -1, nw = 0;
            // The dpre tile is only read by products 1 and the x tile only by the epilogue's first phase: the next unit's copies
            // of the two are requested as soon as those are done, ahead of the m and dy tiles, which products 2 still read.
            auto load_dpre = [&](int n) {
                const int tile = (u_lo + n) % tiles, t0 = (tile % tiles_per_seq) * BM, bi = tile / tiles_per_seq;
                mbar_expect(&ctrl->full_a, (uint32_t)(KB * TILE));
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) tma_load_3d(sb + kb * TILE, &maps.dpre, &ctrl->full_a, kb * 64, t0, bi);
            };
            auto load_x = [&](int n) {
                const int u = u_lo + n, cb = u / tiles, tile = u % tiles, t0 = (tile % tiles_per_seq) * BM, bi = tile / tiles_per_seq;
                mbar_expect(&ctrl->full_x, (uint32_t)((BM + 1) * 128));
                tma_load_3d(sb + off_x(D), &maps.x, &ctrl->full_x, cb * 64, t0 - 1, bi);
            };
            if (nmine > 0) { load_dpre(0); load_x(0); }
            for (int n = 0; n < nmine; ++n) {
                const int u = u_lo + n, cb = u / tiles, tile = u % tiles, t0 = (tile % tiles_per_seq) * BM, bi = tile / tiles_per_seq;
                if (n > 0) mbar_wait_bounded<true>(&ctrl->unit_free, (n - 1) & 1, &ctrl->abort, status);  // products 2 of the previous unit have read the tiles
                if (cb != cb_prev) {
                    // the weights may be replaced as soon as the previous unit's products are complete (unit_free)
                    cb_prev = cb; ++nw;
                    mbar_expect(&ctrl->wfull, (uint32_t)(2 * KB * 64 * 128));
#pragma unroll
                    for (int kb = 0; kb < KB; ++kb) {
                        tma_load_2d(sb + off_lt(D) + kb * 64 * 128, &maps.lt, &ctrl->wfull, kb * 64, cb * 64);
                        tma_load_2d(sb + off_rp(D) + kb * 64 * 128, &maps.rp, &ctrl->wfull, kb * 64, cb * 64);
                    }
                }
                mbar_expect(&ctrl->full, (uint32_t)(KB * TILE + 4 * TILE));
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) tma_load_3d(sb + off_m(D) + kb * TILE, &maps.m, &ctrl->full, kb * 64, t0, bi);
#pragma unroll
                for (int k = 0; k < 4; ++k) tma_load_3d(sb + off_dy(D) + k * TILE, &maps.dy[k], &ctrl->full, cb * 64, t0, bi);
                if (n + 1 < nmine) {
                    mbar_wait_bounded<true>(&ctrl->acc1, n & 1, &ctrl->abort, status);       // products 1 of this unit have read the dpre tile
                    load_dpre(n + 1);
                    mbar_wait_bounded<true>(&ctrl->dz_ready, n & 1, &ctrl->abort, status);   // every epilogue warp is past the x tile
                    load_x(n + 1);
                }
            }
            (void)nw;
        }
        __syncwarp();
    } else if (warp == EPI_WARPS + 1) {
        if (elect_one()) {
            int cb_prev = -1, nw = 0, nflush = 0;
            for (int n = 0; n < nmine; ++n) {
                const int u = u_lo + n, cb = u / tiles;
                const bool newcb = cb != cb_prev;
                if (newcb) {
                    cb_prev = cb;
                    mbar_wait_bounded<false>(&ctrl->wfull, nw & 1, &ctrl->abort, status);
                    ++nw;
                }
                mbar_wait_bounded<false>(&ctrl->full_a, n & 1, &ctrl->abort, status);
                mbar_wait_bounded<false>(&ctrl->full, n & 1, &ctrl->abort, status);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // products 1: du = dpre L^T-block^T (K = 4D), z_k = m_k R'_k^T (K = D)
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    const uint64_t da = desc_sw128(sb + kb * TILE), db = desc_sw128(sb + off_lt(D) + kb * 64 * 128);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks) mma_f16(tmem + C_DU, da + (uint64_t)(2 * ks), db + (uint64_t)(2 * ks), idesc(64), (kb > 0 || ks > 0) ? 1u : 0u);
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int blk = (k * D) / 64, off = ((k * D) % 64) * 2;
                    const uint64_t da = desc_sw128(sb + off_m(D) + blk * TILE) + (uint64_t)(off >> 4);
                    const uint64_t db = desc_sw128(sb + off_rp(D) + blk * 64 * 128) + (uint64_t)(off >> 4);
#pragma unroll
                    for (int ks = 0; ks < D / 16; ++ks) mma_f16(tmem + C_Z + 64 * k, da + (uint64_t)(2 * ks), db + (uint64_t)(2 * ks), idesc(64), ks > 0 ? 1u : 0u);
                }
                tc_commit(&ctrl->acc1);
                // products 2, once the epilogue has turned dy into dz: dR_k += dz_k^T m_k, dbeta_k += dz_k^T 1 (contraction over the 128 tokens)
                mbar_wait_bounded<false>(&ctrl->dz_ready, n & 1, &ctrl->abort, status);
                if (newcb && n > 0) {  // the accumulators still hold the previous channel block until the epilogue warps have flushed them
                    mbar_wait_bounded<false>(&ctrl->flushed, nflush & 1, &ctrl->abort, status);
                    ++nflush;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int blk = (k * D) / 64, off = ((k * D) % 64) * 2;
                    const uint64_t da = desc_mn(sb + off_dy(D) + k * TILE);
                    const uint64_t dbm = desc_mn(sb + off_m(D) + blk * TILE) + (uint64_t)(off >> 4), dbo = desc_mn(sb + off_ones(D));
#pragma unroll
                    for (int ks = 0; ks < BM / 16; ++ks) {
                        const uint32_t acc = (!newcb || ks > 0) ? 1u : 0u;
                        mma_f16(tmem + C_DR + D * k, da + (uint64_t)(ks * 128), dbm + (uint64_t)(ks * 128), idesc_mn64(D), acc);
                        mma_f16(tmem + C_DB + 8 * k, da + (uint64_t)(ks * 128), dbo + (uint64_t)(ks * 128), idesc_mn64(8), acc);
                    }
                }
                tc_commit(&ctrl->unit_free);
            }
            if (ctrl->abort) drain_products(&ctrl->drain, &ctrl->zero, status);
        }
        __syncwarp();
    } else {
        const int q = warp & 3, g = warp >> 2;   // row quarter (= tensor-memory lane quarter), channel group
        const int r = 32 * q + lane, ch0 = CPT * g;
        const int et = tid;                       // 0..32 EPI_WARPS - 1 among the epilogue warps
        const __nv_bfloat16* dyp[4] = {dyp0, dyp1, dyp2, dyp3};
        const uint32_t tlane = tmem + ((uint32_t)(32 * q) << 16);
        // token-contracted accumulators of channel block cbf -> global memory (vector reductions); the M = 64 products keep
        // channel c in tensor-memory lane 32 (c / 16) + c % 16
        auto flush = [&](int cbf) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (g == 0) {
                const int c = cbf * 64 + 16 * q + (lane & 15);
#pragma unroll
                for (int k = 0; k < 4; ++k)
#pragma unroll
                    for (int d0 = 0; d0 < D; d0 += 16) {
                        uint32_t v[16];
                        tmem_ld16(tlane + C_DR + D * k + d0, v);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (lane < 16) {
                            float* o = dR + ((long long)k * C + c) * D + d0;
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj)
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o + 4 * jj), "f"(__uint_as_float(v[4 * jj])), "f"(__uint_as_float(v[4 * jj + 1])),
                                             "f"(__uint_as_float(v[4 * jj + 2])), "f"(__uint_as_float(v[4 * jj + 3])) : "memory");
                        }
                    }
                uint32_t v0[16], v1[16];   // dbeta_k in column C_DB + 8 k
                tmem_ld16(tlane + C_DB, v0);
                tmem_ld16(tlane + C_DB + 16, v1);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (lane < 16) {
                    atomicAdd(dbeta + c, __uint_as_float(v0[0]));
                    atomicAdd(dbeta + (long long)C + c, __uint_as_float(v0[8]));
                    atomicAdd(dbeta + 2LL * C + c, __uint_as_float(v1[0]));
                    atomicAdd(dbeta + 3LL * C + c, __uint_as_float(v1[8]));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ctrl->flushed)) : "memory");
        };
        if (et < 64) ctrl->halo[et] = 0.f;
        int cb_prev = -1, nwf = 0;
        for (int n = 0; n < nmine; ++n) {
            const int u = u_lo + n, cb = u / tiles, tile = u % tiles, t0 = (tile % tiles_per_seq) * BM, bi = tile / tiles_per_seq;
            if (cb != cb_prev) {
                if (n > 0) {  // the previous channel block's sums are complete once the previous unit's products 2 are
                    mbar_wait_bounded<true>(&ctrl->unit_free, (n - 1) & 1, &ctrl->abort, status);
                    flush(cb_prev);
                }
                cb_prev = cb;
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");  // every epilogue warp has finished the previous unit
                if (et < 64) ctrl->alpha[et] = __bfloat162float(alpha[cb * 64 + et]);
                if (et < 256) ctrl->beta[et >> 6][et & 63] = __bfloat162float(beta[(long long)(et >> 6) * C + cb * 64 + (et & 63)]);
                asm volatile("bar.sync 1, %0;" ::"n"(32 * EPI_WARPS) : "memory");  // alpha and beta of this channel block are in place
                mbar_wait_bounded<true>(&ctrl->wfull, nwf & 1, &ctrl->abort, status);   // and its weight tiles (read for the halo row)
                ++nwf;
            }
            // ---- halo: X of the token after this tile (zero past the sequence's end), accumulated with shared-memory atomics.
            // Thread = (channel c, quarter of the contraction = stream k): D rows of L^T for du, the D ranks of R' for z_k, both
            // read out of the swizzled weight tiles in shared memory (16-byte pieces; lanes are consecutive channels).
            if (t0 + BM < T && et < 256) {
                const long long hrow = (long long)bi * T + t0 + BM;
                const int c = et & 63, k = et >> 6, n0 = k * D;
                const unsigned char* lt = sm + off_lt(D) + (n0 >> 6) * 64 * 128 + c * 128;
                const unsigned char* rp = sm + off_rp(D) + (n0 >> 6) * 64 * 128 + c * 128;
                float du = 0.f, z = 0.f;
#pragma unroll
                for (int pc8 = 0; pc8 < D / 8; ++pc8) {
                    const int slot = ((((n0 & 63) >> 3) + pc8) ^ (c & 7)) << 4;
                    float lv[8], rv[8], dp[8], mv[8];
                    unpack8(*reinterpret_cast<const uint4*>(lt + slot), lv);
                    unpack8(*reinterpret_cast<const uint4*>(rp + slot), rv);
                    unpack8(*reinterpret_cast<const uint4*>(dpre + hrow * N4 + n0 + 8 * pc8), dp);
                    unpack8(*reinterpret_cast<const uint4*>(mten + hrow * N4 + n0 + 8 * pc8), mv);
#pragma unroll
                    for (int j = 0; j < 8; ++j) { du += dp[j] * lv[j]; z += mv[j] * rv[j]; }
                }
                const float dyh = __bfloat162float(dyp[k][hrow * C + cb * 64 + c]);
                atomicAdd(&ctrl->halo[c], du * ctrl->alpha[c] + dyh * (z + ctrl->beta[k][c]));
            }
            // ---- X, Dd and dz for this thread's row and 32 channels ---------------------------------------------------
            mbar_wait_bounded<true>(&ctrl->full_x, n & 1, &ctrl->abort, status);
            mbar_wait_bounded<true>(&ctrl->full, n & 1, &ctrl->abort, status);
            mbar_wait_bounded<true>(&ctrl->acc1, n & 1, &ctrl->abort, status);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool ok = !ctrl->abort;
            float X[CPT], Dd[CPT];
            const unsigned char* xs = sm + off_x(D);
#pragma unroll
            for (int cc = 0; cc < CPT / 16; ++cc) {
                float pvs[16];   // x_{t-1} - x_t of these 16 channels
                {
                    uint32_t du[16];
                    tmem_ld16(tlane + C_DU + ch0 + 16 * cc, du);
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int pc = (ch0 >> 3) + 2 * cc + h;   // 16-byte piece of the 64-channel rows
                        float xv[8], pv[8];
                        unpack8(*reinterpret_cast<const uint4*>(xs + (r + 1) * 128 + ((pc ^ ((r + 1) & 7)) << 4)), xv);
                        unpack8(*reinterpret_cast<const uint4*>(xs + r * 128 + ((pc ^ (r & 7)) << 4)), pv);
#pragma unroll
                        for (int j = 0; j < 8; ++j) pvs[8 * h + j] = pv[j] - xv[j];
                    }
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const float d = __uint_as_float(du[j]);
                        X[16 * cc + j] = d * ctrl->alpha[ch0 + 16 * cc + j];
                        Dd[16 * cc + j] = d;
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    uint32_t zk[16];
                    tmem_ld16(tlane + C_Z + 64 * k + ch0 + 16 * cc, zk);
                    float dv[16];
                    uint4* cell[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int pc = (ch0 >> 3) + 2 * cc + h;
                        cell[h] = reinterpret_cast<uint4*>(sm + off_dy(D) + k * TILE + r * 128 + ((pc ^ (r & 7)) << 4));
                        unpack8(*cell[h], dv + 8 * h);
                    }
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        X[16 * cc + j] += dv[j] * (__uint_as_float(zk[j]) + ctrl->beta[k][ch0 + 16 * cc + j]);
                        Dd[16 * cc + j] += dv[j];
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        uint4 o;
                        o.x = pack2(dv[8 * h + 0] * pvs[8 * h + 0], dv[8 * h + 1] * pvs[8 * h + 1]); o.y = pack2(dv[8 * h + 2] * pvs[8 * h + 2], dv[8 * h + 3] * pvs[8 * h + 3]);
                        o.z = pack2(dv[8 * h + 4] * pvs[8 * h + 4], dv[8 * h + 5] * pvs[8 * h + 5]); o.w = pack2(dv[8 * h + 6] * pvs[8 * h + 6], dv[8 * h + 7] * pvs[8 * h + 7]);
                        *cell[h] = o;
                    }
                }
            }
            // dz is in place: products 2 may start.  X of the first row of every quarter goes to shared memory for the row above.
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < CPT; ++j) ctrl->edge[q][ch0 + j] = X[j];
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the previous unit's dx store has read the staging tile
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ctrl->dz_ready)) : "memory");
            asm volatile("bar.sync 2, %0;" ::"n"(32 * EPI_WARPS) : "memory");   // edges and the halo sums are complete
            // ---- dx_t = Dd_t - X_t + X_{t+1} ------------------------------------------------------------------------------
            unsigned char* dxs = sm + off_dx(D);
#pragma unroll
            for (int pcl = 0; pcl < CPT / 8; ++pcl) {
                float o[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const int cj = 8 * pcl + j;
                    float xn = __shfl_down_sync(0xffffffffu, X[cj], 1);
                    if (lane == 31) xn = q < 3 ? ctrl->edge[q + 1][ch0 + cj] : ctrl->halo[ch0 + cj];
                    o[j] = Dd[cj] - X[cj] + xn;
                }
                uint4 pk;
                pk.x = pack2(o[0], o[1]); pk.y = pack2(o[2], o[3]); pk.z = pack2(o[4], o[5]); pk.w = pack2(o[6], o[7]);
                const int pc = (ch0 >> 3) + pcl;
                *reinterpret_cast<uint4*>(dxs + r * 128 + ((pc ^ (r & 7)) << 4)) = pk;
            }
            if (q == 3 && lane == 31) {
#pragma unroll
                for (int j = 0; j < CPT; ++j) ctrl->halo[ch0 + j] = 0.f;   // read above; the next unit's sums start after the barrier below
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("bar.sync 3, %0;" ::"n"(32 * EPI_WARPS) : "memory");   // staging tile complete; edge and halo values have been read
            if (g == 0 && lane == 0) {
                if (ok && t0 + 32 * q < T)
                    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                                 ::"l"(&maps.dx), "r"(cb * 64), "r"(t0 + 32 * q), "r"(bi), "r"(smem_u32(dxs + 32 * q * 128)) : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            __syncwarp();
        }
        if (nmine > 0) {
            mbar_wait_bounded<true>(&ctrl->unit_free, (nmine - 1) & 1, &ctrl->abort, status);
            flush(cb_prev);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
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
    constexpr int smem = g2::smem_bytes(D);
    static_assert(smem <= 232448, "two stages, the output staging and the control block must fit one CTA");
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    static const int sms = [] {
        int dev = 0, n = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        return n;
    }();
    const long long tiles_per_seq = (p.T + BM - 1) / BM, units = tiles_per_seq * B * (p.C / g2::BN);
    if (units > 0x7fffffffLL) return kTooLarge;
    const unsigned grid = (unsigned)(units < sms ? units : sms);
    kern<<<grid, g2::THREADS, smem, stream>>>(mM, mR, mX, mY, (const __nv_bfloat16*)p.beta, (int)p.C, (int)p.T, (int)tiles_per_seq, (int)units, status);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace dtc

// scratch of the backward: dW2 (fp32 [4D, C]), R^T (bf16 [4D, C]), L^T and R' (bf16 [C, 4D] each)
size_t ddlerp_bwd_tc_workspace_bytes(long long C, int D) { return (size_t)(4 * D) * (size_t)C * 10; }

// dx, dR, dbeta (dR, dbeta zero on entry) on the tensor cores; ranks 16 and 32.  dalpha is NOT formed here (see the dL step).
template <int D> static int launch_main_tc_t(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream) {
    using namespace dtc;
    const long long B = p.rows / p.T, C = p.C, T = p.T;
    const int n4 = 4 * D;
    __nv_bfloat16* Lt = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(ws) + (size_t)n4 * C * 6);  // written by launch_ddlerp_prep_bwd
    __nv_bfloat16* Rp = Lt + (size_t)n4 * C;
    alignas(64) MainMaps mm;
    const long long dx[3] = {C, T, B}, sx[2] = {C, T * C}, dn[3] = {n4, T, B}, sn[2] = {n4, T * n4}, dw[2] = {n4, C}, sw[1] = {n4};
    const int b128[3] = {64, BM, 1}, b129[3] = {64, BM + 1, 1}, bw[2] = {64, 64}, b32[3] = {64, 32, 1};
    for (int k = 0; k < 4; ++k)
        if (!encode(&mm.dy[k], p.dy[k], 3, dx, sx, b128)) return kLaunchFailed;
    if (!(encode(&mm.x, p.x, 3, dx, sx, b129) && encode(&mm.dpre, p.dpre, 3, dn, sn, b128) && encode(&mm.m, p.m, 3, dn, sn, b128) &&
          encode(&mm.lt, Lt, 2, dw, sw, bw) && encode(&mm.rp, Rp, 2, dw, sw, bw) && encode(&mm.dx, p.dx, 3, dx, sx, b32)))
        return kLaunchFailed;
    auto kern = ddlerp_main_tc_kernel<D>;
    constexpr int smem = g5::off_ctrl(D) + (int)sizeof(g5::Ctrl) + 1024;
    static_assert(smem <= 232448, "the unit's tiles must fit one CTA");
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    static const int sms = [] {
        int dev = 0, n = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        return n;
    }();
    const long long tiles_per_seq = (T + BM - 1) / BM, tiles = tiles_per_seq * B, units = tiles * (C / 64);
    if (units > 0x7fffffffLL) return kTooLarge;
    const unsigned grid = (unsigned)(units < sms ? units : sms);
    kern<<<grid, g5::THREADS, smem, stream>>>(mm, (const __nv_bfloat16*)p.dy[0], (const __nv_bfloat16*)p.dy[1], (const __nv_bfloat16*)p.dy[2],
                                             (const __nv_bfloat16*)p.dy[3], (const __nv_bfloat16*)p.dpre, (const __nv_bfloat16*)p.m, (const __nv_bfloat16*)p.alpha,
                                             (const __nv_bfloat16*)p.beta, p.dR, p.dbeta, (int)C, (int)T, (int)tiles_per_seq, (int)tiles, (int)units, status);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}
// returns kBadShape for ranks this form does not cover (the caller then runs the mma.sync kernel)
int launch_ddlerp_main_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream) {
    if (p.D == 16) return launch_main_tc_t<16>(p, ws, status, stream);
    if (p.D == 32) return launch_main_tc_t<32>(p, ws, status, stream);
    return kBadShape;
}

// the rearranged weights of the tcgen05 backward kernels into the scratch: R^T, L^T, R' behind dW2
int launch_ddlerp_prep_bwd(const DdlerpBwdParams& p, void* ws, cudaStream_t stream) {
    const long long C = p.C;
    const int n4 = 4 * p.D;
    __nv_bfloat16* Rt = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(ws) + (size_t)n4 * C * 4);
    const long long n = (long long)n4 * C;
    dtc::ddlerp_prep_bwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)p.L, (const __nv_bfloat16*)p.R, Rt, Rt + n, Rt + 2 * n, (int)C, p.D);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

// dpre (bf16 [rows, 4D]) from dy, x, R and m; ranks 16 and 32
template <int D> static int launch_dpre_tc_t(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream) {
    using namespace dtc;
    const long long B = p.rows / p.T, C = p.C, T = p.T;
    const int n4 = 4 * D;
    __nv_bfloat16* Rt = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<unsigned char*>(ws) + (size_t)n4 * C * 4);  // written by launch_ddlerp_prep_bwd
    if (B > 65535) return kTooLarge;
    alignas(64) DyMaps mY;
    alignas(64) CUtensorMap mX, mRt, mP;
    const long long dx[3] = {C, T, B}, sx[2] = {C, T * C}, dr[2] = {C, n4}, sr[1] = {C}, dp[3] = {n4, T, B}, sp[2] = {n4, T * n4};
    const int by[3] = {64, BM, 1}, bx[3] = {64, BM + 1, 1}, br[2] = {64, n4}, bp[3] = {64, 32, 1};
    for (int k = 0; k < 4; ++k)
        if (!encode(&mY.m[k], p.dy[k], 3, dx, sx, by)) return kLaunchFailed;
    if (!(encode(&mX, p.x, 3, dx, sx, bx) && encode(&mRt, Rt, 2, dr, sr, br) && encode(&mP, p.dpre, 3, dp, sp, bp))) return kLaunchFailed;
    auto kern = ddlerp_dpre_tc_kernel<D>;
    constexpr int smem = g4::STAGES * g4::stage_bytes(D) + (int)sizeof(g4::Ctrl) + 1024;
    static_assert(smem <= 232448, "two stages must fit one CTA");
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    dim3 grid((unsigned)((T + BM - 1) / BM), (unsigned)B);
    kern<<<grid, g4::THREADS, smem, stream>>>(mY, mX, mRt, mP, (const __nv_bfloat16*)p.m, (int)C, (int)T, status);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}
// returns kBadShape for ranks this form does not cover (the caller then runs the mma.sync kernel)
int launch_ddlerp_dpre_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream) {
    if (p.D == 16) return launch_dpre_tc_t<16>(p, ws, status, stream);
    if (p.D == 32) return launch_dpre_tc_t<32>(p, ws, status, stream);
    return kBadShape;
}

// dL (fp32 [4D, C], zero on entry) from dpre and x, and with with_dalpha also dalpha (overwritten); ws: the backward's scratch
int launch_ddlerp_dL_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream, bool with_dalpha) {
    using namespace dtc;
    const long long B = p.rows / p.T, C = p.C, T = p.T;
    const int n4 = 4 * p.D;
    float* dW2 = (float*)ws;
    if (cudaMemsetAsync(dW2, 0, sizeof(float) * n4 * C, stream) != cudaSuccess) return kLaunchFailed;
    alignas(64) CUtensorMap mD, mX;
    const long long dd[3] = {n4, T, B}, sd[2] = {n4, T * n4}, dx[3] = {C, T, B}, sx[2] = {C, T * C};
    const int bx[3] = {64, BM, 1};
    if (!(encode(&mD, p.dpre, 3, dd, sd, bx) && encode(&mX, p.x, 3, dx, sx, bx))) return kLaunchFailed;
    const int smem = g3::STAGES * g3::STAGE_BYTES + (int)sizeof(g3::Ctrl) + 1024;
    if (cudaFuncSetAttribute(ddlerp_dw12_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    static const int sms = [] {
        int dev = 0, n = 148;
        if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        return n;
    }();
    const long long tiles_per_seq = (T + BM - 1) / BM, total = tiles_per_seq * B;
    if (total > 0x7fffffffLL) return kTooLarge;
    const int col_tiles = 2 * (int)((C + g3::BN - 1) / g3::BN), row_tiles = (n4 + BM - 1) / BM;
    long long splits = sms / (col_tiles * row_tiles);  // one CTA per SM (a stage pair fills its shared memory)
    if (splits < 1) splits = 1;
    if (splits > total) splits = total;
    dim3 grid((unsigned)col_tiles, (unsigned)splits, (unsigned)row_tiles);
    ddlerp_dw12_kernel<<<grid, g3::THREADS, smem, stream>>>(mD, mX, p.dL, dW2, (int)C, n4, (int)tiles_per_seq, (int)total, status);
    if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    ddlerp_dl_finish_kernel<<<dim3((unsigned)((C + 127) / 128), (unsigned)((n4 + 7) / 8)), 128, 0, stream>>>(
        p.dL, dW2, (const __nv_bfloat16*)p.alpha, (const __nv_bfloat16*)p.L, with_dalpha ? p.dalpha : nullptr, (int)C, n4);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

size_t ddlerp_fwd_tc_workspace_bytes(long long C, int D) { return (size_t)(4 * D) * (size_t)(3 * C) * 2; }

int launch_ddlerp_fwd_tc(const DdlerpFwdParams& p, void* ws, int* status, cudaStream_t stream) {
    using namespace dtc;
    if (p.rows == 0) return kOk;
    const long long B = p.rows / p.T, C = p.C, T = p.T;
    const int D = p.D, n4 = 4 * D;
    if (D == 64) return launch_ddlerp_fwd(p, stream);  // the lerp kernel's two stages do not fit shared memory at rank 64
    if (D != 16 && D != 32) return kBadShape;
    if (B > 65535 || (T + BM - 1) / BM > 65535) return kTooLarge;
    __nv_bfloat16* W12 = (__nv_bfloat16*)ws;
    __nv_bfloat16* Rp = W12 + (long long)n4 * 2 * C;
    {
        const long long n = (long long)n4 * 3 * C;
        ddlerp_prep_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>((const __nv_bfloat16*)p.L, (const __nv_bfloat16*)p.alpha, (const __nv_bfloat16*)p.R,
                                                                          W12, Rp, (int)C, D);
        if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    }
    alignas(64) CUtensorMap mX, mXl, mW, mMs, mMl, mR, mY;
    {
        const long long dx[3] = {C, T, B}, sx[2] = {C, T * C};
        const int bx[3] = {BK, BM, 1}, bxl[3] = {g2::BN, g2::XROWS, 1};
        const long long dw[2] = {2 * C, n4}, sw[1] = {2 * C};
        const int bw[2] = {BK, g1::BN};
        const long long dm[3] = {n4, T, B}, sm_[2] = {n4, T * n4};
        const int bms[3] = {64, 32, 1}, bml[3] = {64, BM, 1};
        const long long dr[2] = {n4, C}, sr[1] = {n4};
        const int br[2] = {64, g2::BN};
        const long long dy[4] = {C, T, B, 4}, sy[3] = {C, T * C, B * T * C};
        const int by[4] = {g2::BN, 32, 1, 1};
        if (!(encode(&mX, p.x, 3, dx, sx, bx) && encode(&mXl, p.x, 3, dx, sx, bxl) && encode(&mW, W12, 2, dw, sw, bw) && encode(&mMs, p.m, 3, dm, sm_, bms) &&
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
    return D == 16 ? launch_lerp<16>(mMl, mR, mXl, mY, p, B, status, stream) : launch_lerp<32>(mMl, mR, mXl, mY, p, B, status, stream);
}

}  // namespace wkv7
