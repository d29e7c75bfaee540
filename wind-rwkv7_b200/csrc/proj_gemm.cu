// Projection GEMM of the time mixer on the 5th-generation tensor cores:  C = act(A W^T)
//     A [M, K] bf16 (activations, rows = tokens),  W [N, K] bf16 (an nn.Linear weight),  C [M, N] bf16,
//     act = tanh on the columns [tanh_from, tanh_to) (the first stage of a LoRA feeds its second stage through tanh),
//     identity elsewhere.
// Replaces the torch matmuls of the reference's mixer (wind_rwkv/rwkv7/time_mixer.py:120-131, 167: x @ W.bfloat16().mT
// followed by a separate tanh pass) for the forward direction.
//
// One CTA computes one 128 x 128 tile of C.  Both operands are K-major, so a [128 rows x 64 k] bf16 block is 128-byte rows:
// TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) brings blocks of A and W into a ring of STAGES shared-memory stages, one
// elected thread issues tcgen05.mma.kind::f16 (M = 128, N = 128, K = 16; four per block) with the fp32 accumulator in
// tensor memory, tcgen05.commit hands a stage back to the producer, and four warps read the accumulator back
// (tcgen05.ld, one row per lane), apply the activation and store the tile through shared memory with bulk tensor stores.  96 KB of shared memory and 128 tensor-memory
// columns per CTA, so two CTAs share an SM and one's epilogue overlaps the other's main loop.
// Rows and columns beyond M and N read as zeros and are not stored (the tensor maps clip).  Every wait is bounded (see
// mbar_wait_bounded): a wait that runs out reports kDeviceTimeout and the CTA leaves without storing.
#include <cuda.h>
#include <cstring>

#include "wkv7_kernels.h"

namespace wkv7 {
namespace gemm {

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 3;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int THREADS = 192;  // warps 0-3: epilogue (tensor-memory lane quarters 0-3), warp 4: TMA, warp 5: MMA

struct Ctrl {
    uint64_t full[STAGES], empty[STAGES], accum, drain;
    uint32_t tmem_base;
    volatile int abort, zero;
};

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ uint32_t elect_one() {
    uint32_t p;
    asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}\n" : "=r"(p));
    return p;
}
// K-major operand block with 128-byte rows and the 128-byte swizzle: 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_sw128(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// fp32 accumulate, bf16 operands, both K-major, M = 128, N = 128
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(THREADS) proj_gemm_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                                                           const __grid_constant__ CUtensorMap mapC, long long M, long long N, long long K,
                                                           int tanh_from, int tanh_to, int* status) {
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(sm + STAGES * STAGE_BYTES);
    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nkb = (int)((K + BK - 1) / BK);

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&ctrl->full[s], 1); mbar_init(&ctrl->empty[s], 1); }
        mbar_init(&ctrl->accum, 1); mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0; ctrl->zero = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = ctrl->tmem_base;

    if (warp == 4) {
        if (elect_one()) {  // producer: one TMA request per operand block
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES, round = kb / STAGES;
                if (round > 0) mbar_wait_bounded<true>(&ctrl->empty[s], (round - 1) & 1, &ctrl->abort, status);
                const uint32_t bar = smem_u32(&ctrl->full[s]), dst = smem_u32(sm + s * STAGE_BYTES);
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)STAGE_BYTES) : "memory");
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                             ::"r"(dst), "l"(&mapA), "r"(bar), "r"(kb * BK), "r"(m0) : "memory");
                asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                             ::"r"(dst + A_BYTES), "l"(&mapB), "r"(bar), "r"(kb * BK), "r"(n0) : "memory");
            }
        }
        __syncwarp();
    } else if (warp == 5) {
        if (elect_one()) {  // MMA issuer
            for (int kb = 0; kb < nkb; ++kb) {
                const int s = kb % STAGES, round = kb / STAGES;
                mbar_wait_bounded<false>(&ctrl->full[s], round & 1, &ctrl->abort, status);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = desc_sw128(smem_u32(sm + s * STAGE_BYTES)), db = desc_sw128(smem_u32(sm + s * STAGE_BYTES + A_BYTES));
#pragma unroll
                for (int ks = 0; ks < BK / 16; ++ks) {
                    const uint32_t acc = (kb > 0 || ks > 0) ? 1u : 0u;
                    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                                 ::"r"(tmem), "l"(da + (uint64_t)(2 * ks)), "l"(db + (uint64_t)(2 * ks)), "r"(IDESC), "r"(acc) : "memory");
                }
                // the stage may be refilled once these products have read it
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&ctrl->empty[s])) : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&ctrl->accum)) : "memory");
            if (ctrl->abort) {
                // a bounded wait gave up and the later waits fell through: commit everything issued to a barrier of its own and
                // wait for it, bounded and regardless of the abort flag, before tensor memory is released
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&ctrl->drain)) : "memory");
                mbar_wait_bounded<false>(&ctrl->drain, 0, &ctrl->zero, status);
            }
        }
        __syncwarp();
    } else {
        // epilogue: warp q owns tensor-memory lanes 32q..32q+31 = rows m0 + 32q + lane
        mbar_wait_bounded<true>(&ctrl->accum, 0, &ctrl->abort, status);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        // The tile leaves through shared memory (the operand stages are free now): every lane writes its row, as bf16, into two
        // [128 rows][64 columns] halves in the 128-byte-swizzled layout (16-byte piece p of row r at p ^ (r % 8): lanes are
        // consecutive rows, so a store instruction touches 32 different bank groups), and each warp stores its 32 rows
        // with two bulk tensor stores, which undo the swizzle and clip at M and N.
        const bool ok = !ctrl->abort;
        const int r = 32 * warp + lane;
#pragma unroll 1
        for (int cb = 0; cb < BN; cb += 32) {
            uint32_t v[32];
            const uint32_t ta = tmem + ((uint32_t)(32 * warp) << 16) + cb;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                         : "=r"(v[0]),"=r"(v[1]),"=r"(v[2]),"=r"(v[3]),"=r"(v[4]),"=r"(v[5]),"=r"(v[6]),"=r"(v[7]),"=r"(v[8]),"=r"(v[9]),"=r"(v[10]),"=r"(v[11]),"=r"(v[12]),"=r"(v[13]),"=r"(v[14]),"=r"(v[15]),
                           "=r"(v[16]),"=r"(v[17]),"=r"(v[18]),"=r"(v[19]),"=r"(v[20]),"=r"(v[21]),"=r"(v[22]),"=r"(v[23]),"=r"(v[24]),"=r"(v[25]),"=r"(v[26]),"=r"(v[27]),"=r"(v[28]),"=r"(v[29]),"=r"(v[30]),"=r"(v[31])
                         : "r"(ta));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            unsigned char* half = sm + (cb >> 6) * (BM * 128);
#pragma unroll
            for (int c8 = 0; c8 < 32; c8 += 8) {
                const int col = n0 + cb + c8;
                float f[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    f[i] = __uint_as_float(v[c8 + i]);
                    if (col + i >= tanh_from && col + i < tanh_to) f[i] = tanh_approx(f[i]);
                }
                uint4 pk;
                __nv_bfloat162 h;
                h = __floats2bfloat162_rn(f[0], f[1]); pk.x = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(f[2], f[3]); pk.y = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(f[4], f[5]); pk.z = *reinterpret_cast<uint32_t*>(&h);
                h = __floats2bfloat162_rn(f[6], f[7]); pk.w = *reinterpret_cast<uint32_t*>(&h);
                const int piece = ((cb & 63) + c8) >> 3;
                *reinterpret_cast<uint4*>(half + r * 128 + ((piece ^ (r & 7)) << 4)) = pk;
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (ok && lane == 0) {
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
                if (n0 + 64 * h2 < N)
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                                 ::"l"(&mapC), "r"(n0 + 64 * h2), "r"(m0 + 32 * warp), "r"(smem_u32(sm + h2 * (BM * 128) + 32 * warp * 128)) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory must outlive the stores' reads
        }
        __syncwarp();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BN) : "memory");
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
// [rows, K] bf16 row-major; box = 64 k x 128 rows, 128-byte swizzle; out-of-range parts of a box read as zeros
static bool encode_kmajor(CUtensorMap* m, const void* base, long long rows, long long K, int box_rows = BM) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    const cuuint32_t es[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace gemm

int launch_proj_gemm(const void* A, const void* W, void* C, long long M, long long N, long long K, int tanh_from, int tanh_to,
                     int* status, cudaStream_t stream) {
    using namespace gemm;
    alignas(64) CUtensorMap ma, mb, mc;
    // C [M, N]: the same kind of map (64 columns x 32 rows per store, one per warp and half tile)
    if (!encode_kmajor(&ma, A, M, K) || !encode_kmajor(&mb, W, N, K) || !encode_kmajor(&mc, C, M, N, 32)) return kLaunchFailed;
    const int smem = STAGES * STAGE_BYTES + (int)sizeof(Ctrl) + 1024;
    if (cudaFuncSetAttribute(proj_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    dim3 grid((unsigned)((N + BN - 1) / BN), (unsigned)((M + BM - 1) / BM));
    proj_gemm_kernel<<<grid, gemm::THREADS, smem, stream>>>(ma, mb, mc, M, N, K, tanh_from, tanh_to, status);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace wkv7
