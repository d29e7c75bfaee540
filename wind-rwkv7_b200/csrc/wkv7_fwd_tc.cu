// WKV7 forward on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory), bf16 IO.
//
// Same mathematics as wkv7_fwd.cu (the reference's forward_kernel, wind_rwkv/rwkv7/attn.cu:11-106, and
// with LN = true its fused GroupNorm + bonus + gate variant, wind_rwkv/rwkv7/attn_ln.cu:106-212),
// different machine mapping.  One CTA walks one (batch, head) chain.  The 64x64 state S[value][key]
// lives in tensor memory for the whole sequence and is never held in registers: per 16-step chunk
// one elected thread issues 26 tcgen05.mma instructions (M = 64 value rows, TF32 operands, fp32
// accumulate)
//     hop 1   [X | Yp] = S [wa;wq]^T + V^T [AK;QK]^T        A = S straight from tensor memory
//     hop 2   U  = X AI^T                                    A = X from tensor memory
//     hop 3   Y  = Yp + U QB^T                               A = U from tensor memory
//     hop 4   S' = S diag(fw) + V^T kwf + U bwf              eight N = 8 products apply the decay
// with kwf = kwi*fw, bwf = bwi*fw, so the column scaling of the state never touches a CUDA core.
// An accumulator that the next product reads as its A operand needs an explicit completion wait
// (tcgen05.commit -> mbarrier); only same-accumulator chains are ordered by the tensor pipe, so the
// decay product and the V^T kwf product are issued inside those waits.
//
// Everything state-independent is done by G "preparation groups" of four warps, each working on
// its own chunk (c, c+G, ...): cp.async of the six input tiles, the decay scan, the operand tiles
// in the shared-memory layouts the tensor core reads directly, the four 16x16 score matrices as
// ONE tcgen05 product ([wa;wq] x [kwi;bwi]^T, M = 64 of which 32 rows are used), masking, the
// triangular inverse, and afterwards the read-back of Y (and of the chunk-end state for the
// checkpoints) from tensor memory.  A group's loop is software-pipelined: the decay scan of its next
// chunk is computed into registers while the chain works on its previous chunk, and the read-back of
// that chunk's results happens just before the operand tiles are overwritten.
//
// Warp roles (128 (G+1) threads): warps 0..4G-1 are the preparation groups, warp 4G+3 issues the chain,
// the other three warps of its warp group only exist so that setmaxnreg can be used: the chain
// warp group shrinks to 32 registers per thread and the preparation warps grow to 112 (a kernel-wide
// 96, which is all that 20 warps leave, makes the decay scan spill, and the spills cost more than
// the whole scan).  The chain thread waits for "operands of chunk c ready" and "results of chunk c-2
// read", so the 16-step dependency is ~1100 cycles per chunk.
//
// Shared-memory operand layouts (no TMA: the tiles are produced by threads, not copied):
//   K-major (contraction index contiguous): 16-byte chunks [row/8][k/4][row%8][k%4], descriptor
//     LBO = 128 B (next k-chunk), SBO = bytes per 8-row group, no swizzle.
//   MN-major TF32 (V, kwf, bwf: contraction index = time): only the 128-byte swizzle with 32-byte
//     base exists for 32-bit MN-major operands: rows of 32 channels (128 B) per time step, the
//     32-byte unit index XOR-ed with (t % 4); LBO = stride between the two 32-channel halves,
//     SBO = 512 B (four time steps).
// Checkpoint states leave through shared memory: tensor memory holds one state row per lane, so a warp-wide
// store from registers can write one 32-byte sector per lane at best (512 wavefronts of the SM's L1 data
// pipe per 16 KB state).  Instead each thread writes its row into a 128-byte-swizzled staging tile (two
// [64 rows][32 floats] halves in the dead [wa;wq] / [kwi;bwi] tiles, conflict-free 16-byte stores) and one
// thread issues two tensor-map bulk stores (cp.async.bulk.tensor.2d, shared -> global), which undo the
// swizzle: the record in global memory stays plain row-major.
// Every wait on an mbarrier is bounded; a wait that runs out raises an abort flag that makes all
// later waits of the CTA return at once, records kDeviceTimeout and lets the CTA finish (tensor
// memory is still released).
#include <cuda.h>
#include <cstring>

#include "wkv7_kernels.h"
namespace wkv7 {
namespace tc {

constexpr int ROWB = 2 * N;         // staging row of a bf16 input tile: 128 bytes, its eight 16-byte segments XOR-ed with (row % 8)
constexpr int RAW_TILE = L * ROWB;  // 2048

// per-group shared memory (byte offsets; tensor-core tiles first, all 1024-byte aligned)
constexpr int G_WAQ = 0;       // [wa;wq]   32 rows x 64, K-major            8192
constexpr int G_KB = 8192;     // [kwi;bwi] 32 rows x 64, K-major            8192 (directly after WAQ: the M = 64 score
                               //                                                 product reads rows 32..63 from here, unused)
constexpr int G_V = 16384;     // V   [time][value]  MN-major                4096
constexpr int G_KWF = 20480;   // kwf [time][key]    MN-major                4096
constexpr int G_BWF = 24576;   // bwf [time][key]    MN-major                4096
constexpr int G_SC = 28672;    // [AK;QK]  32 rows x 16, K-major             2048
constexpr int G_AI = 30720;    // AI       16 x 16, K-major                  1024
constexpr int G_QB = 31744;    // QB       16 x 16, K-major                  1024
static_assert(G_AI == G_SC + 2048 && G_QB == G_AI + 1024, "[AK;QK], AI, QB must be contiguous: they leave as one bulk copy");
constexpr int G_DF = 32768;    // eight 8x8 diagonal blocks of fw, K-major   2048
constexpr int G_ABT = 34816;   // AB transposed, fp32 [16][SCS]              1536
constexpr int G_RAW = 36352;   // q, w, k, a, b, v staging                   6 * 2048
constexpr int G_GRAW = 48640;  // attn_ln only: the gate tile, double buffered (read one iteration later)  2 * 2048
constexpr int G_BYTES_PLAIN = 49152;  // 48 KB (48640 rounded up to 1 KB)
constexpr int G_BYTES_LN = 53248;     // 52 KB
// attn_ln epilogue scratch inside the kwf / bwf tiles, which are dead once the chain step has completed
constexpr int LN_YS = 68;                  // row stride (floats) of the fp32 [time][value] staging of Y
constexpr int LN_PART = L * LN_YS * 4;     // byte offset of the per-warp partial sums [4][16][2] behind it

// tensor-memory columns (32-bit each, 128 lanes; the M = 64 products use lanes 0-15 of each 32-lane quarter)
constexpr int C_S = 0;      // two 64-column state buffers
constexpr int C_XY = 128;   // two buffers of X (16) | Y (16)
constexpr int C_U = 192;    // U (16)
constexpr int C_SCORE = 208;  // + 32 * group: [AK|AB] in lanes 0-15, [QK|QB] in lanes 32-47

constexpr long long WAIT_LIMIT = MBAR_WAIT_LIMIT;

struct Ctrl {
    uint64_t full[4], done[4], rdone[4], score[4], hop;
    uint64_t drain;            // abort path only: completion of the chain thread's outstanding tensor-core work
    uint32_t tmem_base;
    volatile int abort;
    volatile int zero;         // stays 0: the abort-path drain waits with this in place of the abort flag
    float lnp[3 * N];          // attn_ln: GroupNorm weight, bias, bonus of this head
    float bdot[4][2][4][L];    // attn_ln: per-warp partial bonus dots [group][iteration parity][warp][time]
};

__device__ __forceinline__ uint32_t elect_one() {
    uint32_t p;
    asm volatile("{\n.reg .pred P;\nelect.sync _|P, 0xffffffff;\nselp.u32 %0, 1, 0, P;\n}\n" : "=r"(p));
    return p;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait for the phase with the given parity.  Returns at once when the CTA has aborted.
// SLEEP: the thread is suspended by the hardware (try_wait with a time hint) instead of polling, so
// that the many warps that wait for the chain do not take issue slots from the warps that work; the
// chain's own short waits poll.
template <bool SLEEP>
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity, Ctrl* ctrl, int* status, long long limit = WAIT_LIMIT) {
    mbar_wait_bounded<SLEEP>(bar, parity, &ctrl->abort, status, limit);
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Abort path: commits everything this thread has issued to the tensor core to a barrier of its own and waits for
// it, bounded and regardless of the CTA's abort flag, so that tensor memory is not released under products in flight.
__device__ __forceinline__ void drain_tensor_work(uint64_t* bar, volatile int* never_set, int* status) {
    tc_commit(bar);
    mbar_wait_bounded<false>(bar, 0, never_set, status);
}
// named barrier of one preparation group; immediate ids, so that ptxas counts G + 1 barriers for the CTA
// and not all sixteen
__device__ __forceinline__ void group_bar(int grp) {
    switch (grp) {
        case 0: asm volatile("bar.sync 1, 128;" ::: "memory"); break;
        case 1: asm volatile("bar.sync 2, 128;" ::: "memory"); break;
        case 2: asm volatile("bar.sync 3, 128;" ::: "memory"); break;
        default: asm volatile("bar.sync 4, 128;" ::: "memory"); break;
    }
}

// shared-memory matrix descriptor (sm_100 version field set); byte offsets are added to the low word
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr, uint32_t sbo) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {  // 128-byte swizzle with 32-byte base
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)(2048 >> 4) << 16) | ((uint64_t)(512 >> 4) << 32) | (1ull << 46) | (1ull << 61);
}
// instruction descriptor: fp32 accumulate, TF32 operands, M = 64
__host__ __device__ constexpr uint32_t idesc(int n, bool a_mn, bool b_mn) {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) | (4u << 24);
}
__device__ __forceinline__ void mma_ss(uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(d), "l"(a), "l"(b), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void mma_ts(uint32_t d, uint32_t a, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n}\n"
                 ::"r"(d), "r"(a), "l"(b), "r"(id), "r"(acc) : "memory");
}
// 16 consecutive columns of this thread's lane
__device__ __forceinline__ void tmem_ld16(uint32_t ta, uint32_t* v) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]),"=r"(v[1]),"=r"(v[2]),"=r"(v[3]),"=r"(v[4]),"=r"(v[5]),"=r"(v[6]),"=r"(v[7]),"=r"(v[8]),"=r"(v[9]),"=r"(v[10]),"=r"(v[11]),"=r"(v[12]),"=r"(v[13]),"=r"(v[14]),"=r"(v[15]) : "r"(ta));
}
__device__ __forceinline__ void tmem_st16(uint32_t ta, const uint32_t* v) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15};"
        :: "r"(v[0]),"r"(v[1]),"r"(v[2]),"r"(v[3]),"r"(v[4]),"r"(v[5]),"r"(v[6]),"r"(v[7]),"r"(v[8]),"r"(v[9]),"r"(v[10]),"r"(v[11]),"r"(v[12]),"r"(v[13]),"r"(v[14]),"r"(v[15]), "r"(ta) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float rnd(float x) { return __uint_as_float(tf32_rna(x)); }

// byte offset of the 16-byte chunk holding (row, k..k+3) in a K-major tile; sbo = bytes per 8-row group
__device__ __forceinline__ int kchunk(int row, int kc, int sbo) { return (row >> 3) * sbo + kc * 128 + (row & 7) * 16; }

// Column `col` of AI = (I - AB)^-1 (AB strictly lower triangular), written into the K-major AI tile
// as element (row S_, k = col).  Right-looking substitution as in tri_inverse_column().
template <int S_> __device__ __forceinline__ void tri_step_tc(float (&r)[L], const float (&c)[L], float (&cn)[L], const float* ABt, unsigned char* AI, int col) {
    if (S_ + 1 < L) tri_fetch_row<(S_ + 1 < L ? S_ + 1 : 0)>(cn, ABt);
    const float ms = r[S_], msr = rnd(ms);
    *reinterpret_cast<float*>(AI + kchunk(S_, col >> 2, 512) + (col & 3) * 4) = msr;
#pragma unroll
    for (int tq = S_ + 1; tq < L; ++tq) r[tq] = fmaf(c[tq], ms, r[tq]);
}
__device__ __forceinline__ void tri_inverse_tc(const float* ABt, unsigned char* AI, int col) {
    float r[L], ca[L], cb[L];
#pragma unroll
    for (int tq = 0; tq < L; ++tq) r[tq] = (tq == col) ? 1.f : 0.f;
    tri_fetch_row<0>(ca, ABt);
    tri_step_tc<0>(r, ca, cb, ABt, AI, col);   tri_step_tc<1>(r, cb, ca, ABt, AI, col);
    tri_step_tc<2>(r, ca, cb, ABt, AI, col);   tri_step_tc<3>(r, cb, ca, ABt, AI, col);
    tri_step_tc<4>(r, ca, cb, ABt, AI, col);   tri_step_tc<5>(r, cb, ca, ABt, AI, col);
    tri_step_tc<6>(r, ca, cb, ABt, AI, col);   tri_step_tc<7>(r, cb, ca, ABt, AI, col);
    tri_step_tc<8>(r, ca, cb, ABt, AI, col);   tri_step_tc<9>(r, cb, ca, ABt, AI, col);
    tri_step_tc<10>(r, ca, cb, ABt, AI, col);  tri_step_tc<11>(r, cb, ca, ABt, AI, col);
    tri_step_tc<12>(r, ca, cb, ABt, AI, col);  tri_step_tc<13>(r, cb, ca, ABt, AI, col);
    tri_step_tc<14>(r, ca, cb, ABt, AI, col);  tri_step_tc<15>(r, cb, ca, ABt, AI, col);
}

// two 16-byte chunks of an operand tile; R: round to TF32 (nearest) first, otherwise the tensor core
// truncates the low 13 mantissa bits when it reads the operand
template <bool R> __device__ __forceinline__ void store8t(unsigned char* p0, unsigned char* p1, const float (&f)[8]) {
    if (R) {
        *reinterpret_cast<float4*>(p0) = make_float4(rnd(f[0]), rnd(f[1]), rnd(f[2]), rnd(f[3]));
        *reinterpret_cast<float4*>(p1) = make_float4(rnd(f[4]), rnd(f[5]), rnd(f[6]), rnd(f[7]));
    } else {
        *reinterpret_cast<float4*>(p0) = make_float4(f[0], f[1], f[2], f[3]);
        *reinterpret_cast<float4*>(p1) = make_float4(f[4], f[5], f[6], f[7]);
    }
}
// 32 bytes of an MN-major tile in two 16-byte stores; `flip` swaps the order of the two halves so that the
// eight lanes of a quarter-warp (rows r..r+7, where r and r+4 share a 32-byte unit) never hit the same bank
template <bool R> __device__ __forceinline__ void store8mn(unsigned char* p, const float (&f)[8], bool flip) {
    float x[4], y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float lo = R ? rnd(f[i]) : f[i], hi = R ? rnd(f[4 + i]) : f[4 + i];
        x[i] = flip ? hi : lo;  // goes out first
        y[i] = flip ? lo : hi;
    }
    const int off = flip ? 16 : 0;
    *reinterpret_cast<float4*>(p + off) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(p + (16 - off)) = make_float4(y[0], y[1], y[2], y[3]);
}
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// TAIL: the sequence length is not a multiple of 16 (a build of its own, so that whole-chunk sequences carry none of
// the row tests in their register budget).
template <int G, bool RND, bool LN, bool TAIL>
__global__ void __launch_bounds__(128 * (G + 1), 1) wkv7_fwd_tc_kernel(FwdParams p, const __grid_constant__ CUtensorMap ckmap) {
    using IoT = __nv_bfloat16;
    constexpr int G_BYTES = LN ? G_BYTES_LN : G_BYTES_PLAIN;
    constexpr int NCOLS = 512;
    static_assert(C_SCORE + 32 * G <= NCOLS, "tensor memory columns");
    // Register reallocation (G == 4 only).  setmaxnreg.inc blocks, without a bound, until the CTA's
    // register pool can satisfy it, and the pool is what the CTA was launched with: 640 threads x 96
    // registers (65536 / 640 rounded down to a multiple of 8; build.py checks that ptxas reports 96).
    // The raised and lowered counts must therefore fit into that pool exactly or with room to spare.
    constexpr int LAUNCH_REGS = 96, PREP_REGS = 112, CHAIN_REGS = 32;
    static_assert(G != 4 || 128 * G * PREP_REGS + 128 * CHAIN_REGS <= 128 * (G + 1) * LAUNCH_REGS, "setmaxnreg would never be satisfied");
    extern __shared__ unsigned char smem_dyn[];
    unsigned char* sm = smem_dyn + ((1024u - (smem_u32(smem_dyn) & 1023u)) & 1023u);
    Ctrl* ctrl = reinterpret_cast<Ctrl*>(sm + G * G_BYTES);

    const int tid = threadIdx.x, lane = tid & 31;
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);  // provably warp-uniform
    const long long bh = blockIdx.x;
    const long long bi = bh / p.H, hi = bh % p.H;
    const long long base = bi * p.st.b + hi * p.st.h;
    const int nchunks = (int)((p.T + L - 1) / L);  // the last chunk may be partial: its missing rows read as zeros
    const int tail = TAIL ? (int)(p.T - (long long)(nchunks - 1) * L) : L;  // time steps of the last chunk (1..16)

    if (tid == 0) {
        for (int g = 0; g < G; ++g) {
            mbar_init(&ctrl->full[g], 128);
            mbar_init(&ctrl->done[g], 1);
            mbar_init(&ctrl->rdone[g], 128);
            mbar_init(&ctrl->score[g], 1);
        }
        mbar_init(&ctrl->hop, 1);
        mbar_init(&ctrl->drain, 1);
        ctrl->abort = 0;
        ctrl->zero = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (LN) {
        for (int i = tid; i < 3 * N; i += blockDim.x) ctrl->lnp[i] = p.params[(long long)(i / N) * p.H * N + hi * N + (i % N)];
    }
    // the off-diagonal zeros of the decay blocks are written once
    for (int i = tid; i < G * (2048 / 16); i += blockDim.x)
        *reinterpret_cast<uint4*>(sm + (i / 128) * G_BYTES + G_DF + (i % 128) * 16) = make_uint4(0, 0, 0, 0);
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&ctrl->tmem_base)), "r"(NCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctrl->tmem_base;

    // initial state -> tensor memory buffer 0 (and checkpoint 0): warp w of group 0 owns lanes 32w..32w+31,
    // of which lanes 0-15 hold value rows 16w..16w+15
    if (warp < 4) {
        const int i = 16 * warp + (lane & 15);
        const float* s0 = p.s0 ? p.s0 + bh * N * N + i * N : nullptr;
        float* ck = (p.ckpt && lane < 16) ? p.ckpt + bh * nchunks * (long long)CK_FLOATS + i * N : nullptr;
#pragma unroll
        for (int cb = 0; cb < N; cb += 16) {
            uint32_t v[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 x = s0 ? *reinterpret_cast<const float4*>(s0 + cb + 4 * q) : make_float4(0.f, 0.f, 0.f, 0.f);
                x.x *= STATE_SCALE; x.y *= STATE_SCALE; x.z *= STATE_SCALE; x.w *= STATE_SCALE;  // the state is carried as S~ = 2^-64 S (see ANCHOR_LN)
                v[4 * q] = __float_as_uint(x.x); v[4 * q + 1] = __float_as_uint(x.y); v[4 * q + 2] = __float_as_uint(x.z); v[4 * q + 3] = __float_as_uint(x.w);
                if (ck) *reinterpret_cast<float4*>(ck + cb + 4 * q) = x;
            }
            tmem_st16(tmem + ((uint32_t)(32 * warp) << 16) + C_S + cb, v);
        }
        tmem_st_wait();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();

    if (warp >= 4 * G) {
        // ------------------------------ chain warp group -----------------------------------------
        if (G == 4) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(CHAIN_REGS));
        // The chain is issued by the LAST warp of its warp group: warp 4G + 3 shares its scheduler (warp index mod 4) with
        // warp 3 of every preparation group, which has the least to do (no score read-back, no inverse); on the
        // scheduler of the groups' warps 0 the chain's instructions waited longer for issue slots (forward +5 %).
        if (warp == 4 * G + 3 && elect_one()) {
            const uint32_t sb = smem_u32(sm);
            uint32_t hop_phase = 0;
            for (int c = 0; c < nchunks; ++c) {
                const int g = c % G, k = c / G;
                const uint32_t gb = sb + g * G_BYTES;
                const uint64_t dWAQ = desc_kmajor(gb + G_WAQ, 2048), dSC = desc_kmajor(gb + G_SC, 512), dAI = desc_kmajor(gb + G_AI, 512),
                               dQB = desc_kmajor(gb + G_QB, 512), dDF = desc_kmajor(gb + G_DF, 256);
                const uint64_t dV = desc_mnmajor(gb + G_V), dKWF = desc_mnmajor(gb + G_KWF), dBWF = desc_mnmajor(gb + G_BWF);
                const uint32_t Sa = tmem + C_S + 64 * (c & 1), Sn = tmem + C_S + 64 * ((c + 1) & 1), XY = tmem + C_XY + 32 * (c & 1), U = tmem + C_U;
                mbar_wait<true>(&ctrl->full[g], k & 1, ctrl, p.status);
                // the Y buffer and the state buffer about to be overwritten were last read for chunk c-2
                if (c > 1) mbar_wait<true>(&ctrl->rdone[(c - 2) % G], ((c - 2) / G) & 1, ctrl, p.status);
                tc_fence_after();
                // hop 1
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) mma_ts(XY, Sa + 8 * ks, dWAQ + (uint64_t)(ks * 16), idesc(32, false, false), ks > 0);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) mma_ss(XY, dV + (uint64_t)(ks * 64), dSC + (uint64_t)(ks * 16), idesc(32, true, false), 1);
                tc_commit(&ctrl->hop);
                // the decay of the old state goes into the other buffer while hop 1 drains
#pragma unroll
                for (int s = 0; s < 8; ++s) mma_ts(Sn + 8 * s, Sa + 8 * s, dDF + (uint64_t)(s * 16), idesc(8, false, false), 0);
                mbar_wait<false>(&ctrl->hop, hop_phase++ & 1, ctrl, p.status);
                tc_fence_after();
                // hop 2
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) mma_ts(U, XY + 8 * ks, dAI + (uint64_t)(ks * 16), idesc(16, false, false), ks > 0);
                tc_commit(&ctrl->hop);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) mma_ss(Sn, dV + (uint64_t)(ks * 64), dKWF + (uint64_t)(ks * 64), idesc(64, true, true), 1);
                mbar_wait<false>(&ctrl->hop, hop_phase++ & 1, ctrl, p.status);
                tc_fence_after();
                // hop 3 and the U part of the state update
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) mma_ts(XY + 16, U + 8 * ks, dQB + (uint64_t)(ks * 16), idesc(16, false, false), 1);
#pragma unroll
                for (int ks = 0; ks < 2; ++ks) mma_ts(Sn, U + 8 * ks, dBWF + (uint64_t)(ks * 64), idesc(64, false, true), 1);
                tc_commit(&ctrl->done[g]);
                tc_commit(&ctrl->hop);
                mbar_wait<false>(&ctrl->hop, hop_phase++ & 1, ctrl, p.status);  // S' is the next chunk's A operand
                tc_fence_after();
            }
            if (ctrl->abort) drain_tensor_work(&ctrl->drain, &ctrl->zero, p.status);
        }
        __syncwarp();
    } else {
        // ------------------------------ preparation group ---------------------------------------
        if (G == 4) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(PREP_REGS));
        const int grp = warp >> 2, wg = warp & 3, gt = tid & 127;
        unsigned char* gs = sm + grp * G_BYTES;
        const uint32_t tlane = tmem + ((uint32_t)(32 * wg) << 16);
        const IoT* gin[6] = {(const IoT*)p.r + base, (const IoT*)p.w + base, (const IoT*)p.k + base,
                             (const IoT*)p.a + base, (const IoT*)p.b + base, (const IoT*)p.v + base};
        IoT* gy = (IoT*)p.y + base;
        const IoT* gg = LN ? (const IoT*)p.g + base : nullptr;
        auto issue_raw = [&](int c, int gbuf) {  // gbuf: parity of the iteration that will process chunk c
            const int r = gt >> 3, seg = gt & 7;
            const bool live = !TAIL || c + 1 < nchunks || r < tail;  // rows beyond the end of the sequence are filled with zeros, nothing is read
            const long long goff = ((long long)c * L + (live ? r : 0)) * p.st.t;
            const int at = r * ROWB + ((seg ^ (r & 7)) << 4);
#pragma unroll
            for (int ten = 0; ten < 6; ++ten) {
                if (TAIL) cp_async16_zfill(gs + G_RAW + ten * RAW_TILE + at, reinterpret_cast<const unsigned char*>(gin[ten] + goff) + seg * 16, live);
                else cp_async16(gs + G_RAW + ten * RAW_TILE + at, reinterpret_cast<const unsigned char*>(gin[ten] + goff) + seg * 16);
            }
            if (LN) {
                if (TAIL) cp_async16_zfill(gs + G_GRAW + gbuf * RAW_TILE + at, reinterpret_cast<const unsigned char*>(gg + goff) + seg * 16, live);
                else cp_async16(gs + G_GRAW + gbuf * RAW_TILE + at, reinterpret_cast<const unsigned char*>(gg + goff) + seg * 16);
            }
            cp_async_commit();
        };
        // Results of own chunk number kk (chunk cc): Y^T into registers, the chunk-end state straight to the
        // checkpoint (or the final state) in two halves, then "results read" for the chain.
        auto read_results = [&](int cc, int kk) {
            mbar_wait<true>(&ctrl->done[grp], kk & 1, ctrl, p.status);
            tc_fence_after();
            const bool last = cc + 1 == nchunks;
            float* sdst = last ? (p.sT ? p.sT + bh * N * N : nullptr)
                               : (p.ckpt ? p.ckpt + (bh * nchunks + cc + 1) * (long long)CK_FLOATS : nullptr);
#ifdef WKV7_TC_NOCKPT
            sdst = nullptr;
#endif
            if (!LN) {
                // Y^T sits one value row per thread.  Lanes i and i^1 swap half of their 16 time steps, so that
                // every lane holds (row i&~1, row i|1) pairs for 8 time steps and stores them as bf16x2.
                uint32_t yv[16];
                tmem_ld16(tlane + C_XY + 32 * (cc & 1) + 16, yv);
                tmem_ld_wait();
                const int odd = lane & 1;
                IoT* yo = gy + ((long long)cc * L + odd) * p.st.t + 16 * wg + (lane & 14);
#pragma unroll
                for (int m = 0; m < 8; ++m) {
                    const float mine = __uint_as_float(odd ? yv[2 * m + 1] : yv[2 * m]);
                    const float give = __uint_as_float(odd ? yv[2 * m] : yv[2 * m + 1]);
                    const float got = __shfl_xor_sync(0xffffffffu, give, 1);
                    const __nv_bfloat162 pr = odd ? __floats2bfloat162_rn(got, mine) : __floats2bfloat162_rn(mine, got);
                    if (lane < 16 && (!TAIL || !last || 2 * m + odd < tail)) *reinterpret_cast<__nv_bfloat162*>(yo + (long long)(2 * m) * p.st.t) = pr;
                }
            } else {
                // attn_ln epilogue (reference: wind_rwkv/rwkv7/attn_ln.cu:176-205): GroupNorm over the head's 64
                // value channels of each time step, + bonus dot * v, * gate.  Y^T goes to shared memory as
                // fp32 [time][value] (in the dead kwf / bwf tiles); then one thread = one time step x 8 value channels, the mapping of the scan.
                float* ysf = reinterpret_cast<float*>(gs + G_KWF);
                float* part = reinterpret_cast<float*>(gs + G_KWF + LN_PART);
                {
                    uint32_t yv[16];
                    tmem_ld16(tlane + C_XY + 32 * (cc & 1) + 16, yv);
                    tmem_ld_wait();
                    if (lane < 16) {
#pragma unroll
                        for (int t = 0; t < 16; ++t) ysf[t * LN_YS + 16 * wg + lane] = __uint_as_float(yv[t]);
                    }
                }
                group_bar(grp);
                const int t = lane & 15, i0 = 16 * wg + 8 * (lane >> 4);
                float yv8[8];
                {
                    const float4 a4 = *reinterpret_cast<const float4*>(ysf + t * LN_YS + i0), b4 = *reinterpret_cast<const float4*>(ysf + t * LN_YS + i0 + 4);
                    yv8[0] = a4.x; yv8[1] = a4.y; yv8[2] = a4.z; yv8[3] = a4.w; yv8[4] = b4.x; yv8[5] = b4.y; yv8[6] = b4.z; yv8[7] = b4.w;
                }
                // sums about a pivot (the row's first element) keep the one-pass variance well conditioned
                const float pivot = ysf[t * LN_YS];
                float s1 = 0.f, s2 = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) { const float dd = yv8[i] - pivot; s1 += dd; s2 = fmaf(dd, dd, s2); }
                s1 += __shfl_xor_sync(0xffffffffu, s1, 16);
                s2 += __shfl_xor_sync(0xffffffffu, s2, 16);
                if (lane < 16) *reinterpret_cast<float2*>(part + (wg * L + t) * 2) = make_float2(s1, s2);
                group_bar(grp);
                {
                    float a1 = 0.f, a2 = 0.f, bd = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < 4; ++w2) {
                        const float2 pp = *reinterpret_cast<const float2*>(part + (w2 * L + t) * 2);
                        a1 += pp.x; a2 += pp.y;
                        bd += ctrl->bdot[grp][kk & 1][w2][t];
                    }
                    const float md = a1 * (1.f / N);
                    const float mu = pivot + md;
                    const float rstd = rsqrtf(fmaxf(a2 * (1.f / N) - md * md, 0.f) + p.eps);
                    // v of this chunk is still in the fp32 MN-major tile, the gate in its own double buffer
                    const int mo = (i0 >> 5) * 2048 + t * 128 + ((((i0 & 31) >> 3) ^ (t & 3)) << 5);
                    const float4 v0 = *reinterpret_cast<const float4*>(gs + G_V + mo), v1 = *reinterpret_cast<const float4*>(gs + G_V + mo + 16);
                    const float vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
                    float gv[8];
                    load8<IoT>(gs + G_GRAW + (kk & 1) * RAW_TILE + t * ROWB + (((i0 >> 3) ^ (t & 7)) << 4), gv);
                    float o8[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        o8[i] = ((yv8[i] - mu) * rstd * ctrl->lnp[i0 + i] + ctrl->lnp[N + i0 + i] + bd * vv[i]) * gv[i];
                    uint4 pk;
                    pk.x = pack_bf16x2_rn(o8[0], o8[1]); pk.y = pack_bf16x2_rn(o8[2], o8[3]);
                    pk.z = pack_bf16x2_rn(o8[4], o8[5]); pk.w = pack_bf16x2_rn(o8[6], o8[7]);
                    if (!TAIL || !last || t < tail) *reinterpret_cast<uint4*>(gy + ((long long)cc * L + t) * p.st.t + i0) = pk;
                }
                group_bar(grp);  // the scratch lies in an operand tile that is rewritten next
            }
            if (sdst && !last) {
                // checkpoint state: exact fp32 (the backward's tensor-core products read its upper 19 bits, its carried
                // decay term all of them), staged in the 128-byte-swizzled layout the tensor-map store expects: half h = columns 32h..32h+31,
                // row i at i*128 bytes, its 16-byte unit u at (u ^ (i & 7))
                unsigned char* stage = gs + G_WAQ;
                const int i = 16 * wg + (lane & 15);
#pragma unroll
                for (int qt = 0; qt < 4; ++qt) {
                    uint32_t sv[16];
                    tmem_ld16(tlane + C_S + 64 * ((cc + 1) & 1) + 16 * qt, sv);
                    tmem_ld_wait();
                    if (qt == 3) {
                        tc_fence_before();
                        mbar_arrive(&ctrl->rdone[grp]);
                    }
                    if (lane < 16) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int u = 4 * qt + j;
                            *reinterpret_cast<uint4*>(stage + (u >> 3) * 8192 + i * 128 + (((u & 7) ^ (i & 7)) << 4)) =
                                make_uint4(sv[4 * j], sv[4 * j + 1], sv[4 * j + 2], sv[4 * j + 3]);
                        }
                    }
                }
                fence_async_smem();
                group_bar(grp);
                if (wg == 0 && elect_one()) {
                    const int rec_row = (int)((bh * nchunks + cc + 1) * (CK_FLOATS / N));  // a record is 80 rows of 64 floats
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                                 ::"l"(&ckmap), "r"(0), "r"(rec_row), "r"(smem_u32(stage)) : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                                 ::"l"(&ckmap), "r"(32), "r"(rec_row), "r"(smem_u32(stage + 8192)) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                __syncwarp();
            } else if (sdst) {
                // final state: exact, straight from registers (32-byte stores: whole sectors of the lane's 256-byte row)
                float* d = sdst + (16 * wg + (lane & 15)) * N;
#pragma unroll
                for (int qt = 0; qt < 4; ++qt) {
                    uint32_t sv[16];
                    tmem_ld16(tlane + C_S + 64 * ((cc + 1) & 1) + 16 * qt, sv);
                    tmem_ld_wait();
                    if (qt == 3) {
                        tc_fence_before();
                        mbar_arrive(&ctrl->rdone[grp]);
                    }
#pragma unroll
                    for (int e = 0; e < 16; ++e) sv[e] = __float_as_uint(__uint_as_float(sv[e]) * STATE_UNSCALE);  // S = 2^64 S~
                    if (lane < 16) {
#pragma unroll
                        for (int q8 = 0; q8 < 2; ++q8)
                            asm volatile("st.global.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(d + 16 * qt + 8 * q8), "r"(sv[8 * q8]), "r"(sv[8 * q8 + 1]),
                                         "r"(sv[8 * q8 + 2]), "r"(sv[8 * q8 + 3]), "r"(sv[8 * q8 + 4]), "r"(sv[8 * q8 + 5]), "r"(sv[8 * q8 + 6]), "r"(sv[8 * q8 + 7]) : "memory");
                    }
                }
            } else {
                tc_fence_before();
                mbar_arrive(&ctrl->rdone[grp]);
            }
        };
        const int row = lane & 15, j0 = 16 * wg + 8 * (lane >> 4);
        if (grp < nchunks) issue_raw(grp, 0);
        int k = 0, cprev = -1;
        for (int c = grp; c < nchunks; c += G, ++k) {
            cp_async_wait<0>();
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // the matrix copy of the previous own chunk (its issuer only)
            group_bar(grp);
            // ---------------- decay scan, into registers ---------------------------------------------
            // One thread = one time step x 8 adjacent key channels.  The three transcendentals per
            // element go to the special-function unit: with the matrix products on tcgen05 the FMA
            // pipe and the issue slots are what this kernel runs out of, not MUFU throughput.
            float o[4][8], v[8], fwv[8];  // kwf, bwf are formed from kwi, bwi and fw when the tiles are written
            {
                const unsigned char* raw = gs + G_RAW + row * ROWB + (((j0 >> 3) ^ (row & 7)) << 4);
                float cum[8], q[8], kk[8], a[8], b[8];
                load8<IoT>(raw + 1 * RAW_TILE, cum);
                load8<IoT>(raw + 0 * RAW_TILE, q);
                load8<IoT>(raw + 2 * RAW_TILE, kk);
                load8<IoT>(raw + 3 * RAW_TILE, a);
                load8<IoT>(raw + 4 * RAW_TILE, b);
                load8<IoT>(raw + 5 * RAW_TILE, v);
                if (LN) {  // bonus dot sum_j r_j k_j bonus_j of this time step: 8 channels here, the rest by shuffle and in the epilogue
                    float acc = 0.f;
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc = fmaf(q[i] * kk[i], ctrl->lnp[2 * N + j0 + i], acc);
                    acc += __shfl_xor_sync(0xffffffffu, acc, 16);
                    if (lane < 16) ctrl->bdot[grp][k & 1][wg][row] = acc;
                }
                // log2 of the per-step decay: -exp(w) * log2(e); running sum along the 16 time rows
#pragma unroll
                for (int i = 0; i < 8; ++i)  // with the per-step floor (see MIN_STEP_LOG_DECAY)
                    cum[i] = fmaxf(ex2_approx(cum[i] * 1.4426950408889634f) * -1.4426950408889634f, MIN_STEP_LOG_DECAY * 1.4426950408889634f);  // log2 units
                if (TAIL && c + 1 == nchunks && row >= tail) {  // a row beyond the end of the sequence: no decay, the state passes through
#pragma unroll
                    for (int i = 0; i < 8; ++i) cum[i] = 0.f;
                }
                float step[8];  // this row's own log2 decay: P_{t-1} = 2^(cum_t - step_t), cheaper than a shuffle for the row above
#pragma unroll
                for (int i = 0; i < 8; ++i) step[i] = cum[i];
#pragma unroll
                for (int d = 1; d < 16; d <<= 1)
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float up = __shfl_up_sync(0xffffffffu, cum[i], d, 16);
                        if (row >= d) cum[i] += up;
                    }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    // P~_t = 2^64 P_t and its reciprocal (see ANCHOR_LN): both finite for cum >= -179 (2^-115 ~ e^-80)
                    const float ca = cum[i] + ANCHOR_LOG2;
                    const float cc = fmaxf(ca, -115.f);
                    const float incl = ex2_approx(cc);
                    const float inv = ex2_approx(-cc);
                    const float non = ex2_approx(fmaxf(ca - step[i], -115.f));
                    const float fw = __shfl_sync(0xffffffffu, incl, 15, 16);  // P~_L = 2^64 P_L (P_L itself may lie below fp32's normal range)
                    o[0][i] = q[i] * incl;   // wq
                    o[1][i] = a[i] * non;    // wa
                    o[2][i] = kk[i] * inv;   // kwi
                    o[3][i] = b[i] * inv;    // bwi
                    fwv[i] = fw;
                }
            }
            // ---------------- results of the previous own chunk (its operand tiles are free afterwards) --
            if (cprev >= 0) {
                read_results(cprev, k - 1);
                if (p.ckpt) {  // the staging tiles are operand tiles: wait until the bulk stores have read them
                    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    group_bar(grp);
                }
            }
            // ---------------- operand tiles -----------------------------------------------------------
            {
                const int jc = j0 >> 2;
                store8t<RND>(gs + G_WAQ + kchunk(row, jc, 2048), gs + G_WAQ + kchunk(row, jc + 1, 2048), o[1]);
                store8t<RND>(gs + G_WAQ + kchunk(16 + row, jc, 2048), gs + G_WAQ + kchunk(16 + row, jc + 1, 2048), o[0]);
                store8t<RND>(gs + G_KB + kchunk(row, jc, 2048), gs + G_KB + kchunk(row, jc + 1, 2048), o[2]);
                store8t<RND>(gs + G_KB + kchunk(16 + row, jc, 2048), gs + G_KB + kchunk(16 + row, jc + 1, 2048), o[3]);
                const int mo = (j0 >> 5) * 2048 + row * 128 + ((((j0 & 31) >> 3) ^ (row & 3)) << 5);
#pragma unroll
                for (int i = 0; i < 8; ++i) { o[2][i] = o[2][i] * fwv[i] * STATE_SCALE; o[3][i] = o[3][i] * fwv[i] * STATE_SCALE; }  // k P_L / P_t first, then 2^-64
                const bool flip = (row >> 2) & 1;
                store8mn<RND>(gs + G_KWF + mo, o[2], flip);
                store8mn<RND>(gs + G_BWF + mo, o[3], flip);
                store8mn<false>(gs + G_V + mo, v, flip);  // bf16 values are exact in TF32
                if (row == 15) {
                    unsigned char* df = gs + G_DF + (j0 >> 3) * 256;
#pragma unroll
                    for (int n = 0; n < 8; ++n) {
                        const float pl = fwv[n] * STATE_SCALE;  // P_L; where it underflows, so does S~ P_L
                        *reinterpret_cast<float*>(df + (n >> 2) * 128 + n * 16 + (n & 3) * 4) = RND ? rnd(pl) : pl;
                    }
                }
            }
            fence_async_smem();
            group_bar(grp);
            if (c + G < nchunks) issue_raw(c + G, (k + 1) & 1);
            // ---------------- the four score matrices as one product ---------------------------------
            if (wg == 0 && elect_one()) {
                const uint64_t dA = desc_kmajor(smem_u32(gs + G_WAQ), 2048), dB = desc_kmajor(smem_u32(gs + G_KB), 2048);
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) mma_ss(tmem + C_SCORE + 32 * grp, dA + (uint64_t)(ks * 16), dB + (uint64_t)(ks * 16), idesc(32, false, false), ks > 0);
                tc_commit(&ctrl->score[grp]);
            }
            __syncwarp();
            if (wg < 2) {
                mbar_wait<true>(&ctrl->score[grp], k & 1, ctrl, p.status);
                tc_fence_after();
                uint32_t sv[32];
                tmem_ld16(tlane + C_SCORE + 32 * grp, sv);
                tmem_ld16(tlane + C_SCORE + 32 * grp + 16, sv + 16);
                tmem_ld_wait();
                const int t = lane;
                if (wg == 0) {
                    // lane t: row t of AK (strictly lower) and of AB (strictly lower, kept transposed for the inverse)
                    if (lane < 16) {
                        float* ABt = reinterpret_cast<float*>(gs + G_ABT);
#pragma unroll
                        for (int qd = 0; qd < 4; ++qd) {
                            float4 x;
                            x.x = (4 * qd + 0 < t) ? rnd(__uint_as_float(sv[4 * qd + 0])) : 0.f;
                            x.y = (4 * qd + 1 < t) ? rnd(__uint_as_float(sv[4 * qd + 1])) : 0.f;
                            x.z = (4 * qd + 2 < t) ? rnd(__uint_as_float(sv[4 * qd + 2])) : 0.f;
                            x.w = (4 * qd + 3 < t) ? rnd(__uint_as_float(sv[4 * qd + 3])) : 0.f;
                            *reinterpret_cast<float4*>(gs + G_SC + kchunk(t, qd, 512)) = x;
                        }
#pragma unroll
                        for (int s = 0; s < 16; ++s) ABt[s * SCS + t] = (s < t) ? __uint_as_float(sv[16 + s]) : 0.f;
                    }
                    __syncwarp();
                    if (lane < 16) tri_inverse_tc(reinterpret_cast<const float*>(gs + G_ABT), gs + G_AI, lane);
                } else if (lane < 16) {
                    // lane t: row t of QK and QB (lower triangular including the diagonal)
#pragma unroll
                    for (int qd = 0; qd < 4; ++qd) {
                        float4 x, x2;
                        x.x = (4 * qd + 0 <= t) ? rnd(__uint_as_float(sv[4 * qd + 0])) : 0.f;
                        x.y = (4 * qd + 1 <= t) ? rnd(__uint_as_float(sv[4 * qd + 1])) : 0.f;
                        x.z = (4 * qd + 2 <= t) ? rnd(__uint_as_float(sv[4 * qd + 2])) : 0.f;
                        x.w = (4 * qd + 3 <= t) ? rnd(__uint_as_float(sv[4 * qd + 3])) : 0.f;
                        x2.x = (4 * qd + 0 <= t) ? rnd(__uint_as_float(sv[16 + 4 * qd + 0])) : 0.f;
                        x2.y = (4 * qd + 1 <= t) ? rnd(__uint_as_float(sv[16 + 4 * qd + 1])) : 0.f;
                        x2.z = (4 * qd + 2 <= t) ? rnd(__uint_as_float(sv[16 + 4 * qd + 2])) : 0.f;
                        x2.w = (4 * qd + 3 <= t) ? rnd(__uint_as_float(sv[16 + 4 * qd + 3])) : 0.f;
                        *reinterpret_cast<float4*>(gs + G_SC + kchunk(16 + t, qd, 512)) = x;
                        *reinterpret_cast<float4*>(gs + G_QB + kchunk(t, qd, 512)) = x2;
                    }
                }
            }
            fence_async_smem();
            tc_fence_before();
            mbar_arrive(&ctrl->full[grp]);
            // The chunk's four 16x16 matrices go into its checkpoint record: the three tiles [AK;QK], AI, QB are
            // contiguous in shared memory and are stored as they are, by one bulk copy issued after the chain
            // has been given the go-ahead.  The issuing thread waits on the same barrier as the chain (all 128
            // threads have written and fenced their part of the tiles by then).
#ifndef WKV7_TC_NOCKPT
            if (p.ckpt && wg == 0) {
                if (elect_one()) {
                    mbar_wait<true>(&ctrl->full[grp], k & 1, ctrl, p.status);
                    float* ckm = p.ckpt + (bh * nchunks + c) * (long long)CK_FLOATS + CK_MATS;
                    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                                 ::"l"(__cvta_generic_to_global(ckm)), "r"(smem_u32(gs + G_SC)), "n"(4 * L * L * 4) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                __syncwarp();
            }
#endif
            cprev = c;
        }
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory must outlive the last matrix copy
        if (cprev >= 0) {
            read_results(cprev, k - 1);
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // ... and the last state copy
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(NCOLS) : "memory");
    }
}

// Tensor map over the checkpoint buffer seen as an fp32 matrix [records * 80 rows][64 floats]; box = 64 rows x
// 32 floats (128 bytes) with the 128-byte swizzle.  Encoded through the runtime's driver-entry-point query
// (the library does not link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static bool encode_checkpoint_map(CUtensorMap* m, float* base, long long records) {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(records * (CK_FLOATS / N))};
    const cuuint64_t strides[1] = {(cuuint64_t)(N * sizeof(float))};
    const cuuint32_t box[2] = {32, (cuuint32_t)N};
    const cuuint32_t es[2] = {1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int G, bool RND, bool LN, bool TAIL> static int launch_tt(const FwdParams& p, cudaStream_t stream) {
    auto kern = wkv7_fwd_tc_kernel<G, RND, LN, TAIL>;
    const int smem = G * (LN ? G_BYTES_LN : G_BYTES_PLAIN) + (int)sizeof(Ctrl) + 1024;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    alignas(64) CUtensorMap ckmap;
    memset(&ckmap, 0, sizeof(ckmap));
    if (p.ckpt && !encode_checkpoint_map(&ckmap, p.ckpt, p.B * p.H * ((p.T + L - 1) / L))) return kLaunchFailed;
    kern<<<(unsigned)(p.B * p.H), 128 * (G + 1), smem, stream>>>(p, ckmap);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

template <int G, bool RND, bool LN> static int launch_t(const FwdParams& p, cudaStream_t stream) {
    return p.T % L ? launch_tt<G, RND, LN, true>(p, stream) : launch_tt<G, RND, LN, false>(p, stream);
}

// Exercises the bounded wait and the abort path with the kernel's own mbar_wait: one CTA of four warps;
// warp 0 waits (polling) and warp 1 waits (suspended) on mbarriers that nothing ever arrives on, with a
// short limit; warps 2 and 3 then wait on a third barrier with the full limit and must fall through at
// once because the CTA has aborted.  Leaves kDeviceTimeout in the status word and writes, per warp, the
// cycles its wait took.  No tensor memory, no tcgen05: nothing here can fault or hang.
__global__ void __launch_bounds__(128) bounded_wait_selftest_kernel(long long limit, int* status, long long* cycles) {
    __shared__ Ctrl ctrl;
    const int tid = threadIdx.x, warp = tid >> 5;
    if (tid == 0) {
        for (int g = 0; g < 3; ++g) mbar_init(&ctrl.full[g], 1);
        ctrl.abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    // clock reads that cannot be scheduled across the barrier / the wait: they take a value produced there as input
    auto clock_after = [](int dep) { long long t; asm volatile("mov.u64 %0, %%clock64;" : "=l"(t) : "r"(dep) : "memory"); return t; };
    const long long t0 = clock_after(__syncthreads_or(0));
    if (warp == 0) mbar_wait<false>(&ctrl.full[0], 0, &ctrl, status, limit);
    else if (warp == 1) mbar_wait<true>(&ctrl.full[1], 0, &ctrl, status, limit);
    const long long t1 = clock_after(__syncthreads_or(0));
    if (warp >= 2) mbar_wait<true>(&ctrl.full[2], 0, &ctrl, status);  // full limit, but the abort flag is up
    const long long t2 = clock_after(ctrl.abort);
    if ((tid & 31) == 0) cycles[warp] = warp < 2 ? t1 - t0 : t2 - t1;
}

}  // namespace tc

int launch_bounded_wait_selftest(long long limit_cycles, int* status, long long* cycles, cudaStream_t stream) {
    tc::bounded_wait_selftest_kernel<<<1, 128, 0, stream>>>(limit_cycles, status, cycles);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

template <bool LN> static int launch_ln(const FwdParams& p, int groups, cudaStream_t stream) {
    switch (groups) {
        case 2: return tc::launch_t<2, true, LN>(p, stream);
        case 3: return tc::launch_t<3, true, LN>(p, stream);
        case 4: return tc::launch_t<4, true, LN>(p, stream);
        case -2: return tc::launch_t<2, false, LN>(p, stream);
        case -3: return tc::launch_t<3, false, LN>(p, stream);
        case -4: return tc::launch_t<4, false, LN>(p, stream);
        default: return kBadShape;
    }
}

int launch_fwd_tc(const FwdParams& p, int groups, bool ln, cudaStream_t stream) {
    return ln ? launch_ln<true>(p, groups, stream) : launch_ln<false>(p, groups, stream);
}

}  // namespace wkv7
