// Shared device helpers for the sm_100a WKV7 kernels: TF32 warp-MMA fragments,
// bulk-async (TMA engine) row copies with mbarrier completion, bounded waits,
// and the status codes of the C ABI.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace wkv7 {

constexpr int N = 64;        // head size (value and key width of the state)
constexpr int L = 16;        // chunk length in time steps
constexpr int WARPS = 4;     // one warp per 16 value rows of the state
constexpr int THREADS = 32 * WARPS;
constexpr int OPS = N + 8;   // row stride (floats) of the [time][key] operand buffers
constexpr int SCS = L + 8;   // row stride (floats) of the [time][time] score buffers

// ---- status codes (mirrored in include/wkv7_sm100.h) -------------------------------------
enum Status : int {
    kOk = 0,
    kBadShape = -1,        // negative or inconsistent dimensions
    kBadHeadSize = -2,     // only N == 64 is built
    kBadChunk = -3,        // T is not a multiple of 16
    kBadAlign = -4,        // pointer or stride not 16-byte aligned
    kBadDtype = -5,
    kNullPointer = -6,
    kLaunchFailed = -7,    // cudaGetLastError() after launch was not cudaSuccess
    kTooLarge = -8,
    kDeviceTimeout = -9,   // a bounded device-side wait gave up (see wkv7_device_status)
};

// ---- IO element access ----------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f32(T x);
template <> __device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// ---- TF32 operands ---------------------------------------------------------------------------
// PREC == 1: one TF32 MMA per product (operands rounded to 10 mantissa bits, fp32 accumulate).
// PREC == 3: hi/lo split, three MMAs per product (error ~2^-21: the fp32 path).
__device__ __forceinline__ uint32_t tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

template <int PREC> struct Op {  // one scalar operand
    uint32_t h, l;
    __device__ __forceinline__ void set(float x) {
        h = tf32_rna(x);
        if (PREC == 3) l = tf32_rna(x - __uint_as_float(h));
        else l = 0;
    }
};

template <int PREC> struct FragA { Op<PREC> x[4]; };  // 16x8, (g,t) (g+8,t) (g,t+4) (g+8,t+4)
template <int PREC> struct FragB { Op<PREC> x[2]; };  // 8x8,  (k=t,n=g) (k=t+4,n=g)

__device__ __forceinline__ void mma_tf32_raw(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int PREC>
__device__ __forceinline__ void mma(float (&d)[4], const FragA<PREC>& a, const FragB<PREC>& b) {
    if (PREC == 3) {
        mma_tf32_raw(d, a.x[0].l, a.x[1].l, a.x[2].l, a.x[3].l, b.x[0].h, b.x[1].h);
        mma_tf32_raw(d, a.x[0].h, a.x[1].h, a.x[2].h, a.x[3].h, b.x[0].l, b.x[1].l);
    }
    mma_tf32_raw(d, a.x[0].h, a.x[1].h, a.x[2].h, a.x[3].h, b.x[0].h, b.x[1].h);
}

// Every contraction here sums over an index block of 8; the two k-slots a thread feeds
// (slot t and slot t+4) are mapped to the ADJACENT actual indices 2t and 2t+1 of the block,
// consistently for A and B.  That makes an accumulator tile (thread holds columns 2t, 2t+1)
// directly usable as the A operand of the next product, and turns every shared-memory
// operand fetch along the contraction index into one 8-byte load.

// A operand from an accumulator tile whose 8 columns are the contraction block.
template <int PREC> __device__ __forceinline__ FragA<PREC> fragA_from_acc(const float (&c)[4]) {
    FragA<PREC> f;
    f.x[0].set(c[0]);  // (g,   2t)
    f.x[1].set(c[2]);  // (g+8, 2t)
    f.x[2].set(c[1]);  // (g,   2t+1)
    f.x[3].set(c[3]);  // (g+8, 2t+1)
    return f;
}

// A operand from memory laid out [m][k] (row stride ld floats), rows m0+g, m0+g+8, block k0.
template <int PREC>
__device__ __forceinline__ FragA<PREC> fragA_mk(const float* p, int ld, int m0, int k0, int g, int t) {
    FragA<PREC> f;
    float2 lo = *reinterpret_cast<const float2*>(p + (m0 + g) * ld + k0 + 2 * t);
    float2 hi = *reinterpret_cast<const float2*>(p + (m0 + g + 8) * ld + k0 + 2 * t);
    f.x[0].set(lo.x); f.x[1].set(hi.x); f.x[2].set(lo.y); f.x[3].set(hi.y);
    return f;
}

// A operand from memory laid out [k][m] (the transpose), rows k0+2t, k0+2t+1, columns m0+g, m0+g+8.
template <int PREC>
__device__ __forceinline__ FragA<PREC> fragA_km(const float* p, int ld, int m0, int k0, int g, int t) {
    FragA<PREC> f;
    const float* r0 = p + (k0 + 2 * t) * ld + m0 + g;
    f.x[0].set(r0[0]); f.x[1].set(r0[8]); f.x[2].set(r0[ld]); f.x[3].set(r0[ld + 8]);
    return f;
}

// B operand from memory laid out [n][k]: row n0+g, block k0 (one 8-byte load).
template <int PREC>
__device__ __forceinline__ FragB<PREC> fragB_nk(const float* p, int ld, int n0, int k0, int g, int t) {
    FragB<PREC> f;
    float2 v = *reinterpret_cast<const float2*>(p + (n0 + g) * ld + k0 + 2 * t);
    f.x[0].set(v.x); f.x[1].set(v.y);
    return f;
}

// B operand from memory laid out [k][n]: rows k0+2t, k0+2t+1, column n0+g.
template <int PREC>
__device__ __forceinline__ FragB<PREC> fragB_kn(const float* p, int ld, int n0, int k0, int g, int t) {
    FragB<PREC> f;
    const float* r0 = p + (k0 + 2 * t) * ld + n0 + g;
    f.x[0].set(r0[0]); f.x[1].set(r0[ld]);
    return f;
}

// ---- mbarrier + bulk async copy (TMA engine, untiled) -----------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded wait on a phase parity: gives up after about a second of SM clocks.  Returns false if
// the limit ran out (the caller records it and leaves its loop); never spins forever.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    uint32_t addr = smem_u32(bar);
    long long start = 0;
    for (int it = 0;; ++it) {
        uint32_t done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (it == 64) start = clock64();
        if (it > 64 && clock64() - start > 2000000000LL) return false;
    }
}

// One contiguous row global -> shared; 16-byte aligned on both sides, size a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// exp() by precision class: the single-TF32 path tolerates the fast intrinsic.
template <int PREC> __device__ __forceinline__ float exp_p(float x) { return PREC == 3 ? expf(x) : __expf(x); }

// Tensor addressing shared by all launchers: element (b,t,h,0) of a [B,T,H,N] tensor.
struct Strides {
    long long b, t, h;  // in elements
};

}  // namespace wkv7
