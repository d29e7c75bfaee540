// Shared device helpers for the sm_100a WKV7 kernels: TF32 warp-MMA fragments, the chunk
// preparation (decay scan, triangular inverse), MUFU-free exp / reciprocal, cp.async copies, and
// the status codes of the C ABI.
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
// One checkpoint record per 16-step chunk, written by the forward for the backward: the fp32 state at
// the start of the chunk [N][N], then the chunk's four state-independent 16x16 matrices QK, QB (lower
// triangular), AK (strictly lower), AI = (I - AB)^-1.  The backward loads them instead of rebuilding
// them (two score products per warp and the 16-step inverse).  The matrices are kept in the layout of
// the tcgen05 forward's operand tiles, so that that kernel can copy them out with one bulk copy:
// three K-major tiles of 16-byte chunks, element (row, col) at float (row/8)*128 + (col/4)*32 + (row%8)*4
// + col%4; the first tile has 32 rows (AK in rows 0-15, QK in rows 16-31), then AI, then QB.
constexpr int CK_STATE = 0, CK_MATS = N * N;
constexpr int CK_SC = CK_MATS, CK_AI = CK_SC + 2 * L * L, CK_QB = CK_AI + L * L;
__host__ __device__ constexpr int ck_tile_at(int row, int chunk) { return (row >> 3) * 128 + chunk * 32 + (row & 7) * 4; }
constexpr int CK_FLOATS = CK_QB + L * L;  // 5120 floats = 20 KB
// Range of the decay within a chunk.  The kernels factor the decay between two steps of a chunk as P_t * (1 / P_s), with
// P_t the running decay product since the chunk start: over 16 steps of strong decay P_t leaves what fp32 holds.  Two
// measures keep every chunk inside, without a data-dependent branch:
//  * the products are kept as P~_t = 2^64 P_t and 1 / P~_t, so that both use the exponent range on either side of 1
//    (P~ from 2^64 down to e^-80, its reciprocal from 2^-64 up to e^80); every formula of the chunked algorithm is invariant
//    under P -> 2^64 P when the state is carried as S~ = 2^-64 S and its gradient as 2^64 dS (power-of-two scalings,
//    exact): initial states are scaled on the way in, final states and state gradients on the way out, and the
//    checkpoints hold S~;
//  * the per-step log-decay -exp(w) has a floor of -7.75 (16 * 7.75 = 124 = 80 + 64 ln 2): a step that would multiply the
//    state by less than e^-7.75 = 4.3e-4 (w > 2.05) multiplies it by e^-7.75.  RWKV-7 parameterises w <= -0.5 (per-step
//    log-decay >= -0.61) and never comes near it; N(-0.6, 0.5^2) inputs reach it at 5.3 sigma.
constexpr float ANCHOR_LN = 44.361419555836498f;      // 64 ln 2
constexpr float ANCHOR_LOG2 = 64.f;
constexpr float STATE_SCALE = 5.421010862427522e-20f;  // 2^-64
constexpr float STATE_UNSCALE = 18446744073709551616.f;  // 2^64
constexpr float MIN_CUM_LOG_DECAY = -(80.f + ANCHOR_LN);
constexpr float MIN_STEP_LOG_DECAY = -7.75f;

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
    kDeviceTimeout = -9,   // a bounded device-side wait (mbar_wait_bounded) gave up
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
// Round to nearest (ties away from zero) to 10 mantissa bits with two integer instructions.  The
// conversion instruction (cvt.rna.tf32.f32) and MUFU share the XU pipe, which profiling showed
// ~90% busy in these kernels; integer adds run on a pipe with headroom.  Finite inputs only.
__device__ __forceinline__ uint32_t tf32_rna(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }

// Value as it is kept in shared memory for later use as an MMA operand: in the single-TF32 class
// it is rounded once by its producer, so that the (many) consumers need no conversion.
template <int PREC> __device__ __forceinline__ float pre(float x) { return PREC == 1 ? __uint_as_float(tf32_rna(x)) : x; }

template <int PREC> struct Op {  // one scalar operand
    uint32_t h, l;
    __device__ __forceinline__ void set(float x) {
        h = tf32_rna(x);
        if (PREC == 3) l = tf32_rna(x - __uint_as_float(h));
        else l = 0;
    }
    // x was stored through pre<PREC>() or is exactly representable in TF32 (a bf16 value)
    __device__ __forceinline__ void setr(float x) {
        if (PREC == 1) { h = __float_as_uint(x); l = 0; }
        else set(x);
    }
    template <bool R> __device__ __forceinline__ void put(float x) { if (R) setr(x); else set(x); }
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

// Column swizzles of the fp32 tiles of the backward kernel.  A tile is read in two ways: along the
// contraction index (lanes = rows g, 8-byte loads at columns 2t) and across it (lanes = columns g,
// rows 2t and 2t+1).
// X = 1, for row strides of 8 or 24 mod 32 words (the padded operand and score tiles): the first
//   pattern is conflict-free by the padding, in the second rows 2t and 2t+4 fall on the same banks;
//   XOR-ing the column with 8 for rows 4..7 of every block of 8 rows separates them.
// X = 2, for unpadded 64-float rows: the column is XOR-ed with 8 * ((row ^ (row >> 2)) & 3), which gives
//   rows g = 0..3, rows g = 4..7, rows 0,2,4,6 and rows 1,3,5,7 four different values each, so both
//   patterns are conflict-free.
// Groups of 8 floats stay contiguous under both.  X = 0: plain layout.
template <int X> __device__ __forceinline__ int xcol(int row, int col) {
    return X == 1 ? (col ^ ((row & 4) << 1)) : X == 2 ? (col ^ (((row ^ (row >> 2)) & 3) << 3)) : col;
}

// A operand from memory laid out [m][k] (row stride ld floats), rows m0+g, m0+g+8, block k0.
// The loaders' template argument R says the source was stored through pre<PREC>(), X that the
// tile carries the column swizzle above.
template <int PREC, bool R = false, int X = 0>
__device__ __forceinline__ FragA<PREC> fragA_mk(const float* p, int ld, int m0, int k0, int g, int t) {
    FragA<PREC> f;
    float2 lo = *reinterpret_cast<const float2*>(p + (m0 + g) * ld + xcol<X>(m0 + g, k0 + 2 * t));
    float2 hi = *reinterpret_cast<const float2*>(p + (m0 + g + 8) * ld + xcol<X>(m0 + g + 8, k0 + 2 * t));
    f.x[0].template put<R>(lo.x); f.x[1].template put<R>(hi.x); f.x[2].template put<R>(lo.y); f.x[3].template put<R>(hi.y);
    return f;
}

// A operand from memory laid out [k][m] (the transpose), rows k0+2t, k0+2t+1, columns m0+g, m0+g+8.
template <int PREC, bool R = false, int X = 0>
__device__ __forceinline__ FragA<PREC> fragA_km(const float* p, int ld, int m0, int k0, int g, int t) {
    FragA<PREC> f;
    const int k = k0 + 2 * t;
    const float *r0 = p + k * ld, *r1 = r0 + ld;
    f.x[0].template put<R>(r0[xcol<X>(k, m0 + g)]); f.x[1].template put<R>(r0[xcol<X>(k, m0 + g + 8)]);
    f.x[2].template put<R>(r1[xcol<X>(k + 1, m0 + g)]); f.x[3].template put<R>(r1[xcol<X>(k + 1, m0 + g + 8)]);
    return f;
}

// B operand from memory laid out [n][k]: row n0+g, block k0 (one 8-byte load).
template <int PREC, bool R = false, int X = 0>
__device__ __forceinline__ FragB<PREC> fragB_nk(const float* p, int ld, int n0, int k0, int g, int t) {
    FragB<PREC> f;
    float2 v = *reinterpret_cast<const float2*>(p + (n0 + g) * ld + xcol<X>(n0 + g, k0 + 2 * t));
    f.x[0].template put<R>(v.x); f.x[1].template put<R>(v.y);
    return f;
}

// B operand from memory laid out [k][n]: rows k0+2t, k0+2t+1, column n0+g.
template <int PREC, bool R = false, int X = 0>
__device__ __forceinline__ FragB<PREC> fragB_kn(const float* p, int ld, int n0, int k0, int g, int t) {
    FragB<PREC> f;
    const int k = k0 + 2 * t;
    f.x[0].template put<R>(p[k * ld + xcol<X>(k, n0 + g)]); f.x[1].template put<R>(p[(k + 1) * ld + xcol<X>(k + 1, n0 + g)]);
    return f;
}

// exp(x) on the FMA and integer pipes only (for kernels whose special-function unit is the busier pipe: expand_loras,
// with seven transcendentals per element, splits them between the two).  2^t with t = x*log2(e): round(t) goes into the
// exponent field (the low mantissa bits of t + 1.5*2^23 are round(t); shifted left by 23 they land on the exponent, the
// constant's own bits fall off the top), the fraction in [-0.5, 0.5] through a degree-5 polynomial (relative error 2e-6,
// far below TF32 operand rounding).  x is clamped to [-80, 80].
__device__ __forceinline__ float exp_poly(float x) {
    const float t = fminf(fmaxf(x, -80.f), 80.f) * 1.4426950408889634f;
    const float tm = t + 12582912.f;
    const float f = t - (tm - 12582912.f);
    float p = 1.3333558e-3f;
    p = fmaf(p, f, 9.6181291e-3f);
    p = fmaf(p, f, 5.5504109e-2f);
    p = fmaf(p, f, 2.4022651e-1f);
    p = fmaf(p, f, 6.9314718e-1f);
    p = fmaf(p, f, 1.f);
    return __int_as_float(__float_as_int(p) + (__float_as_int(tm) << 23));
}
// 1/x for positive normal x without MUFU: exponent-flip seed (12% error), three Newton steps.
__device__ __forceinline__ float rcp_newton(float x) {
    float y = __int_as_float(0x7EF311C7 - __float_as_int(x));
    y = y * fmaf(-x, y, 2.f);
    y = y * fmaf(-x, y, 2.f);
    y = y * fmaf(-x, y, 2.f);
    return y;
}
// The same two functions on the special-function unit (one MUFU instruction each, relative error about 2^-22): what the
// WKV7 kernels use, whose XU pipe is otherwise idle (TF32 rounding is done with integer instructions).
__device__ __forceinline__ float exp_mufu(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(fminf(fmaxf(x, -80.f), 80.f) * 1.4426950408889634f));
    return y;
}
__device__ __forceinline__ float rcp_mufu(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// exp() and 1/x by precision class: MUFU for the single-TF32 class, libdevice for the fp32 class.
template <int PREC> __device__ __forceinline__ float exp_p(float x) { return PREC == 3 ? expf(x) : exp_mufu(x); }
template <int PREC> __device__ __forceinline__ float rcp_p(float x) { return PREC == 3 ? 1.f / x : rcp_mufu(x); }
// P~ = 2^64 exp(c) for a running log-decay c <= 0 (clamped at MIN_CUM_LOG_DECAY).  fp32 class: exact power-of-two scaling
// of expf(c) wherever that has not underflowed.
template <int PREC> __device__ __forceinline__ float decay_up(float c) {
    if (PREC == 3) return c >= -80.f ? expf(c) * STATE_UNSCALE : expf(fmaxf(c, MIN_CUM_LOG_DECAY) + ANCHOR_LN);
    return exp_mufu(c + ANCHOR_LN);  // exp_mufu clamps its argument at -80
}

// ---- decay scan (state-independent chunk preparation, shared by forward and backward) ----------
// 8 consecutive IO elements (16 or 32 bytes) -> floats
template <typename T> __device__ __forceinline__ void load8(const unsigned char* p, float (&f)[8]);
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const unsigned char* p, float (&f)[8]) {
    const uint4 u = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        f[2 * i] = __uint_as_float(w[i] << 16);
        f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}
template <> __device__ __forceinline__ void load8<float>(const unsigned char* p, float (&f)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 16);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
// Eight floats of a row in two 16-byte stores.  With the 72-float row pitch rows r and r + 4 start on the same banks
// (also under the column swizzle, which moves both by the same 8 floats), and the eight lanes of a quarter-warp are
// rows r..r+7: `flip` (set for rows 4..7 of every eight) makes those lanes store their second half first, so that
// each of the two instructions touches eight different 16-byte bank groups.
__device__ __forceinline__ void store8(float* p, const float (&f)[8], bool flip = false) {
    float x[4], y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[i] = flip ? f[4 + i] : f[i];  // goes out first
        y[i] = flip ? f[i] : f[4 + i];
    }
    const int off = flip ? 4 : 0;
    *reinterpret_cast<float4*>(p + off) = make_float4(x[0], x[1], x[2], x[3]);
    *reinterpret_cast<float4*>(p + (4 - off)) = make_float4(y[0], y[1], y[2], y[3]);
}

// One thread = one time step x 8 adjacent key channels (lane = row + 16 * channel-half, warp =
// 16-channel group).  The running log-decay along the 16 time rows is a 4-step warp-shuffle scan,
// eight independent channels per thread keep the pipes busy, and all shared-memory traffic is 16
// bytes wide.  Writes wq = q*P_t, wa = a*P_{t-1}, kwi = k/P_t, bwi = b/P_t (row stride OPS), the
// chunk decay fw = P_L, and optionally the running log-decay and the per-step log-decay.
// tq/tw/tk/ta/tb: staging tiles with row stride `rowb` bytes.
// RAWX: the staging tiles have unpadded 128-byte rows (bf16) whose eight 16-byte segments are XOR-ed
// with (row % 8), so that cp.async writes whole aligned lines and these 16-byte reads stay conflict-free.
// live: number of time steps of this chunk that exist (16 except in the last chunk of a sequence whose length
// is not a multiple of 16); rows beyond it carry zero inputs and a per-step log-decay of zero, so that the state
// passes through them unchanged.
template <typename IoT, int PREC, int X = 0, bool RAWX = false>
__device__ __forceinline__ void decay_scan(const unsigned char* tq, const unsigned char* tw, const unsigned char* tk,
                                           const unsigned char* ta, const unsigned char* tb, int rowb, float* wq, float* wa,
                                           float* kwi, float* bwi, float* fw, float* cum_out, float* lw_out, int warp, int lane,
                                           int live = L) {
    const int row = lane & 15, j0 = 16 * warp + 8 * (lane >> 4);
    const int off = RAWX ? row * rowb + ((((j0 * (int)sizeof(IoT)) >> 4) ^ (row & 7)) << 4) : row * rowb + j0 * (int)sizeof(IoT);
    float lw[8], cum[8], q[8], k[8], a[8], b[8];
    load8<IoT>(tw + off, lw);
    load8<IoT>(tq + off, q);
    load8<IoT>(tk + off, k);
    load8<IoT>(ta + off, a);
    load8<IoT>(tb + off, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) lw[i] = row < live ? fmaxf(-exp_p<PREC>(lw[i]), MIN_STEP_LOG_DECAY) : 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) cum[i] = lw[i];
#pragma unroll
    for (int d = 1; d < 16; d <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float up = __shfl_up_sync(0xffffffffu, cum[i], d, 16);
            if (row >= d) cum[i] += up;
        }
    // P_t from one exp (argument clamped so that P_t and 1/P_t stay finite), 1/P_t from a reciprocal.
    float o[4][8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const float incl = decay_up<PREC>(cum[i]);   // P~_t
        const float inv = rcp_p<PREC>(incl);
        // P_{t-1} = exp(cum_t - lw_t) (row 0: exp(0) = 1): one more exponential on the idle special-function unit is
        // cheaper here than fetching the row above with a shuffle
        const float non = decay_up<PREC>(cum[i] - lw[i]);
        o[0][i] = pre<PREC>(q[i] * incl);
        o[1][i] = pre<PREC>(a[i] * non);
        o[2][i] = pre<PREC>(k[i] * inv);
        o[3][i] = pre<PREC>(b[i] * inv);
        if (row == 15) fw[j0 + i] = incl;  // P~_16 = 2^64 P_16: users multiply by it first and by 2^-64 afterwards
    }
    const int at = row * OPS + xcol<X>(row, j0);
    const bool flip = (row >> 2) & 1;
    store8(wq + at, o[0], flip);
    store8(wa + at, o[1], flip);
    store8(kwi + at, o[2], flip);
    store8(bwi + at, o[3], flip);
    if (cum_out) store8(cum_out + at, cum, flip);
    if (lw_out) store8(lw_out + at, lw, flip);
}

// Column `col` of AI = (I - AB)^-1 for a strictly lower-triangular 16x16 AB, one lane per column.
// ABt holds AB TRANSPOSED (ABt[s][tq] = AB[tq][s], row stride SCS), so that everything step s needs
// is one contiguous row.  Right-looking substitution: as soon as entry s is final it is pushed
// into all later rows, so the dependent chain is 16 steps long rather than 120.
template <int S_> __device__ __forceinline__ void tri_fetch_row(float (&dst)[L], const float* ABt) {
    // entries tq > S_ of row S_ of ABt, in 16-byte pieces
#pragma unroll
    for (int v = (S_ + 1) / 4; v < L / 4; ++v) {
        const float4 x = *reinterpret_cast<const float4*>(ABt + S_ * SCS + 4 * v);
        dst[4 * v] = x.x; dst[4 * v + 1] = x.y; dst[4 * v + 2] = x.z; dst[4 * v + 3] = x.w;
    }
}
template <int PREC, int S_, int X>
__device__ __forceinline__ void tri_step(float (&r)[L], const float (&c)[L], float (&cn)[L], const float* ABt, float* AI, int col) {
    if (S_ + 1 < L) tri_fetch_row<(S_ + 1 < L ? S_ + 1 : 0)>(cn, ABt);  // one step ahead of its use
    const float ms = r[S_];
    AI[S_ * SCS + xcol<X>(S_, col)] = pre<PREC>(ms);
#pragma unroll
    for (int tq = S_ + 1; tq < L; ++tq) r[tq] = fmaf(c[tq], ms, r[tq]);
}
template <int PREC, int X = 0> __device__ __forceinline__ void tri_inverse_column(const float* ABt, float* AI, int col) {
    float r[L], ca[L], cb[L];
#pragma unroll
    for (int tq = 0; tq < L; ++tq) r[tq] = (tq == col) ? 1.f : 0.f;
    tri_fetch_row<0>(ca, ABt);
    tri_step<PREC, 0, X>(r, ca, cb, ABt, AI, col);   tri_step<PREC, 1, X>(r, cb, ca, ABt, AI, col);
    tri_step<PREC, 2, X>(r, ca, cb, ABt, AI, col);   tri_step<PREC, 3, X>(r, cb, ca, ABt, AI, col);
    tri_step<PREC, 4, X>(r, ca, cb, ABt, AI, col);   tri_step<PREC, 5, X>(r, cb, ca, ABt, AI, col);
    tri_step<PREC, 6, X>(r, ca, cb, ABt, AI, col);   tri_step<PREC, 7, X>(r, cb, ca, ABt, AI, col);
    tri_step<PREC, 8, X>(r, ca, cb, ABt, AI, col);   tri_step<PREC, 9, X>(r, cb, ca, ABt, AI, col);
    tri_step<PREC, 10, X>(r, ca, cb, ABt, AI, col);  tri_step<PREC, 11, X>(r, cb, ca, ABt, AI, col);
    tri_step<PREC, 12, X>(r, ca, cb, ABt, AI, col);  tri_step<PREC, 13, X>(r, cb, ca, ABt, AI, col);
    tri_step<PREC, 14, X>(r, ca, cb, ABt, AI, col);  tri_step<PREC, 15, X>(r, cb, ca, ABt, AI, col);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Bounded wait for the phase of an mbarrier with the given parity; the one wait every kernel of this library uses.
// Returns at once when the CTA has aborted.  When `limit` clocks pass without the phase completing it raises the
// CTA's abort flag (every later wait then falls through), records kDeviceTimeout in the device status word and
// returns: a lost copy or a missing arrival ends with an error code, never with a hung GPU.
// SLEEP: the thread is suspended by the hardware (try_wait with a time hint) instead of polling.
constexpr long long MBAR_WAIT_LIMIT = 1LL << 28;  // clocks (~0.15 s): far beyond any legitimate wait
template <bool SLEEP>
__device__ __forceinline__ void mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile int* abort, int* status, long long limit = MBAR_WAIT_LIMIT) {
    const uint32_t addr = smem_u32(bar);
    long long start = 0;
    // (Polling variant: the abort flag is read after every failed probe.  A tighter loop that looked at it only every
    // 32nd probe made the tcgen05 forward 1.3 % slower: the chain's polls take issue slots from the working warps.)
    for (int spin = 0;; ++spin) {
        uint32_t ok;
        if (SLEEP)
            asm volatile("{\n.reg .pred P;\nmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\nselp.u32 %0, 1, 0, P;\n}\n"
                         : "=r"(ok) : "r"(addr), "r"(parity), "r"(4000u) : "memory");
        else
            asm volatile("{\n.reg .pred P;\nmbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\nselp.u32 %0, 1, 0, P;\n}\n"
                         : "=r"(ok) : "r"(addr), "r"(parity) : "memory");
        if (ok) return;
        if (*abort) return;
        if (spin == 0) start = clock64();
        else if ((SLEEP || (spin & 63) == 0) && clock64() - start > limit) {
            *abort = 1;
            *reinterpret_cast<volatile int*>(status) = (int)kDeviceTimeout;  // the launchers always pass the status word (host-visible)
            __threadfence_system();
            return;
        }
    }
}

// 16-byte asynchronous copy global -> shared through the load/store unit (no TMA request)
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem)), "l"(gmem) : "memory");
}
// The same copy for a row that may lie beyond the end of the sequence: when `live` is false nothing is read and the
// 16 bytes are filled with zeros (the source address must still be a valid one).
__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool live) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem), "r"(live ? 16 : 0) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }


// Tensor addressing shared by all launchers: element (b,t,h,0) of a [B,T,H,N] tensor.
struct Strides {
    long long b, t, h;  // in elements
};

}  // namespace wkv7
