// WKV7 backward for sm_100a: one CTA per (batch, head) chain, 4 warps, chunks of 16 time steps
// walked in reverse; the gradient dS of the state stays in registers across chunks.
//
// Replaces the reference's backward_kernel (wind_rwkv/rwkv7/attn.cu:131-326).  The forward
// intermediates of a chunk are rebuilt from the fp32 chunk-start state S0 the forward wrote (exact fp32; in the
// single-TF32 class the tensor core reads the upper 19 bits of it as an operand, no conversion instruction).
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
// With LN = true the kernel is the backward of the fused attn_ln op (reference:
// wind_rwkv/rwkv7/attn_ln.cu:40-104, 237-464): `dy` is then the gradient of the fused output; the
// chunk's recurrence output Y is rebuilt, the GroupNorm / bonus / gate backward runs on it in the
// transposed register layout (three cross-warp reductions per time step through shared memory),
// and its result replaces dY for everything below.  Parameter gradients are accumulated in
// registers over the whole chain and written as per-(batch, head) partials (no atomics).
//
// Stage B (rows = value index, per warp, no cross-warp traffic): U^T, du^T, dabu^T, dV^T, dS0.
// Stage C (contractions over the value index, warp owns 16 key columns): the four score
// gradients and DA, DQ, DB, DK with S0 and dSf read from shared memory.
#include <cuda.h>
#include <cstddef>
#include <cstring>

#include "wkv7_kernels.h"

namespace wkv7 {

// Tensor maps of the five [time x key] outputs (dq, dw, dk, da, db) for the bulk-store epilogue.
// ck: the checkpoint states, for the bulk tensor loads of the chunk-start state.
struct alignas(64) OutMaps { CUtensorMap m[7]; CUtensorMap ck, ckm; };  // m[5]: dv, m[6]: dg (attn_ln); ck, ckm: checkpoint states, matrices

constexpr int SS = N + 8;  // row stride (floats) of the [value][key] state buffers
constexpr int MAT_BLK = 8 * 4 * SCS;  // floats per block of the matrices buffer
static_assert(SCS == L + 8, "the matrix loads copy boxes of L + 8 floats per row");
// All fp32 tiles of this kernel (operands, scores, score gradients, U, dabu, the two state buffers)
// carry the column swizzle xcol<1>() of wkv7_common.cuh: each is read both along and across its
// contraction index.

// Staging tiles [time][channel] in the IO dtype.  bf16: 128-byte rows, the eight 16-byte segments of a
// row XOR-ed with (row % 8) (cp.async then writes whole aligned 128-byte lines: padded rows cost it
// 2.5 times the shared-memory wavefronts); fp32: 256-byte rows padded by 16 bytes.
template <typename IoT> struct BwdLayout {
    static constexpr bool SWZ = sizeof(IoT) == 2;
    static constexpr int ROWB = N * (int)sizeof(IoT) + (SWZ ? 0 : 16);
    // byte offset of element (row, col)
    __device__ static __forceinline__ int at(int row, int col) {
        const int b = col * (int)sizeof(IoT);
        return SWZ ? row * ROWB + ((((b >> 4) ^ (row & 7)) << 4) | (b & 15)) : row * ROWB + b;
    }
    static constexpr int TILEB = L * ROWB;
    static constexpr int YS = (sizeof(IoT) == 2) ? 24 : 20;
};

template <typename IoT, int PREC, bool LN> struct BwdSmem {
    using Lay = BwdLayout<IoT>;
    alignas(16) unsigned char st_in[5][Lay::TILEB];  // q, w, k, a, b (dead after the scan)
    alignas(16) unsigned char st_v[2][Lay::TILEB];
    alignas(16) unsigned char st_dy[2][Lay::TILEB];
    alignas(16) unsigned char st_g[LN ? 2 : 1][LN ? Lay::TILEB : 16];
    alignas(16) float wq[L * OPS], wa[L * OPS], kwi[L * OPS], bwi[L * OPS];
    alignas(16) float cum[L * OPS];
    alignas(16) float lw[PREC == 3 ? L * OPS : 4];   // single-TF32 path derives it from cum
    // The chunk's four 16x16 matrices AK, QK, AI, QB (matrix m, row r: row group 2m + r/8 of the record's 64-row operand
    // tile), filled by two bulk tensor loads: rows with (r & 4) == 0 form a dense block of [8 row groups][4 rows][24 floats]
    // (16 values, 8 floats of fill), the other rows a second block whose rows start with the fill.  See mat_at().
    alignas(128) float mats[2 * MAT_BLK];
    // Score gradients (stage C).  While stage B runs they are dead, and the same bytes serve as
    // the per-warp transposition scratch for dv / dg and as the GroupNorm reduction buffers.
    static constexpr int SCRATCH_FLOATS = WARPS * L * Lay::YS * (int)sizeof(IoT) / 4 + WARPS * L * 5;
    static constexpr int SGRAD_FLOATS = 4 * L * SCS > SCRATCH_FLOATS ? 4 * L * SCS : SCRATCH_FLOATS;
    alignas(LN && sizeof(IoT) == 2 ? 1024 : 16) float sgrad[SGRAD_FLOATS];  // score gradient i at sgrad + i * L * SCS
    // attn_ln: Ut, Dt, Yt are dead between stage C and the next chunk's stage B and double as the output staging tiles
    alignas(LN ? 1024 : 16) float Ut[L * OPS];  // U and dabu as [time][value]
    alignas(16) float Dt[L * OPS];
    alignas(16) float Yt[LN ? L * OPS : 4];      // recurrence-output gradient as [time][value]
    // Chunk-start state [value][key], filled by two bulk tensor loads per chunk: rows with (row & 4) == 0 form a dense
    // block of 32 rows x 72 floats (64 values, 8 floats of fill), the other rows a second block whose rows start with
    // the 8 floats of fill (the load starts at column -8).  See s0_at().
    alignas(128) float S0s[N * SS];
    alignas(16) float dSs[N * SS];  // dSf as [value][key], column swizzle 1
    alignas(8) uint64_t s0_bar;     // completion of the state loads
    volatile int abort;             // set when a bounded wait gave up
    alignas(16) float fw[N];
    alignas(16) float Gp[2][WARPS][N];
    alignas(16) float lnp[LN ? 3 * N : 4];
    float bdot[L], sbon[L];
    // bf16: the five [16 x 64] output tiles of a chunk, 128-byte rows with the 16-byte unit index XOR-ed
    // with (row % 8) (what a 128-byte-swizzle tensor map expects), stored by five bulk tensor copies per chunk
    static constexpr bool TMA_OUT = sizeof(IoT) == 2;
    // (attn: a sixth tile carries dv, which is formed one stage earlier)
    // (attn_ln: the five tiles alias Ut, Dt, Yt; only dv's tile lives here)
    alignas(TMA_OUT ? 1024 : 16) unsigned char ostage[TMA_OUT ? (LN ? 1 : 6) * 2048 : 16];
    __device__ __forceinline__ unsigned char* out_tiles() { return LN ? reinterpret_cast<unsigned char*>(Ut) : ostage; }
    __device__ __forceinline__ unsigned char* dv_tile() { return ostage + (TMA_OUT && !LN ? 5 * 2048 : 0); }
};
static_assert(sizeof(BwdSmem<__nv_bfloat16, 1, false>) <= 115712, "bf16 backward must fit two CTAs per SM");
static_assert(sizeof(BwdSmem<__nv_bfloat16, 1, true>) <= 115712, "bf16 attn_ln backward must fit two CTAs per SM");
using BwdSmemLnBf16 = BwdSmem<__nv_bfloat16, 1, true>;
static_assert(offsetof(BwdSmemLnBf16, Yt) - offsetof(BwdSmemLnBf16, Ut) == 2 * L * OPS * 4 && 3 * L * OPS * 4 >= 5 * 2048 &&
                  offsetof(BwdSmemLnBf16, Ut) % 1024 == 0,
              "attn_ln output staging tiles alias Ut, Dt, Yt");

template <typename IoT> __device__ __forceinline__ float bst_elem(const unsigned char* tile, int row, int col) {
    return to_f32<IoT>(*reinterpret_cast<const IoT*>(tile + BwdLayout<IoT>::at(row, col)));
}
// two adjacent elements (col even) of a staging tile
template <typename IoT> __device__ __forceinline__ float2 bst_pair(const unsigned char* tile, int row, int col);
template <> __device__ __forceinline__ float2 bst_pair<float>(const unsigned char* tile, int row, int col) {
    return *reinterpret_cast<const float2*>(tile + BwdLayout<float>::at(row, col));
}
template <> __device__ __forceinline__ float2 bst_pair<__nv_bfloat16>(const unsigned char* tile, int row, int col) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(tile + BwdLayout<__nv_bfloat16>::at(row, col)));
}
// A operand [m = time][k = value] straight from a staging tile laid out [time][value]
template <typename IoT, int PREC>
__device__ __forceinline__ FragA<PREC> fragA_mk_st(const unsigned char* tile, int k0, int g, int t4) {
    FragA<PREC> f;
    float2 lo = bst_pair<IoT>(tile, g, k0 + 2 * t4), hi = bst_pair<IoT>(tile, g + 8, k0 + 2 * t4);
    constexpr bool EXACT = sizeof(IoT) == 2;  // a bf16 value is a TF32 value
    f.x[0].template put<EXACT>(lo.x); f.x[1].template put<EXACT>(hi.x); f.x[2].template put<EXACT>(lo.y); f.x[3].template put<EXACT>(hi.y);
    return f;
}
// B operand [k = value][n = time] from a staging tile laid out [time][value]
template <typename IoT, int PREC>
__device__ __forceinline__ FragB<PREC> fragB_nk_st(const unsigned char* tile, int n0, int k0, int g, int t4) {
    FragB<PREC> f;
    float2 v = bst_pair<IoT>(tile, n0 + g, k0 + 2 * t4);
    constexpr bool EXACT = sizeof(IoT) == 2;
    f.x[0].template put<EXACT>(v.x); f.x[1].template put<EXACT>(v.y);
    return f;
}
// A operand [m = value][k = time] (the transpose) from a staging tile laid out [time][value]
template <typename IoT, int PREC>
__device__ __forceinline__ FragA<PREC> fragA_km_st(const unsigned char* tile, int m0, int k0, int g, int t4) {
    FragA<PREC> f;
    const int tr = k0 + 2 * t4, vc = m0 + g;
    constexpr bool EXACT = sizeof(IoT) == 2;
    f.x[0].template put<EXACT>(bst_elem<IoT>(tile, tr, vc));
    f.x[1].template put<EXACT>(bst_elem<IoT>(tile, tr, vc + 8));
    f.x[2].template put<EXACT>(bst_elem<IoT>(tile, tr + 1, vc));
    f.x[3].template put<EXACT>(bst_elem<IoT>(tile, tr + 1, vc + 8));
    return f;
}

template <typename IoT> __device__ __forceinline__ void store_pair(IoT* p, float x, float y);
template <> __device__ __forceinline__ void store_pair<float>(float* p, float x, float y) {
    *reinterpret_cast<float2*>(p) = make_float2(x, y);
}
template <> __device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16* p, float x, float y) {
    *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(x, y);
}

// Epilogue stores.  A thread holds columns (2*t4, 2*t4+1) of two adjacent 8-column tiles; stored as they
// are, a warp-wide store writes 16 bytes per row (half a 32-byte sector).  Lanes t4 and t4^1 swap one
// pair, after which the even lane holds columns 4m..4m+3 of the first tile and the odd lane the same
// columns of the second tile (m = t4 / 2): 8-byte stores (bf16), whole sectors per row.
// `row` points at column 16*warp of the output row; live = false (rows beyond the end of the sequence) keeps the
// exchange but skips the store.
__device__ __forceinline__ void store_quad(__nv_bfloat16* row, float a0, float a1, float b0, float b1, int t4, bool live) {
    const __nv_bfloat162 p0 = __floats2bfloat162_rn(a0, a1), p1 = __floats2bfloat162_rn(b0, b1);  // tile 0, tile 1
    const uint32_t u0 = *reinterpret_cast<const uint32_t*>(&p0), u1 = *reinterpret_cast<const uint32_t*>(&p1);
    const bool odd = t4 & 1;
    const uint32_t got = __shfl_xor_sync(0xffffffffu, odd ? u0 : u1, 1);
    const uint2 v = odd ? make_uint2(got, u1) : make_uint2(u0, got);
    if (live) *reinterpret_cast<uint2*>(row + 8 * (t4 & 1) + 4 * (t4 >> 1)) = v;
}
__device__ __forceinline__ void store_quad(float* row, float a0, float a1, float b0, float b1, int t4, bool live) {
    const bool odd = t4 & 1;
    const float g0 = __shfl_xor_sync(0xffffffffu, odd ? a0 : b0, 1), g1 = __shfl_xor_sync(0xffffffffu, odd ? a1 : b1, 1);
    const float4 v = odd ? make_float4(g0, g1, b0, b1) : make_float4(a0, a1, g0, g1);
    if (live) *reinterpret_cast<float4*>(row + 8 * (t4 & 1) + 4 * (t4 >> 1)) = v;
}

// Offset of element (row = value, col = key) of the chunk-start state in shared memory.  With the 72-float row pitch
// (8 banks) both access patterns of the tensor-core fragments are free of bank conflicts: lanes over rows g = 0..3 or
// 4..7 of one block with 8-byte loads, and lanes over rows 0,2,4,6 (or 1,3,5,7) x 8 columns, where the second block's
// shift by 8 floats separates rows r and r + 4.
constexpr int S0_BLK = 32 * SS;
// Offset of element (row, col) of matrix m (0 AK, 1 QK, 2 AI, 3 QB) in the matrices buffer; the same split by row bit 2
// and the same shift of the second block by 8 floats as for the state, here with the 24-float row pitch.
__device__ __forceinline__ int mat_at(int m, int row, int col) {
    return ((row >> 2) & 1) * (MAT_BLK + 8) + ((2 * m + (row >> 3)) * 4 + (row & 3)) * SCS + col;
}
__device__ __forceinline__ int s0_at(int row, int col) {
    return ((row >> 2) & 1) * (S0_BLK + 8) + (((row >> 3) << 2) | (row & 3)) * SS + col;
}
static_assert(SS == N + 8, "the state loads copy boxes of N + 8 floats per row");

// Waits (polling, bounded) for a phase of the state-load barrier: the library's common wait, which the forward's
// self-test exercises on barriers nothing arrives on.
__device__ __forceinline__ void s0_wait(uint64_t* bar, uint32_t parity, volatile int* abort, int* status) {
    mbar_wait_bounded<false>(bar, parity, abort, status);
}

// TAIL: the sequence length is not a multiple of 16 (an instantiation of its own, so that whole-chunk sequences carry
// none of the row tests).
template <typename IoT, int PREC, bool LN, bool TAIL>
__global__ void __launch_bounds__(THREADS) wkv7_bwd_kernel(BwdParams p, const __grid_constant__ OutMaps omaps) {
    using Lay = BwdLayout<IoT>;
    using Smem = BwdSmem<IoT, PREC, LN>;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    constexpr bool TMA_OUT = Smem::TMA_OUT;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const long long bh = blockIdx.x;
    const long long bi = bh / p.H, hi = bh % p.H;
    const long long base = bi * p.st.b + hi * p.st.h;
    const int nchunks = (int)((p.T + L - 1) / L);  // the last chunk may be partial: its missing rows read as zeros
    constexpr bool has_tail = TAIL;
    const IoT* gin[5] = {(const IoT*)p.r + base, (const IoT*)p.w + base, (const IoT*)p.k + base,
                         (const IoT*)p.a + base, (const IoT*)p.b + base};
    const IoT* gv = (const IoT*)p.v + base;
    const IoT* gdy = (const IoT*)p.dy + base;
    IoT* gout[5] = {(IoT*)p.dr + base, (IoT*)p.dw + base, (IoT*)p.dk + base, (IoT*)p.da + base, (IoT*)p.db + base};
    IoT* gdv = (IoT*)p.dv + base;
    const IoT* gg = LN ? (const IoT*)p.g + base : nullptr;
    IoT* gdg = LN ? (IoT*)p.dg + base : nullptr;
    constexpr uint32_t ROW_BYTES = N * sizeof(IoT);

    if (LN) {
        for (int i = tid; i < 3 * N; i += THREADS) sm.lnp[i] = p.params[(long long)(i / N) * p.H * N + hi * N + (i % N)];
    }
    // stage-B scratch aliased onto the score-gradient buffers
    IoT* const dvsc = reinterpret_cast<IoT*>(sm.sgrad) + warp * (L * Lay::YS);
    float* const red = sm.sgrad + (WARPS * L * Lay::YS * (int)sizeof(IoT)) / 4;  // [WARPS][L][2]
    float* const red2 = red + WARPS * L * 2;                                             // [WARPS][L][3]
    float dlnw_acc[2] = {0.f, 0.f}, dlnb_acc[2] = {0.f, 0.f}, dbon_acc[2][2] = {{0.f, 0.f}, {0.f, 0.f}};
    // Carried decay term for the last chunk: sum_i dsT[i,:] * sT[i,:] (zero without dsT).
    for (int i = tid; i < WARPS * N; i += THREADS) sm.Gp[1][i / N][i % N] = 0.f;
    if (tid == 0) {
        sm.abort = 0;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&sm.s0_bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (p.dsT && p.sT && tid < N) {
        const float* d = p.dsT + bh * N * N;
        const float* s = p.sT + bh * N * N;
        float acc = 0.f;
        for (int i = 0; i < N; ++i) acc += d[i * N + tid] * s[i * N + tid];
        sm.Gp[1][0][tid] = acc;
    }

    // iteration `it` handles chunk c = nchunks-1-it.  All threads fetch 16-byte pieces with
    // cp.async; a chunk's loads are issued one iteration ahead and waited for before the barrier
    // that ends the iteration.
    constexpr int CH = ROW_BYTES / 16;
    auto issue_in = [&](int c) {
        for (int i = tid; i < 5 * L * CH; i += THREADS) {
            const int ten = i / (L * CH), row = (i / CH) % L, ch = i % CH;
            const long long tt = (long long)c * L + row;
            if (has_tail) cp_async16_zfill(sm.st_in[ten] + Lay::at(row, ch * (16 / (int)sizeof(IoT))),
                             reinterpret_cast<const unsigned char*>(gin[ten] + (tt < p.T ? tt : p.T - 1) * p.st.t) + ch * 16, tt < p.T);
            else cp_async16(sm.st_in[ten] + Lay::at(row, ch * (16 / (int)sizeof(IoT))), reinterpret_cast<const unsigned char*>(gin[ten] + tt * p.st.t) + ch * 16);
        }
    };
    auto issue_vdy = [&](int c, int s) {
        for (int i = tid; i < (LN ? 3 : 2) * L * CH; i += THREADS) {
            const int ten = i / (L * CH), row = (i / CH) % L, ch = i % CH;
            const long long tt = (long long)c * L + row;
            const IoT* src = (ten == 0 ? gv : ten == 1 ? gdy : gg) + (!TAIL || tt < p.T ? tt : p.T - 1) * p.st.t;
            unsigned char* dst = (ten == 0 ? sm.st_v[s] : ten == 1 ? sm.st_dy[s] : sm.st_g[LN ? s : 0]) + Lay::at(row, ch * (16 / (int)sizeof(IoT)));
            if (has_tail) cp_async16_zfill(dst, reinterpret_cast<const unsigned char*>(src) + ch * 16, tt < p.T);
            else cp_async16(dst, reinterpret_cast<const unsigned char*>(src) + ch * 16);
        }
    };
    // the checkpoint record of chunk c: its start state and its four 16x16 matrices (QK, QB, AK, AI), which the
    // forward left there so that the scores and the triangular inverse are not rebuilt here
    auto issue_s0 = [&](int c) {
        if (tid == 0) {
            // two boxes of [8][4 rows][72 floats]: rows 8a + b and rows 8a + 4 + b (a < 8, b < 4); the second starts at
            // column -8, so that its fill comes first in each row
            const uint32_t bar = smem_u32(&sm.s0_bar);
            const int record = (int)(bh * nchunks + c);
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"((uint32_t)((N * SS + 2 * MAT_BLK) * 4)) : "memory");
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
                asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                             ::"r"(smem_u32(sm.S0s + blk * S0_BLK)), "l"(&omaps.ck), "r"(bar), "r"(-8 * blk), "r"(0), "r"(blk), "r"(0), "r"(record) : "memory");
            // the matrices: the record keeps them as the forward's operand tiles, 16-byte pieces [row / 8][column / 4][row % 8];
            // seen as [row group][row bit 2][row % 4][piece][4 floats], a box of 6 pieces per row (2 of them beyond the
            // row: zero fill) lands as rows of 24 floats; the second block starts at piece -2
#pragma unroll
            for (int blk = 0; blk < 2; ++blk)
                asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
                             ::"r"(smem_u32(sm.mats + blk * MAT_BLK)), "l"(&omaps.ckm), "r"(bar), "r"(0), "r"(-2 * blk), "r"(0), "r"(blk), "r"(record * (CK_FLOATS / 128) + CK_MATS / 128) : "memory");
        }
    };
    if (nchunks > 0) {
        issue_in(nchunks - 1);
        issue_vdy(nchunks - 1, 0);
        issue_s0(nchunks - 1);
        cp_async_commit();
        cp_async_wait<0>();
    }
    __syncthreads();

    // dS: warp owns value rows 16*warp + {g, g+8}; tile nt covers key columns 8nt..8nt+7.
    float dS[8][4];
    {
        const float* d = p.dsT ? p.dsT + bh * N * N : nullptr;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            if (d) {
                float2 lo = *reinterpret_cast<const float2*>(d + (16 * warp + g) * N + 8 * nt + 2 * t4);
                float2 hi2 = *reinterpret_cast<const float2*>(d + (16 * warp + g + 8) * N + 8 * nt + 2 * t4);
                // the state gradient is carried as 2^64 dS, the counterpart of the forward's S~ = 2^-64 S (see ANCHOR_LN)
                dS[nt][0] = lo.x * STATE_UNSCALE; dS[nt][1] = lo.y * STATE_UNSCALE; dS[nt][2] = hi2.x * STATE_UNSCALE; dS[nt][3] = hi2.y * STATE_UNSCALE;
            } else {
                dS[nt][0] = dS[nt][1] = dS[nt][2] = dS[nt][3] = 0.f;
            }
        }
    }

    // this thread's offsets into the chunk-start state: rows 16*warp + g (and + 8) at columns 2*t4 + 8*block, and
    // rows 2*t4 (and + 1) + 8*block at column 16*warp + g
    const float* const s0_mk = sm.S0s + s0_at(16 * warp + g, 2 * t4);
    const float* const s0_kn = sm.S0s + s0_at(2 * t4, 16 * warp + g);
    // matrix m as a B operand: [n][k] (row 8*nt + g, columns 8*kk + 2*t4, +1) and [k][n] (rows 8*tb + 2*t4, +1, column 8*sb + g)
    const float* const mat_g = sm.mats + mat_at(0, g, 2 * t4);
    const float* const mat_t = sm.mats + mat_at(0, 2 * t4, g);
    auto mat_nk = [&](int m, int nt, int kk) {
        FragB<PREC> f;
        const float2 v = *reinterpret_cast<const float2*>(mat_g + (2 * m + nt) * (4 * SCS) + 8 * kk);
        f.x[0].setr(v.x); f.x[1].setr(v.y);
        return f;
    };
    auto mat_kn = [&](int m, int sb, int tb) {
        FragB<PREC> f;
        const float* q = mat_t + (2 * m + tb) * (4 * SCS) + 8 * sb;
        f.x[0].setr(q[0]); f.x[1].setr(q[SCS]);
        return f;
    };
    for (int it = 0; it < nchunks; ++it) {
        const int c = nchunks - 1 - it;
        const int vs = it & 1;
        // ---------------- P1: decay scan and scaled operands -------------------------------------
        {
            decay_scan<IoT, PREC, 1, Lay::SWZ>(sm.st_in[0], sm.st_in[1], sm.st_in[2], sm.st_in[3], sm.st_in[4], Lay::ROWB, sm.wq, sm.wa,
                                  sm.kwi, sm.bwi, sm.fw, sm.cum, PREC == 3 ? sm.lw : nullptr, warp, lane,
                                  TAIL ? (int)min((long long)L, p.T - (long long)c * L) : L);
            if (LN) {  // bonus dot  sum_j r_j k_j bonus_j  per time step: 8 threads per row
                const int row = tid >> 3, part = tid & 7;
                float acc = 0.f;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const int ch = part * 8 + i;
                    acc += bst_elem<IoT>(sm.st_in[0], row, ch) * bst_elem<IoT>(sm.st_in[2], row, ch) * sm.lnp[2 * N + ch];
                }
                acc += __shfl_xor_sync(0xffffffffu, acc, 1);
                acc += __shfl_xor_sync(0xffffffffu, acc, 2);
                acc += __shfl_xor_sync(0xffffffffu, acc, 4);
                if (part == 0) sm.bdot[row] = acc;
            }
        }
        if (TMA_OUT && !LN) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // previous chunk's output tiles have been read
        __syncthreads();  // (A)
        if (c > 0) {
            issue_in(c - 1);
            issue_vdy(c - 1, vs ^ 1);
        }

        // ---------------- stage B: rows = value index -----------------------------------------
        const unsigned char* vt = sm.st_v[vs];
        const unsigned char* dyt = sm.st_dy[vs];
        FragA<PREC> vf[2], dyf[2];
#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            vf[kk] = fragA_km_st<IoT, PREC>(vt, 16 * warp, 8 * kk, g, t4);
            if (!LN) dyf[kk] = fragA_km_st<IoT, PREC>(dyt, 16 * warp, 8 * kk, g, t4);
        }
        // dS <- dSf = dS * fw, then du and the first part of dV.  None of this needs the chunk-start state, so the
        // attn kernel does it before it waits for the state's copy; attn_ln needs the state first (for dy).
        float du[2][4] = {}, dV[2][4] = {};
        float X[2][4] = {};
        if (!LN) s0_wait(&sm.s0_bar, it & 1, &sm.abort, p.status);  // this chunk's start state has landed
        // attn: the X = S0 wa^T products ride in the same loop, six independent accumulator chains instead of four, then two
        auto du_dv = [&]() {
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const float2 f = *reinterpret_cast<const float2*>(sm.fw + 8 * nt + 2 * t4);  // P~_L = 2^64 P_L
                dS[nt][0] = dS[nt][0] * STATE_SCALE * f.x; dS[nt][1] = dS[nt][1] * STATE_SCALE * f.y;
                dS[nt][2] = dS[nt][2] * STATE_SCALE * f.x; dS[nt][3] = dS[nt][3] * STATE_SCALE * f.y;
            }
#pragma unroll
            for (int sb = 0; sb < 2; ++sb)
#pragma unroll
                for (int tb = sb; tb < 2; ++tb) {
                    mma<PREC>(du[sb], dyf[tb], mat_kn(3, sb, tb));
                    mma<PREC>(dV[sb], dyf[tb], mat_kn(1, sb, tb));
                }
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                FragA<PREC> a = fragA_from_acc<PREC>(dS[kk]);
#pragma unroll
                for (int sb = 0; sb < 2; ++sb) {
                    mma<PREC>(du[sb], a, fragB_nk<PREC, true, 1>(sm.bwi, OPS, 8 * sb, 8 * kk, g, t4));
                    mma<PREC>(dV[sb], a, fragB_nk<PREC, true, 1>(sm.kwi, OPS, 8 * sb, 8 * kk, g, t4));
                }
                if (!LN) {
                    FragA<PREC> a0;
                    const float2 lo = *reinterpret_cast<const float2*>(s0_mk + 8 * kk), hi2 = *reinterpret_cast<const float2*>(s0_mk + 4 * SS + 8 * kk);
                    a0.x[0].setr(lo.x); a0.x[1].setr(hi2.x); a0.x[2].setr(lo.y); a0.x[3].setr(hi2.y);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) mma<PREC>(X[nt], a0, fragB_nk<PREC, true, 1>(sm.wa, OPS, 8 * nt, 8 * kk, g, t4));
                }
            }
        };
        if (!LN) du_dv();
        if (LN) s0_wait(&sm.s0_bar, it & 1, &sm.abort, p.status);
        float U[2][4] = {};
        float dvx[2][4] = {};  // LN: bonus-term contribution to dv
        {
            float Y[2][4] = {};
#pragma unroll
            for (int kk = 0; kk < (LN ? 8 : 0); ++kk) {
                FragA<PREC> a;
                {
                    const float2 lo = *reinterpret_cast<const float2*>(s0_mk + 8 * kk), hi2 = *reinterpret_cast<const float2*>(s0_mk + 4 * SS + 8 * kk);
                    a.x[0].setr(lo.x); a.x[1].setr(hi2.x); a.x[2].setr(lo.y); a.x[3].setr(hi2.y);
                }
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    mma<PREC>(X[nt], a, fragB_nk<PREC, true, 1>(sm.wa, OPS, 8 * nt, 8 * kk, g, t4));
                    if (LN) mma<PREC>(Y[nt], a, fragB_nk<PREC, true, 1>(sm.wq, OPS, 8 * nt, 8 * kk, g, t4));
                }
            }
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int kk = 0; kk <= nt; ++kk) {
                    mma<PREC>(X[nt], vf[kk], mat_nk(0, nt, kk));
                    if (LN) mma<PREC>(Y[nt], vf[kk], mat_nk(1, nt, kk));
                }
            FragA<PREC> xa[2] = {fragA_from_acc<PREC>(X[0]), fragA_from_acc<PREC>(X[1])};
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int kk = 0; kk <= nt; ++kk) mma<PREC>(U[nt], xa[kk], mat_nk(2, nt, kk));
            if (LN) {
                // ---- rebuild Y, then GroupNorm / bonus / gate backward in the [value][time] layout ----
                FragA<PREC> ua0[2] = {fragA_from_acc<PREC>(U[0]), fragA_from_acc<PREC>(U[1])};
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int kk = 0; kk <= nt; ++kk) mma<PREC>(Y[nt], ua0[kk], mat_nk(3, nt, kk));
                // statistics: per-warp mean and centred sum of squares over 16 rows, merged below
                // (a thread's four time steps i4 = 2 * nt + e go through every shuffle level together; sums that only one
                // lane has to store are formed as a reduce-scatter over the row lanes, which halves the values per level)
                const bool b0 = g & 1, b1 = g & 2, b2 = g & 4;
                {
                    float sy[4], q2[4];
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) sy[i4] = Y[i4 >> 1][i4 & 1] + Y[i4 >> 1][(i4 & 1) + 2];
#pragma unroll
                    for (int m = 4; m <= 16; m <<= 1)
#pragma unroll
                        for (int i4 = 0; i4 < 4; ++i4) sy[i4] += __shfl_xor_sync(0xffffffffu, sy[i4], m);
#pragma unroll
                    for (int i4 = 0; i4 < 4; ++i4) {
                        sy[i4] *= (1.f / 16.f);  // the warp's mean
                        const float d0 = Y[i4 >> 1][i4 & 1] - sy[i4], d1 = Y[i4 >> 1][(i4 & 1) + 2] - sy[i4];
                        q2[i4] = d0 * d0 + d1 * d1;
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float send = b0 ? q2[i] : q2[i + 2], keep = b0 ? q2[i + 2] : q2[i];
                        q2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                    }
                    {
                        const float send = b1 ? q2[0] : q2[1], keep = b1 ? q2[1] : q2[0];
                        q2[0] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
                    q2[0] += __shfl_xor_sync(0xffffffffu, q2[0], 16);
                    if (!b2) {  // this lane holds time step i4 = 2 * b0 + b1
                        const int tq = 8 * (b0 ? 1 : 0) + 2 * t4 + (b1 ? 1 : 0);
                        red[(warp * L + tq) * 2 + 0] = b0 ? (b1 ? sy[3] : sy[2]) : (b1 ? sy[1] : sy[0]);
                        red[(warp * L + tq) * 2 + 1] = q2[0];
                    }
                }
                __syncthreads();  // (D1)
                const unsigned char* gt = sm.st_g[LN ? vs : 0];
                float xh[2][4], dxh[2][4], rstd_t[4];
                float asum[16];  // [a1 | a2 | a3 | unused][i4]
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) asum[12 + i4] = 0.f;
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const int nt = i4 >> 1, e = i4 & 1, tq = 8 * nt + 2 * t4 + e;
                    float mu = 0.f, m2 = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < WARPS; ++w2) mu += red[(w2 * L + tq) * 2];
                    mu *= 0.25f;
#pragma unroll
                    for (int w2 = 0; w2 < WARPS; ++w2) {
                        const float dm = red[(w2 * L + tq) * 2] - mu;
                        m2 += red[(w2 * L + tq) * 2 + 1] + 16.f * dm * dm;
                    }
                    const float rstd = 1.f / sqrtf(m2 * (1.f / N) + p.eps);
                    rstd_t[i4] = rstd;
                    const float bd = sm.bdot[tq];
                    float a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow) {
                        const int vc = 16 * warp + g + 8 * hrow, i = e + 2 * hrow;
                        const float x = (Y[nt][i] - mu) * rstd;
                        const float ve = bst_elem<IoT>(vt, tq, vc), ge = bst_elem<IoT>(gt, tq, vc), de = bst_elem<IoT>(dyt, tq, vc);
                        const float z = x * sm.lnp[vc] + sm.lnp[N + vc] + bd * ve;
                        const float dz = de * ge;
                        Y[nt][i] = de * z;  // dg, stored below
                        dlnw_acc[hrow] += dz * x;
                        dlnb_acc[hrow] += dz;
                        dvx[nt][i] = dz * bd;
                        const float dx = dz * sm.lnp[vc];
                        xh[nt][i] = x;
                        dxh[nt][i] = dx;
                        a1 += dx; a2 += dx * x; a3 += dz * ve;
                    }
                    asum[i4] = a1; asum[4 + i4] = a2; asum[8 + i4] = a3;
                }
                {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float send = b0 ? asum[i] : asum[i + 8], keep = b0 ? asum[i + 8] : asum[i];
                        asum[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
                    }
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float send = b1 ? asum[i] : asum[i + 4], keep = b1 ? asum[i + 4] : asum[i];
                        asum[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
                    }
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float send = b2 ? asum[i] : asum[i + 2], keep = b2 ? asum[i + 2] : asum[i];
                        asum[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
                    }
                    // the lane now holds entries 8 * b0 + 4 * b1 + 2 * b2 + {0, 1}: sum number 2 * b0 + b1 of time steps i4 = 2 * b2 + {0, 1}
                    const int which = (b0 ? 2 : 0) + (b1 ? 1 : 0);
                    if (which < 3) {
                        const int tq = 8 * (b2 ? 1 : 0) + 2 * t4;
                        red2[(warp * L + tq) * 3 + which] = asum[0];
                        red2[(warp * L + tq + 1) * 3 + which] = asum[1];
                    }
                }
                // dg out.  bf16: as a 128-byte-swizzled [time][value] tile at the start of the score-gradient buffer (dead
                // until the end of stage C's first part), stored by a bulk tensor copy issued after the barrier below and
                // waited for before barrier (C1); otherwise through the per-warp scratch tile
                if constexpr (TMA_OUT) {
                    unsigned char* dgt = reinterpret_cast<unsigned char*>(sm.sgrad);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int tq = 8 * nt + 2 * t4 + (i & 1), vc = 16 * warp + g + 8 * (i >> 1);
                            *reinterpret_cast<__nv_bfloat16*>(dgt + tq * 128 + (((vc >> 3) ^ (tq & 7)) << 4) + (vc & 7) * 2) = __float2bfloat16_rn(Y[nt][i]);
                        }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                } else {
                    IoT* sc = dvsc;
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const int tq = 8 * nt + 2 * t4;
                        sc[tq * Lay::YS + g] = from_f32<IoT>(Y[nt][0]);
                        sc[(tq + 1) * Lay::YS + g] = from_f32<IoT>(Y[nt][1]);
                        sc[tq * Lay::YS + g + 8] = from_f32<IoT>(Y[nt][2]);
                        sc[(tq + 1) * Lay::YS + g + 8] = from_f32<IoT>(Y[nt][3]);
                    }
                    __syncwarp();
                    const int row = lane >> 1, hf = lane & 1;
                    const uint4* src = reinterpret_cast<const uint4*>(sc + row * Lay::YS + 8 * hf);
                    uint4* dst = reinterpret_cast<uint4*>(gdg + ((long long)c * L + row) * p.st.t + 16 * warp + 8 * hf);
                    if (!TAIL || (long long)c * L + row < p.T) {
                        dst[0] = src[0];
                        if (sizeof(IoT) == 4) dst[1] = src[1];
                    }
                    __syncwarp();
                }
                if (TMA_OUT) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // previous chunk's output tiles (in Ut, Dt, Yt) have been read
                __syncthreads();  // (D2)
                if (TMA_OUT && tid == 0) {
                    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
                                 ::"l"(&omaps.m[6]), "r"(0), "r"((int)hi), "r"(c * L), "r"((int)bi), "r"(smem_u32(sm.sgrad)) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
#pragma unroll
                for (int i4 = 0; i4 < 4; ++i4) {
                    const int nt = i4 >> 1, e = i4 & 1, tq = 8 * nt + 2 * t4 + e;
                    float m1 = 0.f, m2 = 0.f, sb = 0.f;
#pragma unroll
                    for (int w2 = 0; w2 < WARPS; ++w2) {
                        m1 += red2[(w2 * L + tq) * 3];
                        m2 += red2[(w2 * L + tq) * 3 + 1];
                        sb += red2[(w2 * L + tq) * 3 + 2];
                    }
                    m1 *= (1.f / N); m2 *= (1.f / N);
                    if (warp == 0 && g == 0) sm.sbon[tq] = sb;
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow) {
                        const int i = e + 2 * hrow;
                        Y[nt][i] = rstd_t[i4] * (dxh[nt][i] - m1 - xh[nt][i] * m2);  // gradient of the recurrence output
                    }
                }
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    dyf[nt] = fragA_from_acc<PREC>(Y[nt]);
                    const int tq = 8 * nt + 2 * t4, vc = 16 * warp + g;
                    const int c0 = xcol<1>(tq, vc), c1 = xcol<1>(tq, vc + 8);  // rows tq, tq+1 share the swizzle
                    sm.Yt[tq * OPS + c0] = pre<PREC>(Y[nt][0]); sm.Yt[(tq + 1) * OPS + c0] = pre<PREC>(Y[nt][1]);
                    sm.Yt[tq * OPS + c1] = pre<PREC>(Y[nt][2]); sm.Yt[(tq + 1) * OPS + c1] = pre<PREC>(Y[nt][3]);
                }
            }
        }
        if (LN) du_dv();
        float dabu[2][4] = {};
        {
            FragA<PREC> da2[2] = {fragA_from_acc<PREC>(du[0]), fragA_from_acc<PREC>(du[1])};
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
#pragma unroll
                for (int kb = nb; kb < 2; ++kb) mma<PREC>(dabu[nb], da2[kb], mat_kn(2, nb, kb));
        }
        FragA<PREC> dbf[2] = {fragA_from_acc<PREC>(dabu[0]), fragA_from_acc<PREC>(dabu[1])};
#pragma unroll
        for (int sb = 0; sb < 2; ++sb)
#pragma unroll
            for (int tb = sb; tb < 2; ++tb) mma<PREC>(dV[sb], dbf[tb], mat_kn(0, sb, tb));

        // dv out: the bf16 kernels write it into its staging tile; otherwise transposed through a per-warp scratch tile
        // for 16-byte stores
        if constexpr (TMA_OUT) {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tq = 8 * nt + 2 * t4 + (i & 1), vc = 16 * warp + g + 8 * (i >> 1);
                    *reinterpret_cast<__nv_bfloat16*>(sm.dv_tile() + tq * 128 + (((vc >> 3) ^ (tq & 7)) << 4) + (vc & 7) * 2) = __float2bfloat16_rn(dV[nt][i] + dvx[nt][i]);
                }
        } else {
            IoT* sc = dvsc;
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int tq = 8 * nt + 2 * t4;
                sc[tq * Lay::YS + g] = from_f32<IoT>(dV[nt][0] + dvx[nt][0]);
                sc[(tq + 1) * Lay::YS + g] = from_f32<IoT>(dV[nt][1] + dvx[nt][1]);
                sc[tq * Lay::YS + g + 8] = from_f32<IoT>(dV[nt][2] + dvx[nt][2]);
                sc[(tq + 1) * Lay::YS + g + 8] = from_f32<IoT>(dV[nt][3] + dvx[nt][3]);
            }
            __syncwarp();
            const int row = lane >> 1, hf = lane & 1;
            const uint4* src = reinterpret_cast<const uint4*>(sc + row * Lay::YS + 8 * hf);
            uint4* dst = reinterpret_cast<uint4*>(gdv + ((long long)c * L + row) * p.st.t + 16 * warp + 8 * hf);
            if (!TAIL || (long long)c * L + row < p.T) {
                dst[0] = src[0];
                if (sizeof(IoT) == 4) dst[1] = src[1];
            }
        }
        // dSf, U, dabu to shared memory for stage C
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(sm.dSs + (16 * warp + g) * SS + xcol<1>(g, 8 * nt + 2 * t4)) = make_float2(pre<PREC>(dS[nt][0]), pre<PREC>(dS[nt][1]));
            *reinterpret_cast<float2*>(sm.dSs + (16 * warp + g + 8) * SS + xcol<1>(g, 8 * nt + 2 * t4)) = make_float2(pre<PREC>(dS[nt][2]), pre<PREC>(dS[nt][3]));
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int tq = 8 * nt + 2 * t4, vc = 16 * warp + g;
            const int c0 = xcol<1>(tq, vc), c1 = xcol<1>(tq, vc + 8);  // rows tq, tq+1 share the swizzle
            sm.Ut[tq * OPS + c0] = pre<PREC>(U[nt][0]); sm.Ut[(tq + 1) * OPS + c0] = pre<PREC>(U[nt][1]);
            sm.Ut[tq * OPS + c1] = pre<PREC>(U[nt][2]); sm.Ut[(tq + 1) * OPS + c1] = pre<PREC>(U[nt][3]);
            sm.Dt[tq * OPS + c0] = pre<PREC>(dabu[nt][0]); sm.Dt[(tq + 1) * OPS + c0] = pre<PREC>(dabu[nt][1]);
            sm.Dt[tq * OPS + c1] = pre<PREC>(dabu[nt][2]); sm.Dt[(tq + 1) * OPS + c1] = pre<PREC>(dabu[nt][3]);
        }
        // dS0 = dSf + dY^T wq + dabu^T wa ; carried decay term sum_i dS0[i,:] S0[i,:]
        {
            float gp[16];  // this thread's two rows: [2 * nt + e] for key column 8 * nt + 2 * t4 + e
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
                for (int kk = 0; kk < 2; ++kk) {
                    mma<PREC>(dS[nt], dyf[kk], fragB_kn<PREC, true, 1>(sm.wq, OPS, 8 * nt, 8 * kk, g, t4));
                    mma<PREC>(dS[nt], dbf[kk], fragB_kn<PREC, true, 1>(sm.wa, OPS, 8 * nt, 8 * kk, g, t4));
                }
                const float2 lo = *reinterpret_cast<const float2*>(s0_mk + 8 * nt);
                const float2 hi2 = *reinterpret_cast<const float2*>(s0_mk + 4 * SS + 8 * nt);
                gp[2 * nt] = dS[nt][0] * lo.x + dS[nt][2] * hi2.x;
                gp[2 * nt + 1] = dS[nt][1] * lo.y + dS[nt][3] * hi2.y;
            }
            // Sum over the eight row lanes g as a reduce-scatter: every step halves the values a lane carries (8 + 4 + 2
            // shuffles instead of 3 per value), and lane g ends with the two sums of tile nt = bit-reversed g.
            const bool b0 = g & 1, b1 = g & 2, b2 = g & 4;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float send = b0 ? gp[i] : gp[i + 8], keep = b0 ? gp[i + 8] : gp[i];
                gp[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float send = b1 ? gp[i] : gp[i + 4], keep = b1 ? gp[i + 4] : gp[i];
                gp[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float send = b2 ? gp[i] : gp[i + 2], keep = b2 ? gp[i + 2] : gp[i];
                gp[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
            }
            const int nt_own = (b2 ? 1 : 0) + (b1 ? 2 : 0) + (b0 ? 4 : 0);
            *reinterpret_cast<float2*>(&sm.Gp[it & 1][warp][8 * nt_own + 2 * t4]) = make_float2(gp[0], gp[1]);
        }
        if (TMA_OUT && LN) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // dg's tile lies where stage C writes the score gradients
        __syncthreads();  // (C1)
        // ---------------- stage C: contractions over the value index --------------------------
        float DA[2][4] = {}, DQ[2][4] = {}, DB[2][4] = {}, DK[2][4] = {};
        {
            // one score gradient per warp: 0 dQK = tril(dY V^T), 1 dAK = stril(dabu V^T),
            // 2 dQB = tril(dY U^T), 3 dAB = stril(dabu U^T)
            float d[2][4] = {};
            const bool strict = warp & 1;
            float* dst = sm.sgrad + warp * (L * SCS);  // 0 dQK, 1 dAK, 2 dQB, 3 dAB
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                FragA<PREC> aD = fragA_mk<PREC, true, 1>(sm.Dt, OPS, 0, 8 * kk, g, t4);
                FragA<PREC> aY = LN ? fragA_mk<PREC, true, 1>(sm.Yt, OPS, 0, 8 * kk, g, t4) : fragA_mk_st<IoT, PREC>(dyt, 8 * kk, g, t4);
                FragA<PREC> aU = fragA_mk<PREC, true, 1>(sm.Ut, OPS, 0, 8 * kk, g, t4);
                FragA<PREC> aV = fragA_mk_st<IoT, PREC>(vt, 8 * kk, g, t4);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    FragB<PREC> bsc = (warp >> 1) ? fragB_nk<PREC, true, 1>(sm.Ut, OPS, 8 * nt, 8 * kk, g, t4)
                                                  : fragB_nk_st<IoT, PREC>(vt, 8 * nt, 8 * kk, g, t4);
                    mma<PREC>(d[nt], strict ? aD : aY, bsc);
                    FragB<PREC> bS;
                    bS.x[0].setr(s0_kn[4 * kk * SS + 8 * nt]); bS.x[1].setr(s0_kn[(4 * kk + 1) * SS + 8 * nt]);
                    FragB<PREC> bD = fragB_kn<PREC, true, 1>(sm.dSs, SS, 16 * warp + 8 * nt, 8 * kk, g, t4);
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
                *reinterpret_cast<float2*>(dst + g * SCS + xcol<1>(g, s)) =
                    make_float2(keep(g, s) ? pre<PREC>(d[nt][0]) : 0.f, keep(g, s + 1) ? pre<PREC>(d[nt][1]) : 0.f);
                *reinterpret_cast<float2*>(dst + (g + 8) * SCS + xcol<1>(g, s)) =
                    make_float2(keep(g + 8, s) ? pre<PREC>(d[nt][2]) : 0.f, keep(g + 8, s + 1) ? pre<PREC>(d[nt][3]) : 0.f);
            }
        }
        __syncthreads();  // (C2) score gradients visible; S0s free
        if (c > 0) issue_s0(c - 1);
        cp_async_commit();

#pragma unroll
        for (int kk = 0; kk < 2; ++kk) {
            const float *dQK = sm.sgrad, *dAK = sm.sgrad + L * SCS, *dQB = sm.sgrad + 2 * L * SCS, *dAB = sm.sgrad + 3 * L * SCS;
            FragA<PREC> aAB = fragA_mk<PREC, true, 1>(dAB, SCS, 0, 8 * kk, g, t4), aAK = fragA_mk<PREC, true, 1>(dAK, SCS, 0, 8 * kk, g, t4);
            FragA<PREC> aQB = fragA_mk<PREC, true, 1>(dQB, SCS, 0, 8 * kk, g, t4), aQK = fragA_mk<PREC, true, 1>(dQK, SCS, 0, 8 * kk, g, t4);
            FragA<PREC> tAB = fragA_km<PREC, true, 1>(dAB, SCS, 0, 8 * kk, g, t4), tAK = fragA_km<PREC, true, 1>(dAK, SCS, 0, 8 * kk, g, t4);
            FragA<PREC> tQB = fragA_km<PREC, true, 1>(dQB, SCS, 0, 8 * kk, g, t4), tQK = fragA_km<PREC, true, 1>(dQK, SCS, 0, 8 * kk, g, t4);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int n0 = 16 * warp + 8 * nt;
                FragB<PREC> bb = fragB_kn<PREC, true, 1>(sm.bwi, OPS, n0, 8 * kk, g, t4), bk = fragB_kn<PREC, true, 1>(sm.kwi, OPS, n0, 8 * kk, g, t4);
                FragB<PREC> ba = fragB_kn<PREC, true, 1>(sm.wa, OPS, n0, 8 * kk, g, t4), bq = fragB_kn<PREC, true, 1>(sm.wq, OPS, n0, 8 * kk, g, t4);
                mma<PREC>(DA[nt], aAB, bb); mma<PREC>(DA[nt], aAK, bk);
                mma<PREC>(DQ[nt], aQB, bb); mma<PREC>(DQ[nt], aQK, bk);
                mma<PREC>(DB[nt], tAB, ba); mma<PREC>(DB[nt], tQB, bq);
                mma<PREC>(DK[nt], tAK, ba); mma<PREC>(DK[nt], tQK, bq);
            }
        }
        // ---------------- epilogue: thread holds rows g, g+8 x key columns n0+2*t4, +1 ---------
        float outv[5][2][2][2];  // [dq, dw, dk, da, db][tile][row half][column]
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int key = 16 * warp + 8 * nt + 2 * t4;
            float x[2][2], e2[2][2], lwv[2][2];  // [row half][column]
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const int tq = g + 8 * hrow;
                const int kx = xcol<1>(tq, key);
                const float2 cu = *reinterpret_cast<const float2*>(sm.cum + tq * OPS + kx);
                float2 lwp;
                if (PREC == 3) {
                    lwp = *reinterpret_cast<const float2*>(sm.lw + tq * OPS + kx);
                } else {  // running log-decay difference; row -1 is zero
                    const float2 cp = tq > 0 ? *reinterpret_cast<const float2*>(sm.cum + (tq - 1) * OPS + xcol<1>(tq - 1, key)) : make_float2(0.f, 0.f);
                    lwp = make_float2(cu.x - cp.x, cu.y - cp.y);
                }
                const float2 oq = *reinterpret_cast<const float2*>(sm.wq + tq * OPS + kx);
                const float2 oa = *reinterpret_cast<const float2*>(sm.wa + tq * OPS + kx);
                const float2 okw = *reinterpret_cast<const float2*>(sm.kwi + tq * OPS + kx);
                const float2 ob = *reinterpret_cast<const float2*>(sm.bwi + tq * OPS + kx);
                const float cuv[2] = {cu.x, cu.y}, lwa[2] = {lwp.x, lwp.y};
                const float wqv[2] = {oq.x, oq.y}, wav[2] = {oa.x, oa.y}, kwv[2] = {okw.x, okw.y}, bwv[2] = {ob.x, ob.y};
                float o_q[2], o_k[2], o_a[2], o_b[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int i = e + 2 * hrow;
                    const float incl = decay_up<PREC>(cuv[e]);   // P~_t, as the scan formed it
                    const float inv = rcp_p<PREC>(incl);
                    // P_{t-1} = exp(cum_{t-1}) with cum_{t-1} = cum_t - lw_t (0 for the first row): an exponential on the idle
                    // special-function unit instead of two shuffles for the row above
                    const float non = decay_up<PREC>(cuv[e] - lwa[e]);
                    o_a[e] = non * DA[nt][i];
                    o_q[e] = incl * DQ[nt][i];
                    o_b[e] = inv * DB[nt][i];
                    o_k[e] = inv * DK[nt][i];
                    if (LN) {  // bonus term: y += (sum_j q_j k_j bonus_j) v
                        const float sbv = sm.sbon[tq], bo = sm.lnp[2 * N + key + e];
                        const float q_raw = wqv[e] * inv, k_raw = kwv[e] * incl;
                        o_q[e] += sbv * k_raw * bo;
                        o_k[e] += sbv * q_raw * bo;
                        dbon_acc[nt][e] += sbv * q_raw * k_raw;
                    }
                    e2[hrow][e] = wav[e] * DA[nt][i];
                    x[hrow][e] = wqv[e] * DQ[nt][i] - kwv[e] * DK[nt][i] - bwv[e] * DB[nt][i] + e2[hrow][e];
                    lwv[hrow][e] = lwa[e];
                }
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    outv[0][nt][hrow][e] = o_q[e]; outv[2][nt][hrow][e] = o_k[e];
                    outv[3][nt][hrow][e] = o_a[e]; outv[4][nt][hrow][e] = o_b[e];
                }
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
                const float d0 = (x[hrow][0] - e2[hrow][0] + Gc.x) * lwv[hrow][0];
                const float d1 = (x[hrow][1] - e2[hrow][1] + Gc.y) * lwv[hrow][1];
                outv[1][nt][hrow][0] = d0; outv[1][nt][hrow][1] = d1;
            }
        }
        if (TMA_OUT) {
            // into the swizzled staging tiles: 4-byte stores, a warp-wide store covers 8 rows x 16 bytes in 8 different
            // 16-byte units (conflict-free); the tiles leave by bulk tensor stores after the barrier below
#pragma unroll
            for (int ten = 0; ten < 5; ++ten)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow) {
                        const int tq = g + 8 * hrow;
                        const __nv_bfloat162 v2 = __floats2bfloat162_rn(outv[ten][nt][hrow][0], outv[ten][nt][hrow][1]);
                        *reinterpret_cast<__nv_bfloat162*>(sm.out_tiles() + ten * 2048 + tq * 128 + ((((2 * warp + nt) ^ (tq & 7))) << 4) + 4 * t4) = v2;
                    }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        } else {
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                const long long off = ((long long)c * L + g + 8 * hrow) * p.st.t + 16 * warp;
                const bool live = !TAIL || (long long)c * L + g + 8 * hrow < p.T;  // uniform over the lanes that exchange values
#pragma unroll
                for (int ten = 0; ten < 5; ++ten)
                    store_quad(gout[ten] + off, outv[ten][0][hrow][0], outv[ten][0][hrow][1], outv[ten][1][hrow][0], outv[ten][1][hrow][1], t4, live);
            }
        }
        cp_async_wait<0>();
        __syncthreads();  // (E)
        if (TMA_OUT && tid == 0) {
#pragma unroll
            for (int ten = 0; ten < 6; ++ten)
                asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3, %4}], [%5];"
                             ::"l"(&omaps.m[ten]), "r"(0), "r"((int)hi), "r"(c * L), "r"((int)bi), "r"(smem_u32(ten < 5 ? sm.out_tiles() + ten * 2048 : sm.dv_tile())) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
    if (TMA_OUT) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");  // shared memory must outlive the last stores

    if (LN) {
        // per-(batch, head) partial parameter gradients: ws[b][0..2][h*N + channel]
        float* ws = p.dparams_ws + bi * 3 * p.H * N + hi * N;
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            float a = dlnw_acc[hrow], b2 = dlnb_acc[hrow];
            a += __shfl_xor_sync(0xffffffffu, a, 1); a += __shfl_xor_sync(0xffffffffu, a, 2);
            b2 += __shfl_xor_sync(0xffffffffu, b2, 1); b2 += __shfl_xor_sync(0xffffffffu, b2, 2);
            if (t4 == 0) {
                ws[16 * warp + g + 8 * hrow] = a;
                ws[p.H * N + 16 * warp + g + 8 * hrow] = b2;
            }
        }
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float a = dbon_acc[nt][e];
                a += __shfl_xor_sync(0xffffffffu, a, 4); a += __shfl_xor_sync(0xffffffffu, a, 8); a += __shfl_xor_sync(0xffffffffu, a, 16);
                if (g == 0) ws[2 * p.H * N + 16 * warp + 8 * nt + 2 * t4 + e] = a;
            }
    }
    if (p.ds0) {
        float* o = p.ds0 + bh * N * N;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) {
            *reinterpret_cast<float2*>(o + (16 * warp + g) * N + 8 * nt + 2 * t4) = make_float2(dS[nt][0] * STATE_SCALE, dS[nt][1] * STATE_SCALE);
            *reinterpret_cast<float2*>(o + (16 * warp + g + 8) * N + 8 * nt + 2 * t4) = make_float2(dS[nt][2] * STATE_SCALE, dS[nt][3] * STATE_SCALE);
        }
    }
}

// dparams[i][c] = sum over batch of the per-(batch, head) partials, in a fixed order.
__global__ void reduce_dparams_kernel(const float* __restrict__ ws, float* __restrict__ out, long long B, long long n3) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (i >= n3) return;
    float acc = 0.f;
    for (long long b = 0; b < B; ++b) acc += ws[b * n3 + i];
    out[i] = acc;
}

// Tensor map of a bf16 [B,T,H,N] tensor with element strides st; box = one head, 16 time steps, 64 channels,
// 128-byte swizzle.  Encoded through the runtime's driver-entry-point query (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}
// Tensor map over the states of `records` checkpoint records (fp32 [64][64] at the start of each record of CK_FLOATS
// floats), seen as [record][a = row / 8][row bit 2][b = row % 4][column]; a box is the 32 rows of one value of bit 2,
// N + 8 floats wide (the part outside the 64 columns reads as zero).
static bool encode_ckpt_state_map(CUtensorMap* m, const float* ckpt, long long records) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[5] = {(cuuint64_t)N, 4, 2, 8, (cuuint64_t)records};
    const cuuint64_t strides[4] = {N * 4, 4 * N * 4, 8 * N * 4, (cuuint64_t)CK_FLOATS * 4};
    const cuuint32_t box[5] = {(cuuint32_t)SS, 4, 1, 8, 1};
    const cuuint32_t es[5] = {1, 1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(ckpt + CK_STATE), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
// Tensor map over the matrices part of the checkpoint records.  A record is 40 row groups of 128 floats (32 of state, then
// 8 of matrices: [AK;QK], AI, QB as operand tiles, a row group = [4 pieces][8 rows][4 floats]); the map sees the whole
// buffer as [row group][row bit 2][row % 4][piece][4 floats]; a box is the rows of one value of bit 2 in 8 row groups,
// 6 pieces wide (pieces 4, 5 do not exist and read as zero).
static bool encode_ckpt_mats_map(CUtensorMap* m, const float* ckpt, long long records) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    static_assert(CK_FLOATS % 128 == 0 && CK_MATS % 128 == 0, "records and their matrices part are whole row groups");
    const cuuint64_t dims[5] = {4, 4, 4, 2, (cuuint64_t)(records * (CK_FLOATS / 128))};
    const cuuint64_t strides[4] = {32 * 4, 4 * 4, 16 * 4, 128 * 4};
    const cuuint32_t box[5] = {4, (cuuint32_t)(SCS / 4), 4, 1, 8};
    const cuuint32_t es[5] = {1, 1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 5, const_cast<float*>(ckpt), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}
static bool encode_bthn_map(CUtensorMap* m, void* base, long long B, long long T, long long H, const Strides& st) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
    // a dimension of extent 1 may carry any stride; give it a valid (16-byte multiple, non-zero) one
    auto sb = [&](long long s, long long fallback) { return (cuuint64_t)((s > 0 ? s : fallback) * 2); };
    const cuuint64_t strides[3] = {sb(st.h, N), sb(st.t, H * N), sb(st.b, T * H * N)};
    const cuuint32_t box[4] = {(cuuint32_t)N, 1, (cuuint32_t)L, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename IoT, int PREC, bool LN> static int launch_bwd_t(const BwdParams& p, cudaStream_t stream) {
    using Smem = BwdSmem<IoT, PREC, LN>;
    auto kern = p.T % L ? wkv7_bwd_kernel<IoT, PREC, LN, true> : wkv7_bwd_kernel<IoT, PREC, LN, false>;
    const int smem = (int)sizeof(Smem);
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return kLaunchFailed;
    OutMaps omaps;
    memset(&omaps, 0, sizeof(omaps));
    if (Smem::TMA_OUT) {
        void* outs[7] = {p.dr, p.dw, p.dk, p.da, p.db, p.dv, p.dg};
        for (int i = 0; i < (LN ? 7 : 6); ++i)
            if (!encode_bthn_map(&omaps.m[i], outs[i], p.B, p.T, p.H, p.st)) return kLaunchFailed;
    }
    const long long records = p.B * p.H * ((p.T + L - 1) / L);
    if (!(encode_ckpt_state_map(&omaps.ck, p.ckpt, records) && encode_ckpt_mats_map(&omaps.ckm, p.ckpt, records)))
        return kLaunchFailed;
    kern<<<(unsigned)(p.B * p.H), THREADS, smem, stream>>>(p, omaps);
    if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    if (LN) {
        const long long n3 = 3 * p.H * N;
        reduce_dparams_kernel<<<(unsigned)((n3 + 255) / 256), 256, 0, stream>>>(p.dparams_ws, p.dparams, p.B, n3);
        if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    }
    return kOk;
}

int launch_bwd(const BwdParams& p, int io_dtype, bool ln, cudaStream_t stream) {
    if (io_dtype == 0) return ln ? launch_bwd_t<__nv_bfloat16, 1, true>(p, stream) : launch_bwd_t<__nv_bfloat16, 1, false>(p, stream);
    if (io_dtype == 2) return ln ? launch_bwd_t<float, 1, true>(p, stream) : launch_bwd_t<float, 1, false>(p, stream);
    return ln ? launch_bwd_t<float, 3, true>(p, stream) : launch_bwd_t<float, 3, false>(p, stream);
}

}  // namespace wkv7
