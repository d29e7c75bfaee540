// expand_loras for sm_100a: second-stage LoRA expansion producing (w, k, kk, b) for the WKV7 mixer.
// Replaces fw_triton_ / bw_triton_ of the reference (wind_rwkv/rwkv7/rwkv7_expand_loras.py:32-79, 91-211):
//     w  = -softplus(-(w_bias + w_in)) - 0.5
//     z  = tanh(z_in) @ Wz^T + k_in ;   kk = z / sqrt(max(sum_head z^2, 1e-12))
//     a  = sigmoid(a_in @ Wa^T + a_bias)   ma, mk likewise
//     k  = k_in * (ma + a - ma*a) * exp(w * mk) ;   b = -kk * a
// One warp handles 16 tokens x one head (64 channels): the rank-D products are bf16 m16n8k16 MMAs
// with the head's weight slices staged in shared memory, the per-head L2 norm is a 4-lane shuffle.
// Forward: grid (H, rows/64).  Backward: grid (H, B), walking the sequence in 64-token tiles so the
// weight gradients stay in registers (one LoRA per warp; bias gradients ride along as an extra
// all-ones input column) and are flushed once with fp32 atomics; the input gradients, which
// contract over all heads, are written as per-head partials and summed by a small kernel.
#include "expand_loras.h"
#include "mma_bf16.cuh"

namespace wkv7 {

constexpr int HC = 64;  // channels per head

// The gates of one element:  a, ma, mk = sigmoid(xa, xm, xk);  w = -softplus(-v) - 0.5;  E = exp(w * mk).
// Six special-function instructions (three tanh for the sigmoids, ex2 + lg2 for the softplus, ex2 for E) and one
// exponential as a polynomial on the FMA pipe: the op is bound by issue slots, and the textbook forms (expf, a
// division per sigmoid) cost three to four times the instructions.
struct Gates { float a, ma, mk, w, E, ev; };  // ev = exp(-v) (for the backward: sigmoid(-v) = ev / (1 + ev))
__device__ __forceinline__ Gates lora_gates(float xa, float xm, float xk, float v) {
    Gates o;
    o.a = sigmoid_f(xa);
    o.ma = sigmoid_f(xm);
    o.mk = sigmoid_f(xk);
    o.ev = exp_poly(-v);  // exp_poly clamps its argument to +-80
    o.w = -0.6931471805599453f * __log2f(1.f + o.ev) - 0.5f;
    o.E = __expf(o.w * o.mk);
    return o;
}

constexpr int GLD = HC + 8;  // row stride (bf16) of the [token][channel] tiles: 4-byte accesses in the MMA fragment pattern
                             // (rows g, columns 2 * t4) and 16-byte row accesses are both free of bank conflicts
template <int D> struct LorasFwdSmem {
    bf16 W[4][HC][D + 8];  // [channel][rank]
    // [token][channel] tiles of one head: w_in, k_in on the way in (16-byte cp.async, whole 128-byte rows), the four
    // outputs on the way out (written in the fragment pattern, stored as whole rows).  Global accesses in the
    // fragment pattern itself would touch 16 bytes per row and instruction.
    bf16 io[4][64][GLD];
};

// A fragments of a [16, D] input block straight from global memory (rows r0+g, r0+g+8).
template <int D, bool TANH>
__device__ __forceinline__ void load_in_frags(uint32_t (&a)[D / 16][4], const bf16* base, long long r0, int g, int t4) {
    const bf16* p0 = base + (r0 + g) * D + 2 * t4;
    const bf16* p1 = p0 + 8 * D;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t v[4] = {*reinterpret_cast<const uint32_t*>(p0 + 16 * ks), *reinterpret_cast<const uint32_t*>(p1 + 16 * ks),
                         *reinterpret_cast<const uint32_t*>(p0 + 16 * ks + 8), *reinterpret_cast<const uint32_t*>(p1 + 16 * ks + 8)};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (TANH) {
                float2 f = unpack_bf16x2(v[i]);
                v[i] = pack_bf16x2(tanh_f(f.x), tanh_f(f.y));
            }
            a[ks][i] = v[i];
        }
    }
}

template <int D>
__global__ void __launch_bounds__(128) loras_fwd_kernel(LorasParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sm = *reinterpret_cast<LorasFwdSmem<D>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int h = blockIdx.x, C = (int)p.C;
    const long long r0 = (long long)blockIdx.y * 64 + 16 * warp;
    for (int i = tid; i < 4 * HC * (D / 8); i += 128) {
        const int l = i / (HC * (D / 8)), r = (i / (D / 8)) % HC, ch = i % (D / 8);
        cp_async16(&sm.W[l][r][ch * 8], (const bf16*)p.W[l] + (long long)(h * HC + r) * D + ch * 8);
    }
    {   // this CTA's 64 tokens of w_in and k_in; rows past the end are filled with zeros
        const long long t0 = (long long)blockIdx.y * 64;
        for (int i = tid; i < 2 * 64 * 8; i += 128) {
            const int ten = i / 512, r = (i / 8) % 64, ch = i % 8;
            const bool live = t0 + r < p.rows;
            const bf16* src = (const bf16*)(ten ? p.k_in : p.w_in) + (live ? t0 + r : 0) * C + h * HC + ch * 8;
            cp_async16_zfill(&sm.io[ten][r][ch * 8], src, live);
        }
    }
    cp_async_commit();
    // the LoRA inputs come straight from global memory into MMA fragments: requested before the wait for the asynchronous
    // copies, so that the two latencies overlap
    uint32_t az[D / 16][4], aa[D / 16][4], am[D / 16][4], ak[D / 16][4];
    if (r0 < p.rows) {
        load_in_frags<D, true>(az, (const bf16*)p.lin[0], r0, g, t4);
        load_in_frags<D, false>(aa, (const bf16*)p.lin[1], r0, g, t4);
        load_in_frags<D, false>(am, (const bf16*)p.lin[2], r0, g, t4);
        load_in_frags<D, false>(ak, (const bf16*)p.lin[3], r0, g, t4);
    }
    cp_async_wait<0>();
    __syncthreads();
    if (r0 >= p.rows) return;
    const int lr = 16 * warp;  // this warp's first tile row

    float z[8][4];
    float ss0 = 0.f, ss1 = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        z[j][0] = z[j][1] = z[j][2] = z[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t b[2];
            ldB_nk(b, &sm.W[0][0][0], D + 8, 8 * j, 16 * ks, g, t4);
            mma_bf16(z[j], az[ks], b);
        }
        const float2 k0 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.io[1][lr + g][8 * j + 2 * t4]));
        const float2 k1 = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.io[1][lr + g + 8][8 * j + 2 * t4]));
        z[j][0] += k0.x; z[j][1] += k0.y; z[j][2] += k1.x; z[j][3] += k1.y;
        ss0 += z[j][0] * z[j][0] + z[j][1] * z[j][1];
        ss1 += z[j][2] * z[j][2] + z[j][3] * z[j][3];
    }
    ss0 += __shfl_xor_sync(0xffffffffu, ss0, 1); ss0 += __shfl_xor_sync(0xffffffffu, ss0, 2);
    ss1 += __shfl_xor_sync(0xffffffffu, ss1, 1); ss1 += __shfl_xor_sync(0xffffffffu, ss1, 2);
    const float in0 = rsqrtf(fmaxf(ss0, 1e-12f)), in1 = rsqrtf(fmaxf(ss1, 1e-12f));

#pragma unroll
    for (int j = 0; j < 8; ++j) {
        float fa[4] = {}, fm[4] = {}, fk[4] = {};
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
            uint32_t b[2];
            ldB_nk(b, &sm.W[1][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(fa, aa[ks], b);
            ldB_nk(b, &sm.W[2][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(fm, am[ks], b);
            ldB_nk(b, &sm.W[3][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(fk, ak[ks], b);
        }
        const int c = h * HC + 8 * j + 2 * t4;
        const float2 wb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.w_bias + c));
        const float2 ab = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.bias[0] + c));
        const float2 mb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.bias[1] + c));
        const float2 kb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.bias[2] + c));
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int tr = lr + g + 8 * hrow, tc = 8 * j + 2 * t4;
            const float2 wi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.io[0][tr][tc]));
            const float2 ki = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.io[1][tr][tc]));
            const float inorm = hrow ? in1 : in0;
            float ow[2], ok[2], okk[2], ob[2];
#pragma unroll
            for (int x = 0; x < 2; ++x) {
                const int i = 2 * hrow + x;
                const Gates gt = lora_gates(fa[i] + (x ? ab.y : ab.x), fm[i] + (x ? mb.y : mb.x), fk[i] + (x ? kb.y : kb.x),
                                            (x ? wb.y : wb.x) + (x ? wi.y : wi.x));
                const float kk = z[j][i] * inorm;
                ow[x] = gt.w;
                ok[x] = (x ? ki.y : ki.x) * (gt.ma + gt.a - gt.ma * gt.a) * gt.E;
                okk[x] = kk;
                ob[x] = -kk * gt.a;
            }
            // w and k replace w_in and k_in in their tiles (this thread's element, already read); kk and b get their own
            *reinterpret_cast<uint32_t*>(&sm.io[0][tr][tc]) = pack_bf16x2(ow[0], ow[1]);
            *reinterpret_cast<uint32_t*>(&sm.io[1][tr][tc]) = pack_bf16x2(ok[0], ok[1]);
            *reinterpret_cast<uint32_t*>(&sm.io[2][tr][tc]) = pack_bf16x2(okk[0], okk[1]);
            *reinterpret_cast<uint32_t*>(&sm.io[3][tr][tc]) = pack_bf16x2(ob[0], ob[1]);
        }
    }
    __syncwarp();
    {   // the warp's 16 rows of the four outputs leave as whole 128-byte rows (live rows only)
        bf16* outs[4] = {(bf16*)p.w_out, (bf16*)p.k_out, (bf16*)p.kk_out, (bf16*)p.b_out};
#pragma unroll
        for (int ten = 0; ten < 4; ++ten)
#pragma unroll
            for (int it = 0; it < 4; ++it) {
                const int r = lr + 4 * it + (lane >> 3), ch = lane & 7;
                const long long row = (long long)blockIdx.y * 64 + r;
                if (row < p.rows) *reinterpret_cast<uint4*>(outs[ten] + row * C + h * HC + ch * 8) = *reinterpret_cast<const uint4*>(&sm.io[ten][r][ch * 8]);
            }
    }
}

// ------------------------------------------------------------------------------------------------

template <int D> struct LorasBwdSmem {
    bf16 W[4][HC][D + 8];        // [channel][rank]: B operand of the forward, [k][n] operand of d(input)
    bf16 in[4][64][D + 16];      // tanh(z_in), a_in, ma_in, mk_in; column D is all ones (bias gradient)
    // [token][channel] tiles of one head.  On the way in (16-byte cp.async, whole 128-byte rows) tiles 0..5 hold
    // w_in, k_in, dw_out, dk_out, db_out, dkk_out.  Each thread replaces, element by element, what it has read: tiles
    // 0..4 become the pre-activation gradients of z, a, ma, mk and dw_in (the gradient of w_in), tile 5 becomes dk_in.
    bf16 gr[6][64][GLD];
};

template <int D>
__global__ void __launch_bounds__(128) loras_bwd_kernel(LorasParams p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sm = *reinterpret_cast<LorasBwdSmem<D>*>(smem_raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    const int h = blockIdx.x, C = (int)p.C, T = (int)p.T, H = C / HC;
    const long long b0 = (long long)blockIdx.y * T;

    for (int i = tid; i < 4 * HC * (D / 8); i += 128) {
        const int l = i / (HC * (D / 8)), r = (i / (D / 8)) % HC, ch = i % (D / 8);
        cp_async16(&sm.W[l][r][ch * 8], (const bf16*)p.W[l] + (long long)(h * HC + r) * D + ch * 8);
    }
    cp_async_commit();
    for (int i = tid; i < 4 * 64 * 16; i += 128) {  // ones column and padding
        const int l = i / (64 * 16), r = (i / 16) % 64, c = i % 16;
        sm.in[l][r][D + c] = __float2bfloat16(c == 0 ? 1.f : 0.f);
    }

    // weight-gradient accumulators: warp w owns LoRA w: [64 channels] x [D ranks + ones column],
    // plus channel m-tile w of the dw_bias column
    constexpr int NT = D / 8 + 1;
    float dWacc[4][NT][4] = {};
    float dwb[4] = {};

    // gridDim.z CTAs share a sequence: each walks a contiguous range of 64-token tiles (more resident
    // CTAs per SM; the price is one more flush of the weight-gradient accumulators per extra CTA)
    const int tiles = (T + 63) / 64, per = (tiles + (int)gridDim.z - 1) / (int)gridDim.z;
    const int tbeg = (int)blockIdx.z * per * 64, tend = min(T, tbeg + per * 64);
    for (int t0 = tbeg; t0 < tend; t0 += 64) {
        const long long r0 = b0 + t0 + 16 * warp;
        const bool valid = t0 + 16 * warp < T;
        // ---- the six [token][channel] tiles first (asynchronous copies), then this tile's LoRA inputs under them ------------
        {
            const bf16* src6[6] = {(const bf16*)p.w_in, (const bf16*)p.k_in, (const bf16*)p.dw_out, (const bf16*)p.dk_out,
                                   (const bf16*)p.db_out, (const bf16*)p.dkk_out};
            for (int i = tid; i < 6 * 64 * 8; i += 128) {
                const int ten = i / 512, r = (i / 8) % 64, ch = i % 8;
                const bool live = t0 + r < T;
                cp_async16_zfill(&sm.gr[ten][r][ch * 8], src6[ten] + (b0 + (live ? t0 + r : 0)) * C + h * HC + ch * 8, live);
            }
            cp_async_commit();
        }
        // LoRA inputs (tanh applied to z_in): the loads of a group of four are issued together, so that their latencies overlap
        {
            constexpr int ITEMS = 4 * 64 * (D / 8) / 128;  // per thread
            static_assert(ITEMS % 4 == 0, "groups of four loads per thread");
#pragma unroll
            for (int i0 = 0; i0 < ITEMS; i0 += 4) {
                uint4 v[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = tid + 128 * (i0 + u);
                    const int l = i / (64 * (D / 8)), r = (i / (D / 8)) % 64, ch = i % (D / 8);
                    v[u] = make_uint4(0, 0, 0, 0);
                    if (t0 + r < T) v[u] = *reinterpret_cast<const uint4*>((const bf16*)p.lin[l] + (b0 + t0 + r) * D + ch * 8);
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int i = tid + 128 * (i0 + u);
                    const int l = i / (64 * (D / 8)), r = (i / (D / 8)) % 64, ch = i % (D / 8);
                    if (l == 0) {
                        float f[8];
                        unpack8(v[u], f);
#pragma unroll
                        for (int q = 0; q < 8; ++q) f[q] = tanh_f(f[q]);
                        v[u] = pack8(f);
                    }
                    *reinterpret_cast<uint4*>(&sm.in[l][r][ch * 8]) = v[u];
                }
            }
        }
        cp_async_wait<0>();
        __syncthreads();

        if (valid) {
            const int lr = 16 * warp;  // first tile row of this warp
            uint32_t az[D / 16][4], aa[D / 16][4], am[D / 16][4], ak[D / 16][4];
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
                ldA_mk(az[ks], &sm.in[0][0][0], D + 16, lr, 16 * ks, g, t4);
                ldA_mk(aa[ks], &sm.in[1][0][0], D + 16, lr, 16 * ks, g, t4);
                ldA_mk(am[ks], &sm.in[2][0][0], D + 16, lr, 16 * ks, g, t4);
                ldA_mk(ak[ks], &sm.in[3][0][0], D + 16, lr, 16 * ks, g, t4);
            }
            // ---- pass A: z, a; row sums for the norm and its gradient -----------------------------------
            float z[8][4], dzo[8][4];
            float ss[2] = {0.f, 0.f}, dn[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float fa[4] = {};
                z[j][0] = z[j][1] = z[j][2] = z[j][3] = 0.f;
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t b[2];
                    ldB_nk(b, &sm.W[0][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(z[j], az[ks], b);
                    ldB_nk(b, &sm.W[1][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(fa, aa[ks], b);
                }
                const float2 ab = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.bias[0] + h * HC + 8 * j + 2 * t4));
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int tr = lr + g + 8 * hrow, tc = 8 * j + 2 * t4;
                    const float2 ki = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[1][tr][tc]));
                    const float2 dk = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[5][tr][tc]));
                    const float2 db = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[4][tr][tc]));
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int i = 2 * hrow + x;
                        z[j][i] += x ? ki.y : ki.x;
                        const float a = sigmoid_f(fa[i] + (x ? ab.y : ab.x));
                        dzo[j][i] = (x ? dk.y : dk.x) - (x ? db.y : db.x) * a;  // gradient of kk
                        ss[hrow] += z[j][i] * z[j][i];
                        dn[hrow] += dzo[j][i] * z[j][i];
                    }
                }
            }
#pragma unroll
            for (int hrow = 0; hrow < 2; ++hrow) {
                ss[hrow] += __shfl_xor_sync(0xffffffffu, ss[hrow], 1); ss[hrow] += __shfl_xor_sync(0xffffffffu, ss[hrow], 2);
                dn[hrow] += __shfl_xor_sync(0xffffffffu, dn[hrow], 1); dn[hrow] += __shfl_xor_sync(0xffffffffu, dn[hrow], 2);
            }
            const float inorm[2] = {rsqrtf(fmaxf(ss[0], 1e-12f)), rsqrtf(fmaxf(ss[1], 1e-12f))};
            // ---- pass B: everything elementwise, gradients into the shared tiles ----------------------------
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float fa[4] = {}, fm[4] = {}, fk[4] = {};
#pragma unroll
                for (int ks = 0; ks < D / 16; ++ks) {
                    uint32_t b[2];
                    ldB_nk(b, &sm.W[1][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(fa, aa[ks], b);
                    ldB_nk(b, &sm.W[2][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(fm, am[ks], b);
                    ldB_nk(b, &sm.W[3][0][0], D + 8, 8 * j, 16 * ks, g, t4); mma_bf16(fk, ak[ks], b);
                }
                const int c = h * HC + 8 * j + 2 * t4;
                const float2 wb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.w_bias + c));
                const float2 ab = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.bias[0] + c));
                const float2 mb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.bias[1] + c));
                const float2 kb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>((const bf16*)p.bias[2] + c));
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int tr = lr + g + 8 * hrow, tc = 8 * j + 2 * t4;
                    const float2 wi = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[0][tr][tc]));
                    const float2 ki = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[1][tr][tc]));
                    const float2 gw = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[2][tr][tc]));
                    const float2 gk = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[3][tr][tc]));
                    const float2 gb = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.gr[4][tr][tc]));
                    float o_dw[2], o_dk[2], o_z[2], o_a[2], o_m[2], o_k[2];
#pragma unroll
                    for (int x = 0; x < 2; ++x) {
                        const int i = 2 * hrow + x;
                        const float v = (x ? wb.y : wb.x) + (x ? wi.y : wi.x);
                        const Gates gt = lora_gates(fa[i] + (x ? ab.y : ab.x), fm[i] + (x ? mb.y : mb.x), fk[i] + (x ? kb.y : kb.x), v);
                        const float a = gt.a, ma = gt.ma, mk = gt.mk, w = gt.w, E = gt.E;
                        const float kin = x ? ki.y : ki.x;
                        const float kmix = ma + a - ma * a;
                        const float zz = z[j][i], kk = zz * inorm[hrow];
                        const float dkE = (x ? gk.y : gk.x) * E;
                        const float de = dkE * kin * kmix;                       // gradient of w*mk
                        const float dwt = (x ? gw.y : gw.x) + de * mk;
                        const float dmk = de * w;
                        const float dma = dkE * (kin - kin * a);
                        const float da = -(x ? gb.y : gb.x) * kk + dkE * (kin - kin * ma);
                        const float in3 = inorm[hrow] * inorm[hrow] * inorm[hrow];
                        const float dz = dzo[j][i] * inorm[hrow] - in3 * dn[hrow] * zz;
                        o_dw[x] = dwt * sigmoid_f(-v);
                        o_dk[x] = dkE * kmix + dz;
                        o_z[x] = dz;
                        o_a[x] = da * a * (1.f - a);
                        o_m[x] = dma * ma * (1.f - ma);
                        o_k[x] = dmk * mk * (1.f - mk);
                    }
                    *reinterpret_cast<uint32_t*>(&sm.gr[5][tr][tc]) = pack_bf16x2(o_dk[0], o_dk[1]);
                    *reinterpret_cast<uint32_t*>(&sm.gr[0][tr][tc]) = pack_bf16x2(o_z[0], o_z[1]);
                    *reinterpret_cast<uint32_t*>(&sm.gr[1][tr][tc]) = pack_bf16x2(o_a[0], o_a[1]);
                    *reinterpret_cast<uint32_t*>(&sm.gr[2][tr][tc]) = pack_bf16x2(o_m[0], o_m[1]);
                    *reinterpret_cast<uint32_t*>(&sm.gr[3][tr][tc]) = pack_bf16x2(o_k[0], o_k[1]);
                    *reinterpret_cast<uint32_t*>(&sm.gr[4][tr][tc]) = pack_bf16x2(o_dw[0], o_dw[1]);
                }
            }
            __syncwarp();
            {   // dw_in (tile 4) and dk_in (tile 5) of the warp's 16 rows leave as whole 128-byte rows (live rows only)
#pragma unroll
                for (int ten = 4; ten < 6; ++ten)
#pragma unroll
                    for (int it = 0; it < 4; ++it) {
                        const int r = lr + 4 * it + (lane >> 3), ch = lane & 7;
                        if (t0 + r < T)
                            *reinterpret_cast<uint4*>((bf16*)(ten == 4 ? p.dw_in : p.dk_in) + (b0 + t0 + r) * C + h * HC + ch * 8) =
                                *reinterpret_cast<const uint4*>(&sm.gr[ten][r][ch * 8]);
                    }
            }
            // ---- d(input) partial of this head: [16, D] = grad[16, 64] @ W[64, D] ----------------------------
#pragma unroll
            for (int l = 0; l < 4; ++l) {
                float acc[D / 8][4] = {};
#pragma unroll
                for (int ks = 0; ks < HC / 16; ++ks) {
                    uint32_t a[4];
                    ldA_mk(a, &sm.gr[l][0][0], GLD, lr, 16 * ks, g, t4);
#pragma unroll
                    for (int j = 0; j < D / 8; ++j) {
                        uint32_t b[2];
                        ldB_kn_trans(b, &sm.W[l][0][0], D + 8, 8 * j, 16 * ks, lane);
                        mma_bf16(acc[j], a, b);
                    }
                }
                bf16* po = (bf16*)p.partial + (((long long)l * p.rows + r0 + g) * H + h) * D + 2 * t4;
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    float v0 = acc[j][0], v1 = acc[j][1], v2 = acc[j][2], v3 = acc[j][3];
                    if (l == 0) {  // through the tanh of z_in
                        const float2 t0v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.in[0][lr + g][8 * j + 2 * t4]));
                        const float2 t1v = unpack_bf16x2(*reinterpret_cast<const uint32_t*>(&sm.in[0][lr + g + 8][8 * j + 2 * t4]));
                        v0 *= 1.f - t0v.x * t0v.x; v1 *= 1.f - t0v.y * t0v.y;
                        v2 *= 1.f - t1v.x * t1v.x; v3 *= 1.f - t1v.y * t1v.y;
                    }
                    *reinterpret_cast<uint32_t*>(po + 8 * j) = pack_bf16x2(v0, v1);
                    *reinterpret_cast<uint32_t*>(po + 8LL * H * D + 8 * j) = pack_bf16x2(v2, v3);
                }
            }
        } else {
            // rows past the end of the sequence contribute nothing to the weight gradients
            for (int i = lane; i < 5 * 16 * (HC / 8); i += 32) {
                const int l = i / (16 * (HC / 8)), r = (i / (HC / 8)) % 16, ch = i % (HC / 8);
                *reinterpret_cast<uint4*>(&sm.gr[l][16 * warp + r][ch * 8]) = make_uint4(0, 0, 0, 0);
            }
        }
        __syncthreads();
        // ---- weight gradients: dW_l[64, D+ones] += grad_l^T[64, tokens] @ in_l[tokens, D+ones] ---------------
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            uint32_t b[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) ldB_kn_trans(b[j], &sm.in[warp][0][0], D + 16, 8 * j, 16 * ks, lane);
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                uint32_t a[4];
                ldA_km_trans(a, &sm.gr[warp][0][0], GLD, 16 * mt, 16 * ks, lane);
#pragma unroll
                for (int j = 0; j < NT; ++j) mma_bf16(dWacc[mt][j], a, b[j]);
            }
            uint32_t a[4];
            ldA_km_trans(a, &sm.gr[4][0][0], GLD, 16 * warp, 16 * ks, lane);
            mma_bf16(dwb, a, b[NT - 1]);
        }
        __syncthreads();
    }

    // ---- flush ------------------------------------------------------------------------------------------
    float* dWo = p.dW[warp];
    float* dbo = warp == 0 ? nullptr : p.dbias[warp - 1];  // LoRA 0 (z) has no bias
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int hrow = 0; hrow < 2; ++hrow) {
            const int ch = h * HC + 16 * mt + g + 8 * hrow;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                atomicAdd(dWo + (long long)ch * D + 8 * j + 2 * t4, dWacc[mt][j][2 * hrow]);
                atomicAdd(dWo + (long long)ch * D + 8 * j + 2 * t4 + 1, dWacc[mt][j][2 * hrow + 1]);
            }
            if (dbo && t4 == 0) atomicAdd(dbo + ch, dWacc[mt][NT - 1][2 * hrow]);
        }
    if (t4 == 0) {
        atomicAdd(p.dw_bias + h * HC + 16 * warp + g, dwb[0]);
        atomicAdd(p.dw_bias + h * HC + 16 * warp + g + 8, dwb[2]);
    }
}

// sums the per-head partials: out[l][row][d] = sum_h partial[l][row][h][d]
__global__ void loras_reduce_heads_kernel(LorasParams p, int H, int D) {
    const long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;  // index over [4, rows, D]
    const long long per = p.rows * D;
    if (i >= 4 * per) return;
    const int l = (int)(i / per);
    const long long rd = i % per, row = rd / D;
    const int d = (int)(rd % D);
    const bf16* src = (const bf16*)p.partial + ((long long)l * p.rows + row) * H * D + d;
    float acc = 0.f;
    for (int hh = 0; hh < H; ++hh) acc += __bfloat162float(src[(long long)hh * D]);
    ((bf16*)p.dlin[l])[rd] = __float2bfloat16_rn(acc);
}

template <int D> static int launch_loras_fwd_t(const LorasParams& p, cudaStream_t stream) {
    auto kern = loras_fwd_kernel<D>;
    const int smem = (int)sizeof(LorasFwdSmem<D>);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    kern<<<dim3((unsigned)(p.C / HC), (unsigned)((p.rows + 63) / 64)), 128, smem, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

template <int D> static int launch_loras_bwd_t(const LorasParams& p, cudaStream_t stream) {
    const int C = (int)p.C, H = C / HC;
    for (int l = 0; l < 4; ++l)
        if (cudaMemsetAsync(p.dW[l], 0, sizeof(float) * C * D, stream) != cudaSuccess) return kLaunchFailed;
    if (cudaMemsetAsync(p.dw_bias, 0, sizeof(float) * C, stream) != cudaSuccess) return kLaunchFailed;
    for (int l = 0; l < 3; ++l)
        if (cudaMemsetAsync(p.dbias[l], 0, sizeof(float) * C, stream) != cudaSuccess) return kLaunchFailed;
    auto kern = loras_bwd_kernel<D>;
    const int smem = (int)sizeof(LorasBwdSmem<D>);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return kLaunchFailed;
    // enough CTAs for about eight per SM (three are resident at a time), at most one per 64-token tile
    const long long seqs = (long long)H * (p.rows / p.T), tiles = (p.T + 63) / 64;
    long long nseg = (8 * 148 + seqs - 1) / seqs;
    if (nseg > tiles) nseg = tiles;
    if (nseg < 1) nseg = 1;
    kern<<<dim3((unsigned)H, (unsigned)(p.rows / p.T), (unsigned)nseg), 128, smem, stream>>>(p);
    if (cudaGetLastError() != cudaSuccess) return kLaunchFailed;
    const long long n = 4 * p.rows * D;
    loras_reduce_heads_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(p, H, D);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

int launch_loras_fwd(const LorasParams& p, cudaStream_t stream) {
    switch (p.D) {
        case 16: return launch_loras_fwd_t<16>(p, stream);
        case 32: return launch_loras_fwd_t<32>(p, stream);
        case 64: return launch_loras_fwd_t<64>(p, stream);
        case 128: return launch_loras_fwd_t<128>(p, stream);
        default: return kBadShape;
    }
}
int launch_loras_bwd(const LorasParams& p, cudaStream_t stream) {
    switch (p.D) {
        case 16: return launch_loras_bwd_t<16>(p, stream);
        case 32: return launch_loras_bwd_t<32>(p, stream);
        case 64: return launch_loras_bwd_t<64>(p, stream);
        case 128: return launch_loras_bwd_t<128>(p, stream);
        default: return kBadShape;
    }
}

}  // namespace wkv7
