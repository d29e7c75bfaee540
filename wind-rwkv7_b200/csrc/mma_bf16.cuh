// bf16 warp-MMA helpers (m16n8k16, fp32 accumulate), ldmatrix, cp.async: shared by the ddlerp
// and expand_loras kernels, whose contractions take bf16 operands exactly as their inputs are.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "wkv7_common.cuh"

namespace wkv7 {

using bf16 = __nv_bfloat16;

// Fragment layouts (g = lane/4, t = lane%4), each register two bf16 with the lower index low:
//   A 16x16: a0 (g, 2t..2t+1)  a1 (g+8, 2t..)  a2 (g, 2t+8..)  a3 (g+8, 2t+8..)
//   B 16x8 : b0 (k=2t..2t+1, n=g)  b1 (k=2t+8.., n=g)
//   C 16x8 : c0 (g,2t) c1 (g,2t+1) c2 (g+8,2t) c3 (g+8,2t+1)
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}

// A fragment from shared memory laid out [m][k] (ld in elements): rows m0+g, m0+g+8; k block k0.
__device__ __forceinline__ void ldA_mk(uint32_t (&a)[4], const bf16* p, int ld, int m0, int k0, int g, int t) {
    const bf16* r0 = p + (m0 + g) * ld + k0 + 2 * t;
    const bf16* r1 = r0 + 8 * ld;
    a[0] = *reinterpret_cast<const uint32_t*>(r0);
    a[1] = *reinterpret_cast<const uint32_t*>(r1);
    a[2] = *reinterpret_cast<const uint32_t*>(r0 + 8);
    a[3] = *reinterpret_cast<const uint32_t*>(r1 + 8);
}
// B fragment from shared memory laid out [n][k]: row n0+g, k block k0.
__device__ __forceinline__ void ldB_nk(uint32_t (&b)[2], const bf16* p, int ld, int n0, int k0, int g, int t) {
    const bf16* r0 = p + (n0 + g) * ld + k0 + 2 * t;
    b[0] = *reinterpret_cast<const uint32_t*>(r0);
    b[1] = *reinterpret_cast<const uint32_t*>(r0 + 8);
}

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return smem_u32(p); }

// B fragment from shared memory laid out [k][n] (row = contraction index): transposing ldmatrix.
// Rows k0..k0+15, columns n0..n0+7; rows must be 16-byte aligned.
__device__ __forceinline__ void ldB_kn_trans(uint32_t (&b)[2], const bf16* p, int ld, int n0, int k0, int lane) {
    const bf16* row = p + (k0 + (lane & 15)) * ld + n0;
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b[0]), "=r"(b[1]) : "r"(smem_addr(row)));
}
// A fragment from shared memory laid out [k][m] (the transpose of the operand): rows k0..k0+15,
// columns m0..m0+15.
__device__ __forceinline__ void ldA_km_trans(uint32_t (&a)[4], const bf16* p, int ld, int m0, int k0, int lane) {
    // matrices: 0 (k 0-7, m 0-7) -> a0, 1 (k 0-7, m 8-15) -> a1, 2 (k 8-15, m 0-7) -> a2, 3 (k 8-15, m 8-15) -> a3
    const int mat = lane >> 3, r = lane & 7;
    const bf16* row = p + (k0 + r + 8 * (mat >> 1)) * ld + m0 + 8 * (mat & 1);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3])
                 : "r"(smem_addr(row)));
}

// tanh on the special-function unit (one MUFU instruction, relative error 2^-11: below the bf16 rounding of every value
// these kernels pass through it), and the logistic function through it: sigmoid(x) = 0.5 tanh(x / 2) + 0.5.
__device__ __forceinline__ float tanh_f(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sigmoid_f(float x) { return fmaf(0.5f, tanh_f(0.5f * x), 0.5f); }

// 8 consecutive bf16 <-> 8 floats
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

}  // namespace wkv7
