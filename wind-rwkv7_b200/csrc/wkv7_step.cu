// WKV7 decode step: the recurrence itself, one time step at a time, for generation after a prefill.
//
//     S <- S diag(exp(-exp(w_t))) + (S a_t) b_t^T + v_t k_t^T ,   y_t = S r_t
//
// (the loop body of the reference's naive recurrence, wind_rwkv/rwkv7/time_mixer.py:13-15; the
// reference has no kernel for it: its chunked kernels need T % 16 == 0, rwkv7_attn.py:22).  The
// state uses the fp32 [B,H,N,N] format of wkv7_fwd's s0 / sT, so a prefill's final state is this
// kernel's input.  Meant for T of one to a few steps: no chunking, no tensor cores, no checkpoints;
// plain fp32 FMAs, exact to fp32 rounding.
//
// One CTA of 256 threads per (batch, head) chain.  Thread (i, q) = (tid / 4, tid % 4) keeps columns
// 16q..16q+15 of state row i in registers for all T steps; the two row contractions (S a and S r)
// are 16 FMAs per thread and two shuffles across the row's four threads.  The kernel is bound by
// the state traffic: 2 * 16 KB per chain and call, 64-byte pieces per thread, 2 KB contiguous per
// warp.
#include "wkv7_kernels.h"

namespace wkv7 {

template <typename IoT> __device__ __forceinline__ void load16(const IoT* p, float (&f)[16]);
template <> __device__ __forceinline__ void load16<float>(const float* p, float (&f)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 x = *reinterpret_cast<const float4*>(p + 4 * i);
        f[4 * i] = x.x; f[4 * i + 1] = x.y; f[4 * i + 2] = x.z; f[4 * i + 3] = x.w;
    }
}
template <> __device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[16]) {
    float lo[8], hi[8];
    load8<__nv_bfloat16>(reinterpret_cast<const unsigned char*>(p), lo);
    load8<__nv_bfloat16>(reinterpret_cast<const unsigned char*>(p + 8), hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) { f[i] = lo[i]; f[8 + i] = hi[i]; }
}

template <typename IoT>
__global__ void __launch_bounds__(256) wkv7_step_kernel(StepParams p) {
    const int tid = threadIdx.x, i = tid >> 2, q = tid & 3;
    const long long bh = blockIdx.x;
    const long long bi = bh / p.H, hi = bh % p.H;
    const long long base = bi * p.st.b + hi * p.st.h;
    float S[16];
    if (p.s0) {
        load16<float>(p.s0 + bh * N * N + i * N + 16 * q, S);
    } else {
#pragma unroll
        for (int j = 0; j < 16; ++j) S[j] = 0.f;
    }
    for (long long t = 0; t < p.T; ++t) {
        const long long off = base + t * p.st.t + 16 * q;
        float w[16], a[16], b[16], k[16], r[16];
        load16<IoT>((const IoT*)p.w + off, w);
        load16<IoT>((const IoT*)p.a + off, a);
        load16<IoT>((const IoT*)p.b + off, b);
        load16<IoT>((const IoT*)p.k + off, k);
        load16<IoT>((const IoT*)p.r + off, r);
        const float v = to_f32<IoT>(((const IoT*)p.v)[base + t * p.st.t + i]);
        float sa = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sa = fmaf(S[j], a[j], sa);
        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
        sa += __shfl_xor_sync(0xffffffffu, sa, 2);
        float y = 0.f;
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            S[j] = fmaf(S[j], expf(-expf(w[j])), fmaf(sa, b[j], v * k[j]));
            y = fmaf(S[j], r[j], y);
        }
        y += __shfl_xor_sync(0xffffffffu, y, 1);
        y += __shfl_xor_sync(0xffffffffu, y, 2);
        if (q == 0) ((IoT*)p.y)[base + t * p.st.t + i] = from_f32<IoT>(y);
    }
    if (p.sT) {
        float* o = p.sT + bh * N * N + i * N + 16 * q;
#pragma unroll
        for (int j = 0; j < 4; ++j) *reinterpret_cast<float4*>(o + 4 * j) = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    }
}

int launch_step(const StepParams& p, int io_dtype, cudaStream_t stream) {
    if (io_dtype == 0) wkv7_step_kernel<__nv_bfloat16><<<(unsigned)(p.B * p.H), 256, 0, stream>>>(p);
    else wkv7_step_kernel<float><<<(unsigned)(p.B * p.H), 256, 0, stream>>>(p);
    return cudaGetLastError() == cudaSuccess ? kOk : kLaunchFailed;
}

}  // namespace wkv7
