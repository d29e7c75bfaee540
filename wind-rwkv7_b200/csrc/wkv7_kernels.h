// Internal launcher interface between the C ABI (capi.cu) and the kernel translation units.
#pragma once
#include "wkv7_common.cuh"

namespace wkv7 {

struct FwdParams {
    const void *r, *w, *k, *v, *a, *b;  // [B,T,H,N], io dtype
    const void* g;                      // attn_ln only
    const float* params;                // attn_ln only: [3, H*N] = ln_weight, ln_bias, bonus
    const float* s0;                    // [B,H,N,N] or null (zeros)
    void* y;                            // [B,T,H,N]
    float* sT;                          // [B,H,N,N] or null
    float* ckpt;                        // [B,H,T/16,CK_FLOATS] checkpoint records (chunk-start state + 4 matrices), or null
    long long B, T, H;
    Strides st;
    float eps;
    int* status;                        // device status word
};

struct BwdParams {
    const void *r, *w, *k, *v, *a, *b, *dy;  // dy: gradient of y (attn) or of the fused output (attn_ln)
    const void* g;           // attn_ln only
    const float* params;     // attn_ln only
    void* dg;                // attn_ln only
    float* dparams;          // attn_ln only: [3, H*N]
    float* dparams_ws;       // attn_ln only: [B, 3, H*N] per-(batch, head) partials
    float eps;
    const float* ckpt;   // written by the forward
    const float* dsT;    // [B,H,N,N] or null (zeros)
    const float* sT;     // final state of the forward; needed only when dsT is given
    void *dr, *dw, *dk, *dv, *da, *db;
    float* ds0;          // or null
    long long B, T, H;
    Strides st;
    int* status;
};

struct StepParams {
    const void *r, *w, *k, *v, *a, *b;  // [B,T,H,N], io dtype
    const float* s0;                    // [B,H,N,N] or null (zeros); may be the same buffer as sT
    void* y;                            // [B,T,H,N]
    float* sT;                          // [B,H,N,N] or null
    long long B, T, H;
    Strides st;
};

int launch_fwd(const FwdParams& p, int io_dtype, bool ln, cudaStream_t stream);
// the recurrence step by step on fp32 FMAs (decode); io_dtype 0 = bf16, otherwise fp32 tensors
int launch_step(const StepParams& p, int io_dtype, cudaStream_t stream);
int launch_bwd(const BwdParams& p, int io_dtype, bool ln, cudaStream_t stream);
// tcgen05 forward (bf16 IO; attn, or attn_ln with ln = true); |groups| = preparation groups per CTA (2..4); negative: operands are
// not rounded to TF32 by their producer (the tensor core truncates them)
int launch_fwd_tc(const FwdParams& p, int groups, bool ln, cudaStream_t stream);
// C[M,N] = act(A[M,K] W[N,K]^T), bf16, tanh on columns [tanh_from, tanh_to); tcgen05 + TMA (proj_gemm.cu)
int launch_proj_gemm(const void* A, const void* W, void* C, long long M, long long N, long long K, int tanh_from, int tanh_to,
                     int* status, cudaStream_t stream);
// one small CTA running the tcgen05 forward's bounded mbarrier wait on barriers nothing arrives on
int launch_bounded_wait_selftest(long long limit_cycles, int* status, long long* cycles, cudaStream_t stream);

}  // namespace wkv7
