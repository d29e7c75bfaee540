// Launcher interface of the expand_loras kernels (expand_loras.cu).
#pragma once
#include "wkv7_common.cuh"

namespace wkv7 {

struct LorasParams {
    // forward inputs (bf16): w_in,k_in [rows,C]; z_in,a_in,ma_in,mk_in [rows,D]; W* [C,D]; biases [C]
    const void *w_in, *k_in, *lin[4];   // lin: z_in, a_in, ma_in, mk_in
    const void* W[4];                   // Wz, Wa, Wma, Wmk
    const void *w_bias, *bias[3];       // bias: a_bias, ma_bias, mk_bias
    // forward outputs (bf16 [rows,C])
    void *w_out, *k_out, *kk_out, *b_out;
    // backward inputs (bf16 [rows,C]) and outputs
    const void *dw_out, *dk_out, *dkk_out, *db_out;
    void *dw_in, *dk_in;                // bf16 [rows,C]
    void* dlin[4];                      // bf16 [rows,D]: dz_in, da_in, dma_in, dmk_in
    void* partial;                      // bf16 [4, rows, H, D] per-head partials of dlin
    float* dW[4];                       // fp32 [C,D]
    float *dw_bias, *dbias[3];          // fp32 [C]
    long long rows, T, C;               // rows = B*T
    int D;
};

int launch_loras_fwd(const LorasParams& p, cudaStream_t stream);
int launch_loras_bwd(const LorasParams& p, cudaStream_t stream);

}  // namespace wkv7
