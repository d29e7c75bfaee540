// Launcher interface of the ddlerp kernels (forward: ddlerp_fwd.cu, backward: ddlerp_bwd.cu).
#pragma once
#include "wkv7_common.cuh"

namespace wkv7 {

struct DdlerpFwdParams {
    const void *x, *alpha, *L, *R, *beta;  // bf16: [rows,C], [C], [4D,C], [4,C,D], [4,C]
    void* m;                                // bf16 [rows,4D]  tanh activations, kept for the backward
    void* y;                                // bf16 [4,rows,C]
    long long rows, T, C;                   // rows = B*T
    int D;
};

struct DdlerpBwdParams {
    const void *x, *alpha, *L, *R, *beta, *m;  // as the forward
    const void* dy[4];                          // bf16 [rows,C] each
    void* dpre;                                 // bf16 [rows,4D] workspace: gradient before the tanh
    void* dx;                                   // bf16 [rows,C]
    float *dalpha, *dL, *dR, *dbeta;            // fp32 [C], [4D,C], [4,C,D], [4,C]; zero-filled by the launcher
    long long rows, T, C;
    int D;
};

int launch_ddlerp_fwd(const DdlerpFwdParams& p, cudaStream_t stream);
// tcgen05 + TMA form of the forward (ddlerp_tc.cu); `ws` holds ddlerp_fwd_tc_workspace_bytes(C, D) bytes of scratch
size_t ddlerp_fwd_tc_workspace_bytes(long long C, int D);
int launch_ddlerp_fwd_tc(const DdlerpFwdParams& p, void* ws, int* status, cudaStream_t stream);
int launch_ddlerp_bwd(const DdlerpBwdParams& p, cudaStream_t stream);
// The backward with dL formed on the tensor cores (ddlerp_tc.cu); `ws`: ddlerp_bwd_tc_workspace_bytes(C, D) bytes of scratch
size_t ddlerp_bwd_tc_workspace_bytes(long long C, int D);
int launch_ddlerp_bwd_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream);
int launch_ddlerp_dL_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream, bool with_dalpha);
int launch_ddlerp_main_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream);  // kBadShape: rank not covered
int launch_ddlerp_prep_bwd(const DdlerpBwdParams& p, void* ws, cudaStream_t stream);  // rearranged weights for the two below
int launch_ddlerp_dpre_tc(const DdlerpBwdParams& p, void* ws, int* status, cudaStream_t stream);  // kBadShape: rank not covered

}  // namespace wkv7
