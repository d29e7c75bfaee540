/*
 * C ABI of libwkv7_sm100.so — the B200 (sm_100a) implementation of the RWKV-7 WKV7 hot path.
 *
 * Plain pointers and sizes only; every buffer (inputs, outputs, checkpoints) is owned and
 * allocated by the caller, the library never allocates device memory.  All pointers are device
 * pointers unless said otherwise.  Every entry point validates its arguments on the host and
 * returns a status code (0 = success, negative = WKV7_ERR_*) without launching anything when
 * validation fails.  Kernels are launched on `stream` (a cudaStream_t passed as void*; 0 = the
 * default stream) and the call returns without synchronising.
 *
 * Tensor layout (the reference's internal op layout, wind_rwkv/rwkv7/rwkv7_attn.py:53-59):
 *   r, w, k, v, a, b, g, y and their gradients: [B, T, H, N] with element strides
 *   (stride_b, stride_t, stride_h, 1); N == 64.  A contiguous [B, T, H*N] tensor has
 *   stride_b = T*H*N, stride_t = H*N, stride_h = N.  Head- or batch-sharded views are
 *   expressed through the strides.  Base pointers and strides must keep every row 16-byte
 *   aligned.  States s0, sT, dsT, ds0: fp32 [B, H, N, N] contiguous, S[value][key].
 *   Checkpoints: fp32 [B, H, ceil(T/16), WKV7_CHECKPOINT_FLOATS] contiguous, one record per 16-step chunk; the
 *   contents are private to the library.  Size the buffer with wkv7_checkpoint_bytes() and nothing else.
 *   io_dtype: WKV7_BF16 (bf16 tensors, single-TF32 tensor-core products, fp32 state) or
 *   WKV7_F32 (fp32 tensors, 3xTF32 split products), or WKV7_F32_TF32 (fp32 tensors, single-TF32
 *   products: what the bf16 path computes, observable without bf16 output rounding).
 *
 * Recurrence (w is the RAW decay input; the op applies exp(-exp(w)) itself):
 *   S_t = S_{t-1} diag(exp(-exp(w_t))) + (S_{t-1} a_t) b_t^T + v_t k_t^T ,   y_t = S_t r_t
 */
#ifndef WKV7_SM100_H
#define WKV7_SM100_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define WKV7_BF16 0
#define WKV7_F32 1
#define WKV7_F32_TF32 2 /* fp32 tensors, single-TF32 products: the bf16 path's arithmetic without output rounding */

#define WKV7_OK 0
#define WKV7_ERR_SHAPE (-1)          /* negative or inconsistent dimensions */
#define WKV7_ERR_HEAD_SIZE (-2)      /* only N == 64 is built */
#define WKV7_ERR_CHUNK (-3)          /* expand_loras: T not a multiple of 16; ddlerp, expand_loras: C not a multiple of 64 */
#define WKV7_ERR_ALIGN (-4)          /* a pointer or stride breaks 16-byte row alignment */
#define WKV7_ERR_DTYPE (-5)
#define WKV7_ERR_NULL (-6)           /* a required pointer is null */
#define WKV7_ERR_LAUNCH (-7)         /* the CUDA launch failed */
#define WKV7_ERR_TOO_LARGE (-8)
#define WKV7_ERR_DEVICE_TIMEOUT (-9) /* reported by wkv7_device_status() */
#define WKV7_ERR_STATIC_SCRATCH (-10) /* problem too large for wkv7_attn_ln_bwd_static's built-in scratch */

/* Size of the scratch array compiled into the library for wkv7_attn_ln_bwd_static. */
#define WKV7_STATIC_SCRATCH_BYTES (4u << 20)

/* Human-readable text for a status code (host pointer, static storage). */
const char* wkv7_status_string(int status);

/* Bytes of checkpoint buffer the forward writes for the backward: B*H*ceil(T/16) records of
 * WKV7_CHECKPOINT_FLOATS floats (the N*N chunk-start state and the chunk's four 16x16 score / inverse
 * matrices, which the backward loads instead of rebuilding).  The contents are private to the library
 * (in the bf16 and F32_TF32 classes the matrices are rounded to TF32): only a buffer written by wkv7_fwd /
 * wkv7_attn_ln_fwd with the same io_dtype may be given to the backward.  0 for N != 64. */
#define WKV7_CHECKPOINT_FLOATS (64 * 64 + 4 * 16 * 16)
int64_t wkv7_checkpoint_bytes(int64_t B, int64_t T, int64_t H, int64_t N);

/* Device-side errors.  The kernels wait on mbarriers with a cycle limit; a wait that runs out makes its CTA finish
 * early and writes WKV7_ERR_DEVICE_TIMEOUT into a status word (one per process, a managed variable inside the library that
 * host and GPUs can both access; nothing is allocated for it).  No reference counterpart (the reference's kernels have no waits that could be bounded).
 * wkv7_device_status(): synchronises the current device (all its streams), then returns the word and clears it, in
 *   one atomic step.  0 = no error since the last call.
 * wkv7_peek_status(): returns the word without synchronising and without clearing it: a plain host load, cheap
 *   enough for every call.  It sees the errors of kernels that have finished; the Python wrappers look at it
 *   before every launch, so a timeout surfaces at the next call at the latest, without a device-wide sync. */
int wkv7_device_status(void);
int wkv7_peek_status(void);

/*
 * Self-test of the bounded device-side wait (no reference counterpart).  Launches one 128-thread CTA in
 * which two warps wait, with a limit of `limit_cycles` SM cycles, on mbarriers that nothing arrives on
 * (one polling, one hardware-suspended: the two forms the tcgen05 forward uses), and two more warps then
 * wait with the kernel's full limit and must return at once because the CTA has aborted.  Synchronises
 * the stream.  cycles_out (host, 4 values, may be null) receives the cycles each warp's wait took.
 * Returns the device status word, read and cleared: WKV7_ERR_DEVICE_TIMEOUT when the path works.  The
 * kernel touches no tensor memory and cannot fault or hang; the context stays usable.
 */
int wkv7_selftest_bounded_wait(int64_t limit_cycles, int64_t* cycles_out, void* stream);

/*
 * Which kernel wkv7_fwd and wkv7_attn_ln_fwd run for io_dtype WKV7_BF16 (no reference counterpart: the reference has one
 * forward kernel per dtype).  0: the warp-MMA kernel (mma.sync TF32, state in registers).  2, 3, 4: the
 * tcgen05 kernel (state in tensor memory) with that many preparation groups per CTA; negative values
 * select the same kernel without the producer-side rounding of operands to TF32 (the tensor core then
 * truncates them: 0.4 % faster, about twice the state error).  The default is 4, or the value of the environment variable WKV7_FWD_TC when the library
 * is loaded.  Returns WKV7_ERR_SHAPE for any other value.  The fp32 dtypes always use the warp-MMA
 * kernel.
 */
int wkv7_set_fwd_impl(int impl);
int wkv7_get_fwd_impl(void);

/*
 * WKV7 forward.  Replaces cuda_forward / forward_kernel of the reference
 * (wind_rwkv/rwkv7/attn.cpp:8-13, attn.cu:11-128) behind th.ops.wind.forward
 * (rwkv7_attn.py:5-11).  s0 may be null (zero initial state), sT may be null (final state not
 * wanted), ckpt may be null (no backward will follow).  Any T >= 0: the reference requires T % 16 == 0
 * (rwkv7_attn.py:22); here the missing time steps of a last, partial chunk are treated as zero inputs with no
 * decay, nothing is read or written beyond row T-1.  WKV7_ERR_TOO_LARGE when B*H*ceil(T/16)*80 >= 2^31.
 */
int wkv7_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
             const float* s0, void* y, float* sT, float* ckpt,
             int64_t B, int64_t T, int64_t H, int64_t N,
             int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream);

/*
 * WKV7 decode step(s): the recurrence itself, time step by time step, for generation after a prefill.
 * Restates the loop body of the reference's naive recurrence (wind_rwkv/rwkv7/time_mixer.py:13-15); the
 * reference has no kernel for it (its chunked kernels require T % 16 == 0, rwkv7_attn.py:22).  Same
 * tensors, strides and fp32 state format as wkv7_fwd, so a prefill's sT is this call's s0; s0 and sT may
 * be the same buffer (update in place); s0 null = zero state, sT null = state not wanted.  Meant for T of
 * one to a few steps (any T >= 0 is accepted; time is linear in T with one CTA per (batch, head)).  Plain
 * fp32 arithmetic for every io_dtype: results equal the chunked kernels' up to fp32 / TF32 rounding, not
 * bit for bit.  No checkpoints, no backward.
 */
int wkv7_step(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
              const float* s0, void* y, float* sT,
              int64_t B, int64_t T, int64_t H, int64_t N,
              int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream);

/*
 * WKV7 backward.  Replaces cuda_backward / backward_kernel of the reference
 * (attn.cpp:15-22, attn.cu:131-348) behind th.ops.wind.backward (rwkv7_attn.py:13-16).
 * ckpt is what wkv7_fwd wrote.  dsT may be null (zero); when dsT is given, sT (the forward's
 * final state) is required.  ds0 may be null.  Gradients use the same strides as the inputs.
 */
int wkv7_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
             const void* dy, const float* ckpt, const float* dsT, const float* sT,
             void* dr, void* dw, void* dk, void* dv, void* da, void* db, float* ds0,
             int64_t B, int64_t T, int64_t H, int64_t N,
             int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream);

/*
 * Fused WKV7 + per-head GroupNorm (eps) + bonus term + output gate, forward.  Replaces the
 * attn_ln variant (wind_rwkv/rwkv7/attn_ln.cpp:10-13, attn_ln.cu:106-234; Python side
 * rwkv7_attn_ln.py:5-11).  params: fp32 [3, H*N] = (GroupNorm weight, GroupNorm bias, bonus).
 *   y = (GroupNorm_head(S_t r_t) + (sum_j r_j k_j bonus_j) v) * g
 */
int wkv7_attn_ln_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                     const void* g, const float* params, const float* s0, void* y, float* sT, float* ckpt,
                     float eps, int64_t B, int64_t T, int64_t H, int64_t N,
                     int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream);

/* Bytes of workspace wkv7_attn_ln_bwd needs: B*3*H*N*4 (per-batch partial parameter gradients). */
int64_t wkv7_attn_ln_bwd_workspace_bytes(int64_t B, int64_t H, int64_t N);

/*
 * Backward of the fused attn_ln op.  Replaces the attn_ln cuda_backward / backward_kernel
 * (wind_rwkv/rwkv7/attn_ln.cpp:15-22, attn_ln.cu:237-486; Python side rwkv7_attn_ln.py:13-17).
 * dy is the gradient of the fused output.  dparams: fp32 [3, H*N], overwritten (the reference
 * accumulates into a zero-filled buffer with atomics; here per-batch partials go to `workspace`
 * and are summed in a fixed order, so the result is deterministic).  Other arguments as wkv7_bwd.
 */
int wkv7_attn_ln_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                     const void* g, const float* params, const void* dy, const float* ckpt, const float* dsT,
                     const float* sT, void* dr, void* dw, void* dk, void* dv, void* da, void* db, void* dg,
                     float* dparams, float* workspace, float* ds0, float eps,
                     int64_t B, int64_t T, int64_t H, int64_t N,
                     int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream);

/*
 * ddlerp: data-dependent token-shift interpolation.  Replaces fw1_triton_ / fw2_triton_
 * (wind_rwkv/rwkv7/rwkv7_ddlerp.py:19-84) behind DDLerp.forward (:307-322).  All tensors bf16,
 * contiguous: x [B,T,C], alpha [C], L [4D,C], R [4,C,D], beta [4,C] (the reference casts its fp32
 * parameters to bf16 first, :309).  Outputs: m [B,T,4D] (tanh activations, input of the backward)
 * and y [4,B,T,C].  Requires C % 64 == 0 and D in {16,32,64}; any T (the reference needs T % 64 == 0
 * for T >= 64, :44-45).
 *   xx = x_{t-1} - x_t ;  m = tanh((x + xx*alpha) @ L^T) ;  y_k = x + xx*(m_k @ R_k^T + beta_k)
 */
int wkv7_ddlerp_fwd(const void* x, const void* alpha, const void* L, const void* R, const void* beta,
                    void* m, void* y, int64_t B, int64_t T, int64_t C, int64_t D, void* stream);

/*
 * ddlerp forward on the tcgen05 tensor cores with bulk tensor (TMA) loads and stores: same arguments, results and
 * limits as wkv7_ddlerp_fwd, plus `workspace`: wkv7_ddlerp_fwd_tc_workspace_bytes(C, D) bytes of device scratch,
 * 16-byte aligned, overwritten (the shifted-weight form of L and the rearranged R).  The time shift is folded into
 * the weights, m = tanh([x_t | x_{t-1}] [L(1-alpha) | L alpha]^T), so m differs from wkv7_ddlerp_fwd's in the last
 * bf16 bits.  May report WKV7_ERR_DEVICE_TIMEOUT through the status word (bounded waits).
 */
size_t wkv7_ddlerp_fwd_tc_workspace_bytes(int64_t C, int64_t D);
int wkv7_ddlerp_fwd_tc(const void* x, const void* alpha, const void* L, const void* R, const void* beta,
                       void* m, void* y, void* workspace, int64_t B, int64_t T, int64_t C, int64_t D, void* stream);

/*
 * ddlerp backward.  Replaces bw1..bw4_triton_ (rwkv7_ddlerp.py:92-303) behind DDLerp.backward
 * (:323-334).  dy0..dy3: bf16 [B,T,C].  dpre_workspace: bf16 [B,T,4D] scratch.  dx: bf16 [B,T,C].
 * Parameter gradients are fp32 and overwritten: dalpha [C], dL [4D,C], dR [4,C,D], dbeta [4,C].
 */
int wkv7_ddlerp_bwd(const void* x, const void* alpha, const void* L, const void* R, const void* beta, const void* m,
                    const void* dy0, const void* dy1, const void* dy2, const void* dy3,
                    void* dpre_workspace, void* dx, float* dalpha, float* dL, float* dR, float* dbeta,
                    int64_t B, int64_t T, int64_t C, int64_t D, void* stream);

/*
 * ddlerp backward on the tcgen05 tensor cores with bulk tensor (TMA) loads and stores: same arguments, results and limits
 * as wkv7_ddlerp_bwd, plus `workspace`: wkv7_ddlerp_bwd_tc_workspace_bytes(C, D) bytes of device scratch, 16-byte aligned,
 * overwritten.  dL is formed as dW12 = dpre^T [x_t | x_{t-1}] and combined with alpha (dalpha is a by-product); at ranks 16
 * and 32 dpre (dz = dy * xx formed in place in the loaded tiles, K = C products with R^T) and the main step (dx, dR, dbeta:
 * token-contracted sums resident in tensor memory) run on the tensor cores as well, at rank 64 the mma.sync kernels of
 * wkv7_ddlerp_bwd.  The two entry points sum differently rounded terms (there u and fp32 dz, here x, the shifted weights and
 * bf16 dz): their outputs agree to bf16 rounding.  May report WKV7_ERR_DEVICE_TIMEOUT through the status word (bounded waits).
 */
size_t wkv7_ddlerp_bwd_tc_workspace_bytes(int64_t C, int64_t D);
int wkv7_ddlerp_bwd_tc(const void* x, const void* alpha, const void* L, const void* R, const void* beta, const void* m,
                       const void* dy0, const void* dy1, const void* dy2, const void* dy3, void* dpre_workspace, void* dx,
                       float* dalpha, float* dL, float* dR, float* dbeta, void* workspace,
                       int64_t B, int64_t T, int64_t C, int64_t D, void* stream);

/*
 * Projection of the time mixer, forward: C = act(A W^T) with A [M,K], W [N,K] (an nn.Linear weight), C [M,N], all bf16,
 * contiguous; act = tanh on the columns tanh_from <= n < tanh_to (a LoRA's first stage feeds its second through tanh),
 * identity elsewhere (tanh_from == tanh_to: a plain projection).  Replaces the torch matmuls `x @ W.bfloat16().mT` and the
 * separate tanh passes of the reference's mixer (wind_rwkv/rwkv7/time_mixer.py:120-131, 167).  tcgen05 products (bf16
 * operands, fp32 accumulation in tensor memory), operands by bulk tensor loads.  N and K multiples of 8; any M.
 */
int wkv7_proj_gemm(const void* A, const void* W, void* C, int64_t M, int64_t N, int64_t K,
                   int64_t tanh_from, int64_t tanh_to, void* stream);

/*
 * expand_loras: second-stage LoRA expansion producing (w, k, kk, b) for the mixer.  Replaces
 * fw_triton_ (wind_rwkv/rwkv7/rwkv7_expand_loras.py:32-89) behind ExpandLoras.forward (:215-231).
 * All tensors bf16, contiguous: w_in,k_in [B,T,C]; z_in,a_in,ma_in,mk_in [B,T,D]; W* [C,D];
 * biases [C]; outputs [B,T,C].  Head size 64 (C % 64 == 0), T % 16 == 0, D in {16,32,64,128}.
 *   w = -softplus(-(w_bias+w_in)) - 0.5 ;  z = tanh(z_in)@Wz^T + k_in ;  kk = z/||z||_head
 *   a, ma, mk = sigmoid(x_in@W^T + bias) ;  k = k_in*(ma+a-ma*a)*exp(w*mk) ;  b = -kk*a
 */
int wkv7_expand_loras_fwd(const void* w_in, const void* k_in, const void* z_in, const void* a_in, const void* ma_in,
                          const void* mk_in, const void* Wz, const void* Wa, const void* Wma, const void* Wmk,
                          const void* w_bias, const void* a_bias, const void* ma_bias, const void* mk_bias,
                          void* w_out, void* k_out, void* kk_out, void* b_out,
                          int64_t B, int64_t T, int64_t C, int64_t D, void* stream);

/* Bytes of workspace wkv7_expand_loras_bwd needs: 4*B*T*(C/64)*D*2 (per-head partials of the
 * rank-D input gradients, bf16, as the reference keeps them, rwkv7_expand_loras.py:201,207-210). */
int64_t wkv7_expand_loras_bwd_workspace_bytes(int64_t B, int64_t T, int64_t C, int64_t D);

/*
 * expand_loras backward.  Replaces bw_triton_ (rwkv7_expand_loras.py:91-211) behind
 * ExpandLoras.backward (:232-239).  Input gradients bf16 (dw_in,dk_in [B,T,C]; dz_in..dmk_in
 * [B,T,D]); weight and bias gradients fp32, overwritten.
 */
int wkv7_expand_loras_bwd(const void* w_in, const void* k_in, const void* z_in, const void* a_in, const void* ma_in,
                          const void* mk_in, const void* Wz, const void* Wa, const void* Wma, const void* Wmk,
                          const void* w_bias, const void* a_bias, const void* ma_bias, const void* mk_bias,
                          const void* dw_out, const void* dk_out, const void* dkk_out, const void* db_out,
                          void* dw_in, void* dk_in, void* dz_in, void* da_in, void* dma_in, void* dmk_in,
                          float* dWz, float* dWa, float* dWma, float* dWmk,
                          float* dw_bias, float* da_bias, float* dma_bias, float* dmk_bias,
                          void* workspace, int64_t B, int64_t T, int64_t C, int64_t D, void* stream);

/*
 * wkv7_attn_ln_bwd for callers that cannot hand over a workspace.  No counterpart in the
 * reference, where PyTorch allocates everything.
 *
 * Who needs it: code that drives the library without an allocator of its own and may not call
 * cudaMalloc at this point -- a runtime that has already handed all device memory to its own
 * pool, a plugin loaded into a host application that owns the memory, or a thread for which
 * cudaMalloc's implicit device-wide synchronisation is not acceptable in the middle of a step.
 * wkv7_attn_ln_bwd needs B*3*H*N floats of scratch for the per-batch partial parameter
 * gradients; this variant keeps that scratch in an array of WKV7_STATIC_SCRATCH_BYTES (4 MiB)
 * that is part of the library's device image.  Every GPU that loads the library holds those
 * 4 MiB until the process exits, whether or not this entry point is ever called.
 *
 * Arguments and results are exactly those of wkv7_attn_ln_bwd without `workspace`; inputs and
 * outputs are still the caller's.  The call itself allocates nothing: no cudaMalloc, cudaFree
 * or allocating library routine.
 *  - Limit: B*3*H*N*4 <= WKV7_STATIC_SCRATCH_BYTES, else WKV7_ERR_STATIC_SCRATCH and nothing runs.
 *  - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *    that device current) and caches it; make that first call before starting a stream capture.
 *  - All calls on a device share the one array.  Each call overwrites the part it uses before
 *    reading it, so nothing has to be cleared between calls, but two calls that can overlap on
 *    the GPU (different streams, no dependency) race on it: serialise them.
 */
int wkv7_attn_ln_bwd_static(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                            const void* g, const float* params, const void* dy, const float* ckpt, const float* dsT,
                            const float* sT, void* dr, void* dw, void* dk, void* dv, void* da, void* db, void* dg,
                            float* dparams, float* ds0, float eps,
                            int64_t B, int64_t T, int64_t H, int64_t N,
                            int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* WKV7_SM100_H */
