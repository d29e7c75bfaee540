// extern "C" entry points of libwkv7_sm100.so (declared in include/wkv7_sm100.h): host-side
// validation, the per-device status word, and dispatch to the kernel launchers.
#include <atomic>
#include <cstdlib>
#include "../../include/wkv7_sm100.h"
#include "wkv7_kernels.h"
#include "ddlerp.h"
#include "expand_loras.h"

#include <mutex>

// Scratch for wkv7_attn_ln_bwd_static: lives in the library's device image, one copy on every GPU
// that loads the library, until the process exits.  Only its ADDRESS ON THE DEVICE may be given
// to a kernel; in host code the name is a host-side stand-in, so the address is fetched once
// per device with cudaGetSymbolAddress (see static_scratch()).
static __device__ __align__(256) float g_attn_ln_static_scratch[WKV7_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {

// The status word that a kernel's bounded wait writes when it gives up: a managed variable, part of the library's
// image (nothing is allocated at run time), one per process, readable by the host while kernels run (concurrent
// managed access), so that wkv7_peek_status() is a plain load that synchronises nothing.  The page stays on the host
// side unless a kernel reports an error.
__managed__ int g_status_word = 0;

int* status_ptr() {
    static int* word = [] {
        int* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_status_word) != cudaSuccess) p = nullptr;
        return p;
    }();
    return word;
}

// Device address of g_attn_ln_static_scratch on the current device, looked up on the first call
// for that device and cached.  Returns nullptr if the lookup fails.
float* static_scratch() {
    constexpr int kMaxDevices = 64;
    static float* cache[kMaxDevices] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev]) {
        float* ptr = nullptr;
        if (cudaGetSymbolAddress((void**)&ptr, g_attn_ln_static_scratch) != cudaSuccess) return nullptr;
        cache[dev] = ptr;
    }
    return cache[dev];
}

// Forward implementation for bf16 attn (see wkv7_set_fwd_impl in the header): 0 = warp-MMA kernel,
// +-2..4 = tcgen05 kernel with that many preparation groups.
bool valid_fwd_impl(int x) { return x == 0 || (x >= 2 && x <= 4) || (x <= -2 && x >= -4); }
std::atomic<int>& fwd_impl() {
    static std::atomic<int> v([] {
        const char* e = std::getenv("WKV7_FWD_TC");
        if (!e) return 4;
        const int x = std::atoi(e);
        return valid_fwd_impl(x) ? x : 0;
    }());
    return v;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_common(int64_t B, int64_t T, int64_t H, int64_t N, int64_t sb, int64_t st, int64_t sh, int io_dtype) {
    if (B < 0 || T < 0 || H < 0 || N <= 0) return wkv7::kBadShape;
    if (N != wkv7::N) return wkv7::kBadHeadSize;
    if (io_dtype != WKV7_BF16 && io_dtype != WKV7_F32 && io_dtype != WKV7_F32_TF32) return wkv7::kBadDtype;
    const int64_t per16 = io_dtype == WKV7_BF16 ? 8 : 4;  // elements per 16 bytes
    if (sb % per16 || st % per16 || sh % per16) return wkv7::kBadAlign;
    if (sb < 0 || st < 0 || sh < 0) return wkv7::kBadShape;
    if (B * H > 0x7fffffffLL) return wkv7::kTooLarge;
    // the kernels address checkpoint records through 32-bit row coordinates of their tensor maps (80 rows of 64 floats
    // per record)
    if (B * H > 0 && (T + wkv7::L - 1) / wkv7::L > (0x7fffffffLL / (wkv7::CK_FLOATS / wkv7::N)) / (B * H)) return wkv7::kTooLarge;
    return wkv7::kOk;
}

}  // namespace

extern "C" {

const char* wkv7_status_string(int status) {
    switch (status) {
        case WKV7_OK: return "ok";
        case WKV7_ERR_SHAPE: return "bad shape: negative or inconsistent dimensions";
        case WKV7_ERR_HEAD_SIZE: return "unsupported head size: only N == 64 is built";
        case WKV7_ERR_CHUNK: return "expand_loras: T must be a multiple of 16; ddlerp, expand_loras: C must be a multiple of 64";
        case WKV7_ERR_ALIGN: return "pointer or stride breaks 16-byte row alignment";
        case WKV7_ERR_DTYPE: return "unknown io_dtype";
        case WKV7_ERR_NULL: return "a required pointer is null";
        case WKV7_ERR_LAUNCH: return "CUDA launch failed";
        case WKV7_ERR_TOO_LARGE: return "B*H exceeds the grid limit, or B*H*ceil(T/16) checkpoint records exceed 32-bit row addressing";
        case WKV7_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case WKV7_ERR_STATIC_SCRATCH: return "problem needs more than WKV7_STATIC_SCRATCH_BYTES of built-in scratch (B*3*H*N*4 bytes); use wkv7_attn_ln_bwd with a caller-provided workspace";
        default: return "unknown status";
    }
}

int64_t wkv7_checkpoint_bytes(int64_t B, int64_t T, int64_t H, int64_t N) {
    if (B < 0 || T < 0 || H < 0 || N < 0) return 0;
    if (N != wkv7::N) return 0;
    return B * H * ((T + wkv7::L - 1) / wkv7::L) * (int64_t)wkv7::CK_FLOATS * (int64_t)sizeof(float);
}

__device__ long long g_selftest_cycles[4];

int wkv7_selftest_bounded_wait(int64_t limit_cycles, int64_t* cycles_out, void* stream) {
    if (limit_cycles <= 0 || limit_cycles > (1LL << 28)) return WKV7_ERR_SHAPE;
    int* status = status_ptr();
    long long* cyc = nullptr;
    if (!status || cudaGetSymbolAddress((void**)&cyc, g_selftest_cycles) != cudaSuccess) return WKV7_ERR_LAUNCH;
    int rc = wkv7::launch_bounded_wait_selftest(limit_cycles, status, cyc, (cudaStream_t)stream);
    if (rc) return rc;
    if (cudaStreamSynchronize((cudaStream_t)stream) != cudaSuccess) return WKV7_ERR_LAUNCH;
    if (cycles_out) {
        long long h[4];
        if (cudaMemcpy(h, cyc, sizeof(h), cudaMemcpyDeviceToHost) != cudaSuccess) return WKV7_ERR_LAUNCH;
        for (int i = 0; i < 4; ++i) cycles_out[i] = h[i];
    }
    return wkv7_device_status();
}

int wkv7_set_fwd_impl(int impl) {
    if (!valid_fwd_impl(impl)) return WKV7_ERR_SHAPE;
    fwd_impl().store(impl, std::memory_order_relaxed);
    return WKV7_OK;
}

int wkv7_get_fwd_impl(void) { return fwd_impl().load(std::memory_order_relaxed); }

int wkv7_device_status(void) {
    int* w = status_ptr();
    if (!w) return WKV7_ERR_LAUNCH;
    if (cudaDeviceSynchronize() != cudaSuccess) return WKV7_ERR_LAUNCH;  // every stream of the current device, non-blocking ones too
    return __atomic_exchange_n(w, 0, __ATOMIC_ACQ_REL);                  // read and clear in one step
}

int wkv7_peek_status(void) {
    int* w = status_ptr();
    return w ? __atomic_load_n(w, __ATOMIC_ACQUIRE) : WKV7_ERR_LAUNCH;
}

static int fwd_common(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                      const void* g, const float* params, bool ln, float eps, const float* s0, void* y, float* sT,
                      float* ckpt, int64_t B, int64_t T, int64_t H, int64_t N, int64_t sb, int64_t st, int64_t sh,
                      int io_dtype, void* stream) {
    int rc = check_common(B, T, H, N, sb, st, sh, io_dtype);
    if (rc) return rc;
    if (B == 0 || H == 0) return WKV7_OK;
    if (T == 0) {  // nothing to scan: the state passes through
        if (sT) {
            size_t bytes = (size_t)B * H * N * N * sizeof(float);
            cudaError_t e = s0 ? cudaMemcpyAsync(sT, s0, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)
                               : cudaMemsetAsync(sT, 0, bytes, (cudaStream_t)stream);
            if (e != cudaSuccess) return WKV7_ERR_LAUNCH;
        }
        return WKV7_OK;
    }
    if (!r || !w || !k || !v || !a || !b || !y || (ln && (!g || !params))) return WKV7_ERR_NULL;
    const void* ptrs[] = {r, w, k, v, a, b, y, g, s0, sT, ckpt, params};
    for (const void* p : ptrs)
        if (p && !aligned16(p)) return WKV7_ERR_ALIGN;
    wkv7::FwdParams p{};
    p.r = r; p.w = w; p.k = k; p.v = v; p.a = a; p.b = b; p.g = g; p.params = params;
    p.s0 = s0; p.y = y; p.sT = sT; p.ckpt = ckpt;
    p.B = B; p.T = T; p.H = H;
    p.st = wkv7::Strides{sb, st, sh};
    p.eps = eps;
    p.status = status_ptr();
    if (!p.status) return WKV7_ERR_LAUNCH;
    if (io_dtype == WKV7_BF16) {
        const int groups = fwd_impl().load(std::memory_order_relaxed);
        if (groups) return wkv7::launch_fwd_tc(p, groups, ln, (cudaStream_t)stream);
    }
    return wkv7::launch_fwd(p, io_dtype, ln, (cudaStream_t)stream);
}

int wkv7_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
             const float* s0, void* y, float* sT, float* ckpt, int64_t B, int64_t T, int64_t H, int64_t N,
             int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream) {
    return fwd_common(r, w, k, v, a, b, nullptr, nullptr, false, 0.f, s0, y, sT, ckpt, B, T, H, N, stride_b, stride_t,
                      stride_h, io_dtype, stream);
}

int wkv7_step(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b, const float* s0,
              void* y, float* sT, int64_t B, int64_t T, int64_t H, int64_t N, int64_t stride_b, int64_t stride_t,
              int64_t stride_h, int io_dtype, void* stream) {
    int rc = check_common(B, T, H, N, stride_b, stride_t, stride_h, io_dtype);
    if (rc) return rc;
    if (B == 0 || H == 0) return WKV7_OK;
    if (T == 0) {
        if (sT && sT != s0) {
            size_t bytes = (size_t)B * H * N * N * sizeof(float);
            cudaError_t e = s0 ? cudaMemcpyAsync(sT, s0, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)
                               : cudaMemsetAsync(sT, 0, bytes, (cudaStream_t)stream);
            if (e != cudaSuccess) return WKV7_ERR_LAUNCH;
        }
        return WKV7_OK;
    }
    if (!r || !w || !k || !v || !a || !b || !y) return WKV7_ERR_NULL;
    const void* ptrs[] = {r, w, k, v, a, b, y, s0, sT};
    for (const void* q : ptrs)
        if (q && !aligned16(q)) return WKV7_ERR_ALIGN;
    wkv7::StepParams p{};
    p.r = r; p.w = w; p.k = k; p.v = v; p.a = a; p.b = b; p.s0 = s0; p.y = y; p.sT = sT;
    p.B = B; p.T = T; p.H = H;
    p.st = wkv7::Strides{stride_b, stride_t, stride_h};
    return wkv7::launch_step(p, io_dtype == WKV7_BF16 ? 0 : 1, (cudaStream_t)stream);
}

int wkv7_attn_ln_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                     const void* g, const float* params, const float* s0, void* y, float* sT, float* ckpt, float eps,
                     int64_t B, int64_t T, int64_t H, int64_t N, int64_t stride_b, int64_t stride_t, int64_t stride_h,
                     int io_dtype, void* stream) {
    return fwd_common(r, w, k, v, a, b, g, params, true, eps, s0, y, sT, ckpt, B, T, H, N, stride_b, stride_t,
                      stride_h, io_dtype, stream);
}

static int bwd_common(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                      const void* g, const float* params, bool ln, float eps, const void* dy, const float* ckpt,
                      const float* dsT, const float* sT, void* dr, void* dw, void* dk, void* dv, void* da, void* db,
                      void* dg, float* dparams, float* dparams_ws, float* ds0, int64_t B, int64_t T, int64_t H, int64_t N,
                      int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream) {
    int rc = check_common(B, T, H, N, stride_b, stride_t, stride_h, io_dtype);
    if (rc) return rc;
    if (B == 0 || H == 0) return WKV7_OK;
    if (T == 0) {
        if (ln && dparams) {
            if (cudaMemsetAsync(dparams, 0, (size_t)3 * H * N * sizeof(float), (cudaStream_t)stream) != cudaSuccess)
                return WKV7_ERR_LAUNCH;
        }
        if (ds0) {
            size_t bytes = (size_t)B * H * N * N * sizeof(float);
            cudaError_t e = dsT ? cudaMemcpyAsync(ds0, dsT, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream)
                                : cudaMemsetAsync(ds0, 0, bytes, (cudaStream_t)stream);
            if (e != cudaSuccess) return WKV7_ERR_LAUNCH;
        }
        return WKV7_OK;
    }
    if (!r || !w || !k || !v || !a || !b || !dy || !ckpt || !dr || !dw || !dk || !dv || !da || !db) return WKV7_ERR_NULL;
    if (dsT && !sT) return WKV7_ERR_NULL;
    if (ln && (!g || !params || !dg || !dparams || !dparams_ws)) return WKV7_ERR_NULL;
    const void* ptrs[] = {r, w, k, v, a, b, dy, ckpt, dsT, sT, dr, dw, dk, dv, da, db, ds0, g, params, dg, dparams, dparams_ws};
    for (const void* p : ptrs)
        if (p && !aligned16(p)) return WKV7_ERR_ALIGN;
    wkv7::BwdParams p{};
    p.r = r; p.w = w; p.k = k; p.v = v; p.a = a; p.b = b; p.dy = dy;
    p.ckpt = ckpt; p.dsT = dsT; p.sT = sT;
    p.g = g; p.params = params; p.dg = dg; p.dparams = dparams; p.dparams_ws = dparams_ws; p.eps = eps;
    p.dr = dr; p.dw = dw; p.dk = dk; p.dv = dv; p.da = da; p.db = db; p.ds0 = ds0;
    p.B = B; p.T = T; p.H = H;
    p.st = wkv7::Strides{stride_b, stride_t, stride_h};
    p.status = status_ptr();
    if (!p.status) return WKV7_ERR_LAUNCH;
    return wkv7::launch_bwd(p, io_dtype, ln, (cudaStream_t)stream);
}

int wkv7_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
             const void* dy, const float* ckpt, const float* dsT, const float* sT, void* dr, void* dw, void* dk,
             void* dv, void* da, void* db, float* ds0, int64_t B, int64_t T, int64_t H, int64_t N, int64_t stride_b,
             int64_t stride_t, int64_t stride_h, int io_dtype, void* stream) {
    return bwd_common(r, w, k, v, a, b, nullptr, nullptr, false, 0.f, dy, ckpt, dsT, sT, dr, dw, dk, dv, da, db, nullptr,
                      nullptr, nullptr, ds0, B, T, H, N, stride_b, stride_t, stride_h, io_dtype, stream);
}

int64_t wkv7_attn_ln_bwd_workspace_bytes(int64_t B, int64_t H, int64_t N) {
    if (B < 0 || H < 0 || N < 0) return 0;
    return B * 3 * H * N * (int64_t)sizeof(float);
}

int wkv7_attn_ln_bwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                     const void* g, const float* params, const void* dy, const float* ckpt, const float* dsT,
                     const float* sT, void* dr, void* dw, void* dk, void* dv, void* da, void* db, void* dg,
                     float* dparams, float* workspace, float* ds0, float eps, int64_t B, int64_t T, int64_t H,
                     int64_t N, int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream) {
    return bwd_common(r, w, k, v, a, b, g, params, true, eps, dy, ckpt, dsT, sT, dr, dw, dk, dv, da, db, dg, dparams,
                      workspace, ds0, B, T, H, N, stride_b, stride_t, stride_h, io_dtype, stream);
}

int wkv7_attn_ln_bwd_static(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
                            const void* g, const float* params, const void* dy, const float* ckpt, const float* dsT,
                            const float* sT, void* dr, void* dw, void* dk, void* dv, void* da, void* db, void* dg,
                            float* dparams, float* ds0, float eps, int64_t B, int64_t T, int64_t H, int64_t N,
                            int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream) {
    if (B < 0 || H < 0 || N < 0) return WKV7_ERR_SHAPE;
    if (wkv7_attn_ln_bwd_workspace_bytes(B, H, N) > (int64_t)WKV7_STATIC_SCRATCH_BYTES) return WKV7_ERR_STATIC_SCRATCH;
    float* scratch = static_scratch();
    if (!scratch) return WKV7_ERR_LAUNCH;
    return bwd_common(r, w, k, v, a, b, g, params, true, eps, dy, ckpt, dsT, sT, dr, dw, dk, dv, da, db, dg, dparams,
                      scratch, ds0, B, T, H, N, stride_b, stride_t, stride_h, io_dtype, stream);
}

int wkv7_proj_gemm(const void* A, const void* W, void* C, int64_t M, int64_t N, int64_t K, int64_t tanh_from,
                   int64_t tanh_to, void* stream) {
    if (M < 0 || N <= 0 || K <= 0 || tanh_from < 0 || tanh_to < tanh_from || tanh_to > N) return WKV7_ERR_SHAPE;
    if (N % 8 != 0 || K % 8 != 0) return WKV7_ERR_ALIGN;   // 16-byte rows for the bulk tensor loads and the stores
    if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL || (M + 127) / 128 > 65535) return WKV7_ERR_TOO_LARGE;
    if (M == 0) return WKV7_OK;
    if (!A || !W || !C) return WKV7_ERR_NULL;
    if (!aligned16(A) || !aligned16(W) || !aligned16(C)) return WKV7_ERR_ALIGN;
    int* status = status_ptr();
    if (!status) return WKV7_ERR_LAUNCH;
    return wkv7::launch_proj_gemm(A, W, C, M, N, K, (int)tanh_from, (int)tanh_to, status, (cudaStream_t)stream);
}

static int ddlerp_check(int64_t B, int64_t T, int64_t C, int64_t D) {
    if (B < 0 || T < 0 || C <= 0 || D <= 0) return WKV7_ERR_SHAPE;
    if (C % 64 != 0) return WKV7_ERR_CHUNK;
    if (D != 16 && D != 32 && D != 64) return WKV7_ERR_SHAPE;  // rank 128: the backward's resident L and R blocks exceed shared memory
    return WKV7_OK;
}

int wkv7_ddlerp_fwd(const void* x, const void* alpha, const void* L, const void* R, const void* beta, void* m, void* y,
                    int64_t B, int64_t T, int64_t C, int64_t D, void* stream) {
    int rc = ddlerp_check(B, T, C, D);
    if (rc) return rc;
    if (B == 0 || T == 0) return WKV7_OK;
    const void* ptrs[] = {x, alpha, L, R, beta, m, y};
    for (const void* q : ptrs) {
        if (!q) return WKV7_ERR_NULL;
        if (!aligned16(q)) return WKV7_ERR_ALIGN;
    }
    wkv7::DdlerpFwdParams p{x, alpha, L, R, beta, m, y, B * T, T, C, (int)D};
    return wkv7::launch_ddlerp_fwd(p, (cudaStream_t)stream);
}

size_t wkv7_ddlerp_fwd_tc_workspace_bytes(int64_t C, int64_t D) {
    if (C <= 0 || D <= 0) return 0;
    return wkv7::ddlerp_fwd_tc_workspace_bytes(C, (int)D);
}

int wkv7_ddlerp_fwd_tc(const void* x, const void* alpha, const void* L, const void* R, const void* beta, void* m, void* y,
                       void* workspace, int64_t B, int64_t T, int64_t C, int64_t D, void* stream) {
    int rc = ddlerp_check(B, T, C, D);
    if (rc) return rc;
    if (B == 0 || T == 0) return WKV7_OK;
    const void* ptrs[] = {x, alpha, L, R, beta, m, y, workspace};
    for (const void* q : ptrs) {
        if (!q) return WKV7_ERR_NULL;
        if (!aligned16(q)) return WKV7_ERR_ALIGN;
    }
    int* status = status_ptr();
    if (!status) return WKV7_ERR_LAUNCH;
    wkv7::DdlerpFwdParams p{x, alpha, L, R, beta, m, y, B * T, T, C, (int)D};
    return wkv7::launch_ddlerp_fwd_tc(p, workspace, status, (cudaStream_t)stream);
}

static int ddlerp_bwd_any(const void* x, const void* alpha, const void* L, const void* R, const void* beta, const void* m,
                          const void* dy0, const void* dy1, const void* dy2, const void* dy3, void* dpre_workspace, void* dx,
                          float* dalpha, float* dL, float* dR, float* dbeta, void* workspace, bool tc, int64_t B, int64_t T, int64_t C,
                          int64_t D, void* stream) {
    int rc = ddlerp_check(B, T, C, D);
    if (rc) return rc;
    if (tc && (!workspace || !aligned16(workspace))) return workspace ? WKV7_ERR_ALIGN : WKV7_ERR_NULL;
    const void* ptrs[] = {x, alpha, L, R, beta, m, dy0, dy1, dy2, dy3, dpre_workspace, dx, dalpha, dL, dR, dbeta};
    for (const void* q : ptrs) {
        if (!q) return WKV7_ERR_NULL;
        if (!aligned16(q)) return WKV7_ERR_ALIGN;
    }
    wkv7::DdlerpBwdParams p{};
    p.x = x; p.alpha = alpha; p.L = L; p.R = R; p.beta = beta; p.m = m;
    p.dy[0] = dy0; p.dy[1] = dy1; p.dy[2] = dy2; p.dy[3] = dy3;
    p.dpre = dpre_workspace; p.dx = dx; p.dalpha = dalpha; p.dL = dL; p.dR = dR; p.dbeta = dbeta;
    p.rows = B * T; p.T = T; p.C = C; p.D = (int)D;
    if (B == 0 || T == 0) {  // parameter gradients of an empty batch are zero
        cudaStream_t s = (cudaStream_t)stream;
        if (cudaMemsetAsync(dalpha, 0, sizeof(float) * C, s) != cudaSuccess || cudaMemsetAsync(dbeta, 0, sizeof(float) * 4 * C, s) != cudaSuccess ||
            cudaMemsetAsync(dR, 0, sizeof(float) * 4 * C * D, s) != cudaSuccess || cudaMemsetAsync(dL, 0, sizeof(float) * 4 * D * C, s) != cudaSuccess)
            return WKV7_ERR_LAUNCH;
        return WKV7_OK;
    }
    if (!tc) return wkv7::launch_ddlerp_bwd(p, (cudaStream_t)stream);
    int* status = status_ptr();
    if (!status) return WKV7_ERR_LAUNCH;
    return wkv7::launch_ddlerp_bwd_tc(p, workspace, status, (cudaStream_t)stream);
}

int wkv7_ddlerp_bwd(const void* x, const void* alpha, const void* L, const void* R, const void* beta, const void* m,
                    const void* dy0, const void* dy1, const void* dy2, const void* dy3, void* dpre_workspace, void* dx,
                    float* dalpha, float* dL, float* dR, float* dbeta, int64_t B, int64_t T, int64_t C, int64_t D,
                    void* stream) {
    return ddlerp_bwd_any(x, alpha, L, R, beta, m, dy0, dy1, dy2, dy3, dpre_workspace, dx, dalpha, dL, dR, dbeta, nullptr, false, B, T, C, D, stream);
}

size_t wkv7_ddlerp_bwd_tc_workspace_bytes(int64_t C, int64_t D) {
    if (C <= 0 || D <= 0) return 0;
    return wkv7::ddlerp_bwd_tc_workspace_bytes(C, (int)D);
}

int wkv7_ddlerp_bwd_tc(const void* x, const void* alpha, const void* L, const void* R, const void* beta, const void* m,
                       const void* dy0, const void* dy1, const void* dy2, const void* dy3, void* dpre_workspace, void* dx,
                       float* dalpha, float* dL, float* dR, float* dbeta, void* workspace, int64_t B, int64_t T, int64_t C, int64_t D,
                       void* stream) {
    return ddlerp_bwd_any(x, alpha, L, R, beta, m, dy0, dy1, dy2, dy3, dpre_workspace, dx, dalpha, dL, dR, dbeta, workspace, true, B, T, C, D, stream);
}

static int loras_check(int64_t B, int64_t T, int64_t C, int64_t D) {
    if (B < 0 || T < 0 || C <= 0 || D <= 0) return WKV7_ERR_SHAPE;
    if (T % 16 != 0 || C % 64 != 0) return WKV7_ERR_CHUNK;
    if (D != 16 && D != 32 && D != 64 && D != 128) return WKV7_ERR_SHAPE;
    return WKV7_OK;
}

int wkv7_expand_loras_fwd(const void* w_in, const void* k_in, const void* z_in, const void* a_in, const void* ma_in,
                          const void* mk_in, const void* Wz, const void* Wa, const void* Wma, const void* Wmk,
                          const void* w_bias, const void* a_bias, const void* ma_bias, const void* mk_bias, void* w_out,
                          void* k_out, void* kk_out, void* b_out, int64_t B, int64_t T, int64_t C, int64_t D, void* stream) {
    int rc = loras_check(B, T, C, D);
    if (rc) return rc;
    if (B == 0 || T == 0) return WKV7_OK;
    const void* ptrs[] = {w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias, w_out, k_out, kk_out, b_out};
    for (const void* q : ptrs) {
        if (!q) return WKV7_ERR_NULL;
        if (!aligned16(q)) return WKV7_ERR_ALIGN;
    }
    wkv7::LorasParams p{};
    p.w_in = w_in; p.k_in = k_in; p.lin[0] = z_in; p.lin[1] = a_in; p.lin[2] = ma_in; p.lin[3] = mk_in;
    p.W[0] = Wz; p.W[1] = Wa; p.W[2] = Wma; p.W[3] = Wmk;
    p.w_bias = w_bias; p.bias[0] = a_bias; p.bias[1] = ma_bias; p.bias[2] = mk_bias;
    p.w_out = w_out; p.k_out = k_out; p.kk_out = kk_out; p.b_out = b_out;
    p.rows = B * T; p.T = T; p.C = C; p.D = (int)D;
    return wkv7::launch_loras_fwd(p, (cudaStream_t)stream);
}

int64_t wkv7_expand_loras_bwd_workspace_bytes(int64_t B, int64_t T, int64_t C, int64_t D) {
    if (B < 0 || T < 0 || C < 0 || D < 0) return 0;
    return 4 * B * T * (C / 64) * D * 2;
}

int wkv7_expand_loras_bwd(const void* w_in, const void* k_in, const void* z_in, const void* a_in, const void* ma_in,
                          const void* mk_in, const void* Wz, const void* Wa, const void* Wma, const void* Wmk,
                          const void* w_bias, const void* a_bias, const void* ma_bias, const void* mk_bias,
                          const void* dw_out, const void* dk_out, const void* dkk_out, const void* db_out, void* dw_in,
                          void* dk_in, void* dz_in, void* da_in, void* dma_in, void* dmk_in, float* dWz, float* dWa,
                          float* dWma, float* dWmk, float* dw_bias, float* da_bias, float* dma_bias, float* dmk_bias,
                          void* workspace, int64_t B, int64_t T, int64_t C, int64_t D, void* stream) {
    int rc = loras_check(B, T, C, D);
    if (rc) return rc;
    const void* ptrs[] = {w_in, k_in, z_in, a_in, ma_in, mk_in, Wz, Wa, Wma, Wmk, w_bias, a_bias, ma_bias, mk_bias,
                          dw_out, dk_out, dkk_out, db_out, dw_in, dk_in, dz_in, da_in, dma_in, dmk_in,
                          dWz, dWa, dWma, dWmk, dw_bias, da_bias, dma_bias, dmk_bias, workspace};
    for (const void* q : ptrs) {
        if (!q) return WKV7_ERR_NULL;
        if (!aligned16(q)) return WKV7_ERR_ALIGN;
    }
    wkv7::LorasParams p{};
    p.w_in = w_in; p.k_in = k_in; p.lin[0] = z_in; p.lin[1] = a_in; p.lin[2] = ma_in; p.lin[3] = mk_in;
    p.W[0] = Wz; p.W[1] = Wa; p.W[2] = Wma; p.W[3] = Wmk;
    p.w_bias = w_bias; p.bias[0] = a_bias; p.bias[1] = ma_bias; p.bias[2] = mk_bias;
    p.dw_out = dw_out; p.dk_out = dk_out; p.dkk_out = dkk_out; p.db_out = db_out;
    p.dw_in = dw_in; p.dk_in = dk_in; p.dlin[0] = dz_in; p.dlin[1] = da_in; p.dlin[2] = dma_in; p.dlin[3] = dmk_in;
    p.dW[0] = dWz; p.dW[1] = dWa; p.dW[2] = dWma; p.dW[3] = dWmk;
    p.dw_bias = dw_bias; p.dbias[0] = da_bias; p.dbias[1] = dma_bias; p.dbias[2] = dmk_bias;
    p.partial = workspace;
    p.rows = B * T; p.T = T; p.C = C; p.D = (int)D;
    if (B == 0 || T == 0) {
        cudaStream_t s = (cudaStream_t)stream;
        float* w4[] = {dWz, dWa, dWma, dWmk};
        float* b4[] = {dw_bias, da_bias, dma_bias, dmk_bias};
        for (int i = 0; i < 4; ++i)
            if (cudaMemsetAsync(w4[i], 0, sizeof(float) * C * D, s) != cudaSuccess || cudaMemsetAsync(b4[i], 0, sizeof(float) * C, s) != cudaSuccess)
                return WKV7_ERR_LAUNCH;
        return WKV7_OK;
    }
    return wkv7::launch_loras_bwd(p, (cudaStream_t)stream);
}

}  // extern "C"
