// extern "C" entry points of libwkv7_sm100.so (declared in include/wkv7_sm100.h): host-side
// validation, the per-device status word, and dispatch to the kernel launchers.
#include "../../include/wkv7_sm100.h"
#include "wkv7_kernels.h"

#include <mutex>

// Scratch for wkv7_attn_ln_bwd_static: lives in the library's device image, one copy on every GPU
// that loads the library, until the process exits.  Only its ADDRESS ON THE DEVICE may be given
// to a kernel; in host code the name is a host-side stand-in, so the address is fetched once
// per device with cudaGetSymbolAddress (see static_scratch()).
static __device__ __align__(256) float g_attn_ln_static_scratch[WKV7_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace {

__device__ int g_status_word = 0;

int* status_ptr() {
    int* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_status_word) != cudaSuccess) return nullptr;
    return p;
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

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int check_common(int64_t B, int64_t T, int64_t H, int64_t N, int64_t sb, int64_t st, int64_t sh, int io_dtype) {
    if (B < 0 || T < 0 || H < 0 || N <= 0) return wkv7::kBadShape;
    if (N != wkv7::N) return wkv7::kBadHeadSize;
    if (T % wkv7::L != 0) return wkv7::kBadChunk;
    if (io_dtype != WKV7_BF16 && io_dtype != WKV7_F32 && io_dtype != WKV7_F32_TF32) return wkv7::kBadDtype;
    const int64_t per16 = io_dtype == WKV7_BF16 ? 8 : 4;  // elements per 16 bytes
    if (sb % per16 || st % per16 || sh % per16) return wkv7::kBadAlign;
    if (sb < 0 || st < 0 || sh < 0) return wkv7::kBadShape;
    if (B * H > 0x7fffffffLL) return wkv7::kTooLarge;
    return wkv7::kOk;
}

}  // namespace

extern "C" {

const char* wkv7_status_string(int status) {
    switch (status) {
        case WKV7_OK: return "ok";
        case WKV7_ERR_SHAPE: return "bad shape: negative or inconsistent dimensions";
        case WKV7_ERR_HEAD_SIZE: return "unsupported head size: only N == 64 is built";
        case WKV7_ERR_CHUNK: return "T must be a multiple of 16";
        case WKV7_ERR_ALIGN: return "pointer or stride breaks 16-byte row alignment";
        case WKV7_ERR_DTYPE: return "unknown io_dtype";
        case WKV7_ERR_NULL: return "a required pointer is null";
        case WKV7_ERR_LAUNCH: return "CUDA launch failed";
        case WKV7_ERR_TOO_LARGE: return "B*H exceeds the grid limit";
        case WKV7_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait ran out";
        case WKV7_ERR_STATIC_SCRATCH: return "problem needs more than WKV7_STATIC_SCRATCH_BYTES of built-in scratch (B*3*H*N*4 bytes); use wkv7_attn_ln_bwd with a caller-provided workspace";
        default: return "unknown status";
    }
}

int64_t wkv7_checkpoint_bytes(int64_t B, int64_t T, int64_t H, int64_t N) {
    if (B < 0 || T < 0 || H < 0 || N < 0) return 0;
    return B * H * (T / wkv7::L) * N * N * (int64_t)sizeof(float);
}

int wkv7_device_status(void) {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status_word, sizeof(int)) != cudaSuccess) return WKV7_ERR_LAUNCH;
    if (v != 0) cudaMemcpyToSymbol(g_status_word, &zero, sizeof(int));
    return v;
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
    return wkv7::launch_fwd(p, io_dtype, ln, (cudaStream_t)stream);
}

int wkv7_fwd(const void* r, const void* w, const void* k, const void* v, const void* a, const void* b,
             const float* s0, void* y, float* sT, float* ckpt, int64_t B, int64_t T, int64_t H, int64_t N,
             int64_t stride_b, int64_t stride_t, int64_t stride_h, int io_dtype, void* stream) {
    return fwd_common(r, w, k, v, a, b, nullptr, nullptr, false, 0.f, s0, y, sT, ckpt, B, T, H, N, stride_b, stride_t,
                      stride_h, io_dtype, stream);
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

}  // extern "C"
