"""ctypes binding of libwkv7_sm100.so (C ABI declared in include/wkv7_sm100.h).

There is no fallback: if the library cannot be loaded, or a call returns a non-zero
status, a RuntimeError is raised.
"""
import ctypes
import os

import torch as th

_PKG_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
LIB_PATH = os.path.join(_PKG_ROOT, 'lib', 'libwkv7_sm100.so')

WKV7_BF16, WKV7_F32 = 0, 1
HEAD_SIZE = 64
CHUNK = 16
# floats per checkpoint record (WKV7_CHECKPOINT_FLOATS of the header): the 64x64 chunk-start state and the
# chunk's four 16x16 matrices; the checkpoint tensor is [B, H, T/16, CKPT_FLOATS] fp32
CKPT_FLOATS = 64 * 64 + 4 * 16 * 16



def chunks(T):
    """Checkpoint records per chain: one per 16 time steps, the last chunk may be partial (upstream requires
    T % 16 == 0, rwkv7_attn.py:22; here any T is accepted)."""
    return (T + CHUNK - 1) // CHUNK


_lib = None

_vp, _i64, _int, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float

_SIGNATURES = {
    'wkv7_status_string': (ctypes.c_char_p, [_int]),
    'wkv7_checkpoint_bytes': (_i64, [_i64] * 4),
    'wkv7_device_status': (_int, []),
    'wkv7_peek_status': (_int, []),
    'wkv7_selftest_bounded_wait': (_int, [_i64, ctypes.POINTER(ctypes.c_int64), _vp]),
    'wkv7_set_fwd_impl': (_int, [_int]),
    'wkv7_get_fwd_impl': (_int, []),
    'wkv7_fwd': (_int, [_vp] * 10 + [_i64] * 7 + [_int, _vp]),
    'wkv7_step': (_int, [_vp] * 9 + [_i64] * 7 + [_int, _vp]),
    'wkv7_bwd': (_int, [_vp] * 17 + [_i64] * 7 + [_int, _vp]),
    'wkv7_attn_ln_fwd': (_int, [_vp] * 12 + [_f32] + [_i64] * 7 + [_int, _vp]),
    'wkv7_attn_ln_bwd_workspace_bytes': (_i64, [_i64] * 3),
    'wkv7_attn_ln_bwd': (_int, [_vp] * 22 + [_f32] + [_i64] * 7 + [_int, _vp]),
    'wkv7_proj_gemm': (_int, [_vp] * 3 + [_i64] * 5 + [_vp]),
    'wkv7_ddlerp_fwd': (_int, [_vp] * 7 + [_i64] * 4 + [_vp]),
    'wkv7_ddlerp_fwd_tc': (_int, [_vp] * 8 + [_i64] * 4 + [_vp]),
    'wkv7_ddlerp_fwd_tc_workspace_bytes': (ctypes.c_size_t, [_i64] * 2),
    'wkv7_ddlerp_bwd': (_int, [_vp] * 16 + [_i64] * 4 + [_vp]),
    'wkv7_ddlerp_bwd_tc': (_int, [_vp] * 17 + [_i64] * 4 + [_vp]),
    'wkv7_ddlerp_bwd_tc_workspace_bytes': (ctypes.c_size_t, [_i64] * 2),
    'wkv7_expand_loras_fwd': (_int, [_vp] * 18 + [_i64] * 4 + [_vp]),
    'wkv7_expand_loras_bwd_workspace_bytes': (_i64, [_i64] * 4),
    'wkv7_expand_loras_bwd': (_int, [_vp] * 33 + [_i64] * 4 + [_vp]),
    'wkv7_attn_ln_bwd_static': (_int, [_vp] * 21 + [_f32] + [_i64] * 7 + [_int, _vp]),
}


def exported_symbols():
    """Names the header declares; used by the symbol-presence test."""
    return list(_SIGNATURES)


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f'{LIB_PATH} is missing: build it with `python wind-rwkv7_b200/build.py` '
                '(needs nvcc; there is no CPU or PyTorch fallback for these ops)')
        L = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in _SIGNATURES.items():
            f = getattr(L, name)
            f.restype, f.argtypes = res, args
        _lib = L
    return _lib


def check(status, what):
    """Raises on a non-zero return code of a C-ABI call, and on a device-side error that an earlier, finished kernel
    left in the status word (looked at without synchronising; see wkv7_peek_status in the header)."""
    if status != 0:
        msg = lib().wkv7_status_string(status).decode()
        raise RuntimeError(f'{what} failed: {msg} (status {status})')
    dev = lib().wkv7_peek_status()
    if dev != 0:
        raise RuntimeError(f'an earlier wkv7 kernel reported: {lib().wkv7_status_string(dev).decode()} (status {dev}); '
                           'its results are invalid.  wkv7_device_status() reads and clears the error.')


def on_device(*tensors):
    """Context manager that makes the tensors' device current for a launch (kernels run on the current device, the
    stream argument alone does not select it); all tensors must live on one CUDA device."""
    devs = {t.device for t in tensors if t is not None}
    if len(devs) != 1:
        raise RuntimeError(f'wkv7 ops need all tensors on one device, got {sorted(str(d) for d in devs)}')
    dev = devs.pop()
    if dev.type != 'cuda':
        raise RuntimeError('wkv7 ops run on CUDA tensors only (sm_100a); there is no CPU path')
    return th.cuda.device(dev)


def io_dtype(t):
    if t.dtype == th.bfloat16:
        return WKV7_BF16
    if t.dtype == th.float32:
        return WKV7_F32
    raise TypeError(f'wkv7 ops take bfloat16 or float32 tensors, got {t.dtype}')


def ptr(t):
    return None if t is None else t.data_ptr()


def stream_of(t):
    return th.cuda.current_stream(t.device).cuda_stream


def require_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError('wkv7 ops run on CUDA tensors only (sm_100a); there is no CPU path')


def strides4(x):
    """Element strides (b, t, h) of a [B,T,H,N] view with unit inner stride."""
    assert x.dim() == 4 and x.stride(3) == 1, 'inner dimension must be contiguous'
    return x.stride(0), x.stride(1), x.stride(2)


def device_status():
    """Reads and clears the device status word (synchronises)."""
    return lib().wkv7_device_status()


def set_fwd_impl(impl):
    """Selects the bf16 attn forward kernel: 0 = warp-MMA, 2..4 = tcgen05 with that many preparation
    groups (negative: operands truncated, not rounded, to TF32).  Returns the previous value."""
    old = lib().wkv7_get_fwd_impl()
    check(lib().wkv7_set_fwd_impl(int(impl)), 'wkv7_set_fwd_impl')
    return old


def opaque_op(name, fn, fake, schema_types):
    """Registers `fn` (a launcher that allocates its outputs and calls the C ABI) as the functional
    custom op wkv7_sm100::<name> with `fake` as its shape function, so that torch.compile can keep
    it in a full graph (upstream gets the same effect from its mutable-alias TORCH_LIBRARY schemas,
    attn.cpp:24-27).  Eager calls do not go through the dispatcher; see `call`."""
    op = th.library.custom_op(f'wkv7_sm100::{name}', fn, mutates_args=(), schema=schema_types)
    op.register_fake(fake)
    return op


def call(op, fn, *args):
    """`fn(*args)` directly in eager mode, the registered custom op while torch.compile traces."""
    return op(*args) if th.compiler.is_compiling() else fn(*args)
