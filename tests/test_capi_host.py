"""Host-side checks of the C ABI that need no GPU: the shared library loads, exports every
symbol include/wkv7_sm100.h declares, and rejects bad arguments before touching CUDA."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope='module')
def lib():
    import __graft_entry__ as ge
    ge.build()
    from wind_rwkv.rwkv7 import _lib
    return _lib.lib()


def declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'wkv7_sm100.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(wkv7_[a-z0-9_]+)\s*\(', text)))


def test_header_symbols_are_exported_and_bound(lib):
    from wind_rwkv.rwkv7 import _lib
    names = declared_symbols()
    assert 'wkv7_fwd' in names and 'wkv7_bwd' in names
    for n in names:
        assert hasattr(lib, n), f'{n} declared in the header but not exported'
    assert sorted(_lib.exported_symbols()) == names, 'ctypes signatures out of sync with the header'


def test_status_strings(lib):
    assert lib.wkv7_status_string(0) == b'ok'
    for code in range(-9, 0):
        assert lib.wkv7_status_string(code) not in (b'', b'unknown status')
    assert lib.wkv7_status_string(-99) == b'unknown status'


def test_checkpoint_bytes(lib):
    assert lib.wkv7_checkpoint_bytes(64, 1024, 12, 64) == 64 * 12 * 64 * (64 * 64 + 4 * 16 * 16) * 4
    assert lib.wkv7_checkpoint_bytes(1, 64, 1, 32) == 0  # only N == 64 is built
    assert lib.wkv7_checkpoint_bytes(1, 0, 1, 64) == 0
    assert lib.wkv7_checkpoint_bytes(1, 17, 1, 64) == 2 * (64 * 64 + 4 * 16 * 16) * 4  # a partial last chunk has a record


def _fwd(lib, T=16, N=64, st=(1024, 64, 64), dtype=0, p=0x1000):
    return lib.wkv7_fwd(p, p, p, p, p, p, None, p, None, None, 1, T, 1, N, st[0], st[1], st[2], dtype, None)


def test_validation_happens_before_any_launch(lib):
    # none of these reach CUDA: the status comes from host-side checks alone
    assert _fwd(lib, T=1 << 40) == -8              # more checkpoint records than 32-bit row coordinates reach
    assert _fwd(lib, N=32) == -2                   # head size
    assert _fwd(lib, dtype=7) == -5                # dtype
    assert _fwd(lib, st=(1024, 60, 64)) == -4      # stride breaks 16-byte rows
    assert _fwd(lib, p=0x1004) == -4               # misaligned pointer
    assert _fwd(lib, T=-16) == -1
    assert lib.wkv7_fwd(None, None, None, None, None, None, None, None, None, None,
                        1, 16, 1, 64, 1024, 64, 64, 0, None) == -6
    # empty problems succeed without a launch
    assert lib.wkv7_fwd(None, None, None, None, None, None, None, None, None, None,
                        0, 16, 4, 64, 1024, 64, 64, 0, None) == 0
    # backward: dsT without sT
    p = 0x1000
    assert lib.wkv7_bwd(p, p, p, p, p, p, p, p, p, None, p, p, p, p, p, p, None,
                        1, 16, 1, 64, 1024, 64, 64, 0, None) == -6


def test_python_ops_refuse_cpu_tensors(lib):
    import torch as th
    from wind_rwkv.rwkv7 import attn
    x = th.zeros(1, 16, 64, dtype=th.bfloat16)
    with pytest.raises(RuntimeError, match='CUDA'):
        attn(x, x, x, x, x, x, 64)


def test_launchers_need_all_tensors_on_one_cuda_device(lib):
    """The wrappers make the tensors' device current for the launch and refuse mixed devices (a kernel launched on
    the current device with another device's pointers would fail or touch the wrong memory)."""
    import torch as th
    from wind_rwkv.rwkv7 import _lib
    with pytest.raises(RuntimeError, match='one device'):
        _lib.on_device(th.zeros(1), th.zeros(1, device='meta'))
    with pytest.raises(RuntimeError, match='CUDA'):
        _lib.on_device(th.zeros(1), None)


def test_status_word_is_readable_without_a_device(lib):
    """wkv7_peek_status is a host load of a managed variable; without a GPU it reports a launch error rather than
    crashing."""
    assert lib.wkv7_peek_status() in (0, -7)
