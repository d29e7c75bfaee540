"""B200 (sm_100a) drop-in for `wind_rwkv.rwkv7` of johanwind/wind-rwkv7 (upstream: rwkv7/__init__.py:1-7)."""
from .rwkv7_ddlerp import ddlerp
from .rwkv7_expand_loras import expand_loras
from .rwkv7_attn import attn, attn_step, load_attn
from .rwkv7_attn_ln import attn_ln, load_attn_ln
from .rwkv7_proj import proj

from .time_mixer import TimeMixer


def _excluded(name):
    def f(*a, **k):
        raise NotImplementedError(f'{name} is the reference\'s Triton backend; this build has one backend (sm_100a CUDA): use attn()')
    return f


attn_triton = _excluded('attn_triton')
attn_triton_bighead = _excluded('attn_triton_bighead')

__version__ = '0.1'
