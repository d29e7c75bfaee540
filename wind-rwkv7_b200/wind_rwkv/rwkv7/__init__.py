"""B200 (sm_100a) drop-in for `wind_rwkv.rwkv7` of johanwind/wind-rwkv7 (upstream: rwkv7/__init__.py:1-7)."""
from .rwkv7_ddlerp import ddlerp
from .rwkv7_expand_loras import expand_loras
from .rwkv7_attn import attn, load_attn
from .rwkv7_attn_ln import attn_ln, load_attn_ln

__version__ = '0.1'
