"""Host-side logic of attn(..., time_split='tail'): which chains are cut in time and into how many segments.
No GPU: the plan is arithmetic on (B, T, H, number of SMs)."""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), '..', 'wind-rwkv7_b200'))

from wind_rwkv.rwkv7.rwkv7_attn import tail_split_plan  # noqa: E402


def test_config4_shapes():
    # 320 chains on 148 SMs: two full rounds and 24 chains (heads 16..39 of the last sequence); 16 segments of 4096 steps
    assert tail_split_plan(8, 65536, 40, 148) == (24, 16)
    # the same model on two GPUs: 160 chains = one round and 12 chains
    tail, n = tail_split_plan(4, 65536, 40, 148)
    assert tail == 12 and 65536 % n == 0 and (65536 // n) % 16 == 0 and n >= 4


def test_declines_when_it_does_not_pay():
    assert tail_split_plan(64, 1024, 12, 148) is None     # the last round's 28 chains span more than one batch entry
    assert tail_split_plan(16, 4096, 32, 148) is None     # 68 chains in the last round: more than one batch entry
    assert tail_split_plan(1, 65536, 12, 148) is None     # fewer chains than SMs: no full round to hide the passes behind
    assert tail_split_plan(4, 1024, 40, 148) is None      # short sequences: the passes' fixed costs exceed the round they replace
    assert tail_split_plan(2, 4096, 74, 148) is None      # chains fill the rounds exactly


def test_segments_divide_the_sequence_into_whole_chunks():
    for T in (8192, 16384, 24576, 65536):
        plan = tail_split_plan(4, T, 40, 148)
        if plan is not None:
            tail, n = plan
            assert tail == 12 and T % n == 0 and (T // n) % 16 == 0
