"""Shared-memory layouts of the backward kernel, restated in Python and checked on the CPU.

The backward (wind-rwkv7_b200/csrc/wkv7_bwd.cu) receives the chunk-start state and the chunk's four 16x16
matrices by bulk tensor loads into "split, shifted" layouts: rows with (row & 4) == 0 form one dense block,
the other rows a second block whose rows start with 8 floats of fill.  These tests pin the index functions
(s0_at, mat_at) against the layout the loads produce, and check the property the layout exists for: both
access patterns of the warp-level tensor-core fragments touch 32 different banks.
"""
import itertools

N, L = 64, 16
SS = N + 8          # row pitch (floats) of the state buffer
SCS = L + 8         # row pitch (floats) of a matrix row
S0_BLK = 32 * SS
MAT_BLK = 8 * 4 * SCS


def s0_at(row, col):
    return ((row >> 2) & 1) * (S0_BLK + 8) + (((row >> 3) << 2) | (row & 3)) * SS + col


def mat_at(m, row, col):
    return ((row >> 2) & 1) * (MAT_BLK + 8) + ((2 * m + (row >> 3)) * 4 + (row & 3)) * SCS + col


def tma_state_layout():
    """Where the two boxes of the state load put element (row, col): box blk holds rows 8a + 4blk + b as
    [a][b][72 floats]; box 0 starts at column 0, box 1 at column -8."""
    where = {}
    for blk in range(2):
        for a, b in itertools.product(range(8), range(4)):
            for x in range(SS):                      # position inside the box row
                col = x - 8 * blk                    # global column this position reads
                if 0 <= col < N:
                    where[(8 * a + 4 * blk + b, col)] = blk * S0_BLK + (a * 4 + b) * SS + x
    return where


def tma_mats_layout():
    """Where the two boxes of the matrices load put element (m, row, col).  Global order of the 4 KB:
    16-byte pieces [row group rg][piece kc][row % 8], rg = 2m + row / 8; box blk holds rows with bit 2 == blk
    as [rg][row % 4][6 pieces][4 floats], starting at piece 0 (box 0) or -2 (box 1)."""
    where = {}
    for blk in range(2):
        for rg, r4 in itertools.product(range(8), range(4)):
            for x in range(6):
                kc = x - 2 * blk
                if 0 <= kc < 4:
                    m, row = rg >> 1, (rg & 1) * 8 + 4 * blk + r4
                    for e in range(4):
                        where[(m, row, 4 * kc + e)] = blk * MAT_BLK + (rg * 4 + r4) * SCS + 4 * x + e
    return where


def test_state_index_function_matches_the_loads():
    where = tma_state_layout()
    assert len(where) == N * N
    assert len(set(where.values())) == N * N
    assert max(where.values()) < N * SS
    for (row, col), off in where.items():
        assert s0_at(row, col) == off


def test_matrix_index_function_matches_the_loads():
    where = tma_mats_layout()
    assert len(where) == 4 * L * L
    assert len(set(where.values())) == 4 * L * L
    assert max(where.values()) < 2 * MAT_BLK
    for (m, row, col), off in where.items():
        assert mat_at(m, row, col) == off


def banks(offsets):
    return [o % 32 for o in offsets]


def test_state_fragment_patterns_are_conflict_free():
    for warp, kk in itertools.product(range(4), range(8)):
        # rows 16*warp + g, 8-byte loads at columns 8*kk + 2*t4: one half-warp (g = 0..3 or 4..7) per wavefront
        for half in range(2):
            offs = []
            for g, t4 in itertools.product(range(4 * half, 4 * half + 4), range(4)):
                base = s0_at(16 * warp + g, 8 * kk + 2 * t4)
                offs += [base, base + 1]
            assert len(set(banks(offs))) == 32
    for warp, nt, kk, odd in itertools.product(range(4), range(2), range(8), range(2)):
        # rows 8*kk + 2*t4 (+1), column 16*warp + 8*nt + g: 4-byte loads, the whole warp in one wavefront
        offs = [s0_at(8 * kk + 2 * t4 + odd, 16 * warp + 8 * nt + g) for g, t4 in itertools.product(range(8), range(4))]
        assert len(set(banks(offs))) == 32


def test_matrix_fragment_patterns_are_conflict_free():
    for m, nt, kk in itertools.product(range(4), range(2), range(2)):
        for half in range(2):
            offs = []
            for g, t4 in itertools.product(range(4 * half, 4 * half + 4), range(4)):
                base = mat_at(m, 8 * nt + g, 8 * kk + 2 * t4)
                offs += [base, base + 1]
            assert len(set(banks(offs))) == 32
    for m, sb, tb, odd in itertools.product(range(4), range(2), range(2), range(2)):
        offs = [mat_at(m, 8 * tb + 2 * t4 + odd, 8 * sb + g) for g, t4 in itertools.product(range(8), range(4))]
        assert len(set(banks(offs))) == 32


def test_scan_store_order_is_conflict_free():
    """Decay scan: lane = time row (0..15) + 16 * channel half, 32 bytes per lane and tile as two 16-byte stores;
    a 16-byte store is served a quarter-warp (eight lanes = rows r..r+7 of one channel group) at a time.  Rows 4..7
    of every eight store their second half first; with the column swizzle (column ^ 8 for those rows) every quarter
    then covers all 32 banks."""
    OPS = N + 8
    for j0 in range(0, N, 8):
        for first in (True, False):
            for quarter in range(2):
                offs = []
                for row in range(8 * quarter, 8 * quarter + 8):
                    flip = (row >> 2) & 1
                    col = j0 ^ (8 if row & 4 else 0)
                    part = (4 if flip else 0) if first else (0 if flip else 4)
                    base = row * OPS + col + part
                    offs += [base + e for e in range(4)]
                assert len(set(banks(offs))) == 32
