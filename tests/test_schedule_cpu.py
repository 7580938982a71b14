"""The GEMM kernels' static tile schedule, checked on the host replica of the
device function: every tile exactly once, block c of every owner before block
c+1 of any owner for the reduce-scatter, own rows first and arrival order after
that for the all-gather."""
import ctypes as C

import pytest

from kernel_b200 import _native as N

PLAIN, RS, AG = 0, 1, 2


def schedule(mode, M, Nn, rank, world, pair):
    lib = N.lib()
    total = lib.kb_gemm_schedule(mode, M, Nn, rank, world, int(pair), -1, None, None)
    if total < 0:
        return None
    blk, nb = C.c_int(), C.c_int()
    out = []
    for pos in range(total):
        lib.kb_gemm_schedule(mode, M, Nn, rank, world, int(pair), pos, C.byref(blk), C.byref(nb))
        out.append((blk.value, nb.value))
    return out


@pytest.mark.parametrize("pair", [False, True])
@pytest.mark.parametrize("M,Nn,world", [(8192, 8192, 8), (2048, 4096, 8), (4096, 2880, 2), (16384, 4096, 8), (1000, 1000, 1), (8192, 29568, 1)])
@pytest.mark.parametrize("mode", [PLAIN, RS, AG])
def test_every_tile_exactly_once(mode, M, Nn, world, pair):
    rows = 256 if pair else 128
    for rank in range(world):
        tiles = schedule(mode, M, Nn, rank, world, pair)
        if tiles is None:
            assert pair and (M // world) % 256 != 0
            continue
        mbq, nbs = -(-M // rows), -(-Nn // 256)
        assert len(tiles) == mbq * nbs and len(set(tiles)) == len(tiles)
        assert all(0 <= b < mbq and 0 <= n < nbs for b, n in tiles)


def _first_appearances(tiles):
    seq = []
    for b, _ in tiles:
        if b not in seq:
            seq.append(b)
    return seq


@pytest.mark.parametrize("pair", [False, True])
def test_reduce_scatter_visits_block_c_of_every_owner_before_block_c_plus_1(pair):
    M, Nn, world = 8192, 8192, 8
    rows = 256 if pair else 128
    per_rank = M // world // rows
    for rank in range(world):
        seq = _first_appearances(schedule(RS, M, Nn, rank, world, pair))
        assert [b % per_rank for b in seq] == sorted(b % per_rank for b in seq)   # chunk-major on every rank
        for c in range(per_rank):
            owners = [b // per_rank for b in seq[c * world:(c + 1) * world]]
            assert owners == [(rank + 1 + d) % world for d in range(world)]         # ring order, own block last


def test_small_m_reduce_scatter_single_block_holds_all_owners():
    tiles = schedule(RS, 64, 2880, 3, 8, False)  # 8 rows per rank: one row block for everybody
    assert {b for b, _ in tiles} == {0} and len(tiles) == 12


@pytest.mark.parametrize("pair", [False, True])
def test_all_gather_order_own_first_then_arrival_order(pair):
    M, Nn, world = 8192, 3696, 8
    rows = 256 if pair else 128
    per_rank = M // world // rows
    for rank in range(world):
        tiles = schedule(AG, M, Nn, rank, world, pair)
        seq = []
        for b, _ in tiles:  # order in which row blocks first appear
            if b not in seq:
                seq.append(b)
        assert seq[:per_rank] == list(range(rank * per_rank, (rank + 1) * per_rank))
        rest = seq[per_rank:]
        # block c of every other source before block c+1 of any source
        chunk_index = [b % per_rank for b in rest]
        assert chunk_index == sorted(chunk_index)
        first_round = rest[:world - 1]
        assert [b // per_rank for b in first_round] == [(rank + d) % world for d in range(1, world)]


def test_schedule_properties_over_random_problems():
    """Random shapes, world sizes and tile configurations: every tile exactly once; for
    the reduce-scatter the blocks appear chunk by chunk (block c of every owner before
    block c+1 of any) when blocks do not straddle owners; for the all-gather the first
    row block visited holds own rows."""
    from hypothesis import given, settings
    from hypothesis import strategies as st

    @settings(max_examples=150, deadline=None)
    @given(mode=st.sampled_from([PLAIN, RS, AG]), world=st.sampled_from([1, 2, 3, 4, 8, 16]), pair=st.booleans(),
           rows_factor=st.sampled_from([8, 16, 32, 64, 128, 256, 384, 512, 1024]), extra_m=st.integers(0, 127),
           n=st.integers(1, 40).map(lambda v: v * 104))
    def check(mode, world, pair, rows_factor, extra_m, n):
        M = rows_factor * world + (extra_m if mode == PLAIN else 0)   # fused modes need M divisible by world
        rpo = M // world
        if mode != PLAIN and world > 1 and rpo % 128 != 0 and 128 % rpo != 0:
            return                                                     # refused by the launcher, not a schedule case
        rows = 256 if pair else 128
        for rank in sorted({0, world // 2, world - 1}):
            tiles = schedule(mode, M, n, rank, world, pair)
            if tiles is None:
                assert pair and mode != PLAIN and world > 1 and rpo % 256 != 0
                continue
            mbq, nbs = -(-M // rows), -(-n // 256)
            assert len(tiles) == mbq * nbs and len(set(tiles)) == len(tiles)
            assert all(0 <= b < mbq and 0 <= c < nbs for b, c in tiles)
            if world == 1 or mode == PLAIN:
                continue
            lo, hi = rank * rpo, (rank + 1) * rpo - 1                  # rows of this rank
            own = [lo // rows <= b <= hi // rows for b, _ in tiles]
            if mode == RS:
                if rpo % rows == 0:
                    chunk = [b % (rpo // rows) for b in _first_appearances(tiles)]
                    assert chunk == sorted(chunk)                      # chunk-major
            else:
                assert own[0]                                          # the all-gather starts on rows it already has

    check()
