"""Host-side checks of the tile scheduler and launch planner (the same functions the kernels
call on the device, reached through the C ABI)."""
import pytest

from mkernel_b200 import _lib
from mkernel_b200._lib import OP_AG, OP_AR, OP_GEMM, OP_RS

CONFIGS = [
    # op, world, M, N, K, layout   (the three headline shapes and the corners of the M x world-size sweep)
    (OP_AG, 8, 8192, 3584, 8192, 0),
    (OP_RS, 8, 8192, 8192, 3584, 0),
    (OP_AR, 8, 128, 8192, 1024, 1),
    (OP_AG, 1, 32768, 28672, 8192, 0),
    (OP_AG, 2, 2048, 14336, 8192, 0),
    (OP_RS, 4, 32768, 8192, 7168, 0),
    (OP_RS, 2, 2048, 8192, 14336, 0),
    (OP_AR, 8, 8192, 8192, 1024, 1),
    (OP_GEMM, 1, 200, 264, 136, 0),
    (OP_AR, 8, 100, 264, 72, 0),
    (OP_AG, 8, 8 * 200, 264, 136, 0),
]


@pytest.mark.parametrize("op,world,M,N,K,layout", CONFIGS)
def test_plan_is_launchable(op, world, M, N, K, layout):
    for rank in range(world):
        p = _lib.plan_op(op, rank, world, M, N, K, layout, 148)
        assert p.smem_bytes <= 232448
        assert 1 <= p.grid <= 148
        assert p.stages >= 2 and p.block_n % (64 if layout else 32) == 0
        assert p.n_comm >= 0 and (p.n_comm == 0 or (world > 1 and op != OP_GEMM))
        cap = {OP_AG: _lib.MK_AG_READY_WORDS, OP_RS: _lib.MK_RS_SYNC_WORDS,
               OP_AR: _lib.MK_AR_BARRIER_WORDS}.get(op)
        if cap:
            assert p.sync_words <= cap


@pytest.mark.parametrize("op,world,M,N,K,layout", CONFIGS)
def test_every_output_element_is_covered_once(op, world, M, N, K, layout):
    p = _lib.plan_op(op, 0, world, M, N, K, layout, 148)
    for rank in {0, world - 1}:
        tiles = _lib.sched_tiles(op, rank, world, M, N, p.block_n, p.group_rows)
        assert len(tiles) == p.row_blocks * p.col_blocks
        seen = set()
        area = 0
        for row0, rows, col0, rb in tiles:
            assert 1 <= rows <= 128 and row0 % 1 == 0
            assert (row0, col0) not in seen
            seen.add((row0, col0))
            area += rows * min(p.block_n, N - col0)
        assert area == M * N


def test_allgather_visits_local_shard_first_then_remote_rows_in_arrival_order():
    world, M, N = 8, 8192, 3584
    rb_per_shard = M // world // 128
    for rank in (0, 3, 7):
        tiles = _lib.sched_tiles(OP_AG, rank, world, M, N, 256, 8)
        seen = []                       # row-blocks in first-visit order: (shard, block)
        for row0, _, _, _ in tiles:
            key = (row0 // (M // world), (row0 % (M // world)) // 128)
            if key not in seen:
                seen.append(key)
        assert seen[:rb_per_shard] == [(rank, j) for j in range(rb_per_shard)]
        rest = seen[rb_per_shard:]
        expect = [((rank + d) % world, j) for j in range(rb_per_shard) for d in range(1, world)]
        # groups of 8 row-blocks are rastered together, so compare as sets per raster group
        for g in range(0, len(rest), 8):
            assert sorted(rest[g:g + 8]) == sorted(expect[g:g + 8])


def test_reduce_scatter_interleaves_owners_own_slice_last():
    world, M, N = 8, 8192, 8192
    rank = 2
    tiles = _lib.sched_tiles(OP_RS, rank, world, M, N, 256, 8)
    # group_rows = 8 = world: each raster group holds one row-block of every owner
    per_group = 8 * (N // 256)
    first = tiles[:per_group]
    owners = sorted({row0 // (M // world) for row0, _, _, _ in first})
    assert owners == list(range(world))
    # within a group the row-block index runs fastest: the 8th tile belongs to this rank
    assert [row0 // (M // world) for row0, _, _, _ in first[:8]] == \
        [(rank + 1 + d) % world for d in range(world)]
    # every owner's j-th row-block is visited in round j
    for idx, (row0, _, _, _) in enumerate(tiles):
        assert (row0 % (M // world)) // 128 == idx // per_group


@pytest.mark.parametrize("op,world,M,N", [(OP_RS, 8, 8192, 8192), (OP_AR, 8, 128, 8192),
                                          (OP_AR, 8, 100, 264), (OP_AR, 4, 1000, 512),
                                          (OP_RS, 2, 384, 256)])
def test_owner_items_partition_the_rows(op, world, M, N):
    covered = []
    for owner in range(world):
        items = _lib.sched_owner_items(op, world, M, N, 128, owner)
        for a, b in items:
            assert 0 <= a < b <= M and b - a <= 128
            assert a // 128 == (b - 1) // 128          # an item never straddles a row-block
            covered.extend(range(a, b))
    assert covered == list(range(M))


def test_block_width_avoids_wave_quantisation():
    # 8192 x 3584 on 148 independent CTAs: 256-wide tiles need 7 waves for 6.05 waves of work,
    # so the planner narrows the tiles (CTA pairs keep 256: narrower halves run the MMA poorly)
    _lib.set_option("cta_pair", 0)
    try:
        p = _lib.plan_op(OP_GEMM, 0, 1, 8192, 3584, 8192, 0, 148)
    finally:
        _lib.set_option("cta_pair", 1)
    tiles = p.row_blocks * p.col_blocks
    waves = -(-tiles // p.grid)
    assert tiles / (waves * p.grid) > 0.95
    assert _lib.plan_op(OP_GEMM, 0, 1, 8192, 3584, 8192, 0, 148).block_n % 128 == 0
    # decode-shaped all-reduce: every tile gets its own CTA
    p = _lib.plan_op(OP_AR, 0, 8, 128, 8192, 1024, 1, 148)
    assert p.row_blocks * p.col_blocks <= p.grid - p.n_comm


@pytest.mark.parametrize("M,N,bn,gr,gc", [(8192, 3584, 256, 12, 7), (8192, 3584, 256, 8, 4),
                                          (1000, 1000, 96, 6, 3), (8192, 28672, 256, 12, 16),
                                          (384, 8192, 128, 2, 5)])
def test_two_level_raster_covers_every_tile_once_and_keeps_pairs_in_one_column(M, N, bn, gr, gc):
    """Column groups outermost, row groups inside, row-block fastest: every tile once; with an
    even number of row-blocks and an even group height tiles 2i and 2i+1 share a column block
    (what a CTA pair needs); a column group is finished before the next one starts."""
    tiles = _lib.sched_tiles(OP_GEMM, 0, 1, M, N, bn, gr, gc)
    P, Q = -(-M // 128), -(-N // bn)
    assert len(tiles) == P * Q
    assert len({(r0, c0) for r0, _, c0, _ in tiles}) == P * Q
    if P % 2 == 0 and gr % 2 == 0:
        for i in range(0, len(tiles), 2):
            assert tiles[i][2] == tiles[i + 1][2] and tiles[i][0] != tiles[i + 1][0]
    groups = [c0 // bn // gc for _, _, c0, _ in tiles]
    assert groups == sorted(groups)
    # more than one GPU: the exchanges are row-ordered, column grouping is ignored
    a = _lib.sched_tiles(OP_AG, 1, 4, 8192, 3584, 256, 8, 4)
    b = _lib.sched_tiles(OP_AG, 1, 4, 8192, 3584, 256, 8, 0)
    assert a == b


@pytest.mark.parametrize("total_tiles,n_comp,cg,k_blocks", [
    (896, 148, 2, 128),     # the up-projection shape: 6.05 rounds, 4 tail pair-tiles cut in 18
    (160, 148, 2, 32),      # 6 tail pair-tiles, pieces capped by four k-blocks each
    (153, 148, 1, 16),      # single-CTA mode
    (224, 148, 2, 128),     # more than half a round left: no cut
    (296, 148, 2, 64),      # exact rounds: no cut
    (100, 148, 1, 64),      # less than one round: no cut
    (300, 146, 2, 9),       # a grid capped below the SM count, few k-blocks
])
def test_work_lists_cover_every_tile_and_k_block_once(total_tiles, n_comp, cg, k_blocks):
    """Whole tiles plus the pieces of a cut last round: every (tile, k-block) exactly once, the
    two CTAs of a pair on consecutive tiles with the same k-range, pieces of a tile in order."""
    seen = {}
    pieces = {}
    for cta in range(n_comp):
        for tile, kb0, kb1, piece in _lib.sched_work_items(total_tiles, n_comp, cg, k_blocks, 32, cta):
            assert 0 <= tile < total_tiles and 0 <= kb0 < kb1 <= k_blocks
            for kb in range(kb0, kb1):
                assert (tile, kb) not in seen, (tile, kb, cta, seen[(tile, kb)])
                seen[(tile, kb)] = cta
            if piece >= 0:
                assert kb1 - kb0 >= 4
                pieces.setdefault(tile, []).append((piece, kb0, kb1, cta))
            else:
                assert (kb0, kb1) == (0, k_blocks)
            if cg == 2:
                assert tile % 2 == cta % 2          # pair member c takes tile 2m + c
    assert len(seen) == total_tiles * k_blocks
    for tile, lst in pieces.items():
        lst.sort()
        assert lst[0][1] == 0 and lst[-1][2] == k_blocks
        assert all(a[2] == b[1] for a, b in zip(lst, lst[1:]))      # contiguous, in piece order
        assert len(lst) >= 2
    # no cut requested: plain round-robin
    plain = [_lib.sched_work_items(total_tiles, n_comp, cg, k_blocks, 0, c) for c in range(n_comp)]
    assert sorted(t for items in plain for t, _, _, _ in items) == list(range(total_tiles))
    assert all(p == -1 for items in plain for _, _, _, p in items)
