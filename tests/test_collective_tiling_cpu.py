"""Index arithmetic of the fused GEMM collectives (``csrc/gemm/tcgen05_gemm.cu``: ``tile_coords_mn``,
``tile_coords_ar``, ``ar_owner_slot``, the unit order of the all-gather form), restated in Python and checked for
every world size the heap supports: each rank visits every output tile exactly once, owners and staging slots are
consistent between the sender's and the owner's view, the staging capacity the launcher checks is enough, and the
pull order of the all-gather form matches the order in which the tiles need the rows."""
import itertools

import pytest

BM = 128


def tile_coords_mn(tile, m_tiles, n_tiles, group_m):
    per_group = group_m * n_tiles
    g = tile // per_group
    first_m = g * group_m
    gsz = min(group_m, m_tiles - first_m)
    i = tile - g * per_group
    return first_m + i % gsz, i // gsz


def tile_coords_ar(mode, rank, world, tile, m_tiles, n_tiles, group_m):
    """mode 0: all-reduce (plain order), 1: reduce-scatter (own block last), 2: all-gather (own block first)."""
    if mode == 0:
        return tile_coords_mn(tile, m_tiles, n_tiles, group_m)
    mt_per = m_tiles // world
    per = mt_per * n_tiles
    blk = tile // per
    owner = (rank + blk + (0 if mode == 2 else 1)) % world
    ml, ni = tile_coords_mn(tile - blk * per, mt_per, n_tiles, group_m)
    return owner * mt_per + ml, ni


def owner_slot(scatter, world, m_tiles, n_tiles, mi, ni):
    if scatter:
        mt_per = m_tiles // world
        owner = mi // mt_per
        return owner, ((mi - owner * mt_per) * n_tiles + ni) * world
    t = mi * n_tiles + ni
    return t % world, (t // world) * world


@pytest.mark.parametrize("world", [2, 3, 4, 5, 8, 16])
@pytest.mark.parametrize("mt_per,n_tiles", [(1, 1), (1, 4), (2, 3), (8, 16), (17, 5), (40, 2)])
def test_every_rank_walks_every_tile_once_and_blocks_are_ordered(world, mt_per, n_tiles):
    m_tiles, group_m = mt_per * world, 16
    total = m_tiles * n_tiles
    for mode, rank in itertools.product((0, 1, 2), range(world)):
        seq = [tile_coords_ar(mode, rank, world, t, m_tiles, n_tiles, group_m) for t in range(total)]
        assert sorted(seq) == sorted(itertools.product(range(m_tiles), range(n_tiles)))
        if mode:
            blocks = [mi // mt_per for mi, _ in seq]
            order = [blocks[i] for i in range(0, total, mt_per * n_tiles)]
            first = rank if mode == 2 else (rank + 1) % world
            assert order == [(first + b) % world for b in range(world)]          # successor ... own, or own ... predecessor
            assert all(blocks[i] == order[i // (mt_per * n_tiles)] for i in range(total))


@pytest.mark.parametrize("world", [2, 3, 4, 8, 16])
@pytest.mark.parametrize("mt_per,n_tiles", [(1, 1), (2, 3), (8, 16), (17, 5)])
@pytest.mark.parametrize("scatter", [False, True])
def test_staging_slots_are_disjoint_per_owner_and_fit_the_checked_capacity(world, mt_per, n_tiles, scatter):
    m_tiles = mt_per * world
    out_tiles = m_tiles * n_tiles
    capacity = (out_tiles + world - 1) // world * world          # slots the launcher requires of every rank's buffer
    used = {r: set() for r in range(world)}
    for mi, ni in itertools.product(range(m_tiles), range(n_tiles)):
        owner, slot0 = owner_slot(scatter, world, m_tiles, n_tiles, mi, ni)
        assert 0 <= owner < world
        if scatter:
            assert owner == mi // mt_per                          # the rank that keeps these rows
        for sender in range(world):
            s = slot0 + sender
            assert s not in used[owner] and 0 <= s < capacity
            used[owner].add(s)
    if scatter or out_tiles % world == 0:           # every owner then reduces the same number of tiles
        assert len({len(v) for v in used.values()}) == 1


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("mt_per,k", [(1, 256), (4, 264), (8, 5376), (3, 8)])
def test_all_gather_units_cover_foreign_rows_in_the_order_the_tiles_need_them(world, mt_per, k):
    unit_cols = 256
    kch = (k + unit_cols - 1) // unit_cols
    units = (world - 1) * mt_per * kch
    for rank in range(world):
        arrived = {}
        first_unit_of_block = {}
        for u in range(units):
            kc, mt, blk = u % kch, (u // kch) % mt_per, u // (kch * mt_per) + 1
            src = (rank + blk) % world
            assert src != rank
            mi = src * mt_per + mt
            cols = min(unit_cols, k - kc * unit_cols)
            assert cols > 0 and cols % 8 == 0
            arrived[mi] = arrived.get(mi, 0) + cols
            first_unit_of_block.setdefault(src, u)
        m_tiles = mt_per * world
        assert arrived == {mi: k for mi in range(m_tiles) if mi // mt_per != rank}     # every foreign row tile, all columns
        # blocks are pulled in the order the tile sequence reaches them
        order = sorted(first_unit_of_block, key=first_unit_of_block.get)
        assert order == [(rank + b) % world for b in range(1, world)]
