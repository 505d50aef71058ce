"""Tile schedule of the persistent GEMM + all-reduce / reduce-scatter kernel (csrc/kernels/tc_gemm_ar.cu), restated on the CPU:
every rank's schedule must be a permutation of the tiles, with the tiles it does not own first and its own tiles last, and in
reduce-scatter mode the foreign owners must be visited in ring order so that no GPU is the target of two senders at once."""
import pytest


def tile_at(pos, ntiles, world, rank, scatter=False, tiles_per_rank=0):
    if world == 1:
        return pos
    if scatter:
        own, foreign = tiles_per_rank, ntiles - tiles_per_rank
        if pos >= foreign:
            return rank * own + (pos - foreign)
        return ((rank + 1 + pos // own) % world) * own + pos % own
    owned = (ntiles - rank + world - 1) // world
    foreign = ntiles - owned
    if pos < foreign:
        g, i = divmod(pos, world - 1)
        return g * world + (i if i < rank else i + 1)
    return (pos - foreign) * world + rank


def owner_of(tile, world, scatter=False, tiles_per_rank=0):
    return min(tile // tiles_per_rank, world - 1) if scatter else tile % world


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("ntiles", [1, 2, 7, 8, 64, 509, 512])
def test_all_reduce_schedule_is_a_permutation_with_own_tiles_last(world, ntiles):
    for rank in range(world):
        order = [tile_at(p, ntiles, world, rank) for p in range(ntiles)]
        assert sorted(order) == list(range(ntiles))
        mine = [owner_of(t, world) == rank for t in order]
        first_own = mine.index(True) if True in mine else ntiles
        assert all(mine[first_own:]) and not any(mine[:first_own])
        foreign = order[:first_own]
        assert foreign == sorted(foreign)          # index order, the order in which the owners consume them


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("per_rank", [1, 3, 16])
def test_reduce_scatter_schedule_visits_owners_in_ring_order(world, per_rank):
    ntiles = world * per_rank
    at_step = {}
    for rank in range(world):
        order = [tile_at(p, ntiles, world, rank, True, per_rank) for p in range(ntiles)]
        assert sorted(order) == list(range(ntiles))
        owners = [owner_of(t, world, True, per_rank) for t in order]
        assert owners[-per_rank:] == [rank] * per_rank and rank not in owners[:-per_rank]
        for j in range(world - 1):
            block = owners[j * per_rank:(j + 1) * per_rank]
            assert block == [(rank + 1 + j) % world] * per_rank
            at_step.setdefault(j, []).append(block[0])
    for j, targets in at_step.items():
        assert sorted(targets) == list(range(world))   # one sender per destination at every step of the ring
