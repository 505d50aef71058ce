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


# ---- the reduce-scatter form's guard against a rank running ahead, restated as a small state machine -------------------------
# Calls are numbered by one counter that every fused kernel of the fabric advances ("S" = GEMM + reduce-scatter, "O" = any other
# fused kernel, e.g. the head's cross-rank argmax). An S call of epoch e pushes partial tiles into the owners' staging half
# e & 1, so before it starts every peer must have finished the PREVIOUS S call that used that half. Each rank leaves, per half,
# the epoch of the last S call it finished, in its own slot table and in every peer's, and an S call waits until every peer
# reports the epoch the rank itself last finished on that half. In this model (as in the kernels) finishing ANY fused call needs
# a push from every peer, which already keeps ranks within one call of each other: the invariant holds with or without the
# guard, so what the guard owes is that it never blocks - whatever other kernels advance the counter in between.
import random


def _simulate(kinds, world, rule, seed):
    rng = random.Random(seed)
    n = len(kinds)
    pc = [0] * world                     # index of the call a rank is in
    started = [False] * world
    slot = [[[0] * world for _ in range(2)] for _ in range(world)]        # slot[r][half][q]
    prev_same_half = {}
    last = {0: None, 1: None}
    for i, k in enumerate(kinds):
        if k == "S":
            prev_same_half[i] = last[(i + 1) & 1]
            last[(i + 1) & 1] = i
    for _ in range(200 * n * world):
        if all(p == n for p in pc):
            return True
        r = rng.randrange(world)
        i = pc[r]
        if i == n:
            continue
        e, h = i + 1, (i + 1) & 1
        if not started[r]:
            if kinds[i] == "S":
                if rule == "none":
                    ok = True
                elif rule == "two_epochs_ago":
                    ok = e <= 2 or all(slot[r][h][q] >= e - 2 for q in range(world) if q != r)
                else:
                    ok = all(slot[r][h][q] >= slot[r][h][r] for q in range(world) if q != r)
                if not ok:
                    continue
                j = prev_same_half[i]
                if j is not None:            # the invariant the guard exists for
                    assert all(pc[q] > j for q in range(world)), f"rank {r} started call {i} while a peer still reduces call {j}"
            started[r] = True
        elif all(pc[q] > i or (pc[q] == i and started[q]) for q in range(world)):      # finishing needs every peer's push
            if kinds[i] == "S":
                for q in range(world):
                    slot[q][h][r] = e
            pc[r], started[r] = i + 1, False
    return False


@pytest.mark.parametrize("world", [2, 4, 8])
def test_reduce_scatter_guard_holds_its_invariant_and_never_blocks(world):
    rng = random.Random(7)
    for trial in range(30):
        kinds = [rng.choice("SSO") for _ in range(rng.randrange(4, 24))]
        assert _simulate(kinds, world, "previous_user", trial), kinds
        assert _simulate(kinds, world, "none", trial), kinds          # the exchange itself keeps the staging halves safe


def test_waiting_for_the_call_two_epochs_ago_blocks_once_other_kernels_interleave():
    assert _simulate(list("SSSSSS"), 2, "two_epochs_ago", 0)               # back-to-back calls: the old rule was enough
    assert not _simulate(list("SSOSS"), 2, "two_epochs_ago", 0)            # call 5 waits for an epoch-3 report nobody makes
    assert _simulate(list("SSOSS"), 2, "previous_user", 0)
