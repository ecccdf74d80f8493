"""Host-side logic of the tensor-parallel split, on CPU: shard ranges, and a world_size-2 gloo run that puts
row-sharded pieces back in rank order the way the model's exchange does."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_leaf_split_is_nested_and_rank_groups_tile_the_axis():
    """The eight leaves of a row-parallel layer's k axis: aligned groups of 8 / world leaves tile the axis for every
    world size, and a group at world w is the union of its two groups at world 2w (so each rank's result is a complete
    subtree of the one summation tree)."""
    from fuel_b200.llama import leaf_split, rank_leaves
    assert leaf_split(16) == [2] * 8 and leaf_split(43) == [5, 5, 5, 6, 5, 6, 5, 6] and leaf_split(4) == [0, 1, 0, 1, 0, 1, 0, 1]
    for nb in (1, 4, 11, 16, 43, 56, 100):
        leaves = leaf_split(nb)
        assert len(leaves) == 8 and sum(leaves) == nb and max(leaves) - min(leaves) <= 1
        for world in (1, 2, 4, 8):
            pos = 0
            for r in range(world):
                b0, mine = rank_leaves(nb, world, r)
                assert b0 == pos and mine == leaves[r * (8 // world):(r + 1) * (8 // world)]
                pos += sum(mine)
            assert pos == nb
        for world in (1, 2, 4):
            for r in range(world):
                b0, mine = rank_leaves(nb, world, r)
                lo, hi = rank_leaves(nb, 2 * world, 2 * r), rank_leaves(nb, 2 * world, 2 * r + 1)
                assert lo[0] == b0 and lo[1] + hi[1] == mine and hi[0] == b0 + sum(lo[1])


def test_pairwise_tree_over_ranks_equals_the_tree_over_all_leaves():
    """f32 model of the row-parallel sum: leaf values added pairwise give the same bits whether one rank adds all
    eight or 2 / 4 / 8 ranks each add their aligned group and the groups are then added pairwise in rank order."""
    rng = np.random.Generator(np.random.PCG64(5))
    leaves = [rng.standard_normal(1000).astype(np.float32) * np.float32(10.0 ** rng.integers(-3, 4)) for _ in range(8)]

    def tree(vals):
        vals = list(vals)
        while len(vals) > 1:
            vals = [(vals[i] + vals[i + 1]).astype(np.float32) for i in range(0, len(vals), 2)]
        return vals[0]

    one = tree(leaves)
    chain = leaves[0]
    for v in leaves[1:]:
        chain = (chain + v).astype(np.float32)
    assert not np.array_equal(one, chain)          # the order matters in f32: that is why it is fixed
    for world in (2, 4, 8):
        per = 8 // world
        assert np.array_equal(tree([tree(leaves[r * per:(r + 1) * per]) for r in range(world)]), one)


def test_shard_range_tiles_the_rows_in_whole_units():
    from fuel_b200.llama import shard_range
    for total, unit in ((11008, 256), (4096, 1), (32000, 1), (2816, 256), (256, 256)):
        for world in (1, 2, 4, 8):
            if total // unit < world:
                continue
            edges = [shard_range(total, world, r, unit) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == total
            for (a0, a1), (b0, b1) in zip(edges, edges[1:]):
                assert a1 == b0
            sizes = [b - a for a, b in edges]
            assert all(sz % unit == 0 and sz > 0 for sz in sizes) and max(sizes) - min(sizes) <= unit
            assert sizes == sorted(sizes, reverse=True)      # the larger shares come first
    # the FFN of the 7B model: 43 blocks
    assert [shard_range(11008, 2, r, 256) for r in range(2)] == [(0, 5632), (5632, 11008)]
    assert [b - a for a, b in (shard_range(11008, 8, r, 256) for r in range(8))] == [1536] * 3 + [1280] * 5


def _worker(rank, world, port, q):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    sys.path.insert(0, ROOT)
    from fuel_b200.llama import shard_range
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, k = 1000, 64
        g = np.random.Generator(np.random.PCG64(0))
        w, x = g.standard_normal((n, k)).astype(np.float32), g.standard_normal(k).astype(np.float32)
        # equal split (library all-gather form)
        lo, hi = shard_range(n, world, rank)
        mine = torch.from_numpy(w[lo:hi] @ x)
        full = torch.empty(n)
        dist.all_gather_into_tensor(full, mine)
        ok_equal = bool(np.array_equal(full.numpy(), np.concatenate([w[a:b] @ x for a, b in
                                                                    (shard_range(n, world, r) for r in range(world))])))
        # uneven whole-unit split (in-kernel exchange form): every rank writes its slice at its own offset
        lo, hi = shard_range(768 * 3, world, rank, 256)
        pieces = [None] * world
        dist.all_gather_object(pieces, (lo, hi, list(range(lo, hi))))
        buf = np.full(768 * 3, -1)
        for a, b, vals in pieces:
            buf[a:b] = vals
        ok_uneven = bool(np.array_equal(buf, np.arange(768 * 3)))
        q.put((rank, ok_equal, ok_uneven))
    finally:
        dist.destroy_process_group()


def test_gloo_two_ranks_reassemble_row_shards_in_rank_order():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, 29541, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(60)
    assert res == [(0, True, True), (1, True, True)]
