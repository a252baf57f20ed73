"""The multi-GPU (root-parallel) path on CPU: two gloo ranks each GROW half of the trees of a search (the CPU oracle
with a tree offset, i.e. with the random streams those trees have in the unsharded search -- what a rank's handle does
on its GPU), form the partial per-action sums of their own trees, all-reduce them and run the final argmax; the result
must equal the unsharded search, which every rank also runs for comparison."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mcts_numba_cuda_b200.distributed import reduce_over_actions_host, shard_trees
from oracle.oracle import OracleMCTSNC


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _partial_sums(orc, lo, hi):
    A = orc.A
    trees, ns, wins = orc.field("trees"), orc.field("trees_ns"), orc.field("trees_ns_wins")
    sums = np.zeros(3 * A, dtype=np.int64)
    expanded = trees[0, 0, 1:] >= 0
    for a in range(A):
        if not expanded[a]:
            continue
        for t in range(lo, hi):
            child = trees[t, 0, 1 + a]
            sums[a] += ns[t, 0]
            sums[A + a] += ns[t, child]
            sums[2 * A + a] += wins[t, child]
    return sums, expanded


def _worker(rank, world, port, variant, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        T_global, steps = 4, 60
        orc = OracleMCTSNC((6, 7), 7, 7, n_trees=T_global, n_playouts=32, variant=variant, seed=3, node_capacity=steps * 7 + 8)
        orc.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1, steps)
        offset, local = shard_trees(T_global, world, rank)
        mine = OracleMCTSNC((6, 7), 7, 7, n_trees=local, n_playouts=32, variant=variant, seed=3, node_capacity=steps * 7 + 8,
                            tree_offset=offset, n_trees_global=T_global)
        mine.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1, steps)
        sums, expanded = _partial_sums(mine, 0, local)
        for t in range(local):      # the shard's trees are the trees [offset, offset + local) of the unsharded search
            n = orc.field("trees_sizes")[offset + t]
            assert mine.field("trees_sizes")[t] == n
            assert np.array_equal(mine.field("trees_ns")[t, :n], orc.field("trees_ns")[offset + t, :n])
            assert np.array_equal(mine.field("trees_ns_wins")[t, :n], orc.field("trees_ns_wins")[offset + t, :n])
        t = torch.from_numpy(sums)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        total = t.numpy()
        A = orc.A
        best = reduce_over_actions_host(mine.field("actions_win_flags") if "prodigal" in variant else
                                        _flags_by_action(mine), total[A:2 * A], total[2 * A:], expanded, "thrifty" in variant)
        ok = best == (orc.best_action, orc.best_win_flag, orc.best_n, orc.best_n_wins)
        root_ok = np.array_equal(total[:A][expanded], np.full(int(expanded.sum()), orc.playouts))
        np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array([ok, root_ok]))
    finally:
        dist.destroy_process_group()


def _flags_by_action(orc):
    # the thrifty variants of the reference index the flags by ordinal; bring them to action order
    flags = np.zeros(orc.A, dtype=np.uint8)
    rae = orc.field("root_actions_expanded")
    for i in range(rae[-1]):
        flags[rae[i]] = orc.field("actions_win_flags")[i]
    return flags


@pytest.mark.parametrize("variant", ["acp_prodigal", "ocp_thrifty"])
def test_two_rank_root_parallel_equals_unsharded(tmp_path, variant):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), variant, str(tmp_path)), nprocs=world, join=True)
    for rank in range(world):
        assert np.load(tmp_path / f"ok_{rank}.npy").all()
