"""More GPU parity cases: the random streams, time-limited (multi-launch) searches, sharded handles, and the
full-size headline workload checked through size-independent invariants."""
import ctypes

import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC, _abi
from mcts_numba_cuda_b200.roots import c4_random_roots
from oracle import oracle as om
from oracle.oracle import OracleMCTSNC
from tests.test_gpu_parity_c4 import compare_trees

pytestmark = pytest.mark.gpu


def _streams(ai, which, n, search=0):
    out = np.zeros((n, 2), dtype=np.uint64)
    _abi.check(_abi.lib().mctsnc_export_rng(ai._handle, search, which, out.ctypes.data, n))
    return out


def test_streams_equal_numba_layout():
    """ACP: stream (tree, action, t) = state[tree*A*P + action*P + t] of create_xoroshiro128p_states(T*A*P, seed)
    (src/mctsnc.py:394, :2028); OCP: playout stream (tree, t) = state[tree*P + t], child-pick stream of tree =
    state[tree*tpb_e1] of a second array with the same seed (:391-392, :1385)."""
    ai = MCTSNC((6, 7), 7, 7, search_steps_limit=5, search_time_limit=np.inf, n_trees=3, n_playouts=64, variant="acp_prodigal",
                seed=42, verbose_info=False)
    ai.init_device_side_arrays()
    assert np.array_equal(_streams(ai, 0, 3 * 7 * 64), om.rng_states(3 * 7 * 64, 42))
    ocp = MCTSNC((6, 7), 7, 7, search_steps_limit=5, search_time_limit=np.inf, n_trees=3, n_playouts=64, variant="ocp_prodigal",
                 seed=42, verbose_info=False)
    ocp.init_device_side_arrays()
    ref = om.rng_states(3 * 64, 42)
    assert np.array_equal(_streams(ocp, 0, 3 * 64), ref)
    assert np.array_equal(_streams(ocp, 1, 3), ref[[0, 64, 128]])   # tpb_e1 = 64 for Connect 4


def test_streams_seeded_on_the_device_equal_the_sequential_chain_for_a_large_configuration():
    """The streams are computed on the device, each from its own index (products of jump matrices); numba and the oracle
    build them one after the other.  Gomoku 4 x 225 x 256 = 230 400 streams, and a shard that starts far into the chain."""
    n = 4 * 225 * 256
    ai = MCTSNC((15, 15), 0, 225, search_steps_limit=2, search_time_limit=np.inf, n_trees=4, n_playouts=256, variant="acp_prodigal",
                device_memory=16.0, seed=11, verbose_info=False)
    ai.init_device_side_arrays()
    ref = om.rng_states(n, 11)
    assert np.array_equal(_streams(ai, 0, n), ref)
    shard = MCTSNC((15, 15), 0, 225, search_steps_limit=2, search_time_limit=np.inf, n_trees=1, n_playouts=256,
                   variant="acp_prodigal", device_memory=16.0, seed=11, verbose_info=False, tree_offset=3, n_trees_global=4)
    shard.init_device_side_arrays()
    assert np.array_equal(_streams(shard, 0, 225 * 256), ref[3 * 225 * 256:])
    ocp = MCTSNC((15, 15), 0, 225, search_steps_limit=2, search_time_limit=np.inf, n_trees=3, n_playouts=64, variant="ocp_thrifty",
                 device_memory=16.0, seed=11, verbose_info=False, tree_offset=2, n_trees_global=5)
    ocp.init_device_side_arrays()
    assert np.array_equal(_streams(ocp, 0, 3 * 64), ref[2 * 64:5 * 64])
    assert np.array_equal(_streams(ocp, 1, 3), ref[[2 * 256, 3 * 256, 4 * 256]])   # tpb_e1 = 256 for Gomoku


def test_sharded_streams_are_a_slice_of_the_global_ones():
    kw = dict(search_steps_limit=5, search_time_limit=np.inf, n_playouts=32, variant="acp_thrifty", seed=7, verbose_info=False)
    part = MCTSNC((6, 7), 7, 7, n_trees=2, tree_offset=4, n_trees_global=8, **kw)
    part.init_device_side_arrays()
    ref = om.rng_states(8 * 7 * 32, 7)
    assert np.array_equal(_streams(part, 0, 2 * 7 * 32), ref[4 * 7 * 32:6 * 7 * 32])


@pytest.mark.parametrize("variant", ["acp_prodigal", "ocp_thrifty"])
def test_two_shards_equal_the_unsharded_search(variant):
    """Root parallelism over two handles (as over two GPUs): partial sums add up to the single search with all trees."""
    steps, T = 80, 4
    kw = dict(search_steps_limit=steps, search_time_limit=np.inf, n_playouts=64, variant=variant, seed=5, verbose_info=False)
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    orc = OracleMCTSNC((6, 7), 7, 7, n_trees=T, n_playouts=64, variant=variant, seed=5, node_capacity=steps * 7 + 8)
    orc.run(board, fills, 1, steps)
    total_n, total_w = np.zeros(7, np.int64), np.zeros(7, np.int64)
    for r in range(2):
        shard = MCTSNC((6, 7), 7, 7, n_trees=2, tree_offset=2 * r, n_trees_global=T, **kw)
        shard.init_device_side_arrays()
        shard.run(board, fills, 1)
        total_n += shard._res["actions_ns"]
        total_w += shard._res["actions_ns_wins"]
        assert np.array_equal(shard.export("trees_ns", max_nodes=500), orc.field("trees_ns")[2 * r:2 * r + 2, :500])
    if "prodigal" in variant:
        assert np.array_equal(total_n, orc.field("actions_ns")) and np.array_equal(total_w, orc.field("actions_ns_wins"))
    else:  # thrifty: the oracle indexes by ordinal; all seven actions are expanded at the empty board
        assert np.array_equal(total_n, orc.field("actions_ns")) and np.array_equal(total_w, orc.field("actions_ns_wins"))


@pytest.mark.parametrize("n_playouts,time_limit", [(64, 0.02), (256, 0.01)])   # 256: a cluster of blocks per tree
def test_time_limited_search_is_a_prefix_of_the_step_limited_one(n_playouts, time_limit):
    """A time budget runs the loop as several launches; the trees must equal those of one launch with as many steps."""
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=time_limit, n_trees=2, n_playouts=n_playouts, variant="acp_prodigal", seed=2,
                verbose_info=False, node_capacity=200000)
    ai.init_device_side_arrays()
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    best = ai.run(board, fills, 1)
    steps = ai.steps
    assert steps > 16          # more than one launch
    orc = OracleMCTSNC((6, 7), 7, 7, n_trees=2, n_playouts=n_playouts, variant="acp_prodigal", seed=2, node_capacity=steps * 7 + 8)
    orc.run(board, fills, 1, steps)
    compare_trees(ai, orc)
    assert int(best) == orc.best_action
    # and the forced step count of experiment replays overrides the clock (src/mctsnc.py:597-599)
    ai.reset_random_streams()
    ai.run(board, fills, 1, forced_search_steps_limit=25)
    assert ai.steps == 25


def test_cluster_of_blocks_per_tree_equals_one_block_per_tree(monkeypatch):
    """Launches with few trees of an ACP search with 256 playouts grow a tree with a cluster of 8 blocks; with the switch
    in the environment, or a fixed number of threads, with one block: same trees, same streams afterwards."""
    boards, fills, turns = c4_random_roots(3, 12, seed=21)
    kw = dict(search_time_limit=np.inf, search_steps_limit=120, n_trees=3, n_playouts=256, variant="acp_thrifty", seed=9,
              verbose_info=False, max_batch=3)
    a = MCTSNC((6, 7), 7, 7, **kw)
    a.init_device_side_arrays()
    out_a = a.run_batch(boards, fills, turns, steps=120, reseed=True)
    assert a.launch_geometry()["threads_per_tree"] == 2048
    monkeypatch.setenv("MCTSNC_B200_NO_CLUSTER", "1")
    b = MCTSNC((6, 7), 7, 7, **kw)
    b.init_device_side_arrays()
    out_b = b.run_batch(boards, fills, turns, steps=120, reseed=True)
    assert b.launch_geometry()["threads_per_tree"] == 1024
    for name in ("best_action", "best_n", "best_n_wins", "actions_ns", "actions_ns_wins", "playouts", "plies", "status"):
        assert np.array_equal(out_a[name], out_b[name]), name
    for search in range(3):
        for field in ("trees_ns", "trees_ns_wins"):
            assert np.array_equal(a.export(field, search=search), b.export(field, search=search))
        assert np.array_equal(_streams(a, 0, 3 * 7 * 256, search), _streams(b, 0, 3 * 7 * 256, search))


def test_info_dicts_have_the_reference_keys(capsys):
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=50, n_trees=2, n_playouts=32)
    ai.init_device_side_arrays()
    ai.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1)
    out = capsys.readouterr().out
    assert "MCTSNC RUN... [MCTSNC(" in out and "MCTSNC RUN DONE. [time:" in out and "calculated max_tree_size: " in out
    best = ai.actions_info["best"]
    assert set(best) == {"index", "name", "n_root", "win_flag", "n", "n_wins", "q", "ucb"}
    assert best["index"] == int(ai.best_action)
    e = ai.actions_info[3]
    assert abs(e["q"] - e["n_wins"] / e["n"]) < 1e-12
    assert abs(e["ucb"] - (e["q"] + 2.0 * np.sqrt(np.log(e["n_root"]) / e["n"]))) <= 1e-6 * abs(e["ucb"])
    perf = ai.performance_info
    assert {"steps", "steps_per_second", "playouts", "playouts_per_second", "times_[ms]", "trees"} <= set(perf)
    assert set(perf["times_[ms]"]) == {"total", "loop", "reduce_over_trees", "reduce_over_actions", "mean_loop", "mean_select",
                                       "mean_expand", "mean_playout", "mean_backup"}
    assert set(perf["trees"]) == {"count", "mean_depth", "max_depth", "mean_size", "max_size"}
    assert perf["playouts"] == int(e["n_root"]) and perf["steps"] == 50
    # every time is a number (the reference fills them all, src/mctsnc.py:448-494), the four stages add up to the loop
    times = perf["times_[ms]"]
    assert all(np.isfinite(v) and v >= 0 for v in times.values()), times
    stages = times["mean_select"] + times["mean_expand"] + times["mean_playout"] + times["mean_backup"]
    assert 0.5 * times["mean_loop"] <= stages <= 1.1 * times["mean_loop"], times
    assert times["reduce_over_trees"] > 0 and times["reduce_over_actions"] > 0


def test_stage_times_of_a_gomoku_search_are_filled():
    ai = MCTSNC((15, 15), 0, 225, search_time_limit=np.inf, search_steps_limit=6, n_trees=2, n_playouts=32, device_memory=16.0,
                verbose_info=False)
    ai.init_device_side_arrays()
    ai.run(np.zeros((15, 15), np.int8), None, 1)
    times = ai.performance_info["times_[ms]"]
    assert all(np.isfinite(v) and v >= 0 for v in times.values()), times
    assert times["mean_playout"] > times["mean_select"] > 0 and times["mean_expand"] > 0 and times["mean_backup"] > 0


def test_json_dump_has_the_reference_keys(tmp_path):
    import json
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=30, n_trees=2, n_playouts=32, verbose_info=False)
    ai.init_device_side_arrays()
    ai.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1)
    ai._json_dump(str(tmp_path / "dump.json"))
    d = json.load(open(tmp_path / "dump.json"))
    assert {"n_trees", "n_playouts", "variant", "search_time_limit", "search_steps_limit", "ucb_c", "seed", "device_memory",
            "trees", "trees_sizes", "trees_depths", "trees_turns", "trees_ns", "trees_ns_wins", "trees_nodes_selected",
            "trees_selected_paths", "trees_actions_expanded", "trees_playout_outcomes",
            "trees_playout_outcomes_children"} == set(d)
    assert np.array(d["trees"]).shape == (2, max(d["trees_sizes"]), 8)


def _oracle_headline_search(job):
    board, fills, turn, steps = job
    orc = OracleMCTSNC((6, 7), 7, 7, n_trees=4, n_playouts=256, variant="acp_prodigal", seed=0, node_capacity=steps * 7 + 8)
    orc.run(board, fills, int(turn), steps)
    return orc


def test_full_size_headline_workload_invariants():
    """256 roots x 4 trees x 256 playouts x 2000 steps (the benchmark's batch, run through the work queue): three of
    its searches are compared with the oracle field by field, all of them through properties that hold at any size."""
    from concurrent.futures import ThreadPoolExecutor
    B, steps = 256, 2000
    boards, fills, turns = c4_random_roots(B, 20, seed=0)
    checked = (0, 101, 255)
    pool = ThreadPoolExecutor(max_workers=len(checked))     # about 16 s each on a host core, while the GPU works
    oracles = [pool.submit(_oracle_headline_search, (boards[b], fills[b], turns[b], steps)) for b in checked]
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=4, n_playouts=256,
                variant="acp_prodigal", verbose_info=False, max_batch=B)
    ai.init_device_side_arrays()
    out = ai.run_batch(boards, fills, turns, steps=steps, reseed=True)
    again = ai.run_batch(boards, fills, turns, steps=steps, reseed=True)
    for name in ("best_action", "best_n", "best_n_wins", "playouts", "plies", "actions_ns", "actions_ns_wins"):
        assert np.array_equal(out[name], again[name]), name          # re-seeded searches repeat exactly
    assert (out["status"] & _abi.STATUS_INTERNAL == 0).all() and (out["status"] & _abi.STATUS_TREE_FULL == 0).all()
    assert (out["steps"] == steps).all()
    exp = out["actions_expanded"][:, :7].astype(bool)
    assert np.array_equal(exp, fills < 6)                              # root children = columns with room
    root_ns = np.where(exp, out["root_ns"][:, :7], 0)
    assert (root_ns.max(axis=1) == out["playouts"]).all()
    assert (np.where(exp, out["actions_ns"][:, :7], 0).sum(axis=1) == out["playouts"]).all()   # every playout passes a root child
    assert (out["actions_ns_wins"][:, :7] <= out["actions_ns"][:, :7]).all()
    assert (out["best_n"] == np.where(out["actions_win_flags"][:, :7].any(axis=1), out["best_n"],
                                      np.where(exp, out["actions_ns"][:, :7], -1).max(axis=1))).all()
    for b in (0, 17, 255):                                             # tree-level invariants on a few searches
        sizes = ai.export("trees_sizes", b)
        smax = int(sizes.max())
        trees, ns, wins = (ai.export(n, b, max_nodes=smax) for n in ("trees", "trees_ns", "trees_ns_wins"))
        depths, leaves = ai.export("trees_depths", b, max_nodes=smax), ai.export("trees_leaves", b, max_nodes=smax)
        for t in range(4):
            n = sizes[t]
            par = trees[t, 1:n, 0]
            assert (par >= 0).all() and (par < np.arange(1, n)).all()
            assert np.array_equal(depths[t, 1:n], depths[t, par] + 1)
            child_sum = np.bincount(par, weights=ns[t, 1:n], minlength=n).astype(np.int64)
            inner = leaves[t, :n] == 0
            own = np.where(np.arange(n) == 0, 0, 256)     # a child got its own 256 playouts at the step that created it
            assert np.array_equal(child_sum[inner] + own[inner], ns[t, :n][inner].astype(np.int64))   # the rest went through its children
            win_sum = np.bincount(par, weights=wins[t, 1:n], minlength=n).astype(np.int64)
            assert (wins[t, :n][inner] + win_sum[inner] <= ns[t, :n][inner]).all()      # the rest are draws
            assert n == 1 + int((trees[t, :n, 1:] >= 0).sum())
    geo = ai.launch_geometry()
    assert B * 4 > geo["blocks_per_sm"] * geo["sm_count"]            # the batch went through the work queue
    for b, fut in zip(checked, oracles):
        orc = fut.result()
        compare_trees(ai, orc, search=b)
        assert out["best_action"][b] == orc.best_action and out["best_n"][b] == orc.best_n
        assert out["best_n_wins"][b] == orc.best_n_wins and out["playouts"][b] == orc.playouts
        assert out["plies"][b] == orc.plies and out["ub_draws"][b] == orc.ub_draws
        assert np.array_equal(out["actions_ns"][b, :7], orc.field("actions_ns"))
        assert np.array_equal(out["actions_ns_wins"][b, :7], orc.field("actions_ns_wins"))
    pool.shutdown()
    # a search does not depend on its position in the batch
    perm = np.random.default_rng(1).permutation(B)
    short = ai.run_batch(boards, fills, turns, steps=100, reseed=True)
    shuffled = ai.run_batch(boards[perm], fills[perm], turns[perm], steps=100, reseed=True)
    assert np.array_equal(short["best_n_wins"][perm], shuffled["best_n_wins"])
    assert np.array_equal(short["actions_ns"][perm], shuffled["actions_ns"])


def test_ub_draws_are_replayed_like_the_oracle():
    """A search long enough to meet draws equal to 1.0f (about 2**-25 per draw): the byte-level replay must agree."""
    steps = 1500
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=4, n_playouts=256,
                variant="acp_prodigal", seed=0, verbose_info=False)
    ai.init_device_side_arrays()
    orc = OracleMCTSNC((6, 7), 7, 7, n_trees=4, n_playouts=256, variant="acp_prodigal", seed=0, node_capacity=steps * 7 + 8)
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    ai.run(board, fills, 1)
    orc.run(board, fills, 1, steps)
    assert orc.ub_draws > 0 and ai._res["ub_draws"] == orc.ub_draws
    assert ai._res["status"] & _abi.STATUS_UB_DRAW
    compare_trees(ai, orc)


@pytest.mark.parametrize("variant,n_trees,n_playouts,steps,ucb_c,seed", [
    ("acp_prodigal", 2, 512, 60, 2.0, 0),      # largest n_playouts: 56 KB of stream states per block (opt-in shared memory)
    ("ocp_prodigal", 3, 512, 150, 0.5, 7),
    ("acp_thrifty", 2, 1, 200, 2.0, 1),        # smallest n_playouts
    ("ocp_thrifty", 5, 2, 300, 1.0, 2),
    ("acp_prodigal", 64, 32, 25, 3.5, 123456789),   # many trees, another seed and exploration constant
    ("ocp_thrifty", 1, 32, 200, 2.0, 0),       # BASELINE config 1 shape
])
def test_edge_sizes_match_oracle(variant, n_trees, n_playouts, steps, ucb_c, seed):
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=n_trees, n_playouts=n_playouts,
                variant=variant, ucb_c=ucb_c, seed=seed, verbose_info=False)
    ai.init_device_side_arrays()
    orc = OracleMCTSNC((6, 7), 7, 7, n_trees=n_trees, n_playouts=n_playouts, variant=variant, ucb_c=ucb_c, seed=seed,
                       node_capacity=steps * 7 + 8)
    boards, fills, turns = c4_random_roots(2, 12, seed=seed % 1000)
    for b in range(2):
        best = ai.run(boards[b], fills[b], int(turns[b]))
        orc.run(boards[b], fills[b], int(turns[b]), steps)
        compare_trees(ai, orc)
        assert int(best) == orc.best_action
        assert ai._res["plies"] == orc.plies


def test_tree_full_is_reported_not_followed():
    """A tiny memory budget (max_tree_size = 40 by the reference's formula, src/mctsnc.py:350-358): the trees stop growing,
    the status says so, nothing is written out of bounds."""
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=100, n_trees=2, n_playouts=32,
                variant="acp_prodigal", verbose_info=False, device_memory=24200 / 2 ** 30)
    ai.init_device_side_arrays()
    assert ai.max_tree_size == 40
    ai.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1)
    assert ai.status & _abi.STATUS_TREE_FULL
    sizes = ai.export("trees_sizes")
    assert (sizes <= 40).all() and (sizes > 30).all()
    ns = ai.export("trees_ns", max_nodes=40)
    assert (ns[:, 0] > 0).all() and ai.steps == 100


@pytest.mark.parametrize("variant", ["acp_prodigal", "ocp_thrifty"])
def test_queued_batch_matches_oracle(variant):
    """More trees than blocks fit on the device: a persistent grid takes 32-step slices of the trees from the work queue
    (whichever tree has most time left first).  Every tree must come out as if it had been grown in one go."""
    B, T, P, steps = 200, 4, 32, 75       # 800 trees; slices of 32, 32 and 11 steps
    boards, fills, turns = c4_random_roots(B, 20, seed=5)
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=T, n_playouts=P, variant=variant,
                seed=4, verbose_info=False, max_batch=B, threads_per_tree=384)   # large blocks: fewer fit than there are trees
    ai.init_device_side_arrays()
    out = ai.run_batch(boards, fills, turns, steps=steps, reseed=True)
    geo = ai.launch_geometry()
    assert B * T > geo["blocks_per_sm"] * geo["sm_count"] and steps > MCTSNC.SLICE_STEPS   # the queue was used
    assert (out["status"] & _abi.STATUS_INTERNAL == 0).all()
    assert (out["steps"] == steps).all()
    again = ai.run_batch(boards, fills, turns, steps=steps, reseed=True)
    for name in ("best_action", "best_n", "best_n_wins", "playouts", "plies", "actions_ns", "actions_ns_wins", "root_ns"):
        assert np.array_equal(out[name], again[name]), name
    for b in (0, 57, 123, 199):
        orc = OracleMCTSNC((6, 7), 7, 7, n_trees=T, n_playouts=P, variant=variant, seed=4, node_capacity=steps * 7 + 8)
        orc.run(boards[b], fills[b], int(turns[b]), steps)
        compare_trees(ai, orc, search=b)
        assert out["best_action"][b] == orc.best_action
        assert out["best_n"][b] == orc.best_n and out["best_n_wins"][b] == orc.best_n_wins
        assert out["playouts"][b] == orc.playouts and out["plies"][b] == orc.plies
    # the same roots a few at a time (one block per tree, no queue) give the same searches
    few = ai.run_batch(boards[:8], fills[:8], turns[:8], steps=steps, reseed=True)
    for name in ("best_action", "best_n", "best_n_wins", "actions_ns", "actions_ns_wins"):
        assert np.array_equal(out[name][:8], few[name]), name


@pytest.mark.parametrize("variant,n_trees,n_playouts,roots,threads", [
    ("acp_prodigal", 4, 256, 128, 320),     # many trees, 1792 games a step: a quarter of the games, capped
    ("ocp_prodigal", 8, 32, 64, 32),        # many trees, 32 games a step: one warp
    ("ocp_prodigal", 8, 512, 64, 128),
    ("ocp_prodigal", 8, 256, 64, 128),      # at most 256 games a step: half of them
    ("acp_prodigal", 4, 256, 1, 2048),      # few trees, more than 256 games a step: 8 blocks of 256 per tree
    ("acp_prodigal", 4, 64, 1, 2048),
    ("acp_prodigal", 4, 32, 1, 224),        # few games a step: a block per tree, one thread per game
    ("ocp_thrifty", 1, 32, 1, 32),
])
def test_block_size_follows_the_games_per_step(variant, n_trees, n_playouts, roots, threads):
    boards, fills, turns = c4_random_roots(roots, 10, seed=2)
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=8, n_trees=n_trees, n_playouts=n_playouts,
                variant=variant, verbose_info=False, max_batch=roots)
    ai.init_device_side_arrays()
    out = ai.run_batch(boards, fills, turns, steps=8, reseed=True)
    assert (out["status"] & _abi.STATUS_INTERNAL == 0).all()
    assert ai.launch_geometry()["threads_per_tree"] == threads


def test_slice_trace_accounts_for_every_step_of_every_tree():
    """The diagnostic record of a queued launch: every tree gets its steps in slices of at most 32, one after the other."""
    B, T, steps = 150, 4, 100
    boards, fills, turns = c4_random_roots(B, 20, seed=9)
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=T, n_playouts=64, variant="acp_prodigal",
                verbose_info=False, max_batch=B, threads_per_tree=384)
    ai.init_device_side_arrays()
    ai.trace_slices(B * T * 4 + 8)
    plain = ai.run_batch(boards, fills, turns, steps=steps, reseed=True)
    rec = ai.read_slices()
    assert len(rec) == B * T * 4                      # 32 + 32 + 32 + 4 steps
    tree, t0, t1, steps_run = rec[:, 0], rec[:, 1], rec[:, 2], rec[:, 3] & 0xFFFFFFFF
    assert (t1 >= t0).all() and set(np.unique(steps_run)) == {4, 32}
    order = np.lexsort((t0, tree))
    tree, t0, t1, steps_run = tree[order].reshape(B * T, 4), t0[order].reshape(B * T, 4), t1[order].reshape(B * T, 4), steps_run[order].reshape(B * T, 4)
    assert (tree == np.arange(B * T)[:, None]).all() and (steps_run.sum(axis=1) == steps).all()
    assert (t0[:, 1:] >= t1[:, :-1]).all()            # a tree's slices never overlap
    ai.trace_slices(0)
    again = ai.run_batch(boards, fills, turns, steps=steps, reseed=True)
    assert len(ai.read_slices()) == 0
    for name in ("best_action", "best_n", "best_n_wins", "actions_ns"):
        assert np.array_equal(plain[name], again[name]), name
