"""GPU parity: the CUDA search (through the C ABI) against the CPU oracle and against the reference's shipped dumps.
Everything here is integer work and must match bit for bit."""
import os

import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC
from mcts_numba_cuda_b200.roots import c4_random_roots
from oracle.oracle import OracleMCTSNC
from tests.test_oracle_golden import check_against_dump

pytestmark = pytest.mark.gpu

FIELDS = ["trees_sizes", "trees_depths", "trees_turns", "trees_leaves", "trees_terminals", "trees_ns", "trees_ns_wins",
          "trees", "trees_boards", "trees_extra_infos", "trees_nodes_selected", "trees_actions_expanded",
          "trees_playout_outcomes"]


def make_pair(variant, n_trees, n_playouts, steps, seed=0, ucb_c=2.0, device_memory=2.0, max_batch=1):
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=n_trees, n_playouts=n_playouts,
                variant=variant, device_memory=device_memory, ucb_c=ucb_c, seed=seed, verbose_info=False,
                max_batch=max_batch)
    ai.init_device_side_arrays()
    orc = OracleMCTSNC((6, 7), 7, 7, n_trees=n_trees, n_playouts=n_playouts, variant=variant, device_memory=device_memory,
                       ucb_c=ucb_c, seed=seed, node_capacity=steps * 7 + 8)
    return ai, orc


def compare_trees(ai, orc, search=0):
    sizes = orc.field("trees_sizes")
    assert np.array_equal(ai.export("trees_sizes", search), sizes)
    smax = int(sizes.max())
    valid = np.arange(smax)[None, :] < sizes[:, None]
    for name in FIELDS[1:]:
        mine = ai.export(name, search, max_nodes=smax)
        ref = np.array(orc.field(name))
        if name == "trees_outcomes":
            continue
        if ref.ndim >= 2 and ref.shape[1] == orc.cap:
            ref = ref[:, :smax].copy()
            ref[~valid] = -1 if name == "trees" else 0
            if name == "trees":
                # child columns of a node that was never expanded are not written by the reference (stale from
                # an earlier search of the same instance); the export gives -1 there
                ref[:, :, 1:][orc.field("trees_leaves")[:, :smax] != 0] = -1
        assert np.array_equal(mine, ref), name
    # outcomes are defined for every node but the root (the reference never writes the root's)
    mine = ai.export("trees_outcomes", search, max_nodes=smax)[:, 1:]
    ref = orc.field("trees_outcomes")[:, 1:smax].copy()
    ref[~valid[:, 1:]] = 0
    assert np.array_equal(mine, ref)
    paths, ref_paths = ai.export("trees_selected_paths", search), orc.field("trees_selected_paths")
    for t in range(len(sizes)):
        n = ref_paths[t, -1]
        assert paths[t, -1] == n and np.array_equal(paths[t, :n], ref_paths[t, :n])
    if "acp" in ai.variant:
        assert np.array_equal(ai.export("trees_playout_outcomes_children", search), orc.field("trees_playout_outcomes_children"))


@pytest.mark.parametrize("variant", MCTSNC.VARIANTS)
@pytest.mark.parametrize("n_trees,n_playouts,steps", [(1, 32, 40), (3, 64, 120), (4, 256, 300)])
def test_search_matches_oracle_from_empty_board(variant, n_trees, n_playouts, steps):
    ai, orc = make_pair(variant, n_trees, n_playouts, steps)
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    best = ai.run(board, fills, 1)
    orc.run(board, fills, 1, steps)
    compare_trees(ai, orc)
    assert int(best) == orc.best_action
    assert (ai.best_win_flag, int(ai.best_n), int(ai.best_n_wins)) == (orc.best_win_flag, orc.best_n, orc.best_n_wins)
    assert ai._res["playouts"] == orc.playouts
    assert ai._res["plies"] == orc.plies
    assert ai._res["ub_draws"] == orc.ub_draws


@pytest.mark.parametrize("variant", ["ocp_thrifty", "acp_prodigal"])
def test_random_roots_match_oracle(variant):
    boards, fills, turns = c4_random_roots(24, 30, seed=11)
    steps = 60
    ai, orc = make_pair(variant, 2, 64, steps, seed=5)
    for b in range(len(boards)):
        ai.reset_random_streams()
        orc.reset_rng()
        best = ai.run(boards[b], fills[b], int(turns[b]))
        orc.run(boards[b], fills[b], int(turns[b]), steps)
        compare_trees(ai, orc)
        assert int(best) == orc.best_action, b


@pytest.mark.parametrize("variant", ["ocp_thrifty", "acp_thrifty"])
def test_reference_dump_reproduced(golden_dir, variant):
    """The two 1000-step dumps shipped by the reference (n_trees=4, n_playouts=128, seed 0, empty board)."""
    g = np.load(os.path.join(golden_dir, f"reference_dump_{variant}.npz"))
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=1000, n_trees=4, n_playouts=128, variant=variant,
                device_memory=1.5, ucb_c=2.0, seed=0, verbose_info=False)
    ai.init_device_side_arrays()
    best = ai.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1)
    smax = int(g["trees_sizes"].max())
    check_against_dump(lambda name: ai.export(name, 0, max_nodes=smax), g)
    table = g["root_actions_table"]
    assert np.array_equal(ai._res["root_ns"], table[:, 1])
    assert np.array_equal(ai._res["actions_win_flags"].astype(np.int64), table[:, 2])
    assert np.array_equal(ai._res["actions_ns"], table[:, 3])
    assert np.array_equal(ai._res["actions_ns_wins"], table[:, 4])
    assert int(best) == int(g["best_index"])


def test_batch_equals_single_runs():
    boards, fills, turns = c4_random_roots(16, 20, seed=3)
    steps = 50
    ai, orc = make_pair("acp_prodigal", 4, 128, steps, seed=9, max_batch=16)
    out = ai.run_batch(boards, fills, turns, steps=steps, reseed=True)
    for b in range(len(boards)):
        # a fresh oracle per root: every slot of a batch has its own "last step" arrays, which start as zeros
        orc = OracleMCTSNC((6, 7), 7, 7, n_trees=4, n_playouts=128, variant="acp_prodigal", seed=9, node_capacity=steps * 7 + 8)
        orc.run(boards[b], fills[b], int(turns[b]), steps)
        compare_trees(ai, orc, search=b)
        assert out["best_action"][b] == orc.best_action
        assert out["best_n"][b] == orc.best_n and out["best_n_wins"][b] == orc.best_n_wins
        assert out["playouts"][b] == orc.playouts


def test_streams_continue_across_runs():
    """The reference never re-seeds inside run() (src/mctsnc.py:390-394): a second search continues the streams."""
    steps = 30
    ai, orc = make_pair("acp_prodigal", 2, 32, steps, seed=1)
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    for _ in range(3):
        ai.run(board, fills, -1)
        orc.run(board, fills, -1, steps)
        compare_trees(ai, orc)


def test_bad_root_is_rejected():
    ai, _ = make_pair("acp_prodigal", 1, 32, 10)
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    board[2, 3] = 1  # a floating disc
    fills[3] = 1
    with pytest.raises(RuntimeError):
        ai.run(board, fills, 1)
