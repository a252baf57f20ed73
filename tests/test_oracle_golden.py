"""Pins the CPU oracle to the two tree dumps the reference ships (1000-step searches from the empty Connect-4 board,
written by ``_json_dump``, ``src/mctsnc.py:2377-2462``) and to the root-action tables printed in the matching logs."""
import os

import numpy as np
import pytest

from oracle.oracle import OracleMCTSNC, reference_max_tree_size


def _run_like_dump(variant, steps=1000):
    o = OracleMCTSNC((6, 7), 7, 7, n_trees=4, n_playouts=128, variant=variant, device_memory=1.5, ucb_c=2.0, seed=0,
                     node_capacity=steps * 7 + 8)
    o.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1, steps)
    return o


def check_against_dump(get, g, variant_is_thrifty=True):
    """``get(name)`` returns the array of the implementation under test; ``g`` is the loaded fixture."""
    sizes = g["trees_sizes"]
    assert np.array_equal(get("trees_sizes"), sizes)
    smax = int(sizes.max())
    valid = np.arange(smax)[None, :] < sizes[:, None]
    for name in ("trees_depths", "trees_turns", "trees_ns", "trees_ns_wins"):
        mine = np.array(get(name)[:, :smax])
        mine[~valid] = 0
        assert np.array_equal(mine, g[name]), name
    trees = np.array(get("trees")[:, :smax, :])
    trees[~valid] = -1
    trees[:, :, 1:][~g["expanded"]] = -1
    assert np.array_equal(trees, g["trees"])
    assert np.array_equal(get("trees_nodes_selected"), g["trees_nodes_selected"])
    paths, gp = get("trees_selected_paths"), g["trees_selected_paths"]
    for t in range(len(sizes)):
        n = gp[t, -1]
        assert paths[t, -1] == n
        assert np.array_equal(paths[t, :n], gp[t, :n])
    assert np.array_equal(get("trees_actions_expanded"), g["trees_actions_expanded"])
    assert np.array_equal(get("trees_playout_outcomes"), g["trees_playout_outcomes"])
    if "trees_playout_outcomes_children" in g:
        assert np.array_equal(get("trees_playout_outcomes_children"), g["trees_playout_outcomes_children"])


@pytest.mark.parametrize("variant", ["ocp_thrifty", "acp_thrifty"])
def test_oracle_reproduces_reference_dump(golden_dir, variant):
    g = np.load(os.path.join(golden_dir, f"reference_dump_{variant}.npz"))
    o = _run_like_dump(variant)
    check_against_dump(o.field, g)
    # root-action table of the log: ordinal == action here (all seven columns legal at the empty board)
    table = g["root_actions_table"]
    assert np.array_equal(o.field("root_ns"), table[:, 1])
    assert np.array_equal(o.field("actions_win_flags"), table[:, 2])
    assert np.array_equal(o.field("actions_ns"), table[:, 3])
    assert np.array_equal(o.field("actions_ns_wins"), table[:, 4])
    assert o.best_action == int(g["best_index"])
    if variant == "acp_thrifty":
        # the dump contains two draws with u == 1.0f; it is reproduced all the same
        assert o.ub_draws == 2


def test_memory_model_matches_log():
    # "calculated max_tree_size: 4238367" in extras/mctsnc_acp_thrifty_c4_1000steps.log (device_memory=1.5)
    assert reference_max_tree_size((6, 7), 7, 7, 4, "acp_thrifty", 1.5) == 4238367


def test_thrifty_and_prodigal_grow_the_same_trees():
    # src/mctsnc.py:1938 -- the RNG index formula makes both ACP variants equal for equal step counts
    a = OracleMCTSNC((6, 7), 7, 7, n_trees=2, n_playouts=32, variant="acp_thrifty", seed=3, node_capacity=2000)
    b = OracleMCTSNC((6, 7), 7, 7, n_trees=2, n_playouts=32, variant="acp_prodigal", seed=3, node_capacity=2000)
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    a.run(board, fills, -1, 150)
    b.run(board, fills, -1, 150)
    for name in ("trees_sizes", "trees_ns", "trees_ns_wins", "trees", "trees_depths"):
        assert np.array_equal(a.field(name), b.field(name)), name
    assert a.best_action == b.best_action
