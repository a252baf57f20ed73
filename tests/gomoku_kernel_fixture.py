"""Shared by the CPU and GPU tests: comparison against ``tests/golden/gomoku_kernel_fixtures.npz``, the arrays the
reference's own kernels produced for two Gomoku search steps (made by ``tests/golden/make_gomoku_kernel_fixtures.py`` with
numba's CUDA simulator; see there for what exactly ran).  A searcher under test runs two steps of acp_prodigal from the
same root with the same seed, node limit and exploration constant; everything the reference's kernels wrote must match."""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "golden", "gomoku_kernel_fixtures.npz")
A = 225


def load():
    data = np.load(PATH)
    cases = sorted({k.split(".")[0] for k in data.files})
    return {c: {k[len(c) + 1:]: data[k] for k in data.files if k.startswith(c + ".")} for c in cases}


def settings(case):
    return dict(n_trees=int(case["n_trees"]), n_playouts=int(case["n_playouts"]), seed=int(case["seed"]),
                ucb_c=float(case["ucb_c"]), max_tree_size=int(case["max_tree_size"]), root_board=case["root_board"],
                root_turn=int(case["root_turn"]))


def check(case, field, best):
    """`field(name)` returns the searcher's array in the reference's format (rows of the node arrays at least up to the
    largest tree size); `best` = (best_action, best_win_flag, best_n, best_n_wins)."""
    sizes = case["trees_sizes"]
    assert np.array_equal(field("trees_sizes"), sizes)
    T, smax = len(sizes), int(sizes.max())
    valid = np.arange(smax)[None, :] < sizes[:, None]
    for name in ("trees_depths", "trees_turns", "trees_leaves", "trees_terminals", "trees_ns", "trees_ns_wins"):
        got, want = np.asarray(field(name))[:, :smax], case[name][:, :smax]
        assert np.array_equal(got[valid].astype(np.int64), want[valid].astype(np.int64)), name
    # outcomes: every node but the root (the reference never writes the root's)
    got, want = np.asarray(field("trees_outcomes"))[:, 1:smax], case["trees_outcomes"][:, 1:smax]
    assert np.array_equal(got[valid[:, 1:]], want[valid[:, 1:]])
    got, want = np.asarray(field("trees_boards"))[:, :smax], case["trees_boards"][:, :smax]
    assert np.array_equal(got[valid], want[valid])
    # parent column everywhere, child columns of the nodes that were expanded (the others are never written)
    got, want = np.asarray(field("trees"))[:, :smax], case["trees"][:, :smax]
    assert np.array_equal(got[:, :, 0][valid], want[:, :, 0][valid])
    expanded = valid & (case["trees_leaves"][:, :smax] == 0)
    assert np.array_equal(got[:, :, 1:][expanded], want[:, :, 1:][expanded])
    assert np.array_equal(field("trees_nodes_selected"), case["trees_nodes_selected"])
    assert np.array_equal(field("trees_actions_expanded"), case["trees_actions_expanded"])
    assert np.array_equal(field("trees_playout_outcomes"), case["trees_playout_outcomes"])
    # per-child tallies: rows of the actions played out in the last step (others keep what an earlier step left, which
    # the fixture also holds: the whole array is compared)
    assert np.array_equal(field("trees_playout_outcomes_children"), case["trees_playout_outcomes_children"])
    paths = np.asarray(field("trees_selected_paths"))
    for t in range(T):
        n = int(case["trees_selected_paths"][t, -1])
        assert paths[t, -1] == n and np.array_equal(paths[t, :n], case["trees_selected_paths"][t, :n])
    want_best = (int(case["best_action"][0]), bool(case["best_win_flag"][0]), int(case["best_n"][0]), int(case["best_n_wins"][0]))
    assert (int(best[0]), bool(best[1]), int(best[2]), int(best[3])) == want_best
