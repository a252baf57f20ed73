"""Shared by the CPU and GPU tests: comparison against ``tests/golden/reference_gpu_dumps.npz`` -- what the reference's
own numba.cuda ``MCTSNC`` (``src/mctsnc.py``, unmodified) left in its device arrays after searches on an NVIDIA B200,
recorded by ``tests/golden/make_reference_gpu_dumps.py``: Connect 4, all four variants, 1-8 trees, 32-256 playouts,
positions from the benchmark's root set and the empty board, up to 2000 steps (the headline search).  The arrays are
the ones ``_json_dump`` writes (``src/mctsnc.py:2377-2462``) plus leaves / terminals / outcomes and the final per-action
sums.  The reference allocates its arrays uninitialised (``cuda.device_array``, ``:372-404``): rows at or beyond a tree's
size and the child columns of nodes that were never expanded hold whatever was in memory and are not compared."""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PATH = os.path.join(HERE, "golden", "reference_gpu_dumps.npz")
VARIANTS = ["ocp_thrifty", "ocp_prodigal", "acp_thrifty", "acp_prodigal"]
A = 7


def load():
    data = np.load(PATH)
    names = sorted({k.split(".")[0] for k in data.files})
    return {n: {k[len(n) + 1:]: data[k] for k in data.files if k.startswith(n + ".")} for n in names}


def settings(case):
    variant, trees, playouts, steps, _ = [int(x) for x in case["settings"]]
    return dict(variant=VARIANTS[variant], n_trees=trees, n_playouts=playouts, steps=steps, board=case["root_board"],
                fills=case["root_fills"], turn=int(case["root_turn"]))


def check(case, field, best):
    """`field(name)` gives the searcher's array in the reference's format, node arrays at least up to the largest tree."""
    s = settings(case)
    sizes = case["trees_sizes"]
    assert np.array_equal(field("trees_sizes"), sizes)
    smax = int(sizes.max())
    valid = np.arange(smax)[None, :] < sizes[:, None]
    for name in ("trees_depths", "trees_turns", "trees_leaves", "trees_terminals", "trees_ns", "trees_ns_wins"):
        got, want = np.asarray(field(name))[:, :smax], case[name][:, :smax]
        assert np.array_equal(got[valid].astype(np.int64), want[valid].astype(np.int64)), name
    got, want = np.asarray(field("trees_outcomes"))[:, 1:smax], case["trees_outcomes"][:, 1:smax]
    assert np.array_equal(got[valid[:, 1:]], want[valid[:, 1:]])
    got, want = np.asarray(field("trees"))[:, :smax], case["trees"][:, :smax]
    assert np.array_equal(got[:, :, 0][valid], want[:, :, 0][valid])
    expanded = valid & (case["trees_leaves"][:, :smax] == 0)
    assert np.array_equal(got[:, :, 1:][expanded], want[:, :, 1:][expanded])
    assert np.array_equal(field("trees_nodes_selected"), case["trees_nodes_selected"])
    assert np.array_equal(field("trees_playout_outcomes"), case["trees_playout_outcomes"])
    ae, want_ae = np.asarray(field("trees_actions_expanded")), case["trees_actions_expanded"]
    assert np.array_equal(ae[:, -2:], want_ae[:, -2:])
    if "prodigal" in s["variant"]:
        assert np.array_equal(ae, want_ae)
    else:
        # thrifty layout: the first [-1] entries are the list of this step; the rest is left over from earlier steps in
        # both, and the search started from zeroed / uninitialised memory respectively
        for t in range(len(sizes)):
            n = int(want_ae[t, -1]) if want_ae[t, -2] != -1 else 0
            assert np.array_equal(ae[t, :n], want_ae[t, :n])
    paths = np.asarray(field("trees_selected_paths"))
    for t in range(len(sizes)):
        n = int(case["trees_selected_paths_len"][t])
        assert paths[t, -1] == n and np.array_equal(paths[t, :n], case["trees_selected_paths_head"][t, :n])
    assert (int(best[0]), int(bool(best[1])), int(best[2]), int(best[3])) == tuple(int(x) for x in case["best"])
