"""Turns the two tree dumps the reference ships into compact fixtures.

Reads ``extras/mctsnc_{ocp,acp}_thrifty_c4_1000steps.json`` (written by the reference's ``_json_dump``,
``src/mctsnc.py:2377-2462``, after a fixed 1000-step search from the empty Connect-4 board with n_trees=4,
n_playouts=128, ucb_c=2.0, seed=0) and the root-action tables of the matching ``.log`` files, and writes
``reference_dump_<variant>.npz`` next to this script.  Rows at or beyond ``trees_sizes[t]`` and child columns of
nodes that were never expanded are uninitialised device memory in the dumps; they are masked to -1 / 0 here.

Run once in a checkout that has the reference mounted:  python tests/golden/make_reference_dump_fixtures.py <reference_root>
"""
import ast
import json
import os
import re
import sys

import numpy as np


def main(ref_root):
    here = os.path.dirname(os.path.abspath(__file__))
    for variant in ("ocp_thrifty", "acp_thrifty"):
        with open(os.path.join(ref_root, "extras", f"mctsnc_{variant}_c4_1000steps.json")) as f:
            d = json.load(f)
        sizes = np.array(d["trees_sizes"], dtype=np.int32)
        T, smax = len(sizes), int(sizes.max())
        valid = np.arange(smax)[None, :] < sizes[:, None]
        out = {"trees_sizes": sizes}
        for name, dt in (("trees_depths", np.int16), ("trees_turns", np.int8), ("trees_ns", np.int32),
                         ("trees_ns_wins", np.int32)):
            a = np.array(d[name], dtype=dt)[:, :smax]
            a[~valid] = 0
            out[name] = a
        trees = np.array(d["trees"], dtype=np.int32)[:, :smax, :]
        trees[~valid] = -1
        # a node is expanded iff some valid node names it as parent
        expanded = np.zeros((T, smax), dtype=bool)
        for t in range(T):
            parents = trees[t, 1:sizes[t], 0]
            expanded[t, parents] = True
        children = trees[:, :, 1:]
        children[~expanded] = -1
        out["trees"] = trees
        out["expanded"] = expanded
        out["trees_nodes_selected"] = np.array(d["trees_nodes_selected"], dtype=np.int32)
        paths = np.array(d["trees_selected_paths"], dtype=np.int32)
        lens = paths[:, -1].copy()
        for t in range(T):
            paths[t, lens[t]:-1] = 0
        out["trees_selected_paths"] = paths
        out["trees_actions_expanded"] = np.array(d["trees_actions_expanded"], dtype=np.int16)
        out["trees_playout_outcomes"] = np.array(d["trees_playout_outcomes"], dtype=np.int32)
        if d.get("trees_playout_outcomes_children") is not None:
            out["trees_playout_outcomes_children"] = np.array(d["trees_playout_outcomes_children"], dtype=np.int32)
        # root-action table of the log: action -> (n_root, win_flag, n, n_wins), and the best action
        with open(os.path.join(ref_root, "extras", f"mctsnc_{variant}_c4_1000steps.log")) as f:
            log = f.read()
        rows = []
        for mt in re.finditer(r"^\s+(\d+): (\{.*?\}),?$", log, flags=re.M):
            e = ast.literal_eval(mt.group(2))
            rows.append((int(mt.group(1)), e["n_root"], int(e["win_flag"]), e["n"], e["n_wins"]))
        out["root_actions_table"] = np.array(rows, dtype=np.int64)
        best = re.search(r"best: (\{.*?\})", log)
        out["best_index"] = np.array(ast.literal_eval(best.group(1))["index"], dtype=np.int64)
        out["params"] = np.array([d["n_trees"], d["n_playouts"], int(d["search_steps_limit"]), d["seed"]], dtype=np.int64)
        np.savez_compressed(os.path.join(here, f"reference_dump_{variant}.npz"), **out)
        print(variant, "->", {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + sys.argv[0] + " <root of the reference checkout>")
    main(sys.argv[1])
