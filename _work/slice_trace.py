"""Timeline of a batched Connect-4 launch: which tree ran on which block when.

    python -m mcts_numba_cuda_b200.slice_trace [--roots 256] [--trees 4] [--playouts 256] [--steps 2000] [--variant acp_prodigal]

Runs the batch twice (the second run is reported), with the library's slice trace switched on, and prints how well the
work queue packed the launch: the launch's span, the sum of the slices' durations divided by the number of resident
blocks (the span a perfect packing would reach), the busy time of the slowest tree (a tree is sequential: no launch is
shorter than that), and the number of blocks busy over time.
"""
import argparse

import numpy as np

from . import MCTSNC
from .roots import c4_random_roots


def summarise(records, resident, bins=20):
    tree, t0, t1 = records[:, 0], records[:, 1].astype(np.float64), records[:, 2].astype(np.float64)
    start = t0.min()
    t0, t1 = (t0 - start) / 1e6, (t1 - start) / 1e6
    busy = np.zeros(int(tree.max()) + 1)
    np.add.at(busy, tree, t1 - t0)
    span = float(t1.max())
    edges = np.linspace(0.0, span, bins + 1)
    active = [float(np.clip(np.minimum(t1, b) - np.maximum(t0, a), 0, None).sum() / (b - a)) for a, b in zip(edges[:-1], edges[1:])]
    return {"slices": int(len(records)), "span_ms": span, "packing_bound_ms": float(busy.sum() / resident),
            "slowest_tree_ms": float(busy.max()), "median_tree_ms": float(np.median(busy)), "fastest_tree_ms": float(busy.min()),
            "mean_slice_ms": float((t1 - t0).mean()), "blocks_busy": [round(a, 1) for a in active]}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--roots", type=int, default=256)
    ap.add_argument("--trees", type=int, default=4)
    ap.add_argument("--playouts", type=int, default=256)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--variant", default="acp_prodigal")
    args = ap.parse_args()
    boards, fills, turns = c4_random_roots(args.roots, 20, seed=0)
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=args.steps, n_trees=args.trees,
                n_playouts=args.playouts, variant=args.variant, verbose_info=False, max_batch=args.roots)
    ai.init_device_side_arrays()
    slices_per_tree = -(-args.steps // MCTSNC.SLICE_STEPS)
    ai.trace_slices(args.roots * args.trees * slices_per_tree + 16)
    for _ in range(2):
        out = ai.run_batch(boards, fills, turns, steps=args.steps, reseed=True)
    geo = ai.launch_geometry()
    resident = geo["blocks_per_sm"] * geo["sm_count"]
    records = ai.read_slices()
    if len(records) == 0:
        print(f"no slices recorded: {args.roots * args.trees} trees fit on the device at once ({resident} blocks), no queue")
        return
    s = summarise(records, resident)
    print(f"{args.roots} roots x {args.trees} trees, {args.steps} steps, {geo['threads_per_tree']} threads per tree, "
          f"{resident} resident blocks; playouts {int(out['playouts'].sum())}")
    for k, v in s.items():
        print(f"{k}: {v if not isinstance(v, float) else round(v, 3)}")


if __name__ == "__main__":
    main()
