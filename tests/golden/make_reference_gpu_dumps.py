"""Runs the reference's numba.cuda ``MCTSNC`` itself on the GPU of this machine (Connect 4 only) and keeps what it
produced: tree dumps for parity tests and its timing on this hardware.

    python baseline/install_reference.py                           # where the reference is mounted
    python tests/golden/make_reference_gpu_dumps.py <output dir>   # on a machine with a GPU

Outputs in <output dir>:
  reference_gpu_dumps.npz    per case the root, the settings and the arrays ``_json_dump`` would write
                             (``src/mctsnc.py:2377-2462``), cut to the nodes in use; copied to ``tests/golden/`` it is
                             the fixture of ``tests/test_reference_gpu_dumps.py``
  reference_gpu_timing.json  playouts/s and steps/s of the reference on the headline configuration (C4 acp_prodigal
                             4 x 256, 2000 steps per root, host-timed the way the reference reports them in
                             ``performance_info``) and of a 1 s time-limited search

Every search is preceded by ``init_device_side_arrays()`` so that its random streams start from the seed
(the reference creates them there, ``src/mctsnc.py:390-394``).  Gomoku is left out on purpose: after a uniform draw equal
to 1.0f the reference's Gomoku playout can loop without end.
"""
import contextlib
import io
import json
import os
import sys
import time

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF_SRC = os.path.join(ROOT, "baseline", "_ref", "src")
sys.path[:0] = [REF_SRC, ROOT]

import numpy as np  # noqa: E402

DUMP_CASES = [
    # name, variant, trees, playouts, steps, index of the root among the benchmark's roots (-1: empty board)
    ("acp_prodigal_4x256_root3", "acp_prodigal", 4, 256, 300, 3),
    ("acp_prodigal_4x256_root101", "acp_prodigal", 4, 256, 300, 101),
    ("acp_thrifty_4x256_root17", "acp_thrifty", 4, 256, 200, 17),
    ("ocp_prodigal_8x256_root40", "ocp_prodigal", 8, 256, 400, 40),
    ("ocp_thrifty_1x32_root7", "ocp_thrifty", 1, 32, 200, 7),
    ("acp_prodigal_4x256_empty_2000", "acp_prodigal", 4, 256, 2000, -1),
]


def quiet(fn, *args, **kwargs):
    with contextlib.redirect_stdout(io.StringIO()):
        return fn(*args, **kwargs)


def dump_arrays(ai):
    sizes = ai.dev_trees_sizes.copy_to_host()
    smax = int(sizes.max())
    out = {"trees_sizes": sizes}
    for name in ("trees", "trees_depths", "trees_turns", "trees_leaves", "trees_terminals", "trees_outcomes", "trees_ns",
                 "trees_ns_wins"):
        out[name] = getattr(ai, "dev_" + name).copy_to_host()[:, :smax].copy()
    for name in ("trees_nodes_selected", "trees_actions_expanded", "trees_playout_outcomes"):
        out[name] = getattr(ai, "dev_" + name).copy_to_host()
    paths = ai.dev_trees_selected_paths.copy_to_host()
    out["trees_selected_paths_head"] = paths[:, :64].copy()
    out["trees_selected_paths_len"] = paths[:, -1].copy()
    if ai.dev_trees_playout_outcomes_children is not None:
        out["trees_playout_outcomes_children"] = ai.dev_trees_playout_outcomes_children.copy_to_host()
    out["root_ns"] = ai.dev_root_ns.copy_to_host()
    out["actions_ns"] = ai.dev_actions_ns.copy_to_host()
    out["actions_ns_wins"] = ai.dev_actions_ns_wins.copy_to_host()
    out["best"] = np.array([int(ai.best_action), int(ai.best_win_flag), int(ai.best_n), int(ai.best_n_wins)], dtype=np.int64)
    return out


def main():
    out_dir = sys.argv[1] if len(sys.argv) > 1 else "."
    os.makedirs(out_dir, exist_ok=True)
    from numba import cuda
    info = {"numba_cuda_available": bool(cuda.is_available())}
    if not info["numba_cuda_available"]:
        raise SystemExit("numba.cuda finds no device")
    import numba
    from mctsnc import MCTSNC                                       # the reference's class (baseline/_ref/src/mctsnc.py)
    import mctsnc as ref_module
    assert os.path.abspath(ref_module.__file__).startswith(os.path.abspath(REF_SRC)), ref_module.__file__
    from mcts_numba_cuda_b200.roots import c4_random_roots
    dev = cuda.get_current_device()
    info.update({"numba": numba.__version__, "device": dev.name.decode() if isinstance(dev.name, bytes) else str(dev.name),
                 "compute_capability": list(dev.compute_capability)})
    boards, fills, turns = c4_random_roots(256, 20, seed=0)          # the benchmark's roots

    def root(i):
        if i < 0:
            return np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1
        return boards[i], fills[i], int(turns[i])

    data = {}
    for name, variant, T, P, steps, idx in DUMP_CASES:
        ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=float(steps), n_trees=T, n_playouts=P,
                    variant=variant, device_memory=0.125, ucb_c=2.0, seed=0, verbose_info=False)
        quiet(ai.init_device_side_arrays)
        b, f, t = root(idx)
        t0 = time.time()
        quiet(ai.run, b, f, t)
        print(f"{name}: {time.time() - t0:.2f} s, best {ai.best_action}, n {ai.best_n}, wins {ai.best_n_wins}", flush=True)
        for k, v in dump_arrays(ai).items():
            data[f"{name}.{k}"] = v
        data[f"{name}.root_board"], data[f"{name}.root_fills"], data[f"{name}.root_turn"] = b, f, np.int8(t)
        data[f"{name}.settings"] = np.array([MCTSNC.VARIANTS.index(variant), T, P, steps, idx], dtype=np.int64)
        del ai
    np.savez_compressed(os.path.join(out_dir, "reference_gpu_dumps.npz"), **data)

    # timing on the headline configuration: 2 GiB of device memory as BASELINE names it
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=2000.0, n_trees=4, n_playouts=256,
                variant="acp_prodigal", device_memory=2.0, ucb_c=2.0, seed=0, verbose_info=True)
    quiet(ai.init_device_side_arrays)
    quiet(ai.run, *root(0))                                            # numba compiles on first use
    rows = []
    for i in range(8):
        quiet(ai.run, *root(i))
        p = ai.performance_info
        rows.append({"root": i, "steps": p["steps"], "playouts": int(p["playouts"]), "playouts_per_second": p["playouts_per_second"],
                     "steps_per_second": p["steps_per_second"], "times_ms": {k: float(v) for k, v in p["times_[ms]"].items()}})
    info["headline_2000_steps"] = {"config": str(ai), "per_root": rows,
                                   "playouts_per_second_mean": float(np.mean([r["playouts_per_second"] for r in rows])),
                                   "steps_per_second_mean": float(np.mean([r["steps_per_second"] for r in rows]))}
    del ai
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=1.0, search_steps_limit=np.inf, n_trees=4, n_playouts=256,
                variant="acp_prodigal", device_memory=2.0, ucb_c=2.0, seed=0, verbose_info=True)
    quiet(ai.init_device_side_arrays)
    quiet(ai.run, *root(-1))
    p = ai.performance_info
    info["time_limited_1s_empty_board"] = {"config": str(ai), "steps": p["steps"], "playouts": int(p["playouts"]),
                                           "playouts_per_second": p["playouts_per_second"]}
    with open(os.path.join(out_dir, "reference_gpu_timing.json"), "w") as f:
        json.dump(info, f, indent=1)
    print(json.dumps(info)[:2000])


if __name__ == "__main__":
    main()
