"""Gomoku fixtures made by the reference's OWN kernels, run on the CPU by numba's CUDA simulator.

    python baseline/install_reference.py            # copy of the reference + its mechanics module switched to Gomoku
    python tests/golden/make_gomoku_kernel_fixtures.py [case ...]

The reference ships no Gomoku artefacts (no dumps, its Gomoku match archives are missing), and it has no GPU in the
build container.  numba's simulator (``NUMBA_ENABLE_CUDASIM=1``) executes the kernels as Python threads; it cannot run
``MCTSNC.run()`` (the constructor asks for a device property the simulator lacks, a step takes seconds) and it exposes a
data race of ``_expand_1_*`` that hardware hides (``src/mctsnc.py:1645-1653``: every thread clears its slot of
``shared_legal_actions_child_shifts`` while thread 0 already fills the array, no barrier in between).  So this script
drives the kernels ONE BY ONE, exactly as the host loop ``_run_acp_prodigal`` does (``src/mctsnc.py:1081-1257``), on
arrays shaped like those of ``init_device_side_arrays`` (``:372-404``), for two search steps:

    _reset, then per step: _select, [expand_1: see below], _expand_2_prodigal, _playout_acp_prodigal,
    _backup_1_acp_prodigal, _backup_2_acp; at the end _reduce_over_trees_prodigal and _reduce_over_actions_prodigal.

All of these are the reference's code, unmodified, with the Gomoku device functions of its mechanics module.  Two
things are restated here, both places where the reference relies on the threads of a warp running in program order:
``_expand_1_acp_prodigal`` (``:1607-1681``), in ``host_expand_1`` below (legality = empty cell, child slots in ascending
action order from ``trees_sizes``), and the last lines of ``_select`` (``:1353-1362``), where thread 0 stores the path
entry of a level into shared memory and the other threads copy the path out with no barrier in between: the selected
node the kernel returns (``trees_nodes_selected``, read after a barrier) is kept, and ``host_path`` rebuilds the path as
the chain of parents from that node to the root, which is what the kernel's copy holds on hardware.  The second step's
``_select`` descends one level (root and its children), where the missing barrier between the read of
``shared_best_child[0]`` (``:1352``) and the next level's write (``:1328``) cannot matter.  Streams:
``create_xoroshiro128p_states(T * A * P, seed)`` as ``:394``.

The result, ``tests/golden/gomoku_kernel_fixtures.npz``, holds the inputs and every array after the two steps.
"""
import os
import sys
import time

os.environ["NUMBA_ENABLE_CUDASIM"] = "1"

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
REF = os.path.join(ROOT, "baseline", "_ref")
sys.path[:0] = [os.path.join(REF, "gomoku"), os.path.join(REF, "src")]

import numpy as np  # noqa: E402
from numba import cuda  # noqa: E402
from numba.cuda.random import create_xoroshiro128p_states  # noqa: E402

import mctsnc as ref  # noqa: E402  (the reference's module: baseline/_ref/src/mctsnc.py)

assert os.path.abspath(ref.__file__).startswith(os.path.abspath(REF)), ref.__file__
K = ref.MCTSNC

M = N = 15
A = 225
MAX_TREE_DEPTH = 2048
TPB = {"r": 256, "s": 512, "e2": 256, "b1": 256, "b2": 512, "roa": 256}   # tpb table of src/mctsnc.py:360-370 for 15x15, 225 actions

# name: (trees, playouts, stones on the root board, seed of the root, seed of the search)
CASES = {"late": (2, 32, 160, 5, 0), "middle": (1, 32, 96, 6, 3), "early": (2, 8, 12, 7, 1)}


def random_root(stones, seed):
    """`stones` uniformly random legal moves from the empty board, re-drawn until nobody has five in a row (the
    reference's CPU class ``Gomoku`` decides)."""
    from gomoku import Gomoku
    rng = np.random.default_rng(seed)
    while True:
        g = Gomoku()
        ok = True
        for _ in range(stones):
            empty = np.flatnonzero(g.get_board().reshape(-1) == 0)
            g = g.take_action(int(rng.choice(empty)))
            if g.compute_outcome() is not None:
                ok = False
                break
        if ok:
            return np.array(g.get_board(), dtype=np.int8), int(g.get_turn())


def host_expand_1(max_tree_size, h):
    """``_expand_1_acp_prodigal`` (``src/mctsnc.py:1607-1681``) without its race: what its threads compute when thread 0's
    loop runs after the others have cleared their slots, which is the order hardware gives (one warp, program order)."""
    T = h["trees"].shape[0]
    for ti in range(T):
        sel = int(h["trees_nodes_selected"][ti])
        ae = h["trees_actions_expanded"][ti]
        if h["trees_terminals"][ti, sel]:
            ae[-1], ae[-2] = 1, -1
            ae[:A] = -1
            h["trees"][ti, sel, 1:] = -1
            ae[0] = 0
            continue
        legal = h["trees_boards"][ti, sel].reshape(-1) == 0
        size = int(h["trees_sizes"][ti])
        shift, shifts = -1, np.full(A, -1, np.int16)
        for a in range(A):
            if legal[a] and size + shift + 1 < max_tree_size:
                shift += 1
            shifts[a] = shift
        if shift >= 0:
            ae[-1], ae[-2] = shift + 1, -2
            h["trees_leaves"][ti, sel] = False
        else:
            ae[-1], ae[-2] = 1, -3
        for a in range(A):
            child = -1
            if legal[a] and shifts[a] >= 0:
                child = size + shifts[a]
                ae[a] = a
            else:
                ae[a] = -1
            h["trees"][ti, sel, 1 + a] = child
        h["trees_sizes"][ti] += shifts[A - 1] + 1
        if ae[-2] == -3:
            ae[0] = 0


def host_path(h):
    """``trees_selected_paths`` as ``_select`` leaves it on hardware: root .. selected node, length in the last column."""
    for ti in range(h["trees"].shape[0]):
        node, chain = int(h["trees_nodes_selected"][ti]), []
        while node != -1:
            chain.append(node)
            node = int(h["trees"][ti, node, 0])
        chain.reverse()
        assert chain[0] == 0
        h["trees_selected_paths"][ti, :len(chain)] = chain
        h["trees_selected_paths"][ti, -1] = len(chain)


def run_case(name):
    T, P, stones, root_seed, seed = CASES[name]
    board, turn = random_root(stones, root_seed)
    n_empty = int((board == 0).sum())
    S = 2 * n_empty + 8                           # nodes per tree: two steps create at most 2 * n_empty - 1 children
    ucb_c = np.float32(2.0)
    h = {"trees": np.full((T, S, 1 + A), -1, np.int32), "trees_sizes": np.zeros(T, np.int32),
         "trees_depths": np.zeros((T, S), np.int16), "trees_turns": np.zeros((T, S), np.int8),
         "trees_leaves": np.zeros((T, S), np.bool_), "trees_terminals": np.zeros((T, S), np.bool_),
         "trees_outcomes": np.zeros((T, S), np.int8), "trees_ns": np.zeros((T, S), np.int32),
         "trees_ns_wins": np.zeros((T, S), np.int32), "trees_boards": np.zeros((T, S, M, N), np.int8),
         "trees_extra_infos": np.zeros((T, S, 1), np.int8), "trees_nodes_selected": np.zeros(T, np.int32),
         "trees_selected_paths": np.zeros((T, MAX_TREE_DEPTH + 2), np.int32),
         "trees_actions_expanded": np.zeros((T, A + 2), np.int16), "trees_playout_outcomes": np.zeros((T, 2), np.int32),
         "trees_playout_outcomes_children": np.zeros((T, A, 2), np.int32)}
    d = {k: cuda.to_device(v) for k, v in h.items()}
    gens = create_xoroshiro128p_states(T * A * P, seed=seed)
    K._reset[T, TPB["r"]](cuda.to_device(board), cuda.to_device(np.zeros(1, np.int8)), turn, d["trees"], d["trees_sizes"],
                          d["trees_depths"], d["trees_turns"], d["trees_leaves"], d["trees_terminals"], d["trees_ns"],
                          d["trees_ns_wins"], d["trees_boards"], d["trees_extra_infos"])
    root_actions_expanded = None
    per_step = []
    for step in range(2):
        t0 = time.time()
        K._select[T, TPB["s"]](ucb_c, d["trees"], d["trees_leaves"], d["trees_ns"], d["trees_ns_wins"],
                               d["trees_nodes_selected"], d["trees_selected_paths"])
        for k in h:
            h[k] = d[k].copy_to_host()
        host_path(h)
        host_expand_1(S, h)
        d = {k: cuda.to_device(v) for k, v in h.items()}
        if step == 0:
            root_actions_expanded = h["trees_actions_expanded"][0].copy()
        K._expand_2_prodigal[(T, A), TPB["e2"]](d["trees"], d["trees_depths"], d["trees_turns"], d["trees_leaves"],
                                                d["trees_terminals"], d["trees_outcomes"], d["trees_ns"], d["trees_ns_wins"],
                                                d["trees_boards"], d["trees_extra_infos"], d["trees_nodes_selected"],
                                                d["trees_actions_expanded"])
        K._playout_acp_prodigal[(T, A), P](d["trees"], d["trees_turns"], d["trees_terminals"], d["trees_outcomes"],
                                           d["trees_boards"], d["trees_extra_infos"], d["trees_nodes_selected"],
                                           d["trees_actions_expanded"], gens, d["trees_playout_outcomes"],
                                           d["trees_playout_outcomes_children"])
        K._backup_1_acp_prodigal[T, TPB["b1"]](P, d["trees"], d["trees_turns"], d["trees_ns"], d["trees_ns_wins"],
                                               d["trees_nodes_selected"], d["trees_actions_expanded"],
                                               d["trees_playout_outcomes"], d["trees_playout_outcomes_children"])
        K._backup_2_acp[T, TPB["b2"]](P, d["trees_turns"], d["trees_ns"], d["trees_ns_wins"], d["trees_selected_paths"],
                                      d["trees_actions_expanded"], d["trees_playout_outcomes"])
        per_step.append({k: d[k].copy_to_host() for k in ("trees_nodes_selected", "trees_playout_outcomes",
                                                          "trees_playout_outcomes_children", "trees_sizes")})
        print(f"[{name}] step {step}: {time.time() - t0:.1f} s, sizes {per_step[-1]['trees_sizes']}", flush=True)
    tpb_rot = 1
    while tpb_rot < T:
        tpb_rot *= 2
    out = {"root_ns": np.zeros(A, np.int64), "actions_win_flags": np.zeros(A, np.bool_), "actions_ns": np.zeros(A, np.int64),
           "actions_ns_wins": np.zeros(A, np.int64), "best_action": np.zeros(1, np.int16), "best_win_flag": np.zeros(1, np.bool_),
           "best_n": np.zeros(1, np.int64), "best_n_wins": np.zeros(1, np.int64)}
    o = {k: cuda.to_device(v) for k, v in out.items()}
    K._reduce_over_trees_prodigal[A, tpb_rot](d["trees"], d["trees_terminals"], d["trees_outcomes"], d["trees_ns"],
                                              d["trees_ns_wins"], cuda.to_device(root_actions_expanded), turn, o["root_ns"],
                                              o["actions_win_flags"], o["actions_ns"], o["actions_ns_wins"])
    K._reduce_over_actions_prodigal[1, TPB["roa"]](o["actions_win_flags"], o["actions_ns"], o["actions_ns_wins"],
                                                   o["best_action"], o["best_win_flag"], o["best_n"], o["best_n_wins"])
    res = {f"{name}.{k}": d[k].copy_to_host() for k in h}
    res.update({f"{name}.{k}": o[k].copy_to_host() for k in out})
    for s, snap in enumerate(per_step):
        res.update({f"{name}.step{s}.{k}": v for k, v in snap.items()})
    res.update({f"{name}.root_board": board, f"{name}.root_turn": np.int8(turn), f"{name}.seed": np.int64(seed),
                f"{name}.n_trees": np.int32(T), f"{name}.n_playouts": np.int32(P), f"{name}.max_tree_size": np.int32(S),
                f"{name}.ucb_c": ucb_c, f"{name}.root_actions_expanded": root_actions_expanded})
    return res


def main():
    names = sys.argv[1:] or list(CASES)
    path = os.path.join(HERE, "gomoku_kernel_fixtures.npz")
    data = dict(np.load(path)) if os.path.exists(path) else {}
    for name in names:
        data = {k: v for k, v in data.items() if not k.startswith(name + ".")}
        data.update(run_case(name))
    np.savez_compressed(path, **data)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
