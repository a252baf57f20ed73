#!/usr/bin/env python
"""Benchmark of the MCTS-NC search hot path: playouts/s for Connect 4, acp_prodigal, 4 trees x 256 playouts,
2000 search steps per root, 256 seeded random roots per pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" of the benchmark is one pass over the whole batch of roots (every root is searched for `--search-steps`
MCTS steps).  With N > 1 (launched by torchrun, one rank per GPU) every rank grows 4 trees of every search with the
random streams of a 4N-tree search, and the per-root-action sums are all-reduced over NCCL once per pass (root
parallelism; per-GPU work is fixed: weak scaling).  Rank 0 prints one JSON line.

`--impl reference` times the CPU restatement of the reference's kernels (oracle/) on all host cores, one tree per
thread, on a bounded sample of the same workload (same search: 4 trees x 256 playouts x 2000 steps per root; fewer roots).

After the headline's timed regions a single-GPU run appends `secondary`: short device-timed runs of the other
configurations (Connect 4 ocp_thrifty 1 x 32, Gomoku acp_prodigal 4 x 256, the PUCT and DUCT selects) and, where a copy of
the reference lies under baseline/_ref (python baseline/install_reference.py), the reference itself on this machine:
its CPU search `MCTS` on the host cores and its numba.cuda `MCTSNC` on this GPU.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GAMES = {"c4": {"shape": (6, 7), "extra": 7, "actions": 7, "inst_per_ply": 65.0, "name": "Connect-4 6x7"},
         "gomoku": {"shape": (15, 15), "extra": 0, "actions": 225, "inst_per_ply": 100.0, "name": "Gomoku 15x15"}}
# inst_per_ply: thread instructions of one playout ply in a bitboard / row-mask formulation: RNG step ~20, draw -> ordinal 5,
# move pick and placement ~18, line test through the new stone 16 (Connect 4) / ~55 (Gomoku), draw test and loop ~6.
# It is the yardstick of the issue roofline, not a count of the compiled code.

KERNEL_SOURCES = {"c4": ("c4_search.cuh", "common.cuh", "rng.cuh"), "gomoku": ("gomoku_search.cuh", "common.cuh", "rng.cuh")}


def kernel_source_sha(game):
    """Identifies the kernel a profile was taken on: hash of the sources the search kernel of `game` is compiled from."""
    import hashlib
    h = hashlib.sha256()
    for name in KERNEL_SOURCES[game]:
        with open(os.path.join(ROOT, "mcts_numba_cuda_b200", "csrc", name), "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def profiler_readings(game, workload_key):
    """Figures read off ncu captures (profiles/search_kernel_ncu.json: DRAM traffic per launch, pipe and issue
    utilisation, lanes per instruction).  They describe the kernel they were captured on: when the kernel sources have
    changed since, or the workload is another one, the answer is None and the bench line carries nulls."""
    path = os.path.join(ROOT, "profiles", "search_kernel_ncu.json")
    if not os.path.exists(path):
        return None
    with open(path) as f:
        entries = json.load(f)
    for e in entries:
        if e.get("game") == game and e.get("kernel_source_sha") == kernel_source_sha(game) and e.get("workload_key") == workload_key:
            return e
    return None


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="search", choices=["search", "puct", "duct"],
                    help="search: the MCTS-NC search (headline); puct: the warp-level PUCT select (BASELINE config 5)")
    ap.add_argument("--puct-trees", type=int, default=4096)
    ap.add_argument("--puct-edges", type=int, default=64)
    ap.add_argument("--puct-depth", type=int, default=16)
    ap.add_argument("--puct-warps", type=int, default=8)
    ap.add_argument("--puct-virtual-loss", type=int, default=3)
    ap.add_argument("--duct-actions", type=int, default=8, help="actions per player of the decoupled-UCT workload")
    ap.add_argument("--game", default="c4", choices=sorted(GAMES))
    ap.add_argument("--roots", type=int, default=256)
    ap.add_argument("--search-steps", type=int, default=2000)
    ap.add_argument("--trees", type=int, default=4)
    ap.add_argument("--playouts", type=int, default=256)
    ap.add_argument("--variant", default="acp_prodigal")
    ap.add_argument("--max-plies", type=int, default=20)
    ap.add_argument("--threads-per-tree", type=int, default=0)
    ap.add_argument("--cpu-sample-roots", type=int, default=0, help="roots of the CPU baseline sample (0 = choose)")
    ap.add_argument("--cpu-sample-steps", type=int, default=0, help="search steps of the CPU legs (0 = reference arm: the workload's; cpu_baseline leg: 400)")
    ap.add_argument("--internal", default="", help=argparse.SUPPRESS)
    ap.add_argument("--no-secondary", action="store_true", help="skip the secondary configurations and the reference's own runs")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--exchange", default="nccl", choices=["nccl", "peer"],
                    help="multi-GPU exchange of the per-action sums: NCCL all-reduce, or the library's own peer stores and flags")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "sm_max_mhz": float(p.get("sm_max_mhz", 1965.0)), "source": "measured"}
    return {"hbm_gbs": 6650.0, "sm_max_mhz": 1965.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                smax.append(float(r[2]))
            except ValueError:
                continue
            for name, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_roots(args):
    from mcts_numba_cuda_b200.roots import c4_random_roots, gomoku_random_roots
    if args.game == "gomoku":
        boards, turns = gomoku_random_roots(args.roots, args.max_plies, seed=0)
        return boards, None, turns
    return c4_random_roots(args.roots, args.max_plies, seed=0)


def oracle_tree_search(job):
    """One tree of one root's search with the oracle: tree `tree` of a search with `trees` trees (its random streams are
    those of that tree in the whole search, so the trees of a root together are exactly the root's search)."""
    from oracle.oracle import OracleMCTSNC
    board, fills, turn, trees, tree, playouts, variant, steps, game = job
    G = GAMES[game]
    o = OracleMCTSNC(G["shape"], G["extra"], G["actions"], n_trees=1, n_playouts=playouts, variant=variant, seed=0,
                     device_memory=16.0 if game == "gomoku" else 2.0, node_capacity=steps * G["actions"] + G["actions"] + 8,
                     tree_offset=tree, n_trees_global=trees)
    o.run(board, fills, int(turn), steps)
    return o.playouts, o.plies


def cpu_port_baseline(args, boards, fills, turns, threads, n_roots, steps):
    """The oracle (CPU restatement of the reference's kernels) on `threads` host threads, one tree of one root per
    thread at a time (the ctypes calls release the interpreter lock).  Returns (playouts, plies, seconds)."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as om
    om.lib()
    jobs = [(boards[i % len(boards)], fills[i % len(boards)] if fills is not None else None, turns[i % len(boards)],
             args.trees, t, args.playouts, args.variant, steps, args.game) for i in range(n_roots) for t in range(args.trees)]
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        res = list(ex.map(oracle_tree_search, jobs))
    wall = time.perf_counter() - t0
    return sum(r[0] for r in res), sum(r[1] for r in res), wall


def config_dict(args, n_gpus, roots=None):
    roots = args.roots if roots is None else roots
    return {"workload": f"{GAMES[args.game]['name']} {args.variant}, n_trees={args.trees} per GPU, n_playouts={args.playouts}, "
                        f"search_steps={args.search_steps}, {roots} seeded random roots (0..{args.max_plies} plies) per pass",
            "trees_per_search_total": args.trees * n_gpus, "parallelism": f"root-parallel x{n_gpus}" if n_gpus > 1 else "single GPU",
            "l2": "no flush: the tree pools of one pass (~0.5 GB) exceed the 126 MB L2", "seed": 0, "ucb_c": 2.0}


def run_reference(args, rank):
    """The reference arm: the CPU restatement of the reference's kernels on every host core.  A pass searches as many of
    the benchmark's roots as keep all cores busy with one tree each (cores / trees roots), with the full step count."""
    if rank != 0:
        return
    boards, fills, turns = make_roots(args)
    cores = os.cpu_count() or 1
    steps = args.cpu_sample_steps or args.search_steps
    n_roots = args.cpu_sample_roots or max(1, cores // args.trees)
    times, total_playouts = [], 0
    for i in range(args.warmup + args.steps):
        # warm-up passes only have to touch the code and the allocator: a tenth of the steps
        playouts, plies, wall = cpu_port_baseline(args, boards, fills, turns, cores, n_roots, steps if i >= args.warmup else max(steps // 10, 1))
        if i >= args.warmup:
            times.append(wall)
            total_playouts += playouts
    value = total_playouts / sum(times)
    sample = (f"{n_roots} of the {args.roots} roots x {steps} search steps per pass (the same search per root as the GPU arm), "
              f"one tree per thread on {cores} threads; warm-up passes run a tenth of the steps")
    cfg = config_dict(args, args.gpus, roots=n_roots)
    cfg["search_steps"] = steps
    print(json.dumps({"impl": "reference", "metric": "playouts/sec", "value": value, "unit": "playouts/s", "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32",
                      "data": "synthetic", "config": cfg,
                      "cpu_baseline": {"value": value, "unit": "playouts/s", "cores": cores, "kind": "port", "sample": sample},
                      "e2e": {"value": value, "unit": "playouts/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


REF_SRC = os.path.join(ROOT, "baseline", "_ref", "src")


def _reference_state(board, fills, turn):
    """A state object of the reference's own class ``C4`` (``src/c4.py``) holding the given position."""
    from c4 import C4
    s = C4()
    s.board[:] = board
    s.column_fills[:] = fills
    s.turn = int(turn)
    return s


def _reference_mcts_one(job):
    """One search of the reference's CPU class ``MCTS`` (``src/mcts.py:482-588``; one playout per step)."""
    import contextlib
    import io
    board, fills, turn, steps = job
    if REF_SRC not in sys.path:
        sys.path.insert(0, REF_SRC)
    from mcts import MCTS
    ai = MCTS(search_time_limit=np.inf, search_steps_limit=steps, vanilla=True, verbose_info=False)
    root = _reference_state(board, fills, turn)
    t0 = time.perf_counter()
    with contextlib.redirect_stdout(io.StringIO()):
        ai.run(root)
    return ai.steps, time.perf_counter() - t0


def internal_reference_mcts(args):
    """Child process: the reference's ``MCTS`` on one core, then one search per core on all cores at once."""
    import multiprocessing as mp
    boards, fills, turns = make_roots(args)
    steps = args.search_steps
    _reference_mcts_one((boards[0], fills[0], turns[0], 200))               # numba compiles the outcome function on first use
    one = [_reference_mcts_one((boards[i], fills[i], turns[i], steps)) for i in range(3)]
    cores = os.cpu_count() or 1
    jobs = [(boards[i % len(boards)], fills[i % len(boards)], turns[i % len(boards)], steps) for i in range(cores)]
    t0 = time.perf_counter()
    with mp.get_context("fork").Pool(cores) as pool:
        pool.map(_reference_mcts_one, jobs[:cores])                           # untimed: every worker compiles
        t0 = time.perf_counter()
        res = pool.map(_reference_mcts_one, jobs)
    wall = time.perf_counter() - t0
    print(json.dumps({"what": "reference src/mcts.py MCTS(vanilla=True), one playout per step", "search_steps": steps,
                      "one_core": {"value": sum(r[0] for r in one) / sum(r[1] for r in one), "unit": "playouts/s", "cores": 1,
                                   "sample": f"3 roots x {steps} steps, sequential"},
                      "all_cores": {"value": sum(r[0] for r in res) / wall, "unit": "playouts/s", "cores": cores,
                                    "sample": f"{cores} roots x {steps} steps, one process per core"}}))


def internal_reference_numba(args):
    """Child process: the reference's numba.cuda ``MCTSNC`` (``src/mctsnc.py``), unmodified, on this machine's GPU for the
    benchmark's configuration; a fresh ``init_device_side_arrays()`` per root, timing as the reference reports it in
    ``performance_info`` (host clock around its whole ``run``)."""
    import contextlib
    import io
    sys.path.insert(0, REF_SRC)
    from mctsnc import MCTSNC
    boards, fills, turns = make_roots(args)
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=float(args.search_steps), n_trees=args.trees,
                n_playouts=args.playouts, variant=args.variant, device_memory=2.0, ucb_c=2.0, seed=0, verbose_info=True)
    rows = []
    with contextlib.redirect_stdout(io.StringIO()):
        ai.init_device_side_arrays()
        ai.run(boards[0], fills[0], int(turns[0]))                            # first use
        for i in range(args.roots):
            ai.init_device_side_arrays()
            ai.run(boards[i], fills[i], int(turns[i]))
            p = ai.performance_info
            rows.append((int(p["playouts"]), float(p["times_[ms]"]["total"]), int(p["steps"]), int(ai.best_action), int(ai.best_n),
                         int(ai.best_n_wins)))
    total_s = sum(r[1] for r in rows) * 1e-3
    print(json.dumps({"what": "reference src/mctsnc.py MCTSNC (numba.cuda), host-timed per run() as its performance_info does",
                      "config": str(ai), "value": sum(r[0] for r in rows) / total_s, "unit": "playouts/s",
                      "steps_per_second": sum(r[2] for r in rows) / total_s, "roots": len(rows),
                      "best": [[r[3], r[4], r[5]] for r in rows]}))


def run_child(mode, args, extra, timeout):
    """Runs this file again as a child process in one of its internal modes and returns the JSON it prints."""
    cmd = [sys.executable, os.path.abspath(__file__), "--internal", mode, "--game", args.game, "--variant", args.variant,
           "--trees", str(args.trees), "--playouts", str(args.playouts), "--search-steps", str(args.search_steps),
           "--max-plies", str(args.max_plies)] + extra
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout)
    except subprocess.TimeoutExpired:
        return {"unavailable": f"no answer within {timeout} s"}
    lines = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
    if res.returncode != 0 or not lines:
        tail = (res.stderr or res.stdout).strip().splitlines()[-1:] or [""]
        return {"unavailable": f"exit code {res.returncode}: {tail[0][:200]}"}
    return json.loads(lines[-1])


def puct_device_case(trees, edges, depth, warps, seed, device):
    """The layered workload of oracle.puct_oracle.layered_case, generated on the device (4096 x 1025 x 64 edges would
    take minutes and gigabytes on the host): level l+1 holds `edges` nodes shared by the nodes of level l, the last level
    is terminal; priors ~ Dirichlet(0.3), visit counts ~ U{0..49}, W = N * U[-1, 1]."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    per = edges
    nodes = 1 + per * depth
    level_of = torch.zeros(nodes, dtype=torch.long, device=device)
    level_of[1:] = (torch.arange(nodes - 1, device=device) // per) + 1
    idx_in_level = torch.zeros(nodes, dtype=torch.long, device=device)
    idx_in_level[1:] = torch.arange(nodes - 1, device=device) % per
    nxt = 1 + per * level_of[:, None] + (torch.arange(edges, device=device)[None, :] + idx_in_level[:, None]) % per
    expanded = torch.full((nodes,), edges, dtype=torch.int32, device=device)
    expanded[level_of == depth] = -1
    nxt[level_of == depth] = -1
    gamma = torch._standard_gamma(torch.full((trees, nodes, edges), 0.3, device=device), generator=g)
    prior = (gamma / gamma.sum(dim=2, keepdim=True).clamp_min(1e-30)).float()
    n = torch.randint(0, 50, (trees, nodes, edges), device=device, generator=g, dtype=torch.int32)
    w = n.float() * (torch.rand((trees, nodes, edges), device=device, generator=g) * 2 - 1)
    return {"edge_child": nxt.to(torch.int32)[None].expand(trees, -1, -1).contiguous(), "edge_prior": prior.contiguous(),
            "edge_w": w.contiguous(), "edge_n": n.contiguous(),
            "edge_inflight": torch.zeros((trees, nodes, edges), dtype=torch.int32, device=device),
            "node_expand_inflight": torch.zeros((trees, nodes), dtype=torch.int32, device=device),
            "node_expanded": expanded[None].expand(trees, -1).contiguous(),
            "node_count": torch.full((trees,), nodes, dtype=torch.int32, device=device),
            "out_selected": torch.zeros((trees, warps), dtype=torch.int32, device=device),
            "out_path": torch.full((trees, warps, depth), -1, dtype=torch.int32, device=device),
            "out_len": torch.zeros((trees, warps), dtype=torch.int32, device=device), "trees": trees, "warps": warps}


def run_puct(args):
    """Select-only timing as the reference's own benchmark does it (src/puct/test_puct_gpu_v3.py:632-650): CUDA events
    around the select launch, an untimed release after each; sel/s = trees * warps / mean select time."""
    import ctypes
    import torch
    from mcts_numba_cuda_b200 import _abi, puct
    _abi.lib()
    dev = "cuda:0"
    T, E, D, Wp, vl = args.puct_trees, args.puct_edges, args.puct_depth, args.puct_warps, args.puct_virtual_loss
    d = puct_device_case(T, E, D, Wp, 0, dev)
    pk = peaks()

    def timed(select):
        times = []
        for i in range(args.warmup + args.steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            select()
            e1.record()
            torch.cuda.synchronize()
            valid = int((((d["out_selected"] >> 22) & 7) != 4).sum())
            puct.launch_release(d, virtual_loss=release_vl[0])
            torch.cuda.synchronize()
            if i >= args.warmup:
                times.append(e0.elapsed_time(e1))
        assert int(d["edge_inflight"].abs().sum()) == 0
        return float(np.mean(times)), valid

    release_vl = [vl]
    sampler = ClockSampler(0)
    sampler.start()
    ms, valid = timed(lambda: puct.launch_select(d, cpuct=1.5, c_pw=0.0, virtual_loss=vl))
    release_vl[0] = 1
    ms_vl1, valid1 = timed(lambda: puct.launch_select(d, cpuct=1.5, c_pw=0.0, virtual_loss=1))
    ref_ms = None
    ref_path = os.path.join(ROOT, "oracle", "_ref", "libpuct_ref_sm100a.so")
    if os.path.exists(ref_path):
        lib = ctypes.CDLL(ref_path)
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.puct_select_winner_recalc_launch.argtypes = [f32, f32, f32, i32] + [vp] * 11 + [i32] * 5 + [vp]
        ptrs = [ctypes.c_void_p(d[k].data_ptr()) for k in ("edge_child", "edge_prior", "edge_w", "edge_n", "edge_inflight",
                                                            "node_expand_inflight", "node_expanded", "node_count",
                                                            "out_selected", "out_path", "out_len")]
        nodes = d["edge_child"].shape[1]
        ref_ms, _ = timed(lambda: lib.puct_select_winner_recalc_launch(1.5, 0.0, 0.5, 0, *ptrs, T, nodes, E, Wp, D,
                                                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    clocks = sampler.stop()
    sel = T * Wp
    bytes_per_sel = D * (16 * E + 16)          # prior, W, N, inflight per edge + node record, child id, path entry, ticket
    achieved = sel * bytes_per_sel / (ms * 1e-3) / 1e9
    line = {"metric": "PUCT selections/sec (select kernel only, CUDA events)", "value": sel / (ms * 1e-3), "unit": "selections/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"PUCT warp-level select: {T} trees x {E} edges, layered depth {D}, {Wp} warps per tree, "
                                   f"virtual loss {vl}, c_puct 1.5, priors ~ Dirichlet(0.3)",
                       "l2": f"edge arrays {5 * 4 * T * (1 + E * D) * E / 1e9:.1f} GB exceed the 126 MB L2"},
            "valid_selections": valid, "virtual_loss_1": {"value": sel / (ms_vl1 * 1e-3), "ms": ms_vl1, "valid": valid1},
            "reference_kernel": None if ref_ms is None else {"value": sel / (ref_ms * 1e-3), "ms": ref_ms,
                                                             "what": "src/puct/puct_gpu_v3_cpp.cu built for sm_100a, virtual loss 1"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                         "kernel": "puct::select_kernel", "bytes_per_selection": bytes_per_sel},
            "gpu_launches": 2 * (args.steps + args.warmup) * 2, "clocks": clocks}
    return line


def duct_device_case(trees, actions, depth, warps, seed, device):
    """Layered trees for the decoupled-UCT select, generated on the device: level l+1 holds A*A nodes shared by the nodes
    of level l (child of joint action j of the i-th node of a level = node (i + j) % (A*A) of the next), the last level is
    terminal; priors ~ Dirichlet(0.3) per player, joint visit counts ~ U{0..49} and joint value sums N * U[-1, 1], from
    which the per-player marginals are summed (player 1's value sums are the negatives)."""
    import torch
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    A, per = actions, actions * actions
    nodes = 1 + per * depth
    level_of = torch.zeros(nodes, dtype=torch.long, device=device)
    level_of[1:] = (torch.arange(nodes - 1, device=device) // per) + 1
    idx_in_level = torch.zeros(nodes, dtype=torch.long, device=device)
    idx_in_level[1:] = torch.arange(nodes - 1, device=device) % per
    nxt = 1 + per * level_of[:, None] + (torch.arange(per, device=device)[None, :] + idx_in_level[:, None]) % per
    nxt[level_of == depth] = -1
    gamma = torch._standard_gamma(torch.full((trees, nodes, 2, A), 0.3, device=device), generator=g)
    prior = (gamma / gamma.sum(dim=3, keepdim=True).clamp_min(1e-30)).float()
    nj = torch.randint(0, 50, (trees, nodes, A, A), device=device, generator=g, dtype=torch.int32)
    wj = nj.float() * (torch.rand((trees, nodes, A, A), device=device, generator=g) * 2 - 1)
    node_n = torch.stack([nj.sum(dim=3), nj.sum(dim=2)], dim=2).to(torch.int32)
    node_w = torch.stack([wj.sum(dim=3), -wj.sum(dim=2)], dim=2).float()
    terminal = (level_of == depth).to(torch.int32)
    return {"child": nxt.to(torch.int32)[None].expand(trees, -1, -1).contiguous(), "node_prior": prior.contiguous(),
            "node_w": node_w.contiguous(), "node_n": node_n.contiguous(),
            "node_inflight": torch.zeros((trees, nodes, 2, A), dtype=torch.int32, device=device),
            "node_terminal": terminal[None].expand(trees, -1).contiguous(),
            "node_count": torch.full((trees,), nodes, dtype=torch.int32, device=device),
            "out_selected": torch.zeros((trees, warps), dtype=torch.int32, device=device),
            "out_path": torch.full((trees, warps, depth + 1), -1, dtype=torch.int32, device=device),
            "out_len": torch.zeros((trees, warps), dtype=torch.int32, device=device), "trees": trees, "warps": warps}


def run_duct(args):
    """Decoupled-UCT select for 2 players x A actions (no counterpart in the reference; the specification is the one of
    include/duct_b200.h): select-only timing as for PUCT, an untimed release after each launch; the CPU baseline is the
    numpy restatement on a sample of the same trees."""
    import torch
    from mcts_numba_cuda_b200 import _abi, duct
    from mcts_numba_cuda_b200.puct import to_host
    _abi.lib()
    dev = "cuda:0"
    T, A, D, Wp, vl = args.puct_trees, args.duct_actions, args.puct_depth, args.puct_warps, args.puct_virtual_loss
    d = duct_device_case(T, A, D, Wp, 0, dev)
    pk = peaks()
    sampler = ClockSampler(0)
    sampler.start()
    times = []
    for i in range(args.warmup + args.steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        duct.launch_select(d, cpuct=1.5, virtual_loss=vl)
        e1.record()
        torch.cuda.synchronize()
        kinds = (d["out_selected"] >> 22) & 7
        mean_len = float(d["out_len"].float().mean())
        duct.launch_backup(d, None, None, virtual_loss=vl)
        torch.cuda.synchronize()
        if i >= args.warmup:
            times.append(e0.elapsed_time(e1))
    assert int(d["node_inflight"].abs().sum()) == 0
    clocks = sampler.stop()
    ms = float(np.mean(times))
    sel = T * Wp
    cpu = None
    if not args.no_cpu_baseline:
        from oracle import duct_oracle as do
        sample = min(T, 1024)
        h = {k: (v[:sample].cpu().numpy() if hasattr(v, "cpu") else v) for k, v in d.items()}
        h["trees"] = sample
        t0 = time.perf_counter()
        do.select(h, cpuct=1.5, virtual_loss=vl)
        dt = time.perf_counter() - t0
        cpu = {"value": sample * Wp / dt, "unit": "selections/s", "cores": 1, "kind": "port",
               "sample": f"{sample} of the {T} trees x {Wp} warps, sequential numpy restatement, {dt:.1f} s"}
    bytes_per_sel = mean_len * (2 * A * 16 + A * A * 4 + 4) + 16
    achieved = sel * bytes_per_sel / (ms * 1e-3) / 1e9
    line = {"metric": "DUCT selections/sec (select kernel only, CUDA events)", "value": sel / (ms * 1e-3), "unit": "selections/s",
            "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"decoupled-UCT select, 2 players x {A} actions: {T} trees, layered depth {D}, {Wp} warps per "
                                   f"tree, virtual loss {vl}, c_puct 1.5, priors ~ Dirichlet(0.3); no counterpart in the reference",
                       "l2": f"node arrays {T * (1 + A * A * D) * (2 * A * 16 + A * A * 4) / 1e9:.1f} GB exceed the 126 MB L2"},
            "mean_path_length": mean_len, "busy_fraction": float((kinds == 4).float().mean()),
            "e2e": {"value": sel / (ms * 1e-3), "unit": "selections/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0,
                    "note": "trees live on the device; a select has no host input"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / pk["hbm_gbs"],
                         "traffic": sel * 10584.0 if (A, D, Wp) == (8, 16, 8) else None,
                         "traffic_unit": "bytes per launch, scaled by traversals from an ncu capture of 1024 trees (10.6 KB each)",
                         "peak_source": pk["source"], "kernel": "duct::select_kernel", "bytes_per_selection": bytes_per_sel},
            "cpu_baseline": cpu, "gpu_launches": 2 * (args.steps + args.warmup), "clocks": clocks}
    return line


def timed_search(game, variant, trees, playouts, steps, roots, max_plies, passes, device):
    """Device-timed playouts/s of one search configuration: roots resident on the device, streams re-seeded every pass,
    CUDA events around `passes` passes after one warm-up pass."""
    import torch
    from mcts_numba_cuda_b200.distributed import RootParallelMCTSNC
    from mcts_numba_cuda_b200.roots import c4_random_roots, gomoku_random_roots
    G = GAMES[game]
    if game == "gomoku":
        boards, turns = gomoku_random_roots(roots, max_plies, seed=0)
        fills = None
    else:
        boards, fills, turns = c4_random_roots(roots, max_plies, seed=0)
    s = RootParallelMCTSNC(G["shape"], G["extra"], G["actions"], n_trees=trees, n_playouts=playouts, variant=variant,
                           search_steps_limit=steps, max_batch=roots, device=device, rank=0, world_size=1, seed=0, ucb_c=2.0,
                           device_memory=16.0 if game == "gomoku" else 2.0)
    s.search_async(boards, fills, turns, steps, reseed=True)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(passes):
        s.search_async(None, None, None, steps, reseed=True)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / passes
    res = s.fetch(roots)
    playouts_pass, plies_pass = int(res["playouts"].sum()), int(res["plies"].sum())
    geo = s.local.launch_geometry()
    peak_inst = geo["sm_count"] * 4 * 32 * peaks()["sm_max_mhz"] * 1e6
    return {"workload": f"{G['name']} {variant}, n_trees={trees}, n_playouts={playouts}, search_steps={steps}, {roots} roots "
                        f"(0..{max_plies} plies)", "value": playouts_pass / (ms * 1e-3), "unit": "playouts/s", "ms_per_pass": ms,
            "passes": passes, "plies_per_playout": plies_pass / max(playouts_pass, 1), "status_bits": int(np.bitwise_or.reduce(res["status"])),
            "issue_frac": plies_pass * G["inst_per_ply"] / (ms * 1e-3) / peak_inst, "threads_per_tree": geo["threads_per_tree"]}


def secondary_runs(args, device):
    """Short runs of the other configurations, and the reference itself where a copy of it is installed; every entry
    stands alone (a failure is recorded in its place)."""
    import copy
    out = {}

    def attempt(name, fn):
        try:
            out[name] = fn()
        except Exception as e:  # noqa: BLE001 - a secondary figure must not take the headline down
            out[name] = {"error": f"{type(e).__name__}: {e}"[:300]}

    attempt("c4_ocp_thrifty_1x32_200steps_64roots", lambda: timed_search("c4", "ocp_thrifty", 1, 32, 200, 64, 10, 5, device))
    attempt("c4_ocp_prodigal_8x128_1000steps_256roots", lambda: timed_search("c4", "ocp_prodigal", 8, 128, 1000, 256, 20, 2, device))
    attempt("gomoku_acp_prodigal_4x256_500steps_1root", lambda: timed_search("gomoku", "acp_prodigal", 4, 256, 500, 1, 30, 2, device))
    attempt("gomoku_acp_prodigal_4x256_500steps_8roots", lambda: timed_search("gomoku", "acp_prodigal", 4, 256, 500, 8, 30, 1, device))
    attempt("single_search_c4_acp_prodigal_4x256_2000steps", lambda: timed_search("c4", "acp_prodigal", 4, 256, 2000, 1, 0, 3, device))
    attempt("four_searches_c4_acp_prodigal_4x256_2000steps", lambda: timed_search("c4", "acp_prodigal", 4, 256, 2000, 4, 20, 3, device))
    for warps in (8, 1):
        a = copy.copy(args)
        a.puct_warps, a.steps, a.warmup = warps, 5, 3

        def puct(a=a):
            line = run_puct(a)
            return {k: line[k] for k in ("value", "unit", "ms_per_step", "config", "valid_selections", "virtual_loss_1",
                                         "reference_kernel", "roofline")}
        attempt(f"puct_select_{warps}_warps", puct)
    a = copy.copy(args)
    a.steps, a.warmup, a.no_cpu_baseline = 5, 3, True
    attempt("duct_select_8_warps", lambda: {k: v for k, v in run_duct(a).items() if k in ("value", "unit", "ms_per_step", "config", "mean_path_length", "busy_fraction", "roofline")})
    if os.path.exists(os.path.join(REF_SRC, "mctsnc.py")):
        out["reference_cpu_mcts"] = run_child("reference-mcts", args, ["--roots", str(args.roots)], 300)
        out["reference_numba_cuda_on_this_gpu"] = run_child("reference-numba", args, ["--roots", "4"], 420)
    else:
        why = {"unavailable": "no copy of the reference under baseline/_ref (python baseline/install_reference.py)"}
        out["reference_cpu_mcts"], out["reference_numba_cuda_on_this_gpu"] = why, why
    return out


def multi_gpu_parity(args, searcher, boards, fills, turns, rank, world, local_rank):
    """Root-parallel result against one GPU growing all the trees: every rank searches 4 roots for 100 steps with its own
    shard of the world * n_trees trees; rank 0 then grows all world * n_trees trees itself and compares the all-reduced
    sums and the chosen action.  Outside every timed region."""
    from mcts_numba_cuda_b200 import MCTSNC
    G = GAMES[args.game]
    A, roots, steps = G["actions"], 4, 100
    got = searcher.run_batch(boards[:roots], None if fills is None else fills[:roots], turns[:roots], steps, reseed=True)
    if rank != 0:
        return None
    whole = MCTSNC(G["shape"], G["extra"], A, search_time_limit=np.inf, search_steps_limit=steps, n_trees=args.trees * world,
                   n_playouts=args.playouts, variant=args.variant, verbose_info=False, device=local_rank, max_batch=roots, seed=0,
                   ucb_c=2.0, device_memory=16.0 if args.game == "gomoku" else 2.0)
    whole.init_device_side_arrays()
    want = whole.run_batch(boards[:roots], None if fills is None else fills[:roots], turns[:roots], steps, reseed=True)
    same = all(np.array_equal(got[k][:, :A] if got[k].ndim > 1 else got[k], want[k][:, :A] if want[k].ndim > 1 else want[k])
               for k in ("root_ns", "actions_ns", "actions_ns_wins", "best_action", "best_n", "best_n_wins", "best_win_flag"))
    return bool(same)


def main():
    args = parse_args()
    if args.internal == "reference-mcts":
        internal_reference_mcts(args)
        return
    if args.internal == "reference-numba":
        internal_reference_numba(args)
        return
    if args.workload == "puct":
        print(json.dumps(run_puct(args)))
        return
    if args.workload == "duct":
        print(json.dumps(run_duct(args)))
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    import torch
    import torch.distributed as dist
    from mcts_numba_cuda_b200 import _abi
    from mcts_numba_cuda_b200.distributed import RootParallelMCTSNC
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the search has no CPU path")
    _abi.lib()  # fails loudly if the extension was not built
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group(backend="nccl", device_id=torch.device(f"cuda:{local_rank}"))
    n_gpus = world
    boards, fills, turns = make_roots(args)
    B = args.roots
    G = GAMES[args.game]
    A = G["actions"]
    searcher = RootParallelMCTSNC(G["shape"], G["extra"], A, n_trees=args.trees, n_playouts=args.playouts, variant=args.variant,
                                  search_steps_limit=args.search_steps, max_batch=B, device=local_rank, rank=rank,
                                  world_size=world, seed=0, ucb_c=2.0, threads_per_tree=args.threads_per_tree,
                                  device_memory=16.0 if args.game == "gomoku" else 2.0, exchange=args.exchange)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---------------------------------------------------------------- device-resident passes (value, roofline)
    searcher.search_async(boards, fills, turns, args.search_steps, reseed=True)  # stages the roots once
    torch.cuda.synchronize()
    for _ in range(max(args.warmup - 1, 0)):
        searcher.search_async(None, None, None, args.search_steps, reseed=True)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for k in range(args.steps):
        searcher.search_async(None, None, None, args.search_steps, reseed=True)
    searcher.drain()      # the exchange of the last pass (all-reduce + argmax) is part of the timed region
    ev1.record()
    barrier()
    dev_ms = ev0.elapsed_time(ev1)
    res = searcher.fetch(B)
    local_playouts = int(res["playouts"].sum())   # this rank's trees
    local_plies = int(res["plies"].sum())
    kernel_ms = float(res["device_ms"][0])         # search kernel of the last pass (CUDA events inside the library)
    status = int(np.bitwise_or.reduce(res["status"]))
    ub_draws = int(res["ub_draws"].sum())
    # ---------------------------------------------------------------- end-to-end passes through the public API
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = searcher.run_batch(boards, fills, turns, args.search_steps, reseed=True)
    barrier()
    e2e_s = time.perf_counter() - t0
    clocks = sampler.stop() if rank == 0 else None
    geo = searcher.local.launch_geometry()   # of the timed launches (the parity check below launches a smaller search)
    parity = multi_gpu_parity(args, searcher, boards, fills, turns, rank, world, local_rank) if world > 1 else None
    exchange_status = searcher.exchange_status()
    # max over ranks of the timed regions, sums of the work
    stats = torch.tensor([dev_ms, e2e_s * 1e3, kernel_ms], dtype=torch.float64, device="cuda")
    work = torch.tensor([local_playouts, local_plies], dtype=torch.int64, device="cuda")
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(work, op=dist.ReduceOp.SUM)
    dev_ms, e2e_ms, kernel_ms = [float(x) for x in stats.tolist()]
    playouts_per_pass, plies_per_pass = [int(x) for x in work.tolist()]
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    pk = peaks()
    value = playouts_per_pass * args.steps / (dev_ms * 1e-3)
    e2e_value = playouts_per_pass * args.steps / (e2e_ms * 1e-3)
    sm_count, per_sm = geo["sm_count"], geo["blocks_per_sm"]
    # dominant kernel: the search kernel.  Per rank and launch it plays plies_per_pass / n_gpus plies.
    plies_per_launch = plies_per_pass / n_gpus
    playouts_per_launch = playouts_per_pass / n_gpus
    tree_steps_per_launch = B * args.trees * args.search_steps
    # algorithmic HBM bytes: a tree-step touches ~1.3 KB of tree records; every stream state is read and written once
    # per launch, or once per 32-step slice when a Connect-4 batch with more trees than resident blocks runs through the
    # work queue (the streams of the headline batch stay in L2 between slices)
    queued = args.game == "c4" and B * args.trees > per_sm * sm_count and args.search_steps > 32
    slices = -(-args.search_steps // 32) if queued else 1
    n_streams = B * args.trees * (A if "acp" in args.variant else 1) * args.playouts
    algo_bytes = 32.0 * n_streams * slices + 1300.0 * tree_steps_per_launch
    hbm_achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
    # the binding roofline: instruction issue.  Work unit = one playout ply, yardstick thread instructions per ply;
    # peak = SMs x 4 schedulers x 32 lanes x SM clock
    peak_inst = sm_count * 4 * 32 * pk["sm_max_mhz"] * 1e6
    inst_achieved = plies_per_launch * G["inst_per_ply"] / (kernel_ms * 1e-3)
    workload_key = f"{args.variant},{args.trees},{args.playouts},{args.search_steps},{B}"
    prof = profiler_readings(args.game, workload_key)
    kernel_name = "c4::search_kernel" if args.game == "c4" else "gomoku::playout_dynamic_kernel (+ tree_step_kernel)"
    line = {
        "metric": "playouts/sec", "value": value, "unit": "playouts/s", "n_gpus": n_gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic", "config": config_dict(args, n_gpus),
        "e2e": {"value": e2e_value, "unit": "playouts/s", "h2d_bytes_per_step": int(B * (17 if args.game == "c4" else 65)),
                "d2h_bytes_per_step": int(B * (3 * A * 8 + 2 * A + 80)), "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": args.steps * ((6 if queued else 4) if args.game == "c4" else 4 + 2 * args.search_steps),
        "roofline": {"bound": "issue", "achieved": inst_achieved / 1e12, "peak": peak_inst / 1e12, "unit": "T thread-inst/s",
                     "frac": inst_achieved / peak_inst, "peak_source": f"{sm_count} SMs x 4 schedulers x 32 lanes x {pk['sm_max_mhz']:.0f} MHz ({pk['source']} clock)",
                     "traffic": None if prof is None else prof.get("dram_bytes_per_launch"),
                     "traffic_unit": "DRAM bytes per launch (ncu)", "kernel": kernel_name, "kernel_ms": kernel_ms,
                     "work_unit": "playout ply", "inst_per_ply_yardstick": G["inst_per_ply"],
                     "plies_per_playout": plies_per_launch / max(playouts_per_launch, 1), "plies_per_launch": plies_per_launch,
                     "profiler": None if prof is None else {k: prof.get(k) for k in ("case", "alu_pipe_pct", "issue_active_pct",
                                                                                        "lanes_per_instruction", "thread_inst_per_ply")},
                     "note": "integer, branch-heavy work without a dense contraction: the limit is instruction issue, not HBM (hbm_roofline)"},
        "hbm_roofline": {"bound": "hbm", "achieved": hbm_achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": hbm_achieved / pk["hbm_gbs"], "algorithmic_bytes": algo_bytes, "peak_source": pk["source"]},
        "clocks": clocks, "threads_per_tree": geo["threads_per_tree"], "blocks_per_sm": per_sm,
        "device_bytes": geo["device_bytes"], "status_bits": status, "ub_draws_per_pass": ub_draws,
        "playouts_per_pass": playouts_per_pass, "best_action_checksum": int(out["best_action"].astype(np.int64).sum()),
        "multi_gpu_parity": parity, "exchange": args.exchange if n_gpus > 1 else None,
        "exchange_status": exchange_status,
    }
    if n_gpus == 1 and not args.no_cpu_baseline:
        steps = args.cpu_sample_steps or 400
        n_roots = args.cpu_sample_roots or 8
        playouts, plies, wall = cpu_port_baseline(args, boards, fills, turns, 1, n_roots, steps)
        line["cpu_baseline"] = {"value": playouts / wall, "unit": "playouts/s", "cores": 1, "kind": "port",
                                "sample": f"{n_roots} roots x {steps} search steps, sequential, {wall:.1f} s"}
    if n_gpus == 1 and not args.no_secondary:
        del searcher
        torch.cuda.empty_cache()
        line["secondary"] = secondary_runs(args, local_rank)
        ref_cpu = line["secondary"].get("reference_cpu_mcts", {})
        if "cpu_baseline" in line and "one_core" in ref_cpu:
            line["cpu_baseline"]["reference_mcts"] = {"one_core": ref_cpu["one_core"], "all_cores": ref_cpu["all_cores"],
                                                      "what": ref_cpu["what"]}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
