#!/usr/bin/env python
"""Benchmark of the MCTS-NC search hot path: playouts/s for Connect 4, acp_prodigal, 4 trees x 256 playouts,
2000 search steps per root, 256 seeded random roots per pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" of the benchmark is one pass over the whole batch of roots (every root is searched for `--search-steps`
MCTS steps).  With N > 1 (launched by torchrun, one rank per GPU) every rank grows 4 trees of every search with the
random streams of a 4N-tree search, and the per-root-action sums are all-reduced over NCCL once per pass (root
parallelism; per-GPU work is fixed: weak scaling).  Rank 0 prints one JSON line.

`--impl reference` times the CPU restatement of the reference's kernels (oracle/) on the host cores, one root per
thread, on a bounded sample of the same workload.
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

# dram__bytes_read.sum + dram__bytes_write.sum of one search-kernel launch, from a one-pass ncu capture of the default
# workload; key: game, variant, trees, playouts, search steps, roots
MEASURED_TRAFFIC_BYTES = {("c4", "acp_prodigal", 4, 256, 2000, 256): 133639424 + 409819136}


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
    ap.add_argument("--cpu-sample-steps", type=int, default=400)
    ap.add_argument("--no-cpu-baseline", action="store_true")
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


def oracle_search(job):
    from oracle.oracle import OracleMCTSNC
    board, fills, turn, trees, playouts, variant, steps, game = job
    G = GAMES[game]
    o = OracleMCTSNC(G["shape"], G["extra"], G["actions"], n_trees=trees, n_playouts=playouts, variant=variant, seed=0,
                     device_memory=16.0 if game == "gomoku" else 2.0, node_capacity=steps * G["actions"] + G["actions"] + 8)
    t0 = time.perf_counter()
    o.run(board, fills, int(turn), steps)
    return o.playouts, o.plies, time.perf_counter() - t0


def cpu_port_baseline(args, boards, fills, turns, threads, n_roots, steps):
    """The oracle (CPU restatement of the reference's kernels) on `threads` host threads, one root per thread."""
    from concurrent.futures import ThreadPoolExecutor
    from oracle import oracle as om
    om.lib()
    jobs = [(boards[i % len(boards)], fills[i % len(boards)] if fills is not None else None, turns[i % len(boards)],
             args.trees, args.playouts, args.variant, steps, args.game) for i in range(n_roots)]
    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        res = list(ex.map(oracle_search, jobs))
    wall = time.perf_counter() - t0
    playouts = sum(r[0] for r in res)
    plies = sum(r[1] for r in res)
    return playouts, plies, wall


def config_dict(args, n_gpus):
    return {"workload": f"{GAMES[args.game]['name']} {args.variant}, n_trees={args.trees} per GPU, n_playouts={args.playouts}, "
                        f"search_steps={args.search_steps}, {args.roots} seeded random roots (0..{args.max_plies} plies) per pass",
            "trees_per_search_total": args.trees * n_gpus, "parallelism": f"root-parallel x{n_gpus}" if n_gpus > 1 else "single GPU",
            "l2": "no flush: the tree pools of one pass (~0.5 GB) exceed the 126 MB L2", "seed": 0, "ucb_c": 2.0}


def run_reference(args, rank):
    if rank != 0:
        return
    boards, fills, turns = make_roots(args)
    cores = os.cpu_count() or 1
    steps = args.cpu_sample_steps
    n_roots = args.cpu_sample_roots or cores
    times, total_playouts = [], 0
    for i in range(args.warmup + args.steps):
        playouts, plies, wall = cpu_port_baseline(args, boards, fills, turns, cores, n_roots, steps)
        if i >= args.warmup:
            times.append(wall)
            total_playouts += playouts
    value = total_playouts / sum(times)
    sample = f"{n_roots} roots x {steps} search steps per pass, one root per thread"
    print(json.dumps({"impl": "reference", "metric": "playouts/sec", "value": value, "unit": "playouts/s", "n_gpus": args.gpus,
                      "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(times) / len(times),
                      "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int32",
                      "data": "synthetic", "config": config_dict(args, args.gpus),
                      "cpu_baseline": {"value": value, "unit": "playouts/s", "cores": cores, "kind": "port", "sample": sample},
                      "e2e": {"value": value, "unit": "playouts/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                      "gpu_launches": 0}))


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
    print(json.dumps(line))


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
    print(json.dumps(line))


def main():
    args = parse_args()
    if args.workload == "puct":
        run_puct(args)
        return
    if args.workload == "duct":
        run_duct(args)
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
                                  device_memory=16.0 if args.game == "gomoku" else 2.0)

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
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    ev[0].record()
    for k in range(args.steps):
        searcher.search_async(None, None, None, args.search_steps, reseed=True)
        ev[k + 1].record()
    barrier()
    dev_ms = ev[0].elapsed_time(ev[-1])
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
    thr, per_sm, sms, nbytes = (np.zeros(1, np.int32), np.zeros(1, np.int32), np.zeros(1, np.int32), np.zeros(1, np.int64))
    import ctypes
    _abi.lib().mctsnc_query(searcher.local._handle, thr.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                            per_sm.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                            sms.ctypes.data_as(ctypes.POINTER(ctypes.c_int32)),
                            nbytes.ctypes.data_as(ctypes.POINTER(ctypes.c_int64)))
    sm_count = int(sms[0])
    # dominant kernel: the search kernel.  Per rank and launch it plays plies_per_pass / n_gpus plies.
    plies_per_launch = plies_per_pass / n_gpus
    playouts_per_launch = playouts_per_pass / n_gpus
    tree_steps_per_launch = B * args.trees * args.search_steps
    # algorithmic HBM bytes: every stream state is read and written once per launch (2 x 16 B), and a
    # tree-step touches ~1.3 KB of tree records
    # A Connect-4 batch with more trees than resident blocks runs in slices of 32 steps taken from a work queue; a
    # tree's streams are then read and written once per slice (they fit in L2 between slices for the headline batch).
    queued = args.game == "c4" and B * args.trees > int(per_sm[0]) * sm_count and args.search_steps > 32
    slices = -(-args.search_steps // 32) if queued else 1
    n_streams = B * args.trees * (A if "acp" in args.variant else 1) * args.playouts
    algo_bytes = 32.0 * n_streams * slices + 1300.0 * tree_steps_per_launch
    hbm_achieved = algo_bytes / (kernel_ms * 1e-3) / 1e9
    peak_inst = sm_count * 4 * 32 * pk["sm_max_mhz"] * 1e6
    inst_achieved = plies_per_launch * G["inst_per_ply"] / (kernel_ms * 1e-3)
    line = {
        "metric": "playouts/sec", "value": value, "unit": "playouts/s", "n_gpus": n_gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic", "config": config_dict(args, n_gpus),
        "e2e": {"value": e2e_value, "unit": "playouts/s", "h2d_bytes_per_step": int(B * (17 if args.game == "c4" else 65)),
                "d2h_bytes_per_step": int(B * (3 * A * 8 + 2 * A + 80)), "ms_per_step": e2e_ms / args.steps},
        "gpu_launches": args.steps * ((6 if queued else 4) if args.game == "c4" else 4 + 2 * args.search_steps),
        "roofline": {"bound": "hbm", "achieved": hbm_achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": hbm_achieved / pk["hbm_gbs"],
                     "traffic": MEASURED_TRAFFIC_BYTES.get((args.game, args.variant, args.trees, args.playouts, args.search_steps, B)),
                     "traffic_unit": "bytes per launch (ncu, one capture)", "algorithmic_bytes": algo_bytes,
                     "peak_source": pk["source"],
                     "kernel": "c4::search_kernel" if args.game == "c4" else "gomoku::playout_kernel (+ tree_step_kernel)", "kernel_ms": kernel_ms,
                     "note": "the search is instruction-issue bound, not HBM bound: see issue_roofline"},
        "issue_roofline": {"bound": "issue", "achieved": inst_achieved / 1e12, "peak": peak_inst / 1e12,
                           "unit": "T thread-inst/s", "frac": inst_achieved / peak_inst,
                           "binding_unit": ("integer/logic pipe (16 lanes per clock and scheduler): 87.8 % of its peak, 71.5 % of "
                                            "issue slots, 21.9 of 32 lanes active (ncu capture of the 256-root, 200-step case)"
                                            if args.game == "c4" else
                                            "integer/logic pipe: 76.4 % of its peak, 72.0 % of issue slots, 21.2 of 32 lanes active "
                                            "(ncu capture of one step of a 4 x 256 search)"),
                           "plies_per_playout": plies_per_launch / max(playouts_per_launch, 1),
                           "inst_per_ply_yardstick": G["inst_per_ply"], "sm_count": sm_count,
                           "peak_clock_mhz": pk["sm_max_mhz"]},
        "clocks": clocks, "threads_per_tree": int(thr[0]), "blocks_per_sm": int(per_sm[0]),
        "device_bytes": int(nbytes[0]), "status_bits": status, "ub_draws_per_pass": ub_draws,
        "playouts_per_pass": playouts_per_pass, "best_action_checksum": int(out["best_action"].astype(np.int64).sum()),
    }
    if n_gpus == 1 and not args.no_cpu_baseline:
        steps = args.cpu_sample_steps
        n_roots = args.cpu_sample_roots or 8
        playouts, plies, wall = cpu_port_baseline(args, boards, fills, turns, 1, n_roots, steps)
        line["cpu_baseline"] = {"value": playouts / wall, "unit": "playouts/s", "cores": 1, "kind": "port",
                                "sample": f"{n_roots} roots x {steps} search steps, sequential, {wall:.1f} s"}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
