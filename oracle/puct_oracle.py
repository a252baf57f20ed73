"""CPU restatement of the reference's warp-level PUCT select and of the backup that follows it.

TEST INFRASTRUCTURE ONLY (imported by tests and by the CPU-baseline leg of the PUCT benchmark).

Follows ``puct_select_winner_recalc_kernel`` of ``src/puct/puct_gpu_v3_cpp.cu:277-448`` (numba twin
``src/puct/puct_gpu_v3.py:426-630``), with the warps of a tree executed ONE AFTER ANOTHER, each to the end of its
traversal.  That is one of the schedules the GPU may take; with one warp per tree it is the only one, so single-warp
results must match exactly, while multi-warp GPU results are checked through invariants.  All arithmetic in float32,
in the order of the reference (``:171-180``, ``:150-157``).

Pinned by the known-answer cases of the reference's own test script (``src/puct/test_puct_gpu_v3.py:1154-1416``,
restated in ``tests/test_puct_oracle.py``) and, on a GPU, by the reference kernel itself compiled from its source into
``oracle/_ref/`` (see ``oracle/Makefile``).
"""
import numpy as np

NODE_TERMINAL = -1
NODE_LIMIT, NODE_MASK, EDGE_LIMIT = 16384, 0x3FFF, 256
KIND_SHIFT, SLOT_SHIFT, REASON_SHIFT = 22, 14, 25
INVALID, EXPAND, TERMINAL, DEPTH_LIMIT, BUSY = 0, 1, 2, 3, 4
(R_UNSET, R_OK_EXPAND, R_OK_TERMINAL, R_OK_DEPTH_LIMIT, R_BUSY_EXPAND_INFLIGHT, R_BUSY_WINNER_RECALC) = (0, 1, 2, 3, 4, 5)
R_INVALID_SHAPE, R_INVALID_NODE_INFO, R_INVALID_NO_VALID_EDGE, R_INVALID_CHILD_OOB, R_INVALID_UNKNOWN = 10, 11, 14, 15, 16
LOWEST = np.float32(-3.4028234663852886e38)
f32 = np.float32


def pack(kind, node, slot, reason):
    return (reason << REASON_SHIFT) | (kind << KIND_SHIFT) | (slot << SLOT_SHIFT) | node


def decode(raw):
    """(kind, slot, node, reason) of a packed result (``:38-41``)."""
    raw = int(raw)
    return (raw >> KIND_SHIFT) & 7, (raw >> SLOT_SHIFT) & 0xFF, raw & NODE_MASK, (raw >> REASON_SHIFT) & 0x3F


def make_case(trees=1, nodes=4, actions=4, warps=1, path_depth=4):
    """Empty arrays in the layout of the select ABI (names as in the reference's tests, ``test_puct_gpu_v3.py:85-111``)."""
    return {"edge_child": np.full((trees, nodes, actions), -1, np.int32),
            "edge_prior": np.ones((trees, nodes, actions), np.float32),
            "edge_w": np.zeros((trees, nodes, actions), np.float32),
            "edge_n": np.zeros((trees, nodes, actions), np.int32),
            "edge_inflight": np.zeros((trees, nodes, actions), np.int32),
            "node_expand_inflight": np.zeros((trees, nodes), np.int32),
            "node_expanded": np.zeros((trees, nodes), np.int32),
            "node_count": np.full((trees,), nodes, np.int32),
            "out_selected": np.full((trees, warps), pack(INVALID, NODE_MASK, 0, 0), np.int32),
            "out_path": np.full((trees, warps, max(1, path_depth)), -1, np.int32),
            "out_len": np.zeros((trees, warps), np.int32), "warps": warps, "trees": trees}


def _allowed_children(c_pw, alpha_pw, n_node, max_edges):
    n = f32(n_node)
    val = f32(c_pw) * np.sqrt(n, dtype=np.float32) if f32(alpha_pw) == f32(0.5) else f32(c_pw) * np.power(n, f32(alpha_pw), dtype=np.float32)
    if val >= f32(max_edges):
        return max_edges
    return max(1, int(np.ceil(val)))


def _score(cpuct, prior, w, n, inflight, sqrt_parent):
    q = f32(0.0) if n <= 0 else f32(w) / f32(n)
    u = f32(f32(f32(cpuct) * f32(prior)) * sqrt_parent) / f32(n + inflight + 1)
    return f32(q + u)


def _rollback(d, tree, wid, depth, amount):
    node_cnt = int(d["node_count"][tree])
    edges = d["edge_child"].shape[2]
    for k in range(depth):
        enc = int(d["out_path"][tree, wid, k])
        parent, slot = enc >> 8, enc & 0xFF
        if 0 <= parent < node_cnt and slot < edges:
            d["edge_inflight"][tree, parent, slot] -= amount


def select(d, cpuct=1.0, c_pw=1.0, alpha_pw=0.5, soft_winner=0, virtual_loss=1):
    """Runs every (tree, warp) traversal in order on the numpy arrays of ``d`` (modified in place)."""
    trees, nodes, edges = d["edge_child"].shape
    warps = d["out_selected"].shape[1]
    path_depth = d["out_path"].shape[2]
    for tree in range(trees):
        for wid in range(warps):
            d["out_selected"][tree, wid], d["out_len"][tree, wid] = _traverse(d, tree, wid, nodes, edges, path_depth, cpuct,
                                                                              c_pw, alpha_pw, soft_winner, virtual_loss)
    return d


def _traverse(d, tree, wid, nodes, edges, path_depth, cpuct, c_pw, alpha_pw, soft_winner, vl):
    node_cnt = int(d["node_count"][tree])
    if not (path_depth >= 1 and nodes > 0 and 0 < node_cnt <= nodes and node_cnt <= NODE_LIMIT and 0 < edges <= EDGE_LIMIT):
        return pack(INVALID, NODE_MASK, 0, R_INVALID_SHAPE), 0
    node, depth = 0, 0
    N, W, P, F = d["edge_n"], d["edge_w"], d["edge_prior"], d["edge_inflight"]
    while True:
        info = int(d["node_expanded"][tree, node])
        if info == NODE_TERMINAL:
            return pack(TERMINAL, node, 0, R_OK_TERMINAL), depth + 1
        if info < 0 or info > edges:
            _rollback(d, tree, wid, depth, vl)
            return pack(INVALID, NODE_MASK, 0, R_INVALID_NODE_INFO), 0
        if depth >= path_depth:
            return pack(DEPTH_LIMIT, node, 0, R_OK_DEPTH_LIMIT), depth + 1
        n_exp = info
        parent_eff, allowed = 1, 1
        if n_exp != 1 or f32(c_pw) != f32(0.0):
            parent_eff = max(int(N[tree, node, :n_exp].sum()) + int(F[tree, node, :n_exp].sum()), 1)
            allowed = _allowed_children(c_pw, alpha_pw, parent_eff, edges)
        if allowed > n_exp:
            tickets = int(d["node_expand_inflight"][tree, node])
            if n_exp + tickets < allowed:
                slot = n_exp + tickets          # atomicAdd returns the old value
                d["node_expand_inflight"][tree, node] += 1
                if slot < allowed:
                    return pack(EXPAND, node, slot, R_OK_EXPAND), depth + 1
                d["node_expand_inflight"][tree, node] -= 1
            if n_exp == 0:
                _rollback(d, tree, wid, depth, vl)
                return pack(BUSY, node, 0, R_BUSY_EXPAND_INFLIGHT), 0
        best = None
        if n_exp == 1:
            F[tree, node, 0] += vl
            best = 0
        else:
            rot = wid % n_exp if wid >= n_exp else wid
            sqrt_parent = np.sqrt(f32(parent_eff), dtype=np.float32)
            best_score, best_tie = None, None
            for e in range(n_exp):
                s = _score(cpuct, P[tree, node, e], W[tree, node, e], int(N[tree, node, e]), int(F[tree, node, e]), sqrt_parent)
                if not (s >= LOWEST):
                    continue
                tie = (e - rot) % n_exp
                if best is None or s > best_score or (s == best_score and tie < best_tie):
                    best, best_score, best_tie = e, s, tie
            if best is None:
                _rollback(d, tree, wid, depth, vl)
                return pack(INVALID, NODE_MASK, 0, R_INVALID_NO_VALID_EDGE), 0
            F[tree, node, best] += vl            # executed alone, the compare-and-swap always succeeds
        child = int(d["edge_child"][tree, node, best])
        if child < 0 or child >= node_cnt:
            F[tree, node, best] -= vl
            _rollback(d, tree, wid, depth, vl)
            return pack(INVALID, NODE_MASK, 0, R_INVALID_CHILD_OOB), 0
        d["out_path"][tree, wid, depth] = (node << 8) | best
        node = child
        depth += 1


def backup(d, values=None, virtual_loss=1):
    """The backup (``src/puct/puct_gpu_v2.py:847-927`` moved to the per-edge inflight layout of v3) or, with
    ``values=None``, the release of the claims only (``src/puct/test_puct_gpu_v3.py:274-332``)."""
    trees, nodes, edges = d["edge_child"].shape
    warps = d["out_selected"].shape[1]
    for tree in range(trees):
        node_cnt = int(d["node_count"][tree])
        if node_cnt <= 0 or node_cnt > nodes or node_cnt > NODE_LIMIT:
            continue
        for wid in range(warps):
            raw = int(d["out_selected"][tree, wid])
            kind = (raw >> KIND_SHIFT) & 7
            plen = int(d["out_len"][tree, wid])
            if raw < 0 or kind in (INVALID, BUSY) or plen <= 0:
                continue
            for k in range(plen - 1):
                enc = int(d["out_path"][tree, wid, k])
                if enc < 0:
                    continue
                parent, slot = enc >> 8, enc & 0xFF
                if parent < node_cnt and slot < edges:
                    d["edge_inflight"][tree, parent, slot] -= virtual_loss
                    if values is not None:
                        d["edge_n"][tree, parent, slot] += 1
                        d["edge_w"][tree, parent, slot] = f32(d["edge_w"][tree, parent, slot]) + f32(values[tree, wid, k])
            if kind == EXPAND:
                leaf = raw & NODE_MASK
                if leaf < node_cnt:
                    d["node_expand_inflight"][tree, leaf] -= 1
    return d


def layered_case(trees, edges, depth, warps, seed, nodes_per_level=None, dirichlet_alpha=0.3):
    """Seeded synthetic workload for the PUCT benchmark and tests: an acyclic layered tree per `tree` -- every node of
    level l has `edges` expanded children in level l+1 (shared within the level so that the array stays small), the
    last level is terminal.  Priors ~ Dirichlet(alpha) per node, visit counts random, W = N * mean leaf value with
    values ~ U[-1, 1]."""
    rng = np.random.default_rng(seed)
    per = nodes_per_level or edges
    nodes = 1 + per * depth
    case = make_case(trees=trees, nodes=nodes, actions=edges, warps=warps, path_depth=depth)
    level_start = [0] + [1 + per * l for l in range(depth)]
    level_size = [1] + [per] * depth
    for l in range(depth):
        for i in range(level_size[l]):
            node = level_start[l] + i
            case["node_expanded"][:, node] = edges
            nxt = level_start[l + 1] + (np.arange(edges) + i) % level_size[l + 1]
            case["edge_child"][:, node, :] = nxt[None, :]
    last = level_start[depth]
    case["node_expanded"][:, last:last + level_size[depth]] = NODE_TERMINAL
    case["edge_prior"][:] = rng.dirichlet(np.full(edges, dirichlet_alpha), size=(trees, nodes)).astype(np.float32)
    n = rng.integers(0, 50, size=(trees, nodes, edges)).astype(np.int32)
    case["edge_n"][:] = n
    case["edge_w"][:] = (n * rng.uniform(-1.0, 1.0, size=(trees, nodes, edges))).astype(np.float32)
    return case
