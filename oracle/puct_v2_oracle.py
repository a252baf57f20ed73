"""CPU restatement of the reference's two older PUCT select kernels and their backup, for trees that keep virtual
visits per child node.

TEST INFRASTRUCTURE ONLY (imported by tests).

Follows ``_select_kernel_native`` (preclaim, ``src/puct/puct_gpu_v2.py:573-697``), ``_select_kernel_winner_recalc``
(counter-CAS, ``:700-840``) and ``_backup_kernel_native`` (``:847-927``) with the warps of a tree executed one after
another, each to the end of its traversal -- one of the schedules a GPU may take, and the only one with a single warp
per tree.  Float32 arithmetic in the reference's order (``_puct_score`` ``:265-288``, ``_allowed_children`` ``:237-262``).
Pinned by the known-answer cases of the reference's test script (``src/puct/test_puct_gpu_v2.py:1006-1166``), restated
in ``tests/test_puct_v2_oracle.py``.
"""
import numpy as np

NODE_TERMINAL = -1
NODE_LIMIT, NODE_MASK, EDGE_LIMIT = 16384, 0x3FFF, 256
KIND_SHIFT, SLOT_SHIFT = 22, 14
INVALID, EXPAND, TERMINAL, DEPTH_LIMIT = 0, 1, 2, 3
PACKED_INVALID = (INVALID << KIND_SHIFT) | NODE_MASK
PRECLAIM, COUNTER_CAS = 0, 1
MAX_RECALC = 2
f32 = np.float32


def pack(kind, node, slot):
    return (kind << KIND_SHIFT) | (slot << SLOT_SHIFT) | node


def decode(raw):
    """(kind, slot, node) of a packed result (``:351-354``)."""
    raw = int(raw)
    return raw >> KIND_SHIFT, (raw >> SLOT_SHIFT) & 0xFF, raw & NODE_MASK


def make_case(trees=1, nodes=4, actions=4, warps=1, path_depth=4):
    """Empty arrays in the layout of the v2 kernels (names as in ``test_puct_gpu_v2.py:78-106``)."""
    return {"edge_child": np.full((trees, nodes, actions), -1, np.int32),
            "edge_prior": np.ones((trees, nodes, actions), np.float32),
            "edge_w": np.zeros((trees, nodes, actions), np.float32),
            "edge_n": np.zeros((trees, nodes, actions), np.int32),
            "node_inflight": np.zeros((trees, nodes), np.int32),
            "node_expand_inflight": np.zeros((trees, nodes), np.int32),
            "node_expanded": np.zeros((trees, nodes), np.int32),
            "node_count": np.full((trees,), nodes, np.int32),
            "out_selected": np.full((trees, warps), PACKED_INVALID, np.int32),
            "out_path": np.full((trees, warps, max(1, path_depth)), -1, np.int32),
            "out_len": np.zeros((trees, warps), np.int32), "warps": warps, "trees": trees}


def _allowed_children(c_pw, alpha_pw, n_node, max_edges):
    n = f32(max(n_node, 1))
    val = f32(c_pw) * np.sqrt(n, dtype=np.float32) if f32(alpha_pw) == f32(0.5) else f32(c_pw) * np.power(n, f32(alpha_pw), dtype=np.float32)
    if val >= f32(max_edges):
        return max_edges
    return max(1, int(np.ceil(val)))


def _score(cpuct, prior, w, n, inflight, sqrt_parent):
    q = f32(0.0) if n <= 0 else f32(w) / f32(n)
    return f32(q + f32(f32(f32(cpuct) * f32(prior)) * sqrt_parent) / f32(n + inflight + 1))


def _rollback(d, tree, wid, depth, node_cnt):
    edges = d["edge_child"].shape[2]
    for k in range(depth):
        enc = int(d["out_path"][tree, wid, k])
        if enc < 0:
            continue
        parent, slot = enc >> 8, enc & 0xFF
        if parent < node_cnt and slot < edges:
            child = int(d["edge_child"][tree, parent, slot])
            if 0 <= child < node_cnt:
                d["node_inflight"][tree, child] -= 1


def select(d, cpuct=1.0, c_pw=1.0, alpha_pw=0.5, variant=PRECLAIM):
    trees, nodes, edges = d["edge_child"].shape
    warps = d["out_selected"].shape[1]
    path_depth = d["out_path"].shape[2]
    for tree in range(trees):
        for wid in range(warps):
            d["out_selected"][tree, wid], d["out_len"][tree, wid] = _traverse(d, tree, wid, nodes, edges, path_depth, cpuct,
                                                                              c_pw, alpha_pw, variant)
    return d


def _traverse(d, tree, wid, nodes, edges, path_depth, cpuct, c_pw, alpha_pw, variant):
    node_cnt = int(d["node_count"][tree])
    if not (path_depth >= 1 and nodes > 0 and 0 < node_cnt <= nodes and node_cnt <= NODE_LIMIT and 0 < edges <= EDGE_LIMIT):
        return PACKED_INVALID, 0
    C, N, W, P, F = d["edge_child"], d["edge_n"], d["edge_w"], d["edge_prior"], d["node_inflight"]
    node, depth = 0, 0
    while True:
        if node < 0 or node >= node_cnt:
            _rollback(d, tree, wid, depth, node_cnt)
            return PACKED_INVALID, 0
        if depth >= path_depth:
            return pack(DEPTH_LIMIT, node, 0), depth + 1
        info = int(d["node_expanded"][tree, node])
        if info == NODE_TERMINAL:
            return pack(TERMINAL, node, 0), depth + 1
        if info < 0 or info > edges:
            _rollback(d, tree, wid, depth, node_cnt)
            return PACKED_INVALID, 0
        n_exp = info
        valid = [e for e in range(n_exp) if 0 <= int(C[tree, node, e]) < node_cnt]
        parent_eff = max(sum(int(N[tree, node, e]) + int(F[tree, int(C[tree, node, e])]) for e in valid), 1)
        allowed = 1 if (variant == PRECLAIM and n_exp == 0) else _allowed_children(c_pw, alpha_pw, parent_eff, edges)
        if allowed > n_exp:
            slot = n_exp + int(d["node_expand_inflight"][tree, node])       # atomic add returns the old value
            d["node_expand_inflight"][tree, node] += 1
            if slot < allowed:
                return pack(EXPAND, node, slot), depth + 1
            d["node_expand_inflight"][tree, node] -= 1
            _rollback(d, tree, wid, depth, node_cnt)
            return PACKED_INVALID, 0
        sqrt_parent = np.sqrt(f32(parent_eff), dtype=np.float32)
        best = None
        if variant == PRECLAIM:
            rot = wid % n_exp if wid >= n_exp else wid
            best_score, best_tie = None, None
            for e in valid:
                child = int(C[tree, node, e])
                old = int(F[tree, child])
                F[tree, child] += 1
                s = _score(cpuct, P[tree, node, e], W[tree, node, e], int(N[tree, node, e]), old, sqrt_parent)
                if s != s:
                    continue
                tie = (e - rot) % n_exp
                if best is None or s > best_score or (s == best_score and tie < best_tie):
                    best, best_score, best_tie = e, s, tie
            for e in valid:
                if e != best:
                    F[tree, int(C[tree, node, e])] -= 1
        else:
            skip = -1
            for attempt in range(MAX_RECALC):
                cand, cand_score = None, None
                for e in valid:
                    if e == skip:
                        continue
                    s = _score(cpuct, P[tree, node, e], W[tree, node, e], int(N[tree, node, e]), int(F[tree, int(C[tree, node, e])]),
                               sqrt_parent)
                    if s != s:
                        continue
                    if cand is None or s > cand_score:     # ascending e: the lowest edge wins ties
                        cand, cand_score = e, s
                if cand is None:
                    if skip < 0:
                        break
                    cand = skip
                child = int(C[tree, node, cand])
                old = int(F[tree, child])
                if old < 0 or old >= 0x7FFFFFFF:
                    break                                   # not claimable
                F[tree, child] += 1                         # alone, the compare-and-swap succeeds at once
                best = cand
                if old == 0 or n_exp <= 1 or attempt + 1 >= MAX_RECALC:
                    break
                F[tree, child] -= 1                         # somebody was there: give it back, choose again without it
                best, skip = None, cand
        if best is None:
            _rollback(d, tree, wid, depth, node_cnt)
            return PACKED_INVALID, 0
        d["out_path"][tree, wid, depth] = (node << 8) | best
        node = int(C[tree, node, best])
        depth += 1


def backup(d, values=None, virtual_loss=1):
    """``_backup_kernel_native`` (``:847-927``); with ``values=None`` only the visits and the ticket are released."""
    trees, nodes, edges = d["edge_child"].shape
    warps = d["out_selected"].shape[1]
    for tree in range(trees):
        node_cnt = int(d["node_count"][tree])
        if node_cnt <= 0 or node_cnt > nodes or node_cnt > NODE_LIMIT:
            continue
        for wid in range(warps):
            raw = int(d["out_selected"][tree, wid])
            plen = int(d["out_len"][tree, wid])
            if raw < 0 or (raw >> KIND_SHIFT) == INVALID or plen <= 0:
                continue
            for k in range(plen - 1):
                enc = int(d["out_path"][tree, wid, k])
                if enc < 0:
                    continue
                parent, slot = enc >> 8, enc & 0xFF
                if parent < node_cnt and slot < edges:
                    child = int(d["edge_child"][tree, parent, slot])
                    if 0 <= child < node_cnt:
                        d["node_inflight"][tree, child] -= virtual_loss
                    if values is not None:
                        d["edge_n"][tree, parent, slot] += 1
                        d["edge_w"][tree, parent, slot] = f32(d["edge_w"][tree, parent, slot]) + f32(values[tree, wid, k])
            if (raw >> KIND_SHIFT) == EXPAND:
                leaf = raw & NODE_MASK
                if leaf < node_cnt:
                    d["node_expand_inflight"][tree, leaf] -= 1
    return d


def from_v3_case(case):
    """A case built for the per-edge layout (``oracle.puct_oracle.layered_case``) in the per-node layout."""
    out = {k: v for k, v in case.items() if k != "edge_inflight"}
    out["node_inflight"] = np.zeros(case["node_expanded"].shape, np.int32)
    out["out_selected"] = np.full_like(case["out_selected"], PACKED_INVALID)
    return out
