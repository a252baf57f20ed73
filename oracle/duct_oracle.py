"""CPU restatement of the decoupled-UCT (DUCT) select and backup of ``include/duct_b200.h``.

TEST INFRASTRUCTURE ONLY (tests, the benchmark's CPU leg).  The reference has no DUCT: this file restates the
library's OWN specification, so agreement with it pins the CUDA kernels to that specification, not to the reference
("parity unpinned").  Warps are run one after the other, each seeing the claims of the earlier ones; with one warp per
tree the CUDA kernel must agree exactly, with several it agrees only in the invariants (claims add up, one expansion per
joint action, everything returned after the backup).
"""
import numpy as np

KIND_INVALID, KIND_EXPAND, KIND_TERMINAL, KIND_DEPTH_LIMIT, KIND_BUSY = 0, 1, 2, 3, 4
R_OK_EXPAND, R_OK_TERMINAL, R_OK_DEPTH_LIMIT, R_BUSY_EXPAND_INFLIGHT, R_INVALID_SHAPE, R_INVALID_CHILD_OOB = 1, 2, 3, 4, 10, 15
CHILD_NONE, CHILD_CLAIMED = -1, -2
f32 = np.float32


def pack(kind, node, slot, reason):
    return (reason << 25) | (kind << 22) | (slot << 14) | node


def decode(selected):
    selected = np.asarray(selected)
    return (selected >> 22) & 7, selected & 0x3FFF, (selected >> 14) & 0xFF, (selected >> 25) & 0x3F


def scores(cpuct, prior, w, n, inflight, virtual_loss):
    """float32 scores of one player's actions, every operation rounded once in the order of the header."""
    n_eff = n.astype(np.int64) + virtual_loss * inflight.astype(np.int64)
    w_eff = (w.astype(f32) - (virtual_loss * inflight).astype(f32)).astype(f32)
    with np.errstate(divide="ignore", invalid="ignore"):
        q = np.where(n_eff > 0, (w_eff / np.maximum(n_eff, 1).astype(f32)).astype(f32), f32(0))
    sqrt_total = np.sqrt(f32(max(int(n_eff.sum()), 1)), dtype=f32)
    u = ((f32(cpuct) * prior.astype(f32)).astype(f32) * sqrt_total).astype(f32) / (1 + n_eff).astype(f32)
    return (q.astype(f32) + u.astype(f32)).astype(f32)


def select(d, cpuct=1.5, virtual_loss=1):
    """In-place on the numpy arrays of ``d`` (same names and shapes as the device dict)."""
    trees, warps = int(d["trees"]), int(d["warps"])
    A = d["node_prior"].shape[3]
    nodes = d["node_prior"].shape[1]
    depth_cap = d["out_path"].shape[2]
    for t in range(trees):
        cnt = int(d["node_count"][t])
        for wp in range(warps):
            if cnt <= 0 or cnt > nodes:
                d["out_selected"][t, wp] = pack(KIND_INVALID, 0, 0, R_INVALID_SHAPE)
                d["out_len"][t, wp] = 0
                continue
            node, depth, path = 0, 0, []
            while True:
                if d["node_terminal"][t, node]:
                    result = pack(KIND_TERMINAL, node, 0, R_OK_TERMINAL)
                    break
                if depth >= depth_cap:
                    result = pack(KIND_DEPTH_LIMIT, node, 0, R_OK_DEPTH_LIMIT)
                    break
                picks = []
                for p in range(2):
                    s = scores(cpuct, d["node_prior"][t, node, p], d["node_w"][t, node, p], d["node_n"][t, node, p],
                               d["node_inflight"][t, node, p], virtual_loss)
                    picks.append(int(np.argmax(s)))       # first maximum = lowest action on ties
                for p in range(2):
                    d["node_inflight"][t, node, p, picks[p]] += virtual_loss
                joint = picks[0] * A + picks[1]
                path.append((node, joint))
                d["out_path"][t, wp, depth] = (node << 8) | joint
                depth += 1
                kid = int(d["child"][t, node, joint])
                if kid >= 0:
                    if kid >= cnt:
                        result, depth = pack(KIND_INVALID, node, joint, R_INVALID_CHILD_OOB), 0
                        _rollback(d, t, path, A, virtual_loss)
                        break
                    node = kid
                    continue
                if kid == CHILD_NONE:
                    d["child"][t, node, joint] = CHILD_CLAIMED
                    result = pack(KIND_EXPAND, node, joint, R_OK_EXPAND)
                else:
                    result, depth = pack(KIND_BUSY, node, joint, R_BUSY_EXPAND_INFLIGHT), 0
                    _rollback(d, t, path, A, virtual_loss)
                break
            d["out_selected"][t, wp] = result
            d["out_len"][t, wp] = depth


def _rollback(d, t, path, A, virtual_loss):
    for node, joint in path:
        d["node_inflight"][t, node, 0, joint // A] -= virtual_loss
        d["node_inflight"][t, node, 1, joint % A] -= virtual_loss


def backup(d, values=None, new_child=None, virtual_loss=1):
    trees, warps = int(d["trees"]), int(d["warps"])
    A = d["node_prior"].shape[3]
    for t in range(trees):
        for wp in range(warps):
            for e in range(int(d["out_len"][t, wp])):
                enc = int(d["out_path"][t, wp, e])
                node, joint = enc >> 8, enc & 0xFF
                a0, a1 = joint // A, joint % A
                d["node_inflight"][t, node, 0, a0] -= virtual_loss
                d["node_inflight"][t, node, 1, a1] -= virtual_loss
                if values is not None:
                    v = f32(values[t, wp, e])
                    d["node_n"][t, node, 0, a0] += 1
                    d["node_n"][t, node, 1, a1] += 1
                    d["node_w"][t, node, 0, a0] = f32(d["node_w"][t, node, 0, a0] + v)
                    d["node_w"][t, node, 1, a1] = f32(d["node_w"][t, node, 1, a1] - v)
            kind, node, joint, _ = decode(int(d["out_selected"][t, wp]))
            if kind == KIND_EXPAND:
                kid = int(new_child[t, wp]) if new_child is not None else CHILD_NONE
                d["child"][t, node, joint] = kid if kid >= 0 else CHILD_NONE


def make_case(trees, actions=8, depth=16, nodes=None, warps=1, path_depth=None, seed=0, expanded_fraction=0.6, alpha=0.3):
    """Seeded synthetic trees: a random tree per search in which a node's joint actions have children with probability
    `expanded_fraction` while nodes last, nodes at `depth` are terminal; priors ~ Dirichlet(alpha) per player, counts and
    value sums consistent with leaf values ~ U[-1, 1] (player 1's sums are the negatives)."""
    rng = np.random.default_rng(seed)
    A = actions
    nodes = nodes or 512
    path_depth = path_depth or depth + 1
    d = {"trees": trees, "warps": warps,
         "child": np.full((trees, nodes, A * A), CHILD_NONE, np.int32),
         "node_prior": np.zeros((trees, nodes, 2, A), f32), "node_w": np.zeros((trees, nodes, 2, A), f32),
         "node_n": np.zeros((trees, nodes, 2, A), np.int32), "node_inflight": np.zeros((trees, nodes, 2, A), np.int32),
         "node_terminal": np.zeros((trees, nodes), np.int32), "node_count": np.zeros(trees, np.int32),
         "out_selected": np.zeros((trees, warps), np.int32), "out_len": np.zeros((trees, warps), np.int32),
         "out_path": np.zeros((trees, warps, path_depth), np.int32)}
    for t in range(trees):
        level_of = [0]
        frontier = [0]
        while frontier:
            node = frontier.pop(0)
            lvl = level_of[node]
            d["node_prior"][t, node] = rng.dirichlet([alpha] * A, size=2).astype(f32)
            if lvl >= depth:
                d["node_terminal"][t, node] = 1
                continue
            for joint in rng.permutation(A * A):
                if len(level_of) >= nodes or rng.random() > expanded_fraction:
                    continue
                kid = len(level_of)
                level_of.append(lvl + 1)
                d["child"][t, node, joint] = kid
                frontier.append(kid)
                visits = int(rng.integers(1, 20))
                value = f32(rng.uniform(-1, 1) * visits)
                a0, a1 = joint // A, joint % A
                d["node_n"][t, node, 0, a0] += visits
                d["node_n"][t, node, 1, a1] += visits
                d["node_w"][t, node, 0, a0] += value
                d["node_w"][t, node, 1, a1] -= value
        d["node_count"][t] = len(level_of)
    return d


def grow_case(trees, actions=8, nodes=256, rounds=150, terminal_depth=5, warps=1, path_depth=None, seed=0, cpuct=1.5,
              virtual_loss=1, alpha=0.3):
    """Trees grown from a bare root by `rounds` rounds of select -> expand -> backup of this restatement (one traversal
    per tree and round, leaf values ~ U[-1, 1], priors ~ Dirichlet(alpha), nodes at `terminal_depth` terminal): the
    statistics a real search leaves.  Returned with `warps` output slots and no claim in flight."""
    rng = np.random.default_rng(seed)
    A = actions
    d = make_case(trees, actions=A, depth=terminal_depth, nodes=nodes, warps=1, path_depth=terminal_depth + 1, seed=seed,
                  expanded_fraction=0.0)
    d["node_prior"][:] = rng.dirichlet([alpha] * A, size=(trees, nodes, 2)).astype(f32)
    depth_of = np.zeros((trees, nodes), np.int32)
    for _ in range(rounds):
        select(d, cpuct=cpuct, virtual_loss=virtual_loss)
        kind, node, _, _ = decode(d["out_selected"])
        values = rng.uniform(-1, 1, d["out_path"].shape).astype(f32)
        new_child = np.full((trees, 1), -1, np.int32)
        for t in range(trees):
            if kind[t, 0] == KIND_EXPAND and d["node_count"][t] < nodes:
                kid = int(d["node_count"][t])
                new_child[t, 0] = kid
                depth_of[t, kid] = depth_of[t, node[t, 0]] + 1
                d["node_terminal"][t, kid] = 1 if depth_of[t, kid] >= terminal_depth else 0
                d["node_count"][t] += 1
        backup(d, values, new_child, virtual_loss=virtual_loss)
    path_depth = path_depth or terminal_depth + 1
    d["warps"] = warps
    d["out_selected"] = np.zeros((trees, warps), np.int32)
    d["out_len"] = np.zeros((trees, warps), np.int32)
    d["out_path"] = np.zeros((trees, warps, path_depth), np.int32)
    return d


def copy_case(d):
    return {k: (v.copy() if isinstance(v, np.ndarray) else v) for k, v in d.items()}
