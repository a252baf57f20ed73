"""Known-answer cases of the warp-level PUCT select, restated from the reference's own test script
(``src/puct/test_puct_gpu_v3.py:1154-1416``): hand-built trees of 2-4 nodes with the result every backend has to give.
Each entry: (name, build() -> (case, select kwargs), check(h) -> bool) where h is the case after select (numpy)."""
import numpy as np

from oracle import puct_oracle as po


def _inflight_sum(h):
    return int(h["edge_inflight"].sum()) + int(h["node_expand_inflight"].sum())


def fresh_root():
    return po.make_case(nodes=2, actions=4, path_depth=2), {}


def check_fresh_root(h):
    kind, slot, node, _ = po.decode(h["out_selected"][0, 0])
    return (kind, slot, node) == (po.EXPAND, 0, 0) and h["out_len"][0, 0] == 1 and h["node_expand_inflight"][0, 0] == 1


def terminal_root():
    c = po.make_case(nodes=2, actions=4, path_depth=2)
    c["node_expanded"][0, 0] = po.NODE_TERMINAL
    return c, {}


def check_terminal_root(h):
    kind, _, node, _ = po.decode(h["out_selected"][0, 0])
    return kind == po.TERMINAL and node == 0 and h["out_len"][0, 0] == 1 and _inflight_sum(h) == 0


def invalid_child_node():
    c = po.make_case(nodes=2, actions=4, path_depth=4)
    c["node_expanded"][0, 0] = 1
    c["node_expanded"][0, 1] = -2
    c["edge_child"][0, 0, 0] = 1
    c["edge_n"][0, 0, 0] = 1
    return c, {}


def check_invalid_rolled_back(h):
    return po.decode(h["out_selected"][0, 0])[0] == po.INVALID and _inflight_sum(h) == 0


def child_beyond_node_count():
    c = po.make_case(nodes=4, actions=4, path_depth=3)
    c["node_count"][0] = 2
    c["node_expanded"][0, 0] = 1
    c["edge_child"][0, 0, 0] = 3
    c["edge_n"][0, 0, 0] = 1
    return c, {}


def fully_expanded():
    c = po.make_case(nodes=3, actions=4, path_depth=4)
    c["node_expanded"][0, 0] = 2
    c["edge_child"][0, 0, :2] = (1, 2)
    c["edge_prior"][0, 0, :2] = (0.1, 0.9)
    c["edge_n"][0, 0, :2] = 1
    return c, {}


def check_fully_expanded(h):
    kind, slot, node, _ = po.decode(h["out_selected"][0, 0])
    return ((kind, slot, node) == (po.EXPAND, 0, 2) and h["out_path"][0, 0, 0] == 1 and h["out_len"][0, 0] == 2
            and h["edge_inflight"][0, 0, 1] == 1 and h["node_expand_inflight"][0, 2] == 1)


def depth_limit():
    c = po.make_case(nodes=3, actions=4, path_depth=1)
    c["node_expanded"][0, :2] = 1
    c["edge_child"][0, 0, 0] = 1
    c["edge_child"][0, 1, 0] = 2
    c["edge_n"][0, 0, 0] = 1
    c["edge_n"][0, 1, 0] = 1
    return c, {}


def check_depth_limit(h):
    kind, _, node, _ = po.decode(h["out_selected"][0, 0])
    return kind == po.DEPTH_LIMIT and node == 1 and h["out_len"][0, 0] == 2 and h["edge_inflight"][0, 0, 0] == 1


def zero_n_edge():
    c = po.make_case(nodes=3, actions=4, path_depth=3)
    c["node_expanded"][0, 0] = 1
    c["edge_child"][0, 0, 0] = 1
    c["edge_n"][0, 0, 0] = 0
    return c, {}


def check_zero_n_edge(h):
    kind, _, node, _ = po.decode(h["out_selected"][0, 0])
    return kind == po.EXPAND and node == 1 and h["out_len"][0, 0] == 2


def edges_256():
    return po.make_case(nodes=2, actions=256, path_depth=2), {}


def edges_257():
    return po.make_case(nodes=2, actions=257, path_depth=2), {}


def too_many_nodes():
    return po.make_case(nodes=po.NODE_LIMIT + 1, actions=4, path_depth=2), {}


def node_count_gates():
    c = po.make_case(nodes=po.NODE_LIMIT + 1, actions=4, path_depth=2)
    c["node_count"][0] = po.NODE_LIMIT
    return c, {}


def check_kind(kind):
    return lambda h: po.decode(h["out_selected"][0, 0])[0] == kind


SINGLE_WARP_CASES = [
    ("fresh root expands slot 0", fresh_root, check_fresh_root),
    ("terminal root", terminal_root, check_terminal_root),
    ("invalid child node rolls back", invalid_child_node, check_invalid_rolled_back),
    ("child beyond node_count is invalid", child_beyond_node_count, check_invalid_rolled_back),
    ("fully expanded picks the high-prior edge", fully_expanded, check_fully_expanded),
    ("depth limit", depth_limit, check_depth_limit),
    ("zero-N edge is selectable", zero_n_edge, check_zero_n_edge),
    ("256 edges are fine", edges_256, check_kind(po.EXPAND)),
    ("257 edges are an invalid shape", edges_257, check_kind(po.INVALID)),
    ("more nodes than the packing allows", too_many_nodes, check_kind(po.INVALID)),
    ("node_count gates the packed node ids", node_count_gates, check_kind(po.EXPAND)),
]


# ---- multi-warp cases: the outcome depends on the schedule, the checks are the reference's invariants
def pw_multi_warp():
    c = po.make_case(nodes=3, actions=4, warps=4, path_depth=2)
    c["node_expanded"][0, 0] = 1
    c["edge_child"][0, 0, 0] = 1
    c["edge_n"][0, 0, 0] = 16
    return c, {"c_pw": 1.0, "alpha_pw": 0.5}


def check_pw_multi_warp(h):
    root_slots, child_expands = [], 0
    for wid in range(4):
        kind, slot, node, _ = po.decode(h["out_selected"][0, wid])
        if kind == po.EXPAND:
            if node == 0:
                root_slots.append(slot)
            elif node == 1:
                child_expands += 1
            else:
                return False
        elif kind != po.BUSY:
            return False
    return sorted(root_slots) == [1, 2, 3] and child_expands <= 1 and h["node_expand_inflight"][0, 0] == 3


def single_edge_contention():
    c = po.make_case(nodes=2, actions=4, warps=8, path_depth=2)
    c["node_expanded"][0, 0] = 1
    c["edge_child"][0, 0, 0] = 1
    c["edge_n"][0, 0, 0] = 1
    c["node_expanded"][0, 1] = po.NODE_TERMINAL
    return c, {"c_pw": 0.0}


def check_single_edge_contention(h):
    kinds = [po.decode(h["out_selected"][0, w])[0] for w in range(8)]
    valid, busy = kinds.count(po.TERMINAL), kinds.count(po.BUSY)
    return valid > 0 and valid + busy == 8 and h["edge_inflight"][0, 0, 0] == valid


def ticket_quota_full():
    c = po.make_case(nodes=3, actions=4, warps=2, path_depth=2)
    c["node_expanded"][0, 0] = 1
    c["node_expand_inflight"][0, 0] = 3
    c["edge_child"][0, 0, 0] = 1
    c["edge_n"][0, 0, 0] = 16
    c["node_expanded"][0, 1] = po.NODE_TERMINAL
    return c, {"c_pw": 1.0, "alpha_pw": 0.5}


def check_ticket_quota_full(h):
    kinds = [po.decode(h["out_selected"][0, w])[0] for w in range(2)]
    nodes = [po.decode(h["out_selected"][0, w])[2] for w in range(2)]
    valid, busy = kinds.count(po.TERMINAL), kinds.count(po.BUSY)
    return (valid > 0 and valid + busy == 2 and all(n in (0, 1) for n in nodes) and h["edge_inflight"][0, 0, 0] == valid
            and h["node_expand_inflight"][0, 0] == 3)


def two_edges_eight_warps(soft):
    def build():
        c = po.make_case(nodes=4, actions=4, warps=8, path_depth=2)
        c["node_expanded"][0, 0] = 2
        for slot, child in enumerate((1, 2)):
            c["edge_child"][0, 0, slot] = child
            c["edge_n"][0, 0, slot] = 1
            c["node_expanded"][0, child] = po.NODE_TERMINAL
        return c, {"c_pw": 0.0, "soft_winner": soft}
    return build


def check_soft_all_valid(h):
    return all(po.decode(h["out_selected"][0, w])[0] == po.TERMINAL for w in range(8))


def check_strict_valid_or_busy(h):
    kinds = [po.decode(h["out_selected"][0, w])[0] for w in range(8)]
    return kinds.count(po.TERMINAL) > 0 and kinds.count(po.TERMINAL) + kinds.count(po.BUSY) == 8


MULTI_WARP_CASES = [
    ("progressive widening: unique slots", pw_multi_warp, check_pw_multi_warp),
    ("single-edge contention", single_edge_contention, check_single_edge_contention),
    ("full ticket quota falls through", ticket_quota_full, check_ticket_quota_full),
    ("soft winner: every warp gets a claim", two_edges_eight_warps(1), check_soft_all_valid),
    ("strict winner: claims or busy", two_edges_eight_warps(0), check_strict_valid_or_busy),
]
