"""Known-answer cases of the two older PUCT select kernels (virtual visits per child node), restated from the reference's
own test script (``src/puct/test_puct_gpu_v2.py:1006-1166``).  Each entry: (name, build() -> (case, select kwargs),
check(h) -> bool) where h is the case after select (numpy); every case is run for both variants."""
from oracle import puct_v2_oracle as pv


def _inflight_sum(h):
    return int(h["node_inflight"].sum()) + int(h["node_expand_inflight"].sum())


def fresh_root():
    return pv.make_case(nodes=2, actions=4, path_depth=2), {}


def check_fresh_root(h):
    return pv.decode(h["out_selected"][0, 0]) == (pv.EXPAND, 0, 0) and h["out_len"][0, 0] == 1 and h["node_expand_inflight"][0, 0] == 1


def terminal_root():
    c = pv.make_case(nodes=2, actions=4, path_depth=2)
    c["node_expanded"][0, 0] = pv.NODE_TERMINAL
    return c, {}


def check_terminal_root(h):
    kind, _, node = pv.decode(h["out_selected"][0, 0])
    return kind == pv.TERMINAL and node == 0 and h["out_len"][0, 0] == 1 and _inflight_sum(h) == 0


def invalid_child_node():
    c = pv.make_case(nodes=2, actions=4, path_depth=4)
    c["node_expanded"][0, 0] = 1
    c["node_expanded"][0, 1] = -2
    c["edge_child"][0, 0, 0] = 1
    c["edge_n"][0, 0, 0] = 1
    return c, {}


def check_invalid_rolled_back(h):
    return pv.decode(h["out_selected"][0, 0])[0] == pv.INVALID and _inflight_sum(h) == 0


def child_beyond_node_count():
    c = pv.make_case(nodes=4, actions=4, path_depth=3)
    c["node_count"][0] = 2
    c["node_expanded"][0, 0] = 1
    c["edge_child"][0, 0, 0] = 3
    c["edge_n"][0, 0, 0] = 1
    return c, {}


def fully_expanded():
    c = pv.make_case(nodes=3, actions=4, path_depth=4)
    c["node_expanded"][0, 0] = 2
    c["edge_child"][0, 0, :2] = (1, 2)
    c["edge_prior"][0, 0, :2] = (0.1, 0.9)
    c["edge_n"][0, 0, :2] = 1
    return c, {}


def check_fully_expanded(h):
    # the edge with prior 0.9 is taken, node 2 gets a visit and is expanded at slot 0
    return (pv.decode(h["out_selected"][0, 0]) == (pv.EXPAND, 0, 2) and h["out_path"][0, 0, 0] == 1 and h["out_len"][0, 0] == 2
            and h["node_inflight"][0, 2] == 1 and h["node_inflight"][0, 1] == 0 and h["node_expand_inflight"][0, 2] == 1)


def depth_limit():
    c = pv.make_case(nodes=3, actions=4, path_depth=1)
    c["node_expanded"][0, :2] = 1
    c["edge_child"][0, 0, 0] = 1
    c["edge_child"][0, 1, 0] = 2
    c["edge_n"][0, :2, 0] = 1
    return c, {}


def check_depth_limit(h):
    kind, _, node = pv.decode(h["out_selected"][0, 0])
    return kind == pv.DEPTH_LIMIT and node == 1 and h["out_len"][0, 0] == 2 and h["node_inflight"][0, 1] == 1


def widening_four_warps():
    c = pv.make_case(nodes=3, actions=4, warps=4, path_depth=2)
    c["node_expanded"][0, 0] = 1
    c["edge_child"][0, 0, 0] = 1
    c["edge_n"][0, 0, 0] = 16
    return c, {"c_pw": 1.0, "alpha_pw": 0.5}


def check_widening_four_warps(h):
    # quota ceil(sqrt(16)) = 4 with one child: three traversals get the slots 1, 2, 3, the fourth finds the quota taken
    slots = []
    for wid in range(4):
        kind, slot, node = pv.decode(h["out_selected"][0, wid])
        if kind == pv.EXPAND:
            if node != 0:
                return False
            slots.append(slot)
        elif kind != pv.INVALID:
            return False
    return sorted(slots) == [1, 2, 3] and h["node_expand_inflight"][0, 0] == 3


def edges_256():
    return pv.make_case(nodes=2, actions=256, path_depth=2), {}


def edges_257():
    return pv.make_case(nodes=2, actions=257, path_depth=2), {}


def nodes_beyond_packing():
    return pv.make_case(nodes=pv.NODE_LIMIT + 1, actions=4, path_depth=2), {}


def nodes_gated_by_count():
    c = pv.make_case(nodes=pv.NODE_LIMIT + 1, actions=4, path_depth=2)
    c["node_count"][0] = pv.NODE_LIMIT
    return c, {}


def check_expand(h):
    return pv.decode(h["out_selected"][0, 0])[0] == pv.EXPAND


def check_invalid(h):
    return pv.decode(h["out_selected"][0, 0])[0] == pv.INVALID


CASES = [
    ("fresh root expands with packed slot", fresh_root, check_fresh_root),
    ("terminal root returns terminal without virtual visits", terminal_root, check_terminal_root),
    ("invalid child node rolls the path back", invalid_child_node, check_invalid_rolled_back),
    ("child id beyond the tree's node count is invalid", child_beyond_node_count, check_invalid_rolled_back),
    ("fully expanded node: the high-prior edge is taken", fully_expanded, check_fully_expanded),
    ("depth limit returns the leaf reached", depth_limit, check_depth_limit),
    ("progressive widening: four traversals, unique slots", widening_four_warps, check_widening_four_warps),
    ("256 edges are accepted", edges_256, check_expand),
    ("257 edges are refused", edges_257, check_invalid),
    ("more nodes than the packing holds are refused", nodes_beyond_packing, check_invalid),
    ("the tree's node count gates the packed node ids", nodes_gated_by_count, check_expand),
]
