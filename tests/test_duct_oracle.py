"""CPU tests of the decoupled-UCT restatement (``oracle/duct_oracle.py``): hand-worked cases of the specification in
``include/duct_b200.h``.  The reference has no DUCT, so these pin the oracle to the written specification only."""
import numpy as np

from oracle import duct_oracle as do

f32 = np.float32


def one_node_case(A=8, warps=1, path_depth=4):
    d = do.make_case(1, actions=A, depth=3, nodes=8, warps=warps, path_depth=path_depth, seed=0, expanded_fraction=0.0)
    assert d["node_count"][0] == 1 and (d["child"] == -1).all()
    return d


def test_unvisited_node_follows_the_priors_and_claims_the_joint_action():
    d = one_node_case()
    d["node_prior"][0, 0, 0] = [0.05, 0.6, 0.05, 0.05, 0.05, 0.05, 0.1, 0.05]
    d["node_prior"][0, 0, 1] = [0.3, 0.05, 0.05, 0.05, 0.05, 0.05, 0.05, 0.4]
    do.select(d, cpuct=1.5)
    kind, node, joint, reason = do.decode(d["out_selected"][0, 0])
    assert (kind, node, joint, reason) == (do.KIND_EXPAND, 0, 1 * 8 + 7, do.R_OK_EXPAND)
    assert d["out_len"][0, 0] == 1 and d["out_path"][0, 0, 0] == (0 << 8) | 15
    assert d["node_inflight"][0, 0, 0, 1] == 1 and d["node_inflight"][0, 0, 1, 7] == 1 and d["node_inflight"].sum() == 2
    assert d["child"][0, 0, 15] == do.CHILD_CLAIMED


def test_score_formula_by_hand():
    prior = np.array([0.5, 0.5], f32)
    w = np.array([3.0, -1.0], f32)
    n = np.array([4, 2], np.int32)
    inflight = np.array([1, 0], np.int32)
    s = do.scores(1.5, prior, w, n, inflight, virtual_loss=3)
    # action 0: n' = 7, w' = 0, q = 0, u = 1.5 * 0.5 * sqrt(9) / 8;  action 1: n' = 2, q = -0.5, u = 1.5 * 0.5 * 3 / 3
    assert s[0] == f32(f32(0.75) * f32(3.0)) / f32(8) and s[1] == f32(-0.5) + f32(f32(0.75) * f32(3.0)) / f32(3)


def test_ties_go_to_the_lowest_action_and_second_warp_sees_the_virtual_loss():
    d = one_node_case(warps=2)
    d["node_prior"][0, 0] = f32(1 / 8)
    do.select(d, cpuct=1.0, virtual_loss=1)
    k0, _, j0, _ = do.decode(d["out_selected"][0, 0])
    k1, _, j1, _ = do.decode(d["out_selected"][0, 1])
    assert (k0, j0) == (do.KIND_EXPAND, 0)            # all equal: action 0 for both players
    assert (k1, j1) == (do.KIND_EXPAND, 1 * 8 + 1)    # action 0 now carries a loss in flight: next lowest for both
    assert d["node_inflight"][0, 0].sum() == 4


def test_a_claimed_joint_action_makes_later_traversals_busy_and_they_give_back_their_claims():
    d = one_node_case(warps=2)
    d["node_prior"][0, 0, :, 0] = 0.93
    d["node_prior"][0, 0, :, 1:] = 0.01
    do.select(d, cpuct=5.0, virtual_loss=1)
    assert do.decode(d["out_selected"][0, 0])[0] == do.KIND_EXPAND
    kind, node, joint, reason = do.decode(d["out_selected"][0, 1])
    assert (kind, joint, reason) == (do.KIND_BUSY, 0, do.R_BUSY_EXPAND_INFLIGHT) and d["out_len"][0, 1] == 0
    assert d["node_inflight"][0, 0].sum() == 2     # only the expanding traversal still holds claims


def test_backup_is_zero_sum_installs_children_and_returns_every_claim():
    d = do.make_case(3, actions=8, depth=6, nodes=64, warps=1, seed=3, expanded_fraction=0.05)
    before_n, before_w = d["node_n"].copy(), d["node_w"].copy()
    do.select(d, cpuct=1.5, virtual_loss=3)
    values = np.random.default_rng(0).uniform(-1, 1, d["out_path"].shape).astype(f32)
    new_child = d["node_count"].copy().reshape(3, 1)
    do.backup(d, values, new_child, virtual_loss=3)
    assert (d["node_inflight"] == 0).all() and (d["child"] != do.CHILD_CLAIMED).all()
    for t in range(3):
        kind, node, joint, _ = do.decode(d["out_selected"][t, 0])
        length = d["out_len"][t, 0]
        assert d["node_n"][t].sum() - before_n[t].sum() == 2 * length
        assert abs(float((d["node_w"][t] - before_w[t]).sum())) < 1e-5      # what one player gains the other loses
        if kind == do.KIND_EXPAND:
            assert d["child"][t, node, joint] == new_child[t, 0]


def test_terminal_and_depth_limit():
    d = one_node_case(path_depth=4)
    d["node_terminal"][0, 0] = 1
    do.select(d)
    assert do.decode(d["out_selected"][0, 0])[:2] == (do.KIND_TERMINAL, 0) and d["out_len"][0, 0] == 0
    d = do.make_case(1, actions=2, depth=9, nodes=600, warps=1, path_depth=3, seed=1, expanded_fraction=1.0)
    do.select(d)
    kind, node, _, reason = do.decode(d["out_selected"][0, 0])
    assert (kind, reason) == (do.KIND_DEPTH_LIMIT, do.R_OK_DEPTH_LIMIT) and d["out_len"][0, 0] == 3
