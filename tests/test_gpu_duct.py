"""GPU tests of the decoupled-UCT (DUCT) select / backup (``include/duct_b200.h``) against the CPU restatement of the same
specification.  The reference has no DUCT: this is parity with the library's own written semantics.  With one warp per
tree the schedule is deterministic and everything must match bit for bit (float32 scores and value sums included);
with several warps the results depend on the schedule and the invariants of the claim protocol are checked."""
import numpy as np
import pytest

from mcts_numba_cuda_b200 import duct
from mcts_numba_cuda_b200.puct import to_device, to_host
from oracle import duct_oracle as do

pytestmark = pytest.mark.gpu

STATE_KEYS = ("child", "node_w", "node_n", "node_inflight", "out_selected", "out_len")


def assert_same(host, ref):
    for k in STATE_KEYS:
        assert np.array_equal(host[k], ref[k]), k
    for t in range(ref["out_len"].shape[0]):
        for w in range(ref["out_len"].shape[1]):
            n = ref["out_len"][t, w]
            assert np.array_equal(host["out_path"][t, w, :n], ref["out_path"][t, w, :n])


@pytest.mark.parametrize("actions,virtual_loss,cpuct,seed", [(8, 1, 1.5, 0), (8, 3, 1.5, 1), (16, 1, 0.7, 2), (3, 2, 4.0, 3)])
def test_one_warp_per_tree_matches_the_specification_exactly(actions, virtual_loss, cpuct, seed):
    import torch
    case = do.grow_case(24, actions=actions, nodes=256, rounds=160, terminal_depth=3, seed=seed, cpuct=cpuct,
                        virtual_loss=virtual_loss)
    ref = do.copy_case(case)
    d = to_device(case)
    duct.launch_select(d, cpuct=cpuct, virtual_loss=virtual_loss)
    torch.cuda.synchronize()
    do.select(ref, cpuct=cpuct, virtual_loss=virtual_loss)
    assert_same(to_host(d), ref)
    assert len(set(do.decode(ref["out_selected"])[0].ravel().tolist())) >= 2     # expansions and terminals both occur
    values = np.random.default_rng(seed).uniform(-1, 1, case["out_path"].shape).astype(np.float32)
    new_child = np.where(case["node_count"] < 256, case["node_count"], -1).astype(np.int32).reshape(-1, 1)
    duct.launch_backup(d, torch.from_numpy(values).cuda(), torch.from_numpy(new_child).cuda(), virtual_loss=virtual_loss)
    torch.cuda.synchronize()
    do.backup(ref, values, new_child, virtual_loss=virtual_loss)
    assert_same(to_host(d), ref)
    assert (ref["node_inflight"] == 0).all()


def test_growing_trees_from_the_root_stays_equal_to_the_specification():
    """120 rounds of select -> expand -> backup from a bare root: the search the kernels are for."""
    import torch
    trees, A, nodes, rounds, vl = 6, 8, 128, 120, 3
    rng = np.random.default_rng(7)
    case = do.make_case(trees, actions=A, depth=5, nodes=nodes, warps=1, path_depth=8, seed=5, expanded_fraction=0.0)
    case["node_prior"][:] = rng.dirichlet([0.3] * A, size=(trees, nodes, 2)).astype(np.float32)
    ref = do.copy_case(case)
    d = to_device(case)
    depth_of = np.zeros((trees, nodes), np.int32)
    kinds_seen = set()
    for r in range(rounds):
        duct.launch_select(d, cpuct=1.5, virtual_loss=vl)
        do.select(ref, cpuct=1.5, virtual_loss=vl)
        kind, node, joint, _ = do.decode(ref["out_selected"])
        kinds_seen.update(kind.ravel().tolist())
        values = rng.uniform(-1, 1, ref["out_path"].shape).astype(np.float32)
        new_child = np.full((trees, 1), -1, np.int32)
        for t in range(trees):
            if kind[t, 0] == do.KIND_EXPAND and ref["node_count"][t] < nodes:
                kid = int(ref["node_count"][t])
                new_child[t, 0] = kid
                depth_of[t, kid] = depth_of[t, node[t, 0]] + 1
                terminal = 1 if depth_of[t, kid] >= 5 else 0
                ref["node_terminal"][t, kid] = terminal
                ref["node_count"][t] += 1
        d["node_terminal"].copy_(torch.from_numpy(ref["node_terminal"]))
        d["node_count"].copy_(torch.from_numpy(ref["node_count"]))
        duct.launch_backup(d, torch.from_numpy(values).cuda(), torch.from_numpy(new_child).cuda(), virtual_loss=vl)
        do.backup(ref, values, new_child, virtual_loss=vl)
        if r % 20 == 19:
            torch.cuda.synchronize()
            assert_same(to_host(d), ref)
    assert {do.KIND_EXPAND, do.KIND_TERMINAL} <= kinds_seen
    assert ref["node_count"].min() > 40 and (ref["node_inflight"] == 0).all()


@pytest.mark.parametrize("warps,virtual_loss", [(8, 1), (32, 3)])
def test_many_warps_keep_the_claim_protocol(warps, virtual_loss):
    import torch
    A = 8
    case = do.grow_case(64, actions=A, nodes=256, rounds=100, terminal_depth=5, warps=warps, seed=11)
    clean = do.copy_case(case)
    d = to_device(case)
    duct.launch_select(d, cpuct=1.5, virtual_loss=virtual_loss)
    torch.cuda.synchronize()
    h = to_host(d)
    kind, node, joint, reason = do.decode(h["out_selected"])
    assert np.isin(kind, (do.KIND_EXPAND, do.KIND_TERMINAL, do.KIND_DEPTH_LIMIT, do.KIND_BUSY)).all()
    assert (h["out_len"][kind == do.KIND_BUSY] == 0).all()
    assert (h["node_inflight"] >= 0).all()
    # every path entry holds one claim per player
    assert h["node_inflight"].sum() == 2 * virtual_loss * h["out_len"].sum()
    for t in range(64):
        slots = [(int(node[t, w]), int(joint[t, w])) for w in range(warps) if kind[t, w] == do.KIND_EXPAND]
        assert len(slots) == len(set(slots))                                   # one expansion per joint action
        assert (h["child"][t] == do.CHILD_CLAIMED).sum() == len(slots)
        for n_, j_ in slots:
            assert h["child"][t, n_, j_] == do.CHILD_CLAIMED and clean["child"][t, n_, j_] == do.CHILD_NONE
        for w in range(warps):      # paths are chains of existing children
            for e in range(1, h["out_len"][t, w]):
                prev = int(h["out_path"][t, w, e - 1])
                assert clean["child"][t, prev >> 8, prev & 0xFF] == int(h["out_path"][t, w, e]) >> 8
    assert (kind == do.KIND_EXPAND).sum() >= 64 * 2      # concurrent traversals spread over several joint actions
    # releasing without values restores the untouched trees
    duct.launch_backup(d, None, None, virtual_loss=virtual_loss)
    torch.cuda.synchronize()
    h = to_host(d)
    for k in ("child", "node_w", "node_n", "node_inflight"):
        assert np.array_equal(h[k], clean[k]), k


def test_bad_shapes_are_refused():
    case = do.make_case(2, actions=8, depth=3, nodes=32, warps=1, seed=0)
    d = to_device(case)
    d["warps"] = 33
    with pytest.raises(RuntimeError):
        duct.launch_select(d)
