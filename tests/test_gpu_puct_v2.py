"""The two older PUCT select kernels (virtual visits per child node: preclaim and counter-CAS, ``src/puct/puct_gpu_v2.py:
573-840``) and their backup on the GPU: the reference's known-answer cases, exact agreement with the CPU restatement for
one traversal per tree, and the invariants of its stress tests (``src/puct/test_puct_gpu_v2.py:1169-1260``) for many."""
import copy

import numpy as np
import pytest

from mcts_numba_cuda_b200 import puct
from oracle import puct_oracle as po
from oracle import puct_v2_oracle as pv
from tests.puct_v2_cases import CASES

pytestmark = pytest.mark.gpu

VARIANTS = [puct.V2_PRECLAIM, puct.V2_COUNTER_CAS]


def run_select(case, variant, **kw):
    d = puct.to_device(case)
    puct.launch_select_v2(d, variant=variant, **kw)
    return d, puct.to_host(d)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("name,build,check", CASES, ids=[c[0] for c in CASES])
def test_known_answer_case(name, build, check, variant):
    case, kw = build()
    d, h = run_select(case, variant, **kw)
    assert check(h)
    puct.launch_backup_v2(d)
    h = puct.to_host(d)
    assert int(h["node_inflight"].sum()) == 0 and int(h["node_expand_inflight"].sum()) == 0


@pytest.mark.parametrize("variant", VARIANTS)
def test_select_then_backup_known_answer(variant):
    import torch
    case, _ = [c for c in CASES if c[0].startswith("fully expanded")][0][1]()
    d, h = run_select(case, variant)
    values = torch.full((1, 1, 4), 0.7, dtype=torch.float32, device="cuda")
    puct.launch_backup_v2(d, values)
    h = puct.to_host(d)
    assert h["edge_n"][0, 0, 1] == 2 and h["edge_w"][0, 0, 1] == np.float32(0.7)
    assert int(h["node_inflight"].sum()) == 0 and int(h["node_expand_inflight"].sum()) == 0


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("edges,depth", [(5, 4), (64, 6), (200, 3)])
def test_one_traversal_per_tree_equals_the_cpu_restatement(variant, edges, depth):
    base = pv.from_v3_case(po.layered_case(trees=40, edges=edges, depth=depth, warps=1, seed=edges))
    want = pv.select(copy.deepcopy(base), cpuct=1.5, c_pw=0.0, variant=variant)
    _, got = run_select(copy.deepcopy(base), variant, cpuct=1.5, c_pw=0.0)
    for key in ("out_selected", "out_path", "out_len", "node_inflight", "node_expand_inflight"):
        assert np.array_equal(got[key], want[key]), key


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("warps", [4, 8, 32])
def test_many_traversals_per_tree_keep_the_invariants(variant, warps):
    """Traversals of a tree race for the same counters: whatever the schedule, no counter goes negative, every finished
    traversal holds exactly one visit per path edge, and the backup brings all counters back to zero."""
    base = pv.from_v3_case(po.layered_case(trees=64, edges=16, depth=6, warps=warps, seed=warps))
    d, h = run_select(base, variant, cpuct=1.5, c_pw=0.0)
    assert (h["node_inflight"] >= 0).all() and (h["node_expand_inflight"] >= 0).all()
    kinds = h["out_selected"] >> pv.KIND_SHIFT
    assert np.isin(kinds, [pv.INVALID, pv.EXPAND, pv.TERMINAL, pv.DEPTH_LIMIT]).all()
    ok = kinds != pv.INVALID
    assert ok.any()
    assert int(h["node_inflight"].sum()) == int((h["out_len"][ok] - 1).sum())     # one visit per edge of the kept paths
    assert (h["out_len"][~ok] == 0).all()
    puct.launch_backup_v2(d)
    h = puct.to_host(d)
    assert int(np.abs(h["node_inflight"]).sum()) == 0 and int(np.abs(h["node_expand_inflight"]).sum()) == 0


@pytest.mark.parametrize("variant", VARIANTS)
def test_widening_tickets_are_unique_under_contention(variant):
    case = pv.make_case(trees=32, nodes=3, actions=16, warps=8, path_depth=2)
    case["node_expanded"][:, 0] = 1
    case["edge_child"][:, 0, 0] = 1
    case["edge_n"][:, 0, 0] = 25                          # quota ceil(sqrt(25)) = 5: four new slots
    d, h = run_select(case, variant, c_pw=1.0, alpha_pw=0.5)
    for t in range(32):
        slots = [pv.decode(x)[1] for x in h["out_selected"][t] if pv.decode(x)[0] == pv.EXPAND]
        assert sorted(slots) == [1, 2, 3, 4]
    assert (h["node_expand_inflight"][:, 0] == 4).all()
