"""The CPU restatement of the PUCT select / backup on the reference's known-answer cases (no GPU needed)."""
import copy

import numpy as np
import pytest

from oracle import puct_oracle as po
from tests.puct_cases import MULTI_WARP_CASES, SINGLE_WARP_CASES


@pytest.mark.parametrize("name,build,check", SINGLE_WARP_CASES + MULTI_WARP_CASES, ids=[c[0] for c in SINGLE_WARP_CASES + MULTI_WARP_CASES])
def test_known_answer_case(name, build, check):
    case, kw = build()
    h = po.select(case, **kw)
    assert check(h)
    po.backup(h)                      # release only
    assert int(h["edge_inflight"].sum()) == 0
    if "quota" not in name:
        assert int(h["node_expand_inflight"].sum()) == 0


def test_select_then_backup_known_answer():
    # src/puct/test_puct_gpu_v2.py:1091-1119 moved to the v3 layout: priors 0.1 / 0.9 -> path [(0 << 8) | 1], expansion at
    # node 2 slot 0; after the backup with value 0.7: N 1 -> 2, W -> 0.7, nothing in flight
    c = po.make_case(nodes=3, actions=4, path_depth=4)
    c["node_expanded"][0, 0] = 2
    c["edge_child"][0, 0, :2] = (1, 2)
    c["edge_prior"][0, 0, :2] = (0.1, 0.9)
    c["edge_n"][0, 0, :2] = 1
    h = po.select(c)
    assert h["out_path"][0, 0, 0] == 1 and po.decode(h["out_selected"][0, 0])[:3] == (po.EXPAND, 0, 2)
    values = np.full((1, 1, 4), 0.7, np.float32)
    po.backup(h, values)
    assert h["edge_n"][0, 0, 1] == 2 and h["edge_w"][0, 0, 1] == np.float32(0.7)
    assert int(h["edge_inflight"].sum()) == 0 and int(h["node_expand_inflight"].sum()) == 0


def test_layered_workload_is_acyclic_and_seeded():
    a = po.layered_case(trees=3, edges=8, depth=5, warps=2, seed=1)
    b = po.layered_case(trees=3, edges=8, depth=5, warps=2, seed=1)
    assert all(np.array_equal(a[k], b[k]) for k in a if hasattr(a[k], "dtype"))
    child = a["edge_child"][0]
    nodes = child.shape[0]
    expanded = a["node_expanded"][0] > 0
    assert (child[expanded] > np.arange(nodes)[expanded][:, None]).all()      # children lie in later levels
    assert np.allclose(a["edge_prior"].sum(axis=2), 1.0, atol=1e-5)
    h = po.select(copy.deepcopy(a), cpuct=1.5, c_pw=0.0)
    kinds = [po.decode(x)[0] for x in h["out_selected"].reshape(-1)]
    assert all(k == po.TERMINAL for k in kinds) and (h["out_len"] == 6).all()
