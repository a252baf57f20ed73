"""The CPU restatement of the two older PUCT select kernels (preclaim, counter-CAS) and their backup on the reference's
known-answer cases (``src/puct/test_puct_gpu_v2.py:1006-1166``); no GPU needed."""
import copy

import numpy as np
import pytest

from oracle import puct_oracle as po
from oracle import puct_v2_oracle as pv
from tests.puct_v2_cases import CASES


@pytest.mark.parametrize("variant", [pv.PRECLAIM, pv.COUNTER_CAS])
@pytest.mark.parametrize("name,build,check", CASES, ids=[c[0] for c in CASES])
def test_known_answer_case(name, build, check, variant):
    case, kw = build()
    h = pv.select(case, variant=variant, **kw)
    assert check(h)
    pv.backup(h)                                       # release only
    assert int(h["node_inflight"].sum()) == 0 and int(h["node_expand_inflight"].sum()) == 0


@pytest.mark.parametrize("variant", [pv.PRECLAIM, pv.COUNTER_CAS])
def test_select_then_backup_known_answer(variant):
    # src/puct/test_puct_gpu_v2.py:1091-1119: priors 0.1 / 0.9 -> path [(0 << 8) | 1], expansion at node 2 slot 0; after the
    # backup with value 0.7: N 1 -> 2, W -> 0.7, nothing in flight
    case, _ = [c for c in CASES if c[0].startswith("fully expanded")][0][1]()
    h = pv.select(case, variant=variant)
    values = np.full((1, 1, 4), 0.7, np.float32)
    pv.backup(h, values)
    assert h["edge_n"][0, 0, 1] == 2 and h["edge_w"][0, 0, 1] == np.float32(0.7)
    assert int(h["node_inflight"].sum()) == 0 and int(h["node_expand_inflight"].sum()) == 0


def test_variants_agree_with_the_per_edge_select_when_alone():
    """One warp per tree on an acyclic tree: no traversal meets another's visits, so preclaim, counter-CAS and the per-edge
    select of the newer layout all take the same path (ties aside: the tree has none)."""
    base = po.layered_case(trees=6, edges=12, depth=5, warps=1, seed=3)
    v3 = po.select(copy.deepcopy(base), cpuct=1.5, c_pw=0.0)
    for variant in (pv.PRECLAIM, pv.COUNTER_CAS):
        h = pv.select(pv.from_v3_case(copy.deepcopy(base)), cpuct=1.5, c_pw=0.0, variant=variant)
        assert np.array_equal(h["out_path"], v3["out_path"]) and np.array_equal(h["out_len"], v3["out_len"])
        assert [pv.decode(x)[2] for x in h["out_selected"].reshape(-1)] == [po.decode(x)[2] for x in v3["out_selected"].reshape(-1)]
        assert h["node_inflight"].sum() == 6 * 5       # one visit per child on the path
