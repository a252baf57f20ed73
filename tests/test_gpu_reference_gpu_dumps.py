"""The CUDA search against what the reference's own numba.cuda ``MCTSNC`` produced on a B200 (``tests/reference_gpu_dumps.py``,
``tests/golden/reference_gpu_dumps.npz``): same roots, seed and step counts, compared array by array.  Integer work: exact."""
import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC
from tests import reference_gpu_dumps as rd

pytestmark = pytest.mark.gpu

CASES = rd.load()


@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_search_reproduces_the_reference_on_b200(name):
    case = CASES[name]
    s = rd.settings(case)
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=s["steps"], n_trees=s["n_trees"],
                n_playouts=s["n_playouts"], variant=s["variant"], device_memory=0.125, ucb_c=2.0, seed=0, verbose_info=False)
    ai.init_device_side_arrays()
    ai.run(s["board"], s["fills"], s["turn"])
    smax = int(case["trees_sizes"].max())
    rd.check(case, lambda name: ai.export(name, max_nodes=smax), (ai.best_action, ai.best_win_flag, ai.best_n, ai.best_n_wins))
    # the per-action sums behind actions_info: by action for prodigal variants, by ordinal among the root's expanded
    # actions for thrifty ones (src/mctsnc.py:2223-2296)
    r = ai._res
    acts = np.flatnonzero(r["actions_expanded"])
    if "prodigal" in s["variant"]:
        for key in ("root_ns", "actions_ns", "actions_ns_wins"):
            assert np.array_equal(r[key][acts], case[key][acts]), key
    else:
        for key in ("root_ns", "actions_ns", "actions_ns_wins"):
            assert np.array_equal(r[key][acts], case[key][:len(acts)]), key
