"""The CUDA Gomoku search against the reference's own kernels: ``tests/golden/gomoku_kernel_fixtures.npz`` holds what the
reference's ``_select`` / ``_expand_2_prodigal`` / ``_playout_acp_prodigal`` / ``_backup_*`` / ``_reduce_over_*`` kernels
(with its Gomoku device functions) produce for two search steps, run through numba's CUDA simulator by
``tests/golden/make_gomoku_kernel_fixtures.py``.  Integer work: everything must match exactly."""
import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC
from tests import gomoku_kernel_fixture as gk

pytestmark = pytest.mark.gpu

CASES = gk.load()


def searcher_for(case, steps):
    s = gk.settings(case)
    ai = MCTSNC((15, 15), 0, 225, search_time_limit=np.inf, search_steps_limit=steps, n_trees=s["n_trees"],
                n_playouts=s["n_playouts"], variant="acp_prodigal", device_memory=16.0, ucb_c=s["ucb_c"], seed=s["seed"],
                verbose_info=False, node_capacity=s["max_tree_size"])
    ai.init_device_side_arrays()
    ai.run(s["root_board"], None, s["root_turn"])
    return ai


@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_search_reproduces_two_steps_of_the_reference_kernels(name):
    case = CASES[name]
    ai = searcher_for(case, 2)
    smax = int(case["trees_sizes"].max())
    gk.check(case, lambda field: ai.export(field, max_nodes=smax), (ai.best_action, ai.best_win_flag, ai.best_n, ai.best_n_wins))
    r = ai._res
    expanded = r["actions_expanded"]
    assert np.array_equal(r["root_ns"][expanded], case["root_ns"][expanded])
    assert np.array_equal(r["actions_ns"][expanded], case["actions_ns"][expanded])
    assert np.array_equal(r["actions_ns_wins"][expanded], case["actions_ns_wins"][expanded])
    assert np.array_equal(r["actions_win_flags"][expanded], case["actions_win_flags"][expanded])


@pytest.mark.parametrize("name", sorted(CASES))
def test_cuda_search_reproduces_the_first_step(name):
    case = CASES[name]
    ai = searcher_for(case, 1)
    for key in ("trees_sizes", "trees_nodes_selected", "trees_playout_outcomes", "trees_playout_outcomes_children"):
        assert np.array_equal(ai.export(key), case["step0." + key]), key
