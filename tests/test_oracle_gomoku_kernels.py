"""The oracle's Gomoku search against the reference's own kernels (``tests/golden/gomoku_kernel_fixtures.npz``: two
search steps driven kernel by kernel through numba's CUDA simulator, see ``tests/golden/make_gomoku_kernel_fixtures.py``).
This pins the oracle's Gomoku child creation, playouts (swap-remove move order, exactly-five rule, per-thread stream
indices), backups, 225-wide select and the final reductions to the reference's code, not only to its CPU classes."""
import numpy as np
import pytest

from oracle.oracle import OracleMCTSNC
from tests import gomoku_kernel_fixture as gk

CASES = gk.load()


def oracle_for(case, steps):
    s = gk.settings(case)
    orc = OracleMCTSNC((15, 15), 0, 225, n_trees=s["n_trees"], n_playouts=s["n_playouts"], variant="acp_prodigal",
                       ucb_c=s["ucb_c"], seed=s["seed"], max_tree_size=s["max_tree_size"], node_capacity=s["max_tree_size"])
    orc.run(s["root_board"], None, s["root_turn"], steps)
    return orc


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_two_steps_of_the_reference_kernels(name):
    case = CASES[name]
    orc = oracle_for(case, 2)
    gk.check(case, orc.field, (orc.best_action, orc.best_win_flag, orc.best_n, orc.best_n_wins))
    assert np.array_equal(orc.field("root_ns"), case["root_ns"])
    assert np.array_equal(orc.field("actions_ns"), case["actions_ns"])
    assert np.array_equal(orc.field("actions_ns_wins"), case["actions_ns_wins"])
    assert np.array_equal(orc.field("actions_win_flags").astype(bool), case["actions_win_flags"])


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_the_first_step(name):
    case = CASES[name]
    orc = oracle_for(case, 1)
    for key in ("trees_sizes", "trees_nodes_selected", "trees_playout_outcomes", "trees_playout_outcomes_children"):
        assert np.array_equal(orc.field(key), case["step0." + key]), key
