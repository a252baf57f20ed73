"""The oracle against what the reference's own numba.cuda kernels produced on a B200 (``tests/reference_gpu_dumps.py``,
``tests/golden/reference_gpu_dumps.npz``): 256 playouts, non-empty roots, all four variants, and the headline search of
2000 steps -- none of which the two dumps shipped with the reference cover."""
import pytest

from oracle.oracle import OracleMCTSNC
from tests import reference_gpu_dumps as rd

CASES = rd.load()


@pytest.mark.parametrize("name", sorted(CASES))
def test_oracle_reproduces_the_reference_on_b200(name):
    case = CASES[name]
    s = rd.settings(case)
    orc = OracleMCTSNC((6, 7), 7, 7, n_trees=s["n_trees"], n_playouts=s["n_playouts"], variant=s["variant"], device_memory=0.125,
                       ucb_c=2.0, seed=0, node_capacity=s["steps"] * 7 + 8)
    orc.run(s["board"], s["fills"], s["turn"], s["steps"])
    rd.check(case, orc.field, (orc.best_action, orc.best_win_flag, orc.best_n, orc.best_n_wins))
