"""The drop-in ``MCTSNC`` class against matches recorded by the reference's authors on their GPU (``experiments/*.zip``,
reduced to ``tests/golden/experiment_replays.json``): the reference's own REPRODUCE_EXPERIMENT procedure
(``src/game_runner.py:86-92``: ``ai.run(board, extra_info, turn, forced_search_steps_limit)`` with the recorded step
counts), with the archive as the expected ``actions_info["best"]`` and ``performance_info``.  One instance per recorded
player, initialised once per match as ``src/main.py:181-186`` does, so the random streams run on over searches and games."""
import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC
from tests import experiment_replay as er

pytestmark = pytest.mark.gpu

FIXTURE = er.load()


def player(cfg):
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=cfg["search_time_limit"], search_steps_limit=np.inf, n_trees=cfg["n_trees"],
                n_playouts=cfg["n_playouts"], variant=cfg["variant"], device_memory=cfg["device_memory"], ucb_c=cfg["ucb_c"],
                seed=cfg["seed"], verbose_info=False)
    ai.init_device_side_arrays()
    return ai


def replay(key, side, limit):
    entry = FIXTURE[key]
    ai = player(entry[side + "_config"])
    done = 0
    for board, fills, turn, rec in list(er.searches_of(entry, side))[:limit]:
        move = ai.run(board, fills, turn, rec[1])
        best, perf = ai.actions_info["best"], ai.performance_info
        assert int(move) == best["index"] and perf["steps"] == rec[1]
        er.check(rec, best["index"], best["win_flag"], best["n_root"], best["n"], best["n_wins"], perf["playouts"],
                 perf["trees"]["max_depth"], perf["trees"]["max_size"], perf["trees"]["mean_size"], perf["trees"]["mean_depth"])
        done += 1
    return done


# Limits below the number of recorded searches mark where the record stops being reproducible: a draw equal to 1.0f makes
# the reference read legal_actions_with_count[count] (src/mctsnc.py:2061-2062); when no earlier ply of the same playout
# wrote that slot and a column is already full, what it finds is whatever its thread's local memory held before, which
# no restatement can know.  Oracle and CUDA agree with each other there (zeros) and part from the record; every search
# before that point, hundreds of such draws included, is reproduced.
@pytest.mark.parametrize("key,side,limit", [
    ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_ocp_thrifty", "ai_b", 90),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_ocp_prodigal", "ai_b", 99),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_acp_thrifty", "ai_b", 94),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_acp_prodigal", "ai_b", 108),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_2_64_ocp_thrifty", "ai_b", 91),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_4_128_acp_thrifty", "ai_b", 82),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_8_256_ocp_prodigal", "ai_b", 89),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_4_256_acp_prodigal", "ai_b", 53),
    ("mcts_5_inf_vanilla;mctsnc_5_inf_4_256_acp_prodigal", "ai_b", 66),
    ("mctsnc_5_inf_4_256_acp_thrifty;mctsnc_5_inf_4_256_acp_prodigal", "ai_a", 72),
    ("mctsnc_5_inf_4_256_acp_thrifty;mctsnc_5_inf_4_256_acp_prodigal", "ai_b", 36),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_8_256_acp_thrifty", "ai_b", 79),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_8_32_acp_prodigal", "ai_b", 97),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_2_256_ocp_prodigal", "ai_b", 90),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_4_64_ocp_thrifty", "ai_b", 79),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_1_256_acp_thrifty", "ai_b", 96),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_8_128_ocp_thrifty", "ai_b", 71),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_2_128_acp_prodigal", "ai_b", 88),
    ("mctsnc_5_inf_4_128_ocp_thrifty;mctsnc_5_inf_4_256_ocp_prodigal", "ai_a", 105),
    ("mctsnc_5_inf_4_128_ocp_thrifty;mctsnc_5_inf_4_256_ocp_prodigal", "ai_b", 107),
])
def test_recorded_matches_are_reproduced(key, side, limit):
    assert replay(key, side, limit) == limit
