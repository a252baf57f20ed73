"""The CPU oracle against matches the reference's authors recorded on their GPU (``experiments/*.zip`` of the reference,
reduced to ``tests/golden/experiment_replays.json``): every search of a match, repeated with its recorded step count in
the recorded order from one instance seeded once, must give the recorded move, visit and win counts, playouts, depths
and tree sizes.  This pins the oracle to hundreds of outputs of the reference itself, over all four variants, with the
random streams running on across searches and games, and through draws equal to 1.0f."""
import numpy as np
import pytest

from oracle.oracle import OracleMCTSNC
from tests import experiment_replay as er

FIXTURE = er.load()


def oracle_for(cfg, most_steps):
    return OracleMCTSNC((6, 7), 7, 7, n_trees=cfg["n_trees"], n_playouts=cfg["n_playouts"], variant=cfg["variant"],
                        device_memory=cfg["device_memory"], ucb_c=cfg["ucb_c"], seed=cfg["seed"],
                        node_capacity=most_steps * 7 + 16)


def replay_with_oracle(key, side, limit):
    entry = FIXTURE[key]
    cfg = entry[side + "_config"]
    todo = list(er.searches_of(entry, side))[:limit]
    orc = oracle_for(cfg, max(rec[1] for _, _, _, rec in todo))
    ub = 0
    for board, fills, turn, rec in todo:
        orc.run(board, fills, turn, rec[1])
        sizes, depths = orc.field("trees_sizes"), orc.field("trees_depths")
        valid = np.arange(depths.shape[1])[None, :] < sizes[:, None]
        er.check(rec, orc.best_action, orc.best_win_flag, orc.field("root_ns").max(), orc.best_n, orc.best_n_wins, orc.playouts,
                 depths[valid].max(), sizes.max(), float(sizes.mean()), float(depths[valid].astype(np.float64).mean()))
        ub += orc.ub_draws
    return len(todo), ub


@pytest.mark.parametrize("key,limit", [
    ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_ocp_thrifty", 90), ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_ocp_prodigal", 99),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_acp_thrifty", 40), ("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_acp_prodigal", 40),
    ("mcts_5_inf_vanilla;mctsnc_1_inf_2_64_ocp_thrifty", 60), ("mcts_5_inf_vanilla;mctsnc_1_inf_4_128_acp_thrifty", 3)])
def test_oracle_reproduces_recorded_matches(key, limit):
    done, _ = replay_with_oracle(key, "ai_b", limit)
    assert done == limit


def test_recorded_matches_include_draws_equal_to_one():
    """The 1 x 32 acp_prodigal match meets draws of exactly 1.0f within its first searches; the replay above goes through
    them, so the convention for what the reference reads there (an uninitialised local array) is the one its GPU showed."""
    _, ub = replay_with_oracle("mcts_5_inf_vanilla;mctsnc_1_inf_1_32_acp_prodigal", "ai_b", 40)
    assert ub >= 1
