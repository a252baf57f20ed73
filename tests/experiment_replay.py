"""Replays matches recorded by the reference's authors (``tests/golden/experiment_replays.json``, made by
``tests/golden/make_experiment_replays.py`` from the reference's ``experiments/*.zip``): every MCTSNC search of a match is
repeated with its recorded number of steps, in the recorded order (one instance plays all games of a match and its random
streams run on), and must give the recorded move and statistics — the reference's own REPRODUCE_EXPERIMENT procedure
(``src/game_runner.py:86-92``) with the archive as the expected answer."""
import json
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load():
    with open(os.path.join(HERE, "golden", "experiment_replays.json")) as f:
        return json.load(f)


def searches_of(entry, side):
    """(board, column fills, turn, recorded search) for every search of instance `side` ("ai_a" / "ai_b"), in order."""
    me = entry[side]
    for game in entry["games"]:
        board, fills, turn = np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1      # black moves first, as +1
        mine_is_black = game["black"] == me
        by_ply = {s[0]: s for s in game["searches"]}
        for ply, action in enumerate(game["moves"]):
            black_moves = ply % 2 == 0
            if ply in by_ply and black_moves == mine_is_black:
                yield board.copy(), fills.copy(), turn, by_ply[ply]
            board[5 - fills[action], action] = turn
            fills[action] += 1
            turn = -turn


def check(recorded, best_action, win_flag, n_root, n, n_wins, playouts, max_depth, max_size, mean_size, mean_depth):
    _, steps, r_action, r_n_root, r_flag, r_n, r_wins, r_playouts, r_max_depth, r_max_size, r_mean_size, r_mean_depth = recorded
    got = (int(best_action), int(n_root), int(bool(win_flag)), int(n), int(n_wins), int(playouts), int(max_depth), int(max_size))
    want = (r_action, r_n_root, r_flag, r_n, r_wins, r_playouts, r_max_depth, r_max_size)
    assert got == want, (got, want)
    assert abs(mean_size - r_mean_size) < 1e-9 * max(1.0, r_mean_size) and abs(mean_depth - r_mean_depth) < 1e-9 * max(1.0, r_mean_depth)
