"""Random games played with the reference's own CPU state classes (``C4`` in ``src/c4.py``, ``Gomoku`` in
``src/gomoku.py``): for every game the actions taken and, after every action, what ``compute_outcome()`` returned
(-1 / 0 / +1, or 2 for "game goes on").  Written to ``mechanics_vectors.npz`` next to this script; the tests replay the
actions through the oracle's restatement of the device functions of ``src/mctsnc_game_mechanics.py``.

Run once in a checkout that has the reference mounted:  python tests/golden/make_mechanics_vectors.py <reference_root>
"""
import os
import sys

import numpy as np


def play(cls, rng, n_games, max_len, want_draws=0):
    """n_games random games; with want_draws > 0 the last want_draws slots are filled with drawn games only."""
    actions = -np.ones((n_games, max_len), dtype=np.int16)
    outcomes = np.full((n_games, max_len), 3, dtype=np.int8)
    lengths = np.zeros(n_games, dtype=np.int32)
    boards = [None] * n_games
    g = 0
    while g < n_games:
        state = cls()
        k = 0
        actions[g] = -1
        outcomes[g] = 3
        while True:
            legal = [a for a in range(cls.get_max_actions()) if _legal(cls, state, a)]
            a = int(rng.choice(legal))
            state = state.take_action(a)
            out = state.compute_outcome()
            actions[g, k] = a
            outcomes[g, k] = 2 if out is None else out
            k += 1
            if out is not None:
                break
        if g >= n_games - want_draws and out != 0:
            continue  # this slot waits for a draw
        lengths[g] = k
        boards[g] = state.get_board().copy()
        g += 1
    return actions, outcomes, lengths, np.array(boards, dtype=np.int8)


def _legal(cls, state, a):
    board = state.get_board()
    if cls.__name__ == "C4":
        return state.get_extra_info()[a] < cls.M
    return board[a // cls.N, a % cls.N] == 0


def main(ref_root):
    sys.path.insert(0, os.path.join(ref_root, "src"))
    from c4 import C4
    from gomoku import Gomoku
    rng = np.random.default_rng(2024)
    out = {}
    for name, cls, n_games, max_len, draws in (("c4", C4, 300, 42, 4), ("gomoku", Gomoku, 60, 225, 0)):
        a, o, l, b = play(cls, rng, n_games, max_len, draws)
        out[f"{name}_actions"], out[f"{name}_outcomes"], out[f"{name}_lengths"], out[f"{name}_boards"] = a, o, l, b
        print(name, "games", n_games, "mean length", l.mean(), "outcomes", {v: int((o[np.arange(n_games), l - 1] == v).sum()) for v in (-1, 0, 1)})
    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "mechanics_vectors.npz"), **out)


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python " + sys.argv[0] + " <root of the reference checkout>")
    main(sys.argv[1])
