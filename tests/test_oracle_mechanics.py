"""The oracle's game mechanics (restated device functions of ``src/mctsnc_game_mechanics.py:89-281``) against games
played with the reference's CPU state classes ``C4`` and ``Gomoku`` (fixture made by
``tests/golden/make_mechanics_vectors.py``)."""
import os

import numpy as np
import pytest

from oracle import oracle as om


@pytest.mark.parametrize("name,game,shape", [("c4", om.GAME_C4, (6, 7)), ("gomoku", om.GAME_GOMOKU, (15, 15))])
def test_outcomes_after_every_move_match_the_reference_classes(golden_dir, name, game, shape):
    v = np.load(os.path.join(golden_dir, "mechanics_vectors.npz"))
    actions, outcomes, lengths, boards = (v[f"{name}_{k}"] for k in ("actions", "outcomes", "lengths", "boards"))
    finals = set()
    for g in range(len(lengths)):
        n = lengths[g]
        got, board = om.replay_game(game, shape[0], shape[1], actions[g, :n])
        assert np.array_equal(got, outcomes[g, :n]), g
        assert np.array_equal(board, boards[g]), g
        assert (got[:-1] == 2).all() and got[-1] in (-1, 0, 1)
        finals.add(int(got[-1]))
    assert {-1, 1} <= finals
    if name == "c4":
        assert 0 in finals   # the fixture holds drawn games too


def test_gomoku_overline_does_not_win():
    # six in a row is not a win (total == 4 exactly, src/mctsnc_game_mechanics.py:235), five is
    moves_plus = [(7, 3), (7, 4), (7, 5), (7, 7), (7, 8)]          # +1 leaves a gap at (7, 6)
    moves_minus = [(0, 0), (0, 2), (0, 4), (0, 6), (0, 8)]
    seq = []
    for a, b in zip(moves_plus, moves_minus):
        seq += [a[0] * 15 + a[1], b[0] * 15 + b[1]]
    seq.append(7 * 15 + 6)                                           # closes a line of SIX for +1
    out, _ = om.replay_game(om.GAME_GOMOKU, 15, 15, seq)
    assert (out == 2).all()
    seq2 = [7 * 15 + 3, 0, 7 * 15 + 4, 2, 7 * 15 + 5, 4, 7 * 15 + 6, 6, 7 * 15 + 7]   # exactly five
    out2, _ = om.replay_game(om.GAME_GOMOKU, 15, 15, seq2)
    assert out2[-1] == 1 and (out2[:-1] == 2).all()
