"""Seeded synthetic root positions: k uniform-random legal moves from the empty board, unfinished games only.

Stands in for positions met in real games (the reference ships no data set); the move mechanics follow the reference's
``C4.take_action_job`` / ``compute_outcome_job`` (``src/c4.py``) and ``Gomoku`` (``src/gomoku.py``).
"""
import numpy as np


def _c4_won(board, i, j):
    m, n = board.shape
    token = board[i, j]
    for di, dj in ((1, 0), (0, 1), (1, 1), (1, -1)):
        total = 1
        for sign in (1, -1):
            ii, jj = i + sign * di, j + sign * dj
            while 0 <= ii < m and 0 <= jj < n and board[ii, jj] == token:
                total += 1
                ii += sign * di
                jj += sign * dj
        if total >= 4:
            return True
    return False


def c4_random_roots(count, max_plies, seed, first_turn=1):
    """Returns (boards int8[count,6,7], column_fills int8[count,7], turns int8[count]).  The first player is +1, as in
    the reference's ``State`` (``src/mcts.py:63``); the turn flips after every move."""
    rng = np.random.default_rng(seed)
    boards = np.zeros((count, 6, 7), dtype=np.int8)
    fills = np.zeros((count, 7), dtype=np.int8)
    turns = np.zeros(count, dtype=np.int8)
    r = 0
    while r < count:
        k = int(rng.integers(0, max_plies + 1))
        board = np.zeros((6, 7), dtype=np.int8)
        fill = np.zeros(7, dtype=np.int8)
        turn = first_turn
        ok = True
        for _ in range(k):
            legal = np.nonzero(fill < 6)[0]
            if legal.size == 0:
                ok = False
                break
            j = int(rng.choice(legal))
            i = 5 - fill[j]
            board[i, j] = turn
            fill[j] += 1
            if _c4_won(board, i, j):
                ok = False
                break
            turn = -turn
        if not ok or (fill >= 6).all():
            continue  # finished game: draw again
        boards[r], fills[r], turns[r] = board, fill, turn
        r += 1
    return boards, fills, turns


def _gomoku_five(board, i, j):
    m, n = board.shape
    token = board[i, j]
    for di, dj in ((1, 0), (0, 1), (1, 1), (1, -1)):
        total = 0
        for sign in (1, -1):
            for k in range(1, 6):
                ii, jj = i + sign * k * di, j + sign * k * dj
                if not (0 <= ii < m and 0 <= jj < n) or board[ii, jj] != token:
                    break
                total += 1
        if total == 4:
            return True
    return False


def gomoku_random_roots(count, max_plies, seed, first_turn=1, size=15):
    """Returns (boards int8[count,15,15], turns int8[count]); Gomoku has no extra information."""
    rng = np.random.default_rng(seed)
    boards = np.zeros((count, size, size), dtype=np.int8)
    turns = np.zeros(count, dtype=np.int8)
    r = 0
    while r < count:
        k = int(rng.integers(0, max_plies + 1))
        board = np.zeros((size, size), dtype=np.int8)
        turn = first_turn
        ok = True
        for _ in range(k):
            empty = np.flatnonzero(board == 0)
            a = int(rng.choice(empty))
            board[a // size, a % size] = turn
            if _gomoku_five(board, a // size, a % size):
                ok = False
                break
            turn = -turn
        if not ok or not (board == 0).any():
            continue
        boards[r], turns[r] = board, turn
        r += 1
    return boards, turns
