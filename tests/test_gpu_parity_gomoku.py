"""GPU parity for Gomoku 15x15: the CUDA search against the CPU oracle, bit for bit.  The reference ships no Gomoku tree
dumps (its experiment archives for Gomoku are missing), so these searches are pinned through the oracle only: its game
mechanics are checked against the reference's ``Gomoku`` class and its search skeleton against the Connect-4 dumps."""
import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC
from mcts_numba_cuda_b200.roots import gomoku_random_roots
from oracle.oracle import OracleMCTSNC

pytestmark = pytest.mark.gpu

NODE_FIELDS = ["trees_depths", "trees_turns", "trees_leaves", "trees_terminals", "trees_ns", "trees_ns_wins", "trees",
               "trees_boards"]


def make_pair(variant, n_trees, n_playouts, steps, seed=0, max_batch=1):
    ai = MCTSNC((15, 15), 0, 225, search_time_limit=np.inf, search_steps_limit=steps, n_trees=n_trees,
                n_playouts=n_playouts, variant=variant, device_memory=16.0, seed=seed, verbose_info=False, max_batch=max_batch)
    ai.init_device_side_arrays()
    orc = OracleMCTSNC((15, 15), 0, 225, n_trees=n_trees, n_playouts=n_playouts, variant=variant, device_memory=16.0,
                       seed=seed, node_capacity=steps * 225 + 230)
    return ai, orc


def compare(ai, orc, search=0):
    sizes = orc.field("trees_sizes")
    assert np.array_equal(ai.export("trees_sizes", search), sizes)
    smax = int(sizes.max())
    valid = np.arange(smax)[None, :] < sizes[:, None]
    for name in NODE_FIELDS:
        mine = ai.export(name, search, max_nodes=smax)
        ref = np.array(orc.field(name))[:, :smax].copy()
        ref[~valid] = -1 if name == "trees" else 0
        if name == "trees":
            ref[:, :, 1:][orc.field("trees_leaves")[:, :smax] != 0] = -1
        assert np.array_equal(mine, ref), name
    assert np.array_equal(ai.export("trees_outcomes", search, max_nodes=smax)[:, 1:][valid[:, 1:]],
                          orc.field("trees_outcomes")[:, 1:smax][valid[:, 1:]])
    assert np.array_equal(ai.export("trees_nodes_selected", search), orc.field("trees_nodes_selected"))
    assert np.array_equal(ai.export("trees_actions_expanded", search), orc.field("trees_actions_expanded"))
    assert np.array_equal(ai.export("trees_playout_outcomes", search), orc.field("trees_playout_outcomes"))
    paths, ref_paths = ai.export("trees_selected_paths", search), orc.field("trees_selected_paths")
    for t in range(len(sizes)):
        n = ref_paths[t, -1]
        assert paths[t, -1] == n and np.array_equal(paths[t, :n], ref_paths[t, :n])
    if "acp" in ai.variant:
        assert np.array_equal(ai.export("trees_playout_outcomes_children", search), orc.field("trees_playout_outcomes_children"))


@pytest.mark.parametrize("variant", MCTSNC.VARIANTS)
def test_gomoku_search_matches_oracle_from_empty_board(variant):
    steps = 8 if "acp" in variant else 40
    ai, orc = make_pair(variant, 2, 32, steps)
    board = np.zeros((15, 15), np.int8)
    best = ai.run(board, None, 1)
    orc.run(board, None, 1, steps)
    compare(ai, orc)
    assert int(best) == orc.best_action
    assert (ai.best_win_flag, int(ai.best_n), int(ai.best_n_wins)) == (orc.best_win_flag, orc.best_n, orc.best_n_wins)
    assert ai._res["playouts"] == orc.playouts
    assert ai._res["plies"] == orc.plies
    assert ai._res["ub_draws"] == orc.ub_draws


@pytest.mark.parametrize("variant", ["acp_thrifty", "ocp_prodigal"])
def test_gomoku_random_roots_match_oracle(variant):
    boards, turns = gomoku_random_roots(6, 120, seed=4)
    steps = 6 if "acp" in variant else 30
    for b in range(len(boards)):
        ai, orc = make_pair(variant, 2, 32, steps, seed=b)
        best = ai.run(boards[b], None, int(turns[b]))
        orc.run(boards[b], None, int(turns[b]), steps)
        compare(ai, orc)
        assert int(best) == orc.best_action


@pytest.mark.parametrize("variant,root_index,steps", [("acp_prodigal", 0, 8), ("acp_thrifty", 1, 8), ("acp_prodigal", 1, 40)])
def test_gomoku_headline_shape_4_trees_256_playouts_matches_oracle(variant, root_index, steps):
    """The launch shape of BASELINE's Gomoku configuration (4 trees x 256 playouts, device_memory 16 GiB): up to 225
    children x 256 games per tree and step through the persistent playout grid, compared with the oracle field by field
    after 8 steps, and after 40 (trees three levels deep, 9 000 nodes each, 2 M playouts).  The oracle searches run on host
    threads meanwhile (the ctypes calls release the interpreter lock)."""
    from concurrent.futures import ThreadPoolExecutor
    boards, turns = gomoku_random_roots(2, 30, seed=11)
    board, turn = boards[root_index], int(turns[root_index])
    ai, orc = make_pair(variant, 4, 256, steps, seed=0)
    with ThreadPoolExecutor(max_workers=1) as ex:
        fut = ex.submit(orc.run, board, None, turn, steps)
        best = ai.run(board, None, turn)
        again = ai.run(board, None, turn)      # streams run on: a different search, must still be a valid one
        fut.result()
    assert ai.status & 4 == 0 and int(again) >= 0
    ai.reset_random_streams()
    best2 = ai.run(board, None, turn)
    assert int(best2) == int(best)
    compare(ai, orc)
    assert int(best) == orc.best_action
    assert (ai.best_win_flag, int(ai.best_n), int(ai.best_n_wins)) == (orc.best_win_flag, orc.best_n, orc.best_n_wins)
    assert ai._res["playouts"] == orc.playouts and ai._res["plies"] == orc.plies and ai._res["ub_draws"] == orc.ub_draws


def nearly_full_board(n_empty, seed):
    """A 15x15 position without any line of five (stones in an XXOO pattern shifted by two per row) with n_empty holes."""
    i, j = np.meshgrid(np.arange(15), np.arange(15), indexing="ij")
    board = np.where(((2 * i + j) % 4) < 2, 1, -1).astype(np.int8)
    holes = np.random.default_rng(seed).choice(225, size=n_empty, replace=False)
    board.reshape(-1)[holes] = 0
    return board


@pytest.mark.parametrize("n_empty,variant", [(4, "acp_prodigal"), (5, "ocp_thrifty"), (3, "acp_thrifty")])
def test_gomoku_nearly_full_boards(n_empty, variant):
    """Few legal moves: terminal (drawn) children, terminal nodes selected again and again, games ending in draws."""
    steps = 60
    ai, orc = make_pair(variant, 3, 64, steps, seed=7)
    board = nearly_full_board(n_empty, seed=n_empty)
    best = ai.run(board, None, -1)
    orc.run(board, None, -1, steps)
    compare(ai, orc)
    assert int(best) == orc.best_action
    assert orc.field("trees_terminals").any()


def test_gomoku_batch_equals_single_runs():
    boards, turns = gomoku_random_roots(4, 60, seed=2)
    steps = 5
    ai, _ = make_pair("acp_prodigal", 2, 32, steps, seed=3, max_batch=4)
    out = ai.run_batch(boards, None, turns, steps=steps, reseed=True)
    for b in range(len(boards)):
        orc = OracleMCTSNC((15, 15), 0, 225, n_trees=2, n_playouts=32, variant="acp_prodigal", device_memory=16.0, seed=3,
                           node_capacity=steps * 225 + 230)
        orc.run(boards[b], None, int(turns[b]), steps)
        compare(ai, orc, search=b)
        assert out["best_action"][b] == orc.best_action and out["playouts"][b] == orc.playouts


def test_gomoku_overlines_are_not_wins_in_playouts():
    """Rows of six stones on the board (they cannot arise by play, but the search does not mind): a stone added at either
    end makes a row of seven, which the reference does not count as a win (it looks at most five stones either way and
    wants exactly four, ``src/mctsnc_game_mechanics.py:220-272``).  The playouts meet this in all four directions."""
    board = np.zeros((15, 15), np.int8)
    board[7, 2:8] = 1                                   # horizontal
    board[1:7, 12] = 1                                  # vertical
    for k in range(6):
        board[8 + k, 2 + k] = 1                         # diagonal, (8,2) .. (13,7)
        board[13 - k, 9 + k] = 1                        # anti-diagonal, (13,9) .. (8,14)
    # as many stones of the other side, none of them next to another
    spots = [(0, c) for c in range(0, 15, 2)] + [(14, c) for c in range(0, 15, 2)] + [(r, 10) for r in range(2, 7, 2)] + \
            [(3, c) for c in range(0, 10, 2)]
    for r, c in spots[:int((board == 1).sum())]:
        assert board[r, c] == 0
        board[r, c] = -1
    assert (board == 1).sum() == (board == -1).sum() == 24
    steps = 5
    for seed, turn in ((0, 1), (1, -1)):
        ai, orc = make_pair("acp_prodigal", 1, 64, steps, seed=seed)
        best = ai.run(board, None, turn)
        orc.run(board, None, turn, steps)
        compare(ai, orc)
        assert int(best) == orc.best_action and ai._res["plies"] == orc.plies
        assert (ai.best_win_flag, int(ai.best_n), int(ai.best_n_wins)) == (orc.best_win_flag, orc.best_n, orc.best_n_wins)
