"""The allocation-free entry point ``mctsnc_search_c4_static`` against the ordinary one (``mctsnc_run`` on a fresh
handle).  It serves callers that may not allocate device memory -- code living under a framework's caching allocator,
services that allocate only at start-up -- by keeping all working memory of a search in a fixed array inside the
library.  The array is shared by all calls and keeps the previous call's contents, so the check is made on two calls
in a row: the second must not see anything of the first.  This file sorts last on purpose: a run that stops at the
first failure has then already run every other test."""
import ctypes

import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC, _abi
from mcts_numba_cuda_b200.roots import c4_random_roots

pytestmark = pytest.mark.gpu

A = 7


def static_search(board, fills, turn, variant, n_trees, n_playouts, steps, ucb_c=2.0, seed=0):
    import torch
    out = torch.full((3 * A + 4,), -7, dtype=torch.int64, device="cuda")   # the caller's buffer; the call allocates nothing
    stream = torch.cuda.current_stream().cuda_stream
    board = np.ascontiguousarray(board, dtype=np.int8)
    fills = np.ascontiguousarray(fills, dtype=np.int8)
    code = _abi.lib().mctsnc_search_c4_static(board.ctypes.data, fills.ctypes.data, int(turn), MCTSNC.VARIANTS.index(variant),
                                              n_trees, n_playouts, steps, ctypes.c_float(ucb_c), ctypes.c_uint64(seed),
                                              ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(stream))
    _abi.check(code)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def ordinary_search(board, fills, turn, variant, n_trees, n_playouts, steps, ucb_c=2.0, seed=0):
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=n_trees, n_playouts=n_playouts,
                variant=variant, ucb_c=ucb_c, seed=seed, verbose_info=False)
    ai.init_device_side_arrays()
    ai.run(board, fills, int(turn))
    r = ai._res
    return np.concatenate([r["root_ns"], r["actions_ns"], r["actions_ns_wins"],
                           [int(ai.best_action), int(ai.best_win_flag), int(ai.best_n), int(ai.best_n_wins)]]).astype(np.int64)


@pytest.mark.parametrize("variant", ["acp_prodigal", "ocp_thrifty"])
def test_static_entry_point_equals_the_ordinary_one_twice_in_a_row(variant):
    boards, fills, turns = c4_random_roots(2, 16, seed=21)
    cases = [(boards[0], fills[0], turns[0], 4, 256, 300), (boards[1], fills[1], turns[1], 3, 64, 120)]
    for board, fill, turn, n_trees, n_playouts, steps in cases:       # two different calls in a row on the shared array
        expected = ordinary_search(board, fill, turn, variant, n_trees, n_playouts, steps)
        got = static_search(board, fill, turn, variant, n_trees, n_playouts, steps)
        assert np.array_equal(got, expected)                           # integer work: exact
    board, fill, turn, n_trees, n_playouts, steps = cases[0]           # and the first one once more, after the other
    assert np.array_equal(static_search(board, fill, turn, variant, n_trees, n_playouts, steps),
                          ordinary_search(board, fill, turn, variant, n_trees, n_playouts, steps))


def test_static_entry_point_rejects_sizes_beyond_its_array():
    board, fills = np.zeros((6, 7), np.int8), np.zeros(7, np.int8)
    for n_trees, n_playouts, steps in [(5, 256, 100), (4, 512, 100), (4, 256, 513)]:
        with pytest.raises(_abi.MctsncError) as e:
            static_search(board, fills, 1, "acp_prodigal", n_trees, n_playouts, steps)
        assert e.value.code == _abi.E_CAPACITY
        assert "capacity" in str(e.value)
