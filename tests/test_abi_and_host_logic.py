"""CPU-side checks: the C-ABI library loads and exports what the header declares, the host logic of the drop-in class
follows the reference (validation messages, memory model, tpb table, budget rule), and nothing computes without a GPU."""
import ctypes
import os
import re

import numpy as np
import pytest

from mcts_numba_cuda_b200 import MCTSNC, _abi
from mcts_numba_cuda_b200.distributed import reduce_over_actions_host, shard_trees
from mcts_numba_cuda_b200.roots import c4_random_roots

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions(header, prefix):
    with open(os.path.join(ROOT, "include", header)) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(" + prefix + r"_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(_abi.LIB_PATH)
    for header, prefix, listed in (("mctsnc_b200.h", "mctsnc", _abi.EXPORTED), ("puct_b200.h", "puct", _abi.EXPORTED_PUCT),
                                   ("duct_b200.h", "duct", _abi.EXPORTED_DUCT)):
        names = declared_functions(header, prefix)
        assert sorted(listed) == names
        for name in names:
            assert hasattr(lib, name), name


def test_result_struct_layout_matches_numpy_dtype():
    assert ctypes.sizeof(_abi.Result) == _abi.RESULT_DTYPE.itemsize
    for name, _ in _abi.Result._fields_:
        assert getattr(_abi.Result, name).offset == _abi.RESULT_DTYPE.fields[name][1], name


def test_error_strings():
    lib = _abi.lib()
    assert b"bad argument" in lib.mctsnc_error_string(_abi.E_BAD_ARGUMENT)
    assert b"reachable" in lib.mctsnc_error_string(_abi.E_BAD_ROOT)
    assert lib.mctsnc_error_string(0) == b"success"


def test_bad_config_is_rejected_before_any_device_work():
    cfg = _abi.Config(board_rows=6, board_cols=7, extra_info_memory=7, max_actions=7, game=0, variant=3, n_trees=4,
                      n_playouts=100, ucb_c=2.0, device=0, seed=0, max_tree_size=1000, node_capacity=1000, max_batch=1,
                      tree_offset=0, n_trees_global=4)
    handle = ctypes.c_void_p()
    assert _abi.lib().mctsnc_create(ctypes.byref(cfg), ctypes.byref(handle)) == _abi.E_BAD_ARGUMENT  # not a power of 2
    cfg.n_playouts = 128
    cfg.n_trees_global = 2
    assert _abi.lib().mctsnc_create(ctypes.byref(cfg), ctypes.byref(handle)) == _abi.E_BAD_ARGUMENT  # shard past the end
    assert _abi.lib().mctsnc_create(None, ctypes.byref(handle)) == _abi.E_BAD_ARGUMENT


@pytest.mark.skipif(os.path.exists("/dev/nvidia0"), reason="a GPU is present")
def test_no_gpu_means_a_loud_failure_not_a_fallback():
    ai = MCTSNC((6, 7), 7, 7, search_steps_limit=10, search_time_limit=np.inf, verbose_info=False)
    with pytest.raises(_abi.MctsncError):
        ai.init_device_side_arrays()
    with pytest.raises(RuntimeError):
        ai.run(np.zeros((6, 7), np.int8), np.zeros(7, np.int8), 1)


def test_constructor_defaults_and_str():
    ai = MCTSNC((6, 7), 7, 7)
    assert (ai.search_time_limit, ai.search_steps_limit, ai.n_trees, ai.n_playouts, ai.variant) == (5.0, np.inf, 8, 128, "acp_prodigal")
    assert str(ai) == ("MCTSNC(search_time_limit=5.0, search_steps_limit=inf, n_trees=8, n_playouts=128, "
                       "variant='acp_prodigal', device_memory=2.0, ucb_c=2.0, seed: 0)")
    assert repr(ai).endswith("state_board_shape=(6, 7), state_extra_info_memory=7, state_max_actions=7)")


def test_invalid_parameters_fall_back_with_the_reference_messages(capsys):
    ai = MCTSNC((6, 7), 7, 7, n_trees=1000, n_playouts=100, variant="xyz", ucb_c=-1.0, search_time_limit=0.0)
    out = capsys.readouterr().out
    assert "[invalid param n_trees: 1000 changed to default: 8; correct range: [1, 512], correct type: <class 'int'>]" in out
    assert "[n_playouts: 100 is not a power of 2; changed to default: 128]" in out
    assert "[invalid variant: 'xyz' changed to default: 'acp_prodigal'; possible variants:" in out
    assert "[invalid param ucb_c: -1.0 changed to default: 2.0; correct range: [0.0, inf], correct type: <class 'float'>]" in out
    assert "[invalid param search_time_limit: 0.0 changed to default: 5.0; correct range: (0.0, inf], correct type: <class 'float'>]" in out
    assert (ai.n_trees, ai.n_playouts, ai.variant, ai.ucb_c, ai.search_time_limit) == (8, 128, "acp_prodigal", 2.0, 5.0)


def test_hard_limits_raise():
    with pytest.raises(ValueError, match="state board shape exceeded"):
        MCTSNC((33, 7), 7, 7)
    with pytest.raises(ValueError, match="extra info memory exceeded"):
        MCTSNC((6, 7), 5000, 7, game="c4")
    with pytest.raises(ValueError, match="max actions"):
        MCTSNC((6, 7), 7, 600, game="c4")


def test_memory_model_and_tpb_table_follow_the_reference():
    ai = MCTSNC((6, 7), 7, 7, n_trees=4, n_playouts=256, variant="acp_prodigal", device_memory=2.0)
    assert ai._memory_model() == (95, 5651185)          # per_state_memory, max_tree_size for the headline configuration
    ai._tpb_table()
    assert (ai.tpb_r, ai.tpb_s, ai.tpb_e1, ai.tpb_e2, ai.tpb_b1, ai.tpb_b2, ai.tpb_rot, ai.tpb_roa) == (64, 512, 64, 64, 8, 512, 4, 8)
    old = MCTSNC((6, 7), 7, 7, n_trees=4, n_playouts=128, variant="acp_thrifty", device_memory=1.5)
    assert old._memory_model()[1] == 4238367            # printed in extras/mctsnc_acp_thrifty_c4_1000steps.log
    gomoku = MCTSNC((15, 15), 0, 225, n_trees=4, n_playouts=256, device_memory=16.0)
    assert gomoku.game == _abi.GAME_GOMOKU
    gomoku._tpb_table()
    assert (gomoku.tpb_r, gomoku.tpb_e1, gomoku.tpb_b1, gomoku.tpb_roa) == (256, 256, 256, 256)
    assert gomoku._memory_model()[0] == 1144


def test_budget_rule():
    ai = MCTSNC((6, 7), 7, 7, search_time_limit=2.0, search_steps_limit=300)
    assert ai._steps_budget() == (300, 2.0)
    assert ai._steps_budget(forced_search_steps_limit=17) == (17, 0.0)   # a forced step count ignores the clock
    assert MCTSNC((6, 7), 7, 7)._steps_budget() == (-1, 5.0)
    assert MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=10)._steps_budget() == (10, 0.0)


def test_roots_are_seeded_legal_and_unfinished():
    a = c4_random_roots(32, 20, seed=0)
    b = c4_random_roots(32, 20, seed=0)
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    boards, fills, turns = a
    assert np.array_equal((boards != 0).sum(axis=1), fills)
    assert set(np.unique(turns)) <= {-1, 1}
    for board, fill, turn in zip(boards, fills, turns):
        stones = int(fill.sum())
        assert turn == (1 if stones % 2 == 0 else -1)
        for j in range(7):  # no floating discs
            assert (board[6 - fill[j]:, j] != 0).all() and (board[:6 - fill[j], j] == 0).all()


def test_shard_trees():
    assert [shard_trees(32, 8, r) for r in (0, 3, 7)] == [(0, 4), (12, 4), (28, 4)]
    with pytest.raises(ValueError):
        shard_trees(6, 4, 0)


def test_final_argmax_tie_rule():
    # equal keys: the stride-halving reduction keeps the left operand, so among ties the smallest bit-reversed slot wins
    flags = np.zeros(7, bool)
    n = np.array([5, 9, 9, 1, 9, 0, 9])
    w = np.array([1, 4, 4, 0, 4, 0, 4])
    expanded = np.ones(7, bool)
    assert reduce_over_actions_host(flags, n, w, expanded, thrifty=False)[0] == 4      # slots 1,2,4,6 tie: order 4,2,6,1
    expanded[0] = False                                                                 # thrifty: ordinals 0..5 = actions 1..6
    assert reduce_over_actions_host(flags, n, w, expanded, thrifty=True)[0] == 1       # ordinals 0,1,3,5 tie -> ordinal 0
    flags[3] = True
    assert reduce_over_actions_host(flags, n, w, np.ones(7, bool), thrifty=False) == (3, True, 1, 0)


def test_drop_in_import_as_top_level_module():
    """The reference's callers do `from mctsnc import MCTSNC` (src/game_runner.py:2, src/main.py:27): with the package
    directory on sys.path that import gives this implementation."""
    import subprocess
    import sys
    pkg = os.path.join(ROOT, "mcts_numba_cuda_b200")
    code = ("import sys; sys.path.insert(0, %r); from mctsnc import MCTSNC; "
            "ai = MCTSNC((6, 7), 7, 7, verbose_info=False); print(type(ai).__module__, ai.variant)" % pkg)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True).stdout.split()
    assert out == ["mctsnc", "acp_prodigal"]
