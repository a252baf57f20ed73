"""The drop-in class under the reference's OWN match driver: ``GameRunner`` (``src/game_runner.py``) and the ``C4`` state
class (``src/c4.py``) are imported unmodified from the copy that ``baseline/install_reference.py`` places under
``baseline/_ref/src``, with this package's directory ahead of it on ``sys.path`` so that the driver's
``from mctsnc import MCTSNC`` (``src/game_runner.py:2``) binds this library's class.

The match replayed is one the reference's authors recorded on their GPU between two MCTSNC players
(``experiments/*[mctsnc_5_inf_4_128_ocp_thrifty;mctsnc_5_inf_4_256_ocp_prodigal;C4_6x7;100].zip``, reduced in
``tests/golden/experiment_replays.json``).  ``GameRunner`` is given the recorded step counts as ``experiment_info_old``,
which is how the reference reproduces an experiment (``src/main.py:168-170``, ``src/game_runner.py:86-92``, ``:124-130``);
the games it plays must then be the recorded ones move for move, with the recorded statistics of every search."""
import contextlib
import io
import os
import sys

import numpy as np
import pytest

from tests import experiment_replay as er

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SRC = os.path.join(ROOT, "baseline", "_ref", "src")
PACKAGE_DIR = os.path.join(ROOT, "mcts_numba_cuda_b200")
MATCH = "mctsnc_5_inf_4_128_ocp_thrifty;mctsnc_5_inf_4_256_ocp_prodigal"
N_GAMES = 2     # game 1: player A moves first; game 2: player B does


@contextlib.contextmanager
def reference_driver_on_path():
    """``sys.path`` as a user of the reference would set it up to switch to this library: the package directory (which
    holds ``mctsnc.py``) first, the reference's ``src`` after it."""
    saved_path, saved_modules = list(sys.path), {k: sys.modules.get(k) for k in ("mctsnc", "game_runner", "c4", "mcts", "utils")}
    for k in saved_modules:
        sys.modules.pop(k, None)
    sys.path[:0] = [PACKAGE_DIR, REF_SRC]
    try:
        yield
    finally:
        sys.path[:] = saved_path
        for k, v in saved_modules.items():
            sys.modules.pop(k, None)
            if v is not None:
                sys.modules[k] = v


@pytest.mark.skipif(not os.path.exists(os.path.join(REF_SRC, "game_runner.py")),
                    reason="no copy of the reference under baseline/_ref (python baseline/install_reference.py)")
def test_reference_game_runner_replays_a_recorded_match_with_the_drop_in_class():
    entry = er.load()[MATCH]
    with reference_driver_on_path():
        import mctsnc
        from c4 import C4
        from game_runner import GameRunner
        assert os.path.dirname(os.path.abspath(mctsnc.__file__)) == PACKAGE_DIR          # this library's class ...
        assert sys.modules["game_runner"].MCTSNC is mctsnc.MCTSNC                        # ... is the one the driver sees

        def player(cfg):   # as src/main.py:63-144 builds its instances, init_device_side_arrays() once (:181-186)
            ai = mctsnc.MCTSNC(C4.get_board_shape(), C4.get_extra_info_memory(), C4.get_max_actions(),
                               search_time_limit=cfg["search_time_limit"], search_steps_limit=np.inf, n_trees=cfg["n_trees"],
                               n_playouts=cfg["n_playouts"], variant=cfg["variant"], device_memory=cfg["device_memory"],
                               ucb_c=cfg["ucb_c"], seed=cfg["seed"], verbose_info=False,
                               action_index_to_name_function=C4.action_index_to_name)
            ai.init_device_side_arrays()
            return ai

        ai_a, ai_b = player(entry["ai_a_config"]), player(entry["ai_b_config"])
        assert str(ai_a) == entry["ai_a"] and str(ai_b) == entry["ai_b"]                 # the strings the experiment hash uses
        # the recorded step counts in the layout of the reference's archives
        old = {"games_infos": {}}
        for g, game in enumerate(entry["games"][:N_GAMES], start=1):
            rounds = {}
            for ply, steps, *_ in game["searches"]:
                rounds.setdefault(str(ply // 2 + 1), {})[("black" if ply % 2 == 0 else "white") + "_performance_info"] = {"steps": steps}
            old["games_infos"][str(g)] = {"moves_rounds": rounds}
        for g, game in enumerate(entry["games"][:N_GAMES], start=1):
            a_starts = (g - 1) % 2 == 0                                                   # src/main.py:194-196
            black, white = (ai_a, ai_b) if a_starts else (ai_b, ai_a)
            assert game["black"] == str(black)
            with contextlib.redirect_stdout(io.StringIO()):
                outcome, info = GameRunner(C4, black, white, g, N_GAMES, old).run()
            assert outcome == game["outcome"]
            recorded = {s[0]: s for s in game["searches"]}
            moves = []
            for r in range(1, len(info["moves_rounds"]) + 1):
                rnd = info["moves_rounds"][str(r)]
                for colour in ("black", "white"):
                    if colour + "_best_action_info" not in rnd:
                        continue
                    best, perf = rnd[colour + "_best_action_info"], rnd[colour + "_performance_info"]
                    ply = len(moves)
                    moves.append(int(best["index"]))
                    er.check(recorded[ply], best["index"], best["win_flag"], best["n_root"], best["n"], best["n_wins"],
                             perf["playouts"], perf["trees"]["max_depth"], perf["trees"]["max_size"],
                             perf["trees"]["mean_size"], perf["trees"]["mean_depth"])
                    assert perf["steps"] == recorded[ply][1]
            assert moves == game["moves"]
