"""Drop-in ``MCTSNC`` for the reference's ``src/mctsnc.py``: same constructor, ``init_device_side_arrays()``,
``run(root_board, root_extra_info, root_turn, forced_search_steps_limit)``, ``actions_info`` / ``performance_info`` and
``_json_dump`` -- with the search loop running inside ``libmctsnc_b200.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/mctsnc_b200.h``) instead of 4-6 numba.cuda launches per step driven from Python.

Put this directory on ``sys.path`` and the reference's ``game_runner.py`` / ``main.py`` import it unchanged
(``from mctsnc import MCTSNC``).  There is no CPU fallback: without the built library or without a CUDA device,
``init_device_side_arrays()`` raises.

Deliberate differences from the reference, all additive:

* the game is chosen from the shapes (6x7 board with 7 actions: Connect 4) or the keyword ``game=``; the reference
  switches games by editing comments in ``src/mctsnc_game_mechanics.py:59-87``;
* hard limit violations raise ``ValueError`` with the reference's message (the reference calls ``sys.exit`` without
  importing ``sys``, ``src/mctsnc.py:238-249``);
* keyword-only extras: ``device``, ``max_batch`` and ``run_batch`` (many roots in one launch), ``tree_offset`` /
  ``n_trees_global`` (root-parallel sharding over several GPUs), ``node_capacity``.
"""
import ctypes
import json
import time

import numpy as np
from numpy import inf

try:  # imported as top-level module `mctsnc` (drop-in) or as part of the package
    from . import _abi
except ImportError:  # pragma: no cover - exercised by the drop-in import test
    import _abi

__version__ = "0.1.0"


def _dict_to_str(d, indent=0):
    """Vertical rendering of a dictionary, one entry per line, as the reference's ``utils.dict_to_str`` prints it."""
    pad = indent * " "
    out = pad + "{"
    for i, key in enumerate(d):
        out += "\n" + pad + "  " + str(key) + ": " + str(d[key]) + ("," if i < len(d) - 1 else "")
    return out + "\n" + pad + "}"


class MCTSNC:
    """Monte Carlo Tree Search with many concurrent trees and playouts on one GPU (four variants), API of the
    reference class ``MCTSNC`` (``src/mctsnc.py:174-563``)."""

    VARIANTS = ["ocp_thrifty", "ocp_prodigal", "acp_thrifty", "acp_prodigal"]
    DEFAULT_SEARCH_TIME_LIMIT = 5.0
    DEFAULT_SEARCH_STEPS_LIMIT = np.inf
    DEFAULT_N_TREES = 8
    DEFAULT_N_PLAYOUTS = 128
    DEFAULT_VARIANT = VARIANTS[-1]
    DEFAULT_DEVICE_MEMORY = 2.0
    DEFAULT_UCB_C = 2.0
    DEFAULT_SEED = 0
    DEFAULT_VERBOSE_DEBUG = False
    DEFAULT_VERBOSE_INFO = True
    MAX_STATE_BOARD_SHAPE = (32, 32)
    MAX_STATE_EXTRA_INFO_MEMORY = 4096
    MAX_STATE_MAX_ACTIONS = 512
    MAX_TREE_SIZE = 2 ** 24
    MAX_N_TREES = 512
    MAX_N_PLAYOUTS = 512
    MAX_TREE_DEPTH = 2048
    CUDA_TPB_DEFAULT = 512  # MAX_THREADS_PER_BLOCK // 2 of every CUDA GPU since sm_20 (src/mctsnc.py:281)

    def __init__(self, state_board_shape, state_extra_info_memory, state_max_actions,
                 search_time_limit=DEFAULT_SEARCH_TIME_LIMIT, search_steps_limit=DEFAULT_SEARCH_STEPS_LIMIT,
                 n_trees=DEFAULT_N_TREES, n_playouts=DEFAULT_N_PLAYOUTS, variant=DEFAULT_VARIANT,
                 device_memory=DEFAULT_DEVICE_MEMORY, ucb_c=DEFAULT_UCB_C, seed=DEFAULT_SEED,
                 verbose_debug=DEFAULT_VERBOSE_DEBUG, verbose_info=DEFAULT_VERBOSE_INFO,
                 action_index_to_name_function=None, *, game=None, device=0, max_batch=1, tree_offset=0,
                 n_trees_global=None, node_capacity=None, threads_per_tree=0):
        self.cuda_tpb_default = self.CUDA_TPB_DEFAULT
        self.state_board_shape = tuple(int(x) for x in state_board_shape)
        if self.state_board_shape[0] > self.MAX_STATE_BOARD_SHAPE[0] or self.state_board_shape[1] > self.MAX_STATE_BOARD_SHAPE[1]:
            raise ValueError("[MCTSNC.__init__(): exiting due to allowed state board shape exceeded]")
        self._extra_info_given = int(state_extra_info_memory)
        self.state_extra_info_memory = max(int(state_extra_info_memory), 1)
        if self.state_extra_info_memory > self.MAX_STATE_EXTRA_INFO_MEMORY:
            raise ValueError("[MCTSNC.__init__(): exiting due to allowed state extra info memory exceeded]")
        self.state_max_actions = int(state_max_actions)
        if self.state_max_actions > self.MAX_STATE_MAX_ACTIONS:
            raise ValueError("[MCTSNC.__init__(): exiting due to allowed state max actions memory exceeded]")
        if self.state_max_actions > self.cuda_tpb_default:
            raise ValueError("[MCTSNC.__init__(): exiting due to state max actions exceeding half of cuda default tpb]")
        self.search_time_limit = search_time_limit
        self._validate_param("search_time_limit", float, True, 0.0, False, np.inf, self.DEFAULT_SEARCH_TIME_LIMIT)
        self.search_steps_limit = float(search_steps_limit)
        self._validate_param("search_steps_limit", float, True, 0.0, False, np.inf, self.DEFAULT_SEARCH_STEPS_LIMIT)
        self.n_trees = n_trees
        self._validate_param("n_trees", int, False, 1, False, self.MAX_N_TREES, self.DEFAULT_N_TREES)
        if n_playouts <= 0 or 2 ** np.round(np.log2(n_playouts)) != n_playouts:
            invalid_n_playouts = n_playouts
            n_playouts = self.DEFAULT_N_PLAYOUTS
            print(f"[n_playouts: {invalid_n_playouts} is not a power of 2; changed to default: {n_playouts}]")
        self.n_playouts = n_playouts
        self._validate_param("n_playouts", int, False, 1, False, self.MAX_N_PLAYOUTS, self.DEFAULT_N_PLAYOUTS)
        if variant not in self.VARIANTS:
            invalid_variant = variant
            variant = self.DEFAULT_VARIANT
            print(f"[invalid variant: '{invalid_variant}' changed to default: '{variant}'; possible variants: {self.VARIANTS}]")
        self.variant = variant
        self.ucb_c = ucb_c
        self._validate_param("ucb_c", float, False, 0.0, False, np.inf, self.DEFAULT_UCB_C)
        self.device_memory = device_memory * 1024 ** 3
        self._validate_param("device_memory", float, True, 0.0, False, np.inf, self.DEFAULT_DEVICE_MEMORY)
        self.seed = seed
        self.verbose_debug = verbose_debug
        self._validate_param("verbose_debug", bool, False, False, False, True, self.DEFAULT_VERBOSE_DEBUG)
        self.verbose_info = verbose_info
        self._validate_param("verbose_info", bool, False, False, False, True, self.DEFAULT_VERBOSE_INFO)
        self.action_index_to_name_function = action_index_to_name_function
        # extras
        self.game = self._detect_game(game)
        self.device = int(device)
        self.max_batch = int(max_batch)
        self.tree_offset = int(tree_offset)
        self.n_trees_global = int(n_trees_global) if n_trees_global is not None else self.tree_offset + int(self.n_trees)
        self.node_capacity = node_capacity
        self.threads_per_tree = int(threads_per_tree)
        self._handle = None
        self._handle_capacity = 0

    # ------------------------------------------------------------------------------------------------ host logic
    def _detect_game(self, game):
        if game is not None:
            names = {"c4": _abi.GAME_C4, "connect4": _abi.GAME_C4, "gomoku": _abi.GAME_GOMOKU}
            if isinstance(game, str):
                if game.lower() not in names:
                    raise ValueError(f"[MCTSNC.__init__(): unknown game '{game}'; known: {sorted(names)}]")
                return names[game.lower()]
            return int(game)
        m, n = self.state_board_shape
        if self.state_max_actions == n and self._extra_info_given == n:
            return _abi.GAME_C4       # column fills as extra info, one action per column (src/c4.py)
        if self.state_max_actions == m * n:
            return _abi.GAME_GOMOKU   # one action per cell (src/gomoku.py)
        raise ValueError("[MCTSNC.__init__(): cannot tell the game from the shapes; pass game='c4' or game='gomoku']")

    def _validate_param(self, name, ptype, leq, low, geq, high, default):
        """Type and range check with fallback to the default and a message, as ``src/mctsnc.py:283-296``."""
        value = getattr(self, name)
        try:
            invalid = value <= low if leq else value < low
            if not invalid:
                invalid = value >= high if geq else value > high
        except TypeError:
            invalid = True
        if not invalid:
            invalid = not isinstance(value, ptype)
        if invalid:
            correct_range_str = ("(" if leq else "[") + f"{low}, {high}" + (")" if geq else "]")
            setattr(self, name, default)
            print(f"[invalid param {name}: {value} changed to default: {default}; correct range: {correct_range_str}, correct type: {ptype}]")

    def __str__(self):
        return (f"MCTSNC(search_time_limit={self.search_time_limit}, search_steps_limit={self.search_steps_limit}, "
                f"n_trees={self.n_trees}, n_playouts={self.n_playouts}, variant='{self.variant}', "
                f"device_memory={np.round(self.device_memory / 1024**3, 2)}, ucb_c={self.ucb_c}, seed: {self.seed})")

    def __repr__(self):
        return (f"{str(self)}, state_board_shape={self.state_board_shape}, "
                f"state_extra_info_memory={self.state_extra_info_memory}, state_max_actions={self.state_max_actions})")

    def _memory_model(self):
        """``per_state_memory`` and ``max_tree_size`` exactly as ``src/mctsnc.py:350-358`` computes them."""
        per_state_additional = 2 + 1 + 2 * 1 + 1 + 2 * 4
        per_tree_additional = 4 + 4 + 2 * (self.state_max_actions + 2) + 4 * 2 + 4 * (self.MAX_TREE_DEPTH + 2)
        if "acp" in self.variant:
            per_tree_additional += 4 * self.state_max_actions * 2
        per_state = int(np.prod(self.state_board_shape)) + self.state_extra_info_memory + 4 * (1 + self.state_max_actions) \
            + per_state_additional
        max_tree_size = (int(self.device_memory) - self.n_trees * per_tree_additional) // (per_state * self.n_trees)
        return per_state, min(max_tree_size, self.MAX_TREE_SIZE)

    def _tpb_table(self):
        """Threads-per-block table of ``src/mctsnc.py:360-370`` (kept as attributes; only tpb_e1 and tpb_roa influence
        results: the index of the OCP child-pick stream and the width of the final argmax)."""
        tpb_board = int(2 ** np.ceil(np.log2(np.prod(self.state_board_shape))))
        tpb_extra_info = int(2 ** np.ceil(np.log2(self.state_extra_info_memory))) if self.state_extra_info_memory > 0 else 1
        tpb_max_actions = int(2 ** np.ceil(np.log2(self.state_max_actions)))
        self.tpb_r = min(max(tpb_board, tpb_extra_info), self.cuda_tpb_default)
        self.tpb_s = self.cuda_tpb_default
        self.tpb_e1 = min(max(self.tpb_r, tpb_max_actions), self.cuda_tpb_default)
        self.tpb_e2 = self.tpb_r
        self.tpb_b1 = tpb_max_actions
        self.tpb_b2 = self.cuda_tpb_default
        self.tpb_rot = int(2 ** np.ceil(np.log2(self.n_trees)))
        self.tpb_roa = tpb_max_actions

    def _steps_budget(self, forced_search_steps_limit=np.inf):
        """(steps_limit, time_limit) for the C ABI following ``src/mctsnc.py:597-601``; -1 / 0.0 mean "none"."""
        if forced_search_steps_limit < np.inf:
            return int(forced_search_steps_limit), 0.0
        steps = int(self.search_steps_limit) if self.search_steps_limit < np.inf else -1
        tlim = float(self.search_time_limit) if self.search_time_limit < np.inf else 0.0
        return steps, tlim

    def _needed_capacity(self, steps):
        """A search of s steps creates at most s * max_actions nodes besides the root."""
        if steps < 0:
            return self.max_tree_size
        return min(self.max_tree_size, steps * self.state_max_actions + 1 + self.state_max_actions)

    # ------------------------------------------------------------------------------------------------ device side
    def init_device_side_arrays(self, node_capacity=None):
        """Allocates the tree pools on the device and (re)creates the random streams (``src/mctsnc.py:318-407``)."""
        if self.verbose_info:
            print(f"[MCTSNC._init_device_side_arrays()... for {self}]")
        t1 = time.time()
        per_state_memory, self.max_tree_size = self._memory_model()
        self._tpb_table()
        if node_capacity is None:
            node_capacity = self.node_capacity
        if node_capacity is None:
            steps, _ = self._steps_budget()
            node_capacity = self._needed_capacity(steps)
        self._create_handle(int(node_capacity))
        t2 = time.time()
        if self.verbose_info:
            print(f"[MCTSNC._init_device_side_arrays() done; time: {t2 - t1} s, per_state_memory: {per_state_memory} B,  calculated max_tree_size: {self.max_tree_size}]")

    def _create_handle(self, node_capacity):
        self._destroy_handle()
        cfg = _abi.Config()
        cfg.board_rows, cfg.board_cols = self.state_board_shape
        cfg.extra_info_memory = self.state_extra_info_memory
        cfg.max_actions = self.state_max_actions
        cfg.game = self.game
        cfg.variant = self.VARIANTS.index(self.variant)
        cfg.n_trees = int(self.n_trees)
        cfg.n_playouts = int(self.n_playouts)
        cfg.ucb_c = float(self.ucb_c)
        cfg.device = self.device
        cfg.seed = int(self.seed) & 0xFFFFFFFFFFFFFFFF
        cfg.max_tree_size = int(self.max_tree_size)
        cfg.node_capacity = int(max(2, min(node_capacity, self.max_tree_size)))
        cfg.max_batch = self.max_batch
        cfg.tree_offset = self.tree_offset
        cfg.n_trees_global = self.n_trees_global
        cfg.threads_per_tree = self.threads_per_tree
        handle = ctypes.c_void_p()
        _abi.check(_abi.lib().mctsnc_create(ctypes.byref(cfg), ctypes.byref(handle)))
        self._handle = handle
        self._handle_capacity = cfg.node_capacity

    def _destroy_handle(self):
        if getattr(self, "_handle", None):
            _abi.lib().mctsnc_destroy(self._handle)
            self._handle = None
            self._handle_capacity = 0

    def __del__(self):
        try:
            self._destroy_handle()
        except Exception:
            pass

    def _require_handle(self, steps):
        if self._handle is None:
            raise RuntimeError("[MCTSNC: init_device_side_arrays() has to be called before run()]")
        if self._needed_capacity(steps) > self._handle_capacity:
            # a forced step count beyond what the pools were sized for: grow them, keeping the random streams
            # as a fresh init would not (documented difference: streams restart)
            self._create_handle(self._needed_capacity(steps))

    def reset_random_streams(self):
        """Re-creates the xoroshiro128+ streams from the seed, the effect a fresh ``init_device_side_arrays()`` has on
        the reference's generators (``src/mctsnc.py:390-394``), without re-allocating."""
        _abi.check(_abi.lib().mctsnc_reset_rng(self._handle))

    def run(self, root_board, root_extra_info, root_turn, forced_search_steps_limit=np.inf):
        """One search from one root; returns the best action (``src/mctsnc.py:409-434`` and the four ``_run_*`` loops)."""
        print(f"MCTSNC RUN... [{self}]")
        t1 = time.time()
        steps_limit, time_limit = self._steps_budget(forced_search_steps_limit)
        self._require_handle(steps_limit)
        board = np.ascontiguousarray(root_board, dtype=np.int8)
        if board.shape != self.state_board_shape:
            raise ValueError(f"[MCTSNC.run(): root board of shape {board.shape}, expected {self.state_board_shape}]")
        extra = None
        if root_extra_info is not None:
            extra = np.ascontiguousarray(root_extra_info, dtype=np.int8)
            if extra.size != self.state_extra_info_memory:
                raise ValueError(f"[MCTSNC.run(): root extra info of {extra.size} bytes, expected {self.state_extra_info_memory}]")
        res = _abi.Result()
        _abi.check(_abi.lib().mctsnc_run(self._handle, board.ctypes.data, extra.ctypes.data if extra is not None else None,
                                         int(root_turn), steps_limit, time_limit, ctypes.byref(res)))
        self._adopt_result(res)
        t2 = time.time()
        self.time_total = t2 - t1
        # the reference builds the two dictionaries only when it prints them (src/mctsnc.py:731-733); they cost nothing
        # here, so they are always there for a caller like game_runner.py
        self._make_actions_info()
        self._make_performance_info()
        if self.verbose_info:
            print(f"[actions info:\n{_dict_to_str(self.actions_info)}]")
            print(f"[performance info:\n{_dict_to_str(self.performance_info)}]")
        best_action_label = str(self.best_action)
        if self.action_index_to_name_function is not None:
            best_action_label += f" ({self.action_index_to_name_function(self.best_action)})"
        print(f"MCTSNC RUN DONE. [time: {self.time_total} s; best action: {best_action_label}, best win_flag: {self.best_win_flag}, best n: {self.best_n}, best n_wins: {self.best_n_wins}, best q: {self.best_q}]")
        return self.best_action

    def _adopt_result(self, res):
        A = self.state_max_actions
        self._res = {
            "root_ns": np.array(res.root_ns[:A], dtype=np.int64), "actions_ns": np.array(res.actions_ns[:A], dtype=np.int64),
            "actions_ns_wins": np.array(res.actions_ns_wins[:A], dtype=np.int64),
            "actions_win_flags": np.array(res.actions_win_flags[:A], dtype=bool),
            "actions_expanded": np.array(res.actions_expanded[:A], dtype=bool),
            "playouts": int(res.playouts), "plies": int(res.plies), "ub_draws": int(res.ub_draws), "status": int(res.status),
            "max_depth": int(res.max_depth), "total_nodes": int(res.total_nodes), "depth_sum": int(res.depth_sum),
            "max_size": int(res.max_size), "device_ms": float(res.device_ms),
            "stage_ms": [float(x) for x in res.stage_ms], "reduce_ms": [float(x) for x in res.reduce_ms]}
        self.best_action = np.int16(res.best_action)
        self.best_win_flag = bool(res.best_win_flag)
        self.best_n = np.int64(res.best_n)
        self.best_n_wins = np.int64(res.best_n_wins)
        self.best_q = self.best_n_wins / self.best_n if self.best_n > 0 else np.nan
        self.steps = int(res.steps)
        self.status = int(res.status)
        self.ub_draws = int(res.ub_draws)
        self.device_time = float(res.device_ms) * 1e-3
        # The loop runs on the device in one piece: its CUDA-event time is the loop time.  The per-stage times of the
        # reference (host clocks around each launch, src/mctsnc.py:606-686) are here the time a tree's thread block spent in
        # each stage, counted on the device (mean over the trees, which run side by side); the two reductions are timed
        # with CUDA events.
        self.time_loop = self.device_time
        self.time_select, self.time_expand, self.time_playout, self.time_backup = (1e-3 * float(x) for x in res.stage_ms)
        self.time_reduce_over_trees, self.time_reduce_over_actions = (1e-3 * float(x) for x in res.reduce_ms)

    def _make_actions_info(self):
        """``actions_info`` with the keys of ``src/mctsnc.py:496-563`` (one layout for thrifty and prodigal: keyed by action)."""
        r = self._res
        actions_info = {}
        best_entry = None
        for a in range(self.state_max_actions):
            if not r["actions_expanded"][a]:
                continue
            entry = {}
            entry["name"] = self.action_index_to_name_function(a) if self.action_index_to_name_function else str(a)
            entry["n_root"] = int(r["root_ns"][a])
            entry["win_flag"] = bool(r["actions_win_flags"][a])
            entry["n"] = int(r["actions_ns"][a])
            entry["n_wins"] = int(r["actions_ns_wins"][a])
            entry["q"] = entry["n_wins"] / entry["n"] if entry["n"] > 0 else np.nan
            entry["ucb"] = entry["q"] + self.ucb_c * np.sqrt(np.log(entry["n_root"]) / entry["n"]) if entry["n"] > 0 else np.inf
            actions_info[a] = entry
            if a == self.best_action:
                best_entry = {"index": int(a), **entry}
        actions_info["best"] = best_entry
        self.actions_info = actions_info
        return actions_info

    _make_actions_info_thrifty = _make_actions_info
    _make_actions_info_prodigal = _make_actions_info

    def _make_performance_info(self):
        """``performance_info`` with the keys of ``src/mctsnc.py:448-494``; adds ``device_times_[ms]`` and ``plies``."""
        r = self._res
        performance_info = {}
        performance_info["steps"] = int(self.steps)
        performance_info["steps_per_second"] = self.steps / self.time_total
        performance_info["playouts"] = int(r["playouts"])
        performance_info["playouts_per_second"] = performance_info["playouts"] / self.time_total
        ms = 10.0 ** 3
        steps = max(self.steps, 1)
        times_info = {"total": ms * self.time_total, "loop": ms * self.time_loop,
                      "reduce_over_trees": ms * self.time_reduce_over_trees,
                      "reduce_over_actions": ms * self.time_reduce_over_actions, "mean_loop": ms * self.time_loop / steps,
                      "mean_select": ms * self.time_select / steps, "mean_expand": ms * self.time_expand / steps,
                      "mean_playout": ms * self.time_playout / steps, "mean_backup": ms * self.time_backup / steps}
        performance_info["times_[ms]"] = times_info
        total_size = r["total_nodes"]
        performance_info["trees"] = {"count": int(self.n_trees), "mean_depth": r["depth_sum"] / max(total_size, 1),
                                     "max_depth": int(r["max_depth"]), "mean_size": total_size / self.n_trees,
                                     "max_size": int(r["max_size"])}
        performance_info["device"] = {"loop_ms": r["device_ms"], "plies": r["plies"], "ub_draws": r["ub_draws"],
                                      "status": r["status"],
                                      "playouts_per_second": r["playouts"] / (r["device_ms"] * 1e-3) if r["device_ms"] > 0 else np.nan}
        self.performance_info = performance_info
        return performance_info

    # ------------------------------------------------------------------------------------------------ batch form
    def run_batch(self, root_boards, root_extra_infos, root_turns, steps=None, reseed=True):
        """Searches ``len(root_boards)`` roots at once (one launch); returns a structured array with one
        ``mctsnc_result`` per root (fields of ``include/mctsnc_b200.h``).  With ``reseed`` every search starts from freshly
        seeded streams, i.e. equals ``init_device_side_arrays(); run(root)`` of the reference."""
        if steps is None:
            steps, _ = self._steps_budget()
        if steps < 0:
            raise ValueError("[MCTSNC.run_batch(): a finite number of steps is needed]")
        boards = np.ascontiguousarray(root_boards, dtype=np.int8)
        batch = boards.shape[0]
        if boards.shape[1:] != self.state_board_shape:
            raise ValueError(f"[MCTSNC.run_batch(): boards of shape {boards.shape[1:]}, expected {self.state_board_shape}]")
        extras = None
        if root_extra_infos is not None:
            extras = np.ascontiguousarray(root_extra_infos, dtype=np.int8).reshape(batch, self.state_extra_info_memory)
        turns = np.ascontiguousarray(root_turns, dtype=np.int8).reshape(batch)
        self._require_handle(steps)
        out = np.zeros(batch, dtype=_abi.RESULT_DTYPE)
        _abi.check(_abi.lib().mctsnc_run_batch(self._handle, batch, boards.ctypes.data,
                                               extras.ctypes.data if extras is not None else None, turns.ctypes.data,
                                               int(steps), 1 if reseed else 0, out.ctypes.data))
        return out

    # ------------------------------------------------------------------------------------------------ tree export
    _EXPORT = {"trees": (0, np.int32), "trees_sizes": (1, np.int32), "trees_depths": (2, np.int16),
               "trees_turns": (3, np.int8), "trees_leaves": (4, np.uint8), "trees_terminals": (5, np.uint8),
               "trees_outcomes": (6, np.int8), "trees_ns": (7, np.int32), "trees_ns_wins": (8, np.int32),
               "trees_boards": (9, np.int8), "trees_extra_infos": (10, np.int8), "trees_nodes_selected": (11, np.int32),
               "trees_selected_paths": (12, np.int32), "trees_actions_expanded": (13, np.int16),
               "trees_playout_outcomes": (14, np.int32), "trees_playout_outcomes_children": (15, np.int32)}

    SLICE_STEPS = 32  # steps a block runs of one tree before it takes another from the work queue (batched launches)

    def launch_geometry(self):
        """Geometry of the last search launch: threads per tree, resident blocks per SM, SMs of the device and the bytes
        of device memory the handle holds.  A Connect-4 batch with more trees than ``blocks_per_sm * sm_count`` and more
        than ``SLICE_STEPS`` steps runs as a persistent grid fed by the work queue."""
        if self._handle is None:
            raise RuntimeError("[MCTSNC: init_device_side_arrays() has to be called first]")
        i32, i64 = ctypes.c_int32, ctypes.c_int64
        thr, per_sm, sms, nbytes = i32(0), i32(0), i32(0), i64(0)
        _abi.check(_abi.lib().mctsnc_query(self._handle, ctypes.byref(thr), ctypes.byref(per_sm), ctypes.byref(sms),
                                           ctypes.byref(nbytes)))
        return {"threads_per_tree": thr.value, "blocks_per_sm": per_sm.value, "sm_count": sms.value,
                "device_bytes": nbytes.value}

    def trace_slices(self, max_records):
        """Diagnostic: record every slice of the following batched launches that go through the work queue
        (``max_records`` = 0 switches it off); see ``read_slices``."""
        if self._handle is None:
            raise RuntimeError("[MCTSNC: init_device_side_arrays() has to be called first]")
        _abi.check(_abi.lib().mctsnc_trace_slices(self._handle, int(max_records)))
        self._trace_cap = int(max_records)

    def read_slices(self):
        """Slices of the last batched launch as int64[n, 4]: tree, start ns, end ns (device global timer),
        (SM id << 32) | steps."""
        cap = getattr(self, "_trace_cap", 0)
        out = np.zeros((max(cap, 1), 4), dtype=np.int64)
        n = ctypes.c_int32(0)
        _abi.check(_abi.lib().mctsnc_read_slices(self._handle, out.ctypes.data, cap, ctypes.byref(n)))
        return out[:n.value]

    def export(self, name, search=0, max_nodes=None):
        """Device arrays of the last run in the reference's formats (what ``_json_dump`` copies to the host)."""
        fid, dtype = self._EXPORT[name]
        T, A = int(self.n_trees), self.state_max_actions
        if max_nodes is None:
            sizes = np.zeros(T, dtype=np.int32)
            _abi.check(_abi.lib().mctsnc_export(self._handle, search, 1, sizes.ctypes.data, 1))
            max_nodes = int(sizes.max())
        m, n = self.state_board_shape
        shape = {"trees": (T, max_nodes, 1 + A), "trees_sizes": (T,), "trees_boards": (T, max_nodes, m, n),
                 "trees_extra_infos": (T, max_nodes, self.state_extra_info_memory), "trees_nodes_selected": (T,),
                 "trees_selected_paths": (T, self.MAX_TREE_DEPTH + 2), "trees_actions_expanded": (T, A + 2),
                 "trees_playout_outcomes": (T, 2), "trees_playout_outcomes_children": (T, A, 2)}.get(name, (T, max_nodes))
        out = np.zeros(shape, dtype=dtype)
        _abi.check(_abi.lib().mctsnc_export(self._handle, search, fid, out.ctypes.data, max_nodes))
        return out

    def _json_dump(self, fname):
        """Writes the trees of the last run as json with the keys of ``src/mctsnc.py:2384-2452``."""
        if self.verbose_info:
            print(f"JSON DUMP... [to file: {fname}]")
        t1 = time.time()
        d = {"n_trees": self.n_trees, "n_playouts": self.n_playouts, "variant": self.variant,
             "search_time_limit": self.search_time_limit if self.search_time_limit < np.inf else "inf",
             "search_steps_limit": self.search_steps_limit if self.search_steps_limit < np.inf else "inf",
             "ucb_c": self.ucb_c, "seed": self.seed, "device_memory": self.device_memory}
        sizes = self.export("trees_sizes")
        size_max = int(sizes.max())
        depths = self.export("trees_depths", max_nodes=size_max)
        depth_max = int(max(depths[i, :sizes[i]].max() for i in range(int(self.n_trees))))
        paths = self.export("trees_selected_paths")
        short_paths = paths[:, :depth_max + 2].copy()
        short_paths[:, -1] = paths[:, -1]
        d["trees"] = self.export("trees", max_nodes=size_max).tolist()
        d["trees_sizes"] = sizes.tolist()
        d["trees_depths"] = depths.tolist()
        for name in ("trees_turns", "trees_ns", "trees_ns_wins"):
            d[name] = self.export(name, max_nodes=size_max).tolist()
        d["trees_nodes_selected"] = self.export("trees_nodes_selected").tolist()
        d["trees_selected_paths"] = short_paths.tolist()
        d["trees_actions_expanded"] = self.export("trees_actions_expanded").tolist()
        d["trees_playout_outcomes"] = self.export("trees_playout_outcomes").tolist()
        if "acp" in self.variant:
            d["trees_playout_outcomes_children"] = self.export("trees_playout_outcomes_children").tolist()
        with open(fname, "w+") as f:
            json.dump(d, f, indent=2)
        t2 = time.time()
        if self.verbose_info:
            print(f"JSON DUMP DONE. [time: {t2 - t1} s]")
