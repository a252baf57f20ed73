"""ctypes wrapper around the CPU oracle (``mctsnc_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke check and by the CPU-baseline legs of the
benchmark.  The product package never imports this module.

The oracle restates the reference's numba.cuda kernels (``src/mctsnc.py:1259-2375``), its game mechanics
(``src/mctsnc_game_mechanics.py:89-281``) and numba's xoroshiro128+ streams sequentially on the CPU; see the
header of ``mctsnc_oracle.c`` for the per-routine citations and for the conventions used where the reference is
undefined.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libmctsnc_oracle.so")

VARIANTS = ["ocp_thrifty", "ocp_prodigal", "acp_thrifty", "acp_prodigal"]
GAME_C4, GAME_GOMOKU = 0, 1
MAX_TREE_DEPTH = 2048

_FIELDS = {
    # name: (id, dtype, shape builder)
    "trees": (0, np.int32, lambda o: (o.T, o.cap, 1 + o.A)),
    "trees_sizes": (1, np.int32, lambda o: (o.T,)),
    "trees_depths": (2, np.int16, lambda o: (o.T, o.cap)),
    "trees_turns": (3, np.int8, lambda o: (o.T, o.cap)),
    "trees_leaves": (4, np.uint8, lambda o: (o.T, o.cap)),
    "trees_terminals": (5, np.uint8, lambda o: (o.T, o.cap)),
    "trees_outcomes": (6, np.int8, lambda o: (o.T, o.cap)),
    "trees_ns": (7, np.int32, lambda o: (o.T, o.cap)),
    "trees_ns_wins": (8, np.int32, lambda o: (o.T, o.cap)),
    "trees_boards": (9, np.int8, lambda o: (o.T, o.cap, o.m, o.n)),
    "trees_extra_infos": (10, np.int8, lambda o: (o.T, o.cap, o.extra)),
    "trees_nodes_selected": (11, np.int32, lambda o: (o.T,)),
    "trees_selected_paths": (12, np.int32, lambda o: (o.T, MAX_TREE_DEPTH + 2)),
    "trees_actions_expanded": (13, np.int16, lambda o: (o.T, o.A + 2)),
    "trees_playout_outcomes": (14, np.int32, lambda o: (o.T, 2)),
    "trees_playout_outcomes_children": (15, np.int32, lambda o: (o.T, o.A, 2)),
    "root_actions_expanded": (16, np.int16, lambda o: (o.A + 2,)),
    "root_ns": (17, np.int64, lambda o: (o.A,)),
    "actions_win_flags": (18, np.uint8, lambda o: (o.A,)),
    "actions_ns": (19, np.int64, lambda o: (o.A,)),
    "actions_ns_wins": (20, np.int64, lambda o: (o.A,)),
}

_lib = None


def build(force=False):
    """Compiles ``libmctsnc_oracle.so`` next to its source (gcc through the Makefile)."""
    src = os.path.join(_HERE, "mctsnc_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "libmctsnc_oracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = ctypes.CDLL(_LIB_PATH)
        L.mo_create.restype = ctypes.c_void_p
        L.mo_create.argtypes = [ctypes.c_int] * 8 + [ctypes.c_int64, ctypes.c_int64, ctypes.c_float, ctypes.c_uint64]
        L.mo_destroy.argtypes = [ctypes.c_void_p]
        L.mo_reset_rng.argtypes = [ctypes.c_void_p]
        L.mo_set_tree_offset.argtypes = [ctypes.c_void_p, ctypes.c_int64]
        L.mo_run.restype = ctypes.c_int
        L.mo_run.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                             ctypes.c_int64, ctypes.c_void_p]
        L.mo_field.restype = ctypes.c_void_p
        L.mo_field.argtypes = [ctypes.c_void_p, ctypes.c_int]
        for name in ("mo_cap", "mo_steps", "mo_ub_draws", "mo_plies", "mo_tree_full_events", "mo_best_n",
                     "mo_best_n_wins"):
            getattr(L, name).restype = ctypes.c_int64
            getattr(L, name).argtypes = [ctypes.c_void_p]
        for name in ("mo_error", "mo_best_action", "mo_best_win_flag", "mo_tpb_e1"):
            getattr(L, name).restype = ctypes.c_int
            getattr(L, name).argtypes = [ctypes.c_void_p]
        L.mo_rng_init_states.argtypes = [ctypes.c_void_p, ctypes.c_int64, ctypes.c_uint64]
        L.mo_rng_uniform_f32.restype = ctypes.c_float
        L.mo_rng_uniform_f32.argtypes = [ctypes.c_void_p]
        L.mo_rng_next.restype = ctypes.c_uint64
        L.mo_rng_next.argtypes = [ctypes.c_void_p]
        L.mo_replay_game.restype = ctypes.c_int
        L.mo_replay_game.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                                     ctypes.c_void_p, ctypes.c_void_p]
        _lib = L
    return _lib


def reference_max_tree_size(board_shape, extra_info_memory, max_actions, n_trees, variant, device_memory_gib):
    """The reference's memory model, ``src/mctsnc.py:350-358``."""
    extra = max(extra_info_memory, 1)
    per_state_additional = 2 + 1 + 2 * 1 + 1 + 2 * 4
    per_tree_additional = 4 + 4 + 2 * (max_actions + 2) + 4 * 2 + 4 * (MAX_TREE_DEPTH + 2)
    if "acp" in variant:
        per_tree_additional += 4 * max_actions * 2
    per_state = int(np.prod(board_shape)) + extra + 4 * (1 + max_actions) + per_state_additional
    size = (int(device_memory_gib * 1024 ** 3) - n_trees * per_tree_additional) // (per_state * n_trees)
    return min(size, 2 ** 24)


def rng_states(n, seed):
    """``create_xoroshiro128p_states(n, seed)`` as an ``uint64[n, 2]`` array (s0, s1)."""
    out = np.zeros((n, 2), dtype=np.uint64)
    lib().mo_rng_init_states(out.ctypes.data, n, ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF))
    return out


def replay_game(game, m, n, actions):
    """Plays `actions` from the empty board with the oracle's game mechanics; returns (outcomes after every action,
    final board).  Outcome 2 means "game goes on"."""
    actions = np.ascontiguousarray(actions, dtype=np.int16)
    outcomes = np.zeros(len(actions), dtype=np.int8)
    board = np.zeros((m, n), dtype=np.int8)
    rc = lib().mo_replay_game(game, m, n, actions.ctypes.data, len(actions), outcomes.ctypes.data, board.ctypes.data)
    if rc != 0:
        raise RuntimeError(f"oracle replay failed with {rc}")
    return outcomes, board


class OracleMCTSNC:
    """One search instance of the oracle; argument names follow ``MCTSNC.__init__`` (``src/mctsnc.py:199-204``)."""

    def __init__(self, state_board_shape, state_extra_info_memory, state_max_actions, n_trees=8, n_playouts=128,
                 variant="acp_prodigal", device_memory=2.0, ucb_c=2.0, seed=0, game=None, max_tree_size=None,
                 node_capacity=None, tree_offset=0, n_trees_global=None):
        self.m, self.n = state_board_shape
        self.extra = max(state_extra_info_memory, 1)
        self.A = state_max_actions
        self.T, self.P = n_trees, n_playouts
        self.variant = variant
        if game is None:
            game = GAME_C4 if self.A == self.n else GAME_GOMOKU
        self.game = game
        # a context that grows the trees [tree_offset, tree_offset + n_trees) of a search with n_trees_global trees
        self.tree_offset = int(tree_offset)
        self.n_trees_global = int(n_trees_global) if n_trees_global is not None else self.tree_offset + n_trees
        self.max_tree_size = max_tree_size if max_tree_size is not None else reference_max_tree_size(
            state_board_shape, state_extra_info_memory, state_max_actions, self.n_trees_global, variant, device_memory)
        cap = node_capacity if node_capacity is not None else min(self.max_tree_size, 1 << 16)
        self._ctx = lib().mo_create(self.m, self.n, self.extra, self.A, game, self.T, self.P, VARIANTS.index(variant),
                                    self.max_tree_size, cap, ucb_c, ctypes.c_uint64(seed & 0xFFFFFFFFFFFFFFFF))
        if not self._ctx:
            raise MemoryError("oracle allocation failed")
        self.cap = lib().mo_cap(self._ctx)
        if self.tree_offset:
            lib().mo_set_tree_offset(self._ctx, self.tree_offset)

    def __del__(self):
        if getattr(self, "_ctx", None):
            lib().mo_destroy(self._ctx)
            self._ctx = None

    def reset_rng(self):
        lib().mo_reset_rng(self._ctx)

    def run(self, root_board, root_extra_info, root_turn, steps, trace=False):
        board = np.ascontiguousarray(root_board, dtype=np.int8)
        if root_extra_info is None:
            extra_ptr, extra_len, extra = None, 0, None
        else:
            extra = np.ascontiguousarray(root_extra_info, dtype=np.int8)
            extra_ptr, extra_len = extra.ctypes.data, extra.size
        tr = np.zeros((steps, self.T, 4), dtype=np.int32) if trace else None
        err = lib().mo_run(self._ctx, board.ctypes.data, extra_ptr, extra_len, int(root_turn), int(steps),
                           tr.ctypes.data if trace else None)
        if err:
            raise RuntimeError(f"oracle error flags {err}")
        self.trace = tr
        self.best_action = lib().mo_best_action(self._ctx)
        self.best_win_flag = bool(lib().mo_best_win_flag(self._ctx))
        self.best_n = lib().mo_best_n(self._ctx)
        self.best_n_wins = lib().mo_best_n_wins(self._ctx)
        return self.best_action

    def field(self, name):
        fid, dtype, shape = _FIELDS[name]
        shape = shape(self)
        ptr = lib().mo_field(self._ctx, fid)
        n = int(np.prod(shape))
        buf = (ctypes.c_char * (n * np.dtype(dtype).itemsize)).from_address(ptr)
        return np.frombuffer(buf, dtype=dtype).reshape(shape)

    @property
    def ub_draws(self):
        return lib().mo_ub_draws(self._ctx)

    @property
    def plies(self):
        return lib().mo_plies(self._ctx)

    @property
    def tree_full_events(self):
        return lib().mo_tree_full_events(self._ctx)

    @property
    def playouts(self):
        return int(self.field("trees_ns")[:, 0].astype(np.int64).sum())
