"""ctypes binding of ``libmctsnc_b200.so`` (declarations: ``include/mctsnc_b200.h``).

The pattern follows the reference's own precedent for native code, ``src/puct/puct_gpu_v3_cpp.py:84-156``: a lazily
loaded shared library, raw pointers, integer return codes turned into ``RuntimeError``.  There is no fallback: if the
library is missing or cannot be loaded, importing a searcher fails with the reason.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MCTSNC_B200_LIB") or os.path.join(HERE, "libmctsnc_b200.so")

MAX_ACTIONS = 512
GAME_C4, GAME_GOMOKU = 0, 1
VARIANTS = ["ocp_thrifty", "ocp_prodigal", "acp_thrifty", "acp_prodigal"]
STATUS_TREE_FULL, STATUS_UB_DRAW, STATUS_INTERNAL = 1, 2, 4

E_BAD_ARGUMENT, E_UNSUPPORTED, E_NO_MEMORY, E_BAD_ROOT, E_CAPACITY, E_NO_DEVICE = -1, -2, -3, -4, -5, -6

# symbols declared in include/mctsnc_b200.h; the CPU test-suite checks that the library exports every one of them
EXPORTED = ["mctsnc_create", "mctsnc_destroy", "mctsnc_reset_rng", "mctsnc_run", "mctsnc_run_batch",
            "mctsnc_search_batch_device", "mctsnc_finish_batch_device", "mctsnc_launch_batch_device",
            "mctsnc_reduce_trees_device", "mctsnc_export", "mctsnc_export_rng",
            "mctsnc_query", "mctsnc_search_c4_static", "mctsnc_trace_slices", "mctsnc_read_slices",
            "mctsnc_exchange_create", "mctsnc_exchange_connect", "mctsnc_exchange_allreduce", "mctsnc_exchange_status",
            "mctsnc_exchange_destroy", "mctsnc_error_string"]
EXCHANGE_HANDLE_BYTES, EXCHANGE_TIMEOUT = 64, 1
# the PUCT entry points keep the names of the reference's native library (include/puct_b200.h)
EXPORTED_PUCT = ["puct_select_winner_recalc_launch", "puct_select_virtual_loss_launch", "puct_backup_launch",
                 "puct_cpp_cuda_error_string", "puct_v2_select_launch", "puct_v2_backup_launch"]
# decoupled-UCT select for simultaneous moves: no counterpart in the reference (include/duct_b200.h)
EXPORTED_DUCT = ["duct_select_launch", "duct_backup_launch"]


class Config(ctypes.Structure):
    _fields_ = [("board_rows", ctypes.c_int32), ("board_cols", ctypes.c_int32), ("extra_info_memory", ctypes.c_int32),
                ("max_actions", ctypes.c_int32), ("game", ctypes.c_int32), ("variant", ctypes.c_int32),
                ("n_trees", ctypes.c_int32), ("n_playouts", ctypes.c_int32), ("ucb_c", ctypes.c_float),
                ("device", ctypes.c_int32), ("seed", ctypes.c_uint64), ("max_tree_size", ctypes.c_int64),
                ("node_capacity", ctypes.c_int64), ("max_batch", ctypes.c_int32), ("tree_offset", ctypes.c_int32),
                ("n_trees_global", ctypes.c_int32), ("threads_per_tree", ctypes.c_int32), ("reserved", ctypes.c_int32)]


class Result(ctypes.Structure):
    _fields_ = [("best_action", ctypes.c_int32), ("best_win_flag", ctypes.c_int32), ("best_n", ctypes.c_int64),
                ("best_n_wins", ctypes.c_int64), ("steps", ctypes.c_int64), ("playouts", ctypes.c_int64),
                ("plies", ctypes.c_int64), ("ub_draws", ctypes.c_int64), ("status", ctypes.c_uint32),
                ("n_root_actions", ctypes.c_int32), ("device_ms", ctypes.c_float), ("max_depth", ctypes.c_int32),
                ("total_nodes", ctypes.c_int64), ("depth_sum", ctypes.c_int64), ("max_size", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("stage_ms", ctypes.c_float * 4), ("reduce_ms", ctypes.c_float * 2),
                ("root_ns", ctypes.c_int64 * MAX_ACTIONS), ("actions_ns", ctypes.c_int64 * MAX_ACTIONS),
                ("actions_ns_wins", ctypes.c_int64 * MAX_ACTIONS), ("actions_win_flags", ctypes.c_uint8 * MAX_ACTIONS),
                ("actions_expanded", ctypes.c_uint8 * MAX_ACTIONS)]


RESULT_DTYPE = np.dtype([("best_action", np.int32), ("best_win_flag", np.int32), ("best_n", np.int64),
                         ("best_n_wins", np.int64), ("steps", np.int64), ("playouts", np.int64), ("plies", np.int64),
                         ("ub_draws", np.int64), ("status", np.uint32), ("n_root_actions", np.int32),
                         ("device_ms", np.float32), ("max_depth", np.int32), ("total_nodes", np.int64),
                         ("depth_sum", np.int64), ("max_size", np.int32), ("reserved", np.int32),
                         ("stage_ms", np.float32, (4,)), ("reduce_ms", np.float32, (2,)),
                         ("root_ns", np.int64, (MAX_ACTIONS,)), ("actions_ns", np.int64, (MAX_ACTIONS,)),
                         ("actions_ns_wins", np.int64, (MAX_ACTIONS,)), ("actions_win_flags", np.uint8, (MAX_ACTIONS,)),
                         ("actions_expanded", np.uint8, (MAX_ACTIONS,))], align=True)

_lib = None


class MctsncError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"{text} ({code})")
        self.code = code


def lib():
    """Loads the library once.  Raises ``RuntimeError`` if it has not been built: there is no CPU path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m mcts_numba_cuda_b200.build` (needs nvcc). "
                "This package has no CPU fallback.")
        L = ctypes.CDLL(LIB_PATH)
        vp, i32, i64 = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64
        L.mctsnc_create.argtypes = [ctypes.POINTER(Config), ctypes.POINTER(vp)]
        L.mctsnc_destroy.argtypes = [vp]
        L.mctsnc_reset_rng.argtypes = [vp]
        L.mctsnc_run.argtypes = [vp, vp, vp, i32, i64, ctypes.c_double, vp]
        L.mctsnc_run_batch.argtypes = [vp, i32, vp, vp, vp, i64, i32, vp]
        L.mctsnc_search_batch_device.argtypes = [vp, i32, vp, vp, vp, i64, i32, vp, vp]
        L.mctsnc_finish_batch_device.argtypes = [vp, i32, vp, vp, vp]
        L.mctsnc_launch_batch_device.argtypes = [vp, i32, vp, vp, vp, i64, i32, vp]
        L.mctsnc_reduce_trees_device.argtypes = [vp, i32, vp, vp]
        L.mctsnc_export.argtypes = [vp, i32, i32, vp, i64]
        L.mctsnc_export_rng.argtypes = [vp, i32, i32, vp, i64]
        L.mctsnc_query.argtypes = [vp, ctypes.POINTER(i32), ctypes.POINTER(i32), ctypes.POINTER(i32), ctypes.POINTER(i64)]
        L.mctsnc_search_c4_static.argtypes = [vp, vp, i32, i32, i32, i32, i64, ctypes.c_float, ctypes.c_uint64, vp, vp]
        L.mctsnc_exchange_create.argtypes = [i32, i32, i64, i32, ctypes.POINTER(vp), vp]
        L.mctsnc_exchange_connect.argtypes = [vp, vp]
        L.mctsnc_exchange_allreduce.argtypes = [vp, vp, i64, i32, vp]
        L.mctsnc_exchange_status.argtypes = [vp, ctypes.POINTER(i32), vp]
        L.mctsnc_exchange_destroy.argtypes = [vp]
        L.mctsnc_trace_slices.argtypes = [vp, i32]
        L.mctsnc_read_slices.argtypes = [vp, vp, i32, ctypes.POINTER(i32)]
        L.mctsnc_error_string.argtypes = [ctypes.c_int]
        L.mctsnc_error_string.restype = ctypes.c_char_p
        for name in EXPORTED[:-1]:
            getattr(L, name).restype = ctypes.c_int
        assert ctypes.sizeof(Result) == RESULT_DTYPE.itemsize
        _lib = L
    return _lib


def check(code):
    if code != 0:
        raise MctsncError(code, lib().mctsnc_error_string(code).decode("utf-8", "replace"))
