"""Host side of the decoupled-UCT (DUCT) select for simultaneous-move games (``csrc/duct_select.cu``,
``include/duct_b200.h``).  The reference has no such component; the interface follows the one of the PUCT select
(``puct.py``): a dict of device arrays and two launches.

``d`` holds ``child`` int32[trees, nodes, A*A], ``node_prior`` / ``node_w`` float32[trees, nodes, 2, A], ``node_n`` /
``node_inflight`` int32[trees, nodes, 2, A], ``node_terminal`` int32[trees, nodes], ``node_count`` int32[trees],
``out_selected`` / ``out_len`` int32[trees, warps], ``out_path`` int32[trees, warps, path_depth] and the ints ``trees``,
``warps`` — torch CUDA tensors or anything with ``__cuda_array_interface__``.
"""
import ctypes

from . import _abi
from .puct import _ptr, _stream

KIND_INVALID, KIND_EXPAND, KIND_TERMINAL, KIND_DEPTH_LIMIT, KIND_BUSY = 0, 1, 2, 3, 4

_configured = False


def _lib():
    global _configured
    L = _abi.lib()
    if not _configured:
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.duct_select_launch.argtypes = [f32, i32] + [vp] * 10 + [i32] * 5 + [vp]
        L.duct_select_launch.restype = i32
        L.duct_backup_launch.argtypes = [i32] + [vp] * 9 + [i32] * 5 + [vp]
        L.duct_backup_launch.restype = i32
        L.puct_cpp_cuda_error_string.argtypes = [i32]
        L.puct_cpp_cuda_error_string.restype = ctypes.c_char_p
        _configured = True
    return L


def _check(code, what):
    if code != 0:
        msg = _lib().puct_cpp_cuda_error_string(code).decode("utf-8", "replace")
        raise RuntimeError(f"DUCT {what} launch failed: {msg} ({code})")


def _shape(d):
    prior = d["node_prior"]
    return int(d["trees"]), int(prior.shape[1]), int(prior.shape[3]), int(d["warps"]), int(d["out_path"].shape[2])


def decode(selected):
    """(kind, node, joint action, reason) of packed results (array or int)."""
    return (selected >> 22) & 7, selected & 0x3FFF, (selected >> 14) & 0xFF, (selected >> 25) & 0x3F


def launch_select(d, cpuct=1.5, virtual_loss=1, stream=None):
    """One traversal per (tree, warp); results in ``d["out_selected"], d["out_path"], d["out_len"]``."""
    trees, nodes, actions, warps, path_depth = _shape(d)
    args = [_ptr(d[k]) for k in ("child", "node_prior", "node_w", "node_n", "node_inflight", "node_terminal", "node_count",
                                 "out_selected", "out_path", "out_len")]
    _check(_lib().duct_select_launch(cpuct, int(virtual_loss), *args, trees, nodes, actions, warps, path_depth,
                                     _stream(stream)), "select")


def launch_backup(d, values=None, new_child=None, virtual_loss=1, stream=None):
    """Returns the claims of the last select; with ``values`` (float32[trees, warps, path_depth], player 0's point of
    view) also updates counts and value sums; ``new_child`` (int32[trees, warps]) installs the expanded children."""
    trees, nodes, actions, warps, path_depth = _shape(d)
    args = [_ptr(d[k]) for k in ("child", "node_w", "node_n", "node_inflight", "out_selected", "out_path", "out_len")]
    _check(_lib().duct_backup_launch(int(virtual_loss), *args, _ptr(values), _ptr(new_child), trees, nodes, actions, warps,
                                     path_depth, _stream(stream)), "backup")
