"""Host side of the warp-level PUCT select: the same ``launch_select(d, cpuct, c_pw, alpha_pw, soft_winner)`` call on a
dict of device arrays that the reference's ``src/puct/puct_gpu_v3_cpp.py:118-156`` offers, bound to the sm_100a kernels
in ``libmctsnc_b200.so`` (``csrc/puct_select.cu``), plus the backup / release step.

``d`` maps the names the reference's tests use (``edge_child, edge_prior, edge_w, edge_n, edge_inflight,
node_expand_inflight, node_expanded, node_count, out_selected, out_path, out_len`` and the ints ``trees``, ``warps``) to
arrays that live on the device: torch CUDA tensors, or anything with ``__cuda_array_interface__`` (numba / cupy arrays).
"""
import ctypes

from . import _abi

_configured = False


def _lib():
    global _configured
    L = _abi.lib()
    if not _configured:
        vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        L.puct_select_winner_recalc_launch.argtypes = [f32, f32, f32, i32] + [vp] * 11 + [i32] * 5 + [vp]
        L.puct_select_winner_recalc_launch.restype = i32
        L.puct_select_virtual_loss_launch.argtypes = [f32, f32, f32, i32, i32] + [vp] * 11 + [i32] * 5 + [vp]
        L.puct_select_virtual_loss_launch.restype = i32
        L.puct_backup_launch.argtypes = [i32] + [vp] * 9 + [i32] * 5 + [vp]
        L.puct_backup_launch.restype = i32
        L.puct_v2_select_launch.argtypes = [i32, f32, f32, f32] + [vp] * 11 + [i32] * 5 + [vp]
        L.puct_v2_select_launch.restype = i32
        L.puct_v2_backup_launch.argtypes = [i32] + [vp] * 10 + [i32] * 5 + [vp]
        L.puct_v2_backup_launch.restype = i32
        L.puct_cpp_cuda_error_string.argtypes = [i32]
        L.puct_cpp_cuda_error_string.restype = ctypes.c_char_p
        _configured = True
    return L


def _ptr(a):
    if a is None:
        return None
    if hasattr(a, "data_ptr"):
        return ctypes.c_void_p(a.data_ptr())
    if hasattr(a, "__cuda_array_interface__"):
        return ctypes.c_void_p(a.__cuda_array_interface__["data"][0])
    raise TypeError(f"not a device array: {type(a)}")


def _stream(stream):
    if stream is not None:
        return ctypes.c_void_p(stream)
    try:
        import torch
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    except Exception:
        return ctypes.c_void_p(0)


def _check(code, what):
    if code != 0:
        msg = _lib().puct_cpp_cuda_error_string(code).decode("utf-8", "replace")
        raise RuntimeError(f"PUCT {what} launch failed: {msg} ({code})")


def _shape(d):
    ec = d["edge_child"]
    return int(d["trees"]), int(ec.shape[1]), int(ec.shape[2]), int(d["warps"]), int(d["out_path"].shape[2])


def launch_select(d, cpuct=1.0, c_pw=1.0, alpha_pw=0.5, soft_winner=0, virtual_loss=1, stream=None):
    """One traversal per (tree, warp); results in ``d["out_selected"], d["out_path"], d["out_len"]``."""
    trees, nodes, edges, warps, path_depth = _shape(d)
    args = [_ptr(d[k]) for k in ("edge_child", "edge_prior", "edge_w", "edge_n", "edge_inflight", "node_expand_inflight",
                                 "node_expanded", "node_count", "out_selected", "out_path", "out_len")]
    if virtual_loss == 1:
        code = _lib().puct_select_winner_recalc_launch(cpuct, c_pw, alpha_pw, int(soft_winner), *args, trees, nodes, edges,
                                                       warps, path_depth, _stream(stream))
    else:
        code = _lib().puct_select_virtual_loss_launch(cpuct, c_pw, alpha_pw, int(soft_winner), int(virtual_loss), *args,
                                                      trees, nodes, edges, warps, path_depth, _stream(stream))
    _check(code, "select")


def launch_backup(d, values=None, virtual_loss=1, stream=None):
    """Turns the claims of the last select into statistics (``values``: float32[trees, warps, path_depth] on the device),
    or only releases them (``values=None``)."""
    trees, nodes, edges, warps, path_depth = _shape(d)
    code = _lib().puct_backup_launch(int(virtual_loss), _ptr(d["edge_w"]), _ptr(d["edge_n"]), _ptr(d["edge_inflight"]),
                                     _ptr(d["node_expand_inflight"]), _ptr(d["node_count"]), _ptr(d["out_selected"]),
                                     _ptr(d["out_path"]), _ptr(d["out_len"]), _ptr(values), trees, nodes, edges, warps,
                                     path_depth, _stream(stream))
    _check(code, "backup")


def launch_release(d, virtual_loss=1, stream=None):
    launch_backup(d, None, virtual_loss, stream)


V2_PRECLAIM, V2_COUNTER_CAS = 0, 1


def launch_select_v2(d, cpuct=1.0, c_pw=1.0, alpha_pw=0.5, variant=V2_PRECLAIM, stream=None):
    """The two older select kernels of the reference (``src/puct/puct_gpu_v2.py:573-840``), for trees that keep virtual
    visits per child node: ``d`` holds ``node_inflight`` (int32[trees, nodes]) in place of ``edge_inflight``.
    ``variant``: preclaim (every candidate is visited before it is scored, losers leave) or counter-CAS (the winner alone
    is claimed by compare-and-swap; a claim that met other visits is given back once)."""
    trees, nodes, edges, warps, path_depth = _shape(d)
    args = [_ptr(d[k]) for k in ("edge_child", "edge_prior", "edge_w", "edge_n", "node_inflight", "node_expand_inflight",
                                 "node_expanded", "node_count", "out_selected", "out_path", "out_len")]
    _check(_lib().puct_v2_select_launch(int(variant), cpuct, c_pw, alpha_pw, *args, trees, nodes, edges, warps, path_depth,
                                        _stream(stream)), "v2 select")


def launch_backup_v2(d, values=None, virtual_loss=1, stream=None):
    """``_backup_kernel_native`` of ``src/puct/puct_gpu_v2.py:847-927`` (``values=None``: release only)."""
    trees, nodes, edges, warps, path_depth = _shape(d)
    _check(_lib().puct_v2_backup_launch(int(virtual_loss), _ptr(d["edge_child"]), _ptr(d["edge_w"]), _ptr(d["edge_n"]),
                                        _ptr(d["node_inflight"]), _ptr(d["node_expand_inflight"]), _ptr(d["node_count"]),
                                        _ptr(d["out_selected"]), _ptr(d["out_path"]), _ptr(d["out_len"]), _ptr(values), trees,
                                        nodes, edges, warps, path_depth, _stream(stream)), "v2 backup")


def to_device(case, device="cuda"):
    """numpy case (as built by the tests) -> dict of torch CUDA tensors."""
    import torch
    return {k: (torch.from_numpy(v).to(device) if hasattr(v, "dtype") else v) for k, v in case.items()}


def to_host(d):
    return {k: (v.cpu().numpy() if hasattr(v, "cpu") else v) for k, v in d.items()}
