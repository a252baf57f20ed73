"""Root-parallel search over the GPUs of one box: one process per GPU (``torch.distributed``), each growing its own
trees of every search; the per-root-action sums are combined by one all-reduce per batch, then every rank runs the same
final argmax.

The reference is single-GPU: its "root parallelism" is ``n_trees`` blocks on one device followed by
``_reduce_over_trees_*`` / ``_reduce_over_actions_*`` (``src/mctsnc.py:2223-2375``).  Sharding keeps those two steps
and puts the exchange between them.  Rank r grows trees ``[r*n_trees, (r+1)*n_trees)`` of a search with
``world*n_trees`` trees and draws from the random streams those trees have in the single-GPU search, so the result
equals a single-GPU search with ``world*n_trees`` trees bit for bit (integer sums commute).
"""
import ctypes

import numpy as np

from . import _abi
from .mctsnc import MCTSNC


def shard_trees(n_trees_global, world_size, rank):
    """Contiguous split of the global tree indices; returns (tree_offset, n_trees_local)."""
    if n_trees_global % world_size != 0:
        raise ValueError(f"n_trees_global={n_trees_global} is not a multiple of world_size={world_size}")
    per_rank = n_trees_global // world_size
    return rank * per_rank, per_rank


def reduce_over_actions_host(actions_win_flags, actions_ns, actions_ns_wins, expanded, thrifty):
    """Host restatement of the final argmax (``_reduce_over_actions_*``, ``src/mctsnc.py:2299-2375``) for callers that
    combine partial sums themselves: lexicographic maximum of (win_flag, n, n_wins); ties go to the candidate that the
    stride-halving reduction keeps, i.e. the smallest bit-reversed slot index.  Thrifty variants reduce over ordinals
    of the expanded root actions, prodigal ones over action indices.  Returns (best_action, win_flag, n, n_wins)."""
    A = len(actions_ns)
    width = 1
    while width < A:
        width <<= 1
    slots = [a for a in range(A) if expanded[a]] if thrifty else list(range(A))
    keys = [(int(actions_win_flags[a]), int(actions_ns[a]), int(actions_ns_wins[a])) for a in slots]
    keys += [(0, 0, 0)] * (width - len(keys))
    idx = list(range(width))
    stride = width >> 1
    while stride > 0:
        for t in range(stride):
            if keys[t] < keys[t + stride]:
                keys[t] = keys[t + stride]
                idx[t] = idx[t + stride]
        stride >>= 1
    best = idx[0]
    if thrifty:
        best = slots[best] if best < len(slots) else 0
    return best, bool(keys[0][0]), keys[0][1], keys[0][2]


class RootParallelMCTSNC:
    """``MCTSNC`` sharded over the ranks of an initialised ``torch.distributed`` process group (backend nccl).

    ``n_trees`` is the number of trees PER RANK; the search has ``world_size * n_trees`` trees.  ``run_batch`` returns
    the same results on every rank.
    """

    def __init__(self, state_board_shape, state_extra_info_memory, state_max_actions, n_trees, n_playouts, variant,
                 search_steps_limit, max_batch, device, rank, world_size, process_group=None, **kwargs):
        self.rank, self.world_size, self.group = rank, world_size, process_group
        self.local = MCTSNC(state_board_shape, state_extra_info_memory, state_max_actions, search_time_limit=np.inf,
                            search_steps_limit=search_steps_limit, n_trees=n_trees, n_playouts=n_playouts, variant=variant,
                            verbose_info=False, device=device, max_batch=max_batch, tree_offset=rank * n_trees,
                            n_trees_global=world_size * n_trees, **kwargs)
        self.local.init_device_side_arrays()
        self.max_batch = max_batch
        self._sums = None
        self._batch = 0   # roots staged by the last call that brought boards (0: none yet; the library then refuses boards=None)

    def search_async(self, boards, extras, turns, steps, reseed=True, stream=None):
        """Launches the searches, the all-reduce and the final argmax on one CUDA stream (torch's current stream, or the
        ``cudaStream_t`` handle given as ``stream``); nothing is copied back."""
        import torch
        if stream is not None and stream != torch.cuda.current_stream().cuda_stream:
            # the all-reduce is ordered against torch's current stream: make the given stream that one
            with torch.cuda.stream(torch.cuda.ExternalStream(stream)):
                return self.search_async(boards, extras, turns, steps, reseed)
        import torch.distributed as dist
        ai = self.local
        A = ai.state_max_actions
        batch = max(self._batch, 1) if boards is None else len(boards)
        if self._sums is None:
            self._sums = torch.empty((self.max_batch, 3 * A), dtype=torch.int64, device=f"cuda:{ai.device}")
        cu_stream = torch.cuda.current_stream().cuda_stream
        if boards is not None:
            boards = np.ascontiguousarray(boards, dtype=np.int8)
            extras = np.ascontiguousarray(extras, dtype=np.int8) if extras is not None else None
            turns = np.ascontiguousarray(turns, dtype=np.int8)
            self._batch = batch
        _abi.check(_abi.lib().mctsnc_search_batch_device(
            ai._handle, batch, boards.ctypes.data if boards is not None else None,
            extras.ctypes.data if boards is not None and extras is not None else None,
            turns.ctypes.data if boards is not None else None, int(steps), 1 if reseed else 0, self._sums.data_ptr(),
            ctypes.c_void_p(cu_stream)))
        if self.world_size > 1:
            dist.all_reduce(self._sums[:batch], op=dist.ReduceOp.SUM, group=self.group)
        _abi.check(_abi.lib().mctsnc_finish_batch_device(ai._handle, batch, self._sums.data_ptr(), None,
                                                         ctypes.c_void_p(cu_stream)))
        return batch

    def fetch(self, batch, stream=None):
        """Copies the results of the last ``search_async`` to the host (synchronises)."""
        import torch
        ai = self.local
        cu_stream = torch.cuda.current_stream().cuda_stream if stream is None else stream
        out = np.zeros(batch, dtype=_abi.RESULT_DTYPE)
        _abi.check(_abi.lib().mctsnc_finish_batch_device(ai._handle, batch, self._sums.data_ptr(), out.ctypes.data,
                                                         ctypes.c_void_p(cu_stream)))
        return out

    def run_batch(self, boards, extras, turns, steps, reseed=True):
        batch = self.search_async(boards, extras, turns, steps, reseed)
        return self.fetch(batch)
