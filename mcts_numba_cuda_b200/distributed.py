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


class PeerExchange:
    """In-place sum of an int64 CUDA tensor over the ranks of one box by peer stores and flags
    (``mctsnc_exchange_*`` of ``include/mctsnc_b200.h``, ``csrc/peer_exchange.cu``), one process per GPU.  The CUDA IPC
    handles of the ranks' buffers travel through ``torch.distributed.all_gather_object``; nothing else uses the process
    group.  ``loopback=True`` maps every peer onto the local buffer (tests on one GPU)."""

    DEFAULT_WAIT_LIMIT = 1 << 23      # polls of ~0.25 us: about two seconds before a missing rank is reported

    def __init__(self, rank, world_size, n_values_max, device, group=None, loopback=False):
        lib = _abi.lib()
        self.rank, self.world_size = rank, world_size
        self._ex = ctypes.c_void_p()
        mine = (ctypes.c_ubyte * _abi.EXCHANGE_HANDLE_BYTES)()
        _abi.check(lib.mctsnc_exchange_create(rank, world_size, int(n_values_max), int(device), ctypes.byref(self._ex), mine))
        if loopback or world_size == 1:
            _abi.check(lib.mctsnc_exchange_connect(self._ex, None))
        else:
            import torch.distributed as dist
            gathered = [None] * world_size
            dist.all_gather_object(gathered, bytes(mine), group=group)
            blob = (ctypes.c_ubyte * (_abi.EXCHANGE_HANDLE_BYTES * world_size)).from_buffer_copy(b"".join(gathered))
            _abi.check(lib.mctsnc_exchange_connect(self._ex, blob))
            dist.barrier(group=group)          # every rank has opened every buffer before anybody stores into one

    def all_reduce(self, values, wait_limit=None, stream=None):
        """Queues the sum on a CUDA stream (torch's current stream unless a ``cudaStream_t`` handle is given)."""
        import torch
        cu = torch.cuda.current_stream().cuda_stream if stream is None else stream
        _abi.check(_abi.lib().mctsnc_exchange_allreduce(self._ex, values.data_ptr(), values.numel(),
                                                        int(wait_limit or self.DEFAULT_WAIT_LIMIT), ctypes.c_void_p(cu)))

    def status(self, stream=None):
        """Status word (``_abi.EXCHANGE_TIMEOUT`` once a wait has run out); synchronises the stream."""
        import torch
        cu = torch.cuda.current_stream().cuda_stream if stream is None else stream
        out = ctypes.c_int32(0)
        _abi.check(_abi.lib().mctsnc_exchange_status(self._ex, ctypes.byref(out), ctypes.c_void_p(cu)))
        return out.value

    def close(self):
        if getattr(self, "_ex", None):
            _abi.lib().mctsnc_exchange_destroy(self._ex)
            self._ex = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class RootParallelMCTSNC:
    """``MCTSNC`` sharded over the ranks of an initialised ``torch.distributed`` process group (backend nccl).

    ``n_trees`` is the number of trees PER RANK; the search has ``world_size * n_trees`` trees.  ``run_batch`` returns
    the same results on every rank.
    """

    def __init__(self, state_board_shape, state_extra_info_memory, state_max_actions, n_trees, n_playouts, variant,
                 search_steps_limit, max_batch, device, rank, world_size, process_group=None, exchange="nccl", **kwargs):
        if exchange not in ("nccl", "peer"):
            raise ValueError(f"exchange must be 'nccl' or 'peer', not {exchange!r}")
        self.rank, self.world_size, self.group, self.exchange = rank, world_size, process_group, exchange
        self._peer = None
        self.local = MCTSNC(state_board_shape, state_extra_info_memory, state_max_actions, search_time_limit=np.inf,
                            search_steps_limit=search_steps_limit, n_trees=n_trees, n_playouts=n_playouts, variant=variant,
                            verbose_info=False, device=device, max_batch=max_batch, tree_offset=rank * n_trees,
                            n_trees_global=world_size * n_trees, **kwargs)
        self.local.init_device_side_arrays()
        self.max_batch = max_batch
        self._sums = None     # two buffers of partial sums, used by alternate calls
        self._batch = 0       # roots staged by the last call that brought boards (0: none yet; the library then refuses boards=None)
        self._calls = 0
        self._side = None     # stream of the exchange (all-reduce + final argmax) when there is more than one rank
        self._reduced = None  # per buffer: event "partial sums written" (main stream) ...
        self._finished = None  # ... and event "argmax done" (exchange stream)

    def _prepare(self):
        import torch
        if self._sums is None:
            A = self.local.state_max_actions
            dev = f"cuda:{self.local.device}"
            self._sums = [torch.empty((self.max_batch, 3 * A), dtype=torch.int64, device=dev) for _ in range(2)]
            self._reduced = [torch.cuda.Event(), torch.cuda.Event()]
            self._finished = [None, None]
            if self.world_size > 1:
                self._side = torch.cuda.Stream(device=dev)
                if self.exchange == "peer":   # peer stores and flags instead of the NCCL all-reduce
                    self._peer = PeerExchange(self.rank, self.world_size, self.max_batch * 3 * A, self.local.device, self.group)

    def search_async(self, boards, extras, turns, steps, reseed=True, stream=None):
        """Launches the searches of one batch on a CUDA stream (torch's current stream, or the ``cudaStream_t`` handle
        given as ``stream``) and their exchange -- all-reduce of the per-action sums, final argmax -- behind them; nothing
        is copied back.  With more than one rank the exchange runs on a stream of its own: the all-reduce is a meeting
        point of the ranks, and on the search stream it would make every rank wait for the slowest one after every batch
        (the ranks grow different trees, their launches differ by a few per cent).  Here the next call's searches start at
        once; only its partial sums wait for this call's argmax, because the two share the handle's flag and statistics
        buffers.  Results are read with ``fetch``."""
        import torch
        if stream is not None and stream != torch.cuda.current_stream().cuda_stream:
            with torch.cuda.stream(torch.cuda.ExternalStream(stream)):
                return self.search_async(boards, extras, turns, steps, reseed)
        import torch.distributed as dist
        self._prepare()
        ai, lib = self.local, _abi.lib()
        batch = max(self._batch, 1) if boards is None else len(boards)
        main = torch.cuda.current_stream()
        cu_main = ctypes.c_void_p(main.cuda_stream)
        if boards is not None:
            boards = np.ascontiguousarray(boards, dtype=np.int8)
            extras = np.ascontiguousarray(extras, dtype=np.int8) if extras is not None else None
            turns = np.ascontiguousarray(turns, dtype=np.int8)
        _abi.check(lib.mctsnc_launch_batch_device(
            ai._handle, batch, boards.ctypes.data if boards is not None else None,
            extras.ctypes.data if boards is not None and extras is not None else None,
            turns.ctypes.data if boards is not None else None, int(steps), 1 if reseed else 0, cu_main))
        if boards is not None:
            self._batch = batch
        k = self._calls % 2
        prev = self._finished[1 - k]
        if prev is not None:
            main.wait_event(prev)          # the previous call's argmax reads what reduce_trees is about to overwrite
        sums = self._sums[k]
        _abi.check(lib.mctsnc_reduce_trees_device(ai._handle, batch, sums.data_ptr(), cu_main))
        if self._side is None:
            _abi.check(lib.mctsnc_finish_batch_device(ai._handle, batch, sums.data_ptr(), None, cu_main))
            self._finished[k] = None
        else:
            self._reduced[k].record(main)
            with torch.cuda.stream(self._side):
                self._side.wait_event(self._reduced[k])
                if self._peer is not None:
                    self._peer.all_reduce(sums[:batch])
                else:
                    dist.all_reduce(sums[:batch], op=dist.ReduceOp.SUM, group=self.group)
                _abi.check(lib.mctsnc_finish_batch_device(ai._handle, batch, sums.data_ptr(), None,
                                                          ctypes.c_void_p(self._side.cuda_stream)))
                done = torch.cuda.Event()
                done.record(self._side)
            self._finished[k] = done
        self._last = k
        self._calls += 1
        return batch

    def exchange_status(self):
        """0, or ``_abi.EXCHANGE_TIMEOUT`` once a wait of the peer exchange has run out (a rank did not arrive in time:
        results since then are sums over the local trees only).  Always 0 with the NCCL exchange."""
        if self._peer is None:
            return 0
        return self._peer.status(self._side.cuda_stream)

    def drain(self):
        """Makes the current stream wait for the exchange of the last ``search_async`` call (for timing with events)."""
        import torch
        done = self._finished[self._last] if self._calls else None
        if done is not None:
            torch.cuda.current_stream().wait_event(done)

    def fetch(self, batch, stream=None):
        """Copies the results of the last ``search_async`` to the host (synchronises)."""
        import torch
        ai = self.local
        self.drain()
        cu_stream = torch.cuda.current_stream().cuda_stream if stream is None else stream
        out = np.zeros(batch, dtype=_abi.RESULT_DTYPE)
        _abi.check(_abi.lib().mctsnc_finish_batch_device(ai._handle, batch, self._sums[self._last].data_ptr(), out.ctypes.data,
                                                         ctypes.c_void_p(cu_stream)))
        return out

    def run_batch(self, boards, extras, turns, steps, reseed=True):
        batch = self.search_async(boards, extras, turns, steps, reseed)
        return self.fetch(batch)
