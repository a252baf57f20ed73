"""Root-parallel search on two GPUs (one process per GPU, NCCL for the plumbing): the result of the sharded search --
with the NCCL all-reduce and with the library's own peer-store exchange -- must equal one GPU growing all the trees, and
calls that overlap the exchange with the next batch must give what one call at a time gives.  Skipped on a box with a
single GPU; the same check runs inside ``bench.py --gpus N`` (``multi_gpu_parity``)."""
import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch
    import torch.distributed as dist
    from mcts_numba_cuda_b200 import MCTSNC
    from mcts_numba_cuda_b200.distributed import RootParallelMCTSNC
    from mcts_numba_cuda_b200.roots import c4_random_roots
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device(f"cuda:{rank}"))
    ok = {}
    try:
        roots, steps, T, P = 12, 150, 3, 64
        boards, fills, turns = c4_random_roots(roots, 16, seed=8)
        keys = ("root_ns", "actions_ns", "actions_ns_wins", "best_action", "best_n", "best_n_wins", "best_win_flag")
        want = None
        if rank == 0:
            whole = MCTSNC((6, 7), 7, 7, search_time_limit=np.inf, search_steps_limit=steps, n_trees=T * world, n_playouts=P,
                           variant="acp_prodigal", verbose_info=False, device=0, max_batch=roots, seed=5)
            whole.init_device_side_arrays()
            want = whole.run_batch(boards, fills, turns, steps, reseed=True)
        for exchange in ("nccl", "peer"):
            s = RootParallelMCTSNC((6, 7), 7, 7, n_trees=T, n_playouts=P, variant="acp_prodigal", search_steps_limit=steps,
                                   max_batch=roots, device=rank, rank=rank, world_size=world, seed=5, exchange=exchange)
            got = s.run_batch(boards, fills, turns, steps, reseed=True)
            # three calls in flight one behind the other, results read at the end: the last one must equal a single call
            for _ in range(3):
                s.search_async(boards, fills, turns, steps, reseed=True)
            piped = s.fetch(roots)
            same = all(np.array_equal(got[k], piped[k]) for k in keys)
            if rank == 0:
                same = same and all(np.array_equal(got[k], want[k]) for k in keys)
            ok[exchange] = bool(same) and s.exchange_status() == 0
            del s
        np.save(os.path.join(out_dir, f"ok_{rank}.npy"), np.array([ok["nccl"], ok["peer"]]))
    finally:
        dist.destroy_process_group()


def test_two_gpus_equal_one_gpu_with_all_the_trees(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for rank in range(2):
        assert np.load(tmp_path / f"ok_{rank}.npy").all()
