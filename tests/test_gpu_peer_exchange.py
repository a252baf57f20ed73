"""The exchange step without a collective library (``mctsnc_exchange_*``: peer stores, flags, a bounded wait) on one
GPU: a single rank, and a rank whose peer never arrives -- the wait must run out, say so in the status word, and leave
the values alone.  The missing peer is made on the host (loop-back mapping: nothing ever raises the second rank's flag);
no GPU is faulted or hung, the wait is a bounded loop of a few thousand polls."""
import time

import pytest

from mcts_numba_cuda_b200 import _abi
from mcts_numba_cuda_b200.distributed import PeerExchange

pytestmark = pytest.mark.gpu


def test_single_rank_sum_is_the_identity_over_many_calls():
    import torch
    ex = PeerExchange(0, 1, 1000, 0)
    for k in range(5):                       # both halves of the buffer, several times
        v = torch.arange(1000, dtype=torch.int64, device="cuda") * (k + 1)
        ex.all_reduce(v)
        assert torch.equal(v.cpu(), torch.arange(1000, dtype=torch.int64) * (k + 1))
    assert ex.status() == 0
    ex.close()


def test_loopback_ranks_add_up():
    """world = 3 with every peer mapped onto the local buffer: the rank's own slot is written three times, the other two
    slots never -- so the flags of ranks 1 and 2 stay down and the wait runs out."""
    import torch
    ex = PeerExchange(0, 3, 64, 0, loopback=True)
    v = torch.full((64,), 7, dtype=torch.int64, device="cuda")
    t0 = time.perf_counter()
    ex.all_reduce(v, wait_limit=4000)        # about a millisecond of polling
    status = ex.status()
    assert time.perf_counter() - t0 < 5.0
    assert status & _abi.EXCHANGE_TIMEOUT
    assert torch.equal(v.cpu(), torch.full((64,), 7, dtype=torch.int64))      # untouched
    ex.close()


def test_sizes_beyond_the_buffer_are_refused():
    import torch
    ex = PeerExchange(0, 1, 16, 0)
    with pytest.raises(_abi.MctsncError) as e:
        ex.all_reduce(torch.zeros(17, dtype=torch.int64, device="cuda"))
    assert e.value.code == _abi.E_CAPACITY
    ex.close()
