"""The oracle's xoroshiro128+ restatement against numba's own CPU routines (the third-party module the reference calls:
``numba.cuda.random``, src/mctsnc.py:162, :391-394).  numba is part of the test environment, not of the product."""
import ctypes

import numpy as np
import pytest

from oracle import oracle as om

numba_random = pytest.importorskip("numba.cuda.random")


@pytest.mark.parametrize("seed", [0, 1, 12345, 2 ** 63 + 11])
def test_stream_states_match_numba(seed):
    n = 300
    ref = np.empty(n, dtype=numba_random.xoroshiro128p_dtype)
    numba_random.init_xoroshiro128p_states_cpu(ref, np.uint64(seed), np.uint64(0))
    mine = om.rng_states(n, seed)
    assert np.array_equal(mine[:, 0], ref["s0"])
    assert np.array_equal(mine[:, 1], ref["s1"])


def test_uniform_float32_matches_numba():
    import numba

    @numba.njit
    def draw(states, idx, k):
        out = np.empty(k, dtype=np.float32)
        for i in range(k):
            out[i] = numba_random.xoroshiro128p_uniform_float32(states, idx)
        return out

    ref = np.empty(4, dtype=numba_random.xoroshiro128p_dtype)
    numba_random.init_xoroshiro128p_states_cpu(ref, np.uint64(7), np.uint64(0))
    mine = om.rng_states(4, 7)
    k = 20000
    expected = draw(ref, 2, k)
    state = mine[2].copy()
    got = np.array([om.lib().mo_rng_uniform_f32(state.ctypes.data) for _ in range(k)], dtype=np.float32)
    assert np.array_equal(got, expected)


def test_uniform_float32_can_be_exactly_one():
    """float32(float64(x >> 11) * 2**-53) rounds up to 1.0 for the largest 2**28 values of x >> 11: the reference then
    indexes one past the list of legal actions (src/mctsnc.py:2061-2062)."""
    state = np.array([0xFFFFFFFFFFFFFFFF, 0], dtype=np.uint64)   # next() returns s0 + s1
    assert om.lib().mo_rng_uniform_f32(state.ctypes.data) == 1.0
    v = np.uint64((2 ** 53 - 2 ** 28 - 1) << 11)                 # just below the rounding boundary
    state = np.array([v, 0], dtype=np.uint64)
    assert om.lib().mo_rng_uniform_f32(state.ctypes.data) < 1.0
