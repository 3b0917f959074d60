"""CPU tests of the sampler oracle (non-greedy branch of the reference's sample(), sampler.h:85-115)."""
import numpy as np
import pytest

from oracle import q4_oracle as O


def xorshift_u32(state):
    state ^= state >> 12
    state ^= (state << 25) & 0xFFFFFFFFFFFFFFFF
    state ^= state >> 27
    return state, ((state * 0x2545F4914F6CDD1D) & 0xFFFFFFFFFFFFFFFF) >> 32


def test_coin_sequence_matches_xorshift_star():
    """random_f32 (sampler.h:66-75) restated with Python integers."""
    r = O.Rng(1234567)
    state = 1234567
    for _ in range(16):
        state, u = xorshift_u32(state)
        assert r.f32() == np.float32((u >> 8) / 16777216.0)


def test_library_coin_matches_oracle():
    """q4_random_f32 of the shared library (host code, no GPU needed) draws the reference's sequence."""
    import ctypes as C

    from llama_cu_awq_b200 import _lib
    L = _lib.lib()
    st = C.c_ulonglong(987654321)
    r = O.Rng(987654321)
    for _ in range(32):
        assert float(L.q4_random_f32(C.byref(st))) == r.f32()


def select_float64(p16, topp, coin):
    """The selection rule in float64 on the fp16 probabilities (sums of multiples of 2^-24 are exact in float64)."""
    p = p16.astype(np.float64)
    if 0.0 < topp < 1.0:
        order = np.lexsort((np.arange(p.size), -p))   # probability descending, equal values by index (stable sort)
        thr = float(np.float32(coin) * np.float32(topp))
    else:
        order = np.arange(p.size)
        thr = float(np.float32(coin))
    cs = np.cumsum(p[order])
    hit = np.nonzero(cs >= thr)[0]
    return int(order[hit[0]]) if hit.size else int(order[-1])


@pytest.mark.parametrize("n", [32000, 1000, 37])
@pytest.mark.parametrize("topp", [0.9, 0.3, 0.0, 1.0])
def test_sampler_oracle_selection(n, topp):
    rng = np.random.default_rng(n + int(topp * 10))
    logits = (rng.standard_normal(n) * 2.5).astype(np.float16)
    for temperature in (0.5, 1.0, 2.0):
        for coin in (0.0, 1e-7, 0.25, 0.6180339, 0.99, 0.99999994):
            tok, p = O.sample_topp(logits, temperature, topp, coin)
            assert abs(float(p.astype(np.float64).sum()) - 1.0) < 2e-3
            assert tok == select_float64(p, topp, coin)


def test_sampler_oracle_threshold_never_reached():
    """fp16 rounding can leave the probabilities summing to less than the threshold: the last element of the order wins."""
    logits = np.zeros(4096, np.float16)         # uniform: p = fp16(1/4096) each, the sum is exactly 1
    logits[7] = np.float16(-20.0)               # one negligible element: lowest probability
    tok, p = O.sample_topp(logits, 1.0, 0.999, 0.99999994)
    assert tok == select_float64(p, 0.999, 0.99999994)
    tok, p = O.sample_topp(logits, 1.0, 0.0, 0.99999994)
    assert tok == select_float64(p, 0.0, 0.99999994)
