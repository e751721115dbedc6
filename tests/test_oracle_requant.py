"""CPU: the re-quantiser oracle (oracle/requant.py) against properties the fit has by construction."""
import numpy as np
import pytest

from oracle import affine, requant


def test_four_equally_spaced_values_are_reproduced_exactly():
    """A group that already lies on a 4-level line (values exact in f16) is fitted with zero error."""
    rng = np.random.default_rng(0)
    lv = rng.integers(0, 4, size=(8, 256))
    lv[:, ::64] = 0
    lv[:, 1::64] = 3        # both ends present in every group of 64
    w = (0.25 * lv - 0.5).astype(np.float32)
    words, s, b, q = requant.quantize_affine(w, 64, 2, "float16")
    assert np.array_equal(q, lv)
    assert np.all(s == 0.25) and np.all(b == -0.5)
    deq = affine.dequantize_affine(words, s.reshape(8, -1).astype(np.float16), b.reshape(8, -1).astype(np.float16), bits=2, group_size=64)
    assert np.array_equal(deq, w)


@pytest.mark.parametrize("store", ["float16", "bfloat16"])
def test_search_and_refinement_never_lose_to_the_minmax_fit(store):
    rng = np.random.default_rng(1)
    w = rng.standard_normal((16, 512)).astype(np.float32)
    g = w.reshape(-1, 128)
    levels = np.float32(3)
    lo, hi = g.min(-1, keepdims=True), g.max(-1, keepdims=True)
    e_minmax = requant._error(g, np.maximum((hi - lo) / levels, 1e-8), lo, levels)
    s, b = requant.fit_search(g, 2)
    e_search = requant._error(g, s, b, levels)
    assert np.all(e_search <= e_minmax)
    s2, b2 = requant.refine_lsq(g, s, b, 2, store=store)
    e_ref = requant._error(g, s2, b2, levels)
    e_start = requant._error(g, requant._store(s, store), requant._store(b, store), levels)
    assert np.all(e_ref <= e_start)
    assert e_ref.sum() < 0.9 * e_minmax.sum()      # a normal group gains clearly from the shrunk range


def test_packing_round_trips_and_constant_group_is_safe():
    w = np.full((2, 128), 0.75, dtype=np.float32)
    words, s, b, q = requant.quantize_affine(w, 128, 2, "float16")
    assert np.all(np.isfinite(s)) and np.all(np.isfinite(b))
    assert np.array_equal(affine.unpack_bits(words, 2, 128), q)
    rec = np.repeat(s, 128) * q.reshape(-1) + np.repeat(b, 128)
    assert np.allclose(rec, 0.75, atol=1e-3)
