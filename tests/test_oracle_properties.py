"""Property tests of the CPU oracle against torch CPU EmbeddingBag on random shapes (hypothesis):
every mode, both table types, ragged bags with empties, padding, include_last_offset, weights."""
import numpy as np
from hypothesis import given, settings, strategies as st

from oracle import eb_oracle as O


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


@settings(max_examples=60, deadline=None, derandomize=True)
@given(seed=st.integers(0, 2**31 - 1), rows=st.integers(1, 60), dim=st.integers(1, 70),
       bags=st.integers(1, 25), max_len=st.integers(0, 40), mode=st.sampled_from([0, 1, 2]),
       half=st.booleans(), pad=st.booleans(), last=st.booleans(), weighted=st.booleans())
def test_oracle_equals_torch_cpu(seed, rows, dim, bags, max_len, mode, half, pad, last, weighted):
    rng = np.random.default_rng(seed)
    dtype = np.float16 if half else np.float32
    table = rng.standard_normal((rows, dim)).astype(dtype)
    if mode == 2:
        table = (np.round(table.astype(np.float32) * 2) / 2).astype(dtype)   # make ties likely
    lengths = rng.integers(0, max_len + 1, bags)
    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
    n = int(offsets[-1])
    indices = rng.integers(0, rows, n).astype(np.int64)
    padding = int(rng.integers(0, rows)) if pad else -1
    weighted = weighted and mode == 0 and not half       # torch multiplies fp16 weights in half
    psw = rng.random(n).astype(np.float32) if weighted else None
    off_arg = offsets if last else offsets[:-1]
    got = O.pool(table, indices, off_arg, mode=mode, padding_idx=padding, include_last_offset=last,
                 per_sample_weights=psw)
    exp = O.torch_pool(table, indices, off_arg, mode=mode, padding_idx=padding,
                       include_last_offset=last, per_sample_weights=psw).numpy()
    assert got.shape == exp.shape
    if weighted:
        # torch fuses the multiply-add on its fast path but not on the path it takes when a
        # padding_idx is set (one ulp apart); the oracle always fuses
        np.testing.assert_allclose(got, exp, rtol=1e-5, atol=1e-5)
    else:
        assert np.array_equal(_bits(got), _bits(exp))


@settings(max_examples=40, deadline=None, derandomize=True)
@given(seed=st.integers(0, 2**31 - 1), shards=st.integers(1, 6), rows=st.integers(6, 80),
       dim=st.integers(1, 33))
def test_row_windows_partition_the_sum(seed, shards, rows, dim):
    """Partial bags over disjoint row windows fold to the unsharded sum (fp64-checked), and the
    mean's denominator counts indices that fall outside the window (reference .cu:112)."""
    rng = np.random.default_rng(seed)
    table = rng.standard_normal((rows, dim)).astype(np.float32)
    lengths = rng.integers(0, 20, 9)
    offsets = np.concatenate([[0], np.cumsum(lengths)])[:-1].astype(np.int32)
    indices = rng.integers(0, rows, int(lengths.sum())).astype(np.int32)
    per = -(-rows // shards)
    parts = []
    for r in range(shards):
        lo, n = min(r * per, rows), max(0, min(per, rows - r * per))
        parts.append(O.pool(table[lo:lo + n] if n else table[:0], indices, offsets, mode=O.MODE_MEAN,
                            row_lo=lo) if n else np.zeros((9, dim), np.float32))
    folded = O.combine_partials(np.stack(parts))
    whole = O.pool(table, indices, offsets, mode=O.MODE_MEAN)
    np.testing.assert_allclose(folded, whole, rtol=1e-5, atol=1e-5)
