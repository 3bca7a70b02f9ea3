"""Our kernels against the reference's own kernels, both on the GPU.

oracle/_ref/libref_eb.so holds embedding_bag_plugin.cu of the reference compiled unmodified for
sm_100a (oracle/build_ref.py; present only where the reference tree was mounted at build time).
Sum, square-sum, the fixed-length form, the row window and gather must agree (the reference adds
through shared-memory atomics in no fixed order and is built with -use_fast_math, so sums are
compared to 1e-5 of the sum of magnitudes); for op codes 1 and 2 the reference kernel computes
max-from-zero / length and a plain sum, which the oracle's literal mode reproduces."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from forward_b200 import capi, workloads  # noqa: E402
from oracle import eb_oracle as O  # noqa: E402
from oracle import ref_kernels as R  # noqa: E402

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not R.available(), reason="reference kernels were not built here")]
DEV = "cuda:0"


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _close(got, ref, mags, rtol=1e-5):
    assert np.all(np.abs(got.astype(np.float64) - ref.astype(np.float64)) <= rtol * mags + 1e-6)


@pytest.mark.parametrize("dim", [4, 64, 128])
def test_sum_square_sum_window_and_literal_ops(dim):
    rng = np.random.default_rng(dim)
    rows = 5000
    table = rng.standard_normal((rows, dim)).astype(np.float32)
    bags = workloads.ragged_bags(rows, rng.integers(0, 50, 700), rng)
    t, i, o = _cuda(table), _cuda(bags.indices), _cuda(bags.offsets)
    stream = capi.current_stream_ptr()
    absum = O.pool(np.abs(table), bags.indices, bags.offsets).astype(np.float64)
    sqsum = O.pool(table, bags.indices, bags.offsets, mode=O.MODE_SQUARE_SUM).astype(np.float64)
    for op, mags in ((0, absum), (3, sqsum)):
        ref = torch.empty((700, dim), device=DEV)
        R.bag(i, o, ref, t, 0, op, stream)
        ours = capi.embedding_bag(t, i, o, mode=op)
        torch.cuda.synchronize()
        _close(ours.cpu().numpy(), ref.cpu().numpy(), mags)
    # row window: the reference's data_offset / count filter
    lo, n = 1000, 2500
    shard = _cuda(table[lo:lo + n])
    ref = torch.empty((700, dim), device=DEV)
    R.bag(i, o, ref, shard, lo, 0, stream)
    ours = capi.embedding_bag(shard, i, o, mode=capi.MODE_SUM, row_lo=lo)
    torch.cuda.synchronize()
    _close(ours.cpu().numpy(), ref.cpu().numpy(), absum)
    # op codes 1 and 2 as the reference kernel really treats them == the oracle's literal mode
    for op in (1, 2):
        ref = torch.empty((700, dim), device=DEV)
        R.bag(i, o, ref, t, 0, op, stream)
        torch.cuda.synchronize()
        lit = O.pool(table, bags.indices, bags.offsets, mode=op, semantics=O.SEM_KERNEL)
        _close(lit, ref.cpu().numpy(), absum, rtol=1e-5)
    enum_mean = O.pool(table, bags.indices, bags.offsets, mode=O.MODE_MEAN)
    assert not np.allclose(enum_mean, lit if op == 1 else enum_mean + 1)   # they do differ


def test_fixed_length_and_gather():
    rng = np.random.default_rng(1)
    table = rng.standard_normal((3000, 64)).astype(np.float32)
    idx = rng.integers(0, 3000, (300, 20)).astype(np.int32)
    t, i = _cuda(table), _cuda(idx)
    stream = capi.current_stream_ptr()
    ref = torch.empty((300, 64), device=DEV)
    R.bag_fixed(i, ref, t, 0, 0, stream)
    ours = capi.embedding_bag(t, i, mode=capi.MODE_SUM, fixed_len=20)
    torch.cuda.synchronize()
    _close(ours.cpu().numpy(), ref.cpu().numpy(), np.abs(table[idx]).sum(1).astype(np.float64))
    ref = torch.zeros((300 * 20, 64), device=DEV)
    R.gather(i, ref, t, 0, stream)
    ours = capi.embedding_bag(t, i, mode=capi.MODE_GATHER)
    torch.cuda.synchronize()
    assert torch.equal(ours, ref)                     # gather is bit-exact
