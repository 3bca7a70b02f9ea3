"""The streaming and the lean lane-group kernels (FWD_EB_STRATEGY_STREAM / _LITE) and the window compaction, against
the CPU oracle: bit for bit in every mode (the kernel adds rows in bag order, like the oracle)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from forward_b200 import capi, workloads  # noqa: E402
from oracle import eb_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
NP = {"f32": np.float32, "f16": np.float16}


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _bits(a):
    return a.view(np.uint32 if a.dtype == np.float32 else np.uint16)


def _batch(rng, rows, nb, maxlen, empty_frac=0.0):
    lengths = rng.integers(0, maxlen + 1, nb)
    if empty_frac:
        lengths[rng.random(nb) < empty_frac] = 0
    bags = workloads.ragged_bags(rows, lengths, rng)
    bags.indices[::11] = 7
    return bags


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("dim", [40, 64, 96, 128, 200, 256])   # rows of 128..512 bytes, some not a power of two
def test_stream_equals_oracle_all_modes(dt, dim):
    if NP[dt] == np.float32 and dim > 128:
        pytest.skip("fp32 rows wider than 512 bytes are outside the streaming kernel's shapes")
    if NP[dt] == np.float16 and dim < 64:
        pytest.skip("fp16 rows under 128 bytes are outside the streaming kernel's shapes")
    rng = np.random.default_rng(dim + (dt == "f16"))
    rows = 4000
    table = rng.standard_normal((rows, dim)).astype(NP[dt])
    qtable = (np.round(table * 2) / 2).astype(NP[dt])          # few distinct values: max ties
    for nb, maxlen, empty in ((1, 3, 0), (37, 5, 0.5), (700, 20, 0.3), (300, 70, 0), (33, 400, 0), (2000, 9, 0.1)):
        bags = _batch(rng, rows, nb, maxlen, empty)
        i, o = _cuda(bags.indices), _cuda(bags.offsets)
        w_np = rng.random(bags.num_indices).astype(np.float32)
        for mode, tab in ((capi.MODE_SUM, table), (capi.MODE_MEAN, table), (capi.MODE_MAX, qtable),
                          (capi.MODE_SQUARE_SUM, table)):
            for row_lo, nrows in ((0, rows), (500, 2500)):
                t = _cuda(tab[row_lo:row_lo + nrows])
                exp = O.pool(tab[row_lo:row_lo + nrows], bags.indices, bags.offsets, mode=mode,
                             padding_idx=7, row_lo=row_lo)
                for strat in (capi.STRATEGY_STREAM, capi.STRATEGY_LITE):
                    got = capi.embedding_bag(t, i, o, mode=mode, padding_idx=7, row_lo=row_lo, strategy=strat)
                    assert np.array_equal(_bits(got.cpu().numpy()), _bits(exp)), (nb, maxlen, mode, row_lo, strat)
        exp = O.pool(table, bags.indices, bags.offsets, mode=O.MODE_SUM, per_sample_weights=w_np,
                     out_dtype=np.float32)
        for strat in (capi.STRATEGY_STREAM, capi.STRATEGY_LITE):
            got = capi.embedding_bag(_cuda(table), i, o, mode=capi.MODE_SUM, per_sample_weights=_cuda(w_np),
                                     strategy=strat, out_dtype=torch.float32)
            assert np.array_equal(_bits(got.cpu().numpy()), _bits(exp)), strat


def test_stream_fixed_length_and_include_last_offset():
    rng = np.random.default_rng(5)
    rows, dim, nb, L = 3000, 128, 513, 20
    table = rng.standard_normal((rows, dim)).astype(np.float32)
    idx = rng.integers(0, rows, (nb, L)).astype(np.int32)
    w = rng.random(nb * L).astype(np.float32)
    t = _cuda(table)
    exp = O.pool(table, idx, fixed_len=L, per_sample_weights=w)
    for strat in (capi.STRATEGY_STREAM, capi.STRATEGY_LITE, capi.STRATEGY_AUTO):
        got = capi.embedding_bag(t, _cuda(idx), None, fixed_len=L, per_sample_weights=_cuda(w), strategy=strat)
        assert np.array_equal(_bits(got.cpu().numpy()), _bits(exp)), strat
    bags = _batch(rng, rows, 300, 30, 0.2)
    off = np.append(bags.offsets, bags.num_indices).astype(np.int32)
    exp = O.pool(table, bags.indices, off, mode=O.MODE_MEAN, include_last_offset=True)
    for strat in (capi.STRATEGY_STREAM, capi.STRATEGY_LITE):
        got = capi.embedding_bag(t, _cuda(bags.indices), _cuda(off), mode=capi.MODE_MEAN,
                                 include_last_offset=True, strategy=strat)
        assert np.array_equal(_bits(got.cpu().numpy()), _bits(exp)), strat


def test_stream_refuses_shapes_outside_its_limits_and_auto_falls_back():
    rng = np.random.default_rng(6)
    table = _cuda(rng.standard_normal((100, 8)).astype(np.float32))          # 32-byte rows
    idx = _cuda(rng.integers(0, 100, 50).astype(np.int32))
    off = _cuda(np.arange(0, 50, 5, dtype=np.int32))
    with pytest.raises(capi.FwdEbError) as e:
        capi.embedding_bag(table, idx, off, strategy=capi.STRATEGY_STREAM)
    assert e.value.code == capi.EUNSUPPORTED
    capi.embedding_bag(table, idx, off)                                        # AUTO picks another kernel
    wide = _cuda(rng.standard_normal((100, 128)).astype(np.float32))
    with pytest.raises(capi.FwdEbError):                                        # int64 indices
        capi.embedding_bag(wide, idx.long(), off.long(), strategy=capi.STRATEGY_STREAM)


def test_stream_survives_malformed_offsets():
    """Offsets that go backwards or past the end must not become wild reads (results for such
    bags are unspecified; the call has to finish and leave well-formed bags' neighbours alone)."""
    rng = np.random.default_rng(7)
    table = _cuda(rng.standard_normal((500, 64)).astype(np.float32))
    idx = _cuda(rng.integers(0, 500, 400).astype(np.int32))
    off = _cuda(np.array([0, 50, 20, 900, 100, -5, 300, 399], dtype=np.int32))
    for strat in (capi.STRATEGY_STREAM, capi.STRATEGY_LITE):
        out = capi.embedding_bag(table, idx, off, strategy=strat)
        torch.cuda.synchronize()
        assert out.shape == (8, 64)


@pytest.mark.parametrize("idx64", [False, True])
@pytest.mark.parametrize("mode", [capi.MODE_SUM, capi.MODE_MAX, "weighted"])
def test_window_compaction_then_pooling_equals_filtering_inside_the_pool(idx64, mode):
    rng = np.random.default_rng(11 + idx64)
    rows, dim = 9000, 64
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    lo, n = 3000, 2000                                           # this "rank" holds rows [3000, 5000)
    t = _cuda(table[lo:lo + n])
    for nb, maxlen in ((1, 10), (15, 40), (16, 40), (17, 40), (33, 40), (1000, 100), (257, 3)):
        bags = _batch(rng, rows, nb, maxlen, 0.2)
        idt = np.int64 if idx64 else np.int32
        i, o = _cuda(bags.indices.astype(idt)), _cuda(bags.offsets.astype(idt))
        w_np = rng.random(bags.num_indices).astype(np.float32) if mode == "weighted" else None
        w = _cuda(w_np) if w_np is not None else None
        m = capi.MODE_SUM if mode == "weighted" else mode
        kept = torch.full((max(1, bags.num_indices),), -7, dtype=torch.int32, device=DEV)
        kept_w = torch.zeros(max(1, bags.num_indices), dtype=torch.float32, device=DEV) if w is not None else None
        bounds = torch.zeros((nb, 2), dtype=torch.int32, device=DEV)
        counts = torch.zeros(nb, dtype=torch.int32, device=DEV)
        out = torch.empty((nb, dim), dtype=torch.float32, device=DEV)
        p = capi.make_params(t, i, o, out=out, mode=m, per_sample_weights=w, padding_idx=7, row_lo=lo)
        capi.compact_window(p, kept, bounds, kept_weights=kept_w, counts=counts)
        torch.cuda.synchronize()
        ends = np.append(bags.offsets, bags.num_indices)
        bh, kh, ch = bounds.cpu().numpy(), kept.cpu().numpy(), counts.cpu().numpy()
        for b in range(nb):
            seg = bags.indices[ends[b]:ends[b + 1]].astype(np.int64)
            live = seg[seg != 7]
            sur = live[(live >= lo) & (live < lo + n)] - lo
            assert ch[b] == live.size
            assert np.array_equal(kh[bh[b, 0]:bh[b, 1]], sur)
            if b % 16:
                assert bh[b, 0] == bh[b - 1, 1]                  # sub-bags of a run are back to back
        exp = O.pool(table[lo:lo + n], bags.indices, bags.offsets, mode=m, padding_idx=7, row_lo=lo,
                     per_sample_weights=w_np, out_dtype=np.float32)
        for strat in (capi.STRATEGY_GROUP, capi.STRATEGY_STREAM, capi.STRATEGY_LITE, capi.STRATEGY_AUTO):
            out.fill_(float("nan"))
            q = capi.make_compacted_params(t, kept, bounds, out=out, mode=m, kept_weights=kept_w,
                                           strategy=strat)
            capi.forward(q)
            torch.cuda.synchronize()
            assert np.array_equal(_bits(out.cpu().numpy()), _bits(exp)), (nb, maxlen, strat)


def test_config3_and_config5_shapes_through_the_streaming_kernel():
    """512-byte rows, max with padding (config 3's shape, fewer rows) and 128-byte rows, short
    dense bags (what config 5 pools after compaction): AUTO must pick the lean kernel and agree
    with the lane-group kernel bit for bit."""
    import ctypes as C
    rng = np.random.default_rng(3)
    t3 = _cuda((rng.standard_normal((100_000, 256)) * 0.1).astype(np.float16))
    bags = workloads.config3_bags(seed=2, num_rows=100_000, num_bags=8192)
    i, o = _cuda(bags.indices), _cuda(bags.offsets)
    out = torch.empty((8192, 256), dtype=torch.float16, device=DEV)
    p = capi.make_params(t3, i, o, out=out, mode=capi.MODE_MAX, padding_idx=0)
    assert capi.lib().fwd_eb_pick_strategy(C.byref(p)) == capi.STRATEGY_LITE
    a = capi.embedding_bag(t3, i, o, mode=capi.MODE_MAX, padding_idx=0)
    b = capi.embedding_bag(t3, i, o, mode=capi.MODE_MAX, padding_idx=0, strategy=capi.STRATEGY_GROUP)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    t5 = _cuda((rng.standard_normal((200_000, 64)) * 0.05).astype(np.float16))
    lengths = rng.binomial(rng.integers(1, 101, 50_000), 1 / 8)
    bags = workloads.ragged_bags(200_000, lengths, rng)
    i, o = _cuda(bags.indices), _cuda(bags.offsets)
    a = capi.embedding_bag(t5, i, o, out_dtype=torch.float32)
    b = capi.embedding_bag(t5, i, o, out_dtype=torch.float32, strategy=capi.STRATEGY_GROUP)
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
