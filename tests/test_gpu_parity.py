"""GPU parity: the CUDA path, called through the C ABI, against the CPU oracle.

Bars (from the task's stated tolerances): bit-exact for gather, max and every result
whose summation order is fixed (the lane-group strategy adds rows in bag order, as the
oracle does); relative 1e-5 (fp32) / 1e-3 (fp16) where the CTA and split strategies fold
partial sums in a different association.
"""
import ctypes as C
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from forward_b200 import capi, workloads  # noqa: E402
from oracle import eb_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
NP = {"f32": np.float32, "f16": np.float16}


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


def _cuda(a):
    return None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def gpu_pool(table, indices, offsets=None, **kw):
    """numpy in, numpy out, through fwd_eb_forward."""
    out_dtype = kw.pop("out_dtype", None)
    tdt = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16}
    out = capi.embedding_bag(_cuda(table), _cuda(indices), _cuda(offsets),
                             per_sample_weights=_cuda(kw.pop("per_sample_weights", None)),
                             out_dtype=None if out_dtype is None else tdt[np.dtype(out_dtype)], **kw)
    torch.cuda.synchronize()
    return out.cpu().numpy()


def assert_close(got, exp, dtype, exact):
    assert got.shape == exp.shape and got.dtype == exp.dtype
    if exact:
        bad = np.nonzero(_bits(got) != _bits(exp))
        assert bad[0].size == 0, f"{bad[0].size} mismatching elements, first at {[b[0] for b in bad]}"
    else:
        rtol = 1e-5 if dtype == np.float32 else 1e-3
        np.testing.assert_allclose(got.astype(np.float64), exp.astype(np.float64), rtol=rtol,
                                   atol=rtol * 4)


# ---- the reference's own fixture -----------------------------------------------

def test_reference_fixture_through_legacy_launcher(golden_dir):
    """embedding_bag.pth + the inputs of test_torch_nodes.h:178-185, through the entry point
    with the reference launcher's argument list (int32 indices, fp32, 32-bit sizes)."""
    g = np.load(os.path.join(golden_dir, "embedding_bag_pth.npz"))
    w = _cuda(g["weight"])
    for case in ("unit_test", "trace"):
        idx = _cuda(g[f"{case}_indices"].astype(np.int32))
        off = _cuda(g[f"{case}_offsets"].astype(np.int32))
        out = torch.full((off.numel(), 4), 9.0, device=DEV)
        rc = capi.lib().fwd_eb_bag_f32(idx.data_ptr(), off.data_ptr(), out.data_ptr(), idx.numel(),
                                       off.numel(), w.data_ptr(), 5, 4, 0, capi.MODE_SUM,
                                       C.c_void_p(capi.current_stream_ptr()))
        capi.check(rc)
        torch.cuda.synchronize()
        exp = g[f"{case}_expected"]
        got = out.cpu().numpy()
        assert np.max(np.abs(got - exp)) <= 1e-3  # the reference test's own threshold
        assert np.array_equal(_bits(got), _bits(exp))


def test_committed_torch_cases_on_gpu(golden_dir):
    g = np.load(os.path.join(golden_dir, "torch_cpu_cases.npz"))
    modes = {"sum": capi.MODE_SUM, "mean": capi.MODE_MEAN, "max": capi.MODE_MAX}
    for name in g["names"]:
        key, dtype, dim, mode, variant, pad, ilo = str(name).split("|")
        psw = g[f"{key}_psw"].astype(np.float32) if variant == "weights" else None
        got = gpu_pool(g[f"{key}_table"], g[f"{key}_indices"], g[f"{key}_offsets"],
                       mode=modes[mode], padding_idx=int(pad), include_last_offset=bool(int(ilo)),
                       per_sample_weights=psw)
        exp = g[f"{key}_expected"]
        assert_close(got, exp, np.dtype(dtype).type,
                     exact=not (variant == "weights" and dtype == "float16"))


# ---- exhaustive small shapes -----------------------------------------------------

DIMS = [1, 3, 4, 5, 8, 20, 64, 96, 100, 128, 192, 256, 264, 520, 1024, 1100]


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("dim", DIMS)
def test_small_shapes_all_modes_all_strategies(dt, dim):
    rng = np.random.default_rng(dim * 7 + (dt == "f16"))
    rows = 300
    table = rng.standard_normal((rows, dim)).astype(NP[dt])
    lengths = np.concatenate([np.arange(0, 71), rng.integers(0, 300, 9)])
    rng.shuffle(lengths)
    offsets = workloads.offsets_from_lengths(lengths).astype(np.int32)
    n = int(lengths.sum())
    indices = rng.integers(0, rows, n).astype(np.int32)
    indices[rng.random(n) < 0.1] = 17
    psw = rng.random(n).astype(np.float32)
    for mode in (capi.MODE_SUM, capi.MODE_MEAN, capi.MODE_MAX, capi.MODE_SQUARE_SUM):
        exp = O.pool(table, indices, offsets, mode=mode, padding_idx=17)
        for strat in (capi.STRATEGY_GROUP, capi.STRATEGY_CTA):
            got = gpu_pool(table, indices, offsets, mode=mode, padding_idx=17, strategy=strat)
            exact = strat == capi.STRATEGY_GROUP or mode == capi.MODE_MAX
            assert_close(got, exp, NP[dt], exact)
    expw = O.pool(table, indices, offsets, mode=capi.MODE_SUM, per_sample_weights=psw)
    gotw = gpu_pool(table, indices, offsets, mode=capi.MODE_SUM, per_sample_weights=psw,
                    strategy=capi.STRATEGY_GROUP)
    assert_close(gotw, expw, NP[dt], exact=True)


@pytest.mark.parametrize("dt", ["f32", "f16"])
@pytest.mark.parametrize("mode", [capi.MODE_SUM, capi.MODE_MEAN, capi.MODE_MAX])
def test_long_bags_cta_and_split(dt, mode):
    """Few very long bags: AUTO goes to the split strategy when scratch is offered; the
    forced CTA strategy and the split one agree with the oracle (max bit for bit)."""
    rng = np.random.default_rng(11)
    rows, dim = 5000, 128
    table = rng.standard_normal((rows, dim)).astype(NP[dt])
    if mode == capi.MODE_MAX:
        table = (np.round(table.astype(np.float32) * 4) / 4).astype(NP[dt])
    lengths = np.array([30000, 1, 0, 12345, 70001, 4096])
    offsets = workloads.offsets_from_lengths(lengths).astype(np.int32)
    indices = rng.integers(0, rows, int(lengths.sum())).astype(np.int32)
    indices[rng.random(indices.size) < 0.05] = 0
    exp = O.pool(table, indices, offsets, mode=mode, padding_idx=0)
    t, i, o = _cuda(table), _cuda(indices), _cuda(offsets)
    out = torch.empty((len(lengths), dim), dtype=t.dtype, device=DEV)
    p = capi.make_params(t, i, o, out=out, mode=mode, padding_idx=0)
    need = capi.lib().fwd_eb_workspace_size(C.byref(p))
    assert need > 0
    ws = torch.empty(need, dtype=torch.uint8, device=DEV)
    p.workspace, p.workspace_bytes = ws.data_ptr(), need
    assert capi.lib().fwd_eb_pick_strategy(C.byref(p)) == capi.STRATEGY_SPLIT
    # Sums of tens of thousands of terms: the bar for a re-associated fp32 sum is an error
    # bound relative to the sum of magnitudes (1e-5 fp32 / 1e-3 fp16), measured against a
    # float64 sum, not agreement with one particular fp32 order.
    keep = indices != 0
    vals = np.where(keep[:, None], table[indices].astype(np.float64), 0.0)
    bag_of = np.repeat(np.arange(len(lengths)), lengths)
    exact64 = np.zeros((len(lengths), dim))
    mags = np.zeros((len(lengths), dim))
    np.add.at(exact64, bag_of, vals)
    np.add.at(mags, bag_of, np.abs(vals))
    counts = np.maximum(np.bincount(bag_of, weights=keep, minlength=len(lengths)), 1)[:, None]
    if mode == capi.MODE_MEAN:
        exact64, mags = exact64 / counts, mags / counts
    for strat in (capi.STRATEGY_AUTO, capi.STRATEGY_CTA, capi.STRATEGY_GROUP):
        out.fill_(float("nan"))
        p.strategy = strat
        capi.forward(p)
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        if mode == capi.MODE_MAX or strat == capi.STRATEGY_GROUP:
            assert_close(got, exp, NP[dt], exact=True)
        else:
            rtol = 1e-5 if dt == "f32" else 1e-3
            assert np.all(np.abs(got.astype(np.float64) - exact64) <= rtol * mags + 1e-6)


# ---- API surface: dtypes, strides, windows, gather ---------------------------------

def test_int64_indices_strided_table_and_output_fp32_from_fp16():
    rng = np.random.default_rng(2)
    big = rng.standard_normal((400, 160)).astype(np.float16)
    tview = _cuda(big)[:, :128]                      # row stride 160 elements, still 16 B aligned
    lengths = rng.integers(0, 40, 200)
    offsets = workloads.offsets_from_lengths(lengths)
    indices = rng.integers(0, 400, int(lengths.sum()))
    outbuf = torch.zeros((200, 192), dtype=torch.float32, device=DEV)
    out = outbuf[:, :128]
    p = capi.make_params(tview, _cuda(indices), _cuda(offsets), out=out, mode=capi.MODE_MEAN)
    capi.forward(p)
    torch.cuda.synchronize()
    exp = O.pool(big[:, :128], indices, offsets, mode=O.MODE_MEAN, out_dtype=np.float32)
    assert np.array_equal(_bits(out.cpu().numpy()), _bits(exp))
    assert not outbuf[:, 128:].any()                 # nothing written past the row


def test_misaligned_table_takes_the_scalar_path():
    rng = np.random.default_rng(3)
    flat = _cuda(rng.standard_normal(300 * 64 + 1).astype(np.float32))
    tview = flat[1:].view(300, 64)                   # 4-byte aligned only
    lengths = rng.integers(0, 30, 64)
    offsets = workloads.offsets_from_lengths(lengths).astype(np.int32)
    indices = rng.integers(0, 300, int(lengths.sum())).astype(np.int32)
    out = capi.embedding_bag(tview, _cuda(indices), _cuda(offsets), mode=capi.MODE_SUM)
    torch.cuda.synchronize()
    exp = O.pool(tview.cpu().numpy(), indices, offsets)
    assert np.array_equal(_bits(out.cpu().numpy()), _bits(exp))


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_fixed_length_and_legacy_fixed_launcher(dt):
    rng = np.random.default_rng(4)
    table = rng.standard_normal((1000, 64)).astype(NP[dt])
    idx = rng.integers(0, 1000, (257, 20)).astype(np.int32)
    for mode in (capi.MODE_SUM, capi.MODE_MEAN, capi.MODE_MAX, capi.MODE_SQUARE_SUM):
        got = gpu_pool(table, idx, mode=mode, fixed_len=20)
        assert_close(got, O.pool(table, idx, mode=mode, fixed_len=20), NP[dt], exact=True)
    if dt == "f32":
        t, i = _cuda(table), _cuda(idx)
        out = torch.empty((257, 64), device=DEV)
        capi.check(capi.lib().fwd_eb_bag_fixed_f32(i.data_ptr(), out.data_ptr(), 257, 20,
                                                   t.data_ptr(), 1000, 64, 0, capi.MODE_SUM,
                                                   C.c_void_p(capi.current_stream_ptr())))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), O.pool(table, idx, fixed_len=20))


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_gather_and_window(dt):
    rng = np.random.default_rng(5)
    table = rng.standard_normal((512, 24)).astype(NP[dt])
    idx = rng.integers(0, 512, (33, 7)).astype(np.int32)
    got = gpu_pool(table, idx, mode=capi.MODE_GATHER)
    assert np.array_equal(_bits(got), _bits(table[idx.reshape(-1)]))
    shard = table[128:384]
    got = gpu_pool(shard, idx, mode=capi.MODE_GATHER, row_lo=128)
    exp = O.pool(shard, idx, mode=O.MODE_GATHER, row_lo=128)
    assert np.array_equal(_bits(got), _bits(exp))
    # reference behaviour on request: skipped rows are left as they were
    out = torch.full((idx.size, 24), 5.0, dtype=_cuda(table).dtype, device=DEV)
    capi.embedding_bag(_cuda(shard), _cuda(idx), mode=capi.MODE_GATHER, row_lo=128, out=out,
                       flags=capi.FLAG_GATHER_KEEP_SKIPPED)
    torch.cuda.synchronize()
    inside = ((idx >= 128) & (idx < 384)).reshape(-1)
    o = out.cpu().numpy()
    assert np.all(o[~inside] == 5.0) and np.array_equal(_bits(o[inside]), _bits(exp[inside]))
    if dt == "f32":
        t, i = _cuda(shard), _cuda(idx)
        out = torch.zeros((idx.size, 24), device=DEV)
        capi.check(capi.lib().fwd_eb_gather_f32(i.data_ptr(), out.data_ptr(), 33, 7, t.data_ptr(),
                                                256, 24, 128,
                                                C.c_void_p(capi.current_stream_ptr())))
        torch.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy(), exp)


def test_row_shards_sum_to_the_whole():
    """Pool each of four row windows into an fp32 partial, fold them: equals the unsharded
    result (the window test is the reference's data_offset / count filter, .cu:94)."""
    rng = np.random.default_rng(6)
    rows, dim, shards = 4000, 64, 4
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    bags = workloads.ragged_bags(rows, rng.integers(1, 101, 2000), rng)
    parts = torch.empty((shards, bags.num_bags, dim), dtype=torch.float32, device=DEV)
    idx, off = _cuda(bags.indices), _cuda(bags.offsets)
    for r in range(shards):
        lo = r * rows // shards
        capi.embedding_bag(_cuda(table[lo:lo + rows // shards]), idx, off, mode=capi.MODE_SUM,
                           row_lo=lo, out=parts[r])
    out = torch.empty((bags.num_bags, dim), dtype=torch.float16, device=DEV)
    capi.combine_partials(parts, out)
    torch.cuda.synchronize()
    host_parts = np.stack([O.pool(table[r * 1000:(r + 1) * 1000], bags.indices, bags.offsets,
                                  row_lo=r * 1000, out_dtype=np.float32) for r in range(shards)])
    assert np.array_equal(_bits(parts.cpu().numpy()), _bits(host_parts))
    assert np.array_equal(_bits(out.cpu().numpy()),
                          _bits(O.combine_partials(host_parts, np.float16)))
    whole = O.pool(table, bags.indices, bags.offsets)
    np.testing.assert_allclose(out.cpu().numpy().astype(np.float32), whole.astype(np.float32),
                               rtol=1e-3, atol=4e-3)


def test_empty_inputs_and_guard_rows():
    t = _cuda(np.ones((10, 8), dtype=np.float32))
    empty_i = torch.empty(0, dtype=torch.int32, device=DEV)
    out = capi.embedding_bag(t, empty_i, empty_i, mode=capi.MODE_SUM)       # zero bags
    assert out.shape == (0, 8)
    off = torch.zeros(5, dtype=torch.int32, device=DEV)
    guard = torch.full((7, 8), 3.0, device=DEV)
    capi.embedding_bag(t, empty_i, off, mode=capi.MODE_MAX, out=guard[1:6])  # five empty bags
    torch.cuda.synchronize()
    g = guard.cpu().numpy()
    assert not g[1:6].any() and np.all(g[0] == 3.0) and np.all(g[6] == 3.0)


def test_fill_table_matches_host_twin():
    for dt, tdt in (("f32", torch.float32), ("f16", torch.float16)):
        t = torch.empty((3000, 64), dtype=tdt, device=DEV)
        capi.fill_table(t, row_lo=123_456_789, seed=4, scale=0.05)
        torch.cuda.synchronize()
        rows = np.arange(3000, dtype=np.int64) + 123_456_789
        exp = O.table_rows(rows, 64, seed=4, scale=0.05, dtype=NP[dt])
        assert np.array_equal(_bits(t.cpu().numpy()), _bits(exp))


# ---- the named configurations at full size ------------------------------------------

def test_config1_full():
    table, bags = workloads.config1()
    got = gpu_pool(table, bags.indices, bags.offsets, mode=capi.MODE_SUM)
    assert np.array_equal(_bits(got), _bits(O.pool(table, bags.indices, bags.offsets)))
    ref = O.torch_pool(table, bags.indices, bags.offsets).numpy()
    np.testing.assert_allclose(got, ref, rtol=1e-5, atol=1e-6)


def test_config2_full_mean_fp16_bit_exact_and_deterministic():
    """1M x 128 fp16, 16384 bags, Zipf indices, mean: whole output against the oracle and
    torch CPU; two runs give the same bits (no atomics anywhere)."""
    table = workloads.config2_table()
    bags = workloads.config2_bags()
    t, i, o = _cuda(table), _cuda(bags.indices), _cuda(bags.offsets)
    a = capi.embedding_bag(t, i, o, mode=capi.MODE_MEAN)
    b = capi.embedding_bag(t, i, o, mode=capi.MODE_MEAN)
    torch.cuda.synchronize()
    assert torch.equal(a, b)
    exp = O.pool(table, bags.indices, bags.offsets, mode=O.MODE_MEAN)
    assert_close(a.cpu().numpy(), exp, np.float16, exact=True)
    ref = O.torch_pool(table, bags.indices, bags.offsets, mode=O.MODE_MEAN).numpy()
    np.testing.assert_allclose(a.cpu().numpy().astype(np.float32), ref.astype(np.float32),
                               rtol=1e-3, atol=1e-4)


def test_config3_full_max_padding_ties_bit_exact():
    """4M x 256 fp16 filled on the device by the counter generator; the oracle regenerates
    only the rows the batch touches.  Also a tie-stress variant on a coarsely quantised
    table, where first-of-equals decides many outputs."""
    rows, dim = 4_000_000, 256
    bags = workloads.config3_bags()
    t = torch.empty((rows, dim), dtype=torch.float16, device=DEV)
    capi.fill_table(t, 0, seed=2, scale=0.1)
    got = capi.embedding_bag(t, _cuda(bags.indices), _cuda(bags.offsets), mode=capi.MODE_MAX,
                             padding_idx=0)
    torch.cuda.synchronize()
    uniq, inv = np.unique(bags.indices, return_inverse=True)
    compact = O.table_rows(uniq, dim, seed=2, scale=0.1, dtype=np.float16)
    pad_local = int(np.searchsorted(uniq, 0))
    assert uniq[pad_local] == 0
    exp = O.pool(compact, inv.astype(np.int32), bags.offsets, mode=O.MODE_MAX,
                 padding_idx=pad_local)
    g = got.cpu().numpy()
    assert_close(g, exp, np.float16, exact=True)
    lengths = np.diff(np.append(bags.offsets, bags.num_indices))
    assert not g[lengths == 0].any()                  # empty bags give zeros
    del t
    # tie stress: 3 distinct magnitudes incl. +-0
    rng = np.random.default_rng(9)
    q = rng.choice(np.float16([-0.0, 0.0, -1.0, 1.0, 0.5]), size=(20000, dim))
    tb = workloads.config3_bags(seed=12, num_rows=20000, num_bags=4096)
    got = gpu_pool(q, tb.indices, tb.offsets, mode=capi.MODE_MAX, padding_idx=0)
    assert_close(got, O.pool(q, tb.indices, tb.offsets, mode=O.MODE_MAX, padding_idx=0),
                 np.float16, exact=True)
    ref = O.torch_pool(q, tb.indices, tb.offsets, mode=O.MODE_MAX, padding_idx=0).numpy()
    assert np.array_equal(_bits(got), _bits(ref))


def test_config4_one_table_weighted_sum():
    """One table of the 26 (fixed pooling factor 20, fp32, per-sample weights, Zipf 1.1)."""
    rows = int(workloads.config4_rows()[5])
    bags = workloads.config4_bags(5, rows, batch=8192)
    t = torch.empty((rows, 128), dtype=torch.float32, device=DEV)
    capi.fill_table(t, 0, seed=305, scale=1.0)
    got = capi.embedding_bag(t, _cuda(bags.indices), mode=capi.MODE_SUM, fixed_len=20,
                             per_sample_weights=_cuda(bags.per_sample_weights))
    torch.cuda.synchronize()
    uniq, inv = np.unique(bags.indices, return_inverse=True)
    compact = O.table_rows(uniq, 128, seed=305, scale=1.0, dtype=np.float32)
    exp = O.pool(compact, inv.astype(np.int32), mode=O.MODE_SUM, fixed_len=20,
                 per_sample_weights=bags.per_sample_weights)
    assert_close(got.cpu().numpy(), exp, np.float32, exact=True)


def test_config4_all_26_tables_full_batch_every_strategy():
    """Config 4 as stated: all 26 tables (row counts log-uniform 1e3..4e7, here capped at 2e6 rows so
    that the tables fit next to each other; the indices keep the configuration's Zipf(1.1) law),
    batch 65536, pooling factor 20, per-sample weights, sum — pooled into one [65536, 26, 128]
    result as the table-wise placement lays it out, by the strategy AUTO picks and by the two other
    lane-group kernels; a sample of bags of every table against the CPU oracle, bit for bit."""
    rows_all = [int(min(r, 2_000_000)) for r in workloads.config4_rows()]
    B, L, D, T = 65536, 20, 128, len(rows_all)
    strategies = (capi.STRATEGY_AUTO, capi.STRATEGY_LITE, capi.STRATEGY_GROUP)
    outs = [torch.full((B, T, D), float("nan"), dtype=torch.float32, device=DEV) for _ in strategies]
    take = np.arange(0, B, 97)
    for t, rows in enumerate(rows_all):
        bags = workloads.config4_bags(t, rows)
        table = torch.empty((rows, D), dtype=torch.float32, device=DEV)
        capi.fill_table(table, 0, seed=300 + t, scale=0.1)
        d_idx, d_w = _cuda(bags.indices), _cuda(bags.per_sample_weights)
        for out, strat in zip(outs, strategies):
            capi.forward(capi.make_params(table, d_idx, None, out=out[:, t, :], mode=capi.MODE_SUM, fixed_len=L,
                                          per_sample_weights=d_w, strategy=strat))
        torch.cuda.synchronize()
        idx = bags.indices.reshape(B, L)[take].reshape(-1)
        w = bags.per_sample_weights.reshape(B, L)[take].reshape(-1)
        uniq, inv = np.unique(idx, return_inverse=True)
        compact = O.table_rows(uniq, D, seed=300 + t, scale=0.1, dtype=np.float32)
        exp = O.pool(compact, inv.astype(np.int32), mode=O.MODE_SUM, fixed_len=L, per_sample_weights=w)
        got = outs[0][:, t, :].cpu().numpy()[take]
        assert_close(got, exp, np.float32, exact=True)
    for other in outs[1:]:
        assert torch.equal(other.view(torch.int32), outs[0].view(torch.int32))
    assert not torch.isnan(outs[0]).any()


def test_forward_many_equals_one_call_after_the_other():
    """Seven independent tables of different shapes and modes through fwd_eb_forward_many (the
    caller's stream + the library's auxiliary streams), twice in a row into the same outputs, then
    a dependent kernel on the caller's stream: same bits as fwd_eb_forward on each, and the
    consumer sees finished results (the auxiliary streams are joined)."""
    rng = np.random.default_rng(31)
    shapes = [(3000, 64, torch.float16, capi.MODE_SUM), (500, 128, torch.float32, capi.MODE_MEAN),
              (70000, 256, torch.float16, capi.MODE_MAX), (1200, 32, torch.float32, capi.MODE_SUM),
              (9000, 128, torch.float16, capi.MODE_MEAN), (100, 64, torch.float32, capi.MODE_MAX),
              (40000, 96, torch.float16, capi.MODE_SUM)]
    keep, ps, outs, singles = [], [], [], []
    for k, (rows, dim, dt, mode) in enumerate(shapes):
        table = torch.from_numpy(rng.standard_normal((rows, dim)).astype(np.float32)).to(DEV).to(dt)
        bags = workloads.ragged_bags(rows, rng.integers(0, 50, 3000 + 500 * k), rng)
        i, o = _cuda(bags.indices), _cuda(bags.offsets)
        out = torch.full((bags.num_bags, dim), float("nan"), dtype=dt, device=DEV)
        ref = torch.empty_like(out)
        keep += [table, i, o]
        ps.append(capi.make_params(table, i, o, out=out, mode=mode))
        capi.forward(capi.make_params(table, i, o, out=ref, mode=mode))
        outs.append(out)
        singles.append(ref)
    packed = capi.pack_params(ps)
    capi.forward_many(packed)
    capi.forward_many(packed)
    total = sum(o.float().nan_to_num().sum() for o in outs)      # the caller's stream reads every output
    torch.cuda.synchronize()
    for out, ref in zip(outs, singles):
        assert torch.equal(out.view(torch.int16 if out.dtype == torch.float16 else torch.int32),
                           ref.view(torch.int16 if ref.dtype == torch.float16 else torch.int32))
    assert torch.isfinite(total)
    # an invalid call anywhere in the list: nothing is launched, the others' outputs stay as they were
    for o in outs:
        o.fill_(7.0)
    bad = capi.make_params(keep[0], keep[1], keep[2], out=outs[0], mode=capi.MODE_SUM)
    bad.dim = -5
    with pytest.raises(capi.FwdEbError):
        capi.forward_many(capi.pack_params(ps[1:] + [bad]))
    torch.cuda.synchronize()
    assert all(bool((o == 7.0).all()) for o in outs)
    capi.forward_many(capi.pack_params([]))
    capi.forward_many(capi.pack_params(ps[:1]))


def test_int32_filter_edges_negative_indices_and_window_origin():
    """int32 indices take a 32-bit filter: negative indices, indices below the window origin and
    a negative origin (the reference's data_offset is a signed int) must behave as in the oracle."""
    rng = np.random.default_rng(77)
    table = rng.standard_normal((100, 16)).astype(np.float32)
    idx = rng.integers(-50, 300, 4000).astype(np.int32)
    idx[::50] = np.iinfo(np.int32).min
    idx[1::50] = np.iinfo(np.int32).max
    lengths = rng.integers(0, 40, 200)
    lengths[-1] += 4000 - lengths.sum() if lengths.sum() < 4000 else 0
    off = workloads.offsets_from_lengths(lengths).astype(np.int32)
    n = int(lengths.sum())
    idx = idx[:n] if n <= idx.size else np.resize(idx, n)
    for row_lo in (0, 120, -30):
        for mode in (capi.MODE_SUM, capi.MODE_MEAN, capi.MODE_MAX):
            got = gpu_pool(table, idx, off, mode=mode, row_lo=row_lo, padding_idx=7)
            exp = O.pool(table, idx, off, mode=mode, row_lo=row_lo, padding_idx=7)
            assert_close(got, exp, np.float32, exact=True)
            got64 = gpu_pool(table, idx.astype(np.int64), off.astype(np.int64), mode=mode,
                             row_lo=row_lo, padding_idx=7)
            assert_close(got64, exp, np.float32, exact=True)


@pytest.mark.parametrize("dt", ["f32", "f16"])
def test_max_with_nan_rows_follows_torch_in_every_strategy(dt):
    """torch's max keeps the bag's first entry as is and later entries only when strictly greater:
    a NaN in the middle of a bag is ignored.  The CTA and split strategies cut a bag into slices;
    a slice that starts with a NaN row must not lose the larger values behind it."""
    rng = np.random.default_rng(71)
    rows, dim = 500, 64
    table = rng.standard_normal((rows, dim)).astype(NP[dt])
    table[7] = np.nan                     # a whole NaN row
    table[11, ::3] = np.nan               # NaN in some columns only
    table[13] = 100.0                     # the value that must survive
    lengths = np.array([4000, 1, 2500, 300, 0, 5000])
    offsets = workloads.offsets_from_lengths(lengths).astype(np.int32)
    idx = rng.integers(14, rows, int(lengths.sum())).astype(np.int32)   # no NaN rows yet
    idx[1::5] = 7                          # NaN rows all over every bag, never at a bag's start
    idx[3::11] = 11
    idx[offsets[0] + 3999] = 13            # 100 at the very end of bag 0, behind many NaN rows
    idx[offsets[2] + 1300] = 13
    idx[offsets[:4]] = 20                  # every non-empty bag starts with an ordinary row
    idx[offsets[5]] = 20
    t, i, o = torch.from_numpy(table), torch.from_numpy(idx.astype(np.int64)), torch.from_numpy(offsets.astype(np.int64))
    exp = torch.nn.functional.embedding_bag(i, t.float(), o, mode="max").numpy().astype(NP[dt])
    assert not np.isnan(exp).any() and exp[0].max() == 100.0
    ws = torch.empty(1 << 24, dtype=torch.uint8, device=DEV)
    for strat in (capi.STRATEGY_GROUP, capi.STRATEGY_CTA, capi.STRATEGY_SPLIT, capi.STRATEGY_AUTO):
        out = torch.empty((lengths.size, dim), dtype=torch.float16 if dt == "f16" else torch.float32, device=DEV)
        p = capi.make_params(_cuda(table), _cuda(idx), _cuda(offsets), out=out, mode=capi.MODE_MAX,
                             strategy=strat, workspace=ws)
        capi.forward(p)
        torch.cuda.synchronize()
        assert np.array_equal(_bits(out.cpu().numpy()), _bits(exp)), strat
