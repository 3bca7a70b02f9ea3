"""The fused pool-and-push kernels on ONE GPU: every "rank" is a set of buffers on the same
device and the ranks' launches run one after another on one stream.  A fold / wait kernel
raises its own rank's flag and then waits for the others', so here every rank's flag is raised
explicitly (fwd_eb_shard_signal) before the first fold runs: no kernel ever waits for a kernel
queued behind it.  Real multi-GPU runs are in test_gpu_multi.py."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from forward_b200 import capi, workloads  # noqa: E402
from forward_b200 import dist as fd  # noqa: E402
from oracle import eb_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _cuda(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def _setup(world, per, dim, wire, layout=fd.LAYOUT_ROW_SHARD, num_tables=0, max_spins=0):
    lib = fd._lib()
    nbytes = (lib.fwd_eb_shard_tablewise_bytes(per, num_tables, dim, wire) if num_tables else
              lib.fwd_eb_shard_slots_bytes(world, per, dim, wire))
    bufs = fd.PeerBuffers(nbytes, world, 0, local_world=world)
    xs, keep = [], []
    for r in range(world):
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        keep += [status]
        xs.append(fd.make_exchange(bufs, r, per, wire, status, layout=layout,
                                   num_tables=num_tables, max_spins=max_spins))
    return lib, bufs, xs, keep


@pytest.mark.parametrize("wire", [capi.F32, capi.F16])
@pytest.mark.parametrize("mode", [capi.MODE_SUM, capi.MODE_MEAN])
def test_row_shard_push_and_combine_four_ranks(wire, mode):
    rng = np.random.default_rng(8)
    world, rows, dim, nb = 4, 8000, 64, 1000          # 1000 bags: the last rank owns fewer
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, wire)
    stream = C.c_void_p(capi.current_stream_ptr())
    shards = [fd.shard_rows(rows, world, r) for r in range(world)]
    tabs = [_cuda(table[lo:lo + n]) for lo, n in shards]
    for epoch in (1, 2, 3):                            # both buffer halves, fresh inputs each call
        bags = workloads.ragged_bags(rows, rng.integers(0, 60, nb), rng)
        bags.indices[::7] = 5
        i, o = _cuda(bags.indices), _cuda(bags.offsets)
        for r in range(world):
            xs[r].epoch = epoch
            p = capi.make_params(tabs[r], i, o, out=tabs[r][:1], mode=mode, padding_idx=5,
                                 row_lo=shards[r][0])
            capi.check(lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[r]), stream))
        for r in range(world):
            capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
        parts = np.stack([O.pool(table[lo:lo + n], bags.indices, bags.offsets, mode=mode,
                                 padding_idx=5, row_lo=lo, out_dtype=np.float32)
                          for lo, n in shards])
        if wire == capi.F16:
            parts = parts.astype(np.float16)
        expect = O.combine_partials(parts, np.float32)
        for r in range(world):
            lo, mine = fd.owned_bags(nb, world, r)
            out = torch.full((per, dim), float("nan"), device=DEV)
            capi.check(lib.fwd_eb_shard_combine(C.byref(xs[r]), dim, mine, out.data_ptr(), capi.F32,
                                                stream))
            torch.cuda.synchronize()
            assert np.array_equal(out[:mine].cpu().numpy(), expect[lo:lo + mine])
            assert torch.isnan(out[mine:]).all()
    assert all(int(k.item()) == 0 for k in keep)       # no timeouts
    whole = O.pool(table, bags.indices, bags.offsets, mode=mode, padding_idx=5, out_dtype=np.float32)
    np.testing.assert_allclose(expect, whole, rtol=1e-3, atol=2e-2 if wire == capi.F16 else 1e-4)


@pytest.mark.parametrize("wire", [capi.F32, capi.F16])
def test_row_shard_staged_send_equals_push(wire):
    """The copy-engine exchange: plain pooling into a staging buffer, one copy per owner, then the
    same flags and fold; bit-identical to the CPU fold of the ranks' partials."""
    rng = np.random.default_rng(18)
    world, rows, dim, nb = 4, 6000, 64, 1000
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, wire)
    stream = C.c_void_p(capi.current_stream_ptr())
    shards = [fd.shard_rows(rows, world, r) for r in range(world)]
    tabs = [_cuda(table[lo:lo + n]) for lo, n in shards]
    wdt = torch.float16 if wire == capi.F16 else torch.float32
    for epoch, mode in ((1, capi.MODE_SUM), (2, capi.MODE_MEAN)):
        bags = workloads.ragged_bags(rows, rng.integers(0, 60, nb), rng)
        i, o = _cuda(bags.indices), _cuda(bags.offsets)
        for r in range(world):
            xs[r].epoch = epoch
            stage = torch.empty((nb, dim), dtype=wdt, device=DEV)
            p = capi.make_params(tabs[r], i, o, out=stage, mode=mode, row_lo=shards[r][0],
                                 flags=capi.FLAG_MEAN_SINGLE_ROUNDING)
            capi.forward(p)
            capi.check(lib.fwd_eb_shard_send_staged(C.byref(xs[r]), dim, nb, stage.data_ptr(), stream))
        for r in range(world):
            capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
        parts = np.stack([O.pool(table[lo:lo + n], bags.indices, bags.offsets, mode=mode, row_lo=lo,
                                 out_dtype=np.float32) for lo, n in shards])
        if wire == capi.F16:
            parts = parts.astype(np.float16)
        expect = O.combine_partials(parts, np.float32)
        for r in range(world):
            lo, mine = fd.owned_bags(nb, world, r)
            out = torch.empty((per, dim), device=DEV)
            capi.check(lib.fwd_eb_shard_combine(C.byref(xs[r]), dim, mine, out.data_ptr(), capi.F32,
                                                stream))
            torch.cuda.synchronize()
            assert np.array_equal(out[:mine].cpu().numpy(), expect[lo:lo + mine])
    assert all(int(k.item()) == 0 for k in keep)


@pytest.mark.parametrize("wire", [capi.F32, capi.F16])
@pytest.mark.parametrize("mode", [capi.MODE_SUM, capi.MODE_MEAN])
def test_row_shard_compacted_push_equals_the_replicated_scan(wire, mode):
    """Window compaction first, then the pooling kernel pushes the dense sub-bags' partial rows:
    for SUM the result is bit-identical to the fold of the ranks' partials (what the push and the
    staged exchange give); a MEAN is folded as sums and divided by the bag's full count."""
    rng = np.random.default_rng(28)
    world, rows, dim, nb = 4, 8000, 64, 1000
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, wire)
    stream = C.c_void_p(capi.current_stream_ptr())
    shards = [fd.shard_rows(rows, world, r) for r in range(world)]
    tabs = [_cuda(table[lo:lo + n]) for lo, n in shards]
    for epoch in (1, 2):
        bags = workloads.ragged_bags(rows, rng.integers(0, 60, nb), rng)
        bags.indices[::7] = 5
        i, o = _cuda(bags.indices), _cuda(bags.offsets)
        counts = []
        for r in range(world):
            xs[r].epoch = epoch
            kept = torch.empty(bags.num_indices, dtype=torch.int32, device=DEV)
            bounds = torch.empty((nb, 2), dtype=torch.int32, device=DEV)
            cnt = torch.zeros(nb, dtype=torch.int32, device=DEV)
            p = capi.make_params(tabs[r], i, o, out=tabs[r][:1], mode=mode, padding_idx=5,
                                 row_lo=shards[r][0])
            capi.compact_window(p, kept, bounds, counts=cnt)
            q = capi.make_compacted_params(tabs[r], kept, bounds, out=tabs[r][:1], mode=capi.MODE_SUM)
            capi.check(lib.fwd_eb_shard_push(C.byref(q), C.byref(xs[r]), stream))
            counts.append(cnt)
            keep += [kept, bounds]
        for r in range(world):
            capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
        parts = np.stack([O.pool(table[lo:lo + n], bags.indices, bags.offsets, mode=O.MODE_SUM,
                                 padding_idx=5, row_lo=lo, out_dtype=np.float32) for lo, n in shards])
        if wire == capi.F16:
            parts = parts.astype(np.float16)
        expect = O.combine_partials(parts, np.float32)
        if mode == capi.MODE_MEAN:
            ends = np.append(bags.offsets, bags.num_indices)
            full = np.array([np.count_nonzero(bags.indices[ends[b]:ends[b + 1]] != 5) for b in range(nb)])
            expect = (expect / np.maximum(full, 1)[:, None].astype(np.float32)).astype(np.float32)
        for r in range(world):
            lo, mine = fd.owned_bags(nb, world, r)
            out = torch.full((per, dim), float("nan"), device=DEV)
            cptr = C.c_void_p(counts[r][lo:].data_ptr()) if mode == capi.MODE_MEAN else None
            capi.check(lib.fwd_eb_shard_combine_div(C.byref(xs[r]), dim, mine, cptr, out.data_ptr(),
                                                    capi.F32, stream))
            torch.cuda.synchronize()
            assert np.array_equal(out[:mine].cpu().numpy(), expect[lo:lo + mine])
    assert all(int(k.item()) == 0 for k in keep if k.numel() == 1 and k.dtype == torch.int32)


@pytest.mark.parametrize("wire", [capi.F32, capi.F16])
def test_staged_rows_shipped_by_the_copy_kernel_equal_the_fused_push(wire):
    """x->stage set: the pooling kernel writes every partial row locally and fwd_eb_shard_ship sends
    them on.  Row shards (3 ranks, the last one owning fewer bags) and table-wise placement
    (5 tables on 2 ranks): the owners' results are those of the fused push, bit for bit."""
    rng = np.random.default_rng(61)
    world, rows, dim, nb = 3, 6000, 64, 1000
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, wire)
    stream = C.c_void_p(capi.current_stream_ptr())
    shards = [fd.shard_rows(rows, world, r) for r in range(world)]
    tabs = [_cuda(table[lo:lo + n]) for lo, n in shards]
    stage_bytes = lib.fwd_eb_shard_stage_bytes(world, per, 1, dim, wire)
    for epoch in (1, 2, 9):                          # 9: the part after a wrap of the eight
        bags = workloads.ragged_bags(rows, rng.integers(0, 60, nb), rng)
        i, o = _cuda(bags.indices), _cuda(bags.offsets)
        for r in range(world):
            stage = torch.zeros(stage_bytes, dtype=torch.uint8, device=DEV)
            keep.append(stage)
            xs[r].epoch = epoch
            xs[r].stage = stage.data_ptr()
            xs[r].stage_tables = 1
            p = capi.make_params(tabs[r], i, o, out=tabs[r][:1], mode=capi.MODE_SUM, row_lo=shards[r][0])
            capi.check(lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[r]), stream))
            capi.check(lib.fwd_eb_shard_ship(C.byref(xs[r]), dim, nb, None, stream))
        for r in range(world):
            capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
        parts = np.stack([O.pool(table[lo:lo + n], bags.indices, bags.offsets, mode=O.MODE_SUM, row_lo=lo,
                                 out_dtype=np.float32) for lo, n in shards])
        if wire == capi.F16:
            parts = parts.astype(np.float16)
        expect = O.combine_partials(parts, np.float32)
        for r in range(world):
            lo, mine = fd.owned_bags(nb, world, r)
            out = torch.empty((per, dim), device=DEV)
            capi.check(lib.fwd_eb_shard_combine(C.byref(xs[r]), dim, mine, out.data_ptr(), capi.F32, stream))
            torch.cuda.synchronize()
            assert np.array_equal(out[:mine].cpu().numpy(), expect[lo:lo + mine])
    # table-wise: tables 0, 2, 4 on rank 0 and 1, 3 on rank 1
    world, ntab, L, dim, nb = 2, 5, 6, 32, 999
    owner = [0, 1, 0, 1, 0]
    tables = [rng.standard_normal((800 + 50 * t, dim)).astype(np.float32) for t in range(ntab)]
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep2 = _setup(world, per, dim, capi.F32, layout=fd.LAYOUT_TABLE_WISE, num_tables=ntab)
    idx = [rng.integers(0, tables[t].shape[0], (nb, L)).astype(np.int32) for t in range(ntab)]
    for r in range(world):
        mine_t = [t for t in range(ntab) if owner[t] == r]
        stage = torch.zeros(lib.fwd_eb_shard_stage_bytes(world, per, len(mine_t), dim, capi.F32),
                            dtype=torch.uint8, device=DEV)
        keep2.append(stage)
        xs[r].epoch = 1
        xs[r].stage = stage.data_ptr()
        xs[r].stage_tables = len(mine_t)
        for j, t in enumerate(mine_t):
            tt, ii = _cuda(tables[t]), _cuda(idx[t])
            keep2 += [tt, ii]
            xs[r].table_index, xs[r].stage_slot = t, j
            p = capi.make_params(tt, ii, None, out=tt[:1], mode=capi.MODE_SUM, fixed_len=L)
            capi.check(lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[r]), stream))
        ids = (C.c_int32 * len(mine_t))(*mine_t)
        capi.check(lib.fwd_eb_shard_ship(C.byref(xs[r]), dim, nb, ids, stream))
    for r in range(world):
        capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
    expect = np.stack([O.pool(tables[t], idx[t], fixed_len=L) for t in range(ntab)], axis=1)
    for r in range(world):
        res = C.c_void_p()
        capi.check(lib.fwd_eb_shard_wait(C.byref(xs[r]), dim, C.byref(res), stream))
        torch.cuda.synchronize()
        lo, mine = fd.owned_bags(nb, world, r)
        got = torch.as_tensor(fd._DeviceView(res.value, (per, ntab, dim), "<f4"), device="cuda")
        assert np.array_equal(got[:mine].cpu().numpy(), expect[lo:lo + mine])


def test_row_shard_config5_geometry_small_window():
    """Config 5's numbers on a small physical window: logical rows up to 10^9 (int32 indices near
    2^30), a shard whose row_lo lies beyond 5*10^8, G = 8 windows of which this GPU holds one.
    The compacted path and the replicated scan must agree bit for bit with the CPU oracle."""
    rng = np.random.default_rng(45)
    G, dim, nb = 8, 64, 4096
    logical = 1_000_000_000
    per_rows = logical // G
    rank = 5                                             # row_lo = 625,000,000
    row_lo = rank * per_rows
    phys = 50_000                                        # rows actually held: the head of the window
    table = torch.empty((phys, dim), dtype=torch.float16, device=DEV)
    capi.fill_table(table, row_lo, seed=4, scale=0.05)
    lengths = rng.integers(1, 101, nb)
    n = int(lengths.sum())
    idx = rng.integers(0, logical, n)
    near = rng.random(n) < 0.3                           # a third of the lookups land in the held rows
    idx[near] = row_lo + rng.integers(0, phys, int(near.sum()))
    idx[rng.random(n) < 0.01] = logical - 1              # the largest index of the table
    idx = idx.astype(np.int32)
    off = workloads.offsets_from_lengths(lengths).astype(np.int32)
    host_rows = O.table_rows(np.arange(row_lo, row_lo + phys, dtype=np.int64), dim, seed=4, scale=0.05,
                             dtype=np.float16)
    exp = O.pool(host_rows, idx, off, mode=O.MODE_SUM, row_lo=row_lo, out_dtype=np.float32)
    i, o = _cuda(idx), _cuda(off)
    scan = capi.embedding_bag(table, i, o, row_lo=row_lo, out_dtype=torch.float32)
    kept = torch.empty(n, dtype=torch.int32, device=DEV)
    bounds = torch.empty((nb, 2), dtype=torch.int32, device=DEV)
    out = torch.empty((nb, dim), dtype=torch.float32, device=DEV)
    p = capi.make_params(table, i, o, out=out, row_lo=row_lo)
    capi.compact_window(p, kept, bounds)
    capi.forward(capi.make_compacted_params(table, kept, bounds, out=out))
    torch.cuda.synchronize()
    assert np.array_equal(scan.cpu().numpy(), exp)
    assert np.array_equal(out.cpu().numpy(), exp)


def _tricky_table(rng, rows, dim, dtype):
    """Few distinct values (many ties), signed zeros and some NaN rows."""
    t = rng.integers(-2, 3, (rows, dim)).astype(dtype)
    t[rng.random((rows, dim)) < 0.15] = -0.0
    t[::17] = np.nan
    return t


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_max_with_positions_matches_the_sequential_rule(dtype):
    rng = np.random.default_rng(31)
    rows, dim, nb = 300, 40, 257                      # dim 40: fp32 rows of 160 B, 10 chunks
    table = _tricky_table(rng, rows, dim, dtype)
    bags = workloads.ragged_bags(rows, rng.integers(0, 45, nb), rng)
    bags.indices[::5] = 7
    lo, n = 100, 120                                  # a row window in the middle
    out = torch.empty((nb, dim, 2), dtype=torch.float32, device=DEV)
    p = capi.make_params(_cuda(table[lo:lo + n]), _cuda(bags.indices), _cuda(bags.offsets),
                         out=out.view(nb, 2 * dim)[:, :dim], mode=capi.MODE_MAX, padding_idx=7, row_lo=lo)
    p.out, p.out_dtype, p.out_stride = out.data_ptr(), capi.F32_POS, 0
    capi.forward(p)
    torch.cuda.synchronize()
    got = out.cpu().numpy()
    val, pos = O.max_with_positions(table[lo:lo + n], bags.indices, bags.offsets, row_lo=lo, padding_idx=7)
    assert np.array_equal(got[..., 1].view(np.int32), pos)
    gv = np.ascontiguousarray(got[..., 0])
    same = gv.view(np.uint32) == val.view(np.uint32)
    assert (same | (np.isnan(gv) & np.isnan(val))).all()      # NaN payloads may differ


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
def test_row_shard_max_equals_torch_on_the_whole_table(dtype):
    """Sharded MAX (staged exchange, {value, position} partials) against torch CPU EmbeddingBag on
    the unsharded table, bit for bit: ties, signed zeros, a NaN as first entry, padding, empty bags."""
    import torch.nn.functional as F
    rng = np.random.default_rng(32)
    world, rows, dim, nb = 4, 400, 64, 600
    table = _tricky_table(rng, rows, dim, dtype)
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, capi.F32_POS)
    stream = C.c_void_p(capi.current_stream_ptr())
    shards = [fd.shard_rows(rows, world, r) for r in range(world)]
    tabs = [_cuda(table[lo:lo + n]) for lo, n in shards]
    tdt = torch.float16 if dtype == np.float16 else torch.float32
    for epoch in (1, 2):
        bags = workloads.ragged_bags(rows, rng.integers(0, 30, nb), rng)
        bags.indices[::9] = 3
        i, o = _cuda(bags.indices), _cuda(bags.offsets)
        for r in range(world):
            xs[r].epoch = epoch
            stage = torch.empty((nb, 2 * dim), dtype=torch.float32, device=DEV)
            p = capi.make_params(tabs[r], i, o, out=stage[:, :dim], mode=capi.MODE_MAX, padding_idx=3,
                                 row_lo=shards[r][0])
            p.out, p.out_dtype, p.out_stride = stage.data_ptr(), capi.F32_POS, 0
            capi.forward(p)
            capi.check(lib.fwd_eb_shard_send_staged(C.byref(xs[r]), dim, nb, stage.data_ptr(), stream))
        for r in range(world):
            capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
        expect = F.embedding_bag(torch.from_numpy(bags.indices.astype(np.int64)), torch.from_numpy(table),
                                 torch.from_numpy(bags.offsets.astype(np.int64)), mode="max",
                                 padding_idx=3).numpy()
        bits = np.uint16 if dtype == np.float16 else np.uint32
        for r in range(world):
            lo, mine = fd.owned_bags(nb, world, r)
            out = torch.empty((per, dim), dtype=tdt, device=DEV)
            capi.check(lib.fwd_eb_shard_combine(C.byref(xs[r]), dim, mine, out.data_ptr(),
                                                capi.F16 if dtype == np.float16 else capi.F32, stream))
            torch.cuda.synchronize()
            got = out[:mine].cpu().numpy()
            same = got.view(bits) == expect[lo:lo + mine].view(bits)
            both_nan = np.isnan(got) & np.isnan(expect[lo:lo + mine])   # NaN payloads may differ
            assert (same | both_nan).all()
    assert all(int(k.item()) == 0 for k in keep)


def test_table_wise_push_lands_in_result_layout():
    rng = np.random.default_rng(9)
    world, ntab, dim, nb, L = 2, 5, 32, 96, 4
    owner = fd.place_tables([1] * ntab, world)
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, capi.F32, layout=fd.LAYOUT_TABLE_WISE,
                                 num_tables=ntab)
    stream = C.c_void_p(capi.current_stream_ptr())
    tables = [rng.standard_normal((200 + 10 * t, dim)).astype(np.float32) for t in range(ntab)]
    idx = [rng.integers(0, tables[t].shape[0], (nb, L)).astype(np.int32) for t in range(ntab)]
    w = [rng.random(nb * L).astype(np.float32) for _ in range(ntab)]
    keepalive = []
    for r in range(world):
        mine = [t for t in range(ntab) if owner[t] == r]
        xs[r].epoch = 1
        for k, t in enumerate(mine):
            tt, ii, ww = _cuda(tables[t]), _cuda(idx[t]), _cuda(w[t])
            keepalive += [tt, ii, ww]
            p = capi.make_params(tt, ii, None, out=tt[:1], mode=capi.MODE_SUM, fixed_len=L,
                                 per_sample_weights=ww)
            xs[r].table_index = t
            capi.check(lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[r]), stream))
    for r in range(world):
        capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
    expect = np.stack([O.pool(tables[t], idx[t], mode=O.MODE_SUM, fixed_len=L, per_sample_weights=w[t])
                       for t in range(ntab)], axis=1)                      # [nb, T, dim]
    for r in range(world):
        res = C.c_void_p()
        capi.check(lib.fwd_eb_shard_wait(C.byref(xs[r]), dim, C.byref(res), stream))
        torch.cuda.synchronize()
        got = torch.as_tensor(fd._DeviceView(res.value, (per, ntab, dim), "<f4"), device="cuda")
        assert np.array_equal(got.cpu().numpy(), expect[r * per:(r + 1) * per])
    assert all(int(k.item()) == 0 for k in keep)


@pytest.mark.parametrize("wire", [capi.F32, capi.F16])
def test_table_wise_with_replicated_tables_pooled_by_each_rank_for_its_own_bags(wire):
    """Three ranks, five tables: the two large ones live on one rank each and are pushed, the
    three small ones are held by every rank, which pools only the bags it owns straight into its
    own buffer (fwd_eb_shard_pool_local).  Ragged bags, mean, 100 bags on 3 ranks (the last rank
    owns fewer); every rank's [per, T, dim] equals the single-GPU result."""
    rng = np.random.default_rng(19)
    world, ntab, dim, nb = 3, 5, 64, 100
    sizes = [300, 4000, 200, 5000, 250]
    owner = fd.place_tables([n * dim * 2 for n in sizes], world, replicate_below_bytes=1000 * dim * 2)
    assert [o == fd.REPLICATED for o in owner] == [True, False, True, False, True]
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, wire, layout=fd.LAYOUT_TABLE_WISE, num_tables=ntab)
    stream = C.c_void_p(capi.current_stream_ptr())
    tables = [rng.standard_normal((n, dim)).astype(np.float16) for n in sizes]
    bags = [workloads.ragged_bags(n, rng.integers(0, 30, nb), rng) for n in sizes]
    d_tab = [_cuda(t) for t in tables]
    d_idx = [_cuda(b.indices) for b in bags]
    d_off = [_cuda(b.offsets) for b in bags]
    for r in range(world):
        xs[r].epoch = 2
        for t in range(ntab):
            xs[r].table_index = t
            if owner[t] == r:
                p = capi.make_params(d_tab[t], d_idx[t], d_off[t], out=d_tab[t][:1], mode=capi.MODE_MEAN)
                capi.check(lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[r]), stream))
            elif owner[t] == fd.REPLICATED:
                lo, hi = r * per, min(nb, (r + 1) * per)
                last = hi == nb
                off = d_off[t][lo:hi] if last else d_off[t][lo:hi + 1]
                p = capi.make_params(d_tab[t], d_idx[t], off, out=d_tab[t][:1], mode=capi.MODE_MEAN,
                                     include_last_offset=not last)
                assert p.num_bags == hi - lo
                capi.check(lib.fwd_eb_shard_pool_local(C.byref(p), C.byref(xs[r]), stream))
    for r in range(world):
        capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
    odt = np.float16 if wire == capi.F16 else np.float32
    expect = np.stack([O.pool(tables[t], bags[t].indices, bags[t].offsets, mode=O.MODE_MEAN, out_dtype=odt)
                       for t in range(ntab)], axis=1)
    for r in range(world):
        res = C.c_void_p()
        capi.check(lib.fwd_eb_shard_wait(C.byref(xs[r]), dim, C.byref(res), stream))
        torch.cuda.synchronize()
        got = torch.as_tensor(fd._DeviceView(res.value, (per, ntab, dim), "<f2" if wire == capi.F16 else "<f4"),
                              device="cuda").cpu().numpy()
        mine = min(nb, (r + 1) * per) - r * per
        assert np.array_equal(got[:mine].view(np.uint16 if wire == capi.F16 else np.uint32),
                              expect[r * per:r * per + mine].view(np.uint16 if wire == capi.F16 else np.uint32))
    assert all(int(k.item()) == 0 for k in keep)
    # a batch larger than a rank's share is refused
    p = capi.make_params(d_tab[0], d_idx[0], d_off[0], out=d_tab[0][:1], mode=capi.MODE_MEAN)
    assert lib.fwd_eb_shard_pool_local(C.byref(p), C.byref(xs[0]), stream) == capi.EINVAL


def test_wait_gives_up_and_reports_instead_of_hanging():
    """Nothing raises rank 1's flag: the bounded wait runs out after a few thousand polls, sets
    the status word and leaves the output alone; the context stays usable."""
    world, per, dim = 2, 8, 16
    lib, bufs, xs, keep = _setup(world, per, dim, capi.F32, max_spins=2000)
    stream = C.c_void_p(capi.current_stream_ptr())
    xs[0].epoch = 1                                              # rank 0's fold raises its own flag;
                                                                 # rank 1 never raises its
    out = torch.full((per, dim), 7.0, device=DEV)
    capi.check(lib.fwd_eb_shard_combine(C.byref(xs[0]), dim, per, out.data_ptr(), capi.F32, stream))
    torch.cuda.synchronize()
    status0 = keep[0]
    assert int(status0.item()) == fd.SHARD_TIMEOUT
    assert torch.all(out == 7.0)
    assert float((out + 1).sum().item()) == per * dim * 8.0       # device still answers


def test_argument_errors():
    lib, bufs, xs, keep = _setup(2, 8, 16, capi.F32)
    t = torch.zeros((4, 16), device=DEV)
    i = torch.zeros(4, dtype=torch.int32, device=DEV)
    p = capi.make_params(t, i, i, out=t, mode=capi.MODE_MAX)
    xs[0].epoch = 1
    assert lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[0]), None) == capi.EUNSUPPORTED
    p.mode = capi.MODE_SUM
    xs[0].epoch = 0
    assert lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[0]), None) == capi.EINVAL
    xs[0].epoch, xs[0].world = 1, 99
    assert lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[0]), None) == capi.EINVAL


def test_row_shard_push_wide_rows_span_column_tiles():
    """2304 fp16 columns = 288 chunks: three column tiles per bag tile through the work dispenser."""
    rng = np.random.default_rng(10)
    world, rows, dim, nb = 2, 600, 2304, 70
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    per = fd.bags_per_rank(nb, world)
    lib, bufs, xs, keep = _setup(world, per, dim, capi.F32)
    stream = C.c_void_p(capi.current_stream_ptr())
    bags = workloads.ragged_bags(rows, rng.integers(0, 20, nb), rng)
    i, o = _cuda(bags.indices), _cuda(bags.offsets)
    shards = [fd.shard_rows(rows, world, r) for r in range(world)]
    tabs = [_cuda(table[lo:lo + n]) for lo, n in shards]
    for r in range(world):
        xs[r].epoch = 1
        p = capi.make_params(tabs[r], i, o, out=tabs[r][:1], mode=capi.MODE_SUM, row_lo=shards[r][0])
        capi.check(lib.fwd_eb_shard_push(C.byref(p), C.byref(xs[r]), stream))
    for r in range(world):
        capi.check(lib.fwd_eb_shard_signal(C.byref(xs[r]), stream))
    parts = np.stack([O.pool(table[lo:lo + n], bags.indices, bags.offsets, row_lo=lo,
                             out_dtype=np.float32) for lo, n in shards])
    expect = O.combine_partials(parts, np.float32)
    for r in range(world):
        lo, mine = fd.owned_bags(nb, world, r)
        out = torch.empty((per, dim), device=DEV)
        capi.check(lib.fwd_eb_shard_combine(C.byref(xs[r]), dim, mine, out.data_ptr(), capi.F32, stream))
        torch.cuda.synchronize()
        assert np.array_equal(out[:mine].cpu().numpy(), expect[lo:lo + mine])
