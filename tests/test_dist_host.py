"""Host-side logic of the multi-GPU paths on CPU: shard geometry, table placement, and the
exchange + fold plumbing run as two gloo ranks (partials come from the oracle here — the
product has no CPU pooling path)."""
import os
import sys

import numpy as np
import pytest

from forward_b200 import dist as fd
from forward_b200 import workloads

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rows_cover_the_table_once():
    for rows, world in [(10, 3), (1_000_000_000, 8), (7, 8), (16, 4), (1, 2)]:
        spans = [fd.shard_rows(rows, world, r) for r in range(world)]
        assert spans[0][0] == 0 and sum(n for _, n in spans) == rows
        for (lo, n), (lo2, _) in zip(spans, spans[1:]):
            assert lo + n == lo2 or n == 0
        assert max(n for _, n in spans) - min(n for _, n in spans if n) <= max(n for _, n in spans)


def test_owned_bags_partition_the_batch():
    for bags, world in [(131072, 8), (10, 4), (3, 8), (16384, 2)]:
        per = fd.bags_per_rank(bags, world)
        got = [fd.owned_bags(bags, world, r) for r in range(world)]
        assert sum(n for _, n in got) == bags and all(n <= per for _, n in got)
        assert [lo for lo, _ in got] == [min(r * per, bags) for r in range(world)]


def test_table_placement_balances_count_and_bytes():
    rng = np.random.default_rng(3)
    rows = np.round(np.exp(rng.uniform(np.log(1e3), np.log(4e7), 26))).astype(np.int64)
    nbytes = [int(r) * 128 * 4 for r in rows]
    owner = fd.place_tables(nbytes, 8)
    counts = np.bincount(owner, minlength=8)
    assert counts.max() - counts.min() <= 1 and counts.sum() == 26      # 4,4,3,3,3,3,3,3
    held = np.bincount(owner, weights=nbytes, minlength=8)
    assert held.max() < 0.5 * sum(nbytes)
    assert owner == fd.place_tables(nbytes, 8)                          # deterministic
    assert fd.place_tables(nbytes, 1) == [0] * 26
    skew = fd.place_tables([1, 1, 1, 1], 2, lookups=[100, 1, 1, 1])
    assert skew.count(skew[0]) == 1                                     # the heavy table sits alone


def _worker(rank, world, port, method, tmp):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from forward_b200 import dist as fd2
    from forward_b200 import workloads
    from oracle import eb_oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    rng = np.random.default_rng(5)                       # same draw on every rank
    rows, dim, bags_n = 999, 24, 50
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    bags = workloads.ragged_bags(rows, rng.integers(0, 30, bags_n), rng)
    lo, n = fd2.shard_rows(rows, world, rank)
    per = fd2.bags_per_rank(bags_n, world)
    partial = np.zeros((per * world, dim), dtype=np.float32)
    partial[:bags_n] = O.pool(table[lo:lo + n], bags.indices, bags.offsets, mode=O.MODE_MEAN,
                              row_lo=lo, out_dtype=np.float32)
    fold = lambda recv: torch.from_numpy(O.combine_partials(recv.numpy()))
    mine = fd2.exchange_partials(torch.from_numpy(partial), world, per, method=method, fold=fold)
    np.save(os.path.join(tmp, f"{method}_{rank}.npy"), mine.numpy())
    dist.destroy_process_group()


def test_small_tables_are_replicated_and_the_rest_placed_evenly():
    rows = workloads.config4_rows()
    nbytes = [int(r) * 128 * 4 for r in rows]
    owner = fd.place_tables(nbytes, 8, replicate_below_bytes=256 << 20)
    rep = [t for t, r in enumerate(owner) if r == fd.REPLICATED]
    assert len(rep) == 18 and all(nbytes[t] < (256 << 20) for t in rep)
    placed = [r for r in owner if r != fd.REPLICATED]
    assert sorted(placed) == list(range(8))                  # the eight large tables: one per rank
    assert sum(nbytes[t] for t in rep) < 1.2e9               # 1.15 GB on every rank
    assert fd.REPLICATED not in fd.place_tables(nbytes, 1, replicate_below_bytes=256 << 20)   # one rank: nothing to replicate


def test_a_rank_s_own_bags_of_a_replicated_table():
    """TableWiseBags._own_bags: the slice of a whole-batch input that a rank pools itself."""
    import types

    import torch
    own = fd.TableWiseBags._own_bags
    idx = torch.arange(40, dtype=torch.int32)
    w = torch.arange(40, dtype=torch.float32)
    # fixed length 4, 10 bags on 3 ranks (4 + 4 + 2)
    for rank, (lo, n) in enumerate([(0, 4), (4, 4), (8, 2)]):
        me = types.SimpleNamespace(rank=rank, per=4, fixed_len=4)
        i, o, ww, incl = own(me, idx.view(10, 4), None, w)
        assert o is None and not incl
        assert i.tolist() == list(range(lo * 4, (lo + n) * 4)) and ww.tolist() == i.float().tolist()
    assert own(types.SimpleNamespace(rank=3, per=4, fixed_len=4), idx.view(10, 4), None, w) is None
    # ragged: offsets stay absolute, the next rank's first start closes the last bag
    off = torch.tensor([0, 3, 3, 10, 12, 20, 31, 31, 35, 36], dtype=torch.int32)
    me = types.SimpleNamespace(rank=1, per=4, fixed_len=0)
    i, o, ww, incl = own(me, idx, off, None)
    assert i is idx and ww is None and incl and o.tolist() == [12, 20, 31, 31, 35]
    me = types.SimpleNamespace(rank=2, per=4, fixed_len=0)
    i, o, ww, incl = own(me, idx, off, None)
    assert not incl and o.tolist() == [35, 36]               # the batch's last bags end at num_indices


@pytest.mark.parametrize("method", ["a2a", "nccl"])
def test_two_gloo_ranks_exchange_and_fold(method, tmp_path):
    import torch.multiprocessing as mp

    from forward_b200 import workloads
    from oracle import eb_oracle as O
    world = 2
    port = 29600 + (os.getpid() % 200) + (0 if method == "a2a" else 1)
    mp.spawn(_worker, args=(world, port, method, str(tmp_path)), nprocs=world, join=True)
    rng = np.random.default_rng(5)
    table = rng.standard_normal((999, 24)).astype(np.float16)
    bags = workloads.ragged_bags(999, rng.integers(0, 30, 50), rng)
    parts = np.stack([O.pool(table[lo:lo + n], bags.indices, bags.offsets, mode=O.MODE_MEAN, row_lo=lo,
                             out_dtype=np.float32)
                      for lo, n in (fd.shard_rows(999, world, r) for r in range(world))])
    expect = O.combine_partials(parts)                    # fold in rank order
    got = np.concatenate([np.load(tmp_path / f"{method}_{r}.npy") for r in range(world)])[:50]
    if method == "a2a":
        assert np.array_equal(got, expect)                # fixed order: bit-identical
    else:
        np.testing.assert_allclose(got, expect, rtol=1e-6, atol=1e-7)
    whole = O.pool(table, bags.indices, bags.offsets, mode=O.MODE_MEAN, out_dtype=np.float32)
    np.testing.assert_allclose(got, whole, rtol=1e-5, atol=1e-6)


def _validation_worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    from forward_b200 import capi
    from forward_b200 import dist as fd2
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    table = torch.zeros((10, 8), dtype=torch.float16)
    seen = []
    for kw in (dict(mode=capi.MODE_MAX, exchange="push"),            # max travels staged only
               dict(mode=capi.MODE_MAX, exchange="nccl"),
               dict(mode=capi.MODE_SUM, exchange="stage", wire_dtype=capi.F32_POS),
               dict(mode=capi.MODE_SQUARE_SUM, exchange="push")):
        try:
            fd2.RowShardedBag(table, 0, max_bags=16, **kw)
            seen.append("accepted")
        except ValueError as e:
            seen.append(str(e))
    with open(os.path.join(tmp, f"validation_{rank}.txt"), "w") as f:
        f.write("\n".join(seen))
    dist.destroy_process_group()


def test_sharded_bag_refuses_combinations_it_cannot_honour(tmp_path):
    """Argument checks of RowShardedBag run before anything touches a GPU (two gloo ranks)."""
    import torch.multiprocessing as mp
    world = 2
    port = 29850 + (os.getpid() % 100)
    mp.spawn(_validation_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        lines = (tmp_path / f"validation_{r}.txt").read_text().splitlines()
        assert len(lines) == 4 and "accepted" not in lines
        assert "exchange='stage'" in lines[0] and "exchange='stage'" in lines[1]
        assert "belongs to max" in lines[2] and "sum, mean and max" in lines[3]


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("num_bags", [1022, 1024, 5, 1])
def test_own_bags_of_all_ranks_cover_a_batch_exactly_once(world, num_bags):
    """Replicated tables: the ranks' own-bag slices, fixed-length and ragged, put together give the
    whole batch, each bag once and with its own indices."""
    import types

    import torch
    own = fd.TableWiseBags._own_bags
    per = fd.bags_per_rank(num_bags, world)
    L = 3
    idx = torch.arange(num_bags * L, dtype=torch.int32)
    seen = []
    for rank in range(world):
        got = own(types.SimpleNamespace(rank=rank, per=per, fixed_len=L), idx.view(num_bags, L), None, None)
        if got is not None:
            seen += got[0].tolist()
    assert seen == idx.tolist()
    rng = np.random.default_rng(num_bags * 10 + world)
    lengths = rng.integers(0, 5, num_bags)
    off = torch.from_numpy(np.concatenate([[0], np.cumsum(lengths)[:-1]]).astype(np.int32))
    total = int(lengths.sum())
    ridx = torch.arange(total, dtype=torch.int32)
    bags = []
    for rank in range(world):
        got = own(types.SimpleNamespace(rank=rank, per=per, fixed_len=0), ridx, off, None)
        if got is None:
            continue
        i, o, _, incl = got
        starts = o.tolist()
        n = len(starts) - (1 if incl else 0)
        ends = starts[1:] + ([] if incl else [total])
        bags += [(starts[b], ends[b]) for b in range(n)]
    expect = list(zip(off.tolist(), off.tolist()[1:] + [total]))
    assert bags == expect
