"""Row shards and table-wise placement across real GPUs (one process per GPU, NCCL for the
rendezvous and the plain variants, peer stores for the fused ones).  Skipped on a single GPU."""
import os
import sys

import numpy as np
import pytest

torch = pytest.importorskip("torch")

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, tmp):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    from forward_b200 import capi, workloads
    from forward_b200 import dist as fd
    from oracle import eb_oracle as O
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    failures = []
    rng = np.random.default_rng(13)
    rows, dim, nb = 40_000, 128, 4096
    table = rng.standard_normal((rows, dim)).astype(np.float16)
    lo, n = fd.shard_rows(rows, world, rank)
    local = torch.from_numpy(table[lo:lo + n]).to(dev)
    shards = [fd.shard_rows(rows, world, r) for r in range(world)]
    for exchange, wire in (("compact", capi.F32), ("compact", capi.F16), ("compact+lanes", capi.F32),
                           ("compact+lanes", capi.F16), ("push+lanes", capi.F32), ("stage+lanes", capi.F16),
                           ("compact+tickets", capi.F32),
                           ("compact+ship", capi.F32), ("compact+ship", capi.F16), ("push+ship", capi.F32),
                           ("push", capi.F32), ("push", capi.F16), ("push+tickets", capi.F16),
                           ("stage", capi.F32),
                           ("stage", capi.F16), ("a2a", capi.F32), ("nccl", capi.F32)):
        tickets = exchange.endswith("+tickets")      # the pooling grid raises the flag itself
        ship = exchange.endswith("+ship")            # rows staged locally, sent by the copy kernel
        lanes = 2 if exchange.endswith("+lanes") else 1   # consecutive steps on two alternating streams
        exchange = exchange.split("+")[0]
        for mode in (capi.MODE_SUM, capi.MODE_MEAN):
            bag = fd.RowShardedBag(local, lo, mode=mode, max_bags=nb, exchange=exchange,
                                   wire_dtype=wire, padding_idx=3, max_indices=80 * nb,
                                   flag_from_pool=tickets, ship=ship, lanes=lanes)
            for step in range(20 if (exchange in ("compact", "push") or lanes > 1) else 3):   # beyond the buffer parts
                brng = np.random.default_rng(100 + step)
                bags = workloads.ragged_bags(rows, brng.integers(0, 80, nb), brng)
                bags.indices[::11] = 3
                got = bag.forward(torch.from_numpy(bags.indices).to(dev),
                                  torch.from_numpy(bags.offsets).to(dev))
                if step % 5 != 4:
                    continue      # several steps queued back to back, then one is checked
                bag.sync_result()
                torch.cuda.synchronize()
                parts = np.stack([O.pool(table[a:a + c], bags.indices, bags.offsets, mode=mode,
                                         padding_idx=3, row_lo=a, out_dtype=np.float32)
                                  for a, c in shards])
                if exchange == "compact" and mode == capi.MODE_MEAN:
                    # partials are sums; the owner divides by the bag's full count after the fold
                    parts = np.stack([O.pool(table[a:a + c], bags.indices, bags.offsets, mode=O.MODE_SUM,
                                             padding_idx=3, row_lo=a, out_dtype=np.float32)
                                      for a, c in shards])
                if wire == capi.F16:
                    parts = parts.astype(np.float16)
                expect = O.combine_partials(parts, np.float32)
                if exchange == "compact" and mode == capi.MODE_MEAN:
                    ends = np.append(bags.offsets, bags.num_indices)
                    full = np.array([np.count_nonzero(bags.indices[ends[b]:ends[b + 1]] != 3)
                                     for b in range(nb)])
                    expect = (expect / np.maximum(full, 1)[:, None].astype(np.float32)).astype(np.float32)
                blo, mine = fd.owned_bags(nb, world, rank)
                g = got.cpu().numpy()
                if exchange == "nccl":
                    ok = np.allclose(g, expect[blo:blo + mine], rtol=1e-5, atol=1e-5)
                else:
                    ok = np.array_equal(g, expect[blo:blo + mine])
                if not ok or bag.check_status() != 0:
                    failures.append(f"rowshard {exchange} wire{wire} mode{mode} step{step}")
            dist.barrier()
            bag.close()
    # sharded max (staged exchange, {value, position} partials): the whole-table max, bit for bit
    bag = fd.RowShardedBag(local, lo, mode=capi.MODE_MAX, max_bags=nb, exchange="stage", padding_idx=3,
                           out_dtype=torch.float16)
    for step in range(2):
        brng = np.random.default_rng(200 + step)
        bags = workloads.ragged_bags(rows, brng.integers(0, 40, nb), brng)
        bags.indices[::11] = 3
        got = bag.forward(torch.from_numpy(bags.indices).to(dev), torch.from_numpy(bags.offsets).to(dev))
        bag.sync_result()
        torch.cuda.synchronize()
        expect = O.pool(table, bags.indices, bags.offsets, mode=O.MODE_MAX, padding_idx=3)
        blo, mine = fd.owned_bags(nb, world, rank)
        if not np.array_equal(got.cpu().numpy().view(np.uint16), expect[blo:blo + mine].view(np.uint16)) \
                or bag.check_status() != 0:
            failures.append(f"rowshard max step{step}")
    dist.barrier()
    bag.close()
    # table-wise: 5 tables over the ranks, fixed pooling factor, weights
    ntab, L, dim2, nb2 = 5, 8, 64, 1024
    owner = fd.place_tables([1] * ntab, world)
    trng = np.random.default_rng(17)
    tables = [trng.standard_normal((3000 + 100 * t, dim2)).astype(np.float32) for t in range(ntab)]
    for exchange in ("push", "push+lanes", "push+tickets", "push+ship", "nccl"):
        mine_t = [t for t in range(ntab) if owner[t] == rank]
        tw = fd.TableWiseBags({t: torch.from_numpy(tables[t]).to(dev) for t in mine_t}, owner,
                              dim=dim2, max_bags=nb2, exchange=exchange.split("+")[0], fixed_len=L,
                              flag_from_pool=exchange.endswith("+tickets"), ship=exchange.endswith("+ship"),
                              lanes=2 if exchange.endswith("+lanes") else 1)
        for step in range(20 if exchange != "nccl" else 2):
            irng = np.random.default_rng(200 + step)
            idx = [irng.integers(0, tables[t].shape[0], (nb2, L)).astype(np.int32) for t in range(ntab)]
            w = [irng.random(nb2 * L).astype(np.float32) for _ in range(ntab)]
            inputs = {t: (torch.from_numpy(idx[t]).to(dev), None, torch.from_numpy(w[t]).to(dev))
                      for t in mine_t}
            res = tw.forward(inputs)
            if step % 3 != 2 and exchange != "nccl":
                continue          # steps queued back to back (on alternating streams with lanes), then one is checked
            tw.sync_result()
            torch.cuda.synchronize()
            expect = np.stack([O.pool(tables[t], idx[t], fixed_len=L, per_sample_weights=w[t])
                               for t in range(ntab)], axis=1)
            per = fd.bags_per_rank(nb2, world)
            if not np.array_equal(res.cpu().numpy(), expect[rank * per:(rank + 1) * per]) or \
                    tw.check_status() != 0:
                failures.append(f"tablewise {exchange} step{step}")
        dist.barrier()
        tw.close()
    # table-wise with replicated tables: the two large tables live on one rank each, the three
    # small ones on every rank (pooled there for the rank's own bags); fixed-length weighted bags
    # and ragged bags, 1022 bags (the last rank owns fewer)
    sizes = [600, 9000, 500, 12000, 700]
    nb3 = 1022
    owner = fd.place_tables([n * dim2 * 4 for n in sizes], world, replicate_below_bytes=1000 * dim2 * 4)
    tables = [trng.standard_normal((n, dim2)).astype(np.float32) for n in sizes]
    here = [t for t in range(ntab) if owner[t] in (rank, fd.REPLICATED)]
    d_tables = {t: torch.from_numpy(tables[t]).to(dev) for t in here}
    per = fd.bags_per_rank(nb3, world)
    blo, mine_b = fd.owned_bags(nb3, world, rank)
    for exchange in ("push", "push+lanes", "nccl"):
        for fixed in (L, 0):
            tw = fd.TableWiseBags(d_tables, owner, dim=dim2, max_bags=nb3, exchange=exchange.split("+")[0],
                                  fixed_len=fixed, mode=capi.MODE_SUM if fixed else capi.MODE_MEAN,
                                  lanes=2 if exchange.endswith("+lanes") else 1)
            for step in range(20 if exchange != "nccl" else 2):
                irng = np.random.default_rng(300 + step)
                if fixed:
                    idx = [irng.integers(0, sizes[t], (nb3, L)).astype(np.int32) for t in range(ntab)]
                    w = [irng.random(nb3 * L).astype(np.float32) for _ in range(ntab)]
                    inputs = {t: (torch.from_numpy(idx[t]).to(dev), None, torch.from_numpy(w[t]).to(dev))
                              for t in here}
                else:
                    bgs = [workloads.ragged_bags(sizes[t], irng.integers(0, 20, nb3), irng) for t in range(ntab)]
                    inputs = {t: (torch.from_numpy(bgs[t].indices).to(dev), torch.from_numpy(bgs[t].offsets).to(dev),
                                  None) for t in here}
                res = tw.forward(inputs)
                if step % 5 != 4 and exchange != "nccl":
                    continue
                tw.sync_result()
                torch.cuda.synchronize()
                if fixed:
                    expect = np.stack([O.pool(tables[t], idx[t], fixed_len=L, per_sample_weights=w[t])
                                       for t in range(ntab)], axis=1)
                else:
                    expect = np.stack([O.pool(tables[t], bgs[t].indices, bgs[t].offsets, mode=O.MODE_MEAN)
                                       for t in range(ntab)], axis=1)
                if not np.array_equal(res.cpu().numpy()[:mine_b], expect[blo:blo + mine_b]) or \
                        tw.check_status() != 0:
                    failures.append(f"tablewise replicated {exchange} fixed{fixed} step{step}")
            dist.barrier()
            tw.close()
    with open(os.path.join(tmp, f"rank{rank}.txt"), "w") as f:
        f.write("\n".join(failures))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
def test_row_shards_and_table_wise_across_gpus(tmp_path):
    import torch.multiprocessing as mp
    world = min(4, torch.cuda.device_count())
    port = 29800 + os.getpid() % 100
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        text = (tmp_path / f"rank{r}.txt").read_text()
        assert text == "", f"rank {r}: {text}"
