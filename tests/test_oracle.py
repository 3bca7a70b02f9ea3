"""The CPU oracle against the reference's fixture, committed torch outputs and live torch CPU."""
import os

import numpy as np
import pytest

from oracle import eb_oracle as O


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


def test_reference_fixture_unit_test_inputs(golden_dir):
    """data/torch_unit_tests/nodes/embedding_bag.pth with the inputs of
    source/unit_test/test_torch_nodes.h:178-185: four empty bags, then all five rows.
    The reference test allows an absolute error of 1e-3 (test_torch_nodes.h:40)."""
    g = np.load(os.path.join(golden_dir, "embedding_bag_pth.npz"))
    for case in ("unit_test", "trace"):
        got = O.pool(g["weight"], g[f"{case}_indices"], g[f"{case}_offsets"], mode=O.MODE_SUM)
        exp = g[f"{case}_expected"]
        assert got.shape == exp.shape
        assert np.max(np.abs(got - exp)) <= 1e-3
        assert np.array_equal(_bits(got), _bits(exp))  # in fact bit-identical
    unit = O.pool(g["weight"], g["unit_test_indices"], g["unit_test_offsets"])
    assert not unit[:4].any()


def test_committed_torch_cases(golden_dir):
    g = np.load(os.path.join(golden_dir, "torch_cpu_cases.npz"))
    modes = {"sum": O.MODE_SUM, "mean": O.MODE_MEAN, "max": O.MODE_MAX}
    assert len(g["names"]) >= 60
    for name in g["names"]:
        key, dtype, dim, mode, variant, pad, ilo = str(name).split("|")
        table = g[f"{key}_table"]
        psw = g[f"{key}_psw"].astype(np.float32) if variant == "weights" else None
        got = O.pool(table, g[f"{key}_indices"], g[f"{key}_offsets"], mode=modes[mode],
                     padding_idx=int(pad), include_last_offset=bool(int(ilo)),
                     per_sample_weights=psw)
        exp = g[f"{key}_expected"]
        assert got.dtype == exp.dtype and got.shape == exp.shape, name
        if variant == "weights" and dtype == "float16":
            # torch multiplies in half precision here; the plugin takes fp32 weights
            np.testing.assert_allclose(got.astype(np.float32), exp.astype(np.float32),
                                       rtol=1e-3, atol=2e-3, err_msg=str(name))
        else:
            assert np.array_equal(_bits(got), _bits(exp)), name


@pytest.mark.parametrize("dtype", [np.float32, np.float16])
@pytest.mark.parametrize("mode", [O.MODE_SUM, O.MODE_MEAN, O.MODE_MAX])
def test_live_torch_cpu(dtype, mode):
    rng = np.random.default_rng(7)
    table = rng.standard_normal((500, 96)).astype(dtype)
    lengths = rng.integers(0, 70, 50)
    offsets = np.concatenate([[0], np.cumsum(lengths)])[:-1].astype(np.int64)
    indices = rng.integers(0, 500, int(lengths.sum())).astype(np.int64)
    indices[rng.random(indices.size) < 0.1] = 11
    got = O.pool(table, indices, offsets, mode=mode, padding_idx=11)
    exp = O.torch_pool(table, indices, offsets, mode=mode, padding_idx=11).numpy()
    assert np.array_equal(_bits(got), _bits(exp))


def test_half_conversion_matches_numpy():
    lib = O.lib()
    for h in list(range(0, 0x10000, 7)) + [0x0001, 0x03FF, 0x0400, 0x7BFF, 0x7C00, 0xFC00, 0x8000]:
        f = lib.oracle_half_to_float(h)
        ref = np.array([h], dtype=np.uint16).view(np.float16).astype(np.float32)[0]
        if np.isnan(ref):
            assert np.isnan(f)
        else:
            assert np.float32(f).tobytes() == ref.tobytes(), hex(h)
    rng = np.random.default_rng(3)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s
                           for s in (1e-8, 1e-5, 1e-3, 1.0, 100.0, 7e4)])
    vals = np.concatenate([vals, np.float32([0.0, -0.0, 65504, 65520, 65519.99, 2**-24, 2**-25,
                                             1.5 * 2**-25, np.inf, -np.inf])])
    for v in vals:
        assert lib.oracle_float_to_half(float(v)) == int(np.float16(v).view(np.uint16)), v


def test_kernel_semantics_differ_from_enum_where_the_reference_is_inconsistent():
    """The reference .cu treats op 1 as max-from-zero divided by the length and op 2 as a
    sum (embedding_bag_plugin.cu:50-64,111) while its enum says 1 = MEAN, 2 = MAX
    (embedding_bag_plugin.h:39).  Sum and square-sum agree between the two readings."""
    rng = np.random.default_rng(0)
    table = rng.standard_normal((30, 8)).astype(np.float32)
    idx = rng.integers(0, 30, 20).astype(np.int32)
    off = np.array([0, 5, 5, 12], dtype=np.int32)
    for mode in (O.MODE_SUM, O.MODE_SQUARE_SUM):
        a = O.pool(table, idx, off, mode=mode, semantics=O.SEM_ENUM)
        b = O.pool(table, idx, off, mode=mode, semantics=O.SEM_KERNEL)
        assert np.array_equal(a, b)
    lit_mean = O.pool(table, idx, off, mode=1, semantics=O.SEM_KERNEL)
    lens = np.array([5, 0, 7, 8])
    manual = np.stack([np.maximum(table[idx[s:s + n]].max(0), 0) / max(n, 1) if n else np.zeros(8)
                       for s, n in zip(off, lens)]).astype(np.float32)
    np.testing.assert_allclose(lit_mean, manual, rtol=1e-6)
    assert not np.allclose(lit_mean, O.pool(table, idx, off, mode=O.MODE_MEAN))
    lit_max = O.pool(table, idx, off, mode=2, semantics=O.SEM_KERNEL)
    assert np.array_equal(lit_max, O.pool(table, idx, off, mode=O.MODE_SUM))


def test_fixed_length_and_window_and_gather():
    rng = np.random.default_rng(5)
    table = rng.standard_normal((64, 12)).astype(np.float32)
    idx = rng.integers(0, 64, (10, 5)).astype(np.int32)
    fixed = O.pool(table, idx, mode=O.MODE_SUM, fixed_len=5)
    np.testing.assert_allclose(fixed, table[idx].sum(1), rtol=1e-6, atol=1e-6)
    # window [16, 48): rows outside are skipped, mean still counts them (reference .cu:94,112)
    shard = table[16:48]
    part = O.pool(shard, idx, mode=O.MODE_MEAN, fixed_len=5, row_lo=16)
    inside = (idx >= 16) & (idx < 48)
    manual = np.where(inside[..., None], table[idx], 0).sum(1) / 5
    np.testing.assert_allclose(part, manual, rtol=1e-6, atol=1e-6)
    gathered = O.pool(shard, idx, mode=O.MODE_GATHER, row_lo=16)
    exp = np.where(inside.reshape(-1, 1), table[idx.reshape(-1)], 0)
    assert np.array_equal(gathered, exp)
    kept = np.full((50, 12), 7.0, dtype=np.float32)
    O.pool(shard, idx, mode=O.MODE_GATHER, row_lo=16, flags=O.FLAG_GATHER_KEEP_SKIPPED, out=kept)
    assert np.all(kept[~inside.reshape(-1)] == 7.0)


def test_table_generator_is_seeded_and_roughly_normal():
    rows = np.arange(0, 4000, dtype=np.int64) * 250_007
    t = O.table_rows(rows, 64, seed=4, scale=0.05, dtype=np.float32)
    assert np.array_equal(t, O.table_rows(rows, 64, seed=4, scale=0.05, dtype=np.float32))
    assert not np.array_equal(t, O.table_rows(rows, 64, seed=5, scale=0.05, dtype=np.float32))
    assert abs(t.mean()) < 1e-3 and abs(t.std() - 0.05) < 1e-3


def test_sharded_max_rule_equals_torch_on_the_whole_table():
    """Per-shard {value, position} partials folded by "greater value, earlier position among equals,
    NaN only as the bag's first entry" reproduce torch CPU's max on the unsharded table bit for bit:
    ties, signed zeros, NaN rows, padding, empty bags; 1 to 5 shards."""
    import torch
    import torch.nn.functional as F
    rng = np.random.default_rng(32)
    rows, dim, nb = 200, 8, 150
    for dtype in (np.float32, np.float16):
        table = rng.integers(-2, 3, (rows, dim)).astype(dtype)
        table[rng.random((rows, dim)) < 0.15] = -0.0
        table[::17] = np.nan
        lengths = rng.integers(0, 25, nb)
        offsets = np.zeros(nb, dtype=np.int32)
        offsets[1:] = np.cumsum(lengths[:-1])
        indices = rng.integers(0, rows, int(lengths.sum())).astype(np.int32)
        indices[::9] = 3
        expect = F.embedding_bag(torch.from_numpy(indices.astype(np.int64)), torch.from_numpy(table),
                                 torch.from_numpy(offsets.astype(np.int64)), mode="max",
                                 padding_idx=3).numpy().astype(np.float32)
        assert np.isnan(expect).any() and (np.signbit(expect) & (expect == 0)).any()
        for shards in (1, 2, 5):
            cuts = np.linspace(0, rows, shards + 1).astype(int)
            parts = [O.max_with_positions(table[a:b], indices, offsets, row_lo=int(a), padding_idx=3)
                     for a, b in zip(cuts[:-1], cuts[1:])]
            got = O.fold_max_partials(np.stack([v for v, _ in parts]), np.stack([p for _, p in parts]))
            same = got.view(np.uint32) == expect.view(np.uint32)
            assert (same | (np.isnan(got) & np.isnan(expect))).all(), (dtype, shards)
