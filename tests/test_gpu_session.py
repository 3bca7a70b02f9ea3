"""The host-buffer session on a GPU: blocking calls and the in-flight pipeline vs the oracle."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")

from forward_b200 import capi, workloads  # noqa: E402
from forward_b200.session import Session  # noqa: E402
from oracle import eb_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def _bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


@pytest.mark.parametrize("mode", [capi.MODE_SUM, capi.MODE_MEAN, capi.MODE_MAX])
def test_blocking_run_matches_oracle(mode):
    rng = np.random.default_rng(21)
    table = rng.standard_normal((5000, 128)).astype(np.float16)
    with Session(table_dtype=capi.F16, dim=128, num_rows=5000, mode=mode, max_indices=100_000,
                 max_bags=2048, padding_idx=5, depth=2) as s:
        s.load_table(table)
        for trial in range(3):
            bags = workloads.ragged_bags(5000, rng.integers(0, 60, 1500 + trial), rng)
            bags.indices[::11] = 5
            got = s.run(bags.indices, bags.offsets)
            exp = O.pool(table, bags.indices, bags.offsets, mode=mode, padding_idx=5)
            assert np.array_equal(_bits(got), _bits(exp))


def test_pipeline_slots_weighted_fixed_length_fp32():
    rng = np.random.default_rng(22)
    table = rng.standard_normal((3000, 64)).astype(np.float32)
    depth, L, B = 4, 20, 512
    with Session(table_dtype=capi.F32, dim=64, num_rows=3000, mode=capi.MODE_SUM,
                 max_indices=B * L, max_bags=B, fixed_len=L, weighted=True, depth=depth) as s:
        s.load_table(table[:1000], 0)
        s.load_table(table[1000:], 1000)
        inputs = []
        for k in range(depth):
            idx = rng.integers(0, 3000, B * L).astype(np.int32)
            w = rng.random(B * L).astype(np.float32)
            vi, vo, vw, vout = s.slot(k)
            assert vo is None
            vi[:] = idx
            vw[:] = w
            inputs.append((idx, w))
            s.submit(k, B * L, B)
        with pytest.raises(capi.FwdEbError):
            s.submit(0, B * L, B)            # slot still in flight
        for k in range(depth):
            s.wait(k)
            exp = O.pool(table, inputs[k][0], mode=O.MODE_SUM, fixed_len=L,
                         per_sample_weights=inputs[k][1])
            assert np.array_equal(_bits(s.slot(k)[3].copy()), _bits(exp))
        h2d, d2h = s.copy_bytes(B * L, B)
        assert h2d == B * L * 8 and d2h == B * 64 * 4
        with pytest.raises(capi.FwdEbError):
            s.submit(0, B * L + 1, B)        # beyond capacity
