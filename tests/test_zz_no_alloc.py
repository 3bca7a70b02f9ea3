"""fwd_eb_forward_static_scratch: the split-bag path with its scratch inside the library.

Written for hosts that cannot allocate (a plugin that was promised no workspace, a serving
loop with a frozen memory pool).  The entry point must give exactly what fwd_eb_forward gives
with the split strategy and a caller-allocated workspace — the kernels are the same, only the
scratch differs — on two calls in a row, the second of which finds the first call's leftovers
in the shared array.  This file sorts last on purpose: a run that stops at the first failure
has already exercised everything else.
"""
import ctypes as C

import numpy as np
import pytest

from forward_b200 import capi

SCRATCH_BYTES = 8 << 20


def _bind():
    fn = capi.lib().fwd_eb_forward_static_scratch
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(capi.Params), C.c_void_p]
    return fn


def test_oversized_call_is_refused_before_any_cuda_call():
    """Pure host check, so it runs without a GPU: 8 bags x 64 splits x 4096 columns of fp32
    partials is a little over 8 MiB, more than the built-in array holds."""
    p = capi.Params()
    p.table, p.indices, p.offsets, p.out = 0x1000, 0x2000, 0x3000, 0x4000
    p.table_dtype, p.out_dtype, p.dim = capi.F32, capi.F32, 4096
    p.num_rows, p.num_bags, p.num_indices = 1000, 8, 8 * 100_000
    p.mode, p.padding_idx = capi.MODE_SUM, -1
    before = capi.lib().fwd_eb_launch_count()
    rc = _bind()(C.byref(p), None)
    assert rc == capi.ETOOBIG
    assert b"built-in array" in capi.lib().fwd_eb_last_error_string()
    assert capi.lib().fwd_eb_launch_count() == before
    q = capi.Params.from_buffer_copy(p)
    q.strategy = capi.STRATEGY_SPLIT
    assert capi.lib().fwd_eb_workspace_size(C.byref(q)) > SCRATCH_BYTES


@pytest.mark.gpu
@pytest.mark.parametrize("mode", [capi.MODE_SUM, capi.MODE_MEAN, capi.MODE_MAX])
def test_two_calls_in_a_row_match_the_allocating_entry_point(mode):
    torch = pytest.importorskip("torch")
    dev = "cuda:0"
    fn = _bind()
    rng = np.random.default_rng(31 + mode)
    table = torch.from_numpy(rng.standard_normal((20000, 128)).astype(np.float16)).to(dev)
    stream = C.c_void_p(capi.current_stream_ptr())
    # second call is smaller: it sees the first call's partials in the slots it does not rewrite
    for lengths in ([40000, 3, 0, 25000, 9000, 65000, 1], [5000, 0, 12000]):
        lengths = np.array(lengths)
        offsets = np.zeros(len(lengths), dtype=np.int32)
        offsets[1:] = np.cumsum(lengths[:-1])
        indices = rng.integers(0, 20000, int(lengths.sum())).astype(np.int32)
        indices[::17] = 4
        i = torch.from_numpy(indices).to(dev)
        o = torch.from_numpy(offsets).to(dev)
        got = torch.full((len(lengths), 128), float("nan"), dtype=torch.float16, device=dev)
        ref = torch.full_like(got, float("nan"))
        p = capi.make_params(table, i, o, out=got, mode=mode, padding_idx=4)
        capi.check(fn(C.byref(p), stream))
        q = capi.make_params(table, i, o, out=ref, mode=mode, padding_idx=4,
                             strategy=capi.STRATEGY_SPLIT)
        need = capi.lib().fwd_eb_workspace_size(C.byref(q))
        assert 0 < need <= SCRATCH_BYTES
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        q.workspace, q.workspace_bytes = ws.data_ptr(), need
        capi.forward(q)
        torch.cuda.synchronize()
        assert not torch.isnan(got).any()
        assert torch.equal(got, ref)   # same kernels, same order of folding: identical bits
