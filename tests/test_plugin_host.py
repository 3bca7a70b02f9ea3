"""The EmbeddingBag_TRT plugin driven in TensorRT's call order by the stand-in host
(description -> layer creator -> network -> configure -> serialise -> load -> enqueue).

CPU tests cover what needs no device: registry lookup, creator fields, output shapes, format
rules, the engine-blob layout (byte-compatible with the reference's serialize.hpp order).  GPU
tests run enqueue against the oracle, including the reference unit test's fixture."""
import ctypes as C
import os
import struct

import numpy as np
import pytest

from forward_b200 import capi
from oracle import eb_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
KINT32, KFLOAT, KHALF = 3, 0, 1          # nvinfer1::DataType values used by the plugin
PF_F16, PF_F32, PF_I32 = 0, 1, 5         # nvinfer1::PluginFieldType values


@pytest.fixture(scope="module")
def host():
    capi.lib()
    h = C.CDLL(os.path.join(ROOT, "forward_b200", "lib", "libfwd_eb_plugin.so"))
    h.fwd_eb_host_build.restype = C.c_void_p
    h.fwd_eb_host_build.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                    C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                    C.c_void_p, C.c_int, C.c_void_p]
    h.fwd_eb_host_free.argtypes = [C.c_void_p]
    h.fwd_eb_host_blob.restype = C.c_size_t
    h.fwd_eb_host_blob.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    h.fwd_eb_host_load.restype = C.c_void_p
    h.fwd_eb_host_load.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p]
    h.fwd_eb_host_clone_context.restype = C.c_void_p
    h.fwd_eb_host_clone_context.argtypes = [C.c_void_p]
    h.fwd_eb_host_output_dims.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    h.fwd_eb_host_layer_name.restype = C.c_char_p
    h.fwd_eb_host_layer_name.argtypes = [C.c_void_p]
    h.fwd_eb_host_table_uploads.argtypes = [C.c_void_p]
    h.fwd_eb_host_shares_table.argtypes = [C.c_void_p, C.c_void_p]
    h.fwd_eb_host_format_ok.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int]
    h.fwd_eb_host_workspace.restype = C.c_size_t
    h.fwd_eb_host_workspace.argtypes = [C.c_void_p]
    h.fwd_eb_host_run.argtypes = [C.c_void_p] * 6
    h.fwd_eb_host_last_log.restype = C.c_char_p
    h.fwd_eb_host_creator_accepts.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    h.fwd_eb_host_creator_field_names.argtypes = [C.c_char_p, C.c_size_t]
    h.fwd_eb_host_build_external.restype = C.c_void_p
    h.fwd_eb_host_build_external.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                             C.c_longlong, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                             C.c_void_p, C.c_int, C.c_void_p]
    h.fwd_eb_plugin_register_weights.argtypes = [C.c_char_p, C.c_void_p, C.c_int, C.c_longlong, C.c_int, C.c_int]
    h.fwd_eb_plugin_unregister_weights.argtypes = [C.c_char_p]
    return h


def _dims(*d):
    return (C.c_int * max(len(d), 1))(*d), len(d)


def build(host, table, op, idx_dims, off_dims=(), w_dims=(), offset=0, padding=-1, last=0, half_out=0):
    table = np.ascontiguousarray(table)
    i, ir = _dims(*idx_dims)
    o, orank = _dims(*off_dims)
    w, wr = _dims(*w_dims)
    h = host.fwd_eb_host_build(table.ctypes.data, int(table.dtype == np.float16), table.shape[0],
                               table.shape[1], offset, op, padding, last, half_out, ir, i, orank, o,
                               wr, w)
    return h


def out_dims(host, h):
    d = (C.c_int * 8)()
    t = C.c_int()
    n = host.fwd_eb_host_output_dims(h, d, C.byref(t))
    return tuple(d[:n]), t.value


def blob_of(host, h):
    n = host.fwd_eb_host_blob(h, None, 0)
    buf = (C.c_char * n)()
    host.fwd_eb_host_blob(h, buf, n)
    return bytes(buf)


# ---- CPU ------------------------------------------------------------------------------------

def test_registry_creator_fields(host):
    buf = C.create_string_buffer(256)
    n = host.fwd_eb_host_creator_field_names(buf, 256)
    names = buf.value.decode().split(",")
    assert names[:5] == ["dim", "count", "offset", "op", "data"] and n == len(names)  # reference's five first

    table = np.arange(12, dtype=np.float32)
    ints = [np.array([v], dtype=np.int32) for v in (3, 4, 0, 0)]

    def accepts(extra=(), drop=None, data_type=PF_F32, op=0):
        ints[3][0] = op
        fields = [("dim", PF_I32, ints[0]), ("count", PF_I32, ints[1]), ("offset", PF_I32, ints[2]),
                  ("op", PF_I32, ints[3]), ("data", data_type, table)] + list(extra)
        fields = [f for f in fields if f[0] != drop]
        k = len(fields)
        names_c = (C.c_char_p * k)(*[f[0].encode() for f in fields])
        types_c = (C.c_int * k)(*[f[1] for f in fields])
        data_c = (C.c_void_p * k)(*[f[2].ctypes.data for f in fields])
        lens_c = (C.c_int * k)(*[f[2].size for f in fields])
        return host.fwd_eb_host_creator_accepts(k, names_c, types_c, data_c, lens_c)

    assert accepts() == 1                                   # exactly the reference's call
    one = np.array([1], dtype=np.int32)
    assert accepts(extra=[("padding_idx", PF_I32, one), ("include_last_offset", PF_I32, one)]) == 1
    assert accepts(drop="count") == 0                       # a required field is missing
    assert accepts(extra=[("bogus", PF_I32, one)]) == 0     # unknown field (reference asserts)
    assert accepts(op=7) == 0
    assert accepts(extra=[("per_sample_weights", PF_I32, one)], op=2) == 0
    assert accepts(data_type=PF_I32) == 0
    assert b"EmbeddingBag_TRT" in host.fwd_eb_host_last_log()


def test_output_shapes_follow_the_reference_rules(host):
    t = np.zeros((50, 16), dtype=np.float32)
    cases = [
        (dict(op=0, idx_dims=(37,), off_dims=(9,)), (9, 16)),            # 1-D indices + offsets
        (dict(op=1, idx_dims=(37,), off_dims=(1, 9)), (9, 16)),          # [1, B] offsets (DLRM slice)
        (dict(op=0, idx_dims=(37,), off_dims=(10,), last=1), (9, 16)),   # include_last_offset
        (dict(op=2, idx_dims=(10, 5)), (10, 16)),                        # 2-D fixed-length
        (dict(op=999, idx_dims=(10, 5)), (10, 5, 16)),                   # gather appends dim
        (dict(op=0, idx_dims=(10, 5), w_dims=(10, 5)), (10, 16)),        # fixed-length + weights
        (dict(op=0, idx_dims=(37,), off_dims=(9,), w_dims=(37,)), (9, 16)),
    ]
    for kw, expect in cases:
        h = build(host, t, **kw)
        assert h, kw
        assert out_dims(host, h) == (expect, KFLOAT)
        assert host.fwd_eb_host_layer_name(h).endswith(b" [Embedding Bag]")
        assert host.fwd_eb_host_workspace(h) == 0
        host.fwd_eb_host_free(h)
    h = build(host, np.zeros((50, 1), dtype=np.float32), op=999, idx_dims=(1, 3))
    assert out_dims(host, h)[0] == (1, 3)        # dim == 1 gather keeps the input shape
    host.fwd_eb_host_free(h)
    assert not build(host, t, op=999, idx_dims=(37,), off_dims=(9,))     # gather with offsets
    assert not build(host, t, op=0, idx_dims=(37,), off_dims=(3, 3))     # offsets neither 1-D nor [1,B]
    assert not build(host, t, op=0, idx_dims=(37,))                      # single 1-D input
    h = build(host, t.astype(np.float16), op=1, idx_dims=(37,), off_dims=(9,), half_out=1)
    assert out_dims(host, h) == ((9, 16), KHALF)
    host.fwd_eb_host_free(h)


def test_format_rules(host):
    t = np.zeros((50, 16), dtype=np.float32)
    h = build(host, t, op=0, idx_dims=(37,), off_dims=(9,), w_dims=(37,))
    LINEAR, CHW4 = 0, 3
    assert host.fwd_eb_host_format_ok(h, 0, KINT32, LINEAR) == 1
    assert host.fwd_eb_host_format_ok(h, 0, KFLOAT, LINEAR) == 0
    assert host.fwd_eb_host_format_ok(h, 1, KINT32, CHW4) == 0
    assert host.fwd_eb_host_format_ok(h, 2, KFLOAT, LINEAR) == 1    # weights
    assert host.fwd_eb_host_format_ok(h, 2, KINT32, LINEAR) == 0
    assert host.fwd_eb_host_format_ok(h, 3, KFLOAT, LINEAR) == 1    # output: fp32 as the reference
    assert host.fwd_eb_host_format_ok(h, 3, KHALF, LINEAR) == 0
    host.fwd_eb_host_free(h)


def test_blob_starts_with_the_reference_layout_and_round_trips(host):
    """[int dim][int count][int data_offset][int op][size_t n][n floats] then our trailer
    (embedding_bag_plugin.cpp:196-202 / serialize.hpp:41-103 in the reference)."""
    rng = np.random.default_rng(0)
    t = rng.standard_normal((7, 12)).astype(np.float32)
    h = build(host, t, op=1, idx_dims=(20,), off_dims=(4,), offset=3, padding=2)
    blob = blob_of(host, h)
    dim, count, off, op, n = struct.unpack_from("<iiiiQ", blob, 0)
    assert (dim, count, off, op, n) == (12, 7, 3, 1, 84)
    assert blob[24:24 + 84 * 4] == t.tobytes()
    magic, flags, pad = struct.unpack_from("<IIq", blob, 24 + 84 * 4)
    assert magic == 0x32424546 and flags == 0 and pad == 2 and len(blob) == 24 + 336 + 16
    # a blob exactly as the reference writes it (no trailer) loads with reference defaults
    legacy = host.fwd_eb_host_load(blob[:24 + 336], 24 + 336, h)
    assert legacy and blob_of(host, legacy)[:360] == blob[:360]
    again = host.fwd_eb_host_load(blob, len(blob), h)
    assert again and blob_of(host, again) == blob
    assert not host.fwd_eb_host_load(blob[:100], 100, h)            # truncated
    assert b"truncated" in host.fwd_eb_host_last_log()
    # fp16 tables ride in the float vector padded to whole floats
    t16 = rng.standard_normal((3, 5)).astype(np.float16)
    h16 = build(host, t16, op=0, idx_dims=(6,), off_dims=(2,))
    b16 = blob_of(host, h16)
    assert struct.unpack_from("<Q", b16, 16)[0] == 8 and b16[24:24 + 30] == t16.tobytes()
    assert struct.unpack_from("<II", b16, 24 + 32) == (0x32424546, 1)
    for x in (h, legacy, again, h16):
        host.fwd_eb_host_free(x)


# ---- GPU ------------------------------------------------------------------------------------

def _run(host, h, torch, arrays, out_shape, out_dtype):
    dev = [None if a is None else torch.from_numpy(np.ascontiguousarray(a)).cuda() for a in arrays]
    out = torch.full(out_shape, float("nan"), dtype=out_dtype, device="cuda")
    ptrs = [C.c_void_p(d.data_ptr()) if d is not None else None for d in dev] + [None] * (3 - len(dev))
    rc = host.fwd_eb_host_run(h, ptrs[0], ptrs[1], ptrs[2], C.c_void_p(out.data_ptr()),
                              C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return rc, out.cpu().numpy()


@pytest.mark.gpu
def test_reference_unit_test_through_build_save_load_run(host, golden_dir):
    """TestTorchNodes.EmbeddingBagModule (test_torch_nodes.h:178-185): build, serialise, load a
    fresh plugin from the blob, run, compare with the TorchScript module's CPU output."""
    torch = pytest.importorskip("torch")
    g = np.load(os.path.join(golden_dir, "embedding_bag_pth.npz"))
    idx = g["unit_test_indices"].astype(np.int32)      # Forward casts int64 -> int32 on the way in
    off = g["unit_test_offsets"].astype(np.int32)
    h = build(host, g["weight"], op=0, idx_dims=idx.shape, off_dims=off.shape)
    blob = blob_of(host, h)
    loaded = host.fwd_eb_host_load(blob, len(blob), h)
    for handle in (h, loaded):
        rc, got = _run(host, handle, torch, [idx, off], (5, 4), torch.float32)
        assert rc == 0
        assert np.max(np.abs(got - g["unit_test_expected"])) <= 1e-3     # the reference's threshold
        assert np.array_equal(got, g["unit_test_expected"])
    host.fwd_eb_host_free(h)
    host.fwd_eb_host_free(loaded)


@pytest.mark.gpu
@pytest.mark.parametrize("half", [False, True])
def test_modes_options_and_shared_table(host, half):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(3)
    table = rng.standard_normal((4000, 64)).astype(np.float16 if half else np.float32)
    lengths = rng.integers(0, 40, 300)
    off = np.zeros(301, dtype=np.int32)
    off[1:] = np.cumsum(lengths)
    idx = rng.integers(0, 4000, int(off[-1])).astype(np.int32)
    idx[::9] = 7
    w = rng.random(idx.size).astype(np.float32)
    tdt = torch.float16 if half else torch.float32
    for op in (0, 1, 2, 3):
        h = build(host, table, op=op, idx_dims=idx.shape, off_dims=(301,), padding=7, last=1,
                  half_out=int(half))
        rc, got = _run(host, h, torch, [idx, off], (300, 64), tdt)
        assert rc == 0
        exp = O.pool(table, idx, off, mode=op, padding_idx=7, include_last_offset=True)
        assert np.array_equal(got.view(np.uint16 if half else np.uint32),
                              exp.view(np.uint16 if half else np.uint32))
        host.fwd_eb_host_free(h)
    # weights + second execution context: clones share one table and one upload
    h = build(host, table, op=0, idx_dims=idx.shape, off_dims=(300,), w_dims=idx.shape)
    ctx = host.fwd_eb_host_clone_context(h)
    assert host.fwd_eb_host_shares_table(h, ctx) == 1
    exp = O.pool(table, idx, off[:-1], per_sample_weights=w, out_dtype=np.float32)
    for handle in (h, ctx):
        rc, got = _run(host, handle, torch, [idx, off[:-1], w], (300, 64), torch.float32)
        assert rc == 0 and np.array_equal(got, exp)
    assert host.fwd_eb_host_table_uploads(ctx) == 1
    # 2-D fixed length, gather, and a row window (the reference's data_offset)
    idx2 = rng.integers(0, 4000, (64, 10)).astype(np.int32)
    h2 = build(host, table[1000:3000], op=1, idx_dims=idx2.shape, offset=1000)
    rc, got = _run(host, h2, torch, [idx2], (64, 64), torch.float32)
    assert rc == 0 and np.array_equal(got, O.pool(table[1000:3000], idx2, mode=1, fixed_len=10,
                                                    row_lo=1000, out_dtype=np.float32))
    hg = build(host, table, op=999, idx_dims=idx2.shape)
    rc, got = _run(host, hg, torch, [idx2], (64, 10, 64), torch.float32)
    assert rc == 0 and np.array_equal(got.reshape(-1, 64), table[idx2.reshape(-1)].astype(np.float32))
    for x in (h, ctx, h2, hg):
        host.fwd_eb_host_free(x)


@pytest.mark.gpu
def test_long_bags_use_the_built_in_scratch_because_the_plugin_gets_no_workspace(host):
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(4)
    table = rng.standard_normal((3000, 32)).astype(np.float32)
    table = np.round(table * 4) / 4
    lengths = np.array([50000, 0, 20000, 7])
    off = np.zeros(4, dtype=np.int32)
    off[1:] = np.cumsum(lengths[:-1])
    idx = rng.integers(0, 3000, int(lengths.sum())).astype(np.int32)
    h = build(host, table, op=2, idx_dims=idx.shape, off_dims=(4,))
    before = capi.lib().fwd_eb_launch_count()
    rc, got = _run(host, h, torch, [idx, off], (4, 32), torch.float32)
    assert rc == 0 and np.array_equal(got, O.pool(table, idx, off, mode=O.MODE_MAX))
    assert capi.lib().fwd_eb_launch_count() - before == 2      # split pass + fold pass
    host.fwd_eb_host_free(h)


def test_external_weights_names_must_be_registered_with_matching_geometry(host):
    """createPlugin with `external_weights`: no table bytes travel; an unknown name, or a table
    registered with another shape or element type, is refused with a logged reason."""
    i, ir = _dims(10)
    o, orank = _dims(3)
    args = (0, 100, 8, 0, 0, -1, 0, 0, ir, i, orank, o, 0, None)
    assert not host.fwd_eb_host_build_external(b"nobody", *args)
    assert b"not registered" in host.fwd_eb_host_last_log()
    fake = 0x7f0000000000      # never dereferenced on the host
    assert host.fwd_eb_plugin_register_weights(b"t", fake, 0, 100, 8, 0) == 0
    assert host.fwd_eb_plugin_register_weights(b"t", fake + 256, 0, 100, 8, 0) == 0    # same shape: pointer replaced
    assert host.fwd_eb_plugin_register_weights(b"t", fake, 0, 100, 16, 0) == -2        # another shape: refused
    h = host.fwd_eb_host_build_external(b"t", *args)
    assert h
    blob = blob_of(host, h)
    assert len(blob) < 128 and struct.unpack_from("<i", blob, 0)[0] == -2 and blob[4:8] == b"002\0"
    assert struct.unpack_from("<iqq", blob, 8) == (8, 100, 0)
    loaded = host.fwd_eb_host_load(blob, len(blob), h)
    assert loaded and host.fwd_eb_host_shares_table(h, loaded) == 0
    host.fwd_eb_host_free(loaded)
    assert not host.fwd_eb_host_build_external(b"t", 0, 101, 8, 0, 0, -1, 0, 0, ir, i, orank, o, 0, None)  # more rows than registered
    assert not host.fwd_eb_host_build_external(b"t", 1, 100, 8, 0, 0, -1, 0, 0, ir, i, orank, o, 0, None)  # fp16 asked, fp32 registered
    assert host.fwd_eb_plugin_unregister_weights(b"t") == 0
    assert not host.fwd_eb_host_load(blob, len(blob), h)          # the name is gone: the blob cannot load
    for cut in range(0, len(blob), 3):                            # truncated "002" blobs are refused, not read past
        assert not host.fwd_eb_host_load(blob[:cut], cut, h)
    host.fwd_eb_host_free(h)


@pytest.mark.gpu
def test_config3_sized_table_stays_outside_the_plan(host):
    """A 2 GB table (config 3: 4,000,000 x 256 fp16) filled on the device, registered by name:
    build -> serialise (a blob of some dozen bytes) -> deserialise -> enqueue, bit-equal to the
    C-ABI result, and no copy of the table is ever made."""
    torch = pytest.importorskip("torch")
    from forward_b200 import workloads
    rows, dim = 4_000_000, 256
    table = torch.empty((rows, dim), dtype=torch.float16, device="cuda:0")
    capi.fill_table(table, 0, seed=2, scale=0.1)
    bags = workloads.config3_bags(seed=2)
    idx, off = bags.indices, bags.offsets
    assert host.fwd_eb_plugin_register_weights(b"c3", table.data_ptr(), 0, rows, dim, 1) == 0
    i, ir = _dims(*idx.shape)
    o, orank = _dims(*off.shape)
    free0 = torch.cuda.mem_get_info()[0]
    h = host.fwd_eb_host_build_external(b"c3", 1, rows, dim, 0, 2, 0, 0, 1, ir, i, orank, o, 0, None)
    assert h, host.fwd_eb_host_last_log()
    blob = blob_of(host, h)
    assert len(blob) < 1024
    loaded = host.fwd_eb_host_load(blob, len(blob), h)
    assert loaded
    assert free0 - torch.cuda.mem_get_info()[0] < (64 << 20)           # nothing of the table's size was allocated
    assert host.fwd_eb_host_table_uploads(loaded) == 0
    exp = capi.embedding_bag(table, torch.from_numpy(idx).cuda(), torch.from_numpy(off).cuda(),
                             mode=capi.MODE_MAX, padding_idx=0)
    for handle in (h, loaded):
        rc, got = _run(host, handle, torch, [idx, off], (off.size, dim), torch.float16)
        assert rc == 0 and np.array_equal(got.view(np.uint16), exp.cpu().numpy().view(np.uint16))
    host.fwd_eb_host_free(h)
    host.fwd_eb_host_free(loaded)
    host.fwd_eb_plugin_unregister_weights(b"c3")


@pytest.mark.gpu
def test_two_contexts_on_two_streams_share_the_built_in_scratch_in_turn(host):
    """Two execution contexts (clones) enqueue long-bag calls on different streams at once; both go
    through the one scratch array of the GPU, which the plugin hands out one call at a time."""
    torch = pytest.importorskip("torch")
    rng = np.random.default_rng(14)
    table = rng.standard_normal((3000, 64)).astype(np.float32)
    table = np.round(table * 4) / 4       # sums of quarters are exact in fp32 whatever the order
    lengths = np.array([60000, 40000, 0, 30000])
    off = np.zeros(4, dtype=np.int32)
    off[1:] = np.cumsum(lengths[:-1])
    batches = [rng.integers(0, 3000, int(lengths.sum())).astype(np.int32) for _ in range(2)]
    h = build(host, table, op=0, idx_dims=batches[0].shape, off_dims=(4,))
    ctx = host.fwd_eb_host_clone_context(h)
    handles = [h, ctx]
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    d_idx = [torch.from_numpy(b).cuda() for b in batches]
    d_off = torch.from_numpy(off).cuda()
    outs = [torch.zeros((4, 64), dtype=torch.float32, device="cuda") for _ in range(2)]
    torch.cuda.synchronize()
    for rep in range(20):
        for k in range(2):
            rc = host.fwd_eb_host_run(handles[k], d_idx[k].data_ptr(), d_off.data_ptr(), None,
                                      outs[k].data_ptr(), streams[k].cuda_stream)
            assert rc == 0
    torch.cuda.synchronize()
    for k in range(2):
        exp = O.pool(table, batches[k], off, mode=O.MODE_SUM)
        assert np.array_equal(outs[k].cpu().numpy(), exp)
    host.fwd_eb_host_free(h)
    host.fwd_eb_host_free(ctx)


def test_damaged_blobs_are_refused_or_loaded_never_crash(host):
    """Random header fields, byte flips and truncations of a valid engine blob: deserializePlugin
    must come back with a plugin or with nullptr (and a logged reason) for every one of them."""
    rng = np.random.default_rng(5)
    t = rng.standard_normal((6, 8)).astype(np.float32)
    h = build(host, t, op=0, idx_dims=(10,), off_dims=(3,))
    blob = blob_of(host, h)
    cases = [blob[:n] for n in range(0, len(blob), 5)]
    for _ in range(300):
        b = bytearray(blob)
        if rng.random() < 0.5:      # one of the five header fields replaced by an arbitrary value
            field = int(rng.integers(0, 5))
            if field < 4:
                struct.pack_into("<i", b, 4 * field, int(rng.integers(-2**31, 2**31)))
            else:
                struct.pack_into("<Q", b, 16, int(rng.integers(0, 2**63)))
        else:
            for _ in range(int(rng.integers(1, 4))):
                b[int(rng.integers(0, len(b)))] = int(rng.integers(0, 256))
        cases.append(bytes(b))
    loaded = refused = 0
    for data in cases:
        got = host.fwd_eb_host_load(data, len(data), h)
        if got:
            loaded += 1
            host.fwd_eb_host_free(got)
        else:
            refused += 1
    assert loaded > 0 and refused > 0
    host.fwd_eb_host_free(h)
