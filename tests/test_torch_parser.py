"""The torch parser slice: TorchScript file -> aten::embedding_bag node -> TrtEmbeddingBagDesc
(-> layer creator -> plugin -> enqueue on a GPU).  Models are traced here, so nothing outside
the repository is read; where the reference's own fixture is mounted it is parsed too."""
import ctypes as C
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")

from forward_b200 import capi  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIB = os.path.join(ROOT, "forward_b200", "lib", "libfwd_eb_torch.so")
from oracle.refpath import reference_root  # noqa: E402

REF_FIXTURE = os.path.join(reference_root() or "", "data", "torch_unit_tests", "nodes", "embedding_bag.pth")


@pytest.fixture(scope="module")
def tl():
    if not os.path.exists(LIB):
        pytest.skip("libfwd_eb_torch.so was not built (libtorch headers missing)")
    capi.lib()
    host = C.CDLL(os.path.join(ROOT, "forward_b200", "lib", "libfwd_eb_plugin.so"), mode=C.RTLD_GLOBAL)
    lib = C.CDLL(LIB)
    lib.fwd_eb_torch_parse.restype = C.c_void_p
    lib.fwd_eb_torch_parse.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
    lib.fwd_eb_torch_free.argtypes = [C.c_void_p]
    lib.fwd_eb_torch_desc_info.argtypes = [C.c_void_p] + [C.c_void_p] * 9
    lib.fwd_eb_torch_input_name.restype = C.c_char_p
    lib.fwd_eb_torch_input_name.argtypes = [C.c_void_p, C.c_int]
    lib.fwd_eb_torch_desc_weights.restype = C.c_size_t
    lib.fwd_eb_torch_desc_weights.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
    lib.fwd_eb_torch_build_engine.restype = C.c_void_p
    lib.fwd_eb_torch_build_engine.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                              C.c_int, C.c_void_p]
    host.fwd_eb_host_run.argtypes = [C.c_void_p] * 6
    host.fwd_eb_host_free.argtypes = [C.c_void_p]
    host.fwd_eb_host_output_dims.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.host = host
    return lib


class Bag(torch.nn.Module):
    def __init__(self, rows, dim, mode, padding_idx=None, include_last_offset=False, half=False,
                 weighted=False):
        super().__init__()
        self.ee = torch.nn.EmbeddingBag(rows, dim, mode=mode, padding_idx=padding_idx,
                                        include_last_offset=include_last_offset)
        if half:
            self.ee = self.ee.half()
        self.weighted = weighted

    def forward(self, index, offset, w=None):
        return self.ee(index, offset, per_sample_weights=w) if self.weighted else self.ee(index, offset)


def save_traced(tmp_path, name, module, example):
    traced = torch.jit.trace(module.eval(), example)
    path = str(tmp_path / name)
    traced.save(path)
    return path


def parse(tl, path):
    err = C.create_string_buffer(512)
    p = tl.fwd_eb_torch_parse(path.encode(), err, 512)
    return p, err.value.decode()


def info(tl, p):
    ints = [C.c_int() for _ in range(4)]
    pad = C.c_longlong()
    rest = [C.c_int() for _ in range(4)]
    n = tl.fwd_eb_torch_desc_info(p, *[C.byref(x) for x in ints], C.byref(pad),
                                  *[C.byref(x) for x in rest])
    keys = ("dim", "count", "offset", "op")
    out = {k: v.value for k, v in zip(keys, ints)}
    out.update(padding_idx=pad.value, include_last_offset=rest[0].value, weighted=rest[1].value,
               half_table=rest[2].value, half_output=rest[3].value, n_inputs=n)
    out["inputs"] = [tl.fwd_eb_torch_input_name(p, i).decode() for i in range(n)]
    return out


def weights(tl, p, dtype, shape):
    n = tl.fwd_eb_torch_desc_weights(p, None, 0)
    buf = np.empty(n, dtype=np.uint8)
    tl.fwd_eb_torch_desc_weights(p, buf.ctypes.data, n)
    return buf.view(dtype).reshape(shape)


EXAMPLE = (torch.tensor([1, 0, 3, 1, 4]), torch.tensor([0, 2]))


@pytest.mark.parametrize("mode,op", [("sum", 0), ("mean", 1), ("max", 2)])
def test_mode_and_weight_are_read_from_the_graph(tl, tmp_path, mode, op):
    m = Bag(5, 4, mode)
    p, err = parse(tl, save_traced(tmp_path, f"{mode}.pt", m, EXAMPLE))
    assert p, err
    d = info(tl, p)
    assert (d["dim"], d["count"], d["offset"], d["op"]) == (4, 5, 0, op)
    assert d["padding_idx"] == -1 and not d["include_last_offset"] and not d["weighted"]
    assert d["n_inputs"] == 2 and not d["half_table"] and not d["half_output"]
    assert np.array_equal(weights(tl, p, np.float32, (5, 4)), m.ee.weight.detach().numpy())
    tl.fwd_eb_torch_free(p)


def test_attributes_the_reference_parser_dropped(tl, tmp_path):
    """padding_idx, include_last_offset, per_sample_weights and fp16 weights (the reference's
    creator reads none of them, torch_embedding_bag_creator.h:54-61)."""
    m = Bag(9, 8, "sum", padding_idx=2, include_last_offset=True, weighted=True)
    ex = (torch.tensor([1, 0, 3, 1, 4]), torch.tensor([0, 2, 5]), torch.rand(5))
    p, err = parse(tl, save_traced(tmp_path, "full.pt", m, ex))
    assert p, err
    d = info(tl, p)
    assert d["padding_idx"] == 2 and d["include_last_offset"] == 1 and d["weighted"] == 1
    assert d["n_inputs"] == 3 and d["inputs"][2].split(".")[0] == "w"
    tl.fwd_eb_torch_free(p)
    neg = Bag(9, 8, "mean", padding_idx=-1)           # torch stores it as 8
    p, err = parse(tl, save_traced(tmp_path, "neg.pt", neg, EXAMPLE))
    assert p and info(tl, p)["padding_idx"] == 8
    tl.fwd_eb_torch_free(p)
    half = Bag(6, 8, "mean", half=True)
    p, err = parse(tl, save_traced(tmp_path, "half.pt", half, EXAMPLE))
    assert p, err
    d = info(tl, p)
    assert d["half_table"] == 1 and d["half_output"] == 1
    assert np.array_equal(weights(tl, p, np.float16, (6, 8)), half.ee.weight.detach().numpy())
    tl.fwd_eb_torch_free(p)


def test_failures_are_reported_not_guessed(tl, tmp_path):
    p, err = parse(tl, str(tmp_path / "missing.pt"))
    assert not p and "load failed" in err
    lin = torch.jit.trace(torch.nn.Linear(4, 2).eval(), torch.zeros(1, 4))
    path = str(tmp_path / "linear.pt")
    lin.save(path)
    p, err = parse(tl, path)
    assert not p and "no aten::embedding_bag" in err


@pytest.mark.skipif(not os.path.exists(REF_FIXTURE), reason="reference tree not mounted")
def test_reference_fixture_parses_to_the_committed_weights(tl, golden_dir):
    p, err = parse(tl, REF_FIXTURE)
    assert p, err
    d = info(tl, p)
    assert (d["dim"], d["count"], d["op"], d["n_inputs"]) == (4, 5, 0, 2)
    assert d["inputs"] == ["input.1", "offsets.1"] or d["inputs"][0].startswith("input")
    g = np.load(os.path.join(golden_dir, "embedding_bag_pth.npz"))
    assert np.array_equal(weights(tl, p, np.float32, (5, 4)), g["weight"])
    tl.fwd_eb_torch_free(p)


@pytest.mark.gpu
@pytest.mark.parametrize("mode", ["sum", "mean", "max"])
@pytest.mark.parametrize("half", [False, True])
def test_parsed_model_runs_through_the_plugin(tl, tmp_path, mode, half):
    """parse -> description -> layer creator -> EmbeddingBag_TRT -> enqueue, against the
    module's own CPU output (the comparison Forward's unit test makes)."""
    torch.manual_seed(3)
    m = Bag(2000, 64, mode, padding_idx=7, half=half)
    rng = np.random.default_rng(5)
    lengths = rng.integers(0, 30, 400)
    off = np.zeros(400, dtype=np.int64)
    off[1:] = np.cumsum(lengths[:-1])
    idx = rng.integers(0, 2000, int(lengths.sum())).astype(np.int64)
    idx[::10] = 7
    ti, to = torch.from_numpy(idx), torch.from_numpy(off)
    p, err = parse(tl, save_traced(tmp_path, "run.pt", m, (ti, to)))
    assert p, err
    dims_i = (C.c_int * 1)(idx.size)
    dims_o = (C.c_int * 1)(off.size)
    h = tl.fwd_eb_torch_build_engine(p, 1, dims_i, 1, dims_o, 0, None)
    assert h
    with torch.no_grad():
        expect = m(ti, to)
    di = ti.to(torch.int32).cuda()                      # Forward casts int64 -> int32 on the way in
    do = to.to(torch.int32).cuda()
    out = torch.empty((400, 64), dtype=torch.float16 if half else torch.float32, device="cuda")
    rc = tl.host.fwd_eb_host_run(h, di.data_ptr(), do.data_ptr(), None, out.data_ptr(),
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0
    assert torch.equal(out.cpu(), expect)               # bit for bit
    tl.host.fwd_eb_host_free(h)
    tl.fwd_eb_torch_free(p)


# ---- whole graphs: several bags, concatenation, stacked offsets, int64 inputs -------------------

class TensorArg(C.Structure):
    _fields_ = [("data", C.c_void_p), ("dtype", C.c_int), ("rank", C.c_int), ("dims", C.c_longlong * 4),
                ("graph_input", C.c_int), ("element", C.c_int)]


def _net_api(tl):
    tl.fwd_eb_torch_parse_network.restype = C.c_void_p
    tl.fwd_eb_torch_parse_network.argtypes = [C.c_char_p, C.c_char_p, C.c_size_t]
    tl.fwd_eb_torch_net_free.argtypes = [C.c_void_p]
    for name in ("num_layers", "num_outputs", "num_graph_inputs"):
        getattr(tl, "fwd_eb_torch_net_" + name).argtypes = [C.c_void_p]
    tl.fwd_eb_torch_net_error.restype = C.c_char_p
    tl.fwd_eb_torch_net_error.argtypes = [C.c_void_p]
    tl.fwd_eb_torch_net_layer_info.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 3
    tl.fwd_eb_torch_net_layer_input.argtypes = [C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 3
    tl.fwd_eb_torch_net_output_layers.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    tl.fwd_eb_torch_net_run.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
    return tl


def parse_network(tl, path):
    _net_api(tl)
    err = C.create_string_buffer(512)
    n = tl.fwd_eb_torch_parse_network(path.encode(), err, 512)
    return n, err.value.decode()


class Tower(torch.nn.Module):
    """DLRM's sparse side (the shape of Forward's own DLRM test, test_torch_dlrm.h:37-56): T bags,
    offsets stacked in one [T, B] tensor, one index tensor per bag, pooled rows concatenated."""

    def __init__(self, tables, dim, mode="sum"):
        super().__init__()
        self.bags = torch.nn.ModuleList([torch.nn.EmbeddingBag(r, dim, mode=mode) for r in tables])

    def forward(self, offsets, *indices):
        return torch.cat([bag(i, offsets[k]) for k, (bag, i) in enumerate(zip(self.bags, indices))], dim=1)


def _tower_inputs(tables, nb, seed):
    g = torch.Generator().manual_seed(seed)
    lengths = [torch.randint(0, 6, (nb,), generator=g) for _ in tables]
    offsets = torch.stack([torch.cumsum(l, 0) - l for l in lengths])
    indices = [torch.randint(0, r, (int(l.sum()),), generator=g) for r, l in zip(tables, lengths)]
    return offsets, indices


@pytest.mark.parametrize("tables", [3, 26])
def test_every_bag_of_a_graph_is_found_with_its_inputs(tl, tmp_path, tables):
    rows = [40 + 7 * t for t in range(tables)]
    tower = Tower(rows, 8)
    offsets, indices = _tower_inputs(rows, 5, 0)
    path = save_traced(tmp_path, f"tower{tables}.pth", tower, (offsets, *indices))
    n, err = parse_network(tl, path)
    assert n, err
    assert tl.fwd_eb_torch_net_num_layers(n) == tables and tl.fwd_eb_torch_net_num_outputs(n) == 1
    assert tl.fwd_eb_torch_net_num_graph_inputs(n) == tables + 1
    order = (C.c_int * 64)()
    assert tl.fwd_eb_torch_net_output_layers(n, 0, order, 64) == tables
    for pos in range(tables):
        layer = order[pos]
        dim, count, op = C.c_int(), C.c_int(), C.c_int()
        assert tl.fwd_eb_torch_net_layer_info(n, layer, C.byref(dim), C.byref(count), C.byref(op)) == 2
        assert (dim.value, count.value, op.value) == (8, rows[pos], 0)       # cat order = table order
        gi, el, fl = C.c_int(), C.c_int(), C.c_int()
        tl.fwd_eb_torch_net_layer_input(n, layer, 0, C.byref(gi), C.byref(el), C.byref(fl))
        assert (gi.value, el.value) == (1 + pos, -1)                          # its own index tensor
        tl.fwd_eb_torch_net_layer_input(n, layer, 1, C.byref(gi), C.byref(el), C.byref(fl))
        assert (gi.value, el.value, fl.value) == (0, pos, 0)                  # row `pos` of the stacked offsets
    tl.fwd_eb_torch_net_free(n)


def test_graphs_with_other_operators_are_refused_with_the_operator_named(tl, tmp_path):
    class Scaled(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ee = torch.nn.EmbeddingBag(30, 4, mode="sum")

        def forward(self, index, offset):
            return torch.relu(self.ee(index, offset))

    n, err = parse_network(tl, save_traced(tmp_path, "relu.pth", Scaled(), EXAMPLE))
    assert not n and "aten::relu" in err

    class Shifted(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.ee = torch.nn.EmbeddingBag(30, 4, mode="sum")

        def forward(self, index, offset):
            return self.ee(index + 1, offset)

    n, err = parse_network(tl, save_traced(tmp_path, "add.pth", Shifted(), EXAMPLE))
    assert not n and "aten::add" in err

    class Stacked(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a = torch.nn.EmbeddingBag(30, 4, mode="sum")
            self.b = torch.nn.EmbeddingBag(30, 4, mode="sum")

        def forward(self, index, offset):
            return torch.cat([self.a(index, offset), self.b(index, offset)], dim=0)

    n, err = parse_network(tl, save_traced(tmp_path, "cat0.pth", Stacked(), EXAMPLE))
    assert not n and "dim 1" in err


def _run_network(tl, n, feeds, out_shape):
    """feeds: list of (graph_input, element, CUDA tensor)."""
    args = (TensorArg * len(feeds))()
    for a, (gi, el, t) in zip(args, feeds):
        a.data, a.rank, a.graph_input, a.element = t.data_ptr(), t.dim(), gi, el
        a.dtype = {torch.int32: 0, torch.int64: 1, torch.float32: 2}[t.dtype]
        for q, d in enumerate(t.shape):
            a.dims[q] = d
    out = torch.full(out_shape, float("nan"), dtype=torch.float32, device="cuda:0")
    outs = (C.c_void_p * 1)(out.data_ptr())
    rc = tl.fwd_eb_torch_net_run(n, args, len(feeds), outs, C.c_void_p(capi.current_stream_ptr()))
    torch.cuda.synchronize()
    assert rc == 0, tl.fwd_eb_torch_net_error(n)
    return out.cpu()


@pytest.mark.gpu
@pytest.mark.parametrize("tables", [3, 26])
def test_a_tower_of_bags_runs_from_int64_inputs_and_matches_the_module(tl, tmp_path, tables):
    """Parse -> one plugin per bag -> int64 inputs cast to int32 on the way in (as Forward's engine
    does) -> enqueue -> concatenate; twice, the second time with fresh indices of the same sizes."""
    rows = [300 + 11 * t for t in range(tables)]
    tower = Tower(rows, 16).eval()
    offsets, indices = _tower_inputs(rows, 64, 1)
    path = save_traced(tmp_path, f"tower{tables}.pth", tower, (offsets, *indices))
    n, err = parse_network(tl, path)
    assert n, err
    for rep in range(2):
        if rep:
            indices = [torch.randint(0, r, i.shape) for r, i in zip(rows, indices)]
        feeds = [(0, -1, offsets.cuda())] + [(1 + k, -1, i.cuda()) for k, i in enumerate(indices)]
        got = _run_network(tl, n, feeds, (64, 16 * tables))
        exp = tower(offsets, *indices).detach()
        assert torch.equal(got, exp)
    tl.fwd_eb_torch_net_free(n)


@pytest.mark.gpu
def test_config1_through_parser_plugin_and_enqueue(tl, tmp_path):
    """BASELINE config 1 (EmbeddingBag(10000, 64, mode='sum'), fp32 N(0,1) weights, 32 bags of 1..20
    uniform indices, seed 0) through parse -> plugin -> enqueue, against torch CPU within 1e-5
    relative (it is bit-identical: the kernel adds in bag order)."""
    from forward_b200 import workloads
    table, bags = workloads.config1(seed=0)
    bag = Bag(10000, 64, "sum")
    with torch.no_grad():
        bag.ee.weight.copy_(torch.from_numpy(table))
    idx = torch.from_numpy(bags.indices.astype(np.int64))
    off = torch.from_numpy(bags.offsets.astype(np.int64))
    path = save_traced(tmp_path, "config1.pth", bag, (idx, off))
    n, err = parse_network(tl, path)
    assert n, err
    got = _run_network(tl, n, [(0, -1, idx.cuda()), (1, -1, off.cuda())], (32, 64))
    exp = torch.nn.functional.embedding_bag(idx, torch.from_numpy(table), off, mode="sum")
    torch.testing.assert_close(got, exp, rtol=1e-5, atol=0)
    assert torch.equal(got, exp)
    tl.fwd_eb_torch_net_free(n)
