"""The TensorFlow parser slice: frozen GraphDef -> Sum(Mul(GatherV2)) / Sum(Square(Mul(GatherV2)))
/ bare GatherV2 patterns -> TrtEmbeddingBagDesc (-> layer creator -> plugin -> enqueue on a GPU).

Graphs are written here with the small protobuf writer in tf_graphdef.py, so nothing outside the
repository is read; where the reference's own fixture is mounted it is parsed too and must give
the table committed under tests/golden/."""
import ctypes as C
import os

import numpy as np
import pytest

import tf_graphdef as G
from forward_b200 import capi
from oracle import eb_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
LIBDIR = os.path.join(ROOT, "forward_b200", "lib")
from oracle.refpath import reference_root  # noqa: E402

REF_FIXTURE = os.path.join(reference_root() or "", "data", "tf_unit_tests", "embedding_bag.pb")


@pytest.fixture(scope="module")
def tf():
    capi.lib()
    host = C.CDLL(os.path.join(LIBDIR, "libfwd_eb_plugin.so"), mode=C.RTLD_GLOBAL)
    lib = C.CDLL(os.path.join(LIBDIR, "libfwd_eb_tf.so"))
    lib.fwd_eb_tf_parse.restype = C.c_void_p
    lib.fwd_eb_tf_parse.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_size_t]
    lib.fwd_eb_tf_free.argtypes = [C.c_void_p]
    lib.fwd_eb_tf_num_descs.argtypes = [C.c_void_p]
    for fn in (lib.fwd_eb_tf_desc_node, lib.fwd_eb_tf_desc_input):
        fn.restype = C.c_char_p
        fn.argtypes = [C.c_void_p, C.c_int]
    lib.fwd_eb_tf_desc_info.argtypes = [C.c_void_p, C.c_int] + [C.c_void_p] * 5
    lib.fwd_eb_tf_desc_weights.restype = C.c_size_t
    lib.fwd_eb_tf_desc_weights.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_size_t]
    lib.fwd_eb_tf_build_engine.restype = C.c_void_p
    lib.fwd_eb_tf_build_engine.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    host.fwd_eb_host_run.argtypes = [C.c_void_p] * 6
    host.fwd_eb_host_free.argtypes = [C.c_void_p]
    host.fwd_eb_host_output_dims.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p]
    lib.host = host
    return lib


def parse(tf, path, outputs):
    err = C.create_string_buffer(512)
    p = tf.fwd_eb_tf_parse(str(path).encode(), outputs.encode(), err, 512)
    return p, err.value.decode("utf-8", "replace")


def descs(tf, p):
    out = []
    for i in range(tf.fwd_eb_tf_num_descs(p)):
        v = [C.c_int() for _ in range(5)]
        assert tf.fwd_eb_tf_desc_info(p, i, *[C.byref(x) for x in v]) == 0
        d = dict(zip(("dim", "count", "offset", "op", "half_table"), (x.value for x in v)))
        d["node"] = tf.fwd_eb_tf_desc_node(p, i).decode()
        d["input"] = tf.fwd_eb_tf_desc_input(p, i).decode()
        n = tf.fwd_eb_tf_desc_weights(p, i, None, 0)
        buf = np.empty(n, dtype=np.uint8)
        tf.fwd_eb_tf_desc_weights(p, i, buf.ctypes.data, n)
        dt = np.float16 if d["half_table"] else np.float32
        d["weights"] = buf.view(dt).reshape(d["count"], -1)
        out.append(d)
    return out


def write(tmp_path, name, graph: bytes):
    path = tmp_path / name
    path.write_bytes(graph)
    return path


def table(rows, dim, dtype=np.float32, seed=0):
    return np.random.default_rng(seed).standard_normal((rows, dim)).astype(dtype)


def test_fm_graph_gives_a_sum_and_a_square_sum_description(tf, tmp_path):
    w = table(50, 10)
    p, err = parse(tf, write(tmp_path, "fm.pb", G.fm_graph(w, 5)), "sub")
    assert p, err
    d = descs(tf, p)
    assert [(x["node"], x["op"]) for x in d] == [("Sum", 0), ("Sum_1", 3)]
    for x in d:
        assert (x["dim"], x["count"], x["offset"], x["input"]) == (10, 50, 0, "ids")
        assert np.array_equal(x["weights"], w)
    tf.fwd_eb_tf_free(p)
    # no Identity between GatherV2 and Mul; table given as float_val instead of tensor_content
    p, err = parse(tf, write(tmp_path, "fm2.pb", G.fm_graph(w, 5, identity=False, table_as_values=True)),
                   "Sum")
    assert p, err
    d = descs(tf, p)
    assert len(d) == 1 and d[0]["op"] == 0 and np.array_equal(d[0]["weights"], w)
    tf.fwd_eb_tf_free(p)


def test_bare_gather_fp16_table_and_weights_node(tf, tmp_path):
    w = table(30, 8, np.float16)
    p, err = parse(tf, write(tmp_path, "g.pb", G.gather_graph(w, 4)), "out")
    assert p, err
    d = descs(tf, p)
    assert len(d) == 1 and d[0]["op"] == 999 and d[0]["node"] == "lookup" and d[0]["half_table"] == 1
    assert np.array_equal(d[0]["weights"], w)
    tf.fwd_eb_tf_free(p)
    # a "<scope>_weights" node takes precedence over the constant feeding GatherV2
    w32, other = table(20, 4), table(20, 4, seed=9)
    p, err = parse(tf, write(tmp_path, "w.pb", G.fm_graph(w32, 3, weights_node=other)), "Sum")
    assert p, err
    assert np.array_equal(descs(tf, p)[0]["weights"], other)
    tf.fwd_eb_tf_free(p)
    # rank-1 table: dim 1
    p, err = parse(tf, write(tmp_path, "r1.pb", G.gather_graph(np.arange(7, dtype=np.float32), 2)), "out")
    assert p, err
    d = descs(tf, p)[0]
    assert (d["dim"], d["count"]) == (1, 7)
    tf.fwd_eb_tf_free(p)


def test_what_cannot_be_converted_faithfully_is_refused(tf, tmp_path):
    w = table(12, 4)
    bad = {
        "axis": G.fm_graph(w, 3, gather_axis=1),
        "sum_axis": G.fm_graph(w, 3, sum_axis=2),
        "keep_dims": G.fm_graph(w, 3, keep_dims=True),
        "table": G.fm_graph(w, 3, table_placeholder=True),
    }
    for name, graph in bad.items():
        p, err = parse(tf, write(tmp_path, name + ".pb", graph), "Sum")
        assert not p and "rejected Sum" in err, (name, err)
    # negative axis counted from the back is the same axis: accepted
    p, err = parse(tf, write(tmp_path, "neg.pb", G.fm_graph(w, 3, sum_axis=-2)), "Sum")
    assert p, err
    tf.fwd_eb_tf_free(p)
    good = G.fm_graph(w, 3)
    p, err = parse(tf, write(tmp_path, "cut.pb", good[:len(good) // 2 + 3]), "sub")
    assert not p and "load failed" in err
    p, err = parse(tf, write(tmp_path, "ok.pb", good), "nope")
    assert not p and "no operation named nope" in err
    p, err = parse(tf, tmp_path / "missing.pb", "sub")
    assert not p and "load failed" in err
    p, err = parse(tf, write(tmp_path, "empty.pb", b""), "sub")
    assert not p and "load failed" in err


def test_python_and_cpp_readers_agree_on_a_written_graph(tf, tmp_path):
    w = table(9, 6, seed=4)
    graph = G.fm_graph(w, 4)
    nodes = G.read_nodes(graph)
    assert nodes["emb/gather"]["inputs"] == ["emb/read", "ids", "emb/axis"]
    assert np.array_equal(G.const_value(nodes["emb/table"]["attrs"]["value"]), w)
    p, err = parse(tf, write(tmp_path, "a.pb", graph), "sub")
    assert p, err
    assert np.array_equal(descs(tf, p)[0]["weights"], w)
    tf.fwd_eb_tf_free(p)


@pytest.mark.skipif(not os.path.exists(REF_FIXTURE), reason="reference tree not mounted")
def test_reference_fixture_parses_to_the_committed_table(tf, golden_dir):
    """data/tf_unit_tests/embedding_bag.pb, output "sub" (source/unit_test/test_tf_nodes.h:199-211)."""
    p, err = parse(tf, REF_FIXTURE, "sub")
    assert p, err
    d = descs(tf, p)
    g = np.load(os.path.join(golden_dir, "embedding_bag_pb.npz"))
    assert [(x["node"], x["op"], x["input"]) for x in d] == [("Sum", 0, "Placeholder"),
                                                             ("Sum_1", 3, "Placeholder")]
    for x in d:
        assert (x["dim"], x["count"]) == (10, 50) and np.array_equal(x["weights"], g["weight"])
    tf.fwd_eb_tf_free(p)


def test_golden_terms_match_the_oracle(golden_dir):
    """The committed numpy evaluation of the reference graph against the CPU oracle's fixed-length
    SUM / SQUARE_SUM (bit for bit: both add in bag order in fp32)."""
    g = np.load(os.path.join(golden_dir, "embedding_bag_pb.npz"))
    idx = g["indices"].reshape(-1)
    s = O.pool(g["weight"], idx, None, mode=O.MODE_SUM, fixed_len=5)
    q = O.pool(g["weight"], idx, None, mode=O.MODE_SQUARE_SUM, fixed_len=5)
    assert np.array_equal(s, g["sum"])
    np.testing.assert_allclose(q, g["square_sum"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(s * s - q, g["sub"], rtol=1e-5, atol=1e-6)


def _run(tf, p, i, idx2d, dim, out_shape, dtype):
    import torch
    dims = (C.c_int * 2)(*idx2d.shape)
    h = tf.fwd_eb_tf_build_engine(p, i, 2, dims)
    assert h
    od = (C.c_int * 8)()
    rank = tf.host.fwd_eb_host_output_dims(h, od, None)
    assert tuple(od[:rank]) == tuple(out_shape)
    d_idx = torch.from_numpy(idx2d).cuda()
    out = torch.empty(out_shape, dtype=dtype, device="cuda")
    rc = tf.host.fwd_eb_host_run(h, d_idx.data_ptr(), None, None, out.data_ptr(),
                                 C.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert rc == 0
    tf.host.fwd_eb_host_free(h)
    return out.cpu().numpy()


@pytest.mark.gpu
def test_golden_graph_runs_through_the_plugin(tf, tmp_path, golden_dir):
    """The reference fixture's table in a graph of the same structure: parse -> descriptions ->
    layer creator -> EmbeddingBag_TRT -> enqueue; the two pooled terms and "sub" against the
    committed numpy evaluation."""
    import torch
    g = np.load(os.path.join(golden_dir, "embedding_bag_pb.npz"))
    p, err = parse(tf, write(tmp_path, "gold.pb", G.fm_graph(g["weight"], 5)), "sub")
    assert p, err
    s = _run(tf, p, 0, g["indices"], 10, (10, 10), torch.float32)
    q = _run(tf, p, 1, g["indices"], 10, (10, 10), torch.float32)
    tf.fwd_eb_tf_free(p)
    assert np.array_equal(s, g["sum"])
    np.testing.assert_allclose(q, g["square_sum"], rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(s * s - q, g["sub"], rtol=1e-5, atol=1e-5)


@pytest.mark.gpu
@pytest.mark.parametrize("half", [False, True])
def test_parsed_patterns_match_the_oracle_at_size(tf, tmp_path, half):
    import torch
    dt = np.float16 if half else np.float32
    w = (table(5000, 64, seed=11) * 0.5).astype(dt)
    rng = np.random.default_rng(12)
    idx = rng.integers(0, 5000, (2048, 20)).astype(np.int32)
    p, err = parse(tf, write(tmp_path, "big.pb", G.fm_graph(w, 20)), "sub")
    assert p, err
    for i, mode in ((0, O.MODE_SUM), (1, O.MODE_SQUARE_SUM)):
        got = _run(tf, p, i, idx, 64, (2048, 64), torch.float32)       # the plugin's output is fp32
        exp = O.pool(w, idx.reshape(-1), None, mode=mode, fixed_len=20, out_dtype=np.float32)
        if mode == O.MODE_SUM:
            assert np.array_equal(got, exp)
        else:
            np.testing.assert_allclose(got, exp, rtol=1e-5, atol=1e-6)
    tf.fwd_eb_tf_free(p)
    p, err = parse(tf, write(tmp_path, "gather.pb", G.gather_graph(w, 20)), "out")
    assert p, err
    got = _run(tf, p, 0, idx, 64, (2048, 20, 64), torch.float32)
    tf.fwd_eb_tf_free(p)
    assert np.array_equal(got, w[idx].astype(np.float32))


def test_damaged_graphs_are_refused_or_parsed_never_crash(tf, tmp_path):
    """Truncations and byte flips of a valid GraphDef: the reader must come back with a handle or
    an error text for every one of them (a wild read would take the test process down)."""
    w = table(20, 4)
    good = G.fm_graph(w, 3)
    rng = np.random.default_rng(77)
    path = tmp_path / "fuzz.pb"
    seen_error = seen_ok = 0
    cases = [good[:n] for n in range(0, len(good), 7)]
    for _ in range(300):
        b = bytearray(good)
        for _ in range(int(rng.integers(1, 4))):
            b[int(rng.integers(0, len(b)))] = int(rng.integers(0, 256))
        cases.append(bytes(b))
    for data in cases:
        path.write_bytes(data)
        p, err = parse(tf, path, "sub")
        if p:
            seen_ok += 1
            for d in descs(tf, p):
                assert d["weights"].size == d["count"] * d["dim"]
            tf.fwd_eb_tf_free(p)
        else:
            seen_error += 1
            assert err
    assert seen_error > 0 and seen_ok > 0


@pytest.mark.skipif(not os.path.exists(REF_FIXTURE), reason="reference tree not mounted")
def test_reference_recommender_graphs_yield_their_gather_descriptions(tf):
    """The reference's larger fixtures (source/unit_test/test_tf_recommender.h:56-71 DeepFM.pb, output
    "Softmax"; test_tf_nodes.h embedding.pb): the walk passes through the dense layers and finds the
    one embedding lookup each holds, as a GATHER description over the graph's own table."""
    root = os.path.dirname(REF_FIXTURE)
    for name, output, node, feed, shape in (
            ("DeepFM.pb", "Softmax", "DNN/GatherV2", "Placeholder_2", (1706, 40)),
            ("embedding.pb", "embedding_4/embedding_lookup/Identity_1", "embedding_4/embedding_lookup",
             "input1_1", (1000, 64))):
        p, err = parse(tf, os.path.join(root, name), output)
        assert p, err
        d = descs(tf, p)
        assert len(d) == 1
        assert (d[0]["node"], d[0]["input"], d[0]["op"]) == (node, feed, 999)
        assert (d[0]["count"], d[0]["dim"]) == shape and d[0]["weights"].shape == shape
        assert np.isfinite(d[0]["weights"]).all() and d[0]["weights"].std() > 0
        tf.fwd_eb_tf_free(p)
