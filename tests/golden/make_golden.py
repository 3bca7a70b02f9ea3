"""Regenerates the golden fixtures in this directory.

Run where the Forward reference tree is mounted (pass its root, or rely on the default):

    python tests/golden/make_golden.py [reference_root]

Outputs
-------
embedding_bag_pth.npz   weights of the reference's own fixture
                        data/torch_unit_tests/nodes/embedding_bag.pth, the inputs of
                        its unit test (source/unit_test/test_torch_nodes.h:178-185)
                        and of its trace call (unit_test_model_factory.py:301), and the
                        outputs the loaded TorchScript module gives for both on CPU —
                        the ground truth the reference test compares its engine with.
embedding_bag_pb.npz    the table of the reference's TensorFlow fixture
                        data/tf_unit_tests/embedding_bag.pb (read with the protobuf
                        reader in tests/tf_graphdef.py; TensorFlow is not needed), seeded
                        indices of the shape its unit test draws
                        (source/unit_test/test_tf_nodes.h:199-211: int32 [10, 5] in
                        [0, 50)), and what the graph computes for them in numpy: the
                        two pooled terms and its output "sub" = Sum^2 - Sum_1.
torch_cpu_cases.npz     torch CPU EmbeddingBag outputs for small seeded cases that
                        the reference never tests (mean, max, fp16, padding_idx,
                        per_sample_weights, include_last_offset, empty bags).
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch
import torch.nn.functional as F

HERE = os.path.dirname(os.path.abspath(__file__))


def reference_fixture(ref_root: str) -> None:
    path = os.path.join(ref_root, "data", "torch_unit_tests", "nodes", "embedding_bag.pth")
    module = torch.jit.load(path, map_location="cpu").eval()
    weight = dict(module.named_parameters())["EE.weight"].detach().clone()
    out = {"weight": weight.numpy()}
    cases = {
        "unit_test": ([1, 0, 3, 1, 4], [0, 0, 0, 0, 0]),   # test_torch_nodes.h:180-181
        "trace": ([1, 0, 3, 1, 4], [0, 2]),                # unit_test_model_factory.py:301
    }
    for name, (idx, off) in cases.items():
        i = torch.tensor(idx, dtype=torch.long)
        o = torch.tensor(off, dtype=torch.long)
        with torch.no_grad():
            y = module(i, o)
        out[f"{name}_indices"] = i.numpy()
        out[f"{name}_offsets"] = o.numpy()
        out[f"{name}_expected"] = y.numpy()
    np.savez(os.path.join(HERE, "embedding_bag_pth.npz"), **out)


def tf_reference_fixture(ref_root: str) -> None:
    sys.path.insert(0, os.path.dirname(HERE))
    import tf_graphdef as G
    path = os.path.join(ref_root, "data", "tf_unit_tests", "embedding_bag.pb")
    nodes = G.read_nodes(open(path, "rb").read())
    gather = nodes["embedding_lookup"]
    assert gather["op"] == "GatherV2" and nodes["Sum"]["op"] == "Sum" and nodes["sub"]["op"] == "Sub"
    table_node = nodes[gather["inputs"][0]]
    while table_node["op"] == "Identity":
        table_node = nodes[table_node["inputs"][0]]
    weight = G.const_value(table_node["attrs"]["value"])
    rng = np.random.default_rng(199)
    indices = rng.integers(0, weight.shape[0], (10, 5)).astype(np.int32)
    e = weight[indices].astype(np.float32)             # mask = sequence_mask(5, 5): all ones
    s = np.zeros((10, weight.shape[1]), dtype=np.float32)
    q = np.zeros_like(s)
    for l in range(indices.shape[1]):                  # in bag order, fp32, like the kernels
        s = s + e[:, l, :]
        q = q + e[:, l, :] * e[:, l, :]
    np.savez(os.path.join(HERE, "embedding_bag_pb.npz"), weight=weight, indices=indices,
             sum=s, square_sum=q, sub=s * s - q)


def torch_cases() -> None:
    rng = np.random.default_rng(20240607)
    out = {}
    names = []
    case_id = 0
    for dtype in (np.float32, np.float16):
        for dim in (4, 8, 20, 40):
            for mode in ("sum", "mean", "max"):
                for variant in ("plain", "padding", "last_offset", "weights"):
                    if variant == "weights" and mode != "sum":
                        continue
                    rows = 24
                    table = rng.standard_normal((rows, dim)).astype(dtype)
                    if mode == "max":  # few distinct values so ties happen
                        table = (np.round(table.astype(np.float32) * 2) / 2).astype(dtype)
                    lengths = rng.integers(0, 9, 7)
                    lengths[2] = 0  # always an empty bag
                    offsets = np.concatenate([[0], np.cumsum(lengths)]).astype(np.int64)
                    n = int(offsets[-1])
                    indices = rng.integers(0, rows, n).astype(np.int64)
                    pad = -1
                    ilo = False
                    psw = None
                    if variant == "padding":
                        pad = 3
                        indices[rng.random(n) < 0.3] = pad
                        # one bag made of padding only
                        s, e = offsets[4], offsets[5]
                        indices[s:e] = pad
                    elif variant == "last_offset":
                        ilo = True
                    elif variant == "weights":
                        psw = rng.random(n).astype(dtype)
                    off_arg = offsets if ilo else offsets[:-1]
                    with torch.no_grad():
                        y = F.embedding_bag(
                            torch.from_numpy(indices), torch.from_numpy(table),
                            torch.from_numpy(off_arg), mode=mode,
                            per_sample_weights=None if psw is None else torch.from_numpy(psw),
                            include_last_offset=ilo, padding_idx=None if pad < 0 else pad)
                    key = f"c{case_id:03d}"
                    case_id += 1
                    names.append(f"{key}|{np.dtype(dtype).name}|{dim}|{mode}|{variant}|{pad}|{int(ilo)}")
                    out[f"{key}_table"] = table
                    out[f"{key}_indices"] = indices
                    out[f"{key}_offsets"] = off_arg
                    out[f"{key}_expected"] = y.numpy()
                    if psw is not None:
                        out[f"{key}_psw"] = psw
    out["names"] = np.array(names)
    np.savez_compressed(os.path.join(HERE, "torch_cpu_cases.npz"), **out)


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
    from oracle.refpath import reference_root
    root = sys.argv[1] if len(sys.argv) > 1 else reference_root()
    if not root:
        sys.exit("no Forward reference tree found: pass its path or set FWD_REFERENCE_ROOT")
    reference_fixture(root)
    tf_reference_fixture(root)
    torch_cases()
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))
