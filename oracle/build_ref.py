"""Compile the reference's EmbeddingBag kernels for sm_100a into oracle/_ref/libref_eb.so.

Sources are compiled where they lie in the reference tree (nothing is copied); the TensorRT
headers they include are satisfied by the interface stand-in under
forward_b200/csrc/plugin/trt_shim (TensorRT itself is not installed).  Only the .cu with the
three kernels and launchers is built — the plugin class needs libnvinfer.  The reference's own
build adds -use_fast_math (CMakeLists.txt:131-137); it is kept here so the kernels run as shipped.

    python oracle/build_ref.py [reference_root]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def main(ref_root: str) -> int:
    src = os.path.join(ref_root, "source", "trt_engine", "trt_network_crt", "plugins",
                       "embedding_bag_plugin", "embedding_bag_plugin.cu")
    if not os.path.exists(src):
        print("reference tree not found; nothing built")
        return 0
    out_dir = os.path.join(HERE, "_ref")
    os.makedirs(out_dir, exist_ok=True)
    out = os.path.join(out_dir, "libref_eb.so")
    deps = [src, os.path.join(HERE, "ref_wrap.cu")]
    if os.path.exists(out) and all(os.path.getmtime(out) >= os.path.getmtime(d) for d in deps):
        return 0
    cmd = ["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-use_fast_math",
           "-Xcompiler", "-fPIC", "-shared", "-Xlinker", "--exclude-libs", "-Xlinker", "ALL",
           "-I", os.path.join(ref_root, "source"),
           "-I", os.path.join(ROOT, "forward_b200", "csrc", "plugin", "trt_shim"),
           "-o", out, src, os.path.join(HERE, "ref_wrap.cu")]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        return proc.returncode
    print(out)
    return 0


if __name__ == "__main__":
    sys.path.insert(0, os.path.dirname(HERE))
    from oracle.refpath import reference_root
    root = sys.argv[1] if len(sys.argv) > 1 else reference_root()
    if not root:
        sys.exit("no Forward reference tree found: pass its path or set FWD_REFERENCE_ROOT")
    sys.exit(main(root))
