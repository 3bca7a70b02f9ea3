"""In-tree build of the native libraries (explicit nvcc / g++ commands).

    python -m forward_b200.build            # build what is stale
    python -m forward_b200.build --force    # rebuild everything
    python -m forward_b200.build --verbose  # also print ptxas resource usage

Outputs (git-ignored, next to the sources so they travel with the tree):
    forward_b200/lib/libfwd_eb.so          kernels + C ABI (include/fwd_eb.h)
    forward_b200/lib/libfwd_eb_plugin.so   EmbeddingBag_TRT plugin, creators and
                                           the host driver used by the tests
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "forward_b200", "csrc")
LIBDIR = os.path.join(ROOT, "forward_b200", "lib")
INCLUDE = os.path.join(ROOT, "include")

ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
              "-shared",
              # keep the statically linked CUDA runtime private to each library
              "-Xlinker", "--exclude-libs", "-Xlinker", "ALL"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: the CUDA toolkit is required to build forward_b200")
    return exe


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _walk(dirpath: str, exts: tuple[str, ...]) -> list[str]:
    out = []
    for base, _, files in os.walk(dirpath):
        for f in files:
            if f.endswith(exts):
                out.append(os.path.join(base, f))
    return sorted(out)


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print(" ".join(cmd), flush=True)
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        sys.stderr.write(proc.stdout + proc.stderr)
        raise RuntimeError(f"build step failed: {' '.join(cmd[:3])} ...")
    if verbose:
        sys.stdout.write(proc.stdout + proc.stderr)


def build_core(force: bool = False, verbose: bool = False) -> str:
    target = os.path.join(LIBDIR, "libfwd_eb.so")
    srcs = [os.path.join(CSRC, f) for f in ("eb_api.cu", "eb_session.cu", "eb_noalloc.cu")]
    srcs = [s for s in srcs if os.path.exists(s)]
    deps = srcs + _walk(CSRC, (".cuh", ".h")) + _walk(INCLUDE, (".h",))
    if force or _stale(target, deps):
        os.makedirs(LIBDIR, exist_ok=True)
        cmd = [_nvcc()] + ARCH + NVCC_FLAGS + ["-DFWD_EB_BUILD", "-I", INCLUDE, "-I", CSRC]
        if verbose:
            cmd += ["-Xptxas", "-v"]
        cmd += ["-o", target] + srcs
        _run(cmd, verbose)
    return target


def build_plugin(force: bool = False, verbose: bool = False) -> str | None:
    pdir = os.path.join(CSRC, "plugin")
    if not os.path.isdir(pdir):
        return None
    target = os.path.join(LIBDIR, "libfwd_eb_plugin.so")
    core = build_core(force, verbose)
    srcs = _walk(pdir, (".cpp", ".cu"))
    deps = srcs + _walk(pdir, (".h", ".hpp")) + _walk(INCLUDE, (".h",)) + [core]
    if force or _stale(target, deps):
        cmd = [_nvcc()] + ARCH + NVCC_FLAGS + [
            "-I", INCLUDE, "-I", pdir, "-I", os.path.join(pdir, "trt_shim"),
            "-o", target] + srcs + [
            "-L", LIBDIR, "-lfwd_eb", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN"]
        _run(cmd, verbose)
    return target


def build_all(force: bool = False, verbose: bool = False) -> list[str]:
    out = [build_core(force, verbose)]
    p = build_plugin(force, verbose)
    if p:
        out.append(p)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ns = ap.parse_args()
    for path in build_all(ns.force, ns.verbose):
        print(path)
