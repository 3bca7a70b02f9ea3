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


CORE_SOURCES = ("eb_api.cu", "eb_session.cu", "eb_noalloc.cu", "eb_shard.cu")


def build_core(force: bool = False, verbose: bool = False) -> str:
    """Compile each translation unit (in parallel) and link libfwd_eb.so."""
    from concurrent.futures import ThreadPoolExecutor

    target = os.path.join(LIBDIR, "libfwd_eb.so")
    srcs = [os.path.join(CSRC, f) for f in CORE_SOURCES]
    headers = _walk(CSRC, (".cuh", ".h")) + _walk(INCLUDE, (".h",))
    headers = [h for h in headers if os.sep + "plugin" + os.sep not in h]
    objdir = os.path.join(ROOT, "build", "obj")
    os.makedirs(objdir, exist_ok=True)
    os.makedirs(LIBDIR, exist_ok=True)
    compile_flags = [f for f in NVCC_FLAGS if f not in ("-shared", "-Xlinker", "--exclude-libs", "ALL")]
    jobs = []
    objs = []
    for src in srcs:
        obj = os.path.join(objdir, os.path.basename(src) + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            cmd = [_nvcc()] + ARCH + compile_flags + ["-DFWD_EB_BUILD", "-I", INCLUDE, "-I", CSRC]
            if verbose:
                cmd += ["-Xptxas", "-v"]
            jobs.append(cmd + ["-c", "-o", obj, src])
    if jobs:
        with ThreadPoolExecutor(max_workers=len(jobs)) as pool:
            list(pool.map(lambda c: _run(c, verbose), jobs))
    if force or jobs or _stale(target, objs):
        _run([_nvcc()] + ARCH + NVCC_FLAGS + ["-o", target] + objs, verbose)
    return target


# Experiment builds of libfwd_eb.so (never loaded by default; FWD_EB_LIB points capi at one).
VARIANTS = {
    # the lean kernel with its table rows staged through shared memory: by cp.async, and by the
    # bulk copy engine (cp.async.bulk + mbarrier); see csrc/eb_lite_staged.cuh
    "row_staging_cp_async": ["-DFWD_EB_ROW_STAGING=1"],
    "row_staging_bulk": ["-DFWD_EB_ROW_STAGING=2"],
    # reads tuning knobs from the environment (FWD_EB_PUSH_CTA, FWD_EB_STREAM_K, FWD_EB_IPL1)
    "tune": ["-DFWD_EB_TUNE"],
}


def build_variant(name: str, verbose: bool = False) -> str:
    """One nvcc call, all translation units, into build/variants/libfwd_eb_<name>.so."""
    flags = VARIANTS[name]
    outdir = os.path.join(ROOT, "build", "variants")
    os.makedirs(outdir, exist_ok=True)
    target = os.path.join(outdir, f"libfwd_eb_{name}.so")
    srcs = [os.path.join(CSRC, f) for f in CORE_SOURCES]
    cmd = [_nvcc()] + ARCH + NVCC_FLAGS + flags + ["-DFWD_EB_BUILD", "-I", INCLUDE, "-I", CSRC]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    _run(cmd + ["-o", target] + srcs, verbose)
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


def build_torch(force: bool = False, verbose: bool = False) -> str | None:
    """The torch parser slice (needs libtorch's C++ headers, which ship with the torch wheel)."""
    tdir = os.path.join(CSRC, "torch_cvt")
    pdir = os.path.join(CSRC, "plugin")
    if not os.path.isdir(tdir):
        return None
    try:
        import torch
    except ImportError:
        return None
    troot = os.path.dirname(torch.__file__)
    tinc = os.path.join(troot, "include")
    if not os.path.exists(os.path.join(tinc, "torch", "script.h")):
        return None
    plugin = build_plugin(force, verbose)
    target = os.path.join(LIBDIR, "libfwd_eb_torch.so")
    srcs = _walk(tdir, (".cpp",))
    deps = srcs + _walk(tdir, (".h",)) + _walk(pdir, (".h",)) + [plugin]
    if force or _stale(target, deps):
        gxx = shutil.which("g++") or "g++"
        abi = int(torch.compiled_with_cxx11_abi())
        cmd = [gxx, "-O2", "-std=c++17", "-fPIC", "-shared", f"-D_GLIBCXX_USE_CXX11_ABI={abi}",
               "-I", tinc, "-I", os.path.join(tinc, "torch", "csrc", "api", "include"),
               "-I", "/usr/local/cuda/include", "-I", tdir, "-I", pdir,
               "-I", os.path.join(pdir, "trt_shim"), "-o", target] + srcs + [
            "-L", LIBDIR, "-lfwd_eb_plugin", "-lfwd_eb", "-L", os.path.join(troot, "lib"), "-ltorch",
            "-ltorch_cpu", "-lc10", "-L", "/usr/local/cuda/lib64", "-lcudart",
            "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + os.path.join(troot, "lib")]
        _run(cmd, verbose)
    return target


def build_tf(force: bool = False, verbose: bool = False) -> str | None:
    """The TensorFlow parser slice (own GraphDef reader: no TensorFlow needed)."""
    tdir = os.path.join(CSRC, "tf_cvt")
    pdir = os.path.join(CSRC, "plugin")
    if not os.path.isdir(tdir):
        return None
    plugin = build_plugin(force, verbose)
    target = os.path.join(LIBDIR, "libfwd_eb_tf.so")
    srcs = _walk(tdir, (".cpp",))
    deps = srcs + _walk(tdir, (".h",)) + _walk(pdir, (".h",)) + [plugin]
    if force or _stale(target, deps):
        gxx = shutil.which("g++") or "g++"
        cmd = [gxx, "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", "/usr/local/cuda/include",
               "-I", tdir, "-I", pdir, "-I", os.path.join(pdir, "trt_shim"), "-o", target] + srcs + [
            "-L", LIBDIR, "-lfwd_eb_plugin", "-Wl,-rpath,$ORIGIN"]
        _run(cmd, verbose)
    return target


def build_all(force: bool = False, verbose: bool = False) -> list[str]:
    out = [build_core(force, verbose)]
    for step in (build_plugin, build_tf, build_torch):
        p = step(force, verbose)
        if p:
            out.append(p)
    return out


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--variant", choices=sorted(VARIANTS), help="build one experiment variant of libfwd_eb.so")
    ns = ap.parse_args()
    if ns.variant:
        print(build_variant(ns.variant, ns.verbose))
        sys.exit(0)
    for path in build_all(ns.force, ns.verbose):
        print(path)
