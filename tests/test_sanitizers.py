"""The GraphDef reader and the TensorFlow pattern matcher under AddressSanitizer and
UndefinedBehaviorSanitizer: the host code that reads untrusted bytes (a frozen graph file) is
compiled with both and fed valid graphs, truncations, byte flips, spliced fragments and inflated
length fields.  Any wild read, signed overflow, misaligned access or leak ends the harness with a
non-zero status.  CPU only."""
import os
import shutil
import subprocess
import sys

import numpy as np
import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import tf_graphdef as G  # noqa: E402

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "forward_b200", "csrc")
LIBDIR = os.path.join(ROOT, "forward_b200", "lib")
SAN = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer"]


def _build(tmp_path):
    gxx = shutil.which("g++")
    if not gxx:
        pytest.skip("no g++")
    probe = tmp_path / "probe.cpp"
    probe.write_text("int main() { return 0; }\n")
    if subprocess.run([gxx] + SAN + ["-o", str(tmp_path / "probe"), str(probe)],
                      capture_output=True).returncode != 0:
        pytest.skip("this g++ has no sanitizer runtime")
    from forward_b200 import build
    if build.build_tf() is None:
        pytest.skip("TensorFlow parser slice not in this tree")
    tdir, pdir = os.path.join(CSRC, "tf_cvt"), os.path.join(CSRC, "plugin")
    exe = tmp_path / "tf_parse_harness"
    srcs = [os.path.join(ROOT, "tests", "sanitize", "tf_parse_harness.cpp")] + \
        [os.path.join(tdir, f) for f in ("tf_graph.cpp", "tf_desc_manager.cpp", "tf_driver.cpp")]
    cmd = [gxx, "-O1", "-g", "-std=c++17"] + SAN + [
        "-I", "/usr/local/cuda/include", "-I", tdir, "-I", pdir, "-I", os.path.join(pdir, "trt_shim"),
        "-o", str(exe)] + srcs + ["-L", LIBDIR, "-lfwd_eb_plugin", f"-Wl,-rpath,{LIBDIR}"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-2000:]
    return exe


def _varint_positions(data: bytes):
    """Offsets of bytes that look like the single-byte length of a length-delimited field (the
    byte after a tag whose wire type is 2)."""
    return [i + 1 for i in range(len(data) - 1) if (data[i] & 7) == 2 and data[i + 1] < 0x80]


def test_graphdef_reader_and_matcher_under_asan_and_ubsan(tmp_path):
    exe = _build(tmp_path)
    rng = np.random.default_rng(5)
    w = rng.standard_normal((24, 4)).astype(np.float32)
    good = [G.fm_graph(w, 3), G.fm_graph(w, 3, identity=False, table_as_values=True),
            G.fm_graph(w.astype(np.float16), 5), G.gather_graph(w, 4)]
    cases = list(good)
    base = good[0]
    cases += [base[:n] for n in range(0, len(base), 5)]                       # truncations
    for _ in range(400):                                                      # byte flips
        b = bytearray(good[int(rng.integers(0, len(good)))])
        for _ in range(int(rng.integers(1, 5))):
            b[int(rng.integers(0, len(b)))] = int(rng.integers(0, 256))
        cases.append(bytes(b))
    for _ in range(100):                                                      # spliced fragments
        a, c = (good[int(rng.integers(0, len(good)))] for _ in range(2))
        i, j = int(rng.integers(0, len(a))), int(rng.integers(0, len(c)))
        cases.append(a[:i] + c[j:])
    lens = _varint_positions(base)
    for _ in range(150):                                                      # inflated / shrunk lengths
        b = bytearray(base)
        at = lens[int(rng.integers(0, len(lens)))]
        b[at] = int(rng.choice([0, 1, 0x7f, 0xff, b[at] + 1 & 0x7f, max(0, b[at] - 1)]))
        if b[at] == 0xff:                                                     # a multi-byte varint that never ends
            b[at + 1:at + 1] = b"\xff" * int(rng.integers(1, 12))
        cases.append(bytes(b))
    paths = []
    for k, data in enumerate(cases):
        p = tmp_path / f"case{k}.pb"
        p.write_bytes(data)
        paths.append(str(p))
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:halt_on_error=1", UBSAN_OPTIONS="print_stacktrace=1")
    for outputs in ("sub", "out", "Sum"):
        done = subprocess.run([str(exe), outputs] + paths, capture_output=True, text=True, env=env, timeout=600)
        assert done.returncode == 0, (done.stdout[-500:], done.stderr[-3000:])
        parsed, refused = (int(done.stdout.split()[i]) for i in (1, 3))
        assert parsed > 0 and refused > 0 and parsed + refused == len(cases)


def test_plugin_blob_deserialiser_under_asan_and_ubsan(tmp_path):
    """The EmbeddingBag_TRT plugin, its creator and the host driver compiled with both sanitizers;
    the harness builds plugins, serialises them and loads damaged copies of the blobs."""
    gxx = shutil.which("g++")
    if not gxx:
        pytest.skip("no g++")
    probe = tmp_path / "probe.cpp"
    probe.write_text("int main() { return 0; }\n")
    if subprocess.run([gxx] + SAN + ["-o", str(tmp_path / "probe"), str(probe)],
                      capture_output=True).returncode != 0:
        pytest.skip("this g++ has no sanitizer runtime")
    from forward_b200 import build
    build.build_core()
    pdir = os.path.join(CSRC, "plugin")
    srcs = [os.path.join(ROOT, "tests", "sanitize", "plugin_blob_harness.cpp")]
    for base, _, files in os.walk(pdir):
        srcs += [os.path.join(base, f) for f in sorted(files) if f.endswith(".cpp")]
    exe = tmp_path / "plugin_blob_harness"
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = [gxx, "-O1", "-g", "-std=c++17"] + SAN + [
        "-I", os.path.join(cuda, "include"), "-I", os.path.join(ROOT, "include"), "-I", pdir,
        "-I", os.path.join(pdir, "trt_shim"), "-o", str(exe)] + srcs + [
        "-L", LIBDIR, "-lfwd_eb", "-L", os.path.join(cuda, "lib64"), "-lcudart", f"-Wl,-rpath,{LIBDIR}",
        f"-Wl,-rpath,{os.path.join(cuda, 'lib64')}"]
    done = subprocess.run(cmd, capture_output=True, text=True)
    assert done.returncode == 0, done.stderr[-3000:]
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:halt_on_error=1:protect_shadow_gap=0",
               UBSAN_OPTIONS="print_stacktrace=1")
    done = subprocess.run([str(exe)], capture_output=True, text=True, env=env, timeout=600)
    assert done.returncode == 0, (done.stdout[-500:], done.stderr[-4000:])
    assert "loaded" in done.stdout
