"""CPU-side checks of the C ABI: the library loads, exports what the header declares, the
ctypes mirror matches the struct, and argument errors are reported before any launch."""
import ctypes as C
import os
import re

import pytest

from forward_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names.update(re.findall(r"\b(fwd_eb_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported_and_bound():
    lib = capi.lib()
    declared = _declared_symbols()
    assert len(declared) >= 11
    handles = [lib]
    plugin = os.path.join(ROOT, "forward_b200", "lib", "libfwd_eb_plugin.so")
    if os.path.exists(plugin):
        handles.append(C.CDLL(plugin))
    for name in declared:
        assert any(hasattr(h, name) for h in handles), f"{name} declared but not exported"
    for name in capi.SIGNATURES:
        assert name in declared, f"{name} bound in capi.py but not declared in include/"


def test_struct_mirror_size_and_version():
    assert capi.lib().fwd_eb_version() == 1
    assert C.sizeof(capi.Params) == capi.lib().fwd_eb_params_size() == 152


def _params(**kw):
    p = capi.Params()
    p.table = 0x1000
    p.table_dtype = capi.F16
    p.dim = 128
    p.num_rows = 1000
    p.indices = 0x2000
    p.offsets = 0x3000
    p.num_indices = 4000
    p.num_bags = 100
    p.mode = capi.MODE_SUM
    p.padding_idx = -1
    p.out = 0x4000
    p.out_dtype = capi.F16
    for k, v in kw.items():
        setattr(p, k, v)
    return p


@pytest.mark.parametrize("kw,code", [
    (dict(dim=0), capi.EINVAL),
    (dict(mode=7), capi.EINVAL),
    (dict(table_dtype=5), capi.EINVAL),
    (dict(offsets=None), capi.EINVAL),
    (dict(num_rows=2**31), capi.ETOOBIG),
    (dict(fixed_len=7), capi.EINVAL),                       # 4000 != 100 * 7
    (dict(per_sample_weights=0x5000, mode=capi.MODE_MAX), capi.EINVAL),
    (dict(strategy=capi.STRATEGY_SPLIT, num_bags=4, num_indices=40000), capi.EWORKSPACE),
    (dict(table_stride=64), capi.EINVAL),
])
def test_bad_arguments_are_rejected_on_the_host(kw, code):
    """No launch happens for these, so they run without a GPU; nothing aborts."""
    lib = capi.lib()
    before = lib.fwd_eb_launch_count()
    p = _params(**kw)
    rc = lib.fwd_eb_forward(C.byref(p), None)
    assert rc == code
    assert lib.fwd_eb_last_error_string() != b""
    assert lib.fwd_eb_launch_count() == before
    with pytest.raises(capi.FwdEbError):
        capi.check(rc)


def test_null_params():
    assert capi.lib().fwd_eb_forward(None, None) == capi.EINVAL


def test_strategy_choice_and_workspace():
    lib = capi.lib()
    many_short = _params(num_bags=16384, num_indices=16384 * 40)
    # a lane group per bag; for rows of 128..512 bytes with int32 indices the lean kernel runs it
    assert lib.fwd_eb_pick_strategy(C.byref(many_short)) == capi.STRATEGY_LITE
    assert lib.fwd_eb_workspace_size(C.byref(many_short)) == 0
    shard = _params(num_bags=16384, num_indices=16384 * 40, row_lo=5000)    # a row window: survivor ring
    assert lib.fwd_eb_pick_strategy(C.byref(shard)) == capi.STRATEGY_GROUP
    wide = _params(num_bags=16384, num_indices=16384 * 40, dim=1024)        # rows beyond 512 bytes
    assert lib.fwd_eb_pick_strategy(C.byref(wide)) == capi.STRATEGY_GROUP
    fixed = _params(num_bags=1000, num_indices=20000, fixed_len=20, offsets=None)
    assert lib.fwd_eb_pick_strategy(C.byref(fixed)) == capi.STRATEGY_LITE
    some_long = _params(num_bags=1000, num_indices=1000 * 500)
    assert lib.fwd_eb_pick_strategy(C.byref(some_long)) == capi.STRATEGY_CTA
    few_huge = _params(num_bags=4, num_indices=4 * 100_000)
    assert lib.fwd_eb_pick_strategy(C.byref(few_huge)) == capi.STRATEGY_CTA  # no scratch offered
    need = lib.fwd_eb_workspace_size(C.byref(few_huge))
    assert need > 0
    few_huge.workspace = 0x10000
    few_huge.workspace_bytes = need
    assert lib.fwd_eb_pick_strategy(C.byref(few_huge)) == capi.STRATEGY_SPLIT
    few_huge.workspace_bytes = need - 1
    assert lib.fwd_eb_pick_strategy(C.byref(few_huge)) == capi.STRATEGY_CTA


def test_session_symbols_and_no_gpu_failure():
    """Every session entry point is exported; without a CUDA device creation fails with
    ENOGPU instead of falling back to anything."""
    from forward_b200 import session
    lib = session._lib()
    declared = _declared_symbols()
    for name in session.SIGNATURES:
        assert name in declared and hasattr(lib, name)
    import torch
    if not torch.cuda.is_available():
        with pytest.raises(capi.FwdEbError) as e:
            session.Session(table_dtype=capi.F16, dim=8, num_rows=4, mode=capi.MODE_SUM,
                            max_indices=4, max_bags=2)
        assert e.value.code == capi.ENOGPU


def test_headers_are_plain_c_and_a_c_host_links(tmp_path):
    """The boundary is a C ABI: a C99 translation unit including every public header compiles
    with -pedantic -Werror, links against libfwd_eb.so and calls into it."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if not gcc:
        pytest.skip("no C compiler")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    libdir = os.path.join(root, "forward_b200", "lib")
    src = tmp_path / "host.c"
    src.write_text('#include "fwd_eb.h"\n#include "fwd_eb_session.h"\n#include "fwd_eb_shard.h"\n'
                   "#include <stdio.h>\n"
                   "int main(void) {\n"
                   "  fwd_eb_params p;\n"
                   '  printf("%d %d\\n", fwd_eb_version(), (int)(fwd_eb_params_size() == sizeof p));\n'
                   "  return fwd_eb_forward(NULL, NULL) == FWD_EB_EINVAL ? 0 : 1;\n"
                   "}\n")
    exe = tmp_path / "host"
    subprocess.check_call([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic",
                           "-I", os.path.join(root, "include"), str(src), "-o", str(exe),
                           "-L", libdir, "-lfwd_eb", "-Wl,-rpath," + libdir])
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.split() == ["1", "1"]
