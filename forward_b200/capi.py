"""ctypes binding of the C ABI in include/fwd_eb.h (libfwd_eb.so).

The binding is deliberately thin: torch is used for device memory and streams
only; every compute call goes through the C entry points.  There is no CPU or
eager fallback — a missing or unloadable library raises at import of the
symbols, and a non-zero status raises ``FwdEbError`` with the library's text.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# FWD_EB_LIB: another build of the library (an experiment variant from forward_b200.build --variant)
LIB_PATH = os.environ.get("FWD_EB_LIB") or os.path.join(_HERE, "lib", "libfwd_eb.so")

MODE_SUM, MODE_MEAN, MODE_MAX, MODE_SQUARE_SUM, MODE_GATHER = 0, 1, 2, 3, 999
F32, F16 = 0, 1
F32_POS = 2          # MODE_MAX only: {fp32 value, int32 position} per column
NO_POS = 0x7FFFFFFF
I32, I64 = 0, 1
STRATEGY_AUTO, STRATEGY_GROUP, STRATEGY_CTA, STRATEGY_SPLIT, STRATEGY_STREAM, STRATEGY_LITE = 0, 1, 2, 3, 4, 5
FLAG_MEAN_RAW_LENGTH, FLAG_GATHER_KEEP_SKIPPED, FLAG_MEAN_SINGLE_ROUNDING = 1, 2, 4
FLAG_OFFSET_PAIRS, FLAG_PAIRS_RUN16 = 8, 16
EINVAL, EUNSUPPORTED, EALIGN, EWORKSPACE, ENOGPU, ETOOBIG = -1, -2, -3, -4, -5, -6


class FwdEbError(RuntimeError):
    def __init__(self, code: int, text: str):
        super().__init__(f"fwd_eb error {code}: {text}")
        self.code = code


class Params(C.Structure):
    """Mirror of struct fwd_eb_params; field order and types must match the header."""
    _fields_ = [
        ("table", C.c_void_p), ("table_dtype", C.c_int32), ("dim", C.c_int32),
        ("num_rows", C.c_int64), ("row_lo", C.c_int64), ("table_stride", C.c_int64),
        ("indices", C.c_void_p), ("offsets", C.c_void_p), ("index_dtype", C.c_int32),
        ("fixed_len", C.c_int32), ("num_indices", C.c_int64), ("num_bags", C.c_int64),
        ("per_sample_weights", C.c_void_p), ("mode", C.c_int32),
        ("include_last_offset", C.c_int32), ("padding_idx", C.c_int64),
        ("out", C.c_void_p), ("out_dtype", C.c_int32), ("strategy", C.c_int32),
        ("out_stride", C.c_int64),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("flags", C.c_uint32),
        ("reserved", C.c_int32),
    ]


# name -> (restype, argtypes); also the list the symbol-export test walks
SIGNATURES = {
    "fwd_eb_version": (C.c_int, []),
    "fwd_eb_params_size": (C.c_size_t, []),
    "fwd_eb_last_error_string": (C.c_char_p, []),
    "fwd_eb_forward": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "fwd_eb_forward_many": (C.c_int, [C.POINTER(C.POINTER(Params)), C.c_int32, C.c_void_p]),
    "fwd_eb_workspace_size": (C.c_size_t, [C.POINTER(Params)]),
    "fwd_eb_pick_strategy": (C.c_int, [C.POINTER(Params)]),
    "fwd_eb_forward_static_scratch": (C.c_int, [C.POINTER(Params), C.c_void_p]),
    "fwd_eb_static_scratch_prepare": (C.c_int, []),
    "fwd_eb_compact_window": (C.c_int, [C.POINTER(Params), C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                        C.c_void_p]),
    "fwd_eb_launch_count": (C.c_uint64, []),
    "fwd_eb_gather_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                    C.c_int, C.c_int, C.c_void_p]),
    "fwd_eb_bag_fixed_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                       C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "fwd_eb_bag_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                 C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]),
    "fwd_eb_fill_table": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_int32, C.c_int64,
                                    C.c_uint64, C.c_float, C.c_void_p]),
    "fwd_eb_cast_i64_to_i32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p]),
    "fwd_eb_combine_partials": (C.c_int, [C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int64,
                                          C.c_void_p, C.c_int32, C.c_void_p]),
}

_lib = None


def lib() -> C.CDLL:
    """Load libfwd_eb.so (building it first if the sources are newer)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            from . import build as _build
            _build.build_core()
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)  # AttributeError here = symbol missing: fail loudly
            fn.restype = res
            fn.argtypes = args
        if handle.fwd_eb_version() != 1:
            raise RuntimeError("libfwd_eb.so ABI version mismatch")
        if handle.fwd_eb_params_size() != C.sizeof(Params):
            raise RuntimeError("ctypes mirror of fwd_eb_params is out of step with the library")
        _lib = handle
    return _lib


def check(code: int) -> None:
    if code != 0:
        raise FwdEbError(code, lib().fwd_eb_last_error_string().decode("utf-8", "replace"))


def _torch_dtype_code(t) -> int:
    import torch
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.float16:
        return F16
    raise TypeError(f"unsupported table/output dtype {t.dtype}")


def _index_code(t) -> int:
    import torch
    if t.dtype == torch.int32:
        return I32
    if t.dtype == torch.int64:
        return I64
    raise TypeError(f"unsupported index dtype {t.dtype}")


def current_stream_ptr() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def make_params(table, indices, offsets=None, *, out, mode=MODE_SUM, fixed_len=0,
                per_sample_weights=None, include_last_offset=False, padding_idx=-1, row_lo=0,
                num_rows=None, strategy=STRATEGY_AUTO, workspace=None, flags=0) -> Params:
    """Fill a Params from torch CUDA tensors (no copies; tensors must stay alive)."""
    for t in (table, indices, out):
        if not t.is_cuda:
            raise ValueError("make_params takes CUDA tensors; there is no CPU path")
    if table.dim() != 2 or table.stride(1) != 1:
        raise ValueError("table must be 2-D with unit column stride")
    p = Params()
    p.table = table.data_ptr()
    p.table_dtype = _torch_dtype_code(table)
    p.dim = table.shape[1]
    p.num_rows = table.shape[0] if num_rows is None else num_rows
    p.row_lo = row_lo
    p.table_stride = table.stride(0)
    idx = indices.reshape(-1)
    if not idx.is_contiguous():
        raise ValueError("indices must be contiguous")
    p.indices = idx.data_ptr()
    p.index_dtype = _index_code(idx)
    p.num_indices = idx.numel()
    p.fixed_len = fixed_len
    if mode == MODE_GATHER:
        p.num_bags = 0
    elif fixed_len > 0:
        p.num_bags = idx.numel() // fixed_len
    else:
        off = offsets.reshape(-1)
        if off.dtype != idx.dtype or not off.is_contiguous() or not off.is_cuda:
            raise ValueError("offsets must be a contiguous CUDA tensor of the indices' dtype")
        p.offsets = off.data_ptr()
        p.num_bags = off.numel() - (1 if include_last_offset else 0)
    if per_sample_weights is not None:
        import torch
        if per_sample_weights.dtype != torch.float32 or not per_sample_weights.is_cuda:
            raise ValueError("per_sample_weights must be fp32 CUDA")
        p.per_sample_weights = per_sample_weights.data_ptr()
    p.mode = mode
    p.include_last_offset = int(include_last_offset)
    p.padding_idx = padding_idx
    p.out = out.data_ptr()
    p.out_dtype = _torch_dtype_code(out)
    p.out_stride = out.stride(0) if out.dim() == 2 else 0
    p.strategy = strategy
    if workspace is not None:
        p.workspace = workspace.data_ptr()
        p.workspace_bytes = workspace.numel() * workspace.element_size()
    p.flags = flags
    return p


def forward(params: Params, stream: int | None = None) -> None:
    check(lib().fwd_eb_forward(C.byref(params), C.c_void_p(stream if stream is not None
                                                           else current_stream_ptr())))


def pack_params(params_list):
    """A C array of pointers to the given Params, for forward_many (keep the list alive)."""
    n = len(params_list)
    return (C.POINTER(Params) * max(n, 1))(*[C.pointer(p) for p in params_list]), n


def forward_many(packed, stream: int | None = None) -> None:
    """Independent calls (one per table of a model) spread over the caller's stream and the
    library's auxiliary streams; `packed` = pack_params([...])."""
    ptrs, n = packed
    check(lib().fwd_eb_forward_many(ptrs, n, C.c_void_p(stream if stream is not None
                                                        else current_stream_ptr())))


def embedding_bag(table, indices, offsets=None, *, mode=MODE_SUM, fixed_len=0,
                  per_sample_weights=None, include_last_offset=False, padding_idx=-1, row_lo=0,
                  out_dtype=None, strategy=STRATEGY_AUTO, flags=0, out=None, use_workspace=True):
    """Gather-and-pool on the current CUDA device and stream; returns the output tensor."""
    import torch
    idx = indices.reshape(-1)
    if mode == MODE_GATHER:
        n_out = idx.numel()
    elif fixed_len > 0:
        n_out = idx.numel() // fixed_len
    else:
        n_out = offsets.numel() - (1 if include_last_offset else 0)
    if out is None:
        out = torch.empty((n_out, table.shape[1]), dtype=out_dtype or table.dtype,
                          device=table.device)
    p = make_params(table, indices, offsets, out=out, mode=mode, fixed_len=fixed_len,
                    per_sample_weights=per_sample_weights,
                    include_last_offset=include_last_offset, padding_idx=padding_idx,
                    row_lo=row_lo, strategy=strategy, flags=flags)
    ws = None
    if use_workspace and mode != MODE_GATHER:
        need = lib().fwd_eb_workspace_size(C.byref(p))
        if need:
            ws = torch.empty(need, dtype=torch.uint8, device=table.device)
            p.workspace = ws.data_ptr()
            p.workspace_bytes = need
    forward(p)
    return out


def compact_window(params: Params, kept, bounds, *, kept_weights=None, counts=None,
                   stream: int | None = None) -> None:
    """fwd_eb_compact_window: keep the indices of `params` that fall inside its row window (and are
    not padding) as dense sub-bags.  kept: int32 [num_indices]; bounds: int32 [num_bags, 2];
    kept_weights: fp32 [num_indices] when params carries per_sample_weights; counts: optional
    int32 [num_bags] (non-padding entries of each whole bag).  Pool the result with
    make_compacted_params()."""
    check(lib().fwd_eb_compact_window(
        C.byref(params), C.c_void_p(kept.data_ptr()),
        C.c_void_p(kept_weights.data_ptr()) if kept_weights is not None else None,
        C.c_void_p(bounds.data_ptr()), C.c_void_p(counts.data_ptr()) if counts is not None else None,
        C.c_void_p(stream if stream is not None else current_stream_ptr())))


def make_compacted_params(table, kept, bounds, *, out, mode=MODE_SUM, kept_weights=None,
                          strategy=STRATEGY_AUTO, flags=0) -> Params:
    """Params that pool what compact_window wrote: local row numbers, {start, end} pairs."""
    p = make_params(table, kept, None, out=out, mode=mode, per_sample_weights=kept_weights,
                    fixed_len=1, strategy=strategy, flags=flags | FLAG_OFFSET_PAIRS | FLAG_PAIRS_RUN16)
    p.fixed_len = 0
    p.offsets = bounds.data_ptr()
    p.num_bags = bounds.shape[0]
    return p


def fill_table(table, row_lo: int, seed: int, scale: float) -> None:
    check(lib().fwd_eb_fill_table(table.data_ptr(), _torch_dtype_code(table), table.shape[0],
                                  table.shape[1], row_lo, seed, scale,
                                  C.c_void_p(current_stream_ptr())))


def combine_partials(parts, out) -> None:
    """parts: [num_parts, ...] contiguous; out: the trailing shape."""
    count = out.numel()
    check(lib().fwd_eb_combine_partials(parts.data_ptr(), _torch_dtype_code(parts), parts.shape[0],
                                        parts.stride(0), count, out.data_ptr(),
                                        _torch_dtype_code(out), C.c_void_p(current_stream_ptr())))
