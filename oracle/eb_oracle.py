"""ctypes front for the CPU oracle (eb_oracle.c) and the torch CPU oracle.

TEST INFRASTRUCTURE ONLY: imported by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline / reference legs.  The product package never imports it.

Two independent answers are offered:

* ``pool`` — the C restatement of the reference plugin's kernels
  (embedding_bag_plugin.cu:66-181 in the Forward tree) with the enum's op
  meanings; ``semantics=1`` selects the literal behaviour of the reference .cu.
* ``torch_pool`` — ``torch.nn.functional.embedding_bag`` on the CPU, which is
  what the reference's own unit test compares its engine with
  (source/unit_test/unit_test_torch_helper.h:147-208).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle_eb.so")

SEM_ENUM, SEM_KERNEL = 0, 1
MODE_SUM, MODE_MEAN, MODE_MAX, MODE_SQUARE_SUM, MODE_GATHER = 0, 1, 2, 3, 999
FLAG_MEAN_RAW_LENGTH, FLAG_GATHER_KEEP_SKIPPED, FLAG_MEAN_SINGLE_ROUNDING = 1, 2, 4

_lib = None


def build(force: bool = False) -> str:
    """Compile eb_oracle.c with gcc via the Makefile beside it."""
    src = os.path.join(_HERE, "eb_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.check_call(["make", "-s", "-C", _HERE, "-f", os.path.join(_HERE, "Makefile")])
    return _LIB_PATH


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.oracle_eb_forward.restype = C.c_int
        _lib.oracle_eb_forward.argtypes = [
            C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int64, C.c_int64,  # table..stride
            C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int64, C.c_int64,  # indices..bags
            C.c_void_p, C.c_int32, C.c_int32, C.c_int64,  # psw, mode, ilo, padding
            C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_int32,  # out.., flags, semantics
        ]
        _lib.oracle_table_value.restype = C.c_float
        _lib.oracle_table_value.argtypes = [C.c_uint64, C.c_int64, C.c_int32, C.c_float]
        _lib.oracle_fill_rows.restype = None
        _lib.oracle_fill_rows.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_int64, C.c_int32,
                                          C.c_uint64, C.c_float]
        _lib.oracle_combine_partials.restype = None
        _lib.oracle_combine_partials.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int64,
                                                 C.c_int64, C.c_void_p, C.c_int32]
        _lib.oracle_half_to_float.restype = C.c_float
        _lib.oracle_half_to_float.argtypes = [C.c_uint16]
        _lib.oracle_float_to_half.restype = C.c_uint16
        _lib.oracle_float_to_half.argtypes = [C.c_float]
    return _lib


def _dt(a: np.ndarray) -> int:
    if a.dtype == np.float32:
        return 0
    if a.dtype == np.float16:
        return 1
    raise TypeError(f"table/out dtype {a.dtype}")


def _it(a: np.ndarray) -> int:
    if a.dtype == np.int32:
        return 0
    if a.dtype == np.int64:
        return 1
    raise TypeError(f"index dtype {a.dtype}")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def pool(table: np.ndarray, indices: np.ndarray, offsets: np.ndarray | None = None, *,
         mode: int = MODE_SUM, fixed_len: int = 0, per_sample_weights: np.ndarray | None = None,
         include_last_offset: bool = False, padding_idx: int = -1, row_lo: int = 0,
         out_dtype=None, flags: int = 0, semantics: int = SEM_ENUM,
         out: np.ndarray | None = None) -> np.ndarray:
    """Pool `table` rows by bags; mirrors fwd_eb_forward argument for argument."""
    table = np.ascontiguousarray(table)
    indices = np.ascontiguousarray(indices).reshape(-1)
    n = indices.size
    dim = table.shape[1]
    if offsets is not None:
        offsets = np.ascontiguousarray(offsets).reshape(-1)
        if offsets.dtype != indices.dtype:
            raise TypeError("indices and offsets must share a dtype")
    if mode == MODE_GATHER:
        n_bags, n_out = 0, n
    elif fixed_len > 0:
        n_bags = n // fixed_len
        n_out = n_bags
    else:
        n_bags = offsets.size - (1 if include_last_offset else 0)
        n_out = n_bags
    out_dtype = np.dtype(out_dtype or table.dtype)
    if out is None:
        out = np.zeros((n_out, dim), dtype=out_dtype)
    psw = None
    if per_sample_weights is not None:
        psw = np.ascontiguousarray(per_sample_weights, dtype=np.float32)
    rc = lib().oracle_eb_forward(
        _ptr(table), _dt(table), dim, table.shape[0], row_lo, 0,
        _ptr(indices), _ptr(offsets), _it(indices), fixed_len, n, n_bags,
        _ptr(psw), mode, int(include_last_offset), padding_idx,
        _ptr(out), _dt(out), 0, flags, semantics)
    if rc != 0:
        raise ValueError("oracle_eb_forward rejected its arguments")
    return out


def table_rows(rows: np.ndarray, dim: int, seed: int, scale: float, dtype=np.float16) -> np.ndarray:
    """Regenerate the listed logical rows of a counter-generated table."""
    rows = np.ascontiguousarray(rows, dtype=np.int64)
    out = np.empty((rows.size, dim), dtype=dtype)
    lib().oracle_fill_rows(_ptr(out), _dt(out), _ptr(rows), rows.size, dim, seed, scale)
    return out


def combine_partials(parts: np.ndarray, out_dtype=np.float32) -> np.ndarray:
    """parts: [num_parts, count] -> sum over axis 0 in slot order, fp32 math."""
    parts = np.ascontiguousarray(parts)
    out = np.empty(parts.shape[1:], dtype=out_dtype)
    count = int(np.prod(parts.shape[1:]))
    lib().oracle_combine_partials(_ptr(parts), _dt(parts), parts.shape[0], count, count,
                                  _ptr(out), _dt(out))
    return out


NO_POS = 0x7FFFFFFF


def max_with_positions(table: np.ndarray, indices: np.ndarray, offsets: np.ndarray, *, row_lo: int = 0,
                       padding_idx: int = -1):
    """A row shard's partial of a max: per bag and column {value (fp32), position inside the bag
    of the index that supplied it}, NO_POS where no row of the bag lies in [row_lo, row_lo+rows).

    The sequential rule torch CPU's max follows (a probe, not a reference file: the reference
    plugin has no sharding and its max op code is wrong, embedding_bag_plugin.cu:51-63): the
    bag's first non-padding entry is taken as is, a later entry only when strictly greater; so a
    NaN counts only when its entry is that first one.  Entries outside the window are skipped but
    still count as "seen".  Plain Python loops: small cases only."""
    nb, dim = offsets.size, table.shape[1]
    ends = np.append(offsets, indices.size)
    val = np.zeros((nb, dim), dtype=np.float32)
    pos = np.full((nb, dim), NO_POS, dtype=np.int32)
    for b in range(nb):
        seen = False
        for p, j in enumerate(range(int(ends[b]), int(ends[b + 1]))):
            idx = int(indices[j])
            if idx == padding_idx:
                continue
            first = not seen
            seen = True
            r = idx - row_lo
            if r < 0 or r >= table.shape[0]:
                continue
            x = table[r].astype(np.float32)
            fresh = pos[b] == NO_POS
            with np.errstate(invalid="ignore"):
                take = np.where(fresh, ~np.isnan(x) | first, x > val[b])
            val[b] = np.where(take, x, val[b])
            pos[b] = np.where(take, p, pos[b])
    return val, pos


def fold_max_partials(values: np.ndarray, positions: np.ndarray) -> np.ndarray:
    """values / positions: [shards, bags, dim] from max_with_positions -> the whole-table max
    [bags, dim] fp32: the greater value, the earlier position among equal values, a NaN partial
    (which exists only where the NaN was the bag's first entry) as is; 0 for a bag without rows."""
    best = np.zeros(values.shape[1:], dtype=np.float32)
    bpos = np.full(values.shape[1:], NO_POS, dtype=np.int32)
    for v, p in zip(values, positions):
        have = p != NO_POS
        with np.errstate(invalid="ignore"):
            later = np.where(np.isnan(best), False,
                             np.where(np.isnan(v), True, (v > best) | ((v == best) & (p < bpos))))
        take = have & np.where(bpos == NO_POS, True, later)
        best = np.where(take, v, best)
        bpos = np.where(take, p, bpos)
    return best


def torch_pool(table, indices, offsets=None, *, mode: int = MODE_SUM, fixed_len: int = 0,
               per_sample_weights=None, include_last_offset: bool = False,
               padding_idx: int = -1, num_threads: int | None = None):
    """torch CPU EmbeddingBag on the same arguments; returns a torch tensor."""
    import torch
    import torch.nn.functional as F

    if num_threads:
        torch.set_num_threads(num_threads)
    t = torch.as_tensor(table)
    idx = torch.as_tensor(indices).reshape(-1).long()
    if fixed_len > 0:
        idx2 = idx.reshape(-1, fixed_len)
        off = None
    else:
        idx2 = idx
        off = torch.as_tensor(offsets).reshape(-1).long()
    psw = None
    if per_sample_weights is not None:
        psw = torch.as_tensor(per_sample_weights).to(t.dtype)
        if fixed_len > 0:
            psw = psw.reshape(-1, fixed_len)
    name = {MODE_SUM: "sum", MODE_MEAN: "mean", MODE_MAX: "max"}[mode]
    with torch.no_grad():
        return F.embedding_bag(idx2, t, off, mode=name, per_sample_weights=psw,
                               include_last_offset=include_last_offset,
                               padding_idx=None if padding_idx < 0 else padding_idx)
