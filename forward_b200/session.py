"""Python face of the host-buffer session API (include/fwd_eb_session.h).

`Session` keeps a table resident on one GPU and runs EmbeddingBag calls whose inputs and
results live in host memory, with `depth` calls in flight.  numpy views of the pinned
staging slots are exposed so a caller can fill inputs in place.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import capi


class SessionConfig(C.Structure):
    """Mirror of struct fwd_eb_session_config."""
    _fields_ = [
        ("table_dtype", C.c_int32), ("dim", C.c_int32), ("num_rows", C.c_int64),
        ("row_lo", C.c_int64), ("mode", C.c_int32), ("out_dtype", C.c_int32),
        ("index_dtype", C.c_int32), ("include_last_offset", C.c_int32),
        ("padding_idx", C.c_int64), ("fixed_len", C.c_int32), ("weighted", C.c_int32),
        ("max_indices", C.c_int64), ("max_bags", C.c_int64), ("depth", C.c_int32),
        ("device", C.c_int32), ("flags", C.c_uint32), ("external_table", C.c_int32),
    ]


SIGNATURES = {
    "fwd_eb_session_create": (C.c_int, [C.POINTER(SessionConfig), C.POINTER(C.c_void_p)]),
    "fwd_eb_session_destroy": (None, [C.c_void_p]),
    "fwd_eb_session_load_table": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_int64]),
    "fwd_eb_session_device_table": (C.c_void_p, [C.c_void_p]),
    "fwd_eb_session_adopt_table": (C.c_int, [C.c_void_p, C.c_void_p]),
    "fwd_eb_session_slot": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_void_p),
                                      C.POINTER(C.c_void_p), C.POINTER(C.c_void_p),
                                      C.POINTER(C.c_void_p)]),
    "fwd_eb_session_submit": (C.c_int, [C.c_void_p, C.c_int32, C.c_int64, C.c_int64]),
    "fwd_eb_session_wait": (C.c_int, [C.c_void_p, C.c_int32]),
    "fwd_eb_session_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64,
                                     C.c_void_p, C.c_void_p]),
    "fwd_eb_session_copy_bytes": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64,
                                            C.POINTER(C.c_int64), C.POINTER(C.c_int64)]),
}

_bound = False


def _lib():
    global _bound
    lib = capi.lib()
    if not _bound:
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _bound = True
    return lib


_NP_F = {capi.F32: np.float32, capi.F16: np.float16}
_NP_I = {capi.I32: np.int32, capi.I64: np.int64}


def _view(ptr, count, dtype):
    if not ptr or count <= 0:
        return None
    nbytes = int(count) * np.dtype(dtype).itemsize
    buf = (C.c_char * nbytes).from_address(ptr)
    return np.frombuffer(buf, dtype=dtype, count=int(count))


class Session:
    def __init__(self, *, table_dtype, dim, num_rows, mode, max_indices, max_bags, row_lo=0,
                 out_dtype=None, index_dtype=capi.I32, include_last_offset=False, padding_idx=-1,
                 fixed_len=0, weighted=False, depth=4, device=-1, flags=0, external_table=False):
        cfg = SessionConfig()
        cfg.table_dtype = table_dtype
        cfg.dim = dim
        cfg.num_rows = num_rows
        cfg.row_lo = row_lo
        cfg.mode = mode
        cfg.out_dtype = table_dtype if out_dtype is None else out_dtype
        cfg.index_dtype = index_dtype
        cfg.include_last_offset = int(include_last_offset)
        cfg.padding_idx = padding_idx
        cfg.fixed_len = fixed_len
        cfg.weighted = int(weighted)
        cfg.max_indices = max_indices
        cfg.max_bags = max_bags
        cfg.depth = depth
        cfg.device = device
        cfg.flags = flags
        cfg.external_table = int(external_table)
        self.cfg = cfg
        self._h = C.c_void_p()
        capi.check(_lib().fwd_eb_session_create(C.byref(cfg), C.byref(self._h)))
        self.depth = depth

    def close(self):
        if self._h:
            _lib().fwd_eb_session_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    @property
    def device_table_ptr(self) -> int:
        return _lib().fwd_eb_session_device_table(self._h) or 0

    def load_table(self, rows: np.ndarray, first_row: int = 0) -> None:
        rows = np.ascontiguousarray(rows, dtype=_NP_F[self.cfg.table_dtype])
        capi.check(_lib().fwd_eb_session_load_table(self._h, rows.ctypes.data, first_row,
                                                    rows.shape[0]))

    def adopt_table(self, device_ptr: int) -> None:
        capi.check(_lib().fwd_eb_session_adopt_table(self._h, C.c_void_p(device_ptr)))

    def slot(self, k: int):
        """numpy views (indices, offsets, weights, out) over slot k's pinned buffers."""
        pi, po, pw, pout = C.c_void_p(), C.c_void_p(), C.c_void_p(), C.c_void_p()
        capi.check(_lib().fwd_eb_session_slot(self._h, k, C.byref(pi), C.byref(po), C.byref(pw),
                                              C.byref(pout)))
        c = self.cfg
        it, ot = _NP_I[c.index_dtype], _NP_F[c.out_dtype]
        n_off = 0 if (c.fixed_len > 0 or c.mode == capi.MODE_GATHER) else c.max_bags + c.include_last_offset
        out_rows = c.max_indices if c.mode == capi.MODE_GATHER else c.max_bags
        out = _view(pout.value, out_rows * c.dim, ot)
        return (_view(pi.value, c.max_indices, it), _view(po.value, n_off, it),
                _view(pw.value, c.max_indices if c.weighted else 0, np.float32),
                None if out is None else out.reshape(out_rows, c.dim))

    def submit(self, k: int, num_indices: int, num_bags: int) -> None:
        capi.check(_lib().fwd_eb_session_submit(self._h, k, num_indices, num_bags))

    def wait(self, k: int) -> None:
        capi.check(_lib().fwd_eb_session_wait(self._h, k))

    def copy_bytes(self, num_indices: int, num_bags: int):
        a, b = C.c_int64(), C.c_int64()
        capi.check(_lib().fwd_eb_session_copy_bytes(self._h, num_indices, num_bags, C.byref(a),
                                                    C.byref(b)))
        return a.value, b.value

    def run(self, indices: np.ndarray, offsets: np.ndarray | None = None,
            per_sample_weights: np.ndarray | None = None) -> np.ndarray:
        """One blocking call on host arrays; returns a fresh host array."""
        c = self.cfg
        it = _NP_I[c.index_dtype]
        idx = np.ascontiguousarray(indices, dtype=it).reshape(-1)
        if c.mode == capi.MODE_GATHER:
            bags, rows = 0, idx.size
        elif c.fixed_len > 0:
            bags = idx.size // c.fixed_len
            rows = bags
        else:
            offsets = np.ascontiguousarray(offsets, dtype=it).reshape(-1)
            bags = offsets.size - c.include_last_offset
            rows = bags
        out = np.empty((rows, c.dim), dtype=_NP_F[c.out_dtype])
        w = None
        if c.weighted:
            w = np.ascontiguousarray(per_sample_weights, dtype=np.float32)
        capi.check(_lib().fwd_eb_session_run(
            self._h, idx.ctypes.data, idx.size,
            None if offsets is None else offsets.ctypes.data, bags,
            None if w is None else w.ctypes.data, out.ctypes.data))
        return out
