"""ctypes front for oracle/_ref/libref_eb.so: the reference's own EmbeddingBag kernels
(embedding_bag_plugin.cu:66-206), compiled unmodified for sm_100a by oracle/build_ref.py.

TEST INFRASTRUCTURE: used by the GPU parity tests and by bench.py's side-by-side timing; absent
on machines where the reference tree was never mounted, in which case `available()` is False."""
from __future__ import annotations

import ctypes as C
import os

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "libref_eb.so")
_lib = None


def available() -> bool:
    return os.path.exists(_PATH)


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(_PATH)
        _lib.ref_eb_bag.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                    C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        _lib.ref_eb_bag_fixed.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,
                                          C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p]
        _lib.ref_eb_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                       C.c_int, C.c_int, C.c_void_p]
    return _lib


def _check_offsets(offsets, num_indices: int) -> None:
    """The reference kernels trust their offsets (embedding_bag_plugin.cu:80-86 reads
    input[offset[b] .. offset[b+1]) unguarded): refuse on the host what would read out of bounds.
    Costs a device-to-host copy; this front is test infrastructure, not a hot path."""
    off = offsets.reshape(-1)
    if off.numel() == 0:
        return
    bad = bool((off < 0).any() or (off > num_indices).any() or (off[1:] < off[:-1]).any())
    if bad:
        raise ValueError("offsets must be non-decreasing and inside [0, num_indices] for the "
                         "reference kernels, which do not check them")


def bag(indices, offsets, out, table, data_offset: int, op: int, stream: int, check: bool = True) -> None:
    """torch CUDA tensors: int32 indices/offsets, fp32 table and output.  `check=False` skips the
    host-side offsets check (it synchronises) for inputs that an earlier call has checked."""
    if check:
        _check_offsets(offsets, indices.numel())
    rc = lib().ref_eb_bag(indices.data_ptr(), offsets.data_ptr(), out.data_ptr(), indices.numel(),
                          offsets.numel(), table.data_ptr(), table.shape[0], table.shape[1],
                          data_offset, op, C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"reference EmbeddingBag launch failed: cudaError {rc}")


def bag_fixed(indices2d, out, table, data_offset: int, op: int, stream: int) -> None:
    rc = lib().ref_eb_bag_fixed(indices2d.data_ptr(), out.data_ptr(), indices2d.shape[0],
                                indices2d.shape[1], table.data_ptr(), table.shape[0],
                                table.shape[1], data_offset, op, C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"reference EmbeddingBagWithFixedOffset launch failed: cudaError {rc}")


def gather(indices2d, out, table, data_offset: int, stream: int) -> None:
    # The reference GatherKernel addresses data[input_id * dim + pos] without subtracting
    # data_offset (embedding_bag_plugin.cu:178): with a non-zero data_offset every in-window
    # index reads past the end of the shard.  That launch is never made from here.
    if data_offset != 0:
        raise ValueError("the reference GatherKernel reads out of bounds for data_offset != 0 "
                         "(embedding_bag_plugin.cu:178); only data_offset == 0 is run")
    rc = lib().ref_eb_gather(indices2d.data_ptr(), out.data_ptr(), indices2d.shape[0],
                             indices2d.shape[1], table.data_ptr(), table.shape[0], table.shape[1],
                             data_offset, C.c_void_p(stream))
    if rc:
        raise RuntimeError(f"reference Gather launch failed: cudaError {rc}")
