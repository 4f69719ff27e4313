"""ctypes binding of libfdma_sm100.so (declarations: include/fdma.h).

The shared library is the only compute backend of this package. If it is missing, importing this module
raises: there is no PyTorch or CPU fallback behind the operator API.
"""
import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FDMA_LIB", os.path.join(_HERE, "lib", "libfdma_sm100.so"))

FDMA_BF16, FDMA_FP16, FDMA_FP32 = 0, 1, 2
PATH_AUTO, PATH_SIMT, PATH_TCGEN05, PATH_DECODE = 0, 1, 2, 3
MASK_TOPK, MASK_RELU = 0, 1
ERR_UNSUPPORTED = -2


class FwdParams(Structure):
    _fields_ = (
        [(n, c_void_p) for n in ("q", "k", "v", "mask", "bias", "out", "lse")]
        + [(f"{t}_{s}_stride", c_int64) for t in ("q", "k", "v", "o") for s in ("batch", "row", "head")]
        + [(f"{t}_{s}_stride", c_int64) for t in ("mask", "bias") for s in ("batch", "head", "row")]
        + [(n, c_int32) for n in ("b", "seqlen_q", "seqlen_k", "h", "h_k", "h_mask", "h_bias", "d")]
        + [("dtype", c_int32), ("is_causal", c_int32), ("softmax_scale", c_float), ("path", c_int32)]
        + [("workspace", c_void_p), ("workspace_bytes", c_size_t)]
        + [("key_pos", c_void_p), ("key_pos_batch_stride", c_int64), ("key_pos_head_stride", c_int64)]
        + [("h_pos", c_int32), ("causal_shift", c_int32)]
        + [("mask_bits", c_int32), ("reserved", c_int32), ("tile_activity", c_void_p)]
    )


class BwdParams(Structure):
    _fields_ = (
        [("f", FwdParams), ("dout", c_void_p)]
        + [(f"do_{s}_stride", c_int64) for s in ("batch", "row", "head")]
        + [(n, c_void_p) for n in ("dq", "dk", "dv", "dbias")]
        + [(f"{t}_{s}_stride", c_int64) for t in ("dq", "dk", "dv") for s in ("batch", "row", "head")]
        + [(f"dbias_{s}_stride", c_int64) for s in ("batch", "head", "row")]
        + [(n, c_int32) for n in ("dbias_b", "dbias_h", "dbias_rows", "dbias_keys", "deterministic", "reserved")]
        + [("softmax_d", c_void_p)]
    )


class MaskParams(Structure):
    _fields_ = (
        [(n, c_void_p) for n in ("bias", "premask", "out")]
        + [(f"bias_{s}_stride", c_int64) for s in ("batch", "head", "row")]
        + [(f"pm_{s}_stride", c_int64) for s in ("batch", "head", "row")]
        + [(n, c_int32) for n in ("out_b", "out_h", "out_rows", "keys", "window", "dtype", "kind", "block_size")]
        + [("min_value", c_float)]
        + [("key_pos", c_void_p), ("count", c_void_p), ("slot_mask", c_void_p), ("capacity", c_int32), ("reserved", c_int32)]
        + [("bits", c_void_p), ("activity", c_void_p)]
    )


# Every symbol include/fdma.h declares; tests check that the library exports each of them.
EXPORTED_SYMBOLS = (
    "fdma_version",
    "fdma_strerror",
    "fdma_fwd_workspace_bytes",
    "fdma_fwd",
    "fdma_bwd_workspace_bytes",
    "fdma_bwd",
    "fdma_create_mask",
    "fdma_last_kernel_status",
    "fdma_poll_kernel_status",
    "fdma_selftest_wait_timeout",
    "fdma_time_next_kernel",
    "fdma_fwd_static_scratch",
    "fdma_static_scratch_limit",
    "fdma_compact_index",
    "fdma_gather_rows",
    "fdma_scatter_rows",
    "fdma_merge_partials",
)



class CompactParams(ctypes.Structure):
    """fdma_compact_params of include/fdma.h."""

    _fields_ = [
        ("mask", c_void_p), ("mask_batch_stride", c_int64), ("mask_head_stride", c_int64),
        ("b_mask", c_int32), ("h_mask", c_int32), ("seqlen_k", c_int32), ("capacity", c_int32),
        ("key_pos", c_void_p), ("count", c_void_p), ("mask_out", c_void_p),
    ]


class RowsParams(ctypes.Structure):
    """fdma_rows_params of include/fdma.h."""

    _fields_ = [
        ("src", c_void_p), ("dst", c_void_p), ("key_pos", c_void_p),
        ("key_pos_batch_stride", c_int64), ("key_pos_head_stride", c_int64),
        ("src_batch_stride", c_int64), ("src_row_stride", c_int64), ("src_head_stride", c_int64),
        ("dst_batch_stride", c_int64), ("dst_row_stride", c_int64), ("dst_head_stride", c_int64),
        ("b", c_int32), ("heads", c_int32), ("h_pos", c_int32), ("rows_full", c_int32),
        ("capacity", c_int32), ("row_elems", c_int32), ("dtype", c_int32), ("reserved_", c_int32),
    ]


class MergeParams(ctypes.Structure):
    """fdma_merge_params of include/fdma.h."""

    _fields_ = [
        ("acc", c_void_p), ("lse_acc", c_void_p), ("part", c_void_p), ("lse_part", c_void_p),
        ("part_batch_stride", c_int64), ("part_row_stride", c_int64), ("part_head_stride", c_int64),
        ("b", c_int32), ("seqlen_q", c_int32), ("h", c_int32), ("d", c_int32), ("dtype", c_int32), ("reserved", c_int32),
    ]


_lib = None


def load():
    """Loads the library once and sets the ctypes prototypes. Raises OSError/RuntimeError if unavailable."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"libfdma_sm100.so not found at {LIB_PATH}: build it with `make -C flash-dmattn_b200/csrc` "
            "(this package has no fallback implementation)"
        )
    lib = ctypes.CDLL(LIB_PATH)
    lib.fdma_version.restype = c_int
    lib.fdma_strerror.restype = c_char_p
    lib.fdma_strerror.argtypes = [c_int]
    lib.fdma_fwd_workspace_bytes.restype = c_size_t
    lib.fdma_fwd_workspace_bytes.argtypes = [POINTER(FwdParams)]
    lib.fdma_fwd.restype = c_int
    lib.fdma_fwd.argtypes = [POINTER(FwdParams), c_void_p]
    lib.fdma_bwd_workspace_bytes.restype = c_size_t
    lib.fdma_bwd_workspace_bytes.argtypes = [POINTER(BwdParams)]
    lib.fdma_bwd.restype = c_int
    lib.fdma_bwd.argtypes = [POINTER(BwdParams), c_void_p]
    lib.fdma_create_mask.restype = c_int
    lib.fdma_create_mask.argtypes = [POINTER(MaskParams), c_void_p]
    lib.fdma_last_kernel_status.restype = c_int
    lib.fdma_last_kernel_status.argtypes = [c_void_p, POINTER(c_int32)]
    lib.fdma_poll_kernel_status.restype = c_int
    lib.fdma_poll_kernel_status.argtypes = [POINTER(c_int32)]
    lib.fdma_selftest_wait_timeout.restype = c_int
    lib.fdma_selftest_wait_timeout.argtypes = [ctypes.c_uint32, c_void_p, c_void_p]
    lib.fdma_fwd_static_scratch.restype = c_int
    lib.fdma_fwd_static_scratch.argtypes = [POINTER(FwdParams), c_void_p]
    lib.fdma_static_scratch_limit.restype = c_size_t
    lib.fdma_compact_index.restype = c_int
    lib.fdma_compact_index.argtypes = [POINTER(CompactParams), c_void_p]
    lib.fdma_gather_rows.restype = c_int
    lib.fdma_gather_rows.argtypes = [POINTER(RowsParams), c_void_p]
    lib.fdma_scatter_rows.restype = c_int
    lib.fdma_scatter_rows.argtypes = [POINTER(RowsParams), c_void_p]
    lib.fdma_merge_partials.restype = c_int
    lib.fdma_merge_partials.argtypes = [POINTER(MergeParams), c_void_p]
    lib.fdma_time_next_kernel.restype = None
    lib.fdma_time_next_kernel.argtypes = [c_void_p, c_void_p]
    _lib = lib
    return lib


def check(status: int, what: str):
    """Turns a non-zero status into the RuntimeError the reference's TORCH_CHECKs would raise."""
    if status != 0:
        msg = load().fdma_strerror(int(status)).decode()
        raise RuntimeError(f"{what} failed: {msg} (status {status})")
