"""ctypes binding of libfstattn_b200.so (the C ABI declared in include/fstattn_b200.h).

There is no fallback: if the library has not been built, loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libfstattn_b200.so")

FST_OK = 0
STATUS_WORDS = 4
DTYPE_F16, DTYPE_BF16, DTYPE_F32 = 0, 1, 2
KERNEL_FLAG_META_STABLE = 0x100
KERNELS = {"auto": 0, "simt": 1, "mma": 2, "tma": 3, "tma_t32": 4, "tma_t64": 5,
           "tma_umma": 6, "persist": 7}
DEV_MALFORMED_TREE, DEV_ANCESTOR_OVERFLOW, DEV_INDEX_RANGE = 16, 17, 18

# every symbol include/fstattn_b200.h declares
EXPORTS = ("fst_version", "fst_status_string", "fst_packed_meta_bytes", "fst_precompute",
           "fst_pack_metadata", "fst_attention_fwd", "fst_attention_ref_workspace_bytes",
           "fst_attention_fwd_ref", "fst_attention_fwd_ref_static",
           "fst_attention_split_workspace_bytes", "fst_attention_fwd_splitkv", "fst_attention_fwd_gqa", "fst_dfs_order",
           "fst_attention_fwd_paged", "fst_selftest_wait_timeout", "fst_tree_topk_nodes",
           "fst_build_tree_topk", "fst_attention_fwd_scatter")
STATIC_SCRATCH_BYTES = 512 * 1024

_lib = None

_i, _i64, _sz, _p, _f = C.c_int, C.c_int64, C.c_size_t, C.c_void_p, C.c_float
_TENSOR_STRIDES = [_i64] * 12


def _declare(lib):
    lib.fst_version.restype = _i
    lib.fst_version.argtypes = []
    lib.fst_status_string.restype = C.c_char_p
    lib.fst_status_string.argtypes = [_i]
    lib.fst_packed_meta_bytes.restype = _sz
    lib.fst_packed_meta_bytes.argtypes = [_i, _i, _i]
    lib.fst_precompute.restype = _i
    lib.fst_precompute.argtypes = [_p, _i, _i, _i, _i, _p, _p, _p, _p, _sz, _p, _p]
    lib.fst_pack_metadata.restype = _i
    lib.fst_pack_metadata.argtypes = [_p, _p, _p, _i, _i, _i, _i, _i64, _p, _sz, _p, _p]
    lib.fst_attention_fwd.restype = _i
    lib.fst_attention_fwd.argtypes = ([_p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _i, _i]
                                      + _TENSOR_STRIDES + [_i, _i, _f, _i, _i, _p, _p])
    lib.fst_attention_fwd_scatter.restype = _i
    lib.fst_attention_fwd_scatter.argtypes = ([_p, _p, _p, _p, _i, _i, _i, _i, _i, _i, _p, _p, _sz, _i, _i, _i, _i, _i]
                                              + _TENSOR_STRIDES + [_i, _i, _f, _i, _i, _p, _p])
    lib.fst_attention_split_workspace_bytes.restype = _sz
    lib.fst_attention_split_workspace_bytes.argtypes = [_i, _i, _i, _i, _i]
    lib.fst_attention_fwd_splitkv.restype = _i
    lib.fst_attention_fwd_splitkv.argtypes = ([_p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _i, _i]
                                              + _TENSOR_STRIDES + [_i, _i, _f, _i, _i, _i, _p, _sz, _p, _p])
    lib.fst_selftest_wait_timeout.restype = _i
    lib.fst_selftest_wait_timeout.argtypes = [_p, _p, _p]
    lib.fst_tree_topk_nodes.restype = C.c_longlong
    lib.fst_tree_topk_nodes.argtypes = [_i, _i, C.c_double]
    lib.fst_build_tree_topk.restype = _i
    lib.fst_build_tree_topk.argtypes = [_p, _i, _i, _i, C.c_double, _i, _p, _p, _p, _p]
    lib.fst_dfs_order.restype = _i
    lib.fst_dfs_order.argtypes = [_p, _i, _i, _p, _p, _p, _p]
    lib.fst_attention_fwd_paged.restype = _i
    lib.fst_attention_fwd_paged.argtypes = ([_p, _p, _p, _p, _p, _p, _sz, _p, _p, _p, _i, _p, _i, _i, _i,
                                             _i64, _i64, _i64, _i, _i, _i, _i, _i]
                                            + _TENSOR_STRIDES + [_i, _i, _f, _i, _i, _p, _sz, _p, _p])
    lib.fst_attention_fwd_gqa.restype = _i
    lib.fst_attention_fwd_gqa.argtypes = ([_p, _p, _p, _p, _p, _p, _sz, _i, _i, _i, _i, _i, _i]
                                          + _TENSOR_STRIDES + [_i, _i, _f, _i, _i, _i, _p, _sz, _p, _p])
    lib.fst_attention_ref_workspace_bytes.restype = _sz
    lib.fst_attention_ref_workspace_bytes.argtypes = [_i, _i, _i, _i]
    lib.fst_attention_fwd_ref.restype = _i
    lib.fst_attention_fwd_ref.argtypes = ([_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i]
                                          + _TENSOR_STRIDES
                                          + [_i, _i, _f, _i, _i, _p, _sz, _p, _p])
    lib.fst_attention_fwd_ref_static.restype = _i
    lib.fst_attention_fwd_ref_static.argtypes = ([_p, _p, _p, _p, _p, _p, _p, _p, _i, _i, _i, _i, _i, _i]
                                                 + _TENSOR_STRIDES + [_i, _i, _f, _i, _i, _p, _p])


def lib():
    """The loaded library; raises RuntimeError when it is missing (build it first)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: the CUDA extension is not built. Run "
                "`python -m fstattention_b200.build` (needs nvcc). There is no CPU fallback.")
        loaded = C.CDLL(LIB_PATH)
        _declare(loaded)
        _lib = loaded
    return _lib


def status_string(code: int) -> str:
    return lib().fst_status_string(int(code)).decode()


def check(rc: int, what: str):
    if rc != FST_OK:
        raise RuntimeError(f"{what}: {status_string(rc)} (status {rc})")
