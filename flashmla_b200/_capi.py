"""ctypes binding of libflashmla_b200.so (declarations: include/flashmla_b200.h).

The library is loaded lazily and loudly: there is no CPU or PyTorch fallback, a missing
or unloadable library raises.
"""
import ctypes
import os
import threading
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_int32, c_int64, c_longlong, c_size_t, c_void_p

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("FLASHMLA_B200_LIB") or os.path.join(_HERE, "libflashmla_b200.so")

MLA_MODE_DENSE_DECODE = 0
MLA_MODE_SPARSE_DECODE = 1

IMPL_AUTO, IMPL_PORTABLE, IMPL_TCGEN05 = 0, 1, 2
NOALLOC_MAX_ROWS = 32768
MLA_DTYPE_BF16, MLA_DTYPE_FP16 = 0, 1
ABI_VERSION = 2


class SchedMetaArgs(Structure):
    _fields_ = [
        ("b", c_int32), ("s_q", c_int32), ("block_size_n", c_int32), ("fixed_overhead_num_blocks", c_int32),
        ("topk", c_int32), ("extra_topk", c_int32),
        ("topk_length", c_void_p), ("extra_topk_length", c_void_p), ("seqlens_k", c_void_p),
        ("meta", c_void_p), ("num_splits", c_void_p), ("num_sm_parts", c_int32), ("stream", c_void_p),
    ]


class DenseDecodeArgs(Structure):
    _fields_ = [
        ("b", c_int32), ("s_q", c_int32), ("h_q", c_int32), ("h_kv", c_int32),
        ("d_qk", c_int32), ("d_v", c_int32), ("num_blocks", c_int32), ("page_block_size", c_int32),
        ("is_causal", c_int32), ("softmax_scale", c_float),
        ("q", c_void_p), ("q_stride_b", c_int64), ("q_stride_s", c_int64), ("q_stride_h", c_int64),
        ("k_cache", c_void_p), ("k_stride_block", c_int64), ("k_stride_row", c_int64), ("k_stride_head", c_int64),
        ("block_table", c_void_p), ("block_table_stride_b", c_int64), ("max_blocks_per_seq", c_int32),
        ("seqlens_k", c_void_p),
        ("out", c_void_p), ("o_stride_b", c_int64), ("o_stride_s", c_int64), ("o_stride_h", c_int64),
        ("lse", c_void_p), ("lse_stride_b", c_int64), ("lse_stride_s", c_int64), ("lse_stride_h", c_int64),
        ("meta", c_void_p), ("num_splits", c_void_p), ("num_sm_parts", c_int32),
        ("lse_accum", c_void_p), ("o_accum", c_void_p),
        ("status", c_void_p), ("impl", c_int32), ("dtype", c_int32), ("stream", c_void_p),
    ]


class SparseDecodeArgs(Structure):
    _fields_ = [
        ("b", c_int32), ("s_q", c_int32), ("h_q", c_int32), ("d_qk", c_int32), ("d_v", c_int32), ("sm_scale", c_float),
        ("q", c_void_p), ("q_stride_b", c_int64), ("q_stride_s", c_int64), ("q_stride_h", c_int64),
        ("kv", c_void_p), ("kv_stride_block_bytes", c_int64), ("num_blocks", c_int32), ("page_block_size", c_int32),
        ("indices", c_void_p), ("indices_stride_b", c_int64), ("indices_stride_s", c_int64), ("topk", c_int32),
        ("topk_length", c_void_p),
        ("extra_kv", c_void_p), ("extra_kv_stride_block_bytes", c_int64), ("extra_num_blocks", c_int32),
        ("extra_page_block_size", c_int32),
        ("extra_indices", c_void_p), ("extra_indices_stride_b", c_int64), ("extra_indices_stride_s", c_int64),
        ("extra_topk", c_int32), ("extra_topk_length", c_void_p),
        ("attn_sink", c_void_p),
        ("out", c_void_p), ("o_stride_b", c_int64), ("o_stride_s", c_int64), ("o_stride_h", c_int64),
        ("lse", c_void_p), ("lse_stride_b", c_int64), ("lse_stride_s", c_int64), ("lse_stride_h", c_int64),
        ("meta", c_void_p), ("num_splits", c_void_p), ("num_sm_parts", c_int32),
        ("lse_accum", c_void_p), ("o_accum", c_void_p),
        ("status", c_void_p), ("impl", c_int32), ("stream", c_void_p),
    ]


class CombineArgs(Structure):
    _fields_ = [
        ("b", c_int32), ("s_q", c_int32), ("h_q", c_int32), ("d_v", c_int32),
        ("lse", c_void_p), ("lse_stride_b", c_int64), ("lse_stride_s", c_int64), ("lse_stride_h", c_int64),
        ("out", c_void_p), ("o_stride_b", c_int64), ("o_stride_s", c_int64), ("o_stride_h", c_int64),
        ("lse_accum", c_void_p), ("o_accum", c_void_p), ("num_splits", c_void_p), ("attn_sink", c_void_p),
        ("dtype", c_int32), ("_pad", c_int32), ("stream", c_void_p),
    ]


class SparsePrefillArgs(Structure):
    _fields_ = [
        ("s_q", c_int32), ("s_kv", c_int32), ("h_q", c_int32), ("h_kv", c_int32),
        ("d_qk", c_int32), ("d_v", c_int32), ("topk", c_int32), ("sm_scale", c_float),
        ("q", c_void_p), ("q_stride_s", c_int64), ("q_stride_h", c_int64),
        ("kv", c_void_p), ("kv_stride_s", c_int64), ("kv_stride_h", c_int64),
        ("indices", c_void_p), ("indices_stride_s", c_int64), ("indices_stride_h", c_int64),
        ("attn_sink", c_void_p), ("topk_length", c_void_p),
        ("out", c_void_p), ("max_logits", c_void_p), ("lse", c_void_p),
        ("status", c_void_p), ("impl", c_int32), ("stream", c_void_p),
    ]


class QuantizeArgs(Structure):
    _fields_ = [
        ("x", c_void_p), ("x_stride_block", c_int64), ("x_stride_row", c_int64),
        ("num_blocks", c_int32), ("block_size", c_int32),
        ("out", c_void_p), ("out_stride_block_bytes", c_int64),
        ("pow2_scale", c_int32), ("layout", c_int32), ("stream", c_void_p),
    ]


# every symbol include/flashmla_b200.h declares, with its signature
SYMBOLS = {
    "mla_last_error": (c_char_p, []),
    "mla_abi_version": (c_int, []),
    "mla_num_sm_parts": (c_int, [c_int, c_int, c_int, c_int, c_int]),
    "mla_num_sm_parts_uniform": (c_int, [c_int, c_int, c_int, c_int, c_int, c_int, c_int]),
    "mla_get_sched_meta": (c_int, [POINTER(SchedMetaArgs)]),
    "mla_dense_decode_fwd": (c_int, [POINTER(DenseDecodeArgs)]),
    "mla_sparse_decode_fwd": (c_int, [POINTER(SparseDecodeArgs)]),
    "mla_combine": (c_int, [POINTER(CombineArgs)]),
    "mla_sparse_prefill_fwd": (c_int, [POINTER(SparsePrefillArgs)]),
    "mla_dense_decode_noalloc": (c_int, [POINTER(DenseDecodeArgs)]),
    "mla_quantize_fp8_kvcache": (c_int, [POINTER(QuantizeArgs)]),
    "mla_workspace_bytes": (c_size_t, [c_int, c_int, c_int, c_int, c_int, POINTER(c_size_t)]),
    "mla_selftest_bounded_wait": (c_int, [c_longlong, c_int, c_void_p, c_void_p, c_void_p]),
}

_lib = None
_lock = threading.Lock()


def lib():
    """The loaded library; raises if it has not been built (python -m flashmla_b200.build)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                if not os.path.exists(LIB_PATH):
                    raise RuntimeError(
                        f"{LIB_PATH} is missing: build it with `python -m flashmla_b200.build` "
                        "(there is no CPU fallback)")
                handle = ctypes.CDLL(LIB_PATH)
                for name, (restype, argtypes) in SYMBOLS.items():
                    fn = getattr(handle, name)
                    fn.restype = restype
                    fn.argtypes = argtypes
                if handle.mla_abi_version() != ABI_VERSION:
                    raise RuntimeError(f"{LIB_PATH} has ABI version {handle.mla_abi_version()}, this package needs "
                                       f"{ABI_VERSION}: rebuild it with `python -m flashmla_b200.build --force`")
                _lib = handle
    return _lib


def check(rc: int, what: str):
    if rc != 0:
        msg = lib().mla_last_error().decode("utf-8", "replace")
        raise RuntimeError(f"{what} failed (code {rc}): {msg}")


def ptr(t):
    """Device pointer of a torch tensor (or None)."""
    return None if t is None else c_void_p(t.data_ptr())
