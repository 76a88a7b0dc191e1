"""ctypes binding of ``libarc_sdpa.so`` (the C ABI declared in ``include/arc_sdpa.h``).

There is no fallback: if the library is missing or cannot be loaded, importing
the operators raises.  ``torch`` must be imported first so the process already
holds the CUDA runtime the library links against.
"""
from __future__ import annotations

import ctypes as C
import os

import torch  # noqa: F401  (loads libcudart.so.12 into the process)

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libarc_sdpa.so")

ARC_OK = 0
ARC_ERR_BAD_SHAPE = 1
ARC_ERR_ALIGNMENT = 2
ARC_ERR_UNSUPPORTED_HEAD_DIM = 3
ARC_ERR_WORKSPACE_TOO_SMALL = 4
ARC_ERR_CUDA = 5
ARC_ERR_COLLECTIVE = 6
ARC_ERR_DEVICE_WAIT_TIMEOUT = 7
ARC_ERR_NULL_POINTER = 8
ARC_ERR_UNSUPPORTED_GQA = 9
ARC_ERR_TOO_LARGE = 10
ARC_ERR_DEVICE_BAD_RANGE = 11

MASK_NONE = 0
MASK_EXPLICIT = 1
MASK_CAUSAL = 3
NO_WINDOW = 2**31 - 1
STATIC_SCRATCH_BYTES = 8 << 20

EXPORTS = (
    "arc_sdpa_status_string", "arc_sdpa_last_error", "arc_sdpa_prefill_workspace_bytes", "arc_sdpa_prefill",
    "arc_sdpa_decode_workspace_bytes", "arc_sdpa_decode", "arc_sdpa_decode_static", "arc_sdpa_exchange_bytes", "arc_sdpa_merge", "arc_mul_sigmoid_inplace",
    "arc_fill_causal_mask", "arc_fill_causal_mask_with_block_ids", "arc_qkv_prepare", "arc_sdpa_device_status", "arc_sdpa_clear_device_status", "arc_sdpa_launch_count",
    "arc_plan_head_shards", "arc_plan_seq_shards", "arc_plan_batch_shards", "arc_sdpa_exchange_init", "arc_sdpa_record_floats",
    "arc_sdpa_allgather_merge",
)


class PrefillParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p),
        ("gate", C.c_void_p), ("mask", C.c_void_p), ("out_lse", C.c_void_p),
        ("batch", C.c_int32), ("seq", C.c_int32), ("kv_len", C.c_int32),
        ("nq", C.c_int32), ("nkv", C.c_int32), ("hd", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64),
        ("k_stride_b", C.c_int64), ("k_stride_t", C.c_int64),
        ("v_stride_b", C.c_int64), ("v_stride_t", C.c_int64),
        ("o_stride_b", C.c_int64), ("o_stride_t", C.c_int64),
        ("scale", C.c_float), ("mask_type", C.c_int32), ("window", C.c_int32), ("num_splits", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("block_ids", C.c_void_p), ("block_ids_offset", C.c_int32),
        ("out_copies", C.c_void_p), ("out_copy_count", C.c_int32),
    ]


class DecodeParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("out", C.c_void_p), ("gate", C.c_void_p),
        ("kv_len", C.c_void_p), ("kv_row_offset", C.c_void_p), ("out_f32", C.c_void_p), ("out_lse", C.c_void_p),
        ("batch", C.c_int32), ("nq", C.c_int32), ("nkv", C.c_int32), ("hd", C.c_int32),
        ("kv_len_uniform", C.c_int32), ("max_kv_len", C.c_int32),
        ("q_stride_b", C.c_int64), ("o_stride_b", C.c_int64), ("kv_stride_b", C.c_int64), ("kv_stride_t", C.c_int64), ("kv_rows_total", C.c_int64),
        ("scale", C.c_float), ("num_ctas", C.c_int32),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("xchg_peers", C.c_void_p), ("xchg_world", C.c_int32), ("xchg_rank", C.c_int32), ("xchg_step", C.c_uint32),
        ("xchg_wait_cycles", C.c_int64),
    ]


class HeadShard(C.Structure):
    _fields_ = [("kv_head_begin", C.c_int32), ("kv_head_end", C.c_int32), ("q_head_begin", C.c_int32),
                ("q_head_end", C.c_int32), ("batch_begin", C.c_int32), ("batch_end", C.c_int32)]


class QkvPrepareParams(C.Structure):
    _fields_ = [
        ("q", C.c_void_p), ("k_src", C.c_void_p), ("v_src", C.c_void_p), ("k_dst", C.c_void_p), ("v_dst", C.c_void_p),
        ("q_weight", C.c_void_p), ("k_weight", C.c_void_p), ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p),
        ("pos_offset", C.c_void_p),
        ("batch", C.c_int32), ("seq", C.c_int32), ("nq", C.c_int32), ("nkv", C.c_int32), ("hd", C.c_int32),
        ("n_active_pairs", C.c_int32),
        ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64),
        ("k_src_stride_b", C.c_int64), ("k_src_stride_t", C.c_int64),
        ("v_src_stride_b", C.c_int64), ("v_src_stride_t", C.c_int64),
        ("k_dst_stride_b", C.c_int64), ("k_dst_stride_t", C.c_int64),
        ("v_dst_stride_b", C.c_int64), ("v_dst_stride_t", C.c_int64),
        ("rope_stride_b", C.c_int64),
        ("pos0", C.c_int32), ("theta", C.c_float), ("eps", C.c_float),
        ("rot_half", C.c_int32), ("freq_denom", C.c_int32), ("mrope_positions", C.c_void_p),
        ("mrope_section", C.c_int32 * 3), ("v_copy", C.c_int32),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the library and declare every exported signature."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m arcaine_b200.build` "
            "(there is no CPU or PyTorch fallback for these operators)")
    L = C.CDLL(LIB_PATH)
    vp = C.c_void_p
    L.arc_sdpa_status_string.restype = C.c_char_p
    L.arc_sdpa_status_string.argtypes = [C.c_int]
    L.arc_sdpa_last_error.restype = C.c_char_p
    L.arc_sdpa_last_error.argtypes = []
    L.arc_sdpa_prefill_workspace_bytes.restype = C.c_size_t
    L.arc_sdpa_prefill_workspace_bytes.argtypes = [C.POINTER(PrefillParams)]
    L.arc_sdpa_prefill.restype = C.c_int
    L.arc_sdpa_prefill.argtypes = [C.POINTER(PrefillParams), vp]
    L.arc_sdpa_decode_workspace_bytes.restype = C.c_size_t
    L.arc_sdpa_decode_workspace_bytes.argtypes = [C.POINTER(DecodeParams)]
    L.arc_sdpa_decode.restype = C.c_int
    L.arc_sdpa_decode.argtypes = [C.POINTER(DecodeParams), vp]
    L.arc_sdpa_exchange_bytes.restype = C.c_size_t
    L.arc_sdpa_exchange_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32]
    L.arc_sdpa_decode_static.restype = C.c_int
    L.arc_sdpa_decode_static.argtypes = [C.POINTER(DecodeParams), vp]
    L.arc_sdpa_merge.restype = C.c_int
    L.arc_sdpa_merge.argtypes = [vp, vp, C.c_int32, C.c_int64, C.c_int32, C.c_int64, C.c_int64, vp, vp, vp, vp, vp]
    L.arc_mul_sigmoid_inplace.restype = C.c_int
    L.arc_mul_sigmoid_inplace.argtypes = [vp, vp, C.c_int64, vp]
    L.arc_fill_causal_mask.restype = C.c_int
    L.arc_fill_causal_mask.argtypes = [vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp]
    L.arc_fill_causal_mask_with_block_ids.restype = C.c_int
    L.arc_fill_causal_mask_with_block_ids.argtypes = [vp, vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp]
    L.arc_qkv_prepare.restype = C.c_int
    L.arc_qkv_prepare.argtypes = [C.POINTER(QkvPrepareParams), vp]
    L.arc_sdpa_device_status.restype = C.c_int
    L.arc_sdpa_device_status.argtypes = [C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
    L.arc_sdpa_clear_device_status.restype = C.c_int
    L.arc_sdpa_clear_device_status.argtypes = []
    L.arc_sdpa_launch_count.restype = C.c_uint64
    L.arc_sdpa_launch_count.argtypes = []
    L.arc_plan_head_shards.restype = C.c_int
    L.arc_plan_head_shards.argtypes = [C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(HeadShard)]
    L.arc_plan_seq_shards.restype = C.c_int
    L.arc_plan_seq_shards.argtypes = [C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64)]
    L.arc_plan_batch_shards.restype = C.c_int
    L.arc_plan_batch_shards.argtypes = [C.POINTER(C.c_int32), C.c_int32, C.c_int32, C.POINTER(C.c_int32)]
    L.arc_sdpa_exchange_init.restype = C.c_int
    L.arc_sdpa_exchange_init.argtypes = [vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.POINTER(C.c_uint64), vp, vp]
    L.arc_sdpa_record_floats.restype = C.c_size_t
    L.arc_sdpa_record_floats.argtypes = [C.c_int32, C.c_int32, C.c_int32]
    L.arc_sdpa_allgather_merge.restype = C.c_int
    L.arc_sdpa_allgather_merge.argtypes = [vp, vp, C.c_int32, C.c_int32, C.c_int32, C.c_int32, vp, vp, vp, vp]
    _lib = L
    return L


class ArcError(RuntimeError):
    """A C-ABI call returned a non-zero status (the reference throws std::runtime_error)."""

    def __init__(self, status: int, where: str):
        self.status = status
        msg = load().arc_sdpa_status_string(status).decode()
        detail = load().arc_sdpa_last_error().decode() if status == ARC_ERR_CUDA else ""
        super().__init__(f"{where}: {msg} (status {status})" + (f" [{detail}]" if detail else ""))


def check(status: int, where: str) -> None:
    if status != ARC_OK:
        raise ArcError(status, where)
