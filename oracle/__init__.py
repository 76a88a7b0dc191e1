"""CPU checker for the SDPA kernels (test infrastructure, never on the product path).

Thin ctypes bindings over ``sdpa_oracle.c`` plus one independent fp32
formulation written with torch CPU ops, used to cross-check the C code.
Parity with the reference itself is unpinned: it ships no attention tests or
golden vectors and cannot be built without a SYCL toolchain.

bf16 tensors are passed as torch CPU ``bfloat16`` tensors (or uint16 numpy
arrays holding the raw bits, the reference's own ``bf16 = uint16_t``
convention, src/common/gpu/buffer.hpp:8).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsdpa_oracle.so")
INT_MAX = 2**31 - 1

MASK_NONE = 0
MASK_EXPLICIT = 1
MASK_CAUSAL = 3


def build(force: bool = False) -> str:
    """Compile the C checker with the Makefile beside it."""
    src = os.path.join(_HERE, "sdpa_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libsdpa_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_LIB_PATH)
        c = ctypes
        vp, i32, i64, f32 = c.c_void_p, c.c_int, c.c_int64, c.c_float
        L.oracle_bf16_to_float.restype = f32
        L.oracle_bf16_to_float.argtypes = [c.c_uint16]
        L.oracle_float_to_bf16.restype = c.c_uint16
        L.oracle_float_to_bf16.argtypes = [f32]
        L.oracle_num_threads.restype = i32
        L.oracle_set_num_threads.restype = None
        L.oracle_set_num_threads.argtypes = [i32]
        L.oracle_lcg_fill.restype = None
        L.oracle_lcg_fill.argtypes = [vp, c.c_size_t, c.POINTER(c.c_uint32)]
        L.oracle_fill_causal_mask.restype = None
        L.oracle_fill_causal_mask.argtypes = [vp, i32, i32, i32, i32]
        L.oracle_fill_causal_mask_with_block_ids.restype = None
        L.oracle_fill_causal_mask_with_block_ids.argtypes = [vp, vp, i32, i32, i32, i32]
        L.oracle_mul_sigmoid_inplace.restype = None
        L.oracle_mul_sigmoid_inplace.argtypes = [vp, vp, c.c_size_t]
        L.oracle_norm_rope.restype = None
        L.oracle_norm_rope.argtypes = [vp, c.c_longlong, vp, c.c_longlong, vp, i32, i32, i32, i32, i32, f32, f32, vp, vp]
        L.oracle_mrope.restype = None
        L.oracle_mrope.argtypes = [vp, vp, i32, i32, i32, i32, f32, vp]
        L.oracle_sdpa_f32.restype = i32
        L.oracle_sdpa_f32.argtypes = [vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32,
                                      f32, vp, i64, vp, vp, vp]
        L.oracle_qwen35_online_attention.restype = i32
        L.oracle_qwen35_online_attention.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, i32, f32]
        L.oracle_gqa_attention.restype = i32
        L.oracle_gqa_attention.argtypes = [vp, i32, i32, i32, vp, vp, i32, i32, i32, i32, i32, vp]
        L.oracle_batched_attention.restype = i32
        L.oracle_batched_attention.argtypes = [vp, i32, i32, i32, vp, vp, i32, i32, i32, i32,
                                               f32, i32, vp]
        L.oracle_merge_partials.restype = None
        L.oracle_merge_partials.argtypes = [vp, vp, i32, i64, i32, vp, vp]
        _lib = L
    return _lib


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    lib().oracle_set_num_threads(int(n))


def _bits(t) -> np.ndarray:
    """Contiguous uint16 view of a bf16 tensor / uint16 array."""
    if isinstance(t, torch.Tensor):
        assert t.dtype == torch.bfloat16 and t.device.type == "cpu"
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    a = np.ascontiguousarray(t)
    assert a.dtype == np.uint16
    return a


def _ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def bits_to_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)


def float_to_bf16_bits(x: float) -> int:
    return int(lib().oracle_float_to_bf16(ctypes.c_float(x)))


def bf16_bits_to_float(b: int) -> float:
    return float(lib().oracle_bf16_to_float(ctypes.c_uint16(b)))


def lcg_fill(n: int, state: int) -> tuple[np.ndarray, int]:
    """Bench input recipe of src/bench/qwen35_attention_bench.cpp:86-94."""
    out = np.empty(n, dtype=np.uint16)
    st = ctypes.c_uint32(state)
    lib().oracle_lcg_fill(_ptr(out), n, ctypes.byref(st))
    return out, int(st.value)


def fill_causal_mask(q_len: int, kv_len: int, past_offset: int, sliding_window: int = INT_MAX) -> np.ndarray:
    m = np.empty((q_len, kv_len), dtype=np.float32)
    lib().oracle_fill_causal_mask(_ptr(m), q_len, kv_len, past_offset, sliding_window)
    return m


def fill_causal_mask_with_block_ids(block_ids, q_len: int, kv_len: int, past_offset: int,
                                    sliding_window: int = INT_MAX) -> np.ndarray:
    m = np.empty((q_len, kv_len), dtype=np.float32)
    ids = None if block_ids is None else np.ascontiguousarray(np.asarray(block_ids), dtype=np.int32)
    lib().oracle_fill_causal_mask_with_block_ids(_ptr(m), _ptr(ids), q_len, kv_len, past_offset, sliding_window)
    return m


def mul_sigmoid_inplace(a: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    ab = _bits(a).copy()
    gb = _bits(gate)
    lib().oracle_mul_sigmoid_inplace(_ptr(ab), _ptr(gb), ab.size)
    return bits_to_bf16(ab).reshape(a.shape)


def norm_rope(x: torch.Tensor, weight: Optional[torch.Tensor], *, eps: float, n_active_pairs: int = 0,
              offset: int = 0, theta: float = 10000.0, rope_cos: Optional[torch.Tensor] = None,
              rope_sin: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMSNorm (+ RoPE) of x (tokens, heads, hd) bf16; returns a new bf16 tensor."""
    tokens, heads, hd = x.shape
    xb = np.ascontiguousarray(_bits(x)).reshape(-1)
    out = np.empty_like(xb)
    wb = _bits(weight) if weight is not None else None
    cos = np.ascontiguousarray(rope_cos.detach().cpu().numpy(), dtype=np.float32) if rope_cos is not None else None
    sin = np.ascontiguousarray(rope_sin.detach().cpu().numpy(), dtype=np.float32) if rope_sin is not None else None
    lib().oracle_norm_rope(_ptr(xb), heads * hd, _ptr(out), heads * hd,
                           _ptr(wb) if wb is not None else None, tokens, heads, hd, n_active_pairs, offset,
                           theta, eps,
                           _ptr(cos) if cos is not None else None, _ptr(sin) if sin is not None else None)
    return bits_to_bf16(out).reshape(x.shape)


def mrope(x: torch.Tensor, positions, rotary_dim: int, theta: float, sections) -> torch.Tensor:
    """Qwen3.5 multi-axis RoPE of x (tokens, heads, head_dim) bf16 with positions (3, tokens); a new tensor."""
    tokens, heads, hd = x.shape
    xb = np.ascontiguousarray(_bits(x)).reshape(-1).copy()
    pos = np.ascontiguousarray(np.asarray(positions), dtype=np.int32)
    sec = np.ascontiguousarray(np.asarray(sections), dtype=np.int32)
    assert pos.shape == (3, tokens) and sec.shape == (3,)
    lib().oracle_mrope(_ptr(xb), _ptr(pos), tokens, heads, hd, rotary_dim, theta, _ptr(sec))
    return bits_to_bf16(xb).reshape(x.shape)


def sdpa_f32(q, k, v, *, scale: float, mask_type: int = MASK_NONE, window: int = INT_MAX,
             mask: Optional[np.ndarray] = None, gate=None, rows: Optional[Sequence[int]] = None,
             want_lse: bool = False):
    """fp32-softmax grading oracle for one sequence.

    q: (seq, nq, hd), k/v: (kv_len, nkv, hd).  Returns (out_f32, out_bf16[, lse]);
    with ``rows`` (flat token*nq+head indices) only those rows, packed.
    """
    qb, kb, vb = _bits(q), _bits(k), _bits(v)
    seq, nq, hd = qb.shape
    kv_len, nkv, _ = kb.shape
    gb = _bits(gate) if gate is not None else None
    rows_a = None if rows is None else np.ascontiguousarray(np.asarray(rows, dtype=np.int64))
    n = seq * nq if rows_a is None else rows_a.size
    out_f = np.empty((n, hd), dtype=np.float32)
    out_b = np.empty((n, hd), dtype=np.uint16)
    lse = np.empty(n, dtype=np.float32) if want_lse else None
    mk = None if mask is None else np.ascontiguousarray(mask, dtype=np.float32)
    rc = lib().oracle_sdpa_f32(_ptr(qb), _ptr(kb), _ptr(vb), _ptr(gb), _ptr(mk), mask_type,
                               int(window), seq, kv_len, nq, nkv, hd, float(scale),
                               _ptr(rows_a), n, _ptr(out_f), _ptr(out_b), _ptr(lse))
    if rc != 0:
        raise RuntimeError(f"oracle_sdpa_f32 failed: {rc}")
    if rows_a is None:
        out_f = out_f.reshape(seq, nq, hd)
        out_b = out_b.reshape(seq, nq, hd)
        if lse is not None:
            lse = lse.reshape(seq, nq)
    res = (torch.from_numpy(out_f), bits_to_bf16(out_b).reshape(out_b.shape))
    return res + (torch.from_numpy(lse),) if want_lse else res


def qwen35_online_attention(q, k, v, *, seq: int, past: int, scale: float) -> torch.Tensor:
    qb, kb, vb = _bits(q), _bits(k), _bits(v)
    _, nq, hd = qb.shape
    nkv = kb.shape[1]
    out = np.empty((seq, nq, hd), dtype=np.uint16)
    rc = lib().oracle_qwen35_online_attention(_ptr(qb), _ptr(kb), _ptr(vb), _ptr(out), seq, past,
                                              nq, nkv, hd, float(scale))
    if rc != 0:
        raise RuntimeError(f"oracle_qwen35_online_attention failed: {rc}")
    return bits_to_bf16(out).reshape(seq, nq, hd)


def gqa_attention(q, k, v, *, past_offset: int, sliding_window: int = INT_MAX, causal: bool) -> torch.Tensor:
    qb, kb, vb = _bits(q), _bits(k), _bits(v)
    seq, nq, hd = qb.shape
    kv_len, nkv, _ = kb.shape
    out = np.empty((seq, nq, hd), dtype=np.uint16)
    rc = lib().oracle_gqa_attention(_ptr(qb), seq, nq, hd, _ptr(kb), _ptr(vb), kv_len, nkv,
                                    past_offset, int(sliding_window), int(causal), _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle_gqa_attention failed: {rc}")
    return bits_to_bf16(out).reshape(seq, nq, hd)


def batched_attention(q, k, v, *, past_offset: int, sliding_window: int = INT_MAX, scale: float = 1.0,
                      skip_mask: bool = False) -> torch.Tensor:
    qb, kb, vb = _bits(q), _bits(k), _bits(v)
    seq, nq, hd = qb.shape
    kv_len, nkv, _ = kb.shape
    out = np.empty((seq, nq, hd), dtype=np.uint16)
    rc = lib().oracle_batched_attention(_ptr(qb), seq, nq, hd, _ptr(kb), _ptr(vb), kv_len, nkv,
                                        past_offset, int(sliding_window), float(scale),
                                        int(skip_mask), _ptr(out))
    if rc != 0:
        raise RuntimeError(f"oracle_batched_attention failed: {rc}")
    return bits_to_bf16(out).reshape(seq, nq, hd)


def merge_partials(o: torch.Tensor, lse: torch.Tensor):
    """o: (parts, rows, hd) f32; lse: (parts, rows) f32 -> (out (rows, hd), lse (rows,))."""
    oa = np.ascontiguousarray(o.numpy(), dtype=np.float32)
    la = np.ascontiguousarray(lse.numpy(), dtype=np.float32)
    parts, rows, hd = oa.shape
    out = np.empty((rows, hd), dtype=np.float32)
    ol = np.empty(rows, dtype=np.float32)
    lib().oracle_merge_partials(_ptr(oa), _ptr(la), parts, rows, hd, _ptr(out), _ptr(ol))
    return torch.from_numpy(out), torch.from_numpy(ol)


def torch_sdpa_f32(q, k, v, *, scale: float, mask_type: int = MASK_NONE, window: int = INT_MAX,
                   mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Independent formulation (torch CPU fp32 matmuls) of the grading oracle,
    used to cross-check the C code.  Shapes as in :func:`sdpa_f32`; returns f32."""
    qf, kf, vf = q.float(), k.float(), v.float()
    seq, nq, hd = qf.shape
    kv_len, nkv, _ = kf.shape
    g = nq // nkv
    kf = kf.repeat_interleave(g, dim=1)
    vf = vf.repeat_interleave(g, dim=1)
    s = torch.einsum("qhd,khd->hqk", qf, kf) * scale
    if mask_type == MASK_EXPLICIT:
        s = s + torch.as_tensor(mask, dtype=torch.float32)[None]
    elif mask_type == MASK_CAUSAL:
        qi = torch.arange(seq)[:, None] + (kv_len - seq)
        kj = torch.arange(kv_len)[None, :]
        dead = kj > qi
        if window != INT_MAX and window > 0:
            dead = dead | (kj < qi - window + 1)
        s = s.masked_fill(dead[None], float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("hqk,khd->qhd", p, vf)


def error_metrics(got: torch.Tensor, want: torch.Tensor) -> tuple[float, float]:
    """(relative L2, max-abs) of got vs want, both taken as fp32."""
    g, w = got.float().flatten(), want.float().flatten()
    den = float(torch.linalg.vector_norm(w))
    rel = float(torch.linalg.vector_norm(g - w)) / (den if den > 0 else 1.0)
    mx = float((g - w).abs().max()) if g.numel() else 0.0
    return rel, mx
