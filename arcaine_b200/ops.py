"""Python host side of the attention path: torch tensors in, C-ABI calls out.

torch is used for device memory and streams only; all arithmetic happens in
``libarc_sdpa.so``.  The functions in the second half keep the names, argument
order and error behaviour of the reference's C++ call sites so its call stacks
map one to one (reference files are cited per function).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Union

import torch

from . import _lib
from ._lib import MASK_CAUSAL, MASK_EXPLICIT, MASK_NONE, NO_WINDOW, ArcError, check

__all__ = [
    "MASK_NONE", "MASK_EXPLICIT", "MASK_CAUSAL", "NO_WINDOW", "ArcError",
    "sdpa_prefill", "sdpa_decode", "sdpa_merge", "mul_sigmoid_inplace", "fill_causal_mask",
    "gqa_attention_sdpa", "gqa_attention", "batched_attention", "qwen35_xmx_attention",
    "qwen35_online_attention", "qwen35_xmx_attention_decode_gqa",
    "device_status", "clear_device_status", "launch_count", "Workspace", "exchange_bytes",
]


def _stream_ptr(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _require(t: torch.Tensor, dtype, name: str) -> None:
    if not isinstance(t, torch.Tensor) or t.device.type != "cuda":
        raise ValueError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")


class Workspace:
    """Grow-only device scratch for split-KV partials, one per device.

    Reallocates only when a call needs more than any earlier call, so steady
    state has no allocation on the hot path (the reference measured what
    per-call attention scratch costs: notes/diffusion_gemma/NVFP4_DPAS_KERNEL.md:243-250).
    """

    _per_device: dict[int, "Workspace"] = {}

    def __init__(self, device: torch.device):
        self.device = device
        self.buf: Optional[torch.Tensor] = None

    @classmethod
    def for_device(cls, device: torch.device) -> "Workspace":
        idx = device.index if device.index is not None else torch.cuda.current_device()
        ws = cls._per_device.get(idx)
        if ws is None:
            ws = cls._per_device[idx] = cls(torch.device("cuda", idx))
        return ws

    def reserve(self, nbytes: int) -> torch.Tensor:
        if self.buf is None or self.buf.numel() < nbytes:
            self.buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=self.device)
        return self.buf


def _token_strides(t: torch.Tensor, name: str) -> tuple[int, int]:
    """(batch stride, token stride) in elements of a (B, T, H, D) tensor whose last two dims are dense."""
    if t.stride(3) != 1 or t.stride(2) != t.shape[3]:
        raise ValueError(f"{name}: the (heads, head_dim) block of every token must be contiguous")
    return t.stride(0), t.stride(1)


def sdpa_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float,
                 mask_type: int = MASK_NONE, window: int = NO_WINDOW, mask: Optional[torch.Tensor] = None,
                 gate: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                 num_splits: int = 0, return_lse: bool = False,
                 workspace: Optional[Workspace] = None,
                 block_ids: Optional[torch.Tensor] = None, block_ids_offset: int = 0,
                 out_copies: Optional[torch.Tensor] = None):
    """Prefill / canvas attention.  q: (B, S, nq, hd) or (S, nq, hd); k, v: (B, L, nkv, hd) or (L, nkv, hd).

    ``out`` may be ``q`` itself.  Returns ``out`` (and the natural-log LSE (B, S, nq) when asked).
    ``block_ids`` (device int32, one per absolute position, -1 = text; causal masks only): Gemma4's
    vision blocks — a query inside a block also sees the block's later keys
    (src/common/kernels/attention_mask.hpp:44-73); ``block_ids[block_ids_offset + j]`` is key j's id.
    ``out_copies`` (device int64, at most 15 addresses): further buffers laid out like ``out`` that the
    kernel's epilogue stores the result to as well — other GPUs' mapped buffers when a head-sharded output
    is to be gathered (see ``sharded.GatheredPrefill``).
    """
    squeeze = q.dim() == 3
    if squeeze:
        q, k, v = q.unsqueeze(0), k.unsqueeze(0), v.unsqueeze(0)
        gate = gate.unsqueeze(0) if gate is not None else None
        out = out.unsqueeze(0) if out is not None else None
    for t, n in ((q, "q"), (k, "k"), (v, "v")):
        _require(t, torch.bfloat16, n)
        if t.dim() != 4:
            raise ValueError(f"{n} must have 3 or 4 dims")
    B, S, nq, hd = q.shape
    Bk, L, nkv, hdk = k.shape
    if v.shape != k.shape or Bk != B or hdk != hd:
        raise ValueError("k/v shape mismatch")
    if out is None:
        out = torch.empty((B, S, nq, hd), dtype=torch.bfloat16, device=q.device)
    _require(out, torch.bfloat16, "out")
    if gate is not None:
        _require(gate, torch.bfloat16, "gate")
        if gate.shape != out.shape or gate.stride() != out.stride():
            raise ValueError("gate must be laid out like out")
    p = _lib.PrefillParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr()
    p.gate = gate.data_ptr() if gate is not None else None
    if mask is not None:
        _require(mask, torch.float32, "mask")
        if tuple(mask.shape) != (S, L) or not mask.is_contiguous():
            raise ValueError("mask must be a contiguous (seq, kv_len) f32 tensor")
        p.mask = mask.data_ptr()
    lse = torch.empty((B, S, nq), dtype=torch.float32, device=q.device) if return_lse else None
    p.out_lse = lse.data_ptr() if lse is not None else None
    p.batch, p.seq, p.kv_len, p.nq, p.nkv, p.hd = B, S, L, nq, nkv, hd
    p.q_stride_b, p.q_stride_t = _token_strides(q, "q")
    p.k_stride_b, p.k_stride_t = _token_strides(k, "k")
    p.v_stride_b, p.v_stride_t = _token_strides(v, "v")
    p.o_stride_b, p.o_stride_t = _token_strides(out, "out")
    p.scale, p.mask_type, p.window, p.num_splits = float(scale), int(mask_type), int(window), int(num_splits)
    if block_ids is not None:
        _require(block_ids, torch.int32, "block_ids")
        if not block_ids.is_contiguous() or block_ids.numel() < block_ids_offset + L or block_ids_offset < 0:
            raise ValueError("block_ids must be contiguous and hold block_ids_offset + kv_len entries")
        p.block_ids, p.block_ids_offset = block_ids.data_ptr(), int(block_ids_offset)
    if out_copies is not None:
        _require(out_copies, torch.int64, "out_copies")
        if not out_copies.is_contiguous() or out_copies.numel() > 15:
            raise ValueError("out_copies must be a contiguous int64 tensor of at most 15 addresses")
        p.out_copies, p.out_copy_count = out_copies.data_ptr(), out_copies.numel()
    L_ = _lib.load()
    with torch.cuda.device(q.device):
        need = L_.arc_sdpa_prefill_workspace_bytes(C.byref(p))
        if need:
            ws = (workspace or Workspace.for_device(q.device)).reserve(need)
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        check(L_.arc_sdpa_prefill(C.byref(p), _stream_ptr(q)), "arc_sdpa_prefill")
    if squeeze:
        out = out.squeeze(0)
        lse = lse.squeeze(0) if lse is not None else None
    return (out, lse) if return_lse else out


def sdpa_decode(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: float,
                kv_len: Union[int, torch.Tensor, None] = None, kv_row_offset: Optional[torch.Tensor] = None,
                gate: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                return_partial: bool = False, want_out: bool = True, num_ctas: int = 0,
                partial_out: Optional[torch.Tensor] = None, partial_lse: Optional[torch.Tensor] = None,
                exchange: Optional[tuple] = None, workspace: Optional[Workspace] = None,
                exchange_wait_cycles: int = 0):
    """Split-KV decode of one query token per sequence.

    q: (B, nq, hd).  k, v: either (B, max_len, nkv, hd) (one cache block per sequence) or
    (rows, nkv, hd) packed with ``kv_row_offset`` (int64 device tensor, first row of each sequence).
    ``kv_len``: int (same for all) or int32 device tensor (B,).
    Returns ``out`` (B, nq, hd) bf16; with ``return_partial`` also (out_f32, lse) — the
    ungated fp32 result and natural-log LSE a sequence-sharded caller exchanges.
    ``exchange`` = (peer_ptrs int64 device tensor (world,), world, rank, step) turns on the
    in-kernel exchange of those records over NVLink peer memory: ``out`` is then the result
    merged over all ranks' key slices (see :class:`arcaine_b200.sharded.SeqShardedDecode`);
    ``exchange_wait_cycles`` bounds the wait for the other ranks' records (0: about a second).
    """
    _require(q, torch.bfloat16, "q")
    _require(k, torch.bfloat16, "k")
    _require(v, torch.bfloat16, "v")
    if q.dim() != 3:
        raise ValueError("q must be (B, nq, hd)")
    B, nq, hd = q.shape
    if q.stride(2) != 1 or q.stride(1) != hd:
        raise ValueError("q: (nq, hd) must be contiguous")
    p = _lib.DecodeParams()
    if k.dim() == 4:
        if kv_row_offset is not None:
            raise ValueError("kv_row_offset needs packed (rows, nkv, hd) caches")
        if k.shape[0] != B or v.shape != k.shape:
            raise ValueError("k/v shape mismatch")
        _, max_len, nkv, hdk = k.shape
        if k.stride(3) != 1 or k.stride(2) != hdk or k.stride() != v.stride() or k.stride(0) % k.stride(1):
            raise ValueError("k/v: unsupported strides")
        p.kv_stride_t = k.stride(1)
        p.kv_stride_b = k.stride(0) // k.stride(1)
        if max_len == 0:  # an empty slice: no rows at all
            p.kv_stride_b = 0
        p.kv_rows_total = (B - 1) * p.kv_stride_b + max_len
    elif k.dim() == 3:
        rows, nkv, hdk = k.shape
        if v.shape != k.shape or k.stride(2) != 1 or k.stride(1) != hdk or k.stride() != v.stride():
            raise ValueError("k/v: unsupported strides")
        max_len = rows
        p.kv_stride_t = k.stride(0)
        p.kv_stride_b = 0
        p.kv_rows_total = rows
        if kv_row_offset is None and B > 1:
            raise ValueError("packed caches need kv_row_offset")
    else:
        raise ValueError("k must have 3 or 4 dims")
    if hdk != hd:
        raise ValueError("head_dim mismatch")
    if isinstance(kv_len, torch.Tensor):
        _require(kv_len, torch.int32, "kv_len")
        if kv_len.shape != (B,) or not kv_len.is_contiguous():
            raise ValueError("kv_len must be a contiguous (B,) int32 tensor")
        p.kv_len = kv_len.data_ptr()
        p.kv_len_uniform = 0
    else:
        p.kv_len_uniform = int(max_len if kv_len is None else kv_len)
        if p.kv_len_uniform > max_len:
            raise ValueError("kv_len exceeds the cache")
    if kv_row_offset is not None:
        _require(kv_row_offset, torch.int64, "kv_row_offset")
        if kv_row_offset.shape != (B,) or not kv_row_offset.is_contiguous():
            raise ValueError("kv_row_offset must be a contiguous (B,) int64 tensor")
        p.kv_row_offset = kv_row_offset.data_ptr()
    p.max_kv_len = int(max_len)
    if want_out and out is None:
        out = torch.empty((B, nq, hd), dtype=torch.bfloat16, device=q.device)
    if out is not None:
        _require(out, torch.bfloat16, "out")
        if out.shape != q.shape or out.stride(2) != 1 or out.stride(1) != hd:
            raise ValueError("out must be laid out like q")
        p.out = out.data_ptr()
        p.o_stride_b = out.stride(0)
    if gate is not None:
        _require(gate, torch.bfloat16, "gate")
        if out is None or gate.shape != out.shape or gate.stride() != out.stride():
            raise ValueError("gate must be laid out like out")
        p.gate = gate.data_ptr()
    out_f32 = lse = None
    if return_partial:
        out_f32 = partial_out if partial_out is not None else torch.empty((B, nq, hd), dtype=torch.float32, device=q.device)
        lse = partial_lse if partial_lse is not None else torch.empty((B, nq), dtype=torch.float32, device=q.device)
        _require(out_f32, torch.float32, "partial_out")
        _require(lse, torch.float32, "partial_lse")
        if tuple(out_f32.shape) != (B, nq, hd) or tuple(lse.shape) != (B, nq) or not out_f32.is_contiguous() \
                or not lse.is_contiguous():
            raise ValueError("partial_out / partial_lse must be contiguous (B, nq, hd) / (B, nq) f32")
        p.out_f32, p.out_lse = out_f32.data_ptr(), lse.data_ptr()
    p.q, p.k, p.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    p.batch, p.nq, p.nkv, p.hd = B, nq, nkv, hd
    p.q_stride_b = q.stride(0)
    p.scale, p.num_ctas = float(scale), int(num_ctas)
    if exchange is not None:
        peers, world, rank, step = exchange
        _require(peers, torch.int64, "exchange peers")
        p.xchg_peers, p.xchg_world, p.xchg_rank, p.xchg_step = peers.data_ptr(), int(world), int(rank), int(step) & 0xFFFFFFFF
        p.xchg_wait_cycles = int(exchange_wait_cycles)
    L_ = _lib.load()
    with torch.cuda.device(q.device):
        need = L_.arc_sdpa_decode_workspace_bytes(C.byref(p))
        if need:
            ws = (workspace or Workspace.for_device(q.device)).reserve(need)
            p.workspace, p.workspace_bytes = ws.data_ptr(), ws.numel()
        check(L_.arc_sdpa_decode(C.byref(p), _stream_ptr(q)), "arc_sdpa_decode")
    return (out, out_f32, lse) if return_partial else out


def sdpa_merge(part_out: torch.Tensor, part_lse: torch.Tensor, *, gate: Optional[torch.Tensor] = None,
               out: Optional[torch.Tensor] = None, want_f32: bool = False, want_lse: bool = False):
    """LSE merge of partial results: part_out (P, rows..., hd) f32, part_lse (P, rows...) f32.

    The leading (part) dimension may be strided — e.g. views into one packed
    ``[out | lse]`` record per rank — as long as each part is dense.
    """
    _require(part_out, torch.float32, "part_out")
    _require(part_lse, torch.float32, "part_lse")
    P, hd = part_out.shape[0], part_out.shape[-1]
    row_shape = tuple(part_out.shape[1:-1])
    rows = 1
    for s in row_shape:
        rows *= s
    if tuple(part_lse.shape) != (P, *row_shape):
        raise ValueError("part_lse shape mismatch")
    if not part_out[0].is_contiguous() or not part_lse[0].is_contiguous():
        raise ValueError("each part must be dense")
    so = part_out.stride(0) if P > 1 else rows * hd
    sl = part_lse.stride(0) if P > 1 else rows
    if out is None:
        out = torch.empty((*row_shape, hd), dtype=torch.bfloat16, device=part_out.device)
    _require(out, torch.bfloat16, "out")
    if not out.is_contiguous():
        raise ValueError("out must be contiguous")
    if gate is not None:
        _require(gate, torch.bfloat16, "gate")
        if not gate.is_contiguous() or gate.numel() != out.numel():
            raise ValueError("gate must be contiguous and shaped like out")
    o32 = torch.empty((*row_shape, hd), dtype=torch.float32, device=part_out.device) if want_f32 else None
    lse = torch.empty(row_shape, dtype=torch.float32, device=part_out.device) if want_lse else None
    with torch.cuda.device(part_out.device):
        check(_lib.load().arc_sdpa_merge(part_out.data_ptr(), part_lse.data_ptr(), P, rows, hd, so, sl,
                                         gate.data_ptr() if gate is not None else None, out.data_ptr(),
                                         o32.data_ptr() if o32 is not None else None,
                                         lse.data_ptr() if lse is not None else None, _stream_ptr(part_out)),
              "arc_sdpa_merge")
    res = (out,)
    if want_f32:
        res += (o32,)
    if want_lse:
        res += (lse,)
    return res[0] if len(res) == 1 else res


def mul_sigmoid_inplace(a: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """a *= sigmoid(gate) in bf16 storage / fp32 math (src/modeling/qwen3_5_moe/kernels.hpp:80-88)."""
    _require(a, torch.bfloat16, "a")
    _require(gate, torch.bfloat16, "gate")
    if not a.is_contiguous() or not gate.is_contiguous() or a.numel() != gate.numel():
        raise ValueError("a and gate must be contiguous and of equal size")
    with torch.cuda.device(a.device):
        check(_lib.load().arc_mul_sigmoid_inplace(a.data_ptr(), gate.data_ptr(), a.numel(), _stream_ptr(a)),
              "arc_mul_sigmoid_inplace")
    return a


def fill_causal_mask(q_len: int, kv_len: int, past_offset: int, sliding_window: int = NO_WINDOW, *,
                     device="cuda", out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Additive (q_len, kv_len) f32 mask (src/common/kernels/attention_mask.hpp:12-38)."""
    if out is None:
        out = torch.empty((q_len, kv_len), dtype=torch.float32, device=device)
    _require(out, torch.float32, "out")
    with torch.cuda.device(out.device):
        check(_lib.load().arc_fill_causal_mask(out.data_ptr(), q_len, kv_len, past_offset, sliding_window,
                                               _stream_ptr(out)), "arc_fill_causal_mask")
    return out


def fill_causal_mask_with_block_ids(block_ids: Optional[torch.Tensor], q_len: int, kv_len: int, past_offset: int,
                                    sliding_window: int = NO_WINDOW, *, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Causal / sliding-window mask with Gemma4's bidirectional vision blocks
    (src/common/kernels/attention_mask.hpp:44-73).  block_ids: device int32, one per absolute position."""
    device = block_ids.device if block_ids is not None else (out.device if out is not None else "cuda")
    if out is None:
        out = torch.empty((q_len, kv_len), dtype=torch.float32, device=device)
    _require(out, torch.float32, "out")
    if block_ids is not None:
        _require(block_ids, torch.int32, "block_ids")
        if block_ids.numel() < past_offset + q_len:
            raise ValueError("block_ids must cover every position up to past_offset + q_len")
    with torch.cuda.device(out.device):
        check(_lib.load().arc_fill_causal_mask_with_block_ids(
            out.data_ptr(), block_ids.data_ptr() if block_ids is not None else None, q_len, kv_len, past_offset,
            sliding_window, _stream_ptr(out)), "arc_fill_causal_mask_with_block_ids")
    return out


# ---------------------------------------------------------------------------
# Reference-named entry points (one sequence, token-major tensors)
# ---------------------------------------------------------------------------
def gqa_attention_sdpa(Q, seq, nq, hd, Kc, Vc, kv_len, nkv, mask=None, mask_type=MASK_NONE, out=None):
    """src/modeling/diffusion_gemma/attention.cpp:930-995 — no scale; mask_type 0 / 1 / 3."""
    q = Q.view(seq, nq, hd)
    k = Kc[: kv_len * nkv * hd].view(kv_len, nkv, hd) if Kc.dim() == 1 else Kc[:kv_len]
    v = Vc[: kv_len * nkv * hd].view(kv_len, nkv, hd) if Vc.dim() == 1 else Vc[:kv_len]
    return sdpa_prefill(q, k, v, scale=1.0, mask_type=mask_type, mask=mask, out=out)


def gqa_attention(Q, seq, nq, hd, Kc, Vc, kv_len, nkv, past_offset, sliding_window, causal, out=None):
    """src/modeling/diffusion_gemma/attention.cpp:706-821 — the matmul/softmax/matmul path's result."""
    del past_offset  # queries and keys share it; the visibility rule does not depend on it
    q = Q.view(seq, nq, hd)
    k, v = Kc[:kv_len], Vc[:kv_len]
    return sdpa_prefill(q, k, v, scale=1.0, mask_type=MASK_CAUSAL if causal else MASK_NONE,
                        window=sliding_window if causal else NO_WINDOW, out=out)


def batched_attention(Q, seq_len, nq_heads, q_head_dim, K, V, kv_len, nkv_heads, kv_head_dim, past_offset,
                      sliding_window, scale=1.0, skip_mask=False, block_ids=None, out=None):
    """src/common/layers/attention_batched.hpp:71-136.  ``block_ids`` (device int32 per absolute position)
    turns on the vision-block rule of fill_causal_mask_with_block_ids, evaluated inside the kernel: key j
    of ``K`` sits at absolute position past_offset - (kv_len - seq_len) + j."""
    if q_head_dim != kv_head_dim:
        raise RuntimeError("batched_attention: q and kv head_dim differ")
    if block_ids is not None and skip_mask:
        block_ids = None  # the reference builds no mask at all in that case
    return sdpa_prefill(Q.view(seq_len, nq_heads, q_head_dim), K[:kv_len], V[:kv_len], scale=scale,
                        mask_type=MASK_NONE if skip_mask else MASK_CAUSAL,
                        window=NO_WINDOW if skip_mask else sliding_window, out=out,
                        block_ids=block_ids, block_ids_offset=past_offset - (kv_len - seq_len) if block_ids is not None else 0)


def gemma4_sliding_decode_attention(Q, K_cache, V_cache, kv_len, kv_start, nq_heads, nkv_heads, head_dim, out=None):
    """Single-token decode of a Gemma4 sliding layer over cache rows [kv_start, kv_start + kv_len)
    (sliding_decode_attention, src/modeling/gemma4_unified/attention.cpp:93-137; no scale: Q and K are
    RMS-normed).  The reference keeps two extra copies of the cache for this call, K head-major
    (nkv, max_seq, hd) and V transposed (nkv, hd, max_seq), because its strided GEMMs want them; here the
    token-major cache (max_seq, nkv, hd) of src/modeling/gemma4_unified/kv_cache.hpp:8-9 is read in place —
    the GQA group is folded into the MMA, so those copies and their upkeep disappear."""
    q = Q.view(1, nq_heads, head_dim)
    o = out.view(1, nq_heads, head_dim) if out is not None else None
    k = K_cache.view(-1, nkv_heads, head_dim)[kv_start:kv_start + kv_len]
    v = V_cache.view(-1, nkv_heads, head_dim)[kv_start:kv_start + kv_len]
    res = sdpa_decode(q, k, v, scale=1.0, kv_len=kv_len, out=o)
    return res.view(nq_heads, head_dim)


def gemma4_full_decode_attention(Q, K_cache, V_cache, kv_len, nq_heads, head_dim, out=None):
    """The nkv == 1 decode path of Gemma4's full-attention layers
    (src/modeling/gemma4_unified/attention.cpp:274-288): every query head shares the one KV head, the cache
    (kv_len, 1, hd) is read once for all of them.  Head dims 128 and 256 (the 512-wide global heads are
    outside what the attention kernels cover)."""
    q = Q.view(1, nq_heads, head_dim)
    o = out.view(1, nq_heads, head_dim) if out is not None else None
    nsplit = 1
    if nq_heads > 16:
        # more than 16 query heads on one KV head: the same cache rows serve several groups of <= 16 heads
        for d in range(1, nq_heads + 1):
            if nq_heads % d == 0 and nq_heads // d <= 16:
                nsplit = d
                break
    k = K_cache.view(-1, 1, head_dim)[:kv_len]
    v = V_cache.view(-1, 1, head_dim)[:kv_len]
    if nsplit == 1:
        return sdpa_decode(q, k, v, scale=1.0, kv_len=kv_len, out=o).view(nq_heads, head_dim)
    # "batch" of nsplit query groups over the same rows (row offset 0 for all)
    qb = q.view(nsplit, nq_heads // nsplit, head_dim)
    ob = o.view(nsplit, nq_heads // nsplit, head_dim) if o is not None else None
    offs = torch.zeros(nsplit, dtype=torch.int64, device=Q.device)
    lens = torch.full((nsplit,), kv_len, dtype=torch.int32, device=Q.device)
    res = sdpa_decode(qb, k, v, scale=1.0, kv_len=lens, kv_row_offset=offs, out=ob)
    return res.view(nq_heads, head_dim)


def qwen35_xmx_attention(query, key, value, output, seq, past, query_heads, key_heads, head_dim, scale):
    """src/modeling/qwen3_5/kernels.hpp:761-905 — causal over past + seq keys; output may alias query."""
    if key_heads <= 0 or query_heads % key_heads != 0:
        raise RuntimeError("Qwen3.5 attention requires integral GQA ratio")
    q = query.view(-1, query_heads, head_dim)[:seq]
    o = output.view(-1, query_heads, head_dim)[:seq]
    k, v = key[: past + seq], value[: past + seq]
    if seq == 1:
        sdpa_decode(q, k, v, scale=scale, kv_len=past + 1, out=o)
    else:
        sdpa_prefill(q, k, v, scale=scale, mask_type=MASK_CAUSAL, out=o)
    return output


qwen35_online_attention = qwen35_xmx_attention  # src/modeling/qwen3_5/kernels.hpp:621-679, same contract


def qwen35_xmx_attention_decode_gqa(query, key, value, output, past, query_heads, key_heads, head_dim, scale,
                                    gate=None):
    """src/modeling/qwen3_5/kernels.hpp:910-1054, optionally with the sigmoid gate of operators.hpp:160 fused."""
    if key_heads <= 0 or query_heads % key_heads != 0:
        raise RuntimeError("Qwen3.5 attention requires integral GQA ratio")
    q = query.view(1, query_heads, head_dim)
    o = output.view(1, query_heads, head_dim)
    g = gate.view(1, query_heads, head_dim) if gate is not None else None
    sdpa_decode(q, key[: past + 1], value[: past + 1], scale=scale, kv_len=past + 1, gate=g, out=o)
    return output


def qkv_prepare(q: Optional[torch.Tensor], k: Optional[torch.Tensor], v: Optional[torch.Tensor], *,
                k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None, past_len: int = 0,
                q_weight: Optional[torch.Tensor] = None, k_weight: Optional[torch.Tensor] = None,
                eps: float = 1e-6, theta: float = 10000.0, partial_rotary_factor: float = 1.0,
                rope_cos: Optional[torch.Tensor] = None, rope_sin: Optional[torch.Tensor] = None,
                pos_offset=None, v_from_k: bool = False, rotary_dim: Optional[int] = None,
                mrope_positions: Optional[torch.Tensor] = None, mrope_section=None, v_copy: bool = False) -> None:
    """RMSNorm (+ RoPE) of the projected Q / K rows, unit-RMS norm of V and the KV-cache append, one launch.

    q: (B, S, nq, hd) or (S, nq, hd), rewritten in place.  k, v: (B, S, nkv, hd) projections.  K and V go to
    ``k_cache`` / ``v_cache`` (B, capacity, nkv, hd) at rows ``past_len .. past_len + S`` (no separate copy);
    without caches K is rewritten in place and V too.  ``v_from_k``: V = unit-RMS norm of the raw K projection
    (full-attention layers, src/modeling/diffusion_gemma/attention.cpp:587-595).  ``pos_offset``: the position
    of the first token, an int or a device int32 tensor (B,); defaults to ``past_len``.  With ``rope_cos`` /
    ``rope_sin`` (S, n_active_pairs) or (B, S, n_active_pairs) f32 the angles are read, otherwise computed.

    Qwen3.5 form (qwen35_apply_mrope, src/modeling/qwen3_5/kernels.hpp:576-617): ``rotary_dim`` rotates pairs
    (f, f + rotary_dim/2) with frequency exponent 2f / rotary_dim; ``mrope_positions`` (B, 3, S) or (3, S) int32
    with ``mrope_section`` (three ints) gives each frequency the position of its axis; ``v_copy`` appends V
    without a norm.
    """
    ref = q if q is not None else k
    if ref is None:
        raise ValueError("qkv_prepare needs q or k")
    three = ref.dim() == 3
    un = (lambda t: t.unsqueeze(0) if (t is not None and three) else t)
    q, k, v, k_cache, v_cache = un(q), un(k), un(v), un(k_cache), un(v_cache)
    ref = q if q is not None else k
    B, S, _, hd = ref.shape
    P = _lib.QkvPrepareParams()
    for t, name in ((q, "q"), (k, "k"), (v, "v"), (k_cache, "k_cache"), (v_cache, "v_cache"), (q_weight, "q_weight"),
                    (k_weight, "k_weight")):
        if t is not None:
            _require(t, torch.bfloat16, name)
    if q is not None:
        P.q = q.data_ptr()
        P.nq = q.shape[2]
        P.q_stride_b, P.q_stride_t = _token_strides(q, "q")
    if k is not None:
        P.k_src = k.data_ptr()
        P.nkv = k.shape[2]
        P.k_src_stride_b, P.k_src_stride_t = _token_strides(k, "k")
        kd = k_cache if k_cache is not None else k
        row0 = past_len if k_cache is not None else 0
        if k_cache is not None and past_len + S > k_cache.shape[1]:
            raise ValueError("KV cache capacity exceeded")
        P.k_dst_stride_b, P.k_dst_stride_t = _token_strides(kd, "k_cache")
        P.k_dst = kd.data_ptr() + row0 * P.k_dst_stride_t * 2
        if v is not None or v_from_k:
            vd = v_cache if v_cache is not None else (v if v is not None else None)
            if vd is None:
                raise ValueError("v_from_k needs v_cache")
            if v_from_k and k_cache is None:
                # K would be rewritten in place while V is still being read from it
                raise ValueError("v_from_k needs k_cache: K cannot be normalised in place when V is taken from it")
            P.v_dst_stride_b, P.v_dst_stride_t = _token_strides(vd, "v_cache")
            P.v_dst = vd.data_ptr() + (past_len if v_cache is not None else 0) * P.v_dst_stride_t * 2
            if v is not None and not v_from_k:
                P.v_src = v.data_ptr()
                P.v_src_stride_b, P.v_src_stride_t = _token_strides(v, "v")
    P.q_weight = q_weight.data_ptr() if q_weight is not None else None
    P.k_weight = k_weight.data_ptr() if k_weight is not None else None
    P.batch, P.seq, P.hd = B, S, hd
    P.n_active_pairs = int(partial_rotary_factor * hd / 2.0)
    if rope_cos is not None:
        _require(rope_cos, torch.float32, "rope_cos")
        _require(rope_sin, torch.float32, "rope_sin")
        if not (rope_cos.is_contiguous() and rope_sin.is_contiguous()):
            raise ValueError("rope tables must be contiguous")
        P.rope_cos, P.rope_sin = rope_cos.data_ptr(), rope_sin.data_ptr()
        P.rope_stride_b = S * P.n_active_pairs if rope_cos.dim() == 3 else 0
    if isinstance(pos_offset, torch.Tensor):
        _require(pos_offset, torch.int32, "pos_offset")
        P.pos_offset = pos_offset.data_ptr()
    else:
        P.pos0 = past_len if pos_offset is None else int(pos_offset)
    P.theta, P.eps = float(theta), float(eps)
    if rotary_dim is not None:
        P.rot_half, P.freq_denom, P.n_active_pairs = rotary_dim // 2, rotary_dim, rotary_dim // 2
    if mrope_positions is not None:
        _require(mrope_positions, torch.int32, "mrope_positions")
        if not mrope_positions.is_contiguous() or mrope_positions.numel() != B * 3 * S:
            raise ValueError("mrope_positions must be a contiguous (B, 3, S) int32 tensor")
        if mrope_section is None or len(mrope_section) != 3:
            raise ValueError("Qwen3.5 MRoPE needs three sections")
        P.mrope_positions = mrope_positions.data_ptr()
        for i in range(3):
            P.mrope_section[i] = int(mrope_section[i])
    P.v_copy = 1 if v_copy else 0
    _lib.check(_lib.load().arc_qkv_prepare(C.byref(P), _stream_ptr(ref)), "arc_qkv_prepare")


def rms_norm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """In-place RMSNorm over the last dimension of (rows, H) / (S, heads, H): rms_norm / rms_norm_no_scale,
    src/common/kernels/rms_norm.hpp:9-56 (weight None = unit scale)."""
    x3 = x if x.dim() == 3 else x.view(x.shape[0], 1, x.shape[-1])
    qkv_prepare(x3, None, None, q_weight=weight, eps=eps, partial_rotary_factor=0.0)
    return x


def fused_norm_rope_inplace(x: torch.Tensor, weight: torch.Tensor, offset: int, theta: float, partial: float,
                            eps: float, rope_cos: Optional[torch.Tensor] = None,
                            rope_sin: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fused_norm_rope_inplace(x (seq, nheads, hd), weight, offset, theta, partial, eps, cos, sin):
    src/modeling/diffusion_gemma/attention_kernels.hpp:99-153."""
    qkv_prepare(x, None, None, q_weight=weight, eps=eps, theta=theta, partial_rotary_factor=partial,
                rope_cos=rope_cos, rope_sin=rope_sin, pos_offset=offset)
    return x


def exchange_bytes(world: int, batch: int, nq: int, hd: int) -> int:
    """Size of one rank's peer-exchange buffer for sequence-sharded decode."""
    return int(_lib.load().arc_sdpa_exchange_bytes(world, batch, nq, hd))


FAULT_WAIT_PEER = 9      # device fault codes (csrc/ptx.cuh)
FAULT_BAD_KV_RANGE = 10


def device_status(device=None) -> tuple[int, int]:
    """(fault code, detail) of the device-side status word; synchronises the device."""
    code, detail = C.c_uint32(0), C.c_uint32(0)
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        rc = _lib.load().arc_sdpa_device_status(C.byref(code), C.byref(detail))
    if rc not in (_lib.ARC_OK, _lib.ARC_ERR_DEVICE_WAIT_TIMEOUT, _lib.ARC_ERR_DEVICE_BAD_RANGE):
        raise ArcError(rc, "arc_sdpa_device_status")
    return int(code.value), int(detail.value)


def clear_device_status(device=None) -> None:
    with torch.cuda.device(device if device is not None else torch.cuda.current_device()):
        check(_lib.load().arc_sdpa_clear_device_status(), "arc_sdpa_clear_device_status")


def launch_count() -> int:
    return int(_lib.load().arc_sdpa_launch_count())
