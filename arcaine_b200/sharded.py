"""Multi-GPU partitioning of the attention path: one process per GPU, torch.distributed plumbing.

Two partitions, both without any collective inside the kernels:

* prefill / canvas — KV heads (with their query-head groups) and, once the heads
  run out, whole sequences are dealt to ranks; each rank computes its slice of the
  output.  The only exchange is an optional all-gather of the output slices.
* long-context decode — the KV *sequence* is cut into one contiguous slice per
  rank, the single-token queries are replicated.  Every rank produces one packed
  record ``[out f32 (B, nq, hd) | lse f32 (B, nq)]``; one all-gather moves the
  records and every rank folds them with the log-sum-exp merge kernel, which also
  applies the optional sigmoid gate.

The reference has neither (its two GPUs split layers and copy activations through
host memory, src/modeling/diffusion_gemma/model.cpp:33-46), so there is no
reference call to mirror; the record layout and merge identity are this
library's own.  The planning and exchange functions below are plain host logic on
torch tensors and run unchanged on CPU tensors over ``gloo``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


# ---------------------------------------------------------------------------
# Partition planning (pure host logic)
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class HeadShard:
    """Slice of a (batch, tokens, heads, hd) problem owned by one rank."""
    kv_head_begin: int
    kv_head_end: int
    q_head_begin: int
    q_head_end: int
    batch_begin: int
    batch_end: int

    @property
    def empty(self) -> bool:
        return self.kv_head_begin >= self.kv_head_end or self.batch_begin >= self.batch_end


def _clib():
    from . import _lib  # the planners live in the C library (include/arc_sdpa.h) so that C and C++ hosts share them
    return _lib, _lib.load()


def plan_head_shards(nq: int, nkv: int, batch: int, world: int) -> list[HeadShard]:
    """Deal KV heads first, then sequences, to ``world`` ranks (``arc_plan_head_shards``).

    ``world`` is factored as head_ways x batch_ways with head_ways the largest
    divisor of ``world`` that also divides ``nkv``; batch_ways must then divide
    into ``batch`` (ranks beyond the available work get an empty shard).
    """
    if nq % nkv != 0:
        raise ValueError("nq must be a multiple of nkv")
    _lib, L = _clib()
    shards = []
    for r in range(world):
        hs = _lib.HeadShard()
        _lib.check(L.arc_plan_head_shards(nq, nkv, batch, world, r, C.byref(hs)), "arc_plan_head_shards")
        shards.append(HeadShard(hs.kv_head_begin, hs.kv_head_end, hs.q_head_begin, hs.q_head_end,
                                hs.batch_begin, hs.batch_end))
    return shards


def plan_seq_shards(kv_len: int, world: int, align: int = 64) -> list[tuple[int, int]]:
    """Contiguous [begin, end) key ranges, one per rank, boundaries aligned to ``align`` keys
    (``arc_plan_seq_shards``).

    A short sequence leaves the last ranks with an empty range ``(kv_len, kv_len)``; such a rank still
    takes part in the step (it sends records with lse = -inf), see :class:`SeqShardedDecode`.
    """
    _lib, L = _clib()
    out = []
    for r in range(world):
        b, e = C.c_int64(0), C.c_int64(0)
        _lib.check(L.arc_plan_seq_shards(kv_len, world, r, align, C.byref(b), C.byref(e)), "arc_plan_seq_shards")
        out.append((int(b.value), int(e.value)))
    return out


def plan_batch_shards(lens, world: int) -> list[list[int]]:
    """Deal whole sequences to ranks so that the ranks' key counts come out even (``arc_plan_batch_shards``).

    Decode time is proportional to the keys a rank reads, not to its number of sequences, so the
    sequences are taken longest first and each goes to the rank with the fewest keys so far (ties: the
    rank with fewer sequences, then the lower rank).  Returns, per rank, the sequence indices in
    ascending order.  Dealing by count instead left the heaviest of 8 ranks 1.27x above the mean for 64
    lengths uniform in [1024, 32768]; this rule leaves it within about 1 %.
    """
    lens = [int(x) for x in lens]
    if world <= 0:
        raise ValueError("world must be positive")
    _lib, L = _clib()
    n = len(lens)
    arr = (C.c_int32 * max(n, 1))(*lens)
    owner = (C.c_int32 * max(n, 1))()
    _lib.check(L.arc_plan_batch_shards(arr, n, world, owner), "arc_plan_batch_shards")
    owned: list[list[int]] = [[] for _ in range(world)]
    for i in range(n):
        owned[owner[i]].append(i)
    return owned


def all_ranks_ok(local_ok: bool, group: Optional[dist.ProcessGroup] = None, device: Optional[torch.device] = None) -> bool:
    """Host-side agreement between steps: True only if every rank reports ``local_ok``.

    Call it after a step has been synchronised and before the next launch — with ``local_ok`` false on
    a rank whose step failed (an exception, a device status) or that is about to leave.  The others
    then skip the launch instead of waiting on the device for records that will never come (the
    in-kernel peer wait is bounded, but it leaves a device status that has to be cleared).  One small
    all-reduce on the host path; works over gloo with CPU tensors and over NCCL with ``device``.
    """
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return bool(local_ok)
    flag = torch.tensor([0.0 if local_ok else 1.0], device=device if device is not None else "cpu")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX, group=group)
    return flag.item() == 0.0


# ---------------------------------------------------------------------------
# Record exchange (works on CPU tensors over gloo and CUDA tensors over NCCL)
# ---------------------------------------------------------------------------
def record_numel(batch: int, nq: int, hd: int) -> int:
    """Floats in one packed record, padded to a multiple of 4 so every part stays 16-byte aligned."""
    _lib, L = _clib()
    return int(L.arc_sdpa_record_floats(batch, nq, hd))


def split_record(record: torch.Tensor, batch: int, nq: int, hd: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Views (out (..., B, nq, hd), lse (..., B, nq)) into packed record(s); the last dim is the record."""
    n_out, n_lse = batch * nq * hd, batch * nq
    out = record[..., :n_out].unflatten(-1, (batch, nq, hd))
    lse = record[..., n_out:n_out + n_lse].unflatten(-1, (batch, nq))
    return out, lse


def exchange_records(record: torch.Tensor, gathered: Optional[torch.Tensor] = None,
                     group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather one packed record per rank into a (world, numel) tensor."""
    world = dist.get_world_size(group)
    if gathered is None:
        gathered = torch.empty((world, record.numel()), dtype=record.dtype, device=record.device)
    if world == 1:
        gathered[0].copy_(record)
        return gathered
    dist.all_gather_into_tensor(gathered.view(-1), record.contiguous().view(-1), group=group)
    return gathered


# ---------------------------------------------------------------------------
# GPU entry points
# ---------------------------------------------------------------------------
class SeqShardedDecode:
    """Sequence-sharded decode step with persistent exchange buffers.

    Each rank holds keys [begin, end) of every sequence (``k_local``/``v_local``:
    (B, local_len, nkv, hd)) and the full query.  Two exchange paths:

    * ``peer`` (default when symmetric memory can be set up): two launches per step.  The decode
      merge kernel stores this rank's ``(out, lse)`` records straight into every rank's exchange
      buffer over NVLink as (value, step) words, waits (bounded) until the words of all ranks for
      its rows show the step, and folds the records — the exchange is part of the kernel, no
      collective call.
    * ``nccl``: local decode writes the packed record, one ``all_gather_into_tensor`` moves it,
      the uniform merge kernel folds the gathered records in place.
    """

    def __init__(self, batch: int, nq: int, hd: int, device: torch.device, group: Optional[dist.ProcessGroup] = None,
                 exchange: str = "auto"):
        from . import ops  # GPU-only import
        self._ops = ops
        self.batch, self.nq, self.hd = batch, nq, hd
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.out = torch.empty((batch, nq, hd), dtype=torch.bfloat16, device=device)
        self.step = 0
        self.mode = "local" if self.world == 1 else exchange
        self.peer_error: Optional[str] = None
        if self.mode in ("auto", "peer"):
            try:
                self._setup_peer(device)
                self.mode = "peer"
            except Exception as e:  # symmetric memory unavailable: fall back to the collective
                if exchange == "peer":
                    raise
                self.peer_error = repr(e)
                self.mode = "nccl"
        if self.mode in ("nccl", "local"):
            n = record_numel(batch, nq, hd)
            self.record = torch.empty(n, dtype=torch.float32, device=device)
            self.gathered = torch.empty((self.world, n), dtype=torch.float32, device=device)
            self.part_out, self.part_lse = split_record(self.record, batch, nq, hd)
            self.all_out, self.all_lse = split_record(self.gathered, batch, nq, hd)

    def _setup_peer(self, device):
        import torch.distributed._symmetric_memory as symm_mem
        nbytes = self._ops.exchange_bytes(self.world, self.batch, self.nq, self.hd)
        self._xbuf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        grp = self.group if self.group is not None else dist.group.WORLD
        self._xhdl = symm_mem.rendezvous(self._xbuf, grp)
        ptrs = [int(x) for x in self._xhdl.buffer_ptrs]
        if len(ptrs) != self.world:
            raise RuntimeError("symmetric memory rendezvous returned an unexpected number of peers")
        # clear this rank's buffer and put the mapped peer addresses where the kernel reads them
        # (arc_sdpa_exchange_init: the same call a C or C++ host makes)
        self._peers = torch.empty(self.world, dtype=torch.int64, device=device)
        _lib, L = _clib()
        host_ptrs = (C.c_uint64 * self.world)(*ptrs)
        with torch.cuda.device(device):
            _lib.check(L.arc_sdpa_exchange_init(self._xbuf.data_ptr(), self.world, self.batch, self.nq, self.hd, host_ptrs,
                                                self._peers.data_ptr(), torch.cuda.current_stream(device).cuda_stream),
                       "arc_sdpa_exchange_init")
        torch.cuda.synchronize(device)
        dist.barrier(group=self.group)  # every rank's flags are zero before anyone stores to them

    def __call__(self, q, k_local, v_local, *, scale, kv_len=None, gate=None):
        ops = self._ops
        if self.mode == "peer":
            self.step += 1
            return ops.sdpa_decode(q, k_local, v_local, scale=scale, kv_len=kv_len, gate=gate, out=self.out,
                                   exchange=(self._peers, self.world, self.rank, self.step))
        if self.world == 1:  # nothing to exchange: the plain decode call
            return ops.sdpa_decode(q, k_local, v_local, scale=scale, kv_len=kv_len, gate=gate, out=self.out)
        ops.sdpa_decode(q, k_local, v_local, scale=scale, kv_len=kv_len, return_partial=True, want_out=False,
                        partial_out=self.part_out, partial_lse=self.part_lse)
        dist.all_gather_into_tensor(self.gathered.view(-1), self.record, group=self.group)
        return ops.sdpa_merge(self.all_out, self.all_lse, gate=gate, out=self.out)


class GatheredPrefill:
    """Head/batch-sharded prefill whose output every rank ends up holding whole, without a collective:
    the gather buffer ``(world, *out_local.shape)`` lives in symmetric memory, and the prefill kernel's
    epilogue stores this rank's slice into slot ``rank`` of every rank's buffer (its own directly, the
    others' through their mapped addresses over NVLink) while it computes.  A rank's slice is in place
    everywhere once its call has completed; ``wait_all()`` is the cross-rank barrier a consumer needs
    before it reads the other slots."""

    def __init__(self, out_local_shape, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        shape = (self.world,) + tuple(out_local_shape)
        numel = 1
        for s in shape:
            numel *= s
        self.copies = None
        if self.world > 1:
            flat = symm_mem.empty(numel, dtype=torch.bfloat16, device=device)
            hdl = symm_mem.rendezvous(flat, group if group is not None else dist.group.WORLD)
            ptrs = [int(x) for x in hdl.buffer_ptrs]
            if len(ptrs) != self.world:
                raise RuntimeError("symmetric memory rendezvous returned an unexpected number of peers")
            slot_bytes = (numel // self.world) * 2
            self.copies = torch.tensor([ptrs[r] + self.rank * slot_bytes for r in range(self.world) if r != self.rank],
                                       dtype=torch.int64, device=device)
            self._flat, self._hdl = flat, hdl
        else:
            flat = torch.empty(numel, dtype=torch.bfloat16, device=device)
        self.gathered = flat.view(shape)

    def __call__(self, q_local, k_local, v_local, *, scale, mask_type, window, gate_local=None):
        from . import ops
        return ops.sdpa_prefill(q_local, k_local, v_local, scale=scale, mask_type=mask_type, window=window,
                                gate=gate_local, out=self.gathered[self.rank], out_copies=self.copies)

    def wait_all(self):
        """Every rank's slice has landed in this rank's buffer (host-side: stream sync + barrier)."""
        torch.cuda.current_stream().synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)
        return self.gathered


def prefill_head_sharded(q_local, k_local, v_local, *, scale, mask_type, window, gate_local=None, out_local=None,
                         gather_into: Optional[torch.Tensor] = None, group: Optional[dist.ProcessGroup] = None):
    """Prefill on this rank's head/batch shard; optionally all-gather the output slices.

    ``gather_into``: (world, *out_local.shape) bf16 buffer; when given, every
    rank ends up with all slices (slice r = what rank r computed).
    """
    from . import ops
    out_local = ops.sdpa_prefill(q_local, k_local, v_local, scale=scale, mask_type=mask_type, window=window,
                                 gate=gate_local, out=out_local)
    if gather_into is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_gather_into_tensor(gather_into.view(-1), out_local.contiguous().view(-1), group=group)
    return out_local
