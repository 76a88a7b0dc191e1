"""Sequence-sharded decode and head-sharded prefill on 2 GPUs (one process per GPU, NCCL plumbing).
Skipped on boxes with fewer than 2 GPUs.  The exchange of partial (out, lse) records is checked
both ways — in-kernel over NVLink peer memory, and NCCL all-gather + merge — against the
single-GPU kernel over the whole key range and against the CPU oracle."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import oracle
    from helpers import assert_close, seeded_bf16
    from arcaine_b200 import ops, sharded
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        B, nq, nkv, hd, L = 3, 16, 2, 128, 5000
        scale = hd ** -0.5
        q = seeded_bf16(B, nq, hd, seed=1)
        k, v = seeded_bf16(B, L, nkv, hd, seed=2), seeded_bf16(B, L, nkv, hd, seed=3)
        gate = seeded_bf16(B, nq, hd, seed=4)
        lo, hi = sharded.plan_seq_shards(L, world)[rank]
        qd, gd = q.to(dev), gate.to(dev)
        kl, vl = k[:, lo:hi].contiguous().to(dev), v[:, lo:hi].contiguous().to(dev)
        whole = ops.sdpa_decode(qd, k.to(dev), v.to(dev), scale=scale, gate=gd)
        results = {}
        for mode in ("nccl", "peer"):
            try:
                runner = sharded.SeqShardedDecode(B, nq, hd, dev, exchange=mode)
            except Exception as e:
                if mode == "peer":
                    print(f"rank {rank}: peer exchange unavailable: {e!r}", flush=True)
                    continue
                raise
            for step in range(3):  # several steps: flags, parities and step numbers keep working
                out = runner(qd, kl, vl, scale=scale, gate=gd)
            torch.cuda.synchronize()
            results[mode] = out.clone()
            assert_close(out, whole.float(), f"{mode}: merged slices vs one pass", rel_tol=4e-3, abs_tol=4e-3)
        assert ops.device_status() == (0, 0)
        if rank == 0:
            for b in range(B):
                _, want = oracle.sdpa_f32(q[b:b + 1], k[b], v[b], scale=scale, gate=gate[b:b + 1])
                for mode, out in results.items():
                    assert_close(out[b:b + 1], want.float(), f"{mode} seq {b} vs oracle")
        # the C-side collective wrapper with an ncclComm_t of the caller's own (as a C++ host has one): a
        # communicator made through the NCCL library already in the process, its id broadcast by torch
        import ctypes as C
        from arcaine_b200 import _lib
        nccl = C.CDLL("libnccl.so.2")

        class UniqueId(C.Structure):
            _fields_ = [("internal", C.c_byte * 128)]

        uid = UniqueId()
        if rank == 0:
            assert nccl.ncclGetUniqueId(C.byref(uid)) == 0
        idt = torch.frombuffer(bytearray(bytes(uid)), dtype=torch.uint8).to(dev)
        dist.broadcast(idt, src=0)
        C.memmove(C.byref(uid), bytes(idt.cpu().numpy().tobytes()), 128)
        comm = C.c_void_p()
        nccl.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, UniqueId, C.c_int]
        assert nccl.ncclCommInitRank(C.byref(comm), world, uid, rank) == 0
        L_ = _lib.load()
        n = L_.arc_sdpa_record_floats(B, nq, hd)
        assert n == sharded.record_numel(B, nq, hd)
        record = torch.zeros(n, dtype=torch.float32, device=dev)
        gathered = torch.zeros(world * n, dtype=torch.float32, device=dev)
        p_out, p_lse = sharded.split_record(record, B, nq, hd)
        ops.sdpa_decode(qd, kl, vl, scale=scale, return_partial=True, want_out=False, partial_out=p_out, partial_lse=p_lse)
        c_out = torch.empty(B, nq, hd, dtype=torch.bfloat16, device=dev)
        rc = L_.arc_sdpa_allgather_merge(record.data_ptr(), gathered.data_ptr(), world, B, nq, hd, gd.data_ptr(),
                                         c_out.data_ptr(), comm, torch.cuda.current_stream().cuda_stream)
        assert rc == _lib.ARC_OK, rc
        torch.cuda.synchronize()
        assert_close(c_out, whole.float(), "arc_sdpa_allgather_merge vs one pass", rel_tol=4e-3, abs_tol=4e-3)
        assert torch.equal(c_out, results["nccl"])  # the same collective and the same merge as the torch path
        assert L_.arc_sdpa_allgather_merge(record.data_ptr(), gathered.data_ptr(), world, B, nq, hd, None,
                                           c_out.data_ptr(), None, None) == _lib.ARC_ERR_NULL_POINTER
        nccl.ncclCommDestroy.argtypes = [C.c_void_p]
        nccl.ncclCommDestroy(comm)
        # head-sharded prefill: each rank its KV heads; gathered slices equal the whole
        S = 300
        qp = seeded_bf16(S, nq, hd, seed=5)
        sh = sharded.plan_head_shards(nq, nkv, 1, world)[rank]
        mine = ops.sdpa_prefill(qp[:, sh.q_head_begin:sh.q_head_end].contiguous().to(dev),
                                k[0, :S, sh.kv_head_begin:sh.kv_head_end].contiguous().to(dev),
                                v[0, :S, sh.kv_head_begin:sh.kv_head_end].contiguous().to(dev),
                                scale=scale, mask_type=ops.MASK_CAUSAL, window=100)
        parts = torch.empty((world, *mine.shape), dtype=mine.dtype, device=dev)
        sharded.prefill_head_sharded(qp[:, sh.q_head_begin:sh.q_head_end].contiguous().to(dev),
                                     k[0, :S, sh.kv_head_begin:sh.kv_head_end].contiguous().to(dev),
                                     v[0, :S, sh.kv_head_begin:sh.kv_head_end].contiguous().to(dev),
                                     scale=scale, mask_type=ops.MASK_CAUSAL, window=100, gather_into=parts)
        torch.cuda.synchronize()
        if rank == 0:
            want, _ = oracle.sdpa_f32(qp, k[0, :S], v[0, :S], scale=scale, mask_type=3, window=100)
            assert_close(torch.cat(list(parts), dim=1), want, "gathered head shards")
        # the same gather done by the kernel's own epilogue: every rank's rows stored into every rank's
        # buffer over NVLink (symmetric memory), no collective; a large case as well, so that both prefill
        # kernels take part
        for S2, win in ((300, 100), (2048, 512)):
            q2 = seeded_bf16(S2, nq, hd, seed=6)
            args = (q2[:, sh.q_head_begin:sh.q_head_end].contiguous().to(dev),
                    k[0, :S2, sh.kv_head_begin:sh.kv_head_end].contiguous().to(dev),
                    v[0, :S2, sh.kv_head_begin:sh.kv_head_end].contiguous().to(dev))
            ref = ops.sdpa_prefill(*args, scale=scale, mask_type=ops.MASK_CAUSAL, window=win)
            gp = sharded.GatheredPrefill(tuple(ref.shape), dev)
            local = gp(*args, scale=scale, mask_type=ops.MASK_CAUSAL, window=win)
            both = gp.wait_all()
            assert torch.equal(local, ref) and torch.equal(both[rank], ref)
            theirs = [torch.empty_like(ref) for _ in range(world)]
            dist.all_gather(theirs, ref)
            for r in range(world):
                assert torch.equal(both[r], theirs[r]), f"slot {r} of rank {rank}'s buffer (S {S2})"
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_rank_main, args=(2, _free_port()), nprocs=2, join=True)
