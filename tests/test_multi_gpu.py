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
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpu_sharding():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    mp.spawn(_rank_main, args=(2, _free_port()), nprocs=2, join=True)
