"""Host logic of the multi-GPU partitions, run as world_size-2 gloo ranks on CPU.

The local attention of each rank is played by the CPU checker (test only); what is
under test is the partition planning, the packed record layout, the all-gather and
the merge identity that the GPU path uses unchanged."""
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

from arcaine_b200 import sharded  # noqa: E402


def test_plan_head_shards_covers_everything_once():
    for nq, nkv, batch, world in [(32, 16, 4, 1), (32, 16, 4, 2), (32, 16, 4, 8), (16, 8, 1, 8), (16, 2, 4, 8),
                                  (24, 4, 64, 8), (8, 4, 1, 8)]:
        shards = sharded.plan_head_shards(nq, nkv, batch, world)
        assert len(shards) == world
        seen = set()
        for s in shards:
            assert (s.q_head_end - s.q_head_begin) == (s.kv_head_end - s.kv_head_begin) * (nq // nkv)
            for b in range(s.batch_begin, s.batch_end):
                for h in range(s.kv_head_begin, s.kv_head_end):
                    assert (b, h) not in seen
                    seen.add((b, h))
        assert len(seen) == batch * nkv


def test_plan_seq_shards():
    for kv_len, world in [(524288, 8), (1000, 3), (63, 4), (1, 2)]:
        r = sharded.plan_seq_shards(kv_len, world)
        assert r[0][0] == 0 and r[-1][1] == kv_len
        for (a, b), (c, d) in zip(r[:-1], r[1:]):
            assert b == c and a <= b
        assert all(a % 64 == 0 for a, _ in r if a < kv_len)


def test_record_views_alias_the_packed_buffer():
    B, nq, hd = 3, 5, 128
    n = sharded.record_numel(B, nq, hd)
    assert n % 4 == 0 and n >= B * nq * (hd + 1)
    rec = torch.zeros(2, n)
    out, lse = sharded.split_record(rec, B, nq, hd)
    assert out.shape == (2, B, nq, hd) and lse.shape == (2, B, nq)
    out[1, 2, 4, 127] = 7.0
    lse[1, 0, 0] = 3.0
    assert rec[1, B * nq * hd - 1] == 7.0 and rec[1, B * nq * hd] == 3.0


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, fail_rank):
    import oracle
    from helpers import seeded_bf16
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, nq, nkv, hd, L = 2, 8, 2, 128, 333
        scale = hd ** -0.5
        q = seeded_bf16(B, nq, hd, seed=1)
        k = seeded_bf16(B, L, nkv, hd, seed=2)
        v = seeded_bf16(B, L, nkv, hd, seed=3)
        # --- sequence-sharded decode: local partial -> packed record -> all-gather -> merge
        lo, hi = sharded.plan_seq_shards(L, world)[rank]
        rec = torch.zeros(sharded.record_numel(B, nq, hd))
        p_out, p_lse = sharded.split_record(rec, B, nq, hd)
        for b in range(B):
            if hi > lo:
                o, _, l = oracle.sdpa_f32(q[b:b + 1], k[b, lo:hi], v[b, lo:hi], scale=scale, want_lse=True)
                p_out[b], p_lse[b] = o[0], l[0]
            else:
                p_out[b], p_lse[b] = 0.0, float("-inf")
        gathered = sharded.exchange_records(rec)
        assert gathered.shape == (world, rec.numel())
        a_out, a_lse = sharded.split_record(gathered, B, nq, hd)
        merged, _ = oracle.merge_partials(a_out.reshape(world, B * nq, hd).contiguous(),
                                          a_lse.reshape(world, B * nq).contiguous())
        for b in range(B):
            want, _ = oracle.sdpa_f32(q[b:b + 1], k[b], v[b], scale=scale)
            assert torch.allclose(merged.view(B, nq, hd)[b], want[0], atol=3e-6), "merge differs from unsplit attention"
        # --- head-sharded prefill: each rank computes its heads; gather reproduces the whole
        S = 9
        qp = seeded_bf16(S, nq, hd, seed=4)
        sh = sharded.plan_head_shards(nq, nkv, 1, world)[rank]
        mine, _ = oracle.sdpa_f32(qp[:, sh.q_head_begin:sh.q_head_end].contiguous(),
                                  k[0][:, sh.kv_head_begin:sh.kv_head_end].contiguous(),
                                  v[0][:, sh.kv_head_begin:sh.kv_head_end].contiguous(), scale=scale, mask_type=3)
        parts = torch.empty(world, *mine.shape)
        dist.all_gather_into_tensor(parts.view(-1), mine.contiguous().view(-1))
        whole, _ = oracle.sdpa_f32(qp, k[0], v[0], scale=scale, mask_type=3)
        assert torch.allclose(torch.cat(list(parts), dim=1), whole, atol=1e-6)
        # --- a rank that fails between steps is seen by the others on the host, before the next launch
        assert sharded.all_ranks_ok(rank != fail_rank) == (fail_rank < 0)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fail_rank", [-1, 1])
def test_world2_gloo(fail_rank):
    port = _free_port()
    mp.spawn(_rank_main, args=(2, port, fail_rank), nprocs=2, join=True)


def test_plan_batch_shards_balances_keys():
    """Longest-first dealing: the heaviest rank stays close to the mean where dealing by count does not."""
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(1024, 32769, (64,), generator=g).tolist()
    for world in (1, 2, 4, 8):
        owned = sharded.plan_batch_shards(lens, world)
        assert sorted(i for o in owned for i in o) == list(range(64))
        loads = [sum(lens[i] for i in o) for o in owned]
        assert max(loads) <= 1.03 * (sum(lens) / world)
        assert all(o == sorted(o) for o in owned)
    by_count = [sum(lens[i] for i in range(r * 8, r * 8 + 8)) for r in range(8)]
    assert max(by_count) > 1.1 * (sum(lens) / 8)  # what the rule replaces
    # more ranks than sequences: the extra ranks own nothing
    owned = sharded.plan_batch_shards([5, 9], 4)
    assert sorted(map(tuple, owned)) == [(), (), (0,), (1,)]


def test_plan_seq_shards_short_sequence_leaves_empty_ranks():
    shards = sharded.plan_seq_shards(100, 8)
    assert shards[0] == (0, 64) and shards[1] == (64, 100)
    assert all(s == (100, 100) for s in shards[2:])
    assert sharded.all_ranks_ok(True) and not sharded.all_ranks_ok(False)  # no process group: local answer


def test_c_planners_against_a_plain_restatement():
    """The planners are C functions of the library (a C++ host uses the same ones); here against the
    rules written out in Python."""
    for nq, nkv, batch, world in [(32, 16, 4, 1), (32, 16, 4, 2), (32, 16, 4, 8), (16, 8, 1, 8), (24, 4, 64, 8), (6, 3, 5, 4), (8, 8, 3, 16)]:
        group = nq // nkv
        head_ways = max(d for d in range(1, world + 1) if world % d == 0 and nkv % d == 0)
        batch_ways, heads_per = world // head_ways, nkv // head_ways
        got = sharded.plan_head_shards(nq, nkv, batch, world)
        for r, sh in enumerate(got):
            hw, bw = r % head_ways, r // head_ways
            b0 = min(batch, (batch * bw + batch_ways - 1) // batch_ways)
            b1 = min(batch, (batch * (bw + 1) + batch_ways - 1) // batch_ways)
            assert (sh.kv_head_begin, sh.kv_head_end) == (hw * heads_per, (hw + 1) * heads_per)
            assert (sh.q_head_begin, sh.q_head_end) == (hw * heads_per * group, (hw + 1) * heads_per * group)
            assert (sh.batch_begin, sh.batch_end) == (b0, b1)
        # every (kv head, sequence) pair is owned exactly once
        owned = sorted((h, b) for sh in got for h in range(sh.kv_head_begin, sh.kv_head_end)
                       for b in range(sh.batch_begin, sh.batch_end))
        assert owned == sorted((h, b) for h in range(nkv) for b in range(batch))
    for kv_len, world, align in [(524288, 8, 64), (5000, 2, 64), (100, 8, 64), (1000, 3, 16), (0, 4, 64)]:
        per = -(-kv_len // world)
        per = -(-per // align) * align
        want = [(min(kv_len, r * per), min(kv_len, (r + 1) * per)) for r in range(world)]
        assert sharded.plan_seq_shards(kv_len, world, align) == want
    assert sharded.record_numel(4, 16, 128) == 4 * 16 * 128 + 4 * 16
    assert sharded.record_numel(3, 5, 128) % 4 == 0
    with pytest.raises(Exception):
        sharded.plan_seq_shards(-1, 2)
