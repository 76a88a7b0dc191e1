"""Parity of the split-KV decode kernel and the LSE merge with the CPU oracle, through the C ABI."""
import ctypes as C

import pytest
import torch

from helpers import assert_close, seeded_bf16
import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from arcaine_b200 import ops as o
    o.clear_device_status()
    yield o
    assert o.device_status() == (0, 0), "a bounded device-side wait gave up during the decode tests"


def oracle_decode(q, k_rows, v_rows, scale, gate=None):
    """q (nq, hd), k/v (len, nkv, hd) -> (f32 out, bf16 out, lse)."""
    return oracle.sdpa_f32(q[None], k_rows, v_rows, scale=scale, gate=gate[None] if gate is not None else None,
                           want_lse=True)


@pytest.mark.parametrize("B,nq,nkv,hd,lens", [
    (1, 8, 2, 128, [37]),
    (2, 8, 2, 128, [100, 300]),
    (3, 24, 4, 256, [17, 1000, 257]),
    (2, 16, 2, 128, [5000, 1]),
    (4, 6, 1, 256, [64, 65, 63, 1024]),
    (2, 32, 2, 128, [333, 77]),       # 16 query heads per KV head: two n-tiles
    (2, 32, 16, 128, [200, 31]),      # 16 KV heads: two head groups per key share
    (3, 4, 4, 256, [0, 50, 0]),       # empty sequences give zeros
])
def test_variable_lengths_block_cache(ops, B, nq, nkv, hd, lens):
    cap = max(max(lens), 1) + 5
    q = seeded_bf16(B, nq, hd, seed=1)
    k, v = seeded_bf16(B, cap, nkv, hd, seed=2), seeded_bf16(B, cap, nkv, hd, seed=3)
    g = seeded_bf16(B, nq, hd, seed=4)
    kd, vd = k.cuda(), v.cuda()
    # rows past each sequence's length are never-written cache: poison them
    for b, n in enumerate(lens):
        kd[b, n:] = float("nan")
        vd[b, n:] = float("nan")
    kl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    scale = hd ** -0.5
    out, o32, lse = ops.sdpa_decode(q.cuda(), kd, vd, scale=scale, kv_len=kl, return_partial=True)
    outg = ops.sdpa_decode(q.cuda(), kd, vd, scale=scale, kv_len=kl, gate=g.cuda())
    for b, n in enumerate(lens):
        if n == 0:
            assert torch.count_nonzero(out[b].float()) == 0 and torch.isinf(lse[b]).all()
            continue
        wf, wb, wl = oracle_decode(q[b], k[b, :n], v[b, :n], scale)
        assert_close(out[b], wf[0], f"seq {b} len {n}")
        assert_close(o32[b], wf[0], f"seq {b} f32", rel_tol=3e-3, abs_tol=5e-3)
        assert torch.allclose(lse[b].cpu(), wl[0], atol=2e-3)
        _, wgb, _ = oracle_decode(q[b], k[b, :n], v[b, :n], scale, gate=g[b])
        assert_close(outg[b], wgb[0].float(), f"seq {b} gated")


def test_packed_cache_with_row_offsets_and_cta_counts(ops):
    B, nq, nkv, hd = 5, 24, 4, 256
    lens = [700, 33, 1500, 1, 260]
    offs = [0]
    for n in lens[:-1]:
        offs.append(offs[-1] + n)
    total = sum(lens)
    q = seeded_bf16(B, nq, hd, seed=11)
    k, v = seeded_bf16(total, nkv, hd, seed=12), seeded_bf16(total, nkv, hd, seed=13)
    kl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    ko = torch.tensor(offs, dtype=torch.int64, device="cuda")
    want = [oracle_decode(q[b], k[offs[b]:offs[b] + lens[b]], v[offs[b]:offs[b] + lens[b]], 0.0625)[0][0] for b in range(B)]
    for nctas in (0, 1, 3, 148, 500):
        out = ops.sdpa_decode(q.cuda(), k.cuda(), v.cuda(), scale=0.0625, kv_len=kl, kv_row_offset=ko, num_ctas=nctas)
        for b in range(B):
            assert_close(out[b], want[b], f"num_ctas {nctas} seq {b}")


def test_qwen_single_token_entry_points(ops):
    """seq == 1 through the reference-named calls, bench-recipe inputs, against the restated scalar kernel."""
    nq, nkv, hd, depth = 24, 4, 256, 512
    state = 42
    qb, state = oracle.lcg_fill(nq * hd, state)
    kb, state = oracle.lcg_fill((depth + 1) * nkv * hd, state)
    vb, state = oracle.lcg_fill((depth + 1) * nkv * hd, state)
    gb, state = oracle.lcg_fill(nq * hd, state)
    q = oracle.bits_to_bf16(qb).reshape(1, nq, hd)
    k = oracle.bits_to_bf16(kb).reshape(depth + 1, nkv, hd)
    v = oracle.bits_to_bf16(vb).reshape(depth + 1, nkv, hd)
    g = oracle.bits_to_bf16(gb).reshape(1, nq, hd)
    want = oracle.qwen35_online_attention(q, k, v, seq=1, past=depth, scale=0.0625)
    buf = q.cuda().clone()
    ops.qwen35_xmx_attention(buf, k.cuda(), v.cuda(), buf, 1, depth, nq, nkv, hd, 0.0625)  # out aliases q
    assert_close(buf, want.float(), "qwen35_xmx_attention seq=1")
    out = torch.empty_like(buf)
    ops.qwen35_xmx_attention_decode_gqa(q.cuda(), k.cuda(), v.cuda(), out, depth, nq, nkv, hd, 0.0625, gate=g.cuda())
    assert_close(out, oracle.mul_sigmoid_inplace(want, g).float(), "decode_gqa + gate")
    # the unfused pair of launches gives the same thing
    ops.mul_sigmoid_inplace(buf, g.cuda())
    assert_close(buf, oracle.mul_sigmoid_inplace(want, g).float(), "attention then mul_sigmoid_inplace")


def test_merge_kernel_against_oracle(ops):
    P, rows, hd = 5, 37, 128
    g = torch.Generator().manual_seed(5)
    po = torch.randn(P, rows, hd, generator=g)
    pl = torch.randn(P, rows, generator=g) * 3
    pl[2] = float("-inf")           # an empty part
    pl[:, 7] = float("-inf")        # a row nobody covers
    gate = seeded_bf16(rows, hd, seed=6)
    want, want_lse = oracle.merge_partials(po, pl)
    out, o32, lse = ops.sdpa_merge(po.cuda(), pl.cuda(), want_f32=True, want_lse=True)
    assert torch.allclose(o32.cpu(), want, atol=1e-5)
    fin = torch.isfinite(want_lse)
    assert torch.allclose(lse.cpu()[fin], want_lse[fin], atol=1e-5) and torch.isinf(lse.cpu()[~fin]).all()
    assert_close(out, want, "bf16 merge", rel_tol=4e-3, abs_tol=2e-2)
    gated = ops.sdpa_merge(po.cuda(), pl.cuda(), gate=gate.cuda())
    assert_close(gated, oracle.mul_sigmoid_inplace(want.bfloat16(), gate).float(), "gated merge", rel_tol=4e-3)
    # strided parts: one packed [out | lse] record per part, merged in place
    from arcaine_b200 import sharded
    n = sharded.record_numel(1, rows, hd)
    rec = torch.zeros(P, n, device="cuda")
    ro, rl = sharded.split_record(rec, 1, rows, hd)
    ro.copy_(po.cuda().view(P, 1, rows, hd))
    rl.copy_(pl.cuda().view(P, 1, rows))
    out2 = ops.sdpa_merge(ro, rl)
    assert torch.equal(out2.view(rows, hd), out)


def test_sequence_sharded_partials_merge_to_the_whole(ops):
    """What each GPU of a sequence-sharded decode computes, emulated on one device: partial
    (out, lse) per key slice, then the merge — must equal decode over the whole range."""
    from arcaine_b200 import sharded
    B, nq, nkv, hd, L, world = 2, 16, 2, 128, 3000, 4
    q = seeded_bf16(B, nq, hd, seed=21)
    k, v = seeded_bf16(B, L, nkv, hd, seed=22), seeded_bf16(B, L, nkv, hd, seed=23)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    n = sharded.record_numel(B, nq, hd)
    gathered = torch.zeros(world, n, device="cuda")
    for r, (lo, hi) in enumerate(sharded.plan_seq_shards(L, world)):
        po, pl = sharded.split_record(gathered[r], B, nq, hd)
        ops.sdpa_decode(qd, kd[:, lo:hi], vd[:, lo:hi], scale=0.09, return_partial=True, want_out=False,
                        partial_out=po, partial_lse=pl)
    ao, al = sharded.split_record(gathered, B, nq, hd)
    merged = ops.sdpa_merge(ao, al)
    whole = ops.sdpa_decode(qd, kd, vd, scale=0.09)
    assert_close(merged, whole.float(), "merged vs unsplit kernel", rel_tol=3e-3, abs_tol=4e-3)
    for b in range(B):
        assert_close(merged[b], oracle_decode(q[b], k[b], v[b], 0.09)[0][0], f"seq {b}")


def test_error_statuses(ops):
    from arcaine_b200 import _lib
    q = torch.zeros(2, 34, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(2, 64, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.ArcError) as e:
        ops.sdpa_decode(q, k, k, scale=1.0)
    assert e.value.status == _lib.ARC_ERR_UNSUPPORTED_GQA
    q = torch.zeros(2, 4, 64, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(2, 64, 2, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.ArcError) as e:
        ops.sdpa_decode(q, k, k, scale=1.0)
    assert e.value.status == _lib.ARC_ERR_UNSUPPORTED_HEAD_DIM
    # raw ABI: workspace too small
    q = torch.zeros(2, 4, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(2, 64, 2, 128, dtype=torch.bfloat16, device="cuda")
    p = _lib.DecodeParams()
    p.q, p.k, p.v, p.out = q.data_ptr(), k.data_ptr(), k.data_ptr(), q.data_ptr()
    p.batch, p.nq, p.nkv, p.hd, p.kv_len_uniform, p.max_kv_len = 2, 4, 2, 128, 64, 64
    p.q_stride_b = p.o_stride_b = 512
    p.kv_stride_b, p.kv_stride_t, p.kv_rows_total, p.scale = 64, 256, 128, 1.0
    L = _lib.load()
    assert L.arc_sdpa_decode_workspace_bytes(C.byref(p)) > 0
    ws = torch.zeros(64, dtype=torch.uint8, device="cuda")
    p.workspace, p.workspace_bytes = ws.data_ptr(), 64
    assert L.arc_sdpa_decode(C.byref(p), None) == _lib.ARC_ERR_WORKSPACE_TOO_SMALL


def test_peer_wait_gives_up_with_a_status_and_the_device_stays_usable(ops):
    """Sequence-sharded decode on one GPU with a second "rank" whose records never come: the merge
    kernel's wait for them is bounded, expires (a few ms here), records FAULT_WAIT_PEER with the
    missing source rank and returns; while the status is set launches do nothing; after a clear the
    same call without the exchange is correct.  Nothing faults or hangs: the flag is simply never set."""
    B, nq, nkv, hd, n = 1, 4, 1, 128, 300
    q, k, v = seeded_bf16(B, nq, hd, seed=71), seeded_bf16(B, n, nkv, hd, seed=72), seeded_bf16(B, n, nkv, hd, seed=73)
    xbuf = torch.zeros(ops.exchange_bytes(2, B, nq, hd), dtype=torch.uint8, device="cuda")
    peers = torch.tensor([xbuf.data_ptr(), xbuf.data_ptr()], dtype=torch.int64, device="cuda")
    out = torch.full((B, nq, hd), 7.0, dtype=torch.bfloat16, device="cuda")
    ops.sdpa_decode(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, out=out, exchange=(peers, 2, 0, 1),
                    exchange_wait_cycles=20_000_000)
    assert ops.device_status() == (ops.FAULT_WAIT_PEER, 1)   # source rank 1 never raised its flag
    assert (out.float() == 7.0).all()                         # the merged result was never written
    # sticky: a launch made while the status is set returns at once without touching its output
    ops.sdpa_decode(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, out=out)
    torch.cuda.synchronize()
    assert (out.float() == 7.0).all()
    ops.clear_device_status()
    assert ops.device_status() == (0, 0)
    got = ops.sdpa_decode(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, out=out)
    wf, _, _ = oracle_decode(q[0], k[0], v[0], hd ** -0.5)
    assert_close(got[0], wf[0], "decode after the status was cleared")


def test_exchange_fold_with_the_other_ranks_record_already_in_place(ops):
    """The cross-rank fold of the sequence-sharded decode on one GPU, without two kernels waiting for each
    other: "rank 1"'s record is computed first (return_partial) and written into rank 0's exchange buffer
    in the wire format — 8-byte (value, step) words, log-sum-exp in word hd — then rank 0's call finds it
    there, never waits, and must produce the attention over both halves of the keys, gate included."""
    B, nq, nkv, hd, n, step = 2, 8, 2, 128, 700, 5
    q, k, v = seeded_bf16(B, nq, hd, seed=91), seeded_bf16(B, n, nkv, hd, seed=92), seeded_bf16(B, n, nkv, hd, seed=93)
    gate = seeded_bf16(B, nq, hd, seed=94)
    qd, kd, vd, gd = q.cuda(), k.cuda(), v.cuda(), gate.cuda()
    half = 384
    _, o1, l1 = ops.sdpa_decode(qd, kd[:, half:].contiguous(), vd[:, half:].contiguous(), scale=hd ** -0.5, return_partial=True)
    rows, words = B * nq, hd + 2
    assert ops.exchange_bytes(2, B, nq, hd) == 2 * 2 * rows * words * 8
    xbuf = torch.zeros(2, 2, rows, words, 2, dtype=torch.int32, device="cuda")  # [parity][source][row][word][value, step]
    rec = xbuf[step & 1, 1]
    rec[:, :hd, 0] = o1.reshape(rows, hd).contiguous().view(torch.int32)
    rec[:, hd, 0] = l1.reshape(rows).contiguous().view(torch.int32)
    rec[:, :, 1] = step
    scratch = torch.zeros_like(xbuf)  # where rank 0's words for "rank 1" go
    peers = torch.tensor([xbuf.data_ptr(), scratch.data_ptr()], dtype=torch.int64, device="cuda")
    out = ops.sdpa_decode(qd, kd[:, :half].contiguous(), vd[:, :half].contiguous(), scale=hd ** -0.5, gate=gd,
                          exchange=(peers, 2, 0, step), exchange_wait_cycles=20_000_000)
    assert ops.device_status() == (0, 0)
    whole = ops.sdpa_decode(qd, kd, vd, scale=hd ** -0.5, gate=gd)
    assert_close(out, whole.float(), "two halves folded vs one pass", rel_tol=4e-3, abs_tol=2e-3)
    for b in range(B):
        _, want, _ = oracle.sdpa_f32(q[b:b + 1], k[b], v[b], scale=hd ** -0.5, gate=gate[b:b + 1], want_lse=True)
        assert_close(out[b], want[0].float(), f"sequence {b}")
    # rank 0's own words went out to both buffers, tagged with the step
    assert (xbuf[step & 1, 0, :, :, 1] == step).all() and (scratch[step & 1, 0, :, :, 1] == step).all()


def test_device_side_length_past_the_cache_is_a_status_not_a_wrong_result(ops):
    from arcaine_b200 import _lib
    B, nq, nkv, hd, cap = 2, 8, 2, 128, 64
    q, k, v = seeded_bf16(B, nq, hd, seed=81), seeded_bf16(B, cap, nkv, hd, seed=82), seeded_bf16(B, cap, nkv, hd, seed=83)
    out = torch.full((B, nq, hd), 3.0, dtype=torch.bfloat16, device="cuda")
    bad = torch.tensor([cap, cap + 1], dtype=torch.int32, device="cuda")  # sequence 1 claims one row too many
    ops.sdpa_decode(q.cuda(), k.cuda(), v.cuda(), scale=0.1, kv_len=bad, out=out)
    assert ops.device_status() == (ops.FAULT_BAD_KV_RANGE, 1)
    code, detail = C.c_uint32(0), C.c_uint32(0)
    assert _lib.load().arc_sdpa_device_status(C.byref(code), C.byref(detail)) == _lib.ARC_ERR_DEVICE_BAD_RANGE
    assert (out.float() == 3.0).all()
    ops.clear_device_status()
    # known on the host: refused before anything is launched
    with pytest.raises(ValueError):
        ops.sdpa_decode(q.cuda(), k.cuda(), v.cuda(), scale=0.1, kv_len=cap + 1, out=out)
    good = torch.tensor([cap, 5], dtype=torch.int32, device="cuda")
    got = ops.sdpa_decode(q.cuda(), k.cuda(), v.cuda(), scale=0.1, kv_len=good, out=out)
    wf, _, _ = oracle_decode(q[1], k[1, :5], v[1, :5], 0.1)
    assert_close(got[1], wf[0], "decode after the status was cleared")


def test_empty_cache_slice_gives_empty_records(ops):
    """A sequence-sharded rank whose slice holds no keys still produces its records: zeros with lse = -inf."""
    B, nq, nkv, hd = 2, 8, 2, 128
    q = seeded_bf16(B, nq, hd, seed=91).cuda()
    k = torch.empty(B, 0, nkv, hd, dtype=torch.bfloat16, device="cuda")
    out, o32, lse = ops.sdpa_decode(q, k, k, scale=0.1, return_partial=True)
    assert torch.count_nonzero(out.float()) == 0 and torch.count_nonzero(o32) == 0
    assert torch.isinf(lse).all() and (lse < 0).all()
