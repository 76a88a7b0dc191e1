"""The benchmark configurations at full size.  Inputs are seeded N(0,1) bf16 drawn on the device;
the rows the CPU oracle checks are copied back bit for bit, so both sides see identical values.
Full-size cases are checked on a sample of output rows plus size-independent properties."""
import pytest
import torch

from helpers import assert_close, sample_rows
import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from arcaine_b200 import ops as o
    o.clear_device_status()
    yield o
    assert o.device_status() == (0, 0)


def dev_randn(*shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(*shape, generator=g, device="cuda", dtype=torch.float32).bfloat16()


def test_config3_sliding_window_prefill_full_size(ops):
    """batch 4, 32Q/16KV, hd128, seq 8192, causal window 1024."""
    B, S, nq, nkv, hd, W = 4, 8192, 32, 16, 128, 1024
    q, k, v = dev_randn(B, S, nq, hd, seed=3), dev_randn(B, S, nkv, hd, seed=4), dev_randn(B, S, nkv, hd, seed=5)
    out = ops.sdpa_prefill(q, k, v, scale=hd ** -0.5, mask_type=ops.MASK_CAUSAL, window=W)
    torch.cuda.synchronize()
    for b in range(B):
        rows = sample_rows(S, nq, 600, seed=30 + b)
        want, _ = oracle.sdpa_f32(q[b].cpu(), k[b].cpu(), v[b].cpu(), scale=hd ** -0.5, mask_type=3, window=W, rows=rows)
        assert_close(out[b].reshape(-1, hd)[rows], want, f"sequence {b}")
    # property: keys outside every window do not matter — perturbing the first 1024 keys of a
    # sequence leaves the outputs of queries >= 2047 bit-identical
    k2, v2 = k.clone(), v.clone()
    k2[1, :1024] = dev_randn(1024, nkv, hd, seed=6)
    v2[1, :1024] = dev_randn(1024, nkv, hd, seed=7)
    out2 = ops.sdpa_prefill(q, k2, v2, scale=hd ** -0.5, mask_type=ops.MASK_CAUSAL, window=W)
    assert torch.equal(out2[1, 2047:], out[1, 2047:])
    assert not torch.equal(out2[1, :1024], out[1, :1024])
    assert torch.equal(out2[0], out[0])
    # property: sequences are independent and heads depend only on their own KV head
    # (eight query heads, so that the sub-problem is still large enough for the same kernel)
    solo = ops.sdpa_prefill(q[2:3, :, 8:16].contiguous(), k[2:3, :, 4:8].contiguous(), v[2:3, :, 4:8].contiguous(),
                            scale=hd ** -0.5, mask_type=ops.MASK_CAUSAL, window=W)
    assert torch.equal(solo[0], out[2, :, 8:16])


def test_config4_gated_decode_full_size(ops):
    """batch 64, 24Q/4KV, hd256, kv_len uniform random in [1024, 32768], sigmoid gate."""
    B, nq, nkv, hd = 64, 24, 4, 256
    g = torch.Generator().manual_seed(4)
    lens = torch.randint(1024, 32769, (B,), generator=g, dtype=torch.int32)
    offs = torch.zeros(B, dtype=torch.int64)
    offs[1:] = torch.cumsum(lens[:-1].long(), 0)
    total = int(lens.sum())
    k, v = dev_randn(total, nkv, hd, seed=41), dev_randn(total, nkv, hd, seed=42)
    q, gate = dev_randn(B, nq, hd, seed=43), dev_randn(B, nq, hd, seed=44)
    out = ops.sdpa_decode(q, k, v, scale=hd ** -0.5, kv_len=lens.cuda(), kv_row_offset=offs.cuda(), gate=gate)
    plain, o32, lse = ops.sdpa_decode(q, k, v, scale=hd ** -0.5, kv_len=lens.cuda(), kv_row_offset=offs.cuda(),
                                      return_partial=True)
    torch.cuda.synchronize()
    shortest, longest = int(torch.argmin(lens)), int(torch.argmax(lens))
    for b in sorted({0, 9, 17, 26, 40, 55, 63, shortest, longest}):
        o0, n = int(offs[b]), int(lens[b])
        _, want, wl = oracle.sdpa_f32(q[b:b + 1].cpu(), k[o0:o0 + n].cpu(), v[o0:o0 + n].cpu(), scale=hd ** -0.5,
                                      gate=gate[b:b + 1].cpu(), want_lse=True)
        assert_close(out[b], want[0].float(), f"sequence {b} (len {n})")
        assert torch.allclose(lse[b].cpu(), wl[0], atol=2e-3)
    # property: the fused gate equals the reference's two launches on the ungated result
    two = plain.clone()
    ops.mul_sigmoid_inplace(two, gate)
    assert torch.equal(two, out)


def test_config5_long_context_decode_full_size(ops):
    """batch 4, 16Q/2KV, hd128, KV length 524288; also the 8-way sequence sharding emulated on one GPU."""
    from arcaine_b200 import sharded
    B, nq, nkv, hd, L = 4, 16, 2, 128, 524288
    k, v = dev_randn(B, L, nkv, hd, seed=51), dev_randn(B, L, nkv, hd, seed=52)
    q = dev_randn(B, nq, hd, seed=53)
    scale = hd ** -0.5
    out = ops.sdpa_decode(q, k, v, scale=scale)
    torch.cuda.synchronize()
    for b in range(B):  # every sequence, all sixteen heads (both KV groups)
        want, _ = oracle.sdpa_f32(q[b:b + 1].cpu(), k[b].cpu(), v[b].cpu(), scale=scale)
        assert_close(out[b], want[0], f"sequence {b}")
    world = 8
    n = sharded.record_numel(B, nq, hd)
    gathered = torch.zeros(world, n, device="cuda")
    for r, (lo, hi) in enumerate(sharded.plan_seq_shards(L, world)):
        po, pl = sharded.split_record(gathered[r], B, nq, hd)
        ops.sdpa_decode(q, k[:, lo:hi], v[:, lo:hi], scale=scale, return_partial=True, want_out=False,
                        partial_out=po, partial_lse=pl)
    merged = ops.sdpa_merge(*sharded.split_record(gathered, B, nq, hd))
    assert_close(merged, out.float(), "8 merged slices vs one pass", rel_tol=4e-3, abs_tol=2e-3)
