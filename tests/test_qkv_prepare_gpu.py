"""RMSNorm + RoPE + KV-cache append in one launch, against the CPU restatement, through the C ABI."""
import pytest
import torch

from helpers import seeded_bf16
import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from arcaine_b200 import ops as o
    return o


def close_bf16(got, want, what):
    """At most one bf16 step apart (plus 2e-6 absolute: a rotation can cancel to nearly zero, where fp32
    rounding of the O(1) operands is all that is left), and only in a small share of the elements (the
    device sums the squares in fp32 with rsqrt.approx, the oracle in double)."""
    g, w = got.detach().cpu().float(), want.float()
    step = w.abs() * 2.0 ** -7 + 2e-6
    assert ((g - w).abs() <= step).all(), f"{what}: max diff {(g - w).abs().max().item()}"
    assert (g != w).float().mean().item() < 5e-3, f"{what}: too many one-step differences"


def rope_tables(seq, nap, hd, offset, theta=10000.0):
    p = torch.arange(nap).float()
    inv = 1.0 / torch.pow(torch.tensor(float(theta)), 2.0 * p / hd)
    ang = (torch.arange(seq).float() + offset)[:, None] * inv[None]
    return torch.cos(ang).contiguous(), torch.sin(ang).contiguous()


@pytest.mark.parametrize("hd,partial", [(128, 1.0), (256, 1.0), (256, 0.25), (512, 0.25)])
def test_table_mode_with_cache_append(ops, hd, partial):
    """Encoder call: Q in place; K normed + rotated and V unit-normed into the cache at past_len; rows outside
    the appended span untouched (src/modeling/diffusion_gemma/attention.cpp:1017-1020)."""
    seq, nq, nkv, past, cap = 70, 8, 4, 33, 128
    nap = int(partial * hd / 2.0)
    q, k, v = seeded_bf16(seq, nq, hd, seed=1), seeded_bf16(seq, nkv, hd, seed=2), seeded_bf16(seq, nkv, hd, seed=3)
    qw = (seeded_bf16(hd, seed=4).float() * 0.1 + 1.0).bfloat16()
    kw = (seeded_bf16(hd, seed=5).float() * 0.1 + 1.0).bfloat16()
    cos, sin = rope_tables(seq, nap, hd, past)
    kc = seeded_bf16(cap, nkv, hd, seed=6)
    vc = seeded_bf16(cap, nkv, hd, seed=7)
    qd, kcd, vcd = q.cuda(), kc.cuda(), vc.cuda()
    ops.qkv_prepare(qd, k.cuda(), v.cuda(), k_cache=kcd, v_cache=vcd, past_len=past, q_weight=qw.cuda(),
                    k_weight=kw.cuda(), eps=1e-6, partial_rotary_factor=partial, rope_cos=cos.cuda(), rope_sin=sin.cuda())
    close_bf16(qd, oracle.norm_rope(q, qw, eps=1e-6, n_active_pairs=nap, rope_cos=cos, rope_sin=sin), "Q")
    close_bf16(kcd[past:past + seq], oracle.norm_rope(k, kw, eps=1e-6, n_active_pairs=nap, rope_cos=cos, rope_sin=sin), "K")
    close_bf16(vcd[past:past + seq], oracle.norm_rope(v, None, eps=1e-6), "V")
    for cache_d, cache in ((kcd, kc), (vcd, vc)):
        assert torch.equal(cache_d[:past].cpu(), cache[:past]) and torch.equal(cache_d[past + seq:].cpu(), cache[past + seq:])


def test_inline_angles_batch_offsets_and_shared_kv_projection(ops):
    """Angles computed on the device from theta; per-sequence positions; V taken from the raw K projection
    (src/modeling/diffusion_gemma/attention.cpp:587-595)."""
    B, seq, nq, nkv, hd, cap = 3, 40, 4, 2, 256, 64
    offs = [0, 5, 17]
    q, k = seeded_bf16(B, seq, nq, hd, seed=11), seeded_bf16(B, seq, nkv, hd, seed=12)
    qw = (seeded_bf16(hd, seed=13).float() * 0.1 + 1.0).bfloat16()
    kw = (seeded_bf16(hd, seed=14).float() * 0.1 + 1.0).bfloat16()
    kc = torch.zeros(B, cap, nkv, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    qd = q.cuda()
    ops.qkv_prepare(qd, k.cuda(), None, k_cache=kc, v_cache=vc, past_len=8, q_weight=qw.cuda(), k_weight=kw.cuda(),
                    eps=1e-6, theta=10000.0, partial_rotary_factor=0.5, v_from_k=True,
                    pos_offset=torch.tensor(offs, dtype=torch.int32, device="cuda"))
    nap = 64
    for b in range(B):
        # fp32 pow / cos / sin differ between libm and the device by a few ulp of the angle; at these small
        # positions that stays well inside one bf16 step
        close_bf16(qd[b], oracle.norm_rope(q[b], qw, eps=1e-6, n_active_pairs=nap, offset=offs[b], theta=10000.0), f"Q{b}")
        close_bf16(kc[b, 8:8 + seq], oracle.norm_rope(k[b], kw, eps=1e-6, n_active_pairs=nap, offset=offs[b], theta=10000.0), f"K{b}")
        close_bf16(vc[b, 8:8 + seq], oracle.norm_rope(k[b], None, eps=1e-6), f"V{b}")
    assert not kc[:, :8].any() and not kc[:, 8 + seq:].any()


def test_reference_named_wrappers(ops):
    x = seeded_bf16(33, 2, 128, seed=21)
    w = (seeded_bf16(128, seed=22).float() * 0.1 + 1.0).bfloat16()
    xd = x.cuda()
    ops.fused_norm_rope_inplace(xd, w.cuda(), 3, 10000.0, 1.0, 1e-6)
    close_bf16(xd, oracle.norm_rope(x, w, eps=1e-6, n_active_pairs=64, offset=3, theta=10000.0), "fused_norm_rope_inplace")
    y = seeded_bf16(50, 256, seed=23)
    yd = y.cuda()
    ops.rms_norm(yd, None, 1e-5)
    close_bf16(yd, oracle.norm_rope(y.view(50, 1, 256), None, eps=1e-5).view(50, 256), "rms_norm_no_scale")


def test_then_attention_reads_the_appended_rows(ops):
    """End to end for one encoder layer call: prepare + append, then causal attention over the cache."""
    seq, nq, nkv, hd, past, cap = 96, 4, 2, 128, 160, 512
    q, k, v = seeded_bf16(seq, nq, hd, seed=31), seeded_bf16(seq, nkv, hd, seed=32), seeded_bf16(seq, nkv, hd, seed=33)
    kc, vc = seeded_bf16(cap, nkv, hd, seed=34).cuda(), seeded_bf16(cap, nkv, hd, seed=35).cuda()
    qd = q.cuda()
    ops.qkv_prepare(qd, k.cuda(), v.cuda(), k_cache=kc, v_cache=vc, past_len=past, eps=1e-6, partial_rotary_factor=1.0)
    out = ops.sdpa_prefill(qd, kc[:past + seq], vc[:past + seq], scale=hd ** -0.5, mask_type=ops.MASK_CAUSAL)
    want, _ = oracle.sdpa_f32(qd.cpu(), kc[:past + seq].cpu(), vc[:past + seq].cpu(), scale=hd ** -0.5, mask_type=3)
    from helpers import assert_close
    assert_close(out, want, "attention over appended cache")


def test_rejects_bad_arguments(ops):
    from arcaine_b200 import _lib
    x = torch.zeros(4, 2, 192, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.ArcError):
        ops.qkv_prepare(x, None, None)
    k = torch.zeros(4, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="capacity"):
        ops.qkv_prepare(None, k, k, k_cache=torch.zeros(3, 2, 128, dtype=torch.bfloat16, device="cuda"),
                        v_cache=torch.zeros(3, 2, 128, dtype=torch.bfloat16, device="cuda"), past_len=0)


def test_against_committed_fixtures(ops):
    """The kernel against tests/golden/preprocess_small.npz (torch-fp32 formulation, see make_golden.py)."""
    import os
    import numpy as np
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "preprocess_small.npz"))
    for name in ("hd128_full", "hd256_quarter", "hd512_norm_only"):
        tokens, heads, hd, nap, offset = (int(v) for v in z[name + "_params"])
        x = oracle.bits_to_bf16(z[name + "_x"]).reshape(tokens, heads, hd)
        w = oracle.bits_to_bf16(z[name + "_w"])
        want = oracle.bits_to_bf16(z[name + "_y"]).reshape(tokens, heads, hd)
        xd = x.cuda()
        ops.fused_norm_rope_inplace(xd, w.cuda(), offset, 10000.0, 2.0 * nap / hd, 1e-6)
        close_bf16(xd, want, name)


@pytest.mark.parametrize("hd,rd", [(256, 64), (128, 32), (256, 128), (512, 64)])
def test_qwen35_form_norm_mrope_and_plain_v_append(ops, hd, rd):
    """Qwen3.5 layer call (src/modeling/qwen3_5/operators.hpp:127-140): q/k RMSNorm with weights, multi-axis
    RoPE on the first rotary_dim values of every row (pairs rotary_dim/2 apart), K and V appended to the
    cache, V as it is."""
    B, seq, nq, nkv, past, cap, theta, sec = 2, 37, 6, 2, 11, 64, 1e6, (11, 11, 10)
    q, k, v = seeded_bf16(B, seq, nq, hd, seed=51), seeded_bf16(B, seq, nkv, hd, seed=52), seeded_bf16(B, seq, nkv, hd, seed=53)
    qw = (seeded_bf16(hd, seed=54).float() * 0.1 + 1.0).bfloat16()
    kw = (seeded_bf16(hd, seed=55).float() * 0.1 + 1.0).bfloat16()
    g = torch.Generator().manual_seed(56)
    pos = torch.randint(0, 300, (B, 3, seq), generator=g, dtype=torch.int32)
    kc = torch.zeros(B, cap, nkv, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    qd = q.cuda()
    ops.qkv_prepare(qd, k.cuda(), v.cuda(), k_cache=kc, v_cache=vc, past_len=past, q_weight=qw.cuda(), k_weight=kw.cuda(),
                    eps=1e-6, theta=theta, rotary_dim=rd, mrope_positions=pos.cuda(), mrope_section=sec, v_copy=True)
    for b in range(B):
        want_q = oracle.mrope(oracle.norm_rope(q[b], qw, eps=1e-6), pos[b].numpy(), rd, theta, sec)
        want_k = oracle.mrope(oracle.norm_rope(k[b], kw, eps=1e-6), pos[b].numpy(), rd, theta, sec)
        close_bf16(qd[b], want_q, f"Q{b}")
        close_bf16(kc[b, past:past + seq], want_k, f"K{b}")
        assert torch.equal(vc[b, past:past + seq].cpu(), v[b]), "V must be appended bit for bit"
    assert not kc[:, :past].any() and not vc[:, past + seq:].any()


def test_qwen35_form_rejects_unsupported_rotary_dim(ops):
    from arcaine_b200 import _lib
    x = torch.zeros(4, 2, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(_lib.ArcError):
        ops.qkv_prepare(x, None, None, rotary_dim=96)   # pairs 48 apart: not a power of two


def test_shared_kv_projection_with_in_place_k_is_refused(ops):
    """V taken from the raw K projection while K is normalised in place would read rows another warp
    has already rewritten: the call is refused (src/modeling/diffusion_gemma/attention.cpp:587-595 norms V
    from a copy of raw K before k_norm runs)."""
    B, seq, nq, nkv, hd = 1, 8, 2, 1, 128
    q, k = seeded_bf16(B, seq, nq, hd, seed=1).cuda(), seeded_bf16(B, seq, nkv, hd, seed=2).cuda()
    vc = torch.zeros(B, 16, nkv, hd, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError, match="k_cache"):
        ops.qkv_prepare(q, k, None, v_from_k=True, v_cache=vc)
