"""CPU tests of the checker itself: the C restatement against independent formulations,
the committed fixtures and the reference's documented rules (no GPU needed)."""
import os

import numpy as np
import pytest
import torch

from helpers import seeded_bf16
import oracle

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "sdpa_small.npz")


def test_bf16_round_to_nearest_even_matches_torch():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(4096, generator=g) * 100
    x = torch.cat([x, torch.tensor([0.0, -0.0, 1.0, 1.00390625, 1.01171875, 3.0e38, 1e-40])])
    want = x.bfloat16().view(torch.int16).numpy().view(np.uint16)
    got = np.array([oracle.float_to_bf16_bits(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got, want)
    back = np.array([oracle.bf16_bits_to_float(int(b)) for b in got], dtype=np.float32)
    assert np.array_equal(back, x.bfloat16().float().numpy())


def test_lcg_fill_matches_the_bench_recipe():
    gold = np.load(GOLDEN)
    bits, state = oracle.lcg_fill(8, 42)
    vals = oracle.bits_to_bf16(bits).float().numpy()
    # x/1024 needs up to 9 significant bits, so the recipe's bf16 store rounds it (RNE)
    want = torch.from_numpy(gold["lcg_first8"]).bfloat16().float().numpy()
    assert np.array_equal(vals, want)
    assert state == int(gold["lcg_state_after8"][0])
    # filling in two calls continues the same stream (Q then K then V in the bench)
    a, s1 = oracle.lcg_fill(5, 42)
    b, _ = oracle.lcg_fill(3, s1)
    assert np.array_equal(np.concatenate([a, b]), bits)


def test_fill_causal_mask_rule():
    # window W keeps the W most recent keys, self included; past_offset cancels out
    m = oracle.fill_causal_mask(4, 6, past_offset=10, sliding_window=3)
    want = np.full((4, 6), -np.inf, dtype=np.float32)
    for qi in range(4):
        diag = qi + 2
        for kj in range(max(0, diag - 2), diag + 1):
            want[qi, kj] = 0.0
    assert np.array_equal(m, want)
    assert np.array_equal(oracle.fill_causal_mask(4, 6, 0, 3), m)
    full = oracle.fill_causal_mask(3, 3, 0)
    assert np.array_equal(np.isinf(full), np.triu(np.ones((3, 3), dtype=bool), 1))


@pytest.mark.parametrize("name", ["noncausal_gqa2", "causal_bottom_right", "window8", "canvas_hd256_scale1",
                                  "decode_gqa6"])
def test_c_oracle_reproduces_committed_fixtures(name):
    gold = np.load(GOLDEN)
    seq, kv_len, nq, nkv, hd, mt, w, seed = (int(x) for x in gold[name + "_params"])
    scale = float(gold[name + "_scale"][0])
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(seq, nq, hd, generator=g).bfloat16()
    k = torch.randn(kv_len, nkv, hd, generator=g).bfloat16()
    v = torch.randn(kv_len, nkv, hd, generator=g).bfloat16()
    got, got_bf16 = oracle.sdpa_f32(q, k, v, scale=scale, mask_type=mt, window=w)
    want = torch.from_numpy(gold[name + "_out_f32"])
    rel, mx = oracle.error_metrics(got, want)
    assert rel < 2e-6 and mx < 2e-5, (rel, mx)
    assert torch.equal(got_bf16, got.bfloat16())


def test_explicit_mask_equals_inline_rule_and_row_sampling():
    q, k, v = seeded_bf16(20, 4, 128, seed=1), seeded_bf16(33, 2, 128, seed=2), seeded_bf16(33, 2, 128, seed=3)
    mask = oracle.fill_causal_mask(20, 33, past_offset=13, sliding_window=7)
    a, _ = oracle.sdpa_f32(q, k, v, scale=0.1, mask_type=oracle.MASK_EXPLICIT, mask=mask)
    b, _ = oracle.sdpa_f32(q, k, v, scale=0.1, mask_type=oracle.MASK_CAUSAL, window=7)
    assert torch.allclose(a, b, atol=1e-6)
    rows = [0, 5, 17, 79]
    c, _, lse = oracle.sdpa_f32(q, k, v, scale=0.1, mask_type=oracle.MASK_CAUSAL, window=7, rows=rows, want_lse=True)
    assert torch.equal(c, b.reshape(-1, 128)[rows])
    assert torch.isfinite(lse).all()


def test_rows_with_no_visible_key_are_zero():
    # more queries than keys, bottom-right aligned: the first queries see nothing
    q, k, v = seeded_bf16(6, 2, 128, seed=4), seeded_bf16(3, 1, 128, seed=5), seeded_bf16(3, 1, 128, seed=6)
    out, _, lse = oracle.sdpa_f32(q, k, v, scale=0.1, mask_type=oracle.MASK_CAUSAL, want_lse=True)
    assert torch.equal(out[:3], torch.zeros(3, 2, 128))
    assert torch.isinf(lse[:3]).all() and torch.isfinite(lse[3:]).all()


def test_online_attention_restatement_agrees_with_fp32_oracle():
    # src/modeling/qwen3_5/kernels.hpp:621-679 against the grading oracle, bench-recipe inputs
    nq, nkv, hd, seq, past = 24, 4, 256, 5, 20
    state = 42
    qb, state = oracle.lcg_fill(seq * nq * hd, state)
    kb, state = oracle.lcg_fill((past + seq) * nkv * hd, state)
    vb, state = oracle.lcg_fill((past + seq) * nkv * hd, state)
    q = oracle.bits_to_bf16(qb).reshape(seq, nq, hd)
    k = oracle.bits_to_bf16(kb).reshape(past + seq, nkv, hd)
    v = oracle.bits_to_bf16(vb).reshape(past + seq, nkv, hd)
    got = oracle.qwen35_online_attention(q, k, v, seq=seq, past=past, scale=0.0625)
    want, _ = oracle.sdpa_f32(q, k, v, scale=0.0625, mask_type=oracle.MASK_CAUSAL)
    rel, mx = oracle.error_metrics(got, want)
    assert rel < 4e-3 and mx < 2e-3, (rel, mx)  # one bf16 rounding of the output


def test_matmul_softmax_matmul_restatements_agree_with_oracle():
    # gqa_attention (bf16 scores / probabilities, no scale) and batched_attention (scale, f32 softmax)
    q = (seeded_bf16(12, 4, 128, seed=7).float() * 0.3).bfloat16()
    k = (seeded_bf16(30, 2, 128, seed=8).float() * 0.3).bfloat16()
    v = seeded_bf16(30, 2, 128, seed=9)
    want, _ = oracle.sdpa_f32(q, k, v, scale=1.0, mask_type=oracle.MASK_CAUSAL, window=9)
    a = oracle.gqa_attention(q, k, v, past_offset=18, sliding_window=9, causal=True)
    b = oracle.batched_attention(q, k, v, past_offset=18, sliding_window=9, scale=1.0)
    for got in (a, b):
        rel, mx = oracle.error_metrics(got, want)
        assert rel < 1e-2 and mx < 2e-2, (rel, mx)
    nc = oracle.gqa_attention(q, k, v, past_offset=0, causal=False)
    want_nc, _ = oracle.sdpa_f32(q, k, v, scale=1.0)
    rel, mx = oracle.error_metrics(nc, want_nc)
    assert rel < 1e-2 and mx < 2e-2, (rel, mx)


def test_gate_matches_reference_formula():
    a, g = seeded_bf16(3, 5, 128, seed=10), seeded_bf16(3, 5, 128, seed=11)
    got = oracle.mul_sigmoid_inplace(a, g)
    want = (a.float() * (1.0 / (1.0 + torch.exp(-g.float())))).bfloat16()
    assert (got.view(torch.int16).int() - want.view(torch.int16).int()).abs().max() <= 1  # expf vs torch.exp ulp
    _, gated = oracle.sdpa_f32(seeded_bf16(3, 4, 128, seed=1), seeded_bf16(9, 2, 128, seed=2),
                               seeded_bf16(9, 2, 128, seed=3), scale=0.1, gate=seeded_bf16(3, 4, 128, seed=12))
    _, plain = oracle.sdpa_f32(seeded_bf16(3, 4, 128, seed=1), seeded_bf16(9, 2, 128, seed=2),
                               seeded_bf16(9, 2, 128, seed=3), scale=0.1)
    assert torch.equal(gated, oracle.mul_sigmoid_inplace(plain, seeded_bf16(3, 4, 128, seed=12)))


def test_split_merge_identity():
    q, k, v = seeded_bf16(1, 8, 128, seed=20), seeded_bf16(301, 2, 128, seed=21), seeded_bf16(301, 2, 128, seed=22)
    whole, _, lse_whole = oracle.sdpa_f32(q, k, v, scale=0.09, want_lse=True)
    cuts = [0, 64, 65, 200, 301]
    outs, lses = [], []
    for a, b in zip(cuts[:-1], cuts[1:]):
        o, _, l = oracle.sdpa_f32(q, k[a:b], v[a:b], scale=0.09, want_lse=True)
        outs.append(o.reshape(-1, 128))
        lses.append(l.reshape(-1))
    # an empty part (lse = -inf) must be ignored
    outs.append(torch.zeros_like(outs[0]))
    lses.append(torch.full_like(lses[0], float("-inf")))
    merged, lse = oracle.merge_partials(torch.stack(outs), torch.stack(lses))
    assert torch.allclose(merged, whole.reshape(-1, 128), atol=2e-6)
    assert torch.allclose(lse, lse_whole.reshape(-1), atol=2e-6)


def _torch_norm_rope(x, w, eps, nap, offset, theta):
    """RMSNorm then RoPE in plain torch fp32, with the reference's rounding points."""
    xf = x.float()
    rms = torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
    n = xf * rms
    if w is not None:
        n = n * w.float()
    n = n.bfloat16().float()
    hd = x.shape[-1]
    if nap:
        p = torch.arange(nap).float()
        inv = 1.0 / torch.pow(torch.tensor(float(theta)), 2.0 * p / hd)
        ang = (torch.arange(x.shape[0]).float() + offset)[:, None] * inv[None]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        o = n.clone()
        o[..., :nap] = n[..., :nap] * c - n[..., hd // 2:hd // 2 + nap] * s
        o[..., hd // 2:hd // 2 + nap] = n[..., :nap] * s + n[..., hd // 2:hd // 2 + nap] * c
        n = o
    return n.bfloat16()


@pytest.mark.parametrize("hd,partial", [(128, 1.0), (256, 0.25), (512, 0.0)])
def test_norm_rope_restatement_matches_torch(hd, partial):
    """rms_norm + fused_norm_rope_inplace (src/common/kernels/rms_norm.hpp:9-49,
    src/modeling/diffusion_gemma/attention_kernels.hpp:99-153) against an independent torch formulation:
    at most one bf16 step apart, and that in very few elements (fp32 vs double sum of squares)."""
    x = seeded_bf16(9, 3, hd, seed=hd)
    w = (seeded_bf16(hd, seed=hd + 1).float() * 0.1 + 1.0).bfloat16()
    nap = int(partial * hd / 2.0)
    for weight in (w, None):
        got = oracle.norm_rope(x, weight, eps=1e-6, n_active_pairs=nap, offset=11, theta=10000.0)
        want = _torch_norm_rope(x, weight, 1e-6, nap, 11, 10000.0)
        diff = (got.float() - want.float()).abs()
        step = want.float().abs() * 2.0 ** -7 + 2e-6
        assert (diff <= step).all()
        assert (got != want).float().mean() < 5e-3
    # table mode reads the angles instead of computing them
    if nap:
        p = torch.arange(nap).float()
        inv = 1.0 / torch.pow(torch.tensor(10000.0), 2.0 * p / hd)
        ang = (torch.arange(9).float() + 11)[:, None] * inv[None]
        got_t = oracle.norm_rope(x, w, eps=1e-6, n_active_pairs=nap, rope_cos=torch.cos(ang), rope_sin=torch.sin(ang))
        want_t = oracle.norm_rope(x, w, eps=1e-6, n_active_pairs=nap, offset=11, theta=10000.0)
        assert (got_t.float() - want_t.float()).abs().max() <= 2.0 ** -7 * want_t.float().abs().max()


def test_block_id_mask_matches_a_numpy_restatement():
    """fill_causal_mask_with_block_ids (src/common/kernels/attention_mask.hpp:44-73): causal plus
    bidirectional attention inside one vision block; no block ids = plain causal mask."""
    q_len, kv_len, past = 24, 40, 30
    ids = np.full(past + q_len, -1, dtype=np.int32)
    ids[20:28] = 0          # a block that straddles the cached part and the new tokens
    ids[33:41] = 1
    for window in (oracle.INT_MAX, 12):
        got = oracle.fill_causal_mask_with_block_ids(ids, q_len, kv_len, past, window)
        qg = past + np.arange(q_len)[:, None]
        kg = past - (kv_len - q_len) + np.arange(kv_len)[None, :]
        same = (ids[qg] >= 0) & (ids[qg] == ids[kg])
        hidden = (~same & (kg > qg)) | ((window != oracle.INT_MAX) & (kg < qg - window + 1))
        assert np.array_equal(np.isneginf(got), hidden) and np.all((got == 0) | np.isneginf(got))
        assert np.array_equal(oracle.fill_causal_mask_with_block_ids(None, q_len, kv_len, past, window),
                              oracle.fill_causal_mask(q_len, kv_len, past, window))
    assert np.isfinite(oracle.fill_causal_mask_with_block_ids(ids, q_len, kv_len, past)[4, 23])  # q=34 sees k=37


PRE_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "preprocess_small.npz")


def test_preprocess_fixtures():
    """Committed fixtures for the pre-processing restatements (made by tests/golden/make_golden.py from torch /
    numpy formulations): RMSNorm + RoPE within one bf16 step, the vision-block mask exactly."""
    z = np.load(PRE_GOLDEN)
    for name in ("hd128_full", "hd256_quarter", "hd512_norm_only"):
        tokens, heads, hd, nap, offset = (int(v) for v in z[name + "_params"])
        x = oracle.bits_to_bf16(z[name + "_x"]).reshape(tokens, heads, hd)
        w = oracle.bits_to_bf16(z[name + "_w"])
        want = oracle.bits_to_bf16(z[name + "_y"]).reshape(tokens, heads, hd).float()
        got = oracle.norm_rope(x, w, eps=1e-6, n_active_pairs=nap, offset=offset, theta=10000.0).float()
        assert ((got - want).abs() <= want.abs() * 2.0 ** -7 + 2e-6).all(), name
        assert (got != want).float().mean() < 5e-3, name
    q_len, kv_len, past, window = (int(v) for v in z["blockmask_params"])
    m = oracle.fill_causal_mask_with_block_ids(z["blockmask_ids"], q_len, kv_len, past, window)
    assert np.array_equal(np.isneginf(m), z["blockmask_hidden"])


def test_mrope_restatement_matches_torch():
    """qwen35_apply_mrope (src/modeling/qwen3_5/kernels.hpp:576-617) against a torch formulation."""
    tokens, heads, hd, rd, theta, sec = 9, 3, 256, 64, 1e6, (11, 11, 10)
    x = seeded_bf16(tokens, heads, hd, seed=77)
    g = torch.Generator().manual_seed(78)
    pos = torch.randint(0, 500, (3, tokens), generator=g, dtype=torch.int32)
    got = oracle.mrope(x, pos.numpy(), rd, theta, sec)
    half = rd // 2
    f = torch.arange(half)
    axis = torch.zeros(half, dtype=torch.long)
    for a in (1, 2):
        axis[(f >= a) & (f < sec[a] * 3) & (f % 3 == a)] = a
    inv = 1.0 / torch.pow(torch.tensor(theta), 2.0 * f.float() / rd)
    ang = pos.float()[axis, :].T * inv[None, :]             # (tokens, half)
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    xf = x.float()
    want = xf.clone()
    want[..., :half] = xf[..., :half] * c - xf[..., half:rd] * s
    want[..., half:rd] = xf[..., :half] * s + xf[..., half:rd] * c
    want = want.bfloat16().float()
    assert ((got.float() - want).abs() <= want.abs() * 2.0 ** -7 + 2e-6).all()
    assert torch.equal(got[..., rd:], x[..., rd:])          # the tail of every row is untouched
