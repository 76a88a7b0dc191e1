"""Generates tests/golden/sdpa_small.npz and tests/golden/preprocess_small.npz.

The reference ships no attention golden vectors and cannot be built or imported
here (SYCL + oneDNN), so these fixtures do not pin the oracle to the reference.
They are regression anchors: small seeded cases whose expected outputs come from
an independent torch-fp32 formulation (``oracle.torch_sdpa_f32``), committed so
that a later change to the C checker cannot drift unnoticed.  The one recipe that
does come from the reference — the bench's LCG input fill,
src/bench/qwen35_attention_bench.cpp:86-94 — is recorded as the first values it
must produce, worked out by hand from the recurrence.

Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import oracle  # noqa: E402

CASES = [
    # name, seq, kv_len, nq, nkv, hd, scale, mask_type, window, seed
    ("noncausal_gqa2", 24, 40, 4, 2, 128, 128 ** -0.5, 0, oracle.INT_MAX, 11),
    ("causal_bottom_right", 16, 37, 4, 2, 128, 128 ** -0.5, 3, oracle.INT_MAX, 12),
    ("window8", 32, 32, 2, 1, 128, 128 ** -0.5, 3, 8, 13),
    ("canvas_hd256_scale1", 8, 48, 4, 2, 256, 1.0, 0, oracle.INT_MAX, 14),
    ("decode_gqa6", 1, 65, 6, 1, 256, 0.0625, 3, oracle.INT_MAX, 15),
]


def make_inputs(seq, kv_len, nq, nkv, hd, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(seq, nq, hd, generator=g).bfloat16()
    k = torch.randn(kv_len, nkv, hd, generator=g).bfloat16()
    v = torch.randn(kv_len, nkv, hd, generator=g).bfloat16()
    return q, k, v


def lcg_first_values(n=8, state=42):
    vals = []
    for _ in range(n):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        vals.append((((state >> 16) & 1023) - 512) / 1024.0)
    return np.asarray(vals, dtype=np.float32), state


def main():
    out = {}
    for name, seq, kv_len, nq, nkv, hd, scale, mt, w, seed in CASES:
        q, k, v = make_inputs(seq, kv_len, nq, nkv, hd, seed)
        want = oracle.torch_sdpa_f32(q, k, v, scale=scale, mask_type=mt, window=w)
        out[name + "_out_f32"] = want.numpy().astype(np.float32)
        out[name + "_params"] = np.asarray([seq, kv_len, nq, nkv, hd, mt, min(w, oracle.INT_MAX), seed], dtype=np.int64)
        out[name + "_scale"] = np.asarray([scale], dtype=np.float64)
    vals, state = lcg_first_values()
    out["lcg_first8"] = vals
    out["lcg_state_after8"] = np.asarray([state], dtype=np.int64)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "sdpa_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")
    make_preprocess()


def torch_norm_rope(x, w, eps, nap, offset, theta):
    """RMSNorm then RoPE in plain torch fp32 with the reference's rounding points
    (src/common/kernels/rms_norm.hpp:9-49, src/modeling/diffusion_gemma/attention_kernels.hpp:99-153)."""
    xf = x.float()
    n = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps)
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


def make_preprocess():
    """tests/golden/preprocess_small.npz: RMSNorm + RoPE outputs and a vision-block mask, from formulations that
    do not go through the C checker (torch fp32 / numpy)."""
    out = {}
    for name, tokens, heads, hd, partial, offset, seed in (("hd128_full", 7, 3, 128, 1.0, 5, 41),
                                                          ("hd256_quarter", 5, 2, 256, 0.25, 100, 42),
                                                          ("hd512_norm_only", 4, 2, 512, 0.0, 0, 43)):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn(tokens, heads, hd, generator=g).bfloat16()
        w = (torch.randn(hd, generator=g) * 0.1 + 1.0).bfloat16()
        nap = int(partial * hd / 2.0)
        y = torch_norm_rope(x, w, 1e-6, nap, offset, 10000.0)
        out[name + "_x"] = x.view(torch.int16).numpy().view(np.uint16)
        out[name + "_w"] = w.view(torch.int16).numpy().view(np.uint16)
        out[name + "_y"] = y.view(torch.int16).numpy().view(np.uint16)
        out[name + "_params"] = np.asarray([tokens, heads, hd, nap, offset], dtype=np.int64)
    q_len, kv_len, past, window = 12, 20, 14, 9
    ids = np.full(past + q_len, -1, dtype=np.int32)
    ids[10:16] = 0
    ids[19:24] = 1
    qg = past + np.arange(q_len)[:, None]
    kg = past - (kv_len - q_len) + np.arange(kv_len)[None, :]
    same = (ids[qg] >= 0) & (ids[qg] == ids[kg])
    hidden = (~same & (kg > qg)) | (kg < qg - window + 1)
    out["blockmask_ids"] = ids
    out["blockmask_params"] = np.asarray([q_len, kv_len, past, window], dtype=np.int64)
    out["blockmask_hidden"] = hidden
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "preprocess_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
