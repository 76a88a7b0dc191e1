"""Generates tests/golden/sdpa_small.npz.

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


if __name__ == "__main__":
    main()
