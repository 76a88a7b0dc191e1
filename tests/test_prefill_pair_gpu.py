"""Parity of the two-tiles-per-CTA prefill kernel (head dim 128) with the CPU oracle.

The library picks this kernel by a cost model (large problems); ARC_SDPA_PREFILL_KERNEL=pair, read once per
process, forces it for every head-dim-128 call, so the small cases here run in a child process with that
variable set: two token tiles of one head (odd GQA group), two heads of one KV group over the same tokens (even
group), masks, windows, gate and ragged ends.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[1] + '/tests')
import torch
from helpers import assert_close, seeded_bf16
import oracle
from arcaine_b200 import ops
ops.clear_device_status()
cases = [  # seq, kv_len, nq, nkv, mask_type, window, gate
    (300, 300, 8, 4, 0, oracle.INT_MAX, False),
    (300, 300, 8, 4, 3, oracle.INT_MAX, True),
    (1000, 1000, 4, 2, 3, 100, False),
    (1, 129, 4, 2, 3, oracle.INT_MAX, False),
    (129, 127, 4, 2, 3, 64, False),      # kv_len < seq: leading queries see nothing
    (130, 1000, 4, 2, 3, oracle.INT_MAX, False),
    (257, 257, 2, 1, 0, oracle.INT_MAX, False),
    (2048, 2048, 4, 2, 3, 1024, False),
    (600, 600, 3, 3, 3, 200, False),     # one query head per KV head: a CTA takes 256 tokens of one head
    (520, 700, 6, 2, 3, oracle.INT_MAX, True),  # three per KV head: the same
    (384, 384, 8, 2, 0, oracle.INT_MAX, False),  # four per KV head: two heads of a group per CTA
]
for i, (seq, kv, nq, nkv, mt, w, gate) in enumerate(cases):
    q, k, v = seeded_bf16(seq, nq, 128, seed=900 + i), seeded_bf16(kv, nkv, 128, seed=950 + i), seeded_bf16(kv, nkv, 128, seed=990 + i)
    g = seeded_bf16(seq, nq, 128, seed=930 + i) if gate else None
    out, lse = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=0.09, mask_type=mt, window=w, num_splits=1,
                                gate=g.cuda() if gate else None, return_lse=True)
    want = oracle.sdpa_f32(q, k, v, scale=0.09, mask_type=mt, window=w, gate=g, want_lse=True)
    assert_close(out, want[0], f"case {i}")
    finite = torch.isfinite(want[2])
    assert torch.equal(torch.isfinite(lse.cpu()), finite), f"case {i}: lse finiteness"
    assert torch.allclose(lse.cpu()[finite], want[2][finite], atol=2e-3), f"case {i}: lse"
# Scores that grow along the keys: the one-pass blocks must move their reference, both between blocks
# (growth of 2^8 .. 2^32) and inside a block (more than 2^32), without losing accuracy.
for i, (seq, kv, gain_at, gain) in enumerate([(384, 1024, 512, 6.0), (384, 1024, 300, 60.0), (256, 2048, 1900, 200.0),
                                              (300, 1500, 130, 25.0)]):
    q, k, v = seeded_bf16(seq, 4, 128, seed=1200 + i), seeded_bf16(kv, 2, 128, seed=1250 + i), seeded_bf16(kv, 2, 128, seed=1290 + i)
    k = k.float()
    k[gain_at:] *= gain
    k[gain_at + 37::53] *= 3.0   # and a few outliers inside the blocks
    k = k.bfloat16()
    for mt in (0, 3):
        out, lse = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=0.09, mask_type=mt, num_splits=1, return_lse=True)
        want = oracle.sdpa_f32(q, k, v, scale=0.09, mask_type=mt, want_lse=True)
        assert_close(out, want[0], f"growing scores {i} mask {mt}")
        finite = torch.isfinite(want[2])
        assert torch.allclose(lse.cpu()[finite], want[2][finite], atol=2e-3, rtol=1e-5), f"growing scores {i}: lse"
# batch > 1 and many tiles per CTA: against the default kernel's own parity-tested output is not possible in
# this process, so check sampled rows against the oracle
B, S, nq, nkv = 2, 4096, 16, 8
g = torch.Generator(device='cuda').manual_seed(5)
q = torch.randn(B, S, nq, 128, generator=g, device='cuda').bfloat16()
k = torch.randn(B, S, nkv, 128, generator=g, device='cuda').bfloat16()
v = torch.randn(B, S, nkv, 128, generator=g, device='cuda').bfloat16()
out = ops.sdpa_prefill(q, k, v, scale=128 ** -0.5, mask_type=3, window=1024)
from helpers import sample_rows
rows = sample_rows(S, nq, 400, seed=77)
want, _ = oracle.sdpa_f32(q[1].cpu(), k[1].cpu(), v[1].cpu(), scale=128 ** -0.5, mask_type=3, window=1024, rows=rows)
assert_close(out[1].reshape(-1, 128)[rows], want, "batch 2 x 4096")
# output copies from this kernel's epilogue, several units per CTA, tiles of a single key block among them
# (S = 8192, window 1024: the first token tile of every head sees one block)
q1, k1, v1 = q[:1].repeat(1, 2, 1, 1), k[:1].repeat(1, 2, 1, 1), v[:1].repeat(1, 2, 1, 1)
ref = ops.sdpa_prefill(q1, k1, v1, scale=128 ** -0.5, mask_type=3, window=1024)
bufs = [torch.zeros_like(ref) for _ in range(3)]
copies = torch.tensor([b.data_ptr() for b in bufs], dtype=torch.int64, device='cuda')
got = ops.sdpa_prefill(q1, k1, v1, scale=128 ** -0.5, mask_type=3, window=1024, out_copies=copies)
torch.cuda.synchronize()
assert torch.equal(got, ref) and all(torch.equal(b, ref) for b in bufs), "output copies"
assert ops.device_status() == (0, 0)
assert ops.launch_count() > 0
print("PAIR-OK")
"""


def test_pair_kernel_matches_oracle():
    env = dict(os.environ, ARC_SDPA_PREFILL_KERNEL="pair")
    res = subprocess.run([sys.executable, "-c", CHILD, ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0 and "PAIR-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]
