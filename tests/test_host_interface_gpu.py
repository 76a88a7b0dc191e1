"""The C++ host interface (reference-shaped free functions) driven by the kbench-style program,
checked the way the reference's own bench checks its kernels: against the scalar online-softmax
kernel (src/bench/qwen35_attention_bench.cpp:124-159), here restated on the CPU."""
import os
import re
import subprocess

import numpy as np
import pytest
import torch

from helpers import assert_close
import oracle

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "arcaine_b200", "arc_attention_bench")


def test_bench_cells_match_the_scalar_reference_kernel(tmp_path):
    if not os.path.exists(BIN):
        from arcaine_b200 import build
        build.build_attention_bench()
    prefills, depths = [128, 512], [0, 512, 1024]
    res = subprocess.run([BIN, "qwen35-attention", "--warmup", "1", "--runs", "3", "--dump", str(tmp_path)],
                         capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stderr
    rows = re.findall(r"qwen35_attention kind=(\w+) kernel=(sdpa\S*) q=(\d+) kv=(\d+) mean_ms=([\d.]+) sd_ms=[\d.]+ "
                      r"max_abs=([\d.]+) max_rel=([\d.]+)", res.stdout)
    assert len(rows) == len(prefills) + 2 * len(depths)
    # the row's own check: the library against the bench's scalar kernel on the device
    assert all(float(r[5]) <= 2e-2 for r in rows), rows
    assert len(re.findall(r"kernel=baseline", res.stdout)) == len(rows)
    listing = subprocess.run([BIN, "--list"], capture_output=True, text=True, timeout=60).stdout
    assert all(name in listing for name in ("qwen35-attention", "sdpa-prefill", "sdpa-decode"))
    nq, nkv, hd, scale = 24, 4, 256, 0.0625
    max_q, max_kv = max(prefills), max(max(prefills), max(depths) + 1)
    state = 42
    qb, state = oracle.lcg_fill(max_q * nq * hd, state)
    kb, state = oracle.lcg_fill(max_kv * nkv * hd, state)
    vb, state = oracle.lcg_fill(max_kv * nkv * hd, state)
    gb, state = oracle.lcg_fill(max_q * nq * hd, state)
    q = oracle.bits_to_bf16(qb).reshape(max_q, nq, hd)
    k = oracle.bits_to_bf16(kb).reshape(max_kv, nkv, hd)
    v = oracle.bits_to_bf16(vb).reshape(max_kv, nkv, hd)
    g = oracle.bits_to_bf16(gb).reshape(max_q, nq, hd)

    def load(kind, seq, kv):
        a = np.fromfile(os.path.join(tmp_path, f"{kind}_q{seq}_kv{kv}.bin"), dtype=np.uint16)
        return oracle.bits_to_bf16(a).reshape(seq, nq, hd)

    for seq in prefills:
        want = oracle.qwen35_online_attention(q[:seq], k[:seq], v[:seq], seq=seq, past=0, scale=scale)
        assert_close(load("prefill", seq, seq), want.float(), f"prefill {seq}")
    for d in depths:
        want = oracle.qwen35_online_attention(q[:1], k[:d + 1], v[:d + 1], seq=1, past=d, scale=scale)
        assert_close(load("decode", 1, d + 1), want.float(), f"decode depth {d}")
        assert_close(load("decode_gated", 1, d + 1), oracle.mul_sigmoid_inplace(want, g[:1]).float(), f"gated depth {d}")
