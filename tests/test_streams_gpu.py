"""Calls on two CUDA streams at once, each with a workspace of its own: the library keeps no per-call state
outside the caller's buffers (the status word is the one thing the calls share), so the results must be the ones
the same calls give one after the other."""
import pytest
import torch

from helpers import seeded_bf16

pytestmark = pytest.mark.gpu


def test_prefill_and_decode_on_two_streams_equal_the_serial_results():
    from arcaine_b200 import ops
    ops.clear_device_status()
    dev = torch.device("cuda", 0)
    # stream A: canvas-like prefill (key-range splits as a cluster) and a windowed hd128 prefill (two-tile kernel)
    qa, ka, va = (seeded_bf16(256, 8, 256, seed=1).cuda(), seeded_bf16(2304, 4, 256, seed=2).cuda(),
                  seeded_bf16(2304, 4, 256, seed=3).cuda())
    qw, kw, vw = (seeded_bf16(2048, 16, 128, seed=4).cuda(), seeded_bf16(2048, 8, 128, seed=5).cuda(),
                  seeded_bf16(2048, 8, 128, seed=6).cuda())
    # stream B: gated decode with per-sequence lengths and a long single-sequence decode
    qd, kd, vd = (seeded_bf16(6, 24, 256, seed=7).cuda(), seeded_bf16(6, 3000, 4, 256, seed=8).cuda(),
                  seeded_bf16(6, 3000, 4, 256, seed=9).cuda())
    gd = seeded_bf16(6, 24, 256, seed=10).cuda()
    lens = torch.tensor([3000, 17, 1024, 2999, 1, 512], dtype=torch.int32, device=dev)
    ql, kl, vl = (seeded_bf16(1, 16, 128, seed=11).cuda(), seeded_bf16(1, 40000, 2, 128, seed=12).cuda(),
                  seeded_bf16(1, 40000, 2, 128, seed=13).cuda())

    def side_a(ws):
        return (ops.sdpa_prefill(qa, ka, va, scale=0.0625, workspace=ws),
                ops.sdpa_prefill(qw, kw, vw, scale=128 ** -0.5, mask_type=ops.MASK_CAUSAL, window=512, workspace=ws))

    def side_b(ws):
        return (ops.sdpa_decode(qd, kd, vd, scale=0.0625, kv_len=lens, gate=gd, workspace=ws),
                ops.sdpa_decode(ql, kl, vl, scale=128 ** -0.5, workspace=ws))

    ws_a, ws_b = ops.Workspace(dev), ops.Workspace(dev)
    want = side_a(ws_a) + side_b(ws_b)
    torch.cuda.synchronize()
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    got_a, got_b = [], []
    for _ in range(8):  # several rounds, so that the two sides really overlap
        with torch.cuda.stream(sa):
            got_a.append(side_a(ws_a))
        with torch.cuda.stream(sb):
            got_b.append(side_b(ws_b))
    torch.cuda.synchronize()
    assert ops.device_status() == (0, 0)
    for ra, rb in zip(got_a, got_b):
        for g, w in zip(ra + rb, want):
            assert torch.equal(g, w)
