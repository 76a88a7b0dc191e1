"""Parity of the sm_100a prefill / canvas kernel with the CPU oracle, through the C ABI."""
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
    assert o.device_status() == (0, 0), "a bounded device-side wait gave up during the prefill tests"


def run_case(ops, seq, kv_len, nq, nkv, hd, scale, mask_type, window, seed, num_splits=0, gate=False, lse=False):
    q, k, v = seeded_bf16(seq, nq, hd, seed=seed), seeded_bf16(kv_len, nkv, hd, seed=seed + 1), \
        seeded_bf16(kv_len, nkv, hd, seed=seed + 2)
    g = seeded_bf16(seq, nq, hd, seed=seed + 3) if gate else None
    res = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=scale, mask_type=mask_type, window=window,
                           num_splits=num_splits, gate=g.cuda() if gate else None, return_lse=lse)
    want = oracle.sdpa_f32(q, k, v, scale=scale, mask_type=mask_type, window=window, gate=g, want_lse=lse)
    if lse:
        assert_close(res[0], want[0], "out")
        finite = torch.isfinite(want[2])
        assert torch.equal(torch.isfinite(res[1].cpu()), finite)
        assert torch.allclose(res[1].cpu()[finite], want[2][finite], atol=2e-3)
    else:
        assert_close(res, want[0], f"S{seq} L{kv_len} nq{nq}/{nkv} hd{hd} mask{mask_type} w{window}")


@pytest.mark.parametrize("hd", [128, 256])
@pytest.mark.parametrize("mask_type,window", [(0, oracle.INT_MAX), (3, oracle.INT_MAX), (3, 100), (3, 1)])
def test_single_sequence(ops, hd, mask_type, window):
    run_case(ops, 300, 300, 8, 4, hd, hd ** -0.5, mask_type, window, seed=100 + hd)


@pytest.mark.parametrize("seq,kv_len", [(1, 1), (1, 129), (77, 300), (128, 128), (129, 127), (130, 1000), (200, 517)])
@pytest.mark.parametrize("mask_type,window", [(0, oracle.INT_MAX), (3, oracle.INT_MAX), (3, 64)])
def test_ragged_shapes(ops, seq, kv_len, mask_type, window):
    # includes kv_len < seq with bottom-right causal: leading queries see no key and must be zero
    run_case(ops, seq, kv_len, 4, 2, 128, 0.09, mask_type, window, seed=seq * 7 + kv_len, lse=True)


def test_config1_cpu_runnable_case(ops):
    """B1, 8Q/4KV, hd128, seq 512, non-causal, scale 1/sqrt(128)."""
    run_case(ops, 512, 512, 8, 4, 128, 128 ** -0.5, 0, oracle.INT_MAX, seed=1)


@pytest.mark.parametrize("scale", [1.0, 256 ** -0.5])
def test_config2_canvas_over_prompt_steps(ops, scale):
    """DiffusionGemma denoising steps: 2048 cached prompt rows + a 256-row canvas written at the cache
    tail each step (src/modeling/diffusion_gemma/attention.cpp:1079-1103), all 32 steps
    (src/modeling/diffusion_gemma/generate.cpp:123): every output row of the first and the last step,
    every fifth row of the others.  Scale 1.0 is what the reference runs, 1/sqrt(256) the conditioned
    variant."""
    nq, nkv, hd, prompt, canvas, steps = 16, 8, 256, 2048, 256, 32
    kc = torch.empty(prompt + canvas, nkv, hd, dtype=torch.bfloat16)
    vc = torch.empty_like(kc)
    kc[:prompt], vc[:prompt] = seeded_bf16(prompt, nkv, hd, seed=2000), seeded_bf16(prompt, nkv, hd, seed=2001)
    kd, vd = kc.cuda(), vc.cuda()
    prompt_k, prompt_v = kd[:prompt].clone(), vd[:prompt].clone()
    worst = 0.0
    for step in range(steps):
        q = seeded_bf16(canvas, nq, hd, seed=2100 + step)
        kc[prompt:], vc[prompt:] = seeded_bf16(canvas, nkv, hd, seed=2200 + step), seeded_bf16(canvas, nkv, hd, seed=2300 + step)
        kd[prompt:].copy_(kc[prompt:])
        vd[prompt:].copy_(vc[prompt:])
        got = ops.gqa_attention_sdpa(q.cuda(), canvas, nq, hd, kd, vd, prompt + canvas, nkv) if scale == 1.0 else \
            ops.sdpa_prefill(q.cuda(), kd, vd, scale=scale)
        rows = list(range(canvas * nq)) if step in (0, steps - 1) else list(range(step % 5, canvas * nq, 5))
        want, _ = oracle.sdpa_f32(q, kc, vc, scale=scale, rows=rows)
        rel, _ = assert_close(got.reshape(-1, hd)[rows], want, f"step {step}")
        worst = max(worst, rel)
    assert worst < 5e-3  # the tolerance is 1e-2; the steps sit well inside it
    # the prompt rows of the cache are read, never written
    assert torch.equal(kd[:prompt], prompt_k) and torch.equal(vd[:prompt], prompt_v)


@pytest.mark.parametrize("splits", [1, 2, 3, 5, 0])
def test_key_range_splits_agree(ops, splits):
    run_case(ops, 256, 1100, 4, 2, 256, 0.0625, 3, 700, seed=31, num_splits=splits, lse=True)


@pytest.mark.parametrize("hd", [128, 256])
@pytest.mark.parametrize("seq,kv_len,nq,nkv,mask_type,window,parts", [
    (256, 1300, 28, 4, 0, oracle.INT_MAX, 2),   # 56 tiles on 148 SMs, 11 key blocks: two parts
    (200, 1300, 28, 4, 3, 300, 2),              # the same ragged and windowed: CTAs of a cluster without keys
    (256, 2100, 16, 8, 0, oracle.INT_MAX, 4),   # 32 tiles, 17 key blocks (the last one ragged): four parts
    (130, 2100, 16, 2, 3, 100, 4),              # 32 tiles, a window: most CTAs of a cluster see no key
    (130, 2100, 4, 2, 0, oracle.INT_MAX, 8),    # 8 tiles: eight parts, always two launches
    (256, 1200, 8, 4, 3, oracle.INT_MAX, 5),    # 16 tiles, 10 key blocks: five parts, two launches
])
def test_key_range_splits_the_library_chooses(ops, hd, seq, kv_len, nq, nkv, mask_type, window, parts):
    """Splits the library chooses itself: two or four parts at head dim 256 run as one thread-block cluster per
    tile whose CTAs fold their accumulators through distributed shared memory (one launch); everything else as
    partial records and a merge launch.  With the gate and the log-sum-exp output."""
    before = ops.launch_count()
    run_case(ops, seq, kv_len, nq, nkv, hd, hd ** -0.5, mask_type, window, seed=500 + hd + seq, gate=True, lse=True)
    torch.cuda.synchronize()
    assert ops.launch_count() - before == (1 if hd == 256 and parts in (2, 4) else 2)
    run_case(ops, seq, kv_len, nq, nkv, hd, hd ** -0.5, mask_type, window, seed=600 + hd + seq)


@pytest.mark.parametrize("case", ["hd128", "single", "cluster", "two_launch", "nothing_visible"])
def test_output_copies_are_written_by_every_epilogue(ops, case):
    """out_copies: further buffers that receive the same rows at the same offsets (other GPUs' buffers when
    a head-sharded output is gathered; here two more buffers on the same device), through every kernel
    that writes output."""
    seq, kv, nq, nkv, hd, mask, win, splits = {
        "hd128": (1024, 1024, 8, 4, 128, 3, 256, 0),         # (the two-tile kernel's copies: test_prefill_pair_gpu.py)
        "single": (300, 300, 4, 2, 256, 3, oracle.INT_MAX, 1),
        "cluster": (256, 2100, 16, 8, 256, 0, oracle.INT_MAX, 0),    # 32 tiles, 17 key blocks: clusters of four
        "two_launch": (256, 1200, 4, 2, 128, 0, oracle.INT_MAX, 3),
        "nothing_visible": (200, 100, 4, 2, 128, 3, oracle.INT_MAX, 0),  # the first 100 queries see no key
    }[case]
    q, k, v = seeded_bf16(seq, nq, hd, seed=700), seeded_bf16(kv, nkv, hd, seed=701), seeded_bf16(kv, nkv, hd, seed=702)
    g = seeded_bf16(seq, nq, hd, seed=703)
    plain = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, mask_type=mask, window=win,
                             num_splits=splits, gate=g.cuda())
    # the copies sit inside a wider buffer (a head slice of a full-width output), like the gathered layout
    wide = [torch.full((seq, 2 * nq, hd), 9.0, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
    out = torch.empty(seq, 2 * nq, hd, dtype=torch.bfloat16, device="cuda")[:, nq:]
    copies = torch.tensor([w[:, nq:].data_ptr() for w in wide], dtype=torch.int64, device="cuda")
    gate_wide = torch.empty(seq, 2 * nq, hd, dtype=torch.bfloat16, device="cuda")[:, nq:]  # laid out like out
    gate_wide.copy_(g)
    got = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, mask_type=mask, window=win,
                           num_splits=splits, gate=gate_wide, out=out, out_copies=copies)
    torch.cuda.synchronize()
    assert torch.equal(got, plain)
    for w in wide:
        assert torch.equal(w[:, nq:], plain) and (w[:, :nq].float() == 9.0).all()


@pytest.mark.parametrize("gate", [False, True])
def test_two_tile_launch_with_a_single_head_tail(ops, gate):
    """13 token tiles x 16 head pairs = 208 two-tile units on 148 SMs: one whole wave of pairs, and the 60 pairs
    left over are cut into 120 single heads that a second launch (the one-tile kernel, one CTA per tile) takes
    behind the first.  Every row must come out exactly once, from either launch."""
    run_case(ops, 1664, 1664, 32, 16, 128, 128 ** -0.5, 3, 300, seed=800, gate=gate, lse=True)


def test_consumer_right_behind_the_two_launch_form_sees_finished_rows(ops):
    """The single-head tail runs beside the two-tile launch in front of it; what follows in the stream waits for
    the tail launch only, so the tail must not complete first.  A copy enqueued right behind the call, with no
    host synchronisation in between, has to see every row."""
    q, k, v = seeded_bf16(1664, 32, 128, seed=810).cuda(), seeded_bf16(1664, 16, 128, seed=811).cuda(), \
        seeded_bf16(1664, 16, 128, seed=812).cuda()
    ref = ops.sdpa_prefill(q, k, v, scale=128 ** -0.5, mask_type=ops.MASK_CAUSAL, window=300).clone()
    torch.cuda.synchronize()
    for _ in range(20):
        out = torch.zeros_like(ref)
        ops.sdpa_prefill(q, k, v, scale=128 ** -0.5, mask_type=ops.MASK_CAUSAL, window=300, out=out)
        snap = out.clone()
        torch.cuda.synchronize()
        assert torch.equal(snap, ref)


def test_gate_epilogue_and_split_gate(ops):
    run_case(ops, 150, 400, 6, 2, 256, 0.0625, 3, oracle.INT_MAX, seed=41, gate=True)
    run_case(ops, 150, 400, 6, 2, 256, 0.0625, 3, oracle.INT_MAX, seed=41, gate=True, num_splits=2)


def test_explicit_mask_equals_inline_rule(ops):
    seq, kv_len, nq, nkv, hd = 140, 260, 4, 2, 128
    q, k, v = seeded_bf16(seq, nq, hd, seed=51).cuda(), seeded_bf16(kv_len, nkv, hd, seed=52).cuda(), \
        seeded_bf16(kv_len, nkv, hd, seed=53).cuda()
    mask = ops.fill_causal_mask(seq, kv_len, past_offset=kv_len - seq, sliding_window=50)
    assert torch.equal(mask.cpu(), torch.from_numpy(oracle.fill_causal_mask(seq, kv_len, kv_len - seq, 50)))
    a = ops.sdpa_prefill(q, k, v, scale=0.1, mask_type=ops.MASK_EXPLICIT, mask=mask)
    b = ops.sdpa_prefill(q, k, v, scale=0.1, mask_type=ops.MASK_CAUSAL, window=50)
    assert_close(a, b.float(), "explicit vs inline", rel_tol=2e-3, abs_tol=4e-3)


def test_batched_strided_inputs_and_output_aliasing_query(ops):
    """batch 3 inside a larger cache allocation (token and batch strides), out written over q."""
    B, S, L, cap, nq, nkv, hd = 3, 140, 200, 256, 8, 4, 128
    q = seeded_bf16(B, S, nq, hd, seed=61)
    kc = seeded_bf16(B, cap, nkv, hd, seed=62)
    vc = seeded_bf16(B, cap, nkv, hd, seed=63)
    qd = q.cuda()
    out = ops.sdpa_prefill(qd, kc.cuda()[:, :L], vc.cuda()[:, :L], scale=0.09, mask_type=3, out=qd)
    assert out.data_ptr() == qd.data_ptr()
    for b in range(B):
        want, _ = oracle.sdpa_f32(q[b], kc[b, :L], vc[b, :L], scale=0.09, mask_type=3)
        assert_close(out[b], want, f"batch {b}")


def test_reference_named_entry_points(ops):
    seq, past, nq, nkv, hd = 130, 70, 8, 2, 256
    q, k, v = seeded_bf16(seq, nq, hd, seed=71), seeded_bf16(past + seq, nkv, hd, seed=72), seeded_bf16(past + seq, nkv, hd, seed=73)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    # qwen35_xmx_attention: causal over past + seq keys, output aliasing the query buffer
    buf = qd.clone()
    ops.qwen35_xmx_attention(buf, kd, vd, buf, seq, past, nq, nkv, hd, 0.0625)
    assert_close(buf, oracle.qwen35_online_attention(q, k, v, seq=seq, past=past, scale=0.0625).float(), "qwen35")
    # gqa_attention: no scale; inputs scaled down so the softmax is not one-hot
    qs = (q.float() * 0.25).bfloat16()
    got = ops.gqa_attention(qs.cuda(), seq, nq, hd, kd, vd, past + seq, nkv, past, 64, True)
    want, _ = oracle.sdpa_f32(qs, k, v, scale=1.0, mask_type=3, window=64)
    assert_close(got, want, "gqa_attention")
    # the restated matmul path keeps scores and probabilities in bf16, so it is itself
    # ~5e-2 away from the fp32 oracle at these magnitudes; this is a sanity bound, not the gate
    assert_close(got, oracle.gqa_attention(qs, k, v, past_offset=past, sliding_window=64, causal=True).float(),
                 "gqa_attention vs its restatement", rel_tol=2e-2, abs_tol=1.5e-1)
    got = ops.batched_attention(q.cuda(), seq, nq, hd, kd, vd, past + seq, nkv, hd, past, oracle.INT_MAX, scale=0.0625)
    assert_close(got, oracle.batched_attention(q, k, v, past_offset=past, scale=0.0625).float(), "batched_attention",
                 rel_tol=2e-2, abs_tol=1.5e-1)
    assert_close(got, oracle.sdpa_f32(q, k, v, scale=0.0625, mask_type=3)[0], "batched_attention vs fp32 oracle")
    with pytest.raises(ValueError):  # block ids must cover every key position
        ops.batched_attention(q.cuda(), seq, nq, hd, kd, vd, past + seq, nkv, hd, past, oracle.INT_MAX,
                              block_ids=torch.zeros(1, dtype=torch.int32, device="cuda"))


def test_error_statuses(ops):
    from arcaine_b200 import _lib
    q = torch.zeros(8, 4, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.ArcError) as e:
        ops.sdpa_prefill(q, q, q, scale=1.0)
    assert e.value.status == _lib.ARC_ERR_UNSUPPORTED_HEAD_DIM
    q = torch.zeros(8, 6, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(8, 4, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.ArcError) as e:
        ops.sdpa_prefill(q, k, k, scale=1.0)
    assert e.value.status == _lib.ARC_ERR_BAD_SHAPE
    q = torch.zeros(8, 4, 128, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.ArcError) as e:
        ops.sdpa_prefill(q, k, k, scale=-1.0)
    assert e.value.status == _lib.ARC_ERR_BAD_SHAPE
    # raw ABI: misaligned pointer, missing workspace for a forced split
    p = _lib.PrefillParams()
    big = torch.zeros(600, 4, 128, dtype=torch.bfloat16, device="cuda")
    p.q = p.k = p.v = p.out = big.data_ptr()
    p.batch, p.seq, p.kv_len, p.nq, p.nkv, p.hd = 1, 600, 600, 4, 4, 128
    for f in ("q", "k", "v", "o"):
        setattr(p, f + "_stride_t", 512)
        setattr(p, f + "_stride_b", 600 * 512)
    p.scale, p.mask_type, p.window, p.num_splits = 1.0, 0, ops.NO_WINDOW, 2
    L = _lib.load()
    assert L.arc_sdpa_prefill(C.byref(p), None) == _lib.ARC_ERR_WORKSPACE_TOO_SMALL
    p.num_splits = 1
    p.q = big.data_ptr() + 2
    assert L.arc_sdpa_prefill(C.byref(p), None) == _lib.ARC_ERR_ALIGNMENT
    assert L.arc_sdpa_prefill(None, None) == _lib.ARC_ERR_NULL_POINTER


def test_vision_block_mask_buffer_and_attention(ops):
    """Gemma4 vision blocks: the mask kernel against its restatement (bit for bit), then attention through
    the explicit-mask path against the oracle with the same buffer."""
    import numpy as np
    seq, kv_len, past, nq, nkv, hd = 150, 230, 80, 4, 2, 128
    ids = np.full(past + seq, -1, dtype=np.int32)
    ids[70:100] = 0
    ids[140:200] = 1
    for window in (oracle.INT_MAX, 64):
        want_mask = oracle.fill_causal_mask_with_block_ids(ids, seq, kv_len, past, window)
        mask = ops.fill_causal_mask_with_block_ids(torch.from_numpy(ids).cuda(), seq, kv_len, past, window)
        assert np.array_equal(mask.cpu().numpy(), want_mask)
        q, k, v = seeded_bf16(seq, nq, hd, seed=71), seeded_bf16(kv_len, nkv, hd, seed=72), seeded_bf16(kv_len, nkv, hd, seed=73)
        out = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, mask_type=ops.MASK_EXPLICIT, mask=mask)
        want = oracle.sdpa_f32(q, k, v, scale=hd ** -0.5, mask_type=1, mask=want_mask)
        assert_close(out, want[0], f"vision blocks, window {window}")
    plain = ops.fill_causal_mask_with_block_ids(None, seq, kv_len, past, 64, out=torch.empty(seq, kv_len, device="cuda"))
    assert torch.equal(plain, ops.fill_causal_mask(seq, kv_len, past, 64))


@pytest.mark.parametrize("hd", [128, 256])
def test_vision_block_ids_inside_the_kernel(ops, hd):
    """Gemma4 vision blocks evaluated in the attention kernel (no (seq, kv_len) buffer): against the oracle
    fed with the restated mask of src/common/kernels/attention_mask.hpp:44-73, with and without a window,
    a block that straddles query tiles and one that starts in the past; and through batched_attention."""
    import numpy as np
    seq, kv_len, nq, nkv = 300, 420, 4, 2
    past = kv_len - seq  # the cache holds every position from 0
    ids = np.full(kv_len, -1, dtype=np.int32)
    ids[100:190] = 0      # starts before the first query (position 120), ends inside the first tile
    ids[230:340] = 1      # straddles the first and second query tile
    ids[400:420] = 2      # runs to the end of the sequence
    ids_d = torch.from_numpy(ids).cuda()
    q, k, v = seeded_bf16(seq, nq, hd, seed=171), seeded_bf16(kv_len, nkv, hd, seed=172), seeded_bf16(kv_len, nkv, hd, seed=173)
    for window in (oracle.INT_MAX, 150):
        want_mask = oracle.fill_causal_mask_with_block_ids(ids, seq, kv_len, past, window)
        want = oracle.sdpa_f32(q, k, v, scale=hd ** -0.5, mask_type=1, mask=want_mask)
        out = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, mask_type=ops.MASK_CAUSAL, window=window,
                               block_ids=ids_d)
        assert_close(out, want[0], f"block ids in the kernel, window {window}")
        plain = ops.sdpa_prefill(q.cuda(), k.cuda(), v.cuda(), scale=hd ** -0.5, mask_type=ops.MASK_CAUSAL, window=window)
        assert not torch.equal(plain, out)  # the blocks do change the result
    # the reference-named call: K holds only the last 350 positions, so key 0 sits at absolute position 70
    kv2 = 350
    got = ops.batched_attention(q.cuda(), seq, nq, hd, k.cuda()[kv_len - kv2:], v.cuda()[kv_len - kv2:], kv2, nkv, hd,
                                past, oracle.INT_MAX, scale=0.08, block_ids=ids_d)
    want_mask = oracle.fill_causal_mask_with_block_ids(ids, seq, kv2, past, oracle.INT_MAX)
    want = oracle.sdpa_f32(q, k[kv_len - kv2:], v[kv_len - kv2:], scale=0.08, mask_type=1, mask=want_mask)
    assert_close(got, want[0], "batched_attention with block ids")


def test_gemma4_decode_wrappers(ops):
    """sliding_decode_attention (src/modeling/gemma4_unified/attention.cpp:93-137) over rows
    [kv_start, kv_start + kv_len) of the token-major cache, and the nkv == 1 path (:274-288) with more than
    16 query heads on the one KV head; no scale."""
    nq, nkv, hd, max_seq, kv_start, kv_len = 16, 8, 256, 700, 123, 512
    q = (seeded_bf16(nq, hd, seed=181).float() * 0.25).bfloat16()
    kc, vc = (seeded_bf16(max_seq, nkv, hd, seed=182).float() * 0.25).bfloat16(), seeded_bf16(max_seq, nkv, hd, seed=183)
    got = ops.gemma4_sliding_decode_attention(q.cuda(), kc.cuda(), vc.cuda(), kv_len, kv_start, nq, nkv, hd)
    want, _ = oracle.sdpa_f32(q[None], kc[kv_start:kv_start + kv_len], vc[kv_start:kv_start + kv_len], scale=1.0)
    assert_close(got, want[0], "gemma4 sliding decode")
    nq1, hd1, n = 32, 128, 333
    q1 = (seeded_bf16(nq1, hd1, seed=184).float() * 0.3).bfloat16()
    k1, v1 = (seeded_bf16(n, 1, hd1, seed=185).float() * 0.3).bfloat16(), seeded_bf16(n, 1, hd1, seed=186)
    got1 = ops.gemma4_full_decode_attention(q1.cuda(), k1.cuda(), v1.cuda(), n, nq1, hd1)
    want1, _ = oracle.sdpa_f32(q1[None], k1, v1, scale=1.0)
    assert_close(got1, want1[0], "gemma4 full-attention decode, one KV head")
