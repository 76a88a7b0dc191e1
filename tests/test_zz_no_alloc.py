"""arc_sdpa_decode_static: the decode entry point for callers that cannot supply or allocate scratch
(an arena-owning server, a thin FFI binding).  Called through the C ABI and compared with
arc_sdpa_decode, twice in a row so the second call runs on whatever the first left in the
library's built-in scratch array.  Collected last on purpose."""
import ctypes as C

import pytest
import torch

from helpers import assert_close, seeded_bf16

pytestmark = pytest.mark.gpu


def _params(q, k, v, out, gate, lens):
    from arcaine_b200 import _lib
    B, nq, hd = q.shape
    _, cap, nkv, _ = k.shape
    p = _lib.DecodeParams()
    p.q, p.k, p.v, p.out, p.gate = q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), gate.data_ptr()
    p.kv_len = lens.data_ptr()
    p.batch, p.nq, p.nkv, p.hd = B, nq, nkv, hd
    p.max_kv_len = cap
    p.q_stride_b = p.o_stride_b = nq * hd
    p.kv_stride_b, p.kv_stride_t, p.kv_rows_total = cap, nkv * hd, B * cap
    p.scale = hd ** -0.5
    return p


def test_static_scratch_decode_matches_workspace_decode_twice():
    from arcaine_b200 import _lib, ops
    L = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    for call, (B, nq, nkv, hd, lens) in enumerate([(3, 24, 4, 256, [900, 17, 2049]), (2, 16, 2, 128, [5000, 333])]):
        cap = max(lens)
        q, g = seeded_bf16(B, nq, hd, seed=900 + call).cuda(), seeded_bf16(B, nq, hd, seed=910 + call).cuda()
        k, v = seeded_bf16(B, cap, nkv, hd, seed=920 + call).cuda(), seeded_bf16(B, cap, nkv, hd, seed=930 + call).cuda()
        kl = torch.tensor(lens, dtype=torch.int32, device="cuda")
        want = ops.sdpa_decode(q, k, v, scale=hd ** -0.5, kv_len=kl, gate=g)      # existing entry point
        got = torch.full_like(want, float("nan"))
        p = _params(q, k, v, got, g, kl)                                           # no workspace given
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = L.arc_sdpa_decode_static(C.byref(p), stream)
        assert rc == _lib.ARC_OK, L.arc_sdpa_last_error()
        torch.cuda.synchronize()
        if call > 0:
            # what the name promises: the call took no device memory (the first call on a device may
            # still load the library's kernels; from the second on nothing may move)
            assert torch.cuda.mem_get_info()[0] == free_before
        # same kernels, same schedule: identical bits; the tolerance is the suite's usual one
        assert_close(got, want.float(), f"call {call}")
        assert torch.equal(got, want)
    assert ops.device_status() == (0, 0)


def test_static_scratch_decode_refuses_shapes_beyond_its_array():
    from arcaine_b200 import _lib
    L = _lib.load()
    B, nq, nkv, hd, cap = 512, 64, 8, 256, 16
    q = torch.zeros(B, nq, hd, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(B, cap, nkv, hd, dtype=torch.bfloat16, device="cuda")
    kl = torch.full((B,), cap, dtype=torch.int32, device="cuda")
    p = _params(q, k, k, q, q, kl)
    assert L.arc_sdpa_decode_workspace_bytes(C.byref(p)) > _lib.STATIC_SCRATCH_BYTES
    assert L.arc_sdpa_decode_static(C.byref(p), None) == _lib.ARC_ERR_TOO_LARGE
    assert b"built-in array" in L.arc_sdpa_last_error()
    assert L.arc_sdpa_decode_static(None, None) == _lib.ARC_ERR_NULL_POINTER
