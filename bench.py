#!/usr/bin/env python
"""Benchmark of the attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One JSON line on stdout (rank 0).  The headline workload is the sliding-window
prefill configuration (batch 4, 32Q/16KV, hd128, seq 8192, window 1024) reported
in TFLOP/s; the decode workloads (KV-read GB/s) ride along under "extra" unless
one of them is chosen with --workload.  A "step" is one pass of the operator over
one batch of seeded synthetic inputs.

Workloads
  prefill_window   config 3 — head-sharded over N GPUs (total work fixed)
  canvas           config 2 — 256-token canvas over a 2048-token prompt, hd256
  decode_gated     config 4 — batch 64, kv_len in [1024, 32768], sigmoid gate; sequences dealt to ranks
                   longest first, so that the ranks' key counts are even
  decode_long      config 5 — batch 4, KV 524288, sequence-sharded; the (out, lse) records are exchanged
                   inside the merge kernel by stores into the peers' memory over NVLink (NCCL
                   all-gather + merge as the fallback)
  qkv_prepare      the pre-processing of config 3 (RMSNorm + RoPE + cache append)

Every workload is timed two ways at every N: each step on its own pair of CUDA events after an L2
flush (the reported number), and all steps back to back (under "timing").  With N > 1 the line
also carries "parity": the sequence-sharded decode checked, outside every timed region, against a
plain fp32 softmax on the device and against its NCCL form, and two more lines under "extra":
"prefill_window_gathered" (config 3 with an NCCL all-gather of the output slices inside the step) and
"prefill_window_peer_gathered" (the same gather done by the kernel's own epilogue stores into the
other ranks' buffers over NVLink).

--impl reference times the CPU port of the reference's matmul/softmax/matmul path
(oracle/, all host threads) on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS if k in d} | {"source": "measured"}
    except Exception:
        return dict(FALLBACK_PEAKS) | {"source": "fallback"}


def load_traffic():
    """DRAM bytes per launch from committed ncu captures (profiles/ncu_traffic.json), keyed by workload."""
    try:
        with open(os.path.join(ROOT, "profiles", "ncu_traffic.json")) as f:
            return {k: v for k, v in json.load(f).items() if not k.startswith("_")}
    except Exception:
        return {}


# ---------------------------------------------------------------------------
# Clock / throttle sampling during the timed region
# ---------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) >= 7:
                self.samples.append(parts)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for s in self.samples:
            try:
                sm.append(float(s[0]))
                mx.append(float(s[1]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), s[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------
# Workload descriptions (shapes from the benchmark configurations)
# ---------------------------------------------------------------------------
CFG3 = dict(B=4, S=8192, nq=32, nkv=16, hd=128, W=1024)
CFG2 = dict(nq=16, nkv=8, hd=256, prompt=2048, canvas=256, steps=32)
CFG4 = dict(B=64, nq=24, nkv=4, hd=256, lo=1024, hi=32768)
CFG5 = dict(B=4, nq=16, nkv=2, hd=128, L=524288)


def window_pairs(S: int, W: int) -> int:
    """Unmasked (query, key) pairs of one head of one sequence: sum_i min(i + 1, W)."""
    return sum(min(i + 1, W) for i in range(S))


def cfg3_flops(batch: int, nq: int) -> float:
    return 4.0 * CFG3["hd"] * window_pairs(CFG3["S"], CFG3["W"]) * nq * batch


def cfg4_lengths():
    import torch
    g = torch.Generator().manual_seed(4)
    return torch.randint(CFG4["lo"], CFG4["hi"] + 1, (CFG4["B"],), generator=g, dtype=torch.int32)


# ---------------------------------------------------------------------------
# Workloads.  Each holds this rank's device-resident inputs, pinned host copies
# for the end-to-end arm, and enqueues one pass of the operator per step().
# ---------------------------------------------------------------------------
def workload_text(name: str) -> str:
    """One description per workload, shared by this arm's line and the reference arm's."""
    if name == "prefill_window":
        return "config 3: sliding-window prefill, batch 4, 32Q/16KV, hd128, seq 8192, causal window 1024"
    if name == "canvas":
        return ("config 2: DiffusionGemma denoising-step attention, 16Q/8KV, hd256, 256-token canvas "
                "over a 2048-token cached prompt, bidirectional, scale 1.0")
    if name == "decode_gated":
        return ("config 4: gated decode, batch 64, 24Q/4KV, hd256, kv_len uniform in [1024, 32768] "
                f"(seed 4, {int(sum(cfg4_lengths()))} keys), output * sigmoid(gate)")
    if name == "decode_long":
        return "config 5: long-context decode, batch 4, 16Q/2KV, hd128, KV 524288 per sequence"
    if name == "qkv_prepare":
        return ("pre-processing of config 3: RMSNorm + RoPE (Q, K), unit norm (V), KV-cache append; "
                "batch 4, seq 8192, 32Q/16KV, hd128, angles computed in the kernel")
    raise KeyError(name)


class Workload:
    name = ""
    metric = ""
    unit = ""
    bound = "hbm"
    scaling = "strong"
    dtype = "bf16"
    L2_BYTES = 126 * 1024 * 1024

    def working_set_bytes(self) -> int:  # bytes this rank's step touches in HBM
        raise NotImplementedError

    def timing_note(self) -> str:
        mb = self.working_set_bytes() / 1e6
        return (f"every step timed on its own CUDA event pair after an L2 flush (256 MB written, 256 MB read); "
                f"this rank's working set is {mb:.0f} MB against 126 MB of L2; the back-to-back time is under \"timing\"")

    def units_total(self) -> float:      # algorithmic units per step, whole job (all ranks)
        raise NotImplementedError

    def units_rank(self) -> float:       # algorithmic units per step of this rank's main kernel
        raise NotImplementedError

    def step(self):
        raise NotImplementedError

    def step_e2e(self):
        raise NotImplementedError

    def config(self) -> dict:
        raise NotImplementedError


def _randn_bf16(shape, seed, device):
    import torch
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(*shape, generator=g, device=device, dtype=torch.float32).bfloat16()


class PrefillWindow(Workload):
    """Config 3: KV heads (and then sequences) dealt to ranks; no collective in the timed step."""
    name = "prefill_window"
    metric = "sdpa_prefill_tflops"
    unit = "TFLOP/s"
    bound = "tensor"

    def __init__(self, rank, world, device, pin=True):
        import torch
        from arcaine_b200 import ops, sharded
        self.ops, self.torch = ops, torch
        c = CFG3
        self.world = world
        sh = sharded.plan_head_shards(c["nq"], c["nkv"], c["B"], world)[rank]
        self.B = sh.batch_end - sh.batch_begin
        self.nq = sh.q_head_end - sh.q_head_begin
        self.nkv = sh.kv_head_end - sh.kv_head_begin
        S, hd = c["S"], c["hd"]
        seed = 3000 + rank
        self.q = _randn_bf16((self.B, S, self.nq, hd), seed, device)
        self.k = _randn_bf16((self.B, S, self.nkv, hd), seed + 100, device)
        self.v = _randn_bf16((self.B, S, self.nkv, hd), seed + 200, device)
        self.out = torch.empty_like(self.q)
        self.scale = hd ** -0.5
        if pin:
            self.hq, self.hk, self.hv = (t.cpu().pin_memory() for t in (self.q, self.k, self.v))
            self.hout = torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        self.h2d = (self.q.numel() + self.k.numel() + self.v.numel()) * 2
        self.d2h = self.out.numel() * 2

    def working_set_bytes(self):
        return self.h2d + self.d2h

    def units_total(self):
        return cfg3_flops(CFG3["B"], CFG3["nq"]) / 1e12

    def units_rank(self):
        return cfg3_flops(self.B, self.nq) / 1e12

    def step(self):
        self.ops.sdpa_prefill(self.q, self.k, self.v, scale=self.scale, mask_type=self.ops.MASK_CAUSAL,
                              window=CFG3["W"], out=self.out)

    def step_e2e(self):
        """Host buffers in, host buffers out, through ops.sdpa_prefill: one call per sequence, so that the
        copy-in of sequence b+1, the kernel of b and the copy-out of b-1 overlap (two copy streams)."""
        torch = self.torch
        cur = torch.cuda.current_stream()
        if not hasattr(self, "s_in"):
            self.s_in, self.s_out = torch.cuda.Stream(), torch.cuda.Stream()
            self.ev_in = [torch.cuda.Event() for _ in range(self.B)]
            self.ev_done = [torch.cuda.Event() for _ in range(self.B)]
            for e in self.ev_done:
                e.record(cur)
        for b in range(self.B):
            self.s_in.wait_event(self.ev_done[b])  # the previous step's kernel no longer reads these inputs
            with torch.cuda.stream(self.s_in):
                self.q[b].copy_(self.hq[b], non_blocking=True)
                self.k[b].copy_(self.hk[b], non_blocking=True)
                self.v[b].copy_(self.hv[b], non_blocking=True)
                self.ev_in[b].record(self.s_in)
        for b in range(self.B):
            cur.wait_event(self.ev_in[b])
            self.ops.sdpa_prefill(self.q[b:b + 1], self.k[b:b + 1], self.v[b:b + 1], scale=self.scale,
                                  mask_type=self.ops.MASK_CAUSAL, window=CFG3["W"], out=self.out[b:b + 1])
            self.ev_done[b].record(cur)
            self.s_out.wait_event(self.ev_done[b])
            with torch.cuda.stream(self.s_out):
                self.hout[b].copy_(self.out[b], non_blocking=True)
        cur.wait_stream(self.s_out)  # the step ends when its result is on the host

    def config(self):
        c = CFG3
        return {"workload": workload_text("prefill_window"),
                "partition": f"KV heads then sequences over {self.world} rank(s); per rank batch {self.B}, "
                             f"{self.nq}Q/{self.nkv}KV; output stays head-sharded",
                "timing": self.timing_note()}


class Canvas(Workload):
    """Config 2: one DiffusionGemma denoising-step attention per step (scale 1.0, as the reference runs it)."""
    name = "canvas"
    metric = "sdpa_canvas_tflops"
    unit = "TFLOP/s"
    bound = "tensor"

    def working_set_bytes(self):
        return (self.q.numel() + self.k.numel() + self.v.numel() + self.out.numel()) * 2

    def __init__(self, rank, world, device, pin=True):
        import torch
        from arcaine_b200 import ops, sharded
        self.ops, self.torch = ops, torch
        c = CFG2
        self.world = world
        sh = sharded.plan_head_shards(c["nq"], c["nkv"], 1, world)[rank]
        self.nq, self.nkv = sh.q_head_end - sh.q_head_begin, sh.kv_head_end - sh.kv_head_begin
        L, hd = c["prompt"] + c["canvas"], c["hd"]
        self.q = _randn_bf16((c["canvas"], self.nq, hd), 2000 + rank, device)
        self.k = _randn_bf16((L, self.nkv, hd), 2100 + rank, device)
        self.v = _randn_bf16((L, self.nkv, hd), 2200 + rank, device)
        self.out = torch.empty_like(self.q)
        if pin:
            self.hq = self.q.cpu().pin_memory()
            self.hk = self.k[c["prompt"]:].cpu().pin_memory()
            self.hv = self.v[c["prompt"]:].cpu().pin_memory()
            self.hout = torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        self.h2d = (self.q.numel() + 2 * self.hk.numel()) * 2 if pin else 0
        self.d2h = self.out.numel() * 2

    def _flops(self, nq):
        c = CFG2
        return 4.0 * nq * c["canvas"] * (c["prompt"] + c["canvas"]) * c["hd"] / 1e12

    def units_total(self):
        return self._flops(CFG2["nq"])

    def units_rank(self):
        return self._flops(self.nq)

    def step(self):
        self.ops.sdpa_prefill(self.q, self.k, self.v, scale=1.0, out=self.out)

    def step_e2e(self):
        # each step brings fresh canvas Q/K/V; the prompt rows stay cached on the device
        p = CFG2["prompt"]
        self.q.copy_(self.hq, non_blocking=True)
        self.k[p:].copy_(self.hk, non_blocking=True)
        self.v[p:].copy_(self.hv, non_blocking=True)
        self.step()
        self.hout.copy_(self.out, non_blocking=True)

    def config(self):
        return {"workload": workload_text("canvas"),
                "partition": f"KV heads over {self.world} rank(s)",
                "timing": self.timing_note()}


class DecodeGated(Workload):
    """Config 4: batch 64 gated decode with per-sequence lengths; sequences dealt to ranks."""
    name = "decode_gated"
    metric = "sdpa_decode_kv_read_gbs"
    unit = "GB/s"

    def __init__(self, rank, world, device, pin=True):
        import torch
        from arcaine_b200 import ops
        self.ops, self.torch = ops, torch
        c = CFG4
        self.world = world
        from arcaine_b200 import sharded
        lens_all = cfg4_lengths()
        mine = sharded.plan_batch_shards(lens_all.tolist(), world)[rank]  # longest first: even key counts
        lens = lens_all[mine]
        self.B = len(mine)
        self.total_all = int(lens_all.sum())
        self.total = int(lens.sum())
        offs = torch.zeros(self.B, dtype=torch.int64)
        offs[1:] = torch.cumsum(lens[:-1].long(), 0)
        hd = c["hd"]
        self.k = _randn_bf16((self.total, c["nkv"], hd), 4100 + rank, device)
        self.v = _randn_bf16((self.total, c["nkv"], hd), 4200 + rank, device)
        self.q = _randn_bf16((self.B, c["nq"], hd), 4300 + rank, device)
        self.g = _randn_bf16((self.B, c["nq"], hd), 4400 + rank, device)
        self.lens, self.offs = lens.to(device), offs.to(device)
        self.out = torch.empty_like(self.q)
        self.scale = hd ** -0.5
        if pin:
            self.hq, self.hg = self.q.cpu().pin_memory(), self.g.cpu().pin_memory()
            # one new cache row per sequence arrives with every decode step
            self.hk_new = self.k[:self.B].cpu().pin_memory()
            self.hv_new = self.v[:self.B].cpu().pin_memory()
            self.last_rows = (self.offs + self.lens.long() - 1)
            self.hout = torch.empty(self.out.shape, dtype=self.out.dtype).pin_memory()
        self.h2d = (2 * self.q.numel() + 2 * self.B * c["nkv"] * hd) * 2
        self.d2h = self.out.numel() * 2

    def _bytes(self, total_keys, batch):
        c = CFG4
        return (total_keys * c["nkv"] * c["hd"] * 2 * 2 + 3 * batch * c["nq"] * c["hd"] * 2) / 1e9

    def working_set_bytes(self):
        return int(self._bytes(self.total, self.B) * 1e9)

    def units_total(self):
        return self._bytes(self.total_all, CFG4["B"])

    def units_rank(self):
        return self._bytes(self.total, self.B)

    def step(self):
        self.ops.sdpa_decode(self.q, self.k, self.v, scale=self.scale, kv_len=self.lens, kv_row_offset=self.offs,
                             gate=self.g, out=self.out)

    def step_e2e(self):
        self.q.copy_(self.hq, non_blocking=True)
        self.g.copy_(self.hg, non_blocking=True)
        knew = self.hk_new.to(self.q.device, non_blocking=True)
        vnew = self.hv_new.to(self.q.device, non_blocking=True)
        self.k.index_copy_(0, self.last_rows, knew)
        self.v.index_copy_(0, self.last_rows, vnew)
        self.step()
        self.hout.copy_(self.out, non_blocking=True)

    def config(self):
        return {"workload": workload_text("decode_gated"),
                "partition": f"sequences over {self.world} rank(s), dealt longest first ({self.B} sequences, "
                             f"{self.total} keys on this rank; mean {self.total_all // self.world})",
                "timing": self.timing_note()}


class DecodeLong(Workload):
    """Config 5: KV sequence cut into one slice per rank; partial (out, lse) records all-gathered and merged."""
    name = "decode_long"
    metric = "sdpa_decode_kv_read_gbs"
    unit = "GB/s"

    def __init__(self, rank, world, device, pin=True):
        import torch
        from arcaine_b200 import ops, sharded
        self.ops, self.torch = ops, torch
        c = CFG5
        self.world = world
        lo, hi = sharded.plan_seq_shards(c["L"], world)[rank]
        self.local = hi - lo
        hd = c["hd"]
        self.k = _randn_bf16((c["B"], self.local, c["nkv"], hd), 5100 + rank, device)
        self.v = _randn_bf16((c["B"], self.local, c["nkv"], hd), 5200 + rank, device)
        self.q = _randn_bf16((c["B"], c["nq"], hd), 5300, device)
        self.scale = hd ** -0.5
        self.runner = sharded.SeqShardedDecode(c["B"], c["nq"], hd, device)
        if pin:
            self.hq = self.q.cpu().pin_memory()
            self.hk_new = self.k[:, -1].cpu().pin_memory()
            self.hv_new = self.v[:, -1].cpu().pin_memory()
            self.hout = torch.empty(self.runner.out.shape, dtype=torch.bfloat16).pin_memory()
        self.h2d = (self.q.numel() + 2 * c["B"] * c["nkv"] * hd) * 2
        self.d2h = self.runner.out.numel() * 2

    def _bytes(self, keys):
        c = CFG5
        return c["B"] * keys * c["nkv"] * c["hd"] * 2 * 2 / 1e9

    def working_set_bytes(self):
        return int(self._bytes(self.local) * 1e9)

    def units_total(self):
        return self._bytes(CFG5["L"])

    def units_rank(self):
        return self._bytes(self.local)

    def step(self):
        self.runner(self.q, self.k, self.v, scale=self.scale)

    def step_e2e(self):
        self.q.copy_(self.hq, non_blocking=True)
        self.k[:, -1].copy_(self.hk_new, non_blocking=True)
        self.v[:, -1].copy_(self.hv_new, non_blocking=True)
        self.step()
        self.hout.copy_(self.runner.out, non_blocking=True)

    def config(self):
        return {"workload": workload_text("decode_long"),
                "partition": f"KV sequence over {self.world} rank(s) ({self.local} keys each); (out, lse) records "
                             f"exchanged by: {self.runner.mode}"
                             + (" (in-kernel stores into peers' memory over NVLink, flags, merge in the same kernel)"
                                if self.runner.mode == "peer" else
                                " (NCCL all-gather of the packed record, then the LSE merge kernel)"
                                if self.runner.mode == "nccl" else ""),
                "timing": self.timing_note()}


class QkvPrepare(Workload):
    """The step before config 3's attention: RMSNorm + RoPE of Q and K, unit norm of V, K/V appended to the
    cache, one launch; tokens dealt to ranks by KV head and sequence like the attention itself."""
    name = "qkv_prepare"
    metric = "qkv_prepare_gbs"
    unit = "GB/s"
    bound = "hbm"

    def __init__(self, rank, world, device, pin=True):
        import torch
        from arcaine_b200 import ops, sharded
        self.ops, self.torch = ops, torch
        c = CFG3
        self.world = world
        sh = sharded.plan_head_shards(c["nq"], c["nkv"], c["B"], world)[rank]
        self.B = sh.batch_end - sh.batch_begin
        self.nq = sh.q_head_end - sh.q_head_begin
        self.nkv = sh.kv_head_end - sh.kv_head_begin
        S, hd = c["S"], c["hd"]
        seed = 7000 + rank
        self.q = _randn_bf16((self.B, S, self.nq, hd), seed, device)
        self.k = _randn_bf16((self.B, S, self.nkv, hd), seed + 100, device)
        self.v = _randn_bf16((self.B, S, self.nkv, hd), seed + 200, device)
        self.kc = torch.empty_like(self.k)
        self.vc = torch.empty_like(self.v)
        self.qw = (_randn_bf16((hd,), seed + 300, device).float() * 0.1 + 1.0).bfloat16()
        self.kw = (_randn_bf16((hd,), seed + 400, device).float() * 0.1 + 1.0).bfloat16()
        if pin:
            self.hq, self.hk, self.hv = (t.cpu().pin_memory() for t in (self.q, self.k, self.v))
            self.hout = torch.empty(self.q.shape, dtype=self.q.dtype).pin_memory()
        self.h2d = (self.q.numel() + self.k.numel() + self.v.numel()) * 2
        self.d2h = self.q.numel() * 2

    def _bytes(self, B, nq, nkv):  # every element read once and written once
        return 2.0 * B * CFG3["S"] * (nq + 2 * nkv) * CFG3["hd"] * 2

    def working_set_bytes(self):
        return int(self._bytes(self.B, self.nq, self.nkv))

    def units_total(self):
        return self._bytes(CFG3["B"], CFG3["nq"], CFG3["nkv"]) / 1e9

    def units_rank(self):
        return self._bytes(self.B, self.nq, self.nkv) / 1e9

    def step(self):
        self.ops.qkv_prepare(self.q, self.k, self.v, k_cache=self.kc, v_cache=self.vc, past_len=0,
                             q_weight=self.qw, k_weight=self.kw, eps=1e-6, theta=10000.0, partial_rotary_factor=1.0)

    def step_e2e(self):
        self.q.copy_(self.hq, non_blocking=True)
        self.k.copy_(self.hk, non_blocking=True)
        self.v.copy_(self.hv, non_blocking=True)
        self.step()
        self.hout.copy_(self.q, non_blocking=True)

    def config(self):
        return {"workload": workload_text("qkv_prepare"),
                "partition": f"KV heads then sequences over {self.world} rank(s); per rank batch {self.B}, "
                             f"{self.nq}Q/{self.nkv}KV",
                "timing": self.timing_note()}


class PrefillWindowGathered(PrefillWindow):
    """Config 3 with the output gather inside the step: after the kernel every rank's slice goes to every
    rank by one NCCL all-gather (268 MB of output in total), as the head-sharded form needs when the
    consumer wants whole rows."""
    name = "prefill_window_gathered"

    def __init__(self, rank, world, device, pin=False):
        super().__init__(rank, world, device, pin=False)
        self.gathered = self.torch.empty((world,) + tuple(self.out.shape), dtype=self.out.dtype, device=device)

    def working_set_bytes(self):
        return (self.q.numel() + self.k.numel() + self.v.numel() + self.out.numel() + self.gathered.numel()) * 2

    def step(self):
        from arcaine_b200 import sharded
        sharded.prefill_head_sharded(self.q, self.k, self.v, scale=self.scale, mask_type=self.ops.MASK_CAUSAL,
                                     window=CFG3["W"], out_local=self.out, gather_into=self.gathered)

    def config(self):
        c = super().config()
        c["partition"] = c["partition"].replace("output stays head-sharded",
                                                "output slices all-gathered over NCCL inside the timed step")
        return c


class PrefillWindowPeerGathered(PrefillWindow):
    """Config 3 with the output gather inside the kernel: the epilogue stores every output row into every
    rank's gather buffer (symmetric memory, plain peer stores over NVLink), so the transfer overlaps the
    attention tile by tile and no collective follows."""
    name = "prefill_window_peer_gathered"

    def __init__(self, rank, world, device, pin=False):
        super().__init__(rank, world, device, pin=False)
        from arcaine_b200 import sharded
        self.runner = sharded.GatheredPrefill(tuple(self.out.shape), device)

    def working_set_bytes(self):
        return (self.q.numel() + self.k.numel() + self.v.numel() + self.runner.gathered.numel()) * 2

    def step(self):
        self.runner(self.q, self.k, self.v, scale=self.scale, mask_type=self.ops.MASK_CAUSAL, window=CFG3["W"])

    def config(self):
        c = super().config()
        c["partition"] = c["partition"].replace("output stays head-sharded",
                                                "output rows stored into every rank's buffer by the kernel's epilogue (peer stores over NVLink)")
        return c


WORKLOADS = {w.name: w for w in (PrefillWindow, Canvas, DecodeGated, DecodeLong, QkvPrepare)}


# ---------------------------------------------------------------------------
# Timing
# ---------------------------------------------------------------------------
class Runner:
    def __init__(self, rank, world, device):
        import torch
        import torch.distributed as dist
        self.torch, self.dist = torch, dist
        self.rank, self.world, self.device = rank, world, device
        self.flush_buf = None

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(self, x: float) -> float:
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
        return float(t.item())

    def flush_l2(self):
        """Write 256 MB, then read another 256 MB: whatever the previous step left in L2 is gone, and
        the lines that are left are clean, so the timed step does not pay for the flush's write-backs."""
        if self.flush_buf is None:
            self.flush_buf = self.torch.empty(256 << 20, dtype=self.torch.uint8, device=self.device)
            self.flush_src = self.torch.zeros(64 << 20, dtype=self.torch.int32, device=self.device)
        self.flush_buf.zero_()
        self.flush_sink = self.flush_src.sum()

    def time_steps(self, fn, steps, warmup, flush=False):
        """Device time of exactly `steps` calls (ms, max over ranks), CUDA events on the launching stream."""
        torch = self.torch
        for _ in range(warmup):
            fn()
        self.barrier()
        if not flush:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                fn()
            e1.record()
            self.barrier()
            ms = e0.elapsed_time(e1)
        else:
            pairs = []
            for _ in range(steps):
                self.flush_l2()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn()
                b.record()
                pairs.append((a, b))
            self.barrier()
            ms = sum(a.elapsed_time(b) for a, b in pairs)
        return self.max_over_ranks(ms)


def measure(workload_cls, runner, steps, warmup, peaks, traffic, with_e2e=True, sample_clocks=True):
    """Run one workload: device-resident steps, then the end-to-end arm.  Returns the JSON fields."""
    from arcaine_b200 import ops
    w = workload_cls(runner.rank, runner.world, runner.device, pin=with_e2e)
    sampler = ClockSampler(runner.device.index or 0) if (sample_clocks and runner.rank == 0) else None
    # warm-up happens inside time_steps; start sampling just before the timed loop of a second pass
    runner.time_steps(w.step, min(steps, 3), warmup, True)
    if sampler:
        sampler.start()
    l0 = ops.launch_count()
    ms = runner.time_steps(w.step, steps, 0, True)       # the reported number: L2 flushed before every step
    launches = ops.launch_count() - l0
    ms_b2b = runner.time_steps(w.step, steps, 0, False)  # and the same steps back to back
    clocks = sampler.stop() if sampler else None
    launches_total = int(runner.sum_over_ranks(float(launches)))
    status = ops.device_status()
    if status != (0, 0):
        ops.clear_device_status()  # re-arm the kernels: what follows (extras, parity) must not inherit it
        raise RuntimeError(f"device-side wait timed out during the bench: {status}")
    ms_step = ms / steps
    value = w.units_total() / (ms_step / 1e3)
    peak = peaks["bf16_tflops"] if w.bound == "tensor" else peaks["hbm_gbs"]
    achieved = w.units_rank() / (ms_step / 1e3)
    res = {
        "metric": w.metric, "value": round(value, 3), "unit": w.unit, "ms_per_step": round(ms_step, 6),
        "scaling": w.scaling, "dtype": w.dtype, "config": w.config(),
        "roofline": {"bound": w.bound, "achieved": round(achieved, 3), "peak": peak,
                     "unit": "TFLOP/s" if w.bound == "tensor" else "GB/s", "frac": round(achieved / peak, 4),
                     "traffic": traffic.get(w.name), "peak_source": f"of {peaks['source']}"
                     + (" (burst cuBLAS bf16)" if w.bound == "tensor" else " (copy)"),
                     "kernel_time": "rank 0 step time, all launches of the step (main kernel plus merge where split)"},
        "gpu_launches": launches_total,
        "timing": {"method": "l2_flush_per_step", "ms_per_step_flushed": round(ms_step, 6),
                   "ms_per_step_back_to_back": round(ms_b2b / steps, 6)},
    }
    if clocks:
        res["clocks"] = clocks
    if with_e2e:
        ms_e = runner.time_steps(w.step_e2e, steps, max(3, min(warmup, 5)), False)
        ms_e_step = ms_e / steps
        res["e2e"] = {"value": round(w.units_total() / (ms_e_step / 1e3), 3), "unit": w.unit,
                      "ms_per_step": round(ms_e_step, 6),
                      "h2d_bytes_per_step": int(runner.sum_over_ranks(float(w.h2d))),
                      "d2h_bytes_per_step": int(runner.sum_over_ranks(float(w.d2h)))}
    del w
    runner.torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------
# Correctness record of the multi-GPU paths (outside every timed region)
# ---------------------------------------------------------------------------
def multi_gpu_parity(runner):
    """Sequence-sharded decode on a small case (batch 2, 4096 keys per rank): the in-kernel NVLink
    exchange against a plain fp32 softmax over the whole key range computed with torch on the device,
    and against the NCCL all-gather + merge form on the same inputs.  Every rank draws the same
    seeded K / V and keeps its slice.  Returns the record rank 0 prints."""
    import torch
    from arcaine_b200 import ops, sharded
    world, rank, dev = runner.world, runner.rank, runner.device
    B, nq, nkv, hd = 2, 16, 2, 128
    L = 4096 * world
    k = _randn_bf16((B, L, nkv, hd), 9100, dev)
    v = _randn_bf16((B, L, nkv, hd), 9200, dev)
    q = _randn_bf16((B, nq, hd), 9300, dev)
    gate = _randn_bf16((B, nq, hd), 9400, dev)
    scale = hd ** -0.5
    lo, hi = sharded.plan_seq_shards(L, world)[rank]
    kl, vl = k[:, lo:hi].contiguous(), v[:, lo:hi].contiguous()
    outs = {}
    modes = []
    for mode in ("auto", "nccl"):
        run = sharded.SeqShardedDecode(B, nq, hd, dev, exchange=mode)
        for _ in range(2):  # two steps: both parities of the exchange buffer
            out = run(q, kl, vl, scale=scale, gate=gate)
        torch.cuda.synchronize()
        outs[run.mode] = out.float().clone()
        modes.append(run.mode)
        del run
    # fp32 reference on the device: softmax(scale * q k^T) v per KV group, then the gate on the bf16-rounded result
    G = nq // nkv
    qf = q.float().view(B, nkv, G, hd)
    s = torch.einsum("bhgd,blhd->bhgl", qf, k.float()) * scale
    ref = torch.einsum("bhgl,blhd->bhgd", torch.softmax(s, dim=-1), v.float()).reshape(B, nq, hd)
    ref = ref.bfloat16().float() * torch.sigmoid(gate.float())
    got = outs[modes[0]]
    rel = float((got - ref).norm() / ref.norm())
    mx = float((got - ref).abs().max())
    rec = {"case": f"sequence-sharded gated decode, batch {B}, {nq}Q/{nkv}KV, hd{hd}, {L} keys over {world} ranks",
           "mode": modes[0], "vs_fp32_softmax": {"rel_l2": round(rel, 6), "max_abs": round(mx, 6)},
           "tolerance": {"rel_l2": 1e-2, "max_abs": 2e-2}}
    if modes[0] != modes[1]:
        rec["peer_vs_nccl_max_abs"] = round(float((outs[modes[0]] - outs[modes[1]]).abs().max()), 6)
    bad = runner.max_over_ranks(0.0 if (rel <= 1e-2 and mx <= 2e-2 and rec.get("peer_vs_nccl_max_abs", 0.0) <= 8e-3) else 1.0)
    rec["ok_on_all_ranks"] = bad == 0.0
    status = ops.device_status()
    rec["device_status"] = list(status)
    return rec


# ---------------------------------------------------------------------------
# CPU baseline: the port of the reference's matmul/softmax/matmul path (oracle/)
# ---------------------------------------------------------------------------
def cpu_library_baselines(workload: str):
    """Two more CPU numbers for the prefill workloads, from libraries in the image (torch 2.11 and the
    oneDNN it bundles), on the same bounded sample as the port: torch's fused CPU attention in bf16,
    and bf16 matmul -> fp32 softmax -> bf16 matmul, the closest runnable analogue of the reference's
    own matmul path (src/modeling/diffusion_gemma/attention.cpp:706-821 over src/common/gpu/ops.hpp:233-276).
    The window mask is an explicit boolean mask there: these libraries do not skip masked blocks, the
    figure is algorithmic FLOPs (unmasked pairs only) per second all the same."""
    import torch
    import torch.nn.functional as F
    if workload not in ("prefill_window", "canvas"):
        return {}
    threads = torch.get_num_threads()
    g = torch.Generator().manual_seed(7)
    if workload == "prefill_window":
        c = CFG3
        S, L, nq, nkv, hd, scale = c["S"], c["S"], c["nq"], c["nkv"], c["hd"], c["hd"] ** -0.5
        flops = cfg3_flops(1, nq)
        i = torch.arange(S)
        mask = (i[None, :] <= i[:, None]) & (i[None, :] > i[:, None] - c["W"])
        sample = "1 of 4 sequences, all heads, dense 8192 x 8192 scores with a boolean window mask"
    else:
        c = CFG2
        S, L, nq, nkv, hd, scale = c["canvas"], c["prompt"] + c["canvas"], c["nq"], c["nkv"], c["hd"], 1.0
        flops = 4.0 * nq * S * L * hd
        mask = None
        sample = "all 16 query heads, full canvas and prompt"
    q = (torch.randn(1, nq, S, hd, generator=g) * hd ** -0.25).bfloat16()
    k = (torch.randn(1, nkv, L, hd, generator=g) * hd ** -0.25).bfloat16()
    v = torch.randn(1, nkv, L, hd, generator=g).bfloat16()
    out = {}
    with torch.no_grad():
        F.scaled_dot_product_attention(q[:, :, :128], k, v, attn_mask=None if mask is None else mask[:128],
                                       scale=scale, enable_gqa=True)  # warm-up
        t0 = time.perf_counter()
        F.scaled_dot_product_attention(q, k, v, attn_mask=mask, scale=scale, enable_gqa=True)
        dt = time.perf_counter() - t0
        out["torch_sdpa_bf16"] = {"value": round(flops / dt / 1e12, 4), "unit": "TFLOP/s", "cores": threads,
                                  "seconds": round(dt, 3), "sample": sample}
        # decomposed: per KV head, its query heads as rows of one bf16 GEMM
        G = nq // nkv
        addm = None if mask is None else torch.zeros(S, L).masked_fill_(~mask, float("-inf"))
        t0 = time.perf_counter()
        for h in range(nkv):
            qh = q[0, h * G:(h + 1) * G]                                  # (G, S, hd)
            sc = torch.matmul(qh, k[0, h].transpose(0, 1)).float() * scale  # bf16 GEMM, fp32 scores
            if addm is not None:
                sc += addm
            pr = torch.softmax(sc, dim=-1).bfloat16()
            torch.matmul(pr, v[0, h])
        dt = time.perf_counter() - t0
        out["onednn_matmul_path"] = {"value": round(flops / dt / 1e12, 4), "unit": "TFLOP/s", "cores": threads,
                                     "seconds": round(dt, 3), "sample": sample}
    return out



def cpu_sample(workload: str, reps: int = 1):
    """Time the CPU port on a bounded sample of the workload.  Returns (value, unit, cores, sample text)."""
    import torch
    import oracle
    # all the cores this process may run on, whatever OMP_NUM_THREADS a launcher set
    try:
        avail = len(os.sched_getaffinity(0))
    except AttributeError:
        avail = os.cpu_count() or 1
    oracle.set_num_threads(avail)
    cores = oracle.num_threads()
    if workload in ("prefill_window", "canvas"):
        if workload == "prefill_window":
            c = CFG3
            S, L, nq, nkv, hd = c["S"], c["S"], c["nq"], c["nkv"], c["hd"]
            sample = "1 of 4 sequences, all 32 query heads (16 KV heads), full 8192 tokens, window 1024"
            flops = cfg3_flops(1, nq)
            kw = dict(past_offset=0, sliding_window=c["W"], causal=True)
        else:
            c = CFG2
            S, L, nq, nkv, hd = c["canvas"], c["prompt"] + c["canvas"], 4, 2, c["hd"]
            sample = "4 of 16 query heads (2 KV heads), full canvas and prompt"
            flops = 4.0 * nq * S * L * hd
            kw = dict(past_offset=0, causal=False)
        g = torch.Generator().manual_seed(7)
        q = (torch.randn(S, nq, hd, generator=g) * hd ** -0.25).bfloat16()   # the path has no scale argument
        k = (torch.randn(L, nkv, hd, generator=g) * hd ** -0.25).bfloat16()
        v = torch.randn(L, nkv, hd, generator=g).bfloat16()
        oracle.gqa_attention(q[:64], k, v, **{**kw, "past_offset": 0})  # warm the library / threads
        t0 = time.perf_counter()
        for _ in range(reps):
            oracle.gqa_attention(q, k, v, **kw)
        dt = (time.perf_counter() - t0) / reps
        return flops / dt / 1e12, "TFLOP/s", cores, sample, dt
    if workload == "qkv_prepare":
        c = CFG3
        S, nq, nkv, hd = 1024, c["nq"], c["nkv"], c["hd"]
        sample = "1 of 4 sequences, 1024 of 8192 tokens, all heads (single thread: the restatement is scalar)"
        g = torch.Generator().manual_seed(9)
        q = torch.randn(S, nq, hd, generator=g).bfloat16()
        k = torch.randn(S, nkv, hd, generator=g).bfloat16()
        v = torch.randn(S, nkv, hd, generator=g).bfloat16()
        w = torch.ones(hd).bfloat16()
        t0 = time.perf_counter()
        for _ in range(reps):
            oracle.norm_rope(q, w, eps=1e-6, n_active_pairs=hd // 2, theta=10000.0)
            oracle.norm_rope(k, w, eps=1e-6, n_active_pairs=hd // 2, theta=10000.0)
            oracle.norm_rope(v, None, eps=1e-6)
        dt = (time.perf_counter() - t0) / reps
        return 2.0 * S * (nq + 2 * nkv) * hd * 2 / dt / 1e9, "GB/s", 1, sample, dt
    # decode: the scalar online-softmax kernel's arithmetic over a slice of the KV
    if workload == "decode_gated":
        c = CFG4
        B, L, nq, nkv, hd = 4, 16384, c["nq"], c["nkv"], c["hd"]
        sample = "4 of 64 sequences at 16384 keys each, all heads"
    else:
        c = CFG5
        B, L, nq, nkv, hd = 1, 65536, c["nq"], c["nkv"], c["hd"]
        sample = "1 of 4 sequences, 1/8 of the 524288 keys, all heads"
    g = torch.Generator().manual_seed(8)
    q = torch.randn(B, 1, nq, hd, generator=g).bfloat16()
    k = torch.randn(B, L, nkv, hd, generator=g).bfloat16()
    v = torch.randn(B, L, nkv, hd, generator=g).bfloat16()
    t0 = time.perf_counter()
    for _ in range(reps):
        for b in range(B):
            oracle.sdpa_f32(q[b], k[b], v[b], scale=hd ** -0.5)
    dt = (time.perf_counter() - t0) / reps
    return B * L * nkv * hd * 4 / dt / 1e9, "GB/s", cores, sample, dt


def run_reference_arm(args):
    """CPU port of the reference path on the host cores; rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cls = WORKLOADS[args.workload]
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_sample(args.workload)
    t0 = time.perf_counter()
    vals = []
    for _ in range(args.steps):
        v, unit, cores, sample, dt = cpu_sample(args.workload)
        vals.append((v, dt))
        if time.perf_counter() - t0 > 240:
            break
    steps_done = len(vals)
    ms = sum(d for _, d in vals) / steps_done * 1e3
    value = sum(v for v, _ in vals) / steps_done
    line = {
        "impl": "reference", "metric": cls.metric, "value": round(value, 6), "unit": unit, "n_gpus": args.gpus,
        "steps": steps_done, "warmup": min(args.warmup, 1), "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": cls.scaling, "vs_baseline": None, "dtype": "bf16 storage, fp32 math", "data": "synthetic",
        "config": {"workload": workload_text(args.workload),
                   "note": "each step is a bounded sample of the workload on the host CPU: " + sample},
        "cpu_baseline": {"value": round(value, 6), "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": round(value, 6), "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    if args.workload in ("prefill_window", "canvas"):
        # the two library CPU paths on the same sample, beside the port this arm reports: a reader who wants
        # the ratio against the fastest CPU implementation finds it here
        try:
            others = cpu_library_baselines(args.workload)
            if others:
                line["cpu_baseline"]["others"] = others
                line["cpu_baseline"]["fastest"] = max(others, key=lambda k: others[k]["value"])
        except Exception as e:
            line["cpu_baseline"]["others_error"] = repr(e)
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="prefill_window")
    ap.add_argument("--no-extra", action="store_true", help="skip the ride-along workloads")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        run_reference_arm(args)
        return

    # Libraries (NCCL's version banner, for one) may write to stdout; the contract is ONE JSON
    # line there.  Everything but that line goes to stderr.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the operators have no CPU path")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        log(f"warning: --gpus {args.gpus} but WORLD_SIZE {world}")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    runner = Runner(rank, world, device)
    peaks, traffic = load_peaks(), load_traffic()

    main_res = measure(WORKLOADS[args.workload], runner, args.steps, args.warmup, peaks, traffic,
                       with_e2e=not args.no_e2e)
    extra = {}
    if not args.no_extra:
        for name in ("decode_gated", "decode_long", "canvas", "qkv_prepare", "prefill_window"):
            if name == args.workload:
                continue
            try:
                r = measure(WORKLOADS[name], runner, max(5, min(args.steps, 20)), 3, peaks, traffic,
                            with_e2e=False, sample_clocks=False)
                extra[name] = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "roofline", "config", "timing")}
            except Exception as e:  # an extra never takes the headline down
                extra[name] = {"error": repr(e)}
        if world > 1 and args.workload == "prefill_window":
            for cls in (PrefillWindowGathered, PrefillWindowPeerGathered):
                try:
                    r = measure(cls, runner, max(5, min(args.steps, 20)), 3, peaks, traffic,
                                with_e2e=False, sample_clocks=False)
                    extra[cls.name] = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "roofline", "config", "timing")}
                except Exception as e:
                    extra[cls.name] = {"error": repr(e)}
    parity = None
    if world > 1:
        try:
            parity = multi_gpu_parity(runner)
        except Exception as e:
            parity = {"error": repr(e)}
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        try:
            v, unit, cores, sample, dt = cpu_sample(args.workload)
            cpu = {"value": round(v, 6), "unit": unit, "cores": cores, "kind": "port", "sample": sample,
                   "seconds": round(dt, 3)}
            try:
                others = cpu_library_baselines(args.workload)
                if others:
                    cpu["others"] = others
                    best = max(list(others.items()) + [("port", cpu)], key=lambda kv: kv[1]["value"])
                    cpu["fastest"] = best[0]
            except Exception as e:
                cpu["others"] = {"error": repr(e)}
        except Exception as e:
            cpu = {"error": repr(e)}
    if rank == 0:
        line = {"metric": main_res["metric"], "value": main_res["value"], "unit": main_res["unit"],
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"],
                "higher_is_better": True, "scaling": main_res["scaling"], "vs_baseline": None,
                "dtype": main_res["dtype"], "data": "synthetic", "config": main_res["config"],
                "roofline": main_res["roofline"], "gpu_launches": main_res["gpu_launches"],
                "clocks": main_res.get("clocks"), "timing": main_res["timing"]}
        if parity is not None:
            line["parity"] = parity
        if "e2e" in main_res:
            line["e2e"] = main_res["e2e"]
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if extra:
            line["extra"] = extra
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
