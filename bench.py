#!/usr/bin/env python
"""Benchmark of the low-bit KV-cache decode-attention step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C2]

A *step* is one decode-attention call (split-KV decode kernel + split combine) over one batch of
synthetic, seeded inputs.  The default workload is the Llama-3-8B decode shape the headline metric is
quoted on: batch 8, 32 query / 8 KV heads, head_dim 128, 32768 tokens of 4-bit cache (group 128) plus a
64-token fp16 tail.

With N > 1 (launched by torch.distributed.run, one rank per GPU) the SAME job is sharded over the ranks
(strong scaling): the batch of 8 is split 4/2/1 sequences per GPU with no data-path collective; workloads
sharded by KV heads (C4, C5a) likewise; a single long sequence (C5b) is split along its tokens and the
ranks exchange their (out, lse) partials inside the timed step.  Before timing, the sharded result is
compared with a one-GPU decode of the whole job on rank 0 ("check").

Prints ONE JSON line (rank 0):
  value      whole-job decode throughput in tokens/s (sequences advanced per second), cache resident in
             HBM, device-timed with CUDA events around CUDA-graph replays, max over ranks, median of
             repeated K-step regions
  e2e        the same step through the public Python API with the step's inputs (q and the new token's
             K/V rows) copied from pinned host memory and the output copied back inside the timed region
  roofline   algorithmic HBM bytes per step / measured step time, against the measured copy bandwidth
  cpu_baseline  the CPU oracle (a port of the reference algorithm; the reference has no CPU path) timed
             on a bounded sample on this host's cores
  sharded    (default run only) the other configurations of the baseline, sharded the way each is
             specified, with their own time, roofline fraction and check

`--impl reference` times the CPU port alone with all host threads on the whole batch, same metric and
config, and adds the timing of the reference's own CUDA kernel (recompiled for sm_100a) when built.
"""
from __future__ import annotations

import argparse
import datetime
import json
import math
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode-attn throughput (4/2-bit KV cache, 32k ctx): tokens/s; us/step and HBM TB/s alongside"
UNIT = "tokens/s"
FALLBACK_HBM_GBS = 6650.0
L2_BYTES = 126 * 2**20
CHUNK = 131072          # tokens generated and packed at a time

WORKLOADS = {
    # full problem; `shard` says how it is cut over GPUs
    "C1": dict(b=1, h=32, h_k=8, s=4096, bits=4, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
               shard="batch", desc="b1 32q/8kv d128 s4096 4-bit g128"),
    "C2": dict(b=8, h=32, h_k=8, s=32768, bits=4, group=128, res=64, dtype="fp16", ragged=False, outliers=0.0,
               shard="batch", desc="Llama-3-8B decode: b8 32q/8kv d128 s32768 4-bit g128 + 64-token fp16 tail"),
    "C3": dict(b=1, h=32, h_k=8, s=131072, bits=2, group=64, res=0, dtype="fp16", ragged=False, outliers=0.05,
               shard="sequence", desc="b1 32q/8kv d128 s131072 2-bit g64, 5% K outlier channels x10"),
    "C4": dict(b=32, h=32, h_k=32, s=16384, bits=4, group=128, res=128, dtype="bf16", ragged=True, outliers=0.0,
               shard="kv_heads", desc="Llama-2-7B MHA: b32 32/32 d128 ragged s in [1024,16384] 4-bit g128 bf16"),
    "C5a4": dict(b=16, h=64, h_k=8, s=131072, bits=4, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
                 shard="kv_heads", desc="Llama-3-70B: b16 64q/8kv d128 s131072 4-bit g128"),
    "C5a2": dict(b=16, h=64, h_k=8, s=131072, bits=2, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
                 shard="kv_heads", desc="Llama-3-70B: b16 64q/8kv d128 s131072 2-bit g128"),
    "C5b": dict(b=1, h=64, h_k=8, s=1048576, bits=4, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
                shard="sequence", desc="Llama-3-70B, one sequence of 1 Mi tokens: b1 64q/8kv d128 4-bit g128"),
}
# DRAM bytes (read + write) of one decode launch relative to its algorithmic bytes, from ncu captures of these
# workloads (every block is read once; partials and the tail add the rest)
NCU_TRAFFIC_RATIO = {"C2": 291_137_536 / 287_440_896, "C3": 86_691_072 / 83_902_464,
                     "C4": 1_230_654_464 / 1_212_579_840, "C1": 4_556_544 / 4_472_832}


def algorithmic_bytes(w, seqlens=None, res_lens=None, b=None, h=None, h_k=None, s=None) -> int:
    """HBM bytes one decode step has to move: codes, scales/zeros, tail, q and out."""
    b = w["b"] if b is None else b
    h = w["h"] if h is None else h
    h_k = w["h_k"] if h_k is None else h_k
    s = w["s"] if s is None else s
    d, bits, group = 128, w["bits"], w["group"]
    tok = sum(seqlens) if seqlens is not None else b * s
    rtok = sum(res_lens) if res_lens is not None else b * w["res"]
    codes = 2 * tok * h_k * d * bits // 8
    params = tok * h_k * d * 4 // group + tok * h_k * (d // group) * 4
    tail = 2 * rtok * h_k * d * 2
    qo = 2 * b * h * d * 2
    return codes + params + tail + qo


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return FALLBACK_HBM_GBS, "fallback (6.65 TB/s)"


def shard_range(n, rank, world):
    base, extra = divmod(n, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def job_config(name, w, world):
    """The part of the line that names the job; the same for both arms."""
    mode = w["shard"] if world > 1 else "none"
    how = {"none": "one GPU holds the whole job",
           "batch": f"batch of {w['b']} split over {world} GPUs, no data-path collective",
           "kv_heads": f"{w['h_k']} KV heads (and their query heads) split over {world} GPUs, no data-path collective",
           "sequence": f"{w['s']} tokens split over {world} GPUs; (out, lse) partials exchanged and merged inside the step"}
    return {"workload": f"{name}: {w['desc']}", "global_batch": w["b"], "n_shards": world, "sharding": how[mode]}


# ---------------------------------------------------------------------------
# clocks sampler (read-only NVML queries in a thread)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples = []
        self.sm_max = None
        self._stop = threading.Event()
        self._thread = None
        self.period = period_s
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, mask))
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        mask_all = 0
        for _, m in self.samples:
            mask_all |= m
        reasons = sorted(name for bit, name in self.REASONS.items() if mask_all & bit and name != "gpu_idle")
        return {"sm_mhz": int(statistics.median(s[0] for s in self.samples)), "sm_max_mhz": self.sm_max,
                "reasons": reasons, "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# workload construction: seeded per (sequence, chunk), so that any rank can build any shard and
# rank 0 can build the whole job for the check
# ---------------------------------------------------------------------------
class Shard:
    """Which part of the job one rank (or, with world = 1, one GPU) holds."""

    def __init__(self, w, rank, world):
        mode = w["shard"] if world > 1 else "none"
        self.mode = mode
        self.b_lo, self.b_hi = (shard_range(w["b"], rank, world) if mode == "batch" else (0, w["b"]))
        self.h_lo, self.h_hi = (shard_range(w["h_k"], rank, world) if mode == "kv_heads" else (0, w["h_k"]))
        nb = 32 * (16 // w["bits"])
        if mode == "sequence":
            blo, bhi = shard_range(w["s"] // nb, rank, world)
            self.t_lo, self.t_hi = blo * nb, bhi * nb
        else:
            self.t_lo, self.t_hi = 0, w["s"]
        self.b, self.h_k, self.s = self.b_hi - self.b_lo, self.h_hi - self.h_lo, self.t_hi - self.t_lo
        self.gq = w["h"] // w["h_k"]
        self.h = self.h_k * self.gq
        self.has_tail = w["res"] > 0 and (mode != "sequence" or rank == world - 1)


def _gen(device, *key):
    import torch
    seed = 0x9E3779B97F4A7C15
    for k in key:
        seed = (seed * 6364136223846793005 + int(k) + 1442695040888963407) % (1 << 63)
    return torch.Generator(device=device).manual_seed(seed)


def _ragged_lengths(w, seed):
    import torch
    cg = torch.Generator(device="cpu").manual_seed(seed)
    total = torch.randint(1024, w["s"] + 1, (w["b"],), generator=cg)
    seq = (total // 128) * 128
    return seq, total - seq


_SPACER = {}


def _spacer(device):
    import torch
    key = str(device)
    if key not in _SPACER:
        _SPACER[key] = torch.zeros(48 * 1024 * 1024, dtype=torch.int32, device=device)       # 192 MiB: 1.5 x the L2
    return _SPACER[key]


def build_cache(B, w, sh, device, seed, copy):
    """One packed cache copy of this shard (seeded N(0,1) K/V, generated chunk by chunk on the device and
    packed with the library's own kernel).  Returns (bufs, pack_ms list)."""
    import torch
    tdt = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    d = 128
    bufs = B.alloc_packed_cache(sh.b, max(sh.s, 32 * (16 // w["bits"])), sh.h_k, d, w["bits"], w["group"], device=device)
    pack_ms = []
    outl = {}
    for ib in range(sh.b_lo, sh.b_hi):
        for t0 in range(sh.t_lo, sh.t_hi, CHUNK):
            n = min(CHUNK, sh.t_hi - t0)
            g = _gen(device, seed, copy, ib, t0 // CHUNK)
            k = torch.randn(1, n, w["h_k"], d, generator=g, device=device, dtype=torch.float32)
            v = torch.randn(1, n, w["h_k"], d, generator=g, device=device, dtype=torch.float32)
            if w["outliers"] > 0:
                for ih in range(w["h_k"]):
                    if ih not in outl:
                        outl[ih] = torch.randperm(d, generator=_gen(device, seed, 7777, ih), device=device)[:round(w["outliers"] * d)]
                    k[:, :, ih, outl[ih]] *= 10.0
            k, v = k.to(tdt)[:, :, sh.h_lo:sh.h_hi], v.to(tdt)[:, :, sh.h_lo:sh.h_hi]
            i = ib - sh.b_lo
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            # a read of a buffer larger than the L2 first: the inputs just generated leave the L2 (the pack reads
            # them from HBM, as in a real prefill; a read leaves no dirty lines to write back meanwhile), and the
            # GPU is still busy with it while the host queues the event and the launch, so the interval holds
            # the kernel and not the host's launch latency
            _spacer(device).sum()
            e0.record()
            B.kvcache_pack_int(k, bufs[0][i:i + 1], bufs[1][i:i + 1], v, bufs[2][i:i + 1], bufs[3][i:i + 1],
                               None, None, n, "k-channel", w["group"], w["bits"], dst_token_offset=t0 - sh.t_lo)
            e1.record()
            e1.synchronize()
            if n == CHUNK or n == w["s"]:
                pack_ms.append((e0.elapsed_time(e1), n))
            del k, v
    return bufs, pack_ms


def build_inputs(B, w, sh, device, seed, copies):
    """`copies` packed caches of this shard plus q, tail and lengths (shared by all copies)."""
    import torch
    tdt = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    d = 128
    caches, pack_ms = [], []
    for c in range(copies):
        bufs, ms = build_cache(B, w, sh, device, seed, c)
        caches.append(bufs)
        pack_ms += ms
    gq = _gen(device, seed, 424242)
    q_full = torch.randn(w["b"], 1, w["h"], d, generator=gq, device=device, dtype=torch.float32).to(tdt)
    q = q_full[sh.b_lo:sh.b_hi, :, sh.h_lo * sh.gq:sh.h_hi * sh.gq].contiguous()
    extras, seqlens, res_lens = {}, None, None
    if sh.has_tail:
        kr = torch.randn(w["b"], w["res"], w["h_k"], d, generator=gq, device=device, dtype=torch.float32).to(tdt)
        vr = torch.randn(w["b"], w["res"], w["h_k"], d, generator=gq, device=device, dtype=torch.float32).to(tdt)
        extras["k_res"] = kr[sh.b_lo:sh.b_hi, :, sh.h_lo:sh.h_hi].contiguous()
        extras["v_res"] = vr[sh.b_lo:sh.b_hi, :, sh.h_lo:sh.h_hi].contiguous()
    if w["ragged"]:
        seq, res = _ragged_lengths(w, seed)
        seqlens, res_lens = seq[sh.b_lo:sh.b_hi].tolist(), res[sh.b_lo:sh.b_hi].tolist()
        extras["cache_seqlens"] = seq[sh.b_lo:sh.b_hi].to(torch.int32).to(device)
        extras["res_lens"] = res[sh.b_lo:sh.b_hi].to(torch.int32).to(device)
    pack_gbs = None
    if pack_ms:
        per_tok = 2 * sh.h_k * d * 2 * (1 + w["bits"] / 16.0) + 2 * sh.h_k * d * 4 / w["group"]
        pack_gbs = statistics.median(per_tok * n / (ms * 1e-3) / 1e9 for ms, n in pack_ms)
    return caches, q, extras, seqlens, res_lens, pack_gbs


def decoder_step_extra(B, device, seed):
    """A whole decoder step of the headline shape, captured as one CUDA graph: the decode with the new token
    attended and filed in the tail, rotary embedding of q and the new key at the token's position, and the
    device-side bookkeeping (a tail that fills up is quantize-packed as the sequence's next block, the lengths
    move on).  30 steps per replay from 64-token tails, lengths put back between replays."""
    import torch
    from bitladder_b200.kv_cache import PackedKVCache
    w = WORKLOADS["C2"]
    b, h, h_k, s, d = w["b"], w["h"], w["h_k"], w["s"], 128
    g = _gen(device, seed, 31337)
    caches = []
    for c in range(3):
        cache = PackedKVCache(b, s + 1024, h_k, d, w["bits"], w["group"], dtype=torch.float16, device=device)
        k = torch.randn(1, s + w["res"], h_k, d, generator=g, device=device, dtype=torch.float32).to(torch.float16)
        v = torch.randn(1, s + w["res"], h_k, d, generator=g, device=device, dtype=torch.float32).to(torch.float16)
        cache.prefill(k.expand(b, -1, -1, -1).contiguous(), v.expand(b, -1, -1, -1).contiguous())
        del k, v
        caches.append(cache)
    q = torch.randn(b, 1, h, d, generator=g, device=device, dtype=torch.float32).to(torch.float16)
    kn = torch.randn(b, 1, h_k, d, generator=g, device=device, dtype=torch.float32).to(torch.float16)
    vn = torch.randn(b, 1, h_k, d, generator=g, device=device, dtype=torch.float32).to(torch.float16)
    ang = torch.rand(s + 2048, d // 2, generator=g, device=device) * 6.2831853
    cos, sin = torch.cos(ang).to(torch.float16), torch.sin(ang).to(torch.float16)
    scale = 1.0 / math.sqrt(d)
    out = {}
    for label, kw in (("bookkeeping", {}), ("bookkeeping_and_rotary", dict(rotary_cos=cos, rotary_sin=sin, rotary_interleaved=False))):
        steps = [c.decoder_step(q, kn, vn, scale, **kw) for c in caches]
        saved = [(c.cache_seqlens.clone(), c.res_lens.clone()) for c in caches]
        for st in steps:
            st.step()
        torch.cuda.synchronize()
        per = 30
        gr, side = torch.cuda.CUDAGraph(), torch.cuda.Stream(device)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side), torch.cuda.graph(gr, stream=side):
            for i in range(per):
                steps[i % 3].step()
        torch.cuda.current_stream().wait_stream(side)
        ts = []
        for _ in range(12):
            for c, (a, r) in zip(caches, saved):
                c.cache_seqlens.copy_(a)
                c.res_lens.copy_(r)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gr.replay()
            e1.record()
            e1.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3 / per)
        out[label] = {"us_per_step": statistics.median(ts), "gpu_launches_per_step": steps[0].plan()["launches"]}
        rc = steps[0].status()
        if rc != 0:
            out[label]["device_status"] = rc
        for c, (a, r) in zip(caches, saved):
            c.cache_seqlens.copy_(a)
            c.res_lens.copy_(r)
    out["what"] = ("C2 shape with per-sequence lengths: decode + fused append + device-side roll-over and length update "
                   "(and rotary embedding of q and the new key), one CUDA graph of 30 steps, median of 12 replays")
    del caches
    torch.cuda.empty_cache()
    return out


def copies_for(nbytes, asked):
    """Rotating cache copies: at least three, and enough that the set is several times the L2."""
    if asked > 0:
        return asked
    return int(min(64, max(3, math.ceil(3.2 * L2_BYTES / max(nbytes, 1)))))


# ---------------------------------------------------------------------------
# one measured workload
# ---------------------------------------------------------------------------
def measure(B, name, w, args, device, rank, world, dist, steps, warmup, want_e2e, target_s=0.25):
    import torch
    sh = Shard(w, rank, world)
    seed = 1000 + list(WORKLOADS).index(name)
    scale = 1.0 / math.sqrt(128)
    if sh.b == 0 or sh.h_k == 0 or sh.s == 0:
        raise SystemExit(f"{name} cannot be cut into {world} shards")
    local_bytes = algorithmic_bytes(w, b=sh.b, h=sh.h, h_k=sh.h_k, s=sh.s,
                                    res_lens=None if sh.has_tail else [0] * sh.b)
    copies = copies_for(local_bytes, args.copies)
    caches, q, extras, seqlens, res_lens, pack_gbs = build_inputs(B, w, sh, device, seed, copies)
    if seqlens is not None:
        local_bytes = algorithmic_bytes(w, seqlens, res_lens, b=sh.b, h=sh.h, h_k=sh.h_k)
    total_bytes = local_bytes
    if world > 1:
        t = torch.tensor([float(local_bytes)], device=device, dtype=torch.float64)
        dist.all_reduce(t)
        total_bytes = int(t.item())
    seq_split = sh.mode == "sequence"
    out = torch.empty_like(q)

    if seq_split:
        from bitladder_b200 import sharding as S
        runs = [S.SequenceParallelStep(q, *bufs, scale, w["group"], w["bits"], seqlen_k=sh.s, **extras) for bufs in caches]
        capturable = all(getattr(r, "capturable", False) for r in runs)
        exchange = runs[0].exchange
    else:
        runs = [B.DecodeStep(q, *bufs, None, scale, "k-channel", w["group"], w["bits"], out=out,
                             num_splits=args.num_splits, **extras) for bufs in caches]
        capturable, exchange = True, None
    ncopy = len(runs)

    def step(i):
        runs[i % ncopy].step()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- check: the sharded result against one GPU decoding the whole job (rank 0, copy 0)
    check = None
    if world > 1:
        step(0)
        torch.cuda.synchronize()
        mine = (runs[0].out if seq_split else out).float()
        if seq_split:
            gathered = [mine]
        else:
            shape = [w["b"], 1, w["h"], 128]
            full = torch.zeros(shape, device=device)
            full[sh.b_lo:sh.b_hi, :, sh.h_lo * sh.gq:sh.h_hi * sh.gq] = mine
            dist.all_reduce(full)
            gathered = [full]
        if rank == 0:
            whole = Shard(w, 0, 1)
            bufs0, _ = build_cache(B, w, whole, device, seed, 0)
            _, q0, ex0, _, _, _ = build_inputs(B, w, whole, device, seed, 0)
            ref = B.fwd_kvcache_int(q0, *bufs0, None, scale, "k-channel", w["group"], w["bits"], **ex0).float()
            torch.cuda.synchronize()
            check = {"max_abs_err": float((gathered[0] - ref).abs().max()),
                     "against": "one-GPU decode of the whole job on rank 0 (first cache copy)"}
            del bufs0, q0, ex0, ref
            torch.cuda.empty_cache()
        barrier()

    for i in range(max(warmup, 3)):
        step(i)
    barrier()

    # ---- CUDA graphs: one of `g` steps (whole cache rotations where possible) replayed n times, one for
    # the remainder, so that the timed region is `steps` steps of graph replay whatever `steps` is
    graphs, g, launch = None, 0, "eager"
    if capturable and not args.eager:
        try:
            g = min(steps, max(ncopy, (args.graph_steps // ncopy) * ncopy))
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                main = torch.cuda.CUDAGraph()
                with torch.cuda.graph(main, stream=side):
                    for i in range(g):
                        step(i)
                rest = None
                if steps % g:
                    rest = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(rest, stream=side):
                        for i in range(steps % g):
                            step(g + i)
            torch.cuda.current_stream().wait_stream(side)
            graphs = (main, rest)
            launch = f"cuda graph replay ({steps // g} x {g} steps" + (f" + 1 x {steps % g}" if steps % g else "") + ")"
        except Exception as exc:
            print(f"[bench] graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            graphs = None
    torch.cuda.synchronize()

    def run_region():
        if graphs is None:
            for i in range(steps):
                step(i)
            return
        for _ in range(steps // g):
            graphs[0].replay()
        if graphs[1] is not None:
            graphs[1].replay()

    run_region()
    barrier()
    # how many K-step regions: about `target_s` of device time, the same count on every rank
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_region()
    e1.record()
    torch.cuda.synchronize()
    est = torch.tensor([e0.elapsed_time(e1) * 1e-3], device=device)
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MAX)
    repeats = int(min(400, max(5, math.ceil(target_s / max(float(est.item()), 1e-6)))))

    sampler = ClockSampler(device.index)
    sampler.start()
    if not args.no_preroll:                     # NVML refreshes every few tens of ms: keep the kernels running first
        for _ in range(max(1, repeats // 2)):
            run_region()
    barrier()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(repeats)]
    for a, b_ in evs:
        a.record()
        run_region()
        b_.record()
    barrier()
    clocks = sampler.stop()
    times = torch.tensor([a.elapsed_time(b_) for a, b_ in evs], device=device)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)         # every region: the slowest rank
    per_step = sorted((times / steps).tolist())
    ms_per_step = statistics.median(per_step)
    pct = lambda p: per_step[min(len(per_step) - 1, int(p * len(per_step)))]

    # ---- end to end: the step's inputs come from pinned host memory, the result goes back.  q and, when the
    # workload has a tail, the K/V rows of the token being decoded sit in ONE pinned host buffer and go to the
    # device in one copy; a prepared DecodeStep attends over the new token and files it in the tail itself
    # (fused append); the output comes back to pinned host memory; the stream is synchronised every step.
    e2e = None
    if want_e2e and not seq_split:
        n_q, n_kv = sh.b * sh.h * 128, (sh.b * sh.h_k * 128 if sh.has_tail else 0)
        stage_dev = torch.empty(n_q + 2 * n_kv, dtype=q.dtype, device=device)
        q_dev = stage_dev[:n_q].view(sh.b, 1, sh.h, 128)
        stage_host = torch.empty(n_q + 2 * n_kv, dtype=q.dtype).pin_memory()
        stage_host[:n_q].copy_(q.reshape(-1).cpu())
        kw = dict(extras)
        if sh.has_tail:
            k_new_dev = stage_dev[n_q:n_q + n_kv].view(sh.b, 1, sh.h_k, 128)
            v_new_dev = stage_dev[n_q + n_kv:].view(sh.b, 1, sh.h_k, 128)
            stage_host[n_q:n_q + n_kv].copy_(extras["k_res"][:, -1:].reshape(-1).cpu())
            stage_host[n_q + n_kv:].copy_(extras["v_res"][:, -1:].reshape(-1).cpu())
            base = extras["res_lens"] if "res_lens" in extras else torch.full((sh.b,), w["res"], dtype=torch.int32, device=device)
            kw["res_lens"] = torch.clamp(base - 1, min=0).to(torch.int32)     # the new token takes the last tail slot
            kw.update(k_new=k_new_dev, v_new=v_new_dev)
        out_host = torch.empty(q.shape, dtype=q.dtype).pin_memory()
        e2e_runs = [B.DecodeStep(q_dev, *bufs, None, scale, "k-channel", w["group"], w["bits"],
                                 num_splits=args.num_splits, **kw) for bufs in caches[:8]]
        stream = torch.cuda.current_stream()
        e2e_graphs = []
        if not args.eager:
            try:
                side = torch.cuda.Stream(device)
                side.wait_stream(stream)
                with torch.cuda.stream(side):
                    for run in e2e_runs:
                        stage_dev.copy_(stage_host, non_blocking=True)
                        run.step()
                    side.synchronize()
                    for run in e2e_runs:
                        gr = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(gr, stream=side):
                            stage_dev.copy_(stage_host, non_blocking=True)
                            run.step()
                            out_host.copy_(run.out, non_blocking=True)
                        e2e_graphs.append(gr)
                stream.wait_stream(side)
            except Exception as exc:
                print(f"[bench] e2e graph capture failed ({exc}); three eager operations per step", file=sys.stderr)
                e2e_graphs = []
        torch.cuda.synchronize()

        def e2e_step(i):
            if e2e_graphs:
                e2e_graphs[i % len(e2e_graphs)].replay()
            else:
                stage_dev.copy_(stage_host, non_blocking=True)
                run = e2e_runs[i % len(e2e_runs)]
                run.step()
                out_host.copy_(run.out, non_blocking=True)
            stream.synchronize()                    # the caller needs the result before the next step

        e2e_steps = min(max(steps, 200), 1000)
        for i in range(5):
            e2e_step(i)
        barrier()
        e0.record()
        for i in range(e2e_steps):
            e2e_step(i)
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / e2e_steps
        e2e = {"value": w["b"] / (e2e_ms * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": stage_host.numel() * stage_host.element_size() * world,
               "d2h_bytes_per_step": out_host.numel() * out_host.element_size() * world,
               "us_per_step": e2e_ms * 1e3, "steps": e2e_steps,
               "note": "per rank: q and the new token's K/V rows in one pinned host buffer, one H2D copy, a prepared "
                       "DecodeStep with fused append, out copied back to pinned host memory ("
                       + ("replayed as one CUDA graph" if e2e_graphs else "three eager operations")
                       + "), stream synchronised every step; the packed cache is state resident in HBM; byte counts "
                         "are summed over ranks"}

    sm = torch.cuda.get_device_properties(device).multi_processor_count
    local = runs[0]._local_step if seq_split else runs[0]
    plan = local.plan()                      # what the library does with these arguments on this device
    rows = plan["rows"]
    # the library's own count (prefix table of a ragged batch, decode, parts merge); the exchange of a sequence
    # split merges the parts itself, so its kernel takes the place of the parts merge
    fused_exchange = bool(exchange and exchange.get("merges_local_parts"))
    launches = plan["launches"] - (1 if fused_exchange and rows > 4 * sh.b else 0) + (exchange["launches"] if exchange else 0)
    peak, peak_src = measured_peak_gbs()
    achieved = local_bytes / (ms_per_step * 1e-3) / 1e9        # this rank's bytes over the step time (slowest rank's time)
    ratio = NCU_TRAFFIC_RATIO.get(name if world == 1 else "")
    res = {
        "us_per_step": ms_per_step * 1e3, "ms_per_step": ms_per_step,
        "us_per_step_p20": pct(0.2) * 1e3, "us_per_step_p80": pct(0.8) * 1e3, "regions": repeats,
        "value": w["b"] / (ms_per_step * 1e-3),
        "hbm_tb_s": total_bytes / (ms_per_step * 1e-3) / 1e12,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                     "traffic": (round(local_bytes * ratio) if ratio else None),
                     "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this workload"
                                        if ratio else None),
                     "peak_source": peak_src, "algorithmic_bytes_per_step": local_bytes,
                     "note": "per GPU: this rank's algorithmic bytes per step / CUDA-event time of the whole step"},
        "launch": launch, "rows_per_kv_head": rows, "ctas_per_sm": plan["ctas_per_sm"], "gpu_launches_per_step": launches,
        "l2": f"{copies} rotating packed-cache copies of {local_bytes / 2**20:.1f} MiB each per GPU "
              f"({copies * local_bytes / 2**20:.0f} MiB against {L2_BYTES // 2**20} MiB of L2)",
        "per_gpu": {"batch": sh.b, "kv_heads": sh.h_k, "tokens": sh.s},
        "clocks": clocks, "pack_gb_s": pack_gbs, "e2e": e2e, "check": check, "exchange": exchange,
    }
    del caches, runs
    torch.cuda.empty_cache()
    return res


# ---------------------------------------------------------------------------
# CPU arm
# ---------------------------------------------------------------------------
def cpu_inputs(w, seed, nseq):
    """Seeded inputs of `nseq` sequences of the workload for the CPU port (full length, all KV heads)."""
    import numpy as np
    import torch
    from oracle import c_oracle

    b, h, h_k, s, d = nseq, w["h"], w["h_k"], w["s"], 128
    g = torch.Generator(device="cpu").manual_seed(seed)
    is_bf = w["dtype"] == "bf16"
    tdt = torch.bfloat16 if is_bf else torch.float16
    to_np = (lambda t: t.view(torch.uint16).numpy()) if is_bf else (lambda t: t.numpy())
    q = to_np(torch.randn(b, 1, h, d, generator=g).to(tdt))
    packs = []
    for ib in range(b):       # pack sequence by sequence: bounded staging memory
        k = to_np(torch.randn(1, s, h_k, d, generator=g).to(tdt))
        v = to_np(torch.randn(1, s, h_k, d, generator=g).to(tdt))
        packs.append(c_oracle.quantize_pack(k, v, w["bits"], w["group"], w["dtype"]))
    pk = {key: np.concatenate([p[key] for p in packs], axis=0) for key in ("k_pack", "k_params", "v_pack", "v_params")}
    kr = vr = None
    if w["res"]:
        kr = to_np(torch.randn(b, w["res"], h_k, d, generator=g).to(tdt))
        vr = to_np(torch.randn(b, w["res"], h_k, d, generator=g).to(tdt))
    cs = rl = None
    if w["ragged"]:
        seq, res = _ragged_lengths(w, seed)
        cs, rl = seq[:b].numpy().astype("int32"), res[:b].numpy().astype("int32")
    return q, pk, kr, vr, cs, rl


def cpu_time(w, seed, nseq, steps, warmup):
    """Times the CPU oracle port (dequantize-then-attention in C/OpenMP) on `nseq` sequences of the workload.
    Returns (seconds per step of those nseq sequences, threads)."""
    from oracle import c_oracle
    q, pk, kr, vr, cs, rl = cpu_inputs(w, seed, nseq)
    scale = 1.0 / math.sqrt(128)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        c_oracle.decode(q, pk["k_pack"], pk["k_params"], pk["v_pack"], pk["v_params"], scale, w["bits"], w["group"],
                        w["dtype"], cache_seqlens=cs, k_res=kr, v_res=vr, res_lens=rl)
        if it >= warmup:
            times.append(time.perf_counter() - t0)
    return sum(times) / len(times), c_oracle.num_threads()


def run_reference(args, name, w, rank, world):
    """The reference arm: the CPU port on the WHOLE batch of the job, every step, with all host threads."""
    if rank != 0:
        return
    from oracle import c_oracle
    c_oracle.set_num_threads(len(os.sched_getaffinity(0)))   # a multi-rank launcher exports OMP_NUM_THREADS=1
    steps = args.steps if args.steps is not None else 10
    warmup = args.warmup if args.warmup is not None else 3
    nseq = w["b"]
    sec, cores = cpu_time(w, 1000, nseq, steps, warmup)
    tps = nseq / sec
    sample = (f"all {nseq} sequences, {w['h_k']} KV heads, {w['s']} tokens{' + tail' if w['res'] else ''}: "
              f"dequantize-then-attention in C/OpenMP on {cores} threads, {steps} steps of {sec * 1e3:.0f} ms")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f16 (int4/int2 codes, fp32 accumulate)", "data": "synthetic",
        "config": job_config(name, w, world),
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path; this is the CPU port of its algorithm "
                "(oracle/bd_oracle.c, pinned to the reference kernels' bytes) on the host cores",
    }
    # the reference's OWN implementation is a CUDA kernel: where it was built for sm_100a and a GPU is here,
    # time it too (headline shape without the tail, which it does not have)
    try:
        import torch
        from oracle import build_ref
        if name == "C2" and torch.cuda.is_available() and build_ref.available("fast"):
            us = build_ref.time_decode_c2("fast")
            line["reference_gpu_kernel"] = {
                "us_per_step": us, "value": 8 / (us * 1e-6), "unit": UNIT,
                "what": "the reference's split-KV decode + combine kernels (sm_80-style mma.sync code) recompiled for "
                        "sm_100a, through its own host API with only the architecture check removed, b8 32q/8kv "
                        "s32768 4-bit g128, no tail, eager launches as its API allocates per call"}
    except Exception as exc:                                   # noqa: BLE001
        line["reference_gpu_kernel"] = {"unavailable": str(exc)[:200]}
    print(json.dumps(line))


# ---------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=None, choices=sorted(WORKLOADS))
    ap.add_argument("--copies", type=int, default=0, help="rotating packed-cache copies (0: enough to exceed the L2 several times)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-preroll", action="store_true", help="skip the clock pre-roll (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations (the 'sharded' key)")
    ap.add_argument("--num-splits", type=int, default=0, help="ranges per sequence (0: the library's plan)")
    ap.add_argument("--graph-steps", type=int, default=96, help="most decode steps held by one CUDA graph")
    ap.add_argument("--eager", action="store_true", help="launch every step from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    name = args.workload or "C2"
    w = WORKLOADS[name]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, name, w, rank, world)
        return

    import torch
    import torch.distributed as dist
    import bitladder_b200 as B

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU port")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a short timeout: a rank that falls out of step must end the run, not hold the GPUs for ten minutes
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=120))

    steps = max(args.steps if args.steps is not None else 2000, 1)
    warmup = max(args.warmup if args.warmup is not None else 50, 3)
    main_res = measure(B, name, w, args, device, rank, world, dist, steps, warmup, want_e2e=not args.no_e2e)

    extras = {}
    if args.workload is None and not args.no_extras:
        others = ["C4", "C5a4", "C5a2", "C5b"] + (["C1", "C3"] if world == 1 else [])
        for other in others:
            ow = WORKLOADS[other]
            try:
                r = measure(B, other, ow, args, device, rank, world, dist, steps=min(steps, 48), warmup=5,
                            want_e2e=False, target_s=0.1)
                extras[other] = {"config": job_config(other, ow, world), "us_per_step": r["us_per_step"],
                                 "us_per_step_p20": r["us_per_step_p20"], "us_per_step_p80": r["us_per_step_p80"],
                                 "value": r["value"], "hbm_tb_s": r["hbm_tb_s"], "roofline_frac_per_gpu": r["roofline"]["frac"],
                                 "algorithmic_bytes_per_gpu": r["roofline"]["algorithmic_bytes_per_step"],
                                 "per_gpu": r["per_gpu"], "launch": r["launch"], "gpu_launches_per_step": r["gpu_launches_per_step"],
                                 "rows_per_kv_head": r["rows_per_kv_head"], "ctas_per_sm": r["ctas_per_sm"],
                                 "check": r["check"], "exchange": r["exchange"], "l2": r["l2"]}
            except Exception as exc:                            # noqa: BLE001
                extras[other] = {"error": str(exc)[:300]}
                if world > 1:
                    raise

    decoder_step = None
    if world == 1 and args.workload is None and not args.no_extras:
        try:
            decoder_step = decoder_step_extra(B, device, 1000)
        except Exception as exc:                                # noqa: BLE001
            decoder_step = {"error": str(exc)[:300]}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sec, cores = cpu_time(w, 1000, 1, steps=10, warmup=1)
        cpu = {"value": 1 / sec, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"1 of {w['b']} sequences, {w['h_k']} KV heads, {w['s']} tokens{' + tail' if w['res'] else ''}; "
                         f"dequantize-then-attention in C/OpenMP, 10 steps of {sec * 1e3:.0f} ms"}

    if rank == 0:
        r = main_res
        cfg = job_config(name, w, world)
        cfg.update({"per_gpu": r["per_gpu"], "rows_per_kv_head": r["rows_per_kv_head"], "ctas_per_sm": r["ctas_per_sm"],
                    "launch": r["launch"], "l2": r["l2"],
                    "timed": f"{r['regions']} regions of {steps} steps each, median (p20 {r['us_per_step_p20']:.2f} us, "
                             f"p80 {r['us_per_step_p80']:.2f} us per step)"})
        line = {
            "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": r["ms_per_step"], "us_per_step": r["us_per_step"], "hbm_tb_s": r["hbm_tb_s"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 (int4/int2 codes, fp32 accumulate)", "data": "synthetic",
            "config": cfg, "roofline": r["roofline"], "cpu_baseline": cpu, "e2e": r["e2e"],
            "gpu_launches": r["gpu_launches_per_step"] * steps, "clocks": r["clocks"], "pack_gb_s": r["pack_gb_s"],
            "check": r["check"], "exchange": r["exchange"],
        }
        if extras:
            line["sharded" if world > 1 else "other_configs"] = extras
        if decoder_step is not None:
            line["decoder_step"] = decoder_step
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
