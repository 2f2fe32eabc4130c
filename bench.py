#!/usr/bin/env python
"""Benchmark of the low-bit KV-cache decode-attention step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload C2]

A *step* is one decode-attention call (split-KV decode kernel + split combine)
over one batch of synthetic, seeded inputs.  The default workload is the
Llama-3-8B decode shape the headline metric is quoted on: batch 8, 32 query / 8
KV heads, head_dim 128, 32768 tokens of 4-bit cache (group 128) plus a 64-token
fp16 tail.  With N > 1 (launched by torch.distributed.run, one rank per GPU) the
batch is sharded: every rank holds and decodes its own batch of 8 sequences, no
data-path collective, weak scaling.

Prints ONE JSON line (rank 0):
  value     whole-job decode throughput in tokens/s (sequences advanced per second),
            cache resident in HBM, device-timed with CUDA events, max over ranks
  e2e       the same step through the public Python API with the step's inputs
            (q and the new token's K/V rows) copied from pinned host memory and
            the output copied back inside the timed region
  roofline  algorithmic HBM bytes per step / measured step time, against the
            measured copy bandwidth of this pool's B200s
  cpu_baseline  the CPU oracle (a port of the reference algorithm; the reference
            has no CPU path) timed on a bounded sample on this host's cores

`--impl reference` times that CPU port alone with all host threads, same metric.
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

WORKLOADS = {
    # name: batch, q heads, kv heads, seqlen, bits, group, tail, dtype, ragged, outlier fraction
    "C1": dict(b=1, h=32, h_k=8, s=4096, bits=4, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
               desc="b1 32q/8kv d128 s4096 4-bit g128"),
    "C2": dict(b=8, h=32, h_k=8, s=32768, bits=4, group=128, res=64, dtype="fp16", ragged=False, outliers=0.0,
               desc="Llama-3-8B decode: b8 32q/8kv d128 s32768 4-bit g128 + 64-token fp16 tail"),
    "C3": dict(b=1, h=32, h_k=8, s=131072, bits=2, group=64, res=0, dtype="fp16", ragged=False, outliers=0.05,
               desc="b1 32q/8kv d128 s131072 2-bit g64, 5% K outlier channels x10"),
    "C4": dict(b=32, h=32, h_k=32, s=16384, bits=4, group=128, res=128, dtype="bf16", ragged=True, outliers=0.0,
               desc="Llama-2-7B MHA: b32 32/32 d128 ragged s in [1024,16384] 4-bit g128 bf16"),
    "C5a4": dict(b=16, h=8, h_k=1, s=131072, bits=4, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
                 desc="Llama-3-70B, one KV head of 8 per GPU: b16 8q/1kv d128 s131072 4-bit g128"),
    "C5a2": dict(b=16, h=8, h_k=1, s=131072, bits=2, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
                 desc="Llama-3-70B, one KV head of 8 per GPU: b16 8q/1kv d128 s131072 2-bit g128"),
    # one sequence of 1 Mi tokens split along the sequence over 8 GPUs: every rank streams 131072 tokens and
    # the ranks exchange their (out, lse) partials (all-gather over NCCL + bd_combine) inside the timed step;
    # on fewer ranks each still holds a 131072-token shard (weak scaling of the same per-rank work)
    "C5b": dict(b=1, h=64, h_k=8, s=131072, bits=4, group=128, res=0, dtype="fp16", ragged=False, outliers=0.0,
                seq_split=True,
                desc="Llama-3-70B, 1 Mi-token sequence, 131072-token shard per GPU: b1 64q/8kv d128 4-bit g128"),
}


def algorithmic_bytes(w, seqlens=None, res_lens=None) -> int:
    """HBM bytes one decode step has to move: codes, scales/zeros, tail, q and out."""
    b, h, h_k, d, bits, group = w["b"], w["h"], w["h_k"], 128, w["bits"], w["group"]
    tok = sum(seqlens) if seqlens is not None else b * w["s"]
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


# ---------------------------------------------------------------------------
# clocks sampler (read-only NVML queries in a thread)
# ---------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
               0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}

    def __init__(self, index: int, period_s: float = 0.01):
        self.samples, self.reasons = [], set()
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
                util = nv.nvmlDeviceGetUtilizationRates(self.handle).gpu
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, util, mask))
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
        for _, _, m in self.samples:
            mask_all |= m
        reasons = sorted(name for bit, name in self.REASONS.items() if mask_all & bit and name != "gpu_idle")
        return {"sm_mhz": int(statistics.median(s[0] for s in self.samples)), "sm_max_mhz": self.sm_max,
                "reasons": reasons, "samples": len(self.samples)}


NCU_TRAFFIC_C2 = 291_537_920     # bytes per launch: 287.490 MB read + 4.048 MB written
NCU_ALGO_C2 = 287_440_896        # algorithmic bytes of the same launch

# ---------------------------------------------------------------------------
# workload construction
# ---------------------------------------------------------------------------
def make_inputs(w, device, seed, copies):
    """Seeded N(0,1) K/V generated on the device chunk by chunk, packed with the
    library's own quantize-pack kernel into `copies` independent packed caches."""
    import torch
    import bitladder_b200 as B

    tdt = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    b, h, h_k, s, d = w["b"], w["h"], w["h_k"], w["s"], 128
    gen = torch.Generator(device=device).manual_seed(seed)
    caches = []
    pack_ms = []
    for _ in range(copies):
        bufs = B.alloc_packed_cache(b, s, h_k, d, w["bits"], w["group"], device=device)
        for ib in range(b):   # one sequence at a time keeps the fp16 staging small
            k = torch.randn(1, s, h_k, d, generator=gen, device=device, dtype=torch.float32)
            if w["outliers"] > 0:
                n_out = round(w["outliers"] * d)
                for ih in range(h_k):
                    idx = torch.randperm(d, generator=gen, device=device)[:n_out]
                    k[:, :, ih, idx] *= 10.0
            k = k.to(tdt)
            v = torch.randn(1, s, h_k, d, generator=gen, device=device, dtype=torch.float32).to(tdt)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            B.kvcache_pack_int(k, bufs[0][ib:ib + 1], bufs[1][ib:ib + 1], v, bufs[2][ib:ib + 1], bufs[3][ib:ib + 1],
                               None, None, s, "k-channel", w["group"], w["bits"])
            e1.record()
            e1.synchronize()
            pack_ms.append(e0.elapsed_time(e1))
            del k, v
        caches.append(bufs)
    q = torch.randn(b, 1, h, d, generator=gen, device=device, dtype=torch.float32).to(tdt)
    extras = {}
    if w["res"]:
        extras["k_res"] = torch.randn(b, w["res"], h_k, d, generator=gen, device=device, dtype=torch.float32).to(tdt)
        extras["v_res"] = torch.randn(b, w["res"], h_k, d, generator=gen, device=device, dtype=torch.float32).to(tdt)
    seqlens = res_lens = None
    if w["ragged"]:
        cg = torch.Generator(device="cpu").manual_seed(seed)
        total = torch.randint(1024, s + 1, (b,), generator=cg)
        seq = (total // 128) * 128
        res = total - seq
        seqlens, res_lens = seq.tolist(), res.tolist()
        extras["cache_seqlens"] = seq.to(torch.int32).to(device)
        extras["res_lens"] = res.to(torch.int32).to(device)
    pack_bytes = 2 * s * h_k * d * 2 * (1 + w["bits"] / 16.0) + 2 * s * h_k * d * 4 / w["group"]
    pack_gbs = pack_bytes / (statistics.median(pack_ms) * 1e-3) / 1e9
    return caches, q, extras, seqlens, res_lens, pack_gbs


def cpu_sample(w, seed, steps, warmup):
    """Times the CPU oracle port on a bounded sample: one sequence of the workload
    (all KV heads, full length, tail included).  Returns (tokens/s, cores, sample text)."""
    import numpy as np
    import torch
    from oracle import c_oracle

    b, h, h_k, s, d = 1, w["h"], w["h_k"], min(w["s"], 32768), 128
    g = torch.Generator(device="cpu").manual_seed(seed)
    is_bf = w["dtype"] == "bf16"
    tdt = torch.bfloat16 if is_bf else torch.float16

    def to_np(t):
        return t.view(torch.uint16).numpy() if is_bf else t.numpy()

    q = to_np(torch.randn(b, 1, h, d, generator=g).to(tdt))
    k = to_np(torch.randn(b, s, h_k, d, generator=g).to(tdt))
    v = to_np(torch.randn(b, s, h_k, d, generator=g).to(tdt))
    kr = vr = None
    if w["res"]:
        kr = to_np(torch.randn(b, w["res"], h_k, d, generator=g).to(tdt))
        vr = to_np(torch.randn(b, w["res"], h_k, d, generator=g).to(tdt))
    pk = c_oracle.quantize_pack(k, v, w["bits"], w["group"], w["dtype"])
    scale = 1.0 / math.sqrt(d)
    times = []
    for it in range(warmup + steps):
        t0 = time.perf_counter()
        c_oracle.decode(q, pk["k_pack"], pk["k_params"], pk["v_pack"], pk["v_params"], scale, w["bits"],
                        w["group"], w["dtype"], k_res=kr, v_res=vr)
        t1 = time.perf_counter()
        if it >= warmup:
            times.append(t1 - t0)
    sec = sum(times) / len(times)
    # a sample of `b` sequences of length s stands for s/w["s"] of the same number of full sequences
    frac = s / w["s"]
    tokens_per_s = b * frac / sec
    sample = (f"{b} of {w['b']} sequences, {h_k} KV heads, {s} of {w['s']} tokens"
              f"{' + tail' if w['res'] else ''}; dequantize-then-attention in C/OpenMP, {steps} steps of {sec * 1e3:.0f} ms")
    return tokens_per_s, sec, c_oracle.num_threads(), sample


def run_reference(args, w, rank):
    if rank != 0:
        return
    steps = max(1, min(args.steps, 20))
    warmup = max(1, min(args.warmup, 3))
    if args.gpus > 1:
        # torchrun exports OMP_NUM_THREADS=1 to its ranks; the one rank that runs this arm takes the host's cores
        from oracle import c_oracle
        c_oracle.set_num_threads(len(os.sched_getaffinity(0)))
    tps, sec, cores, sample = cpu_sample(w, 1000, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": UNIT, "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": sec * 1e3 * w["b"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f16 (int4/int2 codes)", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {w['desc']}", "timed": sample},
        "cpu_baseline": {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference has no CPU implementation of this path; this is the CPU port of its algorithm "
                "(oracle/bd_oracle.c) on the host cores; ms_per_step is the sample time scaled to the full batch",
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="C2", choices=sorted(WORKLOADS))
    ap.add_argument("--copies", type=int, default=3, help="rotating packed-cache copies (defeats L2 reuse)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-preroll", action="store_true", help="skip the half-second clock pre-roll (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg (profiling runs)")
    ap.add_argument("--num-splits", type=int, default=0, help="ranges per sequence (0: the library's plan)")
    ap.add_argument("--graph-steps", type=int, default=48, help="decode steps held by one CUDA graph")
    ap.add_argument("--eager", action="store_true", help="launch every step from Python instead of replaying a CUDA graph")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference(args, w, rank)
        return

    import torch
    import torch.distributed as dist
    import bitladder_b200 as B

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU port")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    distributed = world > 1
    if distributed:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # a short timeout: a rank that falls out of step must end the run, not hold the GPUs for ten minutes
        dist.init_process_group("nccl", device_id=device, timeout=datetime.timedelta(seconds=90))

    warmup = max(args.warmup, 3)
    steps = max(args.steps, 1)
    caches, q, extras, seqlens, res_lens, pack_gbs = make_inputs(w, device, 1000 + rank, args.copies)
    scale = 1.0 / math.sqrt(128)
    nbytes = algorithmic_bytes(w, seqlens, res_lens)
    out = torch.empty_like(q)

    ws_bytes = B.decode_workspace_bytes(q, *caches[0], group_size=w["group"], num_bits=w["bits"],
                                        num_splits=args.num_splits, **extras)
    workspace = torch.zeros(max(ws_bytes, 16), dtype=torch.uint8, device=device)

    seq_split = bool(w.get("seq_split")) and distributed
    if seq_split:
        from bitladder_b200 import sharding as S
        args.eager = True                      # the step holds NCCL collectives: launched eagerly
        sp_steps = [S.SequenceParallelStep(q, bufs[0], bufs[1], bufs[2], bufs[3], scale, w["group"], w["bits"])
                    for bufs in caches]

    def step(i):
        bufs = caches[i % len(caches)]
        if seq_split:      # partial (out, lse) of this rank's shard, all-gather, merge: every rank gets the result
            sp_steps[i % len(sp_steps)].step()
            return
        B.fwd_kvcache_int(q, bufs[0], bufs[1], bufs[2], bufs[3], None, scale, "k-channel", w["group"], w["bits"],
                          out=out, workspace=workspace, num_splits=args.num_splits, **extras)

    def barrier():
        if distributed:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(warmup):
        step(i)
    barrier()

    # The timed loop replays a CUDA graph of `copies` consecutive steps (one per
    # rotating cache copy), so the device is never waiting for the Python caller;
    # steps that do not fill a whole graph are launched eagerly.
    ncopy = len(caches)
    per_graph = ncopy * max(1, args.graph_steps // ncopy)     # steps held by one graph (whole rotations)
    graph = None
    if not args.eager:
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for i in range(per_graph):
                        step(i)
            torch.cuda.current_stream().wait_stream(side)
        except Exception as exc:   # capture unsupported: fall back to eager launches
            print(f"[bench] graph capture failed ({exc}); timing eager launches", file=sys.stderr)
            graph = None
    torch.cuda.synchronize()

    def run_steps(n):
        if graph is None:
            for i in range(n):
                step(i)
            return
        for _ in range(n // per_graph):
            graph.replay()
        for i in range(n % per_graph):
            step(i)

    run_steps(max(per_graph, 3))
    barrier()

    sampler = ClockSampler(local_rank)
    sampler.start()
    # Clock pre-roll: NVML refreshes its readings every few tens of ms, so keep the
    # same kernels running for about half a second before the timed region starts.
    t_pre = time.perf_counter()
    if seq_split and not args.no_preroll:
        # the step holds collectives: every rank must run the SAME number of steps, so the pre-roll
        # is a fixed count here, never a wall-clock loop
        run_steps(3000)
        torch.cuda.synchronize()
    while not seq_split and not args.no_preroll and time.perf_counter() - t_pre < 0.5:
        run_steps(60)
        torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_steps(steps)
    e1.record()
    barrier()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1)
    if distributed:
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / steps
    seqs = w["b"] * (1 if seq_split else world)          # sequences advanced per step, whole job
    value = seqs / (ms_per_step * 1e-3)

    # ---- end to end: the step's inputs come from pinned host memory, the result goes back
    e2e_steps = min(steps, 500)
    # End to end through the public API with HOST buffers: the step's inputs (q and, when the
    # workload has a tail, the K/V rows of the token being decoded) sit in ONE pinned host buffer
    # and go to the device in one copy; the decode step (a prepared B.DecodeStep, the call a
    # decoder loop makes) attends over the new token and files it in the tail itself (fused append);
    # the output comes back to pinned host memory and the stream is synchronised every step.
    b_, h_, hk_, d_ = w["b"], w["h"], w["h_k"], 128
    n_q, n_kv = b_ * h_ * d_, (b_ * hk_ * d_ if w["res"] else 0)
    stage_dev = torch.empty(n_q + 2 * n_kv, dtype=q.dtype, device=device)
    q_dev = stage_dev[:n_q].view(b_, 1, h_, d_)
    stage_host = torch.empty(n_q + 2 * n_kv, dtype=q.dtype).pin_memory()
    stage_host[:n_q].copy_(q.reshape(-1).cpu())
    e2e_kw = dict(extras)
    if w["res"]:
        k_new_dev = stage_dev[n_q:n_q + n_kv].view(b_, 1, hk_, d_)
        v_new_dev = stage_dev[n_q + n_kv:].view(b_, 1, hk_, d_)
        stage_host[n_q:n_q + n_kv].copy_(extras["k_res"][:, -1:].reshape(-1).cpu())
        stage_host[n_q + n_kv:].copy_(extras["v_res"][:, -1:].reshape(-1).cpu())
        # the new token takes the last tail slot: the tail holds one token less before the step
        base = extras["res_lens"] if "res_lens" in extras else torch.full((b_,), w["res"], dtype=torch.int32, device=device)
        e2e_kw["res_lens"] = torch.clamp(base - 1, min=0).to(torch.int32)
        e2e_kw.update(k_new=k_new_dev, v_new=v_new_dev)
    out_host = torch.empty(q.shape, dtype=q.dtype).pin_memory()
    h2d = stage_host.numel() * stage_host.element_size()
    d2h = out_host.numel() * out_host.element_size()
    e2e_runs = [] if (args.no_e2e or seq_split) else [
        B.DecodeStep(q_dev, bufs[0], bufs[1], bufs[2], bufs[3], None, scale, "k-channel", w["group"], w["bits"],
                     num_splits=args.num_splits, **e2e_kw) for bufs in caches]
    e2e_stream = torch.cuda.current_stream()

    # One CUDA graph per cache copy holds the whole step (copy in, decode, copy out): the caller pays
    # one graph launch and one synchronisation per step.  DecodeStep allocates nothing in step(), so it
    # can be captured as it is.
    e2e_graphs = []
    if e2e_runs and not args.eager:
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for run in e2e_runs:
                    stage_dev.copy_(stage_host, non_blocking=True)      # warm-up outside capture
                    run.step()
                side.synchronize()
                for run in e2e_runs:
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr, stream=side):
                        stage_dev.copy_(stage_host, non_blocking=True)
                        run.step()
                        out_host.copy_(run.out, non_blocking=True)
                    e2e_graphs.append(gr)
            torch.cuda.current_stream().wait_stream(side)
        except Exception as exc:
            print(f"[bench] e2e graph capture failed ({exc}); launching the step's three operations one by one",
                  file=sys.stderr)
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
        e2e_stream.synchronize()                    # the caller needs the result before the next step

    e2e = None
    if not args.no_e2e and not seq_split:
        for i in range(3):
            e2e_step(i)
        barrier()
        e0.record()
        for i in range(e2e_steps):
            e2e_step(i)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1)
        if distributed:
            t = torch.tensor([e2e_ms], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e2e_ms = float(t.item())
        e2e = {"value": w["b"] * world / (e2e_ms / e2e_steps * 1e-3), "unit": UNIT,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "us_per_step": e2e_ms / e2e_steps * 1e3, "steps": e2e_steps,
               "note": "q and the new token's K/V rows in one pinned host buffer, one H2D copy, a prepared "
                       "DecodeStep with fused append, out copied back to pinned host memory ("
                       + ("the three operations replayed as one CUDA graph" if e2e_graphs else "three eager launches")
                       + "), stream synchronised every step; the packed cache is state resident in HBM"}

    peak, peak_src = measured_peak_gbs()
    achieved = nbytes / (ms_per_step * 1e-3) / 1e9
    # DRAM bytes (read + write) of one decode launch from the ncu capture summarised in
    # profiles/decode_kernel_c2_4bit.md; for the other workloads the same ratio to the
    # algorithmic bytes (every byte is read once, partials add about 1.4 %).
    traffic = NCU_TRAFFIC_C2 if args.workload == "C2" else round(nbytes * NCU_TRAFFIC_C2 / NCU_ALGO_C2)
    traffic_src = ("ncu dram__bytes_read.sum + dram__bytes_write.sum, one launch of this workload"
                   if args.workload == "C2" else "scaled from the C2 capture by algorithmic bytes")
    splits = B.plan_splits(w["b"], w["h_k"], w["s"], w["bits"], torch.cuda.get_device_properties(device).multi_processor_count)
    rows_used = args.num_splits * w["b"] if args.num_splits > 0 else splits

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        tps, sec, cores, sample = cpu_sample(w, 1000, steps=12, warmup=1)
        cpu = {"value": tps, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "us_per_step": ms_per_step * 1e3, "hbm_tb_s": achieved / 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 (int4/int2 codes, fp32 accumulate)", "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['desc']}", "per_gpu_batch": w["b"],
                       "global_batch": w["b"] * (1 if w.get("seq_split") else world),
                       "sharding": ("sequence split: all-gather of (out, lse) partials + merge inside the step"
                                    if seq_split else "batch, no data-path collective"),
                       "rows_per_kv_head": splits, "launch": "cuda graph replay" if graph is not None else "eager",
                       "l2": f"{args.copies} rotating packed-cache copies of {nbytes / 2**20:.0f} MiB each (> 126 MB L2)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_source": traffic_src, "peak_source": peak_src,
                         "note": "achieved = algorithmic bytes per step / CUDA-event time of the whole step "
                                 "(one split-KV decode kernel launch; the range that finishes last merges the partials)",
                         "algorithmic_bytes_per_step": nbytes},
            "cpu_baseline": cpu,
            "e2e": e2e,
            # decode kernel, + the 256-thread prefix kernel for ragged batches, + the parallel merge
            # kernel when a sequence is cut into more than four parts on average
            "gpu_launches": (1 + (1 if w["ragged"] else 0) + (1 if rows_used > 4 * w["b"] else 0)) * steps,
            "clocks": clocks,
            "pack_gb_s": pack_gbs,
        }
        print(json.dumps(line))
    if distributed:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
