#!/usr/bin/env python
"""Benchmark of the FP8 attention-forward + FP8 GEMM hot path on B200.

One "step" = one FP8 attention forward at B=4, H=32 (BH=128), S=8192, D=128,
non-causal, fp16 output + fp32 LSE (4*BH*S^2*D = 4.398e12 FLOP) followed by one
FP8 GEMM 8192^3 with bf16 output scaled by sa*sb (2*M*N*K = 1.0995e12 FLOP),
both on synthetic seeded N(0,1) data quantised per tensor with scale = amax/448.
`value` is total FLOP / time in TFLOPS, whole job (all GPUs).  At N > 1 every
rank runs the same per-GPU workload on its own shard (attention: its own 128
heads of a 128*N-head batch; GEMM: its own 8192 rows of an (8192*N)-row A with
B replicated), no collective on the data path: weak scaling.

Beside `value` the line carries: `parts` (each kernel alone; `parts.sustained`: each kernel back to back for >= 3 s
with the SM clock sampled; `parts.strong` at N > 1: the SAME global problem — BH = 128 heads, 8192 GEMM rows — divided
over the N GPUs; `parts.allgather` at N > 1: the optional NCCL all-gather of the row-sharded C), `roofline` for the
dominant kernel against the burst peak, `e2e` (host buffers, copies inside the timed region, plus a copy-only leg) and
`cpu_baseline` (the reference's own CPU code on a bounded sample).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload both|attn|gemm] [--bh BH] [--causal 0|1] [--hd 64|128]
                    [--mnk M N K] [--brief]
    python bench.py --impl reference ...     # the reference's own CPU code, bounded sample

--bh/--causal/--hd/--mnk change the timed shapes (profiling a smaller case of the same kernels; the line then names the
shape it ran); --brief skips the sustained, end-to-end and CPU legs.  Prints ONE JSON line (rank 0).
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

METRIC = "FP8 attn-fwd & FP8 GEMM TFLOPS/GPU (hd128 S=8192; 8192^3) at 1/2/4/8 B200"
ATT = dict(bh=128, sl=8192, hd=128, causal=0)
GEMM = dict(M=8192, N=8192, K=8192)
NOMINAL_FP8_TFLOPS = 4500.0
FALLBACK_BF16_TFLOPS = 1590.0  # fallback when the measured-peaks file is absent
# dram__bytes_read.sum + dram__bytes_write.sum per launch at the bench shape, from ncu captures of a quarter of it
# (BH=32, S=8192, D=128), times 4 (traffic grows with the number of heads): the attention kernel itself
# (134.27 MB read + 41.31 MB written per quarter) and the fp16-V pre-pass that every call runs before it
# (33.6 MB of codes read + 67.1 MB of fp16 written per quarter: its algorithmic bytes, which a streaming copy moves once)
ATTN_KERNEL_TRAFFIC_BYTES = 4 * (134.27e6 + 41.31e6)
ATTN_PREPASS_TRAFFIC_BYTES = 4 * (33.55e6 + 67.11e6)


def att_flops(a):
    return 4.0 * a["bh"] * a["sl"] ** 2 * a["hd"] / (2 if a["causal"] else 1)


def gemm_flops(g):
    return 2.0 * g["M"] * g["N"] * g["K"]


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d, "measured"
    return {"bf16_tflops": FALLBACK_BF16_TFLOPS, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}, "fallback"


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons every 50 ms.  The sampler is started ahead of the region of
    interest (nvidia-smi takes a few hundred ms to deliver its first line); mark() opens the region, stop() closes
    it and summarises the samples that arrived inside it.  A region shorter than the sampling period can end up with
    no sample of its own: the summary then uses the samples taken under the same load just before it and says so."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.proc = None
        self.lines = []      # (arrival time, text)
        self.t_mark = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "50", "-i", str(self.idx)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_first_sample(self, timeout=3.0):
        t0 = time.time()
        while self.proc is not None and not self.lines and time.time() - t0 < timeout:
            time.sleep(0.02)

    def mark(self):
        self.t_mark = time.time()

    def stop(self):
        t_end = time.time()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.06)     # one more sampling period, so that a sample taken at the end of the region arrives
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def parse(rows):
            sm, mx, reasons = [], [], set()
            for _, ln in rows:
                f = [x.strip() for x in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            return sm, mx, reasons

        t0 = self.t_mark if self.t_mark is not None else 0.0
        inside = [r for r in self.lines if t0 <= r[0] <= t_end + 0.06]
        sm, mx, reasons = parse(inside)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        busy = [x for x in sm if x > 0.5 * max(sm)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------ the reference arm

def reference_cpu_run(steps: int, warmup: int, cores: int | None = None):
    """Times the reference's own CPU code for the path (oracle/_ref: cpu_attention_fp8 of
    libs/flash_attention_v121r_diet_hd128_fp8_forward.cu and the GEMM loop of libs/fp8_gemm_bench.cu)
    when it was compiled, else the oracle's restatement of the same loops; independent heads / row blocks
    are spread over all host threads.  Each step is a bounded sample with the bench's 4:1 FLOP mix."""
    import numpy as np
    from concurrent.futures import ThreadPoolExecutor
    import oracle as O

    cores = cores or os.cpu_count() or 1
    R = O.ref()
    kind = "reference" if R.available else "port"
    sl, hd = 512, 128
    heads = cores
    rows_per_thread, gn, gk = 8, 1024, 2048
    q, _, _ = O.quantize_f32(O.seeded_normal("Q", (heads, sl, hd), config="bench-cpu"))
    k, _, _ = O.quantize_f32(O.seeded_normal("K", (heads, sl, hd), config="bench-cpu"))
    v, _, _ = O.quantize_f32(O.seeded_normal("V", (heads, sl, hd), config="bench-cpu"))
    a, _, _ = O.quantize_f32(O.seeded_normal("A", (cores * rows_per_thread, gk), config="bench-cpu"))
    b, _, _ = O.quantize_f32(O.seeded_normal("B", (gn, gk), config="bench-cpu"))

    def one_head(h):
        if kind == "reference":
            R.cpu_attention_fp8(q[h:h + 1], k[h:h + 1], v[h:h + 1], 0, 0)
        else:
            O.attention_f32(q[h:h + 1], k[h:h + 1], v[h:h + 1], 0, 0)

    def one_block(t):
        blk = a[t * rows_per_thread:(t + 1) * rows_per_thread]
        if kind == "reference":
            R.gemm_cpu_loop(blk, b)
        else:
            O.gemm_f32(blk, b)

    flops = 4.0 * heads * sl * sl * hd + 2.0 * cores * rows_per_thread * gn * gk
    pool = ThreadPoolExecutor(cores)

    def step():
        list(pool.map(one_head, range(heads)))
        list(pool.map(one_block, range(cores)))

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    tflops = flops * steps / dt / 1e12
    sample = (f"per step: attention BH={heads} (one head per host thread) S={sl} D={hd} non-causal + GEMM "
              f"{cores * rows_per_thread}x{gn}x{gk}, same seeded N(0,1)/amax-448 inputs as the GPU workload "
              f"(bounded sample of BH=128 S=8192 / 8192^3; {flops / 1e9:.2f} GFLOP per step)")
    return {"value": tflops, "unit": "TFLOPS", "cores": cores, "kind": kind, "sample": sample}, dt / steps * 1e3


def run_reference_arm(args, emit=print):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    base, ms = reference_cpu_run(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "fp8-e4m3 codes, fp32 arithmetic (CPU)", "data": "synthetic",
        "config": {"workload": "bounded CPU sample of the GPU arm's workload — " + base["sample"],
                   "gpu_arm_workload": workload_config(args.gpus, args.workload)["workload"],
                   "inputs": "seeded N(0,1), per-tensor e4m3 with scale = amax/448"},
        "cpu_baseline": base,
        "e2e": {"value": base["value"], "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(json.dumps(line))
    return 0


def workload_config(n, workload):
    return {
        "workload": {"both": "FP8 attention fwd (B=4,H=32,S=8192,D=128, non-causal, fp16 O + fp32 LSE) + FP8 GEMM 8192^3 (bf16 out, alpha=sa*sb) per GPU",
                     "attn": "FP8 attention fwd (B=4,H=32,S=8192,D=128, non-causal, fp16 O + fp32 LSE) per GPU",
                     "gemm": "FP8 GEMM 8192^3 (bf16 out, alpha=sa*sb) per GPU"}[workload],
        "attention": dict(ATT), "gemm": dict(GEMM),
        "sharding": f"weak: global BH = 128*{n}, global GEMM M = 8192*{n} split by 128-row tiles, B replicated; no collective",
        "l2": "inputs larger than L2 (attention Q+K+V 403 MB + O 268 MB; GEMM A+B 134 MB + C 134 MB), no explicit flush",
        "inputs": "seeded N(0,1), per-tensor e4m3 with scale = amax/448",
    }


# ----------------------------------------------------------------------------- ours

def numa_bind(dev_index: int) -> dict:
    """Binds this process to the CPUs of the NUMA node its GPU hangs off, so that the pinned host buffers allocated
    afterwards (first touch) and the copy threads live next to the GPU's PCIe root.  Returns what was done."""
    info = {"gpu": dev_index, "node": None, "bound": False}
    try:
        import torch
        pr = torch.cuda.get_device_properties(dev_index)
        bus = f"{pr.pci_domain_id:04x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read().strip())
        info["pci"] = bus
        if node < 0:
            return info
        info["node"] = node
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["bound"] = True
            info["cpus"] = len(allowed)
    except (OSError, ValueError, AttributeError) as e:
        info["error"] = str(e)[:80]
    return info


def _json_only_stdout():
    """Libraries (NCCL's version banner, for one) print to the process's stdout; the contract is ONE JSON line there.
    File descriptor 1 is pointed at stderr for the run and the returned writer emits the line on the real stdout."""
    real = os.dup(1)
    sys.stdout.flush()
    os.dup2(2, 1)

    def emit(text: str) -> None:
        sys.stdout.flush()
        os.write(real, (text + "\n").encode())

    return emit


def main():
    emit = _json_only_stdout()
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="both", choices=["both", "attn", "gemm"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--bh", type=int, default=None, help="attention batch*heads per GPU (default 128)")
    ap.add_argument("--sl", type=int, default=None)
    ap.add_argument("--hd", type=int, default=None, choices=[64, 128])
    ap.add_argument("--causal", type=int, default=None, choices=[0, 1])
    ap.add_argument("--mnk", type=int, nargs=3, default=None)
    ap.add_argument("--brief", action="store_true", help="device-timed steps only: no sustained, end-to-end or CPU leg")
    ap.add_argument("--sustain-s", type=float, default=3.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    if args.impl == "reference":
        return run_reference_arm(args, emit)

    import torch
    import torch.distributed as dist
    from goml_b200 import fa_forward as F, fp8_gemm as G, multi_gpu as MG, quantize as Q

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    numa = numa_bind(local)          # before any pinned allocation
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ctx = F.FACreate()
    stream = torch.cuda.current_stream()
    sh = stream.cuda_stream

    att = dict(ATT)
    gm = dict(GEMM)
    custom = False
    for key, val in (("bh", args.bh), ("sl", args.sl), ("hd", args.hd), ("causal", args.causal)):
        if val is not None:
            att[key] = val
            custom = True
    if args.mnk:
        gm = dict(M=args.mnk[0], N=args.mnk[1], K=args.mnk[2])
        custom = True
    do_attn = args.workload in ("both", "attn")
    do_gemm = args.workload in ("both", "gemm")

    # ---- synthetic inputs: seeded N(0,1) generated on the host side of the ABI would take minutes at this
    # size, so they are drawn on the device (seeded per rank) and quantised by the library's own quantiser
    gen = torch.Generator(device=dev).manual_seed(20260000 + rank)
    scales = torch.zeros(16, dtype=torch.float32, device=dev)

    def quantised(shape, slot):
        x = torch.randn(shape, generator=gen, device=dev, dtype=torch.float32)
        c = torch.empty(shape, dtype=torch.uint8, device=dev)
        Q.QuantizeF32ToF8E4M3(x.data_ptr(), c.data_ptr(), scales.data_ptr() + 8 * slot, scales.data_ptr() + 8 * slot + 4, x.numel(), sh)
        return c

    bh, sl, hd = att["bh"], att["sl"], att["hd"]
    M, N, K = gm["M"], gm["N"], gm["K"]
    if do_attn:
        q, k, v = quantised((bh, sl, hd), 0), quantised((bh, sl, hd), 1), quantised((bh, sl, hd), 2)
        o = torch.empty((bh, sl, hd), dtype=torch.float16, device=dev)
        lse = torch.empty((bh, sl), dtype=torch.float32, device=dev)
    if do_gemm:
        a, b = quantised((M, K), 3), quantised((N, K), 4)
        c = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
    torch.cuda.synchronize()
    sp = scales.data_ptr()
    softmax_scale = 1.0 / math.sqrt(hd)

    def attn(heads=None):
        ctx.ForwardEx(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), heads or bh, sl, hd, att["causal"], 0,
                      softmax_scale, 1.0, sp, sp + 8, sp + 16, sh)

    def gemm(rows=None):
        G.FP8GEMMScaled(rows or M, N, K, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, sp + 24, sp + 32, G.OutBF16, sh)

    def barrier():
        if world > 1:
            dist.barrier()

    def max_over_ranks(vals):
        t = torch.tensor(vals, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def timed(fn, iters):
        """Mean device time of `fn` over `iters` back-to-back launches (events on the launching stream)."""
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    sampler = ClockSampler(local).start()
    sampler.wait_first_sample()
    for _ in range(args.warmup):
        if do_attn: attn()
        if do_gemm: gemm()
    torch.cuda.synchronize()

    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    barrier()
    torch.cuda.synchronize()
    sampler.mark()
    t_start = torch.cuda.Event(enable_timing=True); t_end = torch.cuda.Event(enable_timing=True)
    t_start.record(stream)
    for i in range(args.steps):
        ev[i][0].record(stream)
        if do_attn: attn()
        ev[i][1].record(stream)
        if do_gemm: gemm()
        ev[i][2].record(stream)
    t_end.record(stream)
    torch.cuda.synchronize()
    total_ms = t_start.elapsed_time(t_end)
    clock_window = "timed region"
    if total_ms < 300.0:
        # the region is shorter than a few sampling periods: keep the identical launches going (untimed) for 0.3 s
        # so that the clock record describes this load and not an idle gap
        clock_window = "timed region + 0.3 s of the same launches right after it (region shorter than the sampling period)"
        t_extra = time.time()
        while time.time() - t_extra < 0.3:
            if do_attn: attn()
            if do_gemm: gemm()
            torch.cuda.synchronize()
    barrier()
    clocks = sampler.stop()
    clocks["window"] = clock_window
    attn_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev) if do_attn else 0.0
    gemm_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev) if do_gemm else 0.0
    ctx.DeviceStatus()
    if G.device_status() != 0:
        raise SystemExit("bench.py: the GEMM kernel reported a bounded-wait expiry")

    peaks, peak_src = measured_peaks()
    parts = {}

    # ---- sustained leg: each kernel back to back for >= sustain_s seconds (power-capped steady state), SM clock sampled
    if not args.brief:
        sustained = {}
        for name, fn, ms, fl in (("attention", attn, attn_ms, att_flops(att)), ("gemm", gemm, gemm_ms, gemm_flops(gm))):
            if (name == "attention" and not do_attn) or (name == "gemm" and not do_gemm):
                continue
            iters = max(10, int(args.sustain_s * 1e3 / max(ms, 1e-3)) + 1)
            smp = ClockSampler(local).start()
            smp.wait_first_sample()
            barrier()
            smp.mark()
            t_ms = timed(fn, iters)
            ck = smp.stop()
            (t_ms,) = max_over_ranks([t_ms])
            tf = fl / t_ms / 1e9
            sustained[name] = {"launches": iters, "seconds": t_ms * iters / 1e3, "ms": t_ms, "tflops_per_gpu": tf,
                               "sm_mhz_median": ck.get("sm_mhz"), "reasons": ck.get("reasons"),
                               "ms_x_mhz": (t_ms * ck["sm_mhz"]) if ck.get("sm_mhz") else None,
                               "frac_of_2x_bf16_sustained": tf / (2.0 * peaks.get("bf16_tflops_sustained", peaks["bf16_tflops"]))}
        parts["sustained"] = sustained

    # ---- strong scaling: the SAME global problem divided over the ranks (attention: 128 / N heads each; GEMM:
    # 8192 / N rows of A each, cut on 128-row tiles, B replicated); no collective on the data path
    if world > 1 and not custom:
        strong = {}
        iters = max(5, min(args.steps, 30))
        if do_attn:
            h0, h1 = MG.shard_heads(bh, world, rank)
            for _ in range(3): attn(h1 - h0)
            torch.cuda.synchronize(); barrier()
            (ms,) = max_over_ranks([timed(lambda: attn(h1 - h0), iters)])
            per_gpu = att_flops(att) / world / ms / 1e9
            strong["attention"] = {"heads_per_gpu": bh // world, "ms": ms, "tflops_per_gpu": per_gpu, "tflops_whole_job": per_gpu * world,
                                   "efficiency_vs_full_problem_per_gpu": per_gpu / (att_flops(att) / attn_ms / 1e9)}
        if do_gemm:
            r0, r1 = MG.shard_rows(M, world, rank)
            for _ in range(3): gemm(r1 - r0)
            torch.cuda.synchronize(); barrier()
            (ms,) = max_over_ranks([timed(lambda: gemm(r1 - r0), iters)])
            per_gpu = gemm_flops(gm) / world / ms / 1e9
            strong["gemm"] = {"rows_per_gpu": M // world, "ms": ms, "tflops_per_gpu": per_gpu, "tflops_whole_job": per_gpu * world,
                              "efficiency_vs_full_problem_per_gpu": per_gpu / (gemm_flops(gm) / gemm_ms / 1e9)}
            # the optional all-gather of the row-sharded C (bf16): every rank ends with the full [8192, 8192] matrix
            full = torch.empty((M, N), dtype=torch.bfloat16, device=dev)
            mine = c[: r1 - r0]
            for _ in range(3): MG.allgather_rows_into(full, mine, M, world, rank)
            torch.cuda.synchronize(); barrier()
            (ms,) = max_over_ranks([timed(lambda: MG.allgather_rows_into(full, mine, M, world, rank), iters)])
            total_bytes = M * N * 2
            parts["allgather"] = {"what": "NCCL all-gather of C row blocks (bf16) after the row-sharded GEMM, its own call",
                                  "bytes_total": total_bytes, "ms": ms, "algbw_gbs": total_bytes / ms / 1e6,
                                  "busbw_gbs_per_gpu": total_bytes * (world - 1) / world / ms / 1e6,
                                  "nvlink_peer_copy_gbs_measured_on_this_pool": 770.0}
        parts["strong"] = strong

    # ---- end to end through the public API with HOST buffers (pinned): every step copies its inputs host->device
    # and its results device->host inside the timed region.  The caller-side pattern is the usual one for a
    # pointer-based ABI: three streams (copy-in, compute, copy-out) over double-buffered device tensors, so the
    # copies of neighbouring steps overlap the kernels; each step still moves all of its own bytes.
    e2e = None
    if not args.brief:
        e2e_steps = max(4, min(args.steps, 40))   # enough steps that filling and draining the three-stage pipeline is amortised
        h2d = d2h = 0
        host, devbuf = {}, [{}, {}]
        if do_attn:
            for name, t in (("q", q), ("k", k), ("v", v)):
                host[name] = torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t)
                h2d += t.numel()
            host["o"] = torch.empty(o.shape, dtype=o.dtype, pin_memory=True)
            host["lse"] = torch.empty(lse.shape, dtype=lse.dtype, pin_memory=True)
            d2h += o.numel() * 2 + lse.numel() * 4
            devbuf[0].update(q=q, k=k, v=v, o=o, lse=lse)
            devbuf[1].update({n: torch.empty_like(t) for n, t in devbuf[0].items() if n in ("q", "k", "v", "o", "lse")})
        if do_gemm:
            host["a"] = torch.empty(a.shape, dtype=a.dtype, pin_memory=True).copy_(a)   # activations travel; the weight B stays resident
            host["c"] = torch.empty(c.shape, dtype=c.dtype, pin_memory=True)
            h2d += a.numel()
            d2h += c.numel() * 2
            devbuf[0].update(a=a, c=c)
            devbuf[1].update(a=torch.empty_like(a), c=torch.empty_like(c))
        s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        ev_in = [torch.cuda.Event() for _ in range(2)]     # inputs of buffer b are on the device
        ev_comp = [torch.cuda.Event() for _ in range(2)]   # kernels of buffer b have finished
        ev_out = [torch.cuda.Event() for _ in range(2)]    # results of buffer b are on the host
        b_ptr = b.data_ptr() if do_gemm else 0

        def e2e_step(i, kernels=True):
            bi = i & 1
            d = devbuf[bi]
            with torch.cuda.stream(s_in):
                if i >= 2: s_in.wait_event(ev_comp[bi])       # the kernels that read this input buffer two steps ago are done
                if do_attn:
                    d["q"].copy_(host["q"], non_blocking=True); d["k"].copy_(host["k"], non_blocking=True); d["v"].copy_(host["v"], non_blocking=True)
                if do_gemm:
                    d["a"].copy_(host["a"], non_blocking=True)
                ev_in[bi].record(s_in)
            stream.wait_event(ev_in[bi])
            if i >= 2: stream.wait_event(ev_out[bi])          # the results written two steps ago have been read out
            if kernels and do_attn:
                ctx.ForwardEx(d["q"].data_ptr(), d["k"].data_ptr(), d["v"].data_ptr(), d["o"].data_ptr(), d["lse"].data_ptr(), bh, sl, hd,
                              att["causal"], 0, softmax_scale, 1.0, sp, sp + 8, sp + 16, sh)
            if kernels and do_gemm:
                G.FP8GEMMScaled(M, N, K, d["a"].data_ptr(), b_ptr, d["c"].data_ptr(), 1.0, sp + 24, sp + 32, G.OutBF16, sh)
            ev_comp[bi].record(stream)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[bi])
                if do_attn:
                    host["o"].copy_(d["o"], non_blocking=True); host["lse"].copy_(d["lse"], non_blocking=True)
                if do_gemm:
                    host["c"].copy_(d["c"], non_blocking=True)
                ev_out[bi].record(s_out)

        def e2e_run(kernels):
            for i in range(2):
                e2e_step(i, kernels)
            torch.cuda.synchronize()
            barrier(); torch.cuda.synchronize()
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(s_in)
            stream.wait_event(e0); s_out.wait_event(e0)
            for i in range(e2e_steps):
                e2e_step(i, kernels)
            s_out.wait_stream(stream); s_out.wait_stream(s_in)
            e1.record(s_out)
            torch.cuda.synchronize()
            return e0.elapsed_time(e1) / e2e_steps

        e2e_ms = e2e_run(True)
        copy_ms = e2e_run(False)     # the same copies with no kernel in between: what the host side alone allows
        e2e_ms, copy_ms = max_over_ranks([e2e_ms, copy_ms])
        e2e = (e2e_ms, copy_ms, h2d, d2h)

    total_ms, attn_ms, gemm_ms = max_over_ranks([total_ms, attn_ms, gemm_ms])

    flops_step = (att_flops(att) if do_attn else 0.0) + (gemm_flops(gm) if do_gemm else 0.0)
    ms_per_step = total_ms / args.steps
    value = flops_step * world / ms_per_step / 1e9
    # The timed steps last a fraction of a second and run at boost clocks: their denominator is the BURST figure.
    # (MEASURED_PEAKS.json has no FP8 entry; dense FP8 is twice the dense bf16 rate on this part.)
    fp8_burst = 2.0 * peaks["bf16_tflops"]
    dom_ms, dom_flops, dom_name = (attn_ms, att_flops(att), f"fa_fwd_kernel<{hd}>") if do_attn else (gemm_ms, gemm_flops(gm), "fp8_gemm_tcgen05_kernel")
    achieved = dom_flops / dom_ms / 1e9
    # the attention's P.V product runs at the fp16 tensor rate (fp16 P keeps the 1e-2 mean-relative bar): per 128 x 128
    # score tile 256 clk of FP8 Q.K^T + 512 clk of fp16 P.V = 768 clk where an all-FP8 kernel needs 512
    mixed_peak = fp8_burst * 512.0 / 768.0
    cfg = workload_config(world, args.workload)
    if custom:
        cfg["workload"] = (f"custom shape for profiling: attention BH={bh} S={sl} D={hd} causal={att['causal']}; "
                           f"GEMM {M}x{N}x{K} (same kernels as the headline workload)")
        cfg["attention"], cfg["gemm"] = att, gm
    cfg["numa"] = numa
    parts.update({"attention_ms": attn_ms, "attention_tflops_per_gpu": (att_flops(att) / attn_ms / 1e9) if do_attn else None,
                  "gemm_ms": gemm_ms, "gemm_tflops_per_gpu": (gemm_flops(gm) / gemm_ms / 1e9) if do_gemm else None,
                  "gemm_frac_of_2x_bf16_burst": (gemm_flops(gm) / gemm_ms / 1e9 / fp8_burst) if do_gemm else None})
    scale_heads = bh / 32.0 * (sl / 8192.0) * (hd / 128.0)
    traffic = (ATTN_KERNEL_TRAFFIC_BYTES + ATTN_PREPASS_TRAFFIC_BYTES) / 4 * scale_heads if do_attn else None
    line = {
        "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8-e4m3 (fp32 accumulate)", "data": "synthetic",
        "config": cfg,
        "parts": parts,
        "roofline": {"bound": "tensor", "kernel": dom_name, "achieved": achieved, "peak": fp8_burst, "unit": "TFLOP/s",
                     "frac": achieved / fp8_burst, "traffic": traffic,
                     "traffic_parts": ({"attention_kernel": ATTN_KERNEL_TRAFFIC_BYTES / 4 * scale_heads,
                                        "fp16_v_prepass": ATTN_PREPASS_TRAFFIC_BYTES / 4 * scale_heads} if do_attn else None),
                     "peak_source": f"2 x {peak_src} bf16 BURST cuBLAS TFLOP/s (MEASURED_PEAKS.json has no FP8 entry); "
                                    "the timed steps are a sub-second burst, the >= 3 s leg is under parts.sustained",
                     "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                     "frac_of_mixed_fp8_qk_fp16_pv_peak": (achieved / mixed_peak) if do_attn else None},
        # kernels launched inside the timed region: the attention entry launches two (fp16-V pre-pass + forward), the GEMM one
        "gpu_launches": args.steps * (2 * int(do_attn) + int(do_gemm)),
        "clocks": clocks,
    }
    if e2e is not None:
        e2e_ms, copy_ms, h2d, d2h = e2e
        line["e2e"] = {"value": flops_step * world / e2e_ms / 1e9, "unit": "TFLOPS", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                       "ms_per_step": e2e_ms, "copy_only_ms_per_step": copy_ms,
                       "copy_only_gbs_per_gpu": {"h2d": h2d / copy_ms / 1e6, "d2h": d2h / copy_ms / 1e6},
                       "note": "copy_only = the same pinned-host copies with no kernel between them: when it equals ms_per_step the "
                               "step is bound by the host side (PCIe / host memory), not by the kernels"}
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.brief:
        base, _ = reference_cpu_run(steps=4, warmup=1)
        line["cpu_baseline"] = base
    if rank == 0:
        emit(json.dumps(line))
    ctx.Destroy()
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
