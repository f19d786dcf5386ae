#!/usr/bin/env python3
"""Benchmark of the trunk projection GEMMs on B200, one JSON line on stdout.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Workloads (BASELINE.json `configs`, zero-based):
    w8g_down_m900   configs[1]: int8-group down projection, M = 900, K = 9728, N = 2560, fp16 activations, fp16 result   (default)
    f16_up_m900     configs[0]: fp16 up projection, M = 900, K = 2560, N = 9728
    f16_up_m4096 / w8g_down_m4096: the same products at the long-log call size
    f16_dn_out_m900 / f16_o_m900: the DeltaNet out-projection and the attention o-projection with the residual add, 900 rows (lone-CTA kernel)
    attention       the full-attention core over the 15,900-token log in four chained calls
    deltanet        the Gated DeltaNet core over one 4096-token call (--tokens), 16 key / 32 value heads of 128 (--heads128: 16 value heads)
    serve           configs[4]: 64 requests of 600-1200 tokens and 4 of 15,900 through the 36-layer GEMM-chain trunk (configs[3]'s
                    stack), whole requests dealt longest-first to the GPUs; reports prefill tokens/s and p50 / p95 request latency

A step is one batch of `calls_per_step` independent products of that shape (as many requests of M tokens), each on the next of a
ring of operand sets whose total size exceeds the 126 MB L2, so no timed launch finds its operands in cache. `value` is the
whole-job TFLOP/s with operands resident in HBM; `e2e` is the same metric through the host-pointer provider (pinned host X in,
float32 Y out, copies inside the timed region). With N > 1 (torchrun, one rank per GPU) every GPU holds its own replica and runs the
same steps (requests shard whole, no collective on the data path); time is the max over ranks. The default 512 calls a step make
the timed region of the driver's 20 steps longer than half a second: the GPU then runs under its power cap, so `roofline.frac` is
taken against the SUSTAINED measured peak (`roofline.peak_source` says which; `frac_of_burst` is the same time against the burst
peak). Further keys of the default line: `gpu_baseline` (the reference's own GPU kernels and its cuBLAS call, compiled for sm_100
into oracle/_ref, timed on the same box by the reference probe's method; outside the timed region), `shapes` (every named trunk GEMM
with operands from HBM and hot in the L2), `trunk` (whole passes) and `serve` (the request-sharded sweep of configs[4] on the N GPUs
of this run, with each rank's clock so that runs at different N can be compared at equal clock).

`--impl reference` times the reference's own CPU implementation of the same product (its cpu-bf16 packed GEMM compiled from its
sources into oracle/_ref, on all host cores it takes) on the same metric.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, M, N, K, config index in BASELINE.json or None, epilogue)
    "w8g_down_m900": ("w8g", 900, 2560, 9728, 1, "store"),
    "f16_up_m900": ("f16", 900, 9728, 2560, 0, "store"),
    "w8g_down_m4096": ("w8g", 4096, 2560, 9728, 1, "store"),
    "f16_up_m4096": ("f16", 4096, 9728, 2560, 0, "store"),
    # the short, narrow projections that run on lone CTAs at 900 rows (profiling targets): the DeltaNet out-projection and the attention
    # o-projection with the residual add fused (float32 stream updated in place)
    "f16_dn_out_m900": ("f16", 900, 2560, 2048, None, "add"),
    "f16_o_m900": ("f16", 900, 2560, 4096, None, "add"),
    # the down projection as the trunk runs it, the residual add fused: fewer tiles than CTA pairs, so the pairs share the tiles
    "w8g_down_add_m900": ("w8g", 900, 2560, 9728, None, "add"),
    "f16_down_add_m900": ("f16", 900, 2560, 9728, None, "add"),
    # the attention layers' fused q, k, v projection: 72 swapped tiles of 320 tokens, one wave of the 74 CTA pairs
    "f16_qkv_m900": ("f16", 900, 6144, 2560, None, "store"),
}
# Every named trunk GEMM (N x K) for the per-shape table: the projections of a layer at hidden 2560, MLP 9728.
TRUNK_SHAPES = [("gate_up+swiglu", 19456, 2560, "swiglu"), ("up (config 0)", 9728, 2560, "store"), ("down+residual", 2560, 9728, "add"),
                ("q", 4096, 2560, "store"), ("k or v", 1024, 2560, "store"), ("qkv fused", 6144, 2560, "store"), ("o+residual", 2560, 4096, "add"),
                ("dn_in", 8192, 2560, "store"), ("dn_out+residual", 2560, 2048, "add")]
# DRAM bytes of one launch (dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of the workload's kernel; the summaries under
# profiles/ give the command). None: not captured.
NCU_TRAFFIC = {"w8g_down_m900": 43.0e6, "f16_up_m4096": None}
L2_BYTES = 126 * 1024 * 1024
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def bind_near_gpu(local: int):
    """Run this process on the host cores of the GPU's NUMA node, so that the pinned buffers it allocates next (first touch) and the
    threads that fill them sit on the socket whose PCIe root the GPU hangs from. Returns what was done, for the record; does nothing
    where the system does not say (no sysfs entry, a single node)."""
    import torch

    try:
        props = torch.cuda.get_device_properties(local)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        node = int(open(f"/sys/bus/pci/devices/{bus}/numa_node").read())
        if node < 0:
            return {"numa_node": None}
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if not cpus:
            return {"numa_node": node, "bound": False}
        os.sched_setaffinity(0, cpus)
        return {"numa_node": node, "bound": True, "cores": len(cpus)}
    except (OSError, ValueError, AttributeError, RuntimeError):
        return {"numa_node": None}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs (read-only)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown"}

    def __init__(self, index: int) -> None:
        super().__init__(daemon=True)
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self) -> None:
        if not self.ok:
            return
        while not self.stop_flag.is_set():
            try:
                mhz = int(self.nv.nvmlDeviceGetClockInfo(self.handle, self.nv.NVML_CLOCK_SM))
                mask = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)) if hasattr(self.nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else int(self.nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append(mhz)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.02)

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": int(statistics.median(self.samples)), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def make_operand_sets(ctx, kind, m, n, k, device, epilogue="store"):
    """A ring of independent operand sets (seeded synthetic data with BASELINE's distributions) larger than the L2 in total."""
    import torch

    y_bytes = 4 if epilogue == "add" else 2
    per_set = m * k * 2 + (n * k if kind == "w8g" else n * k * 2) + m * n * y_bytes
    sets = max(2, -(-int(1.5 * L2_BYTES) // per_set))
    gen = torch.Generator(device=device).manual_seed(1001)
    out = []
    for _ in range(sets):
        x = torch.randn((m, k), generator=gen, device=device).bfloat16().half()  # N(0, 1), exact in bf16 and fp16
        y = torch.zeros((m, n), dtype=torch.float32, device=device) if epilogue == "add" else torch.empty((m, n), dtype=torch.float16, device=device)
        if kind == "w8g":
            q = torch.randint(-127, 128, (n, k), generator=gen, device=device, dtype=torch.int32).to(torch.int8)
            s = (torch.randn((n, k // 128), generator=gen, device=device) * 0.02).abs() / 127.0
            w = ctx.prepare_w8g(q, s.float().contiguous())
        else:
            w = (torch.randn((n, k), generator=gen, device=device) * 0.02).bfloat16().half()
        out.append((x, w, y))
    return out, sets * per_set


def algorithmic_bytes(kind, m, n, k, epilogue="store"):
    """Bytes one product must move: X once, W once (int8 + scales for w8g), Y once (fp16), or read and written (float32) for the residual add."""
    w = n * k + n * (k // 128) * 2 if kind == "w8g" else n * k * 2
    return m * k * 2 + w + (m * n * 8 if epilogue == "add" else m * n * 2)


def run_ours(args):
    import torch

    import sepal_runner_b200 as sb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    placement = bind_near_gpu(local)
    kind, m, n, k, cfg_index, epilogue = WORKLOADS[args.workload]
    epi = sb.ADD if epilogue == "add" else sb.STORE
    ctx = sb.Context(local)
    ctx.set_static_weights(True)  # the weight matrices are written once, before the first launch, as an engine's are
    sets, ring_bytes = make_operand_sets(ctx, kind, m, n, k, device, epilogue)
    calls = args.calls_per_step
    flops_call = 2.0 * m * n * k

    def call(i):
        x, w, y = sets[i % len(sets)]
        if kind == "w8g":
            ctx.gemm_w8g(x, w, y, epilogue=epi)
        else:
            ctx.gemm_f16(x, w, y, epilogue=epi)

    def step(s):
        for c in range(calls):
            call(s * calls + c)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for s in range(args.warmup):
        step(s)
    ctx.check_status()
    ctx.take_launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(args.steps):
        step(args.warmup + s)
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    launches = ctx.take_launch_count()
    ctx.check_status()

    # ---- end to end through the host-pointer provider: pinned X in, float32 Y out, copies inside the timed region
    import numpy as np

    prov = sb.Provider(local, 1 << 30)
    x0, w0, _ = sets[0]
    if kind == "w8g":
        wd = (w0.q.float() * w0.scales.repeat_interleave(128, dim=1)).cpu().numpy()
        wid = prov.upload_weights_w8g(wd)
    else:
        wid = prov.upload_weights(w0.cpu().numpy())
    hx = torch.empty((m, k), dtype=torch.float16).pin_memory()
    hx.copy_(x0.cpu())
    hy = torch.empty((m, n), dtype=torch.float32).pin_memory()
    e2e_steps = max(1, min(args.steps, 20))
    e2e_calls = min(calls, 8)
    for _ in range(2):
        prov.gemm_f_raw(hx.data_ptr(), 1, m, wid, hy.data_ptr(), 0.0)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps * e2e_calls):
        prov.gemm_f_raw(hx.data_ptr(), 1, m, wid, hy.data_ptr(), 0.0)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    # What the host bus alone allows: the call's X up and Y down as plain pinned copies, each direction timed by itself (they overlap
    # inside a call, so the slower one bounds it).
    dx, dy = torch.empty_like(hx, device=device), torch.empty_like(hy, device=device)
    bus_ms = []
    barrier()  # every rank copies at the same time, as in the timed calls: the bus is shared
    for dst, src in ((dx, hx), (hy, dy)):
        dst.copy_(src, non_blocking=True)
        torch.cuda.synchronize()
        b0, b1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        b0.record()
        for _ in range(10):
            dst.copy_(src, non_blocking=True)
        b1.record()
        torch.cuda.synchronize()
        bus_ms.append(b0.elapsed_time(b1) / 10)
    host_bus = {"h2d_gb_per_s": round(m * k * 2 / bus_ms[0] / 1e6, 1), "d2h_gb_per_s": round(m * n * 4 / bus_ms[1] / 1e6, 1),
                "copies_only_tflops_per_gpu": round(flops_call / (max(bus_ms) * 1e-3) / 1e12, 1),
                "host_placement": placement,
                "note": "pinned copies of one call's X and Y with no multiply, all ranks copying at once: the bound of e2e per GPU when everything else is hidden behind the longer copy"}
    del dx, dy

    times = torch.tensor([elapsed_ms, e2e_s * 1e3], dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(times[0]), float(times[1])

    peaks, peak_kind = measured_peaks()
    burst_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    sustained_tf = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    long_region = elapsed_ms >= 250.0  # a quarter of a second of back-to-back GEMMs runs under the power cap, like the sustained peak's loop
    peak_tf = sustained_tf if long_region else burst_tf
    total_calls = args.steps * calls
    per_call_ms = elapsed_ms / total_calls
    tflops_gpu = flops_call / (per_call_ms * 1e-3) / 1e12
    value = tflops_gpu * world
    e2e_value = flops_call * e2e_steps * e2e_calls / (e2e_ms * 1e-3) / 1e12 * world

    line = {
        "metric": "GEMM TFLOP/s (f16 tensor cores; w8 group) at M=900",
        "value": round(value, 2),
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": round(elapsed_ms / args.steps, 5),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "f16 x int8-group -> f32 accumulate" if kind == "w8g" else "f16 x f16 -> f32 accumulate",
        "data": "synthetic",
        "config": {
            "workload": f"{args.workload}" + (f" (BASELINE configs[{cfg_index}])" if cfg_index is not None else " (a named trunk GEMM, residual add fused)") + f": M={m} K={k} N={n}",
            "calls_per_step": calls,
            "l2": f"ring of {len(sets)} operand sets, {ring_bytes >> 20} MiB > 126 MiB L2: every launch reads its operands from HBM",
            "static_weights": "sepal_b200_set_static_weights(1): no launch writes the weights, so a launch may request its first weight tiles before the one before it has finished",
            "gemm_rows_per_s": round(m * total_calls / (elapsed_ms * 1e-3) * world, 1),
            "timed_region_ms": round(elapsed_ms, 1),
            "parallelism": f"request-sharded x{world}, full replica per GPU, no collective",
        },
        "roofline": {
            "bound": "tensor",
            "achieved": round(tflops_gpu, 2),
            "peak": peak_tf,
            "unit": "TFLOP/s",
            "frac": round(tflops_gpu / peak_tf, 4),
            "frac_of_burst": round(tflops_gpu / burst_tf, 4),
            "peak_source": (f"bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_kind}; the timed region is {elapsed_ms:.0f} ms of back-to-back launches: under the power cap)"
                            if long_region else f"bf16_tflops of MEASURED_PEAKS.json ({peak_kind}; burst: a timed region of {elapsed_ms:.0f} ms)"),
            "traffic": args.traffic if args.traffic is not None else NCU_TRAFFIC.get(args.workload),
            "traffic_source": "--traffic" if args.traffic is not None else ("profiles/gemm_w8t_pair_kernel_w8g_down_m900.md" if NCU_TRAFFIC.get(args.workload) else None),
            "algorithmic_bytes": algorithmic_bytes(kind, m, n, k, epilogue),
            "hbm_gbs_achieved": round(algorithmic_bytes(kind, m, n, k, epilogue) / (per_call_ms * 1e-3) / 1e9, 1),
            "us_per_launch": round(per_call_ms * 1e3, 2),
        },
        "e2e": {
            "value": round(e2e_value, 3),
            "unit": "TFLOP/s",
            "h2d_bytes_per_step": m * k * 2 * e2e_calls,
            "d2h_bytes_per_step": m * n * 4 * e2e_calls,
            "calls_per_step": e2e_calls,
            "steps": e2e_steps,
            "note": f"sepal_b200_provider_gemm_f, pinned host buffers, {e2e_steps} steps of {e2e_calls} calls timed by wall clock around a device sync; "
                    "a call's rows go in up to four pieces whose upload, multiply and download overlap",
            "host_bus": host_bus,
        },
        "gpu_launches": int(launches),
        "clocks": sampler.summary(),
    }
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(kind, m, n, k)
    if rank == 0 and world == 1 and args.gpu_baseline:
        line["gpu_baseline"] = gpu_baseline(ctx, device)
    if rank == 0 and world == 1 and args.shapes:
        line["shapes"] = shape_table(ctx, device, burst_tf)
    prov.close()
    ctx.close()
    del sets
    torch.cuda.empty_cache()
    if rank == 0 and world == 1 and args.trunk:
        line["trunk"] = trunk_numbers(local, sustained_tf)
        line["config"]["prefill_tokens_per_s_per_gpu"] = line["trunk"]["f16"]["log_15900"]["tokens_per_s"]
    if args.serve:
        serve = serve_sweep(local, rank, world, int8=False, passes=3)  # every rank takes part; rank 0 gets the summary
        if rank == 0:
            line["serve"] = serve
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def probe_time_ms(fn, reps: int = 10, batches: int = 3) -> float:
    """Minimum over `batches` of the mean time of `reps` back-to-back calls (the reference probe's method, gemm_probe.cpp:69-89)."""
    import torch

    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    best = None
    for _ in range(batches):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        best = ms if best is None else min(best, ms)
    return best


def shape_table(ctx, device, peak_tf):
    """TFLOP/s of every named trunk GEMM at M = 900 and M = 4096, fp16 and int8-group weights, with the fused epilogues. `us` /
    `tflops` / `frac_of_peak`: consecutive launches rotate over copies of the operands that together exceed the L2 (every launch reads
    from HBM, as in the trunk, where 7 GB of weights pass between two uses of a matrix); `us_hot_l2`: one operand set, relaunched."""
    import torch

    import sepal_runner_b200 as sb

    rows = []
    gen = torch.Generator(device=device).manual_seed(7)
    for m in (900, 4096):
        for name, n, k, ep in TRUNK_SHAPES:
            epi = {"store": sb.STORE, "add": sb.ADD, "swiglu": sb.SWIGLU}[ep]
            n_out = n // 2 if ep == "swiglu" else n
            per_set = m * k * 2 + n * k * 2 + m * n_out * (4 if ep == "add" else 2)
            copies = max(2, -(-int(1.25 * L2_BYTES) // per_set))
            xs = [torch.randn((m, k), generator=gen, device=device).half() for _ in range(copies)]
            ws = [(torch.randn((n, k), generator=gen, device=device) * 0.02).half() for _ in range(copies)]
            ys = [torch.zeros((m, n_out), dtype=torch.float32 if ep == "add" else torch.float16, device=device) for _ in range(copies)]
            variants = [("f16", lambda i: ctx.gemm_f16(xs[i], ws[i], ys[i], epilogue=epi))]
            if k % 128 == 0:
                wqs = []
                for w in ws:
                    q, s = ctx.quantize_group_s8(w.float())
                    wqs.append(ctx.prepare_w8g(q, s))
                variants.append(("w8g", lambda i: ctx.gemm_w8g(xs[i], wqs[i], ys[i], epilogue=epi)))
            for vname, fn in variants:
                turn = [0]

                def rotating():
                    fn(turn[0] % copies)
                    turn[0] += 1

                cold = probe_time_ms(rotating)
                hot = probe_time_ms(lambda: fn(0))
                tf = 2.0 * m * n * k / (cold * 1e-3) / 1e12
                rows.append({"gemm": name, "weights": vname, "m": m, "n": n, "k": k, "us": round(cold * 1e3, 1), "tflops": round(tf, 1),
                             "frac_of_peak": round(tf / peak_tf, 3), "us_hot_l2": round(hot * 1e3, 1), "operand_copies": copies})
            del xs, ws, ys
    # the entry point that allocates nothing, on one shape (the o projection at M = 900: 80 tiles of 128 x 256 ... split evenly over the SMs)
    m, n, k = 900, 2560, 4096
    x = torch.randn((m, k), generator=gen, device=device).half()
    w = (torch.randn((n, k), generator=gen, device=device) * 0.02).half()
    y = torch.zeros((m, n), dtype=torch.float16, device=device)
    ms = probe_time_ms(lambda: sb.gemm_f16_noalloc(x, w, y, wait=False))
    tf = 2.0 * m * n * k / (ms * 1e-3) / 1e12
    rows.append({"gemm": "o (sepal_b200_gemm_f16_noalloc)", "weights": "f16", "m": m, "n": n, "k": k, "us_hot_l2": round(ms * 1e3, 1),
                 "tflops": round(tf, 1), "frac_of_peak": round(tf / peak_tf, 3)})
    ctx.check_status()
    return rows


def gpu_baseline(ctx, device):
    """The reference's own GPU code on this box, on identical buffers: its kernels launch_gemm_nt (float32 accumulation),
    launch_gemm_w8a16 and launch_gemm_simt (Int8Group), compiled unmodified for sm_100, and cublasGemmEx as its engine calls it
    (COMPUTE_32F and COMPUTE_16F), next to this repository's kernels. Timed by the reference probe's method (minimum over three
    batches of back-to-back launches, runner/cuda/tools/gemm_probe.cpp:69-89), operands hot in the L2 for every row alike."""
    import torch

    from oracle.oracle import RefGpu

    if not RefGpu.available():
        return {"unavailable": "oracle/_ref/libsepal_ref_gpu.so was not built (the reference tree was absent at build time)"}
    r = RefGpu()
    out = []
    gen = torch.Generator(device=device).manual_seed(1001)
    for label, m, n, k in (("w8g_down_m900", 900, 2560, 9728), ("f16_up_m900", 900, 9728, 2560), ("f16_up_m4096", 4096, 9728, 2560)):
        flops = 2.0 * m * n * k
        reps = 8 if flops > 2e10 else 20  # the probe's reps_for
        x = torch.randn((m, k), generator=gen, device=device).bfloat16().half()
        w = (torch.randn((n, k), generator=gen, device=device) * 0.02).bfloat16().half()
        y32 = torch.empty((m, n), dtype=torch.float32, device=device)
        y16 = torch.empty((m, n), dtype=torch.float16, device=device)
        q, s = ctx.quantize_group_s8(w.float())
        wq = ctx.prepare_w8g(q, s)
        q_pairs, sw = r.quantize_weights_s8(w, pairs=True)
        x32 = x.float()
        row = {"shape": label, "m": m, "n": n, "k": k, "tflops": {}}

        def tf(fn, reps=reps):
            return round(flops / (probe_time_ms(fn, reps=reps) * 1e-3) / 1e12, 1)

        row["tflops"]["sepal_b200_gemm_f16"] = tf(lambda: ctx.gemm_f16(x, w, y16))
        row["tflops"]["sepal_b200_gemm_w8g"] = tf(lambda: ctx.gemm_w8g(x, wq, y16))
        row["tflops"]["reference cublasGemmEx COMPUTE_32F"] = tf(lambda: r.cublas(x, w, y=y16))
        row["tflops"]["reference cublasGemmEx COMPUTE_16F"] = tf(lambda: r.cublas(x, w, compute16=True, y=y16))
        row["tflops"]["reference launch_gemm_nt Float32"] = tf(lambda: r.gemm_nt(x, w, y=y16, y_half=True))
        row["tflops"]["reference launch_gemm_w8a16"] = tf(lambda: r.gemm_w8a16(x, q_pairs, sw, y_half=True))
        row["tflops"]["reference launch_gemm_simt Int8Group"] = tf(lambda: r.gemm_simt(x32, q, s, y=y32), reps=3)
        out.append(row)
    return {"method": "min over 3 batches of back-to-back launches (CUDA events), operands hot in the L2", "rows": out}


def trunk_numbers(local, peak_tf):
    """Whole passes through the 36-layer GEMM-chain trunk (BASELINE configs[2] and [3]): a 900-token alert and the 15,900-token log in
    calls of 4096, fp16 weights and int8-group MLP weights. Host token ids in, last hidden state out (copies inside the timed region)."""
    import numpy as np

    import sepal_runner_b200 as sb

    out = {}
    rng = np.random.default_rng(4004)
    # "attention": the nine attention layers run the real core (16 query / 4 key-value heads of 256, q_proj carrying the output gate:
    # 8192 rows instead of 4096) instead of the fixed wiring; the DeltaNet layers stay wired.
    real = dict(attn_q=8192, attn_kv=1024, attn_o=4096, attn_heads=16, attn_kv_heads=4, attn_head_dim=256, attn_rotary_dims=64)
    # "cores": as "attention", and the 27 DeltaNet layers run theirs too (16 key / 32 value heads of 128, convolution of 4 taps: an
    # in-projection of 12,352 rows, an out-projection over 4096), the geometry of the 4b model's mixers.
    cores = dict(real, dn_key_heads=16, dn_value_heads=32, dn_in=12352, dn_v=4096, dn_v_offset=0)
    for name, int8, extra in (("f16", 0, {}), ("mlp_int8", 1, {}), ("f16_attention", 0, real), ("f16_cores", 0, cores)):
        trunk = sb.Trunk(local, sb.TrunkConfig(mlp_int8=int8, **extra))
        flops_tok = trunk.gemm_flops_per_token
        row = {"weight_gb": round(trunk.weight_bytes / 1e9, 2), "gemm_gflop_per_token": round(flops_tok / 1e9, 3)}
        for label, n in (("alert_900", 900), ("log_15900", 15900)):
            tokens = rng.integers(0, 151936, n).astype(np.uint32)
            trunk.run(tokens)
            best = None
            for _ in range(3):
                t0 = time.perf_counter()
                _, _, dev_ms = trunk.run(tokens)
                wall = time.perf_counter() - t0
                best = (wall, dev_ms) if best is None or wall < best[0] else best
            row[label] = {"tokens_per_s": round(n / best[0], 1), "ms": round(best[0] * 1e3, 3), "device_ms": round(best[1], 3),
                          "gemm_tflops": round(flops_tok * n / (best[1] * 1e-3) / 1e12, 1),
                          "frac_of_peak": round(flops_tok * n / (best[1] * 1e-3) / 1e12 / peak_tf, 3)}
        out[name] = row
        trunk.close()
    return out


def serve_sweep(local, rank, world, int8: bool, passes: int):
    """BASELINE configs[4] on the GPUs of this run: 64 requests of 600-1200 tokens and 4 of 15,900 through the 36-layer trunk, every rank
    holding a full replica, requests dealt whole, longest first, each to the GPU with the least work so far; all requests arrive at
    time zero, so a request's latency is its completion time (queue + compute, as runner/cuda/tools/gpu_bench.cpp:54-58 defines it).
    Every rank calls this; rank 0 gets the summary, the others None. Needs the process group when world > 1."""
    import numpy as np
    import torch

    import sepal_runner_b200 as sb
    from sepal_runner_b200.sharding import deal_requests, ideal_speedup

    rng = np.random.default_rng(5005)
    lengths = [int(v) for v in rng.integers(600, 1201, 64)] + [15900] * 4
    mine = deal_requests(lengths, world)[rank]
    trunk = sb.Trunk(local, sb.TrunkConfig(mlp_int8=1 if int8 else 0))
    tok_rng = np.random.default_rng(4004 + rank)
    requests = {i: tok_rng.integers(0, 151936, lengths[i]).astype(np.uint32) for i in mine}
    for i in mine[:1]:
        trunk.run(requests[i][:900])  # warm up: first launches, kernel attributes

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    # Short requests first: they share calls of up to 4096 rows (sepal_b200_trunk_score packs them as the reference's engine does), and
    # the long logs, four calls each, follow. A request's latency is the time until its call has finished on the device.
    mine = sorted(mine, key=lambda i: lengths[i])
    sb.Context.take_launch_count()
    results = []
    for _ in range(max(1, passes)):
        sampler = ClockSampler(local)
        sampler.start()
        barrier()
        t0 = time.perf_counter()
        _, done = trunk.score([requests[i] for i in mine])
        span = time.perf_counter() - t0
        sampler.stop_flag.set()
        sampler.join(timeout=2)
        lat = {i: float(done[j]) for j, i in enumerate(mine)}
        dev_ms = float(done.max()) * 1e3 if len(mine) else 0.0
        barrier()
        results.append((span, lat, dev_ms, sampler.summary()))
    launches = int(sb.Context.take_launch_count())
    flops_tok = trunk.gemm_flops_per_token
    trunk.close()
    span, lat, dev_ms, clocks = min(results, key=lambda p: p[0])
    mine_summary = (span, lat, dev_ms, len(mine), sum(lengths[i] for i in mine), clocks)
    if world > 1:
        import torch.distributed as dist

        gathered = [None] * world
        dist.all_gather_object(gathered, mine_summary)
    else:
        gathered = [mine_summary]
    if rank != 0:
        return None
    makespan = max(g[0] for g in gathered)
    all_lat = sorted(v for g in gathered for v in g[1].values())
    total = sum(lengths)
    # The same work at every rank's maximum clock: a rank that sat at a lower clock under the power cap would have finished sooner.
    at_max = [g[0] * (g[5]["sm_mhz"] / g[5]["sm_max_mhz"]) if g[5].get("sm_mhz") and g[5].get("sm_max_mhz") else g[0] for g in gathered]
    return {
        "workload": "serve (BASELINE configs[4]): 64 requests of 600-1200 tokens + 4 of 15900, whole requests per GPU (dealt longest first), packed into calls of up to 4096 rows",
        "weights": "int8-group MLP" if int8 else "fp16",
        "n_gpus": world,
        "tokens_per_s": round(total / makespan, 1),
        "tokens_per_s_at_max_clock": round(total / max(at_max), 1),
        "makespan_s": round(makespan, 4),
        "total_tokens": total,
        "ideal_speedup_over_1_gpu": round(ideal_speedup(lengths, world), 3),
        "p50_latency_s": round(all_lat[len(all_lat) // 2], 4),
        "p95_latency_s": round(all_lat[min(len(all_lat) - 1, int(0.95 * len(all_lat)))], 4),
        "per_gpu": [{"requests": g[3], "tokens": g[4], "span_s": round(g[0], 4), "device_s": round(g[2] / 1e3, 4), "sm_mhz": g[5].get("sm_mhz"),
                     "sm_max_mhz": g[5].get("sm_max_mhz"), "reasons": g[5].get("reasons")} for g in gathered],
        "passes": len(results),
        "gemm_flops_per_token": flops_tok,
        "gpu_launches": launches,
        "note": "speed-up between runs at different N: divide their tokens_per_s_at_max_clock (span x median SM clock / maximum clock per rank, "
                "slowest rank), so that a run that sat lower under the power cap is not flattered or punished",
    }


def run_serve(args):
    """`--workload serve`: the request-sharded sweep of BASELINE configs[4] as the line's own metric."""
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    sampler = ClockSampler(local)
    sampler.start()
    serve = serve_sweep(local, rank, world, args.int8, max(1, args.steps if args.steps <= 5 else 3))
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    if rank == 0:
        total, makespan = serve["total_tokens"], serve["makespan_s"]
        peaks, peak_kind = measured_peaks()
        peak_tf = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
        flops = serve["gemm_flops_per_token"] * total
        line = {
            "metric": "prefill tokens/s (request-sharded, 36-layer GEMM-chain trunk)",
            "value": serve["tokens_per_s"],
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": serve["passes"],
            "warmup": 1,
            "ms_per_step": round(makespan * 1e3, 3),
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "f16 x int8-group MLP" if args.int8 else "f16 x f16 -> f32 accumulate",
            "data": "synthetic",
            "config": {"workload": serve["workload"], "total_tokens": total, "ideal_speedup_over_1_gpu": serve["ideal_speedup_over_1_gpu"],
                       "p50_latency_s": serve["p50_latency_s"], "p95_latency_s": serve["p95_latency_s"], "per_gpu": serve["per_gpu"],
                       "tokens_per_s_at_max_clock": serve["tokens_per_s_at_max_clock"],
                       "l2": "weights 7.3 GB per replica: far larger than the L2", "parallelism": f"request-sharded x{world}, full replica per GPU, no collective"},
            "roofline": {"bound": "tensor", "achieved": round(flops / makespan / 1e12 / world, 1), "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": round(flops / makespan / 1e12 / world / peak_tf, 4),
                         "peak_source": f"bf16_tflops_sustained of MEASURED_PEAKS.json ({peak_kind}; the GEMMs run inside a long step)", "traffic": None},
            "e2e": {"value": serve["tokens_per_s"], "unit": "tokens/s", "h2d_bytes_per_step": total * 4, "d2h_bytes_per_step": 68 * 2560 * 4,
                    "note": "the same number: sepal_b200_trunk_score takes host token ids and returns the last hidden states to the host"},
            "gpu_launches": serve["gpu_launches"],
            "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def run_attention(args):
    """The full-attention core of one layer over the 15,900-token log (BASELINE configs[3]'s request) as four chained calls of 4096 / 4096 /
    4096 / 3612 tokens: norm + RoPE + cache append, then causal grouped-query flash attention times the output gate. A step is the four
    calls. Heads: 16 query / 4 key-value heads of 256 (the served models' attention geometry); --heads128 runs 32 / 8 heads of 128."""
    import torch

    import sepal_runner_b200 as sb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    heads, kvh, hd, rot = (32, 8, 128, 32) if args.heads128 else (16, 4, 256, 64)
    shape = sb.AttentionShape(heads=heads, kv_heads=kvh, head_dim=hd, rotary_dims=rot, rope_theta=1.0e7, eps=1e-6)
    ctx = sb.Context(local)
    total, chunk = 15900, 4096
    gen = torch.Generator(device=device).manual_seed(4004 + rank)
    qg = (torch.randn((total, 2 * heads * hd), generator=gen, device=device) * 1.0).half()
    k = torch.randn((total, kvh * hd), generator=gen, device=device).half()
    v = torch.randn((total, kvh * hd), generator=gen, device=device).half()
    w = (torch.randn(hd, generator=gen, device=device) * 0.1).float()
    k_arena = torch.zeros((total, kvh * hd), dtype=torch.float16, device=device)
    v_arena = torch.zeros_like(k_arena)
    q_out = torch.empty((chunk, heads * hd), dtype=torch.float16, device=device)
    out = torch.empty((total, heads * hd), dtype=torch.float16, device=device)
    calls = [(at, min(chunk, total - at)) for at in range(0, total, chunk)]
    pairs = sum(n * at + n * (n + 1) // 2 for at, n in calls)
    flops = 4.0 * hd * pairs * heads  # Q K^T and P V over the visible (query, key) pairs

    def step():
        for at, n in calls:
            rows = [(0, n, 0, at)]
            sb.attention_prepare(ctx, shape, rows, qg[at:at + n], k[at:at + n], v[at:at + n], w, w, q_out[:n], k_arena, v_arena)
            sb.attention(ctx, shape, rows, q_out[:n], k_arena, v_arena, qg[at:at + n], out[at:at + n])

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for _ in range(args.warmup):
        step()
    ctx.check_status()
    ctx.take_launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    launches = ctx.take_launch_count()
    ctx.check_status()
    # the attention launches alone (the number the roofline is about)
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    attn_ms = 0.0
    for at, n in calls:
        rows = [(0, n, 0, at)]
        sb.attention_prepare(ctx, shape, rows, qg[at:at + n], k[at:at + n], v[at:at + n], w, w, q_out[:n], k_arena, v_arena)
        a0.record()
        for _ in range(3):
            sb.attention(ctx, shape, rows, q_out[:n], k_arena, v_arena, qg[at:at + n], out[at:at + n])
        a1.record()
        torch.cuda.synchronize()
        attn_ms += a0.elapsed_time(a1) / 3
    # end to end: the projections' outputs in pinned host memory in, the o_proj operand back out, copies inside the timed region
    h_qg, h_k, h_v = qg.cpu().pin_memory(), k.cpu().pin_memory(), v.cpu().pin_memory()
    h_out = torch.empty((total, heads * hd), dtype=torch.float16).pin_memory()
    d_qg, d_k, d_v = torch.empty_like(qg[:chunk]), torch.empty_like(k[:chunk]), torch.empty_like(v[:chunk])

    def e2e_step():
        for at, n in calls:
            d_qg[:n].copy_(h_qg[at:at + n], non_blocking=True)
            d_k[:n].copy_(h_k[at:at + n], non_blocking=True)
            d_v[:n].copy_(h_v[at:at + n], non_blocking=True)
            rows = [(0, n, 0, at)]
            sb.attention_prepare(ctx, shape, rows, d_qg[:n], d_k[:n], d_v[:n], w, w, q_out[:n], k_arena, v_arena)
            sb.attention(ctx, shape, rows, q_out[:n], k_arena, v_arena, d_qg[:n], out[at:at + n])
            h_out[at:at + n].copy_(out[at:at + n], non_blocking=True)

    e2e_step()
    barrier()
    e2e_steps = max(1, min(args.steps, 5))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    times = torch.tensor([elapsed_ms, e2e_s * 1e3, attn_ms], dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms, attn_ms = float(times[0]), float(times[1]), float(times[2])
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
        step_ms = elapsed_ms / args.steps
        kernel_tf = flops / (attn_ms * 1e-3) / 1e12
        line = {
            "metric": "attention core TFLOP/s (causal grouped-query, 15,900-token log in four chained calls)",
            "value": round(flops / (step_ms * 1e-3) / 1e12 * world, 2),
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(step_ms, 4),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f16 x f16 -> f32 accumulate, f32 softmax",
            "data": "synthetic",
            "config": {"workload": f"attention: {heads} query / {kvh} key-value heads of {hd}, rotary {rot}, calls of 4096/4096/4096/3612 tokens of one request",
                       "tokens_per_s": round(total / (step_ms * 1e-3) * world, 1),
                       "l2": "q, k, v and the cache of a call are 180 to 400 MB: larger than the 126 MiB L2",
                       "parallelism": f"one request per GPU x{world}, no collective"},
            "roofline": {"bound": "tensor", "achieved": round(kernel_tf, 2), "peak": peak_tf, "unit": "TFLOP/s", "frac": round(kernel_tf / peak_tf, 4),
                         "peak_source": f"bf16_tflops of MEASURED_PEAKS.json ({peak_kind}; burst)", "traffic": None,
                         "kernel": "attention_kernel: algorithmic flops = 4 x head_dim x visible (query, key) pairs x heads; the four launches of a step by CUDA events",
                         "ms_attention_launches": round(attn_ms, 4)},
            "e2e": {"value": round(flops / (e2e_ms * 1e-3) / 1e12 * world, 2), "unit": "TFLOP/s",
                    "h2d_bytes_per_step": total * (2 * heads * hd + 2 * kvh * hd) * 2, "d2h_bytes_per_step": total * heads * hd * 2,
                    "note": "sepal_b200_attention_prepare + sepal_b200_attention per call, q_gate / k / v from pinned host memory, the gated output back to it"},
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    ctx.close()
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def run_deltanet(args):
    """The Gated DeltaNet core of one layer (BASELINE configs[3]'s DeltaNet layers at the 4b geometry: 16 key / 32 value heads of 128, 4 taps)
    over one 4096-token call of a fresh request: convolution + SiLU + q/k normalisation + gates, the chunked delta rule, the gated norm.
    A step is one call of sepal_b200_deltanet. The core is bound by its recurrence (the state of a head is updated chunk after chunk),
    not by memory or by the tensor pipe: the line reports the time per token and, as the roofline, the HBM bytes the call must move
    (bands in, output out, state in and out) against the measured copy bandwidth."""
    import torch

    import sepal_runner_b200 as sb

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    kh, vh, dim, taps, tokens = 16, (16 if args.heads128 else 32), 128, 4, args.tokens
    shape = sb.DeltaNetShape(key_heads=kh, value_heads=vh, head_dim=dim, conv_kernel=taps, eps=1e-6)
    conv_dim, vd = 2 * kh * dim + vh * dim, vh * dim
    ctx = sb.Context(local)
    gen = torch.Generator(device=device).manual_seed(4004 + rank)
    rnd = lambda *sh, s=1.0: (torch.randn(sh, generator=gen, device=device) * s)  # noqa: E731
    sets = []
    per_set = tokens * (conv_dim + vd + 2 * vh) * 2 + tokens * vd * 2
    for _ in range(max(2, -(-int(1.25 * L2_BYTES) // per_set))):  # a ring of inputs larger than the L2
        sets.append((rnd(tokens, conv_dim).half(), rnd(tokens, vd).half(), rnd(tokens, vh).half(), rnd(tokens, vh).half(),
                     torch.empty((tokens, vd), dtype=torch.float16, device=device)))
    conv, a_log, dt_bias, norm = rnd(conv_dim, taps, s=0.5), rnd(vh, s=0.5), rnd(vh, s=0.5), 1.0 + rnd(dim, s=0.1)
    states = torch.zeros((1, vh, dim, dim), dtype=torch.float32, device=device)
    tails = torch.zeros((1, taps - 1, conv_dim), dtype=torch.float32, device=device)
    keep = []

    def step(i):
        mixed, z, b, a, out = sets[i % len(sets)]
        keep.append(sb.deltanet(ctx, shape, [(0, tokens, 0, 1)], mixed, z, b, a, conv, a_log, dt_bias, norm, states, tails, out))
        if len(keep) > 4:
            keep.pop(0)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    ctx.check_status()
    ctx.take_launch_count()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    e1.record()
    barrier()
    elapsed_ms = e0.elapsed_time(e1)
    launches = ctx.take_launch_count()
    ctx.check_status()
    # end to end: the in-projection's bands from pinned host memory, the gated output back to it
    mixed, z, b, a, out = sets[0]
    host = [t.cpu().pin_memory() for t in (mixed, z, b, a)]
    dev = [torch.empty_like(t) for t in (mixed, z, b, a)]
    h_out = torch.empty((tokens, vd), dtype=torch.float16).pin_memory()

    def e2e_step():
        for d, h in zip(dev, host):
            d.copy_(h, non_blocking=True)
        keep.append(sb.deltanet(ctx, shape, [(0, tokens, 0, 1)], *dev, conv, a_log, dt_bias, norm, states, tails, out))
        h_out.copy_(out, non_blocking=True)
        keep.pop(0)

    e2e_step()
    barrier()
    e2e_steps = max(1, min(args.steps, 10))
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    torch.cuda.synchronize()
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
    sampler.stop_flag.set()
    sampler.join(timeout=2)
    times = torch.tensor([elapsed_ms, e2e_ms], dtype=torch.float64, device=device)
    if world > 1:
        import torch.distributed as dist

        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    elapsed_ms, e2e_ms = float(times[0]), float(times[1])
    if rank == 0:
        peaks, peak_kind = measured_peaks()
        step_ms = elapsed_ms / args.steps
        bytes_call = per_set + 2 * vh * dim * dim * 4
        gbs = bytes_call / (step_ms * 1e-3) / 1e9
        peak = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
        line = {
            "metric": "Gated DeltaNet core, tokens/s (one 4096-token call of one request, one layer)",
            "value": round(tokens / (step_ms * 1e-3) * world, 1),
            "unit": "tokens/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": args.warmup,
            "ms_per_step": round(step_ms, 4),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "f16 bands, f32 state, TF32 chunk products",
            "data": "synthetic",
            "config": {"workload": f"deltanet: {kh} key / {vh} value heads of {dim}, {taps} taps, one fresh request of {tokens} tokens",
                       "ns_per_token": round(step_ms * 1e6 / tokens, 1), "l2": f"ring of {len(sets)} input sets > 126 MiB L2",
                       "parallelism": f"one request per GPU x{world}, no collective"},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                         "peak_source": f"hbm_gbs of MEASURED_PEAKS.json ({peak_kind})", "traffic": None,
                         "note": "the recurrence over chunks bounds this core, not memory: the fraction shows how far it is from the bytes it must move"},
            "e2e": {"value": round(tokens / (e2e_ms * 1e-3) * world, 1), "unit": "tokens/s", "h2d_bytes_per_step": tokens * (conv_dim + vd + 2 * vh) * 2,
                    "d2h_bytes_per_step": tokens * vd * 2, "note": "sepal_b200_deltanet with its bands from pinned host memory and the output back to it"},
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    ctx.close()
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def cpu_baseline(kind, m, n, k, reps: int = 5):
    """The reference's cpu-bf16 packed GEMM on this host's cores, on the same product (int8 weights dequantised to float32 first:
    the reference has no group-128 CPU kernel), weights packed once, best of `reps` (runner/tools/sepal_cpu_gemm_bench.cpp:153-201)."""
    import numpy as np

    from oracle.oracle import Oracle, Ref

    rng = np.random.default_rng(1001)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    flops = 2.0 * m * n * k
    if Ref.available():
        r = Ref()
        runs, _ = r.time_gemm(x, w, kind="bf16", reps=reps)
        best = min(p + g for p, g in runs)
        return {"value": round(flops / best / 1e12, 4), "unit": "TFLOP/s", "cores": r.threads(), "kind": "reference",
                "sample": f"{reps} full products of M={m} N={n} K={k} by the reference's gemm_packed ({r.variant()}, {r.brand()}), best, activation packing included",
                "ms": round(best * 1e3, 2)}
    o = Oracle()
    rows = min(m, 64)
    t0 = time.perf_counter()
    o.gemm(x[:rows], w)
    dt = time.perf_counter() - t0
    return {"value": round(2.0 * rows * n * k / dt / 1e12, 5), "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
            "sample": f"{rows} of {m} rows by the float64 oracle (oracle/_ref was not built)", "ms": round(dt * 1e3, 2)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np

    from oracle.oracle import Ref

    kind, m, n, k, cfg_index, _ = WORKLOADS[args.workload]
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not Ref.available():
        print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libsepal_ref.so was not built (the reference tree was absent at build time)"}))
        return
    r = Ref()
    rng = np.random.default_rng(1001)
    x = rng.standard_normal((m, k), dtype=np.float32)
    w = rng.standard_normal((n, k), dtype=np.float32) * np.float32(0.02)
    flops = 2.0 * m * n * k
    steps = max(1, min(args.steps, 50))
    warm = max(1, min(args.warmup, 5))
    runs, _ = r.time_gemm(x, w, kind="bf16", reps=warm + steps)
    timed = runs[warm:]
    total = sum(p + g for p, g in timed)
    value = flops * len(timed) / total / 1e12
    line = {
        "impl": "reference",
        "metric": "GEMM TFLOP/s (f16 tensor cores; w8 group) at M=900",
        "value": round(value, 4),
        "unit": "TFLOP/s",
        "n_gpus": world,
        "steps": len(timed),
        "warmup": warm,
        "ms_per_step": round(total / len(timed) * 1e3, 3),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16 weights x f32/bf16 activations -> f32 accumulate (cpu-bf16)",
        "data": "synthetic",
        "config": {"workload": f"{args.workload} (BASELINE configs[{cfg_index}]): M={m} K={k} N={n}", "calls_per_step": 1,
                   "note": "one full product per step by the reference's cpu-bf16 gemm_packed; int8-group weights run dequantised (no group-128 CPU kernel exists)"},
        "cpu_baseline": {"value": round(value, 4), "unit": "TFLOP/s", "cores": r.threads(), "kind": "reference",
                         "sample": f"{len(timed)} full products, {r.variant()}, {r.brand()}"},
        "e2e": {"value": round(value, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="w8g_down_m900", choices=sorted(WORKLOADS) + ["serve", "attention", "deltanet"])
    ap.add_argument("--tokens", type=int, default=4096, help="deltanet: tokens of the call")
    ap.add_argument("--heads128", action="store_true", help="attention: 32 / 8 heads of 128 instead of 16 / 4 heads of 256")
    ap.add_argument("--int8", action="store_true", help="serve: store the MLP weights as int8 groups")
    ap.add_argument("--no-trunk", dest="trunk", action="store_false", help="skip the whole-trunk passes")
    ap.add_argument("--calls-per-step", type=int, default=512)
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-shapes", dest="shapes", action="store_false", help="skip the per-shape table")
    ap.add_argument("--no-serve", dest="serve", action="store_false", help="skip the request-sharded sweep appended to the default line")
    ap.add_argument("--no-gpu-baseline", dest="gpu_baseline", action="store_false", help="skip the reference's GPU kernels / cuBLAS leg")
    ap.add_argument("--traffic", type=float, default=None, help="DRAM bytes per launch from an ncu capture (reported as roofline.traffic)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        if args.workload in ("serve", "attention", "deltanet") or WORKLOADS[args.workload][4] is None:
            args.workload = "w8g_down_m900"
        run_reference(args)
    elif args.workload == "serve":
        run_serve(args)
    elif args.workload == "attention":
        run_attention(args)
    elif args.workload == "deltanet":
        run_deltanet(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
