#!/usr/bin/env python
"""Benchmark of the hot path: FP8 e4m3 blockwise GEMM with fused 1x128 output
quantisation at M=N=K=4096 (the configuration the headline metric is quoted
on), through the C ABI of libllmmm_b200.so.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one GEMM launch over one batch of synthetic operands.  Prints ONE
JSON line (rank 0).  With N > 1 (launched by torch.distributed.run) every rank
runs the same 4096-row problem on its own GPU: an M-split of a global
M = 4096*N with replicated weights, no data-path collective (weak scaling).

`--impl reference` times the CPU restatement of the reference's own arithmetic
(oracle/, all host threads) on bounded row slabs of the same workload; the
reference project has no CPU implementation of its own.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

M = N = K = 4096
FLOP_PER_STEP = 2.0 * M * N * K
WORKLOAD = ("FP8 e4m3 blockwise GEMM M=N=K=4096: A 1x128 scales, B 128x128 scales, fp32 accumulate with "
            "per-128-K promotion, C emitted as e4m3 with fused 1x128 scales")
METRIC = "fp8_blockwise_gemm_4096_tflops"
UNIT = "TFLOP/s"
SETS = 6  # rotating operand sets: 6 x 49 MB = 294 MB > 126 MB L2
REPEATS = 5  # the timed region of K steps is run this many times; the median region is the one reported


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d, "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ------------------------------------------------------------------ clocks --

class ClockSampler:
    """Samples SM clock, power and clock-event reasons through NVML (read-only) every 10 ms."""

    def __init__(self, index: int):
        self.samples = []
        self.stop_flag = False
        self.ok = False
        self.thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception as e:  # noqa: BLE001
            self.err = repr(e)

    def _reasons(self):
        nv = self.nv
        for name in ("nvmlDeviceGetCurrentClocksEventReasons", "nvmlDeviceGetCurrentClocksThrottleReasons"):
            fn = getattr(nv, name, None)
            if fn is not None:
                try:
                    return int(fn(self.h))
                except Exception:  # noqa: BLE001
                    continue
        return 0

    def _run(self):
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                try:
                    watts = nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0
                except Exception:  # noqa: BLE001
                    watts = 0.0
                self.samples.append((time.perf_counter(), mhz, watts, self._reasons()))
            except Exception:  # noqa: BLE001
                pass
            time.sleep(0.01)

    def start(self):
        if self.ok:
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()

    def stop(self):
        self.stop_flag = True
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self, t0: float, t1: float, window: str):
        if not self.ok:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "note": "NVML unavailable: " + getattr(self, "err", "")}
        names = {0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
                 0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting"}
        inside = [s for s in self.samples if t0 <= s[0] <= t1]
        use = inside if inside else self.samples
        bits = 0
        for s in use:
            bits |= s[3]
        reasons = [n for b, n in names.items() if bits & b and n != "gpu_idle"]
        return {
            "sm_mhz": statistics.median(s[1] for s in use) if use else None,
            "sm_max_mhz": self.max_mhz,
            "power_w_max": max((s[2] for s in use), default=None),
            "reasons": reasons,
            "samples": len(use),
            "window": window,
        }


def prefer_host_memory_near_gpu(index: int):
    """Best effort, for the pinned host buffers of the end-to-end leg: ask the kernel to place this process's new
    pages on the NUMA node the GPU hangs off (set_mempolicy(MPOL_PREFERRED); read-only for the GPU itself).  With
    several ranks on one box each rank then copies from memory next to its own GPU instead of all from the node
    the launcher started on.  Returns what was done, for the JSON line."""
    import ctypes
    try:
        import pynvml
        pynvml.nvmlInit()
        bus = pynvml.nvmlDeviceGetPciInfo(pynvml.nvmlDeviceGetHandleByIndex(index)).busId
        bus = bus.decode() if isinstance(bus, bytes) else bus
        path = Path("/sys/bus/pci/devices") / bus[-12:].lower() / "numa_node"
        node = int(path.read_text())
        if node < 0:
            return {"numa_node": None, "policy": "unchanged (the platform reports no NUMA node for the GPU)"}
        libc = ctypes.CDLL(None, use_errno=True)
        mask = ctypes.c_ulong(1 << node)
        rc = libc.syscall(238, 1, ctypes.byref(mask), ctypes.c_ulong(64))  # x86-64 set_mempolicy, MPOL_PREFERRED
        return {"numa_node": node, "policy": "preferred" if rc == 0 else f"unchanged (set_mempolicy errno {ctypes.get_errno()})"}
    except Exception as e:  # noqa: BLE001
        return {"numa_node": None, "policy": "unchanged (" + repr(e)[:80] + ")"}


# --------------------------------------------------------------- reference --

def reference_arm(args) -> int:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    import numpy as np
    from oracle import oracle as o
    o.build()
    o.set_num_threads(len(os.sched_getaffinity(0)))  # torchrun exports OMP_NUM_THREADS=1; use every core we may
    cores = o.num_threads()
    rows = 256  # one step = a 256-row slab of the 4096-row problem (about 0.5 s on 8 cores)
    rng = np.random.default_rng(0x4C4D4D4D)
    x = rng.standard_normal((rows, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    A_q, A_s = o.quant_1x128(x)
    B_q, B_s = o.quant_128x128(w)

    def step():
        acc = o.fp8_blockwise_acc(A_q, A_s, B_q, B_s)
        o.c_quant_1x128(acc)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    value = 2.0 * rows * N * K / (ms * 1e-3) / 1e12
    sample = f"{rows}-row slab of the 4096-row problem per step (M={rows}, N=K=4096), {cores} OpenMP threads"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp8_e4m3 operands, fp32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference project has no CPU code; this is the CPU restatement of its arithmetic (oracle/)",
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------ ours ----

def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extra", action="store_true", help="skip the secondary configurations")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--quick", action="store_true",
                    help="profiling mode: timed region only (no sustained clock loop, e2e, extra configs or CPU baseline)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, SETS)  # every operand set is touched before the clock starts

    import torch
    import torch.distributed as dist
    from llmmm_b200 import capi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a B200 GPU: the library has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    capi.lib()  # fails loudly if the CUDA library is missing
    stream = torch.cuda.current_stream()
    # caller-owned scratch, registered once: lets the kernel cut the tiles of its last, partly filled wave along K
    capi.ensure_workspace(M, N, K)

    # operands: fp32 N(0,1) sources quantised by the library's own quantisers (1x128 / 128x128)
    gen = torch.Generator(device=dev).manual_seed(0x4C4D4D4D + 2 + rank)
    sets = []
    for _ in range(SETS):
        x = torch.randn(M, K, device=dev, generator=gen)
        w = torch.randn(N, K, device=dev, generator=gen)
        A_q = torch.empty(M, K, dtype=torch.uint8, device=dev)
        A_s = torch.empty(K // 128, M, device=dev)
        B_q = torch.empty(N, K, dtype=torch.uint8, device=dev)
        B_s = torch.empty(N // 128, K // 128, device=dev)
        capi.fp8_quant_1x128(x, A_q, A_s, M, K)
        capi.fp8_quant_128x128(w, B_q, B_s, N, K)
        C_q = torch.empty(M, N, dtype=torch.uint8, device=dev)
        C_s = torch.empty(N // 128, M, device=dev)
        sets.append((A_q, A_s, B_q, B_s, C_q, C_s))
        del x, w
    torch.cuda.synchronize()

    def step(i):
        A_q, A_s, B_q, B_s, C_q, C_s = sets[i % SETS]
        capi.fp8_blockwise_mm(A_q, A_s, B_q, B_s, C_q, C_s, M, N, K)

    sampler = ClockSampler(local)
    sampler.start()
    for i in range(args.warmup):
        step(i)
    launches0 = capi.launch_count()
    split0 = capi.split_launch_count()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    region_ms = []
    for _ in range(REPEATS):
        barrier()
        e0.record(stream)
        for i in range(args.steps):
            step(i)
        e1.record(stream)
        torch.cuda.synchronize()
        region_ms.append(e0.elapsed_time(e1))
    launches = (capi.launch_count() - launches0) // REPEATS  # per region of K steps
    split_launches = (capi.split_launch_count() - split0) // REPEATS  # launches that cut the tiles of their last wave along K
    barrier()
    ms_total = statistics.median(region_ms)
    # sustained loop of the same kernel (about 1 s) so that the clock samples are taken under load
    t_load = time.perf_counter()
    reps = 0 if args.quick else max(200, int(1.0 / max(ms_total / args.steps * 1e-3, 1e-6)))
    for i in range(reps):
        step(i)
    torch.cuda.synchronize()
    t_end = time.perf_counter()
    sampler.stop()
    clocks = sampler.summary(t_begin, t_end, "timed region + 1 s sustained loop of the same kernel")
    capi.check_status()

    ms_fastest_rank = ms_total / args.steps
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_min = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t_min, op=dist.ReduceOp.MIN)
        ms_total, ms_fastest_rank = float(t.item()), float(t_min.item()) / args.steps
    ms_step = ms_total / args.steps
    value = world * FLOP_PER_STEP / (ms_step * 1e-3) / 1e12

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region
    A_q, A_s, B_q, B_s, C_q, C_s = sets[0]
    host_numa = prefer_host_memory_near_gpu(local)
    host_in = [t.cpu().pin_memory() for t in (A_q, A_s, B_q, B_s)]
    host_out = [torch.empty_like(t, device="cpu").pin_memory() for t in (C_q, C_s)]
    h2d = sum(t.numel() * t.element_size() for t in host_in)
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    e2e_steps = 1 if args.quick else max(3, min(args.steps, 30))

    # Every step copies its operands in, runs the GEMM and copies its result out; the package's host-buffer
    # entry overlaps the three phases of successive steps (copy-in of i+1, kernel of i, copy-out of i-1).
    from llmmm_b200.host_pipeline import Fp8GemmHostPipeline
    pipe = Fp8GemmHostPipeline(M, N, K, depth=2, device=dev)
    assert (pipe.h2d_bytes, pipe.d2h_bytes) == (h2d, d2h)

    def e2e_run(n):
        for _ in range(n):
            pipe.submit(*host_in, *host_out)
        pipe.drain()  # every result is in host memory

    e2e_run(0 if args.quick else 3)
    barrier()
    t0 = time.perf_counter()
    e2e_run(e2e_steps)
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3
    # the result that came back is the one the device-resident path produced for the same operands
    capi.fp8_blockwise_mm(A_q, A_s, B_q, B_s, C_q, C_s, M, N, K)
    torch.cuda.synchronize()
    assert torch.equal(host_out[0], C_q.cpu()) and torch.equal(host_out[1], C_s.cpu()), "e2e result differs"
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * FLOP_PER_STEP / (e2e_ms * 1e-3) / 1e12

    peaks, peak_kind = measured_peaks()
    fp8_peak = 2.0 * float(peaks["bf16_tflops"])
    achieved = FLOP_PER_STEP / (ms_step * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s", "frac": achieved / fp8_peak,
        "traffic": 37.7e6,
        "traffic_source": "dram__bytes_read.sum 34.13 MB + dram__bytes_write.sum 3.55 MB of one launch of this kernel on this "
                          "workload, from one ncu --set full capture (not re-measured by this run)",
        "peak_source": f"2 x bf16_tflops ({peak_kind}; the file has no fp8 figure; burst, kernel timed alone)",
        "frac_of_nominal_4500": achieved / 4500.0,
        "kernel": "fp8_blockwise_gemm_pair_kernel<EPI_E4M3>",
    }
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp8_e4m3 operands, fp32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOAD, "per_gpu": "M=N=K=4096", "sharding": "M-split (independent rows), replicated weights, no collective",
                   "l2": f"{SETS} rotating operand sets ({SETS * 49} MB) exceed the 126 MB L2",
                   "scratch": f"{capi.fp8_workspace_bytes(M, N, K)} bytes registered with llmmm_set_workspace"},
        "clocks": clocks,
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": e2e_ms, "steps": e2e_steps, "host_memory": host_numa},
        "gpu_launches": launches,
        "split_launches": split_launches,
        "ms_per_step_fastest_rank": ms_fastest_rank,  # ms_per_step is the slowest rank's (the ranks do not communicate)
        "repeats": REPEATS,  # ms_per_step is the median over this many timed regions of `steps` launches each
        "ms_per_step_of_each_region_rank0": [t / args.steps for t in region_ms],
        "roofline": roofline,
    }

    if world > 1 and not args.no_extra and not args.quick:
        ns = nsplit_config(torch, dist, capi, dev, rank, world)
        if rank == 0:
            line["extra"] = {"mlp7b_split": ns}
    if rank == 0 and world == 1 and not args.no_extra and not args.quick:
        line["extra"] = extra_configs(torch, capi, dev, peaks)
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not args.quick:
        line["cpu_baseline"] = cpu_baseline(sets[0])
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def cpu_baseline(s0):
    """The oracle's restatement of the reference arithmetic, timed on the host cores on a bounded sample."""
    from oracle import oracle as o
    o.build()
    o.set_num_threads(len(os.sched_getaffinity(0)))
    rows = 1024
    A_q, A_s, B_q, B_s = (t.cpu().numpy() for t in s0[:4])
    A_q, A_s = A_q[:rows].copy(), A_s[:, :rows].copy()
    # about 10 s of CPU work: passes over a 1024-row slab of the 4096-row problem until the clock says so
    passes, t0 = 0, time.perf_counter()
    while True:
        acc = o.fp8_blockwise_acc(A_q, A_s, B_q, B_s)
        o.c_quant_1x128(acc)
        passes += 1
        dt = time.perf_counter() - t0
        if dt >= 10.0 or passes >= 64:
            break
    return {"value": 2.0 * passes * rows * N * K / dt / 1e12, "unit": UNIT, "cores": o.num_threads(), "kind": "port",
            "sample": f"first {rows} of the 4096 rows, {passes} passes ({dt:.1f} s)"}


def time_graph(torch, fn_list, iters=5):
    """Median time per call of a CUDA graph that replays fn_list once (launch overhead excluded)."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for f in fn_list:
            f()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fn_list:
            f()
    g.replay()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1) / len(fn_list))
    return statistics.median(times)


def reference_kernels(torch, capi, dev, fp16_sets, our_fp16_us):
    """Times the reference's own GPU kernels (the unmodified sources compiled for sm_100a into oracle/_ref by
    oracle/Makefile: LLMMM::fp16_mm<half>, src/mm/fp16/mm.cu:7-42, and the two fused FP8 launchers
    examples/005.fp8.mm.cu:2499-2577) at 4096^3 beside this library on the same operands.  A bench-side
    comparison like the CPU baseline: nothing under oracle/ is on the product path."""
    import ctypes
    so = ROOT / "oracle" / "_ref" / "libllmmm_ref.so"
    if not so.exists():
        return {"unavailable": "oracle/_ref/libllmmm_ref.so was not built (needs the reference checkout at build time)"}
    ref = ctypes.CDLL(str(so))
    vp = ctypes.c_void_p
    res = {}
    fns = [(lambda s=s: ref.ref_fp16_mm_f16(vp(s[0].data_ptr()), vp(s[1].data_ptr()), vp(s[2].data_ptr()), 4096, 4096, 4096,
                                                vp(torch.cuda.current_stream().cuda_stream)))
           for s in fp16_sets] * 4
    ms = time_graph(torch, fns)
    res["ref_fp16_mm_f16"] = {"us": ms * 1e3, "tflops": 2.0 * 4096 ** 3 / (ms * 1e-3) / 1e12, "ours_us": our_fp16_us,
                              "speedup_ours": ms * 1e3 / our_fp16_us}
    sets = []
    for _ in range(3):
        A = torch.randint(0, 120, (4096, 4096), dtype=torch.uint8, device=dev)
        B = torch.randint(0, 120, (4096, 4096), dtype=torch.uint8, device=dev)
        sets.append((A, torch.rand(32, 4096, device=dev), B, torch.rand(32, 32, device=dev),
                     torch.empty(4096, 4096, dtype=torch.uint8, device=dev), torch.empty(32, 4096, device=dev)))
    capi.ensure_workspace(4096, 4096, 4096)
    ours = time_graph(torch, [(lambda s=s: capi.fp8_blockwise_mm(*s, 4096, 4096, 4096)) for s in sets] * 4)
    for name in ("ref_fp8_mm_opt_reg", "ref_fp8_mm_inner_split"):
        fn = getattr(ref, name)
        ms = time_graph(torch, [(lambda s=s: fn(*(vp(t.data_ptr()) for t in s), 4096, 4096, 4096,
                                                 vp(torch.cuda.current_stream().cuda_stream))) for s in sets] * 4)
        res[name] = {"us": ms * 1e3, "tflops": 2.0 * 4096 ** 3 / (ms * 1e-3) / 1e12, "ours_us": ours * 1e3,
                     "speedup_ours": ms / ours}
    return res


def extra_configs(torch, capi, dev, peaks):
    """Secondary configurations of the same path: FP16 4096^3 and the Qwen3-4B decode shapes."""
    out = {}
    gen = torch.Generator(device=dev).manual_seed(7)
    # FP16 GEMM 4096^3, rotating sets
    sets = []
    for _ in range(3):
        A = (torch.rand(4096, 4096, device=dev, generator=gen) * 2 - 1).half()
        B = (torch.rand(4096, 4096, device=dev, generator=gen) * 2 - 1).half()
        C = torch.empty(4096, 4096, device=dev, dtype=torch.float16)
        sets.append((A, B, C))
    fns = [(lambda s=s: capi.fp16_mm(s[0], s[1], s[2], 4096, 4096, 4096)) for s in sets] * 8
    ms = time_graph(torch, fns)
    tf = 2.0 * 4096 ** 3 / (ms * 1e-3) / 1e12
    out["fp16_gemm_4096"] = {"us": ms * 1e3, "tflops": tf, "frac_of_measured_bf16_burst": tf / float(peaks["bf16_tflops"]),
                             "frac_of_nominal_2250": tf / 2250.0}
    del sets, fns
    # the same FP16 problem through torch.matmul (cuBLAS): a sanity figure for this box and its power state, not
    # part of the product path
    sets = []
    for _ in range(3):
        A = (torch.rand(4096, 4096, device=dev, generator=gen) * 2 - 1).half()
        B = (torch.rand(4096, 4096, device=dev, generator=gen) * 2 - 1).half()
        sets.append((A, B, torch.empty(4096, 4096, device=dev, dtype=torch.float16)))
    ms_cublas = time_graph(torch, [(lambda s=s: torch.matmul(s[0], s[1], out=s[2])) for s in sets] * 8)
    out["fp16_gemm_4096"]["torch_matmul_us"] = ms_cublas * 1e3
    out["fp16_gemm_4096"]["torch_matmul_tflops"] = 2.0 * 4096 ** 3 / (ms_cublas * 1e-3) / 1e12
    out["fp16_gemm_4096"]["ours_over_torch_matmul"] = ms_cublas / ms
    # ... and the reference project's own kernels, rebuilt unmodified for sm_100a (mma.sync / ldmatrix; oracle/_ref,
    # present only if the reference checkout was there at build time), on the same 4096^3 problems
    out["reference_kernels_4096"] = reference_kernels(torch, capi, dev, sets, out["fp16_gemm_4096"]["us"])
    del sets
    # the four Qwen3-4B linears at prefill size (M = 4096)
    pre = []
    for name, (n, k) in (("qkv", (6144, 2560)), ("o", (2560, 4096)), ("gate_up", (19456, 2560)), ("down", (2560, 9728))):
        m = 4096
        ws = [(torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev), torch.rand(n // 128, k // 128, device=dev))
              for _ in range(3)]
        xq = torch.randint(0, 120, (m, k), dtype=torch.uint8, device=dev)
        xs = torch.rand(k // 128, m, device=dev)
        Cq = torch.empty(m, n, dtype=torch.uint8, device=dev)
        Cs = torch.empty(n // 128, m, device=dev)
        capi.ensure_workspace(m, n, k)
        ms_p = time_graph(torch, [(lambda w=w: capi.fp8_blockwise_mm(xq, xs, w[0], w[1], Cq, Cs, m, n, k)) for w in ws] * 4)
        tf_p = 2.0 * m * n * k / (ms_p * 1e-3) / 1e12
        pre.append({"linear": name, "M": m, "N": n, "K": k, "us": ms_p * 1e3, "tflops": tf_p,
                    "frac_of_2x_measured_bf16_burst": tf_p / (2.0 * float(peaks["bf16_tflops"]))})
        del ws
    out["qwen3_4b_prefill"] = pre
    # the two 7B-scale MLP GEMMs at M = 8192 on ONE GPU (the 1-rank point of the N-split configuration)
    mlp7 = []
    for name, (n, k) in (("gate_up", (37888, 3584)), ("down", (3584, 18944))):
        m = 8192
        ws = [(torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev), torch.rand(n // 128, k // 128, device=dev))
              for _ in range(2)]
        xq = torch.randint(0, 120, (m, k), dtype=torch.uint8, device=dev)
        xs = torch.rand(k // 128, m, device=dev)
        Cq = torch.empty(m, n, dtype=torch.uint8, device=dev)
        Cs = torch.empty(n // 128, m, device=dev)
        capi.ensure_workspace(m, n, k)
        ms_p = time_graph(torch, [(lambda w=w: capi.fp8_blockwise_mm(xq, xs, w[0], w[1], Cq, Cs, m, n, k)) for w in ws] * 3)
        tf_p = 2.0 * m * n * k / (ms_p * 1e-3) / 1e12
        mlp7.append({"gemm": name, "M": m, "N": n, "K": k, "ranks": 1, "ms": ms_p, "tflops": tf_p,
                     "frac_of_2x_measured_bf16_burst": tf_p / (2.0 * float(peaks["bf16_tflops"]))})
        del ws, xq, xs, Cq, Cs
    out["mlp7b_one_gpu"] = mlp7
    # decode shapes (HBM-bound): rotate over enough weight copies to exceed L2.  Every shape is timed twice: with the
    # plan the default rule picks, and after llmmm_tune has measured the plans for that weight shape.
    dec = []
    shapes = [(6144, 2560), (2560, 4096), (19456, 2560), (2560, 9728)]
    capi.ensure_workspace(64, 19456, 2560)

    def decode_rows(tag):
        rows = []
        for (n, k) in shapes:
            copies = max(3, int(300e6 // (n * k)) + 1)
            ws = [(torch.randint(0, 120, (n, k), dtype=torch.uint8, device=dev), torch.rand(n // 128, k // 128, device=dev))
                  for _ in range(copies)]
            for m in (1, 16, 64):
                xq = torch.randint(0, 120, (m, k), dtype=torch.uint8, device=dev)
                xs = torch.rand(k // 128, m, device=dev)
                Cq = torch.empty(m, n, dtype=torch.uint8, device=dev)
                Cs = torch.empty(n // 128, m, device=dev)
                fns = [(lambda w=w: capi.fp8_blockwise_mm(xq, xs, w[0], w[1], Cq, Cs, m, n, k)) for w in ws] * 2
                ms_plain = time_graph(torch, fns)
                # the weights of a serving loop are static: with that promise each launch of the chain requests its
                # first weight tiles while the launch before it is still finishing
                capi.set_static_weights(True)
                ms = time_graph(torch, fns)
                capi.set_static_weights(False)
                rows.append({"M": m, "N": n, "K": k, "us": ms * 1e3, "us_without_static_weights": ms_plain * 1e3,
                             "plan": capi.describe_plan("fp8", m, n, k)[:96] + " ... / " + tag})
            del ws
        return rows

    default_rows = decode_rows("default rule")
    capi.set_static_weights(True)
    for (n, k) in shapes:
        capi.tune("fp8", n, k)
    capi.set_static_weights(False)
    tuned_rows = decode_rows("measured by llmmm_tune")
    for d_, t_ in zip(default_rows, tuned_rows):
        m, n, k = t_["M"], t_["N"], t_["K"]
        by = n * k + 4 * (n // 128) * (k // 128) + m * k + 4 * m * k // 128 + m * n + 4 * m * n // 128
        gbs = by / (t_["us"] * 1e-6) / 1e9
        dec.append({**t_, "us_default_rule": d_["us"], "plan_default_rule": d_["plan"], "gbs": gbs,
                    "frac_of_measured_hbm": gbs / float(peaks["hbm_gbs"])})
    out["qwen3_4b_decode"] = dec
    # HBM-bound helpers of the same path at 4096 x 4096: the two quantisers (4 B read + 1 B written per element,
    # plus scales) and the transposes (1 B / 4 B read and written)
    hbm = float(peaks["hbm_gbs"])
    x = torch.randn(3, 4096, 4096, device=dev, generator=gen)
    q = torch.empty(3, 4096, 4096, dtype=torch.uint8, device=dev)
    s1 = torch.empty(32, 4096, device=dev)
    s2 = torch.empty(32, 32, device=dev)
    xt = torch.empty(3, 4096, 4096, device=dev)
    qt = torch.empty(3, 4096, 4096, dtype=torch.uint8, device=dev)
    wn = torch.rand(4096, device=dev, generator=gen) + 0.5
    cases = {
        "quant_1x128": ([lambda i=i: capi.fp8_quant_1x128(x[i], q[i], s1, 4096, 4096) for i in range(3)], 5 * 4096 * 4096 + 4 * 32 * 4096),
        "quant_128x128": ([lambda i=i: capi.fp8_quant_128x128(x[i], q[i], s2, 4096, 4096) for i in range(3)], 5 * 4096 * 4096 + 4 * 32 * 32),
        "rmsnorm_quant_1x128": ([lambda i=i: capi.fp8_rmsnorm_quant_1x128(x[i], wn, 1e-6, q[i], s1, 4096, 4096) for i in range(3)], 5 * 4096 * 4096 + 4 * 32 * 4096 + 4 * 4096),
        "transpose_f32": ([lambda i=i: capi.transpose_aligned_128(xt[i], x[i], 4096, 4096) for i in range(3)], 8 * 4096 * 4096),
        "transpose_e4m3": ([lambda i=i: capi.transpose_aligned_128(qt[i], q[i], 4096, 4096) for i in range(3)], 2 * 4096 * 4096),
    }
    helpers = {}
    for name, (fns, nbytes) in cases.items():
        ms = time_graph(torch, fns * 6)
        helpers[name] = {"us": ms * 1e3, "gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_measured_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm}
    out["hbm_helpers_4096x4096"] = helpers
    del x, q, xt, qt
    # gate_up projection of the Qwen3-4B MLP at M = 4096 with the SwiGLU epilogue fused (H = silu(gate) * up,
    # quantised 1x128 for the down projection), beside the plain GEMM of the same [2I, K] weight
    m, i_, k = 4096, 9728, 2560
    aq = torch.randint(0, 120, (m, k), dtype=torch.uint8, device=dev)
    a_s = torch.rand(k // 128, m, device=dev)
    wsets = [(torch.randint(0, 120, (2 * i_, k), dtype=torch.uint8, device=dev), torch.rand(2 * i_ // 128, k // 128, device=dev))
             for _ in range(3)]
    hq = torch.empty(m, i_, dtype=torch.uint8, device=dev)
    hs = torch.empty(i_ // 128, m, device=dev)
    cq = torch.empty(m, 2 * i_, dtype=torch.uint8, device=dev)
    cs = torch.empty(2 * i_ // 128, m, device=dev)
    capi.ensure_workspace(m, 2 * i_, k)
    ms_f = time_graph(torch, [(lambda w=w: capi.fp8_blockwise_mm_swiglu(aq, a_s, w[0], w[1], hq, hs, m, i_, k)) for w in wsets] * 4)
    ms_p = time_graph(torch, [(lambda w=w: capi.fp8_blockwise_mm(aq, a_s, w[0], w[1], cq, cs, m, 2 * i_, k)) for w in wsets] * 4)
    flop = 2.0 * m * 2 * i_ * k
    out["swiglu_gate_up_4096x19456x2560"] = {
        "us_fused": ms_f * 1e3, "tflops_fused": flop / (ms_f * 1e-3) / 1e12,
        "us_plain_gemm_same_weight": ms_p * 1e3, "tflops_plain": flop / (ms_p * 1e-3) / 1e12,
        "frac_of_2x_measured_bf16_burst": flop / (ms_f * 1e-3) / 1e12 / (2.0 * float(peaks["bf16_tflops"]))}
    # the same MLP front half at decode size (M = 1, 16): decode GEMM into scratch + SwiGLU/quantise kernel
    capi.set_static_weights(True)
    dec_sw = []
    for m_ in (1, 16):
        xq = torch.randint(0, 120, (m_, k), dtype=torch.uint8, device=dev)
        xs = torch.rand(k // 128, m_, device=dev)
        hq_ = torch.empty(m_, i_, dtype=torch.uint8, device=dev)
        hs_ = torch.empty(i_ // 128, m_, device=dev)
        capi.ensure_swiglu_workspace(m_, i_, k)
        ms_d = time_graph(torch, [(lambda w=w: capi.fp8_blockwise_mm_swiglu(xq, xs, w[0], w[1], hq_, hs_, m_, i_, k)) for w in wsets] * 4)
        by = 2 * i_ * k + 4 * (2 * i_ // 128) * (k // 128) + m_ * k + 4 * m_ * k // 128 + m_ * i_ + 4 * m_ * i_ // 128
        dec_sw.append({"M": m_, "us": ms_d * 1e3, "gbs": by / (ms_d * 1e-3) / 1e9, "frac_of_measured_hbm": by / (ms_d * 1e-3) / 1e9 / hbm})
    out["swiglu_gate_up_decode_19456x2560"] = dec_sw
    # the whole Qwen3-4B MLP block as three launches that hand each other 1x128-quantised activations:
    # RMSNorm + quantise (hidden 2560) -> gate_up + SwiGLU + quantise (I = 9728) -> down projection (fp32 out)
    mlp = []
    wd = [(torch.randint(0, 120, (k, i_), dtype=torch.uint8, device=dev), torch.rand(k // 128, i_ // 128, device=dev)) for _ in range(3)]
    gamma = torch.rand(k, device=dev) + 0.5
    for m_ in (1, 16, 4096):
        xin = torch.randn(m_, k, device=dev)
        xq = torch.empty(m_, k, dtype=torch.uint8, device=dev)
        xs = torch.empty(k // 128, m_, device=dev)
        hq_ = torch.empty(m_, i_, dtype=torch.uint8, device=dev)
        hs_ = torch.empty(i_ // 128, m_, device=dev)
        y = torch.empty(m_, k, device=dev)
        if m_ <= 64:
            capi.ensure_swiglu_workspace(m_, i_, k)

        def block(j):
            capi.fp8_rmsnorm_quant_1x128(xin, gamma, 1e-6, xq, xs, m_, k)
            capi.fp8_blockwise_mm_swiglu(xq, xs, wsets[j][0], wsets[j][1], hq_, hs_, m_, i_, k)
            capi.fp8_blockwise_mm_f32(hq_, hs_, wd[j][0], wd[j][1], y, m_, k, i_)

        ms_b = time_graph(torch, [(lambda j=j: block(j)) for j in range(3)] * 4)
        mlp.append({"M": m_, "us_per_block": ms_b * 1e3, "launches_per_block": 3 if m_ > 64 else 4,
                    "weight_bytes": 3 * i_ * k, "tflops": 2.0 * m_ * 3 * i_ * k / (ms_b * 1e-3) / 1e12})
    out["qwen3_4b_mlp_block"] = mlp
    # qkv projection of Qwen3-4B (32 query + 8 key + 8 value heads of 128, hidden 2560) with the per-head q/k
    # RMSNorm and the rotary embedding fused in front of the output quantisation, beside the plain GEMM
    n_q, n_kv = 32, 8
    nq = (n_q + 2 * n_kv) * 128
    wq = [(torch.randint(0, 120, (nq, k), dtype=torch.uint8, device=dev), torch.rand(nq // 128, k // 128, device=dev)) for _ in range(3)]
    ang = torch.arange(8192, device=dev, dtype=torch.float32)[:, None] / (1e6 ** (torch.arange(64, device=dev) / 64.0))[None, :]
    cos_t, sin_t = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    qw, kw = torch.rand(128, device=dev) + 0.5, torch.rand(128, device=dev) + 0.5
    qkv = []
    for m_ in (1, 16, 4096):
        xq = torch.randint(0, 120, (m_, k), dtype=torch.uint8, device=dev)
        xs = torch.rand(k // 128, m_, device=dev)
        oq = torch.empty(m_, nq, dtype=torch.uint8, device=dev)
        os_ = torch.empty(nq // 128, m_, device=dev)
        pos = (torch.arange(m_, device=dev, dtype=torch.int32) + 17) % 8192
        capi.ensure_qk_norm_rope_workspace(m_, nq, k)
        ms_r = time_graph(torch, [(lambda w=w: capi.fp8_blockwise_mm_qk_norm_rope(xq, xs, w[0], w[1], oq, os_, pos, cos_t, sin_t, qw, kw,
                                                                                  1e-6, n_q, n_kv, m_, nq, k)) for w in wq] * 4)
        ms_g = time_graph(torch, [(lambda w=w: capi.fp8_blockwise_mm(xq, xs, w[0], w[1], oq, os_, m_, nq, k)) for w in wq] * 4)
        qkv.append({"M": m_, "us_fused": ms_r * 1e3, "us_plain_gemm": ms_g * 1e3, "launches": 1 if m_ > 64 else 2,
                    "tflops_fused": 2.0 * m_ * nq * k / (ms_r * 1e-3) / 1e12})
    capi.set_static_weights(False)
    out["qwen3_4b_qkv_norm_rope_6144x2560"] = qkv
    capi.check_status()
    return out


def nsplit_config(torch, dist, capi, dev, rank, world):
    """Config 5 of the task: the two 7B-scale MLP GEMMs at M = 8192 partitioned over the ranks.
    gate_up (N = 37888, K = 3584): N-split on 128-column group boundaries, replicated activations; per-rank GEMM,
    GEMM + NCCL all-gather of C_q / C_s into the blocked [ranks][M][N_r] layout (all_gather_into_tensor, nothing
    around the collective), and the GEMM that does the gather itself with peer stores from its epilogue.
    down (N = 3584 = 28 groups, K = 18944): N-split (uneven over 8 ranks) beside an M-split of the same GEMM."""
    from llmmm_b200 import shard
    Mm = 8192

    def timed(fn, n):
        for _ in range(2):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True)
        e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / n], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    gen = torch.Generator(device=dev).manual_seed(11 + rank)
    res = {}

    # ------------------------------------------------------------------ gate_up, N-split
    Nn, Kk = 37888, 3584
    n0, n1 = shard.split_n(Nn, world, rank)
    nr = n1 - n0
    even = all(shard.split_n(Nn, world, r)[1] - shard.split_n(Nn, world, r)[0] == nr for r in range(world))
    A_q = torch.randint(0, 120, (Mm, Kk), dtype=torch.uint8, device=dev, generator=gen)
    A_s = torch.rand(Kk // 128, Mm, device=dev, generator=gen)
    B_q = torch.randint(0, 120, (nr, Kk), dtype=torch.uint8, device=dev, generator=gen)
    B_s = torch.rand(nr // 128, Kk // 128, device=dev, generator=gen)
    C_q = torch.empty(Mm, nr, dtype=torch.uint8, device=dev)
    C_s = torch.empty(nr // 128, Mm, device=dev)
    capi.ensure_workspace(Mm, nr, Kk)

    def gemm():
        capi.fp8_blockwise_mm(A_q, A_s, B_q, B_s, C_q, C_s, Mm, nr, Kk)

    gather = (lambda: shard.all_gather_c_n_blocked(C_q, C_s)) if even else (lambda: shard.all_gather_c_n(C_q, C_s, Nn))
    ms_gemm = timed(gemm, 10)
    ms_both = timed(lambda: (gemm(), gather()), 5)
    flops = 2.0 * Mm * Nn * Kk
    sent = (world - 1) * (Mm * nr + 4 * (nr // 128) * Mm)  # bytes a rank sends (and receives) for the gather
    g = {"shape": "M=8192 N=37888 K=3584, N-split", "ranks": world, "ms_gemm": ms_gemm,
         "tflops_gemm_total": flops / (ms_gemm * 1e-3) / 1e12, "ms_gemm_plus_nccl_allgather": ms_both,
         "nccl_allgather": "all_gather_into_tensor into the blocked [ranks][M][N_r] layout" if even else "padded list all_gather (uneven split)",
         "gathered_bytes_per_rank": Mm * Nn + 4 * (Nn // 128) * Mm, "bytes_sent_per_rank": sent}
    # The same gather done by the GEMM itself: every rank's epilogue stores its column shard into the full C of
    # every rank (peer buffers from torch symmetric memory).  Whether the peer mapping works is agreed on by all
    # ranks before any further collective, so that no rank waits for one that gave up.
    po, err = None, ""
    try:
        po = shard.PeerOutputs(Mm, Nn, dev)
    except Exception as e:  # noqa: BLE001  (a box without peer access between its GPUs)
        err = repr(e)[:200]
    ok = torch.tensor([1 if po is not None else 0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)
    if bool(ok.item()):
        dq, ds = po.dsts()
        ms_fused = timed(lambda: capi.fp8_blockwise_mm_gather(A_q, A_s, B_q, B_s, dq, ds, Nn, n0, Mm, nr, Kk), 10)
        po.wait_all()
        gemm()
        q_ref, s_ref = shard.all_gather_c_n(C_q, C_s, Nn)
        same = torch.tensor([1 if (torch.equal(po.C_q, q_ref) and torch.equal(po.C_s, s_ref)) else 0], device=dev)
        dist.all_reduce(same, op=dist.ReduceOp.MIN)
        g.update({"ms_gemm_with_fused_gather": ms_fused, "tflops_total_with_fused_gather": flops / (ms_fused * 1e-3) / 1e12,
                  "fused_gather_gbs_sent_per_rank": sent / (ms_fused * 1e-3) / 1e9,
                  "fused_gather_frac_of_770_gbs_peer_copy": sent / (ms_fused * 1e-3) / 1e9 / 770.0,
                  "fused_gather_equals_nccl_gather_on_all_ranks": bool(same.item())})
        po.close()
        del q_ref, s_ref
    else:
        g["fused_gather_unavailable"] = err or "another rank could not map the peer buffers"
    res["gate_up"] = g
    del A_q, A_s, B_q, B_s, C_q, C_s, po
    torch.cuda.empty_cache()

    # ------------------------------------------------------------------ down, N-split beside M-split
    Nn, Kk = 3584, 18944
    n0, n1 = shard.split_n(Nn, world, rank)
    nr = n1 - n0
    m0, m1 = shard.split_m(Mm, world, rank)
    mr = m1 - m0
    A_q = torch.randint(0, 120, (Mm, Kk), dtype=torch.uint8, device=dev, generator=gen)
    A_s = torch.rand(Kk // 128, Mm, device=dev, generator=gen)
    B_q = torch.randint(0, 120, (Nn, Kk), dtype=torch.uint8, device=dev, generator=gen)
    B_s = torch.rand(Nn // 128, Kk // 128, device=dev, generator=gen)
    Bq_r, Bs_r = B_q[n0:n1].contiguous(), B_s[n0 // 128:n1 // 128].contiguous()
    Aq_r, As_r = shard.shard_activations_m(A_q, A_s, world, rank)
    Cn_q = torch.empty(Mm, nr, dtype=torch.uint8, device=dev)
    Cn_s = torch.empty(nr // 128, Mm, device=dev)
    Cm_q = torch.empty(mr, Nn, dtype=torch.uint8, device=dev)
    Cm_s = torch.empty(Nn // 128, mr, device=dev)
    capi.ensure_workspace(Mm, nr, Kk)
    capi.ensure_workspace(mr, Nn, Kk)
    ms_n = timed(lambda: capi.fp8_blockwise_mm(A_q, A_s, Bq_r, Bs_r, Cn_q, Cn_s, Mm, nr, Kk), 10)
    ms_m = timed(lambda: capi.fp8_blockwise_mm(Aq_r, As_r, B_q, B_s, Cm_q, Cm_s, mr, Nn, Kk), 10)
    ms_n_g = timed(lambda: (capi.fp8_blockwise_mm(A_q, A_s, Bq_r, Bs_r, Cn_q, Cn_s, Mm, nr, Kk),
                            shard.all_gather_c_n(Cn_q, Cn_s, Nn)), 5)
    ms_m_g = timed(lambda: (capi.fp8_blockwise_mm(Aq_r, As_r, B_q, B_s, Cm_q, Cm_s, mr, Nn, Kk),
                            shard.all_gather_c_m(Cm_q, Cm_s, Mm)), 5)
    flops = 2.0 * Mm * Nn * Kk
    groups = [(shard.split_n(Nn, world, r)[1] - shard.split_n(Nn, world, r)[0]) // 128 for r in range(world)]
    res["down"] = {"shape": "M=8192 N=3584 K=18944", "ranks": world, "n_split_groups_per_rank": groups,
                   "ms_gemm_n_split": ms_n, "tflops_total_n_split": flops / (ms_n * 1e-3) / 1e12,
                   "ms_gemm_m_split": ms_m, "tflops_total_m_split": flops / (ms_m * 1e-3) / 1e12,
                   "ms_n_split_plus_allgather": ms_n_g, "ms_m_split_plus_allgather": ms_m_g,
                   "faster_split": "M" if ms_m < ms_n else "N"}
    return res


if __name__ == "__main__":
    sys.exit(main())
