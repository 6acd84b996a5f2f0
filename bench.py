"""Benchmark of the FP8 hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

A "step" is one FP8 GEMM M=N=K=8192 (e4m3 operands from a seeded N(0,1) draw, y column-major,
fp32 accumulation, bf16 output).  With N GPUs the rows of x and out are split into N contiguous
blocks, one per rank, and y is replicated (no collective on the compute path): the problem is fixed
("strong" scaling) and `value` is 2*8192^3 flop divided by the slowest rank's time per step.  The K
timed steps run back to back inside one CUDA-event pair, on operands that rotate through several
copies so that no step finds its inputs in L2.  The same line carries attention B8 H32 S4096 D128
split by batch*head slices and, on more than one GPU, the optional replicated output (one NCCL
all-gather, checked and timed separately).

Printed (rank 0, one JSON line): the device-timed throughput (`value`), the same metric end to
end through the public API with host buffers (`e2e`), the roofline of the GEMM kernel, the CPU
baseline (the oracle timed on a bounded sample), clocks sampled during the timed region, and --
as additional objects measured in the same run -- FP8 attention (B4 H48 S1024 D64 and
B8 H32 S4096 D128) and the LLM-MLP GEMM shapes.

`--impl reference` times the reference's CPU path instead (the numpy restatement of Helion's
ref-eager arithmetic in oracle/, since the reference itself is Python that does not travel to the
benchmark machine) on a bounded row block of the same workload, on rank 0 only.
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
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

M = N = K = 8192
GEMM_FLOPS = 2.0 * M * N * K
NOMINAL_FP8_TFLOPS = 4500.0
NOMINAL_HBM_GBS = 8000.0
METRIC = "FP8 GEMM TFLOP/s (M=N=K=8192, e4m3 x e4m3, fp32 accumulate, bf16 out)"


def load_peaks():
    """Measured peaks of this pool (driver-written file) or the documented fallback."""
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only queries) in a
    background thread while the timed region runs."""

    def __init__(self, index: int, period_s: float = 0.002) -> None:
        self.index = index
        self.period_s = period_s
        self.samples = []
        self.reasons = set()
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None
        self.sm_max = None

    def start(self) -> None:
        try:
            import pynvml

            pynvml.nvmlInit()
            # honour CUDA_VISIBLE_DEVICES when it lists indices
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = self.index
            if visible:
                ids = [v.strip() for v in visible.split(",") if v.strip()]
                if self.index < len(ids) and ids[self.index].isdigit():
                    phys = int(ids[self.index])
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()

    def _run(self) -> None:
        nv = self._nvml
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4),
        }
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(
            nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        power = 0.0
        n = 0
        while not self._stop.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                if n % 4 == 0:  # a short timed region leaves room for few queries: the clock first, the rest less often
                    power = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                    mask = int(get_reasons(self._handle))
                    for name, bit in names.items():
                        if mask & bit:
                            self.reasons.add(name)
                self.samples.append((power, sm, time.perf_counter()))
                n += 1
            except Exception:
                pass
            if self.period_s >= 0.001:
                time.sleep(self.period_s)

    def stop(self, window=None) -> dict:
        """Ends the sampling.  `window` = (t0, t1) in time.perf_counter() seconds keeps only the samples taken inside
        it (the thread is started a little before the timed region so that it is surely running when that begins)."""
        if self._nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvml unavailable"], "samples": 0}
        self._stop.set()
        self._thread.join(timeout=2)
        where = "the whole sampling period"
        if window is not None:
            inside = [s for s in self.samples if window[0] <= s[2] <= window[1]]
            where = f"inside the timed region of {(window[1] - window[0]) * 1e3:.2f} ms"
            if not inside:  # a region shorter than one query: the nearest sample stands in, and the line says so
                inside = sorted(self.samples, key=lambda s: min(abs(s[2] - window[0]), abs(s[2] - window[1])))[:1]
                where = f"nearest to the timed region of {(window[1] - window[0]) * 1e3:.2f} ms (none fell inside)"
            self.samples = inside
        sm = [s[1] for s in self.samples]
        return {
            "samples_taken": where,
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_min_mhz": min(sm) if sm else None,
            "sm_max_mhz": self.sm_max,
            "power_w_max": max(s[0] for s in self.samples) if self.samples else None,
            "samples": len(sm),
            "reasons": sorted(self.reasons),
        }


def time_steps(fn, steps, warmup, flush, torch, stream=None):
    """Per-step CUDA-event times (ms) on the current stream; L2 is flushed before every step."""
    for _ in range(warmup):
        flush()
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(steps):
        flush()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return times


CPU_SAMPLE_ROWS = 128


def cpu_reference_inputs(rows: int):
    """The first `rows` rows of the benchmark's x and its full y, as e4m3 bit patterns."""
    from oracle import fp8_oracle as o

    x, y = o.gemm_inputs(M, N, K, seed=1)
    return o.torch_fp8_to_bits(x[:rows]), o.torch_fp8_to_bits(y)


def cpu_reference_pass(xb, yb):
    """One pass of the oracle's GEMM (dequantise, fp32 matmul, round to bf16); returns seconds."""
    import numpy as np

    from oracle import fp8_oracle as o

    t0 = time.perf_counter()
    out = o.fp8_gemm(xb, yb, "bf16")
    dt = time.perf_counter() - t0
    assert np.isfinite(out).all()
    return dt


def aten_scaled_mm_cpu_gflops():
    """The call the reference's ref-eager mode really makes on CPU tensors (ATen _scaled_mm,
    helion/language/matmul_ops.py:235-242), timed on a 256^3 problem."""
    import torch

    from oracle import fp8_oracle as o

    x, y = o.gemm_inputs(256, 256, 256, seed=0)
    one = torch.tensor(1.0)
    try:
        torch._scaled_mm(x, y, one, one, use_fast_accum=False, out_dtype=torch.float32)
        t0 = time.perf_counter()
        torch._scaled_mm(x, y, one, one, use_fast_accum=False, out_dtype=torch.float32)
        return 2.0 * 256 ** 3 / (time.perf_counter() - t0) / 1e9
    except Exception:  # not every torch build has the CPU kernel
        return None


def run_reference(args, rank: int, emit) -> None:
    if rank != 0:
        return
    import torch

    rows = CPU_SAMPLE_ROWS
    threads = torch.get_num_threads()
    xb, yb = cpu_reference_inputs(rows)
    for _ in range(args.warmup):
        cpu_reference_pass(xb, yb)
    times = [cpu_reference_pass(xb, yb) for _ in range(args.steps)]
    sec = statistics.mean(times)
    tflops = 2.0 * rows * N * K / sec / 1e12
    sample = f"rows 0..{rows - 1} of x against the full y ({rows}x{N}x{K}) per step"
    line = {
        "impl": "reference",
        "metric": METRIC,
        "value": tflops,
        "unit": "TFLOP/s",
        "n_gpus": args.gpus,
        "steps": args.steps,
        "warmup": args.warmup,
        "ms_per_step": sec * 1e3,
        "higher_is_better": True,
        "scaling": "strong",  # the same fixed 8192^3 product at every N; the CPU arm runs it on rank 0's host cores
        "vs_baseline": None,
        "dtype": "e4m3 x e4m3 -> fp32",
        "data": "synthetic",
        "config": {"workload": "fp8_gemm M=N=K=8192, y column-major, bf16 out (BASELINE config 2), rows of x and out split over the GPUs",
                   "global_M": M, "sample": sample},
        "cpu_baseline": {"value": tflops, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample,
                         "aten_scaled_mm_cpu_gflops_256": aten_scaled_mm_cpu_gflops()},
        "e2e": {"value": tflops, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true", help="skip the attention / MLP-shape sections")
    ap.add_argument("--only", default=None, help="time just one named workload and exit: " + ", ".join(WORKLOADS))
    ap.add_argument("--config", type=int, default=None, help="tile-config id for --only (default: table choice)")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    # Libraries (NCCL's version banner, for one) write to stdout; keep stdout for the one JSON line by
    # pointing file descriptor 1 at stderr until that line is printed.
    sys.stdout.flush()
    saved_stdout = os.dup(1)
    os.dup2(2, 1)

    def emit(obj) -> None:
        sys.stdout.flush()
        os.dup2(saved_stdout, 1)
        print(json.dumps(obj), flush=True)

    if args.impl == "reference":
        run_reference(args, rank, emit)
        return

    import torch
    import torch.distributed as dist

    import helion_b200 as hb
    from helion_b200 import _lib
    from oracle import fp8_oracle as o  # input generators + the CPU baseline leg only

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if args.only is not None:
        run_only(args, torch, dev, hb, _lib, emit)
        return
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    peaks = load_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops"]  # dense FP8 issues at twice the bf16 rate
    from helion_b200.sharding import shard_range, sharded_fp8_gemm

    # ---- workload: the fixed 8192^3 GEMM; this rank owns rows [lo, hi) of x and out, y is replicated ------
    x_full, y_host = o.gemm_inputs(M, N, K, seed=1)  # the same draw on every rank
    lo, hi = shard_range(M, world, rank)
    rows = hi - lo
    x_pin = x_full[lo:hi].contiguous().view(torch.uint8).pin_memory()
    y_pin = y_host.t().contiguous().view(torch.uint8).pin_memory()  # [N, K] bytes = column-major y
    out_pin = torch.empty(rows, N, dtype=torch.bfloat16).pin_memory()
    # REPLICAS copies of every operand, used in rotation: back-to-back steps never find their inputs in L2
    # (4 x (x shard + y + out shard) is 364 MB at 8 GPUs, 1.07 GB at one; L2 holds 126 MB)
    xs = [x_pin.to(dev, non_blocking=True).view(torch.float8_e4m3fn) for _ in range(REPLICAS)]
    ys = [y_pin.to(dev, non_blocking=True).view(torch.float8_e4m3fn).t() for _ in range(REPLICAS)]
    outs = [torch.empty(rows, N, dtype=torch.bfloat16, device=dev) for _ in range(REPLICAS)]
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)

    def flush():
        flush_buf.zero_()

    def step(i=0):
        r = i % REPLICAS
        hb.fp8_gemm(xs[r], ys[r], out_dtype=torch.bfloat16, out=outs[r])

    _lib.reset_status(local_rank)

    # ---- device-timed region: K steps back to back inside one event pair -----------------------------
    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank, period_s=0.0005)
    if rank == 0:
        sampler.start()
        time.sleep(0.02)  # the sampling thread is up and has made its first queries before the region starts
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ev_a = torch.cuda.Event(enable_timing=True)
    ev_b = torch.cuda.Event(enable_timing=True)
    t_region0 = time.perf_counter()
    ev_a.record()
    for i in range(args.steps):
        step(warmup + i)
    ev_b.record()
    torch.cuda.synchronize()
    t_region1 = time.perf_counter()
    if world > 1:
        dist.barrier()
    total_ms = ev_a.elapsed_time(ev_b)
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms_max = float(t.item())
    clocks = sampler.stop(window=(t_region0, t_region1)) if rank == 0 else None
    _lib.check_status(local_rank)
    ms_per_step = total_ms_max / args.steps
    value = GEMM_FLOPS / (ms_per_step * 1e-3) / 1e12  # the whole job: all ranks' rows of the one 8192^3 product
    kernel_ms = total_ms / args.steps  # one launch per step on this rank
    shard_flops = 2.0 * rows * N * K
    achieved = shard_flops / (kernel_ms * 1e-3) / 1e12
    # the same launch timed alone (L2 flushed by a 512 MiB write before it, one event pair per launch)
    iso = time_steps(step, 10, 0, flush, torch)
    isolated_ms = statistics.median(iso)
    # cuBLASLt (torch._scaled_mm, the reference's GPU baseline, examples/fp8_gemm.py:61-78) timed the same two
    # ways on the same operands, for the like-for-like fractions of the roofline object (one GPU only)
    cublas_b2b_ms = cublas_iso_ms = None
    if world == 1 and not args.no_extras:
        try:
            one = torch.tensor(1.0, device=dev)

            def cublas_step(i=0):
                r = i % REPLICAS
                torch._scaled_mm(xs[r], ys[r], one, one, use_fast_accum=False, out_dtype=torch.bfloat16)

            cublas_b2b_ms = timed_back_to_back(cublas_step, args.steps, warmup, torch, dist, dev, world)
            cublas_iso_ms = statistics.median(time_steps(cublas_step, 10, 0, flush, torch))
        except Exception:  # context only
            pass

    # ---- end to end: host buffers in, host buffer out, copies inside the timed region ----------
    # hb.HostGemm is the library's call for operands in host memory: every step uploads this rank's rows of x
    # and y from pinned memory and downloads its rows of out, on three streams so that the two PCIe
    # directions and the kernels overlap (row blocks within a step, double-buffered device copies across steps).
    pipe = hb.HostGemm(rows, N, K, out_dtype=torch.bfloat16, device=dev)

    def timed_e2e(fn, steps):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            last = fn()
        torch.cuda.current_stream().wait_event(last)  # the last download; earlier steps finish before it
        b.record()
        torch.cuda.synchronize()
        ms = torch.tensor([a.elapsed_time(b) / steps], dtype=torch.float64, device=dev)
        if world > 1:
            dist.barrier()
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    e2e_steps = min(args.steps, 20)
    e2e_ms = timed_e2e(lambda: pipe.submit(x_pin, y_pin, out_pin), e2e_steps)
    e2e_value = GEMM_FLOPS / (e2e_ms * 1e-3) / 1e12
    got = out_pin[:64].float().numpy().copy()
    # On several GPUs of one node every rank holds the same y in host memory: each uploads 1/world of it and one
    # NCCL all-gather over NVLink per step completes every GPU's copy, so the node moves y over PCIe once per step
    # instead of once per GPU (HostGemm(..., group=...)).  Same inputs in host memory, same result in host memory.
    e2e_every_rank = None
    if world > 1 and N % world == 0:
        e2e_every_rank = {"value": e2e_value, "ms_per_step": e2e_ms, "h2d_bytes_per_step": int(x_pin.numel() + y_pin.numel())}
        out_pin.zero_()
        shared = hb.HostGemm(rows, N, K, out_dtype=torch.bfloat16, device=dev, group=dist.group.WORLD)
        e2e_ms = timed_e2e(lambda: shared.submit(x_pin, y_pin, out_pin), e2e_steps)
        e2e_value = GEMM_FLOPS / (e2e_ms * 1e-3) / 1e12
        shared.close()
        got = out_pin[:64].float().numpy().copy()
    # y as a weight that stays on the device (uploaded once, outside the timed region): per step only this
    # rank's rows of x go up and its rows of out come back
    pipe.set_weight(y_pin)
    e2e_resident_ms = timed_e2e(lambda: pipe.submit(x_pin, None, out_pin), e2e_steps)
    pipe.synchronize()
    got_resident = out_pin[:64].float().numpy().copy()

    # ---- the other sharded BASELINE configuration and the optional replicated output (all ranks) ----
    sharded = None
    if not args.no_extras:
        sharded = sharded_sections(hb, torch, dist, dev, rank, world, xs[0], ys[0], outs[0], x_full, sharded_fp8_gemm)

    line = None
    if rank == 0:
        # sanity of the e2e results against the oracle on a row block (not timed)
        want = o.fp8_gemm(o.torch_fp8_to_bits(x_full[lo:lo + 64]), o.torch_fp8_to_bits(y_host), "bf16")
        import numpy as np

        np.testing.assert_allclose(got, want, rtol=2e-2, atol=2e-2)
        np.testing.assert_allclose(got_resident, want, rtol=2e-2, atol=2e-2)

        extras = {}
        if not args.no_extras and world == 1:
            extras = run_extras(hb, _lib, o, torch, dev, flush, fp8_peak, peaks)
            extras["sustained"] = sustained_section(hb, torch, dev, local_rank, xs, ys, outs, peaks)
        cpu_sec = cpu_tflops = None
        if world == 1:
            xb, yb = cpu_reference_inputs(CPU_SAMPLE_ROWS)
            cpu_sec = min(cpu_reference_pass(xb, yb) for _ in range(5))
            cpu_tflops = 2.0 * CPU_SAMPLE_ROWS * N * K / cpu_sec / 1e12
        line = {
            "metric": METRIC,
            "value": value,
            "unit": "TFLOP/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": warmup,
            "ms_per_step": ms_per_step,
            "higher_is_better": True,
            "scaling": "strong",
            "vs_baseline": None,
            "dtype": "e4m3 x e4m3 -> fp32",
            "data": "synthetic",
            "config": {
                "workload": "fp8_gemm M=N=K=8192, y column-major, bf16 out (BASELINE config 2), rows of x and out split over the GPUs",
                "global_M": M,
                "rows_per_rank": rows,
                "sharding": "contiguous row blocks of x / out per rank, y replicated, no collective on the compute path",
                "l2": f"steps run back to back; every operand exists {REPLICAS} times and the steps rotate through the copies "
                      f"({REPLICAS * (rows * K + N * K + 2 * rows * N) >> 20} MiB per rank), so no step finds its inputs in the 126 MB L2",
                "timing": "one CUDA-event pair around the K steps on the launching stream, max over ranks",
                "tile_config": _lib.describe_config(_lib.OP_GEMM, _lib.load().hb200_fp8_gemm_select_config(rows, N, K, 1, 1)),
            },
            "gpu_launches": args.steps * world,
            "gpu_launches_per_rank": args.steps,
            "clocks": clocks,
            "e2e": {
                "value": e2e_value,
                "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(x_pin.numel() + (y_pin.numel() // world if e2e_every_rank is not None else y_pin.numel())),
                "d2h_bytes_per_step": int(out_pin.numel() * 2),
                "bytes_are": "per rank" + ("" if e2e_every_rank is None else
                                           "; every rank uploads 1/world of y and one NCCL all-gather over NVLink per step "
                                           "completes it on every GPU (HostGemm(group=...))"),
                "steps": e2e_steps,
                "ms_per_step": e2e_ms,
                **({} if e2e_every_rank is None else {"y_uploaded_by_every_rank": e2e_every_rank}),
            },
            "e2e_weight_resident": {
                "value": GEMM_FLOPS / (e2e_resident_ms * 1e-3) / 1e12,
                "unit": "TFLOP/s",
                "h2d_bytes_per_step": int(x_pin.numel()),
                "d2h_bytes_per_step": int(out_pin.numel() * 2),
                "bytes_are": "per rank; y uploaded once before the timed region (HostGemm.set_weight)",
                "ms_per_step": e2e_resident_ms,
            },
            "roofline": {
                "bound": "tensor",
                "achieved": achieved,
                "peak": fp8_peak,
                "unit": "TFLOP/s",
                "frac": achieved / fp8_peak,
                "peak_source": f"2 x bf16_tflops ({peaks['bf16_tflops']}) of {peaks['source']}; dense FP8 issues at twice the bf16 rate "
                               "(the file holds no FP8 figure)",
                "frac_of_2x_bf16_sustained": achieved / (2.0 * peaks["bf16_tflops_sustained"]),
                "frac_of_cublaslt_fp8_same_run": (cublas_b2b_ms / kernel_ms) if cublas_b2b_ms else None,
                "cublaslt_back_to_back_ms": cublas_b2b_ms,
                "cublaslt_isolated_launch_ms": cublas_iso_ms,
                "isolated_frac_of_cublaslt": (cublas_iso_ms / isolated_ms) if cublas_iso_ms else None,
                "frac_of_nominal_4500": achieved / NOMINAL_FP8_TFLOPS,
                "algorithmic_flops_per_launch": shard_flops,
                "kernel_ms": kernel_ms,
                "isolated_launch_ms": isolated_ms,
                "isolated_launch_tflops": shard_flops / (isolated_ms * 1e-3) / 1e12,
                "traffic": TRAFFIC_BYTES_PER_LAUNCH if world == 1 else None,
                "traffic_source": TRAFFIC_SOURCE if world == 1 else "not captured for a row shard",
                "algorithmic_bytes_per_launch": rows * K + K * N + 2 * rows * N,
            },
        }
        if extras.get("attention"):
            # the other kernels of the metric, beside the dominant one: attention against nominal FP8 and against the
            # softmax-only ceiling measured in this run, the few-row GEMM against the measured HBM bandwidth
            line["roofline"]["other_kernels"] = {
                **{name: {k: v.get(k) for k in ("ms", "tflops", "frac_of_nominal_4500", "frac_of_measured_fp8_peak",
                                                "softmax_ceiling_ms", "frac_of_softmax_ceiling")}
                   for name, v in extras["attention"].items()},
                **{f"mlp_{m}": {k: v.get(k) for k in ("ms", "tflops", "hbm_gbs", "frac_of_measured_hbm", "frac_of_measured_fp8_peak")}
                   for m, v in extras.get("mlp_K4096_N14336", {}).items()},
            }
        if world == 1:
            line["cpu_baseline"] = {
                "value": cpu_tflops,
                "unit": "TFLOP/s",
                "cores": torch.get_num_threads(),
                "kind": "port",
                "sample": f"rows 0..{CPU_SAMPLE_ROWS - 1} of x against the full y ({CPU_SAMPLE_ROWS}x{N}x{K}), best of 5, {cpu_sec:.2f} s per pass",
                "aten_scaled_mm_cpu_gflops_256": aten_scaled_mm_cpu_gflops(),
            }
        line.update(extras)
        if sharded is not None:
            line.update(sharded)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        emit(line)


REPLICAS = 4


def timed_back_to_back(fn, steps, warmup, torch, dist, dev, world):
    """`steps` calls of fn(i) inside one event pair after `warmup` calls; returns ms per step, max over ranks."""
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a = torch.cuda.Event(enable_timing=True)
    b = torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(steps):
        fn(warmup + i)
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b) / steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sharded_sections(hb, torch, dist, dev, rank, world, x_shard, y, out_shard, x_full, sharded_fp8_gemm) -> dict:
    """Measured on all ranks in the same run: attention B8 H32 S4096 D128 split by batch*head slices (no
    collective; time = max over ranks, value = global FLOPs / that time), and -- with more than one rank --
    the optional replicated output of the row-sharded GEMM: one NCCL all-gather of the row blocks, checked bit
    for bit against rank 0's own unsharded product and timed on its own."""
    from helion_b200.sharding import shard_range

    res = {}
    b, h, s, d = ATTN_SHAPES["attn_B8_H32_S4096_D128"]
    b0, b1 = shard_range(b * h, world, rank)
    nbh = b1 - b0
    g = torch.Generator(device=dev).manual_seed(4)
    qs, ks, vs, os_ = [], [], [], []
    for _ in range(2):  # two copies in rotation: 2 x 4 x nbh x S x D bytes is at least 134 MB at 8 GPUs
        qs.append(torch.randn(nbh, s, d, device=dev, generator=g).to(torch.float8_e4m3fn))
        ks.append(torch.randn(nbh, s, d, device=dev, generator=g).to(torch.float8_e4m3fn))
        vs.append(torch.randn(nbh, s, d, device=dev, generator=g).to(torch.float8_e4m3fn).permute(0, 2, 1))
        os_.append(torch.empty(nbh, s, d, dtype=torch.float8_e4m3fn, device=dev))
    ms = timed_back_to_back(lambda i: hb.attention_into(qs[i % 2], ks[i % 2], vs[i % 2], os_[i % 2]), 10, 3, torch, dist, dev,
                            world)
    res["attention_B8_H32_S4096_D128_bh_sharded"] = {
        "ms": ms, "tflops": 4.0 * b * h * s * s * d / (ms * 1e-3) / 1e12, "slices_per_rank": nbh,
        "frac_of_nominal_4500_per_gpu": 4.0 * b * h * s * s * d / (ms * 1e-3) / 1e12 / world / NOMINAL_FP8_TFLOPS,
        "scaling": "strong", "collective": "none"}
    del qs, ks, vs, os_
    if world == 1:
        return res

    # ---- replicated output: every rank ends up with the whole [8192, 8192] bf16 product ----------------
    xd = x_full.to(dev)
    full = sharded_fp8_gemm(xd, y, rank=rank, world_size=world, out_dtype=torch.bfloat16, replicate_output=True)
    torch.cuda.synchronize()
    match = None
    if rank == 0:
        own = hb.fp8_gemm(xd, y, out_dtype=torch.bfloat16)  # the unsharded product on this GPU
        match = bool(torch.equal(full, own))
        del own
    gathered = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
    local = out_shard.contiguous()

    def gather(_i):
        dist.all_gather_into_tensor(gathered, local)

    ag_ms = timed_back_to_back(gather, 10, 3, torch, dist, dev, world)
    recv_bytes = (world - 1) * local.numel() * 2
    res["replicated_output"] = {
        "match": match,
        "checked": "rank 0: all-gathered [8192, 8192] bf16 equals its own unsharded hb.fp8_gemm result bit for bit",
        "allgather_ms": ag_ms,
        "allgather_gbs_in_per_gpu": recv_bytes / (ag_ms * 1e-3) / 1e9,
        "bytes_received_per_gpu": recv_bytes,
        "collective": "NCCL all_gather_into_tensor over NVLink, off the compute path, timed separately (10 calls, max over ranks)",
    }
    return res


def sustained_section(hb, torch, dev, index, xs, ys, outs, peaks, seconds: float = 2.0) -> dict:
    """The 8192^3 GEMM launched back to back for `seconds` without a host synchronisation or an L2 flush in
    between (operands rotate through their copies), clocks sampled under load; cuBLASLt (torch._scaled_mm, the
    reference's GPU baseline, examples/fp8_gemm.py:61-78) run the same way right after."""
    one = torch.tensor(1.0, device=dev)

    def ours(i):
        r = i % REPLICAS
        hb.fp8_gemm(xs[r], ys[r], out_dtype=torch.bfloat16, out=outs[r])

    def cublas(i):
        r = i % REPLICAS
        torch._scaled_mm(xs[r], ys[r], one, one, use_fast_accum=False, out_dtype=torch.bfloat16)

    def run(fn):
        for i in range(5):
            fn(i)
        torch.cuda.synchronize()
        launches = max(20, int(seconds / 0.35e-3))
        sampler = ClockSampler(index, period_s=0.01)
        sampler.start()
        a = torch.cuda.Event(enable_timing=True)
        b = torch.cuda.Event(enable_timing=True)
        a.record()
        for i in range(launches):
            fn(i)
        b.record()
        torch.cuda.synchronize()
        clocks = sampler.stop()
        ms = a.elapsed_time(b) / launches
        tf = GEMM_FLOPS / (ms * 1e-3) / 1e12
        out = {"launches": launches, "ms_per_launch": ms, "tflops": tf, "clocks": clocks,
               "frac_of_2x_bf16_sustained": tf / (2.0 * peaks["bf16_tflops_sustained"]),
               "frac_of_nominal_4500": tf / NOMINAL_FP8_TFLOPS}
        if clocks.get("sm_mhz"):
            out["ms_times_median_sm_mhz"] = ms * clocks["sm_mhz"]
        return out

    res = {"ours": run(ours)}
    try:
        res["cublaslt"] = run(cublas)
        res["ours_over_cublaslt"] = res["ours"]["tflops"] / res["cublaslt"]["tflops"]
    except Exception as ex:  # context only
        res["cublaslt"] = {"error": str(ex)[:120]}
    return res


# DRAM traffic of one 8192^3 launch: dram__bytes_read.sum (331.8 MB) + dram__bytes_write.sum (115.8 MB) of the
# 512x256-tile kernel from one `ncu --set full` capture of `bench.py --only gemm_8192`.  A constant of that
# capture, not something this run measures: it moves only when the tile shape or the epilogue changes.
TRAFFIC_BYTES_PER_LAUNCH = 448_057_344  # 331,254,016 read + 116,803,328 written
TRAFFIC_SOURCE = "ncu capture of one launch of this kernel (not measured by this run)"


ATTN_SHAPES = {"attn_B4_H48_S1024_D64": (4, 48, 1024, 64), "attn_B8_H32_S4096_D128": (8, 32, 4096, 128)}
MLP_M = (16, 128, 2048, 16384)
MLP_K, MLP_N = 4096, 14336


def make_workload(name: str, torch, dev, hb, config=None):
    """Build one named workload on the device: returns (launch fn, flops, algorithmic bytes)."""
    if name == "gemm_8192":
        g = torch.Generator(device=dev).manual_seed(1)
        xa = torch.randn(M, K, device=dev, generator=g).to(torch.float8_e4m3fn)
        ya = torch.randn(N, K, device=dev, generator=g).to(torch.float8_e4m3fn).t()
        outg = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        return (lambda: hb.fp8_gemm(xa, ya, out_dtype=torch.bfloat16, out=outg, config=config),
                GEMM_FLOPS, M * K + K * N + 2 * M * N)
    if name.startswith("gemm_shard_"):  # one rank's rows of the 8192^3 product: gemm_shard_1024 / _2048 / _4096
        rows = int(name[len("gemm_shard_"):])
        g = torch.Generator(device=dev).manual_seed(1)
        xa = torch.randn(rows, K, device=dev, generator=g).to(torch.float8_e4m3fn)
        ya = torch.randn(N, K, device=dev, generator=g).to(torch.float8_e4m3fn).t()
        outg = torch.empty(rows, N, dtype=torch.bfloat16, device=dev)
        return (lambda: hb.fp8_gemm(xa, ya, out_dtype=torch.bfloat16, out=outg, config=config),
                2.0 * rows * N * K, rows * K + K * N + 2 * rows * N)
    if name == "cublaslt_8192":  # context only: torch._scaled_mm on the same workload
        g = torch.Generator(device=dev).manual_seed(1)
        xa = torch.randn(M, K, device=dev, generator=g).to(torch.float8_e4m3fn)
        ya = torch.randn(N, K, device=dev, generator=g).to(torch.float8_e4m3fn).t()
        one = torch.tensor(1.0, device=dev)
        return (lambda: torch._scaled_mm(xa, ya, one, one, use_fast_accum=False, out_dtype=torch.bfloat16),
                GEMM_FLOPS, M * K + K * N + 2 * M * N)
    if name in ATTN_SHAPES or name.startswith("attn_causal_"):
        causal = name.startswith("attn_causal_")
        b, h, s, d = ATTN_SHAPES["attn_" + name[len("attn_causal_"):]] if causal else ATTN_SHAPES[name]
        g = torch.Generator(device=dev).manual_seed(3)
        q = torch.randn(b * h, s, d, device=dev, generator=g).to(torch.float8_e4m3fn)
        k = torch.randn(b * h, s, d, device=dev, generator=g).to(torch.float8_e4m3fn)
        v = torch.randn(b * h, s, d, device=dev, generator=g).to(torch.float8_e4m3fn).permute(0, 2, 1)
        outa = torch.empty(b, h, s, d, dtype=torch.float8_e4m3fn, device=dev)
        # with the mask a query row i multiplies against i + 1 keys: (S^2 + S) / 2 pairs instead of S^2
        pairs = (s * s + s) / 2 if causal else s * s
        return (lambda: hb.fp8_attention(q, k, v, b, h, out=outa, config=config, causal=causal),
                4.0 * b * h * pairs * d, 4 * b * h * s * d)
    if name.startswith("mlp_M"):
        m = int(name[5:])
        g = torch.Generator(device=dev).manual_seed(2)
        xa = torch.randn(m, MLP_K, device=dev, generator=g).to(torch.float8_e4m3fn)
        w = torch.randn(MLP_N, MLP_K, device=dev, generator=g) * 0.02
        w = (w * (448.0 / w.abs().max())).to(torch.float8_e4m3fn).t()
        outm = torch.empty(m, MLP_N, dtype=torch.bfloat16, device=dev)
        return (lambda: hb.fp8_gemm(xa, w, out_dtype=torch.bfloat16, out=outm, config=config),
                2.0 * m * MLP_N * MLP_K, m * MLP_K + MLP_K * MLP_N + 2 * m * MLP_N)
    if name == "gemm_8192_rowwise_scaled":  # hb200_fp8_gemm_scaled: one scale per row of x and per column of y
        g = torch.Generator(device=dev).manual_seed(1)
        xa = torch.randn(M, K, device=dev, generator=g).to(torch.float8_e4m3fn)
        ya = torch.randn(N, K, device=dev, generator=g).to(torch.float8_e4m3fn).t()
        sa = torch.rand(M, 1, device=dev, generator=g) + 0.5
        sb = torch.rand(1, N, device=dev, generator=g) + 0.5
        outg = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        return (lambda: hb.fp8_gemm(xa, ya, out_dtype=torch.bfloat16, out=outg, config=config, scale_a=sa, scale_b=sb),
                GEMM_FLOPS, M * K + K * N + 2 * M * N + 4 * (M + N))
    if name.startswith("attn_bf16_") or name.startswith("sdpa_bf16_"):  # the 16-bit sibling (examples/attention.py); torch SDPA for context
        b, h, s, d = ATTN_SHAPES["attn_" + name[len("attn_bf16_"):]]
        g = torch.Generator(device=dev).manual_seed(6)
        q, k, v = (torch.randn(b, h, s, d, device=dev, generator=g).to(torch.bfloat16) for _ in range(3))
        fn = (lambda: hb.attention(q, k, v)) if name.startswith("attn_") else (
            lambda: torch.nn.functional.scaled_dot_product_attention(q, k, v))
        return fn, 4.0 * b * h * s * s * d, 2 * 4 * b * h * s * d
    if name == "matmul_bf16_8192":  # hb200_gemm_16bit: the reference's examples/matmul.py shape class, row-major y
        g = torch.Generator(device=dev).manual_seed(5)
        xa = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
        ya = torch.randn(K, N, device=dev, generator=g).to(torch.bfloat16)
        bias = torch.randn(N, device=dev, generator=g).to(torch.bfloat16)
        outg = torch.empty(M, N, dtype=torch.bfloat16, device=dev)
        return (lambda: hb.matmul(xa, ya, bias=bias, relu=True, out=outg, config=config),
                GEMM_FLOPS, 2 * (M * K + K * N + M * N) + 2 * N)
    if name.startswith("preprocess_"):  # q, k, v fp16 -> e4m3 in one launch (hb200_fp8_attention_preprocess)
        b, h, s, d = ATTN_SHAPES["attn_" + name[len("preprocess_"):]]
        g = torch.Generator(device=dev).manual_seed(4)
        q, k, v = (torch.randn(b, h, s, d, device=dev, generator=g, dtype=torch.float16) for _ in range(3))
        return (lambda: hb.preprocess_fp8_attention_inputs(q, k, v), 0.0, 3 * b * h * s * d * (2 + 1))
    raise SystemExit(f"unknown workload {name!r}")


PREPROCESS = [f"preprocess_{n[len('attn_'):]}" for n in ATTN_SHAPES]
ATTN16 = [f"attn_bf16_{n[len('attn_'):]}" for n in ATTN_SHAPES]
SDPA16 = [f"sdpa_bf16_{n[len('attn_'):]}" for n in ATTN_SHAPES]
CAUSAL = [f"attn_causal_{n[len('attn_'):]}" for n in ATTN_SHAPES]
WORKLOADS = ["gemm_8192", "gemm_shard_1024", "gemm_shard_2048", "gemm_shard_4096", *ATTN_SHAPES, *CAUSAL, *ATTN16, *SDPA16, *(f"mlp_M{m}" for m in MLP_M), "cublaslt_8192", "gemm_8192_rowwise_scaled",
             "matmul_bf16_8192", *PREPROCESS]


def run_only(args, torch, dev, hb, _lib, emit) -> None:
    """`--only NAME`: time one named workload (used for sweeps and as the command under ncu)."""
    fn, flops, byts = make_workload(args.only, torch, dev, hb, args.config)
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    ts = time_steps(fn, args.steps, max(args.warmup, 3), flush_buf.zero_, torch)
    torch.cuda.synchronize()
    _lib.check_status(dev.index)
    med = statistics.median(ts)
    emit({"only": args.only, "config": args.config, "steps": args.steps, "ms": med, "ms_min": min(ts),
          "tflops": flops / (med * 1e-3) / 1e12, "gbs": byts / (med * 1e-3) / 1e9})


def decode_graph(hb, torch, dev, m: int, timed, peaks, layers: int = 32) -> dict:
    """`layers` MLP GEMMs ([m, 4096] x [4096, 14336], one weight each) captured in one CUDA graph."""
    g = torch.Generator(device=dev).manual_seed(2)
    xa = torch.randn(m, MLP_K, device=dev, generator=g).to(torch.float8_e4m3fn)
    ws = []
    for _ in range(layers):
        w = torch.randn(MLP_N, MLP_K, device=dev, generator=g) * 0.02
        ws.append((w * (448.0 / w.abs().max())).to(torch.float8_e4m3fn).t())
    outm = torch.empty(m, MLP_N, dtype=torch.bfloat16, device=dev)

    def graph_of(config):
        def loop():
            for w in ws:
                hb.fp8_gemm(xa, w, out_dtype=torch.bfloat16, out=outm, config=config)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            loop()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loop()
        return timed(graph.replay, steps=10)

    med, mn = graph_of(None)
    byts = m * MLP_K + MLP_K * MLP_N + 2 * m * MLP_N
    gbs = layers * byts / (med * 1e-3) / 1e9
    res = {"layers": layers, "us_per_layer": med * 1e3 / layers, "us_per_layer_min": mn * 1e3 / layers,
           "tflops": layers * 2.0 * m * MLP_N * MLP_K / (med * 1e-3) / 1e12, "hbm_gbs": gbs,
           "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}
    if m <= 64:
        # table row 23: the caller states that y is a weight no kernel of the chain writes, so each launch asks
        # for its first stages of y while its predecessor still runs
        med23, _ = graph_of(23)
        res["us_per_layer_weights_static_row23"] = med23 * 1e3 / layers
    try:  # context: cuBLASLt in the same graph
        one = torch.ones((), device=dev)

        def lt_loop():
            for w in ws:
                torch._scaled_mm(xa, w, one, one, out_dtype=torch.bfloat16, out=outm)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            lt_loop()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            lt_loop()
        res["cublaslt_us_per_layer"] = timed(graph.replay, steps=10)[0] * 1e3 / layers
    except Exception as ex:
        res["cublaslt_error"] = str(ex)[:100]
    return res


def run_extras(hb, _lib, o, torch, dev, flush, fp8_peak, peaks) -> dict:
    """Other benchmark configurations, measured in the same run (20 timed launches each)."""
    res = {}

    def timed(fn, steps=20):
        ts = time_steps(fn, steps, 3, flush, torch)
        return statistics.median(ts), min(ts)

    def entry(name):
        fn, flops, byts = make_workload(name, torch, dev, hb)
        med, mn = timed(fn)
        tf = flops / (med * 1e-3) / 1e12
        gbs = byts / (med * 1e-3) / 1e9
        return {"ms": med, "ms_min": mn, "tflops": tf, "hbm_gbs": gbs, "frac_of_measured_fp8_peak": tf / fp8_peak,
                "frac_of_nominal_4500": tf / NOMINAL_FP8_TFLOPS, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"]}

    res["attention"] = {name: entry(name) for name in ATTN_SHAPES}
    # The attention kernels' own roofline, measured in this run: the softmax-only kernel (the per-score work of the
    # reference's loop with two warpgroups per SM and nothing else) gives the time one 128x128 step cannot beat;
    # a shape's steps spread evenly over the SMs times that is the shortest kernel any pipeline could reach.
    try:
        from helion_b200 import ceiling

        row = ceiling.measure(steps=1000, device=dev.index or 0, only=[2])[0]
        n_sms = _lib.load().hb200_num_sms(dev.index or 0)
        for name, (b, h, s_len, d) in ATTN_SHAPES.items():
            steps = b * h * (s_len // 128) * (s_len // 128)
            ceiling_ms = steps / n_sms * row["ns_per_step_per_sm"] * 1e-6
            res["attention"][name]["softmax_ceiling_ms"] = ceiling_ms
            res["attention"][name]["frac_of_softmax_ceiling"] = ceiling_ms / res["attention"][name]["ms"]
        res["attention_softmax_ceiling"] = {"cycles_per_128x128_step_per_sm": row["cycles_per_step_per_sm"],
                                            "ns_per_128x128_step_per_sm": row["ns_per_step_per_sm"],
                                            "how": "helion_b200.ceiling, two softmax warpgroups per SM, all exp2 on MUFU, 1000 steps"}
    except Exception as ex:  # context only
        res["attention_softmax_ceiling"] = {"error": str(ex)[:120]}
    res["attention_causal"] = {name: entry(name) for name in CAUSAL}  # FLOPs counted under the mask only
    res["mlp_K4096_N14336"] = {f"M{m}": entry(f"mlp_M{m}") for m in MLP_M}
    # the callers either side of the two kernels: scaled GEMM epilogue, attention input preparation
    res["gemm_8192_rowwise_scaled"] = entry("gemm_8192_rowwise_scaled")
    e = entry("matmul_bf16_8192")  # bf16 operands: fractions are of the measured / nominal bf16 peak, not FP8
    res["matmul_bf16_8192_bias_relu"] = {"ms": e["ms"], "ms_min": e["ms_min"], "tflops": e["tflops"],
                                         "frac_of_measured_bf16_peak": e["tflops"] / peaks["bf16_tflops"],
                                         "frac_of_nominal_2250": e["tflops"] / 2250.0}
    res["attention_bf16"] = {}
    for name, ctx_name in zip(ATTN16, SDPA16):
        e = entry(name)
        item = {"ms": e["ms"], "tflops": e["tflops"], "frac_of_measured_bf16_peak": e["tflops"] / peaks["bf16_tflops"]}
        try:  # context only: torch's scaled_dot_product_attention on the same tensors
            item["torch_sdpa_ms"] = entry(ctx_name)["ms"]
        except Exception as ex:
            item["torch_sdpa_error"] = str(ex)[:100]
        res["attention_bf16"][name] = item
    res["attention_preprocess_fp16"] = {}
    for name in PREPROCESS:
        e = entry(name)
        res["attention_preprocess_fp16"][name] = {"ms": e["ms"], "hbm_gbs": e["hbm_gbs"],
                                                  "frac_of_measured_hbm": e["frac_of_measured_hbm"]}

    # The few-row MLP shapes as a decode loop sees them: 32 layers (32 different weights, 1.9 GB: nothing
    # stays in L2) launched back to back from one CUDA graph, so neither launch latency nor the event
    # pair around a single 20 us kernel is in the number.
    res["mlp_decode_graph_32_layers"] = {}
    for m in (16, 128):
        try:
            res["mlp_decode_graph_32_layers"][f"M{m}"] = decode_graph(hb, torch, dev, m, timed, peaks)
        except Exception as ex:  # context only
            res["mlp_decode_graph_32_layers"][f"M{m}"] = {"error": str(ex)[:120]}

    # cuBLASLt on the same workload, for context (the reference's GPU baseline, examples/fp8_gemm.py:61-78)
    try:
        x, y = o.gemm_inputs(M, N, K, seed=1)
        xd = x.to(dev)
        yd = y.t().contiguous().to(dev).t()
        one = torch.tensor(1.0, device=dev)
        med, mn = timed(lambda: torch._scaled_mm(xd, yd, one, one, use_fast_accum=False, out_dtype=torch.bfloat16))
        res["cublaslt_scaled_mm_8192"] = {"ms": med, "tflops": GEMM_FLOPS / (med * 1e-3) / 1e12}
    except Exception as e:  # context only
        res["cublaslt_scaled_mm_8192"] = {"error": str(e)[:120]}
    return res


if __name__ == "__main__":
    main()
