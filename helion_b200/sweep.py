"""Times every row of the tile-config tables on a set of problem shapes.

This is the measured sweep the table-choice functions of the library (``hb200_fp8_gemm_select_config``
and the attention default) are checked against: it replaces the reference's autotuner search
(helion/autotuner/, run per kernel and shape at first call) by numbers taken once, offline.

    python -m helion_b200.sweep                    # GEMM and attention, the default shape lists
    python -m helion_b200.sweep --op gemm --shape 4096,4096,4096 --shape 2048,14336,4096
    python -m helion_b200.sweep --op attention --shape 8,32,4096,128 --causal
    python -m helion_b200.sweep --library          # adds torch._scaled_mm (cuBLASLt) as a context column
    python -m helion_b200.sweep --op gemm --back-to-back 20 --library   # 20 launches per event pair, rows interleaved

For every shape it prints one markdown table row: the time of each table row that accepts the shape,
the row the library picks by itself (``cfg_id = -1``) and how far that pick is from the best row.
Timing: CUDA events, median of ``--iters`` launches, the L2 flushed before each by writing a buffer
larger than it.  With ``--back-to-back N`` (GEMM) a cell is the median over ``--iters`` rounds of N launches
inside one event pair, operands rotating through four copies, the rows taking turns inside every round so
that clock and power drift hits them alike: the regime of a kernel inside a long step, at the power cap,
which is what the constants of the CTA-pair rows in ``hb200_fp8_gemm_select_config`` are fitted to.
"""
from __future__ import annotations

import argparse
import statistics
import sys
from typing import Callable, List, Optional, Sequence, Tuple

import torch

from . import _lib, ops

#: M, N, K with y column-major and bf16 output: the benchmark shapes (cubes, the K=4096 / N=14336 MLP
#: sweep over M), the per-GPU shards of the 8192 cube on 2 / 4 / 8 GPUs, and a few in between.
GEMM_SHAPES: List[Tuple[int, int, int]] = [
    (256, 256, 256), (1024, 1024, 1024), (2048, 2048, 2048), (4096, 4096, 4096), (8192, 8192, 8192),
    (4096, 8192, 8192), (2048, 8192, 8192), (1024, 8192, 8192),
    (16, 14336, 4096), (64, 14336, 4096), (128, 14336, 4096), (512, 14336, 4096), (2048, 14336, 4096),
    (16384, 14336, 4096), (2048, 4096, 14336), (8192, 1024, 8192),
]
#: batch, heads, seq, head_dim
ATTN_SHAPES: List[Tuple[int, int, int, int]] = [
    (4, 48, 1024, 64), (8, 32, 4096, 128), (8, 32, 4096, 64), (4, 48, 1024, 128), (1, 32, 16384, 128), (16, 16, 512, 64),
]


def _median_us(fn: Callable[[], object], iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    times = []
    for _ in range(iters):
        flush.zero_()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        fn()
        end.record()
        end.synchronize()
        times.append(start.elapsed_time(end) * 1e3)
    return statistics.median(times)


def _row_times(run: Callable[[Optional[int]], object], n_rows: int, iters: int, flush: torch.Tensor):
    """Time of every table row that accepts the problem (None where the library refuses it)."""
    times: List[Optional[float]] = []
    for row in range(n_rows):
        try:
            run(row)
            torch.cuda.synchronize()
        except (ValueError, TypeError, RuntimeError):
            times.append(None)
            continue
        times.append(_median_us(lambda: run(row), iters, flush))
    return times


def _row_times_back_to_back(runs: Sequence[Callable[[int], object]], launches: int, iters: int) -> List[Optional[float]]:
    """Median us per launch of each callable (None where it refuses): ``launches`` per event pair, callables interleaved."""
    alive: List[bool] = []
    for run in runs:
        try:
            for i in range(3):
                run(i)
            torch.cuda.synchronize()
            alive.append(True)
        except (ValueError, TypeError, RuntimeError):
            alive.append(False)
    samples: List[List[float]] = [[] for _ in runs]
    for _ in range(iters):
        for idx, run in enumerate(runs):
            if not alive[idx]:
                continue
            run(0)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for i in range(launches):
                run(i + 1)
            end.record()
            end.synchronize()
            samples[idx].append(start.elapsed_time(end) * 1e3 / launches)
    return [statistics.median(v) if v else None for v in samples]


def _format(label: str, times: Sequence[Optional[float]], auto_us: float, auto_row: Optional[int], extra: str) -> str:
    best_row = min((r for r, t in enumerate(times) if t is not None), key=lambda r: times[r])
    cells = " | ".join("—" if t is None else f"{t:.1f}" for t in times)
    picked = "auto" if auto_row is None else str(auto_row)
    return (f"| {label} | {cells} | {picked}: {auto_us:.1f} | {best_row}: {times[best_row]:.1f} | "
            f"{auto_us / times[best_row]:.2f}{extra} |")


def sweep_gemm(shapes, iters: int, library: bool, dev: torch.device, flush: torch.Tensor, back_to_back: int = 0) -> None:
    lib = _lib.load()
    n_rows = _lib.num_configs(_lib.OP_GEMM)
    if back_to_back:
        print(f"\nFP8 GEMM, y column-major, bf16 out; µs per launch, {back_to_back} launches back to back per event pair "
              f"(operands rotate through 4 copies, rows interleaved), median of {iters} rounds\n")
    else:
        print(f"\nFP8 GEMM, y column-major, bf16 out; µs per launch, cold L2, median of {iters}\n")
    head = " | ".join(str(r) for r in range(n_rows))
    print(f"| M×N×K | {head} | picked | best | picked / best{' | cuBLASLt' if library else ''} |")
    print("|" + "---|" * (n_rows + 4 + int(library)))
    for m, n, k in shapes:
        if back_to_back:
            copies = 4
            xs = [torch.randn(m, k, device=dev).to(torch.float8_e4m3fn) for _ in range(copies)]
            ys = [torch.randn(n, k, device=dev).to(torch.float8_e4m3fn).t() for _ in range(copies)]
            outs = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for _ in range(copies)]
            one = torch.ones((), device=dev)

            def make(row: Optional[int]):
                return lambda i: ops.fp8_gemm(xs[i % copies], ys[i % copies], out_dtype=torch.bfloat16, config=row, out=outs[i % copies])

            runs = [make(row) for row in range(n_rows)] + [make(None)]
            if library:
                runs.append(lambda i: torch._scaled_mm(xs[i % copies], ys[i % copies], one, one, out_dtype=torch.bfloat16))
            res = _row_times_back_to_back(runs, back_to_back, iters)
            auto_row = lib.hb200_fp8_gemm_select_config(m, n, k, 1, 0)
            extra = f" | {res[n_rows + 1]:.1f}" if library else ""
            print(_format(f"{m}×{n}×{k}", res[:n_rows], res[n_rows], auto_row, extra), flush=True)
            _lib.check_status(dev.index or 0)
            del xs, ys, outs
            continue
        x = torch.randn(m, k, device=dev).to(torch.float8_e4m3fn)
        y = torch.randn(n, k, device=dev).to(torch.float8_e4m3fn).t()
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)

        def run(row: Optional[int]):
            return ops.fp8_gemm(x, y, out_dtype=torch.bfloat16, config=row, out=out)

        times = _row_times(run, n_rows, iters, flush)
        auto_us = _median_us(lambda: run(None), iters, flush)
        auto_row = lib.hb200_fp8_gemm_select_config(m, n, k, 1, 0)
        extra = ""
        if library:
            one = torch.ones((), device=dev)
            lib_us = _median_us(lambda: torch._scaled_mm(x, y, one, one, out_dtype=torch.bfloat16), iters, flush)
            extra = f" | {lib_us:.1f}"
        print(_format(f"{m}×{n}×{k}", times, auto_us, auto_row, extra), flush=True)
        _lib.check_status(dev.index or 0)


def sweep_attention(shapes, iters: int, causal: bool, dev: torch.device, flush: torch.Tensor) -> None:
    n_rows = _lib.num_configs(_lib.OP_ATTENTION)
    print(f"\nFP8 attention{' (causal)' if causal else ''}, e4m3 out; µs per launch, cold L2, median of {iters}\n")
    head = " | ".join(str(r) for r in range(n_rows))
    print(f"| B·H·S·D | {head} | picked | best | picked / best |")
    print("|" + "---|" * (n_rows + 4))
    for b, h, s, d in shapes:
        q = torch.randn(b * h, s, d, device=dev).to(torch.float8_e4m3fn)
        k = torch.randn(b * h, s, d, device=dev).to(torch.float8_e4m3fn)
        v = torch.randn(b * h, s, d, device=dev).to(torch.float8_e4m3fn).permute(0, 2, 1)
        out = torch.empty(b, h, s, d, dtype=torch.float8_e4m3fn, device=dev)

        def run(row: Optional[int]):
            return ops.fp8_attention(q, k, v, b, h, config=row, out=out, causal=causal)

        times = _row_times(run, n_rows, iters, flush)
        auto_us = _median_us(lambda: run(None), iters, flush)
        print(_format(f"{b}·{h}·{s}·{d}", times, auto_us, None, ""), flush=True)
        _lib.check_status(dev.index or 0)


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--op", choices=("gemm", "attention", "both"), default="both")
    ap.add_argument("--shape", action="append", default=[], help="M,N,K or B,H,S,D (repeatable); default: the built-in lists")
    ap.add_argument("--iters", type=int, default=11)
    ap.add_argument("--causal", action="store_true", help="attention: with the causal mask")
    ap.add_argument("--library", action="store_true", help="gemm: add torch._scaled_mm as a context column")
    ap.add_argument("--back-to-back", type=int, default=0, metavar="N",
                    help="gemm: N launches per event pair, rows interleaved, instead of single cold-L2 launches")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("the sweep needs a CUDA device; the library has no CPU path", file=sys.stderr)
        return 2
    dev = torch.device("cuda", args.device)
    torch.cuda.set_device(dev)
    flush = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    shapes = [tuple(int(v) for v in s.split(",")) for s in args.shape]
    print(f"device: {torch.cuda.get_device_name(dev)}; rows: " + "; ".join(
        _lib.describe_config(op, r) for op in (_lib.OP_GEMM, _lib.OP_ATTENTION) for r in range(_lib.num_configs(op))))
    if args.op in ("gemm", "both"):
        sweep_gemm([s for s in shapes if len(s) == 3] or GEMM_SHAPES, args.iters, args.library, dev, flush,
                   args.back_to_back)
    if args.op in ("attention", "both"):
        sweep_attention([s for s in shapes if len(s) == 4] or ATTN_SHAPES, args.iters, args.causal, dev, flush)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
