"""Where a chain of GEMM launches spends its time: per-CTA wall-clock stamps of the kernels' phases.

A decode loop runs one ``[M <= 64, K] x [K, N]`` GEMM per layer against a different weight each time
(the reference's ``fp8_gemm``, examples/fp8_gemm.py:29-57, called once per linear layer).  This tool captures
``--layers`` such launches in one CUDA graph, replays it, and reads the stamps that an instrumented build of the
few-row kernel (``-DHB_SKINNY_TRACE``, csrc/fp8_gemm_skinny.cu) writes per CTA: entry, set-up done, predecessor
ended (``griddepcontrol.wait`` returned), first stage landed, first refilled stage landed, last stage landed,
teardown reached.  It prints, for a few launches in the middle of the chain, min / median / max over the CTAs of
every stamp (ns from the first CTA of the replay) and the period from one launch's release to the next.

    python -m helion_b200.build --define HB_SKINNY_TRACE --define HB_GEMM_TRACE --output helion_b200/_C/libhelion_b200_trace.so
    HB200_LIB=helion_b200/_C/libhelion_b200_trace.so python -m helion_b200.chain_trace --rows 18,22,23
    HB200_LIB=helion_b200/_C/libhelion_b200_trace.so python -m helion_b200.chain_trace --kernel pair --m 1024 --rows 21,14

``--kernel pair`` traces the 512-row CTA-pair kernel (csrc/fp8_gemm.cu, ``-DHB_GEMM_TRACE``) instead: ``--launches``
calls of ``fp8_gemm`` back to back on the stream (operands rotate through four copies, N = K = 8192 unless given),
stamps of the leader CTA of every pair -- entry, set-up done, predecessor ended, first operands landed, last
operands of its first tile landed, first tile's accumulators complete, first tile handed to the store engine,
teardown -- and, for one epilogue warp, when each 32-column block was loaded from tensor memory and when its bulk
store was issued.

The product library holds none of this; the tool refuses to run on it.
"""
from __future__ import annotations

import argparse
import ctypes
import sys
from typing import Optional, Sequence

import numpy as np
import torch

from . import _lib, ops

STAMPS = ("entry", "set-up done", "predecessor ended", "first stage landed", "first refilled stage landed",
          "last stage landed", "teardown")
SLOTS = 12      # 64-bit words per record
RECORDS = 8192  # ring of records in the instrumented library


PAIR_STAMPS = ("entry", "set-up done", "predecessor ended", "first operands landed", "last operands of tile 0 landed",
               "tile 0 accumulators complete", "tile 0 handed to the store engine", "teardown")


def trace_pair_kernel(args, lib) -> int:
    """Back-to-back launches of the 512-row CTA-pair kernel; one record per leader CTA (32 words)."""
    try:
        read = lib.hb200_debug_gemm_trace
    except AttributeError:
        print("this library was built without -DHB_GEMM_TRACE (see the module docstring)", file=sys.stderr)
        return 2
    read.restype = ctypes.c_int
    read.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint)]
    dev = torch.device("cuda", 0)
    n_cols, k = (args.n, args.k) if args.n_given else (8192, 8192)
    g = torch.Generator(device=dev).manual_seed(1)
    copies = 4
    ys = [torch.randn(n_cols, k, device=dev, generator=g).to(torch.float8_e4m3fn).t() for _ in range(copies)]
    xs = [torch.randn(args.m, k, device=dev, generator=g).to(torch.float8_e4m3fn) for _ in range(copies)]
    outs = [torch.empty(args.m, n_cols, dtype=torch.bfloat16, device=dev) for _ in range(copies)]
    buf = np.zeros((RECORDS, 32), dtype=np.uint64)
    count = ctypes.c_uint(0)

    def dump():
        if read(buf.ctypes.data_as(ctypes.c_void_p), ctypes.byref(count)) != 0:
            raise RuntimeError("reading the trace failed")
        return buf.copy(), count.value

    for row in (int(r) for r in args.rows.split(",")):
        def launch(i):
            ops.fp8_gemm(xs[i % copies], ys[i % copies], out_dtype=torch.bfloat16, out=outs[i % copies], config=row)

        for i in range(4):
            launch(i)
        torch.cuda.synchronize()
        _, before = dump()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(args.launches):
            launch(i)
        end.record()
        torch.cuda.synchronize()
        rec, after = dump()
        n = after - before
        r = rec[[(before + i) % RECORDS for i in range(n)]].astype(np.int64)
        t0 = r[:, 0].min()
        r[r > 0] -= t0
        r = r[np.argsort(r[:, 2], kind="stable")]
        per = n // args.launches
        print(f"\nrow {row}: {_lib.describe_config(_lib.OP_GEMM, row)}")
        print(f"{args.m} x {n_cols} x {k}: {n} leader-CTA records, {per} per launch; "
              f"{start.elapsed_time(end) * 1e3 / args.launches:.2f} us per launch (CUDA events)")
        li = args.launches // 2
        launch_rows = r[li * per:(li + 1) * per]
        base = int(np.median(launch_rows[:, 2]))
        for c, name in enumerate(PAIR_STAMPS):
            col = launch_rows[:, c]
            print(f"  {name}: {int(col.min()) - base:+d} / {int(np.median(col)) - base:+d} / {int(col.max()) - base:+d} ns "
                  "(min / median / max over the pairs, relative to the launch's release)")
        chunks = launch_rows[:, 8:32].reshape(per, 8, 3) - launch_rows[:, 5][:, None, None]
        med = np.median(chunks, axis=0).astype(int)
        used = [c for c in range(8) if med[c, 0] > 0]
        print("  one epilogue warp, tile 0, ns after its accumulators were complete; per 32-column block "
              "(loaded from tensor memory, staging buffer free, bulk store issued): "
              + "; ".join(f"{med[c, 0]} {med[c, 1]} {med[c, 2]}" for c in used))
        released = np.array([np.median(r[i * per:(i + 1) * per, 2]) for i in range(args.launches)])
        periods = np.diff(released)[2:]
        print(f"  release-to-release period: median {int(np.median(periods))} ns (min {int(periods.min())}, max {int(periods.max())})")
        _lib.check_status(0)
    return 0


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--kernel", choices=("few-row", "pair"), default="few-row")
    ap.add_argument("--rows", default=None, help="table rows to trace (default 18,22,23; 21,14 with --kernel pair)")
    ap.add_argument("--m", type=int, default=None)
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--k", type=int, default=None)
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--launches", type=int, default=24)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("needs a CUDA device", file=sys.stderr)
        return 2
    lib = _lib.load()
    args.n_given = args.n is not None and args.k is not None
    if args.kernel == "pair":
        args.rows = args.rows or "21,14"
        args.m = args.m or 1024
        return trace_pair_kernel(args, lib)
    args.rows = args.rows or "18,22,23"
    args.m, args.n, args.k = args.m or 16, args.n or 14336, args.k or 4096
    try:
        read = lib.hb200_debug_skinny_trace
    except AttributeError:
        print("this library was built without -DHB_SKINNY_TRACE (see the module docstring)", file=sys.stderr)
        return 2
    read.restype = ctypes.c_int
    read.argtypes = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_uint)]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(2)
    ws = [torch.randn(args.n, args.k, device=dev, generator=g).mul_(0.5).to(torch.float8_e4m3fn).t()
          for _ in range(args.layers)]
    x = torch.randn(args.m, args.k, device=dev, generator=g).to(torch.float8_e4m3fn)
    out = torch.empty(args.m, args.n, dtype=torch.bfloat16, device=dev)
    buf = np.zeros((RECORDS, SLOTS), dtype=np.uint64)
    count = ctypes.c_uint(0)

    def dump():
        if read(buf.ctypes.data_as(ctypes.c_void_p), ctypes.byref(count)) != 0:
            raise RuntimeError("reading the trace failed")
        return buf.copy(), count.value

    for row in (int(r) for r in args.rows.split(",")):
        def loop():
            for w in ws:
                ops.fp8_gemm(x, w, out_dtype=torch.bfloat16, out=out, config=row)

        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            loop()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            loop()
        graph.replay()
        torch.cuda.synchronize()
        _, before = dump()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        rec, after = dump()
        n = after - before
        r = rec[[(before + i) % RECORDS for i in range(n)]].astype(np.int64)
        r[:, :7] -= r[:, 0].min()
        r = r[np.argsort(r[:, 2], kind="stable")]  # launches follow one another in the order they were released
        per = n // args.layers
        print(f"\nrow {row}: {_lib.describe_config(_lib.OP_GEMM, row)}")
        print(f"{n} CTA records, {per} per launch; {start.elapsed_time(end) * 1e3 / args.layers:.2f} us per layer (CUDA events)")
        for li in (args.layers // 3, args.layers // 3 + 1):
            launch = r[li * per:(li + 1) * per]
            base = int(np.median(launch[:, 2]))
            cells = ", ".join(f"{name} {int(launch[:, c].min()) - base:+d} / {int(np.median(launch[:, c])) - base:+d} / "
                              f"{int(launch[:, c].max()) - base:+d}" for c, name in enumerate(STAMPS))
            print(f"  launch {li} (min / median / max over its CTAs, ns relative to its release): {cells}")
        released = np.array([np.median(r[li * per:(li + 1) * per, 2]) for li in range(args.layers)])
        periods = np.diff(released)[2:]
        print(f"  release-to-release period: median {int(np.median(periods))} ns (min {int(periods.min())}, max {int(periods.max())})")
        _lib.check_status(0)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
