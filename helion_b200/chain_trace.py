"""Where a chain of few-row GEMM launches spends its time: per-CTA wall-clock stamps of the kernel's phases.

A decode loop runs one ``[M <= 64, K] x [K, N]`` GEMM per layer against a different weight each time
(the reference's ``fp8_gemm``, examples/fp8_gemm.py:29-57, called once per linear layer).  This tool captures
``--layers`` such launches in one CUDA graph, replays it, and reads the stamps that an instrumented build of the
few-row kernel (``-DHB_SKINNY_TRACE``, csrc/fp8_gemm_skinny.cu) writes per CTA: entry, set-up done, predecessor
ended (``griddepcontrol.wait`` returned), first stage landed, first refilled stage landed, last stage landed,
teardown reached.  It prints, for a few launches in the middle of the chain, min / median / max over the CTAs of
every stamp (ns from the first CTA of the replay) and the period from one launch's release to the next.

    python -m helion_b200.build --define HB_SKINNY_TRACE --output helion_b200/_C/libhelion_b200_trace.so
    HB200_LIB=helion_b200/_C/libhelion_b200_trace.so python -m helion_b200.chain_trace --rows 18,22,23

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


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--rows", default="18,22,23", help="table rows of the few-row kernel to trace")
    ap.add_argument("--m", type=int, default=16)
    ap.add_argument("--n", type=int, default=14336)
    ap.add_argument("--k", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=32)
    args = ap.parse_args(argv)
    if not torch.cuda.is_available():
        print("needs a CUDA device", file=sys.stderr)
        return 2
    lib = _lib.load()
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
