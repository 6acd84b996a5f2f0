"""Softmax-only ceiling of the FP8 attention kernels, measured on the GPU.

    python -m helion_b200.ceiling [--steps 2000]

Runs ``hb200_debug_softmax_ceiling``: nothing but the per-score work of the reference's attention loop
(examples/fp8_attention.py:74-94: row max, exp2, row sum, cast of P to e4m3; scores read from and P written
to tensor memory) for a number of 128x128 steps per softmax warpgroup on every SM, and prints, per variant,
the SM cycles one 128x128 step costs per SM (the slowest CTA's clock count divided by the steps all
warpgroups of an SM ran) next to the 1024 cycles the MUFU unit alone needs for 128x128 ``ex2`` at 16 per
clock.  An attention kernel with this arithmetic cannot run a step faster than this, whatever its pipeline;
dividing a shape's step count per SM by it gives the shortest possible kernel time.
"""
from __future__ import annotations

import argparse
import json

import torch

from . import _lib

#: (label, warpgroups per CTA, CTAs per SM, polynomial pairs of 8, mode)
VARIANTS = [
    ("1 warpgroup per SM, all exp2 on MUFU", 1, 1, 0, 0),
    ("2 CTAs x 1 warpgroup per SM, all exp2 on MUFU", 1, 2, 0, 0),
    ("2 warpgroups per SM, all exp2 on MUFU", 2, 1, 0, 0),
    ("2 warpgroups per SM, 2 of 8 pairs polynomial", 2, 1, 2, 0),
    ("2 warpgroups per SM, 3 of 8 pairs polynomial", 2, 1, 3, 0),
    ("2 warpgroups per SM, 4 of 8 pairs polynomial", 2, 1, 4, 0),
    ("2 warpgroups per SM, without the row max", 2, 1, 0, 1),
    ("2 warpgroups per SM, without the exponentials", 2, 1, 0, 2),
    ("2 warpgroups per SM, tensor-memory traffic only", 2, 1, 0, 3),
    ("1 warpgroup per SM, 4 of 8 pairs polynomial", 1, 1, 4, 0),
    # the full step of two warpgroups next to other roles of an attention kernel (mode = 16 + mask)
    ("2 warpgroups + four warps polling a barrier", 2, 1, 0, 17),
    ("2 warpgroups + one thread issuing tensor-core instructions back to back", 2, 1, 0, 18),
    ("2 warpgroups + four warps rescaling tensor memory", 2, 1, 0, 20),
    ("2 warpgroups + the protocol's barrier traffic in the softmax threads", 2, 1, 0, 24),
    ("2 warpgroups + all four", 2, 1, 0, 31),
]


def measure(steps: int = 2000, device: int = 0, only=None):
    """Returns one dict per variant: cycles per 128x128 step per SM (from the SM clock) and the event time.
    ``only``: indices into ``VARIANTS`` to run (default: all)."""
    lib = _lib.load()
    dev = torch.device("cuda", device)
    n_sms = lib.hb200_num_sms(device)
    _lib.raise_for(n_sms, "num_sms")
    stream = torch.cuda.current_stream(device).cuda_stream
    rows = []
    for label, wgs, ctas, poly, mode in (VARIANTS if only is None else [VARIANTS[i] for i in only]):
        cycles = torch.zeros(n_sms * ctas, dtype=torch.int64, device=dev)
        for _ in range(2):  # first launch loads the kernel
            _lib.raise_for(lib.hb200_debug_softmax_ceiling(wgs, ctas, poly, mode, steps, cycles.data_ptr(), device, stream),
                           "softmax_ceiling")
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        _lib.raise_for(lib.hb200_debug_softmax_ceiling(wgs, ctas, poly, mode, steps, cycles.data_ptr(), device, stream),
                       "softmax_ceiling")
        end.record()
        end.synchronize()
        per_sm_steps = steps * wgs * ctas
        rows.append({
            "variant": label,
            "cycles_per_step_per_sm": float(cycles.max().item()) / per_sm_steps,
            "ns_per_step_per_sm": start.elapsed_time(end) * 1e6 / per_sm_steps,
        })
    return rows


def floor_us(cycles_per_step: float, batch_heads: int, seq: int, n_sms: int, mhz: float) -> float:
    """Shortest kernel time for a non-causal shape: its 128x128 steps spread evenly over the SMs."""
    steps = batch_heads * (seq // 128) * (seq // 128)
    return steps / n_sms * cycles_per_step / mhz


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--json", action="store_true")
    args = ap.parse_args()
    rows = measure(args.steps)
    if args.json:
        print(json.dumps(rows))
        return
    print("| variant | SM cycles per 128x128 step per SM | ns per step per SM (CUDA events) | of the 1024-cycle MUFU floor |")
    print("|---|---|---|---|")
    for r in rows:
        print(f"| {r['variant']} | {r['cycles_per_step_per_sm']:.0f} | {r['ns_per_step_per_sm']:.0f} | "
              f"{r['cycles_per_step_per_sm'] / 1024.0:.2f} |")


if __name__ == "__main__":
    main()
