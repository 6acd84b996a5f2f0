"""Multi-GPU driver: one process per GPU, no collective on the compute path.

Both operators split into independent units: rows of ``out`` depend only on the same rows of
``x`` (pytorch-labs/helion examples/fp8_gemm.py:47-56), and every batch*head slice of attention is
independent (examples/fp8_attention.py:54 -- the kernel's only grid axis).  So each rank runs the
single-GPU kernel on a contiguous block of M rows / batch*head slices, with ``y`` replicated.  An
NCCL all-gather over NVLink assembles the replicated output only when the caller asks for it.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist

from . import ops


def shard_range(total: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous near-equal split of ``range(total)``: the first ``total % world_size`` ranks get
    one extra unit.  Returns ``(lo, hi)``; empty when there are more ranks than units."""
    if world_size < 1 or not (0 <= rank < world_size):
        raise ValueError(f"bad rank {rank} for world size {world_size}")
    base, extra = divmod(total, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def _gather_dim0(local: torch.Tensor, total: int, world_size: int, group) -> torch.Tensor:
    """All-gather blocks of ``shard_range`` sizes along dim 0 into a [total, ...] tensor."""
    full = torch.empty((total,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    if total % world_size == 0:
        # Equal blocks are contiguous in the result: one zero-copy all-gather.
        gather_view = full
        local_view = local.contiguous()
        if local.dtype == torch.float8_e4m3fn:  # collectives move bytes
            gather_view = full.view(torch.uint8)
            local_view = local_view.view(torch.uint8)
        dist.all_gather_into_tensor(gather_view, local_view, group=group)
        return full
    sizes = [shard_range(total, world_size, r) for r in range(world_size)]
    longest = max(hi - lo for lo, hi in sizes)
    as_bytes = local.dtype == torch.float8_e4m3fn
    pad = torch.zeros((longest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    bufs = [torch.empty_like(pad) for _ in range(world_size)]
    if as_bytes:
        dist.all_gather([b.view(torch.uint8) for b in bufs], pad.view(torch.uint8), group=group)
    else:
        dist.all_gather(bufs, pad, group=group)
    for (lo, hi), b in zip(sizes, bufs):
        full[lo:hi] = b[: hi - lo]
    return full


def sharded_fp8_gemm(
    x: torch.Tensor,
    y: torch.Tensor,
    *,
    rank: int,
    world_size: int,
    out_dtype: torch.dtype = torch.float16,
    replicate_output: bool = False,
    group=None,
    compute: Optional[Callable[..., torch.Tensor]] = None,
) -> torch.Tensor:
    """Row-sharded ``x @ y``.  ``x`` is the FULL [M, K] operand (each rank reads only its rows) and
    ``y`` is replicated.  Returns this rank's [rows, N] block, or the full [M, N] result on every
    rank when ``replicate_output`` is set (one all-gather, off the compute path)."""
    compute = compute or ops.fp8_gemm
    m = x.shape[0]
    lo, hi = shard_range(m, world_size, rank)
    local = compute(x[lo:hi], y, out_dtype=out_dtype)
    if not replicate_output:
        return local
    return _gather_dim0(local, m, world_size, group)


def sharded_fp8_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    batch: int,
    heads: int,
    *,
    rank: int,
    world_size: int,
    out_dtype: torch.dtype = torch.float8_e4m3fn,
    replicate_output: bool = False,
    group=None,
    compute: Optional[Callable[..., None]] = None,
) -> torch.Tensor:
    """Batch*head-sharded attention.  ``q``, ``k`` ([BH,S,D]) and ``v`` ([BH,D,S]) are the FULL
    operands; each rank computes slices ``shard_range(BH, world_size, rank)``.  Returns this rank's
    [slices, S, D] block, or the full [batch, heads, S, D] output when ``replicate_output`` is set.
    The block need not hold whole batches: slices are independent and keep their global order."""
    compute = compute or ops.attention_into
    bh, s, d = q.shape
    if bh != batch * heads:
        raise ValueError(f"q.size(0)={bh} != batch*heads={batch * heads}")
    lo, hi = shard_range(bh, world_size, rank)
    local = torch.empty((hi - lo, s, d), dtype=out_dtype, device=q.device)
    if hi > lo:
        compute(q[lo:hi], k[lo:hi], v[lo:hi], local)
    if not replicate_output:
        return local
    return _gather_dim0(local, bh, world_size, group).view(batch, heads, s, d)
