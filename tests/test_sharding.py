"""The multi-GPU driver's host logic on CPU: shard arithmetic, and the N>1 path with two gloo
ranks where the oracle stands in for the CUDA kernel (the compute function is injectable)."""
from __future__ import annotations

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from helion_b200.sharding import shard_range, sharded_fp8_attention, sharded_fp8_gemm
from oracle import fp8_oracle as o


@pytest.mark.parametrize("total,world", [(8192, 8), (10, 4), (3, 8), (0, 2), (192, 8), (7, 7)])
def test_shard_range_partitions_exactly(total, world):
    spans = [shard_range(total, world, r) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == total
    for (a, b), (c, d) in zip(spans, spans[1:]):
        assert b == c and a <= b
    sizes = [b - a for a, b in spans]
    assert max(sizes) - min(sizes) <= 1


def test_shard_range_rejects_bad_rank():
    with pytest.raises(ValueError):
        shard_range(10, 2, 2)


def _oracle_gemm(x, y, out_dtype=torch.float16):
    name = {torch.float16: "fp16", torch.bfloat16: "bf16", torch.float32: "fp32"}[out_dtype]
    res = o.fp8_gemm(o.torch_fp8_to_bits(x), o.torch_fp8_to_bits(y), name)
    return torch.from_numpy(res).to(out_dtype)


def _oracle_attention(q, k, v, out3):
    bh = q.shape[0]
    res = o.fp8_attention(o.torch_fp8_to_bits(q), o.torch_fp8_to_bits(k), o.torch_fp8_to_bits(v), 1, bh,
                          "e4m3" if out3.dtype == torch.float8_e4m3fn else "fp32")
    out3.copy_(torch.from_numpy(res[0]).to(out3.dtype))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, m: int, bh: int):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        x, y = o.gemm_inputs(m, 48, 64, seed=21)
        want = _oracle_gemm(x, y, torch.float32)
        lo, hi = shard_range(m, world, rank)
        local = sharded_fp8_gemm(x, y, rank=rank, world_size=world, out_dtype=torch.float32, compute=_oracle_gemm)
        assert torch.equal(local, want[lo:hi])
        full = sharded_fp8_gemm(x, y, rank=rank, world_size=world, out_dtype=torch.float32,
                                replicate_output=True, compute=_oracle_gemm)
        assert torch.equal(full, want)

        q, k, v = o.attention_inputs(1, bh, 32, 64, seed=22)
        q8 = q.to(torch.float8_e4m3fn).reshape(bh, 32, 64)
        k8 = k.to(torch.float8_e4m3fn).reshape(bh, 32, 64)
        v8 = v.permute(0, 1, 3, 2).to(torch.float8_e4m3fn).reshape(bh, 64, 32)
        want8 = torch.empty(bh, 32, 64, dtype=torch.float8_e4m3fn)
        _oracle_attention(q8, k8, v8, want8)
        full8 = sharded_fp8_attention(q8, k8, v8, 1, bh, rank=rank, world_size=world, replicate_output=True,
                                      compute=_oracle_attention)
        assert full8.shape == (1, bh, 32, 64)
        assert torch.equal(full8.view(torch.uint8).reshape(bh, 32, 64), want8.view(torch.uint8))
        lo, hi = shard_range(bh, world, rank)
        part = sharded_fp8_attention(q8, k8, v8, 1, bh, rank=rank, world_size=world, compute=_oracle_attention)
        assert torch.equal(part.view(torch.uint8), want8.view(torch.uint8)[lo:hi])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("m,bh", [(64, 4), (50, 3)])  # equal and ragged shards
def test_two_rank_gloo_sharding_matches_unsharded(m, bh):
    mp.spawn(_worker, args=(2, _free_port(), m, bh), nprocs=2, join=True)
