"""FP8 GEMM on HOST buffers: pinned x, y in, pinned out back, with the PCIe copies overlapped.

A caller whose operands live in host memory pays for three transfers per GEMM (x and y in, out
back); done one after the other on one stream they take ~15x longer than the 8192^3 GEMM itself.
:class:`HostGemm` runs them as a pipeline instead:

* three CUDA streams -- copy-in, compute, copy-out -- so that host->device and device->host
  traffic (PCIe is full duplex) and the kernels overlap;
* x and out are cut into row blocks: block i is multiplied while block i+1 is still arriving and
  block i-1 is already on its way back (row blocks of a GEMM are independent, the same fact the
  multi-GPU sharding uses);
* the device buffers exist ``depth`` times, so the next call's uploads overlap this call's
  downloads;
* ``y`` may be made resident (:meth:`HostGemm.set_weight`): a weight that is the same for every call is
  uploaded once, and a call then moves only ``x`` up and ``out`` back;
* with a process group (one rank per GPU of a node, every rank holding the same ``y`` in host memory and its own
  rows of ``x``), every rank uploads only its 1/world share of ``y`` and the ranks exchange the shares with one
  NCCL all-gather over NVLink: the node moves ``y`` over PCIe once per call instead of once per GPU.

The arithmetic is that of :func:`helion_b200.ops.fp8_gemm` on every row block, so the result is
bit-identical to one call on the whole matrix.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from . import ops


class HostGemm:
    """Pipeline for ``out_host = (x_host @ y_host).to(out_dtype)`` with e4m3 operands in pinned memory.

    ``x_host``: uint8 or float8_e4m3fn ``[M, K]`` row-major; ``y_host``: ``[N, K]`` bytes, i.e. ``y``
    stored column-major (the layout the benchmark configurations and ``torch._scaled_mm`` use);
    ``out_host``: ``[M, N]`` of ``out_dtype``.  All three must be pinned for the copies to be
    asynchronous.
    """

    def __init__(self, m: int, n: int, k: int, *, out_dtype: torch.dtype = torch.bfloat16, device=None,
                 row_blocks: int = 8, depth: int = 2, group=None) -> None:
        if not torch.cuda.is_available():
            raise RuntimeError("HostGemm needs a CUDA device; there is no CPU path")
        self.m, self.n, self.k = m, n, k
        self.out_dtype = out_dtype
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.row_blocks = max(1, min(row_blocks, (m + 127) // 128))
        rows = -(-m // self.row_blocks)
        self.block_rows = -(-rows // 128) * 128  # whole 128-row tiles per block
        self.depth = depth
        self._slot = 0
        self._in, self._compute, self._out = (torch.cuda.Stream(self.device) for _ in range(3))
        # The buffers are only ever used on the three private streams; they are allocated under one of them and
        # recorded on the others, so that torch's caching allocator does not hand them to other work while
        # copies or kernels of a dropped pipeline are still in flight.
        with torch.cuda.stream(self._compute):
            self._x = [torch.empty(m, k, dtype=torch.uint8, device=self.device) for _ in range(depth)]
            self._y = [torch.empty(n, k, dtype=torch.uint8, device=self.device) for _ in range(depth)]
            self._o = [torch.empty(m, n, dtype=out_dtype, device=self.device) for _ in range(depth)]
            self._w = torch.empty(n, k, dtype=torch.uint8, device=self.device)
        for t in (*self._x, *self._y, *self._o, self._w):
            t.record_stream(self._in)
            t.record_stream(self._out)
        self._w_ready: Optional[torch.cuda.Event] = None
        self._done: List[Optional[torch.cuda.Event]] = [None] * depth
        # y shared out over the ranks of `group`: rank r uploads rows [r, r + 1) * n / world of the stored y and an
        # all-gather on a stream of its own completes every rank's copy (all ranks must call submit in step)
        self._group = group
        self._world = self._rank = None
        if group is not None:
            import torch.distributed as dist

            self._world, self._rank = dist.get_world_size(group), dist.get_rank(group)
            if n % self._world != 0:
                raise ValueError(f"sharing y over {self._world} ranks needs N ({n}) to be a multiple of it")
            self._xchg = torch.cuda.Stream(self.device)
            for t in self._y:
                t.record_stream(self._xchg)

    def set_weight(self, y_host: torch.Tensor) -> None:
        """Upload ``y`` (stored as ``[N, K]`` bytes, i.e. column-major) once; later calls of :meth:`submit` with
        ``y_host=None`` multiply by it without moving it again."""
        if tuple(y_host.shape) != (self.n, self.k):
            raise ValueError(f"expected y stored as [{self.n},{self.k}]")
        self.synchronize()  # no call in flight may still read the previous weight
        self._in.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._in):
            self._w.copy_(y_host.view(torch.uint8), non_blocking=True)
            self._w_ready = torch.cuda.Event()
            self._w_ready.record(self._in)

    def submit(self, x_host: torch.Tensor, y_host: Optional[torch.Tensor], out_host: torch.Tensor) -> torch.cuda.Event:
        """Enqueue one GEMM; returns the event that fires when ``out_host`` is complete.  ``y_host=None`` uses
        the resident weight of :meth:`set_weight`."""
        m, n, k = self.m, self.n, self.k
        if tuple(x_host.shape) != (m, k) or tuple(out_host.shape) != (m, n) or (
                y_host is not None and tuple(y_host.shape) != (n, k)):
            raise ValueError(f"expected x [{m},{k}], y stored as [{n},{k}], out [{m},{n}]")
        if y_host is None and self._w_ready is None:
            raise ValueError("no resident weight: call set_weight(y_host) first or pass y_host")
        if out_host.dtype != self.out_dtype:
            raise TypeError(f"out_host must be {self.out_dtype}")
        xh = x_host.view(torch.uint8)
        slot = self._slot
        self._slot = (slot + 1) % self.depth
        xd, yd, od = self._x[slot], self._y[slot], self._o[slot]
        caller = torch.cuda.current_stream(self.device)
        self._in.wait_stream(caller)  # the host buffers may have been produced by work on the caller's stream
        if self._done[slot] is not None:
            self._in.wait_event(self._done[slot])  # this slot's previous download must have left the device buffers
        blocks = [(r, min(r + self.block_rows, m)) for r in range(0, m, self.block_rows)]
        arrived = []
        y_gathered: Optional[torch.cuda.Event] = None
        with torch.cuda.stream(self._in):
            if y_host is not None and self._group is not None:
                import torch.distributed as dist

                share = n // self._world
                mine = slice(self._rank * share, (self._rank + 1) * share)
                yd[mine].copy_(y_host.view(torch.uint8)[mine], non_blocking=True)
                uploaded = torch.cuda.Event()
                uploaded.record(self._in)
                self._xchg.wait_event(uploaded)
                with torch.cuda.stream(self._xchg):  # in place: this rank's share already sits where it belongs
                    dist.all_gather_into_tensor(yd, yd[mine], group=self._group)
                    y_gathered = torch.cuda.Event()
                    y_gathered.record(self._xchg)
            elif y_host is not None:
                yd.copy_(y_host.view(torch.uint8), non_blocking=True)
            else:
                yd = self._w
                self._in.wait_event(self._w_ready)
            for r0, r1 in blocks:
                xd[r0:r1].copy_(xh[r0:r1], non_blocking=True)
                ev = torch.cuda.Event()
                ev.record(self._in)
                arrived.append(ev)
        y_op = yd.view(torch.float8_e4m3fn).t()
        computed = []
        with torch.cuda.stream(self._compute):
            if y_gathered is not None:
                self._compute.wait_event(y_gathered)
            for (r0, r1), ev in zip(blocks, arrived):
                self._compute.wait_event(ev)
                ops.fp8_gemm(xd[r0:r1].view(torch.float8_e4m3fn), y_op, out_dtype=self.out_dtype, out=od[r0:r1])
                ev2 = torch.cuda.Event()
                ev2.record(self._compute)
                computed.append(ev2)
        with torch.cuda.stream(self._out):
            for (r0, r1), ev in zip(blocks, computed):
                self._out.wait_event(ev)
                out_host[r0:r1].copy_(od[r0:r1], non_blocking=True)
            done = torch.cuda.Event()
            done.record(self._out)
        self._done[slot] = done
        return done

    def __call__(self, x_host: torch.Tensor, y_host: torch.Tensor, out_host: torch.Tensor) -> torch.Tensor:
        """Blocking form: returns ``out_host`` once it is complete."""
        self.submit(x_host, y_host, out_host).synchronize()
        return out_host

    def synchronize(self) -> None:
        for ev in self._done:
            if ev is not None:
                ev.synchronize()

    def close(self) -> None:
        """Wait for everything in flight; call before dropping a pipeline whose last results were not awaited."""
        self.synchronize()
        for stream in (self._in, self._compute, self._out, *((self._xchg,) if self._group is not None else ())):
            stream.synchronize()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:  # interpreter shutdown: CUDA may be gone already
            pass
