"""Host-to-host streaming of batches through a layer.

A caller whose activations live in host memory pays two PCIe copies per batch (42 MB each way
for 4096 x 5120 bf16, about as long as the layer itself).  Run one after the other they double
the step time; this helper keeps them off the critical path: the host-to-device copy of batch
``k + 1`` and the device-to-host copy of batch ``k - 1`` run on their own streams (PCIe is full
duplex) while batch ``k`` computes.  Device buffers are double-buffered and guarded by events;
nothing synchronises the host until :meth:`drain`.

Under tensor parallelism every rank needs the whole input and, after the exchange, holds the
whole output.  Copying all of it over every rank's PCIe link would make the host link the
bottleneck (134 MB per rank and step for 8192 x 8192), so each rank copies only its
``tokens / tp`` rows in, an all-gather over NVLink replicates them, and each rank copies only
its own rows of the result out: the batch crosses PCIe once in each direction in total.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class HostStreamedLayer:
    """``submit(x_host, out_host)`` queues one batch; ``layer(x_dev)`` must return the
    ``(tokens, hidden)`` result on the current stream.

    With ``group`` of more than one rank, ``x_host`` / ``out_host`` are this rank's row slice
    ``(tokens / tp, hidden)`` of the batch and of the result (``tokens`` must divide).
    """

    def __init__(self, layer, tokens: int, hidden: int, device=None, group=None, depth: int = 2):
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.layer, self.depth, self.group = layer, depth, group
        self.world = dist.get_world_size(group) if (group is not None or (
            dist.is_available() and dist.is_initialized())) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        if tokens % self.world:
            raise ValueError(f"{tokens} tokens do not split over {self.world} ranks")
        self.rows = tokens // self.world
        bf = torch.bfloat16
        self.x_dev = [torch.empty((tokens, hidden), device=dev, dtype=bf) for _ in range(depth)]
        self.x_in = ([torch.empty((self.rows, hidden), device=dev, dtype=bf) for _ in range(depth)]
                     if self.world > 1 else self.x_dev)
        self.out_dev = [torch.empty((self.rows, hidden), device=dev, dtype=bf) for _ in range(depth)]
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        mk = lambda: [torch.cuda.Event() for _ in range(depth)]
        self.x_ready, self.x_free, self.out_ready, self.out_free = mk(), mk(), mk(), mk()
        self.n = 0

    def begin(self) -> None:
        """Order the copy streams after what is already queued on the current stream."""
        ev = torch.cuda.Event()
        ev.record()
        self.s_in.wait_event(ev)
        self.s_out.wait_event(ev)

    def submit(self, x_host: torch.Tensor, out_host: torch.Tensor | None) -> None:
        i, first_use = self.n % self.depth, self.n < self.depth
        self.n += 1
        compute = torch.cuda.current_stream()
        if not first_use:
            self.s_in.wait_event(self.x_free[i])          # the batch that used this buffer is done
        with torch.cuda.stream(self.s_in):
            self.x_in[i].copy_(x_host, non_blocking=True)
            self.x_ready[i].record()
        compute.wait_event(self.x_ready[i])
        if self.world > 1:
            dist.all_gather_into_tensor(self.x_dev[i], self.x_in[i], group=self.group)
        out = self.layer(self.x_dev[i])
        self.x_free[i].record(compute)
        if out_host is None:
            return
        if not first_use:
            compute.wait_event(self.out_free[i])          # its previous content has left the GPU
        r0 = self.rank * self.rows
        self.out_dev[i].copy_(out[r0:r0 + self.rows])
        self.out_ready[i].record(compute)
        self.s_out.wait_event(self.out_ready[i])
        with torch.cuda.stream(self.s_out):
            out_host.copy_(self.out_dev[i], non_blocking=True)
            self.out_free[i].record()

    def end(self) -> None:
        """Make the current stream wait for every copy queued so far (no host synchronisation)."""
        cur = torch.cuda.current_stream()
        for s in (self.s_in, self.s_out):
            ev = torch.cuda.Event()
            ev.record(s)
            cur.wait_event(ev)

    def drain(self) -> None:
        """Wait for everything queued and raise if a device-side wait ran out on the way (under
        tensor parallelism: a barrier between the ranks that a peer never reached)."""
        from . import ops

        self.s_in.synchronize()
        self.s_out.synchronize()
        torch.cuda.current_stream().synchronize()
        ops.check_status()
