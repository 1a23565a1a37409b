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
``tokens / tp`` rows in, replicates them over NVLink, and copies only its own rows of the result
out: the batch crosses PCIe once in each direction in total.  The replication is part of the
copy-in stage, not of the compute: with ``gather="copy"`` (the default when the ranks share a
node) every rank's input buffers are symmetric-memory allocations and a rank stores its rows into
each peer's buffer with one device-to-device copy per peer on the copy-in stream (DMA engines over
NVLink, no SMs, overlapped with the previous batch's compute); a barrier between the ranks on the
compute stream (``lcg_peer_barrier``, bounded wait) then says that every rank's rows have landed.
``gather="nccl"`` keeps the library all-gather on the compute stream.
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

    def __init__(self, layer, tokens: int, hidden: int, device=None, group=None, depth: int = 2,
                 timeline: bool = False, gather: str = "copy"):
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.layer, self.depth, self.group = layer, depth, group
        self.world = dist.get_world_size(group) if (group is not None or (
            dist.is_available() and dist.is_initialized())) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        if tokens % self.world:
            raise ValueError(f"{tokens} tokens do not split over {self.world} ranks")
        self.rows = tokens // self.world
        bf = torch.bfloat16
        if gather not in ("copy", "nccl"):
            raise ValueError("gather must be 'copy' or 'nccl'")
        self.gather = gather if self.world > 1 else None
        self.peer_rows = None
        if self.gather == "copy":
            import os

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")     # plain peer copies only
            import torch.distributed._symmetric_memory as symm

            grp = group if group is not None else dist.group.WORLD
            self.x_dev = [symm.empty((tokens, hidden), dtype=bf, device=dev) for _ in range(depth)]
            self._flags = symm.empty((16,), dtype=torch.int32, device=dev)
            self._flags.zero_()
            handles = [symm.rendezvous(t, grp) for t in (*self.x_dev, self._flags)]
            # peer_rows[i][p]: this rank's row slice inside rank p's i-th input buffer
            off = self.rank * self.rows * hidden
            self.peer_rows = [[h.get_buffer(p, (self.rows, hidden), bf, off) for p in range(self.world)]
                              for h in handles[:depth]]
            self._flag_ptrs = [int(q) for q in handles[depth].buffer_ptrs]
            self._handles = handles
            torch.cuda.synchronize(dev)
            dist.barrier(grp)            # every rank's flags are zero before the first peer barrier
        else:
            self.x_dev = [torch.empty((tokens, hidden), device=dev, dtype=bf) for _ in range(depth)]
        self.x_in = ([torch.empty((self.rows, hidden), device=dev, dtype=bf) for _ in range(depth)]
                     if self.world > 1 else self.x_dev)
        self.out_dev = [torch.empty((self.rows, hidden), device=dev, dtype=bf) for _ in range(depth)]
        self.s_in, self.s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        mk = lambda: [torch.cuda.Event() for _ in range(depth)]
        self.x_ready, self.x_free, self.out_ready, self.out_free = mk(), mk(), mk(), mk()
        self.n = 0
        # With `timeline`, every step records timed events at the start and end of its copy in,
        # its compute (all-gather + layer + slice copy) and its copy out; `timeline_summary`
        # turns them into durations and the overlap between neighbouring steps.
        self.timeline = [] if timeline else None

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
        ev = None
        if self.timeline is not None:
            ev = {k: torch.cuda.Event(enable_timing=True) for k in
                  ("in0", "in1", "c0", "gathered", "c1", "out0", "out1")}
            self.timeline.append(ev)
        with torch.cuda.stream(self.s_in):
            if ev:
                ev["in0"].record()
            self.x_in[i].copy_(x_host, non_blocking=True)
            if self.gather == "copy":
                # Safe to overwrite the peers' buffer i: a rank frees it only after its layer call,
                # whose closing barrier every rank passes after all of them have read their input.
                # Rank r copies to r + 1, r + 2, ... and to itself last: at any moment every rank's
                # inbound link carries one copy (all ranks copying to peer 0 first, then to peer 1, would
                # queue the whole replication behind one link at a time).
                for j in range(1, self.world + 1):
                    p = (self.rank + j) % self.world
                    self.peer_rows[i][p].copy_(self.x_in[i], non_blocking=True)
            if ev:
                ev["in1"].record()
            self.x_ready[i].record()
        compute.wait_event(self.x_ready[i])
        if ev:
            ev["c0"].record(compute)
        if self.gather == "copy":
            from . import ops

            ops.peer_barrier(self._flag_ptrs, self.rank, 0)       # every rank's rows have landed here
        elif self.world > 1:
            dist.all_gather_into_tensor(self.x_dev[i], self.x_in[i], group=self.group)
        if ev:
            ev["gathered"].record(compute)
        out = self.layer(self.x_dev[i])
        self.x_free[i].record(compute)
        if out_host is None:
            if ev:
                ev["c1"].record(compute)
            return
        if not first_use:
            compute.wait_event(self.out_free[i])          # its previous content has left the GPU
        r0 = self.rank * self.rows
        self.out_dev[i].copy_(out[r0:r0 + self.rows])
        self.out_ready[i].record(compute)
        if ev:
            ev["c1"].record(compute)
        self.s_out.wait_event(self.out_ready[i])
        with torch.cuda.stream(self.s_out):
            if ev:
                ev["out0"].record()
            out_host.copy_(self.out_dev[i], non_blocking=True)
            if ev:
                ev["out1"].record()
            self.out_free[i].record()

    def end(self) -> None:
        """Make the current stream wait for every copy queued so far (no host synchronisation)."""
        cur = torch.cuda.current_stream()
        for s in (self.s_in, self.s_out):
            ev = torch.cuda.Event()
            ev.record(s)
            cur.wait_event(ev)

    def timeline_summary(self, skip: int = 2) -> dict:
        """Mean durations (ms) over the recorded steps after the first `skip`: copy in, all-gather,
        layer + slice copy, copy out, the period between the starts of neighbouring steps' compute,
        and how long the compute stream sat idle between one step's end and the next one's start."""
        if not self.timeline:
            return {}
        self.drain()
        steps = [e for e in self.timeline[skip:] if "out1" in e]
        if len(steps) < 2:
            return {}
        mean = lambda v: sum(v) / len(v)
        dur = lambda a, b: mean([e[a].elapsed_time(e[b]) for e in steps])
        period = mean([steps[j]["c0"].elapsed_time(steps[j + 1]["c0"]) for j in range(len(steps) - 1)])
        idle = mean([steps[j]["c1"].elapsed_time(steps[j + 1]["c0"]) for j in range(len(steps) - 1)])
        return {"steps": len(steps), "h2d_ms": dur("in0", "in1"), "all_gather_ms": dur("c0", "gathered"),
                "layer_ms": dur("gathered", "c1"), "d2h_ms": dur("out0", "out1"),
                "compute_period_ms": period, "compute_idle_ms": idle}

    def drain(self) -> None:
        """Wait for everything queued and raise if a device-side wait ran out on the way (under
        tensor parallelism: a barrier between the ranks that a peer never reached)."""
        from . import ops

        self.s_in.synchronize()
        self.s_out.synchronize()
        torch.cuda.current_stream().synchronize()
        ops.check_status()
