"""Tensor-parallel MLP over the intermediate dimension (2 / 4 / 8 GPUs of one node).

The reference enforces TP = 1 (``lcgemm/integrate/qwen_patch.py:216-217``); this is the
multi-GPU form of the same layer.  Rank ``g`` of ``tp`` holds

* ``gate_up`` shard ``[W_gate[g*I/tp:(g+1)*I/tp]; W_up[g*I/tp:(g+1)*I/tp]]`` -- column
  parallel, and still ``[gate | up]`` halves, which is what the chained kernel's SwiGLU
  epilogue needs (``lcgemm/kernels/sm100.py:239-241``);
* ``down`` shard ``W_down[:, g*I/tp:(g+1)*I/tp]`` -- row parallel.

Each rank runs the whole rank-7 chain on its shard with no communication (the input is
replicated), producing a partial ``(M, H)`` output; an all-reduce (NCCL over
NVLink/NVSwitch, bf16 sum) per layer combines the partials, and the residual is added after
the reduction.  One process per GPU; ``torch.distributed`` provides the process group.

With ``slabs > 1`` the row-parallel ``down`` GEMM is issued as that many slabs of tile rows and
the all-reduce of each finished slab (two row ranges, one per block row) runs asynchronously
while the next slab computes; the GEMM then leaves ``reserve_groups`` CTA pairs' worth of SMs
free, because one of its CTAs fills an SM's shared memory and NCCL's kernels could not start
beside it.

With ``fused=True`` the exchange runs in this package's own kernels over peer memory instead of
the library all-reduce.  Row ``g`` of the output belongs to rank ``g // ceil(M / tp)``.  Each
rank's ``down`` GEMM copies every finished tile, from inside the GEMM kernel, into the owner's
receive region over NVLink (the reduce-scatter half, hidden under the GEMM); after a barrier
each owner sums the ``tp`` partials and the residual in fp32 and stores the finished rows into
every rank's output (the all-gather half), and a second barrier closes the layer.  The buffers
are ``torch.distributed._symmetric_memory`` allocations; the receive regions are double-buffered
so that a fast rank's next layer cannot overwrite what a slow owner is still reading.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_mlp_weights(gate_up_weight: torch.Tensor, down_weight: torch.Tensor, rank: int, world: int):
    """The ``(gate_up_shard, down_shard)`` of one rank from full weights ``(2I, H)``, ``(H, I)``."""
    two_i = gate_up_weight.shape[0]
    inter = two_i // 2
    if two_i % 2 or inter % world or down_weight.shape[1] != inter:
        raise ValueError(f"intermediate size {inter} does not split over {world} ranks")
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside [0, {world})")
    per = inter // world
    lo, hi = rank * per, (rank + 1) * per
    gate_up = torch.cat([gate_up_weight[lo:hi], gate_up_weight[inter + lo:inter + hi]], dim=0)
    return gate_up.contiguous(), down_weight[:, lo:hi].contiguous()


def all_reduce_sum(t: torch.Tensor, group=None) -> torch.Tensor:
    """In-place sum over the group; a no-op without an initialised group or with one rank."""
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=group)
    return t


def rows_per_owner(tokens: int, world: int) -> int:
    """Rows each rank owns in the fused exchange (the last owner may hold fewer)."""
    return -(-tokens // world)


def owner_of_row(row: int, tokens: int, world: int) -> int:
    return row // rows_per_owner(tokens, world)


class PeerExchange:
    """The symmetric buffers of one tensor-parallel group and their peer addresses.

    ``slots[b]``: ``(world, rows_per_owner, hidden)`` receive regions (two, used in turn);
    ``out``: the ``(tokens, hidden)`` layer output every owner writes its rows into;
    ``flags``: sixteen words per rank for the barrier (eight peers, the call counter).  ``slot_ptrs[b][o]`` is the address, in
    owner ``o``'s memory, of the region reserved for this rank.
    """

    def __init__(self, tokens: int, hidden: int, group=None, device=None):
        import os

        # Only plain peer loads and stores are used here: no multicast object is needed.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm

        group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.tokens, self.hidden = tokens, hidden
        if self.world > 8:
            raise ValueError("the peer exchange supports at most 8 ranks")
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.rows = rows_per_owner(tokens, self.world)
        elem = 2
        self.slots = [symm.empty((self.world, self.rows, hidden), dtype=torch.bfloat16, device=dev)
                      for _ in range(2)]
        self.out = symm.empty((tokens, hidden), dtype=torch.bfloat16, device=dev)
        self.flags = symm.empty((16,), dtype=torch.int32, device=dev)
        self.flags.zero_()
        handles = [symm.rendezvous(t, group) for t in (*self.slots, self.out, self.flags)]
        mine = self.rank * self.rows * hidden * elem
        self.slot_ptrs = [[int(p) + mine for p in h.buffer_ptrs] for h in handles[:2]]
        self.out_ptrs = [int(p) for p in handles[2].buffer_ptrs]
        self.flag_ptrs = [int(p) for p in handles[3].buffer_ptrs]
        self._handles = handles
        self.turn = 0
        torch.cuda.synchronize(dev)
        dist.barrier(group)          # every rank's flags are zero before the first peer barrier

    def barrier(self):
        """Epochs are counted on the device, so a recorded layer call can be replayed."""
        from . import ops

        ops.peer_barrier(self.flag_ptrs, self.rank, 0)


class TensorParallelMlp:
    """``h + all_reduce(down_g(SwiGLU(gate_up_g(norm(h)))))`` with ``h = x + delta``.

    ``make_layer(tokens, norm_weight, gate_up_shard, down_shard, eps)`` builds the per-rank
    layer; it must offer ``chain(delta, residual) -> (partial, h)``.  The default is the
    rank-7 chain of this package; tests pass a CPU stand-in to drive the same control flow
    over a ``gloo`` group.
    """

    def __init__(self, tokens: int, norm_weight, gate_up_shard, down_shard, eps: float = 1e-6,
                 group=None, make_layer=None, add=None, slabs: int = 1, reserve_groups: int = 8,
                 fused: bool = False, exchange: "PeerExchange | None" = None):
        if make_layer is None:
            from .layer import Rank7MlpLayer as make_layer
        self.group = group
        self.layer = make_layer(tokens, norm_weight, gate_up_shard, down_shard, eps)
        self._add = add
        self._zero = None
        self.out = None
        self.slabs = max(1, int(slabs))
        self.reserve_groups = reserve_groups
        self.exchange = None
        if fused:
            if not (dist.is_available() and dist.is_initialized()):
                raise RuntimeError("fused tensor parallelism needs an initialised process group")
            down = self.layer.down_plan
            m, _, n = down.shape
            if n % 8 or not down.c.is_contiguous():
                raise ValueError("the fused exchange needs a hidden size that is a multiple of 8")
            # The symmetric buffers (3 * tokens * hidden * 2 bytes) may be shared by all the layers of
            # a model that run one after the other on ONE stream: the second barrier of a layer call
            # orders every rank's reads of the receive regions before the next call's pushes.
            if exchange is not None and (exchange.tokens, exchange.hidden) != (m, n):
                raise ValueError(f"the shared exchange is for {(exchange.tokens, exchange.hidden)}, "
                                 f"this layer needs {(m, n)}")
            self.exchange = exchange if exchange is not None else PeerExchange(m, n, group)
            gate = self.layer.gate_plan
            gate.preclear = gate.c                   # nothing to clear: the push GEMM initialises its output

    def forward(self, x: torch.Tensor, delta: torch.Tensor | None = None) -> torch.Tensor:
        if delta is None and not getattr(self.layer, "accepts_no_delta", False):
            if self._zero is None or self._zero.shape != x.shape:
                self._zero = torch.zeros_like(x)
            delta = self._zero
        if self.exchange is not None:
            return self._forward_fused(x, delta)
        if self.slabs > 1 and hasattr(self.layer, "down_plan") and self.layer.down_plan.c.is_contiguous():
            return self._forward_pipelined(x, delta)
        partial, h = self.layer.chain(delta, x)
        if not partial.is_contiguous():
            partial = partial.contiguous()
        all_reduce_sum(partial, self.group)
        if self._add is not None:
            self.out = self._add(h, partial)
        else:
            from . import ops

            if self.out is None or self.out.shape != h.shape:
                self.out = torch.empty_like(h)
            ops.add(h, partial, out=self.out)
        return self.out

    def _forward_fused(self, x, delta):
        """Nothing here synchronises, so a barrier wait that ran out (status code 106: a rank that
        never arrived) does not raise from this call; the owners then reduce receive regions
        that are not complete.  Callers check ``ops.check_status()`` at a step boundary before
        they use the output (``HostStreamedLayer.drain`` and ``bench.py`` do)."""
        from . import ops

        lay, ex = self.layer, self.exchange
        gate, down = lay.gate_plan, lay.down_plan
        gate(x, delta, lay.norm_weight, lay.eps, prepared_w=lay.gate_bw)
        m, k, n = down.shape
        b = ex.turn
        ex.turn ^= 1
        ops.gemm_r7_push(down.scheme, down.a_planes(), lay.down_bw, m, n, k, down.c, ex.slot_ptrs[b],
                         ex.rank, ex.rows, cta_group=down.cta_group)
        ex.barrier()                 # every rank's pushes have landed
        h = x if delta is None else gate.residual_out      # without a delta the residual stream is x
        ops.reduce_gather(ex.slots[b], h, ex.out_ptrs, ex.rows, ex.rank)
        ex.barrier()                 # every owner's rows have landed here
        self.out = ex.out
        return self.out

    def _forward_pipelined(self, x, delta):
        from . import ops

        lay = self.layer
        gate, down = lay.gate_plan, lay.down_plan
        gate(x, delta, lay.norm_weight, lay.eps, prepared_w=lay.gate_bw)   # also zeroes down.c
        h = x if delta is None else gate.residual_out
        if down.rank_split and gate.preclear is not down.c:
            down.c.zero_()
        total = down.tile_rows
        slabs = min(self.slabs, total)
        edges = [round(s * total / slabs) for s in range(slabs + 1)]
        distributed = dist.is_available() and dist.is_initialized() and dist.get_world_size(self.group) > 1
        max_groups = max(1, 74 - self.reserve_groups) if distributed else 0
        pending = []
        for s in range(slabs):
            down.gemm_slab(down.a_planes(), lay.down_bw, (edges[s], edges[s + 1]), max_groups=max_groups)
            if distributed:
                for r0, r1 in down.slab_rows((edges[s], edges[s + 1])):
                    if r1 > r0:
                        pending.append(dist.all_reduce(down.c[r0:r1], op=dist.ReduceOp.SUM,
                                                       group=self.group, async_op=True))
        for work in pending:
            work.wait()
        if self.out is None or self.out.shape != h.shape:
            self.out = torch.empty_like(h)
        ops.add(h, down.c, out=self.out)
        return self.out

    __call__ = forward


class CapturedTensorParallel:
    """A fused tensor-parallel layer call as CUDA graphs: one replay per step.  The receive
    regions are used in turn, so two recordings are kept (one per region set) and replayed
    alternately; the barriers count their epochs on the device.  Every rank records and
    replays in the same order."""

    def __init__(self, layer: TensorParallelMlp, x: torch.Tensor, warmup: int = 2):
        if layer.exchange is None:
            raise ValueError("only the fused exchange (its own kernels, no library collective) is recorded")
        self.layer, self.x = layer, x
        side = torch.cuda.Stream(x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):
            for _ in range(2 * warmup):
                layer(x)
        torch.cuda.current_stream(x.device).wait_stream(side)
        torch.cuda.synchronize(x.device)
        self.graphs = []
        for _ in range(2):
            self.graphs.append((layer.exchange.turn, torch.cuda.CUDAGraph()))
            with torch.cuda.graph(self.graphs[-1][1]):
                self.out = layer(x)
        self.n = 0

    def __call__(self) -> torch.Tensor:
        self.graphs[self.n & 1][1].replay()
        self.n += 1
        return self.out
