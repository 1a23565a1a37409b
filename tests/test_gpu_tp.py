"""Tensor-parallel layer on two GPUs (skipped on a single-GPU box): each rank runs the rank-7
chain on its shard; the partials are combined by one NCCL all-reduce, by the slab-pipelined
all-reduce, and by this package's own exchange over peer memory (push from the GEMM kernel,
barrier, reduce + gather); all must match the unsharded layer and the functional reference."""
import os
import socket

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    import sys
    from pathlib import Path

    repo = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(repo / "writes-that-matter_b200"), str(repo)]
    import torch.distributed as dist
    from lcgemm import ops, tp
    from lcgemm.layer import DenseMlpLayer, Rank7MlpLayer

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        g = torch.Generator().manual_seed(3)
        m, h, i = 1024, 512, 2048
        mk = lambda shape, scale=1.0: (torch.randn(shape, generator=g) * scale).to(torch.bfloat16).to(dev)
        x, nw, wgu, wd = mk((m, h)), mk((h,), 0.01), mk((2 * i, h), 0.02), mk((h, i), 0.02)
        gu_shard, d_shard = tp.shard_mlp_weights(wgu, wd, rank, world)
        layer = tp.TensorParallelMlp(m, nw, gu_shard, d_shard, 1e-6)
        out = layer(x).clone()
        out2 = layer(x).clone()                       # buffers are reused: a second pass must agree
        piped = tp.TensorParallelMlp(m, nw, gu_shard, d_shard, 1e-6, slabs=2)
        out3 = piped(x).clone()                       # down in two slabs, all-reduce overlapped
        out3 = piped(x).clone()
        fused = tp.TensorParallelMlp(m, nw, gu_shard, d_shard, 1e-6, fused=True)
        out4 = fused(x).clone()                       # exchange in this package's own kernels
        out4 = fused(x).clone()
        # a second layer object on the SAME symmetric buffers (layers of a model share one exchange)
        fused_b = tp.TensorParallelMlp(m, nw, gu_shard, d_shard, 1e-6, fused=True, exchange=fused.exchange)
        out5 = fused_b(out4.clone(), x).clone()       # a second layer call on the other slot set
        ref5 = layer(out4.clone(), x).clone()
        # every rank must hold the same bits: the owners sum in rank order and store one result
        theirs = [torch.empty_like(out4) for _ in range(world)]
        dist.all_gather(theirs, out4)
        ranks_equal = all(torch.equal(t, out4) for t in theirs)
        rel = lambda a, b: ((a.float() - b.float()).norm() / b.float().norm()).item()
        # host-to-host streaming: every rank feeds its rows of the batch and gets its rows back
        from lcgemm.streaming import HostStreamedLayer
        rows = m // world
        xs = x[rank * rows:(rank + 1) * rows].cpu().pin_memory()
        streamed = 0.0
        for gather in ("copy", "nccl"):      # rows replicated by DMA copies + barrier, or by the library
            st = HostStreamedLayer(fused, m, h, group=dist.group.WORLD, gather=gather)
            got = [torch.zeros_like(xs).pin_memory() for _ in range(5)]
            st.begin()
            for o in got:
                st.submit(xs, o)
            st.end()
            st.drain()
            streamed = max([streamed] + [rel(o.to(dev), out4[rank * rows:(rank + 1) * rows]) for o in got])
        # the fused layer recorded into CUDA graphs (one per receive-region set), replayed
        cap = tp.CapturedTensorParallel(fused, x)
        captured = max(rel(cap().clone(), out4) for _ in range(3))
        captured_branch = max(rel(cap().clone().float() - x.float(), out4.float() - x.float()) for _ in range(2))
        full = Rank7MlpLayer(m, nw, wgu, wd, 1e-6)(x)
        dense = DenseMlpLayer(m, nw, wgu, wd, 1e-6, gemm="cublas")(x)
        ops.check_status()
        branch = lambda y: y.float() - x.float()
        ret[rank] = (rel(out, full), rel(branch(out), branch(dense)), rel(out2, out), rel(out3, out),
                     rel(out4, out), rel(out5, ref5), streamed, captured,
                     rel(branch(out4), branch(out)), ranks_equal, captured_branch)
    finally:
        dist.destroy_process_group()


def test_two_gpu_tensor_parallel_layer():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(2, port, ret), nprocs=2, join=True)
        assert len(ret) == 2
        for rank in range(2):
            (vs_full, branch_vs_dense, repeat, piped, fused, fused_next, streamed, captured,
             fused_branch, ranks_equal, captured_branch) = ret[rank]
            # the MLP branch (output minus residual) is ~9 % of the output here, so the bounds on
            # the whole output are loose on the branch; these are on the branch itself
            # (both outputs are rounded to bf16 at the residual's magnitude, which alone is ~1.5 % of
            # this branch; the whole-output bound above allows 4-5 %)
            assert fused_branch < 2.5e-2, (rank, fused_branch)   # fp32 sum of partials vs bf16 all-reduce
            assert ranks_equal, rank                              # all ranks hold identical bits
            # graph replay vs eager launches of the same kernels: the split tail of the push GEMM adds
            # into C in an order the hardware picks, so equal up to that, not bit for bit
            assert captured_branch < 2.5e-2, (rank, captured_branch)     # same rounding argument as above
            assert captured < 4e-3, (rank, captured)
            assert streamed < 4e-3, (rank, streamed)
            assert piped < 4e-3, (rank, piped)
            assert fused < 4e-3, (rank, fused)                   # fp32 sum of the partials vs bf16
            assert fused_next < 4e-3, (rank, fused_next)
            assert vs_full < 4e-3, (rank, vs_full)               # residual-dominated output
            assert branch_vs_dense < 5e-2, (rank, branch_vs_dense)
            assert repeat < 4e-3, (rank, repeat)
        assert ret[0][:9] == pytest.approx(ret[1][:9], rel=0.5, abs=1e-3)
