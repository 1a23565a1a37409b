"""The tensor-parallel plumbing on CPU: two ``gloo`` ranks drive ``TensorParallelMlp`` with a
CPU stand-in for the per-rank layer (the oracle's functional MLP on the rank's shard) and must
reproduce the unsharded layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import lc_oracle as O


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _CpuLayer:
    """Per-rank layer on the CPU: the functional reference applied to the shard."""

    def __init__(self, tokens, norm_weight, gate_up_shard, down_shard, eps):
        self.args = (norm_weight, gate_up_shard, down_shard, eps)

    def chain(self, delta, residual):
        nw, wgu, wd, eps = self.args
        return O.mlp_reference(delta, residual, nw, wgu, wd, eps)


class _CpuLayerSingleInput(_CpuLayer):
    """A layer that takes a call without a delta itself (as the CUDA layers do): the residual
    stream it hands back is then its input."""

    accepts_no_delta = True

    def chain(self, delta, residual):
        self.saw_delta = delta is not None
        if delta is None:
            out, _ = super().chain(torch.zeros_like(residual), residual)
            return out, residual
        return super().chain(delta, residual)


def _worker(rank, world, port, ret):
    import sys
    from pathlib import Path

    repo = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(repo / "writes-that-matter_b200"), str(repo)]
    from lcgemm import tp

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        m, h, i = 32, 128, 256
        x = torch.randn(m, h, generator=g).to(torch.bfloat16)
        nw = (torch.randn(h, generator=g) * 0.01).to(torch.bfloat16)
        wgu = (torch.randn(2 * i, h, generator=g) * 0.02).to(torch.bfloat16)
        wd = (torch.randn(h, i, generator=g) * 0.02).to(torch.bfloat16)
        gu_shard, d_shard = tp.shard_mlp_weights(wgu, wd, rank, world)
        assert gu_shard.shape == (2 * i // world, h) and d_shard.shape == (h, i // world)
        seen = {}

        def add(a, b):
            seen["reduced"] = b.clone()
            return (a.float() + b.float()).to(torch.bfloat16)

        layer = tp.TensorParallelMlp(m, nw, gu_shard, d_shard, 1e-6, make_layer=_CpuLayer, add=add)
        out = layer(x)
        full, href = O.mlp_reference(torch.zeros_like(x), x, nw, wgu, wd, 1e-6)
        want = add(href, full)
        err = ((out.float() - want.float()).norm() / want.float().norm()).item()
        mlp_err = ((seen["reduced"].float() - full.float()).norm() / full.float().norm()).item()
        # a layer that says it takes a missing delta gets None, not a zeros tensor; same result
        single = tp.TensorParallelMlp(m, nw, gu_shard, d_shard, 1e-6, make_layer=_CpuLayerSingleInput, add=add)
        out1 = single(x)
        assert single.layer.saw_delta is False and torch.equal(out1, out)
        single(x, torch.zeros_like(x))
        assert single.layer.saw_delta is True
        assert layer._zero is not None and single._zero is None
        ret[rank] = (err, mlp_err)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_rank_gloo_matches_unsharded(world):
    port = _free_port()
    with mp.Manager() as mgr:
        ret = mgr.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert len(ret) == world
        for rank in range(world):
            err, mlp_err = ret[rank]
            assert err < 2e-3, (rank, err)
            # each rank rounds its partial to bf16 before the sum
            assert mlp_err < 1.5e-2, (rank, mlp_err)


def test_shard_errors():
    import sys
    from lcgemm import tp

    wgu, wd = torch.zeros(12, 4), torch.zeros(4, 6)
    with pytest.raises(ValueError):
        tp.shard_mlp_weights(wgu, wd, 0, 4)
    with pytest.raises(ValueError):
        tp.shard_mlp_weights(wgu, wd, 3, 3)
    g, d = tp.shard_mlp_weights(wgu, wd, 1, 3)
    assert g.shape == (4, 4) and d.shape == (4, 2)
    # without a process group the reduction is the identity
    t = torch.ones(3)
    assert tp.all_reduce_sum(t) is t


def test_owner_arithmetic_of_the_peer_exchange():
    from lcgemm import tp

    assert tp.rows_per_owner(8192, 8) == 1024 and tp.rows_per_owner(1030, 8) == 129
    assert tp.owner_of_row(0, 1030, 8) == 0 and tp.owner_of_row(1029, 1030, 8) == 7
    assert tp.owner_of_row(128, 1030, 8) == 0 and tp.owner_of_row(129, 1030, 8) == 1
    # every row has exactly one owner and owners hold contiguous ranges
    for tokens, world in ((4096, 3), (4096, 4), (1030, 8), (7, 8)):
        owners = [tp.owner_of_row(r, tokens, world) for r in range(tokens)]
        assert owners == sorted(owners) and 0 <= owners[0] and owners[-1] < world
