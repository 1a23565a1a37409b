"""The chained ``down`` seam: a plane-consuming rank-7 GEMM (``lcgemm/seams/down.py``).

    S = silu(Z[:, :I]) * Z[:, I:]        # never lands in HBM as such
    out = S @ W_down^T

The ``gate_up`` epilogue has already applied SwiGLU and written the A planes, so this seam
launches only the GEMM.  Its static weight is permuted into the interleaved-K gauge once,
at installation.
"""
from __future__ import annotations

import math

import torch

from .. import chain_gauge, ops
from .._native import SCHEDULE_ALL_RANKS, SCHEDULE_HYBRID, SCHEDULE_RANK_SPLIT
from ..scheme import Scheme

# Shapes the reference runs rank-split (lcgemm/seams/down.py:42-54); kept as the validated set.
RANK_SPLIT_SHAPES = {
    (512, 19968, 6656), (512, 17408, 5120), (1024, 19968, 6656), (1024, 17408, 5120),
    (2048, 19968, 6656), (2048, 17408, 5120), (4096, 17408, 5120), (8192, 17408, 5120),
}

# Measured exceptions to the rank-split rule: whole waves of tiles walked product by product with
# only the last partial wave split (8192 tokens: 867 us against 888 us rank-split, chained).
HYBRID_SHAPES = {(8192, 17408, 5120)}

_CTA_GROUPS = 74            # 2-CTA groups resident on a 148-SM B200
_SPLIT_PENALTY = 0.97       # reduce-add scatter and pre-zeroing cost of the rank-split form


def wants_rank_split(shape) -> bool:
    """Whether the product index has to carry parallelism: compare the wave-quantisation
    efficiency of ``tiles`` units against ``7 * tiles`` units on the resident CTA groups."""
    if tuple(shape) in HYBRID_SHAPES:
        return False
    if tuple(shape) in RANK_SPLIT_SHAPES:
        return True
    m, _, n = shape
    tiles = math.ceil((m + 1) // 2 / 256) * math.ceil(((n + 1) // 2) / 256)
    eff = lambda units: units / (math.ceil(units / _CTA_GROUPS) * _CTA_GROUPS)
    return eff(7 * tiles) * _SPLIT_PENALTY > eff(tiles)


class DownPlan:
    """The ``down`` plan, coupled to its ``gate_up`` producer."""

    seam = "down"

    def __init__(self, scheme: Scheme, shape, *, producer, cta_group: int = 0):
        m, k, n = shape
        if k % 128:
            raise ValueError(f"down shape {tuple(shape)}: K must be a multiple of 128 (the gauge width)")
        self.scheme = scheme
        self.shape = tuple(shape)                       # (M, K, N)
        self.producer = producer
        self.cta_group = cta_group
        dev = torch.device("cuda", torch.cuda.current_device())
        self._store = torch.empty((m, (n + 7) // 8 * 8), device=dev, dtype=torch.bfloat16)
        self.c = self._store[:, :n] if n % 8 else self._store
        if wants_rank_split(self.shape):
            self.schedule = SCHEDULE_RANK_SPLIT
        else:
            self.schedule = SCHEDULE_HYBRID if self.shape in HYBRID_SHAPES else SCHEDULE_ALL_RANKS
        self._desc = None

    @property
    def rank_split(self) -> bool:
        """Whether every contribution is a reduce-add into an output that must arrive zeroed
        (``lcgemm/seams/down.py:67-68`` of the reference)."""
        return self.schedule == SCHEDULE_RANK_SPLIT

    @rank_split.setter
    def rank_split(self, value: bool) -> None:
        self.schedule = SCHEDULE_RANK_SPLIT if value else SCHEDULE_ALL_RANKS

    # ---------------------------------------------------------------- offline
    def prepare_weight(self, w: torch.Tensor) -> torch.Tensor:
        """The R combined B planes with the K permutation of the gauge folded in."""
        return chain_gauge.prepare_down_b(w, self.scheme, chain_gauge.CHUNK)

    # ------------------------------------------------------------------ parts
    def a_planes(self) -> torch.Tensor:
        """The planes already produced by the chained gate/up epilogue."""
        return self.producer.planes

    def gemm(self, a_planes, prepared_w, *, out=None) -> torch.Tensor:
        c = self.c if out is None else out
        m, k, n = self.shape
        # A rank-split output must arrive zeroed.  The chained producer does that for ``self.c``
        # while it runs; any other destination is cleared here.
        cleared_by_producer = (self.producer is not None and c is self.c
                               and getattr(self.producer, "preclear", None) is self.c)
        ops.gemm_r7_planes(
            self.scheme, a_planes, prepared_w, m, n, k, out=c, schedule=self.schedule,
            cta_group=self.cta_group, zero_out=self.rank_split and not cleared_by_producer)
        return c

    # ------------------------------------------------------- slabs (tensor parallel)
    TILE_ROWS = 256          # rows of a block row per tile row (2-CTA pairing)

    @property
    def tile_rows(self) -> int:
        """Tile rows of one block row of the output."""
        return -(-((self.shape[0] + 1) // 2) // self.TILE_ROWS)

    def slab_rows(self, tile_range):
        """The two output row ranges (one per block row) a slab of tile rows covers."""
        m2 = (self.shape[0] + 1) // 2
        t0, t1 = tile_range
        return [(i * m2 + t0 * self.TILE_ROWS, min(i * m2 + t1 * self.TILE_ROWS, min((i + 1) * m2, self.shape[0])))
                for i in range(2)]

    def gemm_slab(self, a_planes, prepared_w, tile_range, *, max_groups: int = 0) -> torch.Tensor:
        """The tile rows ``tile_range`` of the product into ``self.c`` (which a rank-split plan
        expects zeroed, as the chained producer leaves it); used to pipeline ``down`` with the
        all-reduce of the previous slab."""
        m, k, n = self.shape
        ops.gemm_r7_slab(self.scheme, a_planes, prepared_w, m, n, k, self.c, tile_range,
                         schedule=self.schedule, max_groups=max_groups, cta_group=2)
        return self.c

    def __call__(self, *, prepared_w, out=None):
        return self.gemm(self.a_planes(), prepared_w, out=out)

    def describe(self) -> str:
        if self._desc is None:
            m, k, n = self.shape
            self._desc = "  chained (a_planes are free)\n" + ops.describe_gemm(
                m, n, k, True, self.schedule, self.cta_group)
        return self._desc
