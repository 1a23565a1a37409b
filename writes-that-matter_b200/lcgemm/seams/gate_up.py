"""The MLP entry seam: ``norm(residual + delta) -> gate_up_proj`` (``lcgemm/seams/gate_up.py``).

Two launches:

1. the fused residual + RMSNorm + A-plane kernel reads ``residual`` and ``delta`` and writes
   the R A planes plus the new residual stream; the normalised activations never land;
2. the chained rank-7 GEMM computes the R products into ``Z`` and, one tile behind its
   mainloop, emits the ``down`` seam's A planes ``L_r(SwiGLU(Z))`` in the interleaved gauge
   and zeroes the consumer's output when that consumer is rank-split.
"""
from __future__ import annotations

import torch

from .. import ops, planes as lc_planes
from .._native import SCHEDULE_ALL_RANKS, SCHEDULE_HYBRID
from ..scheme import Scheme


class GateUpPlan:
    """The ``gate_up`` producer with its chained plane epilogue.  Owns its buffers; results
    are views of plan storage, valid until the next call."""

    seam = "gate_up"

    def __init__(self, scheme: Scheme, shape, *, plane_scheme: Scheme, cta_group: int = 0,
                 schedule: int = SCHEDULE_HYBRID):
        m, k, n = shape
        if m % 2 or n % 256 or k % 128:
            raise ValueError(
                f"gate_up shape {tuple(shape)} does not fit the chained kernel: it needs an even M, "
                f"N % 256 == 0 (the gate/up split and the 128-wide gauge) and K % 128 == 0")
        self.scheme = scheme
        self.shape = tuple(shape)                       # (M, K, N)
        self.plane_scheme = plane_scheme
        self.cta_group = cta_group
        # Hybrid: whole waves walk all products per tile, the last partial wave is split by
        # product (the role of the reference's per-shape tail policies, lcgemm/seams/gate_up.py:42-68).
        self.schedule = schedule
        dev = torch.device("cuda", torch.cuda.current_device())
        bf = torch.bfloat16
        self.a = torch.empty(ops.a_plane_shape(scheme, m, k), device=dev, dtype=bf)
        self.c = torch.empty((m, n), device=dev, dtype=bf)
        self.residual_out = torch.empty((m, k), device=dev, dtype=bf)
        # down's A planes: N/2 columns after SwiGLU, halved again by the K split.
        self.planes = torch.empty((plane_scheme.rank * (m // 2), (n // 2) // 2), device=dev, dtype=bf)
        # The consumer's output when it must arrive zeroed; ``self.c`` means "nothing to clear".
        self.preclear = self.c
        # What that output starts from instead of zero (the residual stream, when the layer folds
        # its closing add into the consumer's reduce-adds); None: zero.
        self.init_from = None
        self._desc = None

    # ---------------------------------------------------------------- offline
    def prepare_weight(self, w: torch.Tensor) -> torch.Tensor:
        return lc_planes.prepare_b(w, self.scheme)

    # ------------------------------------------------------------------ parts
    def a_planes(self, residual, delta, norm_weight, eps, *, residual_out=None) -> torch.Tensor:
        """``L_r(RMSNorm(residual + delta))`` as ``(R * M/2, K/2)``; also writes the residual stream."""
        r = self.residual_out if residual_out is None else residual_out
        ops.norm_planes(self.scheme, delta, residual, norm_weight, eps, r, self.a)
        return self.a

    def gemm(self, a_planes, prepared_w, *, out=None) -> torch.Tensor:
        c = self.c if out is None else out
        ops.gate_up_chain(self.scheme, self.plane_scheme, a_planes, prepared_w, c, self.planes,
                          preclear=None if self.preclear is self.c else self.preclear,
                          schedule=self.schedule, cta_group=self.cta_group,
                          init_from=None if self.preclear is self.c else self.init_from)
        return c

    def __call__(self, *pre_inputs, prepared_w, out=None, residual_out=None):
        a = self.a_planes(*pre_inputs, residual_out=residual_out)
        return self.gemm(a, prepared_w, out=out)

    def describe(self) -> str:
        if self._desc is None:
            m, k, n = self.shape
            self._desc = (
                f"FusedNormResidual({self.scheme.name})\n"
                + ops.describe_gemm(m, n, k, True, self.schedule, self.cta_group)
                + f"; chained planes {self.plane_scheme.name}"
                + ("; clears the consumer output" if self.preclear is not self.c else ""))
        return self._desc
