"""One dense-decoder MLP layer in three arms, for the single-layer configuration
``x -> RMSNorm -> gate_up -> SwiGLU -> down -> + residual`` and as the building block of the
tensor-parallel form.

* :class:`Rank7MlpLayer`  the rank-7 chain: fused norm planes, chained gate_up GEMM, down GEMM
  (what ``lcgemm_qwen::mlp_chain`` runs, ``lcgemm/integrate/qwen_patch.py:85-97``), 3 launches
  plus the closing residual add;
* :class:`DenseMlpLayer`  the stock layer (``lcgemm/integrate/qwen_patch.py:41-58``) on the
  dense tcgen05 GEMM of this library, or on cuBLAS through ``torch.matmul`` with
  ``gemm="cublas"``: norm, GEMM, SwiGLU, GEMM, residual add.

Both keep the layer's output buffers and return views of them.
"""
from __future__ import annotations

import torch

from . import ops
from .seams import build_chain


class Rank7MlpLayer:
    def __init__(self, tokens: int, norm_weight, gate_up_weight, down_weight, eps: float = 1e-6,
                 cta_group: int = 0, fuse_residual: bool = False):
        two_i, hidden = gate_up_weight.shape
        out_dim, inter = down_weight.shape
        if two_i != 2 * inter:
            raise ValueError("gate_up weight must have 2 * intermediate rows")
        self.eps = eps
        self.norm_weight = norm_weight
        self.gate_plan, self.down_plan = build_chain((tokens, hidden, two_i), (tokens, inter, out_dim))
        self.gate_plan.cta_group = self.down_plan.cta_group = cta_group
        self.gate_bw = self.gate_plan.prepare_weight(gate_up_weight)
        self.down_bw = self.down_plan.prepare_weight(down_weight)
        self.out = torch.empty((tokens, out_dim), device=gate_up_weight.device, dtype=torch.bfloat16)
        # fuse_residual: the closing `h + mlp` is folded into `down`.  Possible when `down` is
        # rank-split and its output is initialised by the gate_up kernel: that kernel then copies h
        # into it instead of zeroing it, every contribution of `down` is reduce-added onto h, and no
        # add kernel runs.  Off by default: each contribution is then rounded to bf16 at the
        # magnitude of h instead of the branch's (1.7 times the error on the MLP branch where h dominates it).
        self.fuse_residual = bool(fuse_residual) and self.down_plan.rank_split \
            and self.gate_plan.preclear is self.down_plan.c and out_dim == hidden \
            and self.down_plan.c.is_contiguous()
        if fuse_residual and not self.fuse_residual:
            raise ValueError("fuse_residual needs a rank-split `down` whose output the gate_up kernel initialises")

    def chain(self, delta, residual):
        """``(down_out, residual_out)`` exactly as the custom op returns them.  Without a ``delta``
        (``None``: the layer on its own, as in the single-layer configuration) the residual stream is
        ``residual`` itself and the norm kernel reads one operand and stores no sum."""
        self.gate_plan(residual, delta, self.norm_weight, self.eps, prepared_w=self.gate_bw)
        h = residual if delta is None else self.gate_plan.residual_out
        return self.down_plan(prepared_w=self.down_bw), h

    def forward(self, x, delta=None):
        """``h + mlp(norm(h))`` with ``h = x + delta`` (``h = x`` without a ``delta``)."""
        if self.fuse_residual:
            gate = self.gate_plan
            # h is x without a delta, else what the norm kernel stores in front of the GEMM
            gate.init_from = x if delta is None else gate.residual_out
            try:
                down_out, _ = self.chain(delta, x)
            finally:
                gate.init_from = None
            return down_out
        down_out, h = self.chain(delta, x)
        return ops.add(h, down_out if down_out.is_contiguous() else down_out.contiguous(), out=self.out)

    __call__ = forward
    launches_per_forward = 4
    accepts_no_delta = True


class DenseMlpLayer:
    def __init__(self, tokens: int, norm_weight, gate_up_weight, down_weight, eps: float = 1e-6,
                 gemm: str = "tcgen05", cta_group: int = 0):
        if gemm not in ("tcgen05", "cublas"):
            raise ValueError("gemm must be 'tcgen05' or 'cublas'")
        two_i, hidden = gate_up_weight.shape
        out_dim, inter = down_weight.shape
        dev, bf = gate_up_weight.device, torch.bfloat16
        self.eps, self.gemm, self.cta_group = eps, gemm, cta_group
        self.norm_weight, self.w_gu, self.w_down = norm_weight, gate_up_weight, down_weight
        self.h = torch.empty((tokens, hidden), device=dev, dtype=bf)
        self.x = torch.empty((tokens, hidden), device=dev, dtype=bf)
        self.z = torch.empty((tokens, two_i), device=dev, dtype=bf)
        self.s = torch.empty((tokens, inter), device=dev, dtype=bf)
        self.d = torch.empty((tokens, out_dim), device=dev, dtype=bf)
        self.out = torch.empty((tokens, out_dim), device=dev, dtype=bf)

    def _mm(self, a, w, out):
        if self.gemm == "cublas":
            return torch.matmul(a, w.t(), out=out)
        return ops.gemm_dense(a, w, out=out, cta_group=self.cta_group)

    def chain(self, delta, residual):
        _, h = ops.add_rmsnorm(delta, residual, self.norm_weight, self.eps, residual_out=self.h, x=self.x)
        self._mm(self.x, self.w_gu, self.z)
        ops.swiglu(self.z, out=self.s)
        self._mm(self.s, self.w_down, self.d)
        return self.d, h                      # without a delta h is `residual` itself

    def forward(self, x, delta=None):
        d, h = self.chain(delta, x)
        return ops.add(h, d, out=self.out)

    __call__ = forward
    launches_per_forward = 5
    accepts_no_delta = True


class CapturedLayer:
    """One layer call recorded into a CUDA graph and replayed: a single launch per step in place
    of the layer's five or six, which removes the host's launch latency and most of the gaps
    between the dependent kernels (about 20 us of a 1.4 ms layer).  The input tensor's storage
    is part of the recording: the caller refills ``x`` in place between replays.  Every kernel
    of this package can be captured (tensor maps are kernel parameters, nothing allocates or
    synchronises); attributes that are set on first use are set by the warm-up calls here.
    """

    def __init__(self, layer, x: torch.Tensor, delta: torch.Tensor | None = None, warmup: int = 3):
        self.layer, self.x, self.delta = layer, x, delta
        call = (lambda: layer(x)) if delta is None else (lambda: layer(x, delta))
        side = torch.cuda.Stream(x.device)
        side.wait_stream(torch.cuda.current_stream(x.device))
        with torch.cuda.stream(side):
            for _ in range(warmup):
                call()
        torch.cuda.current_stream(x.device).wait_stream(side)
        torch.cuda.synchronize(x.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.out = call()

    def __call__(self) -> torch.Tensor:
        self.graph.replay()
        return self.out
