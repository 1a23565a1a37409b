"""The operand-plane contract of the rank-R GEMM (``lcgemm/planes.py`` of the reference).

Every operand reaches the GEMM mainloop as R planes of signed block sums stacked
along the leading dimension, so one TMA descriptor per operand serves all
products with the rank folded into the row coordinate:

* :func:`prepare_b` forms the B planes once, offline, because weights are fixed;
* :func:`a_planes` forms the A planes of a plain activation matrix (the deployed
  seams produce theirs inside the kernel that precedes the GEMM instead);
* :func:`apply_terms` is the signed sum itself, for host-side code that needs it.
"""
from __future__ import annotations

import torch

from . import ops
from .scheme import Scheme


def apply_terms(terms, frag):
    """``sum coeff * frag[row, col]`` over ``(row, col, coeff)`` terms
    (``lcgemm/planes.py:27-50``).  ``frag`` is any mapping from a block index pair to a
    value that supports ``+``, ``-`` and ``*``; unit coefficients cost no multiply."""
    acc = None
    for row, col, coeff in terms:
        term = frag[row, col]
        if abs(coeff) != 1:
            term = term * float(abs(coeff))
        if acc is None:
            acc = -term if coeff < 0 else term
        elif coeff < 0:
            acc = acc - term
        else:
            acc = acc + term
    return acc


def prepare_b(w: torch.Tensor, scheme: Scheme) -> torch.Tensor:
    """Stack the R combined weight planes of ``w`` ``(N, K)``, K-major
    (``lcgemm/planes.py:54-71``): fp32 summation, one rounding to bf16.

    Returns ``(R * N2, K2p)`` with ``N2 = round_up(ceil(N/2), 8)`` and
    ``K2p = round_up(ceil(K/2), 64)``; for shapes divisible by the tile sizes this is the
    reference's ``(R * N/2, K/2)``.  Runs as a CUDA kernel on ``w``'s device."""
    return ops.prepare_b(w.detach(), scheme)


def a_planes(a: torch.Tensor, scheme: Scheme, out: torch.Tensor | None = None) -> torch.Tensor:
    """The R combined activation planes of ``a`` ``(M, K)``: ``(R * ceil(M/2), K2p)``."""
    return ops.a_planes(a.detach(), scheme, out=out)
