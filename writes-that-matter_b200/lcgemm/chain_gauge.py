"""The interleaved-K gauge of the ``gate_up -> SwiGLU -> down`` chain.

``down``'s A planes are ``L_r(S)`` with ``S = silu(Z[:, :I]) * Z[:, I:]``, and each plane
element pairs S column ``l`` of K block 0 with column ``l`` of K block 1.  With two
contiguous halves those columns are ``I / 2`` apart and belong to different tiles of
the producing ``gate_up`` GEMM.  The partition of K into blocks is a free choice as long
as A's and B's agree (``lcgemm/chain_gauge.py:9-36``), and B is a static weight, so the
blocks are chosen chunk-interleaved with width ``CHUNK = 64``::

    block j = {c : (c // 64) % 2 == j}        index l = (c // 128) * 64 + c % 64

The partner of column ``c`` is then ``c ^ 64`` and both sit in one 256-wide tile of the
producer, which therefore owns every input of the plane elements it writes.
"""
from __future__ import annotations

import torch

from . import ops
from .planes import prepare_b

CHUNK = 64


def interleave_perm(width: int, chunk: int = CHUNK) -> torch.Tensor:
    """Column order that makes the interleaved blocks two contiguous halves:
    ``x[:, interleave_perm(K)]`` is the natural form of the permuted matrix
    (``lcgemm/chain_gauge.py:51-65``)."""
    if width % (2 * chunk):
        raise ValueError(f"width {width} not divisible by 2*chunk {2 * chunk}")
    cols = torch.arange(width)
    block = (cols // chunk) % 2
    index = (cols // (2 * chunk)) * chunk + cols % chunk
    perm = torch.empty(width, dtype=torch.long)
    perm[block * (width // 2) + index] = cols
    return perm


def permute_k(x: torch.Tensor, chunk: int = CHUNK) -> torch.Tensor:
    """Apply the gauge to the last dimension of a K-major tensor (``lcgemm/chain_gauge.py:68-70``)."""
    return x[..., interleave_perm(x.shape[-1], chunk).to(x.device)].contiguous()


def swiglu(z: torch.Tensor) -> torch.Tensor:
    """``bf16(silu(gate)) * up`` of ``z = [gate | up]`` as a CUDA kernel.  (The reference's
    host helper of this name, ``lcgemm/chain_gauge.py:76-79``, keeps fp32; this one has the
    rounding of the stock layer, ``lcgemm/integrate/qwen_patch.py:54-56``.)"""
    return ops.swiglu(z)


def chain_a_planes(z: torch.Tensor, scheme, chunk: int = CHUNK,
                   out: torch.Tensor | None = None) -> torch.Tensor:
    """``L_r(SwiGLU(Z))`` in the interleaved gauge, ``(R * M/2, I/2)``, fp32 with one rounding
    (``lcgemm/chain_gauge.py:82-99``), as a kernel of its own.  The chained ``gate_up`` GEMM
    produces the same planes in its epilogue; this is the unfused form."""
    if chunk != CHUNK:
        raise ValueError(f"the device kernels are built for chunk {CHUNK}")
    return ops.swiglu_planes(scheme, z, out=out)


def prepare_down_b(w: torch.Tensor, scheme, chunk: int = CHUNK) -> torch.Tensor:
    """``down``'s B planes with the gauge folded in: permute the static weight's K, then
    :func:`lcgemm.planes.prepare_b` (``lcgemm/chain_gauge.py:102-111``).  Offline, once per layer."""
    return prepare_b(permute_k(w.detach(), chunk), scheme)
