"""The deployed MLP-chain configuration: postsum-CSE for ``gate_up``, the locality-ordered
decomposition for ``down`` (``lcgemm/seams/__init__.py`` of the reference)."""
from __future__ import annotations

from ..scheme import load
from .down import DownPlan
from .gate_up import GateUpPlan

GATE_UP_SCHEME = "2x2_postsum_cse"
DOWN_SCHEME = "2x2_locality_ordered"


def build_chain(gate_up_shape, down_shape):
    """Build the chained plans for one prefill shape: ``gate_up_shape = (M, H, 2I)``,
    ``down_shape = (M, I, H_out)`` (``lcgemm/seams/__init__.py:19-38``)."""
    gate_scheme = load(GATE_UP_SCHEME)
    down_scheme = load(DOWN_SCHEME)
    gate = GateUpPlan(gate_scheme, tuple(gate_up_shape), plane_scheme=down_scheme)
    down = DownPlan(down_scheme, tuple(down_shape), producer=gate)
    if down.rank_split:
        gate.preclear = down.c      # the producer zeroes the consumer's output while it runs
    return gate, down


__all__ = ["DOWN_SCHEME", "GATE_UP_SCHEME", "build_chain", "GateUpPlan", "DownPlan"]
