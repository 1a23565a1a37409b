"""Plans of the MLP chain.  ``build_chain`` wires the one deployed configuration: the
postsum-CSE decomposition for ``gate_up`` (its epilogue also emits ``down``'s operand planes) and
the locality-ordered one for ``down`` (``lcgemm/seams/__init__.py`` of the reference)."""
from __future__ import annotations

from ..scheme import load
from .down import DownPlan
from .gate_up import GateUpPlan

GATE_UP_SCHEME, DOWN_SCHEME = "2x2_postsum_cse", "2x2_locality_ordered"

__all__ = ["DOWN_SCHEME", "GATE_UP_SCHEME", "build_chain", "GateUpPlan", "DownPlan"]


def build_chain(gate_up_shape, down_shape):
    """``(GateUpPlan, DownPlan)`` for ``gate_up_shape = (M, H, 2I)`` and
    ``down_shape = (M, I, H_out)``.  A rank-split consumer accumulates into its output, so the
    producer is told to zero that buffer while it runs."""
    consumer_scheme = load(DOWN_SCHEME)
    producer = GateUpPlan(load(GATE_UP_SCHEME), tuple(gate_up_shape), plane_scheme=consumer_scheme)
    consumer = DownPlan(consumer_scheme, tuple(down_shape), producer=producer)
    if consumer.rank_split:
        producer.preclear = consumer.c
    return producer, consumer
