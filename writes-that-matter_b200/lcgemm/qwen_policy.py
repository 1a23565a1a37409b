"""Which exact batch-one prefill sizes deploy the rank-7 chain (``lcgemm/qwen_policy.py``).

Stock sizes must use a process in which the decoder patch was never armed; rank-7 sizes
use one engine per exact prefill length.
"""
from __future__ import annotations

import sys
from typing import Literal

Deployment = Literal["stock", "lc_chain"]

STOCK_TOKENS = frozenset((512, 1024))
LC_TOKENS = frozenset((2048, 4096, 8192))
SUPPORTED_TOKENS = STOCK_TOKENS | LC_TOKENS


def deployment_for(tokens: int) -> Deployment:
    """The validated engine kind for an exact batch-one prefill size."""
    if tokens in STOCK_TOKENS:
        return "stock"
    if tokens in LC_TOKENS:
        return "lc_chain"
    raise ValueError(
        f"no validated Qwen engine policy for M={tokens}; supported={sorted(SUPPORTED_TOKENS)}")


def arm_selected_engine(tokens: int):
    """Arm the rank-7 engine before vLLM is imported, or leave a stock engine truly unarmed.
    Returns the patch module to hand to :func:`install_selected_engine`, or ``None`` for stock
    (in which case the patch module is deliberately not imported)."""
    if deployment_for(tokens) == "stock":
        loaded = sys.modules.get("lcgemm.integrate.qwen_patch")
        if loaded is not None and getattr(loaded, "_STATE", {}).get("armed"):
            raise RuntimeError(
                "cannot construct a truly unarmed stock engine after the Qwen decoder patch was "
                "armed in this process; use a fresh process")
        return None
    if "vllm" in sys.modules:
        raise RuntimeError("select and arm the LC engine before importing vLLM")
    from lcgemm.integrate import qwen_patch

    qwen_patch.arm()
    return qwen_patch


def install_selected_engine(patch, llm, tokens: int):
    """Install exactly one validated rank-7 shape after the engine has loaded its weights."""
    if deployment_for(tokens) != "lc_chain":
        raise ValueError(f"M={tokens} is a stock-only policy; do not arm or install the patch")
    if patch is None:
        raise ValueError("the LC patch returned by arm_selected_engine is required")
    return patch.install(llm, tokens=tokens)
