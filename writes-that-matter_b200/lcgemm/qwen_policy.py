"""Engine selection for exact batch-one Qwen prefill lengths.

The reference's policy (``lcgemm/qwen_policy.py``): 512 and 1024 tokens deploy the stock engine
-- in a process where the decoder patch was never armed -- and 2048 / 4096 / 8192 deploy the
rank-7 chain, one engine per exact length; anything else has no validated policy.
"""
from __future__ import annotations

import sys
from typing import Literal

Deployment = Literal["stock", "lc_chain"]

_POLICY: dict = {512: "stock", 1024: "stock", 2048: "lc_chain", 4096: "lc_chain", 8192: "lc_chain"}
STOCK_TOKENS = frozenset(t for t, kind in _POLICY.items() if kind == "stock")
LC_TOKENS = frozenset(t for t, kind in _POLICY.items() if kind == "lc_chain")
SUPPORTED_TOKENS = frozenset(_POLICY)
_PATCH_MODULE = "lcgemm.integrate.qwen_patch"


def deployment_for(tokens: int) -> Deployment:
    """Which engine kind a prefill of exactly ``tokens`` tokens deploys."""
    try:
        return _POLICY[tokens]
    except (KeyError, TypeError):
        known = ", ".join(str(t) for t in sorted(SUPPORTED_TOKENS))
        raise ValueError(f"prefill length {tokens!r} has no Qwen engine policy (known: {known})") from None


def arm_selected_engine(tokens: int):
    """Prepare the process for the engine ``tokens`` deploys.

    Rank-7 lengths: import and arm the patch (this must happen before vLLM is imported) and
    return the patch module for :func:`install_selected_engine`.  Stock lengths: return ``None``
    without importing the patch at all, and refuse if it was already armed in this process."""
    kind = deployment_for(tokens)
    if kind == "lc_chain":
        if "vllm" in sys.modules:
            raise RuntimeError("vLLM is already imported: the rank-7 engine has to be armed first")
        from lcgemm.integrate import qwen_patch

        qwen_patch.arm()
        return qwen_patch
    patch = sys.modules.get(_PATCH_MODULE)
    if patch is not None and getattr(patch, "_STATE", {}).get("armed"):
        raise RuntimeError(
            "this process has armed the Qwen decoder patch, so no stock engine built here would "
            "be unpatched; start the stock engine in a fresh process")
    return None


def install_selected_engine(patch, llm, tokens: int):
    """After the engine has loaded its weights: install the one validated rank-7 shape."""
    if deployment_for(tokens) != "lc_chain":
        raise ValueError(f"{tokens} tokens deploy the stock engine: nothing to install")
    if patch is None:
        raise ValueError("pass the module arm_selected_engine() returned")
    return patch.install(llm, tokens=tokens)
