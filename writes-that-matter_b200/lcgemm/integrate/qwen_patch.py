"""Qwen3.5-style dense decoder: the MLP chain as one opaque vLLM custom op.

Arm before the engine is constructed, install after its weights are loaded
(``lcgemm/integrate/qwen_patch.py`` of the reference).  Only the exact token counts passed
to :func:`install` run the rank-7 chain; profiling, dummy and decode shapes take the
functional reference inside the op, and both kinds of call are counted.
"""
from __future__ import annotations

import functools
import os
import sys
from collections import defaultdict
from typing import Tuple

import torch
import torch.nn.functional as F

from lcgemm.seams import build_chain

_CACHE_PRESET = os.environ.get("VLLM_DISABLE_COMPILE_CACHE") in ("1", "true", "True")
_VLLM_PREIMPORTED = "vllm" in sys.modules
os.environ["VLLM_DISABLE_COMPILE_CACHE"] = "1"

# What the validated model looks like (lcgemm/integrate/qwen_patch.py:209-226).
LAYER_CLASS_NAME = "Qwen3_5DecoderLayer"
EXPECTED_LAYERS = 64
EXPECTED_SHAPES = (5120, 17408, 34816, 5120)        # (H, I, 2I, H_out)
INSTALLABLE_TOKENS = (512, 1024, 2048, 4096, 8192)

_STATE = {"armed": False, "installed": False, "layers": 0, "shapes": ()}
_PLANS: dict = {}            # M -> (GateUpPlan, DownPlan)
_PREPARED: dict = {}         # gate_up weight data_ptr -> (down weight data_ptr, gate planes, down planes)
_CALLS: dict = defaultdict(int)
_RESIDUAL_RING: list = []
_RESIDUAL_TURN = 0
_ORIGINAL_FORWARD = None


def _residual_buf(like: torch.Tensor) -> torch.Tensor:
    """One of two buffers in turn: a custom op may not return an alias of an input, and the
    residual of layer n is an input of layer n + 1."""
    global _RESIDUAL_RING, _RESIDUAL_TURN
    if not _RESIDUAL_RING or _RESIDUAL_RING[0].shape != like.shape or _RESIDUAL_RING[0].device != like.device:
        _RESIDUAL_RING = [torch.empty_like(like), torch.empty_like(like)]
    out = _RESIDUAL_RING[_RESIDUAL_TURN]
    _RESIDUAL_TURN = 1 - _RESIDUAL_TURN
    return out


def _reference(delta, residual, norm_weight, gate_up_weight, down_weight, eps):
    """The functional form of the op, with the stock layer's rounding points
    (``lcgemm/integrate/qwen_patch.py:41-58``)."""
    h = (delta.float() + residual.float()).to(delta.dtype)
    hf = h.float()
    x = hf * torch.rsqrt(hf.square().mean(-1, keepdim=True) + eps)
    x = (x * (norm_weight.float() + 1.0)).to(delta.dtype)
    gate, up = F.linear(x, gate_up_weight).chunk(2, dim=-1)
    act = F.silu(gate.float()).to(gate.dtype) * up
    return F.linear(act, down_weight), h


def _dispatch(m: int, gate_up_weight: torch.Tensor, down_weight: torch.Tensor):
    plans = _PLANS.get(m)
    prepared = _PREPARED.get(gate_up_weight.data_ptr())
    if plans is None or prepared is None or prepared[0] != down_weight.data_ptr():
        return None
    return plans, prepared[1], prepared[2]


@torch.library.custom_op("lcgemm_qwen::mlp_chain", mutates_args=(), device_types="cuda")
def mlp_chain(
    delta: torch.Tensor,
    residual: torch.Tensor,
    norm_weight: torch.Tensor,
    gate_up_weight: torch.Tensor,
    down_weight: torch.Tensor,
    eps: float,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(down(SwiGLU(gate_up(norm(delta + residual)))), delta + residual)``."""
    selected = _dispatch(delta.shape[0], gate_up_weight, down_weight)
    if selected is None:
        _CALLS["chain.reference"] += 1
        return _reference(delta, residual, norm_weight, gate_up_weight, down_weight, eps)
    _CALLS["chain.fused"] += 1
    (gate_plan, down_plan), gate_bw, down_bw = selected
    residual_out = _residual_buf(delta)
    gate_plan(residual, delta, norm_weight, eps, prepared_w=gate_bw, residual_out=residual_out)
    return down_plan(prepared_w=down_bw), residual_out


@mlp_chain.register_fake
def _(delta, residual, norm_weight, gate_up_weight, down_weight, eps):
    return delta.new_empty((delta.shape[0], down_weight.shape[0])), torch.empty_like(delta)


def _make_forward():
    def forward(self, hidden_states, residual, positions=None, **kwargs):
        # Dense TP=1 only: the sequence-parallel MoE path keeps the stock forward.
        if self.use_attn_reduce_scatter_for_moe:
            return _ORIGINAL_FORWARD(self, hidden_states=hidden_states, residual=residual,
                                     positions=positions, **kwargs)
        if residual is None:
            residual = hidden_states
            hidden_states = self.input_layernorm(hidden_states)
        else:
            hidden_states, residual = self.input_layernorm(hidden_states, residual)

        if self.layer_type == "linear_attention":
            hidden_states = self.linear_attn(hidden_states=hidden_states)
        elif self.layer_type == "full_attention":
            hidden_states = self.self_attn(hidden_states=hidden_states, positions=positions)
        else:
            raise ValueError(f"invalid Qwen layer type {self.layer_type}")

        def scaled(x, scale):
            s = scale.to(x.dtype)
            return x * ((s[0] if x.dim() == 2 else s) + 1)

        if self.layer_scale:
            hidden_states = scaled(hidden_states, self.attn_layer_scale)
        hidden_states, residual = torch.ops.lcgemm_qwen.mlp_chain(
            hidden_states, residual, self.post_attention_layernorm.weight,
            self.mlp.gate_up_proj.weight, self.mlp.down_proj.weight,
            self.post_attention_layernorm.variance_epsilon)
        if self.layer_scale:
            hidden_states = scaled(hidden_states, self.ffn_layer_scale)
        return hidden_states, residual

    return forward


def arm() -> None:
    """Replace the decoder layer's forward before vLLM compiles it."""
    global _ORIGINAL_FORWARD
    if _VLLM_PREIMPORTED and not _CACHE_PRESET:
        raise RuntimeError(
            "vLLM was imported before qwen_patch with compile cache enabled; the stock graph "
            "could be reused silently")
    from vllm.model_executor.models.qwen3_5 import Qwen3_5DecoderLayer

    if _ORIGINAL_FORWARD is None:
        _ORIGINAL_FORWARD = Qwen3_5DecoderLayer.forward
    Qwen3_5DecoderLayer.forward = _make_forward()
    _STATE["armed"] = True


def _dry_run(gate_plan, down_plan, gate_bw, down_bw) -> None:
    from lcgemm import ops

    m, k, _ = gate_plan.shape
    delta = torch.zeros((m, k), device="cuda", dtype=torch.bfloat16)
    residual = torch.zeros_like(delta)
    norm = torch.zeros((k,), device="cuda", dtype=torch.bfloat16)
    gate_plan(residual, delta, norm, 1e-6, prepared_w=gate_bw)
    down_plan(prepared_w=down_bw)
    ops.check_status()          # synchronises; raises if a device-side wait ran out


def _prepare(model, tokens: int) -> dict:
    layers = [mod for mod in model.modules() if type(mod).__name__ == LAYER_CLASS_NAME]
    if len(layers) != EXPECTED_LAYERS:
        raise RuntimeError(
            f"expected {EXPECTED_LAYERS} {LAYER_CLASS_NAME} modules, found {len(layers)}")
    if any(getattr(layer, "use_attn_reduce_scatter_for_moe", False) for layer in layers):
        raise RuntimeError("Qwen MLP-chain campaign supports dense TP=1 only")
    if any(getattr(layer, "layer_scale", False) for layer in layers):
        raise RuntimeError("layer_scale was not validated for this campaign")

    gate0 = layers[0].mlp.gate_up_proj.weight.data
    down0 = layers[0].mlp.down_proj.weight.data
    h, two_i = gate0.shape[1], gate0.shape[0]
    i, out = down0.shape[1], down0.shape[0]
    if (h, i, two_i, out) != tuple(EXPECTED_SHAPES):
        raise RuntimeError(f"unexpected Qwen MLP shapes {(h, i, two_i, out)}")

    gate_plan, down_plan = _PLANS[tokens] = build_chain((tokens, h, two_i), (tokens, i, out))
    nbytes = 0
    first = None
    for layer in layers:
        gate_w = layer.mlp.gate_up_proj.weight.data
        down_w = layer.mlp.down_proj.weight.data
        gate_bw = gate_plan.prepare_weight(gate_w)
        down_bw = down_plan.prepare_weight(down_w)
        _PREPARED[gate_w.data_ptr()] = (down_w.data_ptr(), gate_bw, down_bw)
        nbytes += gate_bw.numel() * gate_bw.element_size() + down_bw.numel() * down_bw.element_size()
        first = first or (gate_bw, down_bw)
    _dry_run(gate_plan, down_plan, *first)
    return {
        "layers": len(layers),
        "planes_gib": nbytes / 2**30,
        "tokens": tokens,
        "schemes": {"gate_up": gate_plan.scheme.name, "down": down_plan.scheme.name},
        "describe": {"gate_up": gate_plan.describe(), "down": down_plan.describe()},
    }


def install(llm, tokens: int) -> dict:
    """Prepare one prefill shape: planes for every layer, plans, and a dry run."""
    if not _STATE["armed"]:
        raise RuntimeError("call qwen_patch.arm() before constructing LLM")
    if tokens not in INSTALLABLE_TOKENS:
        raise ValueError(f"no Qwen LC shape for M={tokens}")
    info = llm.apply_model(functools.partial(_prepare, tokens=tokens))
    info = info[0] if isinstance(info, list) else info
    _STATE.update(installed=True, layers=info["layers"], shapes=(tokens,))
    return info


def counts() -> dict:
    return dict(_CALLS)


def check_calls(passes: int, since: dict | None = None) -> dict:
    """Every layer of every pass must have taken the fused branch, none the reference."""
    if not _STATE["installed"]:
        raise RuntimeError("qwen_patch.check_calls before install")
    base = since or {}
    fused = _CALLS["chain.fused"] - base.get("chain.fused", 0)
    reference = _CALLS["chain.reference"] - base.get("chain.reference", 0)
    expected = passes * _STATE["layers"]
    if fused != expected or reference:
        raise RuntimeError(
            f"Qwen chain calls fused={fused}, reference={reference}, expected={expected}")
    return {"fused_calls": fused, "reference_calls": reference, "expected": expected}
