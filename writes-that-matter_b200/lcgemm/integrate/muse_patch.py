"""Muse-Glimmer-style decoder: the MLP chain as TWO opaque vLLM custom ops.

``norm_gateup`` consumes the attention output and the residual stream and returns the new
residual and ``gate_up``'s output; ``swiglu_down`` then only launches the ``down`` GEMM on the
planes the first op's epilogue left in the plan (``lcgemm/integrate/muse_patch.py`` of the
reference).  Same ``arm / install / counts / check_calls`` protocol as the Qwen patch.
"""
from __future__ import annotations

import functools
from typing import Tuple

import torch
import torch.nn.functional as F

from lcgemm.integrate._common import PatchCore, compile_cache_guard, gemma_rmsnorm, stock_swiglu_down

_CACHE_PRESET, _VLLM_PREIMPORTED = compile_cache_guard()

LAYER_CLASS_NAME = "MuseGlimmerDecoderLayer"
EXPECTED_LAYERS = 52
EXPECTED_SHAPES = (6656, 19968, 39936, 6656)
INSTALLABLE_TOKENS = (512, 1024, 2048, 4096, 8192)

_STATE = {"armed": False, "installed": False, "layers": 0, "tokens": 0}
_CORE = PatchCore(_STATE, LAYER_CLASS_NAME)
_PLANS, _PREPARED, _DOWN_PREPARED, _CALLS = _CORE.plans, _CORE.by_gate, _CORE.by_down, _CORE.calls

_rmsnorm = gemma_rmsnorm


@torch.library.custom_op("lcgemm_muse::norm_gateup", mutates_args=(), device_types="cuda")
def norm_gateup(
    delta: torch.Tensor,
    residual: torch.Tensor,
    norm_weight: torch.Tensor,
    gate_up_weight: torch.Tensor,
    eps: float,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(residual + delta, gate_up(norm(residual + delta)))``."""
    plans = _PLANS.get(delta.shape[0])
    entry = _PREPARED.get(gate_up_weight.data_ptr())
    if plans is None or entry is None:
        _CALLS["gate_up.reference"] += 1
        h = residual + delta
        return h, F.linear(_rmsnorm(h, norm_weight, eps), gate_up_weight)
    _CALLS["gate_up.fused"] += 1
    new_residual = _CORE.residual_buffer(delta)
    z = plans[0](residual, delta, norm_weight, eps, prepared_w=entry[1], residual_out=new_residual)
    return new_residual, z


@norm_gateup.register_fake
def _(delta, residual, norm_weight, gate_up_weight, eps):
    return torch.empty_like(delta), delta.new_empty((delta.shape[0], gate_up_weight.shape[0]))


@torch.library.custom_op("lcgemm_muse::swiglu_down", mutates_args=(), device_types="cuda")
def swiglu_down(gate_up: torch.Tensor, down_weight: torch.Tensor) -> torch.Tensor:
    """``down(SwiGLU(gate_up))``; on the fused branch the planes already sit in the plan."""
    plans = _PLANS.get(gate_up.shape[0])
    planes = _DOWN_PREPARED.get(down_weight.data_ptr())
    if plans is None or planes is None:
        _CALLS["down.reference"] += 1
        return stock_swiglu_down(gate_up, down_weight, round_silu=False)
    _CALLS["down.fused"] += 1
    return plans[1](prepared_w=planes)


@swiglu_down.register_fake
def _(gate_up, down_weight):
    return gate_up.new_empty((gate_up.shape[0], down_weight.shape[0]))


def _patched_forward(self, positions, hidden_states, residual):
    """Attention exactly as the model has it; the MLP entry and tail go through the two ops
    (``lcgemm/integrate/muse_patch.py:104-127``)."""
    skip = hidden_states
    attn = self.self_attn(positions=positions, hidden_states=self.input_layernorm(hidden_states))
    attn = self.post_attention_layernorm(attn)
    pre_ffn = self.pre_feedforward_layernorm
    skip, gate_up = torch.ops.lcgemm_muse.norm_gateup(
        attn, skip, pre_ffn.weight, self.mlp.gate_up_proj.weight, pre_ffn.eps)
    mlp_out = torch.ops.lcgemm_muse.swiglu_down(gate_up, self.mlp.down_proj.weight)
    return skip + self.post_feedforward_layernorm(mlp_out), skip


def arm() -> None:
    """Patch the decoder class before vLLM compiles it."""
    if _VLLM_PREIMPORTED and not _CACHE_PRESET:
        raise RuntimeError("muse_patch must be imported before vLLM unless its compile cache is off")
    from vllm.model_executor.models.muse_glimmer import MuseGlimmerDecoderLayer

    MuseGlimmerDecoderLayer.forward = _patched_forward
    _STATE["armed"] = True


def _prepare(model, tokens: int) -> dict:
    layers = _CORE.decoder_layers(model, EXPECTED_LAYERS)
    dims = _CORE.mlp_dims(layers[0])
    if dims != tuple(EXPECTED_SHAPES):
        raise RuntimeError(f"Muse MLP dimensions {dims} are not the validated {tuple(EXPECTED_SHAPES)}")
    return _CORE.prepare(layers, tokens, dry_run_eps=1e-5)


def install(llm, tokens: int) -> dict:
    if not _STATE["armed"]:
        raise RuntimeError("muse_patch.arm() has to run before the engine is built")
    if tokens not in INSTALLABLE_TOKENS:
        raise ValueError(f"{tokens} tokens is not an installable Muse prefill length")
    info = llm.apply_model(functools.partial(_prepare, tokens=tokens))
    if isinstance(info, list):
        info = info[0]
    _STATE.update(installed=True, layers=info["layers"], tokens=tokens)
    return info


def counts() -> dict:
    return dict(_CALLS)


def check_calls(passes: int, since: dict | None = None) -> dict:
    """Two fused ops per layer per pass, no functional branch."""
    if not _STATE["installed"]:
        raise RuntimeError("nothing installed yet: muse_patch.check_calls needs install() first")
    fused, reference = _CORE.tally(("gate_up.fused", "down.fused"),
                                   ("gate_up.reference", "down.reference"), since)
    expected = 2 * passes * _STATE["layers"]
    if fused != expected or reference:
        raise RuntimeError(f"Muse ops: {fused} fused and {reference} functional calls, "
                           f"{expected} fused and 0 functional expected")
    return {"fused_calls": fused, "reference_calls": reference, "expected": expected}
