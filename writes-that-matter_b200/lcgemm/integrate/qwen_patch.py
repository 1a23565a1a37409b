"""Qwen3.5-style dense decoder: the whole MLP chain as ONE opaque vLLM custom op.

Protocol (that of the reference's ``lcgemm/integrate/qwen_patch.py``): ``arm()`` before the
engine is constructed, ``install(llm, tokens)`` once its weights are loaded, then
``counts()`` / ``check_calls()`` to prove which branch ran.  Inside the op only calls with
exactly the installed token count *and* the installed weights take the rank-7 chain;
everything else (profiling, dummy and decode shapes) evaluates the functional form, and both
are counted.
"""
from __future__ import annotations

import functools
from typing import Tuple

import torch
import torch.nn.functional as F

from lcgemm.integrate._common import PatchCore, compile_cache_guard, gemma_rmsnorm, stock_swiglu_down

_CACHE_PRESET, _VLLM_PREIMPORTED = compile_cache_guard()

# The validated model (lcgemm/integrate/qwen_patch.py:209-226 of the reference).
LAYER_CLASS_NAME = "Qwen3_5DecoderLayer"
EXPECTED_LAYERS = 64
EXPECTED_SHAPES = (5120, 17408, 34816, 5120)          # hidden, intermediate, 2 * intermediate, out
INSTALLABLE_TOKENS = (512, 1024, 2048, 4096, 8192)    # 512 / 1024 build for evaluation only

_STATE = {"armed": False, "installed": False, "layers": 0, "shapes": ()}
_CORE = PatchCore(_STATE, LAYER_CLASS_NAME)
_PLANS, _PREPARED, _CALLS = _CORE.plans, _CORE.by_gate, _CORE.calls
_ORIGINAL_FORWARD = None


def _reference(delta, residual, norm_weight, gate_up_weight, down_weight, eps):
    """Functional form of the op with the stock layer's rounding points
    (``lcgemm/integrate/qwen_patch.py:41-58``): sum rounded to bf16 before the norm, bf16 GEMMs,
    SiLU rounded before the product."""
    h = (delta.float() + residual.float()).to(delta.dtype)
    x = gemma_rmsnorm(h, norm_weight, eps)
    return stock_swiglu_down(F.linear(x, gate_up_weight), down_weight, round_silu=True), h


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
    plans = _PLANS.get(delta.shape[0])
    entry = _PREPARED.get(gate_up_weight.data_ptr())
    if plans is None or entry is None or entry[0] != down_weight.data_ptr():
        _CALLS["chain.reference"] += 1
        return _reference(delta, residual, norm_weight, gate_up_weight, down_weight, eps)
    _CALLS["chain.fused"] += 1
    gate_plan, down_plan = plans
    new_residual = _CORE.residual_buffer(delta)
    gate_plan(residual, delta, norm_weight, eps, prepared_w=entry[1], residual_out=new_residual)
    out = down_plan(prepared_w=entry[2])
    # A custom op may not return storage that one of its inputs lives in.  The plans' buffers
    # are shared by all layers, and a compiled engine is free to hand a layer an input that still
    # sits in the buffer the previous layer returned (its in-place norms do); the kernels
    # tolerate that (each reads its inputs before anything overwrites them), the contract does not.
    inputs = (delta.untyped_storage().data_ptr(), residual.untyped_storage().data_ptr())
    if out.untyped_storage().data_ptr() in inputs:
        _CALLS["chain.cloned_output"] += 1
        out = out.clone()
    if new_residual.untyped_storage().data_ptr() in inputs:
        _CALLS["chain.cloned_residual"] += 1
        new_residual = new_residual.clone()
    return out, new_residual


@mlp_chain.register_fake
def _(delta, residual, norm_weight, gate_up_weight, down_weight, eps):
    return delta.new_empty((delta.shape[0], down_weight.shape[0])), torch.empty_like(delta)


_ATTENTION_TAKES_OUTPUT: dict = {}


def _calling_convention(cls):
    import inspect

    names = inspect.signature(cls.forward).parameters
    return "output" in names, "positions" in names


def _record_attention_conventions(module) -> None:
    """Fill the table of attention calling conventions from the classes of the model's module,
    once, at ``arm()``: the patched forward is traced by vLLM's compiler, and traced code must
    only read this table (a write inside ``forward`` is refused when CUDA graphs are compiled in)."""
    import inspect

    for name, obj in vars(module).items():
        if inspect.isclass(obj) and "Attention" in name and callable(getattr(obj, "forward", None)):
            _ATTENTION_TAKES_OUTPUT[obj] = _calling_convention(obj)


def _attention(module, hidden_states, positions=None):
    """Call an attention module under either calling convention vLLM has used for this layer:
    returning its result (the revision the reference pins, ``qwen_patch.py:134-148`` there) or
    filling a caller-allocated ``output`` buffer (the installed 0.22 series)."""
    convention = _ATTENTION_TAKES_OUTPUT.get(type(module))
    if convention is None:                         # a class arm() did not see: work it out, store nothing
        convention = _calling_convention(type(module))
    wants_output, wants_positions = convention
    kwargs = {"hidden_states": hidden_states}
    if wants_positions and positions is not None:
        kwargs["positions"] = positions
    if wants_output:
        out = torch.empty_like(hidden_states)
        module(output=out, **kwargs)
        return out
    return module(**kwargs)


def _plus_one_scale(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    s = scale.to(x.dtype)
    return x * ((s[0] if x.dim() == 2 else s) + 1)


def _patched_forward(self, hidden_states, residual, positions=None, **kwargs):
    """The decoder layer with its MLP half replaced by the custom op; the attention half is the
    model's own (``lcgemm/integrate/qwen_patch.py:116-178``)."""
    if getattr(self, "use_attn_reduce_scatter_for_moe", False):   # sequence-parallel MoE path: stock
        return _ORIGINAL_FORWARD(self, hidden_states=hidden_states, residual=residual,
                                 positions=positions, **kwargs)
    if residual is None:
        residual, hidden_states = hidden_states, self.input_layernorm(hidden_states)
    else:
        hidden_states, residual = self.input_layernorm(hidden_states, residual)

    if self.layer_type == "full_attention":
        hidden_states = _attention(self.self_attn, hidden_states, positions)
    elif self.layer_type == "linear_attention":
        hidden_states = _attention(self.linear_attn, hidden_states)
    else:
        raise ValueError(f"invalid Qwen layer type {self.layer_type}")
    if self.layer_scale:
        hidden_states = _plus_one_scale(hidden_states, self.attn_layer_scale)

    norm = self.post_attention_layernorm
    hidden_states, residual = torch.ops.lcgemm_qwen.mlp_chain(
        hidden_states, residual, norm.weight, self.mlp.gate_up_proj.weight,
        self.mlp.down_proj.weight, norm.variance_epsilon)
    if self.layer_scale:
        hidden_states = _plus_one_scale(hidden_states, self.ffn_layer_scale)
    return hidden_states, residual


def arm() -> None:
    """Swap the decoder layer's forward before vLLM traces it."""
    global _ORIGINAL_FORWARD
    if _VLLM_PREIMPORTED and not _CACHE_PRESET:
        raise RuntimeError("qwen_patch must be imported before vLLM unless its compile cache is "
                           "off: a cached stock graph could otherwise be replayed unnoticed")
    import vllm.model_executor.models.qwen3_5 as qwen3_5
    from vllm.model_executor.models.qwen3_5 import Qwen3_5DecoderLayer

    _record_attention_conventions(qwen3_5)
    if _ORIGINAL_FORWARD is None:
        _ORIGINAL_FORWARD = Qwen3_5DecoderLayer.forward
    Qwen3_5DecoderLayer.forward = _patched_forward
    _STATE["armed"] = True


def _prepare(model, tokens: int) -> dict:
    layers = _CORE.decoder_layers(model, EXPECTED_LAYERS)
    if any(getattr(layer, "use_attn_reduce_scatter_for_moe", False) for layer in layers):
        raise RuntimeError("only the dense TP=1 layer form is supported by the Qwen MLP chain")
    if any(getattr(layer, "layer_scale", False) for layer in layers):
        raise RuntimeError("layers with layer_scale were never validated with the MLP chain")
    dims = _CORE.mlp_dims(layers[0])
    if dims != tuple(EXPECTED_SHAPES):
        raise RuntimeError(f"Qwen MLP dimensions {dims} are not the validated {tuple(EXPECTED_SHAPES)}")
    return _CORE.prepare(layers, tokens, dry_run_eps=1e-6)


def install(llm, tokens: int) -> dict:
    """Build the plans for one prefill length and the planes of every layer; dry-run once."""
    if not _STATE["armed"]:
        raise RuntimeError("qwen_patch.arm() has to run before the engine is built")
    if tokens not in INSTALLABLE_TOKENS:
        raise ValueError(f"{tokens} tokens is not an installable Qwen prefill length")
    info = llm.apply_model(functools.partial(_prepare, tokens=tokens))
    if isinstance(info, list):
        info = info[0]
    _STATE.update(installed=True, layers=info["layers"], shapes=(tokens,))
    return info


def counts() -> dict:
    return dict(_CALLS)


def check_calls(passes: int, since: dict | None = None) -> dict:
    """``passes`` forward passes must have taken the fused branch once per layer, and the
    functional branch never."""
    if not _STATE["installed"]:
        raise RuntimeError("nothing installed yet: qwen_patch.check_calls needs install() first")
    fused, reference = _CORE.tally(("chain.fused",), ("chain.reference",), since)
    expected = passes * _STATE["layers"]
    if fused != expected or reference:
        raise RuntimeError(f"Qwen chain: {fused} fused and {reference} functional calls, "
                           f"{expected} fused and 0 functional expected")
    return {"fused_calls": fused, "reference_calls": reference, "expected": expected}
