"""Shared machinery of the vLLM decoder patches.

A patch owns: whether the decoder class has been swapped (``armed``), the plans built for one
exact prefill length, the operand planes prepared for every layer's weights (keyed by the
weights' device addresses, which is all a custom op can see), counters of which branch each
call took, and a two-buffer ring for the residual stream (a custom op may not hand back an
alias of one of its inputs, and layer n's residual is an input of layer n + 1).
"""
from __future__ import annotations

import os
import sys
from collections import defaultdict

import torch
import torch.nn.functional as F

from lcgemm.seams import build_chain


def compile_cache_guard():
    """Record how vLLM's compile cache stood when the patch module was imported, then switch
    it off: a cached stock graph must never stand in for the patched forward."""
    preset = os.environ.get("VLLM_DISABLE_COMPILE_CACHE") in ("1", "true", "True")
    preimported = "vllm" in sys.modules
    os.environ["VLLM_DISABLE_COMPILE_CACHE"] = "1"
    return preset, preimported


def gemma_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """RMSNorm whose stored weight carries a baked ``-1`` offset (effective scale ``w + 1``)."""
    f = x.float()
    f = f * torch.rsqrt(f.square().mean(-1, keepdim=True) + eps)
    return (f * (weight.float() + 1.0)).to(x.dtype)


class PatchCore:
    """State and installation logic common to the one-op and the two-op boundary."""

    def __init__(self, state: dict, layer_class_name: str):
        self.state = state
        self.layer_class_name = layer_class_name
        self.plans: dict = {}            # tokens -> (GateUpPlan, DownPlan)
        self.by_gate: dict = {}          # gate_up weight address -> (down address, gate planes, down planes)
        self.by_down: dict = {}          # down weight address -> down planes
        self.calls: dict = defaultdict(int)
        self._ring: list = []
        self._turn = 0

    # ------------------------------------------------------------------ residual ring
    def residual_buffer(self, like: torch.Tensor) -> torch.Tensor:
        stale = (not self._ring or self._ring[0].shape != like.shape
                 or self._ring[0].device != like.device or self._ring[0].dtype != like.dtype)
        if stale:
            self._ring = [torch.empty_like(like) for _ in range(2)]
            self._turn = 0
        buf = self._ring[self._turn]
        self._turn ^= 1
        return buf

    # ---------------------------------------------------------------------- install
    def decoder_layers(self, model, expected: int) -> list:
        found = [m for m in model.modules() if type(m).__name__ == self.layer_class_name]
        if len(found) != expected:
            raise RuntimeError(f"expected {expected} {self.layer_class_name} modules, found {len(found)}")
        return found

    @staticmethod
    def mlp_dims(layer):
        gate_up = layer.mlp.gate_up_proj.weight.data
        down = layer.mlp.down_proj.weight.data
        return gate_up.shape[1], down.shape[1], gate_up.shape[0], down.shape[0]    # H, I, 2I, H_out

    def prepare(self, layers: list, tokens: int, dry_run_eps: float) -> dict:
        """Plans for ``tokens``, planes for every layer, one dry run on zeros."""
        from lcgemm import ops

        hidden, inter, two_inter, out_dim = self.mlp_dims(layers[0])
        gate_plan, down_plan = build_chain((tokens, hidden, two_inter), (tokens, inter, out_dim))
        self.plans[tokens] = (gate_plan, down_plan)
        plane_bytes = 0
        sample = None
        for layer in layers:
            w_gate = layer.mlp.gate_up_proj.weight.data
            w_down = layer.mlp.down_proj.weight.data
            gate_planes = gate_plan.prepare_weight(w_gate)
            down_planes = down_plan.prepare_weight(w_down)
            self.by_gate[w_gate.data_ptr()] = (w_down.data_ptr(), gate_planes, down_planes)
            self.by_down[w_down.data_ptr()] = down_planes
            plane_bytes += gate_planes.numel() * gate_planes.element_size()
            plane_bytes += down_planes.numel() * down_planes.element_size()
            if sample is None:
                sample = (gate_planes, down_planes)
        zeros = torch.zeros((tokens, hidden), device="cuda", dtype=torch.bfloat16)
        gate_plan(zeros, zeros.clone(), torch.zeros((hidden,), device="cuda", dtype=torch.bfloat16),
                  dry_run_eps, prepared_w=sample[0])
        down_plan(prepared_w=sample[1])
        ops.check_status()                     # synchronises; raises if a device-side wait ran out
        return {
            "layers": len(layers),
            "planes_gib": plane_bytes / 2 ** 30,
            "tokens": tokens,
            "schemes": {"gate_up": gate_plan.scheme.name, "down": down_plan.scheme.name},
            "describe": {"gate_up": gate_plan.describe(), "down": down_plan.describe()},
        }

    # --------------------------------------------------------------------- counters
    def tally(self, fused_keys, reference_keys, since: dict | None):
        base = since or {}
        fused = sum(self.calls[k] - base.get(k, 0) for k in fused_keys)
        reference = sum(self.calls[k] - base.get(k, 0) for k in reference_keys)
        return fused, reference


def stock_swiglu_down(gate_up: torch.Tensor, down_weight: torch.Tensor, *, round_silu: bool):
    gate, up = gate_up.chunk(2, dim=-1)
    act = (F.silu(gate.float()).to(gate.dtype) if round_silu else F.silu(gate)) * up
    return F.linear(act, down_weight)
