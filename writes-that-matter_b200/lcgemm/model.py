"""A random-init dense decoder for end-to-end prefill comparisons (stock MLP vs rank-7 MLP).

The reference measures its patch inside a vLLM engine on real checkpoints
(``lcgemm/bench/prefill.py:76-176``).  Neither the checkpoints nor the pinned engine are
available to this build, so this module is the stand-in: the same layer recipe as the patched
decoder forward (``lcgemm/integrate/qwen_patch.py:116-178``) -- fused add + RMSNorm with the
``(w + 1)`` scale, attention, then the MLP chain returning ``(down_out, residual)`` -- with
torch attention (SDPA, grouped-query, RoPE) and random weights.  Both arms share every tensor and
every line of code except the MLP, so a difference in the output is the MLP's alone.

Arms of :meth:`RandomInitDecoder.prefill`:

``"stock"``   the stock layer as an engine runs it: fused add + RMSNorm kernel, cuBLAS GEMMs,
              fused SwiGLU kernel (the rounding points of ``qwen_patch.py:41-58``);
``"eager"``   the same layer as plain torch ops, the functional reference itself;
``"rank7"``   the chained rank-7 plans of this package (one ``build_chain`` for the model, B
              planes prepared per layer at :meth:`install`, as ``qwen_patch._prepare`` does);
``"rank7_allranks"``  the same plans on the all-ranks schedule for both GEMMs: every C block
              has one writer and a fixed order of additions, so the result is reproducible bit
              for bit (slower: ``down`` then has fewer tiles than the GPU has CTA pairs);
``"dense"``   the stock layer on this package's dense tcgen05 GEMM.

The input norm of every layer uses the fused add + RMSNorm kernel in all arms.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import ops
from ._native import SCHEDULE_ALL_RANKS
from .seams import build_chain


@dataclass
class DecoderConfig:
    layers: int = 64
    hidden: int = 5120
    q_heads: int = 40
    kv_heads: int = 8
    head_dim: int = 128
    inter: int = 17408
    vocab: int = 151936
    rope_theta: float = 1.0e6
    eps: float = 1.0e-6
    seed: int = 0


def _rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    f = x.float()
    f = f * torch.rsqrt(f.square().mean(-1, keepdim=True) + eps)
    return (f * (weight.float() + 1.0)).to(x.dtype)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on (tokens, heads, head_dim)."""
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half].float(), x[..., half:].float()
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class RandomInitDecoder:
    """Weights ~ N(0, 0.02), norm weights ~ N(0, 0.01) (effective scale 1 + w), fixed seed."""

    def __init__(self, cfg: DecoderConfig, device=None):
        self.cfg = cfg
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        g = torch.Generator(device=self.device).manual_seed(cfg.seed)
        bf = torch.bfloat16

        def w(*shape, scale=0.02):
            return (torch.randn(shape, generator=g, device=self.device) * scale).to(bf)

        qkv = (cfg.q_heads + 2 * cfg.kv_heads) * cfg.head_dim
        self.embed = w(cfg.vocab, cfg.hidden)
        self.lm_head = w(cfg.vocab, cfg.hidden)
        self.final_norm = w(cfg.hidden, scale=0.01)
        self.layers = []
        for _ in range(cfg.layers):
            self.layers.append(dict(
                input_norm=w(cfg.hidden, scale=0.01), qkv=w(qkv, cfg.hidden),
                o=w(cfg.hidden, cfg.q_heads * cfg.head_dim), post_norm=w(cfg.hidden, scale=0.01),
                gate_up=w(2 * cfg.inter, cfg.hidden), down=w(cfg.hidden, cfg.inter)))
        self._plans = {}
        self._plans_det = {}
        self._dense = {}
        self.calls = {"fused": 0, "reference": 0}

    # ------------------------------------------------------------------ install
    def install(self, tokens: int) -> dict:
        """Plans for one exact prefill length and B planes for every layer."""
        cfg = self.cfg
        gate, down = build_chain((tokens, cfg.hidden, 2 * cfg.inter), (tokens, cfg.inter, cfg.hidden))
        det_gate, det_down = build_chain((tokens, cfg.hidden, 2 * cfg.inter), (tokens, cfg.inter, cfg.hidden))
        det_gate.schedule = SCHEDULE_ALL_RANKS
        det_down.rank_split = False
        det_gate.preclear = det_gate.c                    # an all-ranks consumer initialises its own output
        self._plans_det[tokens] = (det_gate, det_down)
        nbytes = 0
        for layer in self.layers:
            if "gate_bw" not in layer:
                layer["gate_bw"] = gate.prepare_weight(layer["gate_up"])
                layer["down_bw"] = down.prepare_weight(layer["down"])
            nbytes += (layer["gate_bw"].numel() + layer["down_bw"].numel()) * 2
        self._plans[tokens] = (gate, down)
        ops.check_status()
        return {"layers": cfg.layers, "tokens": tokens, "planes_gib": nbytes / 2 ** 30,
                "describe": {"gate_up": gate.describe(), "down": down.describe()}}

    # --------------------------------------------------------------------- MLP arms
    def _mlp(self, arm: str, layer: dict, delta, residual, ring):
        cfg = self.cfg
        m = delta.shape[0]
        if arm in ("rank7", "rank7_allranks") and m in self._plans:
            gate, down = self._plans[m] if arm == "rank7" else self._plans_det[m]
            self.calls["fused"] += 1
            res_out = ring[0]
            ring.reverse()
            gate(residual, delta, layer["post_norm"], cfg.eps, prepared_w=layer["gate_bw"],
                 residual_out=res_out)
            return down(prepared_w=layer["down_bw"]), res_out
        self.calls["reference"] += 1
        if arm == "eager":
            h = (delta.float() + residual.float()).to(delta.dtype)
            x = _rmsnorm(h, layer["post_norm"], cfg.eps)
            gate_, up = F.linear(x, layer["gate_up"]).chunk(2, dim=-1)
            act = F.silu(gate_.float()).to(gate_.dtype) * up
            return F.linear(act, layer["down"]), h
        h = ring[0]
        ring.reverse()
        x, _ = ops.add_rmsnorm(delta, residual, layer["post_norm"], cfg.eps, residual_out=h)
        if arm == "dense":
            z = ops.gemm_dense(x, layer["gate_up"])
            return ops.gemm_dense(ops.swiglu(z), layer["down"]), h
        return F.linear(ops.swiglu(F.linear(x, layer["gate_up"])), layer["down"]), h

    # ---------------------------------------------------------------------- forward
    @torch.no_grad()
    def prefill(self, token_ids: torch.Tensor, arm: str = "stock"):
        """Batch-1 prefill; returns (logits of the last position as fp32, final hidden state)."""
        if arm not in ("stock", "eager", "rank7", "rank7_allranks", "dense"):
            raise ValueError(f"unknown arm {arm!r}")
        cfg = self.cfg
        m = token_ids.shape[0]
        if arm in ("rank7", "rank7_allranks") and m not in self._plans:
            raise RuntimeError(f"install({m}) before a rank-7 prefill of {m} tokens")
        pos = torch.arange(m, device=self.device, dtype=torch.float32)
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, cfg.head_dim, 2, device=self.device,
                                                     dtype=torch.float32) / cfg.head_dim))
        ang = pos[:, None] * inv[None, :]
        cos, sin = ang.cos(), ang.sin()
        hidden = self.embed[token_ids]
        residual = None
        ring = [torch.empty_like(hidden), torch.empty_like(hidden)]
        q_dim, kv_dim = cfg.q_heads * cfg.head_dim, cfg.kv_heads * cfg.head_dim
        for layer in self.layers:
            if residual is None:
                residual = hidden
                x = _rmsnorm(hidden, layer["input_norm"], cfg.eps)
            else:
                x, residual = ops.add_rmsnorm(hidden.contiguous(), residual, layer["input_norm"], cfg.eps)
            qkv = F.linear(x, layer["qkv"])
            q = _rope(qkv[:, :q_dim].view(m, cfg.q_heads, cfg.head_dim), cos, sin)
            k = _rope(qkv[:, q_dim:q_dim + kv_dim].view(m, cfg.kv_heads, cfg.head_dim), cos, sin)
            v = qkv[:, q_dim + kv_dim:].view(m, cfg.kv_heads, cfg.head_dim)
            att = F.scaled_dot_product_attention(
                q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None],
                is_causal=True, enable_gqa=True)[0].transpose(0, 1).reshape(m, q_dim)
            delta = F.linear(att, layer["o"])
            hidden, residual = self._mlp(arm, layer, delta, residual, ring)
        final = _rmsnorm((hidden.float() + residual.float()).to(hidden.dtype), self.final_norm, cfg.eps)
        logits = F.linear(final[-1:], self.lm_head).float()[0]
        return logits, final


LOGIT_STEP = 0.125      # one quantisation step of the log-probabilities (lcgemm/bench/prefill.py:180-183)


def tie_aware_overlap(ref_logits: torch.Tensor, got_logits: torch.Tensor, k: int = 20,
                      step: float = LOGIT_STEP) -> int:
    """The agreement count of ``lcgemm/bench/prefill.py:186-197`` /
    ``lcgemm/bench/headline.py:48-64``: a token of the reference arm's top-k counts when the
    other arm's top-k holds it too, or when its log-probability lies within ``step`` of the
    other arm's cut (everything at that boundary competes on values that round alike)."""
    ref_lp = torch.log_softmax(ref_logits.float(), dim=-1)
    got_lp = torch.log_softmax(got_logits.float(), dim=-1)
    ref_top = torch.topk(ref_lp, k)
    got_top = torch.topk(got_lp, k)
    cut = got_top.values.min()
    in_other = torch.isin(ref_top.indices, got_top.indices)
    near_cut = ref_top.values <= cut + step
    return int((in_other | near_cut).sum().item())


def compare_arms(ref_logits, got_logits, ref_hidden, got_hidden) -> dict:
    return {
        "top1_equal": bool(ref_logits.argmax() == got_logits.argmax()),
        "top1_gap": float(torch.topk(ref_logits, 2).values.diff().abs().item()),
        "tie_aware_top20": tie_aware_overlap(ref_logits, got_logits),
        "max_abs_logit_diff": float((ref_logits - got_logits).abs().max().item()),
        "logit_std": float(ref_logits.std().item()),
        "hidden_rel_fro": float(((got_hidden.float() - ref_hidden.float()).norm()
                                 / ref_hidden.float().norm()).item()),
    }
