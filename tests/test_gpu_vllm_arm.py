"""arm() against the vLLM that is actually installed: the decoder class's forward is replaced,
and the replacement drives a layer object through the class's own attention calling convention
and through the custom op (functional branch here: nothing is installed for these weights)."""
import pytest
import torch
import torch.nn as nn

from gpu_util import seeded

pytestmark = pytest.mark.gpu


class _Norm(nn.Module):
    """add + RMSNorm with the (w + 1) scale, under the fused-residual calling convention."""

    def __init__(self, k):
        super().__init__()
        self.weight = nn.Parameter(seeded((k,), 3, 0.01), requires_grad=False)
        self.variance_epsilon = 1e-6

    def forward(self, x, residual=None):
        from lcgemm.integrate._common import gemma_rmsnorm

        if residual is None:
            return gemma_rmsnorm(x, self.weight, self.variance_epsilon)
        h = (x.float() + residual.float()).to(x.dtype)
        return gemma_rmsnorm(h, self.weight, self.variance_epsilon), h


class _AttnFillsOutput(nn.Module):
    def forward(self, hidden_states, output, positions=None):
        output.copy_(hidden_states * 0.5)


class _AttnReturns(nn.Module):
    def forward(self, hidden_states, positions=None):
        return hidden_states * 0.5


class _Proj(nn.Module):
    def __init__(self, w):
        super().__init__()
        self.weight = nn.Parameter(w, requires_grad=False)


def test_arm_replaces_the_installed_decoder_forward():
    import os

    os.environ.setdefault("VLLM_DISABLE_COMPILE_CACHE", "1")
    try:
        from vllm.model_executor.models.qwen3_5 import Qwen3_5DecoderLayer
    except Exception as exc:                      # no vLLM, or a vLLM without this model
        pytest.skip(f"vLLM's Qwen3_5DecoderLayer is not importable here: {exc}")
    from lcgemm.integrate import qwen_patch as qp

    stock_forward = Qwen3_5DecoderLayer.forward
    try:
        qp.arm()
        assert qp._STATE["armed"] and Qwen3_5DecoderLayer.forward is qp._patched_forward
        h, i, m = 256, 512, 64
        for attn in (_AttnFillsOutput(), _AttnReturns()):
            layer = nn.Module()
            layer.input_layernorm, layer.post_attention_layernorm = _Norm(h).cuda(), _Norm(h).cuda()
            layer.self_attn, layer.layer_type, layer.layer_scale = attn, "full_attention", False
            layer.mlp = nn.Module()
            layer.mlp.gate_up_proj = _Proj(seeded((2 * i, h), 5, 0.02))
            layer.mlp.down_proj = _Proj(seeded((h, i), 6, 0.02))
            x, res = seeded((m, h), 1), seeded((m, h), 2)
            before = qp.counts().get("chain.reference", 0)
            out, new_res = Qwen3_5DecoderLayer.forward(layer, x, res, positions=torch.arange(m).cuda())
            assert qp.counts()["chain.reference"] == before + 1
            normed, res1 = layer.input_layernorm(x, res)
            want, want_res = qp._reference(normed * 0.5, res1, layer.post_attention_layernorm.weight,
                                           layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight, 1e-6)
            assert torch.equal(out, want) and torch.equal(new_res, want_res)
    finally:
        Qwen3_5DecoderLayer.forward = stock_forward
        qp._STATE["armed"] = False
