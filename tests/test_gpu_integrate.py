"""The operator boundary: the custom ops dispatch on the exact installed token count and on
the weights' addresses, count fused and reference calls, and agree with the functional form."""
import pytest
import torch
import torch.nn as nn

from gpu_util import rel_fro, seeded

pytestmark = pytest.mark.gpu

H, I, LAYERS = 256, 512, 2


class _Proj(nn.Module):
    def __init__(self, w):
        super().__init__()
        self.weight = nn.Parameter(w, requires_grad=False)


class _Mlp(nn.Module):
    def __init__(self, seed):
        super().__init__()
        self.gate_up_proj = _Proj(seeded((2 * I, H), seed, 0.02))
        self.down_proj = _Proj(seeded((H, I), seed + 1, 0.02))


def _layer_class(name):
    def __init__(self, seed):
        nn.Module.__init__(self)
        self.mlp = _Mlp(seed)
        self.use_attn_reduce_scatter_for_moe = False
        self.layer_scale = False
    return type(name, (nn.Module,), {"__init__": __init__})


class _FakeLLM:
    def __init__(self, cls_name):
        cls = _layer_class(cls_name)
        self.model = nn.ModuleList([cls(100 + 10 * n) for n in range(LAYERS)])

    def apply_model(self, fn):
        return [fn(self.model)]


def test_qwen_custom_op_dispatch_and_counters(monkeypatch):
    from lcgemm import ops
    from lcgemm.integrate import qwen_patch as qp

    monkeypatch.setattr(qp, "EXPECTED_LAYERS", LAYERS)
    monkeypatch.setattr(qp, "EXPECTED_SHAPES", (H, I, 2 * I, H))
    monkeypatch.setitem(qp._STATE, "armed", True)       # arming proper needs a vLLM import
    llm = _FakeLLM(qp.LAYER_CLASS_NAME)
    with pytest.raises(ValueError):
        qp.install(llm, tokens=768)
    info = qp.install(llm, tokens=512)
    assert info["layers"] == LAYERS and info["tokens"] == 512
    assert info["schemes"] == {"gate_up": "2x2_postsum_cse", "down": "2x2_locality_ordered"}
    assert "rank7" in info["describe"]["gate_up"] and info["planes_gib"] > 0

    nw = seeded((H,), 5, 0.01)
    before = qp.counts()
    for layer in llm.model:
        delta, residual = seeded((512, H), 1), seeded((512, H), 2)
        out, res = torch.ops.lcgemm_qwen.mlp_chain(
            delta, residual, nw, layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight, 1e-6)
        want, want_res = qp._reference(delta, residual, nw, layer.mlp.gate_up_proj.weight,
                                       layer.mlp.down_proj.weight, 1e-6)
        assert torch.equal(res, want_res)
        assert rel_fro(out, want) <= 2e-2
        assert res.data_ptr() != residual.data_ptr() and res.data_ptr() != delta.data_ptr()
    assert qp.check_calls(1, since=before) == {"fused_calls": LAYERS, "reference_calls": 0,
                                               "expected": LAYERS}
    # another token count, or weights that were never installed, take the reference branch
    mid = qp.counts()
    layer = llm.model[0]
    torch.ops.lcgemm_qwen.mlp_chain(seeded((64, H), 1), seeded((64, H), 2), nw,
                                    layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight, 1e-6)
    torch.ops.lcgemm_qwen.mlp_chain(seeded((512, H), 1), seeded((512, H), 2), nw,
                                    layer.mlp.gate_up_proj.weight.clone(), layer.mlp.down_proj.weight, 1e-6)
    after = qp.counts()
    assert after["chain.reference"] - mid.get("chain.reference", 0) == 2
    with pytest.raises(RuntimeError):
        qp.check_calls(1, since=mid)
    ops.check_status()


def test_qwen_custom_op_clones_an_output_that_shares_an_input_buffer(monkeypatch):
    """A compiled engine may hand layer n + 1 an input that still sits in the plan buffer layer n
    returned.  The kernels read their inputs before anything overwrites that buffer, so the result
    must be the one a private copy of the input gives; the op must then return storage of its own
    (a custom op may not return storage one of its inputs lives in) and count the copy."""
    from lcgemm import ops
    from lcgemm.integrate import qwen_patch as qp

    monkeypatch.setattr(qp, "EXPECTED_LAYERS", LAYERS)
    monkeypatch.setattr(qp, "EXPECTED_SHAPES", (H, I, 2 * I, H))
    monkeypatch.setitem(qp._STATE, "armed", True)
    llm = _FakeLLM(qp.LAYER_CLASS_NAME)
    qp.install(llm, tokens=512)
    nw = seeded((H,), 5, 0.01)
    layer = llm.model[0]
    w_gu, w_d = layer.mlp.gate_up_proj.weight, layer.mlp.down_proj.weight
    delta, residual = seeded((512, H), 1), seeded((512, H), 2)
    first, _ = torch.ops.lcgemm_qwen.mlp_chain(delta, residual, nw, w_gu, w_d, 1e-6)
    shared = first                                   # lives in the plan's output buffer
    private = first.clone()
    before = qp.counts().get("chain.cloned_output", 0)
    # the shared call first: the call on the private copy overwrites the plan buffer `shared` sits in
    got, _ = torch.ops.lcgemm_qwen.mlp_chain(shared, residual, nw, w_gu, w_d, 1e-6)
    assert qp.counts().get("chain.cloned_output", 0) == before + 1
    assert got.untyped_storage().data_ptr() != shared.untyped_storage().data_ptr()
    want, _ = torch.ops.lcgemm_qwen.mlp_chain(private, residual, nw, w_gu, w_d, 1e-6)
    assert qp.counts().get("chain.cloned_output", 0) == before + 1      # no copy for a private input
    assert rel_fro(got, want) <= 8e-3               # rank-split down: bf16 adds in hardware order
    ops.check_status()


def test_muse_two_op_boundary(monkeypatch):
    from lcgemm import ops
    from lcgemm.integrate import muse_patch as mp

    monkeypatch.setattr(mp, "EXPECTED_LAYERS", LAYERS)
    monkeypatch.setattr(mp, "EXPECTED_SHAPES", (H, I, 2 * I, H))
    monkeypatch.setitem(mp._STATE, "armed", True)
    llm = _FakeLLM(mp.LAYER_CLASS_NAME)
    info = mp.install(llm, tokens=512)
    assert info["layers"] == LAYERS
    nw = seeded((H,), 5, 0.01)
    before = mp.counts()
    layer = llm.model[1]
    delta, residual = seeded((512, H), 3), seeded((512, H), 4)
    res, gate_up = torch.ops.lcgemm_muse.norm_gateup(delta, residual, nw, layer.mlp.gate_up_proj.weight, 1e-5)
    out = torch.ops.lcgemm_muse.swiglu_down(gate_up, layer.mlp.down_proj.weight)
    h = (delta.float() + residual.float()).to(torch.bfloat16)
    assert torch.equal(res, h)
    x = mp._rmsnorm(h, nw, 1e-5)
    want_gu = torch.nn.functional.linear(x, layer.mlp.gate_up_proj.weight)
    assert rel_fro(gate_up, want_gu) <= 1e-2
    g, u = want_gu.chunk(2, dim=-1)
    want = torch.nn.functional.linear(torch.nn.functional.silu(g) * u, layer.mlp.down_proj.weight)
    assert rel_fro(out, want) <= 2.5e-2
    mp._STATE["layers"] = 1                 # one layer exercised: two fused ops expected
    assert mp.check_calls(1, since=before)["fused_calls"] == 2
    ops.check_status()
