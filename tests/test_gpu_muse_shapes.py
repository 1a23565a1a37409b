"""The reference's second model family (hidden 6656, intermediate 19968; its plans at
``lcgemm/seams/down.py:42-54,88-98``) through the same chain and the two-op boundary's plans,
at full size.  The CPU oracle does not finish these sizes in seconds, so the checks are the
size-independent ones: the chained epilogue against the unfused plane kernel bit for bit, the
GEMM outputs against cuBLAS on row and column samples, and the whole layer against the stock
layer's functional form on a row sample.
"""
import pytest
import torch

from gpu_util import rel_fro

pytestmark = pytest.mark.gpu
H, I = 6656, 19968


@pytest.mark.parametrize("tokens", [2048, 4096])
def test_muse_sized_chain(tokens):
    from lcgemm import ops
    from lcgemm.seams import build_chain

    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(tokens)
    bf = torch.bfloat16
    x = torch.randn((tokens, H), generator=g, device=dev).to(bf)
    delta = (torch.randn((tokens, H), generator=g, device=dev) * 0.1).to(bf)
    nw = (torch.randn((H,), generator=g, device=dev) * 0.01).to(bf)
    wgu = (torch.randn((2 * I, H), generator=g, device=dev) * 0.02).to(bf)
    wd = (torch.randn((H, I), generator=g, device=dev) * 0.02).to(bf)
    gate, down = build_chain((tokens, H, 2 * I), (tokens, I, H))
    gate_bw, down_bw = gate.prepare_weight(wgu), down.prepare_weight(wd)
    z = gate(x, delta, nw, 1e-6, prepared_w=gate_bw)
    out = down(prepared_w=down_bw)
    ops.check_status()
    # residual stream and the chained epilogue
    h = (delta.float() + x.float()).to(bf)
    assert torch.equal(gate.residual_out, h)
    assert torch.equal(gate.planes, ops.swiglu_planes(gate.plane_scheme, z))
    # gate_up and the whole layer on a row sample against cuBLAS with the stock rounding points
    rows = torch.arange(0, tokens, tokens // 128, device=dev)
    hf = h[rows].float()
    y = (hf * torch.rsqrt(hf.square().mean(-1, keepdim=True) + 1e-6) * (nw.float() + 1.0)).to(bf)
    want_z = torch.nn.functional.linear(y, wgu)
    assert rel_fro(z[rows], want_z) <= 1.0e-2
    gz, uz = want_z.chunk(2, dim=-1)
    want = torch.nn.functional.linear(torch.nn.functional.silu(gz.float()).to(bf) * uz, wd)
    assert rel_fro(out[rows], want) <= 2.0e-2
    assert out.shape == (tokens, H) and bool(torch.isfinite(out.float()).all())
