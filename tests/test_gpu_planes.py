"""Parity of the plane producers (CUDA, through the C ABI) with the CPU oracle."""
import pytest
import torch

from gpu_util import mismatch_fraction, seeded, within_ulps
from oracle import lc_oracle as O

pytestmark = pytest.mark.gpu
NAMES = ("2x2_postsum_cse", "2x2_locality_ordered")


@pytest.fixture(scope="module")
def lc():
    from lcgemm import chain_gauge, ops, planes, scheme

    return type("LC", (), dict(ops=ops, planes=planes, gauge=chain_gauge, load=staticmethod(scheme.load)))


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("shape", [(512, 256), (192, 256), (1000, 520), (999, 1001), (16, 24), (6999, 2500)])
def test_prepare_b_and_a_planes_bit_exact(lc, name, shape):
    rows, cols = shape
    tb, sch = O.Tables(name), lc.load(name)
    x = seeded(shape, 1 + rows, 0.02)
    got = lc.planes.prepare_b(x, sch)
    want = O.prepare_b(x.cpu(), tb)
    assert got.shape == want.shape
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))
    got = lc.planes.a_planes(x, sch)
    want = O.a_planes(x.cpu(), tb)
    assert got.shape == want.shape
    assert torch.equal(got.cpu().view(torch.int16), want.view(torch.int16))


def test_strided_weight_view(lc):
    sch, tb = lc.load("2x2_postsum_cse"), O.Tables("2x2_postsum_cse")
    big = seeded((300, 640), 5, 0.02)
    view = big[:, 64:576]                      # leading dimension 640, 128-byte offset
    got = lc.planes.prepare_b(view, sch)
    assert torch.equal(got.cpu().view(torch.int16), O.prepare_b(view.cpu(), tb).view(torch.int16))


@pytest.mark.parametrize("shape", [(64, 256), (256, 512), (130, 5120), (32, 8192), (8, 16400)])
def test_norm_planes(lc, shape):
    m, k = shape
    sch, tb = lc.load("2x2_postsum_cse"), O.Tables("2x2_postsum_cse")
    delta, residual = seeded(shape, 3), seeded(shape, 4)
    nw = seeded((k,), 5, 0.01)
    out = torch.empty(lc.ops.a_plane_shape(sch, m, k), device="cuda", dtype=torch.bfloat16)
    res_out = torch.empty_like(delta)
    lc.ops.norm_planes(sch, delta, residual, nw, 1e-6, res_out, out)
    want, h = O.norm_planes(delta.cpu(), residual.cpu(), nw.cpu(), 1e-6, tb)
    assert torch.equal(res_out.cpu().view(torch.int16), h.view(torch.int16))
    # rsqrt and the order of the sum of squares differ from the CPU: allow one bf16 ulp on a
    # small fraction of the elements.
    assert within_ulps(out, want, 1.0, floor=2e-3)
    assert mismatch_fraction(out, want) < 2e-3


@pytest.mark.parametrize("name", NAMES + ("2x2_locality_lead_single",))
@pytest.mark.parametrize("shape", [(64, 256), (130, 5120), (36, 7168), (32, 8192), (12, 9216), (8, 16400)])
def test_norm_planes_without_delta(lc, name, shape):
    """No delta: the residual stream is the input itself.  Every kernel form (register, lean, staged,
    generic; compile-time and run-time tables) must give the bits it gives for a delta of zeros, and
    must leave the residual_out argument alone."""
    m, k = shape
    sch = lc.load(name)
    residual, nw = seeded(shape, 4), seeded((k,), 5, 0.01)
    zero = torch.zeros_like(residual)
    want = torch.empty(lc.ops.a_plane_shape(sch, m, k), device="cuda", dtype=torch.bfloat16)
    lc.ops.norm_planes(sch, zero, residual, nw, 1e-6, torch.empty_like(residual), want)
    got = torch.full_like(want, float("nan"))
    lc.ops.norm_planes(sch, None, residual, nw, 1e-6, None, got)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    lc.ops.check_status()


@pytest.mark.parametrize("name", NAMES)
def test_norm_planes_lean_form_matches_the_other_forms(lc, name):
    """K = 6656 is the widest row the 416-thread register kernel takes, K = 6672 the narrowest the
    lean one takes with a delta, K = 8192 its widest: each against the oracle."""
    tb, sch = O.Tables(name), lc.load(name)
    for m, k in ((20, 6656), (20, 6672), (20, 8192)):
        delta, residual, nw = seeded((m, k), 3), seeded((m, k), 4), seeded((k,), 5, 0.01)
        out = torch.empty(lc.ops.a_plane_shape(sch, m, k), device="cuda", dtype=torch.bfloat16)
        res_out = torch.empty_like(delta)
        lc.ops.norm_planes(sch, delta, residual, nw, 1e-6, res_out, out)
        want, h = O.norm_planes(delta.cpu(), residual.cpu(), nw.cpu(), 1e-6, tb)
        assert torch.equal(res_out.cpu().view(torch.int16), h.view(torch.int16))
        assert within_ulps(out, want, 1.0, floor=2e-3)
        assert mismatch_fraction(out, want) < 2e-3


def test_norm_planes_in_place_residual(lc):
    sch = lc.load("2x2_postsum_cse")
    delta, residual = seeded((64, 512), 8), seeded((64, 512), 9)
    nw = seeded((512,), 10, 0.01)
    out = torch.empty(lc.ops.a_plane_shape(sch, 64, 512), device="cuda", dtype=torch.bfloat16)
    want_h = (delta.float() + residual.float()).to(torch.bfloat16)
    lc.ops.norm_planes(sch, delta, residual, nw, 1e-6, residual, out)     # residual_out aliases residual
    assert torch.equal(residual, want_h)


@pytest.mark.parametrize("shape", [(64, 256), (256, 1280), (34, 17408)])
def test_swiglu_planes_and_gauge(lc, shape):
    m, inter = shape
    sch, tb = lc.load("2x2_locality_ordered"), O.Tables("2x2_locality_ordered")
    z = seeded((m, 2 * inter), 6)
    got = lc.gauge.chain_a_planes(z, sch)
    want = O.chain_a_planes(z.cpu(), tb)
    assert within_ulps(got, want, 1.0, floor=1e-3)
    assert mismatch_fraction(got, want) < 1e-3
    s = lc.gauge.swiglu(z).cpu()
    zc = z.cpu()
    ref = torch.nn.functional.silu(zc[:, :inter].float()).to(torch.bfloat16) * zc[:, inter:]
    assert within_ulps(s, ref, 1.0, floor=1e-3) and mismatch_fraction(s, ref) < 1e-3


def test_prepare_down_b_matches_oracle(lc):
    sch, tb = lc.load("2x2_locality_ordered"), O.Tables("2x2_locality_ordered")
    w = seeded((320, 1280), 12, 0.02)
    got = lc.gauge.prepare_down_b(w, sch)
    assert torch.equal(got.cpu().view(torch.int16), O.prepare_down_b(w.cpu(), tb).view(torch.int16))


@pytest.mark.parametrize("m,k", [(96, 5120), (95, 5120), (64, 8192), (16, 8200)])
def test_dense_arm_seams(lc, m, k):
    """Even row counts up to K = 8192 take the register kernel, the rest the staged one."""
    delta, residual, nw = seeded((m, k), 1), seeded((m, k), 2), seeded((k,), 3, 0.01)
    x, h = lc.ops.add_rmsnorm(delta, residual, nw, 1e-6)
    hc = (delta.cpu().float() + residual.cpu().float()).to(torch.bfloat16)
    hf = hc.float()
    want = (hf * torch.rsqrt(hf.square().mean(-1, keepdim=True) + 1e-6) * (nw.cpu().float() + 1)).to(torch.bfloat16)
    assert torch.equal(h.cpu(), hc)
    assert within_ulps(x, want, 1.0, floor=1e-3) and mismatch_fraction(x, want) < 2e-3
    y = lc.ops.add(delta, residual)
    assert torch.equal(y.cpu(), hc)
    # without a delta: the bits of a zero delta, and the residual handed back as the stream
    x0, _ = lc.ops.add_rmsnorm(torch.zeros_like(residual), residual, nw, 1e-6)
    x1, h1 = lc.ops.add_rmsnorm(None, residual, nw, 1e-6)
    assert torch.equal(x0, x1) and h1 is residual


def test_shape_and_device_errors(lc):
    sch = lc.load("2x2_postsum_cse")
    with pytest.raises(ValueError):
        lc.ops.norm_planes(sch, seeded((63, 256), 1), seeded((63, 256), 2), seeded((256,), 3), 1e-6,
                           torch.empty((63, 256), device="cuda", dtype=torch.bfloat16),
                           torch.empty((7 * 32, 128), device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        lc.gauge.chain_a_planes(seeded((64, 2 * 192), 1), lc.load("2x2_locality_ordered"))
    with pytest.raises(ValueError):
        lc.planes.prepare_b(torch.zeros(64, 64, device="cuda"), sch)         # fp32 is refused
