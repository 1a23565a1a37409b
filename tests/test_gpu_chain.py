"""The chained seams (GateUpPlan / DownPlan / build_chain) and the layer arms against the
CPU oracle, plus bit-level agreement of the fused plane epilogue with the unfused kernels."""
import pytest
import torch

from gpu_util import mismatch_fraction, rel_fro, seeded, within_ulps
from oracle import lc_oracle as O

pytestmark = pytest.mark.gpu
GATE, DOWN = "2x2_postsum_cse", "2x2_locality_ordered"


@pytest.fixture(scope="module")
def lc():
    from lcgemm import chain_gauge, layer, ops, planes, scheme, seams

    return type("LC", (), dict(ops=ops, planes=planes, gauge=chain_gauge, seams=seams, layer=layer,
                               load=staticmethod(scheme.load)))


@pytest.fixture(autouse=True)
def _status_clean(lc):
    yield
    lc.ops.check_status()


def _layer_inputs(m, h, i, seed=0):
    return (seeded((m, h), seed + 1), seeded((m, h), seed + 2), seeded((h,), seed + 3, 0.01),
            seeded((2 * i, h), seed + 4, 0.02), seeded((h, i), seed + 5, 0.02))


@pytest.mark.parametrize("dims", [(256, 256, 512), (512, 384, 1280), (130, 128, 256), (258, 128, 384), (2, 128, 128)])
def test_chain_against_oracle(lc, dims):
    m, h, i = dims
    delta, residual, nw, wgu, wd = _layer_inputs(m, h, i)
    gate, down = lc.seams.build_chain((m, h, 2 * i), (m, i, h))
    assert down.rank_split and gate.preclear is down.c
    gate_bw, down_bw = gate.prepare_weight(wgu), down.prepare_weight(wd)
    z = gate(residual, delta, nw, 1e-6, prepared_w=gate_bw)
    out = down(prepared_w=down_bw)
    want_out, want_h, want_z, want_pl = O.mlp_chain(
        delta.cpu(), residual.cpu(), nw.cpu(), wgu.cpu(), wd.cpu(), 1e-6, O.Tables(GATE), O.Tables(DOWN))
    assert torch.equal(gate.residual_out.cpu().view(torch.int16), want_h.view(torch.int16))
    assert rel_fro(z, want_z) <= 8e-3              # hybrid schedule: split tail, unordered bf16 adds
    # planes from the device's own Z must match the oracle's transform of that same Z
    pl_from_dev_z = O.chain_a_planes(z.cpu(), O.Tables(DOWN))
    assert within_ulps(gate.planes, pl_from_dev_z, 1.0, floor=1e-3)
    assert mismatch_fraction(gate.planes, pl_from_dev_z) < 1e-3
    # down from the device's own planes, against the oracle's rank-split model of it
    prods = O.products(gate.planes.cpu(), O.prepare_down_b(wd.cpu(), O.Tables(DOWN)), 7)
    assert rel_fro(out, O.combine_as_kernel(prods, O.Tables(DOWN), m, h, rank_split=True)) <= 8e-3
    assert rel_fro(out, want_out) <= 2e-2           # whole chain, both stages' tolerances stacked
    ref, _ = O.mlp_reference(delta.cpu(), residual.cpu(), nw.cpu(), wgu.cpu(), wd.cpu(), 1e-6)
    assert rel_fro(out, ref) <= 2e-2


@pytest.mark.parametrize("group", [1, 2])
@pytest.mark.parametrize("dims", [(1024, 512, 1280), (2048, 256, 5120)])
def test_fused_epilogue_equals_unfused_kernels(lc, group, dims):
    m, h, i = dims
    gs, ds = lc.load(GATE), lc.load(DOWN)
    x, w = seeded((m, h), 1), seeded((2 * i, h), 2, 0.02)
    ap, bp = lc.planes.a_planes(x, gs), lc.planes.prepare_b(w, gs)
    z = torch.empty((m, 2 * i), device="cuda", dtype=torch.bfloat16)
    pl = torch.full((7 * m // 2, i // 2), 3.0, device="cuda", dtype=torch.bfloat16)
    pc = torch.ones((m, 520), device="cuda", dtype=torch.bfloat16)
    lc.ops.gate_up_chain(gs, ds, ap, bp, z, pl, preclear=pc, schedule=0, cta_group=group)
    z_plain = lc.ops.gemm_r7_planes(gs, ap, bp, m, 2 * i, h, schedule=0, cta_group=group)
    assert torch.equal(z, z_plain)                          # all-ranks schedule: deterministic
    assert torch.equal(pl, lc.gauge.chain_a_planes(z, ds))
    assert bool((pc == 0).all())
    # Hybrid schedule: the tail tiles' products arrive as reduce-adds from several CTAs, so Z
    # agrees within the rank-split tolerance; the planes must still be exactly the transform
    # of the Z this launch produced (the tail tiles' plane phase runs behind the GEMM kernel).
    for _ in range(2):                                      # twice: no state is carried over
        z2 = torch.full_like(z, 5.0)
        pl2 = torch.full_like(pl, 3.0)
        pc.fill_(1.0)
        lc.ops.gate_up_chain(gs, ds, ap, bp, z2, pl2, preclear=pc, schedule=2, cta_group=group)
        assert rel_fro(z2, z_plain) <= 8e-3
        assert torch.equal(pl2, lc.gauge.chain_a_planes(z2, ds))
        assert bool((pc == 0).all())


def test_full_size_chain_qwen_4096(lc):
    m, h, i = 4096, 5120, 17408
    x = torch.randn((m, h), device="cuda").to(torch.bfloat16)
    nw = (torch.randn(h, device="cuda") * 0.01).to(torch.bfloat16)
    wgu = (torch.randn((2 * i, h), device="cuda") * 0.02).to(torch.bfloat16)
    wd = (torch.randn((h, i), device="cuda") * 0.02).to(torch.bfloat16)
    r7 = lc.layer.Rank7MlpLayer(m, nw, wgu, wd)
    out = r7(x).clone()
    gate, down = r7.gate_plan, r7.down_plan
    assert "rank7/hybrid" in gate.describe() and "734 units" in gate.describe()
    assert "644 units" in down.describe()
    # fused planes == unfused kernel on the same Z, bit for bit
    assert torch.equal(gate.planes, lc.gauge.chain_a_planes(gate.c, gate.plane_scheme))
    # the three arms agree within the stated tolerance
    tc = lc.layer.DenseMlpLayer(m, nw, wgu, wd, gemm="tcgen05")(x).clone()
    cb = lc.layer.DenseMlpLayer(m, nw, wgu, wd, gemm="cublas")(x).clone()
    assert rel_fro(tc[::3], cb[::3]) <= 3e-3
    assert rel_fro(out[::3], cb[::3]) <= 1.5e-2
    # the MLP branch alone (without the residual that dominates `out`)
    mlp_r7 = out[::3].float() - x[::3].float()
    mlp_cb = cb[::3].float() - x[::3].float()
    assert rel_fro(mlp_r7, mlp_cb) <= 5e-2
    # a second pass over the same buffers gives the same answer (pre-clear works every time) up to
    # the order of the rank-split down projection's bf16 reduce-adds, which differs run to run
    # (most on a cold first launch): same 8e-3 as rank-split against the ordered schedule
    out2 = r7(x)
    assert rel_fro(out2, out) < 8e-3


def test_layer_arms_small_against_reference(lc):
    m, h, i = 256, 256, 512
    delta, residual, nw, wgu, wd = _layer_inputs(m, h, i, seed=20)
    ref, href = O.mlp_reference(delta.cpu(), residual.cpu(), nw.cpu(), wgu.cpu(), wd.cpu(), 1e-6)
    for arm in (lc.layer.Rank7MlpLayer(m, nw, wgu, wd), lc.layer.DenseMlpLayer(m, nw, wgu, wd),
                lc.layer.DenseMlpLayer(m, nw, wgu, wd, gemm="cublas")):
        d, hh = arm.chain(delta, residual)
        assert torch.equal(hh.cpu().view(torch.int16), href.view(torch.int16))
        assert rel_fro(d, ref) <= (2e-2 if isinstance(arm, lc.layer.Rank7MlpLayer) else 6e-3)
        out = arm(residual, delta)
        want = (href.float() + d.cpu().float()).to(torch.bfloat16)
        assert torch.equal(out.cpu().view(torch.int16), want.view(torch.int16))


def test_layer_without_a_delta_is_the_layer_with_a_zero_delta(lc):
    """`layer(x)` runs the single-input norm kernels; at this size every arm is bit-reproducible
    (all-ranks schedules), so the outputs must be the bits of `layer(x, zeros)`."""
    m, h, i = 256, 256, 512
    _, x, nw, wgu, wd = _layer_inputs(m, h, i, seed=21)
    zero = torch.zeros_like(x)
    for arm in (lc.layer.Rank7MlpLayer(m, nw, wgu, wd), lc.layer.DenseMlpLayer(m, nw, wgu, wd)):
        if isinstance(arm, lc.layer.Rank7MlpLayer):
            from lcgemm._native import SCHEDULE_ALL_RANKS

            arm.gate_plan.schedule = SCHEDULE_ALL_RANKS
            arm.down_plan.rank_split = False
        want = arm(x, zero).clone()
        d, hh = arm.chain(None, x)
        assert hh is x
        got = arm(x)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    lc.ops.check_status()


@pytest.mark.parametrize("dims", [(256, 256, 512), (512, 384, 1280), (130, 128, 256)])
def test_residual_folded_into_down(lc, dims):
    """The gate_up kernel fills the rank-split consumer's output with the residual stream instead
    of zeros (bit for bit, checked before `down` runs); `down` then reduce-adds onto it and the
    layer needs no add kernel.  Tolerances: against the unfused layer 6e-3 of the output (each of
    down's contributions is rounded at the magnitude of h, ~2^-9 each), against the fp32 reference
    the layer's usual 1.5e-2."""
    m, h, i = dims
    delta, x, nw, wgu, wd = _layer_inputs(m, h, i, seed=30)
    gate, down = lc.seams.build_chain((m, h, 2 * i), (m, i, h))
    assert down.rank_split and gate.preclear is down.c
    gate.init_from = x
    gate(x, None, nw, 1e-6, prepared_w=gate.prepare_weight(wgu))
    assert torch.equal(down.c.view(torch.int16), x.view(torch.int16))
    gate.init_from = None

    plain = lc.layer.Rank7MlpLayer(m, nw, wgu, wd)
    fused = lc.layer.Rank7MlpLayer(m, nw, wgu, wd, fuse_residual=True)
    assert fused.fuse_residual and not plain.fuse_residual
    for dl in (None, delta):
        want = plain(x, dl).clone()
        before = lc.ops.launch_count()
        got = fused(x, dl)
        mid = lc.ops.launch_count()
        plain(x, dl)
        assert mid - before == lc.ops.launch_count() - mid - 1          # one kernel less: no add
        hh = x.cpu() if dl is None else (x.cpu().float() + dl.cpu().float()).to(torch.bfloat16)
        ref, _ = O.mlp_reference(torch.zeros_like(hh) if dl is None else dl.cpu(), x.cpu(), nw.cpu(),
                                 wgu.cpu(), wd.cpu(), 1e-6)
        full = (hh.float() + ref.float()).to(torch.bfloat16)
        assert rel_fro(got, want) <= 6e-3
        assert rel_fro(got, full) <= 1.5e-2
        # on the branch alone the roundings at |h| show (the branch is ~2 % of h at this size, so one
        # rounding of the output is already ~10 % of it): a few such roundings instead of one
        on_branch = lambda o: rel_fro(o.cpu().float() - hh.float(), ref.float())
        assert on_branch(got) <= 3.0 * on_branch(want)
        assert fused.gate_plan.init_from is None


def test_residual_fold_refusals(lc, monkeypatch):
    from lcgemm.seams import down as down_mod

    m, h, i = 256, 256, 512
    _, x, nw, wgu, wd = _layer_inputs(m, h, i, seed=31)
    gate, down = lc.seams.build_chain((m, h, 2 * i), (m, i, h))
    bw = gate.prepare_weight(wgu)
    a = gate.a_planes(x, None, nw, 1e-6)
    with pytest.raises(ValueError):                  # wrong shape
        lc.ops.gate_up_chain(gate.scheme, gate.plane_scheme, a, bw, gate.c, gate.planes, preclear=down.c,
                             init_from=x[:128])
    with pytest.raises(ValueError):                  # nothing to write it to
        lc.ops.gate_up_chain(gate.scheme, gate.plane_scheme, a, bw, gate.c, gate.planes, init_from=x)
    with pytest.raises(Exception, match="overlaps"):  # the consumer output itself
        lc.ops.gate_up_chain(gate.scheme, gate.plane_scheme, a, bw, gate.c, gate.planes, preclear=down.c,
                             init_from=down.c)
    monkeypatch.setattr(down_mod, "HYBRID_SHAPES", {(m, i, h)})
    with pytest.raises(ValueError, match="rank-split"):
        lc.layer.Rank7MlpLayer(m, nw, wgu, wd, fuse_residual=True)


def test_plan_shape_errors(lc):
    gs, ds = lc.load(GATE), lc.load(DOWN)
    with pytest.raises(ValueError):
        lc.seams.GateUpPlan(gs, (255, 256, 512), plane_scheme=ds)
    with pytest.raises(ValueError):
        lc.seams.GateUpPlan(gs, (256, 256, 384), plane_scheme=ds)
    with pytest.raises(ValueError):
        lc.seams.DownPlan(ds, (256, 192, 256), producer=None)
