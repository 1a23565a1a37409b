"""The rank-7 GEMM that forms its A operands itself (``lcg_gemm_r7_fused``): no A planes in
global memory.  The operand tiles it builds in shared memory hold the same bf16 values as the
planes ``lcg_a_planes`` writes (a packed bf16 add of two bf16 values is the fp32 sum rounded
once), so with the deterministic all-ranks schedule the output must equal the plane path bit for
bit; the other schedules add into C in an order the hardware picks and are compared within the
stated tolerance, and every schedule is compared with the CPU oracle.
"""
import pytest
import torch

from gpu_util import rel_fro, seeded
from oracle import lc_oracle as O

pytestmark = pytest.mark.gpu
NAME = "2x2_locality_ordered"
TOL_R7_DENSE, TOL_R7_ORACLE, TOL_R7_ORACLE_SPLIT = 1.0e-2, 2.0e-3, 8.0e-3


@pytest.fixture(scope="module")
def lc():
    from lcgemm import _native, ops, planes, scheme

    return type("LC", (), dict(ops=ops, planes=planes, nat=_native, load=staticmethod(scheme.load)))


@pytest.fixture(autouse=True)
def _status_clean(lc):
    yield
    lc.ops.check_status()


# (M, N, K): one tile; several K blocks; odd M (block rows of 129 and 128 rows) and a ragged N;
# a tile row that overhangs its block row; many tiles; more tiles than CTA groups
SHAPES = [(256, 512, 128), (256, 512, 768), (257, 530, 384), (600, 1000, 512), (1024, 1536, 1024),
          (5120, 9000, 128)]


@pytest.mark.parametrize("group", [1, 2])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_equals_plane_path_bit_for_bit(lc, group, shape):
    m, n, k = shape
    sch = lc.load(NAME)
    a, w = seeded((m, k), 21), seeded((n, k), 22, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    assert lc.ops.fused_a_supported(sch, m, n, k)
    got = lc.ops.gemm_r7(a, bp, n, sch, schedule=0, cta_group=group, fused=True)
    want = lc.ops.gemm_r7(a, bp, n, sch, schedule=0, cta_group=group, fused=False)
    assert got.shape == (m, n)
    assert torch.equal(got, want)


@pytest.mark.parametrize("schedule", [0, 1, 2])
@pytest.mark.parametrize("shape", SHAPES)
def test_fused_against_oracle(lc, schedule, shape):
    m, n, k = shape
    sch, tb = lc.load(NAME), O.Tables(NAME)
    a, w = seeded((m, k), 23), seeded((n, k), 24, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    c = lc.ops.gemm_r7_fused(a, bp, n, sch, schedule=schedule)
    assert rel_fro(c, a.double().cpu() @ w.double().cpu().T) <= TOL_R7_DENSE
    model = O.scheme_matmul(a.cpu(), w.cpu(), tb, mode="kernel_split" if schedule == 1 else "kernel")
    assert rel_fro(c, model) <= (TOL_R7_ORACLE_SPLIT if schedule else TOL_R7_ORACLE)


def test_fused_reads_a_strided_activation_and_leaves_its_neighbours_alone(lc):
    sch = lc.load(NAME)
    m, n, k = 300, 520, 256
    big = seeded((m, 1024), 25)
    a = big[:, 256:256 + k]                                # row pitch 1024, offset 512 bytes
    w = seeded((n, k), 26, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    out = torch.zeros((m, 528), device="cuda", dtype=torch.bfloat16)
    got = lc.ops.gemm_r7_fused(a, bp, n, sch, out=out[:, :n], schedule=0)
    want = lc.ops.gemm_r7(a.contiguous(), bp, n, sch, schedule=0, fused=False)
    assert torch.equal(got, want)
    assert bool((out[:, n:] == 0).all())


def test_fused_refuses_what_it_cannot_form(lc):
    m, n, k = 256, 512, 256
    a, w = seeded((m, k), 27), seeded((n, k), 28, 0.02)
    cse = lc.load("2x2_postsum_cse")                      # rows with three and four terms
    assert not lc.ops.fused_a_supported(cse, m, n, k)
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_fused(a, lc.planes.prepare_b(w, cse), n, cse)
    sch = lc.load(NAME)
    a2, w2 = seeded((m, 192), 29), seeded((n, 192), 30, 0.02)   # K / 2 is not whole K blocks
    assert not lc.ops.fused_a_supported(sch, m, n, 192)
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_fused(a2, lc.planes.prepare_b(w2, sch), n, sch)
    # the dispatcher falls back to the plane path for both
    assert lc.ops.gemm_r7(a2, lc.planes.prepare_b(w2, sch), n, sch).shape == (m, n)


def test_fused_full_size_properties(lc):
    """The down-shaped bare GEMM at its benchmark size: agreement with the dense kernel, exact
    scaling by two, zero rows in / zero rows out, column checksum."""
    m, n, k = 4096, 5120, 17408
    sch = lc.load(NAME)
    a = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), device="cuda") * 0.02).to(torch.bfloat16)
    bp = lc.planes.prepare_b(w, sch)
    c = lc.ops.gemm_r7_fused(a, bp, n, sch, schedule=0).clone()
    d = lc.ops.gemm_dense(a, w)
    assert rel_fro(c[:, ::7], d[:, ::7]) <= TOL_R7_DENSE
    assert torch.equal(c, lc.ops.gemm_r7(a, bp, n, sch, schedule=0, fused=False))
    c2 = lc.ops.gemm_r7_fused((a.float() * 2).to(torch.bfloat16), bp, n, sch, schedule=0)
    assert torch.equal(c2.float(), c.float() * 2)
    az = a.clone()
    az[100:164] = 0
    az[m // 2 + 100:m // 2 + 164] = 0
    cz = lc.ops.gemm_r7_fused(az, bp, n, sch, schedule=2)
    assert bool((cz[100:164] == 0).all()) and bool((cz[m // 2 + 100:m // 2 + 164] == 0).all())
    ones = torch.ones(n, device="cuda")
    assert rel_fro(c.float() @ ones, a.float() @ (w.float().T @ ones)) < 2e-2


# ------------------------------------------------------------- product-ahead form
AHEAD_NAMES = ("2x2_locality_ordered", "2x2_locality_lead_single")


@pytest.mark.parametrize("name", AHEAD_NAMES)
@pytest.mark.parametrize("group", [1, 2])
@pytest.mark.parametrize("shape", SHAPES)
def test_ahead_equals_plane_path_bit_for_bit(lc, name, group, shape):
    """``lcg_gemm_r7_ahead``: the plane warps of all CTAs form each two-term A plane in a global
    scratch one product ahead of the MMAs.  Same values as ``lcg_a_planes`` writes, so the
    deterministic schedule must give the plane path's bits."""
    m, n, k = shape
    sch = lc.load(name)
    a, w = seeded((m, k), 31), seeded((n, k), 32, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    need = lc.ops.ahead_scratch_bytes(sch, m, k)
    assert need == 256 + 5 * ((m + 1) // 2) * (k // 2) * 2
    scratch = torch.full((need,), 0xA5, dtype=torch.uint8, device="cuda")      # stale contents
    got = lc.ops.gemm_r7_ahead(a, bp, n, sch, scratch=scratch, schedule=0, cta_group=group)
    want = lc.ops.gemm_r7(a, bp, n, sch, schedule=0, cta_group=group, fused=False)
    assert torch.equal(got, want)
    again = lc.ops.gemm_r7_ahead(a, bp, n, sch, scratch=scratch, schedule=0, cta_group=group)
    assert torch.equal(again, want)                       # counters are cleared by every call


@pytest.mark.parametrize("name", AHEAD_NAMES)
@pytest.mark.parametrize("schedule", [0, 1, 2])
@pytest.mark.parametrize("shape", SHAPES)
def test_ahead_against_oracle(lc, name, schedule, shape):
    m, n, k = shape
    sch, tb = lc.load(name), O.Tables(name)
    a, w = seeded((m, k), 33), seeded((n, k), 34, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    c = lc.ops.gemm_r7_ahead(a, bp, n, sch, schedule=schedule)
    assert rel_fro(c, a.double().cpu() @ w.double().cpu().T) <= TOL_R7_DENSE
    model = O.scheme_matmul(a.cpu(), w.cpu(), tb, mode="kernel_split" if schedule == 1 else "kernel")
    assert rel_fro(c, model) <= (TOL_R7_ORACLE_SPLIT if schedule else TOL_R7_ORACLE)


def test_ahead_refuses_small_scratch_and_other_schemes(lc):
    m, n, k = 256, 512, 256
    sch = lc.load(NAME)
    a, w = seeded((m, k), 35), seeded((n, k), 36, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_ahead(a, bp, n, sch, scratch=torch.empty(1024, dtype=torch.uint8, device="cuda"))
    cse = lc.load("2x2_postsum_cse")
    assert lc.ops.ahead_scratch_bytes(cse, m, k) == -1
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_ahead(a, lc.planes.prepare_b(w, cse), n, cse)


def test_ahead_full_size_properties(lc):
    m, n, k = 4096, 5120, 17408
    sch = lc.load("2x2_locality_lead_single")
    a = torch.randn((m, k), device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), device="cuda") * 0.02).to(torch.bfloat16)
    bp = lc.planes.prepare_b(w, sch)
    scratch = torch.empty(lc.ops.ahead_scratch_bytes(sch, m, k), dtype=torch.uint8, device="cuda")
    c = lc.ops.gemm_r7_ahead(a, bp, n, sch, scratch=scratch, schedule=0).clone()
    assert torch.equal(c, lc.ops.gemm_r7(a, bp, n, sch, schedule=0, fused=False))
    d = lc.ops.gemm_dense(a, w)
    assert rel_fro(c[:, ::7], d[:, ::7]) <= TOL_R7_DENSE
    c2 = lc.ops.gemm_r7_ahead((a.float() * 2).to(torch.bfloat16), bp, n, sch, scratch=scratch, schedule=0)
    assert torch.equal(c2.float(), c.float() * 2)
    ch = lc.ops.gemm_r7_ahead(a, bp, n, sch, scratch=scratch, schedule=2)
    assert rel_fro(ch, c) < 4e-3
    ones = torch.ones(n, device="cuda")
    assert rel_fro(c.float() @ ones, a.float() @ (w.float().T @ ones)) < 2e-2
