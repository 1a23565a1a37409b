"""Parity of the tcgen05 GEMMs (dense and rank-7, every schedule and CTA grouping) with the
CPU oracle at small sizes, and size-independent properties at the full benchmark shapes.

Stated tolerances (bf16 in, fp32 accumulate, bf16 out):
  * dense vs an fp64 product of the same bf16 inputs: relative Frobenius error <= 2.5e-3
    (the output rounding alone is ~1.7e-3);
  * rank-7 vs the same fp64 product: <= 1.0e-2 (measured 6.3e-3 .. 8.5e-3);
  * rank-7 vs the oracle evaluated with the kernel's own rounding points: <= 2.0e-3 for the
    all-ranks schedule; <= 8.0e-3 for the rank-split schedule and for the split tail of the
    hybrid schedule, whose bf16 adds into C land in an order the hardware picks (the oracle
    adds in ascending product order, and models the hybrid schedule as all-ranks).
"""
import pytest
import torch

from gpu_util import rel_fro, seeded
from oracle import lc_oracle as O

pytestmark = pytest.mark.gpu
NAMES = ("2x2_postsum_cse", "2x2_locality_ordered")
TOL_DENSE, TOL_R7_DENSE, TOL_R7_ORACLE, TOL_R7_ORACLE_SPLIT = 2.5e-3, 1.0e-2, 2.0e-3, 8.0e-3


@pytest.fixture(scope="module")
def lc():
    from lcgemm import _native, ops, planes, scheme

    return type("LC", (), dict(ops=ops, planes=planes, nat=_native, load=staticmethod(scheme.load)))


@pytest.fixture(autouse=True)
def _status_clean(lc):
    yield
    lc.ops.check_status()          # synchronises; fails the test if a device-side wait ran out


@pytest.mark.parametrize("group", [1, 2])
@pytest.mark.parametrize("shape", [(128, 256, 64), (256, 512, 256), (1, 8, 8), (100, 24, 72), (384, 768, 320),
                                   (1000, 1003, 520), (2048, 2560, 1024)])
def test_dense_gemm(lc, group, shape):
    m, n, k = shape
    a, b = seeded((m, k), 1), seeded((n, k), 2, 0.02)
    c = lc.ops.gemm_dense(a, b, cta_group=group)
    assert c.shape == (m, n)
    want = a.double().cpu() @ b.double().cpu().T
    assert rel_fro(c, want) <= TOL_DENSE


def test_dense_gemm_strided_operands(lc):
    a_big, b_big = seeded((300, 1024), 3), seeded((520, 1024), 4, 0.02)
    a, b = a_big[:, 128:640], b_big[:, 128:640]
    out = torch.zeros((300, 528), device="cuda", dtype=torch.bfloat16)
    c = lc.ops.gemm_dense(a, b, out=out[:, :520])
    assert rel_fro(c, a.double().cpu() @ b.double().cpu().T) <= TOL_DENSE
    assert bool((out[:, 520:] == 0).all())                 # nothing written past N


@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("group", [1, 2])
@pytest.mark.parametrize("schedule", [0, 1, 2])
@pytest.mark.parametrize("shape", [(256, 512, 128), (512, 1024, 256), (258, 530, 144), (600, 1000, 520),
                                   (1024, 1536, 1024), (5120, 9000, 128)])
def test_rank7_gemm_against_oracle(lc, name, group, schedule, shape):
    m, n, k = shape
    sch, tb = lc.load(name), O.Tables(name)
    a, w = seeded((m, k), 5), seeded((n, k), 6, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    c = lc.ops.gemm_r7(a, bp, n, sch, schedule=schedule, cta_group=group, fused=False)
    assert c.shape == (m, n)
    dense = a.double().cpu() @ w.double().cpu().T
    assert rel_fro(c, dense) <= TOL_R7_DENSE
    model = O.scheme_matmul(a.cpu(), w.cpu(), tb, mode="kernel_split" if schedule == 1 else "kernel")
    assert rel_fro(c, model) <= (TOL_R7_ORACLE_SPLIT if schedule else TOL_R7_ORACLE)


@pytest.mark.parametrize("shape", [(2, 16, 2), (3, 17, 5), (7, 9, 130), (129, 257, 66)])
def test_rank7_tiny_and_ragged_shapes(lc, shape):
    m, n, k = shape
    sch = lc.load("2x2_locality_ordered")
    a, w = seeded((m, k), 11), seeded((n, k), 12, 0.5)
    for schedule in (0, 1, 2):
        c = lc.ops.gemm_r7(a, lc.planes.prepare_b(w, sch), n, sch, schedule=schedule, fused=False)
        assert c.shape == (m, n)
        want = a.double().cpu() @ w.double().cpu().T
        assert rel_fro(c, want) <= 1.5e-2


def test_rank7_rejects_degenerate_shapes(lc):
    sch = lc.load("2x2_locality_ordered")
    a, w = seeded((4, 16), 1), seeded((8, 16), 2)
    with pytest.raises(ValueError):                        # N = 8 leaves the second column block empty
        lc.ops.gemm_r7(a, lc.planes.prepare_b(w, sch), 8, sch)
    with pytest.raises(ValueError):
        lc.ops.gemm_dense(a, seeded((8, 24), 3))           # inner dimensions differ


def test_rank7_odd_shape_pad_path(lc):
    """K=5000, N=13999 (scaled down in M): planes are zero-padded, C blocks are clipped."""
    m, n, k = 257, 13999, 5000
    sch = lc.load("2x2_locality_ordered")
    a, w = seeded((m, k), 7), seeded((n, k), 8, 0.02)
    bp = lc.planes.prepare_b(w, sch)
    assert bp.shape == (7 * 7000, 2560)
    c = lc.ops.gemm_r7(a, bp, n, sch)
    assert c.shape == (m, n) and c.stride(0) == 14000
    assert rel_fro(c, a.double().cpu() @ w.double().cpu().T) <= TOL_R7_DENSE
    with pytest.raises(ValueError):                        # a row pitch TMA cannot store to
        lc.ops.gemm_r7(a, bp, n, sch, out=torch.empty((m, n), device="cuda", dtype=torch.bfloat16))


def test_rank7_rank_split_needs_a_zeroed_output(lc):
    sch = lc.load("2x2_locality_ordered")
    m, n, k = 256, 512, 256
    a, w = seeded((m, k), 9), seeded((n, k), 10, 0.02)
    ap, bp = lc.planes.a_planes(a, sch), lc.planes.prepare_b(w, sch)
    out = torch.ones((m, n), device="cuda", dtype=torch.bfloat16)
    lc.ops.gemm_r7_planes(sch, ap, bp, m, n, k, out=out, schedule=1, zero_out=False)
    clean = lc.ops.gemm_r7_planes(sch, ap, bp, m, n, k, schedule=0)
    assert rel_fro(out.float() - 1.0, clean) < 6e-2          # contributions were added on top of the ones


# ---------------------------------------------------------------- full-size properties
FULL = [("2x2_postsum_cse", 0, (4096, 34816, 5120)), ("2x2_postsum_cse", 2, (4096, 34816, 5120)), ("2x2_locality_ordered", 1, (4096, 5120, 17408)),
        ("2x2_locality_ordered", 0, (2048, 5120, 17408)), ("2x2_postsum_cse", 0, (8192, 32768, 6144))]


@pytest.mark.parametrize("name,schedule,shape", FULL)
def test_full_size_properties(lc, name, schedule, shape):
    m, n, k = shape
    sch = lc.load(name)
    a = (torch.randn((m, k), device="cuda")).to(torch.bfloat16)
    w = (torch.randn((n, k), device="cuda") * 0.02).to(torch.bfloat16)
    bp = lc.planes.prepare_b(w, sch)
    c = lc.ops.gemm_r7(a, bp, n, sch, schedule=schedule, fused=False).clone()
    # (1) agrees with the dense tcgen05 kernel, which agrees with an fp32 product
    d = lc.ops.gemm_dense(a, w)
    assert rel_fro(c[:, ::7], d[:, ::7]) <= TOL_R7_DENSE
    exact = a[::5].float() @ w[::7].float().T                 # fp32 product of the same bf16 inputs
    assert rel_fro(d[::5, ::7], exact) <= TOL_DENSE
    # (2) scaling A by 2 scales C by 2 exactly (powers of two commute with every rounding)
    c2 = lc.ops.gemm_r7((a.float() * 2).to(torch.bfloat16), bp, n, sch, schedule=schedule, fused=False)
    if schedule == 0:
        assert torch.equal(c2.float(), c.float() * 2)
    else:                          # rank split: the order of the bf16 adds is not fixed
        assert rel_fro(c2.float(), c.float() * 2) < 4e-3
    # (3) permuting the rows of both block rows alike permutes C's rows
    m2 = m // 2
    perm = torch.randperm(m2, device="cuda")
    full = torch.cat([perm, perm + m2])
    cp = lc.ops.gemm_r7(a[full].contiguous(), bp, n, sch, schedule=schedule, fused=False)
    if schedule == 0:
        assert torch.equal(cp, c[full])
    else:
        assert rel_fro(cp, c[full]) < 4e-3
    # (4) zero rows in, zero rows out
    az = a.clone()
    az[100:164] = 0
    az[m2 + 100:m2 + 164] = 0
    cz = lc.ops.gemm_r7(az, bp, n, sch, schedule=schedule, fused=False)
    assert bool((cz[100:164] == 0).all()) and bool((cz[m2 + 100:m2 + 164] == 0).all())
    # (5) column checksum: C @ 1 against A @ (W^T 1) in fp32
    ones = torch.ones(n, device="cuda")
    lhs = c.float() @ ones
    rhs = a.float() @ (w.float().T @ ones)
    assert rel_fro(lhs, rhs) < 2e-2


def test_bounded_wait_reports_instead_of_hanging(lc):
    """A wait nothing satisfies runs out after its limit, leaves its code in the status word
    and the kernel returns; the context keeps working and check_status raises."""
    word = lc.ops.status_word()
    word.zero_()
    finished = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    lc.nat.check(lc.nat.lib().lcg_selftest_wait_timeout(word.data_ptr(), 2000, finished.data_ptr(), stream))
    torch.cuda.synchronize()
    assert finished.item() == 1 and word[0].item() == 199
    with pytest.raises(RuntimeError, match="wait ran out"):
        lc.ops.check_status()
    assert word[0].item() == 0                              # cleared for the next launch
    a, b = seeded((128, 64), 1), seeded((256, 64), 2, 0.02)
    assert rel_fro(lc.ops.gemm_dense(a, b), a.double().cpu() @ b.double().cpu().T) <= TOL_DENSE
