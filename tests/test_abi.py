"""The C ABI surface, without a GPU: the library loads, exports every symbol the header
declares, and its host-side entry points (scheme handle, geometry, describe, argument
checks) behave.  No kernel is launched here."""
import ctypes
import re

import pytest

from conftest import REPO
from lcgemm import _native as nat
from lcgemm import scheme as S

HEADER = (REPO / "include" / "lcgemm_b200.h").read_text()
DECLARED = sorted(set(re.findall(r"\b(lcg_[a-z0-9_]+)\s*\(", HEADER)))


def test_header_declares_what_the_loader_binds():
    assert set(DECLARED) == set(nat.SIGNATURES), set(DECLARED) ^ set(nat.SIGNATURES)


@pytest.mark.parametrize("symbol", DECLARED)
def test_symbol_is_exported(native_lib, symbol):
    assert getattr(native_lib, symbol) is not None


def test_version_and_error_text(native_lib):
    assert native_lib.lcg_version() >= 100
    assert isinstance(native_lib.lcg_last_error(), bytes)


@pytest.mark.parametrize("name", ["2x2_postsum_cse", "2x2_locality_ordered", "2x2_locality_lead_single"])
def test_native_plan_equals_host_plan(native_lib, name):
    s = S.load(name)
    native = nat.NativeScheme(s).plan()
    host = [[(d.row, d.col, g.coeff, bool(d.is_first)) for g in step for d in g.dests]
            for step in s.epi_groups]
    assert native == host


def test_native_scheme_validation(native_lib):
    s = S.load("2x2_postsum_cse")
    flat = lambda rows: (ctypes.c_int8 * 28)(*[v for r in rows for v in r])
    a, b, c = flat(s.a), flat(s.b), flat(s.c)
    out = ctypes.c_void_p()
    bad_c = [list(r) for r in s.c]
    bad_c[2][0] = 1
    assert native_lib.lcg_scheme_create(a, b, flat(bad_c), 7, None, ctypes.byref(out)) == nat.ERR_SCHEME
    assert b"not a decomposition" in native_lib.lcg_last_error()
    clear = (ctypes.c_int8 * 7)(1, 0, 0, 1, 0, 0, 0)
    assert native_lib.lcg_scheme_create(a, b, c, 7, clear, ctypes.byref(out)) == nat.ERR_SCHEME
    assert native_lib.lcg_scheme_create(a, b, c, 9, None, ctypes.byref(out)) == nat.ERR_SCHEME
    assert native_lib.lcg_scheme_create(None, b, c, 7, None, ctypes.byref(out)) == nat.ERR_BAD_ARG
    assert native_lib.lcg_scheme_create(a, b, c, 7, None, ctypes.byref(out)) == nat.OK
    native_lib.lcg_scheme_destroy(out)
    with pytest.raises(ValueError):
        nat.check(nat.ERR_SCHEME)


def test_plane_geometry(native_lib):
    assert nat.plane_geometry(4096, 5120, 1) == (2048, 2560, 2560)
    assert nat.plane_geometry(34816, 5120, 8) == (17408, 2560, 2560)
    assert nat.plane_geometry(13999, 5000, 8) == (7000, 2500, 2560)
    assert nat.plane_geometry(4095, 5000, 1) == (2048, 2500, 2560)
    with pytest.raises(ValueError):
        nat.plane_geometry(0, 5, 1)


def test_describe_and_argument_checks_do_not_need_a_gpu(native_lib):
    from lcgemm import ops

    text = ops.describe_gemm(4096, 34816, 5120, True, nat.SCHEDULE_ALL_RANKS, 2)
    assert "8x68 tiles" in text and "544 units" in text and "40 k-blocks" in text
    text = ops.describe_gemm(4096, 5120, 17408, True, nat.SCHEDULE_RANK_SPLIT, 2)
    assert "644 units" in text and "136 k-blocks" in text      # 518 whole-K units + 42 cut in 3
    # NULL operands and bad shapes are rejected before anything touches the device.
    assert native_lib.lcg_gemm_dense(None, 8, None, 8, None, 8, 8, 8, 8, 0, None, None) == nat.ERR_BAD_ARG
    sch = nat.NativeScheme.of(S.load("2x2_postsum_cse")).handle
    fake = ctypes.c_void_p(4096)
    assert native_lib.lcg_gate_up_chain(sch, sch, fake, 64, fake, 64, fake, 300, 64, 300, 128, fake,
                                        80, None, 0, 0, 0, None, None) == nat.ERR_UNSUPPORTED_SHAPE
    assert native_lib.lcg_norm_planes(sch, fake, fake, fake, 7, 64, 1e-6, fake, fake, 64,
                                      None) == nat.ERR_UNSUPPORTED_SHAPE
    # the chain with an initial content for the consumer output: it must exist, have somewhere to
    # go and not be that output
    other = ctypes.c_void_p(4096 + 160)
    far = ctypes.c_void_p(1 << 20)
    for consumer, nbytes, init in ((fake, 1600, None), (None, 0, far), (fake, 1600, other),
                                   (fake, 1600, ctypes.c_void_p((1 << 20) + 8))):
        assert native_lib.lcg_gate_up_chain_init(sch, sch, fake, 64, fake, 64, fake, 512, 64, 512, 128, fake,
                                                 128, consumer, nbytes, init, 0, 0, None, None) in (
            nat.ERR_BAD_ARG, nat.ERR_MISALIGNED)
    # a delta needs somewhere to store the sum; without a delta neither is needed (the shape check
    # comes next, so a missing delta is past the NULL check)
    assert native_lib.lcg_norm_planes(sch, fake, fake, fake, 8, 64, 1e-6, None, fake, 64,
                                      None) == nat.ERR_BAD_ARG
    assert native_lib.lcg_norm_planes(sch, None, fake, fake, 7, 64, 1e-6, None, fake, 64,
                                      None) == nat.ERR_UNSUPPORTED_SHAPE
    assert native_lib.lcg_add_rmsnorm(fake, fake, fake, 8, 64, 1e-6, None, fake, None) == nat.ERR_BAD_ARG
    assert native_lib.lcg_add_rmsnorm(None, fake, fake, 8, 60, 1e-6, None, fake,
                                      None) == nat.ERR_UNSUPPORTED_SHAPE
    assert native_lib.lcg_gemm_r7(sch, fake, 64, fake, 64, fake, 64, 64, 64, 128, 5, 0, None,
                                  None) == nat.ERR_BAD_ARG
    assert native_lib.lcg_launch_count() == 0


def test_in_kernel_plane_forms_say_what_they_take(native_lib):
    """Host-side answers of the two entry points that form A operands inside the GEMM kernel
    (no launch): which schemes and shapes they take, how much scratch the product-ahead form
    needs, and that bad arguments are refused before anything is launched."""
    loc, lead, cse = (nat.NativeScheme.of(S.load(n)).handle
                      for n in ("2x2_locality_ordered", "2x2_locality_lead_single", "2x2_postsum_cse"))
    m, k = 4096, 17408
    assert native_lib.lcg_gemm_r7_fused_supported(loc, m, 5120, k) == 1
    assert native_lib.lcg_gemm_r7_fused_supported(lead, m, 5120, k) == 1
    assert native_lib.lcg_gemm_r7_fused_supported(cse, m, 5120, k) == 0       # rows of three and four terms
    assert native_lib.lcg_gemm_r7_fused_supported(loc, m, 5120, 5000) == 0    # K / 2 is not whole K blocks
    # five two-term planes of (M / 2, K / 2) bf16 behind a 256-byte header
    assert native_lib.lcg_gemm_r7_ahead_scratch_bytes(loc, m, k) == 256 + 5 * (m // 2) * (k // 2) * 2
    assert native_lib.lcg_gemm_r7_ahead_scratch_bytes(lead, 257, 256) == 256 + 5 * 129 * 128 * 2
    assert native_lib.lcg_gemm_r7_ahead_scratch_bytes(cse, m, k) == -1
    assert native_lib.lcg_gemm_r7_ahead_scratch_bytes(loc, m, 5000) == -1
    fake = 4096                                   # a non-null, 256-byte aligned address; never dereferenced
    assert native_lib.lcg_gemm_r7_ahead(loc, fake, k, fake, k // 2, fake, 5120, m, 5120, k, fake, 1024,
                                        2, 0, None, None) == nat.ERR_BAD_ARG          # scratch too small
    assert b"scratch" in native_lib.lcg_last_error()
    assert native_lib.lcg_gemm_r7_ahead(loc, fake, k, fake, k // 2, fake, 5120, m, 5120, k, fake + 8, 1 << 40,
                                        2, 0, None, None) == nat.ERR_MISALIGNED       # scratch alignment
    assert native_lib.lcg_gemm_r7_ahead(cse, fake, k, fake, k // 2, fake, 5120, m, 5120, k, fake, 1 << 40,
                                        2, 0, None, None) == nat.ERR_SCHEME
    assert native_lib.lcg_gemm_r7_fused(loc, fake, 5000, fake, 2560, fake, 5120, m, 5120, 5000,
                                        2, 0, None, None) == nat.ERR_UNSUPPORTED_SHAPE
