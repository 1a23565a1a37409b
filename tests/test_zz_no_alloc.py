"""The allocation-free rank-7 GEMM entry point, through the C ABI.

Some callers of this library cannot allocate device memory: a server that has given all
free memory to its own pool, or a serving thread that may not call cudaMalloc because it
synchronises the device.  ``lcg_gemm_r7_static`` keeps the A-plane scratch in a fixed
device array inside the library instead of a caller-owned buffer.  This test calls it
twice in a row (different shapes, so the second call runs over the first one's leftovers)
and requires the same bits as the existing path ``lcg_a_planes`` + ``lcg_gemm_r7`` with a
torch-allocated workspace.  It is collected last so that a run that stops at the first
failure has already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_pair(lib, nat, scheme, m, n, k, seed, schedule):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn((m, k), generator=g).to(torch.bfloat16).cuda()
    w = (torch.randn((n, k), generator=g) * 0.02).to(torch.bfloat16).cuda()
    handle = nat.NativeScheme.of(scheme).handle
    stream = torch.cuda.current_stream().cuda_stream
    n2, _, k2p = nat.plane_geometry(n, k, 8)
    m2, _, _ = nat.plane_geometry(m, k, 1)
    bp = torch.empty((scheme.rank * n2, k2p), dtype=torch.bfloat16, device="cuda")
    nat.check(lib.lcg_prepare_b(handle, w.data_ptr(), n, k, w.stride(0), bp.data_ptr(), k2p, stream))
    status = torch.zeros(4, dtype=torch.int32, device="cuda")
    ld = (n + 7) // 8 * 8

    # existing path: caller-owned scratch
    ws = torch.empty((scheme.rank * m2, k2p), dtype=torch.bfloat16, device="cuda")
    want = torch.zeros((m, ld), dtype=torch.bfloat16, device="cuda")
    nat.check(lib.lcg_a_planes(handle, a.data_ptr(), m, k, a.stride(0), ws.data_ptr(), k2p, stream))
    nat.check(lib.lcg_gemm_r7(handle, ws.data_ptr(), k2p, bp.data_ptr(), k2p, want.data_ptr(), ld,
                              m, n, k, schedule, 0, status.data_ptr(), stream))
    # new path: scratch inside the library
    got = torch.zeros((m, ld), dtype=torch.bfloat16, device="cuda")
    nat.check(lib.lcg_static_reserve())           # the array takes its memory here, once per device
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()    # the driver's figure: sees any cudaMalloc, not only torch's
    nat.check(lib.lcg_gemm_r7_static(handle, a.data_ptr(), a.stride(0), bp.data_ptr(), k2p,
                                     got.data_ptr(), ld, m, n, k, schedule, 0, status.data_ptr(),
                                     stream))
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] >= free_before
    assert status.tolist() == [0, 0, 0, 0]
    return got[:, :n], want[:, :n], a, w


def test_static_scratch_matches_caller_owned_scratch_twice():
    from lcgemm import _native as nat
    from lcgemm import scheme as S

    lib = nat.lib()
    assert lib.lcg_static_scratch_bytes() == 32 << 20
    sch = S.load("2x2_locality_ordered")
    # two calls in a row; the second is smaller and odd-shaped, so it runs over stale planes
    for (m, n, k, seed) in ((1024, 1536, 2048, 1), (258, 530, 144, 2)):
        got, want, a, w = _run_pair(lib, nat, sch, m, n, k, seed, nat.SCHEDULE_ALL_RANKS)
        assert torch.equal(got, want)                      # all-ranks schedule is deterministic
        exact = a.double().cpu() @ w.double().cpu().T
        rel = ((got.double().cpu() - exact).norm() / exact.norm()).item()
        assert rel <= 1.0e-2
    # rank split and hybrid: the bf16 adds land in hardware order, so compare within the suite's tolerance
    for schedule, shape in ((nat.SCHEDULE_RANK_SPLIT, (512, 1024, 256)), (nat.SCHEDULE_HYBRID, (1280, 9000, 128))):
        got, want, _, _ = _run_pair(lib, nat, sch, *shape, 3, schedule)
        rel = ((got.float() - want.float()).norm() / want.float().norm()).item()
        assert rel <= 8.0e-3


def test_static_scratch_boundary():
    """The largest shape whose planes fit the 32 MiB passes the size check, one more row pair
    does not.  Both calls name a leading dimension below K, which the host refuses before it
    launches anything, so the first call gets past the size check and stops there."""
    from lcgemm import _native as nat
    from lcgemm import scheme as S

    lib = nat.lib()
    handle = nat.NativeScheme.of(S.load("2x2_locality_ordered")).handle
    x = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    limit = lib.lcg_static_scratch_bytes()
    k = 4096
    m = 2 * (limit // (7 * (k // 2) * 2))    # 7 * (m / 2) * (k / 2) * 2 bytes is the most that fits
    assert 7 * (m // 2) * (k // 2) * 2 <= limit < 7 * (m // 2 + 1) * (k // 2) * 2
    bad_lda = 8
    code = lib.lcg_gemm_r7_static(handle, x.data_ptr(), bad_lda, x.data_ptr(), k // 2, x.data_ptr(), 8,
                                  m, 16, k, 0, 0, None, None)
    assert code == nat.ERR_BAD_ARG and b"scratch" not in lib.lcg_last_error()
    code = lib.lcg_gemm_r7_static(handle, x.data_ptr(), bad_lda, x.data_ptr(), k // 2, x.data_ptr(), 8,
                                  m + 2, 16, k, 0, 0, None, None)
    assert code == nat.ERR_UNSUPPORTED_SHAPE and b"scratch" in lib.lcg_last_error()


def test_static_scratch_rejects_oversized_shapes():
    from lcgemm import _native as nat
    from lcgemm import scheme as S

    lib = nat.lib()
    handle = nat.NativeScheme.of(S.load("2x2_locality_ordered")).handle
    x = torch.zeros(8, dtype=torch.bfloat16, device="cuda")
    code = lib.lcg_gemm_r7_static(handle, x.data_ptr(), 17408, x.data_ptr(), 8704, x.data_ptr(), 5120,
                                  4096, 5120, 17408, 0, 0, None, None)
    assert code == nat.ERR_UNSUPPORTED_SHAPE
    assert b"static" in lib.lcg_last_error() and b"scratch" in lib.lcg_last_error()
    with pytest.raises(ValueError):
        nat.check(code)
