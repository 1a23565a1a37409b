"""The tensor-parallel exchange kernels on ONE GPU: the ranks of a group are emulated one after
the other with every "peer" buffer in local memory, which exercises the push from the GEMM
kernel, the tail push, the owner arithmetic and the reduce + gather kernel bit for bit.  (The
barrier between ranks is only called where nothing has to answer: a group of one, and a group
whose second member never arrives, where the bounded wait must run out and report.)"""
import pytest
import torch

from gpu_util import seeded

pytestmark = pytest.mark.gpu
DOWN = "2x2_locality_ordered"


@pytest.fixture(scope="module")
def lc():
    from lcgemm import ops, planes, scheme, tp

    return type("LC", (), dict(ops=ops, planes=planes, tp=tp, load=staticmethod(scheme.load)))


@pytest.fixture(autouse=True)
def _status_clean(lc):
    yield
    lc.ops.check_status()


# (M, N, K per rank, world): all-tail (few tiles), main + tail tiles, and rows that do not divide
@pytest.mark.parametrize("dims", [(512, 512, 256, 2), (4096, 5120, 256, 4), (4096, 5120, 128, 3),
                                  (1030, 264, 128, 8)])
def test_push_and_reduce_gather_emulated_ranks(lc, dims):
    m, n, k, world = dims
    sch = lc.load(DOWN)
    rows = lc.tp.rows_per_owner(m, world)
    h = seeded((m, n), 100)
    slots = [torch.full((world, rows, n), 7.0, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    outs = [torch.full((m, n), 9.0, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    partials = []
    for r in range(world):
        a, w = seeded((m, k), 10 + r), seeded((n, k), 20 + r, 0.05)
        c = torch.full((m, n), 5.0, device="cuda", dtype=torch.bfloat16)
        slot_ptrs = [slots[o][r].data_ptr() for o in range(world)]
        lc.ops.gemm_r7_push(sch, lc.planes.a_planes(a, sch), lc.planes.prepare_b(w, sch), m, n, k, c,
                            slot_ptrs, r, rows)
        # the partial itself is the hybrid-schedule product
        want = a.double() @ w.double().T
        assert ((c.double() - want).norm() / want.norm()).item() <= 1.5e-2
        partials.append(c)
    torch.cuda.synchronize()
    # every owner holds exactly the rows it owns of every rank's partial
    for o in range(world):
        lo, hi = o * rows, min((o + 1) * rows, m)
        for r in range(world):
            assert torch.equal(slots[o][r, :max(hi - lo, 0)], partials[r][lo:hi]), (o, r)
    for o in range(world):
        lc.ops.reduce_gather(slots[o], h, [t.data_ptr() for t in outs], rows, o)
    acc = h.float()
    for r in range(world):
        acc = acc + partials[r].float()
    want = acc.to(torch.bfloat16)
    for t in outs:
        assert torch.equal(t, want)


def test_push_rejects_bad_arguments(lc):
    sch = lc.load(DOWN)
    a, w = seeded((256, 128), 1), seeded((264, 128), 2)
    ap, bp = lc.planes.a_planes(a, sch), lc.planes.prepare_b(w, sch)
    c = torch.empty((256, 264), device="cuda", dtype=torch.bfloat16)
    slot = torch.empty((2, 128, 264), device="cuda", dtype=torch.bfloat16)
    ptrs = [slot[0].data_ptr(), slot[1].data_ptr()]
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_push(sch, ap, bp, 256, 264, 128, c, ptrs, 2, 128)        # rank outside the group
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_push(sch, ap, bp, 256, 264, 128, c, ptrs, 0, 100)        # owners do not cover M
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_push(sch, ap, bp, 256, 264, 128, c, [ptrs[0], 0], 0, 128)  # NULL slot
    with pytest.raises(ValueError):
        lc.ops.gemm_r7_push(sch, ap, bp, 256, 264, 128, c, ptrs * 5, 0, 128)    # more than 8 ranks


def test_barrier_alone_and_bounded(lc):
    flags = torch.zeros(16, dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):                      # a group of one passes at once
        lc.ops.peer_barrier([flags.data_ptr()], 0, epoch)
    torch.cuda.synchronize()
    assert int(flags[0]) == 3
    for _ in range(2):                           # epoch 0: the kernel counts its own calls
        lc.ops.peer_barrier([flags.data_ptr()], 0, 0)
    torch.cuda.synchronize()
    assert int(flags[8]) == 2 and int(flags[0]) == 2
    flags.zero_()
    for epoch in (1, 2, 3):
        lc.ops.peer_barrier([flags.data_ptr()], 0, epoch)
    lc.ops.check_status()
    # a group of two whose other member never arrives: the wait runs out after 20 ms, the
    # kernel returns, the status word says which wait it was, and the context stays usable
    other = torch.zeros(16, dtype=torch.int32, device="cuda")
    lc.ops.peer_barrier([flags.data_ptr(), other.data_ptr()], 0, 4, limit_us=20_000)
    torch.cuda.synchronize()
    assert int(other[0]) == 4                    # the arrival was announced
    with pytest.raises(RuntimeError, match="106"):
        lc.ops.check_status()
    lc.ops.check_status()                        # cleared
    assert float(torch.ones(4, device="cuda").sum()) == 4.0
