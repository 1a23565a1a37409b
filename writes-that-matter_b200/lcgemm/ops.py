"""Torch-tensor front end of the C ABI: argument checks, output allocation, status word.

Every function here launches CUDA work on the current torch stream through
``include/lcgemm_b200.h`` and never synchronises.  Tensors must be bf16 CUDA
tensors; there is no CPU implementation behind these calls.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native as nat
from ._native import NativeScheme, check, lib, ptr, stream_ptr

BF16 = torch.bfloat16

_STATUS: dict = {}


def _need(t: torch.Tensor, what: str, rows_contig: bool = True) -> None:
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(
            f"{what} must be a CUDA tensor: lcgemm_b200 has no CPU implementation of this path")
    if t.dtype != BF16:
        raise ValueError(f"{what} must be bfloat16, got {t.dtype}")
    if rows_contig and t.dim() == 2 and t.stride(1) != 1:
        raise ValueError(f"{what} must be row-major (unit stride along its last dimension)")


def status_word(device=None) -> torch.Tensor:
    """The per-device int32 word the tcgen05 kernels flag a run-out wait in."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    word = _STATUS.get(dev)
    if word is None:
        word = _STATUS[dev] = torch.zeros(4, dtype=torch.int32, device=dev)
    return word


def check_status(device=None) -> None:
    """Synchronise and raise if any kernel since the last check gave up a wait."""
    word = status_word(device)
    code = int(word[0].item())
    if code != 0:
        word.zero_()
        raise RuntimeError(
            f"lcgemm_b200: a device-side wait ran out (code {code}: 101 producer, 102/103 MMA "
            f"issuer, 104 epilogue, 105 plane warps, 106 barrier between ranks); results of that "
            f"launch are invalid")


def launch_count() -> int:
    return int(lib().lcg_launch_count())


def describe_gemm(m: int, n: int, k: int, rank7: bool = True, schedule: int = 0,
                  cta_group: int = 0) -> str:
    buf = ctypes.create_string_buffer(512)
    got = lib().lcg_describe_gemm(m, n, k, int(rank7), schedule, cta_group, buf, 512)
    if got < 0:
        check(got)
    return buf.value.decode()


# ------------------------------------------------------------------ geometry
def a_plane_shape(scheme, m: int, k: int):
    m2, _, k2p = nat.plane_geometry(m, k, 1)
    return scheme.rank * m2, k2p


def b_plane_shape(scheme, n: int, k: int):
    n2, _, k2p = nat.plane_geometry(n, k, 8)
    return scheme.rank * n2, k2p


# -------------------------------------------------------------------- planes
def prepare_b(w: torch.Tensor, scheme) -> torch.Tensor:
    """B planes ``(rank * N2, K2p)`` of a weight ``(N, K)``."""
    _need(w, "weight")
    n, k = w.shape
    out = torch.empty(b_plane_shape(scheme, n, k), dtype=BF16, device=w.device)
    check(lib().lcg_prepare_b(NativeScheme.of(scheme).handle, ptr(w), n, k, w.stride(0), ptr(out),
                              out.stride(0), stream_ptr()))
    return out


def a_planes(a: torch.Tensor, scheme, out: torch.Tensor | None = None) -> torch.Tensor:
    """A planes ``(rank * M2, K2p)`` of a plain activation matrix ``(M, K)``."""
    _need(a, "activation")
    m, k = a.shape
    shape = a_plane_shape(scheme, m, k)
    if out is None:
        out = torch.empty(shape, dtype=BF16, device=a.device)
    elif tuple(out.shape) != shape:
        raise ValueError(f"A-plane buffer must be {shape}, got {tuple(out.shape)}")
    check(lib().lcg_a_planes(NativeScheme.of(scheme).handle, ptr(a), m, k, a.stride(0), ptr(out),
                             out.stride(0), stream_ptr()))
    return out


def norm_planes(scheme, delta, residual, norm_weight, eps: float, residual_out, out) -> None:
    """A planes of ``norm(delta + residual)`` into ``out``, the sum into ``residual_out``.  Without a
    ``delta`` (``None``) the sum is ``residual`` itself: ``residual_out`` is ignored."""
    tensors = [(residual, "residual"), (norm_weight, "norm weight"), (out, "A planes")]
    shaped = [(residual, "residual")]
    if delta is not None:
        tensors += [(delta, "delta"), (residual_out, "residual_out")]
        shaped += [(delta, "delta"), (residual_out, "residual_out")]
    for t, what in tensors:
        _need(t, what)
    m, k = residual.shape
    for t, what in shaped:
        if tuple(t.shape) != (m, k) or not t.is_contiguous():
            raise ValueError(f"{what} must be a contiguous ({m}, {k}) tensor")
    if tuple(norm_weight.shape) != (k,):
        raise ValueError(f"norm weight must be ({k},)")
    if tuple(out.shape) != a_plane_shape(scheme, m, k):
        raise ValueError(f"A workspace must be {a_plane_shape(scheme, m, k)}, got {tuple(out.shape)}")
    check(lib().lcg_norm_planes(NativeScheme.of(scheme).handle,
                                None if delta is None else ptr(delta), ptr(residual),
                                ptr(norm_weight), m, k, float(eps),
                                None if delta is None else ptr(residual_out), ptr(out),
                                out.stride(0), stream_ptr()))


def swiglu_planes(plane_scheme, z: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``L_r(silu(z[:, :I]) * z[:, I:])`` in the interleaved gauge, ``(rank * M/2, I/2)``."""
    _need(z, "z")
    m, two_i = z.shape
    inter = two_i // 2
    shape = (plane_scheme.rank * (m // 2), inter // 2)
    if out is None:
        out = torch.empty(shape, dtype=BF16, device=z.device)
    elif tuple(out.shape) != shape:
        raise ValueError(f"plane buffer must be {shape}, got {tuple(out.shape)}")
    check(lib().lcg_swiglu_planes(NativeScheme.of(plane_scheme).handle, ptr(z), m, inter,
                                  z.stride(0), ptr(out), out.stride(0), stream_ptr()))
    return out


# --------------------------------------------------------------------- GEMMs
def _padded_out(m: int, n: int, device) -> torch.Tensor:
    """An (m, n) view whose row pitch is a multiple of 8 elements (TMA store needs 16 bytes)."""
    ld = (n + 7) // 8 * 8
    return torch.empty((m, ld), dtype=BF16, device=device)[:, :n]


def gemm_dense(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None,
               cta_group: int = 0) -> torch.Tensor:
    """``a @ b.T`` with ``a (M, K)``, ``b (N, K)`` on the dense tcgen05 kernel."""
    _need(a, "a"), _need(b, "b")
    m, k = a.shape
    n, kb = b.shape
    if kb != k:
        raise ValueError(f"inner dimensions differ: {k} vs {kb}")
    if out is None:
        out = _padded_out(m, n, a.device)
    _need(out, "out")
    check(lib().lcg_gemm_dense(ptr(a), a.stride(0), ptr(b), b.stride(0), ptr(out), out.stride(0),
                               m, n, k, cta_group, ptr(status_word(a.device)), stream_ptr()))
    return out


def gemm_r7_planes(scheme, a_pl: torch.Tensor, b_pl: torch.Tensor, m: int, n: int, k: int,
                   out: torch.Tensor | None = None, schedule: int = nat.SCHEDULE_HYBRID,
                   cta_group: int = 0, zero_out: bool = True) -> torch.Tensor:
    """Rank-7 ``C = A @ B^T`` from prepared planes.  The default hybrid schedule walks whole
    waves of tiles product by product and splits the last partial wave by product (for a shape
    with fewer tiles than CTA groups that is all of it).  With the pure rank-split schedule the
    output must arrive zeroed; ``zero_out`` does that here with a memset on the stream."""
    _need(a_pl, "A planes"), _need(b_pl, "B planes")
    if tuple(a_pl.shape) != a_plane_shape(scheme, m, k):
        raise ValueError(f"A planes must be {a_plane_shape(scheme, m, k)}, got {tuple(a_pl.shape)}")
    if tuple(b_pl.shape) != b_plane_shape(scheme, n, k):
        raise ValueError(f"B planes must be {b_plane_shape(scheme, n, k)}, got {tuple(b_pl.shape)}")
    if out is None:
        out = _padded_out(m, n, a_pl.device)
    _need(out, "out")
    if tuple(out.shape) != (m, n):
        raise ValueError(f"out must be ({m}, {n}), got {tuple(out.shape)}")
    if schedule == nat.SCHEDULE_RANK_SPLIT and zero_out:
        out.zero_()
    check(lib().lcg_gemm_r7(NativeScheme.of(scheme).handle, ptr(a_pl), a_pl.stride(0), ptr(b_pl),
                            b_pl.stride(0), ptr(out), out.stride(0), m, n, k, schedule, cta_group,
                            ptr(status_word(a_pl.device)), stream_ptr()))
    return out


def gemm_r7_slab(scheme, a_pl, b_pl, m: int, n: int, k: int, out: torch.Tensor, tile_rows,
                 schedule: int = nat.SCHEDULE_RANK_SPLIT, max_groups: int = 0, cta_group: int = 0) -> None:
    """The tile rows ``[tile_rows[0], tile_rows[1])`` of the rank-7 product into ``out`` (whole
    ``(m, n)`` output buffer; rank-split slabs accumulate, so it arrives zeroed), on at most
    ``max_groups`` CTA groups."""
    _need(a_pl, "A planes"), _need(b_pl, "B planes"), _need(out, "out")
    check(lib().lcg_gemm_r7_slab(NativeScheme.of(scheme).handle, ptr(a_pl), a_pl.stride(0), ptr(b_pl),
                                 b_pl.stride(0), ptr(out), out.stride(0), m, n, k, schedule, cta_group,
                                 int(tile_rows[0]), int(tile_rows[1]), max_groups,
                                 ptr(status_word(a_pl.device)), stream_ptr()))


def fused_a_supported(scheme, m: int, n: int, k: int) -> bool:
    """Whether the GEMM can form this scheme's A operands itself (no A planes in memory)."""
    return bool(lib().lcg_gemm_r7_fused_supported(NativeScheme.of(scheme).handle, m, n, k))


def gemm_r7_fused(a: torch.Tensor, b_pl: torch.Tensor, n: int, scheme, out: torch.Tensor | None = None,
                  schedule: int = nat.SCHEDULE_HYBRID, cta_group: int = 0, zero_out: bool = True) -> torch.Tensor:
    """Bare rank-7 GEMM straight from the activation matrix ``a (M, K)``: the A operand of every
    product is formed inside the GEMM kernel (TMA for single-block products, producer warps for
    two-block ones), so there is no plane-forming pass and no scratch."""
    _need(a, "activation"), _need(b_pl, "B planes")
    m, k = a.shape
    if tuple(b_pl.shape) != b_plane_shape(scheme, n, k):
        raise ValueError(f"B planes must be {b_plane_shape(scheme, n, k)}, got {tuple(b_pl.shape)}")
    if out is None:
        out = _padded_out(m, n, a.device)
    _need(out, "out")
    if tuple(out.shape) != (m, n):
        raise ValueError(f"out must be ({m}, {n}), got {tuple(out.shape)}")
    if schedule == nat.SCHEDULE_RANK_SPLIT and zero_out:
        out.zero_()
    check(lib().lcg_gemm_r7_fused(NativeScheme.of(scheme).handle, ptr(a), a.stride(0), ptr(b_pl),
                                  b_pl.stride(0), ptr(out), out.stride(0), m, n, k, schedule, cta_group,
                                  ptr(status_word(a.device)), stream_ptr()))
    return out


def ahead_scratch_bytes(scheme, m: int, k: int) -> int:
    """Bytes of scratch :func:`gemm_r7_ahead` needs; -1 when it does not take the scheme / shape."""
    return int(lib().lcg_gemm_r7_ahead_scratch_bytes(NativeScheme.of(scheme).handle, m, k))


def gemm_r7_ahead(a: torch.Tensor, b_pl: torch.Tensor, n: int, scheme, out: torch.Tensor | None = None,
                  scratch: torch.Tensor | None = None, schedule: int = nat.SCHEDULE_HYBRID,
                  cta_group: int = 0, zero_out: bool = True) -> torch.Tensor:
    """Bare rank-7 GEMM from the activation matrix with the A planes formed inside the GEMM
    kernel, one product ahead of the MMAs (``lcg_gemm_r7_ahead``).  ``scratch`` is a byte tensor of
    at least :func:`ahead_scratch_bytes`; it is allocated here when not given."""
    _need(a, "activation"), _need(b_pl, "B planes")
    m, k = a.shape
    if tuple(b_pl.shape) != b_plane_shape(scheme, n, k):
        raise ValueError(f"B planes must be {b_plane_shape(scheme, n, k)}, got {tuple(b_pl.shape)}")
    need = ahead_scratch_bytes(scheme, m, k)
    if need < 0:
        raise ValueError("this scheme / shape has no in-kernel plane form (K % 128 != 0, or an A row "
                         "with more than two terms)")
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.uint8, device=a.device)
    if not scratch.is_cuda or scratch.dtype != torch.uint8 or scratch.numel() < need:
        raise ValueError(f"scratch must be a CUDA uint8 tensor of at least {need} bytes")
    if out is None:
        out = _padded_out(m, n, a.device)
    _need(out, "out")
    if tuple(out.shape) != (m, n):
        raise ValueError(f"out must be ({m}, {n}), got {tuple(out.shape)}")
    if schedule == nat.SCHEDULE_RANK_SPLIT and zero_out:
        out.zero_()
    check(lib().lcg_gemm_r7_ahead(NativeScheme.of(scheme).handle, ptr(a), a.stride(0), ptr(b_pl),
                                  b_pl.stride(0), ptr(out), out.stride(0), m, n, k, ptr(scratch),
                                  scratch.numel(), schedule, cta_group, ptr(status_word(a.device)),
                                  stream_ptr()))
    return out


def gemm_r7(a: torch.Tensor, b_pl: torch.Tensor, n: int, scheme, out: torch.Tensor | None = None,
            a_workspace: torch.Tensor | None = None, schedule: int = nat.SCHEDULE_HYBRID,
            cta_group: int = 0, fused: bool | None = None, form: str | None = None,
            scratch: torch.Tensor | None = None) -> torch.Tensor:
    """Bare rank-7 GEMM ``a (M, K) @ B^T`` with prepared B planes, in one of three forms:

    ``"planes"``  the A planes are written to ``a_workspace`` by a pass in front of the GEMM;
    ``"ahead"``   the GEMM kernel's own plane warps form them, one product ahead of the MMAs,
                  in ``scratch`` (:func:`gemm_r7_ahead`);
    ``"fused"``   the A operand tiles are formed on their way into shared memory, nothing is
                  written to global memory (:func:`gemm_r7_fused`; exact, but far slower: kept
                  as the measured form of that data flow).

    ``form=None`` picks ``"ahead"`` where the scheme and shape allow it and the output is narrow
    (:func:`prefers_ahead`), else ``"planes"``.  ``fused=True / False`` is shorthand for
    ``form="fused" / "planes"``."""
    m, k = a.shape
    if form is None:
        if fused is not None:
            form = "fused" if fused else "planes"
        else:
            form = "ahead" if prefers_ahead(scheme, m, n, k) else "planes"
    if form == "fused":
        return gemm_r7_fused(a, b_pl, n, scheme, out=out, schedule=schedule, cta_group=cta_group)
    if form == "ahead":
        return gemm_r7_ahead(a, b_pl, n, scheme, out=out, scratch=scratch, schedule=schedule,
                             cta_group=cta_group)
    if form != "planes":
        raise ValueError(f"unknown form {form!r}")
    planes = a_planes(a, scheme, out=a_workspace)
    return gemm_r7_planes(scheme, planes, b_pl, m, n, k, out=out, schedule=schedule,
                          cta_group=cta_group)


# Output-column tiles (256 wide, per block column) up to which forming the A planes inside the
# GEMM kernel beats the pass in front of it.  The pass costs the same whatever the output width
# and so weighs most on narrow outputs; inside the kernel the plane warps' traffic shares each
# SM's path to L2 with the operand stream, which the 256 x 256 x 64 pair tile already fills, so
# the in-kernel form costs about half of what the separate pass costs and nothing less.
AHEAD_MAX_TILES_N = 16
_CTA_GROUPS = 74


def prefers_ahead(scheme, m: int, n: int, k: int) -> bool:
    if ahead_scratch_bytes(scheme, m, k) < 0:
        return False
    return -(-((n + 1) // 2) // 256) <= AHEAD_MAX_TILES_N


def prefers_fused_a(scheme, m: int, n: int, k: int) -> bool:
    """The shared-memory form is never the fastest on this GPU (see :func:`gemm_r7`)."""
    return False


def bare_gemm_form(m: int, n: int, k: int):
    """``(scheme name, form, schedule)``: what an exact shape of the bare rank-7 GEMM is
    dispatched to.  Narrow outputs take the locality-ordered products with the two single-block
    ones first and the in-kernel plane form; wide ones the postsum-CSE decomposition (seven
    publications instead of twelve) on planes written by a pass in front.  The in-kernel form
    runs the rank-split unit list when whole waves of tiles would leave a short last wave."""
    tiles_m, tiles_n = -(-((m + 1) // 2) // 256), -(-((n + 1) // 2) // 256)
    if k % 128 == 0 and k >= 128 and tiles_n <= AHEAD_MAX_TILES_N:
        tiles = tiles_m * tiles_n
        tail = tiles % _CTA_GROUPS
        split = tiles >= 2 * _CTA_GROUPS and 0 < tail < _CTA_GROUPS // 4
        return "2x2_locality_lead_single", "ahead", nat.SCHEDULE_RANK_SPLIT if split else nat.SCHEDULE_HYBRID
    return "2x2_postsum_cse", "planes", nat.SCHEDULE_HYBRID


def gate_up_chain(scheme, plane_scheme, a_pl, b_pl, z, down_planes, preclear=None,
                  schedule: int = nat.SCHEDULE_HYBRID, cta_group: int = 0, init_from=None) -> None:
    """The chained gate_up GEMM.  ``preclear``: the rank-split consumer's output, zeroed while the
    kernel runs -- or, with ``init_from`` (same shape, contiguous, another buffer), filled with it, so
    that the consumer's reduce-adds land on the residual stream."""
    for t, what in ((a_pl, "A planes"), (b_pl, "B planes"), (z, "z"), (down_planes, "down planes")):
        _need(t, what)
    m, n = z.shape
    k = 2 * a_pl.shape[1]
    if tuple(a_pl.shape) != a_plane_shape(scheme, m, k) or tuple(b_pl.shape) != b_plane_shape(scheme, n, k):
        raise ValueError("operand planes do not match the output shape")
    if tuple(down_planes.shape) != (plane_scheme.rank * (m // 2), n // 4):
        raise ValueError(
            f"down planes must be ({plane_scheme.rank * (m // 2)}, {n // 4}), got {tuple(down_planes.shape)}")
    pc_ptr, pc_bytes = 0, 0
    if preclear is not None:
        _need(preclear, "preclear")
        if not preclear.is_contiguous():
            raise ValueError("the consumer output to clear must be contiguous")
        pc_ptr, pc_bytes = ptr(preclear), preclear.numel() * preclear.element_size()
    if init_from is not None:
        _need(init_from, "initial content")
        if preclear is None or tuple(init_from.shape) != tuple(preclear.shape) or not init_from.is_contiguous():
            raise ValueError("the initial content must be a contiguous tensor of the consumer output's shape")
        check(lib().lcg_gate_up_chain_init(
            NativeScheme.of(scheme).handle, NativeScheme.of(plane_scheme).handle, ptr(a_pl), a_pl.stride(0),
            ptr(b_pl), b_pl.stride(0), ptr(z), z.stride(0), m, n, k, ptr(down_planes), down_planes.stride(0),
            pc_ptr, pc_bytes, ptr(init_from), schedule, cta_group, ptr(status_word(z.device)), stream_ptr()))
        return
    check(lib().lcg_gate_up_chain(NativeScheme.of(scheme).handle, NativeScheme.of(plane_scheme).handle,
                                  ptr(a_pl), a_pl.stride(0), ptr(b_pl), b_pl.stride(0), ptr(z),
                                  z.stride(0), m, n, k, ptr(down_planes), down_planes.stride(0),
                                  pc_ptr, pc_bytes, schedule, cta_group, ptr(status_word(z.device)),
                                  stream_ptr()))


# ------------------------------------------------- tensor parallel, peer memory
def _ptr_table(ptrs):
    return (ctypes.c_void_p * len(ptrs))(*[int(v) for v in ptrs])


def gemm_r7_push(scheme, a_pl, b_pl, m: int, n: int, k: int, c: torch.Tensor, slot_ptrs, rank: int,
                 rows_per_owner: int, cta_group: int = 0) -> None:
    """Row-parallel rank-7 ``down`` of one rank: the partial into ``c`` and, from the same
    kernel, every finished tile's rows into ``slot_ptrs[owner]`` (device addresses of this
    rank's ``(rows_per_owner, n)`` region in each owner's memory)."""
    _need(a_pl, "A planes"), _need(b_pl, "B planes"), _need(c, "c")
    if tuple(c.shape) != (m, n):
        raise ValueError(f"c must be ({m}, {n}), got {tuple(c.shape)}")
    check(lib().lcg_gemm_r7_push(NativeScheme.of(scheme).handle, ptr(a_pl), a_pl.stride(0), ptr(b_pl),
                                 b_pl.stride(0), ptr(c), c.stride(0), m, n, k, _ptr_table(slot_ptrs),
                                 len(slot_ptrs), rank, rows_per_owner, cta_group,
                                 ptr(status_word(c.device)), stream_ptr()))


def peer_barrier(flag_ptrs, rank: int, epoch: int, limit_us: int = 10_000_000, device=None) -> None:
    """Barrier between the ranks on the current stream (bounded wait; code 106 on run-out)."""
    check(lib().lcg_peer_barrier(_ptr_table(flag_ptrs), len(flag_ptrs), rank, epoch & 0xFFFFFFFF,
                                 limit_us, ptr(status_word(device)), stream_ptr()))


def reduce_gather(slots: torch.Tensor, h: torch.Tensor, out_ptrs, rows_per_owner: int, rank: int) -> None:
    """``out[rows of rank] = bf16(h + sum_w slots[w])`` stored into every rank's output."""
    _need(slots, "slots"), _need(h, "h")
    world, rpo, cols = slots.shape
    if rpo != rows_per_owner or world != len(out_ptrs) or not slots.is_contiguous():
        raise ValueError("slots must be a contiguous (world, rows_per_owner, cols) tensor")
    m = h.shape[0]
    check(lib().lcg_reduce_gather(ptr(slots), ptr(h), h.stride(0), _ptr_table(out_ptrs), m, cols,
                                  rows_per_owner, world, rank, stream_ptr()))


# -------------------------------------------------------------- dense seams
def add_rmsnorm(delta, residual, norm_weight, eps: float, residual_out=None, x=None):
    """``(norm(delta + residual), delta + residual)``; without a ``delta`` the second value is
    ``residual`` itself and nothing is stored for it."""
    for t, what in ((residual, "residual"), (norm_weight, "norm weight")):
        _need(t, what)
    m, k = residual.shape
    if x is None:
        x = torch.empty_like(residual)
    if delta is None:
        for t in (residual, x):
            if tuple(t.shape) != (m, k) or not t.is_contiguous():
                raise ValueError(f"operands must be contiguous ({m}, {k}) tensors")
        check(lib().lcg_add_rmsnorm(None, ptr(residual), ptr(norm_weight), m, k, float(eps),
                                    None, ptr(x), stream_ptr()))
        return x, residual
    _need(delta, "delta")
    if residual_out is None:
        residual_out = torch.empty_like(delta)
    for t in (delta, residual, residual_out, x):
        if tuple(t.shape) != (m, k) or not t.is_contiguous():
            raise ValueError(f"operands must be contiguous ({m}, {k}) tensors")
    check(lib().lcg_add_rmsnorm(ptr(delta), ptr(residual), ptr(norm_weight), m, k, float(eps),
                                ptr(residual_out), ptr(x), stream_ptr()))
    return x, residual_out


def swiglu(z: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _need(z, "z")
    m, two_i = z.shape
    inter = two_i // 2
    if out is None:
        out = torch.empty((m, inter), dtype=BF16, device=z.device)
    check(lib().lcg_swiglu(ptr(z), m, inter, z.stride(0), ptr(out), out.stride(0), stream_ptr()))
    return out


def add(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    _need(a, "a"), _need(b, "b")
    if a.shape != b.shape or not a.is_contiguous() or not b.is_contiguous():
        raise ValueError("operands must be contiguous and of equal shape")
    if out is None:
        out = torch.empty_like(a)
    check(lib().lcg_add(ptr(a), ptr(b), ptr(out), a.numel(), stream_ptr()))
    return out
