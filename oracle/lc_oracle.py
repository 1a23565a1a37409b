"""CPU oracle of the rank-7 MLP prefill path.  TEST INFRASTRUCTURE, not product code.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference arm
of ``bench.py`` may import this module.  Nothing in the package under
``writes-that-matter_b200/`` imports it, and it imports nothing from there except
the scheme coefficient tables, which it reads as JSON data.

It restates, in plain torch on the CPU, the algorithm of the reference project
(lcgemm) for this path; each function names the reference lines it follows.
Parity status: PINNED.  ``tests/golden/make_golden.py`` ran the reference's own
``load``/``prepare_b``/``chain_a_planes``/``permute_k``/``_reference`` (imported
from the reference tree) on seeded inputs and committed the outputs;
``tests/test_oracle.py`` checks this restatement against those fixtures bit for
bit.  The reference ships no numeric golden vectors of its own for the device
kernels; their rounding structure is restated from the kernel sources cited
below and that part is pinned only through those citations.
"""
from __future__ import annotations

import json
from pathlib import Path

import torch

SCHEME_DIR = (Path(__file__).resolve().parent.parent / "writes-that-matter_b200" / "lcgemm"
              / "schemes")
CHUNK = 64   # lcgemm/chain_gauge.py:45


# ------------------------------------------------------------------ scheme tables
class Tables:
    """Coefficient rows of a 2x2x2 scheme and the term lists derived from them
    (lcgemm/scheme.py:150-170)."""

    def __init__(self, name: str):
        raw = json.loads((SCHEME_DIR / f"{name}.json").read_text())
        self.name = name
        self.p, self.q, self.s = raw["shape"]
        self.rank = int(raw["r"])
        self.a, self.b, self.c = raw["A"], raw["B"], raw["C"]
        self.clear = list((raw.get("postsum") or {}).get("clear", []))
        self.a_terms = self._terms(self.a, self.q)
        self.b_terms = self._terms(self.b, self.s)
        self.c_terms = self._terms(self.c, self.s)

    @staticmethod
    def _terms(rows, width):
        return [[(n // width, n % width, v) for n, v in enumerate(row) if v] for row in rows]

    def identity_holds(self) -> bool:
        """lcgemm/scheme.py:324-361, by brute force over the dense 2^6 index grid."""
        for i in range(2):
            for j in range(2):
                for ia in range(2):
                    for ka in range(2):
                        for kb in range(2):
                            for jb in range(2):
                                tot = sum(self.c[r][i * 2 + j] * self.a[r][ia * 2 + ka]
                                          * self.b[r][kb * 2 + jb] for r in range(self.rank))
                                if tot != int(ia == i and ka == kb and jb == j):
                                    return False
        return True

    def chains(self):
        """Accumulator chains t, t+2, ... (lcgemm/scheme.py:204-222)."""
        clear = self.clear or [1] * self.rank
        out, open_ = [], {}
        for t in range(self.rank):
            st = t % 2
            if clear[t] or st not in open_:
                open_[st] = []
                out.append(open_[st])
            open_[st].append(t)
        return out

    def publications(self):
        """Per step the (i, j, sigma) prefix-sum publications, sigma_t = c[t] - c[next(t)]
        (lcgemm/scheme.py:234-248), and the per-step 'is first writer' flags
        (lcgemm/scheme.py:424-429)."""
        nxt = [-1] * self.rank
        for ch in self.chains():
            for x, y in zip(ch, ch[1:]):
                nxt[x] = y
        pubs = []
        for t in range(self.rank):
            after = self.c[nxt[t]] if nxt[t] >= 0 else [0] * 4
            pubs.append([(n // 2, n % 2, self.c[t][n] - after[n]) for n in range(4)
                         if self.c[t][n] - after[n]])
        return pubs


def bf16(x: torch.Tensor) -> torch.Tensor:
    """Round to bfloat16 (nearest even) and return as float32."""
    return x.to(torch.bfloat16).to(torch.float32)


def half_up(n: int, align: int = 1) -> int:
    h = (n + 1) // 2
    return (h + align - 1) // align * align


def _block(x: torch.Tensor, rb: int, cb: int, r2: int, c2: int, c2p: int) -> torch.Tensor:
    """Block (rb, cb) of x as an (r2, c2p) float32 matrix, zero outside x."""
    out = torch.zeros((r2, c2p), dtype=torch.float32)
    src = x[rb * r2:(rb + 1) * r2, cb * c2:(cb + 1) * c2].to(torch.float32)
    out[:src.shape[0], :src.shape[1]] = src
    return out


# ------------------------------------------------------------------------ planes
def prepare_b(w: torch.Tensor, tb: Tables, dtype=torch.bfloat16) -> torch.Tensor:
    """B planes of a weight (N, K): fp32 sum, one rounding (lcgemm/planes.py:54-71).
    Odd shapes use N2 = round_up(ceil(N/2), 8), K2 = ceil(K/2) padded to 64 with zeros."""
    n, k = w.shape
    n2, k2 = half_up(n, 8), half_up(k)
    k2p = (k2 + 63) // 64 * 64
    out = torch.zeros((tb.rank * n2, k2p), dtype=dtype)
    for r in range(tb.rank):
        acc = torch.zeros((n2, k2p), dtype=torch.float32)
        for kk, j, cf in tb.b_terms[r]:
            acc.add_(_block(w, j, kk, n2, k2, k2p), alpha=float(cf))
        out[r * n2:(r + 1) * n2] = acc.to(dtype)
    return out


def a_planes(a: torch.Tensor, tb: Tables, dtype=torch.bfloat16) -> torch.Tensor:
    """A planes of a plain (M, K) activation: the pattern of lcgemm/chain_gauge.py:91-98
    without SwiGLU or gauge.  fp32 sum in term order, one rounding."""
    m, k = a.shape
    m2, k2 = half_up(m), half_up(k)
    k2p = (k2 + 63) // 64 * 64
    out = torch.zeros((tb.rank * m2, k2p), dtype=dtype)
    for r in range(tb.rank):
        acc = torch.zeros((m2, k2p), dtype=torch.float32)
        for i, kk, cf in tb.a_terms[r]:
            acc += float(cf) * _block(a, i, kk, m2, k2, k2p)
        out[r * m2:(r + 1) * m2] = acc.to(dtype)
    return out


def norm_planes(delta, residual, norm_weight, eps, tb: Tables):
    """Fused residual add + RMSNorm + A planes (lcgemm/kernels/fused_norm.py:175-198):
    h is rounded to bf16 before the norm; y = h * rstd * (w + 1); signed sums; one rounding.
    Returns (planes bf16, residual_out bf16)."""
    h = (delta.float() + residual.float()).to(delta.dtype)
    hf = h.float()
    rstd = torch.rsqrt(hf.square().mean(-1, keepdim=True) + eps)
    y = hf * rstd * (norm_weight.float() + 1.0)
    return a_planes(y, tb), h


def interleave_perm(width: int, chunk: int = CHUNK) -> torch.Tensor:
    """lcgemm/chain_gauge.py:51-65: block j = {c : (c // chunk) % 2 == j},
    index l = (c // 2chunk) * chunk + c % chunk."""
    if width % (2 * chunk):
        raise ValueError(f"width {width} not divisible by 2*chunk {2 * chunk}")
    c = torch.arange(width)
    j = (c // chunk) % 2
    l = (c // (2 * chunk)) * chunk + (c % chunk)
    perm = torch.empty(width, dtype=torch.long)
    perm[j * (width // 2) + l] = c
    return perm


def permute_k(x: torch.Tensor, chunk: int = CHUNK) -> torch.Tensor:
    """lcgemm/chain_gauge.py:68-70."""
    return x[..., interleave_perm(x.shape[-1], chunk)].contiguous()


def swiglu(z: torch.Tensor) -> torch.Tensor:
    """lcgemm/chain_gauge.py:76-79 (fp32, no intermediate rounding)."""
    i = z.shape[-1] // 2
    zf = z.float()
    return torch.nn.functional.silu(zf[:, :i]) * zf[:, i:]


def chain_a_planes(z: torch.Tensor, tb: Tables, chunk: int = CHUNK,
                   dtype=torch.bfloat16) -> torch.Tensor:
    """L_r(SwiGLU(Z)) in the interleaved gauge (lcgemm/chain_gauge.py:82-99)."""
    return a_planes(permute_k(swiglu(z), chunk), tb, dtype)


def prepare_down_b(w: torch.Tensor, tb: Tables, chunk: int = CHUNK) -> torch.Tensor:
    """lcgemm/chain_gauge.py:102-111."""
    return prepare_b(permute_k(w, chunk), tb)


# -------------------------------------------------------------------- the products
def products(a_pl: torch.Tensor, b_pl: torch.Tensor, rank: int):
    """P_r = At_r @ Bt_r^T in fp32 (bf16 x bf16 -> fp32 accumulate on the device)."""
    m2, n2 = a_pl.shape[0] // rank, b_pl.shape[0] // rank
    return [a_pl[r * m2:(r + 1) * m2].float() @ b_pl[r * n2:(r + 1) * n2].float().T
            for r in range(rank)]


def combine_exact(prods, tb: Tables, m: int, n: int) -> torch.Tensor:
    """C[i][j] = sum_r c[r][i,j] P_r in fp32 (lcgemm/scheme.py:6-9,160-163)."""
    m2, n2 = prods[0].shape
    c = torch.zeros((2 * m2, 2 * n2), dtype=torch.float32)
    for r, terms in enumerate(tb.c_terms):
        for i, j, cf in terms:
            c[i * m2:(i + 1) * m2, j * n2:(j + 1) * n2] += float(cf) * prods[r]
    return _crop(c, m, n, m2, n2)


def _crop(c, m, n, m2, n2):
    rows = torch.cat([torch.arange(0, m2), torch.arange(m2, m2 + (m - m2))])
    cols = torch.cat([torch.arange(0, n2), torch.arange(n2, n2 + (n - n2))])
    return c[rows][:, cols]


def combine_as_kernel(prods, tb: Tables, m: int, n: int, rank_split: bool = False) -> torch.Tensor:
    """The combine with the device kernels' rounding points.

    All-ranks schedule (lcgemm/kernels/sm100.py:595-625,690-727): products of a chain add
    up in the fp32 accumulator; each publication is rounded to bf16; the first write to a
    block is a store, later ones are bf16 adds in memory.
    Rank-split schedule (lcgemm/kernels/down_rank_split.py:209-216,483-508): every product
    is rounded to bf16 and added into a zeroed bf16 output (addition order is not fixed
    on the device; ascending rank is used here)."""
    m2, n2 = prods[0].shape
    blocks = {(i, j): None for i in range(2) for j in range(2)}

    def publish(i, j, val):
        v = bf16(val)
        blocks[(i, j)] = v if blocks[(i, j)] is None else bf16(blocks[(i, j)] + v)

    if rank_split:
        for key in blocks:
            blocks[key] = torch.zeros((m2, n2))
        for r, terms in enumerate(tb.c_terms):
            for i, j, cf in terms:
                publish(i, j, float(cf) * prods[r])
    else:
        clear = tb.clear or [1] * tb.rank
        acc = {}
        pubs = tb.publications()
        for t in range(tb.rank):
            st = t % 2
            acc[st] = prods[t].clone() if clear[t] or st not in acc else acc[st] + prods[t]
            for i, j, sigma in pubs[t]:
                publish(i, j, float(sigma) * acc[st])
    c = torch.zeros((2 * m2, 2 * n2), dtype=torch.float32)
    for (i, j), v in blocks.items():
        c[i * m2:(i + 1) * m2, j * n2:(j + 1) * n2] = v
    return _crop(c, m, n, m2, n2)


def scheme_matmul(a: torch.Tensor, w: torch.Tensor, tb: Tables, mode: str = "fp32") -> torch.Tensor:
    """C = A @ W^T through the scheme.  ``w`` is (N, K) as the reference stores weights.

    mode "fp32":   planes, products and combine in the input precision (the fp32 CPU configuration);
    mode "planes": bf16 planes (one rounding each), fp32 products and combine;
    mode "kernel": bf16 planes and the kernels' publication rounding, all-ranks schedule;
    mode "kernel_split": the same with the rank-split schedule."""
    m, n = a.shape[0], w.shape[0]
    dt = torch.float32 if mode == "fp32" else torch.bfloat16
    prods = products(a_planes(a, tb, dt), prepare_b(w, tb, dt), tb.rank)
    if mode in ("fp32", "planes"):
        return combine_exact(prods, tb, m, n)
    return combine_as_kernel(prods, tb, m, n, rank_split=(mode == "kernel_split"))


# ------------------------------------------------------------------- the MLP layer
def mlp_reference(delta, residual, norm_weight, gate_up_weight, down_weight, eps):
    """The functional reference of the operator boundary, rounding points included
    (lcgemm/integrate/qwen_patch.py:41-58).  Returns (down_out, residual_out)."""
    F = torch.nn.functional
    h = (delta.float() + residual.float()).to(delta.dtype)
    hf = h.float()
    x = hf * torch.rsqrt(hf.square().mean(-1, keepdim=True) + eps)
    x = (x * (norm_weight.float() + 1.0)).to(delta.dtype)
    gate_up = (x.float() @ gate_up_weight.float().T).to(delta.dtype)
    gate, up = gate_up.chunk(2, dim=-1)
    act = F.silu(gate.float()).to(gate.dtype) * up
    return (act.float() @ down_weight.float().T).to(delta.dtype), h


def mlp_chain(delta, residual, norm_weight, gate_up_weight, down_weight, eps,
              gate_tb: Tables, down_tb: Tables, rank_split_down: bool = True):
    """The chained rank-7 layer with the device rounding structure: fused norm planes ->
    gate_up products with chain publications -> SwiGLU planes in the gauge -> down products
    (lcgemm/integrate/qwen_patch.py:85-97 and the kernels cited above).
    Returns (down_out, residual_out, z, down_planes)."""
    m = delta.shape[0]
    two_i = gate_up_weight.shape[0]
    n_out = down_weight.shape[0]
    a_pl, h = norm_planes(delta, residual, norm_weight, eps, gate_tb)
    prods = products(a_pl, prepare_b(gate_up_weight, gate_tb), gate_tb.rank)
    z = combine_as_kernel(prods, gate_tb, m, two_i).to(torch.bfloat16)
    d_pl = chain_a_planes(z, down_tb)
    prods = products(d_pl, prepare_down_b(down_weight, down_tb), down_tb.rank)
    out = combine_as_kernel(prods, down_tb, m, n_out, rank_split=rank_split_down)
    return out.to(torch.bfloat16), h, z, d_pl
