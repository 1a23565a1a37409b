"""Generate the golden fixtures of tests/golden/ from the reference implementation.

Run once, in a container where the reference tree is importable:

    PYTHONPATH=/path/to/reference python tests/golden/make_golden.py

It imports the reference package ``lcgemm`` (NOT this repository's package of the same
name: the script refuses to run if ``lcgemm`` resolves inside this repository), evaluates
the reference's own host functions on seeded CPU inputs and writes

    scheme_tables.json   derived tables of both deployed schemes
    planes.npz           prepare_b, chain_a_planes, permute_k, interleave_perm, prepare_down_b
    mlp_reference.npz    the functional MLP reference and the Muse RMSNorm helper
    evaluator.npz        the scheme evaluator composed from the reference's pieces
                         (A planes by the chain_a_planes pattern, prepare_b, products,
                         C combine over c_terms), fp32, A ~ N(0,1), B ~ N(0,0.02)

bf16 tensors are stored as their int16 bit patterns.
"""
from __future__ import annotations

import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent

import lcgemm  # noqa: E402  (the reference)

if str(REPO) in str(Path(lcgemm.__file__).resolve()):
    sys.exit("lcgemm resolved inside this repository; put the reference tree on PYTHONPATH")

from lcgemm import chain_gauge, planes  # noqa: E402
from lcgemm.scheme import load  # noqa: E402
from lcgemm.integrate import muse_patch, qwen_patch  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    assert t.dtype == torch.bfloat16
    return t.contiguous().view(torch.int16).numpy()


def main() -> None:
    names = ("2x2_postsum_cse", "2x2_locality_ordered")
    schemes = {n: load(n) for n in names}

    tables = {}
    for n, s in schemes.items():
        tables[n] = {
            "shape": list(s.shape), "rank": s.rank, "has_postsum": s.has_postsum,
            "a_terms": [[list(t) for t in step] for step in s.a_terms],
            "b_terms": [[list(t) for t in step] for step in s.b_terms],
            "c_terms": [[list(t) for t in step] for step in s.c_terms],
            "acc_clear": list(s.acc_clear),
            "postsum_chains": [list(c) for c in s.postsum_chains],
            "postsum_next": list(s.postsum_next),
            "postsum_terms": [[list(t) for t in step] for step in s.postsum_terms],
            "epi_groups": [[[g.coeff, [[d.row, d.col, bool(d.is_first)] for d in g.dests]]
                            for g in step] for step in s.epi_groups],
            "dest_groups": [[[g.coeff, [[d.row, d.col, bool(d.is_first)] for d in g.dests]]
                             for g in step] for step in s.dest_groups],
            "num_writes": s.num_writes, "num_staging_passes": s.num_staging_passes,
            "num_output_writes": s.num_output_writes, "summary": s.summary(),
        }
    (HERE / "scheme_tables.json").write_text(json.dumps(tables, indent=1) + "\n")

    g = torch.Generator().manual_seed(20240607)
    out = {}
    w = (torch.randn(192, 256, generator=g) * 0.02).to(torch.bfloat16)          # (N, K)
    out["w"] = bits(w)
    for n, s in schemes.items():
        out[f"prepare_b.{n}"] = bits(planes.prepare_b(w, s))
    z = torch.randn(64, 512, generator=g).to(torch.bfloat16)                   # (M, 2I), I = 256
    out["z"] = bits(z)
    for n, s in schemes.items():
        out[f"chain_a_planes.{n}"] = bits(chain_gauge.chain_a_planes(z, s))
    out["swiglu_fp32"] = chain_gauge.swiglu(z).numpy()
    for width in (128, 256, 640):
        out[f"interleave_perm.{width}"] = chain_gauge.interleave_perm(width).numpy()
    wd = (torch.randn(96, 256, generator=g) * 0.02).to(torch.bfloat16)          # down weight (N, K=I)
    out["w_down"] = bits(wd)
    out["permute_k.w_down"] = bits(chain_gauge.permute_k(wd))
    out["prepare_down_b"] = bits(chain_gauge.prepare_down_b(wd, schemes["2x2_locality_ordered"]))
    np.savez_compressed(HERE / "planes.npz", **out)

    # The functional MLP reference (bf16 on the CPU) and Muse's RMSNorm helper.
    m, h, i = 32, 128, 256
    delta = torch.randn(m, h, generator=g).to(torch.bfloat16)
    residual = torch.randn(m, h, generator=g).to(torch.bfloat16)
    norm_w = (torch.randn(h, generator=g) * 0.01).to(torch.bfloat16)
    w_gu = (torch.randn(2 * i, h, generator=g) * 0.02).to(torch.bfloat16)
    w_dn = (torch.randn(h, i, generator=g) * 0.02).to(torch.bfloat16)
    down_out, hres = qwen_patch._reference(delta, residual, norm_w, w_gu, w_dn, 1e-6)
    np.savez_compressed(
        HERE / "mlp_reference.npz", delta=bits(delta), residual=bits(residual), norm_w=bits(norm_w),
        w_gate_up=bits(w_gu), w_down=bits(w_dn), down_out=bits(down_out), residual_out=bits(hres),
        muse_rmsnorm=bits(muse_patch._rmsnorm(hres, norm_w, 1e-5)))

    # The composed scheme evaluator in fp32 at the config-1 distribution, small size.
    torch.manual_seed(0)
    a = torch.randn(128, 256)
    b = torch.randn(256, 192) * 0.02
    wt = b.T.contiguous()
    ev = {"a": a.numpy(), "b": b.numpy()}
    for n, s in schemes.items():
        m2, k2, n2 = a.shape[0] // 2, a.shape[1] // 2, wt.shape[0] // 2
        bt = planes.prepare_b(wt, s)
        c = torch.zeros(a.shape[0], wt.shape[0])
        for r in range(s.rank):
            at = torch.zeros(m2, k2)
            for bi, bk, cf in s.a_terms[r]:
                at += float(cf) * a[bi * m2:(bi + 1) * m2, bk * k2:(bk + 1) * k2]
            p = at @ bt[r * n2:(r + 1) * n2].T
            for ci, cj, cf in s.c_terms[r]:
                c[ci * m2:(ci + 1) * m2, cj * n2:(cj + 1) * n2] += float(cf) * p
        ev[f"c.{n}"] = c.numpy()
    ev["dense"] = (a @ b).numpy()
    np.savez_compressed(HERE / "evaluator.npz", **ev)
    print("wrote", sorted(p.name for p in HERE.iterdir()))


if __name__ == "__main__":
    main()
