"""Rank-R bilinear schemes for the block matrix product, and their epilogue plans.

A ``matmul-rabc-v1`` scheme splits A into ``p x q`` blocks and B into ``q x s``
blocks and replaces the ``p*q*s`` block products by ``R`` products of signed
block sums::

    At_r = sum a[r][i,k] A[i][k]     Bt_r = sum b[r][k,j] B[k][j]
    P_r  = At_r @ Bt_r               C[i][j] = sum c[r][i,j] P_r

This module keeps the public surface of the reference's scheme layer
(``lcgemm/scheme.py:68-486``: ``Term``, ``Dest``, ``Group``, ``Scheme`` with its
derived tables, ``load``), because the seams, the native library and the tests
all speak in those tables.  The derivations are done once, eagerly, by
:func:`_derive` when a ``Scheme`` is built, and exact-integer validation is part
of :func:`load`.

Accumulator chains ("postsum" plans, ``lcgemm/scheme.py:18-40``).  The GEMM
kernel owns two accumulator stages and step ``t`` uses stage ``t % 2``.  A step
whose ``clear`` flag is 0 adds its product to whatever step ``t - 2`` left in
that stage, so a run of same-parity steps forms a chain and the only values a
chain can publish are its prefix sums.  Publishing prefix ``t`` with coefficient
``sigma_t = c[t] - c[next(t)]`` makes the prefixes telescope to ``C``; a block
whose coefficient does not change along the chain costs no write at all.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import NamedTuple

FORMAT = "matmul-rabc-v1"
SCHEME_DIR = Path(__file__).resolve().parent / "schemes"


class Term(NamedTuple):
    """``coeff * X[row][col]`` where (row, col) indexes a block grid."""

    row: int
    col: int
    coeff: int

    def __repr__(self) -> str:  # plain-tuple repr, as in lcgemm/scheme.py:86-87
        return f"({self.row}, {self.col}, {self.coeff})"


class Dest(NamedTuple):
    """One output block of a staged tile; ``is_first`` = plain store, else reduce-add."""

    row: int
    col: int
    is_first: bool

    def __repr__(self) -> str:
        return f"({self.row}, {self.col}, {self.is_first})"


class Group(NamedTuple):
    """One accumulator->shared-memory staging pass and the blocks it feeds."""

    coeff: int
    dests: tuple

    def __repr__(self) -> str:
        return f"({self.coeff}, {self.dests!r})"


def _nonzeros(rows, width):
    return tuple(
        tuple(Term(n // width, n % width, v) for n, v in enumerate(row) if v) for row in rows
    )


def _first_writer_of(table):
    seen: dict = {}
    for step, terms in enumerate(table):
        for term in terms:
            seen.setdefault((term.row, term.col), step)
    return seen


def _grouped(table, first):
    """Per step: terms bucketed by coefficient, positive coefficients first."""
    out = []
    for step, terms in enumerate(table):
        buckets: dict = {}
        for term in terms:
            buckets.setdefault(term.coeff, []).append(
                Dest(term.row, term.col, first[(term.row, term.col)] == step))
        out.append(tuple(Group(cf, tuple(buckets[cf])) for cf in sorted(buckets, reverse=True)))
    return tuple(out)


@dataclass(frozen=True)
class Scheme:
    """A rank-R decomposition of the ``p x q x s`` block product plus its epilogue plan."""

    name: str
    shape: tuple            # (p, q, s)
    rank: int
    a: tuple                # rank x (p*q), row-major over (i, k)
    b: tuple                # rank x (q*s), row-major over (k, j)
    c: tuple                # rank x (p*s), row-major over (i, j)
    clear: tuple = ()       # per-step chain flags, () = plain scatter epilogue
    _t: dict = field(default_factory=dict, repr=False, compare=False)

    def __post_init__(self):
        self._t.update(_derive(self))

    # block-grid extents
    p = property(lambda self: self.shape[0])
    q = property(lambda self: self.shape[1])
    s = property(lambda self: self.shape[2])

    # operand transforms
    a_terms = property(lambda self: self._t["a_terms"])
    b_terms = property(lambda self: self._t["b_terms"])
    c_terms = property(lambda self: self._t["c_terms"])

    # plain scatter epilogue
    first_writer = property(lambda self: self._t["first_writer"])
    dest_groups = property(lambda self: self._t["dest_groups"])

    # chain plan
    has_postsum = property(lambda self: bool(self.clear))
    acc_clear = property(lambda self: self._t["acc_clear"])
    postsum_chains = property(lambda self: self._t["chains"])
    postsum_next = property(lambda self: self._t["next"])
    postsum_terms = property(lambda self: self._t["postsum_terms"])
    postsum_groups = property(lambda self: self._t["postsum_groups"])

    @property
    def epi_groups(self):
        """What the kernel walks: the chain plan if there is one, else the plain scatter."""
        return self.postsum_groups if self.has_postsum else self.dest_groups

    @property
    def num_staging_passes(self) -> int:
        return sum(len(step) for step in self.epi_groups)

    @property
    def num_writes(self) -> int:
        return sum(len(g.dests) for step in self.epi_groups for g in step)

    @property
    def num_output_writes(self) -> int:
        return sum(len(t) for t in self.c_terms)

    # ---------------------------------------------------------------- validation
    def validate(self) -> None:
        """Shape, the exact tensor identity, and the chain plan (lcgemm/scheme.py:275-292)."""
        self._validate_shape()
        self._validate_identity()
        if self.has_postsum:
            self.validate_postsum()

    def _validate_shape(self) -> None:
        if len(self.shape) != 3 or min(self.shape) < 1:
            raise ValueError(f"scheme {self.name!r}: shape {self.shape} is not a (p, q, s) block grid")
        if self.rank < 1:
            raise ValueError(f"scheme {self.name!r}: rank {self.rank} must be at least 1")
        wanted = (("A", self.a, self.p * self.q), ("B", self.b, self.q * self.s),
                  ("C", self.c, self.p * self.s))
        for label, rows, width in wanted:
            if len(rows) != self.rank:
                raise ValueError(
                    f"scheme {self.name!r}: {label} has {len(rows)} rows for a rank-{self.rank} "
                    f"decomposition; every product needs one row of {label} coefficients")
            for r, row in enumerate(rows):
                if len(row) != width:
                    raise ValueError(
                        f"scheme {self.name!r}: {label} row of product {r} has {len(row)} "
                        f"coefficients, expected {width}")
                if not any(row):
                    raise ValueError(
                        f"scheme {self.name!r}: product {r} has an all-zero {label} row, so it "
                        f"computes nothing and the rank is overstated")

    def _validate_identity(self) -> None:
        """``sum_r c[r][i,j] a[r][i',k'] b[r][k'',j''] == [i'=i][k'=k''][j''=j]`` in integers."""
        p, q, s = self.shape
        total: dict = {}
        for r in range(self.rank):
            for ct in self.c_terms[r]:
                for at in self.a_terms[r]:
                    for bt in self.b_terms[r]:
                        key = (ct.row, ct.col, at.row, at.col, bt.row, bt.col)
                        total[key] = total.get(key, 0) + ct.coeff * at.coeff * bt.coeff
        for i in range(p):
            for k in range(q):
                for j in range(s):
                    got = total.pop((i, j, i, k, k, j), 0)
                    if got != 1:
                        raise ValueError(
                            f"scheme {self.name!r} is not a decomposition of the matmul: "
                            f"A[{i}][{k}]*B[{k}][{j}] reaches C[{i}][{j}] with coefficient {got}, "
                            f"but the product requires 1")
        for (i, j, ia, ka, kb, jb), v in total.items():
            if v:
                raise ValueError(
                    f"scheme {self.name!r} is not a decomposition of the matmul: "
                    f"A[{ia}][{ka}]*B[{kb}][{jb}] leaks into C[{i}][{j}] with coefficient {v}, "
                    f"but must cancel to 0")

    def validate_postsum(self) -> None:
        """The chain plan is well formed and its prefix sums telescope back to ``C``."""
        if len(self.clear) != self.rank:
            raise ValueError(
                f"scheme {self.name!r}: the chain plan has {len(self.clear)} step flags but the "
                f"decomposition has {self.rank} products")
        if any(v not in (0, 1) for v in self.clear):
            raise ValueError(f"scheme {self.name!r}: clear must be 0/1 per step, got {self.clear}")
        for t in range(min(2, self.rank)):
            if not self.clear[t]:
                raise ValueError(
                    f"scheme {self.name!r}: step {t} continues a chain, but it is the first step "
                    f"on accumulator stage {t % 2}; there is nothing for it to add to")
        width = self.p * self.s
        rebuilt = [[0] * width for _ in range(self.rank)]
        for chain in self.postsum_chains:
            for pos, t in enumerate(chain):
                for term in self.postsum_terms[t]:
                    for earlier in chain[: pos + 1]:
                        rebuilt[earlier][term.row * self.s + term.col] += term.coeff
        for r in range(self.rank):
            if rebuilt[r] != list(self.c[r]):
                raise ValueError(
                    f"scheme {self.name!r}: the chain plan does not reproduce C. Product {r} ends "
                    f"up with output coefficients {rebuilt[r]}, the decomposition says "
                    f"{list(self.c[r])}")

    def summary(self) -> str:
        naive = self.p * self.q * self.s
        a_adds = sum(len(t) - 1 for t in self.a_terms)
        b_adds = sum(len(t) - 1 for t in self.b_terms)
        if self.has_postsum:
            epi = (f"{self.num_writes} output writes (postsum CSE in {len(self.postsum_chains)} "
                   f"chains, from {self.num_output_writes})")
        else:
            epi = f"{self.num_writes} output writes"
        return (f"{self.name}: {self.p}x{self.q}x{self.s} rank {self.rank}/{naive} "
                f"({self.rank / naive:.4f} FLOPs), A adds {a_adds}, B adds {b_adds}, "
                f"{self.num_staging_passes} epilogue staging passes, {epi}")


def _derive(sch: Scheme) -> dict:
    """All tables the kernels and seams read, from the raw coefficient rows."""
    p, q, s = (max(1, int(x)) for x in (tuple(sch.shape) + (1, 1, 1))[:3])
    rank = len(sch.c)
    t: dict = {}
    t["a_terms"] = _nonzeros(sch.a, q)
    t["b_terms"] = _nonzeros(sch.b, s)
    t["c_terms"] = _nonzeros(sch.c, s)
    t["first_writer"] = _first_writer_of(t["c_terms"])
    t["dest_groups"] = _grouped(t["c_terms"], t["first_writer"])

    acc_clear = tuple(sch.clear) if sch.clear else (1,) * rank
    t["acc_clear"] = acc_clear
    # Chains: walk the steps once, keeping the open chain of each accumulator stage.
    chains: list = []
    open_chain: dict = {}
    for step in range(min(rank, len(acc_clear))):
        stage = step % 2
        if acc_clear[step] or stage not in open_chain:
            open_chain[stage] = []
            chains.append(open_chain[stage])
        open_chain[stage].append(step)
    t["chains"] = tuple(tuple(ch) for ch in chains)
    nxt = [-1] * rank
    for ch in chains:
        for here, there in zip(ch, ch[1:]):
            nxt[here] = there
    t["next"] = tuple(nxt)
    width = p * s
    pubs = []
    for step in range(rank):
        follow = sch.c[nxt[step]] if nxt[step] >= 0 else (0,) * width
        row = sch.c[step]
        pubs.append(tuple(
            Term(n // s, n % s, row[n] - follow[n])
            for n in range(min(width, len(row), len(follow))) if row[n] - follow[n]))
    t["postsum_terms"] = tuple(pubs)
    t["postsum_groups"] = _grouped(t["postsum_terms"], _first_writer_of(t["postsum_terms"]))
    return t


def load(name: str) -> Scheme:
    """Load and validate a scheme by path, file name or stem from ``schemes/``."""
    path = Path(name)
    if not path.exists():
        path = SCHEME_DIR / (name if str(name).endswith(".json") else f"{name}.json")
    if not path.exists():
        raise FileNotFoundError(f"no scheme {name!r} here or in {SCHEME_DIR}")
    raw = json.loads(path.read_text())
    if raw.get("format") != FORMAT:
        raise ValueError(f"{path}: unsupported format {raw.get('format')!r}, expected {FORMAT!r}")
    plan = raw.get("postsum") or {}
    as_rows = lambda m: tuple(tuple(int(v) for v in row) for row in m)
    scheme = Scheme(
        name=path.stem,
        shape=tuple(raw["shape"]),
        rank=int(raw["r"]),
        a=as_rows(raw["A"]),
        b=as_rows(raw["B"]),
        c=as_rows(raw["C"]),
        clear=tuple(int(v) for v in plan.get("clear", ())),
    )
    scheme.validate()
    if scheme.has_postsum:
        # ``clear`` alone always telescopes; what pins the plan that was searched for is the
        # recorded publication table (lcgemm/scheme.py:467-485).
        stated = plan.get("dests")
        if stated is None:
            raise ValueError(
                f"{path}: the chain plan has 'clear' but no 'dests' table, so nothing pins which "
                f"prefix sums the plan was searched for")
        want = tuple(tuple(Term(int(i), int(j), int(v)) for i, j, v in step) for step in stated)
        if want != scheme.postsum_terms:
            bad = next(t for t in range(scheme.rank) if want[t] != scheme.postsum_terms[t])
            raise ValueError(
                f"{path}: the recorded 'dests' table disagrees with the plan re-derived from "
                f"'clear'. Step {bad} is recorded as publishing {list(want[bad])} but the chains "
                f"imply {list(scheme.postsum_terms[bad])}")
    return scheme


if __name__ == "__main__":
    import sys

    for n in sys.argv[1:] or sorted(x.name for x in SCHEME_DIR.glob("*.json")):
        sch = load(n)
        print(sch.summary())
        for r in range(sch.rank):
            flag = ("CLEAR " if sch.clear[r] else "accum ") if sch.has_postsum else ""
            print(f"    r{r}: {flag}A{list(sch.a_terms[r])} B{list(sch.b_terms[r])} "
                  f"-> {list(sch.epi_groups[r])}")
