"""Scheme layer: the tables the kernels consume, against the reference's own
(tests/golden/scheme_tables.json, generated from the reference), and the validation
behaviour the reference tests (tests/test_policy.py:11-19 there)."""
import dataclasses
import json

import pytest

from conftest import GOLDEN
from lcgemm import scheme as S

NAMES = ("2x2_postsum_cse", "2x2_locality_ordered")


def _groups(table):
    return [[[g.coeff, [[d.row, d.col, bool(d.is_first)] for d in g.dests]] for g in step]
            for step in table]


@pytest.mark.parametrize("name", NAMES)
def test_tables_match_reference(name):
    want = json.loads((GOLDEN / "scheme_tables.json").read_text())[name]
    s = S.load(name)
    assert list(s.shape) == want["shape"] and s.rank == want["rank"]
    assert s.has_postsum == want["has_postsum"]
    for key in ("a_terms", "b_terms", "c_terms", "postsum_terms"):
        assert [[list(t) for t in step] for step in getattr(s, key)] == want[key], key
    assert list(s.acc_clear) == want["acc_clear"]
    assert [list(c) for c in s.postsum_chains] == want["postsum_chains"]
    assert list(s.postsum_next) == want["postsum_next"]
    assert _groups(s.epi_groups) == want["epi_groups"]
    assert _groups(s.dest_groups) == want["dest_groups"]
    assert (s.num_writes, s.num_staging_passes, s.num_output_writes) == (
        want["num_writes"], want["num_staging_passes"], want["num_output_writes"])
    assert s.summary() == want["summary"]


def test_scheme_files_are_self_contained_and_validated():
    gate, down = S.load("2x2_postsum_cse"), S.load("2x2_locality_ordered")
    assert gate.shape == down.shape == (2, 2, 2)
    assert gate.rank == down.rank == 7
    assert gate.has_postsum and not down.has_postsum
    assert gate.postsum_chains == ((0, 2, 4, 6), (1,), (3, 5))
    assert gate.num_writes == 7 and down.num_writes == 12


def test_load_by_filename_and_missing():
    assert S.load("2x2_postsum_cse.json").name == "2x2_postsum_cse"
    with pytest.raises(FileNotFoundError):
        S.load("no_such_scheme")


def _mutated(s, **kw):
    return dataclasses.replace(s, **kw)


@pytest.mark.parametrize("name", NAMES)
def test_identity_catches_a_flipped_coefficient(name):
    s = S.load(name)
    for table in ("a", "b", "c"):
        rows = [list(r) for r in getattr(s, table)]
        rows[3][1] = rows[3][1] + 1
        bad = _mutated(s, **{table: tuple(tuple(r) for r in rows)})
        with pytest.raises(ValueError, match="not a decomposition"):
            bad.validate()


def test_shape_and_plan_wellformedness():
    s = S.load("2x2_postsum_cse")
    with pytest.raises(ValueError, match="all-zero"):
        _mutated(s, a=((0, 0, 0, 0),) + s.a[1:]).validate()
    with pytest.raises(ValueError, match="rows"):
        _mutated(s, b=s.b[:-1]).validate()
    with pytest.raises(ValueError, match="step flags"):
        _mutated(s, clear=(1, 1, 0)).validate()
    with pytest.raises(ValueError, match="0/1"):
        _mutated(s, clear=(1, 1, 2, 1, 0, 0, 0)).validate()
    with pytest.raises(ValueError, match="continues a chain"):
        _mutated(s, clear=(1, 0, 0, 1, 0, 0, 0)).validate()
    with pytest.raises(ValueError, match="block grid"):
        _mutated(s, shape=(2, 2)).validate()


def test_any_wellformed_clear_telescopes():
    """A different chain plan is costlier, never wrong (lcgemm/scheme.py:363-376 there)."""
    s = S.load("2x2_postsum_cse")
    for clear in ((1,) * 7, (1, 1, 0, 0, 0, 0, 0), (1, 1, 1, 0, 1, 0, 1)):
        alt = _mutated(s, clear=clear)
        alt.validate()
        assert alt.num_writes >= s.num_writes


def test_recorded_dests_pin_the_plan(tmp_path):
    raw = json.loads((S.SCHEME_DIR / "2x2_postsum_cse.json").read_text())
    raw["postsum"]["clear"] = [1, 1, 1, 1, 0, 0, 0]
    p = tmp_path / "tampered.json"
    p.write_text(json.dumps(raw))
    with pytest.raises(ValueError, match="disagrees"):
        S.load(str(p))
    del raw["postsum"]["dests"]
    p.write_text(json.dumps(raw))
    with pytest.raises(ValueError, match="no 'dests'"):
        S.load(str(p))
    raw["format"] = "something-else"
    p.write_text(json.dumps(raw))
    with pytest.raises(ValueError, match="unsupported format"):
        S.load(str(p))


def test_term_reprs_are_plain_tuples():
    assert repr(S.Term(1, 0, -1)) == "(1, 0, -1)"
    assert repr(S.Dest(0, 1, True)) == "(0, 1, True)"
    assert repr(S.Group(1, (S.Dest(0, 0, False),))) == "(1, ((0, 0, False),))"
