"""The CPU checker against the hand-written known-answer cases (tests/golden/kat_cases.py)."""
import numpy as np
import pytest

from golden.kat_cases import CASES
from pj_testlib import KIND_BY_NAME, SCHEMA_BY_NAME, abi, as_u8, records


def expected_split(expected):
    doc = (0, 0)
    recs = []
    for e in expected:
        if isinstance(e, dict) and "doc" in e:
            doc = (KIND_BY_NAME[e["doc"][0]], e["doc"][1])
        else:
            recs.append(e)
    return recs, doc


def check_case(parse, name, schema, framing, data, expected):
    sch = SCHEMA_BY_NAME[schema]
    fr = abi.PJ_FRAMING_ARRAY if framing == "array" else abi.PJ_FRAMING_NDJSON
    cols = parse(sch, as_u8(data), fr)
    got = records(cols.as_dict(), sch)
    want, doc = expected_split(expected)
    assert got == want, name
    assert (int(cols.raw.doc_err_kind), int(cols.raw.doc_err_off)) == doc, name
    n_err = sum(1 for e in want if isinstance(e, tuple))
    assert cols.n_records == len(want) and cols.n_errors == n_err, name
    # rec_start: NDJSON extents begin at line starts
    if fr == abi.PJ_FRAMING_NDJSON and len(want):
        rs = cols.get("rec_start")
        for s in rs:
            assert s == 0 or data[int(s) - 1] == 0x0A, name


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_kat(oracle, case):
    check_case(lambda sch, buf, fr: oracle.parse(sch, buf, fr), *case)


def test_case_names_unique():
    names = [c[0] for c in CASES]
    assert len(names) == len(set(names))
    assert len(CASES) > 150
