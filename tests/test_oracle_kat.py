"""The CPU checker against the hand-written known-answer cases (tests/golden/kat_cases.py) and, when a
maintainer of the reference project has produced it with tests/golden/EmitGolden.java, against
tests/golden/java_golden.jsonl: what Micronaut Serde itself answers for the same inputs."""
import base64
import json
import os

import numpy as np
import pytest

from golden.kat_cases import CASES, HEX_LOWER, OPTION_CASES
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


@pytest.mark.parametrize("case", OPTION_CASES, ids=[c[0] for c in OPTION_CASES])
def test_option_kat(oracle, case):
    """The other answer of a rule (pj_options.flags), and the default answer for the same input: a failure."""
    name, schema, opts, data, expected = case
    check_case(lambda sch, buf, fr: oracle.parse(sch, buf, fr, opts=opts), name, schema, "ndjson", data, expected)
    default = oracle.parse(SCHEMA_BY_NAME[schema], as_u8(data))
    assert default.n_errors >= sum(1 for e in expected if isinstance(e, tuple)), name


def test_hex_case_of_the_writer(oracle):
    cols = oracle.parse(1, as_u8(b'{"name":"a\\u001fb\\u000b\\n","photoUrls":[]}\n'))
    assert bytes(oracle.write(1, cols)) == b'{"name":"a\\u001Fb\\u000B\\n"}\n'
    assert bytes(oracle.write(1, cols, opts=HEX_LOWER)) == b'{"name":"a\\u001fb\\u000b\\n"}\n'


def test_case_names_unique():
    names = [c[0] for c in CASES]
    assert len(names) == len(set(names))
    assert len(CASES) > 150


# ---- vectors from the real library -----------------------------------------------------------------------
JAVA_GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "java_golden.jsonl")


def ndjson_lines(data: bytes):
    """The records of an NDJSON input as EmitGolden.java cuts them: LF-delimited, blank lines skipped."""
    return [ln for ln in data.split(b"\n") if ln.strip(b" \t\r")]


def check_against_java(oracle, golden_lines, inclusion=abi.PJ_INCLUDE_NON_EMPTY):
    """Compares the checker with the emitter's answers; returns a list of disagreements (empty = pinned).
    Per record: accepted or not, and for accepted records the re-serialised bytes. Kind and offset of a failure
    are compared only where the Java side reports a byte offset (Jackson's own parse failures)."""
    by_name = {c[0]: c for c in CASES}
    bad = []
    for ln in golden_lines:
        g = json.loads(ln)
        if g.get("unknown_enum", "throws") != "throws" or g["framing"] != "ndjson" or g["name"] not in by_name:
            continue
        _, schema, _, data, _ = by_name[g["name"]]
        sch = SCHEMA_BY_NAME[schema]
        recs = ndjson_lines(bytes(data))
        if len(recs) != len(g["records"]):
            bad.append((g["name"], "record count", len(recs), len(g["records"])))
            continue
        for k, (rec, jr) in enumerate(zip(recs, g["records"])):
            cols = oracle.parse(sch, as_u8(rec + b"\n"))
            ok = cols.n_records == 1 and cols.n_errors == 0
            if ok != bool(jr["ok"]):
                bad.append((g["name"], k, "accepted" if ok else "rejected", "java: " + ("accepted" if jr["ok"] else jr.get("exception", "rejected"))))
                continue
            if ok:
                mine = bytes(oracle.write(sch, cols, 0, inclusion)).rstrip(b"\n")
                theirs = base64.b64decode(jr["rewritten_b64"])
                if mine != theirs:
                    bad.append((g["name"], k, mine, theirs))
            elif "byte_offset" in jr and int(cols.get("err_off")[0]) != int(jr["byte_offset"]):
                bad.append((g["name"], k, "offset", int(cols.get("err_off")[0]), int(jr["byte_offset"])))
    return bad


@pytest.mark.skipif(not os.path.exists(JAVA_GOLDEN), reason="tests/golden/java_golden.jsonl has not been produced (needs a JVM: see EmitGolden.java)")
def test_checker_against_micronaut_serde(oracle):
    with open(JAVA_GOLDEN) as f:
        bad = check_against_java(oracle, [ln for ln in f if ln.strip()])
    assert not bad, bad[:10]


def test_java_golden_loader_on_a_self_made_file(oracle):
    """The loader itself, exercised on answers the checker produced in the emitter's format (and on one
    falsified answer, which it must report)."""
    from golden.export_kat_inputs import lines as kat_lines

    out = []
    for ln in kat_lines():
        c = json.loads(ln)
        if c["framing"] != "ndjson" or c["schema"] == "mixed":
            continue
        data = base64.b64decode(c["input_b64"])
        sch = SCHEMA_BY_NAME[c["schema"]]
        recs = []
        for rec in ndjson_lines(data):
            cols = oracle.parse(sch, as_u8(rec + b"\n"))
            if cols.n_records == 1 and cols.n_errors == 0:
                recs.append({"ok": True, "rewritten_b64": base64.b64encode(bytes(oracle.write(sch, cols, 0, abi.PJ_INCLUDE_NON_EMPTY)).rstrip(b"\n")).decode()})
            else:
                recs.append({"ok": False, "exception": "x", "message": "y"})
        out.append(json.dumps({"name": c["name"], "schema": c["schema"], "framing": "ndjson", "unknown_enum": "throws", "records": recs}))
    assert len(out) > 100
    assert check_against_java(oracle, out) == []
    g = json.loads(out[1])
    g["records"][0]["ok"] = not g["records"][0]["ok"]
    assert check_against_java(oracle, [json.dumps(g)]) != []
