"""The CPU checker triangulated against independent implementations that are not the reference either:
the seeded generator's own record of what it wrote, Python's json, msgspec and jsonschema (Draft 4,
the dialect of Swagger 2.0 definitions)."""
import json
import random
from datetime import datetime

import jsonschema
import msgspec
import numpy as np
import pytest

from pj_testlib import abi, as_u8, pj, records, same_result

SEED = 0x5EED
FLAG_SETS = [0, abi.PJ_GEN_ESCAPES, abi.PJ_GEN_WHITESPACE, abi.PJ_GEN_MALFORMED, abi.PJ_GEN_SPARSE,
             abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_MALFORMED | abi.PJ_GEN_SPARSE,
             abi.PJ_GEN_ZIPF_LISTS | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE,
             abi.PJ_GEN_ARRAY, abi.PJ_GEN_ARRAY | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_MALFORMED | abi.PJ_GEN_SPARSE]


@pytest.mark.parametrize("schema", [1, 2, 3, 4])
@pytest.mark.parametrize("flags", FLAG_SETS)
def test_generator_values_equal_checker_parse(oracle, native, schema, flags):
    n = 400
    text = pj.gen_text(schema, SEED, 0, n, flags)
    want = pj.gen_columns(schema, SEED, 0, n, flags, text.size)
    got = oracle.parse(schema, text, abi.PJ_FRAMING_ARRAY if flags & abi.PJ_GEN_ARRAY else abi.PJ_FRAMING_NDJSON)
    assert same_result(want, got) == ""
    if flags & abi.PJ_GEN_MALFORMED:
        assert got.n_errors > 0


def test_generator_is_shardable(native):
    a = pj.gen_text(4, 7, 0, 300, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ESCAPES)
    b = np.concatenate([pj.gen_text(4, 7, 0, 100, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ESCAPES),
                        pj.gen_text(4, 7, 100, 200, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ESCAPES)])
    assert np.array_equal(a, b)


def test_generator_distributions(native):
    """The first benchmark configuration: ids in [1, 2^62], name 4-16 letters, 0-4 photoUrls of 20-60, 0-3 tags."""
    n = 3000
    text = pj.gen_text(1, SEED, 0, n, 0)
    lens = []
    for line in bytes(text).split(b"\n")[:-1]:
        d = json.loads(line)
        lens.append(len(line) + 1)
        assert list(d) == ["id", "category", "name", "photoUrls", "tags", "status"]
        assert 1 <= d["id"] <= 2**62 and 1 <= d["category"]["id"] <= 2**62
        assert 4 <= len(d["name"]) <= 16 and d["name"].isalpha()
        assert 3 <= len(d["category"]["name"]) <= 12
        assert 0 <= len(d["photoUrls"]) <= 4 and all(20 <= len(u) <= 60 for u in d["photoUrls"])
        assert 0 <= len(d["tags"]) <= 3 and all(3 <= len(t["name"]) <= 10 for t in d["tags"])
        assert d["status"] in ("available", "pending", "sold")
    assert 250 < np.mean(lens) < 340


# ---- Python json ---------------------------------------------------------------------------------
def _strip_nulls(x):
    if isinstance(x, dict):
        return {k: _strip_nulls(v) for k, v in x.items() if v is not None}
    if isinstance(x, list):
        return [_strip_nulls(v) for v in x]
    return x


def _ship(text):
    dt = datetime.fromisoformat(text)
    frac = text.split(".")[1] if "." in text else ""
    stop = next((i for i, ch in enumerate(frac) if not ch.isdigit()), len(frac))
    digits = frac[:stop]
    nanos = int(digits.ljust(9, "0")) if digits else 0
    off = int(dt.utcoffset().total_seconds())
    return (int(dt.replace(microsecond=0).timestamp()), nanos, off)


KNOWN = {1: {"id", "category", "name", "photoUrls", "tags", "status"},
         2: {"id", "petId", "quantity", "shipDate", "status", "complete"},
         3: {"id", "username", "firstName", "lastName", "email", "password", "phone", "userStatus"}}


def test_long_lists_decode_like_python_json(oracle, native):
    """The checker on the records the warp path of the GPU library is tested with (lists of hundreds of elements, blanks,
    escapes and bytes beyond ASCII in the elements): every decoded value against Python's json."""
    import random

    from test_gpu_wide import pet, url

    rng = random.Random(17)
    specials = ['\\"', "\\\\", "\\u00e9", "\\ud83d\\ude00", "é", "€", "😀", "\\n\\t", "\\/"]
    photo = lambda k: '"' + url(rng, rng.randint(0, 40)) + (rng.choice(specials) if k % 3 == 0 else "") + '"'
    tag = lambda k: '{"id":%d,"name":"%s%s"}' % (k, url(rng, 5), rng.choice(specials) if k % 2 else "")
    lines = [pet(rng, n, m, blanks=b) for n, m, b in [(0, 0, False), (300, 0, False), (0, 200, True), (700, 300, True), (64, 64, False)]]
    lines += [pet(rng, 150, 80, photo=photo, tag=tag, blanks=bool(j & 1)) for j in range(6)]
    text = as_u8(("\n".join(lines) + "\n").encode())
    parsed = oracle.parse(1, text)
    assert parsed.n_errors == 0
    got = records(parsed.as_dict(), 1)
    assert len(got) == len(lines)
    for line, rec in zip(lines, got):
        assert rec == _strip_nulls(json.loads(line))


@pytest.mark.parametrize("schema", [1, 2, 3])
@pytest.mark.parametrize("flags", [0, abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_SPARSE, abi.PJ_GEN_ZIPF_LISTS | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE])
def test_decoded_values_equal_python_json(oracle, native, schema, flags):
    text = pj.gen_text(schema, 99, 0, 500, flags)
    got = records(oracle.parse(schema, text).as_dict(), schema)
    lines = bytes(text).split(b"\n")[:-1]
    assert len(got) == len(lines)
    for line, rec in zip(lines, got):
        want = _strip_nulls(json.loads(line))
        if "shipDate" in want:
            want["shipDate"] = _ship(want["shipDate"])
        assert rec == want


INTERESTING = [b'"', b"\\", b"{", b"}", b"[", b"]", b",", b":", b" ", b"\t", b"\x00", b"\x1f", b"\x7f", b"\x80", b"\xc0", b"\xe0\x80",
               b"\xed\xa0\x80", b"\xf4\x90", b"\xff", b"null", b"true", b"false", b"tru", b"-", b"0", b"01", b"1.5", b"1e5", b"-0", b"1.",
               b"9223372036854775808", b"\\u0041", b"\\ud83d\\ude00", b"\\u00", b"\\x", b"//c", b"/*c*/", b"'", b'"id"', b'"name"',
               b'"x":{"a":[1,{"b":null}],"c":"d"},', b"[" * 70, b"NaN", b"Infinity"]


def mutate(rng, rec: bytes) -> bytes:
    b = bytearray(rec)
    for _ in range(rng.choice([1, 1, 2, 3])):
        if not b:
            break
        op = rng.randrange(5)
        pos = rng.randrange(len(b) + 1)
        if op == 0 and pos < len(b):
            b[pos] = rng.randrange(256)
        elif op == 1 and pos < len(b):
            del b[pos:pos + rng.choice([1, 2, 5, 20])]
        elif op == 2:
            b[pos:pos] = rng.choice(INTERESTING)
        elif op == 3 and pos < len(b):
            b[pos:pos + 1] = rng.choice(INTERESTING)
        else:
            b = b[:pos]
    return bytes(b).replace(b"\n", b" ")


def _reject_constant(name):
    raise ValueError(name)


LEXICAL = {"SYNTAX", "EOF", "CTRL_CHAR", "BAD_ESCAPE", "UTF8"}


def _mutated_corpus(schema, seed, n):
    rng = random.Random(seed)
    lines = bytes(pj.gen_text(schema, seed, 0, n, abi.PJ_GEN_ESCAPES)).split(b"\n")[:-1]
    return [ln if rng.random() < 0.2 else mutate(rng, ln) for ln in lines]


@pytest.mark.parametrize("schema", [1, 2, 3])
def test_syntax_verdicts_agree_with_python_json(oracle, native, schema):
    lines = [ln for ln in _mutated_corpus(schema, 1234 + schema, 1500) if ln.strip(b" \t\r")]
    got = records(oracle.parse(schema, as_u8(b"\n".join(lines) + b"\n")).as_dict(), schema)
    assert len(got) == len(lines)
    seen = set()
    for line, rec in zip(lines, got):
        try:
            val = json.loads(line.decode("utf-8"), parse_constant=_reject_constant)
            py_ok = True
        except (ValueError, RecursionError):
            py_ok, val = False, None
        if isinstance(rec, dict):
            assert py_ok and isinstance(val, dict), line
            seen.add("NONE")
        else:
            seen.add(rec[0])
            if not py_ok:
                continue  # both reject
            # Python accepted: the checker's complaint must be one Python does not make
            assert rec[0] not in LEXICAL, (line, rec)
    assert {"NONE", "SYNTAX", "EOF", "TYPE"} <= seen


# ---- msgspec: typed decode ------------------------------------------------------------------------
class Category(msgspec.Struct):
    id: int | None = None
    name: str | None = None


class Tag(msgspec.Struct):
    id: int | None = None
    name: str | None = None


class Pet(msgspec.Struct):
    name: str
    photoUrls: list[str]
    id: int | None = None
    category: Category | None = None
    tags: list[Tag] | None = None
    status: str | None = None


def test_accepted_pets_decode_with_msgspec(oracle, native):
    lines = [ln for ln in _mutated_corpus(1, 4321, 1500) if ln.strip(b" \t\r")]
    got = records(oracle.parse(1, as_u8(b"\n".join(lines) + b"\n")).as_dict(), 1)
    n_ok = 0
    for line, rec in zip(lines, got):
        if not isinstance(rec, dict):
            continue
        pet = msgspec.json.decode(line, type=Pet, strict=True)
        n_ok += 1
        assert pet.name == rec["name"] and pet.photoUrls == rec["photoUrls"]
        assert pet.id == rec.get("id") and pet.status == rec.get("status")
        if "tags" in rec:
            assert [(t.id, t.name) for t in pet.tags] == [(t.get("id"), t.get("name")) for t in rec["tags"]]
    assert n_ok > 200


@pytest.mark.parametrize("text,kind,needle", [
    (b'{"photoUrls":[]}', "REQUIRED", "missing required field"),
    (b'{"name":1,"photoUrls":[]}', "TYPE", "Expected `str`, got `int`"),
    (b'{"name":"a","photoUrls":[1]}', "TYPE", "Expected `str`, got `int`"),
    (b'{"name":"a","photoUrls":[],"id":"7"}', "TYPE", "Expected `int | null`, got `str`"),
    (b'{"name":"a","photoUrls":[],"id":1.5}', "TYPE", "Expected `int | null`, got `float`"),
    (b'{"name":"a","photoUrls":[],"tags":[3]}', "TYPE", "Expected `object`, got `int`"),
])
def test_typed_rejections_match_msgspec(oracle, text, kind, needle):
    rec = records(oracle.parse(1, as_u8(text + b"\n")).as_dict(), 1)[0]
    assert rec[0] == kind
    with pytest.raises(msgspec.ValidationError) as e:
        msgspec.json.decode(text, type=Pet, strict=True)
    assert needle in str(e.value)


# ---- jsonschema: the Swagger 2.0 definitions restated from petstore.json:823-972 ----------------
DEFS = {
    "Category": {"type": "object", "properties": {"id": {"type": "integer"}, "name": {"type": "string"}}},
    "Tag": {"type": "object", "properties": {"id": {"type": "integer"}, "name": {"type": "string"}}},
    "Pet": {"type": "object", "required": ["name", "photoUrls"],
            "properties": {"id": {"type": "integer"}, "category": {"$ref": "#/definitions/Category"}, "name": {"type": "string"},
                           "photoUrls": {"type": "array", "items": {"type": "string"}},
                           "tags": {"type": "array", "items": {"$ref": "#/definitions/Tag"}},
                           "status": {"type": "string", "enum": ["available", "pending", "sold"]}}},
    "Order": {"type": "object",
              "properties": {"id": {"type": "integer"}, "petId": {"type": "integer"}, "quantity": {"type": "integer"},
                             "shipDate": {"type": "string"}, "status": {"type": "string", "enum": ["placed", "approved", "delivered"]},
                             "complete": {"type": "boolean"}}},
    "User": {"type": "object",
             "properties": {k: {"type": "string"} for k in ["username", "firstName", "lastName", "email", "password", "phone"]}
             | {"id": {"type": "integer"}, "userStatus": {"type": "integer"}}},
}


def _has_null_or_big(x):
    if x is None:
        return True
    if isinstance(x, bool):
        return False
    if isinstance(x, int):
        return not -(2**63) <= x < 2**63
    if isinstance(x, dict):
        return any(_has_null_or_big(v) for v in x.values())
    if isinstance(x, list):
        return any(_has_null_or_big(v) for v in x)
    return False


@pytest.mark.parametrize("schema,model", [(1, "Pet"), (2, "Order"), (3, "User")])
def test_schema_verdicts_agree_with_jsonschema(oracle, native, schema, model):
    validator = jsonschema.Draft4Validator({"$ref": f"#/definitions/{model}", "definitions": DEFS})
    rng = random.Random(schema)
    swaps = [b"1", b'"x"', b"true", b"[]", b"{}", b'"sold"', b'"placed"', b"[1]", b'["a"]', b"1.5", b'[{"id":"q"}]']
    lines = []
    for ln in bytes(pj.gen_text(schema, 555, 0, 1200, 0)).split(b"\n")[:-1]:
        d = json.loads(ln)
        for _ in range(rng.choice([0, 1, 1, 2])):
            k = rng.choice(sorted(KNOWN[schema]))
            if rng.random() < 0.3:
                d.pop(k, None)
            else:
                d[k] = json.loads(rng.choice(swaps))
        lines.append(json.dumps(d, separators=(",", ":")).encode())
    got = records(oracle.parse(schema, as_u8(b"\n".join(lines) + b"\n")).as_dict(), schema)
    checked = rejected = 0
    for line, rec in zip(lines, got):
        d = json.loads(line)
        if _has_null_or_big(d):
            continue
        if not isinstance(rec, dict) and rec[0] == "DATETIME":
            continue  # jsonschema does not check formats
        checked += 1
        ok = validator.is_valid(d)
        assert ok == isinstance(rec, dict), (line, rec)
        if not ok:
            rejected += 1
            assert rec[0] in ("TYPE", "ENUM", "REQUIRED"), (line, rec)
    assert checked > 300 and rejected > 100
