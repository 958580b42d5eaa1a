"""Long records (lists of hundreds of elements) are walked by a whole warp: parity with the CPU checker on lists that
are well formed, on lists that are not, and on everything in between. Needs a B200 (run with -m gpu)."""
import random

import numpy as np
import pytest

from pj_testlib import abi, as_u8, same_result
from test_gpu_parity import gpu_parse_device, gpu_parse_host

pytestmark = pytest.mark.gpu

PET, MIXED = abi.PJ_SCHEMA_PET, abi.PJ_SCHEMA_MIXED


def url(rng, n):
    return "".join(rng.choice("abcdefghijklmnopqrstuvwxyz0123456789-._~/:") for _ in range(n))


def pet(rng, n_photo, n_tags, *, blanks=False, photo=None, tag=None, extra="", order="ipct"):
    """One Pet with the given list lengths; `photo` / `tag` make element k (text of the element as written)."""
    sp = (lambda: rng.choice(["", " ", "  ", "\t", " \r"])) if blanks else (lambda: "")
    photos = [photo(k) if photo else '"' + url(rng, rng.randint(0, 70)) + '"' for k in range(n_photo)]
    tags = [tag(k) if tag else '{%s"id"%s:%s%d%s,%s"name"%s:%s"%s"%s}' % (sp(), sp(), sp(), rng.randint(0, 1 << 40), sp(), sp(), sp(), sp(), url(rng, rng.randint(0, 12)), sp())
            for k in range(n_tags)]
    parts = {
        "i": '"id":%d' % rng.randint(1, 1 << 60),
        "p": '"photoUrls":%s[%s' % (sp(), sp()) + (sp() + "," + sp()).join(photos) + sp() + "]",
        "c": '"category":{"id":7,"name":"cat"},"name":"n%d"' % rng.randint(0, 999),
        "t": '"tags":%s[%s' % (sp(), sp()) + (sp() + "," + sp()).join(tags) + sp() + "]",
    }
    body = ",".join(parts[k] for k in order)
    return "{" + body + extra + ',"status":"sold"}'


def check(ctx, oracle, schema, lines):
    text = as_u8(("\n".join(lines) + "\n").encode("utf-8", "surrogateescape"))  # \udcXX stands for the raw byte XX
    want = oracle.parse(schema, text)
    assert same_result(want, gpu_parse_device(ctx, schema, text)) == ""
    assert same_result(want, gpu_parse_host(ctx, schema, text)) == ""
    return want


def test_long_lists_of_every_length(ctx, oracle):
    rng = random.Random(11)
    lines = [pet(rng, n, m) for n, m in [(0, 0), (1, 0), (40, 0), (0, 40), (31, 33), (64, 64), (200, 3), (3, 200), (700, 300), (2000, 1)]]
    lines += [pet(rng, rng.randint(0, 120), rng.randint(0, 60), blanks=True) for _ in range(200)]
    want = check(ctx, oracle, PET, lines)
    assert want.n_errors == 0


def test_long_lists_between_short_records(ctx, oracle):
    rng = random.Random(12)
    lines = []
    for k in range(400):
        lines.append(pet(rng, rng.randint(0, 3), rng.randint(0, 2)))
        if k % 7 == 0:
            lines.append(pet(rng, rng.randint(30, 400), rng.randint(0, 90), blanks=k % 2 == 0, order=rng.choice(["ipct", "tpci", "ctpi", "pict"])))
    check(ctx, oracle, PET, lines)


def test_strings_that_need_the_exact_lexer(ctx, oracle):
    rng = random.Random(13)
    specials = ['\\"', "\\\\", "\\\\\\\\", '\\\\\\"', "\\u00e9", "\\ud83d\\ude00", "é", "€", "😀", "\\n\\t", "\\/", "x\\\\"]

    def photo(k):
        s = url(rng, rng.randint(0, 40))
        if k % 3 == 0:
            s += rng.choice(specials) + url(rng, rng.randint(0, 30)) + rng.choice(specials)
        return '"' + s + '"'

    def tag(k):
        return '{"id":%d,"name":"%s%s"}' % (k, url(rng, 5), rng.choice(specials) if k % 2 else "")

    lines = [pet(rng, 150, 80, photo=photo, tag=tag, blanks=bool(j & 1)) for j in range(20)]
    # runs of backslashes of every length around the 32-byte blocks a lane owns
    for run in range(1, 70):
        lines.append(pet(rng, 60, 0, photo=lambda k, run=run: '"' + "a" * (k % 5) + "\\\\" * run + '"'))
    want = check(ctx, oracle, PET, lines)
    assert want.n_errors == 0


def test_lists_that_are_not_well_formed(ctx, oracle):
    """Each record breaks one thing inside a long list; the failure has to be the one the sequential walk names."""
    rng = random.Random(14)
    lines = []

    def broken_photos(n, at, text):
        return lambda k: text if k == at else '"' + url(rng, rng.randint(3, 50)) + '"'

    def broken_tags(n, at, text):
        return lambda k: text if k == at else '{"id":%d,"name":"%s"}' % (k, url(rng, 6))

    bad_strings = ['"abc', '"a\\qb"', '"a\x01b"', '"\\ud800x"', '"\udcff"', '"\udce9x"', "abc", "123", "null", '"a" "b"', '"a",', "", '"a"]', "[1]", '{"x":1}', '"\\u12"']
    for at in (0, 1, 31, 32, 33, 99, 149):
        for b in bad_strings:
            lines.append(pet(rng, 150, 5, photo=broken_photos(150, at, b)))
    bad_tags = ['{"id":1,"name":"x"', '{"id":"x"}', '{"id":1.5}', "null", '"t"', '{"id":1,,"name":"x"}', '{"id":1}{"id":2}', '{"id":1},', "",
                '{"id":1,"zz":{"a":[1,2,{"b":3}]},"name":"y"}', '{"zz":[{"id":1},{"id":2}]}', '{"id":99999999999999999999}', '{"name":"a\\qb"}', '{"id":1]']
    for at in (0, 1, 40, 63, 64, 119):
        for b in bad_tags:
            lines.append(pet(rng, 4, 120, tag=broken_tags(120, at, b)))
    # a list that never closes, a list closed by the wrong bracket, lists given twice (the last one counts)
    good = pet(rng, 100, 50)
    lines.append(good.replace("]", "", 1))
    lines.append(good.replace("]", "}", 1))
    lines.append(pet(rng, 90, 40, extra=',"photoUrls":["again","and again"],"tags":[{"id":1}]'))
    lines.append(pet(rng, 2, 2, extra=',"photoUrls":[' + ",".join('"%s"' % url(rng, 30) for _ in range(120)) + "]"))
    lines.append(pet(rng, 90, 40, extra=',"photoUrls":null,"tags":null'))
    lines.append(pet(rng, 90, 40, extra=',"unknown":[' + ",".join('"%s"' % url(rng, 30) for _ in range(120)) + "]"))
    want = check(ctx, oracle, PET, lines)
    assert want.n_errors > 100


def test_long_records_in_a_mixed_stream(ctx, oracle):
    rng = random.Random(15)
    lines = []
    for k in range(300):
        lines.append('{"id":%d,"petId":%d,"quantity":3,"status":"placed","complete":true}' % (k, k * 7))
        lines.append('{"id":%d,"username":"u%d","email":"%s@example.org","userStatus":1}' % (k, k, url(rng, 8)))
        if k % 5 == 0:
            lines.append(pet(rng, rng.randint(20, 300), rng.randint(0, 80), blanks=k % 2 == 0))
    check(ctx, oracle, MIXED, lines)


def test_a_record_longer_than_a_tile(ctx, oracle):
    """Lists that make one record larger than the staged window: the warp reads it where it lies."""
    rng = random.Random(16)
    lines = [pet(rng, 3, 1), pet(rng, 4000, 900), pet(rng, 2, 2), pet(rng, 1, 3000, blanks=True), pet(rng, 5, 0)]
    lines.append(pet(rng, 3000, 10, photo=lambda k: '"abc' if k == 2900 else '"' + url(rng, 30) + '"'))
    lines.append(pet(rng, 3, 1))
    check(ctx, oracle, PET, lines)
