"""The device-side parsers and writers, compiled for the host and fuzzed against the CPU checker (no GPU needed).

tests/host_emu/pj_host_emu.cpp includes the library's host+device headers and runs them one "thread" after
another; what is compared is bit-exact: every column, error kind and offset, and the re-serialised bytes.
"""
import ctypes as C
import os
import random
import re
import subprocess
import sys

import numpy as np
import pytest

from pj_testlib import abi, as_u8, nrec_bound, pj, same_result
from test_oracle_crosscheck import mutate

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "host_emu", "pj_host_emu.cpp")
LIB = os.path.join(HERE, "host_emu", "libpj_host_emu.so")
u32, u64 = C.c_uint32, C.c_uint64
NDJSON, ARRAY = abi.PJ_FRAMING_NDJSON, abi.PJ_FRAMING_ARRAY
G = abi  # generator flags live in the abi module


@pytest.fixture(scope="session")
def emu(native):  # `native` builds libpetjson.so, whose generator the tests use
    csrc = os.path.join(ROOT, "micronaut3-bug_b200", "csrc")
    deps = [SRC] + [os.path.join(csrc, f) for f in os.listdir(csrc) if f.endswith((".cuh", ".h"))]
    # PJ_EMU_SANITIZE=1 (set by test_device_code_under_sanitizers for its child process): the same sources with
    # AddressSanitizer and UndefinedBehaviorSanitizer, every finding fatal
    san = os.environ.get("PJ_EMU_SANITIZE") == "1"
    lib = LIB.replace(".so", "_san.so") if san else LIB
    flags = ["-O1", "-g", "-fsanitize=address,undefined", "-fno-sanitize-recover=all"] if san else ["-O2"]
    if not os.path.exists(lib) or any(os.path.getmtime(d) > os.path.getmtime(lib) for d in deps):
        subprocess.run(["g++", *flags, "-std=c++17", "-fPIC", "-shared", "-I", os.path.join(ROOT, "include"), "-I", csrc,
                        "-x", "c++", SRC, "-o", lib], check=True)
    return C.CDLL(lib)


def garbage_columns(schema, n, nbytes):
    """Buffers pre-filled with 0xA5, so a column the code forgets to write shows up."""
    return abi.HostColumns(schema, abi.default_caps(schema, n, nbytes), alloc=lambda nb: np.full(nb, 0xA5, np.uint8))


def extents(oracle, buf):
    cap = nrec_bound(buf)
    s, e, b, n = np.zeros(cap, np.uint64), np.zeros(cap, np.uint64), np.zeros(cap, np.uint8), u64()
    st = oracle.lib.pjo_extents(u32(ARRAY), C.c_void_p(buf.ctypes.data), u64(buf.size), C.c_void_p(s.ctypes.data), C.c_void_p(e.ctypes.data),
                                C.c_void_p(b.ctypes.data), u64(cap), C.byref(n), None, None)
    assert st == 0
    return s[:n.value], e[:n.value], b[:n.value]


def emu_parse_tiles(emu, oracle, schema, buf, framing=NDJSON, tile=128, win=45056, tape=20, lock=False, opts=0):
    """The tile kernel's per-record work on the host: windows of `win` bytes, tapes of `tape` words, `tile` records a tile.
    lock: the lockstep tokeniser (pj_lock.cuh) gets the first try at every staged NDJSON record, as in the stream kernel."""
    emu.emu_use_lock(1 if lock else 0)
    emu.emu_set_options(u32(opts))
    buf = as_u8(buf)
    hc = garbage_columns(schema, nrec_bound(buf), buf.size)
    if framing == ARRAY:
        s, e, b = extents(oracle, buf)
    else:
        s = e = np.zeros(1, np.uint64)
        b = np.zeros(1, np.uint8)
    nfast = u64()
    pad = np.concatenate([buf, np.zeros(64, np.uint8)])  # the code looks 16 bytes ahead
    st = emu.emu_parse_fast(u32(schema), u32(framing), C.c_void_p(pad.ctypes.data), u64(buf.size), u64(0), 1, 1, u64(0), C.byref(hc.raw),
                            C.byref(nfast), u32(tile), u32(win), u32(tape), C.c_void_p(s.ctypes.data), C.c_void_p(e.ctypes.data),
                            C.c_void_p(b.ctypes.data), u64(len(s) if framing == ARRAY else 0))
    assert st == 0, st
    return hc, nfast.value


def emu_write(emu, fn, schema, cols, framing, inclusion, cap):
    out, ln = np.zeros(cap, np.uint8), u64()
    st = getattr(emu, fn)(u32(schema), u32(framing), inclusion, C.byref(cols.raw), C.c_void_p(out.ctypes.data), u64(cap), C.byref(ln))
    assert st == 0, st
    return out[: ln.value]


ALL = G.PJ_GEN_ESCAPES | G.PJ_GEN_WHITESPACE | G.PJ_GEN_MALFORMED | G.PJ_GEN_SPARSE
FLAG_SETS = [0, G.PJ_GEN_ESCAPES, G.PJ_GEN_WHITESPACE, G.PJ_GEN_MALFORMED, G.PJ_GEN_SPARSE, ALL, G.PJ_GEN_ZIPF_LISTS | ALL]
SHAPES = [(128, 45056, 20), (16, 45056, 8), (128, 2048, 20), (7, 45056, 8)]


@pytest.mark.parametrize("schema", [1, 2, 3, 4])
@pytest.mark.parametrize("flags", FLAG_SETS)
@pytest.mark.parametrize("lock", [False, True])
def test_tile_code_matches_checker_on_generated_text(emu, oracle, schema, flags, lock):
    emu.emu_lock_accepted.restype = C.c_uint64
    text = pj.gen_text(schema, 0xE11, 0, 700, flags)
    want = oracle.parse(schema, text)
    for tile, win, tape in SHAPES:
        got, nfast = emu_parse_tiles(emu, oracle, schema, text, NDJSON, tile, win, tape, lock)
        assert same_result(want, got) == "", (tile, win, tape)
        if flags == 0:
            assert nfast >= want.n_records - 1  # everything but, at most, the record at the very end of the input
            if lock and win > 4096:
                assert emu.emu_lock_accepted() >= want.n_records - 1  # the canonical spelling never needs the second try
        if lock and flags == G.PJ_GEN_SPARSE and win > 4096:
            assert emu.emu_lock_accepted() > want.n_records // 20  # records that only omit properties stay on it


def test_common_failures_are_found_by_the_word_path(emu, oracle):
    """Wrong type, unknown literal, missing required property, record ending in a string: same kind and offset as the checker."""
    emu.emu_fail_fast_count.restype = C.c_uint64
    emu.emu_lock_failed.restype = C.c_uint64
    before = emu.emu_fail_fast_count()
    nerr = nlock = 0
    for schema in (1, 2, 3, 4):
        text = pj.gen_text(schema, 99, 0, 3000, G.PJ_GEN_MALFORMED)
        want = oracle.parse(schema, text)
        got, _ = emu_parse_tiles(emu, oracle, schema, text)
        assert same_result(want, got) == ""
        nerr += want.n_errors
        got, _ = emu_parse_tiles(emu, oracle, schema, text, lock=True)  # the lockstep tokeniser reports them itself
        assert same_result(want, got) == ""
        nlock += emu.emu_lock_failed()
    assert nerr > 60 and emu.emu_fail_fast_count() - before >= nerr * 9 // 10
    assert nlock >= nerr * 9 // 10


@pytest.mark.parametrize("seed", [1, 2, 3])
def test_tile_code_matches_checker_on_mutated_text(emu, oracle, seed):
    rng = random.Random(seed)
    for it in range(60):
        schema = rng.choice([1, 1, 2, 3, 4, 4])
        flags = rng.choice(FLAG_SETS)
        lines = bytes(pj.gen_text(schema, rng.randrange(1 << 30), rng.randrange(1000), 40, flags)).split(b"\n")[:-1]
        out = []
        for ln in lines:
            out.append(ln if rng.random() < 0.2 else mutate(rng, ln))
            if rng.random() < 0.05:
                out.append(rng.choice([b"", b"  ", b"\r", b"\t \r"]))
        body = as_u8(b"\n".join(out) + (b"\n" if rng.random() < 0.8 else b""))
        if body.size == 0:
            continue
        want = oracle.parse(schema, body)
        tile, win, tape = rng.choice(SHAPES)
        for lock in (False, True):
            got, _ = emu_parse_tiles(emu, oracle, schema, body, NDJSON, tile, win, tape, lock)
            assert same_result(want, got) == "", (seed, it, schema, flags, tile, win, tape, lock)
        # whatever parsed goes back to text through both writers
        for incl in (abi.PJ_INCLUDE_NON_EMPTY, abi.PJ_INCLUDE_NON_NULL, abi.PJ_INCLUDE_ALWAYS):
            text = oracle.write(schema, want, NDJSON, incl)
            for fn in ("emu_write", "emu_write_fast"):
                assert np.array_equal(text, emu_write(emu, fn, schema, want, NDJSON, incl, body.size * 8 + 128)), (fn, seed, it)


def test_tile_code_on_array_framing(emu, oracle):
    rng = random.Random(5)
    for it in range(40):
        schema = rng.choice([1, 2, 3, 4])
        flags = G.PJ_GEN_ARRAY | rng.choice([0, G.PJ_GEN_WHITESPACE | G.PJ_GEN_ESCAPES, ALL])
        body = as_u8(pj.gen_text(schema, rng.randrange(1 << 30), 0, 50, flags))
        want = oracle.parse(schema, body, ARRAY)
        tile, win, tape = rng.choice(SHAPES)
        got, _ = emu_parse_tiles(emu, oracle, schema, body, ARRAY, tile, win, tape)
        assert same_result(want, got) == "", (it, schema, flags)


def test_integer_text_at_every_digit_count(emu, oracle):
    """The writer's 8-digit groups: powers of ten, their neighbours, both signs, both widths."""
    vals = [0, 1, -1, 9223372036854775807, -9223372036854775808]
    for d in range(1, 19):
        vals += [10 ** d - 1, 10 ** d, 10 ** d + 1, -(10 ** d - 1), -(10 ** d), 10 ** d * 7 + 12345 % 10 ** d]
    recs = [b'{"id":%d,"category":{"id":%d,"name":"c\\u0001\\"x\\\\y\\n"},"name":"n","photoUrls":["a\\tb","plain-0123456789","\\u00e9\\u20ac\\ud83d\\ude00z"],'
            b'"tags":[{"id":%d,"name":"t"},{"id":%d}],"status":"sold"}' % (v, -v if v > -2 ** 63 else v, v, v // 7) for v in vals]
    orders = [b'{"id":%d,"petId":%d,"quantity":%d,"shipDate":"20%02d-02-28T23:59:59.%03dZ","status":"approved","complete":%s}'
              % (v, v, max(-2 ** 31, min(2 ** 31 - 1, v)), k % 100, k % 1000, b"true" if k & 1 else b"false") for k, v in enumerate(vals)]
    for schema, lines in ((1, recs), (2, orders), (4, recs + orders)):
        body = as_u8(b"\n".join(lines) + b"\n")
        cols = oracle.parse(schema, body)
        assert cols.n_errors == 0
        for lock in (False, True):
            got, _ = emu_parse_tiles(emu, oracle, schema, body, lock=lock)
            assert same_result(cols, got) == ""
        for framing in (NDJSON, ARRAY):
            for incl in (abi.PJ_INCLUDE_NON_EMPTY, abi.PJ_INCLUDE_NON_NULL, abi.PJ_INCLUDE_ALWAYS):
                want = oracle.write(schema, cols, framing, incl)
                assert np.array_equal(want, emu_write(emu, "emu_write_fast", schema, cols, framing, incl, body.size * 4 + 128))


# ---- the stream kernel's line index (pj_stream.cuh) ---------------------------------------------------------
def stream_index(emu, buf, tile_bytes, mis=0, slack=0, is_first=1, is_last=1):
    buf = as_u8(buf)
    cap = nrec_bound(buf) + 2
    starts, n, ov, ll = np.zeros(cap, np.uint64), u64(), u64(), u64()
    st = emu.emu_stream_index(C.c_void_p(buf.ctypes.data), u64(buf.size - slack), u64(slack), int(is_first), int(is_last), u32(tile_bytes), u32(mis),
                              C.c_void_p(starts.ctypes.data), u64(cap), C.byref(n), C.byref(ov), C.byref(ll))
    assert st == 0, st
    return starts[: n.value], ov.value, ll.value


def blank_mutations(rng, text: bytes) -> bytes:
    """Blank lines, CRLF line ends, lines of blanks and a missing final line feed, sprinkled over an NDJSON text."""
    out = bytearray()
    for ln in text.split(b"\n"):
        r = rng.random()
        if r < 0.05:
            out += b"\n"
        elif r < 0.10:
            out += b" \t\r\n"
        elif r < 0.15:
            out += b"  "
        out += ln + (b"\r\n" if rng.random() < 0.1 else b"\n")
    if rng.random() < 0.5:
        while out.endswith(b"\n"):
            out.pop()
    return bytes(out)


@pytest.mark.parametrize("tile_bytes", [1024, 4096, 20480, 32768])
def test_stream_line_index_matches_the_checker(emu, oracle, tile_bytes):
    rng = random.Random(tile_bytes)
    for schema, n, flags in ((abi.PJ_SCHEMA_PET, 700, 0), (abi.PJ_SCHEMA_ORDER, 2500, 0), (abi.PJ_SCHEMA_MIXED, 900, G.PJ_GEN_WHITESPACE),
                             (abi.PJ_SCHEMA_PET, 60, G.PJ_GEN_ZIPF_LISTS)):
        text = blank_mutations(rng, pj.gen_text(schema, 7 + tile_bytes, 0, n, flags).tobytes())
        buf = as_u8(text)
        want = oracle.index(buf)
        for mis in (0, 1, 7, 15):
            got, _, _ = stream_index(emu, buf, tile_bytes, mis)
            assert np.array_equal(got, want), (schema, tile_bytes, mis)


def test_stream_line_index_tiny_records_and_long_lines(emu, oracle):
    """More lines than threads in a tile (the overflow road) and lines that run out of the window."""
    rng = random.Random(5)
    tiny = b"".join(rng.choice([b"{}\n", b"\n", b"1\n", b" \n", b"[]\r\n"]) for _ in range(40000))
    got, ov, _ = stream_index(emu, as_u8(tiny), 32768)
    assert ov > 0 and np.array_equal(got, oracle.index(as_u8(tiny)))
    long_line = b'{"name":"' + b"x" * 100000 + b'","photoUrls":[]}\n'
    text = b'{"id":1}\n' + long_line + b'{"id":2}\n' + b" " * 50000 + b"\n" + b'{"id":3}'
    got, _, ll = stream_index(emu, as_u8(text), 32768, mis=3)
    assert ll >= 1 and np.array_equal(got, oracle.index(as_u8(text)))
    for text in (b"", b"\n", b"{}", b"\n{}", b" ", b"   \n \n"):
        got, _, _ = stream_index(emu, as_u8(text), 4096)
        assert np.array_equal(got, oracle.index(as_u8(text))), text


def test_stream_line_index_of_shards(emu, oracle):
    """Shards with slack own the lines the shard rule gives them, whatever the tile size."""
    rng = random.Random(11)
    text = as_u8(blank_mutations(rng, pj.gen_text(abi.PJ_SCHEMA_PET, 3, 0, 900, 0).tobytes()))
    want = oracle.index(text)
    for parts in (2, 3, 5):
        cuts = [text.size * k // parts for k in range(parts + 1)]
        got = []
        for k in range(parts):
            lo, hi = cuts[k], cuts[k + 1]
            slack = min(65536, text.size - hi)
            s, _, _ = stream_index(emu, text[lo:hi + slack], 8192, mis=k, slack=slack, is_first=k == 0, is_last=hi + slack == text.size)
            got.append(s + np.uint64(lo))
        assert np.array_equal(np.concatenate(got), want), parts


def test_lockstep_tokeniser_edges(emu, oracle):
    """What the lockstep tokeniser accepts it decodes as the checker does; what it may not accept it leaves alone."""
    emu.emu_lock_accepted.restype = C.c_uint64
    ok = [b'{}', b'{"name":"a","photoUrls":[]}', b'{"id":0,"name":"","photoUrls":[""],"tags":[{}],"status":"sold"}',
          b'{"id":9223372036854775807,"category":{},"name":"n","photoUrls":["a","b","c","d","e","f","g","h","i","j","k","l","m","n","o","p","q","r","s","t","u","v","w","x"],"tags":[{"id":1},{"name":"x"},{"id":2,"name":"y"}]}',
          b'{"name":"' + b"x" * 2047 + b'","photoUrls":[]}']
    refused = [b'{"id":-1,"name":"a","photoUrls":[]}', b'{"id":01,"name":"a","photoUrls":[]}', b'{"id":1.0,"name":"a","photoUrls":[]}',
               b'{"id":9223372036854775808,"name":"a","photoUrls":[]}', b'{"id":1e3,"name":"a","photoUrls":[]}', b'{"name":"a","photoUrls":[],}',
               b'{"name":"a","photoUrls":["x",]}', b'{"name":"a","photoUrls":[,]}', b'{"name":"a" ,"photoUrls":[]}', b'{"name":"a","photoUrls":[]} ',
               b'{"name":"a","photoUrls":[]}\r', b'{"photoUrls":[],"name":"a"}', b'{"name":"a","name":"b","photoUrls":[]}', b'{"name":"a\\n","photoUrls":[]}',
               b'{"name":"\xc3\xa9","photoUrls":[]}', b'{"name":null,"photoUrls":[]}', b'{"name":"a","photoUrls":[],"status":"gone"}',
               b'{"name":"a","photoUrls":[],"tags":[{"id":1,}]}', b'{"name":"a","photoUrls":[]', b'{"name":"a","photoUrls":[]}}', b'{"name":"a","photoUrls":[]}x',
               b'{"name":"' + b"x" * 2048 + b'","photoUrls":[]}', b'{"id":123456789012345678901234567890,"name":"a","photoUrls":[]}', b'[]', b'']
    for recs, floor in ((ok, len(ok)), (refused, 0)):
        body = as_u8(b"\n".join(recs) + b"\n")
        want = oracle.parse(1, body)
        got, _ = emu_parse_tiles(emu, oracle, 1, body, lock=True)
        assert same_result(want, got) == ""
        n = emu.emu_lock_accepted()
        assert (n >= floor - 1) if floor else (n <= 1), n  # `{}` of the refused set's neighbours aside, nothing of it is accepted
    for schema, recs in ((2, [b'{"id":1,"petId":2,"quantity":3,"shipDate":"2024-02-29T12:00:01.123Z","status":"placed","complete":true}', b'{"complete":false}', b'{"quantity":2147483648}',
                              b'{"shipDate":"2023-02-29T12:00:01Z"}', b'{"complete":tru}']),
                         (3, [b'{"id":5,"username":"u","firstName":"f","lastName":"l","email":"e@x","password":"p","phone":"1234567890","userStatus":3}', b'{"userStatus":-1}']),
                         (4, [b'{"id":1,"name":"a","photoUrls":[]}', b'{"id":1}', b'{"id":1,"status":"placed","petId":2}', b'{"petId":2,"id":1}', b'{"id":7,"username":"u"}', b'{"id":7,"petId":3}',
                              b'{"name":"a","photoUrls":[],"id":4}', b'{"phone":"1"}', b'{"photoUrls":[]}', b'{"password":"x"}', b'{}'])):
        body = as_u8(b"\n".join(recs) + b"\n")
        got, _ = emu_parse_tiles(emu, oracle, schema, body, lock=True)
        assert same_result(oracle.parse(schema, body), got) == "", schema


# ---- the option switches (pj_options.flags) in the device-side parsers ---------------------------------------
def test_option_switches_known_answers(emu, oracle):
    from golden.kat_cases import OPTION_CASES
    from pj_testlib import SCHEMA_BY_NAME, records

    for name, schema, opts, data, expected in OPTION_CASES:
        sch = SCHEMA_BY_NAME[schema]
        for lock in (False, True):
            got, _ = emu_parse_tiles(emu, oracle, sch, as_u8(data), lock=lock, opts=opts)
            assert records(got.as_dict(), sch) == expected, (name, lock)
    emu.emu_set_options(u32(0))


@pytest.mark.parametrize("opts", [1, 2, 4, 7])
def test_option_switches_on_mutated_text(emu, oracle, opts):
    """Every combination of the three parse switches against the checker with the same switches."""
    rng = random.Random(opts)
    for it in range(25):
        schema = rng.choice([1, 2, 3, 4])
        lines = bytes(pj.gen_text(schema, rng.randrange(1 << 30), 0, 40, rng.choice([0, G.PJ_GEN_ESCAPES, G.PJ_GEN_MALFORMED | G.PJ_GEN_SPARSE]))).split(b"\n")[:-1]
        out = []
        for ln in lines:
            r = rng.random()
            if r < 0.25:
                ln = mutate(rng, ln)
            elif r < 0.45:  # quote a number, unquote a short string, break an enum, plant a lone surrogate
                ln = rng.choice([re.sub(rb':(\d+)', rb':"\1"', ln, count=1), re.sub(rb':"([A-Za-z]{1,6})"', rb':\1', ln, count=1),
                                 ln.replace(b'"status":"', b'"status":"x', 1), re.sub(rb'":"', rb'":"\\ud83d', ln, count=1),
                                 re.sub(rb':"([a-z]+)"', rb':12.5', ln, count=1), ln.replace(b"true", b'"true"').replace(b"false", b'"false"')])
            out.append(ln)
        body = as_u8(b"\n".join(out) + b"\n")
        want = oracle.parse(schema, body, opts=opts)
        for lock in (False, True):
            got, _ = emu_parse_tiles(emu, oracle, schema, body, lock=lock, opts=opts)
            assert same_result(want, got) == "", (opts, it, schema, lock)
    emu.emu_set_options(u32(0))


def test_mask_algebra_of_the_long_record_path(emu):
    """pj_wide.cuh finds the elements of long lists from 32-byte masks: escaped bytes (odd runs of backslashes, carried
    from block to block), unescaped quotes, string interiors by prefix XOR. The same formulas, block after block on
    the host, against a byte-at-a-time state machine: random text rich in backslashes and quotes, runs of every
    length across the block edges."""
    rng = random.Random(23)

    def reference(b):
        quotes, instr, special = np.zeros(len(b), np.uint8), np.zeros(len(b), np.uint8), np.zeros(len(b), np.uint8)
        escaped, inside = False, False
        for k, x in enumerate(b):
            is_q = x == 0x22 and not escaped
            if is_q:
                inside = not inside
            quotes[k], instr[k] = is_q, inside
            special[k] = x < 0x20 or x >= 0x80
            escaped = (x == 0x5C) and not escaped
        return quotes, instr, special

    cases = []
    for run in range(0, 70):
        for lead in (0, 1, 29, 30, 31, 32, 33):
            cases.append(b"a" * lead + b"\\" * run + b'"x"' + b"b" * 5 + b'"\\""')
    alphabet = [b"\\", b'"', b"a", b",", b" ", b"\x01", b"\xc3\xa9", b"{", b"}"]
    for _ in range(300):
        cases.append(b"".join(rng.choice(alphabet) for _ in range(rng.randint(1, 300))))
    checked = 0
    for b in cases:
        buf = as_u8(b)
        q, s_, x = np.zeros(buf.size, np.uint8), np.zeros(buf.size, np.uint8), np.zeros(buf.size, np.uint8)
        refused = emu.emu_wide_masks(C.c_void_p(buf.ctypes.data), u64(buf.size), C.c_void_p(q.ctypes.data), C.c_void_p(s_.ctypes.data), C.c_void_p(x.ctypes.data))
        if refused:  # a block of nothing but backslashes
            assert any(bytes(buf[k:k + 32]) == b"\\" * 32 for k in range(0, buf.size, 32))
            continue
        rq, rs, rx = reference(bytes(buf))
        assert np.array_equal(q, rq) and np.array_equal(s_, rs) and np.array_equal(x, rx), b
        checked += 1
    assert checked > 500


def test_device_code_under_sanitizers():
    """The device-side parsers, line index and writers, compiled for the host with AddressSanitizer and
    UndefinedBehaviorSanitizer, run a slice of the tests above in a child process: an out-of-bounds read of a window,
    a tape or a column, a misaligned word load or a shift by 64 ends the child."""
    asan = subprocess.run(["gcc", "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
    if not os.path.isabs(asan) or not os.path.exists(asan):
        pytest.skip("no libasan beside this gcc")
    env = dict(os.environ, PJ_EMU_SANITIZE="1", LD_PRELOAD=asan, ASAN_OPTIONS="detect_leaks=0:abort_on_error=0", UBSAN_OPTIONS="print_stacktrace=1")
    pick = "mask_algebra or stream_line_index or lockstep_tokeniser_edges or common_failures or (mutated_text and 1) or tiny_records_and_long_lines or integer_text or array_framing or option_switches_known"
    r = subprocess.run([sys.executable, "-m", "pytest", "-x", "-q", "-p", "no:cacheprovider", os.path.abspath(__file__), "-k", pick],
                       env=env, capture_output=True, text=True, cwd=HERE, timeout=1500)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "passed" in r.stdout and "deselected" in r.stdout
