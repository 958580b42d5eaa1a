"""Parity of the CUDA path with the CPU checker, through the C ABI. Needs a B200 (run with -m gpu)."""
import random

import numpy as np
import pytest

from golden.kat_cases import CASES, HEX_LOWER, OPTION_CASES
from pj_testlib import SCHEMA_BY_NAME, abi, as_u8, nrec_bound, pj, same_result
from test_oracle_crosscheck import mutate
from test_oracle_kat import check_case

pytestmark = pytest.mark.gpu

NDJSON, ARRAY = abi.PJ_FRAMING_NDJSON, abi.PJ_FRAMING_ARRAY
FLAG_SETS = [0, abi.PJ_GEN_ESCAPES, abi.PJ_GEN_WHITESPACE, abi.PJ_GEN_MALFORMED, abi.PJ_GEN_SPARSE,
             abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_MALFORMED | abi.PJ_GEN_SPARSE,
             abi.PJ_GEN_ZIPF_LISTS | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE]


def gpu_parse_host(ctx, schema, buf, framing=NDJSON):
    """Host buffers in, host columns out (the end-to-end route)."""
    buf = as_u8(buf)
    out = abi.HostColumns(schema, abi.default_caps(schema, nrec_bound(buf), buf.size))
    ctx.parse(schema, buf, out, framing)
    return out


def gpu_parse_device(ctx, schema, buf, framing=NDJSON, misalign=0):
    """Device buffers in and out."""
    import torch

    buf = as_u8(buf)
    t = torch.empty(buf.size + misalign + 64, dtype=torch.uint8, device="cuda")
    t[misalign:misalign + buf.size].copy_(torch.from_numpy(buf))
    out = pj.DeviceColumns(schema, abi.default_caps(schema, nrec_bound(buf), buf.size), "cuda")
    torch.cuda.synchronize()
    ctx.parse(schema, t[misalign:misalign + buf.size], out, framing)
    return out


@pytest.mark.parametrize("case", CASES, ids=[c[0] for c in CASES])
def test_known_answers_on_gpu(ctx, case):
    check_case(lambda sch, buf, fr: gpu_parse_host(ctx, sch, buf, fr), *case)


@pytest.mark.parametrize("schema", [1, 2, 3, 4])
@pytest.mark.parametrize("flags", FLAG_SETS)
def test_generated_corpora(ctx, oracle, schema, flags):
    text = pj.gen_text(schema, 0x5EED, 0, 3000, flags)
    want = oracle.parse(schema, text)
    assert same_result(want, gpu_parse_device(ctx, schema, text)) == ""
    assert same_result(want, gpu_parse_host(ctx, schema, text)) == ""
    assert same_result(want, pj.gen_columns(schema, 0x5EED, 0, 3000, flags, text.size)) == ""


@pytest.mark.parametrize("misalign", [0, 1, 7, 15, 16, 33])
def test_unaligned_device_input(ctx, oracle, misalign):
    text = pj.gen_text(4, 3, 0, 500, abi.PJ_GEN_WHITESPACE)
    assert same_result(oracle.parse(4, text), gpu_parse_device(ctx, 4, text, misalign=misalign)) == ""


@pytest.mark.parametrize("schema", [1, 2, 3, 4])
def test_mutated_corpora(ctx, oracle, schema):
    rng = random.Random(schema * 17)
    for rnd in range(4):
        lines = bytes(pj.gen_text(schema, 100 + rnd, 0, 1500, rng.choice([0, abi.PJ_GEN_ESCAPES, abi.PJ_GEN_SPARSE]))).split(b"\n")[:-1]
        out = []
        for ln in lines:
            out.append(ln if rng.random() < 0.2 else mutate(rng, ln))
            if rng.random() < 0.05:
                out.append(rng.choice([b"", b"  ", b"\r", b"\t \r"]))
        body = as_u8(b"\n".join(out) + (b"\n" if rnd % 2 else b""))
        want = oracle.parse(schema, body)
        assert want.n_errors > 100
        assert same_result(want, gpu_parse_device(ctx, schema, body)) == ""


@pytest.mark.parametrize("size", [0, 1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 16383, 16384, 16385])
def test_tiny_and_tile_edge_inputs(ctx, oracle, size):
    """Inputs around the 64-byte thread span and the 16 KiB tile of the record index."""
    text = pj.gen_text(2, 5, 0, 400, 0)
    for body in (text[:size], np.concatenate([np.full(size, 0x20, np.uint8), as_u8(b"\n"), text[:300]]),
                 np.concatenate([text[:size], as_u8(b"\n" * 70), text[:200]])):
        assert same_result(oracle.parse(2, body), gpu_parse_device(ctx, 2, body)) == ""


def test_line_feeds_at_every_offset_of_a_tile(ctx, oracle):
    rec = b'{"quantity":1}'
    for pad in range(0, 70, 3):
        body = as_u8((b" " * pad + rec + b"\n") * 600)
        assert same_result(oracle.parse(2, body), gpu_parse_device(ctx, 2, body)) == ""


def test_shards_reassemble(ctx, oracle):
    """Byte-range shards with slack give, together, exactly the records of the whole stream."""
    text = pj.gen_text(4, 11, 0, 4000, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ZIPF_LISTS)
    whole = oracle.parse(4, text)
    rng = random.Random(5)
    for nshards in (2, 3, 8):
        cuts = sorted(rng.sample(range(1, text.size), nshards - 1))
        bounds = [0] + cuts + [text.size]
        starts = []
        for g in range(nshards):
            lo, hi = bounds[g], bounds[g + 1]
            slack = min(65536, text.size - hi)
            sub = text[lo:hi + slack]
            out = abi.HostColumns(4, abi.default_caps(4, nrec_bound(sub), sub.size))
            ctx.parse_shard(4, sub, hi - lo, slack, g == 0, hi + slack == text.size, lo, out)
            want = oracle.parse(4, sub, slack=slack, is_first=g == 0, is_last=hi + slack == text.size, goff=lo)
            assert same_result(want, out) == ""
            starts.append(out.get("rec_start"))
        assert np.array_equal(np.concatenate(starts), whole.get("rec_start"))


def test_slack_too_short_is_reported_per_record(ctx, oracle):
    text = pj.gen_text(1, 12, 0, 50, 0)
    cut = int(text.size // 2)
    for slack in (0, 1, 10, 100):
        sub = text[:cut + slack]
        out = abi.HostColumns(1, abi.default_caps(1, nrec_bound(sub), sub.size))
        ctx.parse_shard(1, sub, cut, slack, True, False, 0, out)
        assert same_result(oracle.parse(1, sub, slack=slack, is_first=1, is_last=0), out) == ""
        assert out.get("err_kind")[-1] == abi.PJ_E_TOO_LONG


def test_capacity_error_reports_needed_counts(ctx, oracle):
    text = pj.gen_text(1, 13, 0, 1000, 0)
    want = oracle.parse(1, text)
    caps = abi.default_caps(1, 1000, text.size)
    small = dict(caps)
    small[abi.COL_BY_NAME["pet_photo_data"].id] = 64
    out = abi.HostColumns(1, small)
    assert ctx.parse(1, text, out, allow_capacity=True) == abi.PJ_ERR_CAPACITY
    for c in abi.schema_columns(1):
        assert out.count(c.id) == want.count(c.id), c.name
    # too few rows in a per-record column, in a row-indexed value column and in a row-indexed offset column (which
    # needs rows + 1 entries): refused before anything is written past them
    for name, nbytes in (("err_kind", 10), ("pet_id", 8 * 999), ("pet_name_off", 4 * 1000), ("pet_status", 512)):
        few = dict(caps)
        few[abi.COL_BY_NAME[name].id] = nbytes
        out = abi.HostColumns(1, few, alloc=lambda nb: np.full(nb + 64, 0xA5, np.uint8))
        assert ctx.parse(1, text, out, allow_capacity=True) == abi.PJ_ERR_CAPACITY, name
        assert out.n_records == 1000
        assert all(int(out.arrays[c][max(few.get(c, 0), 16):].min()) == 0xA5 for c in out.arrays), name
    # the context stays usable
    assert same_result(want, gpu_parse_host(ctx, 1, text)) == ""


def test_index_records_only(ctx, oracle):
    import torch

    text = pj.gen_text(4, 14, 0, 5000, abi.PJ_GEN_WHITESPACE)
    want = oracle.index(text)
    rs = np.zeros(6000, np.uint64)
    assert ctx.index_records(text, rs) == want.size and np.array_equal(rs[:want.size], want)
    d_text = torch.from_numpy(text).cuda()
    d_rs = torch.zeros(6000, dtype=torch.int64, device="cuda")
    assert ctx.index_records(d_text, d_rs) == want.size
    assert np.array_equal(d_rs[:want.size].cpu().numpy().view(np.uint64), want)
    assert ctx.index_records(text, np.zeros(10, np.uint64), allow_capacity=True) == want.size


def test_index_records_of_an_array(ctx, oracle):
    """Index only, array framing: the extent starts the checker finds, including extents without a value."""
    import torch

    text = pj.gen_text(4, 15, 0, 3000, abi.PJ_GEN_ARRAY | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_ESCAPES)
    for body in (text, as_u8(b' [ {"a":"]\\"[,"} , , [1,[2]] ,"x]" ] '), as_u8(b"[]"), as_u8(b"")):
        want = oracle.index(body, ARRAY)
        rs = np.zeros(want.size + 8, np.uint64)
        assert ctx.index_records(body, rs, ARRAY) == want.size and np.array_equal(rs[:want.size], want)
    d_text = torch.from_numpy(text).cuda()
    d_rs = torch.zeros(3100, dtype=torch.int64, device="cuda")
    n = ctx.index_records(d_text, d_rs, ARRAY)
    want = oracle.index(text, ARRAY)
    assert n == want.size and np.array_equal(d_rs[:n].cpu().numpy().view(np.uint64), want)


# ---- writer ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("schema", [1, 2, 3, 4])
@pytest.mark.parametrize("framing", [NDJSON, ARRAY])
@pytest.mark.parametrize("inclusion", [abi.PJ_INCLUDE_NON_EMPTY, abi.PJ_INCLUDE_NON_NULL, abi.PJ_INCLUDE_ALWAYS])
def test_writer_matches_checker(native, oracle, schema, framing, inclusion):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    flags = abi.PJ_GEN_ESCAPES | abi.PJ_GEN_SPARSE | abi.PJ_GEN_MALFORMED
    text = pj.gen_text(schema, 21, 0, 2500, flags)
    cols = oracle.parse(schema, text)
    want = oracle.write(schema, cols, framing, inclusion)
    with native.Context(device=0, inclusion=inclusion) as c:
        out = np.zeros(want.size + 16, np.uint8)
        n = c.write(schema, cols, out, framing)
        assert n == want.size and np.array_equal(out[:n], want)
        dcols = pj.DeviceColumns.from_host(cols, "cuda")
        d_out = torch.zeros(want.size + 16, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        n = c.write(schema, dcols, d_out, framing)
        assert n == want.size and np.array_equal(d_out[:n].cpu().numpy(), want)
        assert c.write(schema, cols, np.zeros(100, np.uint8), framing, allow_capacity=True) == want.size


@pytest.mark.parametrize("framing", [NDJSON, ARRAY])
@pytest.mark.parametrize("misalign", [0, 1, 5, 15])
def test_writer_tiles_larger_than_the_window_and_odd_alignment(native, oracle, framing, misalign):
    """Tiles whose text exceeds the staging window are written straight to global memory; the output pointer
    may have any alignment; records without a value (failed ones of a mixed stream) take no bytes."""
    import torch

    big = b'{"id":7,"name":"big","photoUrls":[' + b",".join(b'"' + bytes([97 + k % 26]) * 60 + b'"' for k in range(900)) + b"]}"
    small = bytes(pj.gen_text(4, 9, 0, 400, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ESCAPES))
    body = as_u8(small + big + b"\n" + small + b"{}\n" + big + b"\n")
    cols = oracle.parse(4, body)
    want = oracle.write(4, cols, framing, abi.PJ_INCLUDE_NON_EMPTY)
    with native.Context(device=0) as c:
        dcols = pj.DeviceColumns.from_host(cols, "cuda")
        d_out = torch.zeros(want.size + 64, dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        n = c.write(4, dcols, d_out[misalign:], framing)
        assert n == want.size and np.array_equal(d_out[misalign:misalign + n].cpu().numpy(), want)
        assert int(d_out[misalign + n:].max()) == 0 and (misalign == 0 or int(d_out[:misalign].max()) == 0)
        st = c.stats()
        assert st.kernel_launches == 3  # the look at the string arenas, the tile writer, the closing kernel
        # too small an output: nothing but the needed size is promised
        assert c.write(4, dcols, d_out[:1000], framing, allow_capacity=True) == want.size


def test_writer_empty_tables(native):
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    with native.Context(device=0) as c:
        empty = abi.HostColumns(1, abi.default_caps(1, 0, 0))
        c.parse(1, np.zeros(0, np.uint8), empty)
        out = np.zeros(8, np.uint8)
        assert c.write(1, empty, out, NDJSON) == 0
        assert c.write(1, empty, out, ARRAY) == 2 and bytes(out[:2]) == b"[]"


def test_canonical_text_round_trips(native, oracle):
    """write(parse(x)) == x for the generator's compact, schema-order text."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    with native.Context(device=0, inclusion=abi.PJ_INCLUDE_NON_NULL) as c:
        for schema in (1, 2, 3, 4):
            text = pj.gen_text(schema, 31, 0, 4000, 0)
            d_text = torch.from_numpy(text).cuda()
            cols = pj.DeviceColumns(schema, abi.default_caps(schema, 4000, text.size), "cuda")
            torch.cuda.synchronize()
            c.parse(schema, d_text, cols)
            assert cols.n_errors == 0
            d_out = torch.zeros(text.size + 16, dtype=torch.uint8, device="cuda")
            n = c.write(schema, cols, d_out)
            assert n == text.size and torch.equal(d_out[:n], d_text)


def test_one_million_pets(native, oracle):
    """The benchmark workload at full size against the checker, column by column."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    n = 1_000_000
    text = pj.gen_text(1, 0x5EED, 0, n, 0)
    want = oracle.parse(1, text)
    assert want.n_records == n and want.n_errors == 0
    with native.Context(device=0, inclusion=abi.PJ_INCLUDE_NON_NULL) as c:
        d_text = torch.from_numpy(text).cuda()
        cols = pj.DeviceColumns.sized_for(1, n, text.size, 8 * n, "cuda")
        torch.cuda.synchronize()
        c.parse(1, d_text, cols)
        assert same_result(want, cols) == ""
        st = c.stats()
        assert st.kernel_launches == 1 and st.algorithmic_bytes == text.size + cols.total_bytes()  # one kernel: index, validation, emission
        assert st.fast_records == n
        d_out = torch.zeros(text.size + 16, dtype=torch.uint8, device="cuda")
        m = c.write(1, cols, d_out)
        assert m == text.size and torch.equal(d_out[:m], d_text)


@pytest.mark.parametrize("schema", [1, 2, 3, 4])
@pytest.mark.parametrize("piece", [1, 700, 4096, 100000, 0xFFFFFFFF])
def test_host_buffers_parsed_in_pieces(native, oracle, schema, piece):
    """Host input + host columns are cut after line feeds into up to 16 pieces that overlap copies and kernels;
    the columns must not depend on where the cuts fall (blank lines, failed records and empty pieces included)."""
    flags = abi.PJ_GEN_ESCAPES | abi.PJ_GEN_MALFORMED | abi.PJ_GEN_SPARSE | abi.PJ_GEN_WHITESPACE
    text = bytes(pj.gen_text(schema, 77, 0, 1500, flags))
    lines = text.split(b"\n")
    body = as_u8(b"\n".join(lines[:200]) + b"\n" * 400 + b" \n\t\n" + b"\n".join(lines[200:-1]) + b"\n" + b'{"id":1,"name":"no line feed at the end","photoUrls":[]}')
    want = oracle.parse(schema, body)
    with native.Context(device=0, host_piece_bytes=piece) as c:
        assert same_result(want, gpu_parse_host(c, schema, body)) == ""
        st = c.stats()
        assert 1 <= st.pieces <= 16
        assert (st.pieces > 1) == (piece != 0xFFFFFFFF)
        # a second call on the same context reuses the streams and staging buffers
        assert same_result(want, gpu_parse_host(c, schema, body)) == ""


def test_pieces_keep_capacity_errors(native, oracle):
    """A call cut into pieces that does not fit the caller's buffers fails as a whole and still reports what it needs."""
    text = as_u8(pj.gen_text(1, 5, 0, 2000, 0))
    want = oracle.parse(1, text)
    caps = abi.default_caps(1, nrec_bound(text), text.size)
    with native.Context(device=0, host_piece_bytes=20000) as c:
        small = dict(caps)
        small[abi.COL_BY_NAME["pet_photo_data"].id] = 1000
        out = abi.HostColumns(1, small)
        assert c.parse(1, text, out, allow_capacity=True) == abi.PJ_ERR_CAPACITY
        assert c.stats().pieces > 1
        for col in abi.schema_columns(1):
            assert out.count(col.id) == want.count(col.id), col.name
        few = dict(caps)
        few[abi.COL_BY_NAME["err_kind"].id] = 700
        out = abi.HostColumns(1, few)
        assert c.parse(1, text, out, allow_capacity=True) == abi.PJ_ERR_CAPACITY
        assert out.n_records == 2000
        assert same_result(want, gpu_parse_host(c, 1, text)) == ""


def test_long_records_fall_back_to_unstaged_reads(ctx, oracle):
    """Records longer than the staging window are parsed straight from global memory."""
    big = b'{"name":"n","photoUrls":[' + b",".join(b'"' + b"u" * 50 + b'"' for _ in range(3000)) + b'],"tags":[' + \
          b",".join(b'{"id":%d,"name":"t%d"}' % (k, k) for k in range(500)) + b"]}"
    small = bytes(pj.gen_text(1, 8, 0, 300, 0))
    body = as_u8(small + big + b"\n" + small + big[:-5] + b"\n" + small)
    want = oracle.parse(1, body)
    assert want.n_errors == 1
    assert same_result(want, gpu_parse_device(ctx, 1, body)) == ""


def test_many_tiny_records(ctx, oracle):
    """Far more records than bytes per tile would suggest: empty objects and one-byte garbage lines."""
    body = as_u8(b"{}\n" * 70000 + b"x\n" * 30000 + b'{"id":1}\n' * 50000)
    for schema in (2, 3, 4):
        assert same_result(oracle.parse(schema, body), gpu_parse_device(ctx, schema, body)) == ""


# ---- array framing -----------------------------------------------------------------------------------
ARRAY_FLAG_SETS = [abi.PJ_GEN_ARRAY, abi.PJ_GEN_ARRAY | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_ESCAPES,
                   abi.PJ_GEN_ARRAY | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_MALFORMED | abi.PJ_GEN_SPARSE]


def same_doc(a, b) -> bool:
    return (int(a.raw.doc_err_kind), int(a.raw.doc_err_off)) == (int(b.raw.doc_err_kind), int(b.raw.doc_err_off))


@pytest.mark.parametrize("schema", [1, 2, 3, 4])
@pytest.mark.parametrize("flags", ARRAY_FLAG_SETS)
def test_array_framing_generated(ctx, oracle, schema, flags):
    """The first benchmark configuration's shape (a JSON array of records) at 1 000 and 20 000 records."""
    for n in (1000, 20000):
        text = pj.gen_text(schema, 0x5EED, 0, n, flags)
        want = oracle.parse(schema, text, ARRAY)
        got = gpu_parse_device(ctx, schema, text, ARRAY)
        assert same_result(want, got) == "" and same_doc(want, got)
        assert same_result(want, gpu_parse_host(ctx, schema, text, ARRAY)) == ""
    assert same_result(want, pj.gen_columns(schema, 0x5EED, 0, 20000, flags, text.size)) == ""


def test_array_framing_over_many_tiles(ctx, oracle):
    """A 10 MB array: hundreds of 16 KiB index tiles, so every lane of the tile scan has a run of its own."""
    text = pj.gen_text(1, 77, 0, 30000, abi.PJ_GEN_ARRAY | abi.PJ_GEN_WHITESPACE | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_MALFORMED)
    want = oracle.parse(1, text, ARRAY)
    got = gpu_parse_device(ctx, 1, text, ARRAY)
    assert same_result(want, got) == "" and same_doc(want, got)
    for cut in (text.size - 1, text.size // 2 + 1, 16384 * 33 + 5):  # documents that end early, inside whatever they end in
        want = oracle.parse(1, text[:cut], ARRAY)
        got = gpu_parse_device(ctx, 1, text[:cut], ARRAY)
        assert same_result(want, got) == "" and same_doc(want, got), cut


def test_array_framing_mutated(ctx, oracle):
    rng = random.Random(99)
    special = [b'"', b"\\", b"\\\\", b'\\"', b"[", b"]", b"{", b"}", b",", b" ", b"\n", b"\\" * 63, b"\\" * 64, b"\\" * 65, b'"a,b]"', b"[]", b"x"]
    for rnd in range(40):
        body = bytearray(pj.gen_text(rng.choice([1, 4]), 200 + rnd, 0, rng.choice([1, 40, 400]), abi.PJ_GEN_ARRAY | rng.choice([0, abi.PJ_GEN_ESCAPES, abi.PJ_GEN_WHITESPACE])))
        for _ in range(rng.randrange(0, 6)):
            pos = rng.randrange(len(body) + 1)
            body[pos:pos] = rng.choice(special)
        if rnd % 5 == 0:
            body = body[: rng.randrange(len(body))]
        buf = as_u8(bytes(body))
        want = oracle.parse(1, buf, ARRAY)
        got = gpu_parse_device(ctx, 1, buf, ARRAY, misalign=rnd % 3)
        assert same_result(want, got) == "" and same_doc(want, got), rnd


@pytest.mark.parametrize("run", [1, 62, 63, 64, 65, 127, 128, 16383, 16384, 16385])
def test_array_backslash_runs_across_word_and_tile_edges(ctx, oracle, run):
    """Escape parity, in-string state and depth must carry across 64-byte words and 16 KiB tiles."""
    for lead in (0, 1, 17):
        body = b"[" + b" " * lead + b'{"name":"' + b"\\" * run + b'","photoUrls":["[,]{}"]},{"name":"b","photoUrls":[]}]'
        buf = as_u8(body)
        want = oracle.parse(1, buf, ARRAY)
        got = gpu_parse_device(ctx, 1, buf, ARRAY)
        assert same_result(want, got) == "" and same_doc(want, got)


# ---- the stream kernel's tiles ------------------------------------------------------------------------
@pytest.mark.parametrize("tile_bytes", [1024, 2064, 8192, 32768])
def test_tile_size_does_not_change_the_result(native, oracle, tile_bytes):
    """Tiles of any size give the same columns: few records per tile, more lines than threads in a tile (the two-pass
    road), records that leave the window, blank lines, failed records, host pieces and shards."""
    rng = random.Random(tile_bytes)
    flags = abi.PJ_GEN_ESCAPES | abi.PJ_GEN_MALFORMED | abi.PJ_GEN_SPARSE | abi.PJ_GEN_WHITESPACE
    big = b'{"name":"n","photoUrls":[' + b",".join(b'"' + b"u" * 50 + b'"' for _ in range(900)) + b"]}\n"
    with native.Context(device=0, tile_bytes=tile_bytes, host_piece_bytes=30000) as c:
        for schema in (1, 2, 3, 4):
            text = bytes(pj.gen_text(schema, 300 + schema, 0, 2500, flags))
            body = as_u8(text[:200000] + b"{}\n" * 3000 + b"\n \r\n" * 50 + big + text[200000:] + b"x\n" * 700 + big[:-3])
            want = oracle.parse(schema, body)
            assert same_result(want, gpu_parse_device(c, schema, body, misalign=rng.randrange(16))) == "", schema
            assert same_result(want, gpu_parse_host(c, schema, body)) == "", schema
            assert c.stats().pieces > 1
        text = pj.gen_text(4, 11, 0, 3000, abi.PJ_GEN_MALFORMED)
        for cut in (1, text.size // 3, text.size - 5):
            slack = min(65536, text.size - cut)
            sub = text[:cut + slack]
            out = abi.HostColumns(4, abi.default_caps(4, nrec_bound(sub), sub.size))
            c.parse_shard(4, sub, cut, slack, True, cut + slack == text.size, 0, out)
            assert same_result(oracle.parse(4, sub, slack=slack, is_first=1, is_last=cut + slack == text.size), out) == "", cut


def test_tile_size_follows_the_records(native, oracle):
    """A context sizes the tiles of a call from the bytes per record of its earlier calls; results stay the same."""
    with native.Context(device=0) as c:
        for schema, n in ((2, 40000), (1, 20000), (2, 40000), (3, 30000)):
            text = pj.gen_text(schema, 9, 0, n, 0)
            want = oracle.parse(schema, text)
            for _ in range(2):
                assert same_result(want, gpu_parse_device(c, schema, text)) == ""
                assert c.stats().tiles >= 1


def test_a_bounded_wait_that_runs_out(native, oracle):
    """Tile 0 of the first call is never handed out (test hook), so the other tiles' waits for it run out after 2 ms:
    the call answers PJ_ERR_TIMEOUT instead of hanging, nothing faults, and the same context parses correctly
    afterwards."""
    import time

    text = pj.gen_text(1, 8, 0, 50000, 0)
    want = oracle.parse(1, text)
    with native.Context(device=0, flags=abi.PJ_OPT_TEST_STALL_ONCE, spin_limit_us=2000) as c:
        t0 = time.perf_counter()
        with pytest.raises(native.PetJsonError) as e:
            gpu_parse_device(c, 1, text)
        assert e.value.status == abi.PJ_ERR_TIMEOUT
        assert time.perf_counter() - t0 < 5.0
        assert same_result(want, gpu_parse_device(c, 1, text)) == ""
        assert same_result(want, gpu_parse_host(c, 1, text)) == ""


# ---- the option switches (pj_options.flags) --------------------------------------------------------------
@pytest.mark.parametrize("case", OPTION_CASES, ids=[c[0] for c in OPTION_CASES])
def test_option_known_answers_on_gpu(native, case):
    name, schema, opts, data, expected = case
    with native.Context(device=0, flags=opts) as c:
        check_case(lambda sch, buf, fr: gpu_parse_host(c, sch, buf, fr), name, schema, "ndjson", data, expected)
        check_case(lambda sch, buf, fr: gpu_parse_device(c, sch, buf, fr), name, schema, "ndjson", data, expected)


@pytest.mark.parametrize("opts", [1, 2, 4, 7])
def test_option_switches_on_corpora(native, oracle, opts):
    """Corpora in which the switches matter (quoted numbers, bare words, unknown literals, lone surrogates) with every
    switch and all of them together, NDJSON and array framing."""
    import re

    rng = random.Random(opts)
    with native.Context(device=0, flags=opts) as c:
        for schema in (1, 2, 3, 4):
            lines = bytes(pj.gen_text(schema, 500 + opts, 0, 3000, abi.PJ_GEN_ESCAPES | abi.PJ_GEN_MALFORMED)).split(b"\n")[:-1]
            out = []
            for ln in lines:
                r = rng.random()
                if r < 0.4:
                    ln = rng.choice([re.sub(rb':(\d+)', rb':"\1"', ln, count=1), re.sub(rb':"([A-Za-z]{1,6})"', rb':\1', ln, count=1),
                                     ln.replace(b'"status":"', b'"status":"x', 1), re.sub(rb'":"', rb'":"\\ud83d', ln, count=1),
                                     re.sub(rb':"([a-z]+)"', rb':12.5', ln, count=1), ln.replace(b"true", b'"true"').replace(b"false", b'"false"')])
                out.append(ln)
            body = as_u8(b"\n".join(out) + b"\n")
            want = oracle.parse(schema, body, opts=opts)
            assert same_result(want, gpu_parse_device(c, schema, body)) == "", schema
            arr = as_u8(b"[" + b",".join(out) + b"]")
            assert same_result(oracle.parse(schema, arr, ARRAY, opts=opts), gpu_parse_device(c, schema, arr, ARRAY)) == "", schema


def test_writer_hex_case(native, oracle):
    cols = oracle.parse(1, as_u8(b'{"name":"a\\u001fb\\u000b\\n\\u0000","photoUrls":["\\u001e"]}\n'))
    for opts in (0, HEX_LOWER):
        want = oracle.write(1, cols, opts=opts)
        with native.Context(device=0, flags=opts) as c:
            out = np.zeros(want.size + 8, np.uint8)
            n = c.write(1, cols, out)
            assert n == want.size and np.array_equal(out[:n], want)
    assert b"\\u001F" in bytes(oracle.write(1, cols)) and b"\\u001f" in bytes(oracle.write(1, cols, opts=HEX_LOWER))


def test_cpp_object_mapper_mirror(native):
    """The C++ mirror of the ObjectMapper surface (host/object_mapper.hpp): its self-checking program runs the calls a
    user of the reference's serde API makes (readValue, writeValueAsString, exceptions with kind and offset)."""
    import subprocess

    import importlib

    exe = importlib.import_module("micronaut3-bug_b200.build").build_facade_demo()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr


@pytest.mark.parametrize("schema", [1, 4])
@pytest.mark.parametrize("piece", [64, 1000, 4096, 100000])
def test_device_input_parsed_in_ranges(native, oracle, schema, piece):
    """pj_options.device_piece_bytes: device-resident NDJSON cut into byte ranges (what a call of 4 GiB and more does
    with ranges of 2 GiB): records that start in one range and end in the next, ranges that hold no line start at
    all, errors at the seams."""
    text = pj.gen_text(schema, 21, 0, 3000, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE)
    if piece * 16 < text.size:
        text = text[: int(np.nonzero(text[: piece * 16] == 10)[0][-1]) + 1]  # at most 16 ranges
    want = oracle.parse(schema, text)
    with native.Context(device_piece_bytes=piece) as ctx:
        assert same_result(want, gpu_parse_device(ctx, schema, text)) == ""
        assert ctx.stats().pieces == -(-text.size // piece)
        # a shard of the same bytes: slack behind the last range, a first range that does not own the line at byte 0
        cut = text.size // 2
        lo, hi = cut, text.size - 300
        shard = oracle.parse(schema, text[lo:], slack=text.size - hi, is_first=False, is_last=True, goff=lo)
        import torch

        t = torch.from_numpy(text[lo:].copy()).cuda()
        out = pj.DeviceColumns(schema, abi.default_caps(schema, nrec_bound(text[lo:]), text.size - lo), "cuda")
        if (hi - lo) <= piece * 16:
            ctx.parse_shard(schema, t, hi - lo, text.size - hi, False, True, lo, out)
            assert same_result(shard, out) == ""


def test_mixed_stream_records_filed_under_the_wrong_model(ctx, oracle):
    """The stream kernel hands the lines of a mixed tile to its threads grouped by the model their first keys suggest.
    Records whose first keys suggest one model and whose later keys make them another (unknown keys that look like
    known ones, `status` first, blanks in front of the keys) must come out as in line order all the same."""
    base = bytes(pj.gen_text(4, 31, 0, 6000, abi.PJ_GEN_MALFORMED)).split(b"\n")[:-1]
    traps = [b'{"id":7,"cat":1,"quantity":2,"petId":3}',            # looks like a Pet (category), is an Order
             b'{"id":8,"usable":true,"name":"rex","photoUrls":[]}',  # looks like a User, is a Pet
             b'{"id":9,"quality":"x","username":"u","email":"e@x"}',  # looks like an Order, is a User
             b'{"status":"sold","id":1,"name":"a","photoUrls":["p"]}',  # decides nothing at first
             b'{ "id":10, "petId":4, "quantity":1 }',                  # blanks: no guess
             b'{"id":11,"cat":1}']                                     # looks like a Pet, is nothing: ambiguous
    rng = random.Random(5)
    for every in (9, 53, 400):
        lines = []
        for k, ln in enumerate(base):
            lines.append(ln)
            if k % every == every - 1:
                lines.append(rng.choice(traps))
        text = as_u8(b"\n".join(lines) + b"\n")
        want = oracle.parse(4, text)
        assert same_result(want, gpu_parse_device(ctx, 4, text)) == "", every
        assert same_result(want, gpu_parse_host(ctx, 4, text)) == "", every
