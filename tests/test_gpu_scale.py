"""The benchmark configurations at (or near) their full sizes against the CPU checker, through the C ABI: every
column is compared by its 64-bit checksum, computed on the GPU (pj_columns_checksum) and by the checker on its own
columns, and the small per-record columns element by element as well. Needs a B200 (-m gpu); each case takes
tens of seconds, most of it the single-threaded checker."""
import numpy as np
import pytest

from pj_testlib import abi, pj

pytestmark = pytest.mark.gpu


def caps_for(schema, n, nbytes, items, arena_share=0.5):
    """Capacities that fit the generated corpora without reserving one input-sized arena per string column
    (arena_share: the largest part of the input that one string arena can hold)."""
    return abi.default_caps(schema, n + 16, int(nbytes * arena_share) + 65536, items)


def parse_both(native, oracle, schema, text, n, items, ctx_kw=None, arena_share=0.5):
    import torch

    want = oracle.parse(schema, text, caps=caps_for(schema, n, text.size, items, arena_share))
    ctx = native.Context(device=0, **(ctx_kw or {}))
    d_text = torch.from_numpy(text).cuda()
    cols = pj.DeviceColumns(schema, caps_for(schema, n, text.size, items, arena_share), "cuda")
    torch.cuda.synchronize()
    ctx.parse(schema, d_text, cols)
    return want, ctx, d_text, cols


def assert_same_by_checksum(oracle, want, ctx, schema, cols):
    assert (want.n_records, want.n_errors, [want.n_rows(t) for t in range(4)]) == (cols.n_records, cols.n_errors, [cols.n_rows(t) for t in range(4)])
    for c in abi.schema_columns(schema):
        assert want.count(c.id) == cols.count(c.id), c.name
    got = ctx.checksums(schema, cols)
    exp = oracle.checksums(want)
    bad = [k for k in exp if exp[k] != got[k]]
    assert not bad, bad
    for name in ("err_kind", "err_off", "rec_start"):
        assert np.array_equal(want.get(name), cols.get(name)), name


def test_ten_million_mixed_records_with_one_percent_malformed(native, oracle):
    """BASELINE configs[2] at its full size: 10 M Pet/Order/User records 50/30/20, 1 % malformed (about 100 000 failed
    records: kind and byte offset of every one are compared element by element)."""
    n = 10_000_000
    text = pj.gen_text(abi.PJ_SCHEMA_MIXED, 0xC2, 0, n, abi.PJ_GEN_MALFORMED)
    want, ctx, d_text, cols = parse_both(native, oracle, abi.PJ_SCHEMA_MIXED, text, n, 4 * n)
    assert 80_000 < want.n_errors < 120_000
    assert_same_by_checksum(oracle, want, ctx, abi.PJ_SCHEMA_MIXED, cols)
    assert np.array_equal(want.get("rec_type"), cols.get("rec_type")) and np.array_equal(want.get("rec_row"), cols.get("rec_row"))
    ctx.close()


def test_one_million_pets_with_zipf_lists_escapes_and_blanks(native, oracle):
    """BASELINE configs[3]'s distributions (zipf(1.2) list lengths up to 64 tags / 256 photoUrls, 5 % escaped strings with
    surrogate pairs, random blanks between tokens) at 1 M records, about 1.8 GB."""
    n = 1_000_000
    flags = abi.PJ_GEN_ZIPF_LISTS | abi.PJ_GEN_ESCAPES | abi.PJ_GEN_WHITESPACE
    text = pj.gen_text(abi.PJ_SCHEMA_PET, 0xC3, 0, n, flags)
    assert text.size > 1_000_000_000
    want, ctx, d_text, cols = parse_both(native, oracle, abi.PJ_SCHEMA_PET, text, n, text.size // 30, arena_share=1.0)
    assert want.n_errors == 0
    assert_same_by_checksum(oracle, want, ctx, abi.PJ_SCHEMA_PET, cols)
    ctx.close()


def test_ten_million_pets_written_back_byte_for_byte(native, oracle):
    """BASELINE configs[4]'s shape at 10 M rows: the columns of 10 M Pets go back to text; the generator's text is the
    canonical spelling, so the writer must reproduce it byte for byte (2.9 GB)."""
    import torch

    n = 10_000_000
    text = pj.gen_text(abi.PJ_SCHEMA_PET, 0xC4, 0, n, 0)
    ctx = native.Context(device=0, inclusion=abi.PJ_INCLUDE_NON_NULL)
    d_text = torch.from_numpy(text).cuda()
    cols = pj.DeviceColumns(abi.PJ_SCHEMA_PET, caps_for(abi.PJ_SCHEMA_PET, n, text.size, 3 * n), "cuda")
    torch.cuda.synchronize()
    ctx.parse(abi.PJ_SCHEMA_PET, d_text, cols)
    assert cols.n_records == n and cols.n_errors == 0
    # the parsed values against the generator's own record of what it wrote, column by column, by checksum
    want = pj.gen_columns(abi.PJ_SCHEMA_PET, 0xC4, 0, n, 0, text.size // 2 + 65536)
    got, exp = ctx.checksums(abi.PJ_SCHEMA_PET, cols), oracle.checksums(want)
    assert not [k for k in exp if exp[k] != got[k]]
    d_out = torch.empty(text.size + 64, dtype=torch.uint8, device="cuda")
    m = ctx.write(abi.PJ_SCHEMA_PET, cols, d_out)
    assert m == text.size and torch.equal(d_out[:m], d_text)
    ctx.close()


def test_more_than_four_gib_in_one_call(native, oracle):
    """One pj_parse call on 4.3 GB of device-resident NDJSON (a launch addresses its input with 32-bit offsets: the call
    cuts the input into ranges of 2 GiB, each launch starting from the totals of the one before it). Compared, column
    by column, with the values the generator knows the text to hold."""
    import torch
    from concurrent.futures import ThreadPoolExecutor

    n, parts = 14_700_000, 12
    per = n // parts
    with ThreadPoolExecutor(max_workers=parts) as pool:  # the generator is plain C behind ctypes: the threads run side by side
        texts = list(pool.map(lambda k: pj.gen_text(abi.PJ_SCHEMA_PET, 0xC5, k * per, per, 0), range(parts)))
        sizes = [t.size for t in texts]
        wants = list(pool.map(lambda k: pj.gen_columns(abi.PJ_SCHEMA_PET, 0xC5, k * per, per, 0, sizes[k]), range(parts)))
    total = sum(sizes)
    assert total >= 1 << 32
    d_text = torch.empty(total + 64, dtype=torch.uint8, device="cuda")
    at = 0
    for t in texts:
        d_text[at: at + t.size].copy_(torch.from_numpy(t))
        at += t.size
    del texts
    cols = pj.DeviceColumns(abi.PJ_SCHEMA_PET, caps_for(abi.PJ_SCHEMA_PET, n, total, 3 * n, arena_share=0.34), "cuda")
    torch.cuda.synchronize()
    with native.Context(device=0) as ctx:
        ctx.parse(abi.PJ_SCHEMA_PET, d_text[:total], cols)
        assert ctx.stats().pieces == 3
        assert (cols.n_records, cols.n_errors) == (n, 0)
        # record starts: the generator's parts are record ranges, so their first offsets are the running sizes
        starts = cols.get("rec_start")
        assert starts.dtype == np.uint64 and int(starts[-1]) > 1 << 32 and bool(np.all(np.diff(starts.astype(np.int64)) > 0))
        first = np.cumsum([0] + sizes[:-1])
        assert np.array_equal(starts[::per][:parts], first.astype(np.uint64))
        # fixed-width columns part by part against the generator's values
        ids = cols.get("pet_id")
        for k, w in enumerate(wants):
            assert np.array_equal(ids[k * per:(k + 1) * per], w.get("pet_id")), k
            assert np.array_equal(starts[k * per:(k + 1) * per] - np.uint64(first[k]), w.get("rec_start")), k
        # arenas: total sizes, and the bytes of the parts that straddle the 2 GiB seams
        names = cols.get("pet_name_data")
        assert names.size == sum(w.count(abi.COL_BY_NAME["pet_name_data"].id) for w in wants)
        off = 0
        for k, w in enumerate(wants):
            m = w.count(abi.COL_BY_NAME["pet_name_data"].id)
            assert np.array_equal(names[off: off + m], w.get("pet_name_data")), k
            off += m
