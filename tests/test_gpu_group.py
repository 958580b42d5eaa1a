"""pj_group_*: several shards (one context, stream and host thread each) behind one handle, through the C ABI.
On one GPU the shards share the device (the counter table then goes through the host); with two or more GPUs the
same tests also run one shard per device with the table exchanged by ncclAllGather. Needs a B200 (-m gpu)."""
import ctypes as C
import random

import numpy as np
import pytest

from pj_testlib import abi, as_u8, nrec_bound, pj, same_result

pytestmark = pytest.mark.gpu


def device_sets():
    import torch

    n = torch.cuda.device_count() if torch.cuda.is_available() else 0
    sets = [[0, 0], [0, 0, 0, 0]]
    if n >= 2:
        sets += [list(range(min(n, 4))), [0, 1, 0, 1]]
    return sets


def read_device_u64(ptr, count, device):
    """count uint64 words of device memory at `ptr` (an address the library handed out)."""
    import torch

    rt = None
    for name in ("libcudart.so.12", "libcudart.so.13", "libcudart.so"):
        try:
            rt = C.CDLL(name)
            break
        except OSError:
            continue
    assert rt is not None, "CUDA runtime library not found"
    out = np.zeros(count, np.uint64)
    with torch.cuda.device(device):
        torch.cuda.synchronize()
        rt.cudaMemcpy.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int]
        assert rt.cudaMemcpy(out.ctypes.data, C.c_void_p(int(ptr)), out.nbytes, 2) == 0
    return out


def put_shards(text: np.ndarray, bounds, devices, room=65536):
    import torch

    bufs = []
    for g, dev in enumerate(devices):
        lo, hi = bounds[g], bounds[g + 1]
        t = torch.zeros(hi - lo + room, dtype=torch.uint8, device=f"cuda:{dev}")
        if hi > lo:
            t[: hi - lo].copy_(torch.from_numpy(text[lo:hi]))
        bufs.append(t)
    for dev in set(devices):
        torch.cuda.synchronize(dev)
    return bufs


@pytest.mark.parametrize("devices", device_sets(), ids=lambda d: "dev" + "".join(map(str, d)))
def test_group_parse_matches_the_checker_shard_by_shard(native, oracle, devices):
    import torch

    rng = random.Random(len(devices))
    schema = 4
    text = pj.gen_text(schema, 11, 0, 6000, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ESCAPES)
    whole = oracle.parse(schema, text)
    n = len(devices)
    with native.Group(devices) as grp:
        assert grp.uses_nccl == (len(set(devices)) == n)
        for trial in range(3):
            cuts = sorted(rng.sample(range(1, text.size), n - 1)) if trial else [text.size * k // n for k in range(1, n)]
            if trial == 2 and n >= 3:
                cuts[1] = cuts[0] + 7  # a shard far shorter than a record: its neighbours' records run through it
            bounds = [0] + cuts + [text.size]
            bufs = put_shards(text, bounds, devices)
            cols = [pj.DeviceColumns(schema, abi.default_caps(schema, nrec_bound(text[bounds[g]:bounds[g + 1]]) + 4, bounds[g + 1] - bounds[g] + 65536), f"cuda:{devices[g]}")
                    for g in range(n)]
            shards = grp.parse(schema, bufs, [bounds[g + 1] - bounds[g] for g in range(n)], cols)
            starts, rec0, rows0 = [], 0, [0, 0, 0, 0]
            for g in range(n):
                lo, hi = bounds[g], bounds[g + 1]
                slack = int(shards[g].slack_bytes)
                assert slack == min(65536, text.size - hi)
                want = oracle.parse(schema, text[lo:hi + slack], slack=slack, is_first=lo == 0, is_last=hi + slack == text.size, goff=lo)
                assert same_result(want, cols[g]) == "", (trial, g)
                assert (int(shards[g].global_offset), int(shards[g].first_record), int(shards[g].bytes)) == (lo, rec0, hi - lo)
                assert [int(x) for x in shards[g].first_row][1:] == rows0[1:]
                rec0 += cols[g].n_records
                for t in (1, 2, 3):
                    rows0[t] += cols[g].n_rows(t)
                starts.append(cols[g].get("rec_start"))
                # the gathered table, as it lies on the shard's device (filled behind the call's back: wait for it)
                grp.sync()
                tab = read_device_u64(shards[g].table_dev, abi.PJ_GROUP_NCOUNT * n, devices[g]).reshape(n, abi.PJ_GROUP_NCOUNT)
                for h in range(n):
                    assert int(tab[h, abi.PJ_GC_BYTES]) == bounds[h + 1] - bounds[h]
                assert int(tab[g, abi.PJ_GC_RECORDS]) == cols[g].n_records and int(tab[g, abi.PJ_GC_ERRORS]) == cols[g].n_errors
            assert np.array_equal(np.concatenate(starts), whole.get("rec_start")), trial
            assert rec0 == whole.n_records


@pytest.mark.parametrize("devices", device_sets(), ids=lambda d: "dev" + "".join(map(str, d)))
@pytest.mark.parametrize("piece", [0, 5000])
def test_group_parse_of_a_host_stream(native, oracle, devices, piece):
    """pj_group_parse_host: the shards are ranges of one host buffer; every shard goes through the host-buffer route
    (in pieces when `piece` is set), host columns out."""
    rng = random.Random(3 + len(devices))
    schema = 4
    text = pj.gen_text(schema, 12, 0, 5000, abi.PJ_GEN_MALFORMED | abi.PJ_GEN_WHITESPACE)
    whole = oracle.parse(schema, text)
    n = len(devices)
    with native.Group(devices, host_piece_bytes=piece) as grp:
        for trial in range(2):
            cuts = sorted(rng.sample(range(1, text.size), n - 1)) if trial else [text.size * k // n for k in range(1, n)]
            bounds = [0] + cuts + [text.size]
            cols = [abi.HostColumns(schema, abi.default_caps(schema, nrec_bound(text[bounds[g]:bounds[g + 1]]) + 4, bounds[g + 1] - bounds[g] + 65536)) for g in range(n)]
            shards = grp.parse_host(schema, text, [bounds[g + 1] - bounds[g] for g in range(n)], cols)
            starts, rec0 = [], 0
            for g in range(n):
                lo, hi = bounds[g], bounds[g + 1]
                slack = int(shards[g].slack_bytes)
                assert slack == min(65536, text.size - hi)
                want = oracle.parse(schema, text[lo:hi + slack], slack=slack, is_first=lo == 0, is_last=hi + slack == text.size, goff=lo)
                assert same_result(want, cols[g]) == "", (trial, g)
                assert (int(shards[g].global_offset), int(shards[g].first_record), int(shards[g].bytes)) == (lo, rec0, hi - lo)
                rec0 += cols[g].n_records
                starts.append(cols[g].get("rec_start"))
            grp.sync()
            tab = read_device_u64(shards[0].table_dev, abi.PJ_GROUP_NCOUNT * n, devices[0]).reshape(n, abi.PJ_GROUP_NCOUNT)
            for h in range(n):
                assert int(tab[h, abi.PJ_GC_RECORDS]) == cols[h].n_records and int(tab[h, abi.PJ_GC_ERRORS]) == cols[h].n_errors
            assert np.array_equal(np.concatenate(starts), whole.get("rec_start")), trial
            assert rec0 == whole.n_records


@pytest.mark.parametrize("devices", device_sets()[:1] + device_sets()[2:3], ids=lambda d: "dev" + "".join(map(str, d)))
def test_group_write_concatenates_to_the_checkers_text(native, oracle, devices):
    import torch

    schema = 1
    n = len(devices)
    text = pj.gen_text(schema, 5, 0, 4000, abi.PJ_GEN_SPARSE | abi.PJ_GEN_ESCAPES)
    lines = bytes(text).split(b"\n")[:-1]
    per = (len(lines) + n - 1) // n
    parts = [as_u8(b"".join(ln + b"\n" for ln in lines[g * per:(g + 1) * per])) for g in range(n)]
    hosts = [oracle.parse(schema, p) for p in parts]
    want = [oracle.write(schema, h, 0, abi.PJ_INCLUDE_NON_NULL) for h in hosts]
    with native.Group(devices, inclusion=abi.PJ_INCLUDE_NON_NULL) as grp:
        dcols = [pj.DeviceColumns.from_host(h, f"cuda:{devices[g]}") for g, h in enumerate(hosts)]
        outs = [torch.zeros(w.size + 64, dtype=torch.uint8, device=f"cuda:{devices[g]}") for g, w in enumerate(want)]
        for dev in set(devices):
            torch.cuda.synchronize(dev)
        shards = grp.write(schema, dcols, outs)
        off = 0
        for g in range(n):
            assert (int(shards[g].bytes), int(shards[g].global_offset)) == (want[g].size, off)
            assert np.array_equal(outs[g][: want[g].size].cpu().numpy(), want[g])
            off += want[g].size
        # an output that is too small: the call reports it, the needed sizes are still exact
        outs[0] = outs[0][:100]
        with pytest.raises(native.PetJsonError) as e:
            grp.write(schema, dcols, outs)
        assert e.value.status == abi.PJ_ERR_CAPACITY
        shards = grp.write(schema, dcols, outs, allow_capacity=True)
        assert int(shards[0].bytes) == want[0].size


def test_group_of_one_and_bad_arguments(native):
    import torch

    with native.Group([0]) as grp:
        assert grp.uses_nccl
        text = pj.gen_text(2, 3, 0, 1000, 0)
        buf = put_shards(text, [0, text.size], [0])
        cols = [pj.DeviceColumns(2, abi.default_caps(2, 1000, text.size + 65536), "cuda:0")]
        shards = grp.parse(2, buf, [text.size], cols)
        assert cols[0].n_records == 1000 and int(shards[0].slack_bytes) == 0
    with pytest.raises(native.PetJsonError):
        native.Group([torch.cuda.device_count() + 3])
