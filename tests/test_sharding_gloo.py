"""The multi-rank path on CPU: `gloo` ranks exchange shard heads and counters exactly as the GPU ranks do
over NCCL; the per-shard parse is done by the CPU checker standing in for the CUDA context."""
import ctypes as C
import os
import tempfile

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pj_testlib import Oracle, abi, nrec_bound, pj, u32, u64

SCHEMA = abi.PJ_SCHEMA_MIXED
FLAGS = abi.PJ_GEN_MALFORMED | abi.PJ_GEN_ZIPF_LISTS | abi.PJ_GEN_ESCAPES
N_RECORDS = 3000
SLACK = 32 * 1024


class CheckerEngine:
    """parse_shard with the signature of petjson.Context, backed by oracle/ (CPU test stand-in)."""

    def __init__(self):
        self.oracle = Oracle()

    def parse_shard(self, schema, buf, length, slack, is_first, is_last, global_offset, out):
        a = buf.numpy()
        st = self.oracle.lib.pjo_parse(u32(schema), u32(0), C.c_void_p(a.ctypes.data), u64(length), u64(slack), int(is_first), int(is_last),
                                       u64(global_offset), C.byref(out.raw))
        assert st == 0


def _rank_main(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sharded = __import__("importlib").import_module("micronaut3-bug_b200.sharded")
    text = pj.gen_text(SCHEMA, 77, 0, N_RECORDS, FLAGS)
    lo, hi = sharded.split_even(text.size, world)[rank]
    buf = torch.zeros(hi - lo + SLACK, dtype=torch.uint8)
    buf[: hi - lo] = torch.from_numpy(text[lo:hi])
    out = abi.HostColumns(SCHEMA, abi.default_caps(SCHEMA, nrec_bound(text), text.size))
    parser = sharded.ShardedParser(CheckerEngine(), SCHEMA, SLACK)
    info = parser.parse(buf, hi - lo, out)
    np.savez(os.path.join(tmp, f"rank{rank}.npz"), **out.as_dict())
    # a second call on the same parser with other shard sizes (rank 0 takes 50 000 bytes more, the last rank fewer):
    # every rank must enter the size exchange again, whatever its own size did
    bounds = [b[0] for b in sharded.split_even(text.size, world)] + [text.size]
    bounds[1] += 50000
    lo2, hi2 = bounds[rank], bounds[rank + 1]
    buf2 = torch.zeros(hi2 - lo2 + SLACK, dtype=torch.uint8)
    buf2[: hi2 - lo2] = torch.from_numpy(text[lo2:hi2])
    out2 = abi.HostColumns(SCHEMA, abi.default_caps(SCHEMA, nrec_bound(text), text.size))
    info2 = parser.parse(buf2, hi2 - lo2, out2)
    info["second_call"] = (info2["total_records"], info2["first_record"], out2.n_records, info2["global_offset"] == lo2)
    torch.save(info, os.path.join(tmp, f"info{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_shards_stitch_to_the_whole_stream(oracle, native, world):
    port = 29600 + world + (os.getpid() % 200)
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_rank_main, args=(world, port, tmp), nprocs=world, join=True)
        text = pj.gen_text(SCHEMA, 77, 0, N_RECORDS, FLAGS)
        whole = oracle.parse(SCHEMA, text).as_dict()
        parts = [dict(np.load(os.path.join(tmp, f"rank{r}.npz"))) for r in range(world)]
        infos = [torch.load(os.path.join(tmp, f"info{r}.pt"), weights_only=False) for r in range(world)]
    assert sum(len(p["err_kind"]) for p in parts) == len(whole["err_kind"]) == infos[0]["total_records"]
    assert [i["first_record"] for i in infos] == list(np.cumsum([0] + [len(p["err_kind"]) for p in parts[:-1]]))
    # the second call, with other shard sizes, found the same stream
    assert all(i["second_call"][0] == len(whole["err_kind"]) and i["second_call"][3] for i in infos)
    assert sum(i["second_call"][2] for i in infos) == len(whole["err_kind"])
    # every shard used the exchanged head of its successor
    assert all(i["slack_used"] > 0 for i in infos[:-1]) and infos[-1]["slack_used"] == 0
    # re-assemble every column from the shards with the bases the stitch reported
    cols = {c.name: c for c in abi.schema_columns(SCHEMA)}
    arena_of = {"pet_photo_off": "pet_photo_str_off", "pet_tags_off": "pet_tag_id", "rec_row": None}
    for name, c in cols.items():
        pieces = []
        for r, p in enumerate(parts):
            a = p[name].astype(np.int64) if c.shape.endswith("+1") else p[name]
            if c.shape.endswith("+1"):
                # offsets are local to the shard's arena / child table: shift by that table's global base
                target = arena_of.get(name, name[:-4] + "_data" if name != "pet_photo_str_off" else "pet_photo_data")
                a = a + infos[r]["column_base"][target]
                if r < world - 1:
                    a = a[:-1]
            pieces.append(a)
        got = np.concatenate(pieces)
        if name == "rec_row":
            # rows are local to the shard's model tables
            got = got.astype(np.int64)
            at = 0
            for r, p in enumerate(parts):
                n = len(p["rec_row"])
                seg = got[at:at + n]
                types = p["rec_type"]
                for t in (1, 2, 3):
                    seg[types == t] += infos[r]["first_row"][t]
                at += n
            want = whole[name].astype(np.int64)
            want[whole["rec_type"] == 0] = 0xFFFFFFFF
            got[np.concatenate([p["rec_type"] for p in parts]) == 0] = 0xFFFFFFFF
            assert np.array_equal(got, want), name
            continue
        assert got.shape == whole[name].shape and np.array_equal(got.astype(np.int64), whole[name].astype(np.int64)), name
        assert infos[0]["column_total"][name] == whole[name].size
