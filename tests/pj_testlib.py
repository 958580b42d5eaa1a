"""Shared helpers of the test suite: the package, the CPU checker (oracle/) and column decoding."""
from __future__ import annotations

import ctypes as C
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

pj = importlib.import_module("micronaut3-bug_b200")
abi = importlib.import_module("micronaut3-bug_b200.abi")
build = importlib.import_module("micronaut3-bug_b200.build")
build.build_generator()  # host-only C: the seeded inputs of every test

u32, u64 = C.c_uint32, C.c_uint64

SCHEMA_BY_NAME = {"pet": abi.PJ_SCHEMA_PET, "order": abi.PJ_SCHEMA_ORDER, "user": abi.PJ_SCHEMA_USER, "mixed": abi.PJ_SCHEMA_MIXED}
KIND_BY_NAME = {n: i for i, n in enumerate(abi.ERROR_KIND_NAMES)}

PET_STATUS = ["available", "pending", "sold"]
ORD_STATUS = ["placed", "approved", "delivered"]


def nrec_bound(buf: np.ndarray) -> int:
    """No more records than LFs + commas + 2."""
    return int(np.count_nonzero(buf == 10) + np.count_nonzero(buf == ord(",")) + 2)


class Oracle:
    """ctypes binding of oracle/libpj_oracle.so (the CPU checker)."""

    def __init__(self):
        path = build.build_oracle()
        self.lib = C.CDLL(path)

    def parse(self, schema, buf, framing=0, slack=0, is_first=1, is_last=1, goff=0, opts=0, caps=None) -> "abi.HostColumns":
        buf = np.ascontiguousarray(buf, dtype=np.uint8)
        hc = abi.HostColumns(schema, caps if caps is not None else abi.default_caps(schema, nrec_bound(buf), buf.size))
        st = self.lib.pjo_parse_opt(u32(schema), u32(framing), C.c_void_p(buf.ctypes.data), u64(buf.size - slack), u64(slack),
                                    int(is_first), int(is_last), u64(goff), u32(opts), C.byref(hc.raw))
        assert st == 0, st
        return hc

    def write(self, schema, cols, framing=0, inclusion=0, cap=None, opts=0) -> np.ndarray:
        if cap is None:
            ln = u64()
            self.lib.pjo_write_opt(u32(schema), u32(framing), int(inclusion), u32(opts), C.byref(cols.raw), None, u64(0), C.byref(ln))
            cap = ln.value
        out = np.zeros(max(cap, 1), np.uint8)
        ln = u64()
        st = self.lib.pjo_write_opt(u32(schema), u32(framing), int(inclusion), u32(opts), C.byref(cols.raw), C.c_void_p(out.ctypes.data), u64(cap), C.byref(ln))
        assert st == 0, st
        return out[: ln.value]

    def checksums(self, cols) -> dict:
        """{column name: 64-bit checksum} of a host column set, by the definition of pj_columns_checksum."""
        self.lib.pjo_checksum_bytes.restype = C.c_uint64
        self.lib.pjo_checksum_bytes.argtypes = [C.c_void_p, C.c_uint64]
        out = {}
        for c in abi.schema_columns(cols.schema):
            a = cols.get(c.id)
            out[c.name] = int(self.lib.pjo_checksum_bytes(a.ctypes.data, a.nbytes)) if a.size else 0
        return out

    def index(self, buf, framing=0) -> np.ndarray:
        buf = np.ascontiguousarray(buf, dtype=np.uint8)
        cap = nrec_bound(buf)
        rs = np.zeros(cap, np.uint64)
        n = u64()
        st = self.lib.pjo_index(u32(framing), C.c_void_p(buf.ctypes.data), u64(buf.size), C.c_void_p(rs.ctypes.data), u64(cap), C.byref(n))
        assert st == 0
        return rs[: n.value]


def as_u8(data) -> np.ndarray:
    if isinstance(data, str):
        data = data.encode("utf-8")
    if isinstance(data, (bytes, bytearray)):
        return np.frombuffer(bytes(data), np.uint8).copy()
    return np.ascontiguousarray(data, dtype=np.uint8)


def _s(cols, off_name, row):
    off = cols[off_name]
    data = cols["pet_photo_data" if off_name == "pet_photo_str_off" else off_name[:-4] + "_data"]
    return bytes(data[off[row]: off[row + 1]]).decode("utf-8", "surrogatepass")


def pet_record(cols, r):
    pr = int(cols["pet_present"][r])
    d = {}
    if pr & 1:
        d["id"] = int(cols["pet_id"][r])
    if pr & 2:
        cp = int(cols["pet_cat_present"][r])
        c = {}
        if cp & 1:
            c["id"] = int(cols["pet_cat_id"][r])
        if cp & 2:
            c["name"] = _s(cols, "pet_cat_name_off", r)
        d["category"] = c
    if pr & 4:
        d["name"] = _s(cols, "pet_name_off", r)
    if pr & 8:
        lo = cols["pet_photo_off"]
        d["photoUrls"] = [_s(cols, "pet_photo_str_off", k) for k in range(lo[r], lo[r + 1])]
    if pr & 16:
        lo = cols["pet_tags_off"]
        tags = []
        for k in range(lo[r], lo[r + 1]):
            tp = int(cols["pet_tag_present"][k])
            t = {}
            if tp & 1:
                t["id"] = int(cols["pet_tag_id"][k])
            if tp & 2:
                t["name"] = _s(cols, "pet_tag_name_off", k)
            tags.append(t)
        d["tags"] = tags
    if pr & 32:
        d["status"] = PET_STATUS[int(cols["pet_status"][r])]
    return d


def order_record(cols, r):
    pr = int(cols["ord_present"][r])
    d = {}
    if pr & 1:
        d["id"] = int(cols["ord_id"][r])
    if pr & 2:
        d["petId"] = int(cols["ord_pet_id"][r])
    if pr & 4:
        d["quantity"] = int(cols["ord_quantity"][r])
    if pr & 8:
        d["shipDate"] = (int(cols["ord_ship_epoch"][r]), int(cols["ord_ship_nanos"][r]), int(cols["ord_ship_offset"][r]))
    if pr & 16:
        d["status"] = ORD_STATUS[int(cols["ord_status"][r])]
    if pr & 32:
        d["complete"] = bool(cols["ord_complete"][r])
    return d


USER_STR = ["username", "firstName", "lastName", "email", "password", "phone"]


def user_record(cols, r):
    pr = int(cols["usr_present"][r])
    d = {}
    if pr & 1:
        d["id"] = int(cols["usr_id"][r])
    for f, k in enumerate(USER_STR):
        if pr & (2 << f):
            d[k] = _s(cols, f"usr_{k.lower()}_off", r)
    if pr & 128:
        d["userStatus"] = int(cols["usr_status"][r])
    return d


def records(cols: dict, schema: int) -> list:
    """Decoded records in input order: dict for an accepted record, (kind, offset) tuple for a failed one."""
    out = []
    n = len(cols["err_kind"])
    fn = {1: pet_record, 2: order_record, 3: user_record}
    for i in range(n):
        if cols["err_kind"][i]:
            out.append((abi.ERROR_KIND_NAMES[int(cols["err_kind"][i])], int(cols["err_off"][i])))
            continue
        if schema == abi.PJ_SCHEMA_MIXED:
            t, r = int(cols["rec_type"][i]), int(cols["rec_row"][i])
        else:
            t, r = schema, i
        out.append(fn[t](cols, r))
    return out


def diff_columns(a: dict, b: dict, limit=5) -> str:
    """Human-readable first differences between two column dicts ('' when equal)."""
    msgs = []
    for k in sorted(set(a) | set(b)):
        if k not in a or k not in b:
            msgs.append(f"{k}: missing on one side")
            continue
        x, y = a[k], b[k]
        if x.shape != y.shape:
            msgs.append(f"{k}: {x.shape} vs {y.shape}")
            continue
        if not np.array_equal(x, y):
            idx = np.nonzero(x != y)[0][:limit]
            msgs.append(f"{k}: at {idx.tolist()} {x[idx].tolist()} vs {y[idx].tolist()}")
    return "; ".join(msgs)


def same_result(a, b) -> str:
    """Compares two column sets (HostColumns / DeviceColumns): '' when identical."""
    meta_a = (a.n_records, a.n_errors, [a.n_rows(t) for t in range(4)])
    meta_b = (b.n_records, b.n_errors, [b.n_rows(t) for t in range(4)])
    msg = "" if meta_a == meta_b else f"meta {meta_a} vs {meta_b}; "
    return msg + diff_columns(a.as_dict(), b.as_dict())
