"""ctypes mirror of include/petjson.h: constants, structs and a numpy-backed column set.

This module only describes the C ABI. It can wrap any shared library that exports functions over
`pj_columns` (the product library, or a checker built for the tests); it contains no parsing logic.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

# ---- call status ------------------------------------------------------------------------------
PJ_OK, PJ_ERR_ARG, PJ_ERR_CAPACITY, PJ_ERR_CUDA, PJ_ERR_TIMEOUT, PJ_ERR_NOMEM, PJ_ERR_TOO_LARGE = range(7)

# ---- per-record validation kinds ---------------------------------------------------------------
(PJ_E_NONE, PJ_E_SYNTAX, PJ_E_EOF, PJ_E_CTRL_CHAR, PJ_E_BAD_ESCAPE, PJ_E_BAD_SURROGATE, PJ_E_UTF8,
 PJ_E_TYPE, PJ_E_NUM_RANGE, PJ_E_ENUM, PJ_E_REQUIRED, PJ_E_DATETIME, PJ_E_DEPTH, PJ_E_AMBIGUOUS,
 PJ_E_TOO_LONG) = range(15)
ERROR_KIND_NAMES = ["NONE", "SYNTAX", "EOF", "CTRL_CHAR", "BAD_ESCAPE", "BAD_SURROGATE", "UTF8", "TYPE",
                    "NUM_RANGE", "ENUM", "REQUIRED", "DATETIME", "DEPTH", "AMBIGUOUS", "TOO_LONG"]

PJ_ERR_TIMEOUT = 4
PJ_ERR_NCCL = 7
PJ_MEM_HOST, PJ_MEM_DEVICE = 0, 1
PJ_SCHEMA_PET, PJ_SCHEMA_ORDER, PJ_SCHEMA_USER, PJ_SCHEMA_MIXED = 1, 2, 3, 4
PJ_TYPE_NONE, PJ_TYPE_PET, PJ_TYPE_ORDER, PJ_TYPE_USER = 0, 1, 2, 3
PJ_FRAMING_NDJSON, PJ_FRAMING_ARRAY = 0, 1
PJ_INCLUDE_NON_EMPTY, PJ_INCLUDE_NON_NULL, PJ_INCLUDE_ALWAYS = 0, 1, 2

PJ_GEN_ZIPF_LISTS, PJ_GEN_ESCAPES, PJ_GEN_WHITESPACE, PJ_GEN_MALFORMED, PJ_GEN_ARRAY, PJ_GEN_SPARSE = (
    1, 2, 4, 8, 16, 32)

PJ_OPT_ENUM_UNKNOWN_AS_NULL, PJ_OPT_LONE_SURROGATE_REPLACE, PJ_OPT_COERCE_SCALARS, PJ_OPT_HEX_LOWER = 1, 2, 4, 8
PJ_OPT_TEST_STALL_ONCE = 1 << 31

PJ_MAX_COLS = 64


@dataclass(frozen=True)
class Col:
    id: int
    name: str
    dtype: str      # numpy dtype string
    owner: int      # PJ_TYPE_* of the model table, 0 = per record
    shape: str      # "rows", "rows+1", "P", "P+1", "T", "T+1", "bytes"


COLUMNS = [
    Col(0, "rec_start", "u8", 0, "rows"),
    Col(1, "err_kind", "u1", 0, "rows"),
    Col(2, "err_off", "u4", 0, "rows"),
    Col(3, "rec_type", "u1", 0, "rows"),
    Col(4, "rec_row", "u4", 0, "rows"),
    Col(8, "pet_present", "u1", 1, "rows"),
    Col(9, "pet_id", "i8", 1, "rows"),
    Col(10, "pet_cat_present", "u1", 1, "rows"),
    Col(11, "pet_cat_id", "i8", 1, "rows"),
    Col(12, "pet_cat_name_off", "u4", 1, "rows+1"),
    Col(13, "pet_cat_name_data", "u1", 1, "bytes"),
    Col(14, "pet_name_off", "u4", 1, "rows+1"),
    Col(15, "pet_name_data", "u1", 1, "bytes"),
    Col(16, "pet_photo_off", "u4", 1, "rows+1"),
    Col(17, "pet_photo_str_off", "u4", 1, "P+1"),
    Col(18, "pet_photo_data", "u1", 1, "bytes"),
    Col(19, "pet_tags_off", "u4", 1, "rows+1"),
    Col(20, "pet_tag_present", "u1", 1, "T"),
    Col(21, "pet_tag_id", "i8", 1, "T"),
    Col(22, "pet_tag_name_off", "u4", 1, "T+1"),
    Col(23, "pet_tag_name_data", "u1", 1, "bytes"),
    Col(24, "pet_status", "u1", 1, "rows"),
    Col(32, "ord_present", "u1", 2, "rows"),
    Col(33, "ord_id", "i8", 2, "rows"),
    Col(34, "ord_pet_id", "i8", 2, "rows"),
    Col(35, "ord_quantity", "i4", 2, "rows"),
    Col(36, "ord_ship_epoch", "i8", 2, "rows"),
    Col(37, "ord_ship_nanos", "i4", 2, "rows"),
    Col(38, "ord_ship_offset", "i4", 2, "rows"),
    Col(39, "ord_status", "u1", 2, "rows"),
    Col(40, "ord_complete", "u1", 2, "rows"),
    Col(44, "usr_present", "u1", 3, "rows"),
    Col(45, "usr_id", "i8", 3, "rows"),
    Col(46, "usr_username_off", "u4", 3, "rows+1"),
    Col(47, "usr_username_data", "u1", 3, "bytes"),
    Col(48, "usr_firstname_off", "u4", 3, "rows+1"),
    Col(49, "usr_firstname_data", "u1", 3, "bytes"),
    Col(50, "usr_lastname_off", "u4", 3, "rows+1"),
    Col(51, "usr_lastname_data", "u1", 3, "bytes"),
    Col(52, "usr_email_off", "u4", 3, "rows+1"),
    Col(53, "usr_email_data", "u1", 3, "bytes"),
    Col(54, "usr_password_off", "u4", 3, "rows+1"),
    Col(55, "usr_password_data", "u1", 3, "bytes"),
    Col(56, "usr_phone_off", "u4", 3, "rows+1"),
    Col(57, "usr_phone_data", "u1", 3, "bytes"),
    Col(58, "usr_status", "i4", 3, "rows"),
]
COL_BY_ID = {c.id: c for c in COLUMNS}
COL_BY_NAME = {c.name: c for c in COLUMNS}


def schema_columns(schema: int) -> list[Col]:
    """Columns a parse of `schema` produces."""
    out = []
    for c in COLUMNS:
        if c.owner == 0:
            if c.id in (3, 4) and schema != PJ_SCHEMA_MIXED:
                continue
            out.append(c)
        elif schema == PJ_SCHEMA_MIXED or c.owner == schema:
            out.append(c)
    return out


class pj_buf(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("bytes", C.c_uint64), ("count", C.c_uint64)]


class pj_columns(C.Structure):
    _fields_ = [("schema", C.c_uint32), ("mem_kind", C.c_uint32), ("n_records", C.c_uint64),
                ("n_errors", C.c_uint64), ("n_rows", C.c_uint64 * 4), ("doc_err_off", C.c_uint64),
                ("doc_err_kind", C.c_uint32), ("reserved", C.c_uint32), ("col", pj_buf * PJ_MAX_COLS)]


class pj_options(C.Structure):
    _fields_ = [("device", C.c_int32), ("inclusion", C.c_int32), ("stream", C.c_void_p),
                ("flags", C.c_uint32), ("host_piece_bytes", C.c_uint32), ("tile_bytes", C.c_uint32), ("spin_limit_us", C.c_uint32),
                ("device_piece_bytes", C.c_uint32), ("reserved", C.c_uint32)]


PJ_GROUP_NCOUNT = 24
PJ_GC_RECORDS, PJ_GC_ERRORS, PJ_GC_BYTES, PJ_GC_ROWS_PET, PJ_GC_ROWS_ORDER, PJ_GC_ROWS_USER, PJ_GC_COUNTER0 = 0, 1, 2, 3, 4, 5, 8


class pj_group_shard(C.Structure):
    _fields_ = [("global_offset", C.c_uint64), ("first_record", C.c_uint64), ("first_row", C.c_uint64 * 4), ("bytes", C.c_uint64),
                ("slack_bytes", C.c_uint64), ("table_dev", C.c_void_p), ("status", C.c_int32), ("slack_copy_ms", C.c_float), ("gather_ms", C.c_float), ("reserved", C.c_uint32)]


class pj_call_stats(C.Structure):
    _fields_ = [("kernel_launches", C.c_uint32), ("pieces", C.c_uint32), ("device_ms", C.c_float),
                ("main_kernel_ms", C.c_float), ("stage_ms", C.c_float * 8), ("stage_launches", C.c_uint32 * 8),
                ("h2d_bytes", C.c_uint64), ("d2h_bytes", C.c_uint64),
                ("algorithmic_bytes", C.c_uint64), ("fast_records", C.c_uint64), ("phase_cycles", C.c_uint64 * 4),
                ("lookback_polls", C.c_uint64), ("lookback_rounds", C.c_uint64), ("tile_records", C.c_uint32), ("tiles", C.c_uint32),
                ("wide_records", C.c_uint64), ("wide_fast_records", C.c_uint64), ("wide_cycles", C.c_uint64 * 2)]


class HostColumns:
    """A pj_columns whose buffers are numpy arrays in host memory."""

    def __init__(self, schema: int, byte_caps: dict[int, int], alloc=None):
        """`alloc(nbytes)` may supply the uint8 arrays (e.g. views of pinned memory); default: np.zeros."""
        self.schema = schema
        self.raw = pj_columns()
        self.raw.schema = schema
        self.raw.mem_kind = PJ_MEM_HOST
        self.arrays: dict[int, np.ndarray] = {}
        for c in schema_columns(schema):
            nbytes = max(int(byte_caps.get(c.id, 0)), 16)
            a = alloc(nbytes) if alloc else np.zeros(nbytes, dtype=np.uint8)
            self.arrays[c.id] = a
            self.raw.col[c.id].ptr = a.ctypes.data
            self.raw.col[c.id].bytes = nbytes
            self.raw.col[c.id].count = 0

    def count(self, col: int) -> int:
        return int(self.raw.col[col].count)

    def get(self, name_or_id) -> np.ndarray:
        c = COL_BY_NAME[name_or_id] if isinstance(name_or_id, str) else COL_BY_ID[name_or_id]
        n = self.count(c.id)
        return self.arrays[c.id].view(np.dtype(c.dtype))[:n] if n else np.zeros(0, np.dtype(c.dtype))

    @property
    def n_records(self) -> int:
        return int(self.raw.n_records)

    @property
    def n_errors(self) -> int:
        return int(self.raw.n_errors)

    def n_rows(self, t: int) -> int:
        return int(self.raw.n_rows[t])

    def as_dict(self) -> dict[str, np.ndarray]:
        return {c.name: self.get(c.id).copy() for c in schema_columns(self.schema)}

    def set_counts_from(self, arrays: dict[str, np.ndarray], n_records: int, n_rows) -> None:
        """Loads values (for pj_write): copies arrays in and sets the counts."""
        for name, a in arrays.items():
            c = COL_BY_NAME[name]
            buf = self.arrays[c.id]
            b = np.ascontiguousarray(a).view(np.uint8).reshape(-1)
            assert b.size <= buf.size, (name, b.size, buf.size)
            buf[: b.size] = b
            self.raw.col[c.id].count = a.size
        self.raw.n_records = n_records
        for t in range(4):
            self.raw.n_rows[t] = int(n_rows[t])


def columns_equal(a: dict[str, np.ndarray], b: dict[str, np.ndarray]) -> list[str]:
    """Names of the columns that differ (length or any element)."""
    bad = []
    for k in a:
        if k not in b or a[k].shape != b[k].shape or not np.array_equal(a[k], b[k]):
            bad.append(k)
    for k in b:
        if k not in a:
            bad.append(k)
    return bad


def default_caps(schema: int, n_records: int, in_bytes: int, list_items: int | None = None) -> dict[int, int]:
    """Generous host-side capacities: enough for any input of `in_bytes` bytes with `n_records` records."""
    items = list_items if list_items is not None else in_bytes // 2 + 1
    caps = {}
    for c in schema_columns(schema):
        w = np.dtype(c.dtype).itemsize
        if c.shape == "bytes":
            caps[c.id] = in_bytes + 16
        elif c.shape in ("rows", "rows+1"):
            caps[c.id] = (n_records + 1) * w
        else:
            caps[c.id] = (items + 1) * w
    return caps
