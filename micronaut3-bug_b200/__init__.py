"""petjson for B200: JSON parse / validate / re-serialise of the Petstore models on sm_100a.

This package is a thin ctypes binding of the C ABI in include/petjson.h (libpetjson.so, built
in-tree by `build.py`) plus helpers that hold column sets in torch device tensors. All parsing,
validation and serialisation happens in the CUDA kernels behind that ABI; there is no Python or CPU
implementation of the path here, and loading fails loudly when the native library is missing.

The directory name contains a hyphen, so import it with
    importlib.import_module("micronaut3-bug_b200")
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import abi
from .abi import *  # noqa: F401,F403  (constants and struct mirrors)

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libpetjson.so")
_lib = None

u32, u64, i32 = C.c_uint32, C.c_uint64, C.c_int32


class PetJsonError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        super().__init__(f"{where}: status {status} {detail}".strip())


def lib() -> C.CDLL:
    """The native library; raises if it has not been built (there is no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise ImportError(f"{LIB_PATH} is missing: run `python {os.path.join(_PKG, 'build.py')}` (needs nvcc)")
        L = C.CDLL(LIB_PATH)
        L.pj_version.restype = i32
        L.pj_status_str.restype = C.c_char_p
        L.pj_status_str.argtypes = [i32]
        L.pj_error_kind_str.restype = C.c_char_p
        L.pj_error_kind_str.argtypes = [i32]
        L.pj_column_info.argtypes = [i32, C.POINTER(C.c_char_p), C.POINTER(u32), C.POINTER(u32)]
        L.pj_create.argtypes = [C.POINTER(abi.pj_options), C.POINTER(C.c_void_p)]
        L.pj_destroy.argtypes = [C.c_void_p]
        L.pj_destroy.restype = None
        L.pj_last_error.argtypes = [C.c_void_p]
        L.pj_last_error.restype = C.c_char_p
        L.pj_last_stats.argtypes = [C.c_void_p, C.POINTER(abi.pj_call_stats)]
        L.pj_trim.argtypes = [C.c_void_p]
        L.pj_columns_sizes.argtypes = [u32, u64, u64, u64, C.POINTER(abi.pj_columns)]
        L.pj_parse.argtypes = [C.c_void_p, u32, u32, C.c_void_p, u64, u32, C.POINTER(abi.pj_columns)]
        L.pj_parse_shard.argtypes = [C.c_void_p, u32, C.c_void_p, u64, u64, i32, i32, u64, u32, C.POINTER(abi.pj_columns)]
        L.pj_index_records.argtypes = [C.c_void_p, u32, C.c_void_p, u64, u32, C.c_void_p, u64, C.POINTER(u64)]
        L.pj_index_records_static.argtypes = [C.c_void_p, u64, C.c_void_p, u64, C.c_void_p, C.c_void_p]
        L.pj_write.argtypes = [C.c_void_p, u32, u32, C.POINTER(abi.pj_columns), C.c_void_p, u64, u32, C.POINTER(u64)]
        L.pj_columns_checksum.argtypes = [C.c_void_p, u32, C.POINTER(abi.pj_columns), C.POINTER(u64)]
        L.pj_group_create.argtypes = [i32, C.POINTER(i32), C.POINTER(abi.pj_options), C.POINTER(C.c_void_p)]
        L.pj_group_destroy.argtypes = [C.c_void_p]
        L.pj_group_destroy.restype = None
        L.pj_group_size.argtypes = [C.c_void_p]
        L.pj_group_ctx.argtypes = [C.c_void_p, i32]
        L.pj_group_ctx.restype = C.c_void_p
        L.pj_group_last_error.argtypes = [C.c_void_p]
        L.pj_group_last_error.restype = C.c_char_p
        L.pj_group_uses_nccl.argtypes = [C.c_void_p]
        L.pj_group_sync.argtypes = [C.c_void_p]
        L.pj_group_parse_host.argtypes = [C.c_void_p, u32, C.c_void_p, C.POINTER(u64), u64, C.POINTER(abi.pj_columns), C.POINTER(abi.pj_group_shard)]
        L.pj_group_parse_host.restype = C.c_int
        L.pj_group_sync.restype = C.c_int
        L.pj_group_parse.argtypes = [C.c_void_p, u32, C.POINTER(C.c_void_p), C.POINTER(u64), C.POINTER(u64), u64, C.POINTER(abi.pj_columns),
                                     C.POINTER(abi.pj_group_shard)]
        L.pj_group_write.argtypes = [C.c_void_p, u32, C.POINTER(abi.pj_columns), C.POINTER(C.c_void_p), C.POINTER(u64), C.POINTER(abi.pj_group_shard)]
        _lib = L
    return _lib


GEN_LIB_PATH = os.path.join(_PKG, "libpj_gen.so")
_gen_lib = None


def gen_lib() -> C.CDLL:
    """The seeded workload generator (host-only C, include/petjson_gen.h): a library of its own, so that a
    process which needs inputs but not the GPU path (the CPU baseline) maps nothing of libpetjson.so."""
    global _gen_lib
    if _gen_lib is None:
        if not os.path.exists(GEN_LIB_PATH):
            raise ImportError(f"{GEN_LIB_PATH} is missing: run `python {os.path.join(_PKG, 'build.py')}`")
        L = C.CDLL(GEN_LIB_PATH)
        L.pj_gen_text.argtypes = [u32, u64, u64, u64, u32, C.c_void_p, u64, C.POINTER(u64)]
        L.pj_gen_columns.argtypes = [u32, u64, u64, u64, u32, C.POINTER(abi.pj_columns)]
        _gen_lib = L
    return _gen_lib


# ---- seeded workloads (host) -------------------------------------------------------------------
def gen_text(schema: int, seed: int, first: int, n: int, flags: int = 0, out: np.ndarray | None = None) -> np.ndarray:
    """JSON text of records [first, first+n) of stream `seed` as a uint8 array."""
    L = gen_lib()
    ln = u64()
    if out is None:
        L.pj_gen_text(schema, seed, first, n, flags, None, 0, C.byref(ln))
        out = np.empty(ln.value, np.uint8)
    st = L.pj_gen_text(schema, seed, first, n, flags, out.ctypes.data, out.size, C.byref(ln))
    if st != abi.PJ_OK:
        raise PetJsonError(st, "pj_gen_text")
    return out[: ln.value]


def gen_columns(schema: int, seed: int, first: int, n: int, flags: int, text_bytes: int) -> abi.HostColumns:
    """The values of the same records as host columns."""
    hc = abi.HostColumns(schema, abi.default_caps(schema, n, text_bytes))
    st = gen_lib().pj_gen_columns(schema, seed, first, n, flags, C.byref(hc.raw))
    if st != abi.PJ_OK:
        raise PetJsonError(st, "pj_gen_columns")
    return hc


# ---- device column sets --------------------------------------------------------------------------
class DeviceColumns:
    """A pj_columns whose buffers are torch uint8 tensors on one CUDA device."""

    def __init__(self, schema: int, byte_caps: dict[int, int], device):
        import torch

        self.schema = schema
        self.device = torch.device(device)
        self.raw = abi.pj_columns()
        self.raw.schema = schema
        self.raw.mem_kind = abi.PJ_MEM_DEVICE
        self.tensors = {}
        for c in abi.schema_columns(schema):
            nbytes = max(int(byte_caps.get(c.id, 0)), 16)
            t = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
            self.tensors[c.id] = t
            self.raw.col[c.id].ptr = t.data_ptr()
            self.raw.col[c.id].bytes = nbytes
            self.raw.col[c.id].count = 0

    @classmethod
    def sized_for(cls, schema: int, max_records: int, max_input_bytes: int, max_list_items: int, device) -> "DeviceColumns":
        probe = abi.pj_columns()
        st = lib().pj_columns_sizes(schema, max_records, max_input_bytes, max_list_items, C.byref(probe))
        if st != abi.PJ_OK:
            raise PetJsonError(st, "pj_columns_sizes")
        return cls(schema, {c.id: int(probe.col[c.id].bytes) for c in abi.schema_columns(schema)}, device)

    @classmethod
    def from_host(cls, hc: abi.HostColumns, device) -> "DeviceColumns":
        """Uploads a host column set (values and counts)."""
        import torch

        caps = {c.id: max(hc.count(c.id) * np.dtype(c.dtype).itemsize, 16) for c in abi.schema_columns(hc.schema)}
        dc = cls(hc.schema, caps, device)
        for c in abi.schema_columns(hc.schema):
            nb = hc.count(c.id) * np.dtype(c.dtype).itemsize
            if nb:
                dc.tensors[c.id][:nb].copy_(torch.from_numpy(hc.arrays[c.id][:nb]))
            dc.raw.col[c.id].count = hc.count(c.id)
        dc.raw.n_records = hc.raw.n_records
        dc.raw.n_errors = hc.raw.n_errors
        for t in range(4):
            dc.raw.n_rows[t] = hc.raw.n_rows[t]
        return dc

    def count(self, col: int) -> int:
        return int(self.raw.col[col].count)

    @property
    def n_records(self) -> int:
        return int(self.raw.n_records)

    @property
    def n_errors(self) -> int:
        return int(self.raw.n_errors)

    def n_rows(self, t: int) -> int:
        return int(self.raw.n_rows[t])

    def get(self, name_or_id) -> np.ndarray:
        """One column copied to the host as a typed numpy array."""
        c = abi.COL_BY_NAME[name_or_id] if isinstance(name_or_id, str) else abi.COL_BY_ID[name_or_id]
        n = self.count(c.id)
        dt = np.dtype(c.dtype)
        if not n:
            return np.zeros(0, dt)
        return self.tensors[c.id][: n * dt.itemsize].cpu().numpy().view(dt).copy()

    def as_dict(self) -> dict[str, np.ndarray]:
        return {c.name: self.get(c.id) for c in abi.schema_columns(self.schema)}

    def total_bytes(self) -> int:
        return sum(self.count(c.id) * np.dtype(c.dtype).itemsize for c in abi.schema_columns(self.schema))


# ---- context ----------------------------------------------------------------------------------
class Context:
    """One pj_ctx: a (device, stream) pair with its scratch memory. Not for concurrent use."""

    def __init__(self, device: int = -1, inclusion: int = abi.PJ_INCLUDE_NON_EMPTY, stream: int | None = None, flags: int = 0,
                 host_piece_bytes: int = 0, tile_bytes: int = 0, spin_limit_us: int = 0, device_piece_bytes: int = 0):
        self._h = C.c_void_p()
        opt = abi.pj_options()
        opt.device = device
        opt.inclusion = inclusion
        opt.stream = stream
        opt.flags = flags
        opt.host_piece_bytes = host_piece_bytes
        opt.tile_bytes = tile_bytes
        opt.spin_limit_us = spin_limit_us
        opt.device_piece_bytes = device_piece_bytes
        st = lib().pj_create(C.byref(opt), C.byref(self._h))
        if st != abi.PJ_OK:
            raise PetJsonError(st, "pj_create", (lib().pj_last_error(None) or b"").decode())

    def close(self) -> None:
        if self._h:
            lib().pj_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def last_error(self) -> str:
        return (lib().pj_last_error(self._h) or b"").decode()

    def stats(self) -> abi.pj_call_stats:
        s = abi.pj_call_stats()
        lib().pj_last_stats(self._h, C.byref(s))
        return s

    def _check(self, st: int, where: str, allow=()):
        if st != abi.PJ_OK and st not in allow:
            raise PetJsonError(st, where, self.last_error())
        return st

    @staticmethod
    def _ptr_len_kind(buf):
        """(address, byte length, memory kind) of a numpy array or torch tensor."""
        if isinstance(buf, np.ndarray):
            assert buf.dtype == np.uint8 and buf.flags.c_contiguous
            return buf.ctypes.data, buf.size, abi.PJ_MEM_HOST
        import torch

        assert isinstance(buf, torch.Tensor) and buf.dtype == torch.uint8 and buf.is_contiguous()
        kind = abi.PJ_MEM_DEVICE if buf.is_cuda else abi.PJ_MEM_HOST
        return buf.data_ptr(), buf.numel(), kind

    def parse(self, schema: int, buf, out, framing: int = abi.PJ_FRAMING_NDJSON, allow_capacity: bool = False) -> int:
        """pj_parse of `buf` (numpy / torch uint8, host or device) into `out` (HostColumns / DeviceColumns)."""
        p, n, kind = self._ptr_len_kind(buf)
        st = lib().pj_parse(self._h, schema, framing, p, n, kind, C.byref(out.raw))
        return self._check(st, "pj_parse", (abi.PJ_ERR_CAPACITY,) if allow_capacity else ())

    def parse_shard(self, schema: int, buf, length: int, slack: int, is_first: bool, is_last: bool, global_offset: int,
                    out, allow_capacity: bool = False) -> int:
        p, n, kind = self._ptr_len_kind(buf)
        assert length + slack <= n
        st = lib().pj_parse_shard(self._h, schema, p, length, slack, int(is_first), int(is_last), global_offset, kind,
                                  C.byref(out.raw))
        return self._check(st, "pj_parse_shard", (abi.PJ_ERR_CAPACITY,) if allow_capacity else ())

    def index_records(self, buf, rec_start, framing: int = abi.PJ_FRAMING_NDJSON, allow_capacity: bool = False) -> int:
        """Record index only; rec_start is a uint64 numpy array (host input) or int64/uint64-sized torch tensor."""
        p, n, kind = self._ptr_len_kind(buf)
        if isinstance(rec_start, np.ndarray):
            rp, cap = rec_start.ctypes.data, rec_start.size
        else:
            rp, cap = rec_start.data_ptr(), rec_start.numel()
        cnt = u64()
        st = lib().pj_index_records(self._h, framing, p, n, kind, rp, cap, C.byref(cnt))
        self._check(st, "pj_index_records", (abi.PJ_ERR_CAPACITY,) if allow_capacity else ())
        return int(cnt.value)

    def checksums(self, schema: int, cols) -> dict:
        """{column name: 64-bit checksum} of a device-resident column set (pj_columns_checksum)."""
        sums = (u64 * abi.PJ_MAX_COLS)()
        self._check(lib().pj_columns_checksum(self._h, schema, C.byref(cols.raw), sums), "pj_columns_checksum")
        return {c.name: int(sums[c.id]) for c in abi.schema_columns(schema)}

    def write(self, schema: int, cols, out, framing: int = abi.PJ_FRAMING_NDJSON, allow_capacity: bool = False) -> int:
        """pj_write of `cols` into `out` (numpy / torch uint8); returns the JSON length in bytes."""
        p, cap, kind = self._ptr_len_kind(out)
        ln = u64()
        st = lib().pj_write(self._h, schema, framing, C.byref(cols.raw), p, cap, kind, C.byref(ln))
        self._check(st, "pj_write", (abi.PJ_ERR_CAPACITY,) if allow_capacity else ())
        return int(ln.value)


def index_records_static(buf, rec_start, n_out, stream: int | None = None) -> None:
    """pj_index_records_static: the allocation-free record index. `buf` (uint8), `rec_start` (8-byte elements)
    and `n_out` (one 8-byte element) are CUDA tensors on the current device; the work is only enqueued on
    `stream` (a raw cudaStream_t value, default stream when None), so synchronise before reading."""
    assert buf.is_cuda and rec_start.is_cuda and n_out.is_cuda and buf.is_contiguous()
    st = lib().pj_index_records_static(buf.data_ptr(), buf.numel(), rec_start.data_ptr(), rec_start.numel(), n_out.data_ptr(), stream)
    if st != abi.PJ_OK:
        raise PetJsonError(st, "pj_index_records_static", (lib().pj_last_error(None) or b"").decode())


class Group:
    """Several GPUs of one machine behind one handle (pj_group_*): one context, stream and host thread per shard inside
    the library. `devices` may repeat a device (several shards on one GPU; the counter table then goes through the
    host instead of NCCL)."""

    def __init__(self, devices, inclusion: int = abi.PJ_INCLUDE_NON_EMPTY, tile_bytes: int = 0, spin_limit_us: int = 0, host_piece_bytes: int = 0):
        self.devices = [int(d) for d in devices]
        self._h = C.c_void_p()
        opt = abi.pj_options()
        opt.device = -1
        opt.inclusion = inclusion
        opt.tile_bytes = tile_bytes
        opt.spin_limit_us = spin_limit_us
        opt.host_piece_bytes = host_piece_bytes
        devs = (i32 * len(self.devices))(*self.devices)
        st = lib().pj_group_create(len(self.devices), devs, C.byref(opt), C.byref(self._h))
        if st != abi.PJ_OK:
            raise PetJsonError(st, "pj_group_create", (lib().pj_last_error(None) or b"").decode())

    def close(self) -> None:
        if self._h:
            lib().pj_group_destroy(self._h)
            self._h = C.c_void_p()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def uses_nccl(self) -> bool:
        return bool(lib().pj_group_uses_nccl(self._h))

    def stats(self, i: int) -> abi.pj_call_stats:
        s = abi.pj_call_stats()
        lib().pj_last_stats(lib().pj_group_ctx(self._h, i), C.byref(s))
        return s

    def sync(self) -> None:
        """pj_group_sync: the device tables (pj_group_shard.table_dev) of the last call are complete on return."""
        st = lib().pj_group_sync(self._h)
        if st != abi.PJ_OK:
            raise PetJsonError(st, "pj_group_sync", (lib().pj_group_last_error(self._h) or b"").decode())

    def _cols_array(self, cols):
        arr = (abi.pj_columns * len(cols))()
        for k, c in enumerate(cols):
            C.memmove(C.byref(arr[k]), C.byref(c.raw), C.sizeof(abi.pj_columns))
        return arr

    def parse(self, schema: int, bufs, lengths, cols, slack: int = 65536, allow_capacity: bool = False):
        """bufs[g]: a uint8 CUDA tensor on device g holding lengths[g] bytes of shard g and writable room behind them;
        cols[g]: DeviceColumns on device g. Returns the list of pj_group_shard."""
        n = len(self.devices)
        ptrs = (C.c_void_p * n)(*[int(b.data_ptr()) for b in bufs])
        lens = (u64 * n)(*[int(x) for x in lengths])
        room = (u64 * n)(*[int(b.numel()) - int(x) for b, x in zip(bufs, lengths)])
        arr = self._cols_array(cols)
        shards = (abi.pj_group_shard * n)()
        st = lib().pj_group_parse(self._h, schema, ptrs, lens, room, slack, arr, shards)
        for k, c in enumerate(cols):
            C.memmove(C.byref(c.raw), C.byref(arr[k]), C.sizeof(abi.pj_columns))
        if st != abi.PJ_OK and not (allow_capacity and st == abi.PJ_ERR_CAPACITY):
            raise PetJsonError(st, "pj_group_parse", (lib().pj_group_last_error(self._h) or b"").decode())
        return list(shards)

    def prepare_parse(self, schema: int, bufs, lengths, cols, slack: int = 65536):
        """The argument arrays of parse(), built once for callers that parse into the same buffers again and again
        (a service loop, the benchmark): run it with parse_prepared()."""
        n = len(self.devices)
        return {"schema": schema, "slack": slack, "cols": list(cols), "keep": list(bufs),
                "ptrs": (C.c_void_p * n)(*[int(b.data_ptr()) for b in bufs]),
                "lens": (u64 * n)(*[int(x) for x in lengths]),
                "room": (u64 * n)(*[int(b.numel()) - int(x) for b, x in zip(bufs, lengths)]),
                "arr": self._cols_array(cols), "shards": (abi.pj_group_shard * n)()}

    def parse_prepared(self, prep, allow_capacity: bool = False):
        """One pj_group_parse call with prepared arguments; the columns' counters are refreshed, the shard table of the
        prepared object is returned (valid until the next call)."""
        st = lib().pj_group_parse(self._h, prep["schema"], prep["ptrs"], prep["lens"], prep["room"], prep["slack"], prep["arr"], prep["shards"])
        arr = prep["arr"]
        for k, c in enumerate(prep["cols"]):
            C.memmove(C.byref(c.raw), C.byref(arr[k]), C.sizeof(abi.pj_columns))
        if st != abi.PJ_OK and not (allow_capacity and st == abi.PJ_ERR_CAPACITY):
            raise PetJsonError(st, "pj_group_parse", (lib().pj_group_last_error(self._h) or b"").decode())
        return prep["shards"]

    def parse_host(self, schema: int, text, lengths, cols, slack: int = 65536, allow_capacity: bool = False):
        """pj_group_parse_host: `text` is one uint8 numpy array in host memory (pinned for full speed) holding all shards
        back to back, lengths[g] the bytes of shard g, cols[g] HostColumns or DeviceColumns. Returns the shard table."""
        n = len(self.devices)
        text = np.ascontiguousarray(text, dtype=np.uint8)
        assert int(sum(lengths)) <= text.size
        lens = (u64 * n)(*[int(x) for x in lengths])
        arr = self._cols_array(cols)
        shards = (abi.pj_group_shard * n)()
        st = lib().pj_group_parse_host(self._h, schema, C.c_void_p(text.ctypes.data), lens, slack, arr, shards)
        for k, c in enumerate(cols):
            C.memmove(C.byref(c.raw), C.byref(arr[k]), C.sizeof(abi.pj_columns))
        if st != abi.PJ_OK and not (allow_capacity and st == abi.PJ_ERR_CAPACITY):
            raise PetJsonError(st, "pj_group_parse_host", (lib().pj_group_last_error(self._h) or b"").decode())
        return list(shards)

    def write(self, schema: int, cols, outs, allow_capacity: bool = False):
        """cols[g]: DeviceColumns on device g; outs[g]: a uint8 CUDA tensor on device g. Returns the list of pj_group_shard
        (bytes = text length of shard g, global_offset = where it starts in the concatenated text)."""
        n = len(self.devices)
        ptrs = (C.c_void_p * n)(*[int(o.data_ptr()) for o in outs])
        caps = (u64 * n)(*[int(o.numel()) for o in outs])
        arr = self._cols_array(cols)
        shards = (abi.pj_group_shard * n)()
        st = lib().pj_group_write(self._h, schema, arr, ptrs, caps, shards)
        if st != abi.PJ_OK and not (allow_capacity and st == abi.PJ_ERR_CAPACITY):
            raise PetJsonError(st, "pj_group_write", (lib().pj_group_last_error(self._h) or b"").decode())
        return list(shards)
