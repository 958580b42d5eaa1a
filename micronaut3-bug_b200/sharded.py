"""Byte-range sharding of one NDJSON stream over the ranks of a torch.distributed group.

Every rank holds one contiguous byte range of the stream in its own memory. A shard owns the
records whose preceding LF lies in its range (rank 0 also owns the record at byte 0), so the only
data that has to move is the head of the following shard, up to `slack` bytes, which the owner of
the straddling record appends to its own buffer before parsing. That is one send/recv per rank;
after the parse one all-gather of a few counters gives every rank the global position of its rows.
No kernel ever reads another GPU's memory.
"""
from __future__ import annotations

import time

import numpy as np
import torch
import torch.distributed as dist

from . import abi

N_COUNTERS = 6 + abi.PJ_MAX_COLS  # records, errors, rows[1..3], bytes, then one count per column


class ShardedParser:
    """Runs pj_parse_shard on every rank and stitches the results.

    `engine` is anything with parse_shard(schema, buf, length, slack, is_first, is_last, global_offset, out)
    -- a petjson Context on GPUs; the tests pass a stand-in to exercise the exchange on CPU ranks.
    """

    def __init__(self, engine, schema: int, slack: int = 64 * 1024, group=None):
        self.engine = engine
        self.schema = schema
        self._cols = list(abi.schema_columns(schema))
        self.slack = int(slack)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self._plan = None

    def plan(self, nbytes: int, device) -> dict:
        """Exchanges the shard sizes (one small all-gather) and derives what the parse needs: global byte offset, how
        much of the next shard to fetch, whether the stream ends in this shard's view. Every rank runs this on every
        call: whether to exchange is never decided from one rank's own size, because a collective that only some ranks
        enter hangs the others. A shard other than the last must hold at least `slack` bytes: the slack of its
        predecessor is taken from it alone (pj_group_parse of the C ABI has no such limit)."""
        r, w = self.rank, self.world
        sizes_h = self._all_gather(torch.tensor([nbytes], dtype=torch.int64, device=device)).view(-1).tolist()
        for k in range(1, w - 1):
            if sizes_h[k] < self.slack:
                raise ValueError(f"shard {k} holds {sizes_h[k]} bytes, fewer than the slack of {self.slack}: records of shard {k - 1} could run through it")
        self._plan = {"nbytes": nbytes, "sizes": sizes_h, "goff": int(sum(sizes_h[:r])),
                      "recv_n": min(self.slack, sizes_h[r + 1]) if r + 1 < w else 0,
                      "send_n": min(self.slack, nbytes) if r > 0 else 0,
                      "is_last": r == w - 1 or (r + 1 == w - 1 and sizes_h[r + 1] <= self.slack)}
        return self._plan

    def parse(self, buf: torch.Tensor, nbytes: int, out, wait: bool = True):
        """`buf` holds this rank's `nbytes` bytes followed by at least `slack` writable bytes.
        Fills `out` with this shard's columns (offsets local to the shard). With wait=True returns the stitch
        (global byte offset, global first record / row / arena positions, totals, time spent on the exchange);
        with wait=False the counter all-gather is only enqueued and the returned object's .result() gives the
        stitch later, so consecutive steps do not stop for it."""
        g, r, w = self.group, self.rank, self.world
        on_gpu = buf.is_cuda
        t0 = time.perf_counter()
        plan = self.plan(nbytes, buf.device)
        recv_n, send_n = plan["recv_n"], plan["send_n"]
        if on_gpu:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        # the head of the next shard becomes this shard's slack
        ops = []
        if send_n:
            ops.append(dist.P2POp(dist.isend, buf[:send_n], self._peer(r - 1), group=g))
        if recv_n:
            ops.append(dist.P2POp(dist.irecv, buf[nbytes:nbytes + recv_n], self._peer(r + 1), group=g))
        if ops:
            for req in dist.batch_isend_irecv(ops):
                req.wait()  # on GPUs: orders the current stream after the transfer, does not block the host
        if on_gpu:
            ev1.record()
        exchange_host_ms = 1e3 * (time.perf_counter() - t0)
        # the local parse
        self.engine.parse_shard(self.schema, buf, nbytes, recv_n, r == 0, plan["is_last"], plan["goff"], out)
        # counters -> global bases
        t1 = time.perf_counter()
        cn = np.zeros(N_COUNTERS, np.int64)  # filled on the host in one go: element-wise tensor writes cost microseconds each
        cn[0], cn[1] = out.n_records, out.n_errors
        cn[2:5] = [out.n_rows(t) for t in (1, 2, 3)]
        cn[5] = nbytes
        for col in self._cols:
            cn[6 + col.id] = out.count(col.id)
        c = torch.from_numpy(cn).to(buf.device)
        if on_gpu:
            gathered = torch.empty(w * N_COUNTERS, dtype=torch.int64, device=buf.device)
            dist.all_gather_into_tensor(gathered, c, group=g)
        else:
            parts = [torch.empty_like(c) for _ in range(w)]
            dist.all_gather(parts, c, group=g)
            gathered = torch.stack(parts)
        gather_host_ms = 1e3 * (time.perf_counter() - t1)
        pending = _Pending(self, plan, gathered, (ev0, ev1) if on_gpu else None, exchange_host_ms, gather_host_ms)
        return pending.result() if wait else pending

    def _all_gather(self, t: torch.Tensor) -> torch.Tensor:
        """[world, len(t)] on the host."""
        if t.is_cuda:
            out = torch.empty(self.world * t.numel(), dtype=t.dtype, device=t.device)
            dist.all_gather_into_tensor(out, t, group=self.group)
            return out.view(self.world, -1).cpu()
        parts = [torch.empty_like(t) for _ in range(self.world)]
        dist.all_gather(parts, t, group=self.group)
        return torch.stack(parts)

    def _peer(self, group_rank: int) -> int:
        return dist.get_global_rank(self.group, group_rank) if self.group is not None else group_rank


class _Pending:
    """The stitch of one ShardedParser.parse call whose counter all-gather may still be in flight."""

    def __init__(self, sp: ShardedParser, plan: dict, gathered: torch.Tensor, events, exchange_host_ms: float, gather_host_ms: float):
        self.sp, self.plan, self.gathered, self.events = sp, plan, gathered, events
        self.exchange_host_ms, self.gather_host_ms = exchange_host_ms, gather_host_ms

    def result(self) -> dict:
        sp, r, w = self.sp, self.sp.rank, self.sp.world
        allc = self.gathered.view(w, N_COUNTERS).cpu().numpy()  # synchronises with the all-gather
        exchange_ms = self.events[0].elapsed_time(self.events[1]) if self.events else self.exchange_host_ms
        before = allc[:r].sum(axis=0)
        total = allc.sum(axis=0)
        # an _OFF column of a shard has rows + 1 entries; globally the closing entries collapse
        bases, totals = {}, {}
        for col in abi.schema_columns(sp.schema):
            closing = 1 if col.shape.endswith("+1") else 0
            bases[col.name] = int(before[6 + col.id] - closing * r)
            totals[col.name] = int(total[6 + col.id] - closing * (w - 1))
        return {"global_offset": self.plan["goff"], "first_record": int(before[0]), "total_records": int(total[0]), "total_errors": int(total[1]),
                "first_row": {t: int(before[1 + t]) for t in (1, 2, 3)}, "total_rows": {t: int(total[1 + t]) for t in (1, 2, 3)},
                "column_base": bases, "column_total": totals, "slack_used": self.plan["recv_n"], "is_last": self.plan["is_last"],
                "stitch_ms": exchange_ms + self.gather_host_ms, "exchange_ms": exchange_ms, "gather_ms": self.gather_host_ms}


def split_even(total_bytes: int, world: int) -> list[tuple[int, int]]:
    """Equal contiguous byte ranges [lo, hi) of a stream, one per rank."""
    return [(total_bytes * r // world, total_bytes * (r + 1) // world) for r in range(world)]
