/*
 * pj_stream_kernel.cuh — k_parse_stream<SCHEMA>: NDJSON bytes to typed columns in ONE kernel and one pass over HBM.
 *
 * One thread block = one tile of the input (pj_stream.cuh): the tile and what follows it are staged in shared memory
 * by one bulk copy (cp.async.bulk, the untiled TMA form, no multicast), the block builds the line index of the window
 * itself (line-feed masks from 16-byte chunks, compacted by a block scan), thread j tokenises owned line j, the
 * per-record counts are scanned inside the block, the tile's first record number and its start in every arena and
 * child table come from ONE decoupled look-back over the earlier tiles, and every column is emitted. There is no
 * separate index kernel and the host never needs the record count to size a launch.
 *
 * Look-back: tiles take their number from an atomic ticket, so every predecessor of a running tile is running or
 * done; a tile publishes its own totals ("aggregate") as soon as its records are sized and its inclusive totals once
 * it has found the nearest predecessor whose inclusive totals are published. Every word carries its own valid bit.
 * Waits are bounded by StreamArgs.spin_limit_ns: when one runs out the kernel raises DevResult.timeout, which every
 * other wait watches too, and the block leaves without emitting; the host answers PJ_ERR_TIMEOUT.
 *
 * Tiles with more owned lines than threads (records much shorter than the tile size was chosen for) take the
 * slow road of stream_overflow_tile(): batches of ST_THREADS lines, sized in a first pass and emitted in a second.
 */
#ifndef PJ_STREAM_KERNEL_CUH
#define PJ_STREAM_KERNEL_CUH

#include "pj_kernels.cuh"
#include "pj_lock.cuh"
#include "pj_wide.cuh"
#include "pj_stream.cuh"

namespace pj {

static constexpr uint32_t ST_NLB = 16;    /* look-back words per tile: the NSLOT counters and the record count */
static constexpr uint32_t ST_REC = NSLOT; /* look-back word of the record count */
static_assert(NSLOT + 1 == ST_NLB, "one more word than counters");
struct StreamTile {
  unsigned long long agg[ST_NLB];
  unsigned long long inc[ST_NLB];
};
static_assert(sizeof(StreamTile) == 256, "two 128-byte lines per tile");

static constexpr uint32_t ST_TAPE_CAP = 20; /* 32-bit tape words per record before it is tokenised a second time at emission */
static constexpr uint32_t ST_SMEM_WIN = ST_WIN_BYTES + ST_WIN_PAD;
static constexpr uint32_t ST_SMEM_LFB = ST_CHUNKS * 2; /* one 16-bit line-feed mask per chunk */
static constexpr uint32_t ST_SMEM_LIST = ST_LF_CAP * 2; /* line starts of the current batch, 16-bit window offsets */
static constexpr uint32_t ST_SMEM_BYTES = ST_SMEM_WIN + ST_SMEM_LFB + ST_SMEM_LIST + ST_TAPE_CAP * ST_THREADS * 4;
static_assert(ST_SMEM_WIN % 16 == 0 && ST_WIN_BYTES + 1 < 65536, "window offsets fit 16 bits");

struct StreamArgs {
  const uint8_t* in;
  uint64_t len, limit, goff;
  uint32_t is_first, is_last;
  uint32_t tile_bytes, ntiles;
  uint32_t opts; /* PJ_OPT_* bits that change a rule */
  unsigned long long spin_limit_ns;
  StreamTile* tiles;
  uint32_t* ticket;
  DevResult* res;
  const DevResult* prev;    /* totals of the pieces of the same call parsed by earlier launches (null: none) */
  uint64_t slot_cap[NSLOT]; /* largest total per slot the caller's buffers can take */
  uint64_t rec_cap;         /* records the per-record and row-indexed buffers can take */
  FinalizePlan plan;
  DevCols cols;
};

template <int SCHEMA> struct StreamSlots {
  static constexpr uint32_t lo = SlotRange<SCHEMA>::lo, hi = SlotRange<SCHEMA>::hi;
  static constexpr uint32_t mask = ((hi > lo ? ((1u << hi) - (1u << lo)) : 0u)) | (1u << ST_REC);
};

/* Exclusive totals of all tiles before `tile` for the words of MASK, into excl[] (every lane gets all of them).
 * Warp 0, all lanes. One round looks at 32 predecessors with one memory round trip. False when the wait ran out. */
template <uint32_t MASK>
__device__ __forceinline__ bool stream_lookback(const StreamArgs& a, uint32_t tile, uint32_t lane, uint32_t* excl) {
#pragma unroll
  for (uint32_t k = 0; k < ST_NLB; ++k) excl[k] = 0;
  int64_t j = (int64_t)tile - 1;
  const unsigned long long t0 = global_ns();
  unsigned polls = 0, rounds = 0;
  while (j >= 0) {
    const int64_t mine = j - lane; /* tiles before the first count as "inclusive, zero" */
    uint32_t va[ST_NLB], vi[ST_NLB];
    uint32_t first_inc;
    for (;;) {
      bool has_inc = true, has_agg = true;
#pragma unroll
      for (uint32_t k = 0; k < ST_NLB; ++k) {
        if (!((MASK >> k) & 1u)) continue;
        unsigned long long wa = TS_VALID, wi = TS_VALID;
        if (mine >= 0) { wi = ld_relaxed_u64(&a.tiles[mine].inc[k]); wa = ld_relaxed_u64(&a.tiles[mine].agg[k]); }
        has_inc = has_inc && (wi & TS_VALID);
        has_agg = has_agg && (wa & TS_VALID);
        va[k] = (uint32_t)wa; vi[k] = (uint32_t)wi;
      }
      const uint32_t inc_mask = __ballot_sync(0xFFFFFFFFu, has_inc);
      const uint32_t ready_mask = __ballot_sync(0xFFFFFFFFu, has_inc || has_agg);
      first_inc = inc_mask ? (uint32_t)(__ffs((int)inc_mask) - 1) : 32u;
      const uint32_t need = first_inc >= 31 ? 0xFFFFFFFFu : ((2u << first_inc) - 1u);
      if ((ready_mask & need) == need) break;
      ++polls;
      uint32_t give_up = 0;
      if (lane == 0) give_up = (global_ns() - t0 > a.spin_limit_ns) || *(volatile uint32_t*)&a.res->timeout;
      give_up = __shfl_sync(0xFFFFFFFFu, give_up, 0);
      if (give_up) { if (lane == 0) atomicExch(&a.res->timeout, 1u); return false; }
      __nanosleep(100);
    }
    ++rounds;
#pragma unroll
    for (uint32_t k = 0; k < ST_NLB; ++k) {
      if (!((MASK >> k) & 1u)) continue;
      uint32_t c = lane < first_inc ? va[k] : (lane == first_inc ? vi[k] : 0u);
#pragma unroll
      for (int d = 16; d; d >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, d);
      excl[k] += c;
    }
    if (first_inc < 32) break;
    j -= 32;
  }
  if (lane == 0) { atomicAdd(&a.res->lookback_polls, (unsigned long long)polls); atomicAdd(&a.res->lookback_rounds, (unsigned long long)rounds); }
  return true;
}

/* Warp 0 of a tile whose records are sized: adds up the warps' totals (warp_tot[word * nwarps + warp]), publishes
 * them, looks back, publishes the inclusive totals, checks the caller's capacities and leaves in sh_base[] where the
 * tile starts over the whole call (earlier launches of the call included) and in *sh_ok whether to emit. The last
 * tile also leaves the call's totals. */
template <uint32_t MASK>
__device__ __forceinline__ void stream_resolve(const StreamArgs& a, uint32_t tile, uint32_t lane, const uint32_t* warp_tot, uint32_t nwarps,
                                               uint32_t* sh_tot, uint32_t* sh_base, uint32_t* sh_ok) {
  StreamTile* me = &a.tiles[tile];
  uint32_t mine = 0;
  if (lane < ST_NLB && ((MASK >> lane) & 1u))
    for (uint32_t q = 0; q < nwarps; ++q) mine += warp_tot[lane * nwarps + q];
  if (lane < ST_NLB) {
    sh_tot[lane] = mine;
    st_relaxed_u64(&me->agg[lane], TS_VALID | mine);
    if (tile == 0) st_relaxed_u64(&me->inc[lane], TS_VALID | mine);
  }
  uint32_t excl_all[ST_NLB];
  const bool ok = stream_lookback<MASK>(a, tile, lane, excl_all);
  uint32_t excl = 0;
#pragma unroll
  for (uint32_t k = 0; k < ST_NLB; ++k) if (lane == k) excl = excl_all[k];
  if (tile != 0 && ok && lane < ST_NLB) st_relaxed_u64(&me->inc[lane], TS_VALID | (unsigned long long)(excl + mine));
  /* the tile's start over the whole call: what earlier launches of the call produced comes first */
  uint64_t prior = 0;
  if (a.prev && lane < ST_NLB) prior = lane == ST_REC ? a.prev->n_records : a.prev->total[lane];
  const uint64_t before = lane < ST_NLB ? prior + excl : 0;
  if (lane < ST_NLB) sh_base[lane] = (uint32_t)before;
  const uint64_t cap = lane == ST_REC ? a.rec_cap : (lane < NSLOT ? a.slot_cap[lane] : ~0ull);
  const bool over = lane < ST_NLB && before + mine > cap;
  const uint32_t any_over = __ballot_sync(0xFFFFFFFFu, over);
  if (lane == 0) {
    *sh_ok = ok && !any_over;
    if (any_over) a.res->over = 1u;
  }
  if (tile == a.ntiles - 1) {
    if (lane < NSLOT) a.res->total[lane] = before + mine;
    if (lane == ST_REC) a.res->n_records = before + mine;
  }
}

/* Writes the line starts number [list_base, list_base + ST_LF_CAP) of the window into list[] (window offset of the
 * first byte of each line). `first_idx` is the number of this thread's first line; the virtual line of the first
 * tile of a first shard (the one at byte 0, which no line feed precedes) is line 0 of thread 0. */
__device__ __forceinline__ void stream_fill_list(uint16_t* list, const uint16_t* lfb, uint32_t tid, uint32_t first_idx, uint32_t list_base,
                                                 bool virtual_first, uint32_t mis) {
  uint32_t idx = first_idx;
  if (virtual_first) { if (idx - list_base < ST_LF_CAP) list[idx - list_base] = (uint16_t)mis; idx++; }
#pragma unroll 1
  for (uint32_t k = 0; k < ST_CPT; ++k) {
    const uint32_t c = tid * ST_CPT + k;
    uint32_t m = lfb[c];
    while (m) {
      const uint32_t b = (uint32_t)__ffs((int)m) - 1u;
      m &= m - 1u;
      if (idx - list_base < ST_LF_CAP) list[idx - list_base] = (uint16_t)(c * 16u + b + 1u);
      idx++;
    }
  }
}

/* One line of a tile, located. */
struct StreamLine {
  uint32_t s;       /* window offset of its first byte */
  uint32_t fits;    /* all of its bytes are staged */
  uint64_t gstart;  /* input offset of its first byte */
};

/* Everything the tokenising step leaves behind for one record. */
template <int SCHEMA>
struct StreamRec {
  FVals v, cv;
  uint32_t cnt[NSLOT];
  uint32_t type, err, err_off, fast, locked, direct, start32, lim32, tape_n;
};

/* What lock_record<>() did not finish: the word-at-a-time tokeniser (staged record, or where it lies when it is not
 * staged: `end_known` = input offset of its end, or ~0) and, behind it, the exact parser of pj_core.cuh. Out of
 * line: it is rare, large and wants more registers than the path in step. */
template <int SCHEMA>
__device__ __noinline__ void stream_tokenise_rest(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, const StreamLine& L, uint64_t end_known,
                                                  Tape& tp, StreamRec<SCHEMA>& r, Win& wd) {
  constexpr uint32_t LO = StreamSlots<SCHEMA>::lo, HI = StreamSlots<SCHEMA>::hi;
  const int64_t w0 = (int64_t)g.v0 - (int64_t)g.mis; /* input offset of window byte 0 */
  Win w;
  w.s = win; w.w0 = w0;
  wd = w;
  const uint32_t open_end = a.is_last ? 0u : 1u;
  r.direct = !L.fits && end_known != ~0ull && end_known + 32 <= a.limit;
  if (r.direct) {
    const uint32_t mis4 = (uint32_t)(reinterpret_cast<uintptr_t>(a.in + L.gstart) & 3u);
    wd.s = a.in + L.gstart - mis4; wd.w0 = (int64_t)L.gstart - mis4;
  }
  {
    const uint64_t rel = (uint64_t)((int64_t)a.limit - wd.w0);
    r.lim32 = rel > 0xFFFFFFF0ull ? 0xFFFFFFF0u : (uint32_t)rel;
    r.start32 = (uint32_t)((int64_t)L.gstart - wd.w0);
  }
  uint32_t verdict = FAST_REFUSED, fpos = 0;
  r.type = PJ_TYPE_NONE; r.err = 0; r.err_off = 0; r.fast = 0;
  if (L.fits || r.direct) {
    if (!r.direct) verdict = fast_record<SCHEMA>(w, r.start32, r.lim32, 0u, open_end, &r.type, r.v, r.cv, r.cnt, tp, &r.err, &fpos);
    else {
      uint32_t cnt_d[NSLOT], type_d = PJ_TYPE_NONE, err_d = 0;
      verdict = fast_outline<SCHEMA>(wd, r.start32, r.lim32, 0u, open_end, nullptr, nullptr, 0, tp, cnt_d, &type_d, &err_d, &fpos);
      r.type = type_d; r.err = err_d;
#pragma unroll
      for (uint32_t k = 0; k < NSLOT; ++k) r.cnt[k] = cnt_d[k];
    }
    r.fast = verdict == FAST_ACCEPTED;
    if (verdict == FAST_FAILED && opt_decides(a.opts, r.err)) { verdict = FAST_REFUSED; r.err = 0; } /* the exact parser knows the options */
  }
  if (verdict == FAST_FAILED) { /* a failure found by the word-at-a-time path: no row values, no bytes anywhere */
    r.type = PJ_TYPE_NONE;
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) r.cnt[k] = 0;
    r.err_off = fpos - r.start32;
  }
  if (verdict == FAST_REFUSED) {
    Rd rd;
    rd.in = L.fits ? win - w0 : a.in; rd.lf_ws = 0; rd.open_end = open_end; rd.limit = a.limit; rd.opts = a.opts;
    PS s;
    s.p = L.gstart; s.err = 0; s.err_pos = 0;
    Out<false> so;
    so.cols = &a.cols;
    r.type = parse_record<false>(c_schema, rd, s, (uint32_t)SCHEMA, so, 0);
    r.err = s.err;
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) r.cnt[k] = (k >= LO && k < HI && !s.err) ? so.cnt[k] : 0u;
    if (s.err) r.type = PJ_TYPE_NONE;
    r.err_off = s.err ? (uint32_t)(s.err_pos - L.gstart) : 0u;
  }
  r.tape_n = tp.n;
}

/* Tokenises the record of line L once. Every thread of the block calls this, `is_rec` or not: staged records go
 * through the lockstep tokeniser, which the lanes of a warp walk together; what it neither accepts nor fails goes
 * to stream_tokenise_rest<>(). */
template <int SCHEMA>
__device__ __forceinline__ void stream_tokenise(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, bool is_rec, const StreamLine& L, uint64_t end_known,
                                                Tape& tp, StreamRec<SCHEMA>& r, Win& w, Win& wd) {
  w.s = win; w.w0 = (int64_t)g.v0 - (int64_t)g.mis;
  wd = w;
  const uint32_t open_end = a.is_last ? 0u : 1u;
  r.direct = 0; r.err_off = 0;
  r.start32 = L.s;
  r.lim32 = g.vlimit - g.v0 > 0xFFFFFFF0ull ? 0xFFFFFFF0u : (uint32_t)(g.vlimit - g.v0); /* window offset of the first byte that is not input */
  uint32_t fpos = 0;
  uint32_t verdict = lock_record<SCHEMA>(w, is_rec && L.fits, L.s, r.lim32, open_end, &r.type, r.v, r.cv, r.cnt, tp, &r.err, &fpos);
  if (verdict == FAST_FAILED && opt_decides(a.opts, r.err)) verdict = FAST_REFUSED; /* the exact parser knows the options */
  r.fast = verdict == FAST_ACCEPTED;
  r.locked = r.fast; /* accepted in step: its tape is in model order */
  r.tape_n = tp.n;
  if (!is_rec || verdict == FAST_FAILED) { /* no record, or a failed one: no row values, no bytes anywhere */
    if (!is_rec) r.err = 0;
    r.type = PJ_TYPE_NONE;
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) r.cnt[k] = 0;
    r.err_off = is_rec ? fpos - L.s : 0u;
    r.tape_n = 0;
  } else if (verdict == FAST_REFUSED) {
    /* through copies, so that the addresses of the hot path's own state never leave it (it stays in registers) */
    StreamRec<SCHEMA> cold;
    StreamLine lc = L;
    Tape tc = tp;
    Win wc;
    stream_tokenise_rest<SCHEMA>(a, g, win, lc, end_known, tc, cold, wc);
    r = cold; tp.n = tc.n; wd = wc;
    r.locked = 0;
  }
}

/* Emission of the records the path in step did not accept (out of line, like their tokenising). */
template <int SCHEMA>
__device__ __noinline__ void stream_emit_rest(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, const StreamLine& L, const Win& wd,
                                              Tape& tp, const StreamRec<SCHEMA>& r, const uint32_t* base, uint64_t i) {
  const int64_t w0 = (int64_t)g.v0 - (int64_t)g.mis;
  Win w;
  w.s = win; w.w0 = w0;
  if (r.fast) {
    if (!r.direct && r.tape_n <= tp.cap) fast_emit<SCHEMA>(w, &a.cols, r.type, r.v, r.cv, tp, base, i);
    else {
      uint32_t base_copy[NSLOT], t_d, e_d, p_d;
#pragma unroll
      for (uint32_t k = 0; k < NSLOT; ++k) base_copy[k] = base[k];
      fast_outline<SCHEMA>(r.direct ? wd : w, r.start32, r.lim32, 0u, a.is_last ? 0u : 1u, &a.cols, base_copy, i, tp, nullptr, &t_d, &e_d, &p_d);
    }
  } else {
    Out<true> o;
    o.cols = &a.cols;
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) { o.base[k] = base[k]; o.room[k] = r.cnt[k]; }
    if (r.err) {
      if (SCHEMA != PJ_SCHEMA_MIXED) store_absent<true>(c_schema, (uint32_t)SCHEMA, o, i);
    } else {
      Rd rd;
      rd.in = L.fits ? win - w0 : a.in; rd.lf_ws = 0; rd.open_end = a.is_last ? 0u : 1u; rd.limit = a.limit; rd.opts = a.opts;
      PS s;
      s.p = L.gstart; s.err = 0; s.err_pos = 0;
      parse_record<true>(c_schema, rd, s, (uint32_t)SCHEMA, o, i);
    }
  }
}

/* Emits record number `i` (base[] = its start in every arena / child table / model table). */
template <int SCHEMA>
__device__ __forceinline__ void stream_emit_head(const StreamArgs& a, const StreamLine& L, const StreamRec<SCHEMA>& r, const uint32_t* base, uint64_t i) {
  colp<uint64_t>(&a.cols, PJ_COL_REC_START)[i] = a.goff + L.gstart;
  colp<uint8_t>(&a.cols, PJ_COL_ERR_KIND)[i] = (uint8_t)r.err;
  colp<uint32_t>(&a.cols, PJ_COL_ERR_OFF)[i] = r.err_off;
  if (SCHEMA == PJ_SCHEMA_MIXED) {
    colp<uint8_t>(&a.cols, PJ_COL_REC_TYPE)[i] = (uint8_t)r.type;
    const uint32_t row = r.type == PJ_TYPE_PET ? base[SLOT_ROWS_PET] : (r.type == PJ_TYPE_ORDER ? base[SLOT_ROWS_ORD] : base[SLOT_ROWS_USR]);
    colp<uint32_t>(&a.cols, PJ_COL_REC_ROW)[i] = r.type == PJ_TYPE_NONE ? 0xFFFFFFFFu : row;
  }
}
template <int SCHEMA>
__device__ __forceinline__ void stream_emit(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, const StreamLine& L, const Win& w, const Win& wd,
                                            Tape& tp, const StreamRec<SCHEMA>& r, const uint32_t* base, uint64_t i) {
  stream_emit_head<SCHEMA>(a, L, r, base, i);
  if (r.locked && r.tape_n <= tp.cap) lock_emit<SCHEMA>(w, &a.cols, r.type, r.v, r.cv, tp, base, r.cnt, i);
  else {
    StreamRec<SCHEMA> cold = r;
    StreamLine lc = L;
    Tape tc = tp;
    Win wc = wd;
    uint32_t bc[NSLOT];
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) bc[k] = base[k];
    stream_emit_rest<SCHEMA>(a, g, win, lc, wc, tc, cold, bc, i);
  }
}

/* ---- long records: a warp each (pj_wide.cuh) ----------------------------------------------------------------- */
static constexpr uint32_t ST_WIDE_MIN = 1024; /* bytes from which a record of a model with lists is walked by a warp */
static constexpr uint32_t ST_WIDE_CAP = 32;   /* such records per tile; what is beyond stays with its thread */
struct WideSlot {
  uint64_t gstart, gend, rec_index; /* input offsets of the record's first byte and of the byte that ends it */
  uint32_t fits, type, err, err_off;
  uint32_t fast; /* the word-at-a-time tokeniser accepted it: it emits it too */
  uint32_t cnt[NSLOT], base[NSLOT];
};
template <int SCHEMA>
__device__ __forceinline__ Rd stream_wide_reader(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, const WideSlot* ws) {
  const int64_t w0 = (int64_t)g.v0 - (int64_t)g.mis;
  Rd rd;
  rd.in = ws->fits ? win - w0 : a.in; rd.lf_ws = 0; rd.open_end = a.is_last ? 0u : 1u; rd.limit = a.limit; rd.opts = a.opts;
  rd.rec_end = ws->gend;
  return rd;
}
/* The record of a slot as the word-at-a-time tokeniser addresses it: the staged window, or the bytes where they lie. */
struct WideWin { Win w; uint32_t start, limit, end; };
__device__ __forceinline__ WideWin stream_wide_win(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, const WideSlot* ws) {
  WideWin r;
  int64_t w0;
  if (ws->fits) { r.w.s = win; w0 = (int64_t)g.v0 - (int64_t)g.mis; }
  else {
    const uint32_t mis4 = (uint32_t)(reinterpret_cast<uintptr_t>(a.in + ws->gstart) & 3u);
    r.w.s = a.in + ws->gstart - mis4; w0 = (int64_t)ws->gstart - mis4;
  }
  r.w.w0 = w0;
  const uint64_t rel = (uint64_t)((int64_t)a.limit - w0), rel_end = (uint64_t)((int64_t)ws->gend - w0);
  r.limit = rel > 0xFFFFFFF0ull ? 0xFFFFFFF0u : (uint32_t)rel;
  r.end = rel_end > 0xFFFFFFF0ull ? 0xFFFFFFF0u : (uint32_t)rel_end;
  r.start = (uint32_t)((int64_t)ws->gstart - w0);
  return r;
}
/* Size pass of one long record, by all lanes of the calling warp: the word-at-a-time tokeniser first, the exact
 * parser for what that one refuses. */
template <int SCHEMA>
__device__ __noinline__ void stream_wide_size(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, uint32_t* tape, WideSlot* ws) {
  constexpr uint32_t LO = StreamSlots<SCHEMA>::lo, HI = StreamSlots<SCHEMA>::hi;
  const bool lane0 = (threadIdx.x & 31u) == 0;
  {
    const WideWin ww = stream_wide_win(a, g, win, ws);
    Tape tp;
    tp.e = tape + threadIdx.x; tp.stride = ST_THREADS; tp.cap = TAPE_MIN_CAP; tp.n = 0;
    uint32_t cnt[NSLOT], type = PJ_TYPE_NONE, err = 0, fpos = 0;
    uint32_t verdict = ww.end - ww.start < 0x7FFF0000u
                           ? wide_outline<SCHEMA>(ww.w, ww.start, ww.limit, ww.end, a.is_last ? 0u : 1u, nullptr, nullptr, 0, tp, cnt, &type, &err, &fpos)
                           : (uint32_t)FAST_REFUSED;
    if (verdict == FAST_FAILED && opt_decides(a.opts, err)) verdict = FAST_REFUSED; /* the exact parser knows the options */
    __syncwarp();
    if (verdict != FAST_REFUSED) {
      if (lane0) {
        const bool ok = verdict == FAST_ACCEPTED;
        ws->fast = ok ? 1u : 0u;
        ws->type = ok ? type : (uint32_t)PJ_TYPE_NONE;
        ws->err = ok ? 0u : err;
        ws->err_off = ok ? 0u : fpos - ww.start;
#pragma unroll
        for (uint32_t k = 0; k < NSLOT; ++k) ws->cnt[k] = ok ? cnt[k] : 0u;
        if (ok) atomicAdd(&a.res->n_wide_fast, 1ull);
      }
      return;
    }
  }
  const Rd rd = stream_wide_reader<SCHEMA>(a, g, win, ws);
  PS s;
  s.p = ws->gstart; s.err = 0; s.err_pos = 0;
  Out<false> so;
  so.cols = &a.cols;
  const uint32_t type = parse_record<false, WarpListHook>(c_schema, rd, s, (uint32_t)SCHEMA, so, 0);
  __syncwarp();
  if (lane0) {
    ws->fast = 0;
    ws->type = s.err ? (uint32_t)PJ_TYPE_NONE : type;
    ws->err = s.err;
    ws->err_off = s.err ? (uint32_t)(s.err_pos - ws->gstart) : 0u;
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) ws->cnt[k] = (k >= LO && k < HI && !s.err) ? so.cnt[k] : 0u;
  }
}
/* Emit pass of one long record that the size pass accepted. */
template <int SCHEMA>
__device__ __noinline__ void stream_wide_emit(const StreamArgs& a, const StreamGeom& g, const uint8_t* win, uint32_t* tape, const WideSlot* ws) {
  if (ws->fast) {
    const WideWin ww = stream_wide_win(a, g, win, ws);
    Tape tp;
    tp.e = tape + threadIdx.x; tp.stride = ST_THREADS; tp.cap = TAPE_MIN_CAP; tp.n = 0;
    uint32_t t_d, e_d, p_d;
    wide_outline<SCHEMA>(ww.w, ww.start, ww.limit, ww.end, a.is_last ? 0u : 1u, &a.cols, ws->base, ws->rec_index, tp, nullptr, &t_d, &e_d, &p_d);
    return;
  }
  const Rd rd = stream_wide_reader<SCHEMA>(a, g, win, ws);
  PS s;
  s.p = ws->gstart; s.err = 0; s.err_pos = 0;
  Out<true> o;
  o.cols = &a.cols;
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) { o.base[k] = ws->base[k]; o.room[k] = ws->cnt[k]; }
  parse_record<true, WarpListHook>(c_schema, rd, s, (uint32_t)SCHEMA, o, ws->rec_index);
}

/* Looks, with the whole block, for the first line feed at or after input offset `from` (the end of the one line of a
 * tile that runs out of the window). Returns its input offset, or a.limit when there is none. */
__device__ __forceinline__ uint64_t stream_find_end(const StreamArgs& a, uint64_t from, uint32_t tid, unsigned long long* sh_min) {
  if (tid == 0) *sh_min = ~0ull;
  __syncthreads();
  for (uint64_t p = from; p < a.limit; p += ST_THREADS * 16ull) {
    const uint64_t q = p + (uint64_t)tid * 16u;
    unsigned long long found = ~0ull;
    for (uint32_t b = 0; b < 16 && q + b < a.limit; ++b) if (a.in[q + b] == '\n') { found = q + b; break; }
    if (found != ~0ull) atomicMin(sh_min, found);
    __syncthreads();
    const bool done = *sh_min != ~0ull;
    __syncthreads(); /* nobody updates the minimum before everybody has read it */
    if (done) break;
  }
  const unsigned long long m = *sh_min;
  return m == ~0ull ? a.limit : (uint64_t)m;
}

/* Closing entries of the offset columns, by the last tile of a launch. */
__device__ __forceinline__ void stream_close_offsets(const StreamArgs& a, uint32_t tid, const uint32_t* sh_base, const uint32_t* sh_tot) {
  if (tid < a.plan.n) {
    const FinalizeItem it = a.plan.item[tid];
    if (it.sentinel_slot != 0xFF) {
      const uint32_t rs = it.rows_slot == 0xFF ? ST_REC : it.rows_slot;
      colp<uint32_t>(&a.cols, it.col)[(uint64_t)sh_base[rs] + sh_tot[rs]] = sh_base[it.sentinel_slot] + sh_tot[it.sentinel_slot];
    }
  }
}

/* A tile with more owned lines than threads: batches of ST_THREADS lines. The first pass sizes every record (the
 * tile's totals are what the look-back needs), the second tokenises each batch again, scans it and emits it. */
template <int SCHEMA>
__device__ __noinline__ void stream_overflow_tile(const StreamArgs& a, const StreamGeom& g, uint8_t* win, const uint16_t* lfb, uint16_t* list, uint32_t* tape,
                                                  uint32_t tile, uint32_t first_idx, uint32_t nlf, uint32_t nown, bool virtual_first) {
  constexpr uint32_t MASK = StreamSlots<SCHEMA>::mask;
  __shared__ uint32_t sh_scan[33];
  __shared__ uint32_t sh_sum[ST_NLB], sh_tot[ST_NLB], sh_base[ST_NLB], sh_ok;
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  Tape tp;
  tp.e = tape + tid; tp.stride = ST_THREADS; tp.cap = ST_TAPE_CAP; tp.n = 0;
  StreamRec<SCHEMA> r;
  Win w, wd;
  if (tid < ST_NLB) sh_sum[tid] = 0;
  for (int pass = 0; pass < 2; ++pass) {
    uint32_t run[ST_NLB];
#pragma unroll
    for (uint32_t k = 0; k < ST_NLB; ++k) run[k] = pass ? sh_base[k] : 0u;
    uint32_t nerr = 0, nfast = 0;
    for (uint32_t b0 = 0; b0 < nown; b0 += ST_THREADS) {
      __syncthreads(); /* the list and the tapes of the batch before are free */
      stream_fill_list(list, lfb, tid, first_idx, b0, virtual_first, g.mis);
      __syncthreads();
      const uint32_t j = b0 + tid;
      StreamLine L;
      L.s = 0; L.fits = 0; L.gstart = 0;
      bool is_rec = false;
      if (j < nown) {
        L.s = list[tid];
        L.fits = (j + 1 < nlf) || g.to_limit; /* the list holds ST_LF_CAP > ST_THREADS lines from b0 on */
        L.gstart = g.v0 + L.s - g.mis;
        is_rec = stream_is_record(win, L.s, g, a.in, a.limit, (int)a.is_last);
      }
      r.type = PJ_TYPE_NONE; r.err = 0; r.err_off = 0; r.fast = 0; r.locked = 0; r.direct = 0; r.tape_n = 0;
#pragma unroll
      for (uint32_t k = 0; k < NSLOT; ++k) r.cnt[k] = 0;
      stream_tokenise<SCHEMA>(a, g, win, is_rec, L, ~0ull, tp, r, w, wd); /* a line that leaves the window: exact parser, where it lies */
      if (pass == 0) {
#pragma unroll
        for (uint32_t k = 0; k < ST_NLB; ++k) {
          if (!((MASK >> k) & 1u)) continue;
          uint32_t c = k == ST_REC ? (is_rec ? 1u : 0u) : r.cnt[k];
#pragma unroll
          for (int d = 16; d; d >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, d);
          if (lane == 0 && c) atomicAdd(&sh_sum[k], c);
        }
      } else {
        nerr += r.err ? 1u : 0u; nfast += r.fast;
        uint32_t base[ST_NLB];
#pragma unroll
        for (uint32_t k = 0; k < ST_NLB; ++k) {
          base[k] = 0;
          if (!((MASK >> k) & 1u)) continue;
          const uint32_t mine_k = k == ST_REC ? (is_rec ? 1u : 0u) : r.cnt[k];
          uint32_t total_k;
          base[k] = run[k] + block_excl_scan(mine_k, &total_k, sh_scan);
          run[k] += total_k;
        }
        if (is_rec) stream_emit<SCHEMA>(a, g, win, L, w, wd, tp, r, base, (uint64_t)base[ST_REC]);
      }
    }
    __syncthreads();
    if (pass == 0) {
      if (warp == 0) stream_resolve<MASK>(a, tile, lane, sh_sum, 1, sh_tot, sh_base, &sh_ok);
      __syncthreads();
      if (!sh_ok) return;
    } else {
      for (int d = 16; d; d >>= 1) { nerr += __shfl_xor_sync(0xFFFFFFFFu, nerr, d); nfast += __shfl_xor_sync(0xFFFFFFFFu, nfast, d); }
      if (lane == 0 && nerr) atomicAdd(&a.res->n_errors, (unsigned long long)nerr);
      if (lane == 0 && nfast) atomicAdd(&a.res->n_fast, (unsigned long long)nfast);
    }
  }
  if (tile == a.ntiles - 1) stream_close_offsets(a, tid, sh_base, sh_tot);
}

/* Which owned line a thread takes (>= nown: none). A tile with at most an eighth, a quarter or half as many lines as
 * threads gives every 8th, 4th or 2nd thread a line: its warps share the work, and fewer lanes of a warp sit on
 * records that make them take different paths. The order of the lines along the threads stays, so the scans do. */
__device__ __forceinline__ uint32_t stream_line_of_thread(uint32_t tid, uint32_t nown) {
  const uint32_t sh = nown <= ST_THREADS / 8 ? 3u : (nown <= ST_THREADS / 4 ? 2u : (nown <= ST_THREADS / 2 ? 1u : 0u));
  return (tid & ((1u << sh) - 1u)) ? ST_NONE : (tid >> sh);
}

/* Everything a tile does once its line list stands: thread j takes owned line j, tokenises it, the tile's counts go
 * through the look-back, every record is emitted. SPECIAL = the tile holds a line that runs out of the window or a
 * long record of a model with lists: the block finds the end of the former together, and whole warps walk the
 * latter (pj_wide.cuh). The common case is compiled without any of that. */
template <int SCHEMA, bool SPECIAL>
__device__ __forceinline__ void stream_tile_rest(const StreamArgs& a, const StreamGeom& g, uint8_t* win, const uint16_t* list, uint32_t* tape,
                                                 uint32_t tile, uint32_t nlf, uint32_t nown, long long c0, long long c1) {
  constexpr uint32_t MASK = StreamSlots<SCHEMA>::mask;
  constexpr uint32_t NWARPS = ST_THREADS / 32;
  constexpr bool LISTS = SCHEMA == PJ_SCHEMA_PET || SCHEMA == PJ_SCHEMA_MIXED;
  __shared__ uint32_t sh_warp[ST_NLB][NWARPS];
  __shared__ uint32_t sh_tot[ST_NLB], sh_base[ST_NLB];
  __shared__ uint32_t sh_ok;
  __shared__ unsigned long long sh_end;
  __shared__ uint32_t sh_nwide, sh_wnext[2];
  __shared__ WideSlot sh_wide[SPECIAL ? ST_WIDE_CAP : 1];
  __shared__ uint32_t sh_wtape[SPECIAL ? ST_THREADS * TAPE_MIN_CAP : 1]; /* the warps' scratch tapes: the threads' own hold records that wait for emission */
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const uint32_t mis = g.mis;

  StreamLine L;
  L.s = 0; L.fits = 0; L.gstart = 0;
  bool is_rec = false;
  const uint32_t nlist = nlf < ST_LF_CAP ? nlf : ST_LF_CAP;
  const uint32_t j = stream_line_of_thread(tid, nown); /* a tile with few lines spreads them over its warps */
  if (j < nown) {
    L.s = list[j];
    L.fits = (j + 1 < nlist) || g.to_limit;
    L.gstart = g.v0 + L.s - mis;
    is_rec = stream_is_record(win, L.s, g, a.in, a.limit, (int)a.is_last);
  }
  uint64_t end_known = ~0ull;
  bool wide = false;
  uint32_t wslot = 0;
  if (SPECIAL) {
    if (tid == 0) { sh_nwide = 0; sh_wnext[0] = 0; sh_wnext[1] = 0; }
    /* at most one line of a tile runs out of the window (the last one): the block finds its end together */
    if (__syncthreads_or(is_rec && !L.fits)) {
      const uint64_t e = stream_find_end(a, g.v0 + ST_WIN_BYTES - mis, tid, &sh_end);
      if (is_rec && !L.fits) end_known = e;
    }
    /* long records of the models with lists leave the thread-per-record path */
    if (LISTS && is_rec) {
      const uint32_t e_w = (j + 1 < nlist) ? (uint32_t)list[j + 1] - 1u : g.hi_valid;
      const uint64_t gend = L.fits ? g.v0 + e_w - mis : end_known;
      if (gend != ~0ull && gend - L.gstart >= ST_WIDE_MIN) {
        wslot = atomicAdd(&sh_nwide, 1u);
        if (wslot < ST_WIDE_CAP) {
          wide = true;
          sh_wide[wslot].gstart = L.gstart; sh_wide[wslot].gend = gend; sh_wide[wslot].fits = L.fits;
        }
      }
    }
  }
  Tape tp;
  tp.e = tape + tid; tp.stride = ST_THREADS; tp.cap = ST_TAPE_CAP; tp.n = 0;
  StreamRec<SCHEMA> r;
  Win w, wd;
  r.type = PJ_TYPE_NONE; r.err = 0; r.err_off = 0; r.fast = 0; r.locked = 0; r.direct = 0; r.tape_n = 0;
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) r.cnt[k] = 0;
  if (SPECIAL) __syncthreads(); /* the slots of the long records stand */
  stream_tokenise<SCHEMA>(a, g, win, is_rec && !wide, L, end_known, tp, r, w, wd);
  uint32_t nw = 0;
  if (SPECIAL) { /* every warp goes on to its share of the long records as soon as its own threads are done */
    nw = sh_nwide < ST_WIDE_CAP ? sh_nwide : ST_WIDE_CAP;
    if (nw) {
      if (tid == 0) atomicAdd(&a.res->n_wide, (unsigned long long)nw);
      const long long w0c = clock64();
      for (;;) { /* the warps take the long records as they get free: they differ a lot in length */
        uint32_t q = 0;
        if (lane == 0) q = atomicAdd(&sh_wnext[0], 1u);
        q = __shfl_sync(0xFFFFFFFFu, q, 0);
        if (q >= nw) break;
        stream_wide_size<SCHEMA>(a, g, win, sh_wtape, &sh_wide[q]);
      }
      __syncthreads();
      if (tid == 0) atomicAdd(&a.res->wide_cycles[0], (unsigned long long)(clock64() - w0c));
      if (wide) {
        r.type = sh_wide[wslot].type; r.err = sh_wide[wslot].err; r.err_off = sh_wide[wslot].err_off;
#pragma unroll
        for (uint32_t k = 0; k < NSLOT; ++k) r.cnt[k] = sh_wide[wslot].cnt[k];
      }
    }
  }
  {
    uint32_t pk = (r.err ? 1u : 0u) | (r.fast << 16);
    for (int d = 16; d; d >>= 1) pk += __shfl_down_sync(0xFFFFFFFFu, pk, d);
    if (lane == 0 && (pk & 0xFFFF)) atomicAdd(&a.res->n_errors, (unsigned long long)(pk & 0xFFFF));
    if (lane == 0 && (pk >> 16)) atomicAdd(&a.res->n_fast, (unsigned long long)(pk >> 16));
  }

  /* ---- positions inside the tile, then the look-back ---- */
  uint32_t base[ST_NLB];
#pragma unroll
  for (uint32_t k = 0; k < ST_NLB; ++k) {
    if (!((MASK >> k) & 1u)) { base[k] = 0; continue; }
    const uint32_t mine_k = k == ST_REC ? (is_rec ? 1u : 0u) : r.cnt[k];
    const uint32_t inc = warp_incl_scan(mine_k);
    if (lane == 31) sh_warp[k][warp] = inc;
    base[k] = inc - mine_k;
  }
  __syncthreads();
  const long long c2 = clock64();
#pragma unroll
  for (uint32_t k = 0; k < ST_NLB; ++k) {
    if (!((MASK >> k) & 1u)) continue;
#pragma unroll
    for (uint32_t q = 0; q < NWARPS; ++q) if (q < warp) base[k] += sh_warp[k][q];
  }
  if (warp == 0) stream_resolve<MASK>(a, tile, lane, &sh_warp[0][0], NWARPS, sh_tot, sh_base, &sh_ok);
  __syncthreads();
  const long long c3 = clock64();
  if (!sh_ok) return;

  /* ---- emit ---- */
  if (is_rec) {
    uint32_t gb[NSLOT];
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) gb[k] = base[k] + sh_base[k];
    const uint64_t i = (uint64_t)sh_base[ST_REC] + base[ST_REC];
    if (SPECIAL && wide && !r.err) { /* its warp writes the rest */
      stream_emit_head<SCHEMA>(a, L, r, gb, i);
      sh_wide[wslot].rec_index = i;
#pragma unroll
      for (uint32_t k = 0; k < NSLOT; ++k) sh_wide[wslot].base[k] = gb[k];
    } else stream_emit<SCHEMA>(a, g, win, L, w, wd, tp, r, gb, i);
  }
  if (SPECIAL && nw) {
    __syncthreads();
    const long long w1c = clock64();
    for (;;) {
      uint32_t q = 0;
      if (lane == 0) q = atomicAdd(&sh_wnext[1], 1u);
      q = __shfl_sync(0xFFFFFFFFu, q, 0);
      if (q >= nw) break;
      if (!sh_wide[q].err) stream_wide_emit<SCHEMA>(a, g, win, sh_wtape, &sh_wide[q]);
    }
    __syncthreads();
    if (tid == 0) atomicAdd(&a.res->wide_cycles[1], (unsigned long long)(clock64() - w1c));
  }
  __syncthreads();
  if (tid == 0) {
    const long long c4 = clock64();
    atomicAdd(&a.res->phase_cycles[0], (unsigned long long)(c1 - c0));
    atomicAdd(&a.res->phase_cycles[1], (unsigned long long)(c2 - c1));
    atomicAdd(&a.res->phase_cycles[2], (unsigned long long)(c3 - c2));
    atomicAdd(&a.res->phase_cycles[3], (unsigned long long)(c4 - c3));
  }
  /* the last tile closes the offset columns */
  if (tile == a.ntiles - 1) stream_close_offsets(a, tid, sh_base, sh_tot);
}
/* The tiles with a line that leaves the window or with long records: out of line, so that the common tile keeps its
 * registers. */
template <int SCHEMA>
__device__ __noinline__ void stream_special_tile(const StreamArgs& a, const StreamGeom& g, uint8_t* win, const uint16_t* list, uint32_t* tape,
                                                 uint32_t tile, uint32_t nlf, uint32_t nown, long long c0, long long c1) {
  stream_tile_rest<SCHEMA, true>(a, g, win, list, tape, tile, nlf, nown, c0, c1);
}

template <int SCHEMA>
__global__ void __launch_bounds__(ST_THREADS, 512 / ST_THREADS) k_parse_stream(const __grid_constant__ StreamArgs a) {
  constexpr bool LISTS = SCHEMA == PJ_SCHEMA_PET || SCHEMA == PJ_SCHEMA_MIXED;
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ uint32_t sh_scan[33];
  __shared__ uint32_t sh_tile;
  __shared__ __align__(8) unsigned long long sh_mbar;
  const uint32_t tid = threadIdx.x;
  uint8_t* win = smem;
  uint16_t* lfb = reinterpret_cast<uint16_t*>(smem + ST_SMEM_WIN);
  uint16_t* list = reinterpret_cast<uint16_t*>(smem + ST_SMEM_WIN + ST_SMEM_LFB);
  uint32_t* tape = reinterpret_cast<uint32_t*>(smem + ST_SMEM_WIN + ST_SMEM_LFB + ST_SMEM_LIST);

  if (tid == 0) { sh_tile = atomicAdd(a.ticket, 1u); mbar_init(&sh_mbar, 1); }
  __syncthreads();
  const uint32_t tile = sh_tile;
  if (tile >= a.ntiles) return;
  const long long c0 = clock64();
  const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(a.in) & 15u);
  const StreamGeom g = stream_geom(mis, a.len, a.limit, a.tile_bytes, tile);

  /* ---- stage the window: one bulk copy of whole 16-byte blocks (the first and the last one may hold bytes that are
     not input: they lie in the same aligned 16 bytes as input bytes, so they are readable; they are masked below) */
  int stage_failed = 0;
  if (g.copy_bytes) {
    if (tid == 0) { mbar_expect_tx(&sh_mbar, g.copy_bytes); bulk_g2s(win, a.in - mis + g.v0, g.copy_bytes, &sh_mbar); }
    if (!mbar_try_wait(&sh_mbar, 0)) {
      const unsigned long long t0 = global_ns();
      while (!mbar_try_wait(&sh_mbar, 0)) {
        if (global_ns() - t0 > a.spin_limit_ns) { stage_failed = 1; break; }
        __nanosleep(64);
      }
    }
  }
  if (__syncthreads_or(stage_failed)) { /* the block gives up together: the results of the call are void */
    if (tid == 0) {
      atomicExch(&a.res->timeout, 1u);
      /* the copy may still be in flight, and the block's shared memory must not pass to another block before it has
         landed: one thread stays and waits for it, again with a limit */
      const unsigned long long t1 = global_ns();
      while (!mbar_try_wait(&sh_mbar, 0) && global_ns() - t1 <= a.spin_limit_ns) __nanosleep(256);
    }
    return;
  }
  if (tid < ST_WIN_PAD) win[g.hi_valid + tid] = '\n';
  __syncthreads();

  /* ---- line index of the window ---- */
  const bool virtual_first = tile == 0 && a.is_first && tid == 0 && a.limit > 0;
  uint32_t packed = virtual_first ? 0x00010001u : 0u; /* lines: low half all, high half owned */
#pragma unroll 1
  for (uint32_t k = 0; k < ST_CPT; ++k) {
    const uint32_t c = tid * ST_CPT + k;
    const uint32_t m = stream_chunk_mask(win, c * 16u, g);
    lfb[c] = (uint16_t)m;
    packed += (uint32_t)__popc(m) + ((uint32_t)__popc(stream_own_bits(m, c * 16u, g)) << 16);
  }
  uint32_t packed_total;
  const uint32_t packed_excl = block_excl_scan(packed, &packed_total, sh_scan);
  const uint32_t nlf = packed_total & 0xFFFFu, nown = packed_total >> 16;
  const uint32_t first_idx = packed_excl & 0xFFFFu;
  if (nown > ST_THREADS) {
    stream_overflow_tile<SCHEMA>(a, g, win, lfb, list, tape, tile, first_idx, nlf, nown, virtual_first);
    return;
  }
  stream_fill_list(list, lfb, tid, first_idx, 0, virtual_first, mis);
  __syncthreads();
  const long long c1 = clock64();

  /* a line that leaves the window, or a long record of a model with lists, sends the tile the other way */
  bool special = false;
  if (tid < nown) { /* any thread may look at any line here */
    const uint32_t nlist = nlf < ST_LF_CAP ? nlf : ST_LF_CAP;
    const bool has_next = tid + 1 < nlist;
    const uint32_t len = (has_next ? (uint32_t)list[tid + 1] : g.hi_valid) - (uint32_t)list[tid];
    special = !(has_next || g.to_limit) || (LISTS && len >= ST_WIDE_MIN);
  }
  if (__syncthreads_or(special)) stream_special_tile<SCHEMA>(a, g, win, list, tape, tile, nlf, nown, c0, c1);
  else stream_tile_rest<SCHEMA, false>(a, g, win, list, tape, tile, nlf, nown, c0, c1);
}

}  // namespace pj
#endif
