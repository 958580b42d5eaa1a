/*
 * pj_host_emu.cpp — TEST INFRASTRUCTURE. Compiles the per-record device code of the library
 * (pj_core.cuh, pj_fast.cuh, pj_write_core.cuh, pj_write_fast.cuh, pj_array.cuh: every function in them is
 * host + device) for the host and runs it one "thread" after another, with the tile kernel's bookkeeping
 * (windows, tapes, tile-local scans) restated sequentially. tests/test_host_emulation.py fuzzes it against
 * the CPU checker, so the exactness of the device-side parsers and writers is tested without a GPU.
 * Nothing in the product links or loads this file.
 */
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <algorithm>
#include <vector>

#include "pj_core.cuh"
#include "pj_index.cuh"
#include "pj_write_core.cuh"

using namespace pj;

/* PJ_OPT_* bits for the exact parser (tests set them before a call) */
static uint32_t g_opts = 0;
extern "C" void emu_set_options(uint32_t opts) { g_opts = opts; }


extern "C" int emu_parse(uint32_t schema, uint32_t framing, const uint8_t* in, uint64_t len, uint64_t slack,
                         int is_first, int is_last, uint64_t goff, pj_columns* out,
                         const uint64_t* ext_s, const uint64_t* ext_e, const uint8_t* ext_blank, uint64_t n_ext) {
  Schema S; build_schema(&S);
  DevCols dc; for (int i = 0; i < PJ_MAX_COLS; ++i) dc.ptr[i] = out->col[i].ptr;
  uint64_t limit = len + slack;
  std::vector<uint64_t> starts, ends; std::vector<uint8_t> blank;
  if (framing == PJ_FRAMING_NDJSON) {
    for (uint64_t p = 0; p <= len; ++p) {
      bool cand = (p == 0) ? is_first : in[p - 1] == '\n';
      if (cand && nd_is_record(in, p, limit, is_last)) { starts.push_back(p); ends.push_back(limit); blank.push_back(0); }
    }
  } else {
    for (uint64_t i = 0; i < n_ext; ++i) { starts.push_back(ext_s[i]); ends.push_back(ext_e[i]); blank.push_back(ext_blank[i]); }
  }
  uint64_t N = starts.size();
  std::vector<uint32_t> cnt((size_t)NSLOT * (N + 1), 0);
  std::vector<uint8_t> types(N, 0);
  uint8_t* ek = (uint8_t*)out->col[PJ_COL_ERR_KIND].ptr; uint32_t* eo = (uint32_t*)out->col[PJ_COL_ERR_OFF].ptr;
  uint64_t* rs = (uint64_t*)out->col[PJ_COL_REC_START].ptr;
  uint64_t nerr = 0;
  for (uint64_t i = 0; i < N; ++i) {
    Rd r; r.in = in; r.lf_ws = framing == PJ_FRAMING_ARRAY; r.limit = r.lf_ws ? ends[i] : limit; r.open_end = r.lf_ws ? 0 : !is_last; r.opts = g_opts;
    PS s; s.p = starts[i]; s.err = 0; s.err_pos = 0;
    Out<false> o; o.cols = &dc;
    uint32_t t;
    if (blank[i]) { fail(s, PJ_E_SYNTAX, ends[i]); t = 0; }
    else t = parse_record<false>(S, r, s, schema, o, i);
    if (s.err) { t = 0; for (uint32_t k = 0; k < NSLOT; ++k) o.cnt[k] = 0; }
    types[i] = (uint8_t)t;
    for (uint32_t k = 0; k < NSLOT; ++k) cnt[(size_t)k * (N + 1) + i] = o.cnt[k];
    rs[i] = starts[i] + goff; ek[i] = (uint8_t)s.err; eo[i] = s.err ? (uint32_t)(s.err_pos - starts[i]) : 0;
    nerr += s.err != 0;
    if (schema == PJ_SCHEMA_MIXED) ((uint8_t*)out->col[PJ_COL_REC_TYPE].ptr)[i] = (uint8_t)t;
  }
  uint32_t total[NSLOT];
  for (uint32_t k = 0; k < NSLOT; ++k) {
    uint32_t acc = 0;
    for (uint64_t i = 0; i <= N; ++i) { uint32_t c = cnt[(size_t)k * (N + 1) + i]; cnt[(size_t)k * (N + 1) + i] = acc; acc += c; }
    total[k] = acc;
  }
  for (uint64_t i = 0; i < N; ++i) {
    Out<true> o; o.cols = &dc;
    for (uint32_t k = 0; k < NSLOT; ++k) { o.base[k] = cnt[(size_t)k * (N + 1) + i]; o.room[k] = cnt[(size_t)k * (N + 1) + i + 1] - o.base[k]; }
    if (schema == PJ_SCHEMA_MIXED) ((uint32_t*)out->col[PJ_COL_REC_ROW].ptr)[i] = ek[i] ? 0xFFFFFFFFu : o.base[types[i] - 1];
    if (ek[i]) { if (schema != PJ_SCHEMA_MIXED) store_absent<true>(S, schema, o, i); continue; }
    Rd r; r.in = in; r.lf_ws = framing == PJ_FRAMING_ARRAY; r.limit = r.lf_ws ? ends[i] : limit; r.open_end = r.lf_ws ? 0 : !is_last; r.opts = g_opts;
    PS s; s.p = starts[i]; s.err = 0; s.err_pos = 0;
    uint32_t t = parse_record<true>(S, r, s, schema, o, i);
    if (s.err || t != types[i]) { fprintf(stderr, "emit pass disagrees at record %llu\n", (unsigned long long)i); return -1; }
  }
  // sentinels + counts
  uint64_t rows[4] = {0, N, N, N};
  if (schema == PJ_SCHEMA_MIXED) { rows[1] = total[0]; rows[2] = total[1]; rows[3] = total[2]; }
  for (int c = 0; c < PJ_MAX_COLS; ++c) out->col[c].count = 0;
  out->col[PJ_COL_REC_START].count = out->col[PJ_COL_ERR_KIND].count = out->col[PJ_COL_ERR_OFF].count = N;
  if (schema == PJ_SCHEMA_MIXED) out->col[PJ_COL_REC_TYPE].count = out->col[PJ_COL_REC_ROW].count = N;
  FinalizePlan plan; build_finalize_plan(S, schema, &plan);
  for (uint32_t k = 0; k < plan.n; ++k) {
    const FinalizeItem& it = plan.item[k];
    uint64_t nrows = it.rows_slot == 0xFF ? N : total[it.rows_slot];
    if (it.sentinel_slot != 0xFF) { ((uint32_t*)out->col[it.col].ptr)[nrows] = total[it.sentinel_slot]; out->col[it.col].count = nrows + 1; }
    else out->col[it.col].count = nrows;
  }
  out->schema = schema; out->n_records = N; out->n_errors = nerr;
  for (int t = 0; t < 4; ++t) out->n_rows[t] = 0;
  if (schema == PJ_SCHEMA_MIXED) { out->n_rows[1] = rows[1]; out->n_rows[2] = rows[2]; out->n_rows[3] = rows[3]; }
  else out->n_rows[schema] = N;
  return 0;
}

extern "C" int emu_write(uint32_t schema, uint32_t framing, int inclusion, const pj_columns* cols, uint8_t* out,
                         uint64_t cap, uint64_t* out_len) {
  Schema S; build_schema(&S);
  DevCols dc; for (int i = 0; i < PJ_MAX_COLS; ++i) dc.ptr[i] = cols->col[i].ptr;
  uint64_t n = schema == PJ_SCHEMA_MIXED ? cols->n_records : cols->n_rows[schema];
  bool arr = framing == PJ_FRAMING_ARRAY;
  std::vector<uint64_t> off(n + 1, 0);
  uint64_t acc = arr ? 1 : 0, written = 0;
  for (uint64_t i = 0; i < n; ++i) {
    WOut w; w.dst = nullptr; w.n = 0;
    uint32_t type; uint64_t row;
    off[i] = acc;
    if (!write_locate(schema, &dc, i, &type, &row)) continue;
    write_record<false>(S, &dc, type, row, inclusion, w);
    acc += w.n + 1; /* + LF, or the separating comma / closing bracket */
    written++;
  }
  off[n] = acc;
  uint64_t total = arr ? (written ? acc : 2) : acc;
  *out_len = total;
  if (total > cap) return PJ_ERR_CAPACITY;
  if (arr) { out[0] = '['; out[total - 1] = ']'; }
  for (uint64_t i = 0; i < n; ++i) {
    uint32_t type; uint64_t row;
    if (!write_locate(schema, &dc, i, &type, &row)) continue;
    WOut w; w.dst = out + off[i]; w.n = 0;
    write_record<true>(S, &dc, type, row, inclusion, w);
    out[off[i] + w.n] = arr ? (uint8_t)(off[i] + w.n + 1 == total ? ']' : ',') : (uint8_t)'\n';
  }
  return 0;
}

#include "pj_write_fast.cuh"
extern "C" int emu_write_fast(uint32_t schema, uint32_t framing, int inclusion, const pj_columns* cols, uint8_t* out,
                         uint64_t cap, uint64_t* out_len) {
  Schema S; build_schema(&S);
  DevCols dc; for (int i = 0; i < PJ_MAX_COLS; ++i) dc.ptr[i] = cols->col[i].ptr;
  uint64_t n = schema == PJ_SCHEMA_MIXED ? cols->n_records : cols->n_rows[schema];
  bool arr = framing == PJ_FRAMING_ARRAY;
  bool plain = true;
  {
    auto scan = [&](const ObjDesc& O, auto&& self) -> void {
      for (int i = 0; i < (int)O.nfields; ++i) {
        const FieldDesc& F = O.f[i]; int col = -1;
        if (F.kind == K_STR) col = F.col + 1; else if (F.kind == K_LIST_STR) col = F.col + 2;
        else if (F.kind == K_OBJ || F.kind == K_LIST_OBJ) self(S.obj[F.child], self);
        if (col >= 0) for (uint64_t k = 0; k < cols->col[col].count; ++k) if (escape_extra_byte(((const uint8_t*)cols->col[col].ptr)[k])) plain = false;
      }
    };
    bool mixed = schema == PJ_SCHEMA_MIXED;
    if (schema == PJ_SCHEMA_PET || mixed) scan(S.obj[OBJ_PET], scan);
    if (schema == PJ_SCHEMA_ORDER || mixed) scan(S.obj[OBJ_ORDER], scan);
    if (schema == PJ_SCHEMA_USER || mixed) scan(S.obj[OBJ_USER], scan);
  }
  std::vector<uint64_t> off(n + 1, 0);
  uint64_t acc = arr ? 1 : 0, written = 0;
  for (uint64_t i = 0; i < n; ++i) {
    WOut w; w.dst = nullptr; w.n = 0;
    uint32_t type; uint64_t row;
    off[i] = acc;
    if (!write_locate(schema, &dc, i, &type, &row)) continue;
    if (plain) fwrite_record<false, true>(&dc, type, row, inclusion, w); else fwrite_record<false, false>(&dc, type, row, inclusion, w);
    acc += w.n + 1; /* + LF, or the separating comma / closing bracket */
    written++;
  }
  off[n] = acc;
  uint64_t total = arr ? (written ? acc : 2) : acc;
  *out_len = total;
  if (total > cap) return PJ_ERR_CAPACITY;
  if (arr) { out[0] = '['; out[total - 1] = ']'; }
  for (uint64_t i = 0; i < n; ++i) {
    uint32_t type; uint64_t row;
    if (!write_locate(schema, &dc, i, &type, &row)) continue;
    WOut w; w.dst = out + off[i]; w.n = 0;
    if (plain) fwrite_record<true, true>(&dc, type, row, inclusion, w); else fwrite_record<true, false>(&dc, type, row, inclusion, w);
    out[off[i] + w.n] = arr ? (uint8_t)(off[i] + w.n + 1 == total ? ']' : ',') : (uint8_t)'\n';
  }
  return 0;
}

#include "pj_fast.cuh"
#include "pj_lock.cuh"
static uint64_t g_fail_fast = 0;
extern "C" uint64_t emu_fail_fast_count() { return g_fail_fast; }
/* the lockstep tokeniser of pj_lock.cuh as the first attempt at every staged NDJSON record (as in the stream kernel) */
static int g_use_lock = 0;
static uint64_t g_lock_accepted = 0, g_lock_failed = 0;
extern "C" void emu_use_lock(int on) { g_use_lock = on; g_lock_accepted = 0; g_lock_failed = 0; }
extern "C" uint64_t emu_lock_accepted() { return g_lock_accepted; }
extern "C" uint64_t emu_lock_failed() { return g_lock_failed; }
template <int SCHEMA>
static int emu_fast_t(uint32_t framing, const uint8_t* in, uint64_t len, uint64_t slack, int is_first, int is_last, uint64_t goff,
                      pj_columns* out, uint64_t* n_fast, uint32_t tile_recs, uint32_t win_bytes, uint32_t tape_cap,
                      const uint64_t* ext_s, const uint64_t* ext_e, const uint8_t* ext_blank, uint64_t n_ext) {
  const uint32_t schema = SCHEMA;
  Schema S; build_schema(&S);
  DevCols dc; for (int i = 0; i < PJ_MAX_COLS; ++i) dc.ptr[i] = out->col[i].ptr;
  uint64_t limit = len + slack;
  std::vector<uint64_t> starts, ends; std::vector<uint8_t> blank;
  if (framing == PJ_FRAMING_NDJSON) {
    for (uint64_t p = 0; p <= len; ++p) {
      bool cand = (p == 0) ? is_first : in[p - 1] == '\n';
      if (cand && nd_is_record(in, p, limit, is_last)) { starts.push_back(p); ends.push_back(limit); blank.push_back(0); }
    }
  } else {
    for (uint64_t i = 0; i < n_ext; ++i) { starts.push_back(ext_s[i]); ends.push_back(ext_e[i]); blank.push_back(ext_blank[i]); }
  }
  uint64_t N = starts.size();
  uint8_t* ek = (uint8_t*)out->col[PJ_COL_ERR_KIND].ptr; uint32_t* eo = (uint32_t*)out->col[PJ_COL_ERR_OFF].ptr;
  uint64_t* rs = (uint64_t*)out->col[PJ_COL_REC_START].ptr;
  uint64_t nerr = 0, nfast = 0; uint64_t& nfail_fast = g_fail_fast;
  uint32_t run[NSLOT]; for (uint32_t k = 0; k < NSLOT; ++k) run[k] = 0;
  const uint32_t lf_ws = framing == PJ_FRAMING_ARRAY;
  for (uint64_t r0 = 0; r0 < N; r0 += tile_recs) {
    uint32_t nrec = (uint32_t)std::min<uint64_t>(tile_recs, N - r0);
    uint64_t span_lo = starts[r0];
    uint64_t span_hi = lf_ws ? ends[r0 + nrec - 1] : (r0 + nrec < N ? starts[r0 + nrec] : limit);
    int64_t w0 = ((int64_t)span_lo / 16) * 16;
    uint64_t copy_hi = std::min<uint64_t>(limit, span_hi + 32);
    bool fits = (copy_hi - w0) + 64 <= win_bytes;
    std::vector<uint8_t> winbuf(win_bytes + 64, 0xEE);
    if (fits) { memcpy(winbuf.data(), in + w0, copy_hi - w0); memset(winbuf.data() + (copy_hi - w0), '\n', 32); }
    Win w; w.s = winbuf.data(); w.w0 = w0;
    std::vector<uint32_t> tape((size_t)tape_cap * tile_recs + 1);
    std::vector<FVals> V(nrec), CV(nrec);
    std::vector<uint32_t> types(nrec), isfast(nrec), islock(nrec, 0), ntape(nrec), st32v(nrec), lim32v(nrec);
    std::vector<Win> wins(nrec);
    std::vector<uint32_t> cnt((size_t)nrec * NSLOT, 0);
    for (uint32_t t = 0; t < nrec; ++t) {
      uint64_t i = r0 + t;
      uint64_t lim = lf_ws ? ends[i] : limit;
      Tape tp; tp.e = tape.data() + t; tp.stride = tile_recs; tp.cap = tape_cap; tp.n = 0;
      uint32_t c[NSLOT]; uint32_t type = 0;
      uint64_t my_end = lf_ws ? ends[i] : (i + 1 < N ? starts[i + 1] : limit);
      bool direct = !fits && my_end + 32 <= limit;
      Win wr = w;
      if (direct) { uint32_t mis4 = (uint32_t)((uintptr_t)(in + starts[i]) & 3u); wr.s = in + starts[i] - mis4; wr.w0 = (int64_t)starts[i] - mis4; }
      wins[t] = wr;
      uint64_t rel = (uint64_t)((int64_t)lim - wr.w0);
      uint32_t lim32 = rel > 0xFFFFFFF0ull ? 0xFFFFFFF0u : (uint32_t)rel;
      uint32_t fk = 0, fp = 0, st32 = (uint32_t)((int64_t)starts[i] - wr.w0);
      st32v[t] = st32; lim32v[t] = lim32;
      uint32_t verdict = 0;
      if (g_use_lock && fits && !lf_ws) {
        verdict = lock_record<SCHEMA>(wr, true, st32, lim32, !is_last, &type, V[t], CV[t], c, tp, &fk, &fp);
        if (verdict == FAST_ACCEPTED) { g_lock_accepted++; islock[t] = 1; }
        if (verdict == FAST_FAILED) g_lock_failed++;
      }
      if (verdict == FAST_FAILED && (((g_opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL) && fk == PJ_E_ENUM) || ((g_opts & PJ_OPT_COERCE_SCALARS) && fk == PJ_E_TYPE))) verdict = FAST_REFUSED;
      if (verdict != FAST_REFUSED) {}
      else if ((fits || direct) && !blank[i]) {
        if (!direct) verdict = fast_record<SCHEMA>(wr, st32, lim32, lf_ws, lf_ws ? 0 : !is_last, &type, V[t], CV[t], c, tp, &fk, &fp);
        else { verdict = fast_outline<SCHEMA>(wr, st32, lim32, lf_ws, lf_ws ? 0 : !is_last, nullptr, nullptr, i, tp, c, &type, &fk, &fp); tp.n = tp.cap + 1; }
      }
      if (verdict == FAST_FAILED && (((g_opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL) && fk == PJ_E_ENUM) || ((g_opts & PJ_OPT_COERCE_SCALARS) && fk == PJ_E_TYPE))) verdict = FAST_REFUSED;
      bool ok = verdict == FAST_ACCEPTED;
      PS s; s.p = starts[i]; s.err = 0; s.err_pos = 0;
      if (verdict == FAST_FAILED) { nfail_fast++; s.err = fk; s.err_pos = starts[i] + (fp - st32); type = 0; for (uint32_t k = 0; k < NSLOT; ++k) cnt[(size_t)t * NSLOT + k] = 0; }
      else if (ok) { nfast++; for (uint32_t k = 0; k < NSLOT; ++k) cnt[(size_t)t * NSLOT + k] = c[k]; ntape[t] = tp.n; }
      else {
        Rd r; r.in = fits ? winbuf.data() - w0 : in; r.lf_ws = lf_ws; r.limit = lim; r.open_end = lf_ws ? 0 : !is_last; r.opts = g_opts;
        Out<false> o; o.cols = &dc;
        if (blank[i]) { fail(s, PJ_E_SYNTAX, ends[i]); type = 0; }
        else type = parse_record<false>(S, r, s, schema, o, i);
        if (s.err) type = 0;
        for (uint32_t k = 0; k < NSLOT; ++k) cnt[(size_t)t * NSLOT + k] = s.err ? 0 : o.cnt[k];
      }
      types[t] = type; isfast[t] = ok;
      rs[i] = starts[i] + goff; ek[i] = (uint8_t)s.err; eo[i] = s.err ? (uint32_t)(s.err_pos - starts[i]) : 0;
      nerr += s.err != 0;
      if (schema == PJ_SCHEMA_MIXED) ((uint8_t*)out->col[PJ_COL_REC_TYPE].ptr)[i] = (uint8_t)type;
    }
    for (uint32_t t = 0; t < nrec; ++t) {
      uint64_t i = r0 + t;
      Out<true> o; o.cols = &dc;
      for (uint32_t k = 0; k < NSLOT; ++k) { o.base[k] = run[k]; o.room[k] = cnt[(size_t)t * NSLOT + k]; run[k] += o.room[k]; }
      if (schema == PJ_SCHEMA_MIXED) ((uint32_t*)out->col[PJ_COL_REC_ROW].ptr)[i] = ek[i] ? 0xFFFFFFFFu : o.base[types[t] - 1];
      if (ek[i]) { if (schema != PJ_SCHEMA_MIXED) store_absent<true>(S, schema, o, i); continue; }
      if (isfast[t]) {
        Tape tp; tp.e = tape.data() + t; tp.stride = tile_recs; tp.cap = tape_cap; tp.n = ntape[t];
        if (islock[t] && tp.n <= tp.cap) lock_emit<SCHEMA>(wins[t], &dc, types[t], V[t], CV[t], tp, o.base, o.room, i);
        else if (tp.n <= tp.cap) fast_emit<SCHEMA>(wins[t], &dc, types[t], V[t], CV[t], tp, o.base, i);
        else { uint32_t a_, b_, c_; fast_outline<SCHEMA>(wins[t], st32v[t], lim32v[t], lf_ws, lf_ws ? 0 : !is_last, &dc, o.base, i, tp, nullptr, &a_, &b_, &c_); }
      } else {
        uint64_t lim = lf_ws ? ends[i] : limit;
        Rd r; r.in = fits ? winbuf.data() - w0 : in; r.lf_ws = lf_ws; r.limit = lim; r.open_end = lf_ws ? 0 : !is_last; r.opts = g_opts;
        PS s; s.p = starts[i]; s.err = 0; s.err_pos = 0;
        uint32_t ty = parse_record<true>(S, r, s, schema, o, i);
        if (s.err || ty != types[t]) { fprintf(stderr, "emit pass disagrees at record %llu\n", (unsigned long long)i); return -1; }
      }
    }
  }
  uint32_t* total = run;
  for (int c = 0; c < PJ_MAX_COLS; ++c) out->col[c].count = 0;
  out->col[PJ_COL_REC_START].count = out->col[PJ_COL_ERR_KIND].count = out->col[PJ_COL_ERR_OFF].count = N;
  if (schema == PJ_SCHEMA_MIXED) out->col[PJ_COL_REC_TYPE].count = out->col[PJ_COL_REC_ROW].count = N;
  FinalizePlan plan; build_finalize_plan(S, schema, &plan);
  for (uint32_t k = 0; k < plan.n; ++k) {
    const FinalizeItem& it = plan.item[k];
    uint64_t nrows = it.rows_slot == 0xFF ? N : total[it.rows_slot];
    if (it.sentinel_slot != 0xFF) { ((uint32_t*)out->col[it.col].ptr)[nrows] = total[it.sentinel_slot]; out->col[it.col].count = nrows + 1; }
    else out->col[it.col].count = nrows;
  }
  out->schema = schema; out->n_records = N; out->n_errors = nerr;
  for (int t = 0; t < 4; ++t) out->n_rows[t] = 0;
  if (schema == PJ_SCHEMA_MIXED) { out->n_rows[1] = total[0]; out->n_rows[2] = total[1]; out->n_rows[3] = total[2]; }
  else out->n_rows[schema] = N;
  *n_fast = nfast;
  return 0;
}
extern "C" int emu_parse_fast(uint32_t schema, uint32_t framing, const uint8_t* in, uint64_t len, uint64_t slack,
                              int is_first, int is_last, uint64_t goff, pj_columns* out, uint64_t* n_fast, uint32_t tile_recs,
                              uint32_t win_bytes, uint32_t tape_cap,
                              const uint64_t* ext_s, const uint64_t* ext_e, const uint8_t* ext_blank, uint64_t n_ext) {
#define EMU_ARGS framing, in, len, slack, is_first, is_last, goff, out, n_fast, tile_recs, win_bytes, tape_cap, ext_s, ext_e, ext_blank, n_ext
  switch (schema) {
    case PJ_SCHEMA_PET: return emu_fast_t<PJ_SCHEMA_PET>(EMU_ARGS);
    case PJ_SCHEMA_ORDER: return emu_fast_t<PJ_SCHEMA_ORDER>(EMU_ARGS);
    case PJ_SCHEMA_USER: return emu_fast_t<PJ_SCHEMA_USER>(EMU_ARGS);
    default: return emu_fast_t<PJ_SCHEMA_MIXED>(EMU_ARGS);
  }
}

#include "pj_array.cuh"
extern "C" int emu_array_index(const uint8_t* in, uint64_t len, uint64_t* s_out, uint64_t* e_out, uint8_t* blank_out, uint64_t cap,
                               uint64_t* n_out, uint32_t* doc_kind, uint64_t* doc_off) {
  uint64_t nwords = (len + 63) >> 6;
  std::vector<ArrState> in_state(nwords + 1);
  ArrState st; st.c = 0; st.s = 0; st.d = 0;
  // pass 1 + 2: summaries composed in order (the kernels do the same with scans)
  for (uint64_t w = 0; w < nwords; ++w) {
    in_state[w] = st;
    uint32_t n = (uint32_t)std::min<uint64_t>(64, len - w * 64);
    WordMasks m = word_masks(in + w * 64, n);
    ArrFn f = fn_of_word(m);
    // also exercise composition: apply through compose with identity
    ArrFn g = fn_compose(fn_identity(), f);
    st = fn_apply(g, st);
  }
  in_state[nwords] = st;
  // pass 3
  std::vector<uint64_t> sep(nwords + 1, 0);
  uint64_t doc_min = ~0ull, first_opener = ~0ull;
  for (uint64_t w = 0; w < nwords; ++w) {
    uint32_t n = (uint32_t)std::min<uint64_t>(64, len - w * 64);
    WordMasks m = word_masks(in + w * 64, n);
    WordEval e = eval_word(m, in_state[w]);
    if (e.out.c != in_state[w + 1].c || e.out.s != in_state[w + 1].s || e.out.d != in_state[w + 1].d) { fprintf(stderr, "state mismatch\n"); return -1; }
    WordMarks k = mark_word(m, e, in_state[w].d);
    sep[w] = k.sep;
    if (k.doc_bit < 64) doc_min = std::min(doc_min, w * 64 + k.doc_bit);
    if (k.opener_bit < 64) first_opener = std::min(first_opener, w * 64 + k.opener_bit);
  }
  // pass 4
  uint64_t n = 0;
  for (uint64_t w = 0; w < nwords; ++w) {
    for (uint64_t m = sep[w]; m; m &= m - 1) {
      uint64_t p = w * 64 + ctz64a(m);
      ExtentOut x = arr_extent(in, len, sep.data(), p, first_opener);
      if (x.second_opener) doc_min = std::min(doc_min, p);
      if (!x.is_record) continue;
      if (n < cap) { s_out[n] = x.start; e_out[n] = x.end; blank_out[n] = (uint8_t)x.blank; }
      n++;
    }
  }
  *n_out = n;
  if (doc_min != ~0ull) { *doc_kind = PJ_E_SYNTAX; *doc_off = doc_min; }
  else if (first_opener == ~0ull || st.s || st.d != 0) { *doc_kind = PJ_E_EOF; *doc_off = len; }
  else { *doc_kind = 0; *doc_off = 0; }
  return 0;
}

/* ---- the line index of the stream kernel (pj_stream.cuh), tile by tile and "thread" by "thread" ---------------
 * `mis` bytes of junk are put before the input in a 16-byte aligned copy, as if the caller's buffer started `mis`
 * bytes into an aligned block. Writes the input offset of every record the tiles find, in order. */
#include "pj_stream.cuh"
extern "C" int emu_stream_index(const uint8_t* in, uint64_t len, uint64_t slack, int is_first, int is_last, uint32_t tile_bytes,
                                uint32_t mis, uint64_t* starts, uint64_t cap, uint64_t* n_out, uint64_t* overflow_tiles, uint64_t* long_lines) {
  const uint64_t limit = len + slack;
  std::vector<uint8_t> base(mis + limit + 64, 0xEE);
  if (limit) memcpy(base.data() + mis, in, limit);
  const uint8_t* ain = base.data() + mis; /* the "caller's pointer" */
  std::vector<uint8_t> win(ST_WIN_BYTES + ST_WIN_PAD);
  uint64_t ntiles = stream_tiles(mis, len, 1u, tile_bytes);
  uint64_t n = 0;
  *overflow_tiles = 0; *long_lines = 0;
  for (uint64_t tile = 0; tile < ntiles; ++tile) {
    const StreamGeom g = stream_geom(mis, len, limit, tile_bytes, (uint32_t)tile);
    std::fill(win.begin(), win.end(), 0xDD);
    if (g.copy_bytes) memcpy(win.data(), base.data() + g.v0, std::min<uint64_t>(g.copy_bytes, base.size() - g.v0));
    for (uint32_t k = 0; k < ST_WIN_PAD; ++k) win[g.hi_valid + k] = '\n';
    /* chunk masks, thread by thread */
    std::vector<uint16_t> lfb(ST_CHUNKS);
    std::vector<uint32_t> first_idx(ST_THREADS);
    uint32_t nlf = 0, nown = 0;
    const bool virtual_first = tile == 0 && is_first && limit > 0;
    for (uint32_t tid = 0; tid < ST_THREADS; ++tid) {
      first_idx[tid] = nlf;
      if (tid == 0 && virtual_first) { nlf++; nown++; }
      for (uint32_t k = 0; k < ST_CPT; ++k) {
        const uint32_t c = tid * ST_CPT + k;
        const uint32_t m = stream_chunk_mask(win.data(), c * 16u, g);
        lfb[c] = (uint16_t)m;
        nlf += __builtin_popcount(m); nown += __builtin_popcount(stream_own_bits(m, c * 16u, g));
      }
    }
    if (nown > ST_THREADS) ++*overflow_tiles;
    for (uint32_t b0 = 0; b0 < nown || b0 == 0; b0 += ST_THREADS) {
      std::vector<uint16_t> list(ST_LF_CAP, 0xFFFF);
      for (uint32_t tid = 0; tid < ST_THREADS; ++tid) {
        uint32_t idx = first_idx[tid];
        if (tid == 0 && virtual_first) { if (idx - b0 < ST_LF_CAP) list[idx - b0] = (uint16_t)mis; idx++; }
        for (uint32_t k = 0; k < ST_CPT; ++k) {
          const uint32_t c = tid * ST_CPT + k;
          for (uint32_t m = lfb[c]; m; m &= m - 1) {
            const uint32_t b = (uint32_t)__builtin_ctz(m);
            if (idx - b0 < ST_LF_CAP) list[idx - b0] = (uint16_t)(c * 16u + b + 1u);
            idx++;
          }
        }
      }
      for (uint32_t tid = 0; tid < ST_THREADS; ++tid) {
        const uint32_t j = b0 + tid;
        if (j >= nown) break;
        const uint32_t s = list[tid];
        const bool fits = (j + 1 < nlf) || g.to_limit;
        if (tid + 1 < ST_LF_CAP && j + 1 < nlf && list[tid + 1] == 0xFFFF) return -2; /* the next line must be in the list */
        if (stream_is_record(win.data(), s, g, ain, limit, is_last)) {
          if (!fits) ++*long_lines;
          if (n < cap) starts[n] = g.v0 + s - mis;
          ++n;
        }
      }
      if (nown == 0) break;
    }
  }
  *n_out = n;
  return 0;
}

/* ---- the mask algebra of the long-record path (pj_wide.cuh), lane after lane ---------------------------------------
 * What a warp does side by side is done here one 32-byte block after the other with the same formulas: backslash /
 * quote masks, escaped bytes with the carry from the block before, string interiors by prefix XOR with the running
 * parity. Per byte: quotes_out = it is an unescaped quote, instr_out = it lies in a string (from the opening quote up
 * to, not including, the closing one), special_out = control character or beyond ASCII. Returns 1 when a block
 * consists of backslashes only (the case the device code refuses). */
#include "pj_wide.cuh"
extern "C" int emu_wide_masks(const uint8_t* buf, uint64_t n, uint8_t* quotes_out, uint8_t* instr_out, uint8_t* special_out) {
  using namespace pj;
  uint32_t esc_c = 0, str_c = 0;
  for (uint64_t off = 0; off < n; off += 32) {
    uint8_t blk[32];
    for (uint32_t k = 0; k < 32; ++k) blk[k] = off + k < n ? buf[off + k] : 0;
    const uint32_t valid = wide_low_mask((int64_t)(n - off));
    uint32_t B, Q, C, X;
    wide_block_masks(blk, valid, &B, &Q, &C, &X);
    if (B == 0xFFFFFFFFu) return 1;
    const uint32_t cout = wide_carry_out(B);
    const uint32_t Qu = Q & ~wide_escaped(B, esc_c);
    const uint32_t instr = wide_prefix_xor(Qu) ^ (str_c ? 0xFFFFFFFFu : 0u);
    for (uint32_t k = 0; k < 32 && off + k < n; ++k) {
      quotes_out[off + k] = (Qu >> k) & 1u;
      instr_out[off + k] = (instr >> k) & 1u;
      special_out[off + k] = (X >> k) & 1u;
    }
    esc_c = cout;
    str_c ^= (uint32_t)__builtin_popcount(Qu) & 1u;
  }
  return 0;
}
