/*
 * pj_write_core.cuh — columns -> JSON text for one record, one record per thread (rules W1-W5 of
 * petjson.h). Template parameter WR: false = measure the record's length only, true = store bytes.
 */
#ifndef PJ_WRITE_CORE_CUH
#define PJ_WRITE_CORE_CUH

#include "pj_core.cuh"

namespace pj {

struct WOut {
  uint8_t* dst;
  uint32_t hexa = 'A'; /* first letter of the hex digits of \u00xx escapes: 'A', or 'a' with PJ_OPT_HEX_LOWER */
  uint64_t n;
};
template <bool WR>
PJ_HD void wput(WOut& w, uint32_t b) {
  if (WR) w.dst[w.n] = (uint8_t)b;
  w.n++;
}
template <bool WR>
PJ_HD void wput_packed(WOut& w, uint64_t lo, uint64_t hi, uint32_t len) {
  for (uint32_t i = 0; i < len; ++i) wput<WR>(w, (uint32_t)((i < 8 ? lo >> (8 * i) : hi >> (8 * (i - 8))) & 0xFF));
}
template <bool WR>
PJ_HD void wput_u64(WOut& w, uint64_t u) {
  uint32_t nd = 1;
  for (uint64_t t = u; t >= 10; t /= 10) nd++;
  if (WR) {
    uint64_t t = u;
    for (uint32_t i = nd; i-- > 0;) { w.dst[w.n + i] = (uint8_t)('0' + t % 10); t /= 10; }
  }
  w.n += nd;
}
template <bool WR>
PJ_HD void wput_i64(WOut& w, int64_t v) {
  if (v < 0) { wput<WR>(w, '-'); wput_u64<WR>(w, 0 - (uint64_t)v); }
  else wput_u64<WR>(w, (uint64_t)v);
}
template <bool WR>
PJ_HD void wput_2d(WOut& w, uint32_t v) { wput<WR>(w, '0' + v / 10); wput<WR>(w, '0' + v % 10); }

/* bytes the escapes of W3 add to the n bytes at s: 1 for the two-character escapes, 5 for \u00XX.
 * Reads aligned 4-byte words where it can and looks closer only at words that hold a byte to escape. */
PJ_HD uint32_t escape_extra_byte(uint32_t c) {
  if (c >= 0x20) return (c == '"' || c == '\\') ? 1u : 0u;
  return (c == 8 || c == 9 || c == 10 || c == 12 || c == 13) ? 1u : 5u;
}
PJ_HD uint32_t str_escape_extra(const uint8_t* s, uint32_t n) {
  uint32_t extra = 0, i = 0;
  while (i < n && ((uintptr_t)(s + i) & 3u)) extra += escape_extra_byte(ld_byte(s + i++));
  for (; i + 4 <= n; i += 4) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(s + i);
    const uint32_t xq = w ^ 0x22222222u, xb = w ^ 0x5C5C5C5Cu;
    const uint32_t m = ((w - 0x20202020u) & ~w) | ((xq - 0x01010101u) & ~xq) | ((xb - 0x01010101u) & ~xb);
    if (m & 0x80808080u)
      for (uint32_t k = 0; k < 4; ++k) extra += escape_extra_byte((w >> (8 * k)) & 0xFFu);
  }
  for (; i < n; ++i) extra += escape_extra_byte(ld_byte(s + i));
  return extra;
}

/* W3 */
template <bool WR>
PJ_HD void wput_str(WOut& w, const uint8_t* s, uint32_t n) {
  if (!WR) { w.n += 2 + (uint64_t)n + str_escape_extra(s, n); return; }
  wput<WR>(w, '"');
  for (uint32_t i = 0; i < n; ++i) {
    uint32_t c = ld_byte(s + i);
    if (c >= 0x20 && c != '"' && c != '\\') { wput<WR>(w, c); continue; }
    wput<WR>(w, '\\');
    switch (c) {
      case '"': wput<WR>(w, '"'); break;
      case '\\': wput<WR>(w, '\\'); break;
      case 8: wput<WR>(w, 'b'); break;
      case 9: wput<WR>(w, 't'); break;
      case 10: wput<WR>(w, 'n'); break;
      case 12: wput<WR>(w, 'f'); break;
      case 13: wput<WR>(w, 'r'); break;
      default:
        wput<WR>(w, 'u'); wput<WR>(w, '0'); wput<WR>(w, '0');
        wput<WR>(w, '0' + (c >> 4));
        wput<WR>(w, (c & 15) < 10 ? '0' + (c & 15) : w.hexa + (c & 15) - 10);
        break;
    }
  }
  wput<WR>(w, '"');
}

PJ_HD void civil_from_days(int64_t z, int64_t* y, uint32_t* m, uint32_t* d) {
  z += 719468;
  int64_t era = (z >= 0 ? z : z - 146096) / 146097;
  uint32_t doe = (uint32_t)(z - era * 146097);
  uint32_t yoe = (doe - doe / 1460 + doe / 36524 - doe / 146096) / 365;
  int64_t yy = (int64_t)yoe + era * 400;
  uint32_t doy = doe - (365 * yoe + yoe / 4 - yoe / 100);
  uint32_t mp = (5 * doy + 2) / 153;
  *d = doy - (153 * mp + 2) / 5 + 1;
  *m = mp < 10 ? mp + 3 : mp - 9;
  *y = yy + (*m <= 2);
}
/* W5 */
template <bool WR>
PJ_HD void wput_datetime(WOut& w, int64_t epoch, int32_t nanos, int32_t off) {
  int64_t local = epoch + off;
  int64_t days = (local >= 0 ? local : local - 86399) / 86400;
  uint32_t sod = (uint32_t)(local - days * 86400);
  int64_t y; uint32_t m, d;
  civil_from_days(days, &y, &m, &d);
  wput<WR>(w, '"');
  wput_2d<WR>(w, (uint32_t)(y / 100)); wput_2d<WR>(w, (uint32_t)(y % 100));
  wput<WR>(w, '-'); wput_2d<WR>(w, m); wput<WR>(w, '-'); wput_2d<WR>(w, d);
  wput<WR>(w, 'T'); wput_2d<WR>(w, sod / 3600); wput<WR>(w, ':'); wput_2d<WR>(w, sod % 3600 / 60);
  wput<WR>(w, ':'); wput_2d<WR>(w, sod % 60);
  if (nanos) {
    uint32_t u = (uint32_t)nanos, nd = 9;
    while (u % 10 == 0) { u /= 10; nd--; }
    wput<WR>(w, '.');
    uint32_t div = 1;
    for (uint32_t i = 1; i < nd; ++i) div *= 10;
    for (; div; div /= 10) wput<WR>(w, '0' + u / div % 10);
  }
  if (off == 0) wput<WR>(w, 'Z');
  else {
    uint32_t a = (uint32_t)(off < 0 ? -off : off);
    wput<WR>(w, off < 0 ? '-' : '+');
    wput_2d<WR>(w, a / 3600); wput<WR>(w, ':'); wput_2d<WR>(w, a % 3600 / 60);
  }
  wput<WR>(w, '"');
}

/* W4 */
PJ_HD bool included(int incl, bool present, bool empty) {
  if (incl == PJ_INCLUDE_ALWAYS) return true;
  if (!present) return false;
  return !(incl == PJ_INCLUDE_NON_EMPTY && empty);
}

/* LEVEL 0: model root (may hold an object or lists); LEVEL 1: Category / Tag (scalars only). */
template <bool WR, int LEVEL>
PJ_HD void write_object(const Schema& S, const DevCols* c, const ObjDesc& O, uint64_t row, int incl, WOut& w) {
  uint32_t present = colp<uint8_t>(c, O.present_col)[row];
  bool first = true;
  wput<WR>(w, '{');
  for (int i = 0; i < (int)O.nfields; ++i) {
    const FieldDesc& F = O.f[i];
    bool pr = (present >> i) & 1;
    bool empty = false;
    uint32_t a = 0, b = 0;
    if (F.kind == K_STR || F.kind == K_LIST_STR || F.kind == K_LIST_OBJ) {
      a = colp<uint32_t>(c, F.col)[row]; b = colp<uint32_t>(c, F.col)[row + 1];
      empty = a == b;
    }
    if (!included(incl, pr, empty)) continue;
    if (!first) wput<WR>(w, ',');
    first = false;
    wput<WR>(w, '"'); wput_packed<WR>(w, F.name_lo, F.name_hi, F.name_len); wput<WR>(w, '"'); wput<WR>(w, ':');
    if (!pr) { wput<WR>(w, 'n'); wput<WR>(w, 'u'); wput<WR>(w, 'l'); wput<WR>(w, 'l'); continue; }
    switch (F.kind) {
      case K_I64: wput_i64<WR>(w, colp<int64_t>(c, F.col)[row]); break;
      case K_I32: wput_i64<WR>(w, colp<int32_t>(c, F.col)[row]); break;
      case K_BOOL:
        if (colp<uint8_t>(c, F.col)[row]) wput_packed<WR>(w, 0x65757274ull, 0, 4); else wput_packed<WR>(w, 0x65736C6166ull, 0, 5);
        break;
      case K_ENUM: {
        const EnumDesc& E = S.en[F.child];
        uint32_t e = colp<uint8_t>(c, F.col)[row] % E.n;
        wput<WR>(w, '"'); wput_packed<WR>(w, E.lo[e], E.hi[e], E.len[e]); wput<WR>(w, '"');
        break;
      }
      case K_DATETIME:
        wput_datetime<WR>(w, colp<int64_t>(c, F.col)[row], colp<int32_t>(c, F.col + 1)[row], colp<int32_t>(c, F.col + 2)[row]);
        break;
      case K_STR: wput_str<WR>(w, colp<uint8_t>(c, F.col + 1) + a, b - a); break;
      case K_OBJ:
        if (LEVEL == 0) write_object<WR, 1>(S, c, S.obj[F.child], row, incl, w);
        break;
      case K_LIST_STR: {
        const uint32_t* so = colp<uint32_t>(c, F.col + 1);
        const uint8_t* data = colp<uint8_t>(c, F.col + 2);
        wput<WR>(w, '[');
        for (uint32_t k = a; k < b; ++k) { if (k > a) wput<WR>(w, ','); uint32_t s0 = so[k], s1 = so[k + 1]; wput_str<WR>(w, data + s0, s1 - s0); }
        wput<WR>(w, ']');
        break;
      }
      case K_LIST_OBJ:
        wput<WR>(w, '[');
        if (LEVEL == 0) for (uint32_t k = a; k < b; ++k) { if (k > a) wput<WR>(w, ','); write_object<WR, 1>(S, c, S.obj[F.child], k, incl, w); }
        wput<WR>(w, ']');
        break;
      default: break;
    }
  }
  wput<WR>(w, '}');
}

/* Which model table and row record i of the column set refers to; false when it has none. */
PJ_HD bool write_locate(uint32_t schema, const DevCols* c, uint64_t i, uint32_t* type, uint64_t* row) {
  if (schema != PJ_SCHEMA_MIXED) { *type = schema; *row = i; return true; }
  *type = colp<uint8_t>(c, PJ_COL_REC_TYPE)[i];
  *row = colp<uint32_t>(c, PJ_COL_REC_ROW)[i];
  return *type != PJ_TYPE_NONE;
}

template <bool WR>
PJ_HD void write_record(const Schema& S, const DevCols* c, uint32_t type, uint64_t row, int incl, WOut& w) {
  const ObjDesc& O = type == PJ_TYPE_PET ? S.obj[OBJ_PET] : (type == PJ_TYPE_ORDER ? S.obj[OBJ_ORDER] : S.obj[OBJ_USER]);
  write_object<WR, 0>(S, c, O, row, incl, w);
}

}  // namespace pj
#endif
