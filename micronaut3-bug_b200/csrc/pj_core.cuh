/*
 * pj_core.cuh — per-record JSON tokeniser / validator / column emitter, one record per thread.
 *
 * The same code runs in two modes (template parameter W):
 *   W = false  "size" pass : validates the record, determines its model, and counts what it will
 *                            emit into every variable-size output (string bytes, list items);
 *   W = true   "emit" pass : re-reads an accepted record and stores values, offsets and decoded
 *                            string bytes at the positions the scanned counters assign to it.
 * The grammar and failure rules implemented here are the ones listed as R1-R12 in petjson.h.
 *
 * Reading is abstracted by Rd (byte source + limit). A byte beyond the limit reads as 0, which no
 * grammar position accepts, so every loop stops there without a separate bounds branch; the failure
 * path then tells "ran out of input" from "wrong byte".
 */
#ifndef PJ_CORE_CUH
#define PJ_CORE_CUH

#include <stdint.h>

#include "pj_schema.h"

#if defined(__CUDACC__)
#define PJ_HD __host__ __device__ __forceinline__
#define PJ_HD_NOINLINE inline __host__ __device__ __noinline__
#else
#define PJ_HD inline
#define PJ_HD_NOINLINE
#endif

/* PJ_COLD: functions of the fall-back paths (the word-at-a-time tokeniser and its emitter, the exact parser). With
 * -DPJ_COLD_OUTLINE they are compiled once and called instead of being expanded at every place that can reach them:
 * the kernels' machine code shrinks several times over. Off by default until it has been measured on the GPU. */
#if defined(PJ_COLD_OUTLINE)
#define PJ_COLD PJ_HD_NOINLINE
#else
#define PJ_COLD PJ_HD
#endif

namespace pj {

struct Rd {
  const uint8_t* in;
  uint64_t limit;    /* first unreadable offset */
  uint32_t lf_ws;    /* array framing: LF is whitespace; otherwise LF ends the record */
  uint32_t open_end; /* the stream continues past `limit` (a shard's slack ran out) */
  uint32_t opts;     /* PJ_OPT_* bits that change a rule (enum, surrogate, coercion) */
  uint64_t rec_end;  /* read by list hooks only: offset of the byte that ends the record (its LF, or `limit`) */
};

struct PS {
  uint64_t p;
  uint64_t err_pos;
  uint32_t err;
};

/* generic load: the byte source may be global memory or a window staged in shared memory */
PJ_HD uint32_t ld_byte(const uint8_t* a) { return *a; }
PJ_HD uint32_t rd_get(const Rd& r, uint64_t p) { return p < r.limit ? ld_byte(r.in + p) : 0u; }

PJ_HD bool fail(PS& s, uint32_t kind, uint64_t pos) {
  if (!s.err) { s.err = kind; s.err_pos = pos; }
  return false;
}
/* A failure caused by the byte at q: if the record's bytes end at q that is reported instead. */
PJ_HD bool fail_byte(const Rd& r, PS& s, uint64_t q, uint32_t kind, uint64_t pos) {
  if (q >= r.limit) return fail(s, r.open_end ? PJ_E_TOO_LONG : PJ_E_EOF, r.limit);
  if (!r.lf_ws && ld_byte(r.in + q) == '\n') return fail(s, PJ_E_EOF, q);
  return fail(s, kind, pos);
}
PJ_HD bool is_value_start(uint32_t x) {
  return x == '"' || x == '-' || (x - '0') <= 9u || x == '{' || x == '[' || x == 't' || x == 'f' || x == 'n';
}
/* R5: the byte at p cannot start a value of the expected type */
PJ_HD bool fail_first(const Rd& r, PS& s, uint32_t x) {
  return fail_byte(r, s, s.p, is_value_start(x) ? PJ_E_TYPE : PJ_E_SYNTAX, s.p);
}
PJ_HD void skip_ws(const Rd& r, PS& s) {
  /* on locals: the position is written back once, and nothing is read again through `r` after a store */
  const uint8_t* const in = r.in;
  const uint64_t limit = r.limit;
  const bool lf = r.lf_ws != 0;
  uint64_t p = s.p;
  for (;;) {
    const uint32_t x = p < limit ? ld_byte(in + p) : 0u;
    if (x == ' ' || x == '\t' || x == '\r' || (lf && x == '\n')) p++;
    else break;
  }
  s.p = p;
}

/* ---- string sink ----------------------------------------------------------------------------- */
enum { SINK_COUNT = 0, SINK_WRITE = 1, SINK_PACK = 2 };
struct Sink {
  uint32_t mode, n, room;
  uint8_t* dst;
  uint64_t w[5]; /* SINK_PACK: first 40 decoded bytes, little-endian */
};
PJ_HD void sink_init(Sink& k, uint32_t mode) { k.mode = mode; k.n = 0; k.room = 0; k.dst = nullptr; k.w[0] = k.w[1] = k.w[2] = k.w[3] = k.w[4] = 0; }
PJ_HD void sink_put(Sink& k, uint32_t b) {
  if (k.mode == SINK_WRITE) { if (k.n < k.room) k.dst[k.n] = (uint8_t)b; }
  else if (k.mode == SINK_PACK) { if (k.n < 40) k.w[k.n >> 3] |= (uint64_t)b << ((k.n & 7) * 8); }
  k.n++;
}
PJ_HD uint32_t sink_byte(const Sink& k, uint32_t i) { return (uint32_t)(k.w[i >> 3] >> ((i & 7) * 8)) & 0xFFu; }
PJ_HD void sink_put_cp(Sink& k, uint32_t cp) {
  if (cp < 0x80) sink_put(k, cp);
  else if (cp < 0x800) { sink_put(k, 0xC0 | (cp >> 6)); sink_put(k, 0x80 | (cp & 63)); }
  else if (cp < 0x10000) { sink_put(k, 0xE0 | (cp >> 12)); sink_put(k, 0x80 | ((cp >> 6) & 63)); sink_put(k, 0x80 | (cp & 63)); }
  else { sink_put(k, 0xF0 | (cp >> 18)); sink_put(k, 0x80 | ((cp >> 12) & 63)); sink_put(k, 0x80 | ((cp >> 6) & 63)); sink_put(k, 0x80 | (cp & 63)); }
}

PJ_HD int hexval(uint32_t x) {
  if (x - '0' <= 9u) return (int)(x - '0');
  uint32_t l = x | 0x20;
  if (l - 'a' <= 5u) return (int)(l - 'a' + 10);
  return -1;
}
/* four hex digits at q..q+3 */
PJ_HD bool hex4(const Rd& r, PS& s, uint64_t q, uint32_t* out) {
  uint32_t v = 0;
  for (uint32_t i = 0; i < 4; ++i) {
    int h = hexval(rd_get(r, q + i));
    if (h < 0) return fail_byte(r, s, q + i, PJ_E_BAD_ESCAPE, q + i);
    v = v << 4 | (uint32_t)h;
  }
  *out = v;
  return true;
}

/* R7. s.p is at the opening quote; on success s.p is after the closing quote. */
PJ_HD bool lex_string_body(const Rd& r, PS& s, Sink& k) {
  uint64_t p = s.p + 1;
  for (;;) {
    uint32_t x = rd_get(r, p);
    if (x == '"') { s.p = p + 1; return true; }
    if (x < 0x20) return fail_byte(r, s, p, PJ_E_CTRL_CHAR, p);
    if (x == '\\') {
      uint32_t y = rd_get(r, p + 1), cp;
      switch (y) {
        case '"': cp = '"'; break;
        case '\\': cp = '\\'; break;
        case '/': cp = '/'; break;
        case 'b': cp = 8; break;
        case 'f': cp = 12; break;
        case 'n': cp = 10; break;
        case 'r': cp = 13; break;
        case 't': cp = 9; break;
        case 'u': {
          if (!hex4(r, s, p + 2, &cp)) return false;
          if (r.opts & PJ_OPT_LONE_SURROGATE_REPLACE) {
            /* a high surrogate takes the low one that follows it at once; whatever is left alone becomes U+FFFD */
            if (cp - 0xD800u < 0x400u && rd_get(r, p + 6) == '\\' && rd_get(r, p + 7) == 'u') {
              uint32_t lo;
              if (!hex4(r, s, p + 8, &lo)) return false;
              if (lo - 0xDC00u < 0x400u) { cp = 0x10000u + ((cp - 0xD800u) << 10) + (lo - 0xDC00u); p += 6; }
            }
            if (cp - 0xD800u < 0x800u) cp = 0xFFFDu;
            p += 4;
            break;
          }
          if (cp - 0xDC00u < 0x400u) return fail(s, PJ_E_BAD_SURROGATE, p);
          if (cp - 0xD800u < 0x400u) {
            if (rd_get(r, p + 6) != '\\') return fail_byte(r, s, p + 6, PJ_E_BAD_SURROGATE, p);
            if (rd_get(r, p + 7) != 'u') return fail_byte(r, s, p + 7, PJ_E_BAD_SURROGATE, p);
            uint32_t lo;
            if (!hex4(r, s, p + 8, &lo)) return false;
            if (lo - 0xDC00u >= 0x400u) return fail(s, PJ_E_BAD_SURROGATE, p);
            cp = 0x10000u + ((cp - 0xD800u) << 10) + (lo - 0xDC00u);
            p += 6;
          }
          p += 4;
          break;
        }
        default: return fail_byte(r, s, p + 1, PJ_E_BAD_ESCAPE, p + 1);
      }
      p += 2;
      sink_put_cp(k, cp);
      continue;
    }
    if (x < 0x80) { sink_put(k, x); p++; continue; }
    /* RFC 3629 */
    uint32_t need, lo = 0x80, hi = 0xBF;
    if (x - 0xC2u <= 0x1Du) need = 1;
    else if (x == 0xE0) { need = 2; lo = 0xA0; }
    else if (x == 0xED) { need = 2; hi = 0x9F; }
    else if (x - 0xE1u <= 0x0Eu) need = 2;
    else if (x == 0xF0) { need = 3; lo = 0x90; }
    else if (x - 0xF1u <= 2u) need = 3;
    else if (x == 0xF4) { need = 3; hi = 0x8F; }
    else return fail(s, PJ_E_UTF8, p);
    uint32_t y1 = rd_get(r, p + 1);
    if (y1 < lo || y1 > hi) return fail_byte(r, s, p + 1, PJ_E_UTF8, p);
    uint32_t y2 = 0, y3 = 0;
    if (need >= 2) { y2 = rd_get(r, p + 2); if (y2 - 0x80u > 0x3Fu) return fail_byte(r, s, p + 2, PJ_E_UTF8, p); }
    if (need >= 3) { y3 = rd_get(r, p + 3); if (y3 - 0x80u > 0x3Fu) return fail_byte(r, s, p + 3, PJ_E_UTF8, p); }
    sink_put(k, x); sink_put(k, y1);
    if (need >= 2) sink_put(k, y2);
    if (need >= 3) sink_put(k, y3);
    p += need + 1;
  }
}

PJ_HD_NOINLINE bool lex_string(const Rd& r0, PS& s, Sink& k0) {
  /* copies that the byte stores of the sink cannot alias: reader and sink stay in registers while the string is read */
  const Rd r = r0;
  Sink k = k0;
  const bool ok = lex_string_body(r, s, k);
  k0 = k;
  return ok;
}

/* R6. s.p at '-' or a digit. */
struct Num { uint64_t mag, start; uint32_t neg, is_int, overflow; };
PJ_HD_NOINLINE bool lex_number(const Rd& r0, PS& s, Num& n) {
  const Rd r = r0;
  uint64_t p = s.p;
  n.start = p; n.neg = 0; n.is_int = 1; n.overflow = 0; n.mag = 0;
  uint32_t x = rd_get(r, p);
  if (x == '-') { n.neg = 1; x = rd_get(r, ++p); }
  if (x - '0' > 9u) return fail_byte(r, s, p, PJ_E_SYNTAX, p);
  if (x == '0') {
    x = rd_get(r, ++p);
    if (x - '0' <= 9u) return fail(s, PJ_E_SYNTAX, p);
  } else {
    uint32_t nd = 0;
    do {
      uint64_t d = x - '0';
      if (nd >= 19) { if (n.mag > (0xFFFFFFFFFFFFFFFFull - d) / 10) n.overflow = 1; else n.mag = n.mag * 10 + d; }
      else n.mag = n.mag * 10 + d;
      nd++;
      x = rd_get(r, ++p);
    } while (x - '0' <= 9u);
  }
  if (x == '.') {
    n.is_int = 0;
    x = rd_get(r, ++p);
    if (x - '0' > 9u) return fail_byte(r, s, p, PJ_E_SYNTAX, p);
    do { x = rd_get(r, ++p); } while (x - '0' <= 9u);
  }
  if ((x | 0x20) == 'e') {
    n.is_int = 0;
    x = rd_get(r, ++p);
    if (x == '+' || x == '-') x = rd_get(r, ++p);
    if (x - '0' > 9u) return fail_byte(r, s, p, PJ_E_SYNTAX, p);
    do { x = rd_get(r, ++p); } while (x - '0' <= 9u);
  }
  s.p = p;
  return true;
}
/* the rest of a literal whose first byte (at s.p) has been recognised: word holds bytes 1.. */
PJ_HD bool lex_literal(const Rd& r, PS& s, uint32_t word, uint32_t n) {
  for (uint32_t i = 1; i <= n; ++i) {
    if (rd_get(r, s.p + i) != ((word >> (8 * (i - 1))) & 0xFFu)) return fail_byte(r, s, s.p + i, PJ_E_SYNTAX, s.p + i);
  }
  s.p += n + 1;
  return true;
}
#define PJ_LIT_RUE 0x657572u   /* "rue"  */
#define PJ_LIT_ALSE 0x65736C61u /* "alse" */
#define PJ_LIT_ULL 0x6C6C75u   /* "ull"  */

/* R4: any JSON value at s.p (whitespace already skipped), validated and discarded. */
PJ_HD_NOINLINE bool skip_value(const Rd& r, PS& s) {
  uint64_t stack = 0; /* bit d: 1 = object, 0 = array */
  uint32_t depth = 0;
  Sink nul;
  for (;;) {
    /* a value starts at s.p */
    uint32_t x = rd_get(r, s.p);
    bool need_key = false;
    if (x == '"') { sink_init(nul, SINK_COUNT); if (!lex_string(r, s, nul)) return false; }
    else if (x == '-' || x - '0' <= 9u) { Num n; if (!lex_number(r, s, n)) return false; }
    else if (x == 't') { if (!lex_literal(r, s, PJ_LIT_RUE, 3)) return false; }
    else if (x == 'f') { if (!lex_literal(r, s, PJ_LIT_ALSE, 4)) return false; }
    else if (x == 'n') { if (!lex_literal(r, s, PJ_LIT_ULL, 3)) return false; }
    else if (x == '[' || x == '{') {
      if (depth >= 64) return fail(s, PJ_E_DEPTH, s.p);
      uint64_t bit = 1ull << depth;
      if (x == '{') stack |= bit; else stack &= ~bit;
      depth++;
      s.p++;
      skip_ws(r, s);
      uint32_t y = rd_get(r, s.p);
      if (y == (x == '[' ? (uint32_t)']' : (uint32_t)'}')) { s.p++; depth--; }
      else if (x == '[') continue;
      else need_key = true;
    } else return fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p);
    /* after a complete value (or before the first key of an object) */
    for (;;) {
      if (!need_key) {
        if (depth == 0) return true;
        skip_ws(r, s);
        uint32_t y = rd_get(r, s.p);
        bool in_obj = (stack >> (depth - 1)) & 1;
        if (y == ',') { s.p++; skip_ws(r, s); if (in_obj) need_key = true; else break; }
        else if (y == (in_obj ? (uint32_t)'}' : (uint32_t)']')) { s.p++; depth--; continue; }
        else return fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p);
      }
      if (need_key) {
        if (rd_get(r, s.p) != '"') return fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p);
        sink_init(nul, SINK_COUNT);
        if (!lex_string(r, s, nul)) return false;
        skip_ws(r, s);
        if (rd_get(r, s.p) != ':') return fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p);
        s.p++;
        skip_ws(r, s);
        break;
      }
    }
  }
}

/* ---- dates ---------------------------------------------------------------------------------- */
PJ_HD int64_t days_from_civil(int64_t y, uint32_t m, uint32_t d) {
  y -= m <= 2;
  int64_t era = (y >= 0 ? y : y - 399) / 400;
  uint32_t yoe = (uint32_t)(y - era * 400);
  uint32_t doy = (153 * (m + (m > 2 ? -3 : 9)) + 2) / 5 + d - 1;
  uint32_t doe = yoe * 365 + yoe / 4 - yoe / 100 + doy;
  return era * 146097 + (int64_t)doe - 719468;
}
/* R9 on the decoded text held by a SINK_PACK sink */
PJ_HD_NOINLINE bool parse_datetime(const Sink& k, int64_t* epoch, int32_t* nanos, int32_t* off) {
  uint32_t n = k.n;
  if (n < 20 || n > 35) return false;
  uint32_t t[35];
  for (uint32_t i = 0; i < 35; ++i) t[i] = i < n ? sink_byte(k, i) : 0;
  for (uint32_t i = 0; i < 19; ++i) {
    uint32_t want_digit = 1, c = 0;
    if (i == 4 || i == 7) { want_digit = 0; c = '-'; }
    else if (i == 10) { want_digit = 0; c = 'T'; }
    else if (i == 13 || i == 16) { want_digit = 0; c = ':'; }
    if (want_digit ? (t[i] - '0' > 9u) : (t[i] != c)) return false;
  }
#define PJ_D2(a) ((t[a] - '0') * 10 + (t[(a) + 1] - '0'))
  uint32_t year = PJ_D2(0) * 100 + PJ_D2(2), mon = PJ_D2(5), day = PJ_D2(8), hh = PJ_D2(11), mi = PJ_D2(14), ss = PJ_D2(17);
  if (mon < 1 || mon > 12 || day < 1) return false;
  uint32_t dim = (mon == 2) ? 28u : ((mon == 4 || mon == 6 || mon == 9 || mon == 11) ? 30u : 31u);
  if (mon == 2 && (year % 4 == 0 && (year % 100 != 0 || year % 400 == 0))) dim = 29;
  if (day > dim || hh > 23 || mi > 59 || ss > 59) return false;
  uint32_t i = 19, ns = 0;
  if (t[i] == '.') {
    uint32_t kd = 0;
    ++i;
    while (i < n && t[i] - '0' <= 9u) { if (kd >= 9) return false; ns = ns * 10 + (t[i] - '0'); ++kd; ++i; }
    if (kd == 0) return false;
    for (; kd < 9; ++kd) ns *= 10;
  }
  if (i >= n) return false;
  int32_t o = 0;
  if (t[i] == 'Z') { if (i + 1 != n) return false; }
  else if (t[i] == '+' || t[i] == '-') {
    if (i + 6 != n) return false;
    if (t[i + 1] - '0' > 9u || t[i + 2] - '0' > 9u || t[i + 3] != ':' || t[i + 4] - '0' > 9u || t[i + 5] - '0' > 9u) return false;
    uint32_t oh = PJ_D2(i + 1), om = PJ_D2(i + 4);
    if (oh > 23 || om > 59) return false;
    o = (int32_t)(oh * 3600 + om * 60);
    if (t[i] == '-') o = -o;
  } else return false;
#undef PJ_D2
  *epoch = days_from_civil((int64_t)year, mon, day) * 86400 + (int64_t)hh * 3600 + (int64_t)(mi * 60 + ss) - o;
  *nanos = (int32_t)ns; *off = o;
  return true;
}

/* ---- per-record output context --------------------------------------------------------------- */
template <bool W>
struct Out {
  uint32_t cnt[NSLOT];  /* running count per slot (both passes) */
  uint32_t base[NSLOT]; /* emit pass: scanned start of this record in every slot */
  uint32_t room[NSLOT]; /* emit pass: final size of this record in every slot (stores are clamped to it) */
  const DevCols* cols;
};
template <class T>
PJ_HD T* colp(const DevCols* c, uint32_t col) { return (T*)c->ptr[col]; }

struct ObjVals {
  int64_t v[8];
  int64_t aux; /* DATETIME: nanos << 32 | (uint32) offset */
  uint32_t present;
};
PJ_HD void vals_reset(ObjVals& o) { for (int i = 0; i < 8; ++i) o.v[i] = 0; o.aux = 0; o.present = 0; }

PJ_HD int find_field(const ObjDesc& O, uint32_t len, uint64_t lo, uint64_t hi) {
  for (int i = 0; i < (int)O.nfields; ++i)
    if (O.f[i].name_len == len && O.f[i].name_lo == lo && O.f[i].name_hi == hi) return i;
  return -1;
}
PJ_HD int find_enum(const EnumDesc& E, uint32_t len, uint64_t lo, uint64_t hi) {
  for (int i = 0; i < (int)E.n; ++i)
    if (E.len[i] == len && E.lo[i] == lo && E.hi[i] == hi) return i;
  return -1;
}
/* exact comparison of a decoded key / literal: the packed words cover 16 bytes, longer never match */
PJ_HD bool sink_small(const Sink& k) { return k.n <= 16 && k.w[2] == 0; }

/* Stores the fixed-width values and string / list offsets of one object at `row`. */
template <bool W>
PJ_HD void store_object(const ObjDesc& O, const ObjVals& v, uint64_t row, const Out<W>& o, const uint32_t* str_start) {
  if (!W) return;
  *(colp<uint8_t>(o.cols, O.present_col) + row) = (uint8_t)v.present;
  for (int i = 0; i < (int)O.nfields; ++i) {
    const FieldDesc& F = O.f[i];
    bool pr = (v.present >> i) & 1;
    switch (F.kind) {
      case K_I64: colp<int64_t>(o.cols, F.col)[row] = pr ? v.v[i] : 0; break;
      case K_I32: colp<int32_t>(o.cols, F.col)[row] = pr ? (int32_t)v.v[i] : 0; break;
      case K_BOOL: colp<uint8_t>(o.cols, F.col)[row] = pr ? (uint8_t)v.v[i] : 0; break;
      case K_ENUM: colp<uint8_t>(o.cols, F.col)[row] = pr ? (uint8_t)v.v[i] : 255; break;
      case K_DATETIME:
        colp<int64_t>(o.cols, F.col)[row] = pr ? v.v[i] : 0;
        colp<int32_t>(o.cols, F.col + 1)[row] = pr ? (int32_t)(v.aux >> 32) : 0;
        colp<int32_t>(o.cols, F.col + 2)[row] = pr ? (int32_t)(uint32_t)v.aux : 0;
        break;
      case K_STR: colp<uint32_t>(o.cols, F.col)[row] = o.base[F.cnt] + str_start[i]; break;
      case K_LIST_STR:
      case K_LIST_OBJ: colp<uint32_t>(o.cols, F.col)[row] = o.base[F.cnt]; break;
      default: break;
    }
  }
}

/* PJ_OPT_COERCE_SCALARS: the integer held by a decoded string (k: SINK_PACK). 0 = ok, else the failure kind. */
PJ_HD uint32_t sink_to_int(const Sink& k, bool is64, int64_t* out) {
  if (k.n == 0 || k.n > 20) return PJ_E_TYPE;
  uint32_t i = 0;
  const bool neg = sink_byte(k, 0) == '-';
  if (neg) i = 1;
  if (i >= k.n) return PJ_E_TYPE;
  if (sink_byte(k, i) == '0' && i + 1 < k.n) return PJ_E_TYPE;
  uint64_t mag = 0;
  bool over = false;
  for (; i < k.n; ++i) {
    const uint32_t d = sink_byte(k, i) - '0';
    if (d > 9u) return PJ_E_TYPE;
    if (mag > (0xFFFFFFFFFFFFFFFFull - d) / 10) over = true; else mag = mag * 10 + d;
  }
  const uint64_t lim = is64 ? (neg ? 0x8000000000000000ull : 0x7FFFFFFFFFFFFFFFull) : (neg ? 0x80000000ull : 0x7FFFFFFFull);
  if (over || mag > lim) return PJ_E_NUM_RANGE;
  *out = neg ? (int64_t)(0 - mag) : (int64_t)mag;
  return 0;
}

/* R5 / R6 for an integer property: x is the byte at s.p (not 'n'). */
PJ_HD bool read_int(const Rd& r, PS& s, uint32_t x, bool is64, int64_t* out) {
  if (x == '"' && (r.opts & PJ_OPT_COERCE_SCALARS)) {
    const uint64_t q = s.p;
    Sink k;
    sink_init(k, SINK_PACK);
    if (!lex_string(r, s, k)) return false;
    const uint32_t e = sink_to_int(k, is64, out);
    return e ? fail(s, e, q) : true;
  }
  if (!(x == '-' || x - '0' <= 9u)) return fail_first(r, s, x);
  Num n;
  if (!lex_number(r, s, n)) return false;
  if (!n.is_int) return fail(s, PJ_E_TYPE, n.start);
  uint64_t lim = is64 ? (n.neg ? 0x8000000000000000ull : 0x7FFFFFFFFFFFFFFFull)
                      : (n.neg ? 0x80000000ull : 0x7FFFFFFFull);
  if (n.overflow || n.mag > lim) return fail(s, PJ_E_NUM_RANGE, n.start);
  *out = n.neg ? (int64_t)(0 - n.mag) : (int64_t)n.mag;
  return true;
}

/* Reads the value of a scalar property (kinds I64 .. DATETIME) at s.p into v.v[i]; sets / clears the
 * presence bit. `start` is the string cursor at which this object's string for that slot begins. */
template <bool W>
PJ_HD bool read_scalar(const Schema& S, const Rd& r, PS& s, const FieldDesc& F, int i, ObjVals& v,
                       Out<W>& o, uint32_t start, bool live) {
  uint32_t x = rd_get(r, s.p);
  uint32_t bit = 1u << i;
  if (x == 'n') {
    if (!lex_literal(r, s, PJ_LIT_ULL, 3)) return false;
    v.present &= ~bit; v.v[i] = 0;
    if (F.kind == K_STR) o.cnt[F.cnt] = start;
    return true;
  }
  switch (F.kind) {
    case K_I64:
    case K_I32: {
      int64_t val;
      if (!read_int(r, s, x, F.kind == K_I64, &val)) return false;
      v.v[i] = val;
      v.present |= bit;
      return true;
    }
    case K_BOOL: {
      if (x == 't') { if (!lex_literal(r, s, PJ_LIT_RUE, 3)) return false; v.v[i] = 1; }
      else if (x == 'f') { if (!lex_literal(r, s, PJ_LIT_ALSE, 4)) return false; v.v[i] = 0; }
      else if (x == '"' && (r.opts & PJ_OPT_COERCE_SCALARS)) {
        const uint64_t q = s.p;
        Sink k;
        sink_init(k, SINK_PACK);
        if (!lex_string(r, s, k)) return false;
        if (k.n == 4 && k.w[0] == 0x65757274ull) v.v[i] = 1;
        else if (k.n == 5 && k.w[0] == 0x65736C6166ull) v.v[i] = 0;
        else return fail(s, PJ_E_TYPE, q);
      }
      else return fail_first(r, s, x);
      v.present |= bit;
      return true;
    }
    case K_STR: {
      const bool coerce = (r.opts & PJ_OPT_COERCE_SCALARS) && (x == '-' || x - '0' <= 9u || x == 't' || x == 'f');
      if (x != '"' && !coerce) return fail_first(r, s, x);
      Sink k;
      sink_init(k, (W && live) ? SINK_WRITE : SINK_COUNT);
      if (W && live) {
        uint32_t rm = o.room[F.cnt];
        k.room = rm > start ? rm - start : 0;
        k.dst = colp<uint8_t>(o.cols, F.col + 1) + o.base[F.cnt] + start;
      }
      if (coerce) { /* the token's text, as written, becomes the string */
        const uint64_t t0 = s.p;
        if (x == 't') { if (!lex_literal(r, s, PJ_LIT_RUE, 3)) return false; }
        else if (x == 'f') { if (!lex_literal(r, s, PJ_LIT_ALSE, 4)) return false; }
        else { Num n; if (!lex_number(r, s, n)) return false; }
        for (uint64_t q = t0; q < s.p; ++q) sink_put(k, rd_get(r, q));
      } else
      if (!lex_string(r, s, k)) return false;
      o.cnt[F.cnt] = start + k.n;
      v.present |= bit;
      return true;
    }
    case K_ENUM: {
      if (x != '"') return fail_first(r, s, x);
      uint64_t q = s.p;
      Sink k;
      sink_init(k, SINK_PACK);
      if (!lex_string(r, s, k)) return false;
      int e = sink_small(k) ? find_enum(S.en[F.child], k.n, k.w[0], k.w[1]) : -1;
      if (e < 0) {
        if (!(r.opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL)) return fail(s, PJ_E_ENUM, q);
        v.present &= ~bit; v.v[i] = 0; /* unknown literal: the property stays absent */
        return true;
      }
      v.v[i] = e; v.present |= bit;
      return true;
    }
    default: { /* K_DATETIME */
      if (x != '"') return fail_first(r, s, x);
      uint64_t q = s.p;
      Sink k;
      sink_init(k, SINK_PACK);
      if (!lex_string(r, s, k)) return false;
      int64_t ep; int32_t ns, of;
      if (!parse_datetime(k, &ep, &ns, &of)) return fail(s, PJ_E_DATETIME, q);
      v.v[i] = ep; v.aux = (int64_t)(((uint64_t)(uint32_t)ns << 32) | (uint32_t)of);
      v.present |= bit;
      return true;
    }
  }
}

/* Member loop step shared by all objects: after '{' (first = true) or after a value.
 * Returns 1 with the key packed in k and s.p at the value, 2 when the object closed
 * (*close_pos = offset of '}'), 0 on failure. */
PJ_HD int next_member(const Rd& r, PS& s, bool& first, Sink& k, uint64_t* close_pos) {
  skip_ws(r, s);
  uint32_t x = rd_get(r, s.p);
  if (x == '}') { *close_pos = s.p; s.p++; return 2; }
  if (first) first = false;
  else {
    if (x != ',') { fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p); return 0; }
    s.p++;
    skip_ws(r, s);
    x = rd_get(r, s.p);
  }
  if (x != '"') { fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p); return 0; }
  sink_init(k, SINK_PACK);
  if (!lex_string(r, s, k)) return 0;
  skip_ws(r, s);
  if (rd_get(r, s.p) != ':') { fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p); return 0; }
  s.p++;
  skip_ws(r, s);
  return 1;
}

/* A flat object (Category, Tag): s.p at '{'. `elem` tells that it is a list element, whose strings
 * continue the record's running cursors; otherwise its strings start at cursor 0. */
template <bool W>
PJ_HD_NOINLINE bool parse_flat(const Schema& S, const Rd& r, PS& s, const ObjDesc& O, ObjVals& v, Out<W>& o,
                               bool elem, bool live, uint32_t* str_start) {
  vals_reset(v);
  for (int i = 0; i < (int)O.nfields; ++i) {
    str_start[i] = 0;
    if (O.f[i].kind == K_STR) {
      if (elem) str_start[i] = o.cnt[O.f[i].cnt]; else o.cnt[O.f[i].cnt] = 0;
    }
  }
  s.p++;
  bool first = true;
  Sink k;
  uint64_t close_pos;
  for (;;) {
    int m = next_member(r, s, first, k, &close_pos);
    if (m == 0) return false;
    if (m == 2) return true;
    int i = sink_small(k) ? find_field(O, k.n, k.w[0], k.w[1]) : -1;
    if (i < 0) { if (!skip_value(r, s)) return false; continue; }
    if (!read_scalar<W>(S, r, s, O.f[i], i, v, o, str_start[i], live)) return false;
  }
}

/* One record. s.p at the start of the extent. On success returns the model (PJ_TYPE_*), leaves the
 * counts in o.cnt and, in the emit pass, has stored every column at `row_of(type)`.
 * `schema` is PJ_SCHEMA_*; row_* give the model-table row per type for the emit pass. */
/* What parse_record<>() asks before it walks a non-empty list element by element: a hook may take the whole list
 * (s.p at its first element; on return 1, s.p is behind the `]` and the list's counters in o.cnt are final) or
 * return 0 and leave everything untouched. */
struct NoListHook {
  static constexpr bool enabled = false;
  template <bool W>
  static PJ_HD int list(const Schema&, const Rd&, PS&, const FieldDesc&, Out<W>&) { return 0; }
};

template <bool W, class LH = NoListHook>
PJ_COLD uint32_t parse_record(const Schema& S, const Rd& r, PS& s, uint32_t schema, Out<W>& o, uint64_t rec_index) {
  for (uint32_t i = 0; i < NSLOT; ++i) o.cnt[i] = 0;
  uint32_t type = schema == PJ_SCHEMA_MIXED ? PJ_TYPE_NONE : schema;
  const ObjDesc* O = type == PJ_TYPE_PET ? &S.obj[OBJ_PET] : (type == PJ_TYPE_ORDER ? &S.obj[OBJ_ORDER] : &S.obj[OBJ_USER]);
  ObjVals v, cv, ev; /* root, child object (Category), list element */
  uint32_t zero_start[8] = {0, 0, 0, 0, 0, 0, 0, 0}, cstart[8], estart[8];
  vals_reset(v); vals_reset(cv);
  for (int i = 0; i < 8; ++i) cstart[i] = 0;
  /* R12: values met before the model is known */
  bool have_id = false, have_status = false;
  int64_t early_id = 0; uint64_t status_q = 0; int st_pet = -1, st_ord = -1;

  skip_ws(r, s);
  uint32_t x = rd_get(r, s.p);
  if (x != '{') { fail_first(r, s, x); return PJ_TYPE_NONE; }
  s.p++;
  bool first = true;
  Sink k;
  uint64_t close_pos = 0;
  for (;;) {
    int m = next_member(r, s, first, k, &close_pos);
    if (m == 0) return PJ_TYPE_NONE;
    if (m == 2) break;
    bool small = sink_small(k);
    if (type == PJ_TYPE_NONE) {
      int kp = small ? find_field(S.obj[OBJ_PET], k.n, k.w[0], k.w[1]) : -1;
      int ko = small ? find_field(S.obj[OBJ_ORDER], k.n, k.w[0], k.w[1]) : -1;
      int ku = small ? find_field(S.obj[OBJ_USER], k.n, k.w[0], k.w[1]) : -1;
      int owners = (kp >= 0) + (ko >= 0) + (ku >= 0);
      if (owners == 1) {
        type = kp >= 0 ? PJ_TYPE_PET : (ko >= 0 ? PJ_TYPE_ORDER : PJ_TYPE_USER);
        O = type == PJ_TYPE_PET ? &S.obj[OBJ_PET] : (type == PJ_TYPE_ORDER ? &S.obj[OBJ_ORDER] : &S.obj[OBJ_USER]);
        if (have_id) { v.v[0] = early_id; v.present |= 1; }
        if (have_status && type != PJ_TYPE_USER) {
          int e = type == PJ_TYPE_PET ? st_pet : st_ord;
          int fi = type == PJ_TYPE_PET ? 5 : 4;
          if (e >= 0) { v.v[fi] = e; v.present |= 1u << fi; }
          else if (!(r.opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL)) { fail(s, PJ_E_ENUM, status_q); return PJ_TYPE_NONE; }
        }
      } else if (owners == 3) { /* `id`, int64 in every model */
        uint32_t y = rd_get(r, s.p);
        if (y == 'n') { if (!lex_literal(r, s, PJ_LIT_ULL, 3)) return PJ_TYPE_NONE; have_id = false; continue; }
        if (!read_int(r, s, y, true, &early_id)) return PJ_TYPE_NONE;
        have_id = true;
        continue;
      } else if (owners == 2) { /* `status` of Pet or Order */
        uint32_t y = rd_get(r, s.p);
        if (y == 'n') { if (!lex_literal(r, s, PJ_LIT_ULL, 3)) return PJ_TYPE_NONE; have_status = false; continue; }
        if (y != '"') { fail_first(r, s, y); return PJ_TYPE_NONE; }
        status_q = s.p;
        Sink e;
        sink_init(e, SINK_PACK);
        if (!lex_string(r, s, e)) return PJ_TYPE_NONE;
        bool sm = sink_small(e);
        st_pet = sm ? find_enum(S.en[0], e.n, e.w[0], e.w[1]) : -1;
        st_ord = sm ? find_enum(S.en[1], e.n, e.w[0], e.w[1]) : -1;
        if (st_pet < 0 && st_ord < 0 && !(r.opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL)) { fail(s, PJ_E_ENUM, status_q); return PJ_TYPE_NONE; }
        have_status = true;
        continue;
      } else {
        if (!skip_value(r, s)) return PJ_TYPE_NONE;
        continue;
      }
    }
    int i = small ? find_field(*O, k.n, k.w[0], k.w[1]) : -1;
    if (i < 0) { if (!skip_value(r, s)) return PJ_TYPE_NONE; continue; }
    const FieldDesc& F = O->f[i];
    uint32_t bit = 1u << i;
    if (F.kind <= K_DATETIME) {
      if (!read_scalar<W>(S, r, s, F, i, v, o, 0, true)) return PJ_TYPE_NONE;
      continue;
    }
    x = rd_get(r, s.p);
    if (F.kind == K_OBJ) {
      const ObjDesc& Cd = S.obj[F.child];
      if (x == 'n') {
        if (!lex_literal(r, s, PJ_LIT_ULL, 3)) return PJ_TYPE_NONE;
        v.present &= ~bit; vals_reset(cv);
        for (int j = 0; j < (int)Cd.nfields; ++j) if (Cd.f[j].kind == K_STR) o.cnt[Cd.f[j].cnt] = 0;
        continue;
      }
      if (x != '{') { fail_first(r, s, x); return PJ_TYPE_NONE; }
      if (!parse_flat<W>(S, r, s, Cd, cv, o, false, true, cstart)) return PJ_TYPE_NONE;
      v.present |= bit;
      continue;
    }
    /* lists: a repeated key starts over (R4) */
    o.cnt[F.cnt] = 0;
    if (F.kind == K_LIST_STR) o.cnt[F.cnt + 1] = 0;
    else { const ObjDesc& Ed = S.obj[F.child]; for (int j = 0; j < (int)Ed.nfields; ++j) if (Ed.f[j].kind == K_STR) o.cnt[Ed.f[j].cnt] = 0; }
    if (x == 'n') { if (!lex_literal(r, s, PJ_LIT_ULL, 3)) return PJ_TYPE_NONE; v.present &= ~bit; continue; }
    if (x != '[') { fail_first(r, s, x); return PJ_TYPE_NONE; }
    s.p++;
    v.present |= bit;
    skip_ws(r, s);
    if (rd_get(r, s.p) == ']') { s.p++; continue; }
    if (LH::enabled && LH::template list<W>(S, r, s, F, o)) continue;
    for (;;) {
      skip_ws(r, s);
      x = rd_get(r, s.p);
      uint32_t j = o.cnt[F.cnt];
      bool live = W && j < o.room[F.cnt];
      if (F.kind == K_LIST_STR) {
        if (x != '"') { fail_first(r, s, x); return PJ_TYPE_NONE; }
        Sink e;
        uint32_t at = o.cnt[F.cnt + 1];
        sink_init(e, live ? SINK_WRITE : SINK_COUNT);
        if (live) {
          uint32_t rm = o.room[F.cnt + 1];
          e.room = rm > at ? rm - at : 0;
          e.dst = colp<uint8_t>(o.cols, F.col + 2) + o.base[F.cnt + 1] + at;
          colp<uint32_t>(o.cols, F.col + 1)[o.base[F.cnt] + j] = o.base[F.cnt + 1] + at;
        }
        if (!lex_string(r, s, e)) return PJ_TYPE_NONE;
        o.cnt[F.cnt + 1] = at + e.n;
      } else {
        if (x != '{') { fail_first(r, s, x); return PJ_TYPE_NONE; } /* null elements are PJ_E_TYPE (R5) */
        const ObjDesc& Ed = S.obj[F.child];
        if (!parse_flat<W>(S, r, s, Ed, ev, o, true, live, estart)) return PJ_TYPE_NONE;
        if (live) store_object<W>(Ed, ev, (uint64_t)o.base[F.cnt] + j, o, estart);
      }
      o.cnt[F.cnt] = j + 1;
      skip_ws(r, s);
      x = rd_get(r, s.p);
      if (x == ',') { s.p++; continue; }
      if (x == ']') { s.p++; break; }
      fail_byte(r, s, s.p, PJ_E_SYNTAX, s.p);
      return PJ_TYPE_NONE;
    }
  }
  if (type == PJ_TYPE_NONE) { fail(s, PJ_E_AMBIGUOUS, close_pos); return PJ_TYPE_NONE; }
  if ((v.present & O->required_mask) != O->required_mask) { fail(s, PJ_E_REQUIRED, close_pos); return PJ_TYPE_NONE; }
  skip_ws(r, s);
  /* the extent must end here: LF (NDJSON) or its limit */
  if (s.p < r.limit) {
    if (r.lf_ws || ld_byte(r.in + s.p) != '\n') { fail(s, PJ_E_SYNTAX, s.p); return PJ_TYPE_NONE; }
  } else if (r.open_end) { fail(s, PJ_E_TOO_LONG, r.limit); return PJ_TYPE_NONE; }
  if (W) {
    uint64_t row = schema == PJ_SCHEMA_MIXED ? (uint64_t)o.base[type - 1] : rec_index;
    store_object<W>(*O, v, row, o, zero_start);
    for (int i = 0; i < (int)O->nfields; ++i) {
      if (O->f[i].kind != K_OBJ) continue;
      if (!((v.present >> i) & 1)) vals_reset(cv);
      store_object<W>(S.obj[O->f[i].child], cv, row, o, zero_start);
    }
  }
  if (schema == PJ_SCHEMA_MIXED) o.cnt[type - 1] = 1;
  return type;
}

/* Emit pass for a record the size pass rejected (single-model streams keep an all-absent row). */
template <bool W>
PJ_HD void store_absent(const Schema& S, uint32_t schema, const Out<W>& o, uint64_t row) {
  const ObjDesc& O = schema == PJ_SCHEMA_PET ? S.obj[OBJ_PET] : (schema == PJ_SCHEMA_ORDER ? S.obj[OBJ_ORDER] : S.obj[OBJ_USER]);
  ObjVals z;
  uint32_t zero_start[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  vals_reset(z);
  store_object<W>(O, z, row, o, zero_start);
  for (int i = 0; i < (int)O.nfields; ++i)
    if (O.f[i].kind == K_OBJ) store_object<W>(S.obj[O.f[i].child], z, row, o, zero_start);
}

}  // namespace pj
#endif
