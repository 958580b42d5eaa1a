/*
 * pj_fast.cuh — the speculative word-at-a-time record tokeniser, instantiated on the compile-time
 * model tables of pj_schema.h.
 *
 * fast_record<>() reads a record 8 bytes at a time from a window staged in shared memory (or, for a record
 * that missed the window, from where it lies in global memory). It gives one of three verdicts:
 *   accepted  the record is valid, every key is known and met once (in any order, with any blanks, with
 *             null values, escapes and UTF-8 in its strings). Its values, counts and the place of every
 *             string are known after ONE pass; they are kept (values in registers, strings as 32-bit tape
 *             words in shared memory) until the record's output positions are known, and then replayed by
 *             fast_emit<>() - or, when they outnumber the tape, by a second pass of fast_outline<>();
 *   failed    the record fails validation in one of the common ways (wrong JSON type, unknown enum literal,
 *             missing required property, bad date-time, record ending inside a string); kind and byte offset
 *             are exactly what the generic parser reports, because everything before was accepted;
 *   refused   anything else (unknown or repeated key, number with a fraction, ...): the caller runs the exact
 *             byte-wise parser of pj_core.cuh on the record.
 * What it accepts it decodes exactly as the generic parser would; a host build of this header is fuzzed
 * against the CPU checker for that.
 *
 * Rare and large parts (escapes and UTF-8 in strings, decoding at emission, the second pass) are out of
 * line on purpose: inlined into the hot loop they made it miss the instruction cache and run 3x slower.
 *
 * All positions here are 32-bit offsets into the window; every property index, kind, column and
 * counter slot is a template constant, so per-record state lives in registers.
 */
#ifndef PJ_FAST_CUH
#define PJ_FAST_CUH

#include "pj_core.cuh"

namespace pj {

/* A staged window: window byte k is input byte w0 + k. The staged bytes are followed by at least 32
 * bytes of LF padding, so 16-byte look-ahead from any byte of a staged record is safe. */
struct Win {
  const uint8_t* s; /* window bytes; 4-byte aligned */
  int64_t w0;       /* input offset of s[0] (can be negative by < 16 for a misaligned input) */
};

PJ_HD uint32_t wbyte(const Win& w, uint32_t p) { return w.s[p]; }
/* 4 / 8 bytes at window offset p, little endian */
PJ_HD uint32_t wpeek4(const Win& w, uint32_t p) {
  const uint32_t* a = reinterpret_cast<const uint32_t*>(w.s) + (p >> 2);
  const uint32_t sh = (p & 3u) * 8u;
  const uint32_t x0 = a[0], x1 = a[1];
#if defined(__CUDA_ARCH__)
  return __funnelshift_r(x0, x1, sh);
#else
  return sh ? (x0 >> sh) | (x1 << (32 - sh)) : x0;
#endif
}
PJ_HD uint64_t wpeek8(const Win& w, uint32_t p) {
  const uint32_t* a = reinterpret_cast<const uint32_t*>(w.s) + (p >> 2);
  const uint32_t sh = (p & 3u) * 8u;
  const uint32_t x0 = a[0], x1 = a[1], x2 = a[2];
#if defined(__CUDA_ARCH__)
  const uint32_t lo = __funnelshift_r(x0, x1, sh), hi = __funnelshift_r(x1, x2, sh);
#else
  const uint32_t lo = sh ? (x0 >> sh) | (x1 << (32 - sh)) : x0, hi = sh ? (x1 >> sh) | (x2 << (32 - sh)) : x1;
#endif
  return (uint64_t)lo | ((uint64_t)hi << 32);
}

PJ_HD uint32_t ctz64(uint64_t x) {
#if defined(__CUDA_ARCH__)
  return (uint32_t)(__ffsll((long long)x) - 1);
#else
  return (uint32_t)__builtin_ctzll(x);
#endif
}

#define PJ_ONES 0x0101010101010101ull
#define PJ_HIGH 0x8080808080808080ull
/* flag (0x80) in the lowest byte of w that equals c; flags above it may be spurious */
PJ_HD uint64_t swar_eq(uint64_t w, uint32_t c) {
  const uint64_t x = w ^ (PJ_ONES * c);
  return (x - PJ_ONES) & ~x & PJ_HIGH;
}
/* flags for bytes that end a plain string run: '"', '\\', < 0x20, >= 0x80 (lowest flag exact) */
PJ_HD uint64_t swar_str_special(uint64_t w) {
  const uint64_t lt20 = (w - PJ_ONES * 0x20) & ~w & PJ_HIGH;
  return swar_eq(w, '"') | swar_eq(w, '\\') | lt20 | (w & PJ_HIGH);
}
/* flags for bytes that are not ASCII digits (lowest flag exact) */
PJ_HD uint64_t swar_nondigit(uint64_t w) { return ((w + PJ_ONES * 0x46) | (w - PJ_ONES * 0x30) | w) & PJ_HIGH; }
/* value of 8 ASCII digits, first digit in the lowest byte */
PJ_HD uint32_t swar_parse8(uint64_t w) {
  w -= PJ_ONES * 0x30;
  w = w * 10 + (w >> 8);
  const uint64_t mask = 0x000000FF000000FFull;
  w = ((w & mask) * 0x000F424000000064ull + ((w >> 16) & mask) * 0x0000271000000001ull) >> 32;
  return (uint32_t)w;
}
/* value of the first k (1..8) digits of w */
PJ_HD uint32_t swar_parse_k(uint64_t w, uint32_t k) {
  if (k < 8) w = (w << (64 - 8 * k)) | ((PJ_ONES * 0x30) >> (8 * k));
  return swar_parse8(w);
}

/* ---- tape ---------------------------------------------------------------------------------------
 * 32-bit words in reading order, kept in shared memory until the record's output positions are known:
 *   string          bits 0..3 byte-counter slot, bits 4..14 decoded length (< 2048), bit 15 "has backslash escapes",
 *                   bits 16..31 window offset of the first content byte
 *   list element    bits 0..3 = TAPE_ELEM, bits 4..11 presence bits, bits 12..15 the list's item-counter slot;
 *                   followed by two words (low, high) for every non-string property of the element, in
 *                   property order, and then by the element's strings as ordinary string words          */
enum { TAPE_ELEM = 15, TAPE_MAX_STR = 2047, TAPE_ESC = 1u << 15 };
static_assert(NSLOT <= 15, "slot numbers share four bits with the element marker");
struct Tape {
  uint32_t* e; /* word k of this thread is e[k * stride] */
  uint32_t stride, cap, n;
};
PJ_HD void tape_push(Tape& t, uint32_t v) {
  if (t.n < t.cap) t.e[(size_t)t.n * t.stride] = v;
  t.n++; /* n > cap afterwards means overflow */
}
PJ_HD void tape_set(Tape& t, uint32_t k, uint32_t v) { if (k < t.cap) t.e[(size_t)k * t.stride] = v; }
PJ_HD uint32_t tape_get(const Tape& t, uint32_t k) { return t.e[(size_t)k * t.stride]; }
PJ_HD uint32_t tape_str(uint32_t slot, uint32_t len, uint32_t pos, uint32_t esc) { return slot | (len << 4) | (esc ? (uint32_t)TAPE_ESC : 0u) | (pos << 16); }

/* tokeniser position: window offsets */
struct FastState {
  uint32_t p, limit; /* limit: window offset of the first byte that is not the record's */
  uint32_t lf_ws;
  uint32_t err, err_pos; /* a validation failure found on this path (kind, window offset); 0 = none */
};

/* Records a failure that the generic parser would report in exactly the same way. Every function below
 * returns false both for "refused" (err stays 0: the generic parser decides) and for "failed" (err set);
 * callers pass false upwards without trying anything else, so the first failure in reading order stands. */
PJ_HD bool fast_fail(FastState& f, uint32_t kind, uint32_t pos) { f.err = kind; f.err_pos = pos; return false; }
/* The byte x at f.p cannot start a value of the expected type. When it starts a value of another type
 * that is PJ_E_TYPE at f.p; null, the end of the record and stray bytes are left to the generic parser. */
PJ_HD bool fast_wrong_type(FastState& f, uint32_t x) {
  if (f.p < f.limit && (x == '"' || x == '-' || x - '0' <= 9u || x == '{' || x == '[' || x == 't' || x == 'f')) return fast_fail(f, PJ_E_TYPE, f.p);
  return false;
}

PJ_HD void fast_ws_slow(const Win& w, FastState& f) {
  for (;;) {
    const uint32_t x = wbyte(w, f.p);
    if ((x == ' ' || x == '\t' || x == '\r' || (f.lf_ws && x == '\n')) && f.p < f.limit) f.p++; else break;
  }
}
/* skips whitespace and returns the byte at the new position; one compare when there is none */
PJ_HD uint32_t fast_ws(const Win& w, FastState& f) {
  uint32_t x = wbyte(w, f.p);
  if (x <= ' ') { fast_ws_slow(w, f); x = wbyte(w, f.p); }
  return x;
}

/* four hex digits at window offset q; false if one is not a hex digit */
PJ_HD bool fast_hex4(const Win& w, uint32_t q, uint32_t* out) {
  uint32_t v = 0;
  for (uint32_t i = 0; i < 4; ++i) {
    const int h = hexval(wbyte(w, q + i));
    if (h < 0) return false;
    v = v << 4 | (uint32_t)h;
  }
  *out = v;
  return true;
}
PJ_HD uint32_t utf8_len(uint32_t cp) { return cp < 0x80 ? 1u : (cp < 0x800 ? 2u : (cp < 0x10000 ? 3u : 4u)); }

/* The part of a string value after its first byte that is not plain (a backslash or a non-ASCII byte, at window
 * offset q, with `dec` decoded bytes before it), out of line because it is rare and large. Accepts what
 * lex_string() of pj_core.cuh accepts (escapes, surrogate pairs, well-formed UTF-8). Result: bits 0..31 offset
 * of the closing quote, bits 32..55 decoded bytes, bit 56 "has backslash escapes", bits 60..61 status
 * (0 accepted, 1 refused, 2 the record ends at bits 0..31 inside the string). */
enum { FS_OK = 0, FS_REFUSED = 1, FS_EOF = 2 };
PJ_HD uint64_t fs_result(uint32_t status, uint32_t q, uint32_t dec, uint32_t esc) {
  return (uint64_t)q | ((uint64_t)(dec & 0xFFFFFFu) << 32) | ((uint64_t)esc << 56) | ((uint64_t)status << 60);
}
PJ_HD_NOINLINE uint64_t fast_string_tail(const uint8_t* ws, uint32_t q, uint32_t dec, uint32_t limit, uint32_t lf_ws) {
  Win w;
  w.s = ws; w.w0 = 0;
  uint32_t any_esc = 0;
  for (;;) {
    const uint64_t m = swar_str_special(wpeek8(w, q));
    if (!m) { q += 8; dec += 8; if (q > limit) return fs_result(FS_REFUSED, 0, 0, 0); continue; }
    const uint32_t k = ctz64(m) >> 3;
    q += k; dec += k;
    if (q >= limit || dec > 0xFFFFFFu) return fs_result(FS_REFUSED, 0, 0, 0);
    const uint32_t x = wbyte(w, q);
    if (x == '"') return fs_result(FS_OK, q, dec, any_esc);
    if (x == '\\') {
      const uint32_t y = wbyte(w, q + 1);
      if (y == 'u') {
        uint32_t cp;
        if (q + 6 > limit || !fast_hex4(w, q + 2, &cp)) return fs_result(FS_REFUSED, 0, 0, 0);
        if (cp - 0xDC00u < 0x400u) return fs_result(FS_REFUSED, 0, 0, 0);
        if (cp - 0xD800u < 0x400u) {
          uint32_t lo;
          if (q + 12 > limit || wbyte(w, q + 6) != '\\' || wbyte(w, q + 7) != 'u' || !fast_hex4(w, q + 8, &lo)) return fs_result(FS_REFUSED, 0, 0, 0);
          if (lo - 0xDC00u >= 0x400u) return fs_result(FS_REFUSED, 0, 0, 0);
          dec += 4; q += 12;
        } else { dec += utf8_len(cp); q += 6; }
      } else if (y == '"' || y == '\\' || y == '/' || y == 'b' || y == 'f' || y == 'n' || y == 'r' || y == 't') {
        if (q + 2 > limit) return fs_result(FS_REFUSED, 0, 0, 0);
        dec += 1; q += 2;
      } else return fs_result(FS_REFUSED, 0, 0, 0);
      any_esc = 1;
      continue;
    }
    if (x < 0x20) return (x == '\n' && !lf_ws) ? fs_result(FS_EOF, q, 0, 0) : fs_result(FS_REFUSED, 0, 0, 0);
    /* RFC 3629, the table of lex_string() */
    uint32_t need, lo = 0x80, hi = 0xBF;
    if (x - 0xC2u <= 0x1Du) need = 1;
    else if (x == 0xE0) { need = 2; lo = 0xA0; }
    else if (x == 0xED) { need = 2; hi = 0x9F; }
    else if (x - 0xE1u <= 0x0Eu) need = 2;
    else if (x == 0xF0) { need = 3; lo = 0x90; }
    else if (x - 0xF1u <= 2u) need = 3;
    else if (x == 0xF4) { need = 3; hi = 0x8F; }
    else return fs_result(FS_REFUSED, 0, 0, 0);
    if (q + need >= limit) return fs_result(FS_REFUSED, 0, 0, 0);
    const uint32_t y1 = wbyte(w, q + 1);
    if (y1 < lo || y1 > hi) return fs_result(FS_REFUSED, 0, 0, 0);
    if (need >= 2 && wbyte(w, q + 2) - 0x80u > 0x3Fu) return fs_result(FS_REFUSED, 0, 0, 0);
    if (need >= 3 && wbyte(w, q + 3) - 0x80u > 0x3Fu) return fs_result(FS_REFUSED, 0, 0, 0);
    dec += need + 1; q += need + 1;
  }
}

/* A string VALUE at f.p (opening quote): *pos = offset of the first content byte, *len = DECODED bytes,
 * *esc = it holds backslash escapes (so raw and decoded bytes differ). Plain strings (printable ASCII, no
 * backslash) are finished here, 8 bytes a step; the rest goes through fast_string_tail(). Refuses what it does not
 * accept, but for the one failure it reports itself: the record ending inside the string. */
template <bool TAPE_LIMITS>
PJ_COLD bool fast_string_t(const Win& w, FastState& f, uint32_t* pos, uint32_t* len, uint32_t* esc) {
  uint32_t q = f.p + 1;
  for (;;) {
    const uint64_t m = swar_str_special(wpeek8(w, q));
    if (m) { q += ctz64(m) >> 3; break; }
    q += 8;
    if (q > f.limit) return false;
  }
  if (q >= f.limit) return false;
  uint32_t dec = q - (f.p + 1), any_esc = 0;
  const uint32_t x = wbyte(w, q);
  if (x != '"') {
    if (x < 0x20) {
      /* a line feed inside a string of an LF-delimited record: the record's bytes end here */
      if (x == '\n' && !f.lf_ws) return fast_fail(f, PJ_E_EOF, q);
      return false;
    }
    const uint64_t r = fast_string_tail(w.s, q, dec, f.limit, f.lf_ws);
    const uint32_t status = (uint32_t)(r >> 60) & 3u;
    if (status == FS_EOF) return fast_fail(f, PJ_E_EOF, (uint32_t)r);
    if (status != FS_OK) return false;
    q = (uint32_t)r; dec = (uint32_t)(r >> 32) & 0xFFFFFFu; any_esc = (uint32_t)(r >> 56) & 1u;
  }
  if (TAPE_LIMITS && (dec > TAPE_MAX_STR || f.p + 1 > 0xFFFFu)) return false; /* what a tape word can hold */
  *pos = f.p + 1; *len = dec; *esc = any_esc;
  f.p = q + 1;
  return true;
}
PJ_HD bool fast_string(const Win& w, FastState& f, uint32_t* pos, uint32_t* len, uint32_t* esc) { return fast_string_t<true>(w, f, pos, len, esc); }

/* A plain short string (key or enum literal, <= 14 bytes) at f.p, packed like the model tables. */
PJ_COLD bool fast_short(const Win& w, FastState& f, uint32_t* len, uint64_t* lo, uint64_t* hi) {
  const uint64_t a = wpeek8(w, f.p + 1);
  const uint64_t ma = swar_str_special(a);
  uint32_t n;
  uint64_t b = 0;
  if (ma) n = ctz64(ma) >> 3;
  else {
    b = wpeek8(w, f.p + 9);
    const uint64_t mb = swar_str_special(b);
    if (!mb) return false;
    n = 8 + (ctz64(mb) >> 3);
  }
  if (f.p + 1 + n >= f.limit || wbyte(w, f.p + 1 + n) != '"') return false;
  if (n < 8) { *lo = n ? a & (~0ull >> (64 - 8 * n)) : 0; *hi = 0; }
  else { *lo = a; *hi = n > 8 ? b & (~0ull >> (64 - 8 * (n - 8))) : 0; }
  *len = n;
  f.p += n + 2;
  return true;
}

/* An integer at f.p: -?(0|[1-9][0-9]{0,18}) not followed by '.', 'e', 'E'. */
PJ_COLD bool fast_int(const Win& w, FastState& f, bool is64, int64_t* out) {
  uint32_t p = f.p;
  const bool neg = wbyte(w, p) == '-';
  if (neg) p++;
  const uint32_t first = wbyte(w, p);
  uint64_t mag = 0;
  uint32_t nd = 0;
  for (;;) {
    const uint64_t x = wpeek8(w, p);
    const uint64_t m = swar_nondigit(x);
    if (!m) { mag = mag * 100000000u + swar_parse8(x); nd += 8; p += 8; if (nd > 19) return false; continue; }
    const uint32_t k = ctz64(m) >> 3;
    if (k) {
      uint32_t scale = (k & 1) ? 10u : 1u;
      if (k & 2) scale *= 100u;
      if (k & 4) scale *= 10000u;
      mag = mag * scale + swar_parse_k(x, k);
    }
    nd += k; p += k;
    break;
  }
  if (nd == 0 || nd > 19 || (first == '0' && nd > 1)) return false;
  const uint32_t t = wbyte(w, p);
  if (t == '.' || (t | 0x20) == 'e') return false;
  /* 19 digits can exceed 2^63 but not 2^64 */
  const uint64_t lim = is64 ? (neg ? 0x8000000000000000ull : 0x7FFFFFFFFFFFFFFFull) : (neg ? 0x80000000ull : 0x7FFFFFFFull);
  if (mag > lim) return false;
  *out = neg ? (int64_t)(0 - mag) : (int64_t)mag;
  f.p = p;
  return p <= f.limit;
}

/* RFC 3339 date-time in the n bytes at window offset pos (plain ASCII, no escapes), decoded exactly as
 * parse_datetime() of pj_core.cuh decodes it; false for anything that function would reject. The fixed
 * part `YYYY-MM-DDThh:mm:ss` is checked as two 8-byte words and one 4-byte word. */
PJ_COLD bool fast_datetime(const Win& w, uint32_t pos, uint32_t n, int64_t* epoch, int32_t* nanos, int32_t* off) {
  if (n < 20 || n > 35) return false;
  const uint64_t a = wpeek8(w, pos), b = wpeek8(w, pos + 8);
  const uint32_t c = wpeek4(w, pos + 16);
  /* separators: a = YYYY-MM-  b = DDThh:mm  c = :ss? */
  if ((a & 0xFF0000FF00000000ull) != 0x2D00002D00000000ull) return false;
  if ((b & 0x0000FF0000FF0000ull) != 0x00003A0000540000ull) return false;
  if ((c & 0xFFu) != ':') return false;
  const uint64_t da = (a & ~0xFF0000FF00000000ull) | 0x3000003000000000ull;
  const uint64_t db = (b & ~0x0000FF0000FF0000ull) | 0x0000300000300000ull;
  const uint64_t dc = ((uint64_t)(c >> 8) & 0xFFFFull) | 0x3030303030300000ull;
  if (swar_nondigit(da) | swar_nondigit(db) | swar_nondigit(dc)) return false;
#define PJ_DG(word, k) ((uint32_t)((word) >> (8 * (k))) & 0xFu)
  const uint32_t year = PJ_DG(a, 0) * 1000 + PJ_DG(a, 1) * 100 + PJ_DG(a, 2) * 10 + PJ_DG(a, 3);
  const uint32_t mon = PJ_DG(a, 5) * 10 + PJ_DG(a, 6), day = PJ_DG(b, 0) * 10 + PJ_DG(b, 1);
  const uint32_t hh = PJ_DG(b, 3) * 10 + PJ_DG(b, 4), mi = PJ_DG(b, 6) * 10 + PJ_DG(b, 7), ss = PJ_DG(c, 1) * 10 + PJ_DG(c, 2);
#undef PJ_DG
  if (mon < 1 || mon > 12 || day < 1) return false;
  uint32_t dim = (mon == 2) ? 28u : ((mon == 4 || mon == 6 || mon == 9 || mon == 11) ? 30u : 31u);
  if (mon == 2 && (year % 4 == 0 && (year % 100 != 0 || year % 400 == 0))) dim = 29;
  if (day > dim || hh > 23 || mi > 59 || ss > 59) return false;
  uint32_t i = 19, ns = 0;
  uint32_t x = c >> 24;
  if (x == '.') {
    uint32_t kd = 0;
    ++i;
    for (;;) {
      x = i < n ? wbyte(w, pos + i) : 0u;
      if (x - '0' > 9u) break;
      if (kd >= 9) return false;
      ns = ns * 10 + (x - '0'); ++kd; ++i;
    }
    if (kd == 0) return false;
    for (; kd < 9; ++kd) ns *= 10;
  }
  if (i >= n) return false;
  int32_t o = 0;
  if (x == 'Z') { if (i + 1 != n) return false; }
  else if (x == '+' || x == '-') {
    if (i + 6 != n) return false;
    const uint64_t z = wpeek8(w, pos + i + 1); /* hh:mm */
    if (((z >> 16) & 0xFFu) != ':') return false;
    const uint64_t dz = ((z & 0xFFFF00FFFFull) | 0x3030300000300000ull);
    if (swar_nondigit(dz)) return false;
    const uint32_t oh = ((uint32_t)z & 0xFu) * 10 + ((uint32_t)(z >> 8) & 0xFu), om = ((uint32_t)(z >> 24) & 0xFu) * 10 + ((uint32_t)(z >> 32) & 0xFu);
    if (oh > 23 || om > 59) return false;
    o = (int32_t)(oh * 3600 + om * 60);
    if (x == '-') o = -o;
  } else return false;
  *epoch = days_from_civil((int64_t)year, mon, day) * 86400 + (int64_t)hh * 3600 + (int64_t)(mi * 60 + ss) - o;
  *nanos = (int32_t)ns; *off = o;
  return true;
}

/* ---- compile-time view of one property ------------------------------------------------------------ */
constexpr uint64_t key_pattern_word(uint64_t lo, uint64_t hi, uint32_t len, uint32_t word) {
  /* bytes of `"name":` number 8*word .. 8*word+7, little endian; 0 past the end */
  uint64_t v = 0;
  for (uint32_t k = 0; k < 8; ++k) {
    const uint32_t b = 8 * word + k;
    uint64_t c = 0;
    if (b == 0 || b == len + 1) c = '"';
    else if (b == len + 2) c = ':';
    else if (b <= len) { const uint32_t q = b - 1; c = q < 8 ? (lo >> (8 * q)) & 0xFF : (hi >> (8 * (q - 8))) & 0xFF; }
    v |= c << (8 * k);
  }
  return v;
}
constexpr uint64_t low_bytes_mask(uint32_t n) { return n >= 8 ? ~0ull : ((1ull << (8 * n)) - 1); }

template <int OBJ, int I>
struct FK {
  static constexpr uint32_t kind = CObj<OBJ>::f[I].kind, col = CObj<OBJ>::f[I].col, cnt = CObj<OBJ>::f[I].cnt,
                            child = CObj<OBJ>::f[I].child, len = CObj<OBJ>::f[I].len;
  static constexpr uint64_t lo = CObj<OBJ>::f[I].lo, hi = CObj<OBJ>::f[I].hi;
  /* the compact spelling `"name":` as one or two 8-byte words */
  static constexpr uint32_t pat_len = len + 3;
  static_assert(pat_len <= 16, "property names of up to 13 bytes");
  static constexpr uint64_t pat0 = key_pattern_word(lo, hi, len, 0), pat1 = key_pattern_word(lo, hi, len, 1);
  static constexpr uint64_t mask0 = low_bytes_mask(pat_len), mask1 = low_bytes_mask(pat_len > 8 ? pat_len - 8 : 0);
};
template <int E, int I>
struct EK {
  static constexpr uint32_t len = CEnum<E>::lit[I].len;
  static constexpr uint64_t lo = CEnum<E>::lit[I].lo, hi = CEnum<E>::lit[I].hi;
};
/* Is the compact spelling of key I at f.p? If so, move past its colon. */
template <int OBJ, int I>
PJ_HD bool at_key(const Win& w, FastState& f) {
  const uint64_t a = wpeek8(w, f.p);
  if ((a & FK<OBJ, I>::mask0) != FK<OBJ, I>::pat0) return false;
  if constexpr (FK<OBJ, I>::pat_len > 8) {
    if ((wpeek8(w, f.p + 8) & FK<OBJ, I>::mask1) != FK<OBJ, I>::pat1) return false;
  }
  f.p += FK<OBJ, I>::pat_len;
  return true;
}
/* index of the property / literal with this packed name, -1 if none (an unrolled compare chain) */
template <int OBJ, int I = 0>
PJ_HD int match_key(uint32_t len, uint64_t lo, uint64_t hi) {
  if constexpr (I >= CObj<OBJ>::N) return -1;
  else {
    if (lo == FK<OBJ, I>::lo && len == FK<OBJ, I>::len && hi == FK<OBJ, I>::hi) return I;
    return match_key<OBJ, I + 1>(len, lo, hi);
  }
}
template <int E, int I = 0>
PJ_HD int match_enum(uint32_t len, uint64_t lo, uint64_t hi) {
  if constexpr (I >= CEnum<E>::N) return -1;
  else {
    if (lo == EK<E, I>::lo && len == EK<E, I>::len && hi == EK<E, I>::hi) return I;
    return match_enum<E, I + 1>(len, lo, hi);
  }
}

/* values of one object; only ever indexed with constants, so it lives in registers */
struct FVals {
  int64_t v[8];
  int64_t aux; /* date-time: nanos << 32 | (uint32) offset */
  uint32_t present;
};

/* Where strings go: while tokenising, onto the tape (and into the counters). Arrays are indexed by
 * constant slot numbers only. */
struct DrainState {
  const DevCols* c;     /* null: nothing is emitted, the tape is only emptied (a counting pass that needs no tape) */
  const uint32_t* base; /* the record's start in every arena / child table */
  uint32_t cur[NSLOT];  /* bytes / items of the record emitted so far */
};
/* DR (a compile-time switch, so the first pass carries none of it): the record is tokenised a second time to be
 * emitted, and the tape is emptied into the columns through d whenever it runs full (records whose strings and
 * list elements outnumber the tape). */
template <bool DR>
struct FSinkT {
  static constexpr bool drain = DR;
  static constexpr bool wide = false;
  Tape* t;
  uint32_t* cnt; /* [NSLOT] bytes / items counted so far */
  DrainState* d;
};
/* The sink of a record that all lanes of a warp tokenise together (same bytes, same steps): non-empty lists are
 * handed to wide_fast_list<>() of pj_wide.cuh, which spreads their elements over the lanes. */
struct FSinkWide {
  static constexpr bool drain = true;
  static constexpr bool wide = true;
  Tape* t;
  uint32_t* cnt;
  DrainState* d;
  uint32_t rec_end; /* window offset of the byte that ends the record (its line feed, or the limit) */
};
template <int OBJ, int I, class S>
PJ_HD bool wide_fast_list(const Win& w, FastState& f, S& s);
/* Tape words one list element of flat object E can take: header, scalars, one string per string property. */
template <int E, int I = 0>
constexpr uint32_t string_fields() {
  if constexpr (I >= CObj<E>::N) return 0;
  else return (CObj<E>::f[I].kind == K_STR ? 1u : 0u) + string_fields<E, I + 1>();
}
enum { TAPE_MIN_CAP = 8 }; /* the largest unit pushed between two drain points is well below this */
template <int OBJ, int I = 0>
PJ_COLD uint32_t replay_word(const Win& w, const DevCols* c, const Tape& t, uint32_t k, uint32_t word, const uint32_t* base, uint32_t* cur);
/* replays what the tape holds into the columns and empties it (a call, not inlined: it is met at many places) */
template <int OBJ>
PJ_HD_NOINLINE void tape_drain(const Win w, const Tape t, DrainState* d) { /* by value: the caller's tape stays in registers */
  if (d->c)
    for (uint32_t k = 0; k < t.n;) k = replay_word<OBJ>(w, d->c, t, k, tape_get(t, k), d->base, d->cur);
}
/* In the emitting pass: make room for `need` more words. */
template <int OBJ, class S>
PJ_HD void tape_room(const Win& w, S& s, uint32_t need) {
  if constexpr (S::drain) { if (s.t->n + need > s.t->cap) { tape_drain<OBJ>(w, *s.t, s.d); s.t->n = 0; } }
}

/* n bytes from window offset pos to dst (global memory): bytes up to 4-byte alignment of dst, then words */
PJ_COLD void copy_win(uint8_t* dst, const Win& w, uint32_t pos, uint32_t n) {
  while (n && (reinterpret_cast<uintptr_t>(dst) & 3u)) { *dst++ = (uint8_t)wbyte(w, pos++); n--; }
  while (n >= 4) { *reinterpret_cast<uint32_t*>(dst) = wpeek4(w, pos); dst += 4; pos += 4; n -= 4; }
  while (n) { *dst++ = (uint8_t)wbyte(w, pos++); n--; }
}

/* n DECODED bytes of the string whose content starts at window offset pos, to dst. The string was accepted by
 * fast_string(), so every escape in it is well formed. */
PJ_HD_NOINLINE void copy_decoded(uint8_t* dst, const uint8_t* ws, uint32_t pos, uint32_t n) {
  Win w;
  w.s = ws; w.w0 = 0;
  uint32_t k = 0;
  while (k < n) {
    const uint32_t x = wbyte(w, pos);
    if (x != '\\') { dst[k++] = (uint8_t)x; pos++; continue; }
    const uint32_t y = wbyte(w, pos + 1);
    uint32_t cp;
    pos += 2;
    switch (y) {
      case 'b': cp = 8; break;
      case 'f': cp = 12; break;
      case 'n': cp = 10; break;
      case 'r': cp = 13; break;
      case 't': cp = 9; break;
      case 'u': {
        cp = 0;
        fast_hex4(w, pos, &cp);
        pos += 4;
        if (cp - 0xD800u < 0x400u) {
          uint32_t lo = 0;
          fast_hex4(w, pos + 2, &lo);
          cp = 0x10000u + ((cp - 0xD800u) << 10) + (lo - 0xDC00u);
          pos += 6;
        }
        break;
      }
      default: cp = y; break; /* '"', '\\', '/' */
    }
    if (cp < 0x80) dst[k++] = (uint8_t)cp;
    else if (cp < 0x800) { dst[k++] = (uint8_t)(0xC0 | (cp >> 6)); dst[k++] = (uint8_t)(0x80 | (cp & 63)); }
    else if (cp < 0x10000) { dst[k++] = (uint8_t)(0xE0 | (cp >> 12)); dst[k++] = (uint8_t)(0x80 | ((cp >> 6) & 63)); dst[k++] = (uint8_t)(0x80 | (cp & 63)); }
    else { dst[k++] = (uint8_t)(0xF0 | (cp >> 18)); dst[k++] = (uint8_t)(0x80 | ((cp >> 12) & 63)); dst[k++] = (uint8_t)(0x80 | ((cp >> 6) & 63)); dst[k++] = (uint8_t)(0x80 | (cp & 63)); }
  }
}
/* the string of one tape word to dst */
PJ_HD void copy_tape_str(uint8_t* dst, const Win& w, uint32_t word) {
  const uint32_t len = (word >> 4) & 0x7FFu, pos = word >> 16;
  if (word & TAPE_ESC) copy_decoded(dst, w.s, pos, len); else copy_win(dst, w, pos, len);
}

/* the literal null at f.p */
PJ_HD bool fast_null(const Win& w, FastState& f) {
  if (wpeek4(w, f.p) != 0x6C6C756Eu || f.p + 4 > f.limit) return false;
  f.p += 4;
  return true;
}
/* Value of scalar property I of OBJ at f.p (kinds I64, I32, BOOL, STR, ENUM, DATETIME), or null. */
template <int OBJ, int I, class S>
PJ_COLD bool fast_scalar(const Win& w, FastState& f, S& s, FVals& v) {
  constexpr uint32_t kind = FK<OBJ, I>::kind, slot = FK<OBJ, I>::cnt;
  if (v.present & (1u << I)) return false; /* repeated key */
  const uint32_t x = wbyte(w, f.p);
  if (x == 'n') return fast_null(w, f); /* null: the property stays absent */
  if constexpr (kind == K_I64 || kind == K_I32) {
    int64_t val;
    if (!(x == '-' || x - '0' <= 9u)) return fast_wrong_type(f, x);
    if (!fast_int(w, f, kind == K_I64, &val)) return false;
    v.v[I] = val;
  } else if constexpr (kind == K_BOOL) {
    const uint64_t k = wpeek8(w, f.p);
    if ((k & 0xFFFFFFFFull) == 0x65757274ull) { v.v[I] = 1; f.p += 4; }
    else if ((k & 0xFFFFFFFFFFull) == 0x65736C6166ull) { v.v[I] = 0; f.p += 5; }
    else if (x != 't' && x != 'f') return fast_wrong_type(f, x);
    else return false;
  } else if constexpr (kind == K_STR) {
    if (x != '"') return fast_wrong_type(f, x);
    uint32_t pos, len, esc;
    if (!fast_string(w, f, &pos, &len, &esc)) return false;
    tape_push(*s.t, tape_str(slot, len, pos, esc));
    s.cnt[slot] += len;
  } else if constexpr (kind == K_ENUM) {
    if (x != '"') return fast_wrong_type(f, x);
    const uint32_t q = f.p;
    uint32_t len; uint64_t lo, hi;
    if (!fast_short(w, f, &len, &lo, &hi)) {
      /* not a short plain string; a long plain one is a well-formed string that is no literal */
      uint32_t pos, esc;
      if (fast_string(w, f, &pos, &len, &esc) && !esc) return fast_fail(f, PJ_E_ENUM, q);
      return false; /* with escapes the decoded text decides: left to the generic parser */
    }
    const int e = match_enum<FK<OBJ, I>::child>(len, lo, hi);
    if (e < 0) return fast_fail(f, PJ_E_ENUM, q);
    v.v[I] = e;
  } else if constexpr (kind == K_DATETIME) {
    if (x != '"') return fast_wrong_type(f, x);
    const uint32_t q = f.p;
    uint32_t pos, len, esc;
    if (!fast_string(w, f, &pos, &len, &esc) || esc) return false;
    int64_t ep; int32_t ns, of;
    if (!fast_datetime(w, pos, len, &ep, &ns, &of)) return fast_fail(f, PJ_E_DATETIME, q);
    v.v[I] = ep; v.aux = (int64_t)(((uint64_t)(uint32_t)ns << 32) | (uint32_t)of);
  } else return false;
  v.present |= 1u << I;
  return true;
}

/* `ws* : ws*` */
PJ_HD bool fast_colon(const Win& w, FastState& f) {
  if (fast_ws(w, f) != ':') return false;
  f.p++;
  fast_ws(w, f);
  return true;
}
/* key at f.p -> property index of OBJ, positioned at the value; -1: refuse */
template <int OBJ>
PJ_COLD int fast_key(const Win& w, FastState& f) {
  if (wbyte(w, f.p) != '"') return -1;
  uint32_t len; uint64_t lo, hi;
  if (!fast_short(w, f, &len, &lo, &hi)) return -1;
  const int i = match_key<OBJ>(len, lo, hi);
  if (i < 0 || !fast_colon(w, f)) return -1;
  return i;
}
/* After a value: `ws* , ws*` (returns 1, positioned at the next key), `ws* }` (returns 2, past the brace), else 0. */
PJ_HD int fast_member_end(const Win& w, FastState& f) {
  const uint32_t x = fast_ws(w, f);
  if (x == ',') { f.p++; fast_ws(w, f); return 1; }
  if (x == '}') { f.p++; return 2; }
  return 0;
}

/* ---- flat objects (Category, Tag): scalar properties only ---------------------------------------- */
template <int OBJ, int I, class S>
PJ_HD bool flat_value(const Win& w, FastState& f, S& s, FVals& v) {
  if constexpr (FK<OBJ, I>::kind <= K_ENUM) return fast_scalar<OBJ, I>(w, f, s, v);
  else return false;
}
template <int OBJ, int I = 0, class S>
PJ_HD bool flat_dispatch(int i, const Win& w, FastState& f, S& s, FVals& v) {
  if constexpr (I >= CObj<OBJ>::N) return false;
  else {
    if (i == I) return flat_value<OBJ, I>(w, f, s, v);
    return flat_dispatch<OBJ, I + 1>(i, w, f, s, v);
  }
}
/* One pass over the properties in model order: every key spelled compactly and in order is matched with
 * one or two word compares. state: 1 = at a key, 2 = object closed, 0 = refuse. */
template <int OBJ, int I = 0, class S>
PJ_HD int flat_inorder(const Win& w, FastState& f, S& s, FVals& v, int state) {
  if constexpr (I >= CObj<OBJ>::N) return state;
  else {
    if (state == 1 && at_key<OBJ, I>(w, f)) {
      fast_ws(w, f);
      if (!flat_value<OBJ, I>(w, f, s, v)) return 0;
      state = fast_member_end(w, f);
    }
    return flat_inorder<OBJ, I + 1>(w, f, s, v, state);
  }
}
/* Flat object at f.p == '{'. */
template <int OBJ, class S>
PJ_COLD bool fast_flat(const Win& w, FastState& f, S& s, FVals& v) {
  v.present = 0;
  f.p++;
  if (fast_ws(w, f) == '}') { f.p++; return true; }
  int state = flat_inorder<OBJ>(w, f, s, v, 1);
  while (state == 1) { /* keys out of order or spelled with blanks */
    const int i = fast_key<OBJ>(w, f);
    if (i < 0 || !flat_dispatch<OBJ>(i, w, f, s, v)) return false;
    state = fast_member_end(w, f);
  }
  return state == 2;
}

/* ---- model roots ------------------------------------------------------------------------------------ */
template <int OBJ, int I = 0>
constexpr uint32_t scalar_words() { /* tape words for the non-string properties of a list element */
  if constexpr (I >= CObj<OBJ>::N) return 0;
  else return (CObj<OBJ>::f[I].kind != K_STR ? 2u : 0u) + scalar_words<OBJ, I + 1>();
}
template <int OBJ, int I = 0>
PJ_HD void tape_put_scalars(Tape& t, uint32_t at, const FVals& v) {
  if constexpr (I < CObj<OBJ>::N) {
    if constexpr (FK<OBJ, I>::kind != K_STR) {
      tape_set(t, at, (uint32_t)(uint64_t)v.v[I]);
      tape_set(t, at + 1, (uint32_t)((uint64_t)v.v[I] >> 32));
      tape_put_scalars<OBJ, I + 1>(t, at + 2, v);
    } else tape_put_scalars<OBJ, I + 1>(t, at, v);
  }
}

/* Property I of a model root at f.p: scalars as above; an embedded object into cv; lists item by item. */
template <int OBJ, int I, class S>
PJ_COLD bool root_value(const Win& w, FastState& f, S& s, FVals& v, FVals& cv) {
  constexpr uint32_t kind = FK<OBJ, I>::kind, cnt = FK<OBJ, I>::cnt;
  if constexpr (kind <= K_ENUM || kind == K_DATETIME) { tape_room<OBJ>(w, s, 1); return fast_scalar<OBJ, I>(w, f, s, v); }
  else {
    if (v.present & (1u << I)) return false;
    if (wbyte(w, f.p) == 'n') return fast_null(w, f); /* null: no object, no list */
    if constexpr (kind == K_OBJ) {
      tape_room<OBJ>(w, s, string_fields<FK<OBJ, I>::child>());
      if (wbyte(w, f.p) != '{') return fast_wrong_type(f, wbyte(w, f.p));
      if (!fast_flat<FK<OBJ, I>::child>(w, f, s, cv)) return false;
    } else {
      if (wbyte(w, f.p) != '[') return fast_wrong_type(f, wbyte(w, f.p));
      f.p++;
      uint32_t j = 0;
      if (fast_ws(w, f) == ']') f.p++;
      else if constexpr (S::wide) {
        if (!wide_fast_list<OBJ, I>(w, f, s)) return false;
        j = s.cnt[cnt];
      } else {
        for (;;) {
          if constexpr (kind == K_LIST_STR) {
            if (wbyte(w, f.p) != '"') return fast_wrong_type(f, wbyte(w, f.p));
            uint32_t pos, len, esc;
            if (!fast_string(w, f, &pos, &len, &esc)) return false;
            if constexpr (S::drain) {
              /* the second pass over a long record: a list of strings is where its bytes are, so the strings go
                 straight to the columns (their slots belong to this list alone, so the order against the words
                 still on the tape does not matter) */
              DrainState& d = *s.d;
              if (d.c) {
                constexpr uint32_t col = FK<OBJ, I>::col;
                colp<uint32_t>(d.c, col + 1)[(uint64_t)d.base[cnt] + d.cur[cnt]] = d.base[cnt + 1] + d.cur[cnt + 1];
                copy_tape_str(colp<uint8_t>(d.c, col + 2) + d.base[cnt + 1] + d.cur[cnt + 1], w, tape_str(0, len, pos, esc));
              }
              d.cur[cnt + 1] += len; d.cur[cnt] += 1;
            } else tape_push(*s.t, tape_str(cnt + 1, len, pos, esc));
            s.cnt[cnt + 1] += len;
          } else {
            /* header word, room for the scalars, then the element's strings as they are met */
            constexpr int E = FK<OBJ, I>::child;
            static_assert(1 + scalar_words<E>() + string_fields<E>() <= TAPE_MIN_CAP, "a list element fits an empty tape");
            tape_room<OBJ>(w, s, 1 + scalar_words<E>() + string_fields<E>());
            if (wbyte(w, f.p) != '{') return fast_wrong_type(f, wbyte(w, f.p));
            const uint32_t at = s.t->n;
            for (uint32_t k = 0; k < 1 + scalar_words<E>(); ++k) tape_push(*s.t, 0);
            FVals ev;
            if (!fast_flat<E>(w, f, s, ev)) return false;
            tape_set(*s.t, at, (uint32_t)TAPE_ELEM | (ev.present << 4) | (cnt << 12));
            tape_put_scalars<E>(*s.t, at + 1, ev);
          }
          j++;
          const uint32_t y = fast_ws(w, f);
          if (y == ',') { f.p++; fast_ws(w, f); continue; }
          if (y == ']') { f.p++; break; }
          return false;
        }
      }
      s.cnt[cnt] = j;
    }
    v.present |= 1u << I;
    return true;
  }
}
template <int OBJ, int I = 0, class S>
PJ_HD bool root_dispatch(int i, const Win& w, FastState& f, S& s, FVals& v, FVals& cv) {
  if constexpr (I >= CObj<OBJ>::N) return false;
  else {
    if (i == I) return root_value<OBJ, I>(w, f, s, v, cv);
    return root_dispatch<OBJ, I + 1>(i, w, f, s, v, cv);
  }
}
template <int OBJ, int I = 0, class S>
PJ_HD int root_inorder(const Win& w, FastState& f, S& s, FVals& v, FVals& cv, int state) {
  if constexpr (I >= CObj<OBJ>::N) return state;
  else {
    if (state == 1 && at_key<OBJ, I>(w, f)) {
      fast_ws(w, f);
      if (!root_value<OBJ, I>(w, f, s, v, cv)) return 0;
      state = fast_member_end(w, f);
    }
    return root_inorder<OBJ, I + 1>(w, f, s, v, cv, state);
  }
}
/* Members of a model root. f.p is after `{ ws*`, or at the value of property `pending` (>= 0) whose key
 * was read already. Ends after the closing brace. */
template <int OBJ, class S>
PJ_COLD bool fast_root(const Win& w, FastState& f, S& s, FVals& v, FVals& cv, int pending) {
  int state = 1;
  if (pending >= 0) {
    if (!root_dispatch<OBJ>(pending, w, f, s, v, cv)) return false;
    state = fast_member_end(w, f);
  } else if (wbyte(w, f.p) == '}') { f.p++; return true; }
  state = root_inorder<OBJ>(w, f, s, v, cv, state);
  while (state == 1) { /* keys out of order or spelled with blanks */
    const int i = fast_key<OBJ>(w, f);
    if (i < 0 || !root_dispatch<OBJ>(i, w, f, s, v, cv)) return false;
    state = fast_member_end(w, f);
  }
  return state == 2;
}

template <int SCHEMA> struct RootOf { static constexpr int obj = SCHEMA == PJ_SCHEMA_PET ? (int)OBJ_PET : (SCHEMA == PJ_SCHEMA_ORDER ? (int)OBJ_ORDER : (int)OBJ_USER); };

enum { FAST_REFUSED = 0, FAST_ACCEPTED = 1, FAST_FAILED = 2 };
template <int SCHEMA, bool DR>
PJ_HD bool fast_record_body(const Win& w, FastState& f, uint32_t open_end, uint32_t* type_out, FVals& v, FVals& cv, uint32_t* cnt, Tape& t, DrainState* d);

/* One record at window offset `start`, ending before window offset `limit`.
 * FAST_ACCEPTED: model in *type_out, root values in v, the embedded object's in cv, counts in cnt[slot]
 *                (all NSLOT entries are reset), strings and list elements on the tape. If t.n > t.cap
 *                afterwards the tape was too small to hold them all: such a record is emitted with
 *                fast_outline<>(), which tokenises it once more.
 * FAST_FAILED:   the record fails validation with *err_kind at window offset *err_pos, exactly as the
 *                generic parser reports it.
 * FAST_REFUSED:  the generic parser has to look at the record. */
template <int SCHEMA>
PJ_HD uint32_t fast_record(const Win& w, uint32_t start, uint32_t limit, uint32_t lf_ws, uint32_t open_end, uint32_t* type_out,
                           FVals& v, FVals& cv, uint32_t* cnt, Tape& t, uint32_t* err_kind, uint32_t* err_pos) {
  FastState f;
  f.p = start; f.limit = limit; f.lf_ws = lf_ws; f.err = 0; f.err_pos = 0;
  if (fast_record_body<SCHEMA, false>(w, f, open_end, type_out, v, cv, cnt, t, nullptr)) return FAST_ACCEPTED;
  if (!f.err) return FAST_REFUSED;
  *err_kind = f.err; *err_pos = f.err_pos;
  return FAST_FAILED;
}
template <int SCHEMA, class S>
PJ_HD bool fast_record_sink(const Win& w, FastState& f, uint32_t open_end, uint32_t* type_out, FVals& v, FVals& cv, S& s);
template <int SCHEMA, bool DR>
PJ_HD bool fast_record_body(const Win& w, FastState& f, uint32_t open_end, uint32_t* type_out, FVals& v, FVals& cv, uint32_t* cnt, Tape& t, DrainState* d) {
  FSinkT<DR> s;
  s.t = &t; s.cnt = cnt; s.d = d;
  return fast_record_sink<SCHEMA>(w, f, open_end, type_out, v, cv, s);
}
template <int SCHEMA, class S>
PJ_HD bool fast_record_sink(const Win& w, FastState& f, uint32_t open_end, uint32_t* type_out, FVals& v, FVals& cv, S& s) {
  const uint32_t limit = f.limit, lf_ws = f.lf_ws;
  uint32_t* const cnt = s.cnt;
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) cnt[k] = 0;
  s.t->n = 0;
  v.present = 0; cv.present = 0;
  if (fast_ws(w, f) != '{' || f.p >= limit) return false;
  f.p++;
  fast_ws(w, f);
  uint32_t type;
  if constexpr (SCHEMA != PJ_SCHEMA_MIXED) {
    constexpr int OBJ = RootOf<SCHEMA>::obj;
    if (!fast_root<OBJ>(w, f, s, v, cv, -1)) return false;
    if ((v.present & CObj<OBJ>::required) != (uint32_t)CObj<OBJ>::required) return fast_fail(f, PJ_E_REQUIRED, f.p - 1);
    type = SCHEMA;
  } else {
    /* only the common `id` may precede the deciding key on this path */
    bool have_id = false;
    int64_t early_id = 0;
    for (;;) {
      if (wbyte(w, f.p) != '"') return false;
      uint32_t len; uint64_t lo, hi;
      if (!fast_short(w, f, &len, &lo, &hi) || !fast_colon(w, f)) return false;
      const int kp = match_key<OBJ_PET>(len, lo, hi), ko = match_key<OBJ_ORDER>(len, lo, hi), ku = match_key<OBJ_USER>(len, lo, hi);
      const int owners = (kp >= 0) + (ko >= 0) + (ku >= 0);
      if (owners == 3) {
        if (have_id) return false;
        const uint32_t x = wbyte(w, f.p);
        if (!(x == '-' || x - '0' <= 9u)) return fast_wrong_type(f, x);
        if (!fast_int(w, f, true, &early_id)) return false;
        have_id = true;
        if (fast_member_end(w, f) != 1) return false;
        continue;
      }
      if (owners != 1) return false; /* unknown key, or `status` before the deciding key */
      if (have_id) { v.v[0] = early_id; v.present = 1; }
      if (kp >= 0) {
        type = PJ_TYPE_PET;
        if (!fast_root<OBJ_PET>(w, f, s, v, cv, kp)) return false;
        if ((v.present & CObj<OBJ_PET>::required) != (uint32_t)CObj<OBJ_PET>::required) return fast_fail(f, PJ_E_REQUIRED, f.p - 1);
      } else if (ko >= 0) {
        type = PJ_TYPE_ORDER;
        if (!fast_root<OBJ_ORDER>(w, f, s, v, cv, ko)) return false;
      } else {
        type = PJ_TYPE_USER;
        if (!fast_root<OBJ_USER>(w, f, s, v, cv, ku)) return false;
      }
      break;
    }
  }
  const uint32_t x = fast_ws(w, f);
  if (f.p > limit) return false;
  if (f.p < limit) { if (lf_ws || x != '\n') return false; }
  else if (open_end) return false;
  if constexpr (SCHEMA == PJ_SCHEMA_MIXED) {
    if (type == PJ_TYPE_PET) cnt[SLOT_ROWS_PET] = 1; else if (type == PJ_TYPE_ORDER) cnt[SLOT_ROWS_ORD] = 1; else cnt[SLOT_ROWS_USR] = 1;
  }
  *type_out = type;
  return true;
}

/* ---- emission -------------------------------------------------------------------------------------- */
/* Fixed-width values, string offsets and list offsets of one object at `row`. ELEM: the object is a
 * list element, whose string offsets are stored by store_elem_str_offsets. */
template <int OBJ, bool ELEM, int I = 0>
PJ_COLD void store_vals(const DevCols* c, const FVals& v, uint64_t row, const uint32_t* base) {
  if constexpr (I == 0) colp<uint8_t>(c, CObj<OBJ>::present_col)[row] = (uint8_t)v.present;
  if constexpr (I < CObj<OBJ>::N) {
    constexpr uint32_t kind = FK<OBJ, I>::kind, col = FK<OBJ, I>::col, cnt = FK<OBJ, I>::cnt;
    const bool pr = (v.present >> I) & 1;
    if constexpr (kind == K_I64) colp<int64_t>(c, col)[row] = pr ? v.v[I] : 0;
    else if constexpr (kind == K_I32) colp<int32_t>(c, col)[row] = pr ? (int32_t)v.v[I] : 0;
    else if constexpr (kind == K_BOOL) colp<uint8_t>(c, col)[row] = pr ? (uint8_t)v.v[I] : 0;
    else if constexpr (kind == K_ENUM) colp<uint8_t>(c, col)[row] = pr ? (uint8_t)v.v[I] : 255;
    else if constexpr (kind == K_STR) { if constexpr (!ELEM) colp<uint32_t>(c, col)[row] = base[cnt]; }
    else if constexpr (kind == K_DATETIME) {
      colp<int64_t>(c, col)[row] = pr ? v.v[I] : 0;
      colp<int32_t>(c, col + 1)[row] = pr ? (int32_t)((uint64_t)v.aux >> 32) : 0;
      colp<int32_t>(c, col + 2)[row] = pr ? (int32_t)(uint32_t)v.aux : 0;
    }
    else if constexpr (kind == K_LIST_STR || kind == K_LIST_OBJ) colp<uint32_t>(c, col)[row] = base[cnt];
    store_vals<OBJ, ELEM, I + 1>(c, v, row, base);
  }
}
/* offsets of the strings of a list element = the cursors as they stand before its strings are copied */
template <int OBJ, int I = 0>
PJ_HD void store_elem_str_offsets(const DevCols* c, uint64_t row, const uint32_t* base, const uint32_t* cur) {
  if constexpr (I < CObj<OBJ>::N) {
    if constexpr (FK<OBJ, I>::kind == K_STR) colp<uint32_t>(c, FK<OBJ, I>::col)[row] = base[FK<OBJ, I>::cnt] + cur[FK<OBJ, I>::cnt];
    store_elem_str_offsets<OBJ, I + 1>(c, row, base, cur);
  }
}
template <int OBJ, int I = 0>
PJ_HD void tape_get_scalars(const Tape& t, uint32_t at, FVals& v) {
  if constexpr (I < CObj<OBJ>::N) {
    if constexpr (FK<OBJ, I>::kind != K_STR) {
      v.v[I] = (int64_t)((uint64_t)tape_get(t, at) | ((uint64_t)tape_get(t, at + 1) << 32));
      tape_get_scalars<OBJ, I + 1>(t, at + 2, v);
    } else tape_get_scalars<OBJ, I + 1>(t, at, v);
  }
}
/* a string word that belongs to a flat object CH (embedded object or list element): copy it to its arena */
template <int CH, int I = 0>
PJ_HD bool replay_flat_string(const Win& w, const DevCols* c, uint32_t word, const uint32_t* base, uint32_t* cur) {
  if constexpr (I >= CObj<CH>::N) return false;
  else {
    if constexpr (FK<CH, I>::kind == K_STR) {
      constexpr uint32_t cnt = FK<CH, I>::cnt;
      if ((word & 15u) == cnt) { copy_tape_str(colp<uint8_t>(c, FK<CH, I>::col + 1) + base[cnt] + cur[cnt], w, word); cur[cnt] += (word >> 4) & 0x7FFu; return true; }
    }
    return replay_flat_string<CH, I + 1>(w, c, word, base, cur);
  }
}

/* One tape word of a record whose root is OBJ (k = its index; returns the index of the next word): finds
 * the property it belongs to by an unrolled chain over the properties and emits it. cur[] holds, per slot,
 * the bytes (byte slots) or items (item slots) emitted so far. */
template <int OBJ, int I>
PJ_COLD uint32_t replay_word(const Win& w, const DevCols* c, const Tape& t, uint32_t k, uint32_t word, const uint32_t* base, uint32_t* cur) {
  if constexpr (I >= CObj<OBJ>::N) return k + 1;
  else {
    constexpr uint32_t kind = FK<OBJ, I>::kind, col = FK<OBJ, I>::col, cnt = FK<OBJ, I>::cnt;
    const uint32_t slot = word & 15u, len = (word >> 4) & 0x7FFu;
    if constexpr (kind == K_STR) {
      if (slot == cnt) { copy_tape_str(colp<uint8_t>(c, col + 1) + base[cnt] + cur[cnt], w, word); cur[cnt] += len; return k + 1; }
    } else if constexpr (kind == K_LIST_STR) {
      if (slot == cnt + 1) {
        colp<uint32_t>(c, col + 1)[(uint64_t)base[cnt] + cur[cnt]] = base[cnt + 1] + cur[cnt + 1];
        copy_tape_str(colp<uint8_t>(c, col + 2) + base[cnt + 1] + cur[cnt + 1], w, word);
        cur[cnt + 1] += len; cur[cnt] += 1;
        return k + 1;
      }
    } else if constexpr (kind == K_OBJ) {
      if (replay_flat_string<FK<OBJ, I>::child>(w, c, word, base, cur)) return k + 1;
    } else if constexpr (kind == K_LIST_OBJ) {
      constexpr int E = FK<OBJ, I>::child;
      if (slot == TAPE_ELEM && (word >> 12 & 15u) == cnt) {
        const uint64_t erow = (uint64_t)base[cnt] + cur[cnt];
        cur[cnt] += 1;
        store_elem_str_offsets<E>(c, erow, base, cur);
        FVals ev;
        ev.present = (word >> 4) & 0xFFu;
        tape_get_scalars<E>(t, k + 1, ev);
        store_vals<E, true>(c, ev, erow, base);
        return k + 1 + scalar_words<E>();
      }
      if (slot != TAPE_ELEM && replay_flat_string<E>(w, c, word, base, cur)) return k + 1;
    }
    return replay_word<OBJ, I + 1>(w, c, t, k, word, base, cur);
  }
}

/* columns of the embedded object of OBJ (if it has one) at the root's row */
template <int OBJ, int I = 0>
PJ_HD void store_embedded(const DevCols* c, const FVals& v, const FVals& cv, uint64_t row, const uint32_t* base) {
  if constexpr (I < CObj<OBJ>::N) {
    if constexpr (FK<OBJ, I>::kind == K_OBJ) {
      FVals z = cv;
      if (!((v.present >> I) & 1)) z.present = 0;
      store_vals<FK<OBJ, I>::child, false>(c, z, row, base);
    }
    store_embedded<OBJ, I + 1>(c, v, cv, row, base);
  }
}

/* cur[]: bytes / items of the record already emitted per slot (zeros, unless the tape was emptied on the way) */
template <int OBJ>
PJ_COLD void emit_root(const Win& w, const DevCols* c, const FVals& v, const FVals& cv, const Tape& t, uint64_t row, const uint32_t* base, uint32_t* cur) {
  store_vals<OBJ, false>(c, v, row, base);
  store_embedded<OBJ>(c, v, cv, row, base);
  for (uint32_t k = 0; k < t.n;) k = replay_word<OBJ>(w, c, t, k, tape_get(t, k), base, cur);
}
template <int SCHEMA>
PJ_HD void emit_typed(const Win& w, const DevCols* c, uint32_t type, const FVals& v, const FVals& cv, const Tape& t, const uint32_t* base,
                      uint64_t rec_index, uint32_t* cur) {
  if constexpr (SCHEMA != PJ_SCHEMA_MIXED) emit_root<RootOf<SCHEMA>::obj>(w, c, v, cv, t, rec_index, base, cur);
  else {
    if (type == PJ_TYPE_PET) emit_root<OBJ_PET>(w, c, v, cv, t, base[SLOT_ROWS_PET], base, cur);
    else if (type == PJ_TYPE_ORDER) emit_root<OBJ_ORDER>(w, c, v, cv, t, base[SLOT_ROWS_ORD], base, cur);
    else emit_root<OBJ_USER>(w, c, v, cv, t, base[SLOT_ROWS_USR], base, cur);
  }
}

/* Replays a record accepted by fast_record<SCHEMA>() whose strings and list elements all fit the tape (t.n <= t.cap):
 * every column of its row, then the tape. base[slot] = the record's start in every arena / child table. */
template <int SCHEMA>
PJ_HD void fast_emit(const Win& w, const DevCols* c, uint32_t type, const FVals& v, const FVals& cv, const Tape& t, const uint32_t* base,
                     uint64_t rec_index) {
  uint32_t cur[NSLOT];
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) cur[k] = 0;
  emit_typed<SCHEMA>(w, c, type, v, cv, t, base, rec_index, cur);
}
/* The out-of-line form of the tokeniser, for the records the inlined first pass does not finish alone:
 *  - c != null: emits a record that fast_record<SCHEMA>() (or a counting call of this function) accepted and whose
 *    strings and list elements outnumber the tape: it is tokenised again, and this time the tape (at least
 *    TAPE_MIN_CAP words) is emptied into the columns whenever the next unit would not fit;
 *  - c == null: the counting pass for a record that is read where it lies instead of from the staged window (w then
 *    points into global memory): verdict as fast_record<>(), counts in cnt_out[NSLOT], nothing is kept on the tape.
 * Arguments are passed by value so that the caller's copies stay in registers. */
template <int SCHEMA>
PJ_HD_NOINLINE uint32_t fast_outline(const Win w, uint32_t start, uint32_t limit, uint32_t lf_ws, uint32_t open_end, const DevCols* c,
                                     const uint32_t* base, uint64_t rec_index, Tape t, uint32_t* cnt_out, uint32_t* type_out,
                                     uint32_t* err_kind, uint32_t* err_pos) {
  FastState f;
  f.p = start; f.limit = limit; f.lf_ws = lf_ws; f.err = 0; f.err_pos = 0;
  DrainState d;
  d.c = c; d.base = base;
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) d.cur[k] = 0;
  FVals v, cv;
  uint32_t cnt[NSLOT], type = PJ_TYPE_NONE;
  if (!fast_record_body<SCHEMA, true>(w, f, open_end, &type, v, cv, cnt, t, &d)) {
    if (!f.err) return FAST_REFUSED;
    *err_kind = f.err; *err_pos = f.err_pos;
    return FAST_FAILED;
  }
  if (c) emit_typed<SCHEMA>(w, c, type, v, cv, t, base, rec_index, d.cur);
  else {
    for (uint32_t k = 0; k < NSLOT; ++k) cnt_out[k] = cnt[k];
    *type_out = type;
  }
  return FAST_ACCEPTED;
}

}  // namespace pj
#endif
