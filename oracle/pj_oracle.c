/*
 * pj_oracle.c — TEST INFRASTRUCTURE, not part of the product.
 *
 * A scalar CPU restatement of the JSON parse / validate / re-serialise path that
 * altro3/micronaut3-bug reaches through io.micronaut.serde.ObjectMapper
 * (src/main/java/com/micronaut/bug/config/MyEntityConfig.java:34 readValue;
 *  src/main/java/com/micronaut/bug/service/MyEntityService.java:45 getDefault;
 *  src/main/java/com/micronaut/bug/controller/MyEntityController.java:48-51 response encoding)
 * for the models of petstore.json:823-972, under the strict parser configuration of
 * src/main/resources/application.yml:23-28.
 *
 * PARITY UNPINNED: the arithmetic of that path lives in third-party libraries that are not part of
 * the reference tree and cannot run where this is built or tested (no JVM):
 *   io.micronaut.serde:micronaut-serde-jackson 2.15.1 and micronaut-serde-processor 2.15.1
 *     (build.gradle:14,89,104), jackson-core at the version managed by io.micronaut.platform 4.10.0
 *     (build.gradle:11,23), io.micronaut.validation:micronaut-validation (build.gradle:98),
 *     model shape from the io.micronaut.openapi plugin 4.6.0 / micronaut-openapi 6.19.1
 *     (build.gradle:4,13,44).
 * The reference holds no test, golden vector or fixture for this path (its only test is
 * src/test/java/com/micronaut/bug/controller/CookieTest.java:28-73, about cookies). This file
 * therefore restates RFC 8259 / RFC 3629 / RFC 3339 and the schemas, with every choice those leave
 * open written down as rules R1-R12 / W1-W5 in include/petjson.h; it is cross-checked in the tests
 * against Python's json, msgspec and jsonschema and against hand-written known-answer cases.
 *
 * Only the tests, the smoke check and the benchmark's CPU-baseline leg may call this code. The
 * product library never links or loads it.
 *
 * Method: one recursive-descent pass per record, byte at a time, every string decoded into a
 * temporary buffer, values collected in a per-record struct and appended to the columns when the
 * record has been accepted. Deliberately shares no code with the CUDA kernels.
 */
#include <stdlib.h>
#include <string.h>

#include "petjson.h"

/* ------------------------------------------------------------------------------------------ */
/* small growable byte buffer                                                                  */
/* ------------------------------------------------------------------------------------------ */
typedef struct { uint8_t* b; size_t n, cap; } sbuf;
static void sb_put(sbuf* s, uint8_t c) {
  if (s->n == s->cap) { s->cap = s->cap ? s->cap * 2 : 64; s->b = (uint8_t*)realloc(s->b, s->cap); }
  s->b[s->n++] = c;
}
static void sb_free(sbuf* s) { free(s->b); s->b = NULL; s->n = s->cap = 0; }
static int sb_eq(const sbuf* s, const char* lit) { size_t n = strlen(lit); return s->n == n && memcmp(s->b, lit, n) == 0; }

/* ------------------------------------------------------------------------------------------ */
/* cursor over one record extent                                                               */
/* ------------------------------------------------------------------------------------------ */
typedef struct {
  const uint8_t* b; /* whole input */
  uint64_t s, e, p; /* extent [s, e), position */
  int lf_ws;        /* LF counts as whitespace (array framing) */
  int open_end;     /* extent end not observed (ran out of shard slack): reaching e is TOO_LONG */
  int err; uint64_t err_pos;
  uint32_t opts;    /* PJ_OPT_* bits that select the other answer of a rule */
} cur;

static int fail(cur* c, int kind, uint64_t pos) {
  if (!c->err) { c->err = kind; c->err_pos = pos; }
  return 0;
}
static int fail_end(cur* c) { return fail(c, c->open_end ? PJ_E_TOO_LONG : PJ_E_EOF, c->e); }
static int is_ws(const cur* c, uint8_t x) { return x == ' ' || x == '\t' || x == '\r' || (c->lf_ws && x == '\n'); }
static void skip_ws(cur* c) { while (c->p < c->e && is_ws(c, c->b[c->p])) c->p++; }
static int is_value_start(uint8_t x) {
  return x == '"' || x == '-' || (x >= '0' && x <= '9') || x == '{' || x == '[' || x == 't' || x == 'f' || x == 'n';
}
/* R5: wrong first byte for the expected type */
static int fail_first_byte(cur* c) {
  if (c->p >= c->e) return fail_end(c);
  return fail(c, is_value_start(c->b[c->p]) ? PJ_E_TYPE : PJ_E_SYNTAX, c->p);
}
/* expects byte x at p (after whitespace) */
static int expect(cur* c, uint8_t x) {
  skip_ws(c);
  if (c->p >= c->e) return fail_end(c);
  if (c->b[c->p] != x) return fail(c, PJ_E_SYNTAX, c->p);
  c->p++;
  return 1;
}

static int hexval(uint8_t x) {
  if (x >= '0' && x <= '9') return x - '0';
  if (x >= 'a' && x <= 'f') return x - 'a' + 10;
  if (x >= 'A' && x <= 'F') return x - 'A' + 10;
  return -1;
}
static void put_utf8(sbuf* o, uint32_t cp) {
  if (!o) return;
  if (cp < 0x80) sb_put(o, (uint8_t)cp);
  else if (cp < 0x800) { sb_put(o, 0xC0 | (cp >> 6)); sb_put(o, 0x80 | (cp & 63)); }
  else if (cp < 0x10000) { sb_put(o, 0xE0 | (cp >> 12)); sb_put(o, 0x80 | ((cp >> 6) & 63)); sb_put(o, 0x80 | (cp & 63)); }
  else { sb_put(o, 0xF0 | (cp >> 18)); sb_put(o, 0x80 | ((cp >> 12) & 63)); sb_put(o, 0x80 | ((cp >> 6) & 63)); sb_put(o, 0x80 | (cp & 63)); }
}
/* reads 4 hex digits at p */
static int hex4(cur* c, uint32_t* out) {
  uint32_t v = 0;
  for (int i = 0; i < 4; ++i) {
    if (c->p >= c->e) return fail_end(c);
    int h = hexval(c->b[c->p]);
    if (h < 0) return fail(c, PJ_E_BAD_ESCAPE, c->p);
    v = v << 4 | (uint32_t)h;
    c->p++;
  }
  *out = v;
  return 1;
}

/* R7. p is at the opening quote; decoded bytes go to o (may be NULL). */
static int lex_string(cur* c, sbuf* o) {
  if (o) o->n = 0;
  c->p++; /* opening quote */
  for (;;) {
    if (c->p >= c->e) return fail_end(c);
    uint8_t x = c->b[c->p];
    if (x == '"') { c->p++; return 1; }
    if (x < 0x20) return fail(c, PJ_E_CTRL_CHAR, c->p);
    if (x == '\\') {
      uint64_t bs = c->p;
      c->p++;
      if (c->p >= c->e) return fail_end(c);
      uint8_t y = c->b[c->p];
      uint32_t cp;
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
          c->p++;
          if (!hex4(c, &cp)) return 0;
          if (c->opts & PJ_OPT_LONE_SURROGATE_REPLACE) {
            /* a high surrogate takes the low one that follows it at once; whatever is left alone becomes U+FFFD */
            if (cp >= 0xD800 && cp <= 0xDBFF && c->p + 1 < c->e && c->b[c->p] == '\\' && c->b[c->p + 1] == 'u') {
              uint64_t keep = c->p;
              uint32_t lo;
              c->p += 2;
              if (!hex4(c, &lo)) return 0;
              if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
              else c->p = keep; /* not its partner: read again as an escape of its own */
            }
            if (cp >= 0xD800 && cp <= 0xDFFF) cp = 0xFFFD;
            put_utf8(o, cp);
            continue;
          }
          if (cp >= 0xDC00 && cp <= 0xDFFF) return fail(c, PJ_E_BAD_SURROGATE, bs);
          if (cp >= 0xD800 && cp <= 0xDBFF) {
            if (c->p >= c->e) return fail_end(c);
            if (c->b[c->p] != '\\') return fail(c, PJ_E_BAD_SURROGATE, bs);
            c->p++;
            if (c->p >= c->e) return fail_end(c);
            if (c->b[c->p] != 'u') return fail(c, PJ_E_BAD_SURROGATE, bs);
            c->p++;
            uint32_t lo;
            if (!hex4(c, &lo)) return 0;
            if (lo < 0xDC00 || lo > 0xDFFF) return fail(c, PJ_E_BAD_SURROGATE, bs);
            cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          put_utf8(o, cp);
          continue;
        }
        default: return fail(c, PJ_E_BAD_ESCAPE, c->p);
      }
      c->p++;
      put_utf8(o, cp);
      continue;
    }
    if (x < 0x80) { if (o) sb_put(o, x); c->p++; continue; }
    /* RFC 3629 well-formedness */
    uint64_t lead = c->p;
    uint32_t need; uint8_t lo = 0x80, hi = 0xBF;
    if (x >= 0xC2 && x <= 0xDF) need = 1;
    else if (x == 0xE0) { need = 2; lo = 0xA0; }
    else if ((x >= 0xE1 && x <= 0xEC) || x == 0xEE || x == 0xEF) need = 2;
    else if (x == 0xED) { need = 2; hi = 0x9F; }
    else if (x == 0xF0) { need = 3; lo = 0x90; }
    else if (x >= 0xF1 && x <= 0xF3) need = 3;
    else if (x == 0xF4) { need = 3; hi = 0x8F; }
    else return fail(c, PJ_E_UTF8, lead);
    for (uint32_t k = 1; k <= need; ++k) {
      if (lead + k >= c->e) { c->p = c->e; return fail_end(c); }
      uint8_t y = c->b[lead + k];
      if (y < lo || y > hi) return fail(c, PJ_E_UTF8, lead);
      lo = 0x80; hi = 0xBF;
    }
    if (o) for (uint32_t k = 0; k <= need; ++k) sb_put(o, c->b[lead + k]);
    c->p = lead + need + 1;
  }
}

/* R6. p at '-' or a digit. */
typedef struct { int neg, is_int, overflow; uint64_t mag; uint64_t start; } num;
static int lex_number(cur* c, num* r) {
  r->start = c->p; r->neg = 0; r->is_int = 1; r->overflow = 0; r->mag = 0;
  if (c->b[c->p] == '-') { r->neg = 1; c->p++; }
  if (c->p >= c->e) return fail_end(c);
  uint8_t x = c->b[c->p];
  if (x < '0' || x > '9') return fail(c, PJ_E_SYNTAX, c->p);
  if (x == '0') {
    c->p++;
    if (c->p < c->e && c->b[c->p] >= '0' && c->b[c->p] <= '9') return fail(c, PJ_E_SYNTAX, c->p);
  } else {
    while (c->p < c->e && c->b[c->p] >= '0' && c->b[c->p] <= '9') {
      uint64_t d = c->b[c->p] - '0';
      if (r->mag > (0xFFFFFFFFFFFFFFFFull - d) / 10) r->overflow = 1; else r->mag = r->mag * 10 + d;
      c->p++;
    }
  }
  if (c->p < c->e && c->b[c->p] == '.') {
    r->is_int = 0; c->p++;
    if (c->p >= c->e) return fail_end(c);
    if (c->b[c->p] < '0' || c->b[c->p] > '9') return fail(c, PJ_E_SYNTAX, c->p);
    while (c->p < c->e && c->b[c->p] >= '0' && c->b[c->p] <= '9') c->p++;
  }
  if (c->p < c->e && (c->b[c->p] == 'e' || c->b[c->p] == 'E')) {
    r->is_int = 0; c->p++;
    if (c->p < c->e && (c->b[c->p] == '+' || c->b[c->p] == '-')) c->p++;
    if (c->p >= c->e) return fail_end(c);
    if (c->b[c->p] < '0' || c->b[c->p] > '9') return fail(c, PJ_E_SYNTAX, c->p);
    while (c->p < c->e && c->b[c->p] >= '0' && c->b[c->p] <= '9') c->p++;
  }
  return 1;
}
static int lex_literal(cur* c, const char* lit) {
  for (; *lit; ++lit) {
    if (c->p >= c->e) return fail_end(c);
    if (c->b[c->p] != (uint8_t)*lit) return fail(c, PJ_E_SYNTAX, c->p);
    c->p++;
  }
  return 1;
}

/* R4: any JSON value, validated and discarded. depth = brackets already open inside the skipped value. */
static int skip_value(cur* c, int depth) {
  skip_ws(c);
  if (c->p >= c->e) return fail_end(c);
  uint8_t x = c->b[c->p];
  if (x == '"') return lex_string(c, NULL);
  if (x == '-' || (x >= '0' && x <= '9')) { num r; return lex_number(c, &r); }
  if (x == 't') return lex_literal(c, "true");
  if (x == 'f') return lex_literal(c, "false");
  if (x == 'n') return lex_literal(c, "null");
  if (x == '[') {
    if (depth >= 64) return fail(c, PJ_E_DEPTH, c->p);
    c->p++;
    skip_ws(c);
    if (c->p < c->e && c->b[c->p] == ']') { c->p++; return 1; }
    for (;;) {
      if (!skip_value(c, depth + 1)) return 0;
      skip_ws(c);
      if (c->p >= c->e) return fail_end(c);
      if (c->b[c->p] == ',') { c->p++; continue; }
      if (c->b[c->p] == ']') { c->p++; return 1; }
      return fail(c, PJ_E_SYNTAX, c->p);
    }
  }
  if (x == '{') {
    if (depth >= 64) return fail(c, PJ_E_DEPTH, c->p);
    c->p++;
    skip_ws(c);
    if (c->p < c->e && c->b[c->p] == '}') { c->p++; return 1; }
    for (;;) {
      skip_ws(c);
      if (c->p >= c->e) return fail_end(c);
      if (c->b[c->p] != '"') return fail(c, PJ_E_SYNTAX, c->p);
      if (!lex_string(c, NULL)) return 0;
      if (!expect(c, ':')) return 0;
      if (!skip_value(c, depth + 1)) return 0;
      skip_ws(c);
      if (c->p >= c->e) return fail_end(c);
      if (c->b[c->p] == ',') { c->p++; continue; }
      if (c->b[c->p] == '}') { c->p++; return 1; }
      return fail(c, PJ_E_SYNTAX, c->p);
    }
  }
  return fail(c, PJ_E_SYNTAX, c->p);
}

/* ---- typed scalar readers; each returns 0 on failure, 1 on a value, 2 on null ---------------- */
static int at_null(cur* c) {
  if (c->p < c->e && c->b[c->p] == 'n') return 1;
  return 0;
}
static int read_int(cur* c, int bits, int64_t* out) {
  skip_ws(c);
  if (c->p >= c->e) return fail_end(c);
  if (at_null(c)) return lex_literal(c, "null") ? 2 : 0;
  uint8_t x = c->b[c->p];
  if (x == '"' && (c->opts & PJ_OPT_COERCE_SCALARS)) {
    /* a string that holds an integer: -?(0|[1-9][0-9]*), nothing else */
    uint64_t q = c->p;
    sbuf t; memset(&t, 0, sizeof t);
    if (!lex_string(c, &t)) { sb_free(&t); return 0; }
    size_t i = 0, n = t.n;
    int neg = n && t.b[0] == '-';
    if (neg) i = 1;
    int ok = i < n && !(t.b[i] == '0' && i + 1 < n);
    uint64_t mag = 0; int over = 0;
    for (; ok && i < n; ++i) {
      if (t.b[i] < '0' || t.b[i] > '9') { ok = 0; break; }
      uint64_t d = (uint64_t)(t.b[i] - '0');
      if (mag > (0xFFFFFFFFFFFFFFFFull - d) / 10) over = 1; else mag = mag * 10 + d;
    }
    sb_free(&t);
    if (!ok) return fail(c, PJ_E_TYPE, q);
    uint64_t lim = bits == 64 ? (neg ? 0x8000000000000000ull : 0x7FFFFFFFFFFFFFFFull) : (neg ? 0x80000000ull : 0x7FFFFFFFull);
    if (over || mag > lim) return fail(c, PJ_E_NUM_RANGE, q);
    *out = neg ? (int64_t)(0 - mag) : (int64_t)mag;
    return 1;
  }
  if (!(x == '-' || (x >= '0' && x <= '9'))) return fail_first_byte(c);
  num r;
  if (!lex_number(c, &r)) return 0;
  if (!r.is_int) return fail(c, PJ_E_TYPE, r.start);
  uint64_t lim = bits == 64 ? (r.neg ? 0x8000000000000000ull : 0x7FFFFFFFFFFFFFFFull)
                            : (r.neg ? 0x80000000ull : 0x7FFFFFFFull);
  if (r.overflow || r.mag > lim) return fail(c, PJ_E_NUM_RANGE, r.start);
  *out = r.neg ? (int64_t)(0 - r.mag) : (int64_t)r.mag;
  return 1;
}
static int read_bool(cur* c, uint8_t* out) {
  skip_ws(c);
  if (c->p >= c->e) return fail_end(c);
  if (at_null(c)) return lex_literal(c, "null") ? 2 : 0;
  if (c->b[c->p] == 't') { *out = 1; return lex_literal(c, "true"); }
  if (c->b[c->p] == 'f') { *out = 0; return lex_literal(c, "false"); }
  if (c->b[c->p] == '"' && (c->opts & PJ_OPT_COERCE_SCALARS)) {
    uint64_t q = c->p;
    sbuf t; memset(&t, 0, sizeof t);
    if (!lex_string(c, &t)) { sb_free(&t); return 0; }
    int v = sb_eq(&t, "true") ? 1 : (sb_eq(&t, "false") ? 0 : -1);
    sb_free(&t);
    if (v < 0) return fail(c, PJ_E_TYPE, q);
    *out = (uint8_t)v;
    return 1;
  }
  return fail_first_byte(c);
}
static int read_str(cur* c, sbuf* o, uint64_t* quote_pos) {
  skip_ws(c);
  if (c->p >= c->e) return fail_end(c);
  if (at_null(c)) return lex_literal(c, "null") ? 2 : 0;
  if (c->b[c->p] != '"') {
    /* a plain string property (the callers that ask for no quote position; enums and date-times do ask) also takes a
       number, true or false under PJ_OPT_COERCE_SCALARS: the token's text, as written, becomes the string */
    uint8_t x = c->b[c->p];
    if (!quote_pos && (c->opts & PJ_OPT_COERCE_SCALARS) && (x == '-' || (x >= '0' && x <= '9') || x == 't' || x == 'f')) {
      uint64_t t0 = c->p;
      if (x == 't') { if (!lex_literal(c, "true")) return 0; }
      else if (x == 'f') { if (!lex_literal(c, "false")) return 0; }
      else { num r; if (!lex_number(c, &r)) return 0; }
      if (o) { o->n = 0; for (uint64_t q = t0; q < c->p; ++q) sb_put(o, c->b[q]); }
      return 1;
    }
    return fail_first_byte(c);
  }
  if (quote_pos) *quote_pos = c->p;
  return lex_string(c, o);
}
static int enum_index(const sbuf* s, const char* const* lits, int n) {
  for (int i = 0; i < n; ++i) if (sb_eq(s, lits[i])) return i;
  return -1;
}
static const char* const PET_STATUS[3] = {"available", "pending", "sold"};   /* petstore.json:912-916 */
static const char* const ORD_STATUS[3] = {"placed", "approved", "delivered"}; /* petstore.json:958-962 */

static int64_t days_from_civil(int64_t y, unsigned m, unsigned d) {
  y -= m <= 2;
  int64_t era = (y >= 0 ? y : y - 399) / 400;
  unsigned yoe = (unsigned)(y - era * 400);
  unsigned doy = (153 * (m + (m > 2 ? -3 : 9)) + 2) / 5 + d - 1;
  unsigned doe = yoe * 365 + yoe / 4 - yoe / 100 + doy;
  return era * 146097 + (int64_t)doe - 719468;
}
static void civil_from_days(int64_t z, int64_t* y, unsigned* m, unsigned* d) {
  z += 719468;
  int64_t era = (z >= 0 ? z : z - 146096) / 146097;
  unsigned doe = (unsigned)(z - era * 146097);
  unsigned yoe = (doe - doe / 1460 + doe / 36524 - doe / 146096) / 365;
  int64_t yy = (int64_t)yoe + era * 400;
  unsigned doy = doe - (365 * yoe + yoe / 4 - yoe / 100);
  unsigned mp = (5 * doy + 2) / 153;
  *d = doy - (153 * mp + 2) / 5 + 1;
  *m = mp < 10 ? mp + 3 : mp - 9;
  *y = yy + (*m <= 2);
}
/* R9 on the decoded text */
static int parse_datetime(const sbuf* s, int64_t* epoch, int32_t* nanos, int32_t* off) {
  const uint8_t* t = s->b; size_t n = s->n, i;
  if (n < 20) return 0;
#define DG(k) (t[k] >= '0' && t[k] <= '9')
#define D2(k) ((unsigned)((t[k] - '0') * 10 + (t[(k) + 1] - '0')))
  for (i = 0; i < 19; ++i) {
    if (i == 4 || i == 7) { if (t[i] != '-') return 0; }
    else if (i == 10) { if (t[i] != 'T') return 0; }
    else if (i == 13 || i == 16) { if (t[i] != ':') return 0; }
    else if (!DG(i)) return 0;
  }
  unsigned year = D2(0) * 100 + D2(2), mon = D2(5), day = D2(8), hh = D2(11), mi = D2(14), ss = D2(17);
  static const unsigned mdays[12] = {31, 28, 31, 30, 31, 30, 31, 31, 30, 31, 30, 31};
  if (mon < 1 || mon > 12 || day < 1) return 0;
  unsigned dim = mdays[mon - 1];
  if (mon == 2 && (year % 4 == 0 && (year % 100 != 0 || year % 400 == 0))) dim = 29;
  if (day > dim || hh > 23 || mi > 59 || ss > 59) return 0;
  i = 19;
  uint32_t ns = 0;
  if (t[i] == '.') {
    size_t k = 0;
    ++i;
    while (i < n && DG(i)) { if (k >= 9) return 0; ns = ns * 10 + (uint32_t)(t[i] - '0'); ++k; ++i; }
    if (k == 0) return 0;
    for (; k < 9; ++k) ns *= 10;
  }
  if (i >= n) return 0;
  int32_t o = 0;
  if (t[i] == 'Z') { if (i + 1 != n) return 0; }
  else if (t[i] == '+' || t[i] == '-') {
    if (i + 6 != n || !DG(i + 1) || !DG(i + 2) || t[i + 3] != ':' || !DG(i + 4) || !DG(i + 5)) return 0;
    unsigned oh = D2(i + 1), om = D2(i + 4);
    if (oh > 23 || om > 59) return 0;
    o = (int32_t)(oh * 3600 + om * 60);
    if (t[i] == '-') o = -o;
  } else return 0;
#undef DG
#undef D2
  *epoch = days_from_civil(year, mon, day) * 86400 + (int64_t)hh * 3600 + mi * 60 + ss - o;
  *nanos = (int32_t)ns; *off = o;
  return 1;
}

/* ------------------------------------------------------------------------------------------ */
/* per-record value holders                                                                    */
/* ------------------------------------------------------------------------------------------ */
typedef struct { sbuf data; uint32_t* off; size_t n, cap; } strlist; /* n strings: off has n+1 entries */
static void sl_reset(strlist* l) { l->n = 0; l->data.n = 0; }
static void sl_push(strlist* l, const sbuf* s) {
  if (l->n + 2 > l->cap) { l->cap = l->cap ? l->cap * 2 : 16; l->off = (uint32_t*)realloc(l->off, l->cap * sizeof(uint32_t)); }
  if (l->n == 0) l->off[0] = 0;
  for (size_t i = 0; i < s->n; ++i) sb_put(&l->data, s->b[i]);
  l->off[++l->n] = (uint32_t)l->data.n;
}
static void sl_free(strlist* l) { sb_free(&l->data); free(l->off); memset(l, 0, sizeof *l); }

typedef struct { uint8_t present; int64_t id; } tagval;
typedef struct {
  uint32_t present;
  int64_t id;
  uint32_t cat_present; int64_t cat_id; sbuf cat_name;
  sbuf name;
  strlist photo;
  tagval* tags; size_t n_tags, cap_tags; strlist tag_names;
  int status;
} petval;
typedef struct {
  uint32_t present;
  int64_t id, pet_id, ship_epoch; int32_t quantity, ship_nanos, ship_off; int status; uint8_t complete;
} ordval;
typedef struct { uint32_t present; int64_t id; sbuf s[6]; int32_t user_status; } usrval;

typedef struct { petval pet; ordval ord; usrval usr; sbuf key, tmp; } scratch;

static void scratch_free(scratch* w) {
  sb_free(&w->pet.cat_name); sb_free(&w->pet.name); sl_free(&w->pet.photo); free(w->pet.tags); sl_free(&w->pet.tag_names);
  for (int i = 0; i < 6; ++i) sb_free(&w->usr.s[i]);
  sb_free(&w->key); sb_free(&w->tmp);
}

/* ---- object member loop helpers --------------------------------------------------------- */
/* After '{' was consumed: returns 1 with the next key decoded in w->key and p after ':',
 * 2 when the object closed (*close_pos = position of '}'), 0 on failure. `first` tells whether a
 * member was already read. */
static int next_member(cur* c, sbuf* key, int* first, uint64_t* close_pos) {
  skip_ws(c);
  if (c->p >= c->e) return fail_end(c);
  if (*first) {
    *first = 0;
    if (c->b[c->p] == '}') { *close_pos = c->p; c->p++; return 2; }
  } else {
    if (c->b[c->p] == '}') { *close_pos = c->p; c->p++; return 2; }
    if (c->b[c->p] != ',') return fail(c, PJ_E_SYNTAX, c->p);
    c->p++;
    skip_ws(c);
    if (c->p >= c->e) return fail_end(c);
  }
  if (c->b[c->p] != '"') return fail(c, PJ_E_SYNTAX, c->p);
  if (!lex_string(c, key)) return 0;
  if (!expect(c, ':')) return 0;
  skip_ws(c);
  return 1;
}

/* Category / Tag share the shape {id:int64, name:string} (petstore.json:858-871, 923-936).
 * p is at the value; returns 0 fail, 1 object read, 2 null. */
static int read_id_name(cur* c, scratch* w, uint32_t* present, int64_t* id, sbuf* name, int null_ok) {
  skip_ws(c);
  if (c->p >= c->e) return fail_end(c);
  if (at_null(c)) {
    if (!null_ok) return fail(c, PJ_E_TYPE, c->p);
    return lex_literal(c, "null") ? 2 : 0;
  }
  if (c->b[c->p] != '{') return fail_first_byte(c);
  c->p++;
  *present = 0; *id = 0; name->n = 0;
  int first = 1; uint64_t close_pos;
  for (;;) {
    int m = next_member(c, &w->key, &first, &close_pos);
    if (m == 0) return 0;
    if (m == 2) return 1;
    if (sb_eq(&w->key, "id")) {
      int r = read_int(c, 64, id);
      if (!r) return 0;
      if (r == 1) *present |= 1; else { *present &= ~1u; *id = 0; }
    } else if (sb_eq(&w->key, "name")) {
      int r = read_str(c, name, NULL);
      if (!r) return 0;
      if (r == 1) *present |= 2; else { *present &= ~2u; name->n = 0; }
    } else if (!skip_value(c, 0)) return 0;
  }
}

static void pet_reset(petval* v) {
  v->present = 0; v->id = 0; v->cat_present = 0; v->cat_id = 0; v->cat_name.n = 0; v->name.n = 0;
  sl_reset(&v->photo); v->n_tags = 0; sl_reset(&v->tag_names); v->status = 255;
}

/* value of a Pet property (p at the value). field: 0..5 in schema order. */
static int pet_field(cur* c, scratch* w, int field) {
  petval* v = &w->pet;
  int r;
  switch (field) {
    case 0:
      r = read_int(c, 64, &v->id); if (!r) return 0;
      if (r == 1) v->present |= 1; else { v->present &= ~1u; v->id = 0; }
      return 1;
    case 1:
      r = read_id_name(c, w, &v->cat_present, &v->cat_id, &v->cat_name, 1); if (!r) return 0;
      if (r == 1) v->present |= 2; else { v->present &= ~2u; v->cat_present = 0; v->cat_id = 0; v->cat_name.n = 0; }
      return 1;
    case 2:
      r = read_str(c, &v->name, NULL); if (!r) return 0;
      if (r == 1) v->present |= 4; else { v->present &= ~4u; v->name.n = 0; }
      return 1;
    case 3: case 4: {
      skip_ws(c);
      if (c->p >= c->e) return fail_end(c);
      uint32_t bit = field == 3 ? 8u : 16u;
      if (field == 3) sl_reset(&v->photo); else { v->n_tags = 0; sl_reset(&v->tag_names); }
      if (at_null(c)) { v->present &= ~bit; return lex_literal(c, "null"); }
      if (c->b[c->p] != '[') return fail_first_byte(c);
      c->p++;
      v->present |= bit;
      skip_ws(c);
      if (c->p < c->e && c->b[c->p] == ']') { c->p++; return 1; }
      for (;;) {
        skip_ws(c);
        if (c->p >= c->e) return fail_end(c);
        if (field == 3) {
          if (c->b[c->p] != '"') return fail_first_byte(c);
          if (!lex_string(c, &w->tmp)) return 0;
          sl_push(&v->photo, &w->tmp);
        } else {
          uint32_t pr; int64_t id;
          if (!read_id_name(c, w, &pr, &id, &w->tmp, 0)) return 0;
          if (v->n_tags == v->cap_tags) { v->cap_tags = v->cap_tags ? v->cap_tags * 2 : 8; v->tags = (tagval*)realloc(v->tags, v->cap_tags * sizeof(tagval)); }
          v->tags[v->n_tags].present = (uint8_t)pr; v->tags[v->n_tags].id = id; v->n_tags++;
          sl_push(&v->tag_names, &w->tmp);
        }
        skip_ws(c);
        if (c->p >= c->e) return fail_end(c);
        if (c->b[c->p] == ',') { c->p++; continue; }
        if (c->b[c->p] == ']') { c->p++; return 1; }
        return fail(c, PJ_E_SYNTAX, c->p);
      }
    }
    default: {
      uint64_t q = 0;
      r = read_str(c, &w->tmp, &q); if (!r) return 0;
      if (r == 2) { v->present &= ~32u; v->status = 255; return 1; }
      int k = enum_index(&w->tmp, PET_STATUS, 3);
      if (k < 0) {
        if (!(c->opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL)) return fail(c, PJ_E_ENUM, q);
        v->present &= ~32u; v->status = 255; /* unknown literal: the property stays absent */
        return 1;
      }
      v->present |= 32; v->status = k;
      return 1;
    }
  }
}
static int pet_key(const sbuf* k) {
  static const char* const names[6] = {"id", "category", "name", "photoUrls", "tags", "status"}; /* petstore.json:878-917 */
  for (int i = 0; i < 6; ++i) if (sb_eq(k, names[i])) return i;
  return -1;
}

static void ord_reset(ordval* v) { memset(v, 0, sizeof *v); v->status = 255; }
static int ord_key(const sbuf* k) {
  static const char* const names[6] = {"id", "petId", "quantity", "shipDate", "status", "complete"}; /* petstore.json:939-966 */
  for (int i = 0; i < 6; ++i) if (sb_eq(k, names[i])) return i;
  return -1;
}
static int ord_field(cur* c, scratch* w, int field) {
  ordval* v = &w->ord;
  int r; int64_t t;
  uint32_t bit = 1u << field;
  switch (field) {
    case 0: r = read_int(c, 64, &v->id); if (!r) return 0; if (r == 1) v->present |= bit; else { v->present &= ~bit; v->id = 0; } return 1;
    case 1: r = read_int(c, 64, &v->pet_id); if (!r) return 0; if (r == 1) v->present |= bit; else { v->present &= ~bit; v->pet_id = 0; } return 1;
    case 2: t = 0; r = read_int(c, 32, &t); if (!r) return 0; if (r == 1) { v->present |= bit; v->quantity = (int32_t)t; } else { v->present &= ~bit; v->quantity = 0; } return 1;
    case 3: {
      uint64_t q = 0;
      r = read_str(c, &w->tmp, &q); if (!r) return 0;
      if (r == 2) { v->present &= ~bit; v->ship_epoch = 0; v->ship_nanos = 0; v->ship_off = 0; return 1; }
      if (!parse_datetime(&w->tmp, &v->ship_epoch, &v->ship_nanos, &v->ship_off)) return fail(c, PJ_E_DATETIME, q);
      v->present |= bit;
      return 1;
    }
    case 4: {
      uint64_t q = 0;
      r = read_str(c, &w->tmp, &q); if (!r) return 0;
      if (r == 2) { v->present &= ~bit; v->status = 255; return 1; }
      int k = enum_index(&w->tmp, ORD_STATUS, 3);
      if (k < 0) {
        if (!(c->opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL)) return fail(c, PJ_E_ENUM, q);
        v->present &= ~bit; v->status = 255;
        return 1;
      }
      v->present |= bit; v->status = k;
      return 1;
    }
    default: r = read_bool(c, &v->complete); if (!r) return 0; if (r == 1) v->present |= bit; else { v->present &= ~bit; v->complete = 0; } return 1;
  }
}

static void usr_reset(usrval* v) { v->present = 0; v->id = 0; v->user_status = 0; for (int i = 0; i < 6; ++i) v->s[i].n = 0; }
static int usr_key(const sbuf* k) {
  static const char* const names[8] = {"id", "username", "firstName", "lastName", "email", "password", "phone", "userStatus"}; /* petstore.json:826-852 */
  for (int i = 0; i < 8; ++i) if (sb_eq(k, names[i])) return i;
  return -1;
}
static int usr_field(cur* c, scratch* w, int field) {
  usrval* v = &w->usr;
  int r; int64_t t;
  uint32_t bit = 1u << field;
  if (field == 0) { r = read_int(c, 64, &v->id); if (!r) return 0; if (r == 1) v->present |= bit; else { v->present &= ~bit; v->id = 0; } return 1; }
  if (field == 7) { t = 0; r = read_int(c, 32, &t); if (!r) return 0; if (r == 1) { v->present |= bit; v->user_status = (int32_t)t; } else { v->present &= ~bit; v->user_status = 0; } return 1; }
  r = read_str(c, &v->s[field - 1], NULL); if (!r) return 0;
  if (r == 1) v->present |= bit; else { v->present &= ~bit; v->s[field - 1].n = 0; }
  return 1;
}

/* Parses one record extent. `schema` fixes the model, or PJ_SCHEMA_MIXED infers it (R12).
 * Returns the model (PJ_TYPE_*) with values in w, or PJ_TYPE_NONE after a failure (c->err set). */
static int parse_record(cur* c, scratch* w, uint32_t schema) {
  int type = schema == PJ_SCHEMA_MIXED ? PJ_TYPE_NONE : (int)schema;
  pet_reset(&w->pet); ord_reset(&w->ord); usr_reset(&w->usr);
  /* values met before the model is known (R12) */
  int have_id = 0; int64_t early_id = 0;
  int have_status = 0; uint64_t status_q = 0; int status_pet = -1, status_ord = -1;
  skip_ws(c);
  if (c->p >= c->e) { fail_end(c); return PJ_TYPE_NONE; }
  if (c->b[c->p] != '{') { fail_first_byte(c); return PJ_TYPE_NONE; }
  c->p++;
  int first = 1; uint64_t close_pos = 0;
  for (;;) {
    int m = next_member(c, &w->key, &first, &close_pos);
    if (m == 0) return PJ_TYPE_NONE;
    if (m == 2) break;
    if (type == PJ_TYPE_NONE) {
      int kp = pet_key(&w->key), ko = ord_key(&w->key), ku = usr_key(&w->key);
      int owners = (kp >= 0) + (ko >= 0) + (ku >= 0);
      if (owners == 1) {
        type = kp >= 0 ? PJ_TYPE_PET : (ko >= 0 ? PJ_TYPE_ORDER : PJ_TYPE_USER);
        /* hand the early values to the model */
        if (have_id) {
          if (type == PJ_TYPE_PET) { w->pet.id = early_id; w->pet.present |= 1; }
          else if (type == PJ_TYPE_ORDER) { w->ord.id = early_id; w->ord.present |= 1; }
          else { w->usr.id = early_id; w->usr.present |= 1; }
        }
        if (have_status) {
          const int lenient = (c->opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL) != 0;
          if (type == PJ_TYPE_PET) {
            if (status_pet >= 0) { w->pet.status = status_pet; w->pet.present |= 32; }
            else if (!lenient) { fail(c, PJ_E_ENUM, status_q); return PJ_TYPE_NONE; }
          } else if (type == PJ_TYPE_ORDER) {
            if (status_ord >= 0) { w->ord.status = status_ord; w->ord.present |= 16; }
            else if (!lenient) { fail(c, PJ_E_ENUM, status_q); return PJ_TYPE_NONE; }
          }
          /* User has no `status`: the early value was an unknown key, already validated as a string */
        }
      } else if (owners == 3) { /* id */
        int r = read_int(c, 64, &early_id);
        if (!r) return PJ_TYPE_NONE;
        have_id = r == 1;
        continue;
      } else if (owners == 2) { /* status of Pet or Order */
        int r = read_str(c, &w->tmp, &status_q);
        if (!r) return PJ_TYPE_NONE;
        have_status = r == 1;
        if (have_status) {
          status_pet = enum_index(&w->tmp, PET_STATUS, 3);
          status_ord = enum_index(&w->tmp, ORD_STATUS, 3);
          if (status_pet < 0 && status_ord < 0 && !(c->opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL)) { fail(c, PJ_E_ENUM, status_q); return PJ_TYPE_NONE; }
        }
        continue;
      } else {
        if (!skip_value(c, 0)) return PJ_TYPE_NONE;
        continue;
      }
    }
    int k, ok;
    if (type == PJ_TYPE_PET) { k = pet_key(&w->key); ok = k >= 0 ? pet_field(c, w, k) : skip_value(c, 0); }
    else if (type == PJ_TYPE_ORDER) { k = ord_key(&w->key); ok = k >= 0 ? ord_field(c, w, k) : skip_value(c, 0); }
    else { k = usr_key(&w->key); ok = k >= 0 ? usr_field(c, w, k) : skip_value(c, 0); }
    if (!ok) return PJ_TYPE_NONE;
  }
  if (type == PJ_TYPE_NONE) { fail(c, PJ_E_AMBIGUOUS, close_pos); return PJ_TYPE_NONE; }
  if (type == PJ_TYPE_PET && (w->pet.present & 12u) != 12u) { fail(c, PJ_E_REQUIRED, close_pos); return PJ_TYPE_NONE; } /* petstore.json:873-876 */
  skip_ws(c);
  if (c->p < c->e) { fail(c, PJ_E_SYNTAX, c->p); return PJ_TYPE_NONE; }
  if (c->open_end) { fail_end(c); return PJ_TYPE_NONE; }
  return type;
}

/* ------------------------------------------------------------------------------------------ */
/* column writer (sequential append with capacity accounting)                                  */
/* ------------------------------------------------------------------------------------------ */
typedef struct { pj_columns* c; uint64_t used[PJ_MAX_COLS]; int overflow; } colw;
static void* slot(colw* w, int col, uint32_t elem, uint64_t idx) {
  if (w->used[col] < idx + 1) w->used[col] = idx + 1;
  pj_buf* b = &w->c->col[col];
  if (!b->ptr || (idx + 1) * elem > b->bytes) { w->overflow = 1; return NULL; }
  return (uint8_t*)b->ptr + idx * elem;
}
static void w_u8(colw* w, int col, uint64_t i, uint8_t v) { uint8_t* p = (uint8_t*)slot(w, col, 1, i); if (p) *p = v; }
static void w_u32(colw* w, int col, uint64_t i, uint32_t v) { uint32_t* p = (uint32_t*)slot(w, col, 4, i); if (p) *p = v; }
static void w_i32(colw* w, int col, uint64_t i, int32_t v) { int32_t* p = (int32_t*)slot(w, col, 4, i); if (p) *p = v; }
static void w_i64(colw* w, int col, uint64_t i, int64_t v) { int64_t* p = (int64_t*)slot(w, col, 8, i); if (p) *p = v; }
static void w_u64(colw* w, int col, uint64_t i, uint64_t v) { uint64_t* p = (uint64_t*)slot(w, col, 8, i); if (p) *p = v; }
static void w_str(colw* w, int off_col, int data_col, uint64_t row, const uint8_t* s, size_t n) {
  uint64_t at = w->used[data_col];
  w_u32(w, off_col, row, (uint32_t)at);
  for (size_t i = 0; i < n; ++i) w_u8(w, data_col, at + i, s[i]);
  w_u32(w, off_col, row + 1, (uint32_t)(at + n));
}
static const int USR_OFF_COLS[6] = {PJ_COL_USR_USERNAME_OFF, PJ_COL_USR_FIRSTNAME_OFF, PJ_COL_USR_LASTNAME_OFF,
                                    PJ_COL_USR_EMAIL_OFF, PJ_COL_USR_PASSWORD_OFF, PJ_COL_USR_PHONE_OFF};
static const int PET_OFF_COLS[6] = {PJ_COL_PET_CAT_NAME_OFF, PJ_COL_PET_NAME_OFF, PJ_COL_PET_PHOTO_OFF,
                                    PJ_COL_PET_PHOTO_STR_OFF, PJ_COL_PET_TAGS_OFF, PJ_COL_PET_TAG_NAME_OFF};

static void append_pet(colw* w, const petval* v, uint64_t row) {
  uint64_t P = w->used[PJ_COL_PET_PHOTO_STR_OFF] - 1, T = w->used[PJ_COL_PET_TAG_NAME_OFF] - 1;
  w_u8(w, PJ_COL_PET_PRESENT, row, (uint8_t)v->present);
  w_i64(w, PJ_COL_PET_ID, row, v->id);
  w_u8(w, PJ_COL_PET_CAT_PRESENT, row, (uint8_t)v->cat_present);
  w_i64(w, PJ_COL_PET_CAT_ID, row, v->cat_id);
  w_str(w, PJ_COL_PET_CAT_NAME_OFF, PJ_COL_PET_CAT_NAME_DATA, row, v->cat_name.b, v->cat_name.n);
  w_str(w, PJ_COL_PET_NAME_OFF, PJ_COL_PET_NAME_DATA, row, v->name.b, v->name.n);
  w_u32(w, PJ_COL_PET_PHOTO_OFF, row, (uint32_t)P);
  for (size_t i = 0; i < v->photo.n; ++i)
    w_str(w, PJ_COL_PET_PHOTO_STR_OFF, PJ_COL_PET_PHOTO_DATA, P + i, v->photo.data.b + v->photo.off[i], v->photo.off[i + 1] - v->photo.off[i]);
  w_u32(w, PJ_COL_PET_PHOTO_OFF, row + 1, (uint32_t)(P + v->photo.n));
  w_u32(w, PJ_COL_PET_TAGS_OFF, row, (uint32_t)T);
  for (size_t i = 0; i < v->n_tags; ++i) {
    w_u8(w, PJ_COL_PET_TAG_PRESENT, T + i, v->tags[i].present);
    w_i64(w, PJ_COL_PET_TAG_ID, T + i, v->tags[i].id);
    w_str(w, PJ_COL_PET_TAG_NAME_OFF, PJ_COL_PET_TAG_NAME_DATA, T + i, v->tag_names.data.b + v->tag_names.off[i], v->tag_names.off[i + 1] - v->tag_names.off[i]);
  }
  w_u32(w, PJ_COL_PET_TAGS_OFF, row + 1, (uint32_t)(T + v->n_tags));
  w_u8(w, PJ_COL_PET_STATUS, row, (uint8_t)v->status);
}
static void append_order(colw* w, const ordval* v, uint64_t row) {
  w_u8(w, PJ_COL_ORD_PRESENT, row, (uint8_t)v->present);
  w_i64(w, PJ_COL_ORD_ID, row, v->id);
  w_i64(w, PJ_COL_ORD_PET_ID, row, v->pet_id);
  w_i32(w, PJ_COL_ORD_QUANTITY, row, v->quantity);
  w_i64(w, PJ_COL_ORD_SHIP_EPOCH, row, v->ship_epoch);
  w_i32(w, PJ_COL_ORD_SHIP_NANOS, row, v->ship_nanos);
  w_i32(w, PJ_COL_ORD_SHIP_OFFSET, row, v->ship_off);
  w_u8(w, PJ_COL_ORD_STATUS, row, (uint8_t)v->status);
  w_u8(w, PJ_COL_ORD_COMPLETE, row, v->complete);
}
static void append_user(colw* w, const usrval* v, uint64_t row) {
  w_u8(w, PJ_COL_USR_PRESENT, row, (uint8_t)v->present);
  w_i64(w, PJ_COL_USR_ID, row, v->id);
  for (int f = 0; f < 6; ++f) w_str(w, USR_OFF_COLS[f], USR_OFF_COLS[f] + 1, row, v->s[f].b, v->s[f].n);
  w_i32(w, PJ_COL_USR_STATUS, row, v->user_status);
}

/* ------------------------------------------------------------------------------------------ */
/* record extents                                                                              */
/* ------------------------------------------------------------------------------------------ */
typedef struct { uint64_t s, e; int open_end; int blank_err; } extent;
typedef struct { extent* x; size_t n, cap; } extlist;
static void ext_push(extlist* l, extent x) {
  if (l->n == l->cap) { l->cap = l->cap ? l->cap * 2 : 1024; l->x = (extent*)realloc(l->x, l->cap * sizeof(extent)); }
  l->x[l->n++] = x;
}

/* NDJSON shard rule: candidates are byte 0 (if is_first) and every byte after an LF in [0, len). */
static void extents_ndjson(const uint8_t* in, uint64_t len, uint64_t slack, int is_first, int is_last, extlist* out) {
  uint64_t limit = len + slack;
  for (uint64_t q = 0; q <= len; ++q) {
    uint64_t p;
    if (q == 0) { if (!is_first) continue; p = 0; }
    else { if (in[q - 1] != '\n') continue; p = q; }
    /* blank check */
    uint64_t t = p;
    while (t < limit && (in[t] == ' ' || in[t] == '\t' || in[t] == '\r')) t++;
    extent x; x.s = p; x.blank_err = 0; x.open_end = 0;
    if (t < limit && in[t] == '\n') continue; /* blank line */
    if (t >= limit) {
      if (is_last) continue; /* blank tail of the stream */
      x.e = limit; x.open_end = 1; ext_push(out, x); continue;
    }
    uint64_t e = t;
    while (e < limit && in[e] != '\n') e++;
    x.e = e;
    x.open_end = (e >= limit && !is_last);
    ext_push(out, x);
  }
}

/* Array framing, stated so that every quantity is a prefix sum over the bytes:
 *   - a quote is escaped iff an odd run of backslashes precedes it; unescaped quotes toggle the
 *     in-string state; the quote bytes themselves count as outside;
 *   - d(p) = openers `{` `[` minus closers `}` `]` among the outside bytes before p;
 *   - separators: `[` at d == 0 (opener), `,` at d == 1, `]` at d == 1 (closer);
 *   - an extent runs from the byte after an opener or comma to the next separator, or to the end
 *     of the input when none follows;
 *   - a blank extent is dropped when it lies between an opener and a closer (`[]`) or runs to the
 *     end of the input; any other blank extent is a record failing with PJ_E_SYNTAX at its end;
 *   - document fault: the first outside non-blank byte with d <= 0 that is not a `[` at d == 0, or
 *     the second opener, whichever comes first (PJ_E_SYNTAX); failing those, an input without
 *     opener, ending inside a string or with d != 0 is (PJ_E_EOF, len). */
static void extents_array(const uint8_t* in, uint64_t len, extlist* out, uint32_t* doc_kind, uint64_t* doc_off) {
  *doc_kind = 0; *doc_off = 0;
  uint64_t bs_run = 0; int in_str = 0; int64_t d = 0;
  int have_left = 0, left_is_opener = 0, blank = 1; uint64_t start = 0; uint64_t openers = 0;
  for (uint64_t p = 0; p < len; ++p) {
    uint8_t x = in[p];
    int escaped = (bs_run & 1) != 0;
    if (x == '\\') bs_run++; else bs_run = 0;
    int is_quote = x == '"' && !escaped;
    if (in_str && !is_quote) continue; /* string interior */
    if (is_quote) in_str = !in_str;
    int ws = x == ' ' || x == '\t' || x == '\r' || x == '\n';
    int sep = 0; /* 1 opener, 2 comma, 3 closer */
    if (x == '[' && d == 0) sep = 1;
    else if (x == ',' && d == 1) sep = 2;
    else if (x == ']' && d == 1) sep = 3;
    if (!*doc_kind) {
      if (sep == 1) { if (openers >= 1) { *doc_kind = PJ_E_SYNTAX; *doc_off = p; } }
      else if (!ws && d <= 0) { *doc_kind = PJ_E_SYNTAX; *doc_off = p; }
    }
    if (sep) {
      if (have_left) {
        extent e; e.s = start; e.e = p; e.open_end = 0; e.blank_err = blank;
        if (!(blank && left_is_opener && sep == 3)) ext_push(out, e);
      }
      have_left = sep != 3; left_is_opener = sep == 1; start = p + 1; blank = 1;
      if (sep == 1) openers++;
    } else if (!ws) blank = 0;
    if (x == '{' || x == '[') d++;
    else if (x == '}' || x == ']') d--;
  }
  if (have_left && !blank) { extent e; e.s = start; e.e = len; e.open_end = 0; e.blank_err = 0; ext_push(out, e); }
  if (!*doc_kind && (openers == 0 || in_str || d != 0)) { *doc_kind = PJ_E_EOF; *doc_off = len; }
}

/* ------------------------------------------------------------------------------------------ */
/* public checker entry points                                                                 */
/* ------------------------------------------------------------------------------------------ */
int pjo_parse_opt(uint32_t schema, uint32_t framing, const uint8_t* in, uint64_t len, uint64_t slack,
                  int is_first, int is_last, uint64_t global_offset, uint32_t opts, pj_columns* out);
int pjo_parse(uint32_t schema, uint32_t framing, const uint8_t* in, uint64_t len, uint64_t slack,
              int is_first, int is_last, uint64_t global_offset, pj_columns* out) {
  return pjo_parse_opt(schema, framing, in, len, slack, is_first, is_last, global_offset, 0, out);
}
/* the same with pj_options.flags (the PJ_OPT_* bits that select the other answer of a rule) */
int pjo_parse_opt(uint32_t schema, uint32_t framing, const uint8_t* in, uint64_t len, uint64_t slack,
                  int is_first, int is_last, uint64_t global_offset, uint32_t opts, pj_columns* out) {
  if (!out || (!in && len + slack) || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return PJ_ERR_ARG;
  extlist xl; memset(&xl, 0, sizeof xl);
  uint32_t doc_kind = 0; uint64_t doc_off = 0;
  if (framing == PJ_FRAMING_NDJSON) extents_ndjson(in, len, slack, is_first, is_last, &xl);
  else if (framing == PJ_FRAMING_ARRAY) extents_array(in, len, &xl, &doc_kind, &doc_off);
  else return PJ_ERR_ARG;

  colw w; memset(&w, 0, sizeof w); w.c = out;
  scratch sc; memset(&sc, 0, sizeof sc);
  int mixed = schema == PJ_SCHEMA_MIXED;
  if (schema == PJ_SCHEMA_PET || mixed) for (int i = 0; i < 6; ++i) w_u32(&w, PET_OFF_COLS[i], 0, 0);
  if (schema == PJ_SCHEMA_USER || mixed) for (int f = 0; f < 6; ++f) w_u32(&w, USR_OFF_COLS[f], 0, 0);
  uint64_t rows[4] = {0, 0, 0, 0}, n_err = 0;
  for (size_t i = 0; i < xl.n; ++i) {
    cur c; memset(&c, 0, sizeof c);
    c.b = in; c.s = c.p = xl.x[i].s; c.e = xl.x[i].e; c.lf_ws = framing == PJ_FRAMING_ARRAY; c.open_end = xl.x[i].open_end; c.opts = opts;
    int type;
    if (xl.x[i].blank_err) { fail(&c, PJ_E_SYNTAX, c.e); type = PJ_TYPE_NONE; }
    else type = parse_record(&c, &sc, schema);
    w_u64(&w, PJ_COL_REC_START, i, c.s + global_offset);
    w_u8(&w, PJ_COL_ERR_KIND, i, (uint8_t)c.err);
    w_u32(&w, PJ_COL_ERR_OFF, i, c.err ? (uint32_t)(c.err_pos - c.s) : 0);
    n_err += c.err != 0;
    if (mixed) {
      w_u8(&w, PJ_COL_REC_TYPE, i, (uint8_t)type);
      w_u32(&w, PJ_COL_REC_ROW, i, type == PJ_TYPE_NONE ? 0xFFFFFFFFu : (uint32_t)rows[type]);
      if (type == PJ_TYPE_NONE) continue;
    } else if (type == PJ_TYPE_NONE) {
      /* R11: the failed record keeps an all-absent row */
      type = (int)schema;
      pet_reset(&sc.pet); ord_reset(&sc.ord); usr_reset(&sc.usr);
    }
    uint64_t row = rows[type]++;
    if (type == PJ_TYPE_PET) append_pet(&w, &sc.pet, row);
    else if (type == PJ_TYPE_ORDER) append_order(&w, &sc.ord, row);
    else append_user(&w, &sc.usr, row);
  }
  out->schema = schema;
  out->n_records = xl.n;
  out->n_errors = n_err;
  for (int t = 0; t < 4; ++t) out->n_rows[t] = rows[t];
  out->doc_err_kind = doc_kind; out->doc_err_off = doc_off;
  for (int k = 0; k < PJ_MAX_COLS; ++k) out->col[k].count = w.used[k];
  scratch_free(&sc);
  free(xl.x);
  return w.overflow ? PJ_ERR_CAPACITY : PJ_OK;
}

int pjo_index(uint32_t framing, const uint8_t* in, uint64_t len, uint64_t* rec_start, uint64_t cap, uint64_t* n) {
  extlist xl; memset(&xl, 0, sizeof xl);
  uint32_t dk; uint64_t doff;
  if (framing == PJ_FRAMING_NDJSON) extents_ndjson(in, len, 0, 1, 1, &xl);
  else extents_array(in, len, &xl, &dk, &doff);
  for (size_t i = 0; i < xl.n && i < cap; ++i) rec_start[i] = xl.x[i].s;
  *n = xl.n;
  free(xl.x);
  return xl.n > cap ? PJ_ERR_CAPACITY : PJ_OK;
}

/* Record extents as the framing rules define them (start, end, "blank extent that is a record"). */
int pjo_extents(uint32_t framing, const uint8_t* in, uint64_t len, uint64_t* s, uint64_t* e, uint8_t* blank,
                uint64_t cap, uint64_t* n, uint32_t* doc_kind, uint64_t* doc_off) {
  extlist xl; memset(&xl, 0, sizeof xl);
  uint32_t dk = 0; uint64_t doff = 0;
  if (framing == PJ_FRAMING_NDJSON) extents_ndjson(in, len, 0, 1, 1, &xl);
  else extents_array(in, len, &xl, &dk, &doff);
  for (size_t i = 0; i < xl.n && i < cap; ++i) { s[i] = xl.x[i].s; e[i] = xl.x[i].e; blank[i] = (uint8_t)xl.x[i].blank_err; }
  *n = xl.n;
  if (doc_kind) *doc_kind = dk;
  if (doc_off) *doc_off = doff;
  free(xl.x);
  return xl.n > cap ? PJ_ERR_CAPACITY : PJ_OK;
}

/* ------------------------------------------------------------------------------------------ */
/* writer (W1-W5)                                                                              */
/* ------------------------------------------------------------------------------------------ */
typedef struct { uint8_t* p; uint64_t cap, n; int incl; int hex_lower; } wout;
static void o_put(wout* o, uint8_t c) { if (o->n < o->cap) o->p[o->n] = c; o->n++; }
static void o_lit(wout* o, const char* s) { while (*s) o_put(o, (uint8_t)*s++); }
static void o_i64(wout* o, int64_t v) {
  char b[24]; int n = 0;
  uint64_t u = v < 0 ? 0 - (uint64_t)v : (uint64_t)v;
  do { b[n++] = (char)('0' + u % 10); u /= 10; } while (u);
  if (v < 0) o_put(o, '-');
  while (n) o_put(o, (uint8_t)b[--n]);
}
static void o_str(wout* o, const uint8_t* s, size_t n) {
  const char* HEX = o->hex_lower ? "0123456789abcdef" : "0123456789ABCDEF";
  o_put(o, '"');
  for (size_t i = 0; i < n; ++i) {
    uint8_t c = s[i];
    if (c == '"') o_lit(o, "\\\"");
    else if (c == '\\') o_lit(o, "\\\\");
    else if (c >= 0x20) o_put(o, c);
    else if (c == 8) o_lit(o, "\\b");
    else if (c == 9) o_lit(o, "\\t");
    else if (c == 10) o_lit(o, "\\n");
    else if (c == 12) o_lit(o, "\\f");
    else if (c == 13) o_lit(o, "\\r");
    else { o_lit(o, "\\u00"); o_put(o, (uint8_t)HEX[c >> 4]); o_put(o, (uint8_t)HEX[c & 15]); }
  }
  o_put(o, '"');
}
static void o_key(wout* o, const char* k, int* first) {
  if (!*first) o_put(o, ',');
  *first = 0;
  o_put(o, '"'); o_lit(o, k); o_lit(o, "\":");
}
/* whether a property is written at all, given presence / emptiness (W4) */
static int included(const wout* o, int present, int empty) {
  if (o->incl == PJ_INCLUDE_ALWAYS) return 1;
  if (!present) return 0;
  if (o->incl == PJ_INCLUDE_NON_EMPTY && empty) return 0;
  return 1;
}
#define COL(T, id) ((const T*)cols->col[id].ptr)
static void o_strcol(wout* o, const pj_columns* cols, int off_col, uint64_t row) {
  const uint32_t* off = COL(uint32_t, off_col);
  o_str(o, COL(uint8_t, off_col + 1) + off[row], off[row + 1] - off[row]);
}
static uint32_t strcol_len(const pj_columns* cols, int off_col, uint64_t row) {
  const uint32_t* off = COL(uint32_t, off_col);
  return off[row + 1] - off[row];
}
static void o_2d(wout* o, unsigned v) { o_put(o, (uint8_t)('0' + v / 10)); o_put(o, (uint8_t)('0' + v % 10)); }

static void write_pet(wout* o, const pj_columns* cols, uint64_t r) {
  uint32_t pr = COL(uint8_t, PJ_COL_PET_PRESENT)[r];
  int first = 1;
  o_put(o, '{');
  if (included(o, pr & 1, 0)) { o_key(o, "id", &first); if (pr & 1) o_i64(o, COL(int64_t, PJ_COL_PET_ID)[r]); else o_lit(o, "null"); }
  if (included(o, pr & 2, 0)) {
    o_key(o, "category", &first);
    if (!(pr & 2)) o_lit(o, "null");
    else {
      uint32_t cp = COL(uint8_t, PJ_COL_PET_CAT_PRESENT)[r];
      int f2 = 1;
      o_put(o, '{');
      if (included(o, cp & 1, 0)) { o_key(o, "id", &f2); if (cp & 1) o_i64(o, COL(int64_t, PJ_COL_PET_CAT_ID)[r]); else o_lit(o, "null"); }
      if (included(o, cp & 2, strcol_len(cols, PJ_COL_PET_CAT_NAME_OFF, r) == 0)) { o_key(o, "name", &f2); if (cp & 2) o_strcol(o, cols, PJ_COL_PET_CAT_NAME_OFF, r); else o_lit(o, "null"); }
      o_put(o, '}');
    }
  }
  if (included(o, pr & 4, strcol_len(cols, PJ_COL_PET_NAME_OFF, r) == 0)) { o_key(o, "name", &first); if (pr & 4) o_strcol(o, cols, PJ_COL_PET_NAME_OFF, r); else o_lit(o, "null"); }
  {
    const uint32_t* lo = COL(uint32_t, PJ_COL_PET_PHOTO_OFF);
    if (included(o, pr & 8, lo[r] == lo[r + 1])) {
      o_key(o, "photoUrls", &first);
      if (!(pr & 8)) o_lit(o, "null");
      else {
        o_put(o, '[');
        for (uint32_t k = lo[r]; k < lo[r + 1]; ++k) { if (k > lo[r]) o_put(o, ','); o_strcol(o, cols, PJ_COL_PET_PHOTO_STR_OFF, k); }
        o_put(o, ']');
      }
    }
  }
  {
    const uint32_t* lo = COL(uint32_t, PJ_COL_PET_TAGS_OFF);
    if (included(o, pr & 16, lo[r] == lo[r + 1])) {
      o_key(o, "tags", &first);
      if (!(pr & 16)) o_lit(o, "null");
      else {
        o_put(o, '[');
        for (uint32_t k = lo[r]; k < lo[r + 1]; ++k) {
          uint32_t tp = COL(uint8_t, PJ_COL_PET_TAG_PRESENT)[k];
          int f2 = 1;
          if (k > lo[r]) o_put(o, ',');
          o_put(o, '{');
          if (included(o, tp & 1, 0)) { o_key(o, "id", &f2); if (tp & 1) o_i64(o, COL(int64_t, PJ_COL_PET_TAG_ID)[k]); else o_lit(o, "null"); }
          if (included(o, tp & 2, strcol_len(cols, PJ_COL_PET_TAG_NAME_OFF, k) == 0)) { o_key(o, "name", &f2); if (tp & 2) o_strcol(o, cols, PJ_COL_PET_TAG_NAME_OFF, k); else o_lit(o, "null"); }
          o_put(o, '}');
        }
        o_put(o, ']');
      }
    }
  }
  if (included(o, pr & 32, 0)) {
    o_key(o, "status", &first);
    if (pr & 32) { o_put(o, '"'); o_lit(o, PET_STATUS[COL(uint8_t, PJ_COL_PET_STATUS)[r] % 3]); o_put(o, '"'); } else o_lit(o, "null");
  }
  o_put(o, '}');
}
static void write_order(wout* o, const pj_columns* cols, uint64_t r) {
  uint32_t pr = COL(uint8_t, PJ_COL_ORD_PRESENT)[r];
  int first = 1;
  o_put(o, '{');
  if (included(o, pr & 1, 0)) { o_key(o, "id", &first); if (pr & 1) o_i64(o, COL(int64_t, PJ_COL_ORD_ID)[r]); else o_lit(o, "null"); }
  if (included(o, pr & 2, 0)) { o_key(o, "petId", &first); if (pr & 2) o_i64(o, COL(int64_t, PJ_COL_ORD_PET_ID)[r]); else o_lit(o, "null"); }
  if (included(o, pr & 4, 0)) { o_key(o, "quantity", &first); if (pr & 4) o_i64(o, COL(int32_t, PJ_COL_ORD_QUANTITY)[r]); else o_lit(o, "null"); }
  if (included(o, pr & 8, 0)) {
    o_key(o, "shipDate", &first);
    if (!(pr & 8)) o_lit(o, "null");
    else {
      int64_t ep = COL(int64_t, PJ_COL_ORD_SHIP_EPOCH)[r];
      int32_t ns = COL(int32_t, PJ_COL_ORD_SHIP_NANOS)[r], off = COL(int32_t, PJ_COL_ORD_SHIP_OFFSET)[r];
      int64_t local = ep + off;
      int64_t days = (local >= 0 ? local : local - 86399) / 86400;
      unsigned sod = (unsigned)(local - days * 86400);
      int64_t y; unsigned m, d;
      civil_from_days(days, &y, &m, &d);
      o_put(o, '"');
      o_2d(o, (unsigned)(y / 100)); o_2d(o, (unsigned)(y % 100)); o_put(o, '-'); o_2d(o, m); o_put(o, '-'); o_2d(o, d);
      o_put(o, 'T'); o_2d(o, sod / 3600); o_put(o, ':'); o_2d(o, sod % 3600 / 60); o_put(o, ':'); o_2d(o, sod % 60);
      if (ns) {
        char f[9]; int k = 9; uint32_t u = (uint32_t)ns;
        for (int i = 8; i >= 0; --i) { f[i] = (char)('0' + u % 10); u /= 10; }
        while (k > 0 && f[k - 1] == '0') --k;
        o_put(o, '.');
        for (int i = 0; i < k; ++i) o_put(o, (uint8_t)f[i]);
      }
      if (off == 0) o_put(o, 'Z');
      else { unsigned a = (unsigned)(off < 0 ? -off : off); o_put(o, off < 0 ? '-' : '+'); o_2d(o, a / 3600); o_put(o, ':'); o_2d(o, a % 3600 / 60); }
      o_put(o, '"');
    }
  }
  if (included(o, pr & 16, 0)) {
    o_key(o, "status", &first);
    if (pr & 16) { o_put(o, '"'); o_lit(o, ORD_STATUS[COL(uint8_t, PJ_COL_ORD_STATUS)[r] % 3]); o_put(o, '"'); } else o_lit(o, "null");
  }
  if (included(o, pr & 32, 0)) { o_key(o, "complete", &first); if (pr & 32) o_lit(o, COL(uint8_t, PJ_COL_ORD_COMPLETE)[r] ? "true" : "false"); else o_lit(o, "null"); }
  o_put(o, '}');
}
static void write_user(wout* o, const pj_columns* cols, uint64_t r) {
  static const char* const keys[6] = {"username", "firstName", "lastName", "email", "password", "phone"};
  uint32_t pr = COL(uint8_t, PJ_COL_USR_PRESENT)[r];
  int first = 1;
  o_put(o, '{');
  if (included(o, pr & 1, 0)) { o_key(o, "id", &first); if (pr & 1) o_i64(o, COL(int64_t, PJ_COL_USR_ID)[r]); else o_lit(o, "null"); }
  for (int f = 0; f < 6; ++f) {
    uint32_t bit = 2u << f;
    if (included(o, pr & bit, strcol_len(cols, USR_OFF_COLS[f], r) == 0)) { o_key(o, keys[f], &first); if (pr & bit) o_strcol(o, cols, USR_OFF_COLS[f], r); else o_lit(o, "null"); }
  }
  if (included(o, pr & 128, 0)) { o_key(o, "userStatus", &first); if (pr & 128) o_i64(o, COL(int32_t, PJ_COL_USR_STATUS)[r]); else o_lit(o, "null"); }
  o_put(o, '}');
}

int pjo_write_opt(uint32_t schema, uint32_t framing, int inclusion, uint32_t opts, const pj_columns* cols, uint8_t* out,
                  uint64_t cap, uint64_t* out_len);
int pjo_write(uint32_t schema, uint32_t framing, int inclusion, const pj_columns* cols, uint8_t* out,
              uint64_t cap, uint64_t* out_len) {
  return pjo_write_opt(schema, framing, inclusion, 0, cols, out, cap, out_len);
}
int pjo_write_opt(uint32_t schema, uint32_t framing, int inclusion, uint32_t opts, const pj_columns* cols, uint8_t* out,
                  uint64_t cap, uint64_t* out_len) {
  if (!cols || !out_len || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return PJ_ERR_ARG;
  wout o; o.p = out; o.cap = out ? cap : 0; o.n = 0; o.incl = inclusion; o.hex_lower = (opts & PJ_OPT_HEX_LOWER) != 0;
  int arr = framing == PJ_FRAMING_ARRAY;
  uint64_t n = schema == PJ_SCHEMA_MIXED ? cols->n_records : cols->n_rows[schema];
  uint64_t written = 0;
  if (arr) o_put(&o, '[');
  for (uint64_t i = 0; i < n; ++i) {
    uint32_t type = schema; uint64_t row = i;
    if (schema == PJ_SCHEMA_MIXED) {
      type = COL(uint8_t, PJ_COL_REC_TYPE)[i];
      row = COL(uint32_t, PJ_COL_REC_ROW)[i];
      if (type == PJ_TYPE_NONE) continue;
    }
    if (arr && written) o_put(&o, ',');
    if (type == PJ_TYPE_PET) write_pet(&o, cols, row);
    else if (type == PJ_TYPE_ORDER) write_order(&o, cols, row);
    else write_user(&o, cols, row);
    if (!arr) o_put(&o, '\n');
    written++;
  }
  if (arr) o_put(&o, ']');
  *out_len = o.n;
  return o.n > cap ? PJ_ERR_CAPACITY : PJ_OK;
}

/* ---- column checksums: the definition in include/petjson.h (pj_columns_checksum), for host columns ---------- */
static uint64_t cs_mix(uint64_t x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}
/* sum over the 8-byte words of p[0..n) */
uint64_t pjo_checksum_bytes(const uint8_t* p, uint64_t n) {
  uint64_t s = 0;
  for (uint64_t j = 0; 8 * j < n; ++j) {
    uint64_t w = 0;
    for (uint32_t b = 0; b < 8 && 8 * j + b < n; ++b) w |= (uint64_t)p[8 * j + b] << (8 * b);
    s += cs_mix(w + 0x9E3779B97F4A7C15ull * (j + 1));
  }
  return s;
}
