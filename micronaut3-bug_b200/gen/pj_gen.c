/*
 * pj_gen.c — seeded synthetic Petstore workloads (host code, no CUDA).
 *
 * Produces, for records [first, first+n) of a stream identified by `seed`,
 *   (a) the JSON text (pj_gen_text), and
 *   (b) the values a correct parse of that text yields, as columns (pj_gen_columns).
 * Record k depends only on (seed, k): every draw is a counter-based hash of (seed, record, field,
 * lane), so byte-range shards of one stream can be produced independently.
 *
 * Value distributions are those of the benchmark configurations: Pet per
 * petstore.json:872-922 (id int64 in [1, 2^62]; name 4-16 letters; category {id, name 3-12
 * letters}; 0-4 photoUrls of 20-60 URL-safe characters; 0-3 tags {id, name 3-10 letters}; status
 * uniform over the three literals), Order per petstore.json:937-971, User per petstore.json:824-857.
 */
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "petjson_gen.h"

/* ------------------------------------------------------------------------------------------ */
/* counter-based randomness                                                                    */
/* ------------------------------------------------------------------------------------------ */
static uint64_t mix64(uint64_t x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}
static uint64_t draw(uint64_t seed, uint64_t rec, uint32_t field, uint32_t lane) {
  uint64_t x = mix64(seed + 0x9E3779B97F4A7C15ull * (rec + 1));
  x ^= ((uint64_t)field << 32 | lane) * 0xD1B54A32D192ED03ull;
  return mix64(x + 0x2545F4914F6CDD1Dull);
}
/* uniform integer in [lo, hi] (range far below 2^32, bias negligible and deterministic) */
static uint32_t uni(uint64_t h, uint32_t lo, uint32_t hi) {
  return lo + (uint32_t)((h >> 11) % (uint64_t)(hi - lo + 1));
}
/* sequential stream for formatting decisions inside one record */
typedef struct { uint64_t s; } fstream;
static uint64_t fnext(fstream* f) { f->s += 0x9E3779B97F4A7C15ull; return mix64(f->s); }

/* field ids for draw() */
enum {
  F_TYPE = 1, F_ID, F_CAT_ID, F_CAT_NAME, F_NAME, F_NPHOTO, F_PHOTO, F_NTAGS, F_TAG_ID, F_TAG_NAME,
  F_STATUS, F_MAL, F_MAL_KIND, F_MAL_POS, F_FMT, F_ESC, F_SPARSE,
  F_PETID, F_QTY, F_DATE, F_COMPLETE,
  F_USERNAME, F_FIRST, F_LAST, F_EMAIL, F_PASSWORD, F_PHONE, F_USTATUS
};

/* ------------------------------------------------------------------------------------------ */
/* record values                                                                               */
/* ------------------------------------------------------------------------------------------ */
#define GSTR_MAX 96
typedef struct { uint8_t b[GSTR_MAX]; uint32_t n; uint8_t special; } gstr;
typedef struct { int64_t id; gstr name; } gtag;

#define MAX_PHOTO 256
#define MAX_TAGS 64

enum { MAL_NONE = 0, MAL_ENUM = 1, MAL_REQUIRED = 2, MAL_TYPE = 3, MAL_TRUNC = 4 };

typedef struct {
  uint32_t type; /* PJ_TYPE_* */
  uint32_t present; /* root presence bits, schema order */
  uint32_t nullmask; /* properties written as `null` (then not present) */
  int mal;
  uint32_t mal_pos;
  /* Pet */
  int64_t id, cat_id;
  uint32_t cat_present, cat_null;
  gstr cat_name, name;
  uint32_t n_photo, n_tags;
  gstr photo[MAX_PHOTO];
  gtag tags[MAX_TAGS];
  uint8_t status;
  /* Order */
  int64_t pet_id, ship_epoch;
  int32_t quantity, ship_nanos, ship_off;
  uint8_t complete;
  char ship_text[40];
  /* User */
  gstr u_str[6];
  int32_t user_status;
} grec;

static const char LETTERS[] = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ";
static const char URLSAFE[] = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789-._~";
static const char ALNUM[] = "abcdefghijklmnopqrstuvwxyzABCDEFGHIJKLMNOPQRSTUVWXYZ0123456789";
static const char DIGITS[] = "0123456789";

static const char* const PET_STATUS[3] = {"available", "pending", "sold"};
static const char* const ORD_STATUS[3] = {"placed", "approved", "delivered"};

/* code points mixed into "special" strings when PJ_GEN_ESCAPES is on */
static const uint32_t SPECIALS[] = {0xE9, 0x20AC, 0x4E2D, 0x1F600, 0x10FFFF, '"', '\\', '/', '\n',
                                    '\t', 0x01, 0x7F, 0x80, 0x7FF, 0x800, 0xFFFD, 0x10000, 0x08,
                                    0x0C, '\r', 0x1F};
#define N_SPECIALS (sizeof(SPECIALS) / sizeof(SPECIALS[0]))

static uint32_t utf8_put(uint8_t* d, uint32_t cp) {
  if (cp < 0x80) { d[0] = (uint8_t)cp; return 1; }
  if (cp < 0x800) { d[0] = 0xC0 | (cp >> 6); d[1] = 0x80 | (cp & 63); return 2; }
  if (cp < 0x10000) { d[0] = 0xE0 | (cp >> 12); d[1] = 0x80 | ((cp >> 6) & 63); d[2] = 0x80 | (cp & 63); return 3; }
  d[0] = 0xF0 | (cp >> 18); d[1] = 0x80 | ((cp >> 12) & 63); d[2] = 0x80 | ((cp >> 6) & 63); d[3] = 0x80 | (cp & 63);
  return 4;
}

static void gen_str(gstr* s, uint64_t seed, uint64_t rec, uint32_t field, uint32_t lane_base,
                    const char* alphabet, uint32_t lo, uint32_t hi, uint32_t flags) {
  uint32_t na = (uint32_t)strlen(alphabet);
  uint64_t h = draw(seed, rec, field, lane_base);
  uint32_t n = uni(h, lo, hi);
  uint8_t tmp[GSTR_MAX];
  for (uint32_t i = 0; i < n; i += 8) {
    uint64_t r = draw(seed, rec, field, lane_base + 1 + i / 8);
    for (uint32_t j = 0; j < 8 && i + j < n; ++j) { tmp[i + j] = (uint8_t)alphabet[(r & 0xFF) % na]; r >>= 8; }
  }
  s->special = 0;
  if ((flags & PJ_GEN_ESCAPES) && (draw(seed, rec, F_ESC, field * 4096 + lane_base) % 100) < 5) {
    /* insert 1-3 special code points at seeded positions */
    uint64_t r = draw(seed, rec, F_ESC, field * 4096 + lane_base + 1);
    uint32_t k = 1 + (uint32_t)(r % 3); r >>= 2;
    uint32_t pos[3], cp[3];
    for (uint32_t i = 0; i < k; ++i) { pos[i] = (uint32_t)(r % (n + 1)); r >>= 8; cp[i] = SPECIALS[r % N_SPECIALS]; r >>= 8; }
    uint32_t o = 0;
    for (uint32_t i = 0; i <= n; ++i) {
      for (uint32_t j = 0; j < k; ++j) if (pos[j] == i) o += utf8_put(s->b + o, cp[j]);
      if (i < n) s->b[o++] = tmp[i];
    }
    s->n = o; s->special = 1;
  } else {
    memcpy(s->b, tmp, n); s->n = n;
  }
}

static int64_t gen_id(uint64_t seed, uint64_t rec, uint32_t field, uint32_t lane) {
  return 1 + (int64_t)(draw(seed, rec, field, lane) % (1ull << 62));
}

/* zipf(1.2) over k = 1..cap+1, list length = k-1; thresholds are cumulative weights scaled to 2^32 */
static uint32_t zipf_thr_photo[MAX_PHOTO + 1], zipf_thr_tags[MAX_TAGS + 1];
static int zipf_ready = 0;
static void zipf_init_one(uint32_t* thr, uint32_t cap) {
  double tot = 0.0, acc = 0.0;
  for (uint32_t k = 1; k <= cap + 1; ++k) tot += pow((double)k, -1.2);
  for (uint32_t k = 1; k <= cap + 1; ++k) {
    acc += pow((double)k, -1.2);
    double t = acc / tot * 4294967295.0;
    thr[k - 1] = (k == cap + 1) ? 0xFFFFFFFFu : (uint32_t)t;
  }
}
static void zipf_init(void) {
  if (zipf_ready) return;
  zipf_init_one(zipf_thr_photo, MAX_PHOTO);
  zipf_init_one(zipf_thr_tags, MAX_TAGS);
  zipf_ready = 1;
}
static uint32_t zipf_len(const uint32_t* thr, uint32_t cap, uint64_t h) {
  uint32_t u = (uint32_t)(h >> 32), lo = 0, hi = cap;
  while (lo < hi) { uint32_t mid = (lo + hi) / 2; if (u <= thr[mid]) hi = mid; else lo = mid + 1; }
  return lo;
}

/* days since 1970-01-01 of a proleptic Gregorian date */
static int64_t days_from_civil(int64_t y, uint32_t m, uint32_t d) {
  y -= m <= 2;
  int64_t era = (y >= 0 ? y : y - 399) / 400;
  uint32_t yoe = (uint32_t)(y - era * 400);
  uint32_t doy = (153 * (m + (m > 2 ? -3 : 9)) + 2) / 5 + d - 1;
  uint32_t doe = yoe * 365 + yoe / 4 - yoe / 100 + doy;
  return era * 146097 + (int64_t)doe - 719468;
}

static uint32_t pick_type(uint32_t schema, uint64_t seed, uint64_t rec) {
  if (schema != PJ_SCHEMA_MIXED) return schema; /* PJ_SCHEMA_x == PJ_TYPE_x for the three models */
  uint32_t r = (uint32_t)(draw(seed, rec, F_TYPE, 0) % 100);
  return r < 50 ? PJ_TYPE_PET : (r < 80 ? PJ_TYPE_ORDER : PJ_TYPE_USER);
}

static void gen_record(grec* g, uint32_t schema, uint64_t seed, uint64_t rec, uint32_t flags) {
  g->type = pick_type(schema, seed, rec);
  g->mal = MAL_NONE; g->mal_pos = 0; g->nullmask = 0; g->cat_null = 0;
  uint32_t nfields = g->type == PJ_TYPE_PET ? 6 : (g->type == PJ_TYPE_ORDER ? 6 : 8);
  g->present = (1u << nfields) - 1;
  g->cat_present = 3;
  if (g->type == PJ_TYPE_PET) {
    g->id = gen_id(seed, rec, F_ID, 0);
    g->cat_id = gen_id(seed, rec, F_CAT_ID, 0);
    gen_str(&g->cat_name, seed, rec, F_CAT_NAME, 0, LETTERS, 3, 12, flags);
    gen_str(&g->name, seed, rec, F_NAME, 0, LETTERS, 4, 16, flags);
    if (flags & PJ_GEN_ZIPF_LISTS) {
      zipf_init();
      g->n_photo = zipf_len(zipf_thr_photo, MAX_PHOTO, draw(seed, rec, F_NPHOTO, 0));
      g->n_tags = zipf_len(zipf_thr_tags, MAX_TAGS, draw(seed, rec, F_NTAGS, 0));
    } else {
      g->n_photo = uni(draw(seed, rec, F_NPHOTO, 0), 0, 4);
      g->n_tags = uni(draw(seed, rec, F_NTAGS, 0), 0, 3);
    }
    for (uint32_t i = 0; i < g->n_photo; ++i) gen_str(&g->photo[i], seed, rec, F_PHOTO, i * 16, URLSAFE, 20, 60, flags);
    for (uint32_t i = 0; i < g->n_tags; ++i) {
      g->tags[i].id = gen_id(seed, rec, F_TAG_ID, i);
      gen_str(&g->tags[i].name, seed, rec, F_TAG_NAME, i * 16, LETTERS, 3, 10, flags);
    }
    g->status = (uint8_t)uni(draw(seed, rec, F_STATUS, 0), 0, 2);
  } else if (g->type == PJ_TYPE_ORDER) {
    g->id = gen_id(seed, rec, F_ID, 0);
    g->pet_id = gen_id(seed, rec, F_PETID, 0);
    g->quantity = (int32_t)uni(draw(seed, rec, F_QTY, 0), 1, 100);
    /* A date-time every ISO-8601 formatter prints the same way: non-zero seconds, exactly three
       fraction digits not ending in 0, offset Z or a non-zero +hh:mm / -hh:mm. */
    uint64_t r = draw(seed, rec, F_DATE, 0);
    uint32_t year = 1970 + (uint32_t)(r % 130); r /= 130;
    uint32_t mon = 1 + (uint32_t)(r % 12); r /= 12;
    uint32_t day = 1 + (uint32_t)(r % 28); r /= 28;
    uint32_t hh = (uint32_t)(r % 24); r /= 24;
    uint32_t mi = (uint32_t)(r % 60); r /= 60;
    uint32_t ss = 1 + (uint32_t)(r % 59); r /= 59;
    uint32_t ms = (uint32_t)(r % 1000); r /= 1000;
    if (ms % 10 == 0) ms += 1 + (uint32_t)(r % 9);
    r = draw(seed, rec, F_DATE, 1);
    int32_t off = 0;
    if (r % 3) {
      uint32_t oh = (uint32_t)((r >> 8) % 14), om = 15 * (uint32_t)((r >> 16) % 4);
      if (oh == 0 && om == 0) oh = 1;
      off = (int32_t)(oh * 3600 + om * 60);
      if ((r >> 24) & 1) off = -off;
    }
    g->ship_nanos = (int32_t)ms * 1000000;
    g->ship_off = off;
    g->ship_epoch = days_from_civil(year, mon, day) * 86400 + hh * 3600 + mi * 60 + ss - off;
    int n = 0;
    char* t = g->ship_text;
    t[n++] = '0' + year / 1000; t[n++] = '0' + year / 100 % 10; t[n++] = '0' + year / 10 % 10; t[n++] = '0' + year % 10;
    t[n++] = '-'; t[n++] = '0' + mon / 10; t[n++] = '0' + mon % 10;
    t[n++] = '-'; t[n++] = '0' + day / 10; t[n++] = '0' + day % 10;
    t[n++] = 'T'; t[n++] = '0' + hh / 10; t[n++] = '0' + hh % 10;
    t[n++] = ':'; t[n++] = '0' + mi / 10; t[n++] = '0' + mi % 10;
    t[n++] = ':'; t[n++] = '0' + ss / 10; t[n++] = '0' + ss % 10;
    t[n++] = '.'; t[n++] = '0' + ms / 100; t[n++] = '0' + ms / 10 % 10; t[n++] = '0' + ms % 10;
    if (off == 0) t[n++] = 'Z';
    else {
      uint32_t a = (uint32_t)(off < 0 ? -off : off);
      t[n++] = off < 0 ? '-' : '+';
      t[n++] = '0' + a / 3600 / 10; t[n++] = '0' + a / 3600 % 10; t[n++] = ':';
      t[n++] = '0' + a % 3600 / 60 / 10; t[n++] = '0' + a % 3600 / 60 % 10;
    }
    t[n] = 0;
    g->status = (uint8_t)uni(draw(seed, rec, F_STATUS, 0), 0, 2);
    g->complete = (uint8_t)(draw(seed, rec, F_COMPLETE, 0) & 1);
  } else {
    g->id = gen_id(seed, rec, F_ID, 0);
    gen_str(&g->u_str[0], seed, rec, F_USERNAME, 0, ALNUM, 6, 20, flags);
    gen_str(&g->u_str[1], seed, rec, F_FIRST, 0, LETTERS, 3, 12, flags);
    gen_str(&g->u_str[2], seed, rec, F_LAST, 0, LETTERS, 3, 12, flags);
    { /* email: local@domain.com */
      gstr a, b;
      gen_str(&a, seed, rec, F_EMAIL, 0, LETTERS, 6, 12, 0);
      gen_str(&b, seed, rec, F_EMAIL, 16, LETTERS, 4, 10, 0);
      gstr* e = &g->u_str[3];
      memcpy(e->b, a.b, a.n); e->n = a.n; e->b[e->n++] = '@';
      memcpy(e->b + e->n, b.b, b.n); e->n += b.n;
      memcpy(e->b + e->n, ".com", 4); e->n += 4; e->special = 0;
    }
    gen_str(&g->u_str[4], seed, rec, F_PASSWORD, 0, ALNUM, 8, 16, flags);
    gen_str(&g->u_str[5], seed, rec, F_PHONE, 0, DIGITS, 10, 10, 0);
    g->user_status = (int32_t)uni(draw(seed, rec, F_USTATUS, 0), 0, 3);
  }
  if (flags & PJ_GEN_SPARSE) {
    uint64_t r = draw(seed, rec, F_SPARSE, 0);
    for (uint32_t f = 0; f < nfields; ++f) {
      uint32_t v = (uint32_t)(r & 15); r >>= 4;
      int required = g->type == PJ_TYPE_PET && (f == 2 || f == 3);
      if (required) continue;
      if (v == 0 || v == 1) g->present &= ~(1u << f);                  /* omitted */
      else if (v == 2) { g->present &= ~(1u << f); g->nullmask |= 1u << f; } /* written as null */
    }
    if (g->type == PJ_TYPE_PET) {
      for (uint32_t f = 0; f < 2; ++f) {
        uint32_t v = (uint32_t)(r & 15); r >>= 4;
        if (v == 0) g->cat_present &= ~(1u << f);
        else if (v == 1) { g->cat_present &= ~(1u << f); g->cat_null |= 1u << f; }
      }
    }
  }
  /* keep at least one property that only this model has, so a mixed stream stays decidable */
  if (g->type == PJ_TYPE_ORDER && !((g->present | g->nullmask) & 0x2Eu)) g->present |= 2u;
  if (g->type == PJ_TYPE_USER && !((g->present | g->nullmask) & 0xFEu)) g->present |= 2u;
  if ((flags & PJ_GEN_MALFORMED) && draw(seed, rec, F_MAL, 0) % 100 == 0) {
    uint32_t k = (uint32_t)(draw(seed, rec, F_MAL_KIND, 0) % 4) + 1;
    if (k == MAL_REQUIRED && g->type != PJ_TYPE_PET) k = MAL_TYPE;        /* only Pet has required */
    if (k == MAL_ENUM && g->type == PJ_TYPE_USER) k = MAL_TYPE;           /* User has no enum      */
    if (k == MAL_TRUNC && (flags & PJ_GEN_ARRAY)) k = MAL_TYPE;           /* would swallow the rest */
    /* the broken property must actually be written */
    if (k == MAL_ENUM && !(g->present & (g->type == PJ_TYPE_PET ? 1u << 5 : 1u << 4))) k = MAL_TYPE;
    g->mal = (int)k;
    g->mal_pos = (uint32_t)draw(seed, rec, F_MAL_POS, 0);
    if (k == MAL_TYPE) g->present |= 1u, g->nullmask &= ~1u; /* the wrong-typed `id` is written */
  }
}

/* ------------------------------------------------------------------------------------------ */
/* text emitter                                                                                */
/* ------------------------------------------------------------------------------------------ */
typedef struct {
  uint8_t* p; uint64_t cap, n; /* n keeps counting past cap */
  fstream fmt; uint32_t flags;
  int err_kind; uint64_t err_off; /* expected validation result for a malformed record */
  uint64_t rec0;
} emit;

static void put(emit* e, uint8_t c) { if (e->p && e->n < e->cap) e->p[e->n] = c; e->n++; }
static void puts_(emit* e, const char* s) { while (*s) put(e, (uint8_t)*s++); }
static void ws(emit* e) {
  if (!(e->flags & PJ_GEN_WHITESPACE)) return;
  uint64_t r = fnext(&e->fmt);
  uint32_t k = (uint32_t)(r & 7); /* 0,1,2 blanks with p = 1/8 each, else none */
  if (k > 2) return;
  r >>= 3;
  for (uint32_t i = 0; i < k + 1; ++i) { put(e, (uint8_t)" \t\r "[r & 3]); r >>= 2; }
}
static void tok(emit* e, char c) { ws(e); put(e, (uint8_t)c); }

static void put_i64(emit* e, int64_t v) {
  char b[24]; int n = 0;
  uint64_t u = v < 0 ? 0 - (uint64_t)v : (uint64_t)v;
  do { b[n++] = (char)('0' + u % 10); u /= 10; } while (u);
  if (v < 0) put(e, '-');
  while (n) put(e, (uint8_t)b[--n]);
}
static void put_hex4(emit* e, uint32_t u, uint64_t r) {
  static const char lo[] = "0123456789abcdef", up[] = "0123456789ABCDEF";
  put(e, '\\'); put(e, 'u');
  for (int s = 12; s >= 0; s -= 4) { put(e, (uint8_t)(((r >> s) & 1) ? up : lo)[(u >> s) & 15]); }
}
/* JSON string literal of UTF-8 value v; "special" strings mix escaped and raw forms */
static void put_str(emit* e, const gstr* v) {
  put(e, '"');
  uint32_t i = 0;
  while (i < v->n) {
    uint8_t c = v->b[i];
    uint32_t cp = c, len = 1;
    if (c >= 0xF0) { cp = (c & 7u) << 18 | (v->b[i + 1] & 63u) << 12 | (v->b[i + 2] & 63u) << 6 | (v->b[i + 3] & 63u); len = 4; }
    else if (c >= 0xE0) { cp = (c & 15u) << 12 | (v->b[i + 1] & 63u) << 6 | (v->b[i + 2] & 63u); len = 3; }
    else if (c >= 0xC0) { cp = (c & 31u) << 6 | (v->b[i + 1] & 63u); len = 2; }
    uint64_t r = v->special ? fnext(&e->fmt) : 0;
    if (cp == '"' || cp == '\\') {
      if (v->special && (r & 3) == 0) put_hex4(e, cp, r >> 8); else { put(e, '\\'); put(e, (uint8_t)cp); }
    } else if (cp < 0x20) {
      const char* s = NULL;
      if (cp == 8) s = "\\b"; else if (cp == 9) s = "\\t"; else if (cp == 10) s = "\\n";
      else if (cp == 12) s = "\\f"; else if (cp == 13) s = "\\r";
      if (s && (r & 1)) puts_(e, s); else put_hex4(e, cp, r >> 8);
    } else if (cp == '/' && v->special && (r & 1)) {
      put(e, '\\'); put(e, '/');
    } else if (cp < 0x80) {
      if (v->special && (r & 7) == 0) put_hex4(e, cp, r >> 8); else put(e, (uint8_t)cp);
    } else if (v->special && (r & 1)) {
      if (cp >= 0x10000) { uint32_t u = cp - 0x10000; put_hex4(e, 0xD800 + (u >> 10), r >> 8); put_hex4(e, 0xDC00 + (u & 1023), r >> 24); }
      else put_hex4(e, cp, r >> 8);
    } else {
      for (uint32_t k = 0; k < len; ++k) put(e, v->b[i + k]);
    }
    i += len;
  }
  put(e, '"');
}
static void key(emit* e, const char* k, int* first) {
  if (!*first) tok(e, ',');
  *first = 0;
  ws(e); put(e, '"'); puts_(e, k); put(e, '"'); tok(e, ':'); ws(e);
}
static void set_err(emit* e, int kind) {
  if (!e->err_kind) { e->err_kind = kind; e->err_off = e->n - e->rec0; }
}
/* a JSON string cut after `keep` bytes of content: the line ends inside it */
static int put_str_truncated(emit* e, const gstr* v, uint32_t pos) {
  uint32_t keep = v->n ? pos % v->n : 0;
  put(e, '"');
  for (uint32_t i = 0; i < keep; ++i) {
    uint8_t c = v->b[i];
    if (c < 0x20 || c == '"' || c == '\\' || c >= 0x80) break; /* keep the prefix plain ASCII */
    put(e, c);
  }
  set_err(e, PJ_E_EOF);
  e->err_off = 0; /* patched by the caller to the record length */
  return 1;
}

static int emit_pet(emit* e, const grec* g) {
  int first = 1;
  tok(e, '{');
  if ((g->present | g->nullmask) & 1) {
    key(e, "id", &first);
    if (g->nullmask & 1) puts_(e, "null");
    else if (g->mal == MAL_TYPE) { set_err(e, PJ_E_TYPE); put(e, '"'); put_i64(e, g->id); put(e, '"'); }
    else put_i64(e, g->id);
  }
  if ((g->present | g->nullmask) & 2) {
    key(e, "category", &first);
    if (g->nullmask & 2) puts_(e, "null");
    else {
      int f2 = 1;
      put(e, '{');
      if ((g->cat_present | g->cat_null) & 1) { key(e, "id", &f2); if (g->cat_null & 1) puts_(e, "null"); else put_i64(e, g->cat_id); }
      if ((g->cat_present | g->cat_null) & 2) { key(e, "name", &f2); if (g->cat_null & 2) puts_(e, "null"); else put_str(e, &g->cat_name); }
      tok(e, '}');
    }
  }
  int drop = g->mal == MAL_REQUIRED ? (int)(g->mal_pos & 1) : -1; /* 0: name, 1: photoUrls */
  if (drop != 0) {
    key(e, "name", &first);
    if (g->mal == MAL_TRUNC) { put_str_truncated(e, &g->name, g->mal_pos); return 1; }
    put_str(e, &g->name);
  }
  if (drop != 1) {
    key(e, "photoUrls", &first);
    put(e, '[');
    for (uint32_t i = 0; i < g->n_photo; ++i) { if (i) tok(e, ','); ws(e); put_str(e, &g->photo[i]); }
    tok(e, ']');
  }
  if ((g->present | g->nullmask) & 16) {
    key(e, "tags", &first);
    if (g->nullmask & 16) puts_(e, "null");
    else {
      put(e, '[');
      for (uint32_t i = 0; i < g->n_tags; ++i) {
        int f2 = 1;
        if (i) tok(e, ',');
        tok(e, '{'); key(e, "id", &f2); put_i64(e, g->tags[i].id); key(e, "name", &f2); put_str(e, &g->tags[i].name); tok(e, '}');
      }
      tok(e, ']');
    }
  }
  if ((g->present | g->nullmask) & 32) {
    key(e, "status", &first);
    if (g->nullmask & 32) puts_(e, "null");
    else if (g->mal == MAL_ENUM) { set_err(e, PJ_E_ENUM); puts_(e, "\"unknown\""); }
    else { put(e, '"'); puts_(e, PET_STATUS[g->status]); put(e, '"'); }
  }
  ws(e);
  if (drop >= 0) set_err(e, PJ_E_REQUIRED);
  put(e, '}');
  return 0;
}

static int emit_order(emit* e, const grec* g) {
  int first = 1;
  uint32_t w = g->present | g->nullmask;
  tok(e, '{');
  if (w & 1) {
    key(e, "id", &first);
    if (g->nullmask & 1) puts_(e, "null");
    else if (g->mal == MAL_TYPE) { set_err(e, PJ_E_TYPE); puts_(e, "true"); }
    else put_i64(e, g->id);
  }
  if (w & 2) { key(e, "petId", &first); if (g->nullmask & 2) puts_(e, "null"); else put_i64(e, g->pet_id); }
  if (w & 4) { key(e, "quantity", &first); if (g->nullmask & 4) puts_(e, "null"); else put_i64(e, g->quantity); }
  if (w & 8) {
    key(e, "shipDate", &first);
    if (g->nullmask & 8) puts_(e, "null");
    else if (g->mal == MAL_TRUNC) { gstr t; t.n = (uint32_t)strlen(g->ship_text); memcpy(t.b, g->ship_text, t.n); t.special = 0; put_str_truncated(e, &t, g->mal_pos); return 1; }
    else { put(e, '"'); puts_(e, g->ship_text); put(e, '"'); }
  }
  if (w & 16) {
    key(e, "status", &first);
    if (g->nullmask & 16) puts_(e, "null");
    else if (g->mal == MAL_ENUM) { set_err(e, PJ_E_ENUM); puts_(e, "\"sold\""); } /* a Pet literal, not an Order one */
    else { put(e, '"'); puts_(e, ORD_STATUS[g->status]); put(e, '"'); }
  }
  if (w & 32) { key(e, "complete", &first); if (g->nullmask & 32) puts_(e, "null"); else puts_(e, g->complete ? "true" : "false"); }
  tok(e, '}');
  return 0;
}

static const char* const USER_KEYS[6] = {"username", "firstName", "lastName", "email", "password", "phone"};

static int emit_user(emit* e, const grec* g) {
  int first = 1;
  uint32_t w = g->present | g->nullmask;
  tok(e, '{');
  if (w & 1) {
    key(e, "id", &first);
    if (g->nullmask & 1) puts_(e, "null");
    else if (g->mal == MAL_TYPE) { set_err(e, PJ_E_TYPE); puts_(e, "[1]"); }
    else put_i64(e, g->id);
  }
  for (uint32_t f = 0; f < 6; ++f) {
    if (!(w & (2u << f))) continue;
    key(e, USER_KEYS[f], &first);
    if (g->nullmask & (2u << f)) puts_(e, "null");
    else if (g->mal == MAL_TRUNC && f == 0) { put_str_truncated(e, &g->u_str[0], g->mal_pos); return 1; }
    else put_str(e, &g->u_str[f]);
  }
  if (w & 128) { key(e, "userStatus", &first); if (g->nullmask & 128) puts_(e, "null"); else put_i64(e, g->user_status); }
  tok(e, '}');
  return 0;
}

/* emits one record; returns expected (err_kind, err_off) through e */
static void emit_record(emit* e, const grec* g, uint64_t seed, uint64_t rec) {
  e->fmt.s = draw(seed, rec, F_FMT, 0);
  e->err_kind = 0; e->err_off = 0; e->rec0 = e->n;
  int truncated;
  /* MAL_TRUNC needs its carrier property written: Pet.name always is; for Order / User fall back */
  grec* gm = (grec*)g;
  if (g->mal == MAL_TRUNC && g->type == PJ_TYPE_ORDER && !(g->present & 8)) gm->present |= 8, gm->nullmask &= ~8u;
  if (g->mal == MAL_TRUNC && g->type == PJ_TYPE_USER && !(g->present & 2)) gm->present |= 2, gm->nullmask &= ~2u;
  if (g->type == PJ_TYPE_PET) truncated = emit_pet(e, g);
  else if (g->type == PJ_TYPE_ORDER) truncated = emit_order(e, g);
  else truncated = emit_user(e, g);
  if (truncated) e->err_off = e->n - e->rec0;
  else ws(e);
}

pj_status pj_gen_text(uint32_t schema, uint64_t seed, uint64_t first, uint64_t n, uint32_t flags,
                      uint8_t* text, uint64_t cap, uint64_t* len) {
  if (!len || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return PJ_ERR_ARG;
  grec* g = (grec*)malloc(sizeof(grec));
  if (!g) return PJ_ERR_NOMEM;
  emit e; memset(&e, 0, sizeof e);
  e.p = text; e.cap = text ? cap : 0; e.flags = flags;
  if (flags & PJ_GEN_ARRAY) put(&e, '[');
  for (uint64_t k = 0; k < n; ++k) {
    gen_record(g, schema, seed, first + k, flags);
    if ((flags & PJ_GEN_ARRAY) && k) put(&e, ',');
    emit_record(&e, g, seed, first + k);
    if (!(flags & PJ_GEN_ARRAY)) put(&e, '\n');
  }
  if (flags & PJ_GEN_ARRAY) put(&e, ']');
  free(g);
  *len = e.n;
  return (text && e.n > cap) ? PJ_ERR_CAPACITY : PJ_OK;
}

/* ------------------------------------------------------------------------------------------ */
/* column emitter                                                                              */
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
/* append a string to (off_col, data_col) at row `row`; writes off[row] and off[row+1] */
static void w_str(colw* w, int off_col, int data_col, uint64_t row, const uint8_t* s, uint32_t n) {
  uint64_t at = w->used[data_col];
  w_u32(w, off_col, row, (uint32_t)at);
  for (uint32_t i = 0; i < n; ++i) w_u8(w, data_col, at + i, s[i]);
  w_u32(w, off_col, row + 1, (uint32_t)(at + n));
}

static const int USR_OFF_COLS[6] = {PJ_COL_USR_USERNAME_OFF, PJ_COL_USR_FIRSTNAME_OFF, PJ_COL_USR_LASTNAME_OFF,
                                    PJ_COL_USR_EMAIL_OFF, PJ_COL_USR_PASSWORD_OFF, PJ_COL_USR_PHONE_OFF};

static void col_pet(colw* w, const grec* g, uint64_t row, int failed) {
  uint64_t P = w->used[PJ_COL_PET_PHOTO_STR_OFF] ? w->used[PJ_COL_PET_PHOTO_STR_OFF] - 1 : 0;
  uint64_t T = w->used[PJ_COL_PET_TAG_NAME_OFF] ? w->used[PJ_COL_PET_TAG_NAME_OFF] - 1 : 0;
  uint32_t pr = failed ? 0 : g->present;
  uint32_t cp = (pr & 2) ? g->cat_present : 0;
  w_u8(w, PJ_COL_PET_PRESENT, row, (uint8_t)pr);
  w_i64(w, PJ_COL_PET_ID, row, (pr & 1) ? g->id : 0);
  w_u8(w, PJ_COL_PET_CAT_PRESENT, row, (uint8_t)cp);
  w_i64(w, PJ_COL_PET_CAT_ID, row, (cp & 1) ? g->cat_id : 0);
  w_str(w, PJ_COL_PET_CAT_NAME_OFF, PJ_COL_PET_CAT_NAME_DATA, row, g->cat_name.b, (cp & 2) ? g->cat_name.n : 0);
  w_str(w, PJ_COL_PET_NAME_OFF, PJ_COL_PET_NAME_DATA, row, g->name.b, (pr & 4) ? g->name.n : 0);
  w_u32(w, PJ_COL_PET_PHOTO_OFF, row, (uint32_t)P);
  if (!w->used[PJ_COL_PET_PHOTO_STR_OFF]) w_u32(w, PJ_COL_PET_PHOTO_STR_OFF, 0, 0);
  if (pr & 8) for (uint32_t i = 0; i < g->n_photo; ++i) w_str(w, PJ_COL_PET_PHOTO_STR_OFF, PJ_COL_PET_PHOTO_DATA, P + i, g->photo[i].b, g->photo[i].n);
  w_u32(w, PJ_COL_PET_PHOTO_OFF, row + 1, (uint32_t)(P + ((pr & 8) ? g->n_photo : 0)));
  w_u32(w, PJ_COL_PET_TAGS_OFF, row, (uint32_t)T);
  if (!w->used[PJ_COL_PET_TAG_NAME_OFF]) w_u32(w, PJ_COL_PET_TAG_NAME_OFF, 0, 0);
  if (pr & 16) for (uint32_t i = 0; i < g->n_tags; ++i) {
    w_u8(w, PJ_COL_PET_TAG_PRESENT, T + i, 3);
    w_i64(w, PJ_COL_PET_TAG_ID, T + i, g->tags[i].id);
    w_str(w, PJ_COL_PET_TAG_NAME_OFF, PJ_COL_PET_TAG_NAME_DATA, T + i, g->tags[i].name.b, g->tags[i].name.n);
  }
  w_u32(w, PJ_COL_PET_TAGS_OFF, row + 1, (uint32_t)(T + ((pr & 16) ? g->n_tags : 0)));
  w_u8(w, PJ_COL_PET_STATUS, row, (pr & 32) ? g->status : 255);
}
static void col_order(colw* w, const grec* g, uint64_t row, int failed) {
  uint32_t pr = failed ? 0 : g->present;
  w_u8(w, PJ_COL_ORD_PRESENT, row, (uint8_t)pr);
  w_i64(w, PJ_COL_ORD_ID, row, (pr & 1) ? g->id : 0);
  w_i64(w, PJ_COL_ORD_PET_ID, row, (pr & 2) ? g->pet_id : 0);
  w_i32(w, PJ_COL_ORD_QUANTITY, row, (pr & 4) ? g->quantity : 0);
  w_i64(w, PJ_COL_ORD_SHIP_EPOCH, row, (pr & 8) ? g->ship_epoch : 0);
  w_i32(w, PJ_COL_ORD_SHIP_NANOS, row, (pr & 8) ? g->ship_nanos : 0);
  w_i32(w, PJ_COL_ORD_SHIP_OFFSET, row, (pr & 8) ? g->ship_off : 0);
  w_u8(w, PJ_COL_ORD_STATUS, row, (pr & 16) ? g->status : 255);
  w_u8(w, PJ_COL_ORD_COMPLETE, row, (pr & 32) ? g->complete : 0);
}
static void col_user(colw* w, const grec* g, uint64_t row, int failed) {
  uint32_t pr = failed ? 0 : g->present;
  w_u8(w, PJ_COL_USR_PRESENT, row, (uint8_t)pr);
  w_i64(w, PJ_COL_USR_ID, row, (pr & 1) ? g->id : 0);
  for (uint32_t f = 0; f < 6; ++f)
    w_str(w, USR_OFF_COLS[f], USR_OFF_COLS[f] + 1, row, g->u_str[f].b, (pr & (2u << f)) ? g->u_str[f].n : 0);
  w_i32(w, PJ_COL_USR_STATUS, row, (pr & 128) ? g->user_status : 0);
}

static const int PET_OFF_COLS[] = {PJ_COL_PET_CAT_NAME_OFF, PJ_COL_PET_NAME_OFF, PJ_COL_PET_PHOTO_OFF,
                                   PJ_COL_PET_PHOTO_STR_OFF, PJ_COL_PET_TAGS_OFF, PJ_COL_PET_TAG_NAME_OFF};

pj_status pj_gen_columns(uint32_t schema, uint64_t seed, uint64_t first, uint64_t n, uint32_t flags,
                         pj_columns* out) {
  if (!out || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return PJ_ERR_ARG;
  grec* g = (grec*)malloc(sizeof(grec));
  if (!g) return PJ_ERR_NOMEM;
  colw w; memset(&w, 0, sizeof w); w.c = out;
  emit e; memset(&e, 0, sizeof e); e.flags = flags; /* length-only pass: offsets and expected errors */
  uint64_t rows[4] = {0, 0, 0, 0}, n_err = 0;
  int mixed = schema == PJ_SCHEMA_MIXED;
  if (flags & PJ_GEN_ARRAY) put(&e, '[');
  /* empty tables still carry their leading 0 offset */
  if (schema == PJ_SCHEMA_PET || mixed) for (size_t i = 0; i < sizeof PET_OFF_COLS / sizeof(int); ++i) w_u32(&w, PET_OFF_COLS[i], 0, 0);
  if (schema == PJ_SCHEMA_USER || mixed) for (uint32_t f = 0; f < 6; ++f) w_u32(&w, USR_OFF_COLS[f], 0, 0);
  for (uint64_t k = 0; k < n; ++k) {
    gen_record(g, schema, seed, first + k, flags);
    if ((flags & PJ_GEN_ARRAY) && k) put(&e, ',');
    uint64_t start = e.n;
    emit_record(&e, g, seed, first + k);
    if (!(flags & PJ_GEN_ARRAY)) put(&e, '\n');
    int failed = e.err_kind != 0;
    n_err += (uint64_t)failed;
    w_u64(&w, PJ_COL_REC_START, k, start);
    w_u8(&w, PJ_COL_ERR_KIND, k, (uint8_t)e.err_kind);
    w_u32(&w, PJ_COL_ERR_OFF, k, (uint32_t)e.err_off);
    if (mixed) {
      w_u8(&w, PJ_COL_REC_TYPE, k, failed ? PJ_TYPE_NONE : (uint8_t)g->type);
      w_u32(&w, PJ_COL_REC_ROW, k, failed ? 0xFFFFFFFFu : (uint32_t)rows[g->type]);
      if (failed) continue;
    }
    uint64_t row = rows[g->type]++;
    if (g->type == PJ_TYPE_PET) col_pet(&w, g, row, failed);
    else if (g->type == PJ_TYPE_ORDER) col_order(&w, g, row, failed);
    else col_user(&w, g, row, failed);
  }
  free(g);
  out->schema = schema;
  out->n_records = n;
  out->n_errors = n_err;
  for (int t = 0; t < 4; ++t) out->n_rows[t] = rows[t];
  for (int c = 0; c < PJ_MAX_COLS; ++c) out->col[c].count = w.used[c];
  return w.overflow ? PJ_ERR_CAPACITY : PJ_OK;
}
