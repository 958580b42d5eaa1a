/*
 * pj_lock.cuh — the lockstep tokeniser: the first attempt at every staged record of the stream kernel.
 *
 * One thread owns one record, as in pj_fast.cuh, but the 32 records of a warp are walked IN STEP. The code has one
 * shape: every property of the model is tried once, in model order; every loop has a single exit; nothing returns
 * from the middle of a record. A lane whose record stops matching only clears its state flag and idles through
 * the remaining steps, so the lanes of a warp meet again after every property and every list element instead of
 * drifting apart for the rest of the record (which is what early returns out of nested loops cost the
 * word-at-a-time tokeniser: it ran with a third of its lanes).
 *
 * It only ACCEPTS or REFUSES, it never reports a failure. Accepted: the canonical spelling a serialiser emits — no
 * blanks between tokens, properties in model order (any of them may be missing), no `null`, plain strings
 * (printable ASCII without backslash), non-negative integers in range, the line feed directly after the closing
 * brace. Everything else (blanks, escapes, UTF-8, other key orders, every malformed record) is refused and goes to
 * fast_record<>() and from there, if need be, to the exact parser; so what this file accepts it must decode exactly
 * as they do. Output is what fast_record<>() leaves: values in registers, strings and list elements on the tape,
 * counts per slot. A host build of this header is fuzzed against the CPU checker.
 */
#ifndef PJ_LOCK_CUH
#define PJ_LOCK_CUH

#include "pj_fast.cuh"

namespace pj {

enum { LK_REFUSED = 0, LK_MEMBER = 1, LK_CLOSED = 2 };
struct LkState {
  uint32_t p;  /* window offset */
  uint32_t st; /* LK_MEMBER: at the first byte of a member; LK_CLOSED: past the closing brace; LK_REFUSED */
};

PJ_HD uint32_t lk_ctz32(uint32_t x) {
#if defined(__CUDA_ARCH__)
  return (uint32_t)(__ffs((int)x) - 1);
#else
  return (uint32_t)__builtin_ctz(x);
#endif
}

/* 0x80 in every byte of x that ends a plain string run: '"', '\\', below 0x20, above 0x7F (exact, byte by byte) */
PJ_HD uint32_t lk_special4(uint32_t x) {
  const uint32_t ge20 = (x & 0x7F7F7F7Fu) + 0x60606060u; /* bit 7: the low seven bits are >= 0x20 */
  const uint32_t tq = x ^ 0x22222222u, nq = ((tq & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | tq; /* bit 7: not '"' */
  const uint32_t tb = x ^ 0x5C5C5C5Cu, nb = ((tb & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | tb; /* bit 7: not '\\' */
  return (~(ge20 & nq & nb) | x) & 0x80808080u;
}

/* Window offset of the first byte at or after p that ends a plain string run. Every staged record is followed by a
 * line feed (its own, or the padding behind the window), so the scan ends. Four aligned words a round. */
PJ_HD uint32_t lk_scan(const Win& w, uint32_t p) {
  const uint32_t* a = reinterpret_cast<const uint32_t*>(w.s) + (p >> 2);
  uint32_t first_mask = 0xFFFFFFFFu << ((p & 3u) * 8u); /* bytes of the first word before p do not count */
  uint32_t base = p & ~3u, f = 0;
  while (!f) {
    const uint32_t f0 = lk_special4(a[0]) & first_mask, f1 = lk_special4(a[1]), f2 = lk_special4(a[2]), f3 = lk_special4(a[3]);
    first_mask = 0xFFFFFFFFu;
    if (f0 | f1 | f2 | f3) {
      if (f0) f = f0;
      else if (f1) { f = f1; base += 4; }
      else if (f2) { f = f2; base += 8; }
      else { f = f3; base += 12; }
    } else { a += 4; base += 16; }
  }
  return base + (lk_ctz32(f) >> 3);
}

/* A non-negative integer at p: 0 | [1-9][0-9]{0,18}, within int64 / int32, not followed by '.', 'e', 'E'. On
 * success p moves past it. (A minus sign, like everything else, is refused: the word-at-a-time path takes it.) */
PJ_HD bool lk_int(const Win& w, uint32_t& p, bool is64, int64_t* out) {
  uint32_t q = p;
  uint64_t x = wpeek8(w, q);
  uint64_t m = swar_nondigit(x);
  uint64_t mag = 0;
  uint32_t nd = 0;
  bool ok = true;
  if (!m) { /* eight digits, and maybe eight more */
    mag = swar_parse8(x); nd = 8; q += 8;
    x = wpeek8(w, q); m = swar_nondigit(x);
    if (!m) {
      mag = mag * 100000000u + swar_parse8(x); nd = 16; q += 8;
      x = wpeek8(w, q); m = swar_nondigit(x);
      if (!m) ok = false; /* 24 digits and more */
    }
  }
  const uint32_t k = m ? ctz64(m) >> 3 : 0u; /* digits of the last group */
  if (k) {
    uint32_t scale = (k & 1) ? 10u : 1u;
    if (k & 2) scale *= 100u;
    if (k & 4) scale *= 10000u;
    mag = mag * scale + swar_parse_k(x, k);
  }
  nd += k; q += k;
  const uint32_t first = wbyte(w, p), t = wbyte(w, q);
  const uint64_t lim = is64 ? 0x7FFFFFFFFFFFFFFFull : 0x7FFFFFFFull;
  ok = ok && nd != 0 && nd <= 19 && !(first == '0' && nd > 1) && mag <= lim && t != '.' && (t | 0x20u) != 'e';
  *out = (int64_t)mag;
  if (ok) p = q;
  return ok;
}

/* A plain string at p (its opening quote): content offset and length; p moves past the closing quote. */
PJ_HD bool lk_string(const Win& w, uint32_t& p, uint32_t* pos, uint32_t* len) {
  const uint32_t q = lk_scan(w, p + 1);
  const uint32_t n = q - (p + 1);
  const bool ok = wbyte(w, q) == '"' && n <= TAPE_MAX_STR;
  *pos = p + 1; *len = n;
  if (ok) p = q + 1;
  return ok;
}

/* Scalar property I of OBJ at f.p (the byte after the colon). Clears f.st when the value is not of the accepted form. */
template <int OBJ, int I>
PJ_HD void lk_scalar(const Win& w, LkState& f, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v) {
  constexpr uint32_t kind = FK<OBJ, I>::kind, slot = FK<OBJ, I>::cnt;
  bool ok = false;
  if constexpr (kind == K_I64 || kind == K_I32) {
    int64_t val = 0;
    ok = lk_int(w, f.p, kind == K_I64, &val);
    v.v[I] = val;
  } else if constexpr (kind == K_BOOL) {
    const uint64_t k = wpeek8(w, f.p);
    if ((k & 0xFFFFFFFFull) == 0x65757274ull) { v.v[I] = 1; f.p += 4; ok = true; }
    else if ((k & 0xFFFFFFFFFFull) == 0x65736C6166ull) { v.v[I] = 0; f.p += 5; ok = true; }
  } else if constexpr (kind == K_STR) {
    if (wbyte(w, f.p) == '"') {
      uint32_t pos, len;
      ok = lk_string(w, f.p, &pos, &len);
      if (ok) { tape_push(t, tape_str(slot, len, pos, 0)); cnt[slot] += len; }
    }
  } else if constexpr (kind == K_ENUM) {
    if (wbyte(w, f.p) == '"') {
      FastState fs;
      fs.p = f.p; fs.limit = limit; fs.lf_ws = 0; fs.err = 0; fs.err_pos = 0;
      uint32_t len; uint64_t lo, hi;
      if (fast_short(w, fs, &len, &lo, &hi)) {
        const int e = match_enum<FK<OBJ, I>::child>(len, lo, hi);
        if (e >= 0) { v.v[I] = e; f.p = fs.p; ok = true; }
      }
    }
  } else if constexpr (kind == K_DATETIME) {
    if (wbyte(w, f.p) == '"') {
      uint32_t q = f.p, pos, len;
      if (lk_string(w, q, &pos, &len)) {
        int64_t ep; int32_t ns, of;
        if (fast_datetime(w, pos, len, &ep, &ns, &of)) {
          v.v[I] = ep; v.aux = (int64_t)(((uint64_t)(uint32_t)ns << 32) | (uint32_t)of);
          f.p = q; ok = true;
        }
      }
    }
  }
  if (ok) v.present |= 1u << I; else f.st = LK_REFUSED;
}

/* after a value: ',' (another member follows), '}' (the object is closed), anything else is refused */
PJ_HD void lk_member_end(const Win& w, LkState& f) {
  const uint32_t x = wbyte(w, f.p);
  f.p++;
  f.st = x == ',' ? (uint32_t)LK_MEMBER : (x == '}' ? (uint32_t)LK_CLOSED : (uint32_t)LK_REFUSED);
}

/* is the compact spelling `"name":` of property I at p? */
template <int OBJ, int I>
PJ_HD bool lk_key(const Win& w, uint32_t p) {
  bool hit = (wpeek8(w, p) & FK<OBJ, I>::mask0) == FK<OBJ, I>::pat0;
  if constexpr (FK<OBJ, I>::pat_len > 8) hit = hit && (wpeek8(w, p + 8) & FK<OBJ, I>::mask1) == FK<OBJ, I>::pat1;
  return hit;
}

/* ---- flat objects (Category, Tag): scalar properties only, in model order ---------------------------------- */
template <int OBJ, int I = 0>
PJ_HD void lk_flat_members(const Win& w, LkState& f, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v) {
  if constexpr (I < CObj<OBJ>::N) {
    if (f.st == LK_MEMBER && lk_key<OBJ, I>(w, f.p)) {
      f.p += FK<OBJ, I>::pat_len;
      if constexpr (FK<OBJ, I>::kind <= K_ENUM) lk_scalar<OBJ, I>(w, f, limit, t, cnt, v); else f.st = LK_REFUSED;
      if (f.st != LK_REFUSED) lk_member_end(w, f);
    }
    lk_flat_members<OBJ, I + 1>(w, f, limit, t, cnt, v);
  }
}
/* Flat object at p ('{'). True when it was closed in the accepted form; p then is past its brace. */
template <int OBJ>
PJ_HD bool lk_flat(const Win& w, uint32_t& p, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v) {
  v.present = 0;
  LkState f;
  f.p = p + 1; f.st = LK_MEMBER;
  if (wbyte(w, f.p) == '}') { f.p++; f.st = LK_CLOSED; }
  lk_flat_members<OBJ>(w, f, limit, t, cnt, v);
  const bool ok = f.st == LK_CLOSED;
  if (ok) p = f.p;
  return ok;
}

/* ---- model roots ---------------------------------------------------------------------------------------------- */
/* value of property I of root OBJ at f.p */
template <int OBJ, int I>
PJ_HD void lk_root_value(const Win& w, LkState& f, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v, FVals& cv) {
  constexpr uint32_t kind = FK<OBJ, I>::kind, slot = FK<OBJ, I>::cnt;
  if constexpr (kind <= K_ENUM || kind == K_DATETIME) lk_scalar<OBJ, I>(w, f, limit, t, cnt, v);
  else if constexpr (kind == K_OBJ) {
    bool ok = false;
    if (wbyte(w, f.p) == '{') ok = lk_flat<FK<OBJ, I>::child>(w, f.p, limit, t, cnt, cv);
    if (ok) v.present |= 1u << I; else f.st = LK_REFUSED;
  } else {
    /* a list: `[]`, or elements separated by single commas */
    bool ok = wbyte(w, f.p) == '[';
    bool more = ok;
    uint32_t j = 0;
    f.p++;
    if (more && wbyte(w, f.p) == ']') { f.p++; more = false; }
    while (more) {
      bool item = false;
      if constexpr (kind == K_LIST_STR) {
        if (wbyte(w, f.p) == '"') {
          uint32_t pos, len;
          item = lk_string(w, f.p, &pos, &len);
          if (item) { tape_push(t, tape_str(slot + 1, len, pos, 0)); cnt[slot + 1] += len; }
        }
      } else {
        constexpr int E = FK<OBJ, I>::child;
        if (wbyte(w, f.p) == '{') {
          /* header word and room for the scalars, then the element's strings as they are met */
          const uint32_t at = t.n;
          for (uint32_t k = 0; k < 1 + scalar_words<E>(); ++k) tape_push(t, 0);
          FVals ev;
          item = lk_flat<E>(w, f.p, limit, t, cnt, ev);
          if (item) {
            tape_set(t, at, (uint32_t)TAPE_ELEM | (ev.present << 4) | (slot << 12));
            tape_put_scalars<E>(t, at + 1, ev);
          }
        }
      }
      if (item) {
        j++;
        const uint32_t x = wbyte(w, f.p);
        f.p++;
        if (x != ',') { more = false; ok = x == ']'; }
      } else { more = false; ok = false; }
    }
    cnt[slot] = j;
    if (ok) v.present |= 1u << I; else f.st = LK_REFUSED;
  }
}
/* the members of root OBJ from property I on, each tried once, in model order */
template <int OBJ, int I = 0>
PJ_HD void lk_root_members(const Win& w, LkState& f, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v, FVals& cv) {
  if constexpr (I < CObj<OBJ>::N) {
    if (f.st == LK_MEMBER && lk_key<OBJ, I>(w, f.p)) {
      f.p += FK<OBJ, I>::pat_len;
      lk_root_value<OBJ, I>(w, f, limit, t, cnt, v, cv);
      if (f.st != LK_REFUSED) lk_member_end(w, f);
    }
    lk_root_members<OBJ, I + 1>(w, f, limit, t, cnt, v, cv);
  }
}

/* Mixed streams. The `id` that the three models share (property 0 of each) may come first ... */
PJ_HD void lk_common_id(const Win& w, LkState& f, FVals& v) {
  static_assert(FK<OBJ_PET, 0>::kind == K_I64 && FK<OBJ_ORDER, 0>::kind == K_I64 && FK<OBJ_USER, 0>::kind == K_I64, "id leads every model");
  if (f.st == LK_MEMBER && lk_key<OBJ_PET, 0>(w, f.p)) {
    f.p += FK<OBJ_PET, 0>::pat_len;
    int64_t val = 0;
    if (lk_int(w, f.p, true, &val)) { v.v[0] = val; v.present |= 1u; lk_member_end(w, f); }
    else f.st = LK_REFUSED;
  }
}
/* ... and the key after it decides the model. This looks at three letters of it only (c0, c1, c3 = first, second and
 * fourth letter): the model's own key compare then accepts the record or refuses it. `status` (Pet and Order have
 * one) and anything unknown decide nothing: 0. */
PJ_HD uint32_t lk_guess_owner(uint32_t c0, uint32_t c1, uint32_t c3) {
  switch (c0) {
    case 'c': return c1 == 'a' ? (uint32_t)PJ_TYPE_PET : (uint32_t)PJ_TYPE_ORDER; /* category | complete */
    case 'n': case 't': return PJ_TYPE_PET;                                        /* name, tags */
    case 'q': return PJ_TYPE_ORDER;                                                /* quantity */
    case 'u': case 'f': case 'l': case 'e': return PJ_TYPE_USER;                   /* username, userStatus, firstName, lastName, email */
    case 's': return c1 == 'h' ? (uint32_t)PJ_TYPE_ORDER : 0u;                     /* shipDate | status */
    case 'p': return c1 == 'e' ? (uint32_t)PJ_TYPE_ORDER : (c1 == 'a' ? (uint32_t)PJ_TYPE_USER : (c3 == 't' ? (uint32_t)PJ_TYPE_PET : (uint32_t)PJ_TYPE_USER)); /* petId | password | photoUrls | phone */
    default: return 0;
  }
}

/* One record at window offset `start` (the first byte of its line); `limit` = window offset of the first byte that
 * is not input. Returns true when the record is accepted: model in *type_out, values in v / cv, counts in cnt[]
 * (all NSLOT entries are reset either way), strings and list elements on the tape; t.n > t.cap afterwards means
 * the tape was too small, as with fast_record<>(). `live` = false lets a lane without a record walk along. */
template <int SCHEMA>
PJ_HD bool lock_record(const Win& w, bool live, uint32_t start, uint32_t limit, uint32_t open_end, uint32_t* type_out, FVals& v, FVals& cv,
                       uint32_t* cnt, Tape& t) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (uint32_t k = 0; k < NSLOT; ++k) cnt[k] = 0;
  t.n = 0;
  v.present = 0; cv.present = 0;
  LkState f;
  f.p = start;
  f.st = live && wbyte(w, start) == '{' ? (uint32_t)LK_MEMBER : (uint32_t)LK_REFUSED;
  f.p++;
  uint32_t type = PJ_TYPE_NONE;
  if constexpr (SCHEMA != PJ_SCHEMA_MIXED) {
    constexpr int OBJ = RootOf<SCHEMA>::obj;
    if (f.st == LK_MEMBER && wbyte(w, f.p) == '}') { f.p++; f.st = LK_CLOSED; }
    lk_root_members<OBJ>(w, f, limit, t, cnt, v, cv);
    if ((v.present & CObj<OBJ>::required) != (uint32_t)CObj<OBJ>::required) f.st = LK_REFUSED;
    type = SCHEMA;
  } else {
    /* the common `id` may come first; the key after it decides the model (a `status` there does not: refused) */
    lk_common_id(w, f, v);
    uint32_t guess = 0;
    if (f.st == LK_MEMBER && wbyte(w, f.p) == '"') guess = lk_guess_owner(wbyte(w, f.p + 1), wbyte(w, f.p + 2), wbyte(w, f.p + 4));
    if (guess == PJ_TYPE_PET) {
      lk_root_members<OBJ_PET, 1>(w, f, limit, t, cnt, v, cv);
      if ((v.present & CObj<OBJ_PET>::required) != (uint32_t)CObj<OBJ_PET>::required) f.st = LK_REFUSED;
      cnt[SLOT_ROWS_PET] = 1;
    } else if (guess == PJ_TYPE_ORDER) {
      lk_root_members<OBJ_ORDER, 1>(w, f, limit, t, cnt, v, cv);
      cnt[SLOT_ROWS_ORD] = 1;
    } else if (guess == PJ_TYPE_USER) {
      lk_root_members<OBJ_USER, 1>(w, f, limit, t, cnt, v, cv);
      cnt[SLOT_ROWS_USR] = 1;
    } else f.st = LK_REFUSED;
    type = guess;
  }
  /* the line feed that ends the line must follow at once (the padding behind the input looks like one; there the
     record is complete only if the stream ends there too) */
  const bool ok = f.st == LK_CLOSED && wbyte(w, f.p) == '\n' && (f.p < limit || (f.p == limit && !open_end));
  *type_out = ok ? type : (uint32_t)PJ_TYPE_NONE;
  return ok;
}

}  // namespace pj
#endif
