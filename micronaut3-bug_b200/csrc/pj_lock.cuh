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
 * Accepted: the canonical spelling a serialiser emits — no blanks between tokens, properties in model order (any of
 * them may be missing), no `null`, plain strings (printable ASCII without backslash), non-negative integers in range,
 * the line feed directly after the closing brace. Reported as failed, with the kind and offset the exact parser
 * gives: the common validation failures of such records (a value of the wrong JSON type, an unknown enum literal, a
 * bad date-time, a missing required property, the line ending inside a string). Everything else (blanks, escapes,
 * UTF-8, other key orders, other malformations) is refused and goes to fast_record<>() and from there, if need be, to
 * the exact parser; so what this file accepts or fails it must decode or report exactly as they do. Output is what fast_record<>() leaves: values in registers, strings and list elements on the tape,
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
  uint32_t err, err_pos; /* a validation failure found here (kind, window offset); 0 = none */
};
/* The record fails validation, in one of the ways fast_record<>() reports itself and exactly as it reports them
 * (everything before this point was accepted, so this is the first failure in reading order). The lane stops. */
PJ_HD void lk_fail(LkState& f, uint32_t kind, uint32_t pos) { f.st = LK_REFUSED; f.err = kind; f.err_pos = pos; }
/* The byte x at f.p cannot start a value of the expected type: PJ_E_TYPE when it starts a value of another type;
 * null, the end of the record and stray bytes are refused (the exact parser decides). */
PJ_HD void lk_wrong_type(LkState& f, uint32_t limit, uint32_t x) {
  if (f.p < limit && (x == '"' || x == '-' || x - '0' <= 9u || x == '{' || x == '[' || x == 't' || x == 'f')) lk_fail(f, PJ_E_TYPE, f.p);
  else f.st = LK_REFUSED;
}

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

/* A plain string at f.p (its opening quote): content offset and length; f.p moves past the closing quote. A line
 * feed before the closing quote (the record's bytes end inside the string) is the failure PJ_E_EOF there; any
 * other byte that ends the plain run is refused. False unless the string was accepted. */
PJ_HD bool lk_string(const Win& w, LkState& f, uint32_t limit, uint32_t* pos, uint32_t* len) {
  const uint32_t q = lk_scan(w, f.p + 1);
  const uint32_t n = q - (f.p + 1);
  const uint32_t x = wbyte(w, q);
  const bool ok = x == '"' && n <= TAPE_MAX_STR && q < limit;
  *pos = f.p + 1; *len = n;
  if (ok) f.p = q + 1;
  else if (x == '\n' && q < limit) lk_fail(f, PJ_E_EOF, q);
  else f.st = LK_REFUSED;
  return ok;
}

/* Scalar property I of OBJ at f.p (the byte after the colon). Stops the lane (refused, or failed with kind and
 * offset) when the value is not of the accepted form. */
template <int OBJ, int I>
PJ_HD void lk_scalar(const Win& w, LkState& f, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v) {
  constexpr uint32_t kind = FK<OBJ, I>::kind, slot = FK<OBJ, I>::cnt;
  const uint32_t x = wbyte(w, f.p);
  bool ok = false;
  if constexpr (kind == K_I64 || kind == K_I32) {
    if (x - '0' <= 9u) {
      int64_t val = 0;
      ok = lk_int(w, f.p, kind == K_I64, &val);
      v.v[I] = val;
      if (!ok) f.st = LK_REFUSED;
    } else if (x == '-' || x == 'n') f.st = LK_REFUSED;
    else lk_wrong_type(f, limit, x);
  } else if constexpr (kind == K_BOOL) {
    const uint64_t k = wpeek8(w, f.p);
    if ((k & 0xFFFFFFFFull) == 0x65757274ull) { v.v[I] = 1; f.p += 4; ok = true; }
    else if ((k & 0xFFFFFFFFFFull) == 0x65736C6166ull) { v.v[I] = 0; f.p += 5; ok = true; }
    else if (x != 't' && x != 'f' && x != 'n') lk_wrong_type(f, limit, x);
    else f.st = LK_REFUSED;
  } else if constexpr (kind == K_STR) {
    if (x == '"') {
      uint32_t pos, len;
      ok = lk_string(w, f, limit, &pos, &len);
      if (ok) { tape_push(t, tape_str(slot, len, pos, 0)); cnt[slot] += len; }
    } else if (x == 'n') f.st = LK_REFUSED;
    else lk_wrong_type(f, limit, x);
  } else if constexpr (kind == K_ENUM) {
    if (x == '"') {
      /* a plain string that is no literal fails with PJ_E_ENUM at its opening quote */
      const uint32_t q0 = f.p;
      uint32_t pos, len;
      if (lk_string(w, f, limit, &pos, &len)) {
        int e = -1;
        if (len <= 14) {
          const uint64_t a = wpeek8(w, pos), b = wpeek8(w, pos + 8);
          const uint64_t lo = len >= 8 ? a : (len ? a & (~0ull >> (64 - 8 * len)) : 0);
          const uint64_t hi = len > 8 ? b & (~0ull >> (64 - 8 * (len - 8))) : 0;
          e = match_enum<FK<OBJ, I>::child>(len, lo, hi);
        }
        if (e >= 0) { v.v[I] = e; ok = true; } else lk_fail(f, PJ_E_ENUM, q0);
      }
    } else if (x == 'n') f.st = LK_REFUSED;
    else lk_wrong_type(f, limit, x);
  } else if constexpr (kind == K_DATETIME) {
    if (x == '"') {
      const uint32_t q0 = f.p;
      uint32_t pos, len;
      if (lk_string(w, f, limit, &pos, &len)) {
        int64_t ep; int32_t ns, of;
        if (fast_datetime(w, pos, len, &ep, &ns, &of)) {
          v.v[I] = ep; v.aux = (int64_t)(((uint64_t)(uint32_t)ns << 32) | (uint32_t)of);
          ok = true;
        } else lk_fail(f, PJ_E_DATETIME, q0);
      }
    } else if (x == 'n') f.st = LK_REFUSED;
    else lk_wrong_type(f, limit, x);
  }
  if (ok) v.present |= 1u << I;
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
/* Flat object at f.p ('{'), inside a record whose state is LK_MEMBER. True when it was closed in the accepted form:
 * f.p then is past its brace and the state is LK_MEMBER again; otherwise the lane is stopped. */
template <int OBJ>
PJ_HD bool lk_flat(const Win& w, LkState& f, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v) {
  v.present = 0;
  f.p++;
  if (wbyte(w, f.p) == '}') { f.p++; f.st = LK_CLOSED; }
  lk_flat_members<OBJ>(w, f, limit, t, cnt, v);
  const bool ok = f.st == LK_CLOSED;
  f.st = ok ? (uint32_t)LK_MEMBER : (uint32_t)LK_REFUSED;
  return ok;
}

/* ---- model roots ---------------------------------------------------------------------------------------------- */
/* value of property I of root OBJ at f.p */
template <int OBJ, int I>
PJ_HD void lk_root_value(const Win& w, LkState& f, uint32_t limit, Tape& t, uint32_t* cnt, FVals& v, FVals& cv) {
  constexpr uint32_t kind = FK<OBJ, I>::kind, slot = FK<OBJ, I>::cnt;
  if constexpr (kind <= K_ENUM || kind == K_DATETIME) lk_scalar<OBJ, I>(w, f, limit, t, cnt, v);
  else if constexpr (kind == K_OBJ) {
    const uint32_t x = wbyte(w, f.p);
    if (x == '{') { if (lk_flat<FK<OBJ, I>::child>(w, f, limit, t, cnt, cv)) v.present |= 1u << I; }
    else if (x == 'n') f.st = LK_REFUSED;
    else lk_wrong_type(f, limit, x);
  } else {
    /* a list: `[]`, or elements separated by single commas */
    const uint32_t x0 = wbyte(w, f.p);
    bool more = x0 == '[';
    if (!more) { if (x0 == 'n') f.st = LK_REFUSED; else lk_wrong_type(f, limit, x0); }
    uint32_t j = 0;
    f.p += more ? 1u : 0u;
    if (more && wbyte(w, f.p) == ']') { f.p++; more = false; }
    while (more) { /* ends with the list closed (f.st unchanged) or the lane stopped (f.st == LK_REFUSED) */
      const uint32_t x = wbyte(w, f.p);
      bool item = false;
      if constexpr (kind == K_LIST_STR) {
        if (x == '"') {
          uint32_t pos, len;
          item = lk_string(w, f, limit, &pos, &len);
          if (item) { tape_push(t, tape_str(slot + 1, len, pos, 0)); cnt[slot + 1] += len; }
        } else lk_wrong_type(f, limit, x); /* null as a list element is PJ_E_TYPE for the exact parser: refused here */
      } else {
        constexpr int E = FK<OBJ, I>::child;
        if (x == '{') {
          /* header word and room for the scalars, then the element's strings as they are met */
          const uint32_t at = t.n;
          for (uint32_t k = 0; k < 1 + scalar_words<E>(); ++k) tape_push(t, 0);
          FVals ev;
          item = lk_flat<E>(w, f, limit, t, cnt, ev);
          if (item) {
            tape_set(t, at, (uint32_t)TAPE_ELEM | (ev.present << 4) | (slot << 12));
            tape_put_scalars<E>(t, at + 1, ev);
          }
        } else lk_wrong_type(f, limit, x);
      }
      if (item) {
        j++;
        const uint32_t y = wbyte(w, f.p);
        f.p++;
        if (y != ',') { more = false; if (y != ']') f.st = LK_REFUSED; }
      } else more = false;
    }
    cnt[slot] = j;
    if (f.st != LK_REFUSED) v.present |= 1u << I;
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
PJ_HD void lk_common_id(const Win& w, LkState& f, uint32_t limit, FVals& v) {
  static_assert(FK<OBJ_PET, 0>::kind == K_I64 && FK<OBJ_ORDER, 0>::kind == K_I64 && FK<OBJ_USER, 0>::kind == K_I64, "id leads every model");
  if (f.st == LK_MEMBER && lk_key<OBJ_PET, 0>(w, f.p)) {
    f.p += FK<OBJ_PET, 0>::pat_len;
    const uint32_t x = wbyte(w, f.p);
    int64_t val = 0;
    if (x - '0' <= 9u) {
      if (lk_int(w, f.p, true, &val)) { v.v[0] = val; v.present |= 1u; lk_member_end(w, f); }
      else f.st = LK_REFUSED;
    } else if (x == '-' || x == 'n') f.st = LK_REFUSED;
    else lk_wrong_type(f, limit, x);
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
 * is not input. Verdicts as fast_record<>(). FAST_ACCEPTED: model in *type_out, values in v / cv, counts in cnt[],
 * strings and list elements on the tape; t.n > t.cap afterwards means the tape was too small. FAST_FAILED: kind and
 * window offset of the failure in *err_kind / *err_pos. FAST_REFUSED: somebody else has to look (cnt[] and the tape
 * then hold nothing of use). `live` = false lets a lane without a record walk along (it is refused). */
template <int SCHEMA>
PJ_HD uint32_t lock_record(const Win& w, bool live, uint32_t start, uint32_t limit, uint32_t open_end, uint32_t* type_out, FVals& v, FVals& cv,
                           uint32_t* cnt, Tape& t, uint32_t* err_kind, uint32_t* err_pos) {
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (uint32_t k = 0; k < NSLOT; ++k) cnt[k] = 0;
  t.n = 0;
  v.present = 0; cv.present = 0;
  LkState f;
  f.p = start; f.err = 0; f.err_pos = 0;
  f.st = live && wbyte(w, start) == '{' ? (uint32_t)LK_MEMBER : (uint32_t)LK_REFUSED;
  f.p++;
  uint32_t type = PJ_TYPE_NONE;
  if constexpr (SCHEMA != PJ_SCHEMA_MIXED) {
    constexpr int OBJ = RootOf<SCHEMA>::obj;
    if (f.st == LK_MEMBER && wbyte(w, f.p) == '}') { f.p++; f.st = LK_CLOSED; }
    lk_root_members<OBJ>(w, f, limit, t, cnt, v, cv);
    if (f.st == LK_CLOSED && (v.present & CObj<OBJ>::required) != (uint32_t)CObj<OBJ>::required) lk_fail(f, PJ_E_REQUIRED, f.p - 1);
    type = SCHEMA;
  } else {
    /* the common `id` may come first; the key after it decides the model (a `status` there does not: refused) */
    lk_common_id(w, f, limit, v);
    uint32_t guess = 0;
    if (f.st == LK_MEMBER && wbyte(w, f.p) == '"') guess = lk_guess_owner(wbyte(w, f.p + 1), wbyte(w, f.p + 2), wbyte(w, f.p + 4));
    if (guess == PJ_TYPE_PET) {
      lk_root_members<OBJ_PET, 1>(w, f, limit, t, cnt, v, cv);
      if (f.st == LK_CLOSED && (v.present & CObj<OBJ_PET>::required) != (uint32_t)CObj<OBJ_PET>::required) lk_fail(f, PJ_E_REQUIRED, f.p - 1);
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
  *err_kind = f.err; *err_pos = f.err_pos;
  return ok ? (uint32_t)FAST_ACCEPTED : (f.err ? (uint32_t)FAST_FAILED : (uint32_t)FAST_REFUSED);
}

/* ---- emission in step --------------------------------------------------------------------------------------
 * A record accepted by lock_record<>() has its tape in MODEL order (that is the only order it accepts), so the tape
 * needs no dispatch: the walk below visits the properties as the tokeniser did and knows what every word is. The
 * lanes of a warp copy "their" name at the same time, then "their" next list element, and so on. */
PJ_HD uint32_t lk_funnel(uint32_t lo, uint32_t hi, uint32_t sh) {
#if defined(__CUDA_ARCH__)
  return __funnelshift_r(lo, hi, sh);
#else
  return sh ? (lo >> sh) | (hi << (32 - sh)) : lo;
#endif
}
/* n bytes from window offset pos to dst (any alignment): up to three bytes until dst is word aligned, whole words
 * (one window load each), up to three bytes at the end */
PJ_HD void lk_copy(uint8_t* dst, const Win& w, uint32_t pos, uint32_t n) {
  uint32_t h = (0u - (uint32_t)reinterpret_cast<uintptr_t>(dst)) & 3u;
  if (h > n) h = n;
  if (h > 0) dst[0] = (uint8_t)wbyte(w, pos);
  if (h > 1) dst[1] = (uint8_t)wbyte(w, pos + 1);
  if (h > 2) dst[2] = (uint8_t)wbyte(w, pos + 2);
  dst += h; pos += h; n -= h;
  const uint32_t* a = reinterpret_cast<const uint32_t*>(w.s) + (pos >> 2);
  const uint32_t sh = (pos & 3u) * 8u, nw = n >> 2;
  uint32_t x0 = a[0];
  uint32_t* d4 = reinterpret_cast<uint32_t*>(dst);
  for (uint32_t i = 0; i < nw; ++i) {
    const uint32_t x1 = a[i + 1];
    d4[i] = lk_funnel(x0, x1, sh);
    x0 = x1;
  }
  const uint32_t t = n & 3u;
  if (t) {
    const uint32_t last = lk_funnel(x0, a[nw + 1], sh);
    uint8_t* e = dst + 4u * nw;
    e[0] = (uint8_t)last;
    if (t > 1) e[1] = (uint8_t)(last >> 8);
    if (t > 2) e[2] = (uint8_t)(last >> 16);
  }
}
PJ_HD void lk_copy_word(uint8_t* dst, const Win& w, uint32_t word) { lk_copy(dst, w, word >> 16, (word >> 4) & 0x7FFu); }

/* the strings of a flat object (embedded object or list element), in property order; cur[] = bytes of the record
 * already emitted per slot */
template <int OBJ, int I = 0>
PJ_HD void lk_emit_flat_strings(const Win& w, const DevCols* c, uint32_t present, const Tape& t, uint32_t& k, const uint32_t* base, uint32_t* cur) {
  if constexpr (I < CObj<OBJ>::N) {
    if constexpr (FK<OBJ, I>::kind == K_STR) {
      constexpr uint32_t slot = FK<OBJ, I>::cnt;
      if ((present >> I) & 1u) {
        const uint32_t word = tape_get(t, k);
        k++;
        lk_copy_word(colp<uint8_t>(c, FK<OBJ, I>::col + 1) + base[slot] + cur[slot], w, word);
        cur[slot] += (word >> 4) & 0x7FFu;
      }
    }
    lk_emit_flat_strings<OBJ, I + 1>(w, c, present, t, k, base, cur);
  }
}
/* everything of root OBJ that lies on the tape, property by property */
template <int OBJ, int I = 0>
PJ_HD void lk_emit_walk(const Win& w, const DevCols* c, const FVals& v, const FVals& cv, const Tape& t, uint32_t& k, const uint32_t* base,
                        const uint32_t* cnt, uint32_t* cur) {
  if constexpr (I < CObj<OBJ>::N) {
    constexpr uint32_t kind = FK<OBJ, I>::kind, col = FK<OBJ, I>::col, slot = FK<OBJ, I>::cnt;
    const bool present = (v.present >> I) & 1u;
    if constexpr (kind == K_STR) {
      if (present) {
        const uint32_t word = tape_get(t, k);
        k++;
        lk_copy_word(colp<uint8_t>(c, col + 1) + base[slot], w, word);
      }
    } else if constexpr (kind == K_OBJ) {
      if (present) lk_emit_flat_strings<FK<OBJ, I>::child>(w, c, cv.present, t, k, base, cur);
    } else if constexpr (kind == K_LIST_STR) {
      const uint32_t n = present ? cnt[slot] : 0u;
      uint32_t at = 0;
      for (uint32_t j = 0; j < n; ++j) {
        const uint32_t word = tape_get(t, k);
        k++;
        colp<uint32_t>(c, col + 1)[(uint64_t)base[slot] + j] = base[slot + 1] + at;
        lk_copy_word(colp<uint8_t>(c, col + 2) + base[slot + 1] + at, w, word);
        at += (word >> 4) & 0x7FFu;
      }
    } else if constexpr (kind == K_LIST_OBJ) {
      constexpr int E = FK<OBJ, I>::child;
      const uint32_t n = present ? cnt[slot] : 0u;
      for (uint32_t j = 0; j < n; ++j) {
        const uint32_t head = tape_get(t, k);
        const uint64_t erow = (uint64_t)base[slot] + j;
        FVals ev;
        ev.present = (head >> 4) & 0xFFu;
        tape_get_scalars<E>(t, k + 1, ev);
        k += 1 + scalar_words<E>();
        store_elem_str_offsets<E>(c, erow, base, cur);
        store_vals<E, true>(c, ev, erow, base);
        lk_emit_flat_strings<E>(w, c, ev.present, t, k, base, cur);
      }
    }
    lk_emit_walk<OBJ, I + 1>(w, c, v, cv, t, k, base, cnt, cur);
  }
}
template <int OBJ>
PJ_HD void lk_emit_root(const Win& w, const DevCols* c, const FVals& v, const FVals& cv, const Tape& t, uint64_t row, const uint32_t* base, const uint32_t* cnt) {
  store_vals<OBJ, false>(c, v, row, base);
  store_embedded<OBJ>(c, v, cv, row, base);
  uint32_t cur[NSLOT];
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (uint32_t q = 0; q < NSLOT; ++q) cur[q] = 0;
  uint32_t k = 0;
  lk_emit_walk<OBJ>(w, c, v, cv, t, k, base, cnt, cur);
}
/* Emits a record that lock_record<SCHEMA>() accepted and whose tape held all of it (t.n <= t.cap): what fast_emit<>()
 * does, without looking a word up. cnt[] = the record's counts, base[] = its start in every arena / child table. */
template <int SCHEMA>
PJ_HD void lock_emit(const Win& w, const DevCols* c, uint32_t type, const FVals& v, const FVals& cv, const Tape& t, const uint32_t* base,
                     const uint32_t* cnt, uint64_t rec_index) {
  if constexpr (SCHEMA != PJ_SCHEMA_MIXED) lk_emit_root<RootOf<SCHEMA>::obj>(w, c, v, cv, t, rec_index, base, cnt);
  else {
    if (type == PJ_TYPE_PET) lk_emit_root<OBJ_PET>(w, c, v, cv, t, base[SLOT_ROWS_PET], base, cnt);
    else if (type == PJ_TYPE_ORDER) lk_emit_root<OBJ_ORDER>(w, c, v, cv, t, base[SLOT_ROWS_ORD], base, cnt);
    else lk_emit_root<OBJ_USER>(w, c, v, cv, t, base[SLOT_ROWS_USR], base, cnt);
  }
}

}  // namespace pj
#endif
