/*
 * pj_array.cuh — structural index of array framing (`[rec, rec, ...]`), word-parallel.
 *
 * Every thread owns one 64-byte word of the input and turns it into 64-bit masks (one bit per byte) of
 * backslashes, quotes, brackets, commas and blanks. From those it derives, exactly as the framing rules
 * of petjson.h say:
 *   escaped bytes      a byte is escaped iff an odd run of backslashes precedes it
 *   in-string mask     prefix-XOR of the unescaped quotes
 *   nesting depth      openers minus closers among the bytes outside strings
 * The three quantities carry from word to word (escape carry c, in-string s, depth d), and every carry is
 * a prefix sum, so a word is first summarised as a FUNCTION of its incoming (c, s) — four cases — and the
 * summaries are composed by scans (warp shuffle, block, then tiles); a second pass re-evaluates each word
 * with its now known incoming state and marks the separators: `[` at depth 0, `,` and `]` at depth 1.
 */
#ifndef PJ_ARRAY_CUH
#define PJ_ARRAY_CUH

#include "pj_core.cuh"

namespace pj {

struct WordMasks {
  uint64_t B, Q, O, C, M, W, LB, RB, valid; /* backslash, quote, { [, } ], comma, blank, [, ], bytes inside the input */
};

/* bit k of the result: byte k of the 8-byte word w equals c (exact for every byte) */
PJ_HD uint32_t eq_bits8(uint64_t w, uint32_t c) {
  const uint64_t x = w ^ (0x0101010101010101ull * c);
  const uint64_t y = ((x & 0x7F7F7F7F7F7F7F7Full) + 0x7F7F7F7F7F7F7F7Full) | x; /* bit 7 of a byte clear iff the byte is 0 */
  const uint64_t m = (~y & 0x8080808080808080ull) >> 7;
  return (uint32_t)((m * 0x0102040810204080ull) >> 56);
}
/* masks of the 64 bytes at p, of which the first `n` (1..64) are input; the rest read as 0 */
PJ_HD WordMasks word_masks(const uint8_t* p, uint32_t n) {
  WordMasks m;
  m.B = m.Q = m.O = m.C = m.M = m.W = m.LB = m.RB = 0;
  for (uint32_t k = 0; k < 8; ++k) {
    uint64_t w = 0;
    if (8 * k < n) {
      const uint32_t take = n - 8 * k >= 8 ? 8 : n - 8 * k;
      for (uint32_t b = 0; b < take; ++b) w |= (uint64_t)p[8 * k + b] << (8 * b);
    }
    const uint64_t lb = eq_bits8(w, '['), rb = eq_bits8(w, ']'), lc = eq_bits8(w, '{'), rc = eq_bits8(w, '}');
    const uint64_t ws = eq_bits8(w, ' ') | eq_bits8(w, '\t') | eq_bits8(w, '\r') | eq_bits8(w, '\n');
    m.B |= (uint64_t)eq_bits8(w, '\\') << (8 * k);
    m.Q |= (uint64_t)eq_bits8(w, '"') << (8 * k);
    m.M |= (uint64_t)eq_bits8(w, ',') << (8 * k);
    m.LB |= lb << (8 * k); m.RB |= rb << (8 * k);
    m.O |= (lb | lc) << (8 * k); m.C |= (rb | rc) << (8 * k);
    m.W |= ws << (8 * k);
  }
  m.valid = n >= 64 ? ~0ull : ((1ull << n) - 1);
  /* bytes past the input are neither blanks nor anything else */
  m.W &= m.valid;
  return m;
}

PJ_HD uint32_t popc64(uint64_t x) {
#if defined(__CUDA_ARCH__)
  return (uint32_t)__popcll(x);
#else
  return (uint32_t)__builtin_popcountll(x);
#endif
}
PJ_HD uint32_t ctz64a(uint64_t x) {
#if defined(__CUDA_ARCH__)
  return (uint32_t)(__ffsll((long long)x) - 1);
#else
  return (uint32_t)__builtin_ctzll(x);
#endif
}

/* state carried between words */
struct ArrState {
  uint32_t c, s; /* first byte of the next word is escaped; the next word starts inside a string */
  int32_t d;     /* nesting depth */
};
struct WordEval {
  uint64_t quotes;   /* unescaped quotes */
  uint64_t interior; /* bytes strictly inside strings */
  uint64_t outside;  /* bytes outside strings that are not quotes */
  ArrState out;
};
/* bytes escaped by an odd run of backslashes, and the carry into the next word */
PJ_HD uint64_t escaped_mask(uint64_t backslash, uint32_t carry_in, uint32_t* carry_out) {
  const uint64_t even = 0x5555555555555555ull;
  backslash &= ~(uint64_t)carry_in; /* an escaped backslash does not escape */
  const uint64_t follows = (backslash << 1) | carry_in;
  const uint64_t odd_starts = backslash & ~even & ~follows;
  const uint64_t sum = odd_starts + backslash;
  *carry_out = sum < odd_starts ? 1u : 0u; /* a run of backslashes reaching past the word, of odd length */
  const uint64_t invert = sum << 1;
  return (even ^ invert) & follows;
}
PJ_HD uint64_t prefix_xor(uint64_t x) {
  x ^= x << 1; x ^= x << 2; x ^= x << 4; x ^= x << 8; x ^= x << 16; x ^= x << 32;
  return x;
}
PJ_HD WordEval eval_word(const WordMasks& m, ArrState in) {
  WordEval e;
  uint32_t c_out;
  const uint64_t esc = escaped_mask(m.B, in.c, &c_out);
  e.quotes = m.Q & ~esc;
  const uint64_t instr = prefix_xor(e.quotes) ^ (in.s ? ~0ull : 0ull); /* from an opening quote up to, not including, the closing one */
  e.interior = instr & ~e.quotes & m.valid;
  e.outside = ~instr & ~e.quotes & m.valid;
  e.out.c = c_out;
  e.out.s = (uint32_t)(instr >> 63) & 1u;
  e.out.d = in.d + (int32_t)popc64(m.O & e.outside) - (int32_t)popc64(m.C & e.outside);
  return e;
}

/* A word (or any run of words) as a function of its incoming (c, s): index x = c | s << 1. */
struct ArrFn {
  uint32_t st;  /* four 2-bit outgoing states, entry x in bits 2x..2x+1 */
  int32_t d[4]; /* depth change for each incoming state */
};
PJ_HD ArrFn fn_identity() { ArrFn f; f.st = 0xE4u; f.d[0] = f.d[1] = f.d[2] = f.d[3] = 0; return f; }
PJ_HD ArrFn fn_of_word(const WordMasks& m) {
  ArrFn f;
  f.st = 0;
  for (uint32_t x = 0; x < 4; ++x) {
    ArrState in;
    in.c = x & 1; in.s = x >> 1; in.d = 0;
    const WordEval e = eval_word(m, in);
    f.st |= (e.out.c | (e.out.s << 1)) << (2 * x);
    f.d[x] = e.out.d;
  }
  return f;
}
PJ_HD int32_t fn_pick(const int32_t* d, uint32_t x) { return x == 0 ? d[0] : (x == 1 ? d[1] : (x == 2 ? d[2] : d[3])); }
/* first f, then g */
PJ_HD ArrFn fn_compose(const ArrFn& f, const ArrFn& g) {
  ArrFn h;
  h.st = 0;
  for (uint32_t x = 0; x < 4; ++x) {
    const uint32_t mid = (f.st >> (2 * x)) & 3u;
    h.st |= ((g.st >> (2 * mid)) & 3u) << (2 * x);
    h.d[x] = f.d[x] + fn_pick(g.d, mid);
  }
  return h;
}
PJ_HD ArrState fn_apply(const ArrFn& f, ArrState in) {
  const uint32_t x = in.c | (in.s << 1);
  const uint32_t o = (f.st >> (2 * x)) & 3u;
  ArrState out;
  out.c = o & 1; out.s = o >> 1; out.d = in.d + fn_pick(f.d, x);
  return out;
}

/* Second pass over a word whose incoming state is known: separators, the lowest byte that breaks
 * `ws [ ... ] ws` (doc_bit, 64 = none) and the lowest opener (opener_bit, 64 = none). */
struct WordMarks {
  uint64_t sep;
  uint32_t doc_bit, opener_bit;
};
PJ_HD WordMarks mark_word(const WordMasks& m, const WordEval& e, int32_t depth_in) {
  WordMarks r;
  uint64_t sep = 0, openers = 0, low = 0; /* low: bytes whose depth is <= 0 */
  int32_t d = depth_in;
  uint32_t seg = 0;
  uint64_t bits = (m.O | m.C) & e.outside;
  while (bits) {
    const uint32_t b = ctz64a(bits);
    const uint64_t bit = 1ull << b;
    bits &= bits - 1;
    /* bytes seg..b see depth d */
    if (d <= 0) low |= (b == 63 ? ~0ull : ((bit << 1) - 1)) & ~((1ull << seg) - 1);
    if (m.O & bit) { if ((m.LB & bit) && d == 0) { sep |= bit; openers |= bit; } d++; }
    else { if ((m.RB & bit) && d == 1) sep |= bit; d--; }
    seg = b + 1;
  }
  if (seg < 64 && d <= 0) low |= ~((1ull << seg) - 1);
  /* commas at depth 1: the bytes at depth exactly 1 are those between the bracket events; redo the walk on commas */
  {
    int32_t dd = depth_in;
    uint64_t ev = (m.O | m.C | m.M) & e.outside;
    while (ev) {
      const uint32_t b = ctz64a(ev);
      const uint64_t bit = 1ull << b;
      ev &= ev - 1;
      if (m.O & bit) dd++;
      else if (m.C & bit) dd--;
      else if (dd == 1) sep |= bit;
    }
  }
  const uint64_t bad = low & ~m.W & ~e.interior & m.valid & ~openers;
  r.sep = sep;
  r.doc_bit = bad ? ctz64a(bad) : 64u;
  r.opener_bit = openers ? ctz64a(openers) : 64u;
  return r;
}

/* The extent that starts after the separator at byte p (a `[` or `,`; a `]` starts none).
 * sep: separator bitmap, one bit per input byte; first_opener: offset of the first `[` at depth 0. */
struct ExtentOut {
  uint32_t is_record, blank, second_opener;
  uint64_t start, end;
};
PJ_HD ExtentOut arr_extent(const uint8_t* in, uint64_t len, const uint64_t* sep, uint64_t p, uint64_t first_opener) {
  ExtentOut r;
  r.is_record = 0; r.blank = 0; r.second_opener = 0; r.start = p + 1; r.end = len;
  const uint32_t x = ld_byte(in + p);
  if (x == ']') return r;
  const bool left_opener = x == '[';
  r.second_opener = left_opener && p > first_opener;
  /* next separator after p */
  const uint64_t nwords = (len + 63) >> 6;
  uint64_t wi = p >> 6;
  const uint32_t b = (uint32_t)(p & 63);
  uint64_t m = b == 63 ? 0 : (sep[wi] & (~0ull << (b + 1)));
  bool has_right = false;
  for (;;) {
    if (m) { r.end = (wi << 6) + ctz64a(m); has_right = true; break; }
    if (++wi >= nwords) break;
    m = sep[wi];
  }
  uint64_t t = p + 1;
  while (t < r.end) {
    const uint32_t y = ld_byte(in + t);
    if (y == ' ' || y == '\t' || y == '\r' || y == '\n') ++t; else break;
  }
  r.blank = t >= r.end;
  const bool right_closer = has_right && ld_byte(in + r.end) == ']';
  r.is_record = !(r.blank && ((left_opener && right_closer) || !has_right));
  return r;
}

}  // namespace pj
#endif
