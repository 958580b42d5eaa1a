/*
 * pj_wide.cuh — long records, a warp at a time.
 *
 * A record whose lists hold hundreds of elements keeps one thread busy for a long time while the other threads of
 * its tile have nothing left to do. Such records are taken out of the thread-per-record path: a whole warp runs the
 * exact parser of pj_core.cuh on the record, every lane executing the same steps on the same bytes (so the lanes
 * never diverge and nothing about the rules changes), and where the parser reaches a non-empty list it hands the
 * list to wide_list<>() below, which spreads the ELEMENTS over the lanes:
 *
 *   1. the warp classifies 1024 bytes per step, 32 per lane: masks of backslashes and quotes (exact SWAR compares),
 *      escaped bytes (odd runs of backslashes, carried from lane to lane), string interiors (prefix XOR of the
 *      unescaped quotes, carried by a ballot). The starts of the elements are the opening quotes (list of strings)
 *      or the `{` outside strings (list of flat objects);
 *   2. every lane reads the elements that start in its 32 bytes with the exact routines (lex_string, parse_flat),
 *      then the separator behind each: blanks, `,`, blanks and the next start — or `]`, which ends the list;
 *   3. the chain is checked link by link: the start that follows an element in the masks must be the position its
 *      separator ended at, the first start must be where the list began. With every link in place the starts found
 *      by the masks are exactly the elements a sequential walk meets;
 *   4. sizes are added up by warp scans; the emit pass gives every element its position in the child table and in
 *      the byte arenas before it writes.
 *
 * Whatever is not a well-formed list in this sense — a failing element, a nested container in an unknown property,
 * a missing comma, a 32-byte block of nothing but backslashes — makes wide_list return 0 with nothing changed, and
 * the parser walks the list element by element as it always did, reporting the failure at the place the rules name.
 */
#ifndef PJ_WIDE_CUH
#define PJ_WIDE_CUH

#include "pj_array.cuh"
#include "pj_fast.cuh"

namespace pj {

static constexpr uint32_t WIDE_NONE = 0xFFFFFFFFu;
static constexpr uint32_t WIDE_STEP = 1024; /* bytes a warp classifies per step */

/* bytes escaped by an odd run of backslashes (32 bytes; carry_in: the first byte is escaped) */
PJ_HD uint32_t wide_escaped(uint32_t bs, uint32_t carry_in) {
  const uint32_t even = 0x55555555u;
  bs &= ~carry_in;
  const uint32_t follows = (bs << 1) | carry_in;
  const uint32_t odd_starts = bs & ~even & ~follows;
  const uint32_t sum = odd_starts + bs;
  const uint32_t invert = sum << 1;
  return (even ^ invert) & follows;
}
PJ_HD uint32_t wide_prefix_xor(uint32_t x) {
  x ^= x << 1; x ^= x << 2; x ^= x << 4; x ^= x << 8; x ^= x << 16;
  return x;
}
PJ_HD uint32_t wide_low_mask(int64_t n) { return n <= 0 ? 0u : (n >= 32 ? 0xFFFFFFFFu : ((1u << (uint32_t)n) - 1u)); }
/* bit 7 of every byte of w that equals c / is below 0x20 */
PJ_HD uint64_t wide_flags_eq(uint64_t w, uint32_t c) {
  const uint64_t x = w ^ (0x0101010101010101ull * c);
  return ~((((x & 0x7F7F7F7F7F7F7F7Full) + 0x7F7F7F7F7F7F7F7Full) | x)) & 0x8080808080808080ull;
}
PJ_HD uint64_t wide_flags_ctrl(uint64_t w) {
  const uint64_t x = w & 0xE0E0E0E0E0E0E0E0ull;
  return ~((((x & 0x7F7F7F7F7F7F7F7Full) + 0x7F7F7F7F7F7F7F7Full) | x)) & 0x8080808080808080ull;
}
PJ_HD uint32_t wide_movemask(uint64_t flags) { return (uint32_t)(((flags >> 7) * 0x0102040810204080ull) >> 56); }

/* parity of the run of backslashes that ends a 32-byte block (B: its backslash mask, not all ones): the carry into the
 * block behind it. Independent of the carry INTO the block, because the run does not span it. */
PJ_HD uint32_t wide_carry_out(uint32_t B) {
  uint32_t n = 0;
  while (n < 32 && ((B >> (31 - n)) & 1u)) ++n; /* leading ones */
  return n & 1u;
}
/* The masks of one lane's 32 bytes p[0..32) (valid: which of them belong to the list): backslashes, quotes, `{`, bytes
 * that are control characters or not ASCII. */
PJ_HD void wide_block_masks(const uint8_t* p, uint32_t valid, uint32_t* B, uint32_t* Q, uint32_t* C, uint32_t* X) {
  uint32_t b = 0, q = 0, c = 0, x = 0;
  for (int h = 0; h < 4; ++h) {
    uint64_t w = 0;
    for (int k = 0; k < 8; ++k) w |= (uint64_t)p[8 * h + k] << (8 * k);
    b |= wide_movemask(wide_flags_eq(w, '\\')) << (8 * h);
    q |= wide_movemask(wide_flags_eq(w, '"')) << (8 * h);
    c |= wide_movemask(wide_flags_eq(w, '{')) << (8 * h);
    x |= wide_movemask(wide_flags_ctrl(w) | (w & 0x8080808080808080ull)) << (8 * h);
  }
  *B = b & valid; *Q = q & valid; *C = c & valid; *X = x & valid;
}

#if defined(__CUDACC__)

__device__ __forceinline__ uint32_t wide_min(uint32_t x) {
#pragma unroll
  for (int d = 16; d; d >>= 1) { const uint32_t y = __shfl_xor_sync(0xFFFFFFFFu, x, d); x = y < x ? y : x; }
  return x;
}
__device__ __forceinline__ uint32_t wide_sum(uint32_t x) {
#pragma unroll
  for (int d = 16; d; d >>= 1) x += __shfl_xor_sync(0xFFFFFFFFu, x, d);
  return x;
}
__device__ __forceinline__ uint32_t wide_excl(uint32_t x, uint32_t lane) {
  uint32_t inc = x;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) { const uint32_t y = __shfl_up_sync(0xFFFFFFFFu, inc, d); if ((int)lane >= d) inc += y; }
  return inc - x;
}

/* The separator behind an element: blanks, then `,` blanks (*nxt = where the next element has to start) or `]`
 * (*endx = the offset behind it). False for anything else. */
__device__ __forceinline__ bool wide_gap(const uint8_t* in, uint64_t limit, uint64_t p, uint64_t* nxt, uint64_t* endx) {
  uint32_t x;
  for (;;) { x = p < limit ? in[p] : 0u; if (x == ' ' || x == '\t' || x == '\r') ++p; else break; }
  *endx = 0;
  if (x == ',') {
    ++p;
    for (;;) { x = p < limit ? in[p] : 0u; if (x == ' ' || x == '\t' || x == '\r') ++p; else break; }
    *nxt = p;
    return true;
  }
  if (x == ']') { *endx = p + 1; *nxt = p + 1; return true; }
  return false;
}

/* What a lane knows about the quotes of the lanes behind it (list of strings): where the string that is still open
 * at the end of its own 32 bytes closes. */
struct WideQuotes {
  uint32_t Qu, Fm;      /* this lane: unescaped quotes; bytes no plain string holds (backslash, control, not ASCII) */
  uint32_t lane_bit;    /* 32 * lane */
  uint32_t next_close;  /* position (in the step) of the first quote of the following lanes, WIDE_NONE = none */
  uint32_t clean_until; /* no byte of Fm between this lane's end and that quote */
};
/* The string opened by the quote at bit b of this lane: its closing quote's position in the step when every byte of
 * it is plain (then its decoded length is the distance), WIDE_NONE otherwise. */
__device__ __forceinline__ uint32_t wide_plain_close(const WideQuotes& q, uint32_t b) {
  const uint32_t above = b == 31 ? 0u : (0xFFFFFFFFu << (b + 1));
  const uint32_t rest = q.Qu & above;
  if (rest) {
    const uint32_t c = (uint32_t)__ffs((int)rest) - 1u;
    return (q.Fm & above & ((1u << c) - 1u)) ? WIDE_NONE : q.lane_bit + c;
  }
  if (q.next_close == WIDE_NONE || !q.clean_until || (q.Fm & above)) return WIDE_NONE;
  return q.next_close;
}

/* One element at es.p, sized (and validated) by the exact routines; then its separator. Returns false when the
 * element fails or what follows is neither `, <next>` nor `]`. *nxt: where the next element must start; *endx != 0:
 * the list closed, *endx is the offset behind its `]`. sb[0..1]: decoded bytes per string column of the element. */
static __device__ __noinline__ bool wide_size_element(const Schema& S, const Rd& r, const FieldDesc& F, uint64_t pos, uint32_t* sb, uint64_t* nxt, uint64_t* endx) {
  PS es;
  es.p = pos; es.err = 0; es.err_pos = 0;
  sb[0] = sb[1] = 0;
  if (F.kind == K_LIST_STR) {
    Sink k;
    sink_init(k, SINK_COUNT);
    if (!lex_string(r, es, k)) return false;
    sb[0] = k.n;
  } else {
    const ObjDesc& Ed = S.obj[F.child];
    Out<false> lo;
    lo.cols = nullptr;
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) lo.cnt[k] = 0;
    ObjVals ev;
    uint32_t est[8];
    if (!parse_flat<false>(S, r, es, Ed, ev, lo, true, false, est)) return false;
    uint32_t q = 0;
    for (int i = 0; i < (int)Ed.nfields; ++i)
      if (Ed.f[i].kind == K_STR && q < 2) sb[q++] = lo.cnt[Ed.f[i].cnt];
  }
  return wide_gap(r.in, r.limit, es.p, nxt, endx);
}

/* The emit pass of one element: number j of its list, its strings at cursor at[0..1] of their arenas. */
template <bool W>
__device__ __noinline__ void wide_write_element(const Schema& S, const Rd& r, const FieldDesc& F, Out<W>& o, uint64_t pos, uint32_t j, uint32_t* at) {
  if (!W) return;
  PS es;
  es.p = pos; es.err = 0; es.err_pos = 0;
  const bool live = j < o.room[F.cnt];
  if (F.kind == K_LIST_STR) {
    Sink e;
    sink_init(e, live ? SINK_WRITE : SINK_COUNT);
    if (live) {
      const uint32_t rm = o.room[F.cnt + 1];
      e.room = rm > at[0] ? rm - at[0] : 0;
      e.dst = colp<uint8_t>(o.cols, F.col + 2) + o.base[F.cnt + 1] + at[0];
      colp<uint32_t>(o.cols, F.col + 1)[o.base[F.cnt] + j] = o.base[F.cnt + 1] + at[0];
    }
    lex_string(r, es, e);
    at[0] += e.n;
  } else {
    const ObjDesc& Ed = S.obj[F.child];
    uint32_t q = 0;
    for (int i = 0; i < (int)Ed.nfields; ++i)
      if (Ed.f[i].kind == K_STR && q < 2) o.cnt[Ed.f[i].cnt] = at[q++];
    ObjVals ev;
    uint32_t est[8];
    parse_flat<W>(S, r, es, Ed, ev, o, true, live, est);
    if (live) store_object<W>(Ed, ev, (uint64_t)o.base[F.cnt] + j, o, est);
    q = 0;
    for (int i = 0; i < (int)Ed.nfields; ++i)
      if (Ed.f[i].kind == K_STR && q < 2) at[q++] = o.cnt[Ed.f[i].cnt];
  }
}

/* The list whose first element is at s.p (the parser has skipped the blanks behind `[` and seen that the list is not
 * empty), by the whole warp. All lanes hold the same r, s and o. Returns 1 with s.p behind the `]` and the list's
 * counters in o.cnt, or 0 with nothing changed. */
template <bool W>
__device__ __noinline__ int wide_list(const Schema& S, const Rd& r, PS& s, const FieldDesc& F, Out<W>& o) {
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t lt = (1u << lane) - 1u, gt = lane == 31 ? 0u : ~((2u << lane) - 1u);
  const bool objs = F.kind == K_LIST_OBJ;
  if (objs) { /* two string columns per element at most */
    const ObjDesc& Ed = S.obj[F.child];
    uint32_t q = 0;
    for (int i = 0; i < (int)Ed.nfields; ++i) q += Ed.f[i].kind == K_STR;
    if (q > 2) return 0;
  }
  const int64_t p0 = (int64_t)s.p;
  const int64_t end = (int64_t)(r.rec_end < r.limit ? r.rec_end : r.limit);
  int64_t cb = p0 - (int64_t)(reinterpret_cast<uintptr_t>(r.in + p0) & 15u);
  uint32_t esc_c = 0, str_c = 0;
  uint64_t pending = (uint64_t)p0; /* where the next element has to start */
  uint32_t n_el = 0, tot0 = 0, tot1 = 0;
  Out<W> lo; /* emit pass: this lane's own cursors */
  if (W) {
    lo.cols = o.cols;
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) { lo.cnt[k] = o.cnt[k]; lo.base[k] = o.base[k]; lo.room[k] = o.room[k]; }
  }
  for (;; cb += WIDE_STEP) {
    if (cb >= end) return 0; /* the record ended inside the list */
    const int64_t lb = cb + 32 * (int64_t)lane;
    /* ---- masks of this lane's 32 bytes ---- */
    uint32_t B = 0, Q = 0, C = 0, X = 0; /* backslashes, quotes, `{`, bytes that are control characters or not ASCII */
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int64_t hb = lb + 16 * h;
      if (hb < end && hb + 16 > p0) {
        const uint4 v = *reinterpret_cast<const uint4*>(r.in + hb);
        const uint64_t w0 = (uint64_t)v.x | ((uint64_t)v.y << 32), w1 = (uint64_t)v.z | ((uint64_t)v.w << 32);
        B |= (wide_movemask(wide_flags_eq(w0, '\\')) | (wide_movemask(wide_flags_eq(w1, '\\')) << 8)) << (16 * h);
        Q |= (wide_movemask(wide_flags_eq(w0, '"')) | (wide_movemask(wide_flags_eq(w1, '"')) << 8)) << (16 * h);
        if (objs) C |= (wide_movemask(wide_flags_eq(w0, '{')) | (wide_movemask(wide_flags_eq(w1, '{')) << 8)) << (16 * h);
        else X |= (wide_movemask(wide_flags_ctrl(w0) | (w0 & 0x8080808080808080ull)) | (wide_movemask(wide_flags_ctrl(w1) | (w1 & 0x8080808080808080ull)) << 8)) << (16 * h);
      }
    }
    const uint32_t valid = wide_low_mask(end - lb) & ~wide_low_mask(p0 - lb);
    B &= valid; Q &= valid; C &= valid; X &= valid;
    if (__any_sync(0xFFFFFFFFu, B == 0xFFFFFFFFu)) return 0;
    const uint32_t cout = (uint32_t)__clz((int)~B) & 1u; /* parity of the run of backslashes that ends the block */
    uint32_t cin = __shfl_up_sync(0xFFFFFFFFu, cout, 1);
    if (lane == 0) cin = esc_c;
    const uint32_t esc = wide_escaped(B, cin);
    const uint32_t Qu = Q & ~esc;
    const uint32_t par = __ballot_sync(0xFFFFFFFFu, __popc(Qu) & 1);
    const uint32_t sin = ((uint32_t)__popc(par & lt) & 1u) ^ str_c;
    const uint32_t instr = wide_prefix_xor(Qu) ^ (sin ? 0xFFFFFFFFu : 0u); /* from an opening quote up to, not including, the closing one */
    const uint32_t starts = objs ? (C & ~instr) : (Qu & instr);
    esc_c = __shfl_sync(0xFFFFFFFFu, cout, 31);
    str_c ^= (uint32_t)__popc(par) & 1u;

    /* ---- the elements that start in this lane's bytes ---- */
    const uint32_t have = __ballot_sync(0xFFFFFFFFu, starts != 0);
    if (!have) continue;
    const uint32_t my_first = starts ? 32u * lane + (uint32_t)(__ffs((int)starts) - 1) : WIDE_NONE;
    const uint32_t after = have & gt;
    const int next_lane = after ? __ffs((int)after) - 1 : 0;
    uint32_t next_first = __shfl_sync(0xFFFFFFFFu, my_first, next_lane);
    if (!after) next_first = WIDE_NONE;
    const uint32_t first_lane = (uint32_t)__ffs((int)have) - 1u, last_lane = 31u - (uint32_t)__clz((int)have);

    WideQuotes wq;
    wq.Qu = Qu; wq.Fm = B | X; wq.lane_bit = 32u * lane; wq.next_close = WIDE_NONE; wq.clean_until = 0;
    if (!objs) {
      const uint32_t qhave = __ballot_sync(0xFFFFFFFFu, Qu != 0), fhave = __ballot_sync(0xFFFFFFFFu, wq.Fm != 0);
      const uint32_t qafter = qhave & gt;
      const int nql = qafter ? __ffs((int)qafter) - 1 : 0;
      const uint32_t nq_bit = __shfl_sync(0xFFFFFFFFu, Qu ? (uint32_t)__ffs((int)Qu) - 1u : 0u, nql);
      const uint32_t nq_f = __shfl_sync(0xFFFFFFFFu, wq.Fm, nql);
      if (qafter) {
        wq.next_close = 32u * (uint32_t)nql + nq_bit;
        wq.clean_until = !(fhave & gt & ((1u << nql) - 1u)) && !(nq_f & ((1u << nq_bit) - 1u));
      }
    }
    uint32_t bad = WIDE_NONE, end_rel = WIDE_NONE, my_n = 0, my0 = 0, my1 = 0;
    uint64_t endx = 0, my_pending = 0;
    {
      uint32_t m = starts;
      bool first = lane == first_lane;
      while (m) {
        const uint32_t b = (uint32_t)__ffs((int)m) - 1u;
        m &= m - 1u;
        const uint32_t rel = 32u * lane + b;
        const uint64_t pos = (uint64_t)(cb + rel);
        const uint32_t succ = m ? 32u * lane + (uint32_t)(__ffs((int)m) - 1) : next_first;
        if (first && pos != pending) { bad = rel; break; }
        first = false;
        uint32_t sb[2];
        uint64_t nxt, ex;
        const uint32_t close = objs ? WIDE_NONE : wide_plain_close(wq, b);
        if (close != WIDE_NONE) { /* a plain string: its length is the distance of its quotes */
          sb[0] = close - rel - 1u; sb[1] = 0;
          if (!wide_gap(r.in, r.limit, (uint64_t)(cb + close) + 1u, &nxt, &ex)) { bad = rel; break; }
        } else if (!wide_size_element(S, r, F, pos, sb, &nxt, &ex)) { bad = rel; break; }
        my_n++; my0 += sb[0]; my1 += sb[1];
        if (ex) { end_rel = rel; endx = ex; break; }
        if (succ == WIDE_NONE) my_pending = nxt;
        else if ((uint64_t)(cb + succ) != nxt) { bad = rel; break; }
      }
    }
    const uint32_t END = wide_min(end_rel), BAD = wide_min(bad);
    if (BAD != WIDE_NONE && (END == WIDE_NONE || BAD <= END)) return 0;
    if (END != WIDE_NONE && lane > (END >> 5)) { my_n = 0; my0 = 0; my1 = 0; }
    const uint32_t ex_n = wide_excl(my_n, lane), ex0 = wide_excl(my0, lane), ex1 = wide_excl(my1, lane);

    if (W) { /* second walk: every element knows its place now */
      uint32_t m = starts, j = n_el + ex_n;
      uint32_t at[2] = {tot0 + ex0, tot1 + ex1};
      const uint32_t stop = END == WIDE_NONE ? WIDE_NONE : END;
      while (m) {
        const uint32_t b = (uint32_t)__ffs((int)m) - 1u;
        m &= m - 1u;
        const uint32_t rel = 32u * lane + b;
        if (rel > stop) break;
        const uint32_t close = objs ? WIDE_NONE : wide_plain_close(wq, b);
        if (close != WIDE_NONE) {
          if (j < lo.room[F.cnt]) {
            const uint32_t n = close - rel - 1u, rm = lo.room[F.cnt + 1];
            const uint32_t take = rm > at[0] ? (rm - at[0] < n ? rm - at[0] : n) : 0u;
            uint8_t* dst = colp<uint8_t>(lo.cols, F.col + 2) + lo.base[F.cnt + 1] + at[0];
            const uint8_t* src = r.in + (cb + rel + 1);
            colp<uint32_t>(lo.cols, F.col + 1)[lo.base[F.cnt] + j] = lo.base[F.cnt + 1] + at[0];
            for (uint32_t i = 0; i < take; ++i) dst[i] = src[i];
          }
          at[0] += close - rel - 1u;
        } else wide_write_element<W>(S, r, F, lo, (uint64_t)(cb + rel), j, at);
        j++;
      }
    }
    n_el += wide_sum(my_n); tot0 += wide_sum(my0); tot1 += wide_sum(my1);
    if (END != WIDE_NONE) {
      const int el = (int)(END >> 5);
      const uint32_t xlo = __shfl_sync(0xFFFFFFFFu, (uint32_t)endx, el), xhi = __shfl_sync(0xFFFFFFFFu, (uint32_t)(endx >> 32), el);
      s.p = (uint64_t)xlo | ((uint64_t)xhi << 32);
      o.cnt[F.cnt] = n_el;
      if (!objs) o.cnt[F.cnt + 1] = tot0;
      else {
        const ObjDesc& Ed = S.obj[F.child];
        uint32_t q = 0;
        for (int i = 0; i < (int)Ed.nfields; ++i)
          if (Ed.f[i].kind == K_STR) { o.cnt[Ed.f[i].cnt] = q == 0 ? tot0 : tot1; q++; }
      }
      return 1;
    }
    {
      const uint32_t plo = __shfl_sync(0xFFFFFFFFu, (uint32_t)my_pending, (int)last_lane), phi = __shfl_sync(0xFFFFFFFFu, (uint32_t)(my_pending >> 32), (int)last_lane);
      pending = (uint64_t)plo | ((uint64_t)phi << 32);
    }
  }
}

/* ---- the same, for the word-at-a-time tokeniser of pj_fast.cuh -------------------------------------------------- *
 * All lanes of the warp tokenise the record with FSinkWide (same bytes, same steps, everything in registers); a
 * non-empty list arrives here with f.p at its first element. Elements are found by the masks as above; a plain
 * string is sized by the distance of its quotes, any other string by fast_string, a flat object by fast_flat with
 * the lane's own tape column as scratch. In the emitting pass (s.d->c set) every lane then writes its elements at
 * the places the warp scans give them. Returns false (f.err untouched: "refused") for whatever it does not finish;
 * the record then goes to the exact parser. */
__device__ __forceinline__ bool wide_gap32(const Win& w, uint32_t limit, uint32_t p, uint32_t* nxt, uint32_t* endx) {
  uint32_t x;
  for (;;) { x = p < limit ? wbyte(w, p) : 0u; if (x == ' ' || x == '\t' || x == '\r') ++p; else break; }
  *endx = 0;
  if (x == ',') {
    ++p;
    for (;;) { x = p < limit ? wbyte(w, p) : 0u; if (x == ' ' || x == '\t' || x == '\r') ++p; else break; }
    *nxt = p;
    return true;
  }
  if (x == ']') { *endx = p + 1; *nxt = p + 1; return true; }
  return false;
}
/* slot of the one string property of flat object E (NSLOT: it has none) */
template <int E, int I = 0>
constexpr uint32_t wide_string_slot() {
  if constexpr (I >= CObj<E>::N) return NSLOT;
  else return CObj<E>::f[I].kind == K_STR ? CObj<E>::f[I].cnt : wide_string_slot<E, I + 1>();
}
template <int E>
struct WideElem { /* evaluated where the class is instantiated, not inside device code */
  static constexpr uint32_t string_slot = wide_string_slot<E>(), scalars = scalar_words<E>(), strings = string_fields<E>();
};
/* One element that is a flat object, onto the lane's tape (header, scalars, strings) as root_value() lays it out.
 * *bytes: decoded bytes of its string property. */
template <int OBJ, int I>
__device__ __noinline__ bool wide_object_to_tape(const Win& w, const FastState& f, uint32_t pos, Tape& lt, uint32_t* bytes, uint32_t* after) {
  constexpr int E = FK<OBJ, I>::child;
  constexpr uint32_t cnt = FK<OBJ, I>::cnt, SS = WideElem<E>::string_slot;
  static_assert(1 + WideElem<E>::scalars + WideElem<E>::strings <= TAPE_MIN_CAP, "a list element fits an empty tape");
  FastState lf = f;
  lf.p = pos; lf.err = 0; lf.err_pos = 0;
  uint32_t lcnt[NSLOT];
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) lcnt[k] = 0;
  FSinkT<false> ls;
  lt.n = 0;
  ls.t = &lt; ls.cnt = lcnt; ls.d = nullptr;
  for (uint32_t k = 0; k < 1 + WideElem<E>::scalars; ++k) tape_push(lt, 0);
  FVals ev;
  if (!fast_flat<E>(w, lf, ls, ev)) return false;
  tape_set(lt, 0, (uint32_t)TAPE_ELEM | (ev.present << 4) | (cnt << 12));
  tape_put_scalars<E>(lt, 1, ev);
  *bytes = SS < NSLOT ? lcnt[SS < NSLOT ? SS : 0] : 0u;
  *after = lf.p;
  return true;
}

__device__ __forceinline__ uint32_t wide_max(uint32_t x) {
#pragma unroll
  for (int d = 16; d; d >>= 1) { const uint32_t y = __shfl_xor_sync(0xFFFFFFFFu, x, d); x = y > x ? y : x; }
  return x;
}
/* a string that is not plain (escapes, bytes beyond ASCII): its decoded length and the offset behind its closing quote */
static __device__ __noinline__ bool wide_fancy_string(const Win& w, const FastState& f, uint32_t pos, uint32_t* bytes, uint32_t* behind) {
  FastState lf = f;
  lf.p = pos; lf.err = 0; lf.err_pos = 0;
  uint32_t spos, sesc;
  if (!fast_string_t<false>(w, lf, &spos, bytes, &sesc)) return false;
  *behind = lf.p;
  return true;
}
static __device__ __noinline__ uint32_t wide_emit_fancy_string(const Win& w, const FastState& f, uint32_t pos, uint8_t* dst) {
  FastState lf = f;
  lf.p = pos; lf.err = 0; lf.err_pos = 0;
  uint32_t spos = 0, slen = 0, sesc = 0;
  fast_string_t<false>(w, lf, &spos, &slen, &sesc);
  if (sesc) copy_decoded(dst, w.s, spos, slen); else copy_win(dst, w, spos, slen);
  return slen;
}
/* element number j of the list, a flat object at `pos`, into its row of the child table; its string at cursor `at` of
 * its arena. Returns the string's decoded bytes. */
template <int OBJ, int I>
__device__ __noinline__ uint32_t wide_emit_object(const Win& w, const FastState& f, uint32_t pos, Tape& ltape, const DevCols* c, const uint32_t* base, uint32_t j, uint32_t at) {
  constexpr int E = FK<OBJ, I>::child;
  constexpr uint32_t cnt = FK<OBJ, I>::cnt, SS = WideElem<E>::string_slot;
  uint32_t bytes = 0, behind = 0;
  wide_object_to_tape<OBJ, I>(w, f, pos, ltape, &bytes, &behind);
  uint32_t cur[NSLOT];
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) cur[k] = 0;
  cur[cnt] = j;
  if constexpr (SS < NSLOT) cur[SS] = at;
  for (uint32_t k = 0; k < ltape.n;) k = replay_word<OBJ>(w, c, ltape, k, tape_get(ltape, k), base, cur);
  return bytes;
}

template <int OBJ, int I, class S>
__device__ __noinline__ bool wide_fast_list_impl(const Win& w, FastState& f, S& s) {
  constexpr uint32_t kind = FK<OBJ, I>::kind, cnt = FK<OBJ, I>::cnt, col = FK<OBJ, I>::col;
  constexpr bool objs = kind == K_LIST_OBJ;
  constexpr int E = objs ? (int)FK<OBJ, I>::child : (int)OBJ;
  constexpr uint32_t SS = objs ? WideElem<E>::string_slot : cnt + 1; /* the slot the elements' bytes go to */
  if constexpr (objs) { if (WideElem<E>::strings > 1) return false; }
  const uint32_t lane = threadIdx.x & 31u;
  const uint32_t lt = (1u << lane) - 1u, gt = lane == 31 ? 0u : ~((2u << lane) - 1u);
  DrainState& d = *s.d;
  const bool emit = d.c != nullptr;
  /* the tape is emptied first: the lanes use their tape columns as scratch for the elements */
  tape_drain<OBJ>(w, *s.t, s.d);
  s.t->n = 0;
  Tape ltape = *s.t;

  const int32_t p0 = (int32_t)f.p;
  const int32_t end = (int32_t)(s.rec_end < f.limit ? s.rec_end : f.limit);
  int32_t cb = p0 - (int32_t)(reinterpret_cast<uintptr_t>(w.s + p0) & 15u);
  uint32_t esc_c = 0, str_c = 0;
  uint32_t pending = (uint32_t)p0;
  uint32_t n_el = 0, tot = 0;
  for (;; cb += (int32_t)WIDE_STEP) {
    if (cb >= end) return false;
    const int32_t lb = cb + 32 * (int32_t)lane;
    uint32_t B = 0, Q = 0, C = 0, X = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int32_t hb = lb + 16 * h;
      if (hb < end && hb + 16 > p0) {
        const uint4 v = *reinterpret_cast<const uint4*>(w.s + hb);
        const uint64_t w0 = (uint64_t)v.x | ((uint64_t)v.y << 32), w1 = (uint64_t)v.z | ((uint64_t)v.w << 32);
        B |= (wide_movemask(wide_flags_eq(w0, '\\')) | (wide_movemask(wide_flags_eq(w1, '\\')) << 8)) << (16 * h);
        Q |= (wide_movemask(wide_flags_eq(w0, '"')) | (wide_movemask(wide_flags_eq(w1, '"')) << 8)) << (16 * h);
        if (objs) C |= (wide_movemask(wide_flags_eq(w0, '{')) | (wide_movemask(wide_flags_eq(w1, '{')) << 8)) << (16 * h);
        else X |= (wide_movemask(wide_flags_ctrl(w0) | (w0 & 0x8080808080808080ull)) | (wide_movemask(wide_flags_ctrl(w1) | (w1 & 0x8080808080808080ull)) << 8)) << (16 * h);
      }
    }
    const uint32_t valid = wide_low_mask((int64_t)end - lb) & ~wide_low_mask((int64_t)p0 - lb);
    B &= valid; Q &= valid; C &= valid; X &= valid;
    if (__any_sync(0xFFFFFFFFu, B == 0xFFFFFFFFu)) return false;
    const uint32_t cout = (uint32_t)__clz((int)~B) & 1u;
    uint32_t cin = __shfl_up_sync(0xFFFFFFFFu, cout, 1);
    if (lane == 0) cin = esc_c;
    const uint32_t Qu = Q & ~wide_escaped(B, cin);
    const uint32_t par = __ballot_sync(0xFFFFFFFFu, __popc(Qu) & 1);
    const uint32_t sin = ((uint32_t)__popc(par & lt) & 1u) ^ str_c;
    const uint32_t instr = wide_prefix_xor(Qu) ^ (sin ? 0xFFFFFFFFu : 0u);
    const uint32_t starts = objs ? (C & ~instr) : (Qu & instr);
    esc_c = __shfl_sync(0xFFFFFFFFu, cout, 31);
    str_c ^= (uint32_t)__popc(par) & 1u;

    const uint32_t have = __ballot_sync(0xFFFFFFFFu, starts != 0);
    if (!have) continue;
    const uint32_t my_first = starts ? 32u * lane + (uint32_t)(__ffs((int)starts) - 1) : WIDE_NONE;
    const uint32_t after = have & gt;
    const int next_lane = after ? __ffs((int)after) - 1 : 0;
    uint32_t next_first = __shfl_sync(0xFFFFFFFFu, my_first, next_lane);
    if (!after) next_first = WIDE_NONE;
    const uint32_t first_lane = (uint32_t)__ffs((int)have) - 1u, last_lane = 31u - (uint32_t)__clz((int)have);
    WideQuotes wq;
    wq.Qu = Qu; wq.Fm = B | X; wq.lane_bit = 32u * lane; wq.next_close = WIDE_NONE; wq.clean_until = 0;
    if (!objs) {
      const uint32_t qhave = __ballot_sync(0xFFFFFFFFu, Qu != 0), fhave = __ballot_sync(0xFFFFFFFFu, wq.Fm != 0);
      const uint32_t qafter = qhave & gt;
      const int nql = qafter ? __ffs((int)qafter) - 1 : 0;
      const uint32_t nq_bit = __shfl_sync(0xFFFFFFFFu, Qu ? (uint32_t)__ffs((int)Qu) - 1u : 0u, nql);
      const uint32_t nq_f = __shfl_sync(0xFFFFFFFFu, wq.Fm, nql);
      if (qafter) {
        wq.next_close = 32u * (uint32_t)nql + nq_bit;
        wq.clean_until = !(fhave & gt & ((1u << nql) - 1u)) && !(nq_f & ((1u << nq_bit) - 1u));
      }
    }

    /* ---- first walk: sizes, separators, links. The lanes walk in step: as many rounds as the busiest lane has
       elements, one exit, a lane that is done (or has found something wrong) idles through the rest ---- */
    const uint32_t rounds = wide_max((uint32_t)__popc(starts));
    uint32_t bad = WIDE_NONE, end_rel = WIDE_NONE, my_n = 0, my_b = 0, endx = 0, my_pending = 0;
    {
      uint32_t m = starts;
      bool go = true, first = lane == first_lane;
      for (uint32_t it = 0; it < rounds; ++it) {
        const bool act = go && m != 0;
        const uint32_t b = act ? (uint32_t)__ffs((int)m) - 1u : 0u;
        if (act) m &= m - 1u;
        const uint32_t rel = 32u * lane + b;
        const uint32_t pos = (uint32_t)(cb + (int32_t)rel);
        const uint32_t succ = m ? 32u * lane + (uint32_t)(__ffs((int)m) - 1) : next_first;
        bool ok = act && !(first && pos != pending);
        if (act) first = false;
        uint32_t bytes = 0, behind = 0, nxt = 0, ex = 0;
        if constexpr (objs) {
          if (ok) ok = wide_object_to_tape<OBJ, I>(w, f, pos, ltape, &bytes, &behind);
        } else {
          const uint32_t close = ok ? wide_plain_close(wq, b) : WIDE_NONE;
          if (close != WIDE_NONE) { bytes = close - rel - 1u; behind = (uint32_t)(cb + (int32_t)close) + 1u; }
          else if (ok) ok = wide_fancy_string(w, f, pos, &bytes, &behind);
        }
        if (ok) ok = wide_gap32(w, f.limit, behind, &nxt, &ex);
        if (ok && !ex && succ != WIDE_NONE && (uint32_t)(cb + (int32_t)succ) != nxt) ok = false;
        if (act) {
          if (!ok) { bad = rel; go = false; }
          else {
            my_n++; my_b += bytes;
            if (ex) { end_rel = rel; endx = ex; go = false; }
            else if (succ == WIDE_NONE) my_pending = nxt;
          }
        }
      }
    }
    const uint32_t END = wide_min(end_rel), BAD = wide_min(bad);
    if (BAD != WIDE_NONE && (END == WIDE_NONE || BAD <= END)) return false;
    if (END != WIDE_NONE && lane > (END >> 5)) { my_n = 0; my_b = 0; }
    const uint32_t ex_n = wide_excl(my_n, lane), ex_b = wide_excl(my_b, lane);

    /* ---- second walk (emitting pass): every element knows its place now ---- */
    if (emit) {
      uint32_t m = starts, j = d.cur[cnt] + n_el + ex_n, at = d.cur[SS < NSLOT ? SS : 0] + tot + ex_b;
      for (uint32_t it = 0; it < rounds; ++it) {
        const uint32_t b = m ? (uint32_t)__ffs((int)m) - 1u : 0u;
        const uint32_t rel = 32u * lane + b;
        const bool act = m != 0 && rel <= END; /* END == WIDE_NONE: no element is beyond it */
        m &= m - 1u;
        const uint32_t pos = (uint32_t)(cb + (int32_t)rel);
        if constexpr (objs) {
          if (act) at += wide_emit_object<OBJ, I>(w, f, pos, ltape, d.c, d.base, j, at);
        } else {
          const uint32_t close = act ? wide_plain_close(wq, b) : WIDE_NONE;
          if (act) {
            uint8_t* dst = colp<uint8_t>(d.c, col + 2) + d.base[cnt + 1] + at;
            colp<uint32_t>(d.c, col + 1)[(uint64_t)d.base[cnt] + j] = d.base[cnt + 1] + at;
            if (close != WIDE_NONE) { copy_win(dst, w, pos + 1u, close - rel - 1u); at += close - rel - 1u; }
            else at += wide_emit_fancy_string(w, f, pos, dst);
          }
        }
        if (act) j++;
      }
    }
    n_el += wide_sum(my_n); tot += wide_sum(my_b);
    if (END != WIDE_NONE) {
      f.p = __shfl_sync(0xFFFFFFFFu, endx, (int)(END >> 5));
      s.cnt[cnt] = n_el;
      d.cur[cnt] += n_el;
      if constexpr (SS < NSLOT) { s.cnt[SS] += tot; d.cur[SS] += tot; }
      return true;
    }
    pending = __shfl_sync(0xFFFFFFFFu, my_pending, (int)last_lane);
  }
}

/* A long record by all lanes of a warp with the word-at-a-time tokeniser: the counting pass (c == null: verdict as
 * fast_record<>(), counts in cnt_out[NSLOT], model in *type_out) or the emitting pass of a record the counting pass
 * accepted. rec_end: window offset of the byte that ends the record. Every lane passes its own tape column. */
template <int SCHEMA>
__device__ __noinline__ uint32_t wide_outline(const Win w, uint32_t start, uint32_t limit, uint32_t rec_end, uint32_t open_end, const DevCols* c,
                                              const uint32_t* base, uint64_t rec_index, Tape t, uint32_t* cnt_out, uint32_t* type_out,
                                              uint32_t* err_kind, uint32_t* err_pos) {
  FastState f;
  f.p = start; f.limit = limit; f.lf_ws = 0; f.err = 0; f.err_pos = 0;
  DrainState d;
  d.c = c; d.base = base;
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) d.cur[k] = 0;
  FVals v, cv;
  uint32_t cnt[NSLOT], type = PJ_TYPE_NONE;
  FSinkWide s;
  s.t = &t; s.cnt = cnt; s.d = &d; s.rec_end = rec_end;
  if (!fast_record_sink<SCHEMA>(w, f, open_end, &type, v, cv, s)) {
    if (!f.err) return FAST_REFUSED;
    *err_kind = f.err; *err_pos = f.err_pos;
    return FAST_FAILED;
  }
  if (c) emit_typed<SCHEMA>(w, c, type, v, cv, t, base, rec_index, d.cur);
  else {
#pragma unroll
    for (uint32_t k = 0; k < NSLOT; ++k) cnt_out[k] = cnt[k];
    *type_out = type;
  }
  return FAST_ACCEPTED;
}
#endif /* __CUDACC__ */

template <int OBJ, int I, class S>
PJ_HD bool wide_fast_list(const Win& w, FastState& f, S& s) {
#if defined(__CUDA_ARCH__)
  return wide_fast_list_impl<OBJ, I>(w, f, s);
#else
  return false;
#endif
}

/* The hook parse_record<>() is instantiated with for records a whole warp walks together. */
struct WarpListHook {
  static constexpr bool enabled = true;
  template <bool W>
  static PJ_HD int list(const Schema& S, const Rd& r, PS& s, const FieldDesc& F, Out<W>& o) {
#if defined(__CUDA_ARCH__)
    return wide_list<W>(S, r, s, F, o);
#else
    return 0;
#endif
  }
};

}  // namespace pj
#endif
