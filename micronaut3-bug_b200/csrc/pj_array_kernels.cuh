/*
 * pj_array_kernels.cuh — kernels of the array-framing record index (see pj_array.cuh for the method).
 *
 *   k_arr_summary   every thread summarises its 64-byte word as a function of the incoming (escape carry,
 *                   in-string) state; an ordered shuffle reduction gives one function per 16 KiB tile
 *   k_arr_scan_tiles   composes the tile functions in order (one warp, 32 runs) -> incoming state of every tile, final state
 *   k_arr_mark      re-evaluates every word with its exact incoming state (ordered scan inside the block),
 *                   writes the separator bitmap, finds the first opener and the first stray byte
 *   k_arr_records<> one candidate per separator: extent, blank test, keep / drop; count per tile, then
 *                   (after a scan) store rec_start / rec_end / rec_blank
 */
#ifndef PJ_ARRAY_KERNELS_CUH
#define PJ_ARRAY_KERNELS_CUH

#include "pj_array.cuh"
#include "pj_kernels.cuh"

namespace pj {

static constexpr int ARR_THREADS = 256; /* words per block: one block covers 16 KiB, like the NDJSON index */

struct ArrArgs {
  const uint8_t* in;
  uint64_t len, nwords;
  ArrFn* tile_fn;      /* [tiles] */
  ArrState* tile_in;   /* [tiles] */
  uint64_t* sep;       /* [nwords] separator bitmap */
  uint32_t* tile_cnt;  /* [tiles + 1] */
  uint64_t* rec_start; /* outputs of k_arr_records<true> */
  uint64_t* rec_end;
  uint8_t* rec_blank;
  uint64_t cap, goff;
  uint32_t ntiles;
  DevResult* res;
};

/* masks of word w of the input: 16-byte loads when the input is 16-byte aligned and the word is whole */
__device__ __forceinline__ WordMasks load_word_masks(const ArrArgs& a, uint64_t w) {
  const uint64_t off = w << 6;
  const uint32_t n = a.len - off >= 64 ? 64u : (uint32_t)(a.len - off);
  if (n == 64 && (reinterpret_cast<uintptr_t>(a.in) & 15u) == 0) {
    const uint4* q = reinterpret_cast<const uint4*>(a.in + off);
    WordMasks m;
    m.B = m.Q = m.O = m.C = m.M = m.W = m.LB = m.RB = 0;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint4 v = __ldg(q + k);
      const uint64_t w2[2] = {(uint64_t)v.x | ((uint64_t)v.y << 32), (uint64_t)v.z | ((uint64_t)v.w << 32)};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint64_t x = w2[h];
        const int sh = 16 * k + 8 * h;
        const uint64_t lb = eq_bits8(x, '['), rb = eq_bits8(x, ']'), lc = eq_bits8(x, '{'), rc = eq_bits8(x, '}');
        const uint64_t ws = eq_bits8(x, ' ') | eq_bits8(x, '\t') | eq_bits8(x, '\r') | eq_bits8(x, '\n');
        m.B |= (uint64_t)eq_bits8(x, '\\') << sh;
        m.Q |= (uint64_t)eq_bits8(x, '"') << sh;
        m.M |= (uint64_t)eq_bits8(x, ',') << sh;
        m.LB |= lb << sh; m.RB |= rb << sh;
        m.O |= (lb | lc) << sh; m.C |= (rb | rc) << sh;
        m.W |= ws << sh;
      }
    }
    m.valid = ~0ull;
    return m;
  }
  return word_masks(a.in + off, n);
}

__device__ __forceinline__ ArrFn fn_shfl_up(const ArrFn& f, int d) {
  ArrFn g;
  g.st = __shfl_up_sync(0xFFFFFFFFu, f.st, d);
#pragma unroll
  for (int k = 0; k < 4; ++k) g.d[k] = __shfl_up_sync(0xFFFFFFFFu, f.d[k], d);
  return g;
}
/* inclusive ordered scan of the warp's functions (lane 0 first) */
__device__ __forceinline__ ArrFn fn_warp_scan(ArrFn f) {
  const unsigned lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const ArrFn g = fn_shfl_up(f, d);
    if (lane >= (unsigned)d) f = fn_compose(g, f);
  }
  return f;
}

static __global__ void __launch_bounds__(ARR_THREADS) k_arr_summary(const __grid_constant__ ArrArgs a) {
  __shared__ ArrFn sh[ARR_THREADS / 32];
  const uint64_t w = (uint64_t)blockIdx.x * ARR_THREADS + threadIdx.x;
  ArrFn f = fn_identity();
  if (w < a.nwords) f = fn_of_word(load_word_masks(a, w));
  f = fn_warp_scan(f);
  if ((threadIdx.x & 31) == 31) sh[threadIdx.x >> 5] = f;
  __syncthreads();
  if (threadIdx.x == 0) {
    ArrFn t = sh[0];
    for (int k = 1; k < ARR_THREADS / 32; ++k) t = fn_compose(t, sh[k]);
    a.tile_fn[blockIdx.x] = t;
  }
}

/* One warp: every lane composes a contiguous run of tile functions, an ordered scan over the 32 runs gives each lane
 * the state its run starts in, and the lane walks its run once more to leave every tile's incoming state. */
static __global__ void k_arr_scan_tiles(const __grid_constant__ ArrArgs a) {
  if (blockIdx.x || threadIdx.x >= 32) return;
  const unsigned lane = threadIdx.x;
  const uint32_t per = (a.ntiles + 31) / 32;
  const uint32_t lo = lane * per < a.ntiles ? lane * per : a.ntiles;
  const uint32_t hi = lo + per < a.ntiles ? lo + per : a.ntiles;
  ArrFn f = fn_identity();
  for (uint32_t t = lo; t < hi; ++t) f = fn_compose(f, a.tile_fn[t]);
  const ArrFn inc = fn_warp_scan(f);
  ArrFn prev = fn_shfl_up(inc, 1);
  if (lane == 0) prev = fn_identity();
  ArrState st;
  st.c = 0; st.s = 0; st.d = 0;
  st = fn_apply(prev, st);
  for (uint32_t t = lo; t < hi; ++t) {
    a.tile_in[t] = st;
    st = fn_apply(a.tile_fn[t], st);
  }
  if (lane == 31) { /* its run is the last one (possibly empty): the state after every tile */
    a.res->arr_final_s = st.s;
    a.res->arr_final_d = st.d;
  }
}

static __global__ void __launch_bounds__(ARR_THREADS) k_arr_mark(const __grid_constant__ ArrArgs a) {
  __shared__ ArrFn sh[ARR_THREADS / 32];
  const uint64_t w = (uint64_t)blockIdx.x * ARR_THREADS + threadIdx.x;
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  WordMasks m;
  ArrFn f = fn_identity();
  const bool live = w < a.nwords;
  if (live) { m = load_word_masks(a, w); f = fn_of_word(m); }
  const ArrFn inc = fn_warp_scan(f);
  if (lane == 31) sh[warp] = inc;
  __syncthreads();
  /* everything before this word inside the tile: the warps before, then the lanes before */
  ArrFn before = fn_identity();
  for (unsigned k = 0; k < warp; ++k) before = fn_compose(before, sh[k]);
  ArrFn prev = fn_shfl_up(inc, 1);
  if (lane == 0) prev = fn_identity();
  before = fn_compose(before, prev);
  if (!live) return;
  const ArrState in = fn_apply(before, a.tile_in[blockIdx.x]);
  const WordEval e = eval_word(m, in);
  const WordMarks k = mark_word(m, e, in.d);
  a.sep[w] = k.sep;
  if (k.doc_bit < 64) atomicMin(&a.res->doc_err_off, (unsigned long long)((w << 6) + k.doc_bit));
  if (k.opener_bit < 64) atomicMin(&a.res->first_opener, (unsigned long long)((w << 6) + k.opener_bit));
}

template <bool WRITE>
__global__ void __launch_bounds__(ARR_THREADS) k_arr_records(const __grid_constant__ ArrArgs a) {
  __shared__ uint32_t sh[33];
  const uint64_t w = (uint64_t)blockIdx.x * ARR_THREADS + threadIdx.x;
  const unsigned long long first_opener = a.res->first_opener;
  uint64_t seps = w < a.nwords ? a.sep[w] : 0;
  uint32_t cnt = 0;
  for (uint64_t t = seps; t; t &= t - 1) {
    const uint64_t p = (w << 6) + ctz64a(t);
    const ExtentOut x = arr_extent(a.in, a.len, a.sep, p, first_opener);
    if (!WRITE && x.second_opener) atomicMin(&a.res->doc_err_off, (unsigned long long)p);
    cnt += x.is_record;
  }
  uint32_t total;
  const uint32_t ex = block_excl_scan(cnt, &total, sh);
  if (!WRITE) {
    if (threadIdx.x == 0) a.tile_cnt[blockIdx.x] = total;
    return;
  }
  uint64_t at = (uint64_t)a.tile_cnt[blockIdx.x] + ex;
  for (uint64_t t = seps; t; t &= t - 1) {
    const uint64_t p = (w << 6) + ctz64a(t);
    const ExtentOut x = arr_extent(a.in, a.len, a.sep, p, first_opener);
    if (!x.is_record) continue;
    if (at < a.cap) {
      a.rec_start[at] = x.start + a.goff;
      if (a.rec_end) a.rec_end[at] = x.end;
      if (a.rec_blank) a.rec_blank[at] = (uint8_t)x.blank;
    }
    at++;
  }
}

}  // namespace pj
#endif
