/*
 * pj_kernels.cuh — sm_100a kernels and the device helpers they share.
 *
 * NDJSON is parsed by k_parse_stream (pj_stream_kernel.cuh), which builds its own line index. This header holds
 *   - the block scan, the look-back words, the bulk-copy (cp.async.bulk / mbarrier) wrappers that every kernel uses;
 *   - the NDJSON record index on its own (k_nd_index<false> / k_scan_single / k_nd_index<true>: pj_index_records and
 *     its allocation-free variant);
 *   - k_parse_tile<SCHEMA>: the tile kernel over a GIVEN record index, 128 records per block (array framing, whose
 *     index comes from pj_array_kernels.cuh);
 *   - the writer: columns --k_arena_flags--> "any byte to escape?" --k_write_tile--> text --k_write_close--> brackets, total.
 *
 * Kernels that wait on other blocks (the look-backs) take their tile from an atomic ticket, so every block they
 * wait for is running or done, and every wait is bounded (the spin limit of the kernel's arguments ->
 * DevResult.timeout -> PJ_ERR_TIMEOUT).
 */
#ifndef PJ_KERNELS_CUH
#define PJ_KERNELS_CUH

#include <cuda_runtime.h>

#include "pj_core.cuh"
#include "pj_fast.cuh"
#include "pj_index.cuh"
#include "pj_write_core.cuh"
#include "pj_write_fast.cuh"

namespace pj {

/* one copy per translation unit that includes this header (each sets its own, see tile_init_*) */
static __constant__ Schema c_schema;

/* Written by the kernels, read back by the host once per call. */
struct DevResult {
  unsigned long long n_records;
  unsigned long long n_errors;
  unsigned long long total[NSLOT];
  unsigned long long out_bytes; /* writer: JSON bytes */
  unsigned long long doc_err_off;
  uint32_t doc_err_kind;
  uint32_t ok;      /* every output fits its buffer */
  uint32_t over;    /* stream kernel: some output does not fit its buffer */
  uint32_t timeout; /* a bounded wait ran out */
  uint32_t needs_escape; /* writer: some string byte of the columns has to be escaped (k_arena_flags) */
  unsigned long long n_fast;  /* records decoded by the speculative pass alone */
  unsigned long long phase_cycles[4]; /* tile kernel, summed over blocks: staging, tokenising, look-back, emit */
  unsigned long long lookback_polls, lookback_rounds;
  unsigned long long n_wide;       /* records walked by a whole warp */
  unsigned long long n_wide_fast;  /* of those, finished by the word-at-a-time tokeniser (the rest: the exact parser) */
  unsigned long long wide_cycles[2]; /* cycles the blocks spent in the warps' size pass / emit pass, summed over blocks */
  unsigned long long first_opener; /* array framing: offset of the first `[` at depth 0 */
  uint32_t arr_final_s;            /* array framing: the input ends inside a string */
  int32_t arr_final_d;             /* array framing: nesting depth at the end of the input */
};

static constexpr int INDEX_THREADS = 256;
static constexpr int INDEX_BYTES_PER_THREAD = 64;
static constexpr int INDEX_TILE = INDEX_THREADS * INDEX_BYTES_PER_THREAD; /* 16 KiB */

/* A failure the word-at-a-time paths report that an option turns into something else (an unknown enum literal into an
 * absent property, a value of another JSON type into a coerced one): such records go to the exact parser, which
 * knows the options. */
__device__ __forceinline__ bool opt_decides(uint32_t opts, uint32_t kind) {
  return ((opts & PJ_OPT_ENUM_UNKNOWN_AS_NULL) && kind == PJ_E_ENUM) || ((opts & PJ_OPT_COERCE_SCALARS) && kind == PJ_E_TYPE);
}

/* ---- block-wide exclusive scan ---------------------------------------------------------------- */
template <class T>
__device__ __forceinline__ T warp_incl_scan(T v) {
  const unsigned lane = threadIdx.x & 31;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    T u = __shfl_up_sync(0xFFFFFFFFu, v, d);
    if (lane >= (unsigned)d) v += u;
  }
  return v;
}
/* Exclusive prefix of v over the block (any multiple of 32 threads up to 1024); *total = block sum.
 * `sh` needs 33 entries. Safe to call repeatedly. */
template <class T>
__device__ __forceinline__ T block_excl_scan(T v, T* total, T* sh) {
  const unsigned lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  T inc = warp_incl_scan(v);
  __syncthreads(); /* protect sh from the previous call */
  if (lane == 31) sh[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    T w = lane < nwarps ? sh[lane] : T(0);
    T wi = warp_incl_scan(w);
    if (lane < nwarps) sh[lane] = wi - w;
    if (lane == nwarps - 1) sh[32] = wi;
  }
  __syncthreads();
  *total = sh[32];
  return sh[warp] + inc - v;
}

/* ---- NDJSON record index ---------------------------------------------------------------------- */
/* 64-bit mask of the LF bytes among the 64 bytes at the 16-byte aligned address a, of which the
 * first `valid` (>= 1) belong to the input. */
__device__ __forceinline__ uint64_t lf_mask64(const uint8_t* a, uint64_t valid) {
  const uint4* q = reinterpret_cast<const uint4*>(a);
  uint64_t m = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    if ((uint64_t)(k * 16) >= valid) break; /* never touch a 16-byte block that holds no input byte */
    uint4 v = __ldg(q + k);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t e = __vcmpeq4(w[j], 0x0A0A0A0Au) & 0x01010101u; /* 1 per matching byte */
      uint32_t nib = (e * 0x01020408u) >> 24;                  /* gather the four flags */
      m |= (uint64_t)(nib & 0xF) << (k * 16 + j * 4);
    }
  }
  return m;
}

struct IndexArgs {
  const uint8_t* in;
  uint64_t len, limit;
  int is_first, is_last;
  uint32_t* tile; /* [tiles + 1]: counts, then (after the scan) exclusive bases */
  uint64_t* rec_start;
  uint64_t cap, goff;
};

/* One thread looks at 64 input bytes. Every LF inside [0, len) makes the following byte a candidate
 * line start; byte 0 is one too when the shard is the first of its stream. WRITE = false counts the
 * candidates that are records per tile; WRITE = true stores their offsets at the scanned positions. */
template <bool WRITE>
__global__ void __launch_bounds__(INDEX_THREADS) k_nd_index(const __grid_constant__ IndexArgs a) {
  __shared__ uint32_t sh[33];
  const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(a.in) & 15u);
  const uint8_t* base = a.in - mis; /* 16-byte aligned */
  const uint64_t v0 = (uint64_t)blockIdx.x * INDEX_TILE + (uint64_t)threadIdx.x * INDEX_BYTES_PER_THREAD; /* offset from base */
  const uint64_t vend = a.len ? a.len + mis : 0; /* an empty input is never dereferenced */
  uint64_t m = 0;
  if (v0 < vend) {
    m = lf_mask64(base + v0, vend - v0);
    if (v0 < mis) m &= ~0ull << (mis - v0);               /* bytes before in[0] */
    if (vend - v0 < 64) m &= ~(~0ull << (vend - v0));      /* bytes at or after in[len] */
  }
  const bool head = a.is_first && blockIdx.x == 0 && threadIdx.x == 0; /* candidate at byte 0 */
  uint32_t cnt = 0;
  if (!WRITE) {
    if (head && nd_is_record(a.in, 0, a.limit, a.is_last)) cnt++;
    for (uint64_t t = m; t; t &= t - 1) {
      uint64_t p = v0 + (uint64_t)(__ffsll((long long)t) - 1) - mis + 1;
      if (nd_is_record(a.in, p, a.limit, a.is_last)) cnt++;
    }
    uint32_t total;
    block_excl_scan(cnt, &total, sh);
    if (threadIdx.x == 0) a.tile[blockIdx.x] = total;
  } else {
    /* recount, then place */
    uint64_t keep = 0;
    bool head_keep = head && nd_is_record(a.in, 0, a.limit, a.is_last);
    cnt = head_keep ? 1u : 0u;
    for (uint64_t t = m; t; t &= t - 1) {
      int b = __ffsll((long long)t) - 1;
      uint64_t p = v0 + (uint64_t)b - mis + 1;
      if (nd_is_record(a.in, p, a.limit, a.is_last)) { keep |= 1ull << b; cnt++; }
    }
    uint32_t total;
    uint64_t at = (uint64_t)a.tile[blockIdx.x] + block_excl_scan(cnt, &total, sh);
    if (head_keep) { if (at < a.cap) a.rec_start[at] = a.goff; at++; }
    for (uint64_t t = keep; t; t &= t - 1) {
      uint64_t p = v0 + (uint64_t)(__ffsll((long long)t) - 1) - mis + 1;
      if (at < a.cap) a.rec_start[at] = p + a.goff;
      at++;
    }
  }
}

/* ---- scans over device-resident lengths -------------------------------------------------------- */
/* Single block: exclusive scan of data[0..n) in place, data[n] = total; also *total_out. */
template <class T>
__global__ void __launch_bounds__(1024) k_scan_single(T* data, uint64_t n, unsigned long long* total_out) {
  __shared__ T sh[33];
  T carry = 0;
  for (uint64_t b = 0; b < n; b += blockDim.x) {
    uint64_t i = b + threadIdx.x;
    T v = i < n ? data[i] : T(0), tot;
    T ex = block_excl_scan(v, &tot, sh);
    if (i < n) data[i] = carry + ex;
    carry += tot;
  }
  if (threadIdx.x == 0) { data[n] = carry; if (total_out) *total_out = (unsigned long long)carry; }
}

/* ---- writer arguments ------------------------------------------------------------------------- */
struct WriteArgs {
  uint64_t n;             /* records (mixed) or rows */
  uint32_t schema, array; /* array: wrap as [r,r,...] */
  int inclusion;
  uint32_t hexa;          /* 'A' or 'a': hex letters of \u00xx escapes */
  uint8_t* out;
  uint64_t cap;
  DevResult* res;
  DevCols cols;
};


/* ================================================================================================
 * Single-pass tile kernel
 *
 * One thread block takes TILE_THREADS consecutive records (a "tile"), stages their bytes in shared
 * memory with coalesced 16-byte loads, lets every thread tokenise its record ONCE (speculative
 * word-at-a-time pass of pj_fast.cuh, exact generic parser as fallback), scans the per-record counts
 * inside the block, obtains the tile's start in every arena by a decoupled look-back over the tiles
 * before it, and then emits every column. Input bytes are read from HBM once, every output byte is
 * written once.
 *
 * Look-back protocol (per tile: aggregate[NSLOT], inclusive[NSLOT], each word with its own valid bit): a
 * tile publishes its aggregate as soon as its records are sized and its inclusive prefix once it has
 * found the nearest predecessor whose inclusive prefix is published and added the aggregates in between. Tiles take their
 * index from an atomic ticket, so every predecessor of a running tile is itself running or done and
 * the waits cannot deadlock. Every wait is bounded: after the spin limit it raises res->timeout,
 * which all other waits also watch, and the block finishes without emitting.
 * ================================================================================================ */
static constexpr int TILE_THREADS = 128;
static constexpr uint32_t TILE_WIN_BYTES = 44 * 1024;  /* staged input bytes per tile */
static constexpr uint32_t TILE_TAPE_CAP = 20;          /* 32-bit tape words per record before the generic parser takes over */
static constexpr uint32_t TILE_SMEM_BYTES = ((TILE_WIN_BYTES + 64 + 15) & ~15u) + TILE_TAPE_CAP * TILE_THREADS * 4;

/* Look-back state of one tile. Every word carries its own "valid" bit (bit 63) next to a 32-bit value and
 * is written once with a single 64-bit store, so a reader needs no fence and gets status and value in the
 * same round trip: agg = the tile's own totals, inc = totals of all tiles up to and including it. */
struct TileState {
  unsigned long long agg[NSLOT];
  unsigned long long inc[NSLOT];
  unsigned long long pad[2];
};
static_assert(sizeof(TileState) == 256, "two 128-byte lines per tile state");
static constexpr unsigned long long TS_VALID = 1ull << 63;

struct TileArgs {
  const uint8_t* in;
  uint64_t limit, goff, n_records;
  uint32_t lf_ws, open_end, schema, slot_lo, slot_hi;
  uint32_t tile_recs, ntiles, win_bytes, tape_cap;
  unsigned long long spin_limit_ns; /* bound of every wait on another block or on the staging copy */
  uint32_t opts;                    /* PJ_OPT_* bits that change a rule */
  const uint64_t* rec_end;  /* array framing: end of every extent, else null */
  const uint8_t* rec_blank; /* array framing: extent without a value */
  TileState* tiles;
  uint32_t* ticket;
  DevResult* res;
  uint64_t slot_cap[NSLOT]; /* largest total per slot the caller's buffers can take */
  uint32_t slot_base[NSLOT]; /* totals of the pieces of the same call parsed before this launch: where this
                                launch starts in every arena / child table (offsets stored are absolute) */
  FinalizePlan plan;
  DevCols cols;
};

__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

/* Exclusive prefix of tile `tile` over all earlier tiles for the slots LO..HI-1, into excl[] (every lane
 * gets all of them). Warp 0 only, all 32 lanes. Each round looks at the 32 tiles before position j with one
 * memory round trip: lane L loads every agg and inc word of tile j - L, the warp finds the nearest tile whose
 * inclusive totals are published, and a shuffle reduction adds its inclusive totals to the aggregates of
 * the tiles after it. Returns false when the bounded wait ran out. */
template <uint32_t LO, uint32_t HI>
__device__ __forceinline__ bool tile_lookback(const TileArgs& a, uint32_t tile, uint32_t lane, uint32_t* excl) {
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) excl[k] = 0;
  int64_t j = (int64_t)tile - 1;
  const unsigned long long t0 = global_ns();
  unsigned polls = 0, rounds = 0;
  while (j >= 0) {
    const int64_t mine = j - lane; /* lane L looks at tile j - L; tiles before the first count as "inclusive, zero" */
    uint32_t va[NSLOT], vi[NSLOT];
    uint32_t first_inc;
    for (;;) {
      bool has_inc = true, has_agg = true;
#pragma unroll
      for (uint32_t k = LO; k < HI; ++k) {
        unsigned long long wa = TS_VALID, wi = TS_VALID;
        if (mine >= 0) { wi = ld_relaxed_u64(&a.tiles[mine].inc[k]); wa = ld_relaxed_u64(&a.tiles[mine].agg[k]); }
        has_inc = has_inc && (wi & TS_VALID);
        has_agg = has_agg && (wa & TS_VALID);
        va[k] = (uint32_t)wa; vi[k] = (uint32_t)wi;
      }
      const uint32_t inc_mask = __ballot_sync(0xFFFFFFFFu, has_inc);
      const uint32_t ready_mask = __ballot_sync(0xFFFFFFFFu, has_inc || has_agg);
      first_inc = inc_mask ? (uint32_t)(__ffs((int)inc_mask) - 1) : 32u;
      const uint32_t need = first_inc >= 31 ? 0xFFFFFFFFu : ((2u << first_inc) - 1u);
      if ((ready_mask & need) == need) break;
      ++polls;
      uint32_t give_up = 0;
      if (lane == 0) give_up = (global_ns() - t0 > a.spin_limit_ns) || *(volatile uint32_t*)&a.res->timeout;
      give_up = __shfl_sync(0xFFFFFFFFu, give_up, 0);
      if (give_up) { if (lane == 0) atomicExch(&a.res->timeout, 1u); return false; }
      __nanosleep(100);
    }
    ++rounds;
#pragma unroll
    for (uint32_t k = LO; k < HI; ++k) {
      uint32_t c = lane < first_inc ? va[k] : (lane == first_inc ? vi[k] : 0u);
#pragma unroll
      for (int d = 16; d; d >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, d);
      excl[k] += c;
    }
    if (first_inc < 32) break;
    j -= 32;
  }
  if (lane == 0) { atomicAdd(&a.res->lookback_polls, (unsigned long long)polls); atomicAdd(&a.res->lookback_rounds, (unsigned long long)rounds); }
  return true;
}

/* ---- bulk asynchronous copy (TMA, untiled form) global -> shared, completion on an mbarrier ------------ */
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long* bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}
/* dst and src 16-byte aligned, bytes a multiple of 16; no multicast: the copy lands in this block's own shared memory */
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, unsigned long long* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst)), "l"(src),
               "r"(bytes), "r"(smem_addr(bar))
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return done != 0;
}
/* bounded: false when the copy has not landed after limit_ns */
__device__ __forceinline__ bool mbar_wait_bounded(unsigned long long* bar, uint32_t parity, unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_ns() - t0 > limit_ns) return false;
    __nanosleep(64);
  }
}

/* bulk asynchronous copy shared -> global (same alignment rules); the issuing thread waits until shared memory
 * has been read before the block may leave */
__device__ __forceinline__ void bulk_s2g(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_addr(src)), "r"(bytes) : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void bulk_s2g_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
/* makes this thread's earlier writes to shared memory visible to the asynchronous proxy (the bulk copy engine) */
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

/* A cheap guess at the model of the record at p (n readable bytes), from the first key that is not `id`:
 * 1 Pet, 2 Order, 3 User, 0 no idea. It only decides which records share a warp, never a result. */
__device__ __forceinline__ uint32_t guess_model(const uint8_t* p, uint64_t n) {
  const uint32_t lim = n < 96 ? (uint32_t)n : 96u;
  uint32_t q = 0;
  for (int key = 0; key < 2; ++key) {
    while (q < lim && (p[q] == ' ' || p[q] == '\t' || p[q] == '\r' || p[q] == '{' || p[q] == ',')) ++q;
    if (q + 6 >= lim || p[q] != '"') return 0;
    const uint32_t c0 = p[q + 1], c1 = p[q + 2], c3 = p[q + 4];
    if (c0 == 'i' && c1 == 'd' && p[q + 3] == '"') { /* common to all: skip its value */
      q += 4;
      while (q < lim && p[q] != ',') ++q;
      continue;
    }
    switch (c0) {
      case 'c': return c1 == 'a' ? 1u : 2u;            /* category | complete */
      case 'n': case 't': return 1u;                  /* name, tags */
      case 'q': return 2u;                            /* quantity */
      case 'u': case 'f': case 'l': case 'e': return 3u; /* username, userStatus, firstName, lastName, email */
      case 's': return c1 == 'h' ? 2u : 0u;            /* shipDate | status (Pet or Order) */
      case 'p': return c1 == 'e' ? 2u : (c1 == 'a' ? 3u : (c3 == 't' ? 1u : 3u)); /* petId | password | photoUrls | phone */
      default: return 0;
    }
  }
  return 0;
}

template <int SCHEMA> struct SlotRange {
  static constexpr uint32_t lo = SCHEMA == PJ_SCHEMA_PET ? (uint32_t)SLOT_PET_CAT_NAME : (SCHEMA == PJ_SCHEMA_USER ? (uint32_t)SLOT_USR_STR0 : 0u);
  static constexpr uint32_t hi = SCHEMA == PJ_SCHEMA_PET ? (uint32_t)SLOT_USR_STR0 : (SCHEMA == PJ_SCHEMA_ORDER ? 0u : (uint32_t)NSLOT);
};

template <int SCHEMA>
__global__ void __launch_bounds__(TILE_THREADS, SCHEMA == PJ_SCHEMA_MIXED ? 3 : 4) k_parse_tile(const __grid_constant__ TileArgs a) {
  constexpr uint32_t LO = SlotRange<SCHEMA>::lo, HI = SlotRange<SCHEMA>::hi;
  constexpr uint32_t NWARPS = TILE_THREADS / 32;
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ uint32_t sh_warp[NSLOT][NWARPS];
  __shared__ uint32_t sh_tot[NSLOT], sh_base[NSLOT];
  __shared__ uint32_t sh_tile, sh_ok;
  __shared__ __align__(8) unsigned long long sh_mbar; /* completion of the bulk copy that stages the window */
  constexpr bool SORTED = SCHEMA == PJ_SCHEMA_MIXED;
  __shared__ uint32_t sh_cls[5][NWARPS];
  __shared__ uint32_t sh_perm[SORTED ? TILE_THREADS : 1];
  __shared__ uint32_t sh_x[SORTED ? NSLOT * TILE_THREADS : 1]; /* counts, then tile-local bases, in record order */
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint8_t* win = smem;
  uint32_t* tape = reinterpret_cast<uint32_t*>(smem + ((a.win_bytes + 64 + 15) & ~15u));

  if (tid == 0) { sh_tile = atomicAdd(a.ticket, 1u); mbar_init(&sh_mbar, 1); }
  __syncthreads();
  const uint32_t tile = sh_tile;
  if (tile >= a.ntiles) return;
  const uint64_t N = a.n_records;
  const uint64_t r0 = (uint64_t)tile * a.tile_recs;
  const uint64_t left = N > r0 ? N - r0 : 0;
  const uint32_t nrec = left < a.tile_recs ? (uint32_t)left : a.tile_recs;
  const uint64_t* rec_start = colp<uint64_t>(&a.cols, PJ_COL_REC_START);
  /* Which record of the tile this thread takes. In a stream of several models the records are first grouped by
     (a guess at) their model, so that the lanes of a warp mostly run the same model's code; everything that depends
     on the order of the records (the scan of the counts) goes through shared memory in record order. */
  uint32_t rid = tid;
  if constexpr (SCHEMA == PJ_SCHEMA_MIXED) {
    uint32_t cls = 4; /* threads without a record go last */
    if (tid < nrec) {
      const uint64_t st = rec_start[r0 + tid] - a.goff;
      cls = guess_model(a.in + st, a.limit - st);
    }
    uint32_t before = 0, rank = 0;
#pragma unroll
    for (uint32_t c = 0; c < 5; ++c) {
      const uint32_t b = __ballot_sync(0xFFFFFFFFu, cls == c);
      if (lane == 0) sh_cls[c][warp] = __popc(b);
      if (cls == c) rank = __popc(b & ((1u << lane) - 1u));
    }
    __syncthreads();
#pragma unroll
    for (uint32_t c = 0; c < 5; ++c) {
#pragma unroll
      for (uint32_t q = 0; q < NWARPS; ++q) {
        const uint32_t n_cq = sh_cls[c][q];
        if (c < cls || (c == cls && q < warp)) before += n_cq;
      }
    }
    sh_perm[before + rank] = tid;
    __syncthreads();
    rid = sh_perm[tid];
  }
  const bool active = rid < nrec;
  const uint64_t i = r0 + rid;
  const uint64_t start = active ? rec_start[i] - a.goff : 0;
  const uint64_t my_limit = (active && a.rec_end) ? a.rec_end[i] : a.limit;

  const long long c0 = clock64();
  /* ---- stage the tile's bytes ------------------------------------------------------------------ */
  /* As much of the tile's span as the window holds; a record is read from the window when all of its bytes
     are in it (for the last record of the input that means: the window reaches the end of the input). */
  int64_t w0 = 0;
  uint64_t win_hi = 0; /* input offset of the first byte that is not staged */
  int stage_failed = 0;
  if (nrec) {
    const uint64_t span_lo = rec_start[r0] - a.goff;
    uint64_t span_hi;
    if (a.rec_end) span_hi = a.rec_end[r0 + nrec - 1];
    else span_hi = r0 + nrec < N ? rec_start[r0 + nrec] - a.goff : a.limit;
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(a.in + span_lo) & 15u);
    w0 = (int64_t)span_lo - mis;
    const uint64_t need_hi = a.limit < span_hi + 32 ? a.limit : span_hi + 32;
    const uint64_t cap_hi = (uint64_t)(w0 + (int64_t)a.win_bytes - 64);
    win_hi = need_hi < cap_hi ? need_hi : cap_hi;
    const uint32_t nbytes = (uint32_t)((int64_t)win_hi - w0);
    /* One bulk copy (cp.async.bulk, the untiled TMA form) brings the whole 16-byte multiples; the threads add the
       last odd bytes and the line-feed padding, which lie behind the bulk region, and then wait for the copy. */
    const uint32_t nb16 = nbytes & ~15u;
    if (tid == 0 && nb16) { mbar_expect_tx(&sh_mbar, nb16); bulk_g2s(win, a.in + w0, nb16, &sh_mbar); }
    if (tid < nbytes - nb16) win[nb16 + tid] = a.in[w0 + (int64_t)(nb16 + tid)];
    if (tid < 32) win[nbytes + tid] = '\n';
    stage_failed = nb16 && !mbar_wait_bounded(&sh_mbar, 0, a.spin_limit_ns);
  }
  if (__syncthreads_or(stage_failed)) { /* the whole block leaves together */
    if (tid == 0) atomicExch(&a.res->timeout, 1u);
    return;
  }
  uint64_t my_end = !active ? 0 : (a.rec_end ? a.rec_end[i] : (i + 1 < N ? rec_start[i + 1] - a.goff : a.limit));
  if (active && !a.rec_end && i + 1 == N && my_end > win_hi && start < win_hi) {
    /* the last record of a shard with slack: it ends at its LF, which may well be staged */
    for (uint32_t q = (uint32_t)((int64_t)start - w0), qe = (uint32_t)((int64_t)win_hi - w0); q < qe; ++q)
      if (win[q] == '\n') { my_end = (uint64_t)(w0 + (int64_t)q) + 1; break; }
  }
  const bool fits = active && my_end <= win_hi;

  const long long c1 = clock64();
  /* ---- tokenise every record once ------------------------------------------------------------------ */
  /* A record that is not (wholly) in the window is read where it lies: the same word-at-a-time code, on global
     memory through L1. It looks up to 16 bytes ahead, so the last bytes of the input are left to the generic parser. */
  const bool direct = active && !fits && my_end + 32 <= a.limit;
  Win w;
  w.s = win; w.w0 = w0;
  Win wd = w; /* the view of a record read where it lies */
  if (direct) {
    const uint32_t mis4 = (uint32_t)(reinterpret_cast<uintptr_t>(a.in + start) & 3u);
    wd.s = a.in + start - mis4; wd.w0 = (int64_t)start - mis4;
  }
  uint32_t start32 = 0, lim32 = 0;
  Tape tp;
  tp.e = tape + tid; tp.stride = TILE_THREADS; tp.cap = a.tape_cap; tp.n = 0;
  uint32_t cnt[NSLOT], base[NSLOT];
#pragma unroll
  for (uint32_t k = 0; k < NSLOT; ++k) { cnt[k] = 0; base[k] = 0; }
  FVals v, cv;
  uint32_t type = PJ_TYPE_NONE, err = 0, fast = 0, verdict = FAST_REFUSED;
  if (active) {
    const bool blank = a.rec_blank && a.rec_blank[i];
    if ((fits || direct) && !blank) {
      const uint64_t rel = (uint64_t)((int64_t)my_limit - wd.w0);
      lim32 = rel > 0xFFFFFFF0ull ? 0xFFFFFFF0u : (uint32_t)rel;
      start32 = (uint32_t)((int64_t)start - wd.w0);
      uint32_t fpos = 0;
      if (!direct) verdict = fast_record<SCHEMA>(w, start32, lim32, a.lf_ws, a.open_end, &type, v, cv, cnt, tp, &err, &fpos);
      else {
        /* out of line, and without a tape: what it accepts is tokenised again when it is emitted */
        uint32_t cnt_d[NSLOT], type_d = PJ_TYPE_NONE, err_d = 0;
        verdict = fast_outline<SCHEMA>(wd, start32, lim32, a.lf_ws, a.open_end, nullptr, nullptr, i, tp, cnt_d, &type_d, &err_d, &fpos);
        type = type_d; err = err_d;
#pragma unroll
        for (uint32_t k = 0; k < NSLOT; ++k) cnt[k] = cnt_d[k];
      }
      fast = verdict == FAST_ACCEPTED;
      if (verdict == FAST_FAILED && opt_decides(a.opts, err)) { verdict = FAST_REFUSED; err = 0; } /* the exact parser knows the options */
      if (verdict == FAST_FAILED) {
        /* a validation failure found by the word-at-a-time path: no row values, no bytes anywhere */
        type = PJ_TYPE_NONE;
#pragma unroll
        for (uint32_t k = 0; k < NSLOT; ++k) cnt[k] = 0;
        colp<uint32_t>(&a.cols, PJ_COL_ERR_OFF)[i] = fpos - start32;
      }
    }
    if (verdict == FAST_REFUSED) {
      Rd r;
      r.in = fits ? win - w0 : a.in; r.lf_ws = a.lf_ws; r.open_end = a.open_end; r.limit = my_limit; r.opts = a.opts;
      PS s;
      s.p = start; s.err = 0; s.err_pos = 0;
      Out<false> so;
      so.cols = &a.cols;
      if (blank) { fail(s, PJ_E_SYNTAX, my_limit); type = PJ_TYPE_NONE; }
      else type = parse_record<false>(c_schema, r, s, a.schema, so, i);
      err = s.err;
#pragma unroll
      for (uint32_t k = 0; k < NSLOT; ++k) cnt[k] = (k >= LO && k < HI && !err) ? so.cnt[k] : 0u;
      if (err) type = PJ_TYPE_NONE;
      colp<uint32_t>(&a.cols, PJ_COL_ERR_OFF)[i] = err ? (uint32_t)(s.err_pos - start) : 0u;
    } else if (fast) colp<uint32_t>(&a.cols, PJ_COL_ERR_OFF)[i] = 0u;
    colp<uint8_t>(&a.cols, PJ_COL_ERR_KIND)[i] = (uint8_t)err;
    if (SCHEMA == PJ_SCHEMA_MIXED) colp<uint8_t>(&a.cols, PJ_COL_REC_TYPE)[i] = (uint8_t)type;
  }
  {
    uint32_t packed = (err ? 1u : 0u) | (fast << 16);
    for (int d = 16; d; d >>= 1) packed += __shfl_down_sync(0xFFFFFFFFu, packed, d);
    if (lane == 0 && (packed & 0xFFFF)) atomicAdd(&a.res->n_errors, (unsigned long long)(packed & 0xFFFF));
    if (lane == 0 && (packed >> 16)) atomicAdd(&a.res->n_fast, (unsigned long long)(packed >> 16));
  }

  /* ---- positions: scan inside the tile (two barriers for all counters), then look back ------------- */
  if (tid < NSLOT) sh_tot[tid] = 0;
  if constexpr (SORTED) {
#pragma unroll
    for (uint32_t k = LO; k < HI; ++k) sh_x[k * TILE_THREADS + rid] = cnt[k];
    __syncthreads();
  }
#pragma unroll
  for (uint32_t k = LO; k < HI; ++k) {
    const uint32_t mine_k = SORTED ? sh_x[k * TILE_THREADS + tid] : cnt[k]; /* the count of record number tid */
    const uint32_t inc = warp_incl_scan(mine_k);
    if (lane == 31) sh_warp[k][warp] = inc;
    base[k] = inc - mine_k;
  }
  __syncthreads();
  const long long c2 = clock64();
#pragma unroll
  for (uint32_t k = LO; k < HI; ++k) {
#pragma unroll
    for (uint32_t q = 0; q < NWARPS; ++q) if (q < warp) base[k] += sh_warp[k][q];
    if constexpr (SORTED) sh_x[k * TILE_THREADS + tid] = base[k]; /* record tid's place in the tile; read back by its owner below */
  }
  if (warp == 0) {
    TileState* me = &a.tiles[tile];
    uint32_t mine = 0;
    if (lane >= LO && lane < HI) {
#pragma unroll
      for (uint32_t q = 0; q < NWARPS; ++q) mine += sh_warp[lane][q];
    }
    if (lane < NSLOT) {
      sh_tot[lane] = mine;
      st_relaxed_u64(&me->agg[lane], TS_VALID | mine);
      if (tile == 0) st_relaxed_u64(&me->inc[lane], TS_VALID | mine);
    }
    uint32_t excl_all[NSLOT];
    const bool ok = tile_lookback<LO, HI>(a, tile, lane, excl_all);
    uint32_t excl = 0;
#pragma unroll
    for (uint32_t k = LO; k < HI; ++k) if (lane == k) excl = excl_all[k];
    if (tile != 0 && ok && lane < NSLOT) st_relaxed_u64(&me->inc[lane], TS_VALID | (unsigned long long)(excl + mine));
    const uint64_t before = lane < NSLOT ? (uint64_t)a.slot_base[lane] + excl : 0; /* the tile's start, over the whole call */
    if (lane < NSLOT) sh_base[lane] = (uint32_t)before;
    /* does the whole tile fit the caller's buffers? (totals only grow, so the last tile's verdict is the call's) */
    const bool over = lane < NSLOT && before + mine > a.slot_cap[lane];
    const uint32_t any_over = __ballot_sync(0xFFFFFFFFu, over);
    if (lane == 0) {
      sh_ok = ok && !any_over;
      if (any_over) a.res->ok = 0;
    }
    if (tile == a.ntiles - 1 && lane < NSLOT) a.res->total[lane] = before + mine;
  }
  __syncthreads();
  const long long c3 = clock64();
  if (!sh_ok) return;

  /* ---- emit ---------------------------------------------------------------------------------------- */
  if (active) {
#pragma unroll
    for (uint32_t k = LO; k < HI; ++k) base[k] = (SORTED ? sh_x[k * TILE_THREADS + rid] : base[k]) + sh_base[k];
    if (SCHEMA == PJ_SCHEMA_MIXED) {
      const uint32_t row = type == PJ_TYPE_PET ? base[SLOT_ROWS_PET] : (type == PJ_TYPE_ORDER ? base[SLOT_ROWS_ORD] : base[SLOT_ROWS_USR]);
      colp<uint32_t>(&a.cols, PJ_COL_REC_ROW)[i] = type == PJ_TYPE_NONE ? 0xFFFFFFFFu : row;
    }
    if (fast) {
      if (!direct && tp.n <= tp.cap) fast_emit<SCHEMA>(w, &a.cols, type, v, cv, tp, base, i);
      else {
        /* an out-of-line call: it gets a copy of the bases, so that base[] itself can stay in registers */
        uint32_t base_copy[NSLOT], t_d, e_d, p_d;
#pragma unroll
        for (uint32_t k = 0; k < NSLOT; ++k) base_copy[k] = base[k];
        fast_outline<SCHEMA>(direct ? wd : w, start32, lim32, a.lf_ws, a.open_end, &a.cols, base_copy, i, tp, nullptr, &t_d, &e_d, &p_d);
      }
    } else {
      Out<true> o;
      o.cols = &a.cols;
#pragma unroll
      for (uint32_t k = 0; k < NSLOT; ++k) { o.base[k] = base[k]; o.room[k] = cnt[k]; }
      if (err) {
        if (SCHEMA != PJ_SCHEMA_MIXED) store_absent<true>(c_schema, a.schema, o, i);
      } else {
        Rd r;
        r.in = fits ? win - w0 : a.in; r.lf_ws = a.lf_ws; r.open_end = a.open_end; r.limit = my_limit; r.opts = a.opts;
        PS s;
        s.p = start; s.err = 0; s.err_pos = 0;
        parse_record<true>(c_schema, r, s, a.schema, o, i);
      }
    }
  }
  __syncthreads();
  if (tid == 0) {
    const long long c4 = clock64();
    atomicAdd(&a.res->phase_cycles[0], (unsigned long long)(c1 - c0));
    atomicAdd(&a.res->phase_cycles[1], (unsigned long long)(c2 - c1));
    atomicAdd(&a.res->phase_cycles[2], (unsigned long long)(c3 - c2));
    atomicAdd(&a.res->phase_cycles[3], (unsigned long long)(c4 - c3));
  }
  /* the last tile closes the offset columns */
  if (tile == a.ntiles - 1 && tid < a.plan.n) {
    const FinalizeItem it = a.plan.item[tid];
    if (it.sentinel_slot != 0xFF) {
      const uint64_t rows = it.rows_slot == 0xFF ? N : (uint64_t)sh_base[it.rows_slot] + sh_tot[it.rows_slot];
      colp<uint32_t>(&a.cols, it.col)[rows] = sh_base[it.sentinel_slot] + sh_tot[it.sentinel_slot];
    }
  }
}

/* ================================================================================================
 * Single-pass tile writer (columns -> JSON text)
 *
 * One block takes TILE_THREADS consecutive records. Every thread measures its record (size pass of
 * pj_write_fast.cuh), the lengths are scanned inside the block, the tile's start in the output comes
 * from a decoupled look-back over the tiles before it (one 64-bit running total; the protocol of the
 * parse kernel), every thread then writes its record into a window in shared memory, and the block
 * copies the window to the output with 16-byte stores. A tile whose text does not fit the window is
 * written to global memory directly. Text is produced once and written to HBM once.
 * ================================================================================================ */
#ifndef PJ_WT_THREADS
#define PJ_WT_THREADS 128 /* records (= threads) per writer tile */
#endif
#ifndef PJ_WT_WIN_KB
#define PJ_WT_WIN_KB 40 /* text window per tile in shared memory */
#endif
#ifndef PJ_WT_BLOCKS
#define PJ_WT_BLOCKS 5 /* resident blocks per SM the kernel is compiled for */
#endif
static constexpr uint32_t WT_THREADS = PJ_WT_THREADS;
static_assert(WT_THREADS % 32 == 0 && WT_THREADS >= 96, "the copy-out of the window's odd ends uses threads 32.. and 64..");
static constexpr uint32_t WTILE_WIN_BYTES = PJ_WT_WIN_KB * 1024;
static constexpr uint32_t WTILE_SMEM_BYTES = WTILE_WIN_BYTES + 32;

struct WTileArgs {
  WriteArgs w;
  unsigned long long* agg; /* [ntiles] text bytes of the tile | TS_VALID */
  unsigned long long* inc; /* [ntiles] text bytes of all tiles up to and including it | TS_VALID */
  uint32_t* ticket;
  uint32_t ntiles;
  unsigned long long spin_limit_ns;
};

/* Exclusive prefix of `tile` over all earlier tiles. Warp 0 only, all lanes; false when the bounded wait ran out. */
__device__ __forceinline__ bool lookback_u64(const unsigned long long* agg, const unsigned long long* inc, uint32_t* timeout_flag, unsigned long long limit_ns,
                                             uint32_t tile, uint32_t lane, unsigned long long* excl_out) {
  unsigned long long excl = 0;
  int64_t j = (int64_t)tile - 1;
  const unsigned long long t0 = global_ns();
  while (j >= 0) {
    const int64_t mine = j - lane;
    unsigned long long wa, wi;
    uint32_t first_inc;
    for (;;) {
      wa = TS_VALID; wi = TS_VALID; /* tiles before the first: inclusive total 0 */
      if (mine >= 0) { wi = ld_relaxed_u64(&inc[mine]); wa = ld_relaxed_u64(&agg[mine]); }
      const bool has_inc = wi & TS_VALID, has_agg = wa & TS_VALID;
      const uint32_t inc_mask = __ballot_sync(0xFFFFFFFFu, has_inc);
      const uint32_t ready_mask = __ballot_sync(0xFFFFFFFFu, has_inc || has_agg);
      first_inc = inc_mask ? (uint32_t)(__ffs((int)inc_mask) - 1) : 32u;
      const uint32_t need = first_inc >= 31 ? 0xFFFFFFFFu : ((2u << first_inc) - 1u);
      if ((ready_mask & need) == need) break;
      uint32_t give_up = 0;
      if (lane == 0) give_up = (global_ns() - t0 > limit_ns) || *(volatile uint32_t*)timeout_flag;
      give_up = __shfl_sync(0xFFFFFFFFu, give_up, 0);
      if (give_up) { if (lane == 0) atomicExch(timeout_flag, 1u); return false; }
      __nanosleep(100);
    }
    unsigned long long c = lane < first_inc ? (wa & ~TS_VALID) : (lane == first_inc ? (wi & ~TS_VALID) : 0ull);
#pragma unroll
    for (int d = 16; d; d >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, d);
    excl += c;
    if (first_inc < 32) break;
    j -= 32;
  }
  *excl_out = excl;
  return true;
}

/* Does any byte of the string arenas need a JSON escape (below 0x20, '"', '\\')? Text is mostly free of
 * them, and knowing so lets the tile writer take string lengths from the offset columns alone. */
struct ArenaArgs {
  const uint8_t* p[12];
  uint64_t n[12];
  uint32_t count;
  DevResult* res;
};
__device__ __forceinline__ uint32_t word_needs_escape(uint32_t x) {
  const uint32_t xq = x ^ 0x22222222u, xb = x ^ 0x5C5C5C5Cu;
  return (((x - 0x20202020u) & ~x) | ((xq - 0x01010101u) & ~xq) | ((xb - 0x01010101u) & ~xb)) & 0x80808080u;
}
static __global__ void __launch_bounds__(256) k_arena_flags(const __grid_constant__ ArenaArgs a) {
  const uint64_t gtid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x, gsize = (uint64_t)gridDim.x * blockDim.x;
  uint32_t any = 0;
  for (uint32_t r = 0; r < a.count; ++r) {
    const uint8_t* p = a.p[r];
    const uint64_t n = a.n[r];
    uint64_t head = (16 - (reinterpret_cast<uintptr_t>(p) & 15u)) & 15u;
    if (head > n) head = n;
    const uint64_t nvec = (n - head) >> 4, tail = head + (nvec << 4);
    const uint4* v = reinterpret_cast<const uint4*>(p + head);
    for (uint64_t k = gtid; k < nvec; k += gsize) {
      const uint4 x = __ldg(v + k);
      any |= word_needs_escape(x.x) | word_needs_escape(x.y) | word_needs_escape(x.z) | word_needs_escape(x.w);
    }
    if (gtid < head) any |= escape_extra_byte(p[gtid]);
    if (gtid < n - tail) any |= escape_extra_byte(p[tail + gtid]);
  }
  if (__syncthreads_or((int)any) && threadIdx.x == 0) a.res->needs_escape = 1u;
}

/* The writer is bound by the latency of its column loads (one dependent chain per property). Asking for all the
 * row-indexed values of a record at once, before the first is needed, lets those latencies overlap. */
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
template <int OBJ, int I = 0>
__device__ __forceinline__ void prefetch_row(const DevCols* c, uint64_t row) {
  if constexpr (I == 0) prefetch_l1(colp<uint8_t>(c, CObj<OBJ>::present_col) + row);
  if constexpr (I < CObj<OBJ>::N) {
    constexpr uint32_t kind = FK<OBJ, I>::kind, col = FK<OBJ, I>::col;
    if constexpr (kind == K_I64) prefetch_l1(colp<int64_t>(c, col) + row);
    else if constexpr (kind == K_I32) prefetch_l1(colp<int32_t>(c, col) + row);
    else if constexpr (kind == K_BOOL || kind == K_ENUM) prefetch_l1(colp<uint8_t>(c, col) + row);
    else if constexpr (kind == K_DATETIME) { prefetch_l1(colp<int64_t>(c, col) + row); prefetch_l1(colp<int32_t>(c, col + 1) + row); prefetch_l1(colp<int32_t>(c, col + 2) + row); }
    else if constexpr (kind == K_STR || kind == K_LIST_STR || kind == K_LIST_OBJ) prefetch_l1(colp<uint32_t>(c, col) + row + 1);
    else if constexpr (kind == K_OBJ) prefetch_row<FK<OBJ, I>::child>(c, row);
    prefetch_row<OBJ, I + 1>(c, row);
  }
}

static __global__ void __launch_bounds__(WT_THREADS, PJ_WT_BLOCKS) k_write_tile(const __grid_constant__ WTileArgs a) {
  constexpr uint32_t NWARPS = WT_THREADS / 32;
  extern __shared__ __align__(16) uint8_t smem[];
  __shared__ uint32_t sh_warp[NWARPS];
  __shared__ uint32_t sh_tile, sh_ok;
  __shared__ unsigned long long sh_base;
  const uint32_t tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) sh_tile = atomicAdd(a.ticket, 1u);
  __syncthreads();
  const uint32_t tile = sh_tile;
  if (tile >= a.ntiles) return;
  const uint64_t i = (uint64_t)tile * WT_THREADS + tid;
  uint32_t type = PJ_TYPE_NONE;
  uint64_t row = 0;
  const bool plain = !a.w.res->needs_escape; /* no string of the columns holds a byte to escape */
  const long long c0 = clock64();
  const bool located = i < a.w.n && write_locate(a.w.schema, &a.w.cols, i, &type, &row);
  uint32_t len = 0;
  if (located) {
    if (type == PJ_TYPE_PET) prefetch_row<OBJ_PET>(&a.w.cols, row);
    else if (type == PJ_TYPE_ORDER) prefetch_row<OBJ_ORDER>(&a.w.cols, row);
    else prefetch_row<OBJ_USER>(&a.w.cols, row);
    WOut w; w.dst = nullptr; w.n = 0; w.hexa = a.w.hexa;
    if (plain) fwrite_record<false, true>(&a.w.cols, type, row, a.w.inclusion, w); else fwrite_record<false, false>(&a.w.cols, type, row, a.w.inclusion, w);
    len = (uint32_t)w.n + 1; /* LF, or the comma / closing bracket that follows the record */
  }
  const uint32_t incl = warp_incl_scan(len);
  if (lane == 31) sh_warp[warp] = incl;
  uint32_t loc = incl - len;
  __syncthreads();
  const long long c1 = clock64();
  uint32_t tile_total = 0;
#pragma unroll
  for (uint32_t q = 0; q < NWARPS; ++q) { if (q < warp) loc += sh_warp[q]; tile_total += sh_warp[q]; }
  const uint64_t lead = a.w.array ? 1 : 0; /* the opening bracket */
  if (warp == 0) {
    if (lane == 0) {
      st_relaxed_u64(&a.agg[tile], TS_VALID | tile_total);
      if (tile == 0) st_relaxed_u64(&a.inc[tile], TS_VALID | tile_total);
    }
    unsigned long long excl = 0;
    const bool ok = lookback_u64(a.agg, a.inc, &a.w.res->timeout, a.spin_limit_ns, tile, lane, &excl);
    if (lane == 0) {
      if (tile != 0 && ok) st_relaxed_u64(&a.inc[tile], TS_VALID | (excl + tile_total));
      const bool room = lead + excl + tile_total <= a.w.cap;
      if (ok && !room) a.w.res->ok = 0;
      if (tile == a.ntiles - 1) a.w.res->out_bytes = excl + tile_total; /* text bytes of all records */
      sh_base = excl;
      sh_ok = ok && room;
    }
  }
  __syncthreads();
  const long long c2 = clock64();
  long long c3 = c2;
  if (!sh_ok) return;
  uint8_t* dst0 = a.w.out + lead + sh_base; /* where the tile's text starts */
  const uint8_t sep = a.w.array ? (uint8_t)',' : (uint8_t)'\n';
  if (tile_total + 16 <= WTILE_WIN_BYTES) {
    /* the window mirrors the output's alignment: window byte k goes to (dst0 - pad)[k] */
    const uint32_t pad = (uint32_t)(reinterpret_cast<uintptr_t>(dst0) & 15u);
    if (located) {
      WOut w; w.dst = smem + pad + loc; w.n = 0; w.hexa = a.w.hexa;
      if (plain) fwrite_record<true, true>(&a.w.cols, type, row, a.w.inclusion, w); else fwrite_record<true, false>(&a.w.cols, type, row, a.w.inclusion, w);
      smem[pad + loc + w.n] = sep;
    }
    fence_async_smem();
    __syncthreads();
    c3 = clock64();
    /* the 16-byte multiples in the middle leave with one bulk copy (cp.async.bulk shared -> global), the odd
       bytes at both ends with plain stores */
    uint8_t* gbase = dst0 - pad;
    const uint32_t end = pad + tile_total;
    const uint32_t lo16 = (pad + 15u) & ~15u, hi16 = end & ~15u;
    if (hi16 > lo16) {
      if (tid == 0) { bulk_s2g(gbase + lo16, smem + lo16, hi16 - lo16); bulk_s2g_wait_read(); }
      if (tid >= 32 && tid < 32 + (lo16 - pad)) gbase[pad + tid - 32] = smem[pad + tid - 32];
      if (tid >= 64 && tid < 64 + (end - hi16)) gbase[hi16 + tid - 64] = smem[hi16 + tid - 64];
    } else {
      for (uint32_t b = pad + tid; b < end; b += WT_THREADS) gbase[b] = smem[b];
    }
  } else if (located) {
    WOut w; w.dst = dst0 + loc; w.n = 0; w.hexa = a.w.hexa;
    if (plain) fwrite_record<true, true>(&a.w.cols, type, row, a.w.inclusion, w); else fwrite_record<true, false>(&a.w.cols, type, row, a.w.inclusion, w);
    dst0[loc + w.n] = sep;
  }
  __syncthreads();
  if (tid == 0) { /* cycles per phase: size pass, look-back, text into the window, copy-out */
    const long long c4 = clock64();
    atomicAdd(&a.w.res->phase_cycles[0], (unsigned long long)(c1 - c0));
    atomicAdd(&a.w.res->phase_cycles[1], (unsigned long long)(c2 - c1));
    atomicAdd(&a.w.res->phase_cycles[2], (unsigned long long)(c3 - c2));
    atomicAdd(&a.w.res->phase_cycles[3], (unsigned long long)(c4 - c3));
  }
}
/* closes the text: brackets of array framing, the total, the verdict */
static __global__ void k_write_close(const __grid_constant__ WriteArgs a) {
  if (threadIdx.x || blockIdx.x) return;
  const uint64_t body = a.res->out_bytes;
  const uint64_t total = a.array ? (body ? body + 1 : 2) : body;
  a.res->out_bytes = total;
  const bool ok = a.res->ok && total <= a.cap;
  a.res->ok = ok;
  if (a.array && ok) { a.out[0] = '['; a.out[total - 1] = ']'; }
}

/* ---- column checksums --------------------------------------------------------------------------------- */
PJ_HD uint64_t checksum_mix(uint64_t x) {
  x ^= x >> 30; x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27; x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}
PJ_HD uint64_t checksum_term(uint64_t word, uint64_t j) { return checksum_mix(word + 0x9E3779B97F4A7C15ull * (j + 1)); }
struct ChecksumArgs {
  const uint8_t* p[PJ_MAX_COLS];
  uint64_t n[PJ_MAX_COLS]; /* bytes */
  unsigned long long* out; /* [PJ_MAX_COLS], zeroed */
};
/* blockIdx.y = column; the blocks of a column stride over its 8-byte words */
static __global__ void __launch_bounds__(256) k_checksum(const __grid_constant__ ChecksumArgs a) {
  const uint32_t col = blockIdx.y;
  const uint8_t* p = a.p[col];
  const uint64_t n = a.n[col];
  const uint64_t nwords = (n + 7) / 8;
  const bool aligned = (reinterpret_cast<uintptr_t>(p) & 7u) == 0;
  unsigned long long s = 0;
  for (uint64_t j = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; j < nwords; j += (uint64_t)gridDim.x * blockDim.x) {
    uint64_t w = 0;
    if (aligned && 8 * j + 8 <= n) w = *reinterpret_cast<const uint64_t*>(p + 8 * j);
    else for (uint32_t b = 0; b < 8 && 8 * j + b < n; ++b) w |= (uint64_t)p[8 * j + b] << (8 * b);
    s += checksum_term(w, j);
  }
  for (int d = 16; d; d >>= 1) s += __shfl_xor_sync(0xFFFFFFFFu, s, d);
  if ((threadIdx.x & 31) == 0 && s) atomicAdd(&a.out[col], s);
}

}  // namespace pj
#endif
