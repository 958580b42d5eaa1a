/*
 * pj_api.cu — the C ABI of libpetjson.so (declared in include/petjson.h): argument checking,
 * staging of host buffers, scratch management and the launch sequence of the kernels.
 *
 * There is deliberately no CPU path: without a CUDA device pj_create fails with PJ_ERR_CUDA.
 */
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <thread>
#include <vector>
#include <dlfcn.h>
#include <new>

#include "petjson.h"
#include "pj_kernels.cuh"
#include "pj_array_kernels.cuh"
#include "pj_stream_kernel.cuh"

using namespace pj;

/* the four instantiations of the tile kernel live in objects of their own (pj_tile_inst.cu) */
namespace pj {
cudaError_t tile_init_1(const Schema*); cudaError_t tile_launch_1(const TileArgs*, unsigned, cudaStream_t);
cudaError_t tile_init_2(const Schema*); cudaError_t tile_launch_2(const TileArgs*, unsigned, cudaStream_t);
cudaError_t tile_init_3(const Schema*); cudaError_t tile_launch_3(const TileArgs*, unsigned, cudaStream_t);
cudaError_t tile_init_4(const Schema*); cudaError_t tile_launch_4(const TileArgs*, unsigned, cudaStream_t);
cudaError_t stream_launch_1(const StreamArgs*, unsigned, cudaStream_t); cudaError_t stream_launch_2(const StreamArgs*, unsigned, cudaStream_t);
cudaError_t stream_launch_3(const StreamArgs*, unsigned, cudaStream_t); cudaError_t stream_launch_4(const StreamArgs*, unsigned, cudaStream_t);
}

namespace {

thread_local char g_create_error[256] = "";

struct ColInfo { const char* name; uint8_t elem, owner; };
/* name, element width, owning model (PJ_TYPE_*, 0 = per record) of every column id */
const ColInfo* col_info(int col) {
  static ColInfo t[PJ_MAX_COLS];
  static bool init = false;
  if (!init) {
    auto set = [&](int id, const char* n, int e, int o) { t[id].name = n; t[id].elem = (uint8_t)e; t[id].owner = (uint8_t)o; };
    set(PJ_COL_REC_START, "rec_start", 8, 0); set(PJ_COL_ERR_KIND, "err_kind", 1, 0); set(PJ_COL_ERR_OFF, "err_off", 4, 0);
    set(PJ_COL_REC_TYPE, "rec_type", 1, 0); set(PJ_COL_REC_ROW, "rec_row", 4, 0);
    set(PJ_COL_PET_PRESENT, "pet_present", 1, 1); set(PJ_COL_PET_ID, "pet_id", 8, 1);
    set(PJ_COL_PET_CAT_PRESENT, "pet_cat_present", 1, 1); set(PJ_COL_PET_CAT_ID, "pet_cat_id", 8, 1);
    set(PJ_COL_PET_CAT_NAME_OFF, "pet_cat_name_off", 4, 1); set(PJ_COL_PET_CAT_NAME_DATA, "pet_cat_name_data", 1, 1);
    set(PJ_COL_PET_NAME_OFF, "pet_name_off", 4, 1); set(PJ_COL_PET_NAME_DATA, "pet_name_data", 1, 1);
    set(PJ_COL_PET_PHOTO_OFF, "pet_photo_off", 4, 1); set(PJ_COL_PET_PHOTO_STR_OFF, "pet_photo_str_off", 4, 1);
    set(PJ_COL_PET_PHOTO_DATA, "pet_photo_data", 1, 1); set(PJ_COL_PET_TAGS_OFF, "pet_tags_off", 4, 1);
    set(PJ_COL_PET_TAG_PRESENT, "pet_tag_present", 1, 1); set(PJ_COL_PET_TAG_ID, "pet_tag_id", 8, 1);
    set(PJ_COL_PET_TAG_NAME_OFF, "pet_tag_name_off", 4, 1); set(PJ_COL_PET_TAG_NAME_DATA, "pet_tag_name_data", 1, 1);
    set(PJ_COL_PET_STATUS, "pet_status", 1, 1);
    set(PJ_COL_ORD_PRESENT, "ord_present", 1, 2); set(PJ_COL_ORD_ID, "ord_id", 8, 2); set(PJ_COL_ORD_PET_ID, "ord_pet_id", 8, 2);
    set(PJ_COL_ORD_QUANTITY, "ord_quantity", 4, 2); set(PJ_COL_ORD_SHIP_EPOCH, "ord_ship_epoch", 8, 2);
    set(PJ_COL_ORD_SHIP_NANOS, "ord_ship_nanos", 4, 2); set(PJ_COL_ORD_SHIP_OFFSET, "ord_ship_offset", 4, 2);
    set(PJ_COL_ORD_STATUS, "ord_status", 1, 2); set(PJ_COL_ORD_COMPLETE, "ord_complete", 1, 2);
    set(PJ_COL_USR_PRESENT, "usr_present", 1, 3); set(PJ_COL_USR_ID, "usr_id", 8, 3);
    set(PJ_COL_USR_USERNAME_OFF, "usr_username_off", 4, 3); set(PJ_COL_USR_USERNAME_DATA, "usr_username_data", 1, 3);
    set(PJ_COL_USR_FIRSTNAME_OFF, "usr_firstname_off", 4, 3); set(PJ_COL_USR_FIRSTNAME_DATA, "usr_firstname_data", 1, 3);
    set(PJ_COL_USR_LASTNAME_OFF, "usr_lastname_off", 4, 3); set(PJ_COL_USR_LASTNAME_DATA, "usr_lastname_data", 1, 3);
    set(PJ_COL_USR_EMAIL_OFF, "usr_email_off", 4, 3); set(PJ_COL_USR_EMAIL_DATA, "usr_email_data", 1, 3);
    set(PJ_COL_USR_PASSWORD_OFF, "usr_password_off", 4, 3); set(PJ_COL_USR_PASSWORD_DATA, "usr_password_data", 1, 3);
    set(PJ_COL_USR_PHONE_OFF, "usr_phone_off", 4, 3); set(PJ_COL_USR_PHONE_DATA, "usr_phone_data", 1, 3);
    set(PJ_COL_USR_STATUS, "usr_status", 4, 3);
    init = true;
  }
  if (col < 0 || col >= PJ_MAX_COLS || !t[col].name) return nullptr;
  return &t[col];
}

struct DeviceGuard {
  int prev = -1;
  bool changed = false;
  explicit DeviceGuard(int dev) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != dev) changed = cudaSetDevice(dev) == cudaSuccess;
  }
  ~DeviceGuard() { if (changed) cudaSetDevice(prev); }
};

struct Buffer {
  void* p = nullptr;
  size_t cap = 0;
};

}  // namespace

enum { PJ_CTX_RESULTS = 16 };
struct pj_ctx {
  int device = 0;
  int inclusion = PJ_INCLUDE_NON_EMPTY;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  Buffer scratch;  /* tile counts, counter matrix, scan partials, writer offsets */
  Buffer in_stage; /* device copy of a host input */
  Buffer col_stage; /* device copies of host columns */
  Buffer out_stage; /* device copy of a host output (writer) */
  Buffer tiles;     /* look-back state of the tile kernel + its ticket */
  DevResult* d_res = nullptr; /* [PJ_CTX_RESULTS]: one per piece of a call; [0] serves every other call */
  DevResult* h_res = nullptr; /* pinned, same shape */
  cudaEvent_t ev[10] = {};
  cudaEvent_t ev_k0[16] = {}, ev_k1[16] = {}; /* around the kernel of every piece */
  cudaEvent_t ev_done[16] = {};               /* the totals of a piece have reached the host */
  uint32_t tile_bytes_opt = 0;                /* pj_options.tile_bytes */
  unsigned long long spin_ns = 2000000000ull; /* bound of every device-side wait */
  double avg_rec_bytes[5] = {0, 0, 0, 0, 0};  /* bytes per record seen per schema (sizes the tiles of the next call) */
  /* host buffers parsed in pieces: copy streams and one "piece is on the device" event per piece */
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t ev_in[16] = {};
  uint32_t piece_bytes = 0;
  uint64_t dev_piece_bytes = 0; /* pj_options.device_piece_bytes */
  uint32_t opt_flags = 0;
  bool stall_once = false; /* PJ_OPT_TEST_STALL_ONCE, not yet used up */
  Schema schema;
  pj_call_stats stats = {};
  char err[256] = "";
};

namespace {

pj_status set_err(pj_ctx* c, pj_status st, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(c ? c->err : g_create_error, 256, fmt, ap);
  va_end(ap);
  return st;
}
#define PJ_CUDA(ctx, call)                                                                              \
  do {                                                                                                  \
    cudaError_t e__ = (call);                                                                           \
    if (e__ != cudaSuccess) return set_err(ctx, e__ == cudaErrorMemoryAllocation ? PJ_ERR_NOMEM : PJ_ERR_CUDA, \
                                           "%s: %s", #call, cudaGetErrorString(e__));                   \
  } while (0)

pj_status ensure(pj_ctx* c, Buffer* b, size_t bytes) {
  if (bytes <= b->cap) return PJ_OK;
  if (b->p) { PJ_CUDA(c, cudaStreamSynchronize(c->stream)); PJ_CUDA(c, cudaFree(b->p)); b->p = nullptr; b->cap = 0; }
  size_t want = bytes + bytes / 8 + 4096;
  cudaError_t e = cudaMalloc(&b->p, want);
  if (e != cudaSuccess) { want = bytes; e = cudaMalloc(&b->p, want); }
  if (e != cudaSuccess) { b->p = nullptr; (void)cudaGetLastError(); return set_err(c, PJ_ERR_NOMEM, "cudaMalloc(%zu): %s", want, cudaGetErrorString(e)); }
  b->cap = want;
  return PJ_OK;
}
inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

/* per-record columns a parse of `schema` fills */
int record_cols(uint32_t schema, int* out) {
  int n = 0;
  out[n++] = PJ_COL_REC_START; out[n++] = PJ_COL_ERR_KIND; out[n++] = PJ_COL_ERR_OFF;
  if (schema == PJ_SCHEMA_MIXED) { out[n++] = PJ_COL_REC_TYPE; out[n++] = PJ_COL_REC_ROW; }
  return n;
}

struct Stage {
  pj_ctx* c;
  int k = 0;
  explicit Stage(pj_ctx* ctx) : c(ctx) { cudaEventRecord(c->ev[0], c->stream); }
  /* closes stage k (its launches were counted by the caller) */
  void next() { ++k; cudaEventRecord(c->ev[k], c->stream); }
};
inline void count_launch(pj_ctx* c, int stage, uint32_t n = 1) { c->stats.kernel_launches += n; c->stats.stage_launches[stage] += n; }

/* adds the stage times of the launches just finished to the call's statistics (a call may run several passes) */
void collect_times(pj_ctx* c, int stages) {
  for (int i = 0; i < stages && i < 8; ++i) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, c->ev[i], c->ev[i + 1]) == cudaSuccess) c->stats.stage_ms[i] += ms;
  }
  float ms = 0.f;
  if (cudaEventElapsedTime(&ms, c->ev[0], c->ev[stages]) == cudaSuccess) c->stats.device_ms += ms;
}

enum { MAX_PIECES = 16 };
static constexpr uint64_t DEFAULT_PIECE_BYTES = 32ull << 20;
pj_status ensure_pipe_streams(pj_ctx* c) {
  if (c->s_in) return PJ_OK;
  PJ_CUDA(c, cudaStreamCreateWithFlags(&c->s_in, cudaStreamNonBlocking));
  PJ_CUDA(c, cudaStreamCreateWithFlags(&c->s_out, cudaStreamNonBlocking));
  for (auto& ev : c->ev_in) PJ_CUDA(c, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  return PJ_OK;
}

int persistent_grid(pj_ctx* c, uint64_t items, int threads) {
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, c->device);
  uint64_t want = (items + threads - 1) / threads;
  uint64_t cap = (uint64_t)sms * 16;
  if (want < 1) want = 1;
  return (int)(want < cap ? want : cap);
}

/* What a parse call needs to know about the caller's columns. */
struct ParsePlan {
  FinalizePlan plan;
  int rcols[5], nrc;          /* per-record columns */
  int need[PJ_MAX_COLS], nneed; /* every column the schema fills */
  uint64_t cap_elems[PJ_MAX_COLS];
  uint64_t rec_cap;           /* records that fit every per-record and row-indexed buffer */
  uint64_t slot_cap[NSLOT];   /* largest total of every counter the buffers can take */
  DevCols dcols;              /* device addresses of the columns (the caller's, or the staging copies) */
};

pj_status plan_columns(pj_ctx* c, uint32_t schema, pj_columns* out, uint64_t limit, bool array, ParsePlan* pp) {
  memset(pp, 0, sizeof *pp);
  build_finalize_plan(c->schema, schema, &pp->plan);
  pp->nrc = record_cols(schema, pp->rcols);
  for (int i = 0; i < pp->nrc; ++i) pp->need[pp->nneed++] = pp->rcols[i];
  for (uint32_t k = 0; k < pp->plan.n; ++k) pp->need[pp->nneed++] = pp->plan.item[k].col;
  for (int i = 0; i < pp->nneed; ++i)
    if (!out->col[pp->need[i]].ptr) return set_err(c, PJ_ERR_ARG, "pj_parse: column %s has no buffer", col_info(pp->need[i])->name);
  const bool host_out = out->mem_kind == PJ_MEM_HOST;
  if (host_out) {
    size_t tot = 0;
    for (int i = 0; i < pp->nneed; ++i) tot += align_up(out->col[pp->need[i]].bytes, 256);
    pj_status st = ensure(c, &c->col_stage, tot + 256);
    if (st) return st;
    size_t at = 0;
    for (int i = 0; i < pp->nneed; ++i) { pp->dcols.ptr[pp->need[i]] = (uint8_t*)c->col_stage.p + at; at += align_up(out->col[pp->need[i]].bytes, 256); }
  } else {
    for (int i = 0; i < pp->nneed; ++i) pp->dcols.ptr[pp->need[i]] = out->col[pp->need[i]].ptr;
  }
  for (int i = 0; i < pp->nneed; ++i) pp->cap_elems[pp->need[i]] = out->col[pp->need[i]].bytes / col_info(pp->need[i])->elem;
  /* records: every per-record column and every column with one row per record (less the closing entry of offsets) */
  uint64_t cap_all = ~0ull;
  for (int i = 0; i < pp->nrc; ++i) if (pp->cap_elems[pp->rcols[i]] < cap_all) cap_all = pp->cap_elems[pp->rcols[i]];
  for (uint32_t k = 0; k < NSLOT; ++k) pp->slot_cap[k] = ~0ull;
  for (uint32_t k = 0; k < pp->plan.n; ++k) {
    const FinalizeItem& it = pp->plan.item[k];
    uint64_t room = pp->cap_elems[it.col];
    if (it.sentinel_slot != 0xFF) room = room ? room - 1 : 0;
    if (it.rows_slot == 0xFF) { if (room < cap_all) cap_all = room; }
    else if (room < pp->slot_cap[it.rows_slot]) pp->slot_cap[it.rows_slot] = room;
  }
  if (cap_all > (1ull << 32)) cap_all = 1ull << 32;
  for (uint32_t k = 0; k < NSLOT; ++k) if (pp->slot_cap[k] > 0xFFFFFFFFull) pp->slot_cap[k] = 0xFFFFFFFFull; /* offsets into arenas and child tables are 32-bit */
  /* no more records than candidate line starts (NDJSON: a record needs a byte and an LF) or separators (array) */
  if (!array && cap_all > limit / 2 + 2) cap_all = limit / 2 + 2;
  if (array && cap_all > limit + 2) cap_all = limit + 2;
  pp->rec_cap = cap_all;
  return PJ_OK;
}

/* What the caller gets back once the totals are known. */
pj_status finish_columns(pj_ctx* c, uint32_t schema, uint64_t len, const ParsePlan& pp, uint64_t N, uint64_t n_errors, const uint64_t* total, bool over, pj_columns* out) {
  out->schema = schema;
  out->n_records = N;
  out->n_errors = n_errors;
  for (int t = 0; t < 4; ++t) out->n_rows[t] = 0;
  if (schema == PJ_SCHEMA_MIXED) { out->n_rows[1] = total[SLOT_ROWS_PET]; out->n_rows[2] = total[SLOT_ROWS_ORD]; out->n_rows[3] = total[SLOT_ROWS_USR]; }
  else out->n_rows[schema] = N;
  for (int i = 0; i < pp.nrc; ++i) out->col[pp.rcols[i]].count = N;
  for (uint32_t k = 0; k < pp.plan.n; ++k) {
    const FinalizeItem& it = pp.plan.item[k];
    const uint64_t rows = it.rows_slot == 0xFF ? N : total[it.rows_slot];
    out->col[it.col].count = rows + (it.sentinel_slot != 0xFF ? 1 : 0);
  }
  uint64_t alg = len;
  for (int i = 0; i < pp.nneed; ++i) alg += out->col[pp.need[i]].count * col_info(pp.need[i])->elem;
  c->stats.algorithmic_bytes = alg;
  if (over) return set_err(c, PJ_ERR_CAPACITY, "pj_parse: %llu records need larger output buffers", (unsigned long long)N);
  return PJ_OK;
}

/* Tile size of the stream kernel: about 104 records per tile of 128 threads, from the bytes per record the context
 * saw in its earlier calls on the schema (before the first one: from the benchmark distributions). The result of a
 * call does not depend on it. */
uint32_t pick_tile_bytes(const pj_ctx* c, uint32_t schema) {
  uint64_t tb;
  if (c->tile_bytes_opt) tb = c->tile_bytes_opt;
  else {
    static const double dflt[5] = {0, 300, 125, 190, 220};
    const double avg = c->avg_rec_bytes[schema] > 0 ? c->avg_rec_bytes[schema] : dflt[schema];
    tb = (uint64_t)(avg * (ST_THREADS * 13 / 16));
  }
  tb &= ~15ull;
  if (tb < ST_MIN_TILE_BYTES) tb = ST_MIN_TILE_BYTES;
  if (tb > ST_MAX_TILE_BYTES) tb = ST_MAX_TILE_BYTES;
  return (uint32_t)tb;
}

cudaError_t stream_launch(uint32_t schema, const StreamArgs* a, unsigned grid, cudaStream_t s) {
  switch (schema) {
    case PJ_SCHEMA_PET: return stream_launch_1(a, grid, s);
    case PJ_SCHEMA_ORDER: return stream_launch_2(a, grid, s);
    case PJ_SCHEMA_USER: return stream_launch_3(a, grid, s);
    default: return stream_launch_4(a, grid, s);
  }
}

/* NDJSON: one launch of k_parse_stream per piece. Host buffers of a whole stream are parsed in pieces cut after line
 * feeds, so that the copy of piece p+1 to the device, the kernel of piece p and the copy of the columns of piece p-1
 * back run at the same time on three streams. Every launch is enqueued before the host waits for anything: a piece
 * starts where the piece before it ended, which it reads from that piece's totals ON THE DEVICE (StreamArgs.prev). */
pj_status parse_stream(pj_ctx* c, uint32_t schema, const uint8_t* in, uint64_t len, uint64_t slack, int is_first, int is_last,
                       uint64_t goff, uint32_t in_kind, pj_columns* out) {
  const uint64_t limit = len + slack;
  ParsePlan pp;
  { pj_status st = plan_columns(c, schema, out, limit, false, &pp); if (st) return st; }
  const bool host_in = in_kind == PJ_MEM_HOST, host_out = out->mem_kind == PJ_MEM_HOST;
  uint64_t cut[MAX_PIECES + 1];
  int np = 1;
  cut[0] = 0; cut[1] = len;
  if (host_in && host_out && slack == 0 && is_first && is_last && c->piece_bytes != 0xFFFFFFFFu) {
    const uint64_t piece = c->piece_bytes ? c->piece_bytes : DEFAULT_PIECE_BYTES;
    uint64_t want = len / piece;
    if (want > MAX_PIECES) want = MAX_PIECES;
    np = 0;
    for (uint64_t k = 1; k < want; ++k) {
      const uint64_t target = len / want * k;
      if (target <= cut[np]) continue;
      const void* q = memrchr(in + cut[np], '\n', target - cut[np]);
      if (!q) continue;
      cut[np + 1] = (uint64_t)((const uint8_t*)q - in) + 1;
      ++np;
    }
    cut[++np] = len;
  }
  /* Input that lies on the device and is too long for 32-bit offsets (or whenever pj_options.device_piece_bytes asks
     for it) is parsed as byte ranges of at most 2 GiB, each with the bytes behind it as its slack: the rule that gives
     the lines of a stream to shards gives them to these ranges, and every launch starts from the totals the one before
     it left on the device. */
  bool ranges = false;
  if (!host_in && len && (limit >= (1ull << 32) || c->dev_piece_bytes)) {
    uint64_t piece = c->dev_piece_bytes ? c->dev_piece_bytes : (1ull << 31);
    if (piece < 64) piece = 64;
    if (piece > (1ull << 31)) piece = 1ull << 31;
    const uint64_t want = (len + piece - 1) / piece;
    if (want > MAX_PIECES) return set_err(c, PJ_ERR_TOO_LARGE, "pj_parse: %llu input bytes are more than %d ranges of %llu bytes", (unsigned long long)len, (int)MAX_PIECES, (unsigned long long)piece);
    np = (int)want;
    for (int k = 1; k < np; ++k) cut[k] = (uint64_t)k * piece;
    cut[np] = len;
    ranges = true;
  }
  const bool pipe = np > 1 && !ranges;
  if (pipe) { pj_status st = ensure_pipe_streams(c); if (st) return st; }
  cudaStream_t s_in = pipe ? c->s_in : c->stream, s_out = pipe ? c->s_out : c->stream;
  /* whatever goes wrong from here on, no copy may still be running when the call returns */
  struct Drain {
    pj_ctx* c; bool pipe;
    ~Drain() { if (pipe) { cudaStreamSynchronize(c->s_in); cudaStreamSynchronize(c->stream); cudaStreamSynchronize(c->s_out); } }
  } drain{c, pipe};

  const uint8_t* d_in = in;
  if (host_in && limit) {
    pj_status st = ensure(c, &c->in_stage, limit + 64);
    if (st) return st;
    d_in = (const uint8_t*)c->in_stage.p;
    if (pipe) { PJ_CUDA(c, cudaEventRecord(c->ev_in[0], c->stream)); PJ_CUDA(c, cudaStreamWaitEvent(s_in, c->ev_in[0], 0)); }
    for (int p = 0; p < np; ++p) {
      const uint64_t nb = cut[p + 1] - cut[p] + (p == np - 1 ? slack : 0);
      if (nb) PJ_CUDA(c, cudaMemcpyAsync((uint8_t*)c->in_stage.p + cut[p], in + cut[p], nb, cudaMemcpyHostToDevice, s_in));
      if (pipe) PJ_CUDA(c, cudaEventRecord(c->ev_in[p], s_in));
      c->stats.h2d_bytes += nb;
    }
  }

  const uint32_t tile_bytes = pick_tile_bytes(c, schema);
  /* look-back states: one buffer per piece, so that no launch waits for the one before it to be read back */
  uint64_t nt[MAX_PIECES], nt_total = 0;
  for (int p = 0; p < np; ++p) {
    const uint8_t* pin = d_in ? d_in + cut[p] : d_in;
    const uint32_t mis = (uint32_t)(reinterpret_cast<uintptr_t>(pin) & 15u);
    nt[p] = stream_tiles(mis, cut[p + 1] - cut[p], 1u, tile_bytes); /* at least one tile: it closes the offset columns */
    if (nt[p] >= (1ull << 31)) return set_err(c, PJ_ERR_TOO_LARGE, "pj_parse: too many tiles");
    nt_total += nt[p];
  }
  { pj_status st = ensure(c, &c->tiles, nt_total * sizeof(StreamTile) + (size_t)np * 256 + 256); if (st) return st; }
  PJ_CUDA(c, cudaMemsetAsync(c->tiles.p, 0, nt_total * sizeof(StreamTile) + (size_t)np * 256, c->stream));
  PJ_CUDA(c, cudaMemsetAsync(c->d_res, 0, sizeof(DevResult) * np, c->stream));
  if (c->stall_once) { /* test hook: tickets start at 1, tile 0 is never processed, the waits for it run out */
    c->stall_once = false;
    for (int p = 0; p < np; ++p) PJ_CUDA(c, cudaMemsetAsync((uint8_t*)c->tiles.p + (size_t)p * 256, 1, 1, c->stream));
  }
  c->stats.tile_records = ST_THREADS;
  uint64_t tiles_at = 0;
  for (int p = 0; p < np; ++p) {
    StreamArgs sa;
    memset(&sa, 0, sizeof sa);
    const uint64_t plen = cut[p + 1] - cut[p];
    sa.in = d_in ? d_in + cut[p] : d_in;
    sa.len = plen; sa.limit = plen + (p == np - 1 ? slack : 0); sa.goff = goff + cut[p];
    sa.is_first = (uint32_t)is_first; sa.is_last = (uint32_t)is_last;
    if (ranges) {
      const uint64_t rest = len - cut[p + 1] + slack; /* readable bytes behind the range */
      const uint64_t room = 0xFFFFFFF0ull - plen;
      const uint64_t sl = rest < room ? rest : room;
      sa.limit = plen + sl;
      sa.is_first = p == 0 ? (uint32_t)is_first : 0u;
      sa.is_last = (is_last && sl == rest) ? 1u : 0u;
    }
    sa.tile_bytes = tile_bytes; sa.ntiles = (uint32_t)nt[p];
    sa.spin_limit_ns = c->spin_ns;
    sa.opts = c->opt_flags;
    sa.ticket = (uint32_t*)((uint8_t*)c->tiles.p + (size_t)p * 256);
    sa.tiles = (StreamTile*)((uint8_t*)c->tiles.p + (size_t)np * 256) + tiles_at;
    tiles_at += nt[p];
    sa.res = c->d_res + p;
    sa.prev = p ? c->d_res + p - 1 : nullptr;
    for (uint32_t k = 0; k < NSLOT; ++k) sa.slot_cap[k] = pp.slot_cap[k];
    sa.rec_cap = pp.rec_cap;
    sa.plan = pp.plan;
    sa.cols = pp.dcols;
    if (pipe) PJ_CUDA(c, cudaStreamWaitEvent(c->stream, c->ev_in[p], 0));
    PJ_CUDA(c, cudaEventRecord(c->ev_k0[p], c->stream));
    PJ_CUDA(c, stream_launch(schema, &sa, (unsigned)nt[p], c->stream));
    PJ_CUDA(c, cudaEventRecord(c->ev_k1[p], c->stream));
    PJ_CUDA(c, cudaMemcpyAsync(c->h_res + p, c->d_res + p, sizeof(DevResult), cudaMemcpyDeviceToHost, c->stream));
    PJ_CUDA(c, cudaEventRecord(c->ev_done[p], c->stream));
    count_launch(c, 2);
    c->stats.tiles += (uint32_t)nt[p];
  }

  /* the pieces come back one by one; the columns of each go to the host while the later ones are parsed */
  uint64_t rows_done = 0, n_errors = 0, n_fast = 0;
  uint64_t total[NSLOT];
  for (uint32_t k = 0; k < NSLOT; ++k) total[k] = 0;
  bool over = false;
  for (int p = 0; p < np; ++p) {
    PJ_CUDA(c, cudaEventSynchronize(c->ev_done[p]));
    const DevResult& r = c->h_res[p];
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, c->ev_k0[p], c->ev_k1[p]) == cudaSuccess) { c->stats.stage_ms[2] += ms; c->stats.device_ms += ms; }
    n_fast += r.n_fast; n_errors += r.n_errors;
    for (int k = 0; k < 4; ++k) c->stats.phase_cycles[k] += r.phase_cycles[k];
    c->stats.lookback_polls += r.lookback_polls; c->stats.lookback_rounds += r.lookback_rounds;
    c->stats.wide_records += r.n_wide; c->stats.wide_fast_records += r.n_wide_fast;
    c->stats.wide_cycles[0] += r.wide_cycles[0]; c->stats.wide_cycles[1] += r.wide_cycles[1];
    if (r.timeout) return set_err(c, PJ_ERR_TIMEOUT, "pj_parse: a bounded device-side wait ran out");
    if (r.over) over = true;
    const uint64_t rows_new = r.n_records;
    if (host_out && !over) {
      if (pipe) PJ_CUDA(c, cudaStreamWaitEvent(s_out, c->ev_done[p], 0));
      auto copy_back = [&](int col, uint64_t from, uint64_t to) -> cudaError_t {
        const size_t e = col_info(col)->elem;
        if (to <= from) return cudaSuccess;
        c->stats.d2h_bytes += (to - from) * e;
        return cudaMemcpyAsync((uint8_t*)out->col[col].ptr + from * e, (uint8_t*)pp.dcols.ptr[col] + from * e, (to - from) * e, cudaMemcpyDeviceToHost, s_out);
      };
      for (int i = 0; i < pp.nrc; ++i) PJ_CUDA(c, copy_back(pp.rcols[i], rows_done, rows_new));
      for (uint32_t k = 0; k < pp.plan.n; ++k) {
        const FinalizeItem& it = pp.plan.item[k];
        const uint64_t from = it.rows_slot == 0xFF ? rows_done : total[it.rows_slot];
        const uint64_t to = (it.rows_slot == 0xFF ? rows_new : r.total[it.rows_slot]) + (it.sentinel_slot != 0xFF ? 1 : 0);
        PJ_CUDA(c, copy_back(it.col, from, to));
      }
    }
    rows_done = rows_new;
    for (uint32_t k = 0; k < NSLOT; ++k) total[k] = r.total[k];
  }
  PJ_CUDA(c, cudaGetLastError());
  c->stats.main_kernel_ms = c->stats.stage_ms[2];
  c->stats.fast_records = n_fast;
  c->stats.pieces = (uint32_t)np;
  out->doc_err_kind = 0; out->doc_err_off = 0;
  const pj_status st = finish_columns(c, schema, len, pp, rows_done, n_errors, total, over, out);
  if (st) return st;
  if (rows_done > 1000 && !c->tile_bytes_opt) c->avg_rec_bytes[schema] = (double)len / (double)rows_done;
  if (host_out) PJ_CUDA(c, cudaStreamSynchronize(s_out));
  return PJ_OK;
}

/* Array framing: the record index of pj_array_kernels.cuh (extent of every element), then the tile kernel over
 * tiles of TILE_THREADS records. */
pj_status parse_array(pj_ctx* c, uint32_t schema, const uint8_t* in, uint64_t len, uint32_t in_kind, pj_columns* out) {
  ParsePlan pp;
  { pj_status st = plan_columns(c, schema, out, len, true, &pp); if (st) return st; }
  const bool host_in = in_kind == PJ_MEM_HOST, host_out = out->mem_kind == PJ_MEM_HOST;
  const uint8_t* d_in = in;
  if (host_in && len) {
    pj_status st = ensure(c, &c->in_stage, len + 64);
    if (st) return st;
    d_in = (const uint8_t*)c->in_stage.p;
    PJ_CUDA(c, cudaMemcpyAsync(c->in_stage.p, in, len, cudaMemcpyHostToDevice, c->stream));
    c->stats.h2d_bytes += len;
  }
  const uint64_t cap_all = pp.rec_cap;
  const uint64_t nwords = (len + 63) >> 6;
  const uint64_t atiles = nwords ? (nwords + ARR_THREADS - 1) / ARR_THREADS : 1;
  const size_t off_fn = align_up((atiles + 1) * 4, 256);
  const size_t off_tin = align_up(off_fn + atiles * sizeof(ArrFn), 256);
  const size_t off_sep = align_up(off_tin + atiles * sizeof(ArrState), 256);
  const size_t off_rend = align_up(off_sep + (nwords + 1) * 8, 256);
  const size_t off_rblank = align_up(off_rend + cap_all * 8, 256);
  { pj_status st = ensure(c, &c->scratch, off_rblank + cap_all + 256); if (st) return st; }
  uint32_t* d_tile = (uint32_t*)c->scratch.p;
  uint64_t* d_rec_end = (uint64_t*)((uint8_t*)c->scratch.p + off_rend);
  uint8_t* d_rec_blank = (uint8_t*)c->scratch.p + off_rblank;
  uint32_t slot_lo, slot_hi;
  slot_range(schema, &slot_lo, &slot_hi);

  PJ_CUDA(c, cudaMemsetAsync(c->d_res, 0, sizeof(DevResult), c->stream));
  Stage stage(c);
  ArrArgs aa;
  aa.in = d_in; aa.len = len; aa.nwords = nwords;
  aa.tile_fn = (ArrFn*)((uint8_t*)c->scratch.p + off_fn); aa.tile_in = (ArrState*)((uint8_t*)c->scratch.p + off_tin);
  aa.sep = (uint64_t*)((uint8_t*)c->scratch.p + off_sep); aa.tile_cnt = d_tile;
  aa.rec_start = (uint64_t*)pp.dcols.ptr[PJ_COL_REC_START]; aa.rec_end = d_rec_end; aa.rec_blank = d_rec_blank;
  aa.cap = cap_all; aa.goff = 0; aa.ntiles = (uint32_t)atiles; aa.res = c->d_res;
  /* the two running minima start at "none" */
  PJ_CUDA(c, cudaMemsetAsync(&c->d_res->doc_err_off, 0xFF, sizeof(unsigned long long), c->stream));
  PJ_CUDA(c, cudaMemsetAsync(&c->d_res->first_opener, 0xFF, sizeof(unsigned long long), c->stream));
  k_arr_summary<<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
  k_arr_scan_tiles<<<1, 32, 0, c->stream>>>(aa);
  k_arr_mark<<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
  k_arr_records<false><<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
  k_scan_single<uint32_t><<<1, 1024, 0, c->stream>>>(d_tile, atiles, &c->d_res->n_records);
  k_arr_records<true><<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
  count_launch(c, 0, 6);
  PJ_CUDA(c, cudaGetLastError());
  stage.next();

  /* the tile kernel needs the record count to size its grid */
  PJ_CUDA(c, cudaMemcpyAsync(c->h_res, c->d_res, sizeof(DevResult), cudaMemcpyDeviceToHost, c->stream));
  PJ_CUDA(c, cudaStreamSynchronize(c->stream));
  const uint64_t N0 = c->h_res->n_records;
  uint64_t total[NSLOT];
  for (uint32_t k = 0; k < NSLOT; ++k) total[k] = 0;
  if (N0 > cap_all) {
    out->schema = schema; out->n_records = N0; out->n_errors = 0;
    for (int i = 0; i < pp.nrc; ++i) out->col[pp.rcols[i]].count = N0;
    return set_err(c, PJ_ERR_CAPACITY, "pj_parse: %llu records, per-record buffers hold %llu", (unsigned long long)N0, (unsigned long long)cap_all);
  }
  TileArgs ta;
  memset(&ta, 0, sizeof ta);
  ta.in = d_in; ta.limit = len; ta.goff = 0; ta.n_records = N0;
  ta.lf_ws = 1u; ta.open_end = 0u; ta.schema = schema; ta.slot_lo = slot_lo; ta.slot_hi = slot_hi;
  ta.win_bytes = TILE_WIN_BYTES; ta.tape_cap = TILE_TAPE_CAP;
  ta.tile_recs = TILE_THREADS;
  const uint64_t ntiles = N0 ? (N0 + TILE_THREADS - 1) / TILE_THREADS : 1;
  ta.ntiles = (uint32_t)ntiles;
  ta.spin_limit_ns = c->spin_ns;
  ta.opts = c->opt_flags;
  c->stats.tile_records = TILE_THREADS; c->stats.tiles += (uint32_t)ntiles;
  ta.rec_end = d_rec_end; ta.rec_blank = d_rec_blank;
  { pj_status st = ensure(c, &c->tiles, ntiles * sizeof(TileState) + 256); if (st) return st; }
  ta.ticket = (uint32_t*)c->tiles.p;
  ta.tiles = (TileState*)((uint8_t*)c->tiles.p + 128);
  ta.res = c->d_res;
  for (uint32_t k = 0; k < NSLOT; ++k) { ta.slot_cap[k] = pp.slot_cap[k]; ta.slot_base[k] = 0; }
  ta.plan = pp.plan;
  ta.cols = pp.dcols;
  PJ_CUDA(c, cudaMemsetAsync(c->tiles.p, 0, ntiles * sizeof(TileState) + 128, c->stream));
  const uint32_t one = 1;
  PJ_CUDA(c, cudaMemcpyAsync(&c->d_res->ok, &one, sizeof one, cudaMemcpyHostToDevice, c->stream));
  stage.next(); /* stage 1: set-up */
  switch (schema) {
    case PJ_SCHEMA_PET: PJ_CUDA(c, tile_launch_1(&ta, (unsigned)ntiles, c->stream)); break;
    case PJ_SCHEMA_ORDER: PJ_CUDA(c, tile_launch_2(&ta, (unsigned)ntiles, c->stream)); break;
    case PJ_SCHEMA_USER: PJ_CUDA(c, tile_launch_3(&ta, (unsigned)ntiles, c->stream)); break;
    default: PJ_CUDA(c, tile_launch_4(&ta, (unsigned)ntiles, c->stream)); break;
  }
  count_launch(c, 2);
  stage.next(); /* stage 2: the tile kernel */
  PJ_CUDA(c, cudaMemcpyAsync(c->h_res, c->d_res, sizeof(DevResult), cudaMemcpyDeviceToHost, c->stream));
  PJ_CUDA(c, cudaStreamSynchronize(c->stream));
  PJ_CUDA(c, cudaGetLastError());
  collect_times(c, 3);
  const DevResult r = *c->h_res;
  for (int k = 0; k < 4; ++k) c->stats.phase_cycles[k] += r.phase_cycles[k];
  c->stats.lookback_polls += r.lookback_polls; c->stats.lookback_rounds += r.lookback_rounds;
  c->stats.main_kernel_ms = c->stats.stage_ms[2];
  c->stats.fast_records = r.n_fast;
  c->stats.pieces = 1;
  if (r.timeout) return set_err(c, PJ_ERR_TIMEOUT, "pj_parse: a bounded device-side wait ran out");
  for (uint32_t k = 0; k < NSLOT; ++k) total[k] = r.total[k];
  out->doc_err_kind = 0; out->doc_err_off = 0;
  if (r.doc_err_off != ~0ull) { out->doc_err_kind = PJ_E_SYNTAX; out->doc_err_off = r.doc_err_off; }
  else if (r.first_opener == ~0ull || r.arr_final_s || r.arr_final_d != 0) { out->doc_err_kind = PJ_E_EOF; out->doc_err_off = len; }
  const pj_status st = finish_columns(c, schema, len, pp, r.n_records, r.n_errors, total, !r.ok, out);
  if (st) return st;
  if (host_out) {
    for (int i = 0; i < pp.nneed; ++i) {
      const int col = pp.need[i];
      const size_t nb = (size_t)out->col[col].count * col_info(col)->elem;
      if (nb) PJ_CUDA(c, cudaMemcpyAsync(out->col[col].ptr, pp.dcols.ptr[col], nb, cudaMemcpyDeviceToHost, c->stream));
      c->stats.d2h_bytes += nb;
    }
    PJ_CUDA(c, cudaStreamSynchronize(c->stream));
  }
  return PJ_OK;
}

pj_status parse_impl(pj_ctx* c, uint32_t schema, uint32_t framing, const uint8_t* in, uint64_t len, uint64_t slack,
                     int is_first, int is_last, uint64_t goff, uint32_t in_kind, pj_columns* out) {
  if (!c) return PJ_ERR_ARG;
  if (!out || (!in && len + slack) || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED || in_kind > PJ_MEM_DEVICE ||
      out->mem_kind > PJ_MEM_DEVICE)
    return set_err(c, PJ_ERR_ARG, "pj_parse: bad argument");
  if (framing > PJ_FRAMING_ARRAY) return set_err(c, PJ_ERR_ARG, "pj_parse: unknown framing %u", framing);
  const bool array = framing == PJ_FRAMING_ARRAY;
  if (array && (slack || !is_first || !is_last)) return set_err(c, PJ_ERR_ARG, "pj_parse: array framing cannot be sharded");
  const uint64_t limit = len + slack;
  /* one launch addresses its input with 32-bit offsets; NDJSON that lies on the device is cut into ranges (parse_stream) */
  if (limit >= (1ull << 32) && (array || in_kind != PJ_MEM_DEVICE))
    return set_err(c, PJ_ERR_TOO_LARGE, "pj_parse: %llu input bytes do not fit 32-bit offsets", (unsigned long long)limit);
  DeviceGuard guard(c->device);
  c->stats = pj_call_stats{};
  return array ? parse_array(c, schema, in, len, in_kind, out) : parse_stream(c, schema, in, len, slack, is_first, is_last, goff, in_kind, out);
}
}  // namespace

/* ================================================================================================ */
extern "C" {

int32_t pj_version(void) { return PJ_VERSION_MAJOR * 1000 + PJ_VERSION_MINOR; }

const char* pj_status_str(pj_status s) {
  switch (s) {
    case PJ_OK: return "PJ_OK";
    case PJ_ERR_ARG: return "PJ_ERR_ARG";
    case PJ_ERR_CAPACITY: return "PJ_ERR_CAPACITY";
    case PJ_ERR_CUDA: return "PJ_ERR_CUDA";
    case PJ_ERR_TIMEOUT: return "PJ_ERR_TIMEOUT";
    case PJ_ERR_NOMEM: return "PJ_ERR_NOMEM";
    case PJ_ERR_TOO_LARGE: return "PJ_ERR_TOO_LARGE";
    default: return "PJ_ERR_?";
  }
}
const char* pj_error_kind_str(int32_t kind) {
  static const char* const names[PJ_E_KIND_COUNT] = {"NONE", "SYNTAX", "EOF", "CTRL_CHAR", "BAD_ESCAPE", "BAD_SURROGATE", "UTF8", "TYPE",
                                                     "NUM_RANGE", "ENUM", "REQUIRED", "DATETIME", "DEPTH", "AMBIGUOUS", "TOO_LONG"};
  return kind >= 0 && kind < PJ_E_KIND_COUNT ? names[kind] : "?";
}
pj_status pj_column_info(int32_t col, const char** name, uint32_t* elem_bytes, uint32_t* owner) {
  const ColInfo* ci = col_info(col);
  if (!ci) return PJ_ERR_ARG;
  if (name) *name = ci->name;
  if (elem_bytes) *elem_bytes = ci->elem;
  if (owner) *owner = ci->owner;
  return PJ_OK;
}

pj_status pj_create(const pj_options* opt, pj_ctx** out) {
  if (!out) return PJ_ERR_ARG;
  *out = nullptr;
  int dev = opt ? opt->device : -1;
  int ndev = 0;
  cudaError_t e = cudaGetDeviceCount(&ndev);
  if (e != cudaSuccess || ndev == 0) { (void)cudaGetLastError(); return set_err(nullptr, PJ_ERR_CUDA, "no CUDA device: %s", cudaGetErrorString(e)); }
  if (dev < 0) { if (cudaGetDevice(&dev) != cudaSuccess) return set_err(nullptr, PJ_ERR_CUDA, "cudaGetDevice failed"); }
  if (dev >= ndev) return set_err(nullptr, PJ_ERR_ARG, "device %d of %d", dev, ndev);
  if (opt && (opt->inclusion < PJ_INCLUDE_NON_EMPTY || opt->inclusion > PJ_INCLUDE_ALWAYS)) return set_err(nullptr, PJ_ERR_ARG, "bad inclusion policy");
  pj_ctx* c = new (std::nothrow) pj_ctx();
  if (!c) return PJ_ERR_NOMEM;
  c->device = dev;
  c->inclusion = opt ? opt->inclusion : PJ_INCLUDE_NON_EMPTY;
  c->opt_flags = opt ? opt->flags : 0;
  c->stall_once = (c->opt_flags & PJ_OPT_TEST_STALL_ONCE) != 0;
  c->piece_bytes = opt ? opt->host_piece_bytes : 0;
  c->dev_piece_bytes = opt ? opt->device_piece_bytes : 0;
  c->tile_bytes_opt = opt ? opt->tile_bytes : 0;
  if (opt && opt->spin_limit_us) c->spin_ns = (unsigned long long)opt->spin_limit_us * 1000ull;
  DeviceGuard guard(dev);
  auto fail_create = [&](cudaError_t err, const char* what) {
    set_err(nullptr, PJ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(err));
    pj_destroy(c);
    return PJ_ERR_CUDA;
  };
  if (opt && opt->stream) c->stream = (cudaStream_t)opt->stream;
  else {
    e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return fail_create(e, "cudaStreamCreate");
    c->own_stream = true;
  }
  e = cudaMalloc(&c->d_res, sizeof(DevResult) * PJ_CTX_RESULTS);
  if (e != cudaSuccess) return fail_create(e, "cudaMalloc");
  e = cudaMallocHost(&c->h_res, sizeof(DevResult) * PJ_CTX_RESULTS);
  if (e != cudaSuccess) return fail_create(e, "cudaMallocHost");
  for (auto& ev : c->ev) { e = cudaEventCreate(&ev); if (e != cudaSuccess) return fail_create(e, "cudaEventCreate"); }
  for (auto& ev : c->ev_k0) { e = cudaEventCreate(&ev); if (e != cudaSuccess) return fail_create(e, "cudaEventCreate"); }
  for (auto& ev : c->ev_k1) { e = cudaEventCreate(&ev); if (e != cudaSuccess) return fail_create(e, "cudaEventCreate"); }
  for (auto& ev : c->ev_done) { e = cudaEventCreateWithFlags(&ev, cudaEventDisableTiming); if (e != cudaSuccess) return fail_create(e, "cudaEventCreate"); }
  build_schema(&c->schema);
  e = tile_init_1(&c->schema);
  if (e == cudaSuccess) e = tile_init_2(&c->schema);
  if (e == cudaSuccess) e = tile_init_3(&c->schema);
  if (e == cudaSuccess) e = tile_init_4(&c->schema);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_write_tile, cudaFuncAttributeMaxDynamicSharedMemorySize, WTILE_SMEM_BYTES);
#ifdef PJ_WT_CARVEOUT
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_write_tile, cudaFuncAttributePreferredSharedMemoryCarveout, PJ_WT_CARVEOUT);
#endif
  if (e != cudaSuccess) return fail_create(e, "cudaFuncSetAttribute");
  build_schema(&c->schema);
  e = cudaMemcpyToSymbol(c_schema, &c->schema, sizeof(Schema));
  if (e != cudaSuccess) return fail_create(e, "cudaMemcpyToSymbol");
  *out = c;
  return PJ_OK;
}

void pj_destroy(pj_ctx* c) {
  if (!c) return;
  DeviceGuard guard(c->device);
  if (c->stream) cudaStreamSynchronize(c->stream);
  for (Buffer* b : {&c->scratch, &c->in_stage, &c->col_stage, &c->out_stage, &c->tiles}) if (b->p) cudaFree(b->p);
  if (c->d_res) cudaFree(c->d_res);
  if (c->h_res) cudaFreeHost(c->h_res);
  for (auto& ev : c->ev) if (ev) cudaEventDestroy(ev);
  for (auto& ev : c->ev_in) if (ev) cudaEventDestroy(ev);
  for (auto& ev : c->ev_k0) if (ev) cudaEventDestroy(ev);
  for (auto& ev : c->ev_k1) if (ev) cudaEventDestroy(ev);
  for (auto& ev : c->ev_done) if (ev) cudaEventDestroy(ev);
  if (c->s_in) cudaStreamDestroy(c->s_in);
  if (c->s_out) cudaStreamDestroy(c->s_out);
  if (c->own_stream && c->stream) cudaStreamDestroy(c->stream);
  delete c;
}

const char* pj_last_error(const pj_ctx* c) { return c ? c->err : g_create_error; }

pj_status pj_last_stats(const pj_ctx* c, pj_call_stats* out) {
  if (!c || !out) return PJ_ERR_ARG;
  *out = c->stats;
  return PJ_OK;
}

pj_status pj_trim(pj_ctx* c) {
  if (!c) return PJ_ERR_ARG;
  DeviceGuard guard(c->device);
  PJ_CUDA(c, cudaStreamSynchronize(c->stream));
  for (Buffer* b : {&c->scratch, &c->in_stage, &c->col_stage, &c->out_stage, &c->tiles}) {
    if (b->p) { PJ_CUDA(c, cudaFree(b->p)); b->p = nullptr; b->cap = 0; }
  }
  return PJ_OK;
}

pj_status pj_columns_sizes(uint32_t schema, uint64_t max_records, uint64_t max_input_bytes, uint64_t max_list_items,
                           pj_columns* out) {
  if (!out || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return PJ_ERR_ARG;
  Schema S;
  build_schema(&S);
  FinalizePlan plan;
  build_finalize_plan(S, schema, &plan);
  /* a list item costs at least two input bytes ("" or {}) plus a separator on average */
  const uint64_t items = max_list_items ? max_list_items : max_input_bytes / 2 + 1;
  out->schema = schema;
  int rcols[5];
  const int nrc = record_cols(schema, rcols);
  for (int i = 0; i < nrc; ++i) out->col[rcols[i]].bytes = (max_records + 1) * col_info(rcols[i])->elem;
  for (uint32_t k = 0; k < plan.n; ++k) {
    const FinalizeItem& it = plan.item[k];
    uint64_t rows;
    if (it.rows_slot == 0xFF || it.rows_slot <= SLOT_ROWS_USR) rows = max_records;
    else if (it.elem == 1 && it.sentinel_slot == 0xFF && it.col != S.obj[OBJ_TAG].present_col) rows = max_input_bytes; /* arena: never more bytes than the input */
    else rows = items;
    out->col[it.col].bytes = (rows + 1) * it.elem;
  }
  return PJ_OK;
}

pj_status pj_parse(pj_ctx* ctx, uint32_t schema, uint32_t framing, const uint8_t* in, uint64_t len, uint32_t in_kind,
                   pj_columns* out) {
  return parse_impl(ctx, schema, framing, in, len, 0, 1, 1, 0, in_kind, out);
}

pj_status pj_parse_shard(pj_ctx* ctx, uint32_t schema, const uint8_t* in, uint64_t len, uint64_t slack, int32_t is_first,
                         int32_t is_last, uint64_t global_offset, uint32_t in_kind, pj_columns* out) {
  return parse_impl(ctx, schema, PJ_FRAMING_NDJSON, in, len, slack, is_first != 0, is_last != 0, global_offset, in_kind, out);
}

pj_status pj_index_records(pj_ctx* c, uint32_t framing, const uint8_t* in, uint64_t len, uint32_t kind, uint64_t* rec_start,
                           uint64_t cap, uint64_t* n) {
  if (!c) return PJ_ERR_ARG;
  if ((!in && len) || !n || (!rec_start && cap) || kind > PJ_MEM_DEVICE) return set_err(c, PJ_ERR_ARG, "pj_index_records: bad argument");
  if (framing > PJ_FRAMING_ARRAY) return set_err(c, PJ_ERR_ARG, "pj_index_records: unknown framing %u", framing);
  if (len >= (1ull << 32)) return set_err(c, PJ_ERR_TOO_LARGE, "pj_index_records: input too large");
  const bool array = framing == PJ_FRAMING_ARRAY;
  DeviceGuard guard(c->device);
  c->stats = pj_call_stats{};
  const uint8_t* d_in = in;
  uint64_t* d_rs = rec_start;
  const uint64_t ntiles = (len + 15 + INDEX_TILE) / INDEX_TILE;
  const uint64_t nwords = (len + 63) >> 6;
  const uint64_t atiles = nwords ? (nwords + ARR_THREADS - 1) / ARR_THREADS : 1;
  size_t off_fn = align_up(((ntiles > atiles ? ntiles : atiles) + 1) * 4, 256);
  size_t off_tin = align_up(off_fn + (array ? atiles * sizeof(ArrFn) : 0), 256);
  size_t off_sep = align_up(off_tin + (array ? atiles * sizeof(ArrState) : 0), 256);
  size_t off_rs = align_up(off_sep + (array ? (nwords + 1) * 8 : 0), 256);
  { pj_status st = ensure(c, &c->scratch, off_rs + (kind == PJ_MEM_HOST ? cap * 8 : 0) + 256); if (st) return st; }
  if (kind == PJ_MEM_HOST) {
    if (len) {
      pj_status st = ensure(c, &c->in_stage, len + 64);
      if (st) return st;
      PJ_CUDA(c, cudaMemcpyAsync(c->in_stage.p, in, len, cudaMemcpyHostToDevice, c->stream));
      c->stats.h2d_bytes += len;
      d_in = (const uint8_t*)c->in_stage.p;
    }
    d_rs = (uint64_t*)((uint8_t*)c->scratch.p + off_rs);
  }
  uint32_t* d_tile = (uint32_t*)c->scratch.p;
  PJ_CUDA(c, cudaMemsetAsync(c->d_res, 0, sizeof(DevResult), c->stream));
  Stage stage(c);
  if (!array) {
    IndexArgs ia;
    ia.in = d_in; ia.len = len; ia.limit = len; ia.is_first = 1; ia.is_last = 1;
    ia.tile = d_tile; ia.rec_start = d_rs; ia.cap = cap; ia.goff = 0;
    k_nd_index<false><<<(unsigned)ntiles, INDEX_THREADS, 0, c->stream>>>(ia);
    k_scan_single<uint32_t><<<1, 1024, 0, c->stream>>>(d_tile, ntiles, &c->d_res->n_records);
    k_nd_index<true><<<(unsigned)ntiles, INDEX_THREADS, 0, c->stream>>>(ia);
    count_launch(c, 0, 3);
  } else {
    ArrArgs aa;
    aa.in = d_in; aa.len = len; aa.nwords = nwords;
    aa.tile_fn = (ArrFn*)((uint8_t*)c->scratch.p + off_fn); aa.tile_in = (ArrState*)((uint8_t*)c->scratch.p + off_tin);
    aa.sep = (uint64_t*)((uint8_t*)c->scratch.p + off_sep); aa.tile_cnt = d_tile;
    aa.rec_start = d_rs; aa.rec_end = nullptr; aa.rec_blank = nullptr; /* an index-only call keeps the starts alone */
    aa.cap = cap; aa.goff = 0; aa.ntiles = (uint32_t)atiles; aa.res = c->d_res;
    PJ_CUDA(c, cudaMemsetAsync(&c->d_res->doc_err_off, 0xFF, sizeof(unsigned long long), c->stream));
    PJ_CUDA(c, cudaMemsetAsync(&c->d_res->first_opener, 0xFF, sizeof(unsigned long long), c->stream));
    k_arr_summary<<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
    k_arr_scan_tiles<<<1, 32, 0, c->stream>>>(aa);
    k_arr_mark<<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
    k_arr_records<false><<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
    k_scan_single<uint32_t><<<1, 1024, 0, c->stream>>>(d_tile, atiles, &c->d_res->n_records);
    k_arr_records<true><<<(unsigned)atiles, ARR_THREADS, 0, c->stream>>>(aa);
    count_launch(c, 0, 6);
  }
  PJ_CUDA(c, cudaGetLastError());
  stage.next();
  PJ_CUDA(c, cudaMemcpyAsync(c->h_res, c->d_res, sizeof(DevResult), cudaMemcpyDeviceToHost, c->stream));
  PJ_CUDA(c, cudaStreamSynchronize(c->stream));
  collect_times(c, 1);
  c->stats.main_kernel_ms = c->stats.stage_ms[0];
  *n = c->h_res->n_records;
  uint64_t got = *n < cap ? *n : cap;
  c->stats.algorithmic_bytes = len + got * 8;
  if (kind == PJ_MEM_HOST && got) {
    PJ_CUDA(c, cudaMemcpyAsync(rec_start, d_rs, got * 8, cudaMemcpyDeviceToHost, c->stream));
    PJ_CUDA(c, cudaStreamSynchronize(c->stream));
    c->stats.d2h_bytes += got * 8;
  }
  return *n > cap ? set_err(c, PJ_ERR_CAPACITY, "pj_index_records: %llu records, room for %llu", (unsigned long long)*n, (unsigned long long)cap) : PJ_OK;
}

/* ---- the allocation-free record index -------------------------------------------------------------
 * Scratch of pj_index_records_static: one count per 16 KiB tile of the largest accepted input, plus the
 * closing entry the scan writes. It lives in the library image; in host code its name only stands for
 * the symbol, so the device address is looked up once per device (static_scratch_for). */
static constexpr uint64_t STATIC_INDEX_TILES = (PJ_STATIC_INDEX_MAX_BYTES + 15 + INDEX_TILE) / INDEX_TILE;
static __device__ __align__(256) uint32_t g_static_index_scratch[STATIC_INDEX_TILES + 1];

static uint32_t* static_scratch_for(int device, cudaError_t* err) {
  static uint32_t* addr[64] = {};
  *err = cudaSuccess;
  if (device < 0 || device >= 64) { *err = cudaErrorInvalidDevice; return nullptr; }
  uint32_t* p = __atomic_load_n(&addr[device], __ATOMIC_ACQUIRE);
  if (!p) {
    /* the calling thread's current device is `device`: the address is that device's copy of the array */
    *err = cudaGetSymbolAddress((void**)&p, g_static_index_scratch);
    if (*err != cudaSuccess) return nullptr;
    __atomic_store_n(&addr[device], p, __ATOMIC_RELEASE);
  }
  return p;
}

pj_status pj_index_records_static(const uint8_t* in, uint64_t len, uint64_t* rec_start, uint64_t cap, uint64_t* n_device,
                                  void* stream) {
  if ((!in && len) || !n_device || (!rec_start && cap)) return set_err(nullptr, PJ_ERR_ARG, "pj_index_records_static: bad argument");
  if (len > PJ_STATIC_INDEX_MAX_BYTES)
    return set_err(nullptr, PJ_ERR_TOO_LARGE, "pj_index_records_static: %llu input bytes, the fixed scratch serves at most %llu",
                   (unsigned long long)len, (unsigned long long)PJ_STATIC_INDEX_MAX_BYTES);
  int device = -1;
  cudaError_t e = cudaGetDevice(&device);
  if (e != cudaSuccess) return set_err(nullptr, PJ_ERR_CUDA, "cudaGetDevice: %s", cudaGetErrorString(e));
  uint32_t* tile = static_scratch_for(device, &e);
  if (!tile) return set_err(nullptr, PJ_ERR_CUDA, "cudaGetSymbolAddress: %s", cudaGetErrorString(e));
  const uint64_t ntiles = (len + 15 + INDEX_TILE) / INDEX_TILE; /* <= STATIC_INDEX_TILES by the size check */
  cudaStream_t st = (cudaStream_t)stream;
  IndexArgs ia;
  ia.in = in; ia.len = len; ia.limit = len; ia.is_first = 1; ia.is_last = 1;
  ia.tile = tile; ia.rec_start = rec_start; ia.cap = cap; ia.goff = 0;
  k_nd_index<false><<<(unsigned)ntiles, INDEX_THREADS, 0, st>>>(ia);
  k_scan_single<uint32_t><<<1, 1024, 0, st>>>(tile, ntiles, (unsigned long long*)n_device);
  k_nd_index<true><<<(unsigned)ntiles, INDEX_THREADS, 0, st>>>(ia);
  e = cudaGetLastError();
  if (e != cudaSuccess) return set_err(nullptr, PJ_ERR_CUDA, "pj_index_records_static launch: %s", cudaGetErrorString(e));
  return PJ_OK;
}

pj_status pj_write(pj_ctx* c, uint32_t schema, uint32_t framing, const pj_columns* cols, uint8_t* out, uint64_t cap,
                   uint32_t out_kind, uint64_t* out_len) {
  if (!c) return PJ_ERR_ARG;
  if (!cols || !out_len || (!out && cap) || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED || framing > PJ_FRAMING_ARRAY ||
      out_kind > PJ_MEM_DEVICE || cols->mem_kind > PJ_MEM_DEVICE)
    return set_err(c, PJ_ERR_ARG, "pj_write: bad argument");
  DeviceGuard guard(c->device);
  c->stats = pj_call_stats{};
  const bool mixed = schema == PJ_SCHEMA_MIXED;
  const uint64_t n = mixed ? cols->n_records : cols->n_rows[schema];
  FinalizePlan plan;
  build_finalize_plan(c->schema, schema, &plan);
  int need[PJ_MAX_COLS], nneed = 0;
  if (mixed) { need[nneed++] = PJ_COL_REC_TYPE; need[nneed++] = PJ_COL_REC_ROW; }
  for (uint32_t k = 0; k < plan.n; ++k) need[nneed++] = plan.item[k].col;
  uint64_t col_bytes = 0;
  for (int i = 0; i < nneed; ++i) {
    const pj_buf& b = cols->col[need[i]];
    if (b.count && !b.ptr) return set_err(c, PJ_ERR_ARG, "pj_write: column %s has no buffer", col_info(need[i])->name);
    col_bytes += b.count * col_info(need[i])->elem;
  }
  /* the columns must describe n rows */
  if (mixed && (cols->col[PJ_COL_REC_TYPE].count < n || cols->col[PJ_COL_REC_ROW].count < n)) return set_err(c, PJ_ERR_ARG, "pj_write: record map shorter than n_records");
  for (uint32_t k = 0; k < plan.n; ++k) {
    const FinalizeItem& it = plan.item[k];
    if (it.rows_slot == 0xFF && cols->col[it.col].count < n + (it.sentinel_slot != 0xFF ? 1 : 0))
      return set_err(c, PJ_ERR_ARG, "pj_write: column %s holds %llu elements for %llu rows", col_info(it.col)->name,
                     (unsigned long long)cols->col[it.col].count, (unsigned long long)n);
  }
  DevCols dcols;
  memset(&dcols, 0, sizeof dcols);
  if (cols->mem_kind == PJ_MEM_HOST) {
    size_t tot = 0;
    for (int i = 0; i < nneed; ++i) tot += align_up(cols->col[need[i]].count * col_info(need[i])->elem, 256);
    pj_status st = ensure(c, &c->col_stage, tot + 256);
    if (st) return st;
    size_t at = 0;
    for (int i = 0; i < nneed; ++i) {
      size_t nb = (size_t)cols->col[need[i]].count * col_info(need[i])->elem;
      dcols.ptr[need[i]] = (uint8_t*)c->col_stage.p + at;
      if (nb) PJ_CUDA(c, cudaMemcpyAsync(dcols.ptr[need[i]], cols->col[need[i]].ptr, nb, cudaMemcpyHostToDevice, c->stream));
      c->stats.h2d_bytes += nb;
      at += align_up(nb, 256);
    }
  } else {
    for (int i = 0; i < nneed; ++i) dcols.ptr[need[i]] = cols->col[need[i]].ptr;
  }
  uint8_t* d_out = out;
  if (out_kind == PJ_MEM_HOST) {
    pj_status st = ensure(c, &c->out_stage, cap + 256);
    if (st) return st;
    d_out = (uint8_t*)c->out_stage.p;
  }
  DevResult init;
  memset(&init, 0, sizeof init);
  init.n_records = n;
  init.ok = 1;
  *c->h_res = init;
  PJ_CUDA(c, cudaMemcpyAsync(c->d_res, c->h_res, sizeof(DevResult), cudaMemcpyHostToDevice, c->stream));
  WriteArgs wa;
  wa.n = n; wa.schema = schema; wa.array = framing == PJ_FRAMING_ARRAY; wa.inclusion = c->inclusion;
  wa.hexa = (c->opt_flags & PJ_OPT_HEX_LOWER) ? 'a' : 'A';
  wa.out = d_out; wa.cap = cap; wa.res = c->d_res; wa.cols = dcols;
  {
    /* the single-pass tile writer; stages: [0] state reset and the look at the string arenas, [1] the closing kernel, [2] the tile kernel */
    const uint64_t ntiles = n ? (n + WT_THREADS - 1) / WT_THREADS : 1;
    { pj_status st = ensure(c, &c->tiles, 256 + ntiles * 16 + 256); if (st) return st; }
    WTileArgs ta;
    ta.w = wa;
    ta.ticket = (uint32_t*)c->tiles.p;
    ta.agg = (unsigned long long*)((uint8_t*)c->tiles.p + 256);
    ta.inc = ta.agg + ntiles;
    ta.ntiles = (uint32_t)ntiles;
    ta.spin_limit_ns = c->spin_ns;
    /* the string arenas of the schema */
    ArenaArgs aa;
    memset(&aa, 0, sizeof aa);
    aa.res = c->d_res;
    auto add_arenas = [&](const ObjDesc& O, auto&& self) -> void {
      for (int i = 0; i < (int)O.nfields; ++i) {
        const FieldDesc& F = O.f[i];
        int col = -1;
        if (F.kind == K_STR) col = F.col + 1;
        else if (F.kind == K_LIST_STR) col = F.col + 2;
        else if (F.kind == K_OBJ || F.kind == K_LIST_OBJ) self(c->schema.obj[F.child], self);
        if (col >= 0 && cols->col[col].count && aa.count < 12) { aa.p[aa.count] = (const uint8_t*)dcols.ptr[col]; aa.n[aa.count] = cols->col[col].count; aa.count++; }
      }
    };
    if (schema == PJ_SCHEMA_PET || mixed) add_arenas(c->schema.obj[OBJ_PET], add_arenas);
    if (schema == PJ_SCHEMA_ORDER || mixed) add_arenas(c->schema.obj[OBJ_ORDER], add_arenas);
    if (schema == PJ_SCHEMA_USER || mixed) add_arenas(c->schema.obj[OBJ_USER], add_arenas);
    Stage stage(c);
    PJ_CUDA(c, cudaMemsetAsync(c->tiles.p, 0, 256 + ntiles * 16, c->stream));
    if (aa.count) { k_arena_flags<<<persistent_grid(c, col_bytes / 16 + 1, 256), 256, 0, c->stream>>>(aa); count_launch(c, 0); }
    stage.next();
    cudaEvent_t ev_tile0 = c->ev[8], ev_tile1 = c->ev[9];
    PJ_CUDA(c, cudaEventRecord(ev_tile0, c->stream));
    k_write_tile<<<(unsigned)ntiles, WT_THREADS, WTILE_SMEM_BYTES, c->stream>>>(ta);
    PJ_CUDA(c, cudaEventRecord(ev_tile1, c->stream));
    k_write_close<<<1, 32, 0, c->stream>>>(wa);
    count_launch(c, 2); count_launch(c, 1);
    PJ_CUDA(c, cudaGetLastError());
    stage.next();
    stage.next();
  }
  PJ_CUDA(c, cudaMemcpyAsync(c->h_res, c->d_res, sizeof(DevResult), cudaMemcpyDeviceToHost, c->stream));
  PJ_CUDA(c, cudaStreamSynchronize(c->stream));
  PJ_CUDA(c, cudaGetLastError());
  collect_times(c, 3);
  {
    /* stage 1 covered both kernels: split it with the events around the tile kernel */
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, c->ev[8], c->ev[9]) == cudaSuccess) { c->stats.stage_ms[2] = ms; c->stats.stage_ms[1] -= ms; }
    c->stats.main_kernel_ms = c->stats.stage_ms[2];
  }
  for (int k = 0; k < 4; ++k) c->stats.phase_cycles[k] = c->h_res->phase_cycles[k];
  c->stats.tiles = (uint32_t)(n ? (n + WT_THREADS - 1) / WT_THREADS : 1);
  if (c->h_res->timeout) return set_err(c, PJ_ERR_TIMEOUT, "pj_write: a bounded device-side wait ran out");
  *out_len = c->h_res->out_bytes;
  c->stats.algorithmic_bytes = col_bytes + *out_len;
  if (!c->h_res->ok) return set_err(c, PJ_ERR_CAPACITY, "pj_write: %llu bytes needed, room for %llu", (unsigned long long)*out_len, (unsigned long long)cap);
  if (out_kind == PJ_MEM_HOST && *out_len) {
    PJ_CUDA(c, cudaMemcpyAsync(out, d_out, *out_len, cudaMemcpyDeviceToHost, c->stream));
    PJ_CUDA(c, cudaStreamSynchronize(c->stream));
    c->stats.d2h_bytes += *out_len;
  }
  return PJ_OK;
}

pj_status pj_columns_checksum(pj_ctx* c, uint32_t schema, const pj_columns* cols, uint64_t* sums) {
  if (!c) return PJ_ERR_ARG;
  if (!cols || !sums || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED || cols->mem_kind != PJ_MEM_DEVICE) return set_err(c, PJ_ERR_ARG, "pj_columns_checksum: bad argument");
  DeviceGuard guard(c->device);
  c->stats = pj_call_stats{};
  FinalizePlan plan;
  build_finalize_plan(c->schema, schema, &plan);
  int rcols[5];
  const int nrc = record_cols(schema, rcols);
  ChecksumArgs a;
  memset(&a, 0, sizeof a);
  uint64_t most = 0, bytes = 0;
  auto add = [&](int col) {
    const uint64_t nb = cols->col[col].count * col_info(col)->elem;
    a.p[col] = (const uint8_t*)cols->col[col].ptr; a.n[col] = a.p[col] ? nb : 0;
    if (a.n[col] > most) most = a.n[col];
    bytes += a.n[col];
  };
  for (int i = 0; i < nrc; ++i) add(rcols[i]);
  for (uint32_t k = 0; k < plan.n; ++k) add(plan.item[k].col);
  { pj_status st = ensure(c, &c->scratch, sizeof(unsigned long long) * PJ_MAX_COLS + 256); if (st) return st; }
  a.out = (unsigned long long*)c->scratch.p;
  PJ_CUDA(c, cudaMemsetAsync(a.out, 0, sizeof(unsigned long long) * PJ_MAX_COLS, c->stream));
  Stage stage(c);
  dim3 grid((unsigned)persistent_grid(c, most / 8 + 1, 256), PJ_MAX_COLS);
  k_checksum<<<grid, 256, 0, c->stream>>>(a);
  count_launch(c, 0);
  PJ_CUDA(c, cudaGetLastError());
  stage.next();
  PJ_CUDA(c, cudaMemcpyAsync(sums, a.out, sizeof(uint64_t) * PJ_MAX_COLS, cudaMemcpyDeviceToHost, c->stream));
  PJ_CUDA(c, cudaStreamSynchronize(c->stream));
  collect_times(c, 1);
  c->stats.main_kernel_ms = c->stats.stage_ms[0];
  c->stats.algorithmic_bytes = bytes;
  c->stats.d2h_bytes = sizeof(uint64_t) * PJ_MAX_COLS;
  return PJ_OK;
}

}  // extern "C"

/* ================================================================================================
 * Several GPUs of one machine: pj_group_*
 *
 * One process, one pj_ctx, one stream and one host thread per shard. The threads are started once (pj_group_create)
 * and sleep between calls. NCCL is bound at run time (dlopen), so the library loads on machines without it; only
 * ncclCommInitAll / ncclAllGather / ncclCommDestroy / ncclGetErrorString are used.
 * ================================================================================================ */
namespace {

typedef struct ncclComm* pj_nccl_comm;
struct NcclApi {
  void* handle = nullptr;
  int (*CommInitAll)(pj_nccl_comm*, int, const int*) = nullptr;
  int (*CommDestroy)(pj_nccl_comm) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, pj_nccl_comm, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  bool load() {
    if (handle) return true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) { handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (handle) break; }
    if (!handle) return false;
    CommInitAll = (int (*)(pj_nccl_comm*, int, const int*))dlsym(handle, "ncclCommInitAll");
    CommDestroy = (int (*)(pj_nccl_comm))dlsym(handle, "ncclCommDestroy");
    AllGather = (int (*)(const void*, void*, size_t, int, pj_nccl_comm, cudaStream_t))dlsym(handle, "ncclAllGather");
    GetErrorString = (const char* (*)(int))dlsym(handle, "ncclGetErrorString");
    return CommInitAll && CommDestroy && AllGather && GetErrorString;
  }
};
constexpr int PJ_NCCL_UINT64 = 5; /* ncclUint64 */

/* A host thread that runs one job at a time. Hand-over in both directions first spins for a while on an atomic
 * sequence number (a job follows the previous one within microseconds in a steady stream of calls; a condition
 * variable alone costs tens of microseconds per wake-up) and only then sleeps. */
struct Worker {
  std::thread th;
  std::mutex m;
  std::condition_variable cv;
  std::function<void()> job;
  std::atomic<uint64_t> submitted{0}, done{0};
  std::atomic<bool> stop{false};
  static constexpr int SPINS = 20000;
  void start() {
    th = std::thread([this] {
      uint64_t seen = 0;
      for (;;) {
        int spins = 0;
        while (submitted.load(std::memory_order_acquire) == seen && !stop.load(std::memory_order_acquire)) {
          if (++spins < SPINS) { std::this_thread::yield(); continue; }
          std::unique_lock<std::mutex> lk(m);
          cv.wait(lk, [&] { return submitted.load(std::memory_order_acquire) != seen || stop.load(std::memory_order_acquire); });
        }
        if (stop.load(std::memory_order_acquire)) return;
        seen = submitted.load(std::memory_order_acquire);
        job();
        { std::lock_guard<std::mutex> lk(m); done.store(seen, std::memory_order_release); }
        cv.notify_all();
      }
    });
  }
  void submit(std::function<void()> j) {
    { std::lock_guard<std::mutex> lk(m); job = std::move(j); submitted.fetch_add(1, std::memory_order_release); }
    cv.notify_all();
  }
  void wait() {
    const uint64_t want = submitted.load(std::memory_order_acquire);
    int spins = 0;
    while (done.load(std::memory_order_acquire) != want) {
      if (++spins < SPINS) { std::this_thread::yield(); continue; }
      std::unique_lock<std::mutex> lk(m);
      cv.wait(lk, [&] { return done.load(std::memory_order_acquire) == want; });
    }
  }
  void finish() {
    { std::lock_guard<std::mutex> lk(m); stop.store(true, std::memory_order_release); }
    cv.notify_all();
    if (th.joinable()) th.join();
  }
};
/* All workers of a group meet here in the middle of a job (every one of them runs the same job at the same time). */
struct Rendezvous {
  std::atomic<uint32_t> arrived{0}, generation{0};
  void meet(uint32_t n) {
    const uint32_t gen = generation.load(std::memory_order_acquire);
    if (arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == n) {
      arrived.store(0, std::memory_order_relaxed);
      generation.fetch_add(1, std::memory_order_release);
    } else {
      while (generation.load(std::memory_order_acquire) == gen) std::this_thread::yield();
    }
  }
};

/* the counters of one shard, as the gathered table holds them, from the result block of its last launch */
__global__ void k_group_counters(const DevResult* res, uint64_t bytes, unsigned long long* out /*[PJ_GROUP_NCOUNT]*/) {
  const uint32_t k = threadIdx.x;
  if (k >= PJ_GROUP_NCOUNT) return;
  unsigned long long v = 0;
  if (k == PJ_GC_RECORDS) v = res->n_records;
  else if (k == PJ_GC_ERRORS) v = res->n_errors;
  else if (k == PJ_GC_BYTES) v = bytes ? bytes : res->out_bytes;
  else if (k == PJ_GC_ROWS_PET) v = res->total[SLOT_ROWS_PET];
  else if (k == PJ_GC_ROWS_ORDER) v = res->total[SLOT_ROWS_ORD];
  else if (k == PJ_GC_ROWS_USER) v = res->total[SLOT_ROWS_USR];
  else if (k >= PJ_GC_COUNTER0 && k < PJ_GC_COUNTER0 + NSLOT) v = res->total[k - PJ_GC_COUNTER0];
  out[k] = v;
}

}  // namespace

struct pj_group {
  int ndev = 0;
  std::vector<int> devs;
  std::vector<pj_ctx*> ctx;
  std::vector<Worker*> workers;
  std::vector<pj_nccl_comm> comms;
  std::vector<unsigned long long*> d_mine;  /* [PJ_GROUP_NCOUNT] on the shard's device */
  std::vector<unsigned long long*> d_table; /* [ndev][PJ_GROUP_NCOUNT] on the shard's device */
  std::vector<unsigned long long*> h_table; /* pinned copy per shard */
  std::vector<cudaStream_t> xs;             /* the exchange's own stream per shard: the next call's kernels do not wait for it */
  std::vector<cudaEvent_t> ev_cnt, ev_xdone; /* counters written (shard's stream) / exchange finished (its own stream) */
  bool nccl = false;
  NcclApi api;
  Rendezvous rendezvous;
  char err[256] = "";
};

namespace {

pj_status group_err(pj_group* g, pj_status st, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g ? g->err : g_create_error, 256, fmt, ap);
  va_end(ap);
  return st;
}

template <class F>
void group_run(pj_group* g, F&& fn) {
  for (int i = 0; i < g->ndev; ++i) g->workers[i]->submit([&fn, i] { fn(i); });
  for (int i = 0; i < g->ndev; ++i) g->workers[i]->wait();
}

/* The counters of one shard as the table holds them, from the host copy of the result block of its last launch
 * (the same rule as k_group_counters). */
void group_host_row(const DevResult& res, uint64_t bytes, unsigned long long* row) {
  for (uint32_t k = 0; k < PJ_GROUP_NCOUNT; ++k) {
    unsigned long long v = 0;
    if (k == PJ_GC_RECORDS) v = res.n_records;
    else if (k == PJ_GC_ERRORS) v = res.n_errors;
    else if (k == PJ_GC_BYTES) v = bytes ? bytes : res.out_bytes;
    else if (k == PJ_GC_ROWS_PET) v = res.total[SLOT_ROWS_PET];
    else if (k == PJ_GC_ROWS_ORDER) v = res.total[SLOT_ROWS_ORD];
    else if (k == PJ_GC_ROWS_USER) v = res.total[SLOT_ROWS_USR];
    else if (k >= PJ_GC_COUNTER0 && k < PJ_GC_COUNTER0 + NSLOT) v = res.total[k - PJ_GC_COUNTER0];
    row[k] = v;
  }
}
/* The exchange of the counter table. A shard's call has read its result block back already, so the HOST table (row i
 * of h_table[0], written by shard i's thread before the rendezvous) is complete once every thread has passed the
 * rendezvous, and the caller's answer needs nothing else. The DEVICE tables are produced without the host, and
 * without the shard's stream, waiting for them: the counters of the result block are gathered by k_group_counters on
 * the shard's stream, and ncclAllGather runs on a stream of its own behind an event — an all-gather of eight ranks
 * takes longer than a tenth of a parse step, and the next step's kernels have no reason to queue behind it. (When
 * the device list repeats a device the host table is uploaded instead.) Called on the shard's thread, its device
 * current. */
pj_status group_gather(pj_group* g, int i, int res_index, uint64_t bytes, bool from_host = false) {
  pj_ctx* c = g->ctx[i];
  if (g->nccl && !from_host) {
    if (cudaStreamWaitEvent(c->stream, g->ev_xdone[i], 0) != cudaSuccess) return PJ_ERR_CUDA; /* the exchange before this one has read d_mine */
    k_group_counters<<<1, 32, 0, c->stream>>>(c->d_res + res_index, bytes, g->d_mine[i]);
    if (cudaGetLastError() != cudaSuccess) return PJ_ERR_CUDA;
    if (cudaEventRecord(g->ev_cnt[i], c->stream) != cudaSuccess || cudaStreamWaitEvent(g->xs[i], g->ev_cnt[i], 0) != cudaSuccess) return PJ_ERR_CUDA;
    const int r = g->api.AllGather(g->d_mine[i], g->d_table[i], PJ_GROUP_NCOUNT, PJ_NCCL_UINT64, g->comms[i], g->xs[i]);
    if (r != 0) return set_err(c, PJ_ERR_NCCL, "ncclAllGather: %s", g->api.GetErrorString(r));
    if (cudaEventRecord(g->ev_xdone[i], g->xs[i]) != cudaSuccess) return PJ_ERR_CUDA;
  } else {
    cudaStreamSynchronize(g->xs[i]); /* the upload (or all-gather) before this one is through with the tables */
    if (i) memcpy(g->h_table[i], g->h_table[0], sizeof(unsigned long long) * PJ_GROUP_NCOUNT * g->ndev);
    if (cudaMemcpyAsync(g->d_table[i], g->h_table[i], sizeof(unsigned long long) * PJ_GROUP_NCOUNT * g->ndev, cudaMemcpyHostToDevice, g->xs[i]) != cudaSuccess) return PJ_ERR_CUDA;
  }
  return PJ_OK;
}
/* the device table of shard i is complete (for a caller that wants to read it) */
pj_status group_wait_table(pj_group* g, int i) {
  DeviceGuard guard(g->devs[i]);
  return cudaStreamSynchronize(g->xs[i]) == cudaSuccess ? PJ_OK : PJ_ERR_CUDA;
}
void group_fill(pj_group* g, pj_group_shard* shards, bool offsets_from_bytes) {
  uint64_t off = 0, rec = 0, rows[4] = {0, 0, 0, 0};
  for (int i = 0; i < g->ndev; ++i) {
    const unsigned long long* t = g->h_table[0] + (size_t)i * PJ_GROUP_NCOUNT;
    if (offsets_from_bytes) shards[i].global_offset = off;
    shards[i].first_record = rec;
    shards[i].first_row[0] = 0;
    for (int k = 1; k < 4; ++k) shards[i].first_row[k] = rows[k];
    shards[i].bytes = t[PJ_GC_BYTES];
    shards[i].table_dev = (const uint64_t*)g->d_table[i];
    off += t[PJ_GC_BYTES]; rec += t[PJ_GC_RECORDS];
    rows[1] += t[PJ_GC_ROWS_PET]; rows[2] += t[PJ_GC_ROWS_ORDER]; rows[3] += t[PJ_GC_ROWS_USER];
  }
}

}  // namespace

extern "C" {

pj_status pj_group_create(int32_t ndev, const int32_t* devs, const pj_options* opt, pj_group** out) {
  if (!out || ndev < 1 || ndev > 64 || !devs) return PJ_ERR_ARG;
  *out = nullptr;
  pj_group* g = new (std::nothrow) pj_group();
  if (!g) return PJ_ERR_NOMEM;
  g->ndev = ndev;
  bool distinct = true;
  for (int i = 0; i < ndev; ++i) {
    for (int k = 0; k < i; ++k) if (devs[k] == devs[i]) distinct = false;
    g->devs.push_back(devs[i]);
  }
  pj_status st = PJ_OK;
  for (int i = 0; i < ndev && st == PJ_OK; ++i) {
    pj_options o;
    memset(&o, 0, sizeof o);
    if (opt) o = *opt;
    o.device = devs[i]; o.stream = nullptr;
    pj_ctx* c = nullptr;
    st = pj_create(&o, &c);
    if (st != PJ_OK) break;
    g->ctx.push_back(c);
    DeviceGuard guard(devs[i]);
    unsigned long long *mine = nullptr, *table = nullptr, *host = nullptr;
    if (cudaMalloc(&mine, sizeof(unsigned long long) * PJ_GROUP_NCOUNT) != cudaSuccess ||
        cudaMalloc(&table, sizeof(unsigned long long) * PJ_GROUP_NCOUNT * ndev) != cudaSuccess ||
        cudaMallocHost(&host, sizeof(unsigned long long) * PJ_GROUP_NCOUNT * ndev) != cudaSuccess) {
      (void)cudaGetLastError();
      st = set_err(nullptr, PJ_ERR_NOMEM, "pj_group_create: allocation failed on device %d", devs[i]);
    }
    g->d_mine.push_back(mine); g->d_table.push_back(table); g->h_table.push_back(host);
    cudaStream_t xs = nullptr;
    cudaEvent_t e1 = nullptr, e2 = nullptr;
    if (st == PJ_OK && (cudaStreamCreateWithFlags(&xs, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) != cudaSuccess ||
                        cudaEventCreateWithFlags(&e2, cudaEventDisableTiming) != cudaSuccess)) {
      (void)cudaGetLastError();
      st = set_err(nullptr, PJ_ERR_CUDA, "pj_group_create: stream / event creation failed on device %d", devs[i]);
    }
    g->xs.push_back(xs); g->ev_cnt.push_back(e1); g->ev_xdone.push_back(e2);
    /* every device may read its neighbours' input buffers (the slack copy) */
    for (int k = 0; k < ndev && st == PJ_OK; ++k) {
      if (devs[k] == devs[i]) continue;
      int can = 0;
      cudaDeviceCanAccessPeer(&can, devs[i], devs[k]);
      if (can) { cudaError_t e = cudaDeviceEnablePeerAccess(devs[k], 0); if (e != cudaSuccess) (void)cudaGetLastError(); /* already enabled is fine; without it the copy is staged by the driver */ }
    }
  }
  if (st == PJ_OK && distinct) {
    if (!g->api.load()) st = set_err(nullptr, PJ_ERR_NCCL, "pj_group_create: libnccl.so.2 could not be loaded (%s)", dlerror() ? dlerror() : "symbols missing");
    else {
      g->comms.resize(ndev);
      const int r = g->api.CommInitAll(g->comms.data(), ndev, g->devs.data());
      if (r != 0) { g->comms.clear(); st = set_err(nullptr, PJ_ERR_NCCL, "ncclCommInitAll: %s", g->api.GetErrorString(r)); }
      else g->nccl = true;
    }
  }
  if (st != PJ_OK) { pj_group_destroy(g); return st; }
  for (int i = 0; i < ndev; ++i) { Worker* w = new Worker(); w->start(); g->workers.push_back(w); }
  *out = g;
  return PJ_OK;
}

void pj_group_destroy(pj_group* g) {
  if (!g) return;
  for (Worker* w : g->workers) { w->finish(); delete w; }
  for (size_t i = 0; i < g->ctx.size(); ++i) {
    DeviceGuard guard(g->devs[i]);
    if (g->ctx[i]) cudaStreamSynchronize(g->ctx[i]->stream);
    if (i < g->xs.size() && g->xs[i]) cudaStreamSynchronize(g->xs[i]);
  }
  for (size_t i = 0; i < g->comms.size(); ++i) if (g->comms[i]) g->api.CommDestroy(g->comms[i]);
  for (size_t i = 0; i < g->d_mine.size(); ++i) {
    DeviceGuard guard(g->devs[i]);
    if (i < g->xs.size() && g->xs[i]) cudaStreamDestroy(g->xs[i]);
    if (i < g->ev_cnt.size() && g->ev_cnt[i]) cudaEventDestroy(g->ev_cnt[i]);
    if (i < g->ev_xdone.size() && g->ev_xdone[i]) cudaEventDestroy(g->ev_xdone[i]);
    if (g->d_mine[i]) cudaFree(g->d_mine[i]);
    if (g->d_table[i]) cudaFree(g->d_table[i]);
    if (g->h_table[i]) cudaFreeHost(g->h_table[i]);
  }
  for (pj_ctx* c : g->ctx) pj_destroy(c);
  delete g;
}

int32_t pj_group_size(const pj_group* g) { return g ? g->ndev : 0; }
pj_ctx* pj_group_ctx(pj_group* g, int32_t i) { return g && i >= 0 && i < g->ndev ? g->ctx[i] : nullptr; }
const char* pj_group_last_error(const pj_group* g) { return g ? g->err : g_create_error; }
int32_t pj_group_uses_nccl(const pj_group* g) { return g && g->nccl ? 1 : 0; }
pj_status pj_group_sync(pj_group* g) {
  if (!g) return PJ_ERR_ARG;
  for (int i = 0; i < g->ndev; ++i) if (group_wait_table(g, i) != PJ_OK) return group_err(g, PJ_ERR_CUDA, "pj_group_sync: shard %d", i);
  return PJ_OK;
}

pj_status pj_group_parse(pj_group* g, uint32_t schema, uint8_t* const* in, const uint64_t* len, const uint64_t* room, uint64_t slack,
                         pj_columns* out, pj_group_shard* shards) {
  if (!g) return PJ_ERR_ARG;
  if (!in || !len || !room || !out || !shards || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return group_err(g, PJ_ERR_ARG, "pj_group_parse: bad argument");
  const int n = g->ndev;
  std::vector<uint64_t> goff(n + 1, 0);
  for (int i = 0; i < n; ++i) {
    if (!in[i] && (len[i] || room[i])) return group_err(g, PJ_ERR_ARG, "pj_group_parse: shard %d has no buffer", i);
    if (out[i].mem_kind != PJ_MEM_DEVICE) return group_err(g, PJ_ERR_ARG, "pj_group_parse: columns of shard %d are not device memory", i);
    goff[i + 1] = goff[i] + len[i];
  }
  group_run(g, [&](int i) {
    DeviceGuard guard(g->devs[i]);
    pj_ctx* c = g->ctx[i];
    pj_group_shard& S = shards[i];
    memset(&S, 0, sizeof S);
    S.global_offset = goff[i];
    /* the head of what follows becomes this shard's slack: from as many following shards as it takes */
    uint64_t want = slack < room[i] ? slack : room[i], got = 0;
    cudaEventRecord(c->ev[6], c->stream);
    for (int h = i + 1; h < n && got < want; ++h) {
      const uint64_t take = len[h] < want - got ? len[h] : want - got;
      if (take) {
        const cudaError_t e = cudaMemcpyPeerAsync(in[i] + len[i] + got, g->devs[i], in[h], g->devs[h], take, c->stream);
        if (e != cudaSuccess) { S.status = set_err(c, PJ_ERR_CUDA, "cudaMemcpyPeerAsync: %s", cudaGetErrorString(e)); break; } /* no early return: every shard must reach the exchange */
      }
      got += take;
    }
    cudaEventRecord(c->ev[7], c->stream);
    S.slack_bytes = got;
    const bool is_last = goff[i] + len[i] + got == goff[n]; /* the readable bytes reach the end of the stream */
    const bool is_first = goff[i] == 0;                     /* nothing precedes: the line at byte 0 is this shard's */
    if (S.status == PJ_OK) S.status = parse_impl(c, schema, PJ_FRAMING_NDJSON, in[i], len[i], got, is_first, is_last, goff[i], PJ_MEM_DEVICE, &out[i]);
    if (S.status != PJ_OK && S.status != PJ_ERR_CAPACITY) {
      /* the table must still be exchanged by every shard (a collective): deliver zeros */
      cudaMemsetAsync(c->d_res, 0, sizeof(DevResult), c->stream);
      memset(c->h_res, 0, sizeof(DevResult));
    }
    group_host_row(c->h_res[0], len[i] ? len[i] : ~0ull, g->h_table[0] + (size_t)i * PJ_GROUP_NCOUNT);
    if (cudaEventElapsedTime(&S.slack_copy_ms, c->ev[6], c->ev[7]) != cudaSuccess) { S.slack_copy_ms = 0.f; (void)cudaGetLastError(); }
    /* The exchange starts only when EVERY shard is through its parse: an all-gather kernel waits on its device for the
       other devices' kernels, and a cudaMalloc on one of those (a parse growing its scratch) waits for the first device
       to go idle, because new memory is mapped into the peers: together they would never finish. Nothing allocates
       from here on. */
    g->rendezvous.meet((uint32_t)n);
    const auto t0 = std::chrono::steady_clock::now();
    const pj_status gs = group_gather(g, i, 0, len[i] ? len[i] : ~0ull);
    S.gather_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (S.status == PJ_OK) S.status = gs;
  });
  pj_status st = PJ_OK;
  group_fill(g, shards, false);
  for (int i = 0; i < n; ++i) if (shards[i].bytes == ~0ull) shards[i].bytes = 0;
  for (int i = 0; i < n && st == PJ_OK; ++i) if (shards[i].status != PJ_OK) { st = shards[i].status; group_err(g, st, "shard %d: %s", i, pj_last_error(g->ctx[i])); }
  return st;
}

pj_status pj_group_parse_host(pj_group* g, uint32_t schema, const uint8_t* text, const uint64_t* len, uint64_t slack, pj_columns* out,
                              pj_group_shard* shards) {
  if (!g) return PJ_ERR_ARG;
  if (!len || !out || !shards || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return group_err(g, PJ_ERR_ARG, "pj_group_parse_host: bad argument");
  const int n = g->ndev;
  std::vector<uint64_t> goff(n + 1, 0);
  for (int i = 0; i < n; ++i) goff[i + 1] = goff[i] + len[i];
  if (!text && goff[n]) return group_err(g, PJ_ERR_ARG, "pj_group_parse_host: no text");
  group_run(g, [&](int i) {
    DeviceGuard guard(g->devs[i]);
    pj_ctx* c = g->ctx[i];
    pj_group_shard& S = shards[i];
    memset(&S, 0, sizeof S);
    S.global_offset = goff[i];
    /* the bytes behind a shard ARE its slack: the shards are ranges of one buffer */
    const uint64_t behind = goff[n] - goff[i + 1];
    const uint64_t got = slack < behind ? slack : behind;
    S.slack_bytes = got;
    S.status = parse_impl(c, schema, PJ_FRAMING_NDJSON, text + goff[i], len[i], got, goff[i] == 0, got == behind, goff[i], PJ_MEM_HOST, &out[i]);
    unsigned long long* row = g->h_table[0] + (size_t)i * PJ_GROUP_NCOUNT;
    memset(row, 0, sizeof(unsigned long long) * PJ_GROUP_NCOUNT);
    if (S.status == PJ_OK || S.status == PJ_ERR_CAPACITY) {
      /* a call in pieces leaves its totals in the result block of the last piece; errors were added up on the host */
      const uint32_t last = c->stats.pieces ? c->stats.pieces - 1 : 0;
      group_host_row(c->h_res[last < 16 ? last : 15], len[i] ? len[i] : ~0ull, row);
      row[PJ_GC_ERRORS] = out[i].n_errors;
    }
    g->rendezvous.meet((uint32_t)n);
    const auto t0 = std::chrono::steady_clock::now();
    const pj_status gs = group_gather(g, i, 0, 0, true); /* the device tables from the host table: the result blocks hold per-piece figures */
    S.gather_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (S.status == PJ_OK) S.status = gs;
  });
  pj_status st = PJ_OK;
  group_fill(g, shards, false);
  for (int i = 0; i < n; ++i) if (shards[i].bytes == ~0ull) shards[i].bytes = 0;
  for (int i = 0; i < n && st == PJ_OK; ++i) if (shards[i].status != PJ_OK) { st = shards[i].status; group_err(g, st, "shard %d: %s", i, pj_last_error(g->ctx[i])); }
  return st;
}

pj_status pj_group_write(pj_group* g, uint32_t schema, const pj_columns* cols, uint8_t* const* out, const uint64_t* cap, pj_group_shard* shards) {
  if (!g) return PJ_ERR_ARG;
  if (!cols || !out || !cap || !shards || schema < PJ_SCHEMA_PET || schema > PJ_SCHEMA_MIXED) return group_err(g, PJ_ERR_ARG, "pj_group_write: bad argument");
  const int n = g->ndev;
  group_run(g, [&](int i) {
    DeviceGuard guard(g->devs[i]);
    pj_ctx* c = g->ctx[i];
    pj_group_shard& S = shards[i];
    memset(&S, 0, sizeof S);
    uint64_t out_len = 0;
    S.status = pj_write(c, schema, PJ_FRAMING_NDJSON, &cols[i], out[i], cap[i], PJ_MEM_DEVICE, &out_len);
    if (S.status != PJ_OK && S.status != PJ_ERR_CAPACITY) { cudaMemsetAsync(c->d_res, 0, sizeof(DevResult), c->stream); memset(c->h_res, 0, sizeof(DevResult)); }
    group_host_row(c->h_res[0], 0, g->h_table[0] + (size_t)i * PJ_GROUP_NCOUNT);
    g->rendezvous.meet((uint32_t)n); /* the exchange, once no shard allocates any more (see pj_group_parse) */
    const auto t0 = std::chrono::steady_clock::now();
    const pj_status gs = group_gather(g, i, 0, 0);
    S.gather_ms = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (S.status == PJ_OK) S.status = gs;
  });
  pj_status st = PJ_OK;
  group_fill(g, shards, true);
  for (int i = 0; i < n && st == PJ_OK; ++i) if (shards[i].status != PJ_OK) { st = shards[i].status; group_err(g, st, "shard %d: %s", i, pj_last_error(g->ctx[i])); }
  return st;
}

}  // extern "C"
