/*
 * pj_stream.cuh — geometry and line index of the single-pass NDJSON kernel (k_parse_stream, pj_stream_kernel.cuh),
 * as host + device functions so that the same code is exercised on the CPU by the host emulation of the tests.
 *
 * A shard of `len` owned bytes (plus slack) is cut into tiles of `tile_bytes` bytes, counted from the 16-byte
 * aligned address at or below the first input byte. One thread block takes one tile:
 *   - it stages ST_WIN_BYTES bytes starting at the tile's first byte in shared memory (tile + at least 2 KiB of
 *     what follows, so that the records which begin in the tile usually end inside the window);
 *   - every thread looks at ST_CPT consecutive 16-byte chunks of the window and builds their line-feed masks;
 *   - the masks are compacted into the list of line starts of the window. A tile OWNS the lines whose preceding
 *     line feed lies in the tile (and, in the first tile of a first shard, the line at byte 0): the same rule
 *     that assigns records to shards, so tiles, pieces and shards compose;
 *   - thread j takes owned line j: it is a record unless it holds only blanks.
 */
#ifndef PJ_STREAM_CUH
#define PJ_STREAM_CUH

#include "pj_core.cuh"
#include "pj_index.cuh"

namespace pj {

static constexpr uint32_t ST_THREADS = 256;
static constexpr uint32_t ST_CPT = 15; /* 16-byte chunks per thread; odd, so that 128-bit loads at this stride are free of bank conflicts */
static constexpr uint32_t ST_CHUNKS = ST_THREADS * ST_CPT;
static constexpr uint32_t ST_WIN_BYTES = ST_CHUNKS * 16; /* 34816 bytes staged per tile */
static constexpr uint32_t ST_WIN_PAD = 48;               /* line feeds behind the staged bytes: look-ahead never leaves the window */
static constexpr uint32_t ST_MAX_TILE_BYTES = ST_WIN_BYTES - 2048; /* leaves 2 KiB of the window for records that run past the tile */
static constexpr uint32_t ST_MIN_TILE_BYTES = 1024;
static constexpr uint32_t ST_LF_CAP = ST_THREADS + 64;     /* line starts kept per batch: the owned ones and what follows */
static constexpr uint32_t ST_NONE = 0xFFFFFFFFu;

/* Where a tile lies. Offsets named v* count from the aligned base (input offset + mis); window offsets count from
 * the tile's first byte. */
struct StreamGeom {
  uint64_t v0;         /* the tile's first byte */
  uint64_t vlimit;     /* first unreadable byte (limit + mis) */
  uint32_t mis;        /* input address & 15 */
  uint32_t lo_valid;   /* window bytes below it are not input (first tile only: mis) */
  uint32_t hi_valid;   /* window bytes at or above it are not input (padding) */
  uint32_t own_end;    /* line feeds at window offsets below it belong to this tile */
  uint32_t copy_bytes; /* multiple of 16: what the bulk copy brings */
  uint32_t to_limit;   /* the window reaches the end of the readable bytes */
};
PJ_HD StreamGeom stream_geom(uint32_t mis, uint64_t len, uint64_t limit, uint32_t tile_bytes, uint32_t tile) {
  StreamGeom g;
  g.mis = mis;
  g.v0 = (uint64_t)tile * tile_bytes;
  g.vlimit = limit + mis;
  const uint64_t vlen = len + mis; /* line feeds below it are the shard's own */
  const uint64_t left = g.vlimit > g.v0 ? g.vlimit - g.v0 : 0;
  g.hi_valid = left < ST_WIN_BYTES ? (uint32_t)left : ST_WIN_BYTES;
  g.to_limit = left <= ST_WIN_BYTES;
  g.copy_bytes = (g.hi_valid + 15u) & ~15u;
  g.lo_valid = tile == 0 ? mis : 0;
  const uint64_t own = vlen > g.v0 ? vlen - g.v0 : 0;
  g.own_end = own < tile_bytes ? (uint32_t)own : tile_bytes;
  return g;
}
/* tiles of a shard: they cover the owned bytes; a first shard has at least one, for the line at byte 0 */
PJ_HD uint64_t stream_tiles(uint32_t mis, uint64_t len, uint32_t is_first, uint32_t tile_bytes) {
  uint64_t n = (len + mis + tile_bytes - 1) / tile_bytes;
  if (len == 0) n = 0;
  if (is_first && n == 0) n = 1;
  return n;
}

/* bit b set = byte b of the 16 bytes (four little-endian words) is a line feed */
PJ_HD uint32_t lf_mask16(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
  uint32_t m = 0;
  const uint32_t w[4] = {w0, w1, w2, w3};
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
  for (int j = 0; j < 4; ++j) {
    const uint32_t t = w[j] ^ 0x0A0A0A0Au;
    const uint32_t nz = ((t & 0x7F7F7F7Fu) + 0x7F7F7F7Fu) | t; /* bit 7 of a byte set = the byte is not a line feed */
    const uint32_t f = (~nz & 0x80808080u) >> 7;              /* bit 0 of a byte set = it is */
    m |= (((f * 0x00204081u) >> 21) & 0xFu) << (4 * j);       /* the four flags side by side */
  }
  return m;
}
/* line-feed mask of the chunk at window offset off (a multiple of 16), bytes outside the input cleared */
PJ_HD uint32_t stream_chunk_mask(const uint8_t* win, uint32_t off, const StreamGeom& g) {
  if (off >= g.hi_valid) return 0;
  const uint32_t* q = reinterpret_cast<const uint32_t*>(win + off);
  uint32_t m = lf_mask16(q[0], q[1], q[2], q[3]);
  if (off < g.lo_valid) m &= g.lo_valid - off >= 16 ? 0u : (0xFFFFu << (g.lo_valid - off));
  if (g.hi_valid - off < 16) m &= (1u << (g.hi_valid - off)) - 1u;
  return m;
}
/* of the chunk's line feeds, those the tile owns */
PJ_HD uint32_t stream_own_bits(uint32_t m, uint32_t off, const StreamGeom& g) {
  if (off >= g.own_end) return 0;
  return g.own_end - off >= 16 ? m : (m & ((1u << (g.own_end - off)) - 1u));
}

/* Line j of the list (window offset s of its first byte): a record, or a line of blanks?
 * Mirrors nd_is_record(): a blank line that runs into the end of the readable bytes is a record only when the
 * stream continues there. `in` (the shard's bytes) is consulted only when the blanks reach the end of a
 * window that does not reach the end of the readable bytes. */
PJ_HD bool stream_is_record(const uint8_t* win, uint32_t s, const StreamGeom& g, const uint8_t* in, uint64_t limit, int is_last) {
  uint32_t q = s;
  for (;;) {
    const uint32_t x = win[q]; /* the padding behind the window is line feeds, so this ends */
    if (x == ' ' || x == '\t' || x == '\r') { ++q; continue; }
    if (x != '\n') return true;
    if (q < g.hi_valid) return false; /* a real line feed: the line is blank */
    if (g.to_limit) return !is_last;
    return nd_is_record(in, g.v0 + q - g.mis, limit, is_last);
  }
}

}  // namespace pj
#endif
