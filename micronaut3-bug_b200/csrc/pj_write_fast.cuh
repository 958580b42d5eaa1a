/*
 * pj_write_fast.cuh — columns -> JSON text for one record, instantiated on the compile-time model
 * tables of pj_schema.h. Same text, byte for byte, as write_record() of pj_write_core.cuh (rules W1-W5);
 * what differs is how it gets there: property names, kinds and columns are template constants, so a
 * record is a straight line of loads and stores; `"name":` is stored from immediates; integers are
 * converted in 8-digit groups with 32-bit arithmetic; strings without a byte to escape are copied
 * four bytes per load.
 */
#ifndef PJ_WRITE_FAST_CUH
#define PJ_WRITE_FAST_CUH

#include "pj_fast.cuh"
#include "pj_write_core.cuh"

namespace pj {

/* number of decimal digits of x < 10^8 (1 for 0) */
PJ_HD uint32_t ndigits8(uint32_t x) {
  return 1u + (x >= 10u) + (x >= 100u) + (x >= 1000u) + (x >= 10000u) + (x >= 100000u) + (x >= 1000000u) + (x >= 10000000u);
}
/* the n lowest decimal digits of x at dst, most significant first */
PJ_HD void put_digits(uint8_t* dst, uint32_t x, uint32_t n) {
  for (uint32_t i = n; i-- > 0;) { const uint32_t q = x / 10u; dst[i] = (uint8_t)('0' + (x - q * 10u)); x = q; }
}
PJ_HD void put_digits8(uint8_t* dst, uint32_t x) {
#pragma unroll
  for (int i = 7; i >= 0; --i) { const uint32_t q = x / 10u; dst[i] = (uint8_t)('0' + (x - q * 10u)); x = q; }
}
PJ_HD uint32_t ndigits_u64(uint64_t u) {
  if (u < 100000000ull) return ndigits8((uint32_t)u);
  if (u < 10000000000000000ull)
    return 9u + (u >= 1000000000ull) + (u >= 10000000000ull) + (u >= 100000000000ull) + (u >= 1000000000000ull) +
           (u >= 10000000000000ull) + (u >= 100000000000000ull) + (u >= 1000000000000000ull);
  return 17u + (u >= 100000000000000000ull) + (u >= 1000000000000000000ull) + (u >= 10000000000000000000ull);
}
template <bool WR>
PJ_HD void fput_u64(WOut& w, uint64_t u) {
  if (!WR) { w.n += ndigits_u64(u); return; }
  const uint64_t q1 = u / 100000000ull; /* < 1.85e11 */
  const uint32_t lo = (uint32_t)(u - q1 * 100000000ull);
  const uint32_t hi = (uint32_t)(q1 / 100000000ull); /* <= 1844 */
  const uint32_t mid = (uint32_t)(q1 - (uint64_t)hi * 100000000ull);
  const uint32_t lead = hi ? hi : (mid ? mid : lo), groups = hi ? 2u : (mid ? 1u : 0u); /* full 8-digit groups after the leading one */
  const uint32_t nl = ndigits8(lead);
  if (WR) {
    uint8_t* d = w.dst + w.n;
    put_digits(d, lead, nl);
    if (groups == 2) { put_digits8(d + nl, mid); put_digits8(d + nl + 8, lo); }
    else if (groups == 1) put_digits8(d + nl, lo);
  }
  w.n += nl + 8 * groups;
}
template <bool WR>
PJ_HD void fput_i64(WOut& w, int64_t v) {
  if (v < 0) { wput<WR>(w, '-'); fput_u64<WR>(w, 0 - (uint64_t)v); }
  else fput_u64<WR>(w, (uint64_t)v);
}
/* len bytes held in (w0, w1), lowest byte first; len is a constant at every call, so the loop unrolls into immediates */
template <bool WR>
PJ_HD void fput_const(WOut& w, uint64_t w0, uint64_t w1, uint32_t len) {
  if (WR) {
#pragma unroll
    for (uint32_t i = 0; i < 16; ++i)
      if (i < len) w.dst[w.n + i] = (uint8_t)((i < 8 ? w0 >> (8 * i) : w1 >> (8 * (i - 8))) & 0xFF);
  }
  w.n += len;
}

/* n bytes from s (global memory) to d, four at a time: d is brought to a 4-byte boundary, the source is then
 * read as aligned words and shifted into place. Reads stay inside the aligned words that hold the n bytes. */
PJ_HD void copy_bytes_fast(uint8_t* d, const uint8_t* s, uint32_t n) {
  while (n && ((uintptr_t)d & 3u)) { *d++ = (uint8_t)ld_byte(s++); n--; }
  if (n >= 4) {
    const uint32_t sh = (uint32_t)((uintptr_t)s & 3u) * 8u;
    const uint32_t* sw = reinterpret_cast<const uint32_t*>((uintptr_t)s & ~(uintptr_t)3);
    if (sh == 0) {
      for (; n >= 16; n -= 16) { /* four loads in flight, then four stores */
        const uint32_t a0 = sw[0], a1 = sw[1], a2 = sw[2], a3 = sw[3];
        uint32_t* dw = reinterpret_cast<uint32_t*>(d);
        dw[0] = a0; dw[1] = a1; dw[2] = a2; dw[3] = a3;
        sw += 4; d += 16; s += 16;
      }
      for (; n >= 4; n -= 4) { *reinterpret_cast<uint32_t*>(d) = *sw++; d += 4; s += 4; }
    } else {
      uint32_t x0 = *sw++;
      for (; n >= 16; n -= 16) { /* the four words that hold the next 16 bytes, loaded together */
        const uint32_t a1 = sw[0], a2 = sw[1], a3 = sw[2], a4 = sw[3];
        uint32_t* dw = reinterpret_cast<uint32_t*>(d);
#if defined(__CUDA_ARCH__)
        dw[0] = __funnelshift_r(x0, a1, sh); dw[1] = __funnelshift_r(a1, a2, sh); dw[2] = __funnelshift_r(a2, a3, sh); dw[3] = __funnelshift_r(a3, a4, sh);
#else
        dw[0] = (x0 >> sh) | (a1 << (32 - sh)); dw[1] = (a1 >> sh) | (a2 << (32 - sh)); dw[2] = (a2 >> sh) | (a3 << (32 - sh)); dw[3] = (a3 >> sh) | (a4 << (32 - sh));
#endif
        x0 = a4; sw += 4; d += 16; s += 16;
      }
      for (; n >= 4; n -= 4) {
        const uint32_t x1 = *sw++;
#if defined(__CUDA_ARCH__)
        *reinterpret_cast<uint32_t*>(d) = __funnelshift_r(x0, x1, sh);
#else
        *reinterpret_cast<uint32_t*>(d) = (x0 >> sh) | (x1 << (32 - sh));
#endif
        x0 = x1; d += 4; s += 4;
      }
    }
  }
  while (n) { *d++ = (uint8_t)ld_byte(s++); n--; }
}

/* W3 with the common case first: the string has no byte to escape. PLAIN: the caller knows that no string
 * of the column set has a byte to escape, so lengths need no look at the bytes and the copy needs no checks. */
template <bool WR, bool PLAIN>
PJ_HD void fput_str(WOut& w, const uint8_t* s, uint32_t n) {
  if (PLAIN) {
    if (WR) { w.dst[w.n] = '"'; copy_bytes_fast(w.dst + w.n + 1, s, n); w.dst[w.n + 1 + n] = '"'; }
    w.n += 2 + (uint64_t)n;
    return;
  }
  if (!WR) { w.n += 2 + (uint64_t)n + str_escape_extra(s, n); return; }
  uint8_t* d = w.dst + w.n;
  *d++ = '"';
  uint32_t i = 0;
  bool plain = true;
  while (i < n && ((uintptr_t)(s + i) & 3u)) {
    const uint32_t c = ld_byte(s + i);
    if (escape_extra_byte(c)) { plain = false; break; }
    *d++ = (uint8_t)c; ++i;
  }
  if (plain) {
    for (; i + 4 <= n; i += 4) {
      const uint32_t x = *reinterpret_cast<const uint32_t*>(s + i);
      const uint32_t xq = x ^ 0x22222222u, xb = x ^ 0x5C5C5C5Cu;
      const uint32_t m = ((x - 0x20202020u) & ~x) | ((xq - 0x01010101u) & ~xq) | ((xb - 0x01010101u) & ~xb);
      if (m & 0x80808080u) { plain = false; break; }
      d[0] = (uint8_t)x; d[1] = (uint8_t)(x >> 8); d[2] = (uint8_t)(x >> 16); d[3] = (uint8_t)(x >> 24);
      d += 4;
    }
  }
  if (plain) {
    for (; i < n; ++i) {
      const uint32_t c = ld_byte(s + i);
      if (escape_extra_byte(c)) { plain = false; break; }
      *d++ = (uint8_t)c;
    }
  }
  w.n = (uint64_t)(d - w.dst);
  if (!plain) {
    /* the rest byte by byte, with the escapes of W3 */
    for (; i < n; ++i) {
      const uint32_t c = ld_byte(s + i);
      if (c >= 0x20 && c != '"' && c != '\\') { wput<WR>(w, c); continue; }
      wput<WR>(w, '\\');
      switch (c) {
        case '"': wput<WR>(w, '"'); break;
        case '\\': wput<WR>(w, '\\'); break;
        case 8: wput<WR>(w, 'b'); break;
        case 9: wput<WR>(w, 't'); break;
        case 10: wput<WR>(w, 'n'); break;
        case 12: wput<WR>(w, 'f'); break;
        case 13: wput<WR>(w, 'r'); break;
        default:
          wput<WR>(w, 'u'); wput<WR>(w, '0'); wput<WR>(w, '0');
          wput<WR>(w, '0' + (c >> 4));
          wput<WR>(w, (c & 15) < 10 ? '0' + (c & 15) : w.hexa + (c & 15) - 10);
          break;
      }
    }
  }
  wput<WR>(w, '"');
}

template <bool WR, int E, int I = 0>
PJ_HD void fput_enum(WOut& w, uint32_t e) {
  if constexpr (I < CEnum<E>::N) {
    if (e == I) { wput<WR>(w, '"'); fput_const<WR>(w, EK<E, I>::lo, EK<E, I>::hi, EK<E, I>::len); wput<WR>(w, '"'); }
    else fput_enum<WR, E, I + 1>(w, e);
  }
}

template <bool WR, bool PLAIN, int OBJ, int LEVEL>
PJ_HD void fwrite_object(const DevCols* c, uint64_t row, int incl, WOut& w);

/* a hint to start fetching the line at p (nothing on the host) */
PJ_HD void wr_prefetch(const void* p) {
#if defined(__CUDA_ARCH__)
  asm volatile("prefetch.global.L1 [%0];" ::"l"(p));
#else
  (void)p;
#endif
}
/* the scalar columns of flat object E (a list element) at `row` */
template <int E, int I = 0>
PJ_HD void wr_prefetch_row(const DevCols* c, uint64_t row) {
  if constexpr (I == 0) wr_prefetch(colp<uint8_t>(c, CObj<E>::present_col) + row);
  if constexpr (I < CObj<E>::N) {
    constexpr uint32_t kind = FK<E, I>::kind, col = FK<E, I>::col;
    if constexpr (kind == K_I64) wr_prefetch(colp<int64_t>(c, col) + row);
    else if constexpr (kind == K_I32 || kind == K_STR) wr_prefetch(colp<uint32_t>(c, col) + row);
    else if constexpr (kind == K_BOOL || kind == K_ENUM) wr_prefetch(colp<uint8_t>(c, col) + row);
    wr_prefetch_row<E, I + 1>(c, row);
  }
}

/* Every row-indexed value of one object, loaded before any of them is used: the loads are issued back to back and
 * their latencies overlap, instead of one load per property each waiting behind the stores of the one before.
 * Indexed with constants only, so it lives in registers. */
struct RowSnap {
  int64_t v[8];       /* I64 / I32 / BOOL / ENUM value, DATETIME seconds */
  uint32_t a[8], b[8]; /* STR / LIST offsets of the row and of the next one; DATETIME nanos and offset */
  uint32_t present;
};
template <int OBJ, int I = 0>
PJ_HD void snap_row(const DevCols* c, uint64_t row, RowSnap& r) {
  if constexpr (I == 0) r.present = colp<uint8_t>(c, CObj<OBJ>::present_col)[row];
  if constexpr (I < CObj<OBJ>::N) {
    constexpr uint32_t kind = FK<OBJ, I>::kind, col = FK<OBJ, I>::col;
    if constexpr (kind == K_I64) r.v[I] = colp<int64_t>(c, col)[row];
    else if constexpr (kind == K_I32) r.v[I] = colp<int32_t>(c, col)[row];
    else if constexpr (kind == K_BOOL || kind == K_ENUM) r.v[I] = colp<uint8_t>(c, col)[row];
    else if constexpr (kind == K_DATETIME) {
      r.v[I] = colp<int64_t>(c, col)[row];
      r.a[I] = (uint32_t)colp<int32_t>(c, col + 1)[row]; r.b[I] = (uint32_t)colp<int32_t>(c, col + 2)[row];
    } else if constexpr (kind == K_STR || kind == K_LIST_STR || kind == K_LIST_OBJ) {
      r.a[I] = colp<uint32_t>(c, col)[row]; r.b[I] = colp<uint32_t>(c, col)[row + 1];
    }
    snap_row<OBJ, I + 1>(c, row, r);
  }
}

/* property I of OBJ and, by recursion, the ones after it */
template <bool WR, bool PLAIN, int OBJ, int LEVEL, int I = 0>
PJ_HD void fwrite_fields(const DevCols* c, uint64_t row, int incl, const RowSnap& r, bool& first, WOut& w) {
  if constexpr (I < CObj<OBJ>::N) {
    constexpr uint32_t kind = FK<OBJ, I>::kind, col = FK<OBJ, I>::col;
    const bool pr = (r.present >> I) & 1;
    bool empty = false;
    uint32_t a = 0, b = 0;
    if constexpr (kind == K_STR || kind == K_LIST_STR || kind == K_LIST_OBJ) {
      a = r.a[I]; b = r.b[I];
      empty = a == b;
      if constexpr (!WR && PLAIN) {
        /* the measuring pass does not look at string bytes or child rows here: ask for them now, the writing pass
           that follows finds them on their way */
        if (a < b) {
          if constexpr (kind == K_STR) wr_prefetch(colp<uint8_t>(c, col + 1) + a);
          else if constexpr (kind == K_LIST_STR) wr_prefetch(colp<uint8_t>(c, col + 2) + colp<uint32_t>(c, col + 1)[a]);
          else if constexpr (LEVEL == 0) wr_prefetch_row<FK<OBJ, I>::child>(c, a);
        }
      }
    }
    if (included(incl, pr, empty)) {
      if (!first) wput<WR>(w, ',');
      first = false;
      fput_const<WR>(w, FK<OBJ, I>::pat0, FK<OBJ, I>::pat1, FK<OBJ, I>::pat_len); /* "name": */
      if (!pr) fput_const<WR>(w, 0x6C6C756Eull, 0, 4); /* null */
      else if constexpr (kind == K_I64 || kind == K_I32) fput_i64<WR>(w, r.v[I]);
      else if constexpr (kind == K_BOOL) {
        if (r.v[I]) fput_const<WR>(w, 0x65757274ull, 0, 4); else fput_const<WR>(w, 0x65736C6166ull, 0, 5);
      } else if constexpr (kind == K_ENUM) {
        constexpr int E = FK<OBJ, I>::child;
        fput_enum<WR, E>(w, (uint32_t)r.v[I] % (uint32_t)CEnum<E>::N);
      } else if constexpr (kind == K_DATETIME) {
        wput_datetime<WR>(w, r.v[I], (int32_t)r.a[I], (int32_t)r.b[I]);
      } else if constexpr (kind == K_STR) {
        fput_str<WR, PLAIN>(w, colp<uint8_t>(c, col + 1) + a, b - a);
      } else if constexpr (kind == K_OBJ) {
        if constexpr (LEVEL == 0) fwrite_object<WR, PLAIN, FK<OBJ, I>::child, 1>(c, row, incl, w);
      } else if constexpr (kind == K_LIST_STR) {
        const uint32_t* so = colp<uint32_t>(c, col + 1);
        const uint8_t* data = colp<uint8_t>(c, col + 2);
        if constexpr (!WR && PLAIN) {
          /* brackets, and per string two quotes and (but for the first) a comma */
          w.n += 2 + (a < b ? (uint64_t)(so[b] - so[a]) + 3ull * (b - a) - 1 : 0);
        } else {
        wput<WR>(w, '[');
        uint32_t s0 = a < b ? so[a] : 0;
        for (uint32_t k = a; k < b; ++k) {
          if (k > a) wput<WR>(w, ',');
          const uint32_t s1 = so[k + 1];
          fput_str<WR, PLAIN>(w, data + s0, s1 - s0);
          s0 = s1;
        }
        wput<WR>(w, ']');
        }
      } else if constexpr (kind == K_LIST_OBJ) {
        wput<WR>(w, '[');
        if constexpr (LEVEL == 0)
          for (uint32_t k = a; k < b; ++k) { if (k > a) wput<WR>(w, ','); fwrite_object<WR, PLAIN, FK<OBJ, I>::child, 1>(c, k, incl, w); }
        wput<WR>(w, ']');
      }
    }
    fwrite_fields<WR, PLAIN, OBJ, LEVEL, I + 1>(c, row, incl, r, first, w);
  }
}
/* LEVEL 0: model root; LEVEL 1: Category / Tag */
template <bool WR, bool PLAIN, int OBJ, int LEVEL>
PJ_HD void fwrite_object(const DevCols* c, uint64_t row, int incl, WOut& w) {
  RowSnap r;
  snap_row<OBJ>(c, row, r);
  bool first = true;
  wput<WR>(w, '{');
  fwrite_fields<WR, PLAIN, OBJ, LEVEL>(c, row, incl, r, first, w);
  wput<WR>(w, '}');
}

template <bool WR, bool PLAIN>
PJ_HD void fwrite_record(const DevCols* c, uint32_t type, uint64_t row, int incl, WOut& w) {
  if (type == PJ_TYPE_PET) fwrite_object<WR, PLAIN, OBJ_PET, 0>(c, row, incl, w);
  else if (type == PJ_TYPE_ORDER) fwrite_object<WR, PLAIN, OBJ_ORDER, 0>(c, row, incl, w);
  else fwrite_object<WR, PLAIN, OBJ_USER, 0>(c, row, incl, w);
}

}  // namespace pj
#endif
