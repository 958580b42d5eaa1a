/*
 * pj_schema.h — compiled form of the validated models (petstore.json:823-972) as plain tables that
 * both the host set-up code and the kernels read.
 *
 * A model is an object descriptor: an ordered list of properties, each with its JSON name packed
 * into two little-endian 64-bit words (names are at most 16 bytes), its kind, the column that
 * receives the value and, for variable-size values, the counter slot that sizes its arena.
 */
#ifndef PJ_SCHEMA_H
#define PJ_SCHEMA_H

#include <stdint.h>

#include "petjson.h"

namespace pj {

enum Kind : uint8_t {
  K_I64 = 0,      /* col: i64 */
  K_I32 = 1,      /* col: i32 */
  K_BOOL = 2,     /* col: u8 */
  K_STR = 3,      /* col: _OFF (u32), col+1: _DATA; cnt: byte counter slot */
  K_ENUM = 4,     /* col: u8; child: enum table */
  K_DATETIME = 5, /* col: epoch i64, col+1: nanos i32, col+2: offset i32 */
  K_OBJ = 6,      /* child: object descriptor (flat), rows shared with the parent */
  K_LIST_STR = 7, /* col: list _OFF, col+1: string _OFF, col+2: _DATA; cnt: item counter, cnt+1: bytes */
  K_LIST_OBJ = 8  /* col: list _OFF; cnt: item counter; child: object descriptor (flat) */
};

/* Counter slots: one running total per variable-size output. */
enum Slot : uint32_t {
  SLOT_ROWS_PET = 0, SLOT_ROWS_ORD = 1, SLOT_ROWS_USR = 2, /* model-table rows (mixed streams) */
  SLOT_PET_CAT_NAME = 3, SLOT_PET_NAME = 4, SLOT_PET_PHOTO_CNT = 5, SLOT_PET_PHOTO_BYTES = 6,
  SLOT_PET_TAG_CNT = 7, SLOT_PET_TAG_NAME = 8,
  SLOT_USR_STR0 = 9, /* .. 14: username, firstName, lastName, email, password, phone */
  NSLOT = 15
};

enum ObjId : uint32_t { OBJ_PET = 0, OBJ_CATEGORY = 1, OBJ_TAG = 2, OBJ_ORDER = 3, OBJ_USER = 4, NOBJ = 5 };

struct FieldDesc {
  uint64_t name_lo, name_hi;
  uint8_t name_len, kind, col, cnt, child, pad[3];
};
struct ObjDesc {
  uint8_t nfields, present_col, required_mask, type; /* type: PJ_TYPE_* for model roots, 0 otherwise */
  uint8_t pad[4];
  FieldDesc f[8];
};
struct EnumDesc {
  uint32_t n, pad;
  uint64_t lo[4], hi[4];
  uint32_t len[4];
  char text[4][16];
};
struct Schema {
  ObjDesc obj[NOBJ];
  EnumDesc en[2]; /* 0: Pet.status, 1: Order.status */
  /* per byte-counter slot: the arena column it fills, the item-counter slot that numbers the rows of
   * its offset column (0xFF: one row per record) and whether it belongs to a list of strings */
  uint8_t slot_data_col[NSLOT], slot_rows_slot[NSLOT], slot_is_list_str[NSLOT];
  uint8_t pad[3];
};

/* Device addresses of the caller's columns plus capacities in elements. */
struct DevCols {
  void* ptr[PJ_MAX_COLS];
};

/* ---- host-side construction ----------------------------------------------------------------- */
inline void pack_name(const char* s, uint64_t* lo, uint64_t* hi, uint8_t* len) {
  *lo = 0; *hi = 0;
  uint32_t n = 0;
  for (; s[n]; ++n) {
    if (n < 8) *lo |= (uint64_t)(uint8_t)s[n] << (8 * n);
    else *hi |= (uint64_t)(uint8_t)s[n] << (8 * (n - 8));
  }
  *len = (uint8_t)n;
}
inline FieldDesc mk_field(const char* name, Kind kind, int col, int cnt = 0, int child = 0) {
  FieldDesc f{};
  pack_name(name, &f.name_lo, &f.name_hi, &f.name_len);
  f.kind = kind; f.col = (uint8_t)col; f.cnt = (uint8_t)cnt; f.child = (uint8_t)child;
  return f;
}
inline void mk_enum(EnumDesc* e, const char* a, const char* b, const char* c) {
  const char* lits[3] = {a, b, c};
  e->n = 3;
  for (int i = 0; i < 3; ++i) {
    uint8_t len;
    pack_name(lits[i], &e->lo[i], &e->hi[i], &len);
    e->len[i] = len;
    int k = 0;
    for (; lits[i][k]; ++k) e->text[i][k] = lits[i][k];
    e->text[i][k] = 0;
  }
}

/* ---- the built-in models as compile-time tables ------------------------------------------------
 * The kernels are instantiated on these (every kind, column and slot is a constant in the generated
 * code); build_schema() copies the same tables into the run-time Schema used by the generic parser,
 * the writer and the host. Property order is the specification's (it is also the output order). */
struct CF {
  uint8_t kind, col, cnt, child, len;
  uint64_t lo, hi;
  const char* name;
};
constexpr int c_strlen(const char* s) { int n = 0; while (s[n]) ++n; return n; }
constexpr uint64_t c_pack(const char* s, int from) {
  uint64_t v = 0;
  const int n = c_strlen(s);
  for (int i = 0; i < 8 && from + i < n; ++i) v |= (uint64_t)(uint8_t)s[from + i] << (8 * i);
  return v;
}
constexpr CF cf(const char* name, Kind kind, int col, int cnt = 0, int child = 0) {
  return CF{(uint8_t)kind, (uint8_t)col, (uint8_t)cnt, (uint8_t)child, (uint8_t)c_strlen(name), c_pack(name, 0), c_pack(name, 8), name};
}

template <int OBJ> struct CObj;
template <int E> struct CEnum;
/* The model tables themselves are GENERATED from the OpenAPI definitions (petstore.json:823-972) by the schema
 * compiler, `python -m micronaut3-bug_b200.schemac`; a test regenerates the file and compares it byte for byte. */
#include "pj_schema_models.inc"

template <int OBJ>
inline void copy_obj(Schema* s) {
  ObjDesc& o = s->obj[OBJ];
  o.nfields = (uint8_t)CObj<OBJ>::N; o.present_col = (uint8_t)CObj<OBJ>::present_col;
  o.required_mask = (uint8_t)CObj<OBJ>::required; o.type = (uint8_t)CObj<OBJ>::type;
  for (int i = 0; i < CObj<OBJ>::N; ++i) {
    const CF c = CObj<OBJ>::f[i];
    o.f[i] = mk_field(c.name, (Kind)c.kind, c.col, c.cnt, c.child);
  }
}
inline void build_schema(Schema* s) {
  *s = Schema{};
  copy_obj<OBJ_PET>(s); copy_obj<OBJ_CATEGORY>(s); copy_obj<OBJ_TAG>(s); copy_obj<OBJ_ORDER>(s); copy_obj<OBJ_USER>(s);
  for (uint32_t k = 0; k < NSLOT; ++k) { s->slot_data_col[k] = 0; s->slot_rows_slot[k] = 0xFF; s->slot_is_list_str[k] = 0; }
  for (uint32_t oi = 0; oi < NOBJ; ++oi) {
    const ObjDesc& O = s->obj[oi];
    for (int i = 0; i < (int)O.nfields; ++i) {
      const FieldDesc& F = O.f[i];
      if (F.kind == K_STR) s->slot_data_col[F.cnt] = (uint8_t)(F.col + 1);
      else if (F.kind == K_LIST_STR) { s->slot_data_col[F.cnt + 1] = (uint8_t)(F.col + 2); s->slot_rows_slot[F.cnt + 1] = F.cnt; s->slot_is_list_str[F.cnt + 1] = 1; }
      else if (F.kind == K_LIST_OBJ) {
        const ObjDesc& E = s->obj[F.child];
        for (int q = 0; q < (int)E.nfields; ++q) if (E.f[q].kind == K_STR) s->slot_rows_slot[E.f[q].cnt] = F.cnt;
      }
    }
  }
  mk_enum(&s->en[0], CEnum<0>::lit[0].name, CEnum<0>::lit[1].name, CEnum<0>::lit[2].name);
  mk_enum(&s->en[1], CEnum<1>::lit[0].name, CEnum<1>::lit[1].name, CEnum<1>::lit[2].name);
}

/* Range of counter slots a schema uses. */
inline void slot_range(uint32_t schema, uint32_t* lo, uint32_t* hi) {
  switch (schema) {
    case PJ_SCHEMA_PET: *lo = SLOT_PET_CAT_NAME; *hi = SLOT_USR_STR0; break;
    case PJ_SCHEMA_USER: *lo = SLOT_USR_STR0; *hi = NSLOT; break;
    case PJ_SCHEMA_MIXED: *lo = 0; *hi = NSLOT; break;
    default: *lo = 0; *hi = 0; break;
  }
}

}  // namespace pj
#endif
