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

/* The built-in models. Property order is the specification's (it is also the output order). */
inline void build_schema(Schema* s) {
  *s = Schema{};
  /* Pet — petstore.json:872-922, required name + photoUrls (:873-876) */
  ObjDesc& pet = s->obj[OBJ_PET];
  pet.nfields = 6; pet.present_col = PJ_COL_PET_PRESENT; pet.required_mask = (1u << 2) | (1u << 3); pet.type = PJ_TYPE_PET;
  pet.f[0] = mk_field("id", K_I64, PJ_COL_PET_ID);
  pet.f[1] = mk_field("category", K_OBJ, 0, 0, OBJ_CATEGORY);
  pet.f[2] = mk_field("name", K_STR, PJ_COL_PET_NAME_OFF, SLOT_PET_NAME);
  pet.f[3] = mk_field("photoUrls", K_LIST_STR, PJ_COL_PET_PHOTO_OFF, SLOT_PET_PHOTO_CNT);
  pet.f[4] = mk_field("tags", K_LIST_OBJ, PJ_COL_PET_TAGS_OFF, SLOT_PET_TAG_CNT, OBJ_TAG);
  pet.f[5] = mk_field("status", K_ENUM, PJ_COL_PET_STATUS, 0, 0);
  /* Category — petstore.json:858-871 */
  ObjDesc& cat = s->obj[OBJ_CATEGORY];
  cat.nfields = 2; cat.present_col = PJ_COL_PET_CAT_PRESENT;
  cat.f[0] = mk_field("id", K_I64, PJ_COL_PET_CAT_ID);
  cat.f[1] = mk_field("name", K_STR, PJ_COL_PET_CAT_NAME_OFF, SLOT_PET_CAT_NAME);
  /* Tag — petstore.json:923-936 */
  ObjDesc& tag = s->obj[OBJ_TAG];
  tag.nfields = 2; tag.present_col = PJ_COL_PET_TAG_PRESENT;
  tag.f[0] = mk_field("id", K_I64, PJ_COL_PET_TAG_ID);
  tag.f[1] = mk_field("name", K_STR, PJ_COL_PET_TAG_NAME_OFF, SLOT_PET_TAG_NAME);
  /* Order — petstore.json:937-971 */
  ObjDesc& ord = s->obj[OBJ_ORDER];
  ord.nfields = 6; ord.present_col = PJ_COL_ORD_PRESENT; ord.type = PJ_TYPE_ORDER;
  ord.f[0] = mk_field("id", K_I64, PJ_COL_ORD_ID);
  ord.f[1] = mk_field("petId", K_I64, PJ_COL_ORD_PET_ID);
  ord.f[2] = mk_field("quantity", K_I32, PJ_COL_ORD_QUANTITY);
  ord.f[3] = mk_field("shipDate", K_DATETIME, PJ_COL_ORD_SHIP_EPOCH);
  ord.f[4] = mk_field("status", K_ENUM, PJ_COL_ORD_STATUS, 0, 1);
  ord.f[5] = mk_field("complete", K_BOOL, PJ_COL_ORD_COMPLETE);
  /* User — petstore.json:824-857 */
  ObjDesc& usr = s->obj[OBJ_USER];
  usr.nfields = 8; usr.present_col = PJ_COL_USR_PRESENT; usr.type = PJ_TYPE_USER;
  usr.f[0] = mk_field("id", K_I64, PJ_COL_USR_ID);
  usr.f[1] = mk_field("username", K_STR, PJ_COL_USR_USERNAME_OFF, SLOT_USR_STR0 + 0);
  usr.f[2] = mk_field("firstName", K_STR, PJ_COL_USR_FIRSTNAME_OFF, SLOT_USR_STR0 + 1);
  usr.f[3] = mk_field("lastName", K_STR, PJ_COL_USR_LASTNAME_OFF, SLOT_USR_STR0 + 2);
  usr.f[4] = mk_field("email", K_STR, PJ_COL_USR_EMAIL_OFF, SLOT_USR_STR0 + 3);
  usr.f[5] = mk_field("password", K_STR, PJ_COL_USR_PASSWORD_OFF, SLOT_USR_STR0 + 4);
  usr.f[6] = mk_field("phone", K_STR, PJ_COL_USR_PHONE_OFF, SLOT_USR_STR0 + 5);
  usr.f[7] = mk_field("userStatus", K_I32, PJ_COL_USR_STATUS);
  mk_enum(&s->en[0], "available", "pending", "sold");     /* petstore.json:912-916 */
  mk_enum(&s->en[1], "placed", "approved", "delivered");  /* petstore.json:958-962 */
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
