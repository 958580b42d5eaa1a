/*
 * pj_index.cuh — small host/device helpers shared by the record-index kernels and the set-up code:
 * the "is this line a record" test of NDJSON framing and the per-schema list of output columns
 * with the counter that sizes each of them.
 */
#ifndef PJ_INDEX_CUH
#define PJ_INDEX_CUH

#include "pj_core.cuh"

namespace pj {

/* NDJSON: p is the first byte of a line (byte 0 of the stream or the byte after an LF). The line is
 * a record unless it holds only space / tab / CR. A line that runs into the end of the readable
 * bytes without showing anything but blanks is a record only when the stream continues there (it
 * then fails with PJ_E_TOO_LONG), and nothing when the stream ends. */
PJ_HD bool nd_is_record(const uint8_t* in, uint64_t p, uint64_t limit, int is_last) {
  uint64_t t = p;
  for (; t < limit; ++t) {
    uint32_t x = ld_byte(in + t);
    if (x == ' ' || x == '\t' || x == '\r') continue;
    return x != '\n';
  }
  return !is_last;
}

/* One output column of a schema: element width, the counter slot that gives its row count (0xFF:
 * one row per record) and, for offset columns, the slot whose total is stored as the closing
 * entry [rows]. */
struct FinalizeItem {
  uint8_t col, elem, rows_slot, sentinel_slot;
};
struct FinalizePlan {
  uint32_t n;
  FinalizeItem item[48];
};

inline void plan_add(FinalizePlan* p, int col, int elem, int rows_slot, int sentinel_slot) {
  FinalizeItem it;
  it.col = (uint8_t)col; it.elem = (uint8_t)elem; it.rows_slot = (uint8_t)rows_slot; it.sentinel_slot = (uint8_t)sentinel_slot;
  p->item[p->n++] = it;
}
inline void plan_object(const Schema& S, const ObjDesc& O, int rows_slot, FinalizePlan* p) {
  plan_add(p, O.present_col, 1, rows_slot, 0xFF);
  for (int i = 0; i < (int)O.nfields; ++i) {
    const FieldDesc& F = O.f[i];
    switch (F.kind) {
      case K_I64: plan_add(p, F.col, 8, rows_slot, 0xFF); break;
      case K_I32: plan_add(p, F.col, 4, rows_slot, 0xFF); break;
      case K_BOOL:
      case K_ENUM: plan_add(p, F.col, 1, rows_slot, 0xFF); break;
      case K_DATETIME:
        plan_add(p, F.col, 8, rows_slot, 0xFF);
        plan_add(p, F.col + 1, 4, rows_slot, 0xFF);
        plan_add(p, F.col + 2, 4, rows_slot, 0xFF);
        break;
      case K_STR:
        plan_add(p, F.col, 4, rows_slot, F.cnt);
        plan_add(p, F.col + 1, 1, F.cnt, 0xFF);
        break;
      case K_OBJ: plan_object(S, S.obj[F.child], rows_slot, p); break;
      case K_LIST_STR:
        plan_add(p, F.col, 4, rows_slot, F.cnt);
        plan_add(p, F.col + 1, 4, F.cnt, F.cnt + 1);
        plan_add(p, F.col + 2, 1, F.cnt + 1, 0xFF);
        break;
      case K_LIST_OBJ:
        plan_add(p, F.col, 4, rows_slot, F.cnt);
        plan_object(S, S.obj[F.child], F.cnt, p);
        break;
      default: break;
    }
  }
}
/* Model-table columns of `schema` (the per-record columns REC_START .. REC_ROW are not listed). */
inline void build_finalize_plan(const Schema& S, uint32_t schema, FinalizePlan* p) {
  p->n = 0;
  bool mixed = schema == PJ_SCHEMA_MIXED;
  if (schema == PJ_SCHEMA_PET || mixed) plan_object(S, S.obj[OBJ_PET], mixed ? (int)SLOT_ROWS_PET : 0xFF, p);
  if (schema == PJ_SCHEMA_ORDER || mixed) plan_object(S, S.obj[OBJ_ORDER], mixed ? (int)SLOT_ROWS_ORD : 0xFF, p);
  if (schema == PJ_SCHEMA_USER || mixed) plan_object(S, S.obj[OBJ_USER], mixed ? (int)SLOT_ROWS_USR : 0xFF, p);
}

}  // namespace pj
#endif
