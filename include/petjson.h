/*
 * petjson.h — C ABI of libpetjson.so: JSON parse + schema validation + re-serialisation of the
 * OpenAPI Petstore models (Pet / Order / User) on one NVIDIA B200 (sm_100a).
 *
 * Every entry point is plain `extern "C"`: pointers, sizes and small POD structs only, so it can
 * be bound from Java (Panama FFM / JNA / JNI), Python ctypes or C++ without any CUDA or torch type
 * in a signature.
 *
 * What this boundary replaces in altro3/micronaut3-bug (paths inside that project):
 *   - io.micronaut.serde.ObjectMapper#readValue as called at
 *     src/main/java/com/micronaut/bug/config/MyEntityConfig.java:34        -> pj_parse / pj_parse_shard
 *   - ObjectMapper.getDefault() at
 *     src/main/java/com/micronaut/bug/service/MyEntityService.java:45      -> pj_create(NULL, ...)
 *   - serialisation of a @Serdeable value on the HTTP response at
 *     src/main/java/com/micronaut/bug/controller/MyEntityController.java:48-51 -> pj_write
 *   - strict parser configuration (no comments) at
 *     src/main/resources/application.yml:23-28                              -> always on, no switch
 *   - the validated schemas petstore.json:823-972 (Pet, Category, Tag, Order, User)
 *                                                                          -> PJ_SCHEMA_* and PJ_COL_*
 *
 * There is no CPU implementation behind these calls: a machine without a usable CUDA device gets
 * PJ_ERR_CUDA from pj_create.
 *
 * ---------------------------------------------------------------------------------------------
 * Data model
 * ---------------------------------------------------------------------------------------------
 * A *record* is one JSON object. Two framings are understood:
 *   PJ_FRAMING_NDJSON  one record per line. A record's extent is the bytes between raw LF (0x0A)
 *                      bytes; lines holding only space / tab / CR are skipped and not counted.
 *   PJ_FRAMING_ARRAY   one top-level JSON array `[rec, rec, ...]`. Brackets and commas are counted
 *                      outside strings only; a record's extent is the bytes between the opening
 *                      `[`, the commas at nesting depth 1 and the `]` that returns to depth 0.
 *                      `[]` holds no record; any other extent without a value is a record failing
 *                      with PJ_E_SYNTAX at the separator that ends it. A non-blank byte outside
 *                      the array is reported once per document as (PJ_E_SYNTAX, offset) in
 *                      pj_columns.doc_err_*; input that ends inside the array as (PJ_E_EOF, len).
 * Parsing turns records into *typed columns* (struct of arrays) plus string arenas, Arrow style:
 * a string column is an `_OFF` array of rows+1 uint32 byte offsets into a `_DATA` arena of decoded
 * (un-escaped) UTF-8; a list column is an `_OFF` array of rows+1 uint32 child indices.
 * Per-record validation failures are DATA, not call failures: PJ_COL_ERR_KIND / PJ_COL_ERR_OFF.
 *
 * ---------------------------------------------------------------------------------------------
 * Parsing and validation rules (the contract shared with the CPU checker used by the tests)
 * ---------------------------------------------------------------------------------------------
 * The rules describe a streaming parser that reads a record's extent [s, e) left to right and
 * stops at the FIRST failure it detects; offsets are relative to s (PJ_COL_REC_START).
 *  R1  Whitespace between tokens: space, tab, CR (and LF in array framing). Input is strict
 *      RFC 8259: comments, trailing commas, single quotes, NaN/Infinity, leading zeros and a
 *      leading '+' are PJ_E_SYNTAX at the first offending byte.
 *  R2  Whenever the extent ends while a token or structure is incomplete: PJ_E_EOF at offset e-s.
 *  R3  The record must be an object: another JSON value start (`"` `-` digit `[` t f n) is
 *      PJ_E_TYPE at that byte, anything else PJ_E_SYNTAX. After the closing brace only whitespace
 *      may follow (else PJ_E_SYNTAX at the first such byte).
 *  R4  Keys are compared after un-escaping, by exact name, in any order. Unknown keys are skipped
 *      with full syntactic validation of their value (nesting inside a skipped value is limited to
 *      64 levels: PJ_E_DEPTH at the bracket that would exceed it). A repeated key replaces the
 *      earlier occurrence completely ("last wins").
 *  R5  A value's type is judged by its FIRST byte before the token is read: a JSON value start of
 *      the wrong type for the field is PJ_E_TYPE at that byte; a byte that starts no JSON value
 *      is PJ_E_SYNTAX. `null` is accepted for every field and means "absent"; null as a list
 *      element is PJ_E_TYPE.
 *  R6  Numbers are lexed as -?(0|[1-9][0-9]*)(\.[0-9]+)?([eE][+-]?[0-9]+)? (a violation is
 *      PJ_E_SYNTAX at the offending byte). For an integer field a fraction or exponent is
 *      PJ_E_TYPE and a value outside int64 / int32 is PJ_E_NUM_RANGE, both at the token's first
 *      byte. There are no minimum/maximum constraints (petstore.json:947-950,848-852 state none).
 *  R7  Strings: a raw byte < 0x20 is PJ_E_CTRL_CHAR at that byte. Escapes \" \\ \/ \b \f \n \r \t
 *      \uXXXX; any other escape letter, or a non-hex digit, is PJ_E_BAD_ESCAPE at that byte. A
 *      \uD800-\uDBFF must be followed at once by \uDC00-\uDFFF (together one code point, 4 UTF-8
 *      bytes); otherwise, and for a lone \uDC00-\uDFFF, PJ_E_BAD_SURROGATE at the backslash of
 *      the first unit. Raw bytes >= 0x80 must be well-formed UTF-8 (RFC 3629: no overlongs, no
 *      surrogates, <= U+10FFFF): PJ_E_UTF8 at the first byte of the bad sequence.
 *  R8  Enum fields (Pet.status petstore.json:909-917, Order.status :955-963): the decoded string
 *      must equal a literal; otherwise PJ_E_ENUM at the opening quote. Stored as the literal's
 *      0-based index, 255 when absent.
 *  R9  Order.shipDate (petstore.json:951-954) is RFC 3339 date-time
 *      YYYY-MM-DDThh:mm:ss[.f{1,9}](Z|+hh:mm|-hh:mm), upper-case T and Z, real calendar dates,
 *      hour <= 23, minute <= 59, second <= 59, offset hour <= 23; otherwise PJ_E_DATETIME at the
 *      opening quote. Stored as (UTC epoch seconds, nanoseconds, offset seconds).
 *  R10 Required fields (Pet.name, Pet.photoUrls: petstore.json:873-876) missing or null when the
 *      object closes: PJ_E_REQUIRED at the closing brace.
 *  R11 A failed record keeps its row: every field absent, every list and string empty.
 *  R12 PJ_SCHEMA_MIXED: a record's model is the owner of the first key that belongs to exactly
 *      one of Pet / Order / User (`id` is common to all, `status` to Pet and Order). A `status`
 *      value met before that must be a literal of Pet or of Order (else PJ_E_ENUM at once) and is
 *      re-checked against the model once known (PJ_E_ENUM at the value's quote). An object that
 *      closes with no deciding key is PJ_E_AMBIGUOUS at the closing brace. Failed records get
 *      PJ_COL_REC_TYPE = PJ_TYPE_NONE and no row in any model table.
 *
 * Serialisation rules (pj_write):
 *  W1  Field order is the schema's property order (petstore.json:878-917, 826-852, 939-966);
 *      compact output, records joined by LF (NDJSON, one LF after every record) or wrapped as
 *      `[r,r,...]` (array framing).
 *  W2  Integers in minimal decimal; booleans `true` / `false`; enums by literal.
 *  W3  Strings: `"` -> \", `\` -> \\, 0x08 0x09 0x0A 0x0C 0x0D -> \b \t \n \f \r, other bytes
 *      < 0x20 -> \u00XX with upper-case hex; `/` and bytes >= 0x80 are written as they are.
 *  W4  Inclusion (pj_options.inclusion): absent fields are omitted (PJ_INCLUDE_NON_NULL), and
 *      additionally empty strings and empty lists (PJ_INCLUDE_NON_EMPTY, the default), or absent
 *      fields are written as `null` (PJ_INCLUDE_ALWAYS).
 *  W5  shipDate: YYYY-MM-DDThh:mm:ss, then `.` and the nanoseconds without trailing zeros when
 *      they are not zero, then `Z` for offset 0 or +hh:mm / -hh:mm.
 */
#ifndef PETJSON_H
#define PETJSON_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PJ_VERSION_MAJOR 0
#define PJ_VERSION_MINOR 1

/* ---- call status ------------------------------------------------------------------------- */
typedef int32_t pj_status;
enum {
  PJ_OK = 0,
  PJ_ERR_ARG = 1,       /* null pointer, unknown schema / framing / column, bad option        */
  PJ_ERR_CAPACITY = 2,  /* an output buffer is too small; required counts are written back     */
  PJ_ERR_CUDA = 3,      /* a CUDA call failed (text via pj_last_error)                         */
  PJ_ERR_TIMEOUT = 4,   /* a bounded device-side wait ran out; the context stays usable        */
  PJ_ERR_NOMEM = 5,     /* host or device allocation failed                                    */
  PJ_ERR_TOO_LARGE = 6, /* the input is larger than one call takes: 4 GiB (32-bit offsets), or 32 GiB for NDJSON in
                           device memory, which is parsed in ranges (pj_options.device_piece_bytes)        */
  PJ_ERR_NCCL = 7       /* pj_group_*: an NCCL call failed or the library could not be loaded    */
};

/* ---- per-record validation result (PJ_COL_ERR_KIND) ------------------------------------- */
enum {
  PJ_E_NONE = 0,
  PJ_E_SYNTAX = 1,
  PJ_E_EOF = 2,
  PJ_E_CTRL_CHAR = 3,
  PJ_E_BAD_ESCAPE = 4,
  PJ_E_BAD_SURROGATE = 5,
  PJ_E_UTF8 = 6,
  PJ_E_TYPE = 7,
  PJ_E_NUM_RANGE = 8,
  PJ_E_ENUM = 9,
  PJ_E_REQUIRED = 10,
  PJ_E_DATETIME = 11,
  PJ_E_DEPTH = 12,
  PJ_E_AMBIGUOUS = 13,
  PJ_E_TOO_LONG = 14, /* record runs past the shard's slack bytes; offset = bytes available   */
  PJ_E_KIND_COUNT = 15
};

enum { PJ_MEM_HOST = 0, PJ_MEM_DEVICE = 1 };
enum { PJ_SCHEMA_PET = 1, PJ_SCHEMA_ORDER = 2, PJ_SCHEMA_USER = 3, PJ_SCHEMA_MIXED = 4 };
enum { PJ_TYPE_NONE = 0, PJ_TYPE_PET = 1, PJ_TYPE_ORDER = 2, PJ_TYPE_USER = 3 };
enum { PJ_FRAMING_NDJSON = 0, PJ_FRAMING_ARRAY = 1 };
enum { PJ_INCLUDE_NON_EMPTY = 0, PJ_INCLUDE_NON_NULL = 1, PJ_INCLUDE_ALWAYS = 2 };

/* ---- column ids --------------------------------------------------------------------------
 * "rows" below: for PJ_SCHEMA_PET/ORDER/USER a model table has one row per record (failed records
 * included, rule R11); for PJ_SCHEMA_MIXED it has one row per valid record of that model and
 * PJ_COL_REC_TYPE / PJ_COL_REC_ROW map a record to its row. P = total photoUrls, T = total tags.
 * Presence bytes hold one bit per property in schema order (bit 0 = first property).          */
enum {
  /* per record, every schema */
  PJ_COL_REC_START = 0,  /* u64[N]   byte offset of the record's extent in the input           */
  PJ_COL_ERR_KIND = 1,   /* u8[N]    PJ_E_*                                                    */
  PJ_COL_ERR_OFF = 2,    /* u32[N]   byte offset of the failure relative to REC_START (0 if ok) */
  PJ_COL_REC_TYPE = 3,   /* u8[N]    PJ_TYPE_*            (PJ_SCHEMA_MIXED only)               */
  PJ_COL_REC_ROW = 4,    /* u32[N]   row in the model table, 0xFFFFFFFF when PJ_TYPE_NONE
                                     (PJ_SCHEMA_MIXED only)                                    */

  /* Pet — petstore.json:872-922; Category :858-871; Tag :923-936 */
  PJ_COL_PET_PRESENT = 8,        /* u8[rows]  bits: id, category, name, photoUrls, tags, status */
  PJ_COL_PET_ID = 9,             /* i64[rows]                                                  */
  PJ_COL_PET_CAT_PRESENT = 10,   /* u8[rows]  bits: id, name                                   */
  PJ_COL_PET_CAT_ID = 11,        /* i64[rows]                                                  */
  PJ_COL_PET_CAT_NAME_OFF = 12,  /* u32[rows+1]                                                */
  PJ_COL_PET_CAT_NAME_DATA = 13, /* u8[]                                                       */
  PJ_COL_PET_NAME_OFF = 14,      /* u32[rows+1]                                                */
  PJ_COL_PET_NAME_DATA = 15,     /* u8[]                                                       */
  PJ_COL_PET_PHOTO_OFF = 16,     /* u32[rows+1] list offsets into the photo string column      */
  PJ_COL_PET_PHOTO_STR_OFF = 17, /* u32[P+1]                                                   */
  PJ_COL_PET_PHOTO_DATA = 18,    /* u8[]                                                       */
  PJ_COL_PET_TAGS_OFF = 19,      /* u32[rows+1] list offsets into the tag table                */
  PJ_COL_PET_TAG_PRESENT = 20,   /* u8[T]     bits: id, name                                   */
  PJ_COL_PET_TAG_ID = 21,        /* i64[T]                                                     */
  PJ_COL_PET_TAG_NAME_OFF = 22,  /* u32[T+1]                                                   */
  PJ_COL_PET_TAG_NAME_DATA = 23, /* u8[]                                                       */
  PJ_COL_PET_STATUS = 24,        /* u8[rows]  0 available, 1 pending, 2 sold, 255 absent       */

  /* Order — petstore.json:937-971 */
  PJ_COL_ORD_PRESENT = 32,     /* u8[rows]  bits: id, petId, quantity, shipDate, status, complete */
  PJ_COL_ORD_ID = 33,          /* i64[rows]                                                    */
  PJ_COL_ORD_PET_ID = 34,      /* i64[rows]                                                    */
  PJ_COL_ORD_QUANTITY = 35,    /* i32[rows]                                                    */
  PJ_COL_ORD_SHIP_EPOCH = 36,  /* i64[rows] seconds since 1970-01-01T00:00:00Z                 */
  PJ_COL_ORD_SHIP_NANOS = 37,  /* i32[rows]                                                    */
  PJ_COL_ORD_SHIP_OFFSET = 38, /* i32[rows] UTC offset in seconds                              */
  PJ_COL_ORD_STATUS = 39,      /* u8[rows]  0 placed, 1 approved, 2 delivered, 255 absent      */
  PJ_COL_ORD_COMPLETE = 40,    /* u8[rows]  0 / 1                                              */

  /* User — petstore.json:824-857 */
  PJ_COL_USR_PRESENT = 44, /* u8[rows] bits: id, username, firstName, lastName, email, password,
                              phone, userStatus */
  PJ_COL_USR_ID = 45,      /* i64[rows] */
  PJ_COL_USR_USERNAME_OFF = 46,
  PJ_COL_USR_USERNAME_DATA = 47,
  PJ_COL_USR_FIRSTNAME_OFF = 48,
  PJ_COL_USR_FIRSTNAME_DATA = 49,
  PJ_COL_USR_LASTNAME_OFF = 50,
  PJ_COL_USR_LASTNAME_DATA = 51,
  PJ_COL_USR_EMAIL_OFF = 52,
  PJ_COL_USR_EMAIL_DATA = 53,
  PJ_COL_USR_PASSWORD_OFF = 54,
  PJ_COL_USR_PASSWORD_DATA = 55,
  PJ_COL_USR_PHONE_OFF = 56,
  PJ_COL_USR_PHONE_DATA = 57,
  PJ_COL_USR_STATUS = 58, /* i32[rows] */

  PJ_MAX_COLS = 64
};

/* One buffer of a column set. The CALLER owns `ptr`; the library never frees it and keeps no
 * pointer past the return of the call.
 *   before pj_parse : ptr / bytes = the caller's buffer and its capacity in bytes
 *   after  pj_parse : count = elements produced (for an _OFF column: rows + 1). On
 *                     PJ_ERR_CAPACITY count holds the number REQUIRED for every column.
 *   for    pj_write : ptr / count describe the columns to serialise; bytes is ignored.        */
typedef struct pj_buf {
  void* ptr;
  uint64_t bytes;
  uint64_t count;
} pj_buf;

typedef struct pj_columns {
  uint32_t schema;     /* PJ_SCHEMA_*; set by pj_columns_sizes / pj_parse                       */
  uint32_t mem_kind;   /* PJ_MEM_HOST or PJ_MEM_DEVICE: where every col[].ptr lives             */
  uint64_t n_records;  /* records found (failed ones included)                                  */
  uint64_t n_errors;   /* records with ERR_KIND != 0                                            */
  uint64_t n_rows[4];  /* rows of the model tables, indexed by PJ_TYPE_* ([0] unused)           */
  uint64_t doc_err_off; /* array framing: offset of the first byte that breaks `ws [ ... ] ws`   */
  uint32_t doc_err_kind; /* array framing: PJ_E_SYNTAX / PJ_E_EOF for the document, else 0       */
  uint32_t reserved;
  pj_buf col[PJ_MAX_COLS];
} pj_columns;

/* pj_options.flags. The first four select the other answer of a rule that rests on behaviour of the reference's
 * third-party serde which could not be observed (no JVM where this was written); the defaults are the rules R1-R12,
 * W1-W5 above. tests/golden/EmitGolden.java, run by someone who has the JVM, says which answers are the library's. */
enum {
  PJ_OPT_ENUM_UNKNOWN_AS_NULL = 1u << 0,   /* R8: a string that is no literal of the enum leaves the property absent (the
                                              convention of api/EnumParam.java:32-34) instead of failing with PJ_E_ENUM (the
                                              convention of config/data/VariantEnum.java:41-46)                              */
  PJ_OPT_LONE_SURROGATE_REPLACE = 1u << 1, /* R7: a \uD800-\uDFFF escape without its partner is accepted and decoded as
                                              U+FFFD (EF BF BD) instead of failing with PJ_E_BAD_SURROGATE                 */
  PJ_OPT_COERCE_SCALARS = 1u << 2,         /* R5: an integer property also takes a JSON string that holds an integer
                                              (-?(0|[1-9][0-9]*); otherwise PJ_E_TYPE, out of range PJ_E_NUM_RANGE, both at the
                                              opening quote); a boolean property the strings "true" / "false"; a string
                                              property of a model, Category or Tag also takes a number, true or false, whose
                                              text as written becomes the string. List elements, enums and date-times are
                                              not coerced                                                                  */
  PJ_OPT_HEX_LOWER = 1u << 3,              /* W3: \u00xx escapes are written with lower-case hex digits                    */
  PJ_OPT_TEST_STALL_ONCE = 1u << 31 /* test hook for the time-out path: in the context's FIRST NDJSON parse call the first
                                       tile is never handed out, so every other tile's bounded wait for it runs out
                                       (after spin_limit_us) and the call answers PJ_ERR_TIMEOUT; later calls are normal */
};

typedef struct pj_options {
  int32_t device;            /* CUDA device ordinal; -1 = the calling thread's current device   */
  int32_t inclusion;         /* PJ_INCLUDE_* for pj_write                                       */
  void* stream;              /* a cudaStream_t to run on, or NULL for a stream the context owns */
  uint32_t flags;            /* PJ_OPT_* bits                                                   */
  uint32_t host_piece_bytes; /* pj_parse with host input and host columns (NDJSON): the input is cut after
                                line feeds into pieces of about this many bytes (at most 16), and the copy of
                                one piece to the device, the kernel of the previous one and the copy of the
                                columns of the one before run at the same time. 0 = 32 MiB; 0xFFFFFFFF = never
                                cut. The result does not depend on it.                            */
  uint32_t tile_bytes;       /* NDJSON: input bytes per thread block of the parse kernel (1024 .. 32768, rounded
                                down to a multiple of 16). 0 = chosen by the library from the bytes per record
                                of the context's earlier calls. The result does not depend on it.  */
  uint32_t spin_limit_us;    /* bound, in microseconds, of every wait of a thread block on another one or on
                                its staging copy; when one runs out the call answers PJ_ERR_TIMEOUT and the
                                context stays usable. 0 = 2 seconds.                               */
  uint32_t device_piece_bytes; /* pj_parse* with NDJSON that lies on the device: the input is parsed as byte ranges
                                of this many bytes (at most 16 of them, at most 2 GiB each), one launch per range,
                                each starting from the totals the one before it left on the device. 0 = only
                                inputs of 4 GiB and more are cut (into ranges of 2 GiB): that is what lets one
                                call take up to 32 GiB although a launch addresses its bytes with 32-bit offsets.
                                The result does not depend on it.                                   */
  uint32_t reserved;
} pj_options;

typedef struct pj_ctx pj_ctx;

/* Kernel accounting of the most recent pj_parse* / pj_write / pj_index_records call on a context. */
typedef struct pj_call_stats {
  uint32_t kernel_launches; /* kernels of this library launched by the call                    */
  uint32_t pieces;          /* pj_parse: pieces the input was parsed in (see pj_options.host_piece_bytes) */
  float device_ms;          /* CUDA-event time from first launch to last, on the call's stream  */
  float main_kernel_ms;     /* CUDA-event time of the dominant kernel(s) of the call            */
  float stage_ms[8];        /* CUDA-event time per stage. parse, NDJSON: [2] the parse kernel(s), nothing else
                               runs; parse, array framing: [0] record index, [1] set-up between the kernels
                               (record count read-back, state reset), [2] the tile kernel; write: [0] state
                               reset and the scan of the string arenas for bytes to escape, [1] the closing
                               kernel, [2] the tile kernel */
  uint32_t stage_launches[8]; /* kernels launched per stage                                      */
  uint64_t h2d_bytes;       /* bytes copied host->device by the call                            */
  uint64_t d2h_bytes;       /* bytes copied device->host by the call                            */
  uint64_t algorithmic_bytes; /* input bytes + bytes of every produced column (parse), or column
                                 bytes read + JSON bytes written (write)                        */
  uint64_t fast_records;    /* parse: records decoded by the speculative word-at-a-time pass alone */
  uint64_t phase_cycles[4]; /* SM cycles summed over the blocks of the tile kernel. parse: staging,
                               tokenising, look-back wait, emission; write: size pass, look-back
                               wait, text into the window, copy-out                              */
  uint64_t lookback_polls;  /* parse: times a block found the block before it not yet sized        */
  uint64_t lookback_rounds; /* parse: 32-block look-back rounds, summed over blocks                 */
  uint32_t tile_records;    /* parse: records per block of the tile kernel                       */
  uint32_t tiles;           /* blocks of the tile kernel                                          */
  uint64_t wide_records;    /* parse: long records walked by a whole warp instead of one thread    */
  uint64_t wide_fast_records; /* parse: of those, finished by the word-at-a-time tokeniser (the rest took the
                                 exact parser, lists still spread over the lanes)                  */
  uint64_t wide_cycles[2];  /* parse: SM cycles the blocks spent in the warps' size pass and emit pass (part of
                               phase_cycles[1] and [3])                                          */
} pj_call_stats;

/* Library version as major * 1000 + minor. */
int32_t pj_version(void);
const char* pj_status_str(pj_status s);
const char* pj_error_kind_str(int32_t kind);

/* Name, element width in bytes and owning model (PJ_TYPE_*, 0 = per record) of a column id.
 * Returns PJ_ERR_ARG for ids that are not columns. */
pj_status pj_column_info(int32_t col, const char** name, uint32_t* elem_bytes, uint32_t* owner);

/* Replaces ObjectMapper.getDefault() (MyEntityService.java:45) / the injected ObjectMapper bean
 * (MyEntityConfig.java:24). `opt` may be NULL: current device, NON_EMPTY inclusion, own stream.
 * One context serves one caller at a time; separate contexts are independent. */
pj_status pj_create(const pj_options* opt, pj_ctx** out);
void pj_destroy(pj_ctx* ctx);
/* Text of the last failure on `ctx` (or of the last failed pj_create when ctx is NULL). */
const char* pj_last_error(const pj_ctx* ctx);
pj_status pj_last_stats(const pj_ctx* ctx, pj_call_stats* out);
/* Release device scratch the context grew for earlier calls. */
pj_status pj_trim(pj_ctx* ctx);

/* Upper bounds for buffer sizes: fills out->col[i].bytes for every column of `schema` so that an
 * input of at most `max_input_bytes` holding at most `max_records` records (and at most
 * `max_list_items` list elements in total; pass 0 to bound them by the input size) always fits. */
pj_status pj_columns_sizes(uint32_t schema, uint64_t max_records, uint64_t max_input_bytes,
                           uint64_t max_list_items, pj_columns* out);

/* Replaces ObjectMapper#readValue (MyEntityConfig.java:34) for a whole batch of records.
 * `in` is `len` bytes of JSON in host or device memory (`in_kind`); `out` carries the caller's
 * buffers (all in out->mem_kind memory). Columns of other schemas are ignored; a column of this
 * schema with ptr == NULL is PJ_ERR_ARG. When the record count itself exceeds the per-record
 * buffers, only n_records and the per-record counts are exact in the PJ_ERR_CAPACITY answer.
 * len must be < 4 GiB; NDJSON in device memory may be up to 32 GiB (it is parsed in ranges of 2 GiB, see
 * pj_options.device_piece_bytes) as long as every arena and child table of the result stays below 2^32 entries
 * (PJ_ERR_CAPACITY otherwise). */
pj_status pj_parse(pj_ctx* ctx, uint32_t schema, uint32_t framing, const uint8_t* in,
                   uint64_t len, uint32_t in_kind, pj_columns* out);

/* One byte-range shard of a larger NDJSON stream (multi-GPU or chunked use). `in` must hold
 * len + slack readable bytes, the slack being the head of the following shard (0 for the last one).
 * The shard owns every record whose preceding LF lies in [0, len) and, if `is_first`, the record
 * that starts at byte 0; so the bytes up to and including a later shard's first LF belong to its
 * predecessor, which reads them from its slack. `is_last` tells that the stream ends at
 * len + slack. `global_offset` is added to PJ_COL_REC_START. A record whose end is not reached
 * within the slack fails with PJ_E_TOO_LONG at the number of bytes that were available.
 * len + slack must be < 4 GiB (device memory: 32 GiB, as for pj_parse). */
pj_status pj_parse_shard(pj_ctx* ctx, uint32_t schema, const uint8_t* in, uint64_t len,
                         uint64_t slack, int32_t is_first, int32_t is_last, uint64_t global_offset,
                         uint32_t in_kind, pj_columns* out);

/* Record index only: writes the extent start of every record into rec_start[0..cap) and the number
 * found into *n (PJ_ERR_CAPACITY if n > cap; *n is still set). `rec_start` lives in `kind` memory,
 * like `in`. */
pj_status pj_index_records(pj_ctx* ctx, uint32_t framing, const uint8_t* in, uint64_t len,
                           uint32_t kind, uint64_t* rec_start, uint64_t cap, uint64_t* n);

/* Record index of an NDJSON buffer for callers that must not allocate. It has no counterpart in the
 * reference; it exists for hosts that run this library where device memory cannot be obtained or
 * released: inside a region whose memory is owned and budgeted by someone else (an embedding runtime's
 * pool allocator, a serving process that froze its heap after start-up), or on a latency-critical thread
 * where the implicit synchronisation of an allocation is not acceptable. pj_index_records grows a
 * per-context scratch buffer on demand; this variant does the same work with its scratch (one 32-bit
 * count per 16 KiB of input) in a fixed array that is part of the loaded library image, at most
 * PJ_STATIC_INDEX_MAX_BYTES of input per call (PJ_ERR_TOO_LARGE beyond that).
 *   - `in`, `rec_start` (room for `cap` offsets) and `n_device` (one uint64) are DEVICE memory of the
 *     device that is current for the calling thread; nothing is copied to the host.
 *   - The kernels are enqueued on `stream` (a cudaStream_t, NULL = the default stream) and the call
 *     returns without waiting: read *n_device and rec_start after synchronising that stream. If more than
 *     `cap` records are found, *n_device still holds the true count and only the first `cap` are stored.
 *   - It calls no allocating routine. Its first call on each device looks up the device address of the
 *     fixed array (a driver query, not an allocation); make that first call before any stream capture.
 *   - Every GPU that loads the library holds the array (about 256 KiB) until the process exits. All calls
 *     on a device share it: two calls whose kernels can overlap on the GPU (different streams) race and
 *     give undefined offsets; calls on one stream are ordered and safe. Nothing in it needs clearing
 *     between calls: every word a call reads, that call has written first. */
#define PJ_STATIC_INDEX_MAX_BYTES (1ull << 30)
pj_status pj_index_records_static(const uint8_t* in, uint64_t len, uint64_t* rec_start, uint64_t cap,
                                  uint64_t* n_device, void* stream);

/* Replaces ObjectMapper#writeValueAsBytes / the response body encoder (MyEntityController.java:48-51)
 * for a whole table: serialises rows [0, cols->n_rows[type]) of the model table(s) of `schema`
 * (for PJ_SCHEMA_MIXED: records in PJ_COL_REC_TYPE / PJ_COL_REC_ROW order, PJ_TYPE_NONE skipped).
 * `out` (cap bytes, `out_kind` memory) receives the JSON; *out_len the byte count, also on
 * PJ_ERR_CAPACITY. Columns live in cols->mem_kind memory. */
pj_status pj_write(pj_ctx* ctx, uint32_t schema, uint32_t framing, const pj_columns* cols,
                   uint8_t* out, uint64_t cap, uint32_t out_kind, uint64_t* out_len);

/* One 64-bit checksum per column of a device-resident column set, computed on the GPU: for checking results at sizes
 * where copying every column to the host for a comparison is not wanted. sums[col] is 0 for columns the schema does
 * not have. The checksum of a column is over its first count * element_width bytes b[0..n): with w_j the little-endian
 * 64-bit word of bytes [8j, 8j+8) (zero padded at the end),
 *     sum = SUM_j mix(w_j + 0x9E3779B97F4A7C15 * (j + 1))  (mod 2^64),
 *     mix(x): x ^= x >> 30; x *= 0xBF58476D1CE4E5B9; x ^= x >> 27; x *= 0x94D049BB133111EB; x ^= x >> 31.
 * The terms commute, so any number of threads may add them in any order; the CPU checker computes the same sums
 * from its own columns. No counterpart in the reference (it has no columns). */
pj_status pj_columns_checksum(pj_ctx* ctx, uint32_t schema, const pj_columns* cols, uint64_t* sums /*[PJ_MAX_COLS]*/);

/* ---- several GPUs of one machine ------------------------------------------------------------------------
 * The reference reaches its mapper as ONE in-process bean (MyEntityConfig.java:24,34): a caller that wants all the
 * GPUs of a box therefore needs them behind one handle in one process. A group holds one context per device and
 * runs one host thread and one stream per device inside its calls. An NDJSON stream is split by the caller into
 * contiguous byte ranges ("shards"), shard g resident on device g; a shard owns the records whose preceding line
 * feed lies in its range (pj_parse_shard's rule). The library copies the head of the following shard(s) into the
 * room behind shard g (device to device, peer copy; no kernel reads another GPU's memory), parses every shard on
 * its own GPU, and exchanges one small table of counters with ncclAllGather, which is left on every device. */
typedef struct pj_group pj_group;

/* words per shard of the gathered table (uint64 each) */
enum {
  PJ_GC_RECORDS = 0, PJ_GC_ERRORS = 1, PJ_GC_BYTES = 2,   /* parse: owned input bytes; write: text bytes produced */
  PJ_GC_ROWS_PET = 3, PJ_GC_ROWS_ORDER = 4, PJ_GC_ROWS_USER = 5,
  PJ_GC_COUNTER0 = 8,                                     /* 15 totals: arena bytes and child-table rows, library order */
  PJ_GROUP_NCOUNT = 24
};

/* What a group call reports per shard. */
typedef struct pj_group_shard {
  uint64_t global_offset;  /* parse: byte offset of the shard in the stream (added to PJ_COL_REC_START);
                              write: byte offset of the shard's text in the concatenation of all outputs */
  uint64_t first_record;   /* number, in the whole stream, of the shard's first record                    */
  uint64_t first_row[4];   /* rows of the model tables that precede the shard's, indexed by PJ_TYPE_*     */
  uint64_t bytes;          /* parse: input bytes the shard owns; write: text bytes it produced             */
  uint64_t slack_bytes;    /* parse: bytes of the following shards that were copied behind this one        */
  const uint64_t* table_dev; /* DEVICE memory of the shard's GPU: the gathered table [ndev][PJ_GROUP_NCOUNT]. The
                                all-gather that fills it is enqueued on a stream of the group's own and not waited
                                for (the answer above comes from host copies): call pj_group_sync() before
                                anything reads it. Valid until the next call on the group                   */
  pj_status status;        /* this shard's own status (the call returns the first one that is not PJ_OK)   */
  float slack_copy_ms;     /* parse: CUDA-event time of the device-to-device copy of the slack bytes        */
  float gather_ms;         /* host time to enqueue the exchange of the device tables (counter kernel and
                              all-gather); the caller's answer comes from the host copies of the counters   */
  uint32_t reserved;
} pj_group_shard;

/* `devs` may name a device more than once (several shards per GPU, e.g. to try a group on one GPU): such a group
 * exchanges its table through the host instead of NCCL. Otherwise NCCL (libnccl.so.2, found with the dynamic
 * loader's search rules) is initialised with ncclCommInitAll; PJ_ERR_NCCL if that fails. `opt` applies to every
 * context (device and stream are ignored). */
pj_status pj_group_create(int32_t ndev, const int32_t* devs, const pj_options* opt, pj_group** out);
void pj_group_destroy(pj_group* grp);
int32_t pj_group_size(const pj_group* grp);
/* the context of shard i (pj_last_stats, pj_last_error); not for concurrent use with a group call */
pj_ctx* pj_group_ctx(pj_group* grp, int32_t i);
const char* pj_group_last_error(const pj_group* grp);
/* 1 when the group exchanges its table with NCCL, 0 when it goes through the host */
int32_t pj_group_uses_nccl(const pj_group* grp);
/* Waits until the device tables (pj_group_shard.table_dev) of the last call are complete on every shard. */
pj_status pj_group_sync(pj_group* grp);

/* Replaces ObjectMapper#readValue (MyEntityConfig.java:34) for a stream spread over the group's GPUs.
 * in[g]: shard g's bytes in device g's memory, len[g] of them, followed by room[g] writable bytes (at least
 * `slack` for every shard but the last, or a record that straddles the boundary fails with PJ_E_TOO_LONG);
 * out[g]: shard g's columns, buffers in device g's memory (mem_kind PJ_MEM_DEVICE). Offsets in the columns are
 * local to the shard; PJ_COL_REC_START is global. shards[g] receives where shard g lies in the whole. */
pj_status pj_group_parse(pj_group* grp, uint32_t schema, uint8_t* const* in, const uint64_t* len, const uint64_t* room,
                         uint64_t slack, pj_columns* out, pj_group_shard* shards);

/* The same for a stream that lies in HOST memory (io.micronaut.serde.ObjectMapper.readValue(byte[], ...) of a large
 * body, MyEntityConfig.java:34): `text` holds all shards back to back, shard i is len[i] bytes, and the bytes behind a
 * shard are its slack. Every shard's thread runs the host-buffer route of pj_parse on its device (pieces whose copies
 * overlap the kernels of the pieces before them; pinned memory makes the overlap real), all devices side by side.
 * out[i] may be host or device columns. */
pj_status pj_group_parse_host(pj_group* grp, uint32_t schema, const uint8_t* text, const uint64_t* len, uint64_t slack, pj_columns* out,
                              pj_group_shard* shards);

/* Replaces ObjectMapper#writeValueAsBytes (MyEntityController.java:48-51) for tables spread over the group's GPUs:
 * device g serialises cols[g] (as pj_write, NDJSON framing) into out[g] (cap[g] bytes, device g's memory). The
 * text of the whole is the concatenation of the outputs in shard order; shards[g].global_offset says where shard
 * g's text starts in it, shards[g].bytes how long it is. */
pj_status pj_group_write(pj_group* grp, uint32_t schema, const pj_columns* cols, uint8_t* const* out, const uint64_t* cap,
                         pj_group_shard* shards);

#ifdef __cplusplus
}
#endif
#endif /* PETJSON_H */
