/*
 * petjson_gen.h — seeded synthetic Petstore workloads (libpj_gen.so: plain C on the host, no CUDA, no
 * link to libpetjson.so). The benchmark, the CPU baseline and the tests draw their inputs from here, so
 * that a process which only times the CPU path maps the generator and nothing of the GPU library.
 * The reference project has no counterpart: its only JSON documents are
 * src/main/resources/configs/var1.json and var2.json.
 */
#ifndef PETJSON_GEN_H
#define PETJSON_GEN_H

#include "petjson.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Record `first + k` of a stream depends only on (seed, first + k), so shards can be generated
 * independently. Distributions follow the benchmark configurations: ids uniform in [1, 2^62],
 * names 4-16 letters, category names 3-12, 0-4 photoUrls of 20-60 URL-safe characters, 0-3 tags
 * with 3-10 letter names, status uniform over the literals. */
enum {
  PJ_GEN_ZIPF_LISTS = 1u << 0,  /* list lengths zipf(1.2), tags <= 64, photoUrls <= 256          */
  PJ_GEN_ESCAPES = 1u << 1,     /* 5% of strings carry \uXXXX escapes incl. surrogate pairs       */
  PJ_GEN_WHITESPACE = 1u << 2,  /* random spaces / tabs / CR between tokens                       */
  PJ_GEN_MALFORMED = 1u << 3,   /* 1% of records broken: enum, required, type, truncated string   */
  PJ_GEN_ARRAY = 1u << 4,       /* `[r,r,...]` instead of one record per line                     */
  PJ_GEN_SPARSE = 1u << 5       /* optional properties randomly omitted or written as null        */
};

/* Writes the JSON text of records [first, first+n) of stream `seed` of `schema` into text[0..cap)
 * (host memory) and its length into *len; returns PJ_ERR_CAPACITY (with *len = needed) if it does
 * not fit. text may be NULL to query the length. */
pj_status pj_gen_text(uint32_t schema, uint64_t seed, uint64_t first, uint64_t n, uint32_t flags,
                      uint8_t* text, uint64_t cap, uint64_t* len);

/* Fills host-memory columns with the VALUES of the same records (what a correct parse of
 * pj_gen_text's output yields, error columns included). Buffers as for pj_parse. */
pj_status pj_gen_columns(uint32_t schema, uint64_t seed, uint64_t first, uint64_t n, uint32_t flags,
                         pj_columns* out);

#ifdef __cplusplus
}
#endif
#endif /* PETJSON_GEN_H */
