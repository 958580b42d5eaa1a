/*
 * pj_tile_inst.cu — one instantiation of the two parse kernels (k_parse_stream for NDJSON, k_parse_tile for a given
 * record index), compiled once per model set with
 * -DPJ_TILE_SCHEMA=1..4 (Pet, Order, User, mixed) so that the four heavy instantiations build in
 * parallel. Each object carries its own copy of the constant model tables, set by its init function.
 */
#include <cuda_runtime.h>

#include "petjson.h"
#include "pj_kernels.cuh"
#include "pj_stream_kernel.cuh"

#ifndef PJ_TILE_SCHEMA
#error "compile with -DPJ_TILE_SCHEMA=<PJ_SCHEMA_* value>"
#endif
#define PJ_CAT2(a, b) a##b
#define PJ_CAT(a, b) PJ_CAT2(a, b)

namespace pj {

cudaError_t PJ_CAT(tile_init_, PJ_TILE_SCHEMA)(const Schema* s) {
  cudaError_t e = cudaFuncSetAttribute(k_parse_tile<PJ_TILE_SCHEMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, TILE_SMEM_BYTES);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(k_parse_stream<PJ_TILE_SCHEMA>, cudaFuncAttributeMaxDynamicSharedMemorySize, ST_SMEM_BYTES);
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(c_schema, s, sizeof(Schema));
  return e;
}
cudaError_t PJ_CAT(tile_launch_, PJ_TILE_SCHEMA)(const TileArgs* a, unsigned grid, cudaStream_t stream) {
  k_parse_tile<PJ_TILE_SCHEMA><<<grid, TILE_THREADS, TILE_SMEM_BYTES, stream>>>(*a);
  return cudaGetLastError();
}

cudaError_t PJ_CAT(stream_launch_, PJ_TILE_SCHEMA)(const StreamArgs* a, unsigned grid, cudaStream_t stream) {
  k_parse_stream<PJ_TILE_SCHEMA><<<grid, ST_THREADS, ST_SMEM_BYTES, stream>>>(*a);
  return cudaGetLastError();
}

}  // namespace pj
