// Tensor-map (TMA) helpers: host-side descriptor construction and the device-side
// cp.async.bulk.tensor loads that fill 128-byte swizzled shared-memory tiles.
//
// The descriptors are built per call on the host stack (cuTensorMapEncodeTiled, reached
// through cudaGetDriverEntryPoint so the library links against libcudart only) and passed
// to the kernel by value as __grid_constant__ parameters: nothing is allocated or cached.
// No load here uses cluster multicast.  Every load starts at channel 0 of a 128-byte row,
// so the innermost coordinate is always 16-byte aligned.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace llsa {
namespace tma {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeFn encode_fn() {
  static EncodeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(p);
  }
  return fn;
}

// bf16 tensor of `rank` dims (dims[0] = 64 channels, unit stride), byte strides for dims 1..rank-1,
// box = box_rows rows of 64 channels, 128-byte swizzle.
inline int make_map(CUtensorMap* m, const void* base, int rank, const uint64_t* dims, const uint64_t* strides_bytes, uint32_t box_rows) {
  EncodeFn fn = encode_fn();
  LLSA_REQUIRE(fn != nullptr, LLSA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t gd[5];
  cuuint64_t gs[4];
  cuuint32_t box[5], es[5];
  for (int i = 0; i < rank; ++i) { gd[i] = dims[i]; box[i] = 1; es[i] = 1; }
  for (int i = 0; i + 1 < rank; ++i) gs[i] = strides_bytes[i];
  box[0] = 64;
  box[1] = box_rows;
  const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, (cuuint32_t) rank, const_cast<void*>(base), gd, gs, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  LLSA_REQUIRE(r == CUDA_SUCCESS, LLSA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int) r);
  return LLSA_OK;
}

// [B,H,N,64] tensor with element strides (sb, sh, sn): a 4-D map (channel, token, head, batch).
inline int make_map_bhnd(CUtensorMap* m, const LlsaTensor* t, uint32_t box_rows) {
  const uint64_t dims[4] = {64, (uint64_t) t->shape[2], (uint64_t) t->shape[1], (uint64_t) t->shape[0]};
  // a size-1 dimension may carry any stride: give it one the encoder accepts
  const uint64_t sn = (uint64_t) t->stride[2] * 2, sh = t->shape[1] > 1 ? (uint64_t) t->stride[1] * 2 : sn * t->shape[2],
                 sb = t->shape[0] > 1 ? (uint64_t) t->stride[0] * 2 : sh * t->shape[1];
  const uint64_t strides[3] = {sn, sh, sb};
  return make_map(m, t->ptr, 4, dims, strides, box_rows);
}

// Contiguous [rows, 64] matrix: a 2-D map.
inline int make_map_rows(CUtensorMap* m, const void* base, uint64_t rows, uint32_t box_rows) {
  const uint64_t dims[2] = {64, rows};
  const uint64_t strides[1] = {128};
  return make_map(m, base, 2, dims, strides, box_rows);
}

#ifdef __CUDACC__
__device__ __forceinline__ void load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* mbar, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                   (uint32_t) __cvta_generic_to_shared(smem_dst)),
               "l"(map), "r"((uint32_t) __cvta_generic_to_shared(mbar)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* mbar, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
                   (uint32_t) __cvta_generic_to_shared(smem_dst)),
               "l"(map), "r"((uint32_t) __cvta_generic_to_shared(mbar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
// Untiled bulk copy of `bytes` (a multiple of 16, both addresses 16-byte aligned) with completion on an mbarrier.
__device__ __forceinline__ void load_bulk(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   (uint32_t) __cvta_generic_to_shared(smem_dst)),
               "l"(gsrc), "r"(bytes), "r"((uint32_t) __cvta_generic_to_shared(mbar))
               : "memory");
}
__device__ __forceinline__ void expect_tx(uint64_t* mbar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"((uint32_t) __cvta_generic_to_shared(mbar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* mbar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"((uint32_t) __cvta_generic_to_shared(mbar)) : "memory");
}
#endif

}  // namespace tma
}  // namespace llsa
