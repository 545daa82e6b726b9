// Shared host/device helpers for the llsa_b200 kernels (sm_100a).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/llsa_b200.h"

namespace llsa {

// ---------------------------------------------------------------- host side
void set_error(const char* fmt, ...);

#define LLSA_REQUIRE(cond, code, ...)     \
  do {                                    \
    if (!(cond)) {                        \
      ::llsa::set_error(__VA_ARGS__);     \
      return (code);                      \
    }                                     \
  } while (0)

#define LLSA_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess) {                                                           \
      ::llsa::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
      return LLSA_ERR_CUDA;                                                             \
    }                                                                                   \
  } while (0)

#define LLSA_LAUNCH_OK(name)                                                            \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess) {                                                           \
      ::llsa::set_error("launch of %s failed: %s", name, cudaGetErrorString(e__));      \
      return LLSA_ERR_CUDA;                                                             \
    }                                                                                   \
  } while (0)

// Raises (never lowers) a kernel's dynamic shared-memory limit on the current device; thread-safe.
int raise_smem_limit(const void* kernel, size_t bytes);
#define LLSA_SMEM_LIMIT(kernel, bytes)                                              \
  do {                                                                              \
    int rc__ = ::llsa::raise_smem_limit((const void*) (kernel), (size_t) (bytes));  \
    if (rc__) return rc__;                                                          \
  } while (0)

// Nominal entries per work range of the fine dK/dV kernel: the index transpose cuts the CSR entry list into ranges of this
// many entries (transpose.cu), one warp of attn_dkv_fine_ring_kernel walks one range (attn_bwd_mma.cu).
constexpr int kRangeEntries = 32;
// Small problems (fewer ranges than about two rounds of the GPU's resident warps) are cut into ranges of half that size, so
// that the dK/dV kernel still fills the SMs: the range size travels with the `ranges` tensor, whose length names it.
constexpr int kRangeEntriesSmall = 16;
// Range size S that a ranges tensor of R ranges over E entries was cut with (0: neither size fits)
inline int range_entries_of(int64_t E, int64_t R) {
  if ((E + kRangeEntries - 1) / kRangeEntries == R) return kRangeEntries;
  if ((E + kRangeEntriesSmall - 1) / kRangeEntriesSmall == R) return kRangeEntriesSmall;
  return 0;
}

inline size_t dtype_size(int dt) {
  switch (dt) {
    case LLSA_F32: return 4;
    case LLSA_BF16: return 2;
    case LLSA_I32: return 4;
    case LLSA_I64: return 8;
  }
  return 0;
}

inline bool is_float_dtype(int dt) { return dt == LLSA_F32 || dt == LLSA_BF16; }
inline bool is_index_dtype(int dt) { return dt == LLSA_I32 || dt == LLSA_I64; }

inline bool is_contiguous(const LlsaTensor* t) {
  int64_t s = 1;
  for (int i = t->ndim - 1; i >= 0; --i) {
    if (t->shape[i] != 1 && t->stride[i] != s) return false;
    s *= t->shape[i];
  }
  return true;
}

// Checks a [B,H,N,D] float tensor: innermost stride 1, rows and base 16-byte aligned.
int check_bhnd(const LlsaTensor* t, const char* name, int dtype, int64_t B, int64_t H, int64_t N, int64_t D);
// Checks a contiguous tensor of the given dtype/shape (ndim entries of shape).
int check_contig(const LlsaTensor* t, const char* name, int dtype, int ndim, const int64_t* shape);

// ------------------------------------------------------------- device views
// A [B,H,N,D] tensor with unit innermost stride; strides in elements.
template <typename T>
struct View {
  T* p;
  int64_t sb, sh, sn;
  __host__ __device__ __forceinline__ T* row(int64_t b, int64_t h, int64_t n) const { return p + b * sb + h * sh + n * sn; }
  __host__ __device__ __forceinline__ T* head(int64_t b, int64_t h) const { return p + b * sb + h * sh; }
};

template <typename T>
inline View<T> make_view(const LlsaTensor* t) {
  View<T> v;
  v.p = reinterpret_cast<T*>(t->ptr);
  v.sb = t->stride[0];
  v.sh = t->stride[1];
  v.sn = t->stride[2];
  return v;
}

// Index tensors may be int32 or int64 (the reference mixes both: topk.py:9,176).
struct IdxView {
  const void* p;
  int is64;
  __device__ __forceinline__ int64_t at(int64_t i) const {
    return is64 ? reinterpret_cast<const int64_t*>(p)[i] : (int64_t) reinterpret_cast<const int32_t*>(p)[i];
  }
};
inline IdxView make_idx(const LlsaTensor* t) {
  IdxView v;
  v.p = t ? t->ptr : nullptr;
  v.is64 = t ? (t->dtype == LLSA_I64) : 0;
  return v;
}

// ------------------------------------------------------------ scalar helpers
template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Round an fp32 value to the precision of T and back (identity for float).
template <typename T>
__device__ __forceinline__ float round_to(float x) { return to_f32<T>(from_f32<T>(x)); }

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);   // .x = lo (low 16 bits), .y = hi
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint4 ldg128(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

}  // namespace llsa
