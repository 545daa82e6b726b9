// Error reporting, argument validation and version of the llsa_b200 C ABI.
#include <stdarg.h>
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "common.cuh"

namespace llsa {

static thread_local char g_err[512] = "no error";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int check_bhnd(const LlsaTensor* t, const char* name, int dtype, int64_t B, int64_t H, int64_t N, int64_t D) {
  LLSA_REQUIRE(t && t->ptr, LLSA_ERR_NULL, "%s: null tensor", name);
  LLSA_REQUIRE(t->dtype == dtype, LLSA_ERR_DTYPE, "%s: dtype %d, expected %d", name, t->dtype, dtype);
  LLSA_REQUIRE(t->ndim == 4 && t->shape[0] == B && t->shape[1] == H && t->shape[2] == N && t->shape[3] == D, LLSA_ERR_SHAPE,
               "%s: shape [%lld,%lld,%lld,%lld], expected [%lld,%lld,%lld,%lld]", name, (long long) t->shape[0],
               (long long) t->shape[1], (long long) t->shape[2], (long long) t->shape[3], (long long) B, (long long) H,
               (long long) N, (long long) D);
  const int64_t per16 = 16 / (int64_t) dtype_size(dtype);
  LLSA_REQUIRE(t->stride[3] == 1 || D == 1, LLSA_ERR_STRIDE, "%s: innermost stride %lld, must be 1", name, (long long) t->stride[3]);
  LLSA_REQUIRE(((uintptr_t) t->ptr % 16) == 0 && (B == 1 || t->stride[0] % per16 == 0) && (H == 1 || t->stride[1] % per16 == 0) &&
                   (N == 1 || t->stride[2] % per16 == 0),
               LLSA_ERR_STRIDE, "%s: rows must start on 16-byte boundaries", name);
  return LLSA_OK;
}

int check_contig(const LlsaTensor* t, const char* name, int dtype, int ndim, const int64_t* shape) {
  LLSA_REQUIRE(t && t->ptr, LLSA_ERR_NULL, "%s: null tensor", name);
  LLSA_REQUIRE(t->dtype == dtype, LLSA_ERR_DTYPE, "%s: dtype %d, expected %d", name, t->dtype, dtype);
  LLSA_REQUIRE(t->ndim == ndim, LLSA_ERR_SHAPE, "%s: ndim %d, expected %d", name, t->ndim, ndim);
  for (int i = 0; i < ndim; ++i)
    LLSA_REQUIRE(t->shape[i] == shape[i], LLSA_ERR_SHAPE, "%s: dim %d is %lld, expected %lld", name, i, (long long) t->shape[i],
                 (long long) shape[i]);
  LLSA_REQUIRE(is_contiguous(t), LLSA_ERR_STRIDE, "%s: must be contiguous", name);
  LLSA_REQUIRE(((uintptr_t) t->ptr % 16) == 0, LLSA_ERR_STRIDE, "%s: base pointer must be 16-byte aligned", name);
  return LLSA_OK;
}

// The dynamic shared-memory limit is an attribute of the kernel, not of a launch: it is only ever raised, under a lock,
// and remembered per (kernel, device), so launches of different sizes from different host threads cannot lower each
// other's limit between the attribute call and the launch.
int raise_smem_limit(const void* kernel, size_t bytes) {
  static std::mutex mu;
  static std::map<std::pair<const void*, int>, size_t> limit;
  int dev = 0;
  LLSA_CUDA_OK(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lock(mu);
  size_t& cur = limit[std::make_pair(kernel, dev)];
  if (bytes > cur) {
    LLSA_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) bytes));
    cur = bytes;
  }
  return LLSA_OK;
}

}  // namespace llsa

extern "C" int llsa_version(void) { return 101; }
extern "C" int llsa_status_check(int32_t w) {
  LLSA_REQUIRE(w == 0, LLSA_ERR_DEVICE_CHECK, "device status 0x%x:%s%s", (unsigned) w,
               (w & LLSA_DEV_BAD_INDEX) ? " a block index outside its range was met;" : "",
               (w & LLSA_DEV_WAIT_EXPIRED) ? " a bounded wait inside a kernel ran out (outputs invalid);" : "");
  return LLSA_OK;
}
extern "C" const char* llsa_last_error_string(void) { return llsa::g_err; }
