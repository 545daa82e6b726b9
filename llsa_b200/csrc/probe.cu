// Issue-rate probe for the tensor instruction the fine-block kernels are built on.
//
// The fine stage multiplies 16 x 16 x 64 tiles that one query block owns alone, so it runs on
// mma.sync.m16n8k16 (bf16 in, fp32 out), not on tcgen05.  Its ceiling is therefore the rate at
// which an SM sub-partition retires that instruction, which this probe measures: every warp of
// the launch issues `ilp` independent accumulator chains `iters` times between two clock64 reads.
#include "common.cuh"

namespace llsa {

template <int ILP>
__global__ void mma_rate_kernel(float* sink, int iters, long long* cycles) {
  float c[ILP][4];
#pragma unroll
  for (int i = 0; i < ILP; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
  const uint32_t a0 = threadIdx.x, a1 = a0 * 3u, a2 = a0 * 5u, a3 = a0 * 7u, b0 = a0 * 11u, b1 = a0 * 13u;
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < ILP; ++i) mma_bf16_16816(c[i], a0, a1, a2, a3, b0, b1);
  }
  const long long t1 = clock64();
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < ILP; ++i) s += c[i][0] + c[i][1] + c[i][2] + c[i][3];
  sink[blockIdx.x * blockDim.x + threadIdx.x] = s;
  if (threadIdx.x == 0 && blockIdx.x == 0) *cycles = t1 - t0;
}

}  // namespace llsa

extern "C" int llsa_probe_mma_rate(int warps_per_sm, int ilp, int iters, int n_sms, float* sink, long long* cycles, void* stream) {
  using namespace llsa;
  LLSA_REQUIRE(warps_per_sm >= 1 && warps_per_sm <= 32 && iters > 0 && n_sms > 0, LLSA_ERR_SHAPE, "mma rate probe: 1..32 warps per SM, iters > 0");
  LLSA_REQUIRE(ilp == 1 || ilp == 2 || ilp == 4 || ilp == 8, LLSA_ERR_SHAPE, "mma rate probe: ilp must be 1, 2, 4 or 8");
  cudaStream_t st = (cudaStream_t) stream;
  const dim3 grid((unsigned) n_sms), block((unsigned) warps_per_sm * 32);
  if (ilp == 1) mma_rate_kernel<1><<<grid, block, 0, st>>>(sink, iters, cycles);
  if (ilp == 2) mma_rate_kernel<2><<<grid, block, 0, st>>>(sink, iters, cycles);
  if (ilp == 4) mma_rate_kernel<4><<<grid, block, 0, st>>>(sink, iters, cycles);
  if (ilp == 8) mma_rate_kernel<8><<<grid, block, 0, st>>>(sink, iters, cycles);
  LLSA_LAUNCH_OK("mma_rate_kernel");
  return LLSA_OK;
}
