// Interleaved-pair RoPE apply, forward and backward (reference: src/llsa/kernel/triton/rope.py).
//
// For pair c of token s: sin = F[s,2c], cos = F[s,2c+1] (rope.py:37-40);
//   fwd: y[2c] = cos*x[2c] - sin*x[2c+1];  y[2c+1] = sin*x[2c] + cos*x[2c+1]   (rope.py:46-47)
//   bwd: dx[2c] = cos*dy[2c] + sin*dy[2c+1]; dx[2c+1] = -sin*dy[2c] + cos*dy[2c+1] (rope.py:93-94)
// evaluated in the promoted type of (x, F) with every product and sum rounded
// separately (no FMA contraction), as an element-wise tensor program does.
// One thread moves 16 bytes of x: x and y may have any batch/head/token strides.
#include <type_traits>

#include "common.cuh"

namespace llsa {

template <typename T>
struct Elems16 { static constexpr int N = 16 / sizeof(T); };

template <typename T, int N>
__device__ __forceinline__ void load_vec(const T* p, float (&v)[N]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      float4 x = __ldg(reinterpret_cast<const float4*>(p + i));
      v[i] = x.x; v[i + 1] = x.y; v[i + 2] = x.z; v[i + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; i += 8) {
      uint4 x = ldg128(p + i);
      v[i] = bf16_lo(x.x); v[i + 1] = bf16_hi(x.x); v[i + 2] = bf16_lo(x.y); v[i + 3] = bf16_hi(x.y);
      v[i + 4] = bf16_lo(x.z); v[i + 5] = bf16_hi(x.z); v[i + 6] = bf16_lo(x.w); v[i + 7] = bf16_hi(x.w);
    }
  }
}

template <typename T, int N>
__device__ __forceinline__ void store_vec(T* p, const float (&v)[N]) {
  if constexpr (sizeof(T) == 4) {
#pragma unroll
    for (int i = 0; i < N; i += 4) *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else {
#pragma unroll
    for (int i = 0; i < N; i += 8) {
      uint4 x;
      x.x = pack_bf16(v[i], v[i + 1]); x.y = pack_bf16(v[i + 2], v[i + 3]);
      x.z = pack_bf16(v[i + 4], v[i + 5]); x.w = pack_bf16(v[i + 6], v[i + 7]);
      *reinterpret_cast<uint4*>(p + i) = x;
    }
  }
}

// T: element type of x / y; TF: element type of the table; math in the wider of the two.
template <typename T, typename TF, bool BWD>
__global__ void rope_kernel(View<const T> x, View<T> y, const TF* __restrict__ freq, int64_t fs, int H, int64_t S, int D, int64_t total) {
  constexpr int N = Elems16<T>::N;
  using P = typename std::conditional<(sizeof(TF) > sizeof(T)), TF, T>::type;  // promoted type
  const int lanes = D / N;
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
    const int c = (int) (i % lanes) * N;
    const int64_t row = i / lanes;
    const int64_t s = row % S, bh = row / S;
    float xv[N], fv[N], yv[N];
    load_vec<T, N>(x.row(bh / H, bh % H, s) + c, xv);
    load_vec<TF, N>(freq + s * fs + c, fv);
#pragma unroll
    for (int j = 0; j < N; j += 2) {
      const float sn = fv[j], cs = fv[j + 1], xe = xv[j], xo = xv[j + 1];
      if (!BWD) {
        yv[j] = round_to<P>(__fsub_rn(round_to<P>(__fmul_rn(cs, xe)), round_to<P>(__fmul_rn(sn, xo))));
        yv[j + 1] = round_to<P>(__fadd_rn(round_to<P>(__fmul_rn(sn, xe)), round_to<P>(__fmul_rn(cs, xo))));
      } else {
        yv[j] = round_to<P>(__fadd_rn(round_to<P>(__fmul_rn(cs, xe)), round_to<P>(__fmul_rn(sn, xo))));
        yv[j + 1] = round_to<P>(__fadd_rn(round_to<P>(__fmul_rn(-sn, xe)), round_to<P>(__fmul_rn(cs, xo))));
      }
    }
    store_vec<T, N>(y.row(bh / H, bh % H, s) + c, yv);
  }
}

template <bool BWD>
static int rope_dispatch(const LlsaTensor* x, const LlsaTensor* freq, const LlsaTensor* y, void* stream) {
  const char* nm = BWD ? "rope_bwd" : "rope_fwd";
  LLSA_REQUIRE(x && freq && y && x->ptr && freq->ptr && y->ptr, LLSA_ERR_NULL, "%s: null tensor", nm);
  LLSA_REQUIRE(x->ndim == 4 && freq->ndim == 2, LLSA_ERR_SHAPE, "%s: x must be [B,H,S,D] and freq [S,D]", nm);
  const int64_t B = x->shape[0], H = x->shape[1], S = x->shape[2], D = x->shape[3];
  LLSA_REQUIRE(is_float_dtype(x->dtype) && is_float_dtype(freq->dtype), LLSA_ERR_DTYPE, "%s: dtypes must be f32 or bf16", nm);
  LLSA_REQUIRE(!(x->dtype == LLSA_F32 && freq->dtype == LLSA_BF16), LLSA_ERR_DTYPE, "%s: a bf16 table with f32 data is not supported", nm);
  LLSA_REQUIRE(freq->shape[0] == S && freq->shape[1] == D && (freq->stride[1] == 1), LLSA_ERR_SHAPE, "%s: freq must be [S,D] with unit inner stride", nm);
  const int per16 = x->dtype == LLSA_F32 ? 4 : 8;
  LLSA_REQUIRE(D % per16 == 0 && D % 2 == 0, LLSA_ERR_SHAPE, "%s: D=%lld must be a multiple of %d", nm, (long long) D, per16);
  LLSA_REQUIRE(((uintptr_t) freq->ptr % 16) == 0 && (freq->stride[0] * (int64_t) dtype_size(freq->dtype)) % 16 == 0, LLSA_ERR_STRIDE,
               "%s: freq rows must be 16-byte aligned", nm);
  int rc = check_bhnd(x, "x", x->dtype, B, H, S, D);
  if (rc) return rc;
  rc = check_bhnd(y, "y", x->dtype, B, H, S, D);
  if (rc) return rc;
  const int64_t total = B * H * S * (D / per16);
  if (total == 0) return LLSA_OK;
  int64_t g = (total + 255) / 256;
  if (g > 148 * 32) g = 148 * 32;
  cudaStream_t st = (cudaStream_t) stream;
  if (x->dtype == LLSA_F32)
    rope_kernel<float, float, BWD><<<(int) g, 256, 0, st>>>(make_view<const float>(x), make_view<float>(y), (const float*) freq->ptr,
                                                            freq->stride[0], (int) H, S, (int) D, total);
  else if (freq->dtype == LLSA_BF16)
    rope_kernel<__nv_bfloat16, __nv_bfloat16, BWD><<<(int) g, 256, 0, st>>>(make_view<const __nv_bfloat16>(x), make_view<__nv_bfloat16>(y),
                                                                            (const __nv_bfloat16*) freq->ptr, freq->stride[0], (int) H, S, (int) D, total);
  else
    rope_kernel<__nv_bfloat16, float, BWD><<<(int) g, 256, 0, st>>>(make_view<const __nv_bfloat16>(x), make_view<__nv_bfloat16>(y),
                                                                    (const float*) freq->ptr, freq->stride[0], (int) H, S, (int) D, total);
  LLSA_LAUNCH_OK("rope_kernel");
  return LLSA_OK;
}

}  // namespace llsa

extern "C" int llsa_rope_fwd(const LlsaTensor* x, const LlsaTensor* freq, const LlsaTensor* y, void* stream) {
  return llsa::rope_dispatch<false>(x, freq, y, stream);
}
extern "C" int llsa_rope_bwd(const LlsaTensor* dy, const LlsaTensor* freq, const LlsaTensor* dx, void* stream) {
  return llsa::rope_dispatch<true>(dy, freq, dx, stream);
}
