// Mean pooling along the token axis (reference: src/llsa/kernel/triton/mean_pool.py).
//
// Arithmetic contract (mean_pool.py:26-30): the k rows are added one after the
// other into an accumulator of the INPUT element type, then divided by k, so a
// bf16 tensor is rounded to bf16 after every add.  The kernels below keep the
// accumulator in fp32 registers but round it to T after each add, which gives
// the same bits.
//
// pool_pyramid_kernel writes every pyramid level of q, k and v in one pass over
// HBM: one CTA owns one level-2 row (bs level-1 rows x bs tokens), each thread
// a 16-byte channel group of one level-1 row; the bs loads of a thread are
// independent 128-bit loads, the level-2 row is reduced through shared memory.
#include <string.h>

#include "common.cuh"

namespace llsa {

template <typename T>
struct Vec16;  // 16 bytes of T
template <>
struct Vec16<float> {
  static constexpr int N = 4;
  __device__ static void load(const float* p, float (&v)[4]) {
    float4 x = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
  __device__ static void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <>
struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
    uint4 x = ldg128(p);
    v[0] = bf16_lo(x.x); v[1] = bf16_hi(x.x); v[2] = bf16_lo(x.y); v[3] = bf16_hi(x.y);
    v[4] = bf16_lo(x.z); v[5] = bf16_hi(x.z); v[6] = bf16_lo(x.w); v[7] = bf16_hi(x.w);
  }
  __device__ static void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 x;
    x.x = pack_bf16(v[0], v[1]); x.y = pack_bf16(v[2], v[3]); x.z = pack_bf16(v[4], v[5]); x.w = pack_bf16(v[6], v[7]);
    *reinterpret_cast<uint4*>(p) = x;
  }
};

template <typename T>
struct PyramidArgs {
  View<const T> x[3];
  T* y1[3];  // contiguous [B,H,n1,C]
  T* y2[3];  // contiguous [B,H,n2,C] or nullptr
  int H, C;
  int64_t n1;  // level-1 rows per (b,h)
  int bs;
  // fused RoPE (ROPE kernels only): tensors whose bit is set in rope_mask are rotated by the [N, C] table `freq` of
  // element type T (even columns sin, odd columns cos) before pooling, and the rotated rows are written to xr
  const T* freq;
  int64_t fs;      // table row stride in elements
  View<T> xr[3];
  int rope_mask;
  // fused RMSNorm (NORM kernels only): tensors whose bit is set in norm_mask are normalised over their C channels before the
  // rotation: y = T((x * rsqrt(mean(x^2) + eps)) * w), fp32 arithmetic, w an fp32 [C] weight (nullptr: ones)
  const float* norm_w[3];
  float eps;
  int norm_mask;
};

// RMSNorm of one token row held by `lanes` neighbouring threads (VEC consecutive channels each; lanes a power of two, the
// group aligned inside its warp): squares summed in channel order per thread, then a butterfly over the group.  The
// stand-alone kernel and the fused pooling pass share this function, so their results are identical bit for bit.
template <typename T, int VEC>
__device__ __forceinline__ void rms_normalise(float (&v)[VEC], const float* w, int c, int lanes, int C, float eps) {
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VEC; ++i) ss = __fmaf_rn(v[i], v[i], ss);
  for (int o = 1; o < lanes; o <<= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, o));
  const float rstd = rsqrtf(__fadd_rn(__fdiv_rn(ss, (float) C), eps));
#pragma unroll
  for (int i = 0; i < VEC; ++i) v[i] = round_to<T>(__fmul_rn(__fmul_rn(v[i], rstd), w ? w[c + i] : 1.f));
}

// Interleaved-pair rotation of VEC channels of one token, every product and sum rounded to T separately
// (rope.py:37-47 evaluated as an element-wise tensor program; the same arithmetic as rope_kernel in rope.cu).
template <typename T, int VEC>
__device__ __forceinline__ void rope_rotate(float (&v)[VEC], const float (&f)[VEC]) {
#pragma unroll
  for (int j = 0; j < VEC; j += 2) {
    const float sn = f[j], cs = f[j + 1], xe = v[j], xo = v[j + 1];
    v[j] = round_to<T>(__fsub_rn(round_to<T>(__fmul_rn(cs, xe)), round_to<T>(__fmul_rn(sn, xo))));
    v[j + 1] = round_to<T>(__fadd_rn(round_to<T>(__fmul_rn(sn, xe)), round_to<T>(__fmul_rn(cs, xo))));
  }
}

// blockDim.x = ROWS * (C / VEC); ROWS level-1 rows per CTA (== bs when LEVELS == 2).
template <typename T, int LEVELS, bool ROPE = false, bool NORM = false>
__global__ void pool_pyramid_kernel(PyramidArgs<T> a, int rows_per_cta, int64_t ctas_per_head) {
  constexpr int VEC = Vec16<T>::N;
  extern __shared__ float smem[];  // LEVELS==2: [rows][C] level-1 results as fp32 images of T
  const int ti = blockIdx.y;
  const int64_t bh = blockIdx.x / ctas_per_head;
  const int64_t grp = blockIdx.x % ctas_per_head;
  const int b = (int) (bh / a.H), h = (int) (bh % a.H);
  const int lanes = a.C / VEC;
  const int r = threadIdx.x / lanes, c = (threadIdx.x % lanes) * VEC;
  const int64_t row1 = grp * rows_per_cta + r;  // level-1 row inside (b,h)
  // NORM: every thread of a warp takes part in the row reductions, so rows past the end are computed on the last row and dropped
  const bool live = row1 < a.n1;
  if (live || NORM) {
    const int64_t row1c = live ? row1 : a.n1 - 1;
    const T* xp = a.x[ti].row(b, h, row1c * a.bs) + c;
    const int64_t sn = a.x[ti].sn;
    const bool rope = ROPE && ((a.rope_mask >> ti) & 1);
    const bool norm = NORM && ((a.norm_mask >> ti) & 1);
    const bool writes = (rope || norm) && live;        // the transformed rows go to xr
    T* rp = (rope || norm) ? a.xr[ti].row(b, h, row1c * a.bs) + c : nullptr;
    const T* fp = rope ? a.freq + row1c * a.bs * a.fs + c : nullptr;
    const float* nw = norm ? a.norm_w[ti] : nullptr;
    float acc[VEC];
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = 0.f;
    int t = 0;
    // 8 independent 128-bit loads in flight per thread, consumed in order
    for (; t + 8 <= a.bs; t += 8) {
      float v[8][VEC];
#pragma unroll
      for (int u = 0; u < 8; ++u) Vec16<T>::load(xp + (int64_t) (t + u) * sn, v[u]);
      if (NORM && norm) {
#pragma unroll
        for (int u = 0; u < 8; ++u) rms_normalise<T, VEC>(v[u], nw, c, lanes, a.C, a.eps);
      }
      if (ROPE && rope) {
        float f[8][VEC];
#pragma unroll
        for (int u = 0; u < 8; ++u) Vec16<T>::load(fp + (int64_t) (t + u) * a.fs, f[u]);
#pragma unroll
        for (int u = 0; u < 8; ++u) rope_rotate<T, VEC>(v[u], f[u]);
      }
      if ((ROPE || NORM) && writes) {
#pragma unroll
        for (int u = 0; u < 8; ++u) Vec16<T>::store(rp + (int64_t) (t + u) * a.xr[ti].sn, v[u]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int i = 0; i < VEC; ++i) acc[i] = round_to<T>(acc[i] + v[u][i]);
    }
    for (; t < a.bs; ++t) {
      float v[VEC];
      Vec16<T>::load(xp + (int64_t) t * sn, v);
      if (NORM && norm) rms_normalise<T, VEC>(v, nw, c, lanes, a.C, a.eps);
      if (ROPE && rope) {
        float f[VEC];
        Vec16<T>::load(fp + (int64_t) t * a.fs, f);
        rope_rotate<T, VEC>(v, f);
      }
      if ((ROPE || NORM) && writes) Vec16<T>::store(rp + (int64_t) t * a.xr[ti].sn, v);
#pragma unroll
      for (int i = 0; i < VEC; ++i) acc[i] = round_to<T>(acc[i] + v[i]);
    }
    const float kf = (float) a.bs;
#pragma unroll
    for (int i = 0; i < VEC; ++i) acc[i] = round_to<T>(__fdiv_rn(acc[i], kf));
    if (live) Vec16<T>::store(a.y1[ti] + (bh * a.n1 + row1) * a.C + c, acc);
    if (LEVELS == 2 && live) {
#pragma unroll
      for (int i = 0; i < VEC; ++i) smem[r * a.C + c + i] = acc[i];
    }
  }
  if (LEVELS == 2) {
    __syncthreads();
    // rows_per_cta == bs: the CTA holds exactly the bs level-1 rows of one level-2 row
    for (int ch = threadIdx.x; ch < a.C; ch += blockDim.x) {
      float acc2 = 0.f;
      for (int rr = 0; rr < a.bs; ++rr) acc2 = round_to<T>(acc2 + smem[rr * a.C + ch]);
      acc2 = round_to<T>(__fdiv_rn(acc2, (float) a.bs));
      a.y2[ti][(bh * ctas_per_head + grp) * a.C + ch] = from_f32<T>(acc2);
    }
  }
}

// One output row chunk per thread, any k; VEC = 1 handles channel counts that are not a multiple of 16 bytes.
template <typename T, int VEC>
__global__ void mean_pool_fwd_kernel(View<const T> x, T* y, int H, int C, int64_t S_out, int k, int64_t total) {
  const int lanes = C / VEC;
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
    const int c = (int) (i % lanes) * VEC;
    const int64_t row = i / lanes;
    const int64_t s = row % S_out, bh = row / S_out;
    const T* xp = x.row(bh / H, bh % H, s * k) + c;
    float acc[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
    for (int t = 0; t < k; ++t) {
      float v[VEC];
      if constexpr (VEC == 1) v[0] = to_f32<T>(xp[(int64_t) t * x.sn]);
      else Vec16<T>::load(xp + (int64_t) t * x.sn, v);
#pragma unroll
      for (int j = 0; j < VEC; ++j) acc[j] = round_to<T>(acc[j] + v[j]);
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j) y[row * C + c + j] = from_f32<T>(__fdiv_rn(acc[j], (float) k));
  }
}

// dx[s*k + t] = dy[s] / k  (mean_pool.py:54-58)
template <typename T>
__global__ void mean_pool_bwd_kernel(View<const T> dy, View<T> dx, int H, int C, int64_t S_out, int k, int64_t total) {
  for (int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x; i < total; i += (int64_t) gridDim.x * blockDim.x) {
    const int c = (int) (i % C);
    const int64_t row = i / C;  // output row in [0, B*H*S_out*k)
    const int64_t sx = row % (S_out * k), bh = row / (S_out * k);
    const float g = to_f32<T>(dy.row(bh / H, bh % H, sx / k)[c]);
    dx.row(bh / H, bh % H, sx)[c] = from_f32<T>(__fdiv_rn(g, (float) k));
  }
}

// Stand-alone RMSNorm over the channels of [B,H,S,C] (the q / k normalisation of the attention block): one thread per
// 16-byte channel group, a row's C / VEC threads neighbours in a warp.  y has x's shape, any strides.
template <typename T>
__global__ void rms_norm_kernel(View<const T> x, View<T> y, const float* __restrict__ w, float eps, int H, int C, int64_t S, int64_t rows) {
  constexpr int VEC = Vec16<T>::N;
  const int lanes = C / VEC;
  const int64_t i = blockIdx.x * (int64_t) blockDim.x + threadIdx.x;
  const int64_t row = min(i / lanes, rows - 1);          // rows past the end take part in the reductions and store nothing
  const int c = (int) (i % lanes) * VEC;
  const int64_t s = row % S, bh = row / S;
  float v[VEC];
  Vec16<T>::load(x.row(bh / H, bh % H, s) + c, v);
  rms_normalise<T, VEC>(v, w, c, lanes, C, eps);
  if (i / lanes < rows) Vec16<T>::store(y.row(bh / H, bh % H, s) + c, v);
}

static int grid_for(int64_t total, int block) {
  int64_t g = (total + block - 1) / block;
  const int64_t cap = 148 * 32;
  return (int) (g < 1 ? 1 : (g > cap ? cap : g));
}

template <typename T>
static int launch_pool_fwd(const LlsaTensor* x, const LlsaTensor* y, int k, cudaStream_t st) {
  const int64_t B = x->shape[0], H = x->shape[1], S = x->shape[2], C = x->shape[3];
  const int64_t S_out = S / k;
  constexpr int VEC = Vec16<T>::N;
  const bool vec_ok = (C % VEC == 0) && ((uintptr_t) x->ptr % 16 == 0) && (x->stride[0] % VEC == 0) &&
                      (x->stride[1] % VEC == 0) && (x->stride[2] % VEC == 0);
  View<const T> xv = make_view<const T>(x);
  if (vec_ok) {
    const int64_t total = B * H * S_out * (C / VEC);
    mean_pool_fwd_kernel<T, VEC><<<grid_for(total, 256), 256, 0, st>>>(xv, (T*) y->ptr, (int) H, (int) C, S_out, k, total);
  } else {
    const int64_t total = B * H * S_out * C;
    mean_pool_fwd_kernel<T, 1><<<grid_for(total, 256), 256, 0, st>>>(xv, (T*) y->ptr, (int) H, (int) C, S_out, k, total);
  }
  LLSA_LAUNCH_OK("mean_pool_fwd_kernel");
  return LLSA_OK;
}

}  // namespace llsa

using namespace llsa;

extern "C" int llsa_mean_pool_fwd(const LlsaTensor* x, const LlsaTensor* y, int k, void* stream) {
  LLSA_REQUIRE(x && y && x->ptr && y->ptr, LLSA_ERR_NULL, "mean_pool_fwd: null tensor");
  LLSA_REQUIRE(x->ndim == 4 && y->ndim == 4, LLSA_ERR_SHAPE, "mean_pool_fwd: tensors must be [B,H,S,C]");
  LLSA_REQUIRE(is_float_dtype(x->dtype) && x->dtype == y->dtype, LLSA_ERR_DTYPE, "mean_pool_fwd: dtype must be f32 or bf16 and equal");
  LLSA_REQUIRE(k >= 1 && x->shape[2] % k == 0, LLSA_ERR_ARG, "mean_pool_fwd: S=%lld not divisible by k=%d", (long long) x->shape[2], k);
  LLSA_REQUIRE(x->stride[3] == 1 || x->shape[3] == 1, LLSA_ERR_STRIDE, "mean_pool_fwd: innermost stride must be 1");
  const int64_t shp[4] = {x->shape[0], x->shape[1], x->shape[2] / k, x->shape[3]};
  int rc = check_contig(y, "y", x->dtype, 4, shp);
  if (rc) return rc;
  if (x->shape[0] * x->shape[1] * x->shape[2] * x->shape[3] == 0) return LLSA_OK;
  cudaStream_t st = (cudaStream_t) stream;
  return x->dtype == LLSA_F32 ? launch_pool_fwd<float>(x, y, k, st) : launch_pool_fwd<__nv_bfloat16>(x, y, k, st);
}

extern "C" int llsa_mean_pool_bwd(const LlsaTensor* dy, const LlsaTensor* dx, int k, void* stream) {
  LLSA_REQUIRE(dy && dx && dy->ptr && dx->ptr, LLSA_ERR_NULL, "mean_pool_bwd: null tensor");
  LLSA_REQUIRE(dy->ndim == 4 && dx->ndim == 4, LLSA_ERR_SHAPE, "mean_pool_bwd: tensors must be [B,H,S,C]");
  LLSA_REQUIRE(is_float_dtype(dy->dtype) && dx->dtype == dy->dtype, LLSA_ERR_DTYPE, "mean_pool_bwd: dtype must be f32 or bf16 and equal");
  LLSA_REQUIRE(k >= 1 && dx->shape[0] == dy->shape[0] && dx->shape[1] == dy->shape[1] && dx->shape[2] == dy->shape[2] * k &&
                   dx->shape[3] == dy->shape[3], LLSA_ERR_SHAPE, "mean_pool_bwd: dx must be [B,H,S*k,C]");
  LLSA_REQUIRE((dy->stride[3] == 1 || dy->shape[3] == 1) && (dx->stride[3] == 1 || dx->shape[3] == 1), LLSA_ERR_STRIDE,
               "mean_pool_bwd: innermost stride must be 1");
  const int64_t total = dx->shape[0] * dx->shape[1] * dx->shape[2] * dx->shape[3];
  if (total == 0) return LLSA_OK;
  cudaStream_t st = (cudaStream_t) stream;
  if (dy->dtype == LLSA_F32)
    mean_pool_bwd_kernel<float><<<grid_for(total, 256), 256, 0, st>>>(make_view<const float>(dy), make_view<float>(dx),
                                                                      (int) dx->shape[1], (int) dx->shape[3], dy->shape[2], k, total);
  else
    mean_pool_bwd_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, st>>>(
        make_view<const __nv_bfloat16>(dy), make_view<__nv_bfloat16>(dx), (int) dx->shape[1], (int) dx->shape[3], dy->shape[2], k, total);
  LLSA_LAUNCH_OK("mean_pool_bwd_kernel");
  return LLSA_OK;
}

struct NormSpec {
  int mask;
  const float* w[3];
  float eps;
};

template <typename T, int LEVELS>
static void launch_pyramid_variant(const PyramidArgs<T>& a, dim3 grid, int threads, size_t smem, int rows, int64_t per_head, cudaStream_t st) {
  if (a.rope_mask && a.norm_mask) pool_pyramid_kernel<T, LEVELS, true, true><<<grid, threads, smem, st>>>(a, rows, per_head);
  else if (a.rope_mask) pool_pyramid_kernel<T, LEVELS, true, false><<<grid, threads, smem, st>>>(a, rows, per_head);
  else if (a.norm_mask) pool_pyramid_kernel<T, LEVELS, false, true><<<grid, threads, smem, st>>>(a, rows, per_head);
  else pool_pyramid_kernel<T, LEVELS, false, false><<<grid, threads, smem, st>>>(a, rows, per_head);
}

template <typename T>
static int launch_pyramid(int n, const LlsaTensor* x, const LlsaTensor* y1, const LlsaTensor* y2, int bs, cudaStream_t st,
                          const LlsaTensor* freq = nullptr, int rope_mask = 0, const LlsaTensor* xr = nullptr, const NormSpec* norm = nullptr) {
  constexpr int VEC = Vec16<T>::N;
  PyramidArgs<T> a;
  memset(&a, 0, sizeof(a));
  a.rope_mask = freq ? rope_mask : 0;
  a.norm_mask = norm ? norm->mask : 0;
  if (a.rope_mask) {
    a.freq = (const T*) freq->ptr;
    a.fs = freq->stride[0];
  }
  if (a.norm_mask) {
    a.eps = norm->eps;
    for (int i = 0; i < n; ++i) a.norm_w[i] = norm->w[i];
  }
  for (int i = 0; i < n; ++i)
    if (((a.rope_mask | a.norm_mask) >> i) & 1) a.xr[i] = make_view<T>(&xr[i]);
  const int64_t B = x[0].shape[0], H = x[0].shape[1], N = x[0].shape[2], C = x[0].shape[3];
  for (int i = 0; i < 3; ++i) {
    const int j = i < n ? i : 0;
    a.x[i] = make_view<const T>(&x[j]);
    a.y1[i] = (T*) y1[j].ptr;
    a.y2[i] = y2 ? (T*) y2[j].ptr : nullptr;
  }
  a.H = (int) H; a.C = (int) C; a.n1 = N / bs; a.bs = bs;
  const int lanes = (int) (C / VEC);
  if (y2) {
    const int64_t n2 = a.n1 / bs;
    dim3 grid((unsigned) (B * H * n2), n);
    launch_pyramid_variant<T, 2>(a, grid, bs * lanes, bs * C * sizeof(float), bs, n2, st);
  } else {
    const int rows = 16;
    const int64_t per_head = (a.n1 + rows - 1) / rows;
    dim3 grid((unsigned) (B * H * per_head), n);
    launch_pyramid_variant<T, 1>(a, grid, rows * lanes, 0, rows, per_head, st);
  }
  LLSA_LAUNCH_OK("pool_pyramid_kernel");
  return LLSA_OK;
}

static int pyramid_entry(int n_tensors, const LlsaTensor* x, const LlsaTensor* y1, const LlsaTensor* y2, int block_size, void* stream,
                         const LlsaTensor* freq, int rope_mask, const LlsaTensor* xr, const LlsaTensor* const* norm_w = nullptr, int norm_mask = 0,
                         float eps = 0.f) {
  LLSA_REQUIRE(x && y1, LLSA_ERR_NULL, "pool_pyramid: null tensor list");
  LLSA_REQUIRE(n_tensors >= 1 && n_tensors <= 3, LLSA_ERR_ARG, "pool_pyramid: n_tensors must be 1..3");
  const int bs = block_size;
  LLSA_REQUIRE(bs >= 1, LLSA_ERR_ARG, "pool_pyramid: bad block size");
  const int dt = x[0].dtype;
  LLSA_REQUIRE(is_float_dtype(dt), LLSA_ERR_DTYPE, "pool_pyramid: dtype must be f32 or bf16");
  const int64_t B = x[0].shape[0], H = x[0].shape[1], N = x[0].shape[2], C = x[0].shape[3];
  const int vec = dt == LLSA_F32 ? 4 : 8;
  LLSA_REQUIRE(C % vec == 0 && (int64_t) bs * (C / vec) <= 1024 && 16 * (C / vec) <= 1024, LLSA_ERR_SHAPE,
               "pool_pyramid: channels=%lld unsupported", (long long) C);
  LLSA_REQUIRE(N % bs == 0 && (!y2 || N % ((int64_t) bs * bs) == 0), LLSA_ERR_SHAPE,
               "pool_pyramid: N=%lld not divisible by the pooling factor", (long long) N);
  for (int i = 0; i < n_tensors; ++i) {
    int rc = check_bhnd(&x[i], "x", dt, B, H, N, C);
    if (rc) return rc;
    const int64_t s1[4] = {B, H, N / bs, C};
    rc = check_contig(&y1[i], "y1", dt, 4, s1);
    if (rc) return rc;
    if (y2) {
      const int64_t s2[4] = {B, H, N / bs / bs, C};
      rc = check_contig(&y2[i], "y2", dt, 4, s2);
      if (rc) return rc;
    }
  }
  if (freq) {
    LLSA_REQUIRE(freq->ptr && xr, LLSA_ERR_NULL, "rope_pool_pyramid: null table or output list");
    LLSA_REQUIRE(freq->ndim == 2 && freq->shape[0] == N && freq->shape[1] == C && freq->stride[1] == 1, LLSA_ERR_SHAPE,
                 "rope_pool_pyramid: freq must be [N,C] with unit inner stride");
    LLSA_REQUIRE(freq->dtype == dt, LLSA_ERR_DTYPE, "rope_pool_pyramid: the table must have the dtype of the data");
    LLSA_REQUIRE(C % 2 == 0 && ((uintptr_t) freq->ptr % 16) == 0 && (freq->stride[0] * (int64_t) dtype_size(dt)) % 16 == 0, LLSA_ERR_STRIDE,
                 "rope_pool_pyramid: table rows must be 16-byte aligned");
    LLSA_REQUIRE(rope_mask >= 0 && rope_mask < (1 << n_tensors), LLSA_ERR_ARG, "rope_pool_pyramid: bad rope mask");
    for (int i = 0; i < n_tensors; ++i) {
      if (!((rope_mask >> i) & 1)) continue;
      int rc = check_bhnd(&xr[i], "xr", dt, B, H, N, C);
      if (rc) return rc;
    }
  }
  NormSpec ns;
  memset(&ns, 0, sizeof(ns));
  if (norm_mask) {
    LLSA_REQUIRE(norm_mask > 0 && norm_mask < (1 << n_tensors) && xr, LLSA_ERR_ARG, "rms_rope_pool_pyramid: bad norm mask");
    const int lanes = (int) (C / vec);
    LLSA_REQUIRE(lanes <= 32 && (lanes & (lanes - 1)) == 0, LLSA_ERR_SHAPE, "rms_rope_pool_pyramid: channels=%lld unsupported for the fused norm",
                 (long long) C);
    LLSA_REQUIRE(eps >= 0.f, LLSA_ERR_ARG, "rms_rope_pool_pyramid: eps must not be negative");
    ns.mask = norm_mask;
    ns.eps = eps;
    for (int i = 0; i < n_tensors; ++i) {
      if (!((norm_mask >> i) & 1)) continue;
      const LlsaTensor* w = norm_w ? norm_w[i] : nullptr;
      if (w) {
        const int64_t sw[1] = {C};
        int rc = check_contig(w, "norm weight", LLSA_F32, 1, sw);
        if (rc) return rc;
        ns.w[i] = (const float*) w->ptr;
      }
      if (!((rope_mask >> i) & 1) || !freq) {
        int rc = check_bhnd(&xr[i], "xr", dt, B, H, N, C);
        if (rc) return rc;
      }
    }
  }
  if (B * H * N * C == 0) return LLSA_OK;
  cudaStream_t st = (cudaStream_t) stream;
  const int rc = dt == LLSA_F32 ? launch_pyramid<float>(n_tensors, x, y1, y2, bs, st, freq, rope_mask, xr, norm_mask ? &ns : nullptr)
                                : launch_pyramid<__nv_bfloat16>(n_tensors, x, y1, y2, bs, st, freq, rope_mask, xr, norm_mask ? &ns : nullptr);
  return rc;
}

extern "C" int llsa_pool_pyramid_fwd(int n_tensors, const LlsaTensor* x, const LlsaTensor* y1, const LlsaTensor* y2,
                                     int block_size, void* stream) {
  return pyramid_entry(n_tensors, x, y1, y2, block_size, stream, nullptr, 0, nullptr);
}

extern "C" int llsa_rope_pool_pyramid_fwd(int n_tensors, const LlsaTensor* x, const LlsaTensor* freq, int rope_mask, const LlsaTensor* xr,
                                          const LlsaTensor* y1, const LlsaTensor* y2, int block_size, void* stream) {
  LLSA_REQUIRE(freq, LLSA_ERR_NULL, "rope_pool_pyramid: null table");
  return pyramid_entry(n_tensors, x, y1, y2, block_size, stream, freq, rope_mask, xr);
}


extern "C" int llsa_rms_rope_pool_pyramid_fwd(int n_tensors, const LlsaTensor* x, const LlsaTensor* const* norm_weight, int norm_mask, float eps,
                                              const LlsaTensor* freq, int rope_mask, const LlsaTensor* xr, const LlsaTensor* y1,
                                              const LlsaTensor* y2, int block_size, void* stream) {
  return pyramid_entry(n_tensors, x, y1, y2, block_size, stream, freq, freq ? rope_mask : 0, xr, norm_weight, norm_mask, eps);
}

extern "C" int llsa_rms_norm_fwd(const LlsaTensor* x, const LlsaTensor* weight, float eps, const LlsaTensor* y, void* stream) {
  LLSA_REQUIRE(x && y && x->ptr && y->ptr, LLSA_ERR_NULL, "rms_norm_fwd: null tensor");
  LLSA_REQUIRE(x->ndim == 4 && is_float_dtype(x->dtype), LLSA_ERR_DTYPE, "rms_norm_fwd: x must be a [B,H,S,C] f32 or bf16 tensor");
  const int64_t B = x->shape[0], H = x->shape[1], S = x->shape[2], C = x->shape[3];
  const int vec = x->dtype == LLSA_F32 ? 4 : 8;
  const int64_t lanes = C / vec;
  LLSA_REQUIRE(C % vec == 0 && lanes <= 32 && (lanes & (lanes - 1)) == 0, LLSA_ERR_SHAPE, "rms_norm_fwd: channels=%lld unsupported", (long long) C);
  LLSA_REQUIRE(eps >= 0.f, LLSA_ERR_ARG, "rms_norm_fwd: eps must not be negative");
  int rc;
  if ((rc = check_bhnd(x, "x", x->dtype, B, H, S, C))) return rc;
  if ((rc = check_bhnd(y, "y", x->dtype, B, H, S, C))) return rc;
  const float* w = nullptr;
  if (weight) {
    const int64_t sw[1] = {C};
    if ((rc = check_contig(weight, "weight", LLSA_F32, 1, sw))) return rc;
    w = (const float*) weight->ptr;
  }
  const int64_t rows = B * H * S;
  if (rows == 0) return LLSA_OK;
  const int64_t threads = rows * lanes;
  cudaStream_t st = (cudaStream_t) stream;
  const unsigned grid = (unsigned) ((threads + 255) / 256);
  if (x->dtype == LLSA_F32)
    rms_norm_kernel<float><<<grid, 256, 0, st>>>(make_view<const float>(x), make_view<float>(y), w, eps, (int) H, (int) C, S, rows);
  else
    rms_norm_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(make_view<const __nv_bfloat16>(x), make_view<__nv_bfloat16>(y), w, eps, (int) H, (int) C, S, rows);
  LLSA_LAUNCH_OK("rms_norm_kernel");
  return LLSA_OK;
}
