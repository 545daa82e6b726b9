// Plain-FFMA attention kernels for any supported dtype (fp32 and bf16).
//
// They follow the reference kernels step by step, including the places where
// the reference rounds to the tensor dtype (q*scale, P before P@V, dS before
// dS@K, k*scale), and serve fp32 tensors -- for which the tensor-core kernels
// do not apply -- as well as a cross-check of the bf16 tensor-core path.
//   attn_fwd_generic   : sparse_attention_res_1.py:9-120 / res_2.py:9-163
//   attn_dq_generic    : preprocess (res_1.py:153-177) + the dQ half of
//                        _attn_bwd_res_dqkv (res_1.py:225-281, res_2.py:287-369)
//   attn_dkv_generic   : the dK/dV half via the CSR (res_1.py:283-327) and the
//                        pooled-key gradients (res_1.py:330-400, res_2.py:418-575)
// Thread layout everywhere: 128 threads = 16 rows x 8 lanes; lane c of row r
// owns the two keys {c, c+8} of a 16-key block and the 8 channels [8c, 8c+8).
#include <string.h>

#include "attn.cuh"

namespace llsa {

constexpr int kLd = kD + 1;  // padded shared-memory row

template <typename T>
__device__ __forceinline__ void load_block_smem(float* dst, const T* src, int64_t stride, float mul, bool round) {
  // 16 rows x 64 channels; thread (r, c) loads channels [8c, 8c+8) of row r
  const int r = threadIdx.x >> 3, c = (threadIdx.x & 7) * 8;
  const T* p = src + (int64_t) r * stride + c;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float x = to_f32<T>(p[i]) * mul;
    dst[r * kLd + c + i] = round ? round_to<T>(x) : x;
  }
}

__device__ __forceinline__ float reduce8_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 4));
  return v;
}
__device__ __forceinline__ float reduce8_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

__device__ __forceinline__ float dot64(const float* a, const float* b) {
  float acc = 0.f;
#pragma unroll 16
  for (int d = 0; d < kD; ++d) acc = fmaf(a[d], b[d], acc);
  return acc;
}

// Resolves key block `i` of the concatenated list [fine | pooled-1 | pooled-2] of a query block.
template <typename T>
__device__ __forceinline__ void key_block(const AttnP<T>& a, int64_t b, int64_t h, int64_t bh, int64_t qb, int i, const T*& kp,
                                          const T*& vp, int64_t& ks, int64_t& vs, float& w, float& kvw) {
  if (i < a.topk) {
    const int64_t j = fine_block(a, bh, qb, i);
    kp = a.k.row(b, h, j * kBS); vp = a.v.row(b, h, j * kBS); ks = a.k.sn; vs = a.v.sn; w = 1.f; kvw = 1.f;
  } else if (i < a.topk + a.p1_blocks) {
    const int64_t j = p1_block(a, bh, qb, i - a.topk);
    kp = a.pk + (bh * a.n1 + j * kBS) * kD; vp = a.pv + (bh * a.n1 + j * kBS) * kD; ks = vs = kD; w = a.w1; kvw = a.kvw1;
  } else {
    const int64_t j = i - a.topk - a.p1_blocks;
    kp = a.pk2 + (bh * a.n2 + j * kBS) * kD; vp = a.pv2 + (bh * a.n2 + j * kBS) * kD; ks = vs = kD; w = a.w2; kvw = a.kvw2;
  }
}

template <typename T>
__global__ void __launch_bounds__(128) attn_fwd_generic(AttnP<T> a) {
  __shared__ float qs[kBS * kLd], ks[kBS * kLd], vs[kBS * kLd], ps[kBS * (kBS + 1)];
  const int64_t qb = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int r = threadIdx.x >> 3, c = threadIdx.x & 7;
  load_block_smem<T>(qs, a.q.row(b, h, qb * kBS), a.q.sn, a.scale, true);   // q *= scale in q.dtype
  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  const int nblk = a.topk + a.p1_blocks + a.p2_blocks;
  for (int i = 0; i < nblk; ++i) {
    const T *kp, *vp;
    int64_t kst, vst;
    float w, kvw;
    key_block(a, b, h, bh, qb, i, kp, vp, kst, vst, w, kvw);
    __syncthreads();
    load_block_smem<T>(ks, kp, kst, 1.f, false);
    load_block_smem<T>(vs, vp, vst, 1.f, false);
    __syncthreads();
    const float s0 = dot64(qs + r * kLd, ks + c * kLd), s1 = dot64(qs + r * kLd, ks + (c + 8) * kLd);
    const float mnew = fmaxf(m, reduce8_max(fmaxf(s0, s1)));
    const float alpha = expf(m - mnew);
    const float p0 = expf(s0 - mnew), p1 = expf(s1 - mnew);
    l = l * alpha + reduce8_sum(p0 + p1) * w;
    ps[r * (kBS + 1) + c] = round_to<T>(p0);        // exp_scores.to(v.dtype)
    ps[r * (kBS + 1) + c + 8] = round_to<T>(p1);
    __syncwarp();
    float pv[8];
#pragma unroll
    for (int d = 0; d < 8; ++d) pv[d] = 0.f;
    for (int kk = 0; kk < kBS; ++kk) {
      const float p = ps[r * (kBS + 1) + kk];
#pragma unroll
      for (int d = 0; d < 8; ++d) pv[d] = fmaf(p, vs[kk * kLd + c * 8 + d], pv[d]);
    }
#pragma unroll
    for (int d = 0; d < 8; ++d) acc[d] = acc[d] * alpha + pv[d] * w;
    m = mnew;
    __syncwarp();
  }
  T* op = a.o.row(b, h, qb * kBS + r) + c * 8;
#pragma unroll
  for (int d = 0; d < 8; ++d) op[d] = from_f32<T>(acc[d] / l);
  if (c == 0) a.lse[bh * a.Nq + qb * kBS + r] = m + logf(l);
}

template <typename T>
__global__ void __launch_bounds__(128) attn_dq_generic(AttnP<T> a) {
  __shared__ float qs[kBS * kLd], dos[kBS * kLd], ks[kBS * kLd], vs[kBS * kLd], dss[kBS * (kBS + 1)];
  const int64_t qb = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int r = threadIdx.x >> 3, c = threadIdx.x & 7;
  load_block_smem<T>(qs, a.q.row(b, h, qb * kBS), a.q.sn, 1.f, false);
  load_block_smem<T>(dos, a.d_o.row(b, h, qb * kBS), a.d_o.sn, 1.f, false);
  __syncthreads();
  float part = 0.f;
  {
    const T* op = a.o_in.row(b, h, qb * kBS + r) + c * 8;
#pragma unroll
    for (int d = 0; d < 8; ++d) part = fmaf(to_f32<T>(op[d]), dos[r * kLd + c * 8 + d], part);
  }
  const float delta = reduce8_sum(part);
  const float lse = a.lse[bh * a.Nq + qb * kBS + r];
  if (c == 0) a.delta[bh * a.Nq + qb * kBS + r] = delta;
  float dq[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) dq[d] = 0.f;
  const int nblk = a.topk + a.p1_blocks + a.p2_blocks;
  for (int i = 0; i < nblk; ++i) {
    const T *kp, *vp;
    int64_t kst, vst;
    float w, kvw;
    key_block(a, b, h, bh, qb, i, kp, vp, kst, vst, w, kvw);
    __syncthreads();
    load_block_smem<T>(ks, kp, kst, a.scale, true);     // arg_k = k * scale, a tensor in k.dtype (res_1.py:420-422)
    load_block_smem<T>(vs, vp, vst, 1.f, false);
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int kk = c + 8 * u;
      const float s = dot64(qs + r * kLd, ks + kk * kLd);
      const float p = expf(s - lse) * w;
      const float dp = dot64(dos + r * kLd, vs + kk * kLd);
      dss[r * (kBS + 1) + kk] = round_to<T>(p * (dp - delta));   // ds.to(k.dtype)
    }
    __syncwarp();
    for (int kk = 0; kk < kBS; ++kk) {
      const float ds = dss[r * (kBS + 1) + kk];
#pragma unroll
      for (int d = 0; d < 8; ++d) dq[d] = fmaf(ds, ks[kk * kLd + c * 8 + d], dq[d]);
    }
    __syncwarp();
  }
  T* dp_ = a.dq.row(b, h, qb * kBS + r) + c * 8;
#pragma unroll
  for (int d = 0; d < 8; ++d) dp_[d] = from_f32<T>(dq[d]);
}

// MODE 0: fine KV block blockIdx.x of head blockIdx.y, query blocks from the CSR; writes dk/dv.
// MODE 1: pooled key tile blockIdx.x of query group blockIdx.z (16 query blocks); atomically
//         accumulates into the fp32 pooled-gradient buffers.
template <typename T, int MODE>
__global__ void __launch_bounds__(128) attn_dkv_generic(AttnP<T> a) {
  __shared__ float qs[kBS * kLd], dos[kBS * kLd], ks[kBS * kLd], vs[kBS * kLd], pt[kBS * (kBS + 1)], dst[kBS * (kBS + 1)];
  __shared__ float lses[kBS], deltas[kBS];
  const int64_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int r = threadIdx.x >> 3, c = threadIdx.x & 7;
  const T *kp, *vp;
  int64_t kst, vst;
  float w = 1.f;
  int64_t list0 = 0, list1 = 0, grp = 0;
  float *gk = nullptr, *gv = nullptr;
  if (MODE == 0) {
    const int64_t j = blockIdx.x;
    kp = a.k.row(b, h, j * kBS); vp = a.v.row(b, h, j * kBS); kst = a.k.sn; vst = a.v.sn;
    if (a.off64) {
      list0 = reinterpret_cast<const int64_t*>(a.offsets)[bh * (a.n1 + 1) + j];
      list1 = reinterpret_cast<const int64_t*>(a.offsets)[bh * (a.n1 + 1) + j + 1];
    } else {
      list0 = reinterpret_cast<const int32_t*>(a.offsets)[bh * (a.n1 + 1) + j];
      list1 = reinterpret_cast<const int32_t*>(a.offsets)[bh * (a.n1 + 1) + j + 1];
    }
    // offsets and list entries handed in by a caller are clamped: nothing is read outside the tensors
    const int64_t E = a.nq1 * a.topk;
    list0 = list0 < 0 ? 0 : (list0 > E ? E : list0);
    list1 = list1 < list0 ? list0 : (list1 > E ? E : list1);
  } else {
    grp = blockIdx.z;
    const int i = blockIdx.x;  // pooled tile of this group: [pooled-1 | pooled-2]
    float wq;
    key_block(a, b, h, bh, grp * kBS, a.topk + i, kp, vp, kst, vst, wq, w);
    const int64_t row0 = (kp - (i < a.p1_blocks ? a.pk : a.pk2)) ;  // element offset of the tile inside its pooled tensor
    gk = (i < a.p1_blocks ? a.dpk : a.dpk2) + row0;
    gv = (i < a.p1_blocks ? a.dpv : a.dpv2) + row0;
    list0 = 0; list1 = kBS;
  }
  load_block_smem<T>(ks, kp, kst, a.scale, true);
  load_block_smem<T>(vs, vp, vst, 1.f, false);
  float dk[8], dv[8];
#pragma unroll
  for (int d = 0; d < 8; ++d) dk[d] = dv[d] = 0.f;
  for (int64_t it = list0; it < list1; ++it) {
    int64_t qb = MODE == 0 ? (int64_t) a.flat[bh * a.nq1 * a.topk + it] : grp * kBS + it;
    qb = qb < 0 ? 0 : (qb >= a.nq1 ? a.nq1 - 1 : qb);
    __syncthreads();
    load_block_smem<T>(qs, a.q.row(b, h, qb * kBS), a.q.sn, 1.f, false);
    load_block_smem<T>(dos, a.d_o.row(b, h, qb * kBS), a.d_o.sn, 1.f, false);
    if (threadIdx.x < kBS) {
      lses[threadIdx.x] = a.lse[bh * a.Nq + qb * kBS + threadIdx.x];
      deltas[threadIdx.x] = a.delta[bh * a.Nq + qb * kBS + threadIdx.x];
    }
    __syncthreads();
    // thread (r, c): key r against query rows c and c+8
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int row = c + 8 * u;
      const float s = dot64(qs + row * kLd, ks + r * kLd);
      const float p = expf(s - lses[row]) * w;
      const float dp = dot64(dos + row * kLd, vs + r * kLd);
      pt[r * (kBS + 1) + row] = round_to<T>(p);
      dst[r * (kBS + 1) + row] = round_to<T>(p * (dp - deltas[row]));
    }
    __syncwarp();
    for (int row = 0; row < kBS; ++row) {
      const float p = pt[r * (kBS + 1) + row], ds = dst[r * (kBS + 1) + row];
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        dv[d] = fmaf(p, dos[row * kLd + c * 8 + d], dv[d]);
        dk[d] = fmaf(ds, qs[row * kLd + c * 8 + d], dk[d]);
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int d = 0; d < 8; ++d) dk[d] *= a.scale;
  if (MODE == 0) {
    const int64_t j = blockIdx.x;
    if (a.fold) {
      // pooling backward folded in: dk += (dpk[j] + dpk2[j/16]/16) / 16  (mean_pool.py:54-58 applied twice)
      const float* g1k = a.dpk + (bh * a.n1 + j) * kD + c * 8;
      const float* g1v = a.dpv + (bh * a.n1 + j) * kD + c * 8;
#pragma unroll
      for (int d = 0; d < 8; ++d) {
        float ek = g1k[d], ev = g1v[d];
        if (a.two_level) {
          ek += a.dpk2[(bh * a.n2 + j / kBS) * kD + c * 8 + d] * (1.f / kBS);
          ev += a.dpv2[(bh * a.n2 + j / kBS) * kD + c * 8 + d] * (1.f / kBS);
        }
        dk[d] += ek * (1.f / kBS);
        dv[d] += ev * (1.f / kBS);
      }
    }
    T* dkp = a.dk.row(b, h, j * kBS + r) + c * 8;
    T* dvp = a.dv.row(b, h, j * kBS + r) + c * 8;
#pragma unroll
    for (int d = 0; d < 8; ++d) { dkp[d] = from_f32<T>(dk[d]); dvp[d] = from_f32<T>(dv[d]); }
  } else {
#pragma unroll
    for (int d = 0; d < 8; ++d) {
      atomicAdd(gk + r * kD + c * 8 + d, dk[d]);
      atomicAdd(gv + r * kD + c * 8 + d, dv[d]);
    }
  }
}

template <typename T>
static int fwd_generic_t(const LlsaAttnArgs* g, cudaStream_t st) {
  AttnP<T> a = build_attn_params<T>(g, false);
  dim3 grid((unsigned) a.nq1, (unsigned) (g->q->shape[0] * a.H));
  attn_fwd_generic<T><<<grid, 128, 0, st>>>(a);
  LLSA_LAUNCH_OK("attn_fwd_generic");
  return LLSA_OK;
}

int zero_pooled_acc(const LlsaAttnArgs* g, cudaStream_t st) {
  const int64_t BH = g->q->shape[0] * g->q->shape[1], n1 = g->k->shape[2] / kBS, n2 = n1 / kBS;
  // accumulators that the caller carved out of one allocation, back to back, are cleared by one memset
  char* ptr[4] = {(char*) g->dpk_acc->ptr, (char*) g->dpv_acc->ptr, g->pk2 ? (char*) g->dpk2_acc->ptr : nullptr,
                  g->pk2 ? (char*) g->dpv2_acc->ptr : nullptr};
  const size_t len[4] = {(size_t) BH * n1 * kD * 4, (size_t) BH * n1 * kD * 4, (size_t) BH * n2 * kD * 4, (size_t) BH * n2 * kD * 4};
  for (int i = 0; i < 4;) {
    if (!ptr[i]) { ++i; continue; }
    size_t run = len[i];
    int j = i + 1;
    while (j < 4 && ptr[j] == ptr[i] + run) run += len[j++];
    LLSA_CUDA_OK(cudaMemsetAsync(ptr[i], 0, run, st));
    i = j;
  }
  return LLSA_OK;
}

template <typename T>
static int bwd_generic_t(const LlsaAttnArgs* g, cudaStream_t st) {
  AttnP<T> a = build_attn_params<T>(g, true);
  const unsigned BH = (unsigned) (g->q->shape[0] * a.H);
  const int mask = g->stage_mask ? g->stage_mask : 7;
  if (mask & 1) {
    int rc = zero_pooled_acc(g, st);
    if (rc) return rc;
    attn_dq_generic<T><<<dim3((unsigned) a.nq1, BH), 128, 0, st>>>(a);
    LLSA_LAUNCH_OK("attn_dq_generic");
  }
  const int ptiles = a.p1_blocks + a.p2_blocks;
  if ((mask & 2) && ptiles > 0) {
    attn_dkv_generic<T, 1><<<dim3((unsigned) ptiles, BH, (unsigned) (a.nq1 / kBS)), 128, 0, st>>>(a);
    LLSA_LAUNCH_OK("attn_dkv_generic<pooled>");
  }
  if (mask & 4) {
    attn_dkv_generic<T, 0><<<dim3((unsigned) a.n1, BH), 128, 0, st>>>(a);
    LLSA_LAUNCH_OK("attn_dkv_generic<fine>");
  }
  return LLSA_OK;
}

int launch_attn_fwd_generic(const LlsaAttnArgs* g, cudaStream_t st) {
  return g->q->dtype == LLSA_F32 ? fwd_generic_t<float>(g, st) : fwd_generic_t<__nv_bfloat16>(g, st);
}
int launch_attn_bwd_generic(const LlsaAttnArgs* g, cudaStream_t st) {
  return g->q->dtype == LLSA_F32 ? bwd_generic_t<float>(g, st) : bwd_generic_t<__nv_bfloat16>(g, st);
}

}  // namespace llsa
