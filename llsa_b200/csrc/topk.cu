// Coarse-to-fine top-k block selection (reference: src/llsa/kernel/triton/topk.py).
//
// coarse_topk_kernel / coarse_topk_mma_kernel (bf16 on the tensor cores)
//                     = gen_sparse_indices (topk.py:6-9): scores pq.pk^T rounded to
//   the input dtype (torch.matmul writes its result in the input dtype), then the
//   top-k columns per row, descending.  The score matrix never leaves the SM: a CTA
//   owns ROWS query rows, streams the keys in chunks through shared memory and
//   carries the running top-k list from chunk to chunk.
// refine_topk_kernel  = compute_topk_indices_sparse (topk.py:102-197): one CTA per
//   level-2 query block scores its bs query rows against the bs*p_topk children of
//   the selected parents in fp32 (not rounded, topk.py:141-143).
// Both pick winners by repeated arg-max with ties going to the smallest index, the
// rule the reference's own kernels use (topk.py:60-62, :159-161).
#include <math_constants.h>

#include "common.cuh"
#include "mma_frag.cuh"

namespace llsa {

constexpr int kMaxTopk = 64;

struct Cand {
  float v;
  int64_t i;
};

__device__ __forceinline__ bool better(float v2, int64_t i2, float v, int64_t i) { return v2 > v || (v2 == v && i2 < i); }

// Scores as the selection sees them: a NaN score ranks as the largest value (torch.topk's order, so a row of
// NaNs still yields topk distinct in-range columns); NaN is thereby free to mark "retired / unused" entries,
// which `better` never prefers.
__device__ __forceinline__ float nan_first(float v) { return v != v ? CUDART_INF_F : v; }

__device__ __forceinline__ Cand warp_argmax(Cand c) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, c.v, o);
    const int64_t i2 = __shfl_xor_sync(0xffffffffu, c.i, o);
    if (better(v2, i2, c.v, c.i)) { c.v = v2; c.i = i2; }
  }
  return c;
}

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int D) {
  float acc = 0.f;
  if constexpr (sizeof(T) == 2) {
    for (int d = 0; d < D; d += 8) {
      uint4 x = ldg128(k + d);
      acc = fmaf(q[d], bf16_lo(x.x), acc); acc = fmaf(q[d + 1], bf16_hi(x.x), acc);
      acc = fmaf(q[d + 2], bf16_lo(x.y), acc); acc = fmaf(q[d + 3], bf16_hi(x.y), acc);
      acc = fmaf(q[d + 4], bf16_lo(x.z), acc); acc = fmaf(q[d + 5], bf16_hi(x.z), acc);
      acc = fmaf(q[d + 6], bf16_lo(x.w), acc); acc = fmaf(q[d + 7], bf16_hi(x.w), acc);
    }
  } else {
    for (int d = 0; d < D; d += 4) {
      float4 x = __ldg(reinterpret_cast<const float4*>(k + d));
      acc = fmaf(q[d], x.x, acc); acc = fmaf(q[d + 1], x.y, acc); acc = fmaf(q[d + 2], x.z, acc); acc = fmaf(q[d + 3], x.w, acc);
    }
  }
  return acc;
}

constexpr int kCoarseRows = 8;
constexpr int kCoarseChunk = 1024;
constexpr int kCoarseThreads = 128;

// pq, pk: contiguous [B*H, M|n, D].  idx out: [B*H, M, topk] int32 or int64.
template <typename T>
__global__ void __launch_bounds__(kCoarseThreads)
coarse_topk_kernel(const T* __restrict__ pq, const T* __restrict__ pk, void* __restrict__ idx_out, int idx64, int64_t M, int64_t n, int D,
                   int topk) {
  extern __shared__ float sm[];
  float* qs = sm;                                   // [ROWS][D]
  float* sc = qs + kCoarseRows * D;                 // [ROWS][CHUNK]
  float* cv = sc + kCoarseRows * kCoarseChunk;      // [ROWS][kMaxTopk] carried values
  int64_t* ci = reinterpret_cast<int64_t*>(cv + kCoarseRows * kMaxTopk);  // carried indices
  float* nv = reinterpret_cast<float*>(ci + kCoarseRows * kMaxTopk);      // [ROWS][kMaxTopk] next list
  int64_t* ni = reinterpret_cast<int64_t*>(nv + kCoarseRows * kMaxTopk);

  const int64_t bh = blockIdx.y;
  const int64_t row0 = (int64_t) blockIdx.x * kCoarseRows;
  const int nrows = (int) min((int64_t) kCoarseRows, M - row0);
  const T* q0 = pq + (bh * M + row0) * D;
  const T* k0 = pk + bh * n * D;
  for (int i = threadIdx.x; i < kCoarseRows * D; i += blockDim.x) qs[i] = (i / D) < nrows ? to_f32<T>(q0[i]) : 0.f;
  for (int i = threadIdx.x; i < kCoarseRows * kMaxTopk; i += blockDim.x) { cv[i] = CUDART_NAN_F; ci[i] = INT64_MAX; }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int64_t base = 0; base < n; base += kCoarseChunk) {
    const int cn = (int) min((int64_t) kCoarseChunk, n - base);
    for (int j = threadIdx.x; j < cn; j += blockDim.x) {
      const T* kr = k0 + (base + j) * D;
#pragma unroll
      for (int r = 0; r < kCoarseRows; ++r) sc[r * kCoarseChunk + j] = nan_first(round_to<T>(dot_row<T>(qs + r * D, kr, D)));
    }
    __syncthreads();
    for (int r = warp; r < nrows; r += nwarps) {
      float* s = sc + r * kCoarseChunk;
      for (int t = 0; t < topk; ++t) {
        Cand best{-CUDART_INF_F, INT64_MAX};
        for (int j = lane; j < cn; j += 32) {
          const float v = s[j];
          if (better(v, base + j, best.v, best.i)) { best.v = v; best.i = base + j; }
        }
        if (lane < topk) {
          const float v = cv[r * kMaxTopk + lane];
          const int64_t i = ci[r * kMaxTopk + lane];
          if (better(v, i, best.v, best.i)) { best.v = v; best.i = i; }
        }
        if (topk > 32 && lane + 32 < topk) {
          const float v = cv[r * kMaxTopk + lane + 32];
          const int64_t i = ci[r * kMaxTopk + lane + 32];
          if (better(v, i, best.v, best.i)) { best.v = v; best.i = i; }
        }
        best = warp_argmax(best);
        if (lane == 0) { nv[r * kMaxTopk + t] = best.v; ni[r * kMaxTopk + t] = best.i; }
        // retire the winner from whichever set holds it
        if (best.i >= base && best.i < base + cn) {
          if (lane == 0) s[best.i - base] = CUDART_NAN_F;
        } else {
          for (int u = lane; u < topk; u += 32)
            if (ci[r * kMaxTopk + u] == best.i) cv[r * kMaxTopk + u] = CUDART_NAN_F;
        }
        __syncwarp();
      }
      for (int u = lane; u < topk; u += 32) { cv[r * kMaxTopk + u] = nv[r * kMaxTopk + u]; ci[r * kMaxTopk + u] = ni[r * kMaxTopk + u]; }
      __syncwarp();
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < nrows * topk; i += blockDim.x) {
    const int r = i / topk, t = i % topk;
    const int64_t o = (bh * M + row0 + r) * topk + t;
    const int64_t v = ci[r * kMaxTopk + t];
    if (idx64) reinterpret_cast<int64_t*>(idx_out)[o] = v;
    else reinterpret_cast<int32_t*>(idx_out)[o] = (int32_t) v;
  }
}

// pq1: contiguous [B*H, M, D] (M query blocks); pk1: contiguous [B*H, Mk, D] (Mk key blocks, Mk != M when the
// queries are a shard of the sequence); p_idx [B*H, M/bs, p_topk] with values in [0, Mk/bs); out [B*H, M, topk].
// MMA = true (bf16, D = 64, bs = 16): the 16 x C score tile comes from mma.sync with fp32
// accumulation of the exact bf16 products, as the reference's tl.dot does.

// ---- coarse selection on the tensor cores (bf16, D = 64, top-k <= 8) ---------------------------
// A CTA owns 64 query rows (16 per warp, the m16 of mma.sync.m16n8k16) and streams the keys through a
// double-buffered shared-memory tile of 64 keys (cp.async).  Scores are rounded to bf16 as torch.matmul
// would store them (topk.py:7); a lane sees columns 2t, 2t+1 (+8) of rows g and g+8 of every 16-key
// block and keeps the best 8 of each of its two rows in sorted registers -- columns arrive in
// increasing order and an equal score never displaces an earlier one, so ties go to the smallest index.
// The four lanes of a quad cover a row between them; their 4 x 8 candidates are merged at the end by
// the warp (two reductions per output, as in the refine kernel below).
constexpr int kCmRows = 64, kCmKeys = 64, kCmTop = 8;

__device__ __forceinline__ uint32_t orderable(float v);

__device__ __forceinline__ void top8_insert(float (&val)[kCmTop], int (&idx)[kCmTop], float v, int i) {
  // NaN ranks first (torch.topk); -inf is lifted above the lists' initial -inf so that every column can enter:
  // a lane always ends with eight real columns, whatever the scores are
  v = v != v ? CUDART_INF_F : fmaxf(v, -3.0e38f);
  if (!(v > val[kCmTop - 1])) return;
  val[kCmTop - 1] = v;
  idx[kCmTop - 1] = i;
#pragma unroll
  for (int u = kCmTop - 1; u > 0; --u) {
    const bool sw = val[u] > val[u - 1];
    const float tv = val[u];
    const int ti = idx[u];
    val[u] = sw ? val[u - 1] : tv;  idx[u] = sw ? idx[u - 1] : ti;
    val[u - 1] = sw ? tv : val[u - 1];  idx[u - 1] = sw ? ti : idx[u - 1];
  }
}

__global__ void __launch_bounds__(128)
coarse_topk_mma_kernel(const bf16* __restrict__ pq, const bf16* __restrict__ pk, void* __restrict__ idx_out, int idx64, int64_t M, int64_t n,
                       int topk) {
  __shared__ __align__(16) bf16 sk[2][kCmKeys * kSmemPitch];
  __shared__ float cand_v[4][16][32];
  __shared__ int cand_i[4][16][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t bh = blockIdx.y, row0 = (int64_t) blockIdx.x * kCmRows + warp * 16;
  const bf16* k0 = pk + bh * n * 64;
  auto stage = [&](int64_t kt, int buf) {               // 64 keys x 128 bytes: 4 chunks of 16 bytes per thread
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int ch = c * 128 + threadIdx.x, r = ch >> 3, col = (ch & 7) * 8;
      cp_async16(&sk[buf][r * kSmemPitch + col], k0 + (kt * kCmKeys + r) * 64 + col);
    }
    cp_async_commit();
  };
  stage(0, 0);
  RowFrag qlo, qhi;
  {
    const int64_t ra = min(row0 + g, M - 1), rb = min(row0 + g + 8, M - 1);     // rows past M are computed and dropped
    load_rowfrag(qlo, pq + (bh * M + ra) * 64, t);
    load_rowfrag(qhi, pq + (bh * M + rb) * 64, t);
  }
  float v0[kCmTop], v1[kCmTop];
  int i0[kCmTop], i1[kCmTop];
#pragma unroll
  for (int u = 0; u < kCmTop; ++u) { v0[u] = v1[u] = -CUDART_INF_F; i0[u] = i1[u] = 0x7FFFFFFF; }
  const int64_t n_tiles = n / kCmKeys;
  for (int64_t kt = 0; kt < n_tiles; ++kt) {
    if (kt + 1 < n_tiles) stage(kt + 1, (int) ((kt + 1) & 1));
    else cp_async_commit();
    cp_async_wait_group<1>();
    __syncthreads();
    const bf16* tile = sk[kt & 1];
#pragma unroll
    for (int blk = 0; blk < 4; ++blk) {
      RowFrag ka, kb;
      load_rowfrag_smem(ka, tile + (blk * 16 + g) * kSmemPitch, t);
      load_rowfrag_smem(kb, tile + (blk * 16 + 8 + g) * kSmemPitch, t);
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
      mma_rows_x_keys(s0, s1, qlo, qhi, ka, kb);
      const int c = (int) (kt * kCmKeys) + blk * 16 + 2 * t;
      top8_insert(v0, i0, round_to<bf16>(s0[0]), c);     top8_insert(v0, i0, round_to<bf16>(s0[1]), c + 1);
      top8_insert(v0, i0, round_to<bf16>(s1[0]), c + 8); top8_insert(v0, i0, round_to<bf16>(s1[1]), c + 9);
      top8_insert(v1, i1, round_to<bf16>(s0[2]), c);     top8_insert(v1, i1, round_to<bf16>(s0[3]), c + 1);
      top8_insert(v1, i1, round_to<bf16>(s1[2]), c + 8); top8_insert(v1, i1, round_to<bf16>(s1[3]), c + 9);
    }
    __syncthreads();          // the buffer read here is refilled by the next iteration's stage()
  }
#pragma unroll
  for (int u = 0; u < kCmTop; ++u) {
    cand_v[warp][g][t * kCmTop + u] = v0[u];      cand_i[warp][g][t * kCmTop + u] = i0[u];
    cand_v[warp][g + 8][t * kCmTop + u] = v1[u];  cand_i[warp][g + 8][t * kCmTop + u] = i1[u];
  }
  __syncwarp();
  for (int r = 0; r < 16; ++r) {
    if (row0 + r >= M) break;
    uint32_t key = orderable(cand_v[warp][r][lane]);
    uint32_t blk = (uint32_t) cand_i[warp][r][lane];
    if (blk == 0x7FFFFFFFu) key = 0u;                    // unused slot
    for (int tt = 0; tt < topk; ++tt) {
      const uint32_t mk = __reduce_max_sync(0xffffffffu, key);
      const uint32_t mb = __reduce_min_sync(0xffffffffu, key == mk ? blk : 0xFFFFFFFFu);
      if (key == mk && blk == mb) { key = 0u; blk = 0xFFFFFFFFu; }
      if (lane == 0) {
        const int64_t o = (bh * M + row0 + r) * topk + tt;
        if (idx64) reinterpret_cast<int64_t*>(idx_out)[o] = (int64_t) mb;
        else reinterpret_cast<int32_t*>(idx_out)[o] = (int32_t) mb;
      }
    }
  }
}

constexpr int kRefineSlots = 8;        // register path of the refine selection: up to 256 candidates per row

// Order-preserving map of a float onto uint32 (larger float <=> larger integer, -0 and +0 share one image so
// that they tie like the float comparison does).
__device__ __forceinline__ uint32_t orderable(float v) {
  uint32_t u = __float_as_uint(v);
  if (u == 0x80000000u) u = 0u;
  if (v != v) u = 0x7FC00000u;           // any NaN ranks above +inf, as in torch.topk
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Refine selection with the candidates of a row in registers: lane l keeps candidates l, l + 32, ... (SLOTS of them) as
// order-preserving 32-bit images of the scores; a round is two warp reductions: the largest score, then the smallest
// block index among its holders.
template <int SLOTS>
__device__ __forceinline__ void refine_select_regs(const float* sc, const int* cand, int C, int bs, int topk, void* idx_out, int idx64,
                                                   int64_t out_row0, int warp, int lane, int nwarps) {
  for (int r = warp; r < bs; r += nwarps) {
    const float* s = sc + r * C;
    uint32_t key[SLOTS], blk[SLOTS];
#pragma unroll
    for (int u = 0; u < SLOTS; ++u) {
      const int j = lane + 32 * u;
      key[u] = (j < C && cand[j] >= 0) ? orderable(s[j]) : 0u;            // 0 is below every real score's image
      blk[u] = j < C ? (uint32_t) cand[j] : 0xFFFFFFFFu;
    }
    for (int t = 0; t < topk; ++t) {
      uint32_t bk = key[0], bb = blk[0];
#pragma unroll
      for (int u = 1; u < SLOTS; ++u)
        if (key[u] > bk || (key[u] == bk && blk[u] < bb)) { bk = key[u]; bb = blk[u]; }
      const uint32_t mk = __reduce_max_sync(0xffffffffu, bk);
      const uint32_t mb = __reduce_min_sync(0xffffffffu, bk == mk ? bb : 0xFFFFFFFFu);
#pragma unroll
      for (int u = 0; u < SLOTS; ++u)
        if (key[u] == mk && blk[u] == mb) { key[u] = 0u; blk[u] = 0xFFFFFFFFu; }      // candidates are distinct blocks: one owner
      if (lane == 0) {
        const int64_t o = (out_row0 + r) * topk + t;
        if (idx64) reinterpret_cast<int64_t*>(idx_out)[o] = (int64_t) mb;
        else reinterpret_cast<int32_t*>(idx_out)[o] = (int32_t) mb;
      }
    }
  }
}

// The same selection for at most 128 candidates and top-k <= 32 with fewer instructions per round: a lane sorts its four
// candidates once (descending score image, ascending block index among equals), so its best is always slot 0; a round is two warp
// reductions, the winner's lane shifts its list up by one, and winner t stays in lane t until one store writes the row's list.
__device__ __forceinline__ void refine_select_sorted4(const float* sc, const int* cand, int C, int bs, int topk, void* idx_out, int idx64,
                                                      int64_t out_row0, int warp, int lane, int nwarps) {
  for (int r = warp; r < bs; r += nwarps) {
    const float* s = sc + r * C;
    uint32_t key[4], blk[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = lane + 32 * u;
      key[u] = (j < C && cand[j] >= 0) ? orderable(s[j]) : 0u;            // 0 is below every real score's image
      blk[u] = j < C ? (uint32_t) cand[j] : 0xFFFFFFFFu;
    }
    auto order = [&](int x, int y) {                     // afterwards slot x is not worse than slot y
      const bool sw = key[y] > key[x] || (key[y] == key[x] && blk[y] < blk[x]);
      const uint32_t kx = sw ? key[y] : key[x], ky = sw ? key[x] : key[y], bx = sw ? blk[y] : blk[x], by = sw ? blk[x] : blk[y];
      key[x] = kx; key[y] = ky; blk[x] = bx; blk[y] = by;
    };
    order(0, 1); order(2, 3); order(0, 2); order(1, 3); order(1, 2);
    uint32_t mine = 0;                                   // winner number `lane` of this row
    for (int t = 0; t < topk; ++t) {
      const uint32_t mk = __reduce_max_sync(0xffffffffu, key[0]);
      const uint32_t mb = __reduce_min_sync(0xffffffffu, key[0] == mk ? blk[0] : 0xFFFFFFFFu);
      if (key[0] == mk && blk[0] == mb) {               // candidates are distinct blocks: one owner
        key[0] = key[1]; blk[0] = blk[1]; key[1] = key[2]; blk[1] = blk[2]; key[2] = key[3]; blk[2] = blk[3];
        key[3] = 0u; blk[3] = 0xFFFFFFFFu;
      }
      if (lane == t) mine = mb;
    }
    if (lane < topk) {
      const int64_t o = (out_row0 + r) * topk + lane;
      if (idx64) reinterpret_cast<int64_t*>(idx_out)[o] = (int64_t) mine;
      else reinterpret_cast<int32_t*>(idx_out)[o] = (int32_t) mine;
    }
  }
}

// Coarse selection of ONE level-2 query block against 64 level-2 keys, inside the refine kernel's CTA (four warps: 16 keys
// each).  The scores are the ones coarse_topk_mma_kernel computes -- the same mma.sync k-steps in the same order on the same
// operands (all 16 A rows hold the query block's row, so every row of the result is that row's), rounded to bf16, NaN first --
// and the winners come out in the same order (descending score, ties to the smaller key), so the fused form returns the
// bits of the two-kernel form while saving its launch and its 64 x 64-score CTAs.
struct FusedCoarse {
  const bf16* pq2;     // [BH, M / bs, 64]
  const bf16* pk2;     // [BH, 64, 64]
  void* pidx_out;      // [BH, M / bs, p_topk]
  int pidx64;
};

__device__ __forceinline__ void coarse_row_64(const FusedCoarse& f, int64_t bh, int64_t P, int64_t n2q, int p_topk, float* sc2, int* s_pidx) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  RowFrag q2, ka, kb;
  load_rowfrag(q2, f.pq2 + (bh * n2q + P) * 64, t);
  const bf16* k0 = f.pk2 + bh * 64 * 64;
  load_rowfrag(ka, k0 + (warp * 16 + g) * 64, t);
  load_rowfrag(kb, k0 + (warp * 16 + 8 + g) * 64, t);
  float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
  mma_rows_x_keys(s0, s1, q2, q2, ka, kb);
  if (g == 0) {
    const int c = warp * 16 + 2 * t;
    sc2[c] = round_to<bf16>(s0[0]); sc2[c + 1] = round_to<bf16>(s0[1]);
    sc2[c + 8] = round_to<bf16>(s1[0]); sc2[c + 9] = round_to<bf16>(s1[1]);
  }
  __syncthreads();
  if (warp == 0) {
    uint32_t key[2], blk[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      float v = sc2[lane + 32 * u];
      v = v != v ? CUDART_INF_F : fmaxf(v, -3.0e38f);       // as top8_insert orders them
      key[u] = orderable(v);
      blk[u] = (uint32_t) (lane + 32 * u);
    }
    uint32_t mine = 0;
    for (int tt = 0; tt < p_topk; ++tt) {
      const uint32_t bk = key[1] > key[0] ? key[1] : key[0];
      const uint32_t bb = key[1] > key[0] ? blk[1] : blk[0];      // equal scores: the smaller key (slot 0) wins
      const uint32_t mk = __reduce_max_sync(0xffffffffu, bk);
      const uint32_t mb = __reduce_min_sync(0xffffffffu, bk == mk ? bb : 0xFFFFFFFFu);
#pragma unroll
      for (int u = 0; u < 2; ++u)
        if (blk[u] == mb) { key[u] = 0u; blk[u] = 0xFFFFFFFFu; }
      if (lane == tt) mine = mb;
    }
    if (lane < p_topk) {
      s_pidx[lane] = (int) mine;
      const int64_t o = (bh * n2q + P) * p_topk + lane;
      if (f.pidx64) reinterpret_cast<int64_t*>(f.pidx_out)[o] = (int64_t) mine;
      else reinterpret_cast<int32_t*>(f.pidx_out)[o] = (int32_t) mine;
    }
  }
  __syncthreads();
}

template <typename T, bool MMA, bool FUSED = false>
__global__ void __launch_bounds__(128)
refine_topk_kernel(const T* __restrict__ pq1, const T* __restrict__ pk1, IdxView p_idx, void* __restrict__ idx_out, int idx64, int64_t M,
                   int64_t Mk, int D, int topk, int p_topk, int bs, FusedCoarse fused) {
  extern __shared__ float sm[];
  __shared__ float s_sc2[64];
  __shared__ int s_pidx[kMaxTopk];
  const int C = p_topk * bs;
  float* qs = sm;                 // [bs][D]
  float* sc = qs + bs * D;        // [bs][C]
  int* cand = reinterpret_cast<int*>(sc + bs * C);  // [C] block index of each candidate
  const int64_t bh = blockIdx.y, P = blockIdx.x, n2q = M / bs, n2 = Mk / bs;
  const T* q0 = pq1 + (bh * M + P * bs) * D;
  const T* k0 = pk1 + bh * Mk * D;
  if constexpr (!MMA)                                    // the tensor-core path takes its query fragments straight from global memory
    for (int i = threadIdx.x; i < bs * D; i += blockDim.x) qs[i] = to_f32<T>(q0[i]);
  if constexpr (FUSED) coarse_row_64(fused, bh, P, n2q, p_topk, s_sc2, s_pidx);
  for (int j = threadIdx.x; j < C; j += blockDim.x) {
    int64_t p = FUSED ? (int64_t) s_pidx[j / bs] : p_idx.at((bh * n2q + P) * p_topk + j / bs);
    p = p < 0 ? 0 : (p >= n2 ? n2 - 1 : p);      // never read outside the tensor
    // a parent listed twice (possible only in a caller-made p_idx) contributes its children once: the selection
    // below relies on distinct candidate blocks; the repeats are marked unused (-1)
    bool repeat = false;
    for (int u = 0; u < j / bs; ++u) {
      int64_t pu = FUSED ? (int64_t) s_pidx[u] : p_idx.at((bh * n2q + P) * p_topk + u);
      pu = pu < 0 ? 0 : (pu >= n2 ? n2 - 1 : pu);
      repeat = repeat || pu == p;
    }
    cand[j] = repeat ? -1 : (int) (p * bs + j % bs);
  }
  __syncthreads();
  if constexpr (MMA) {
    const int warp_ = threadIdx.x >> 5, lane_ = threadIdx.x & 31, g = lane_ >> 2, t = lane_ & 3;
    if constexpr (sizeof(T) == 2) {
      RowFrag qlo, qhi;
      load_rowfrag(qlo, reinterpret_cast<const bf16*>(q0) + g * D, t);
      load_rowfrag(qhi, reinterpret_cast<const bf16*>(q0) + (g + 8) * D, t);
      for (int tile = warp_ * 2; tile < C / 8; tile += 8) {      // two 8-candidate n-tiles per step and warp
        RowFrag ka, kb;
        load_rowfrag(ka, reinterpret_cast<const bf16*>(k0) + (int64_t) max(cand[tile * 8 + g], 0) * D, t);
        load_rowfrag(kb, reinterpret_cast<const bf16*>(k0) + (int64_t) max(cand[tile * 8 + 8 + g], 0) * D, t);
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        mma_rows_x_keys(s0, s1, qlo, qhi, ka, kb);
        // C fragment: rows g / g+8, candidates tile*8 + 2t, +1 (and +8 for the second tile)
        sc[g * C + tile * 8 + 2 * t] = s0[0];       sc[g * C + tile * 8 + 2 * t + 1] = s0[1];
        sc[(g + 8) * C + tile * 8 + 2 * t] = s0[2]; sc[(g + 8) * C + tile * 8 + 2 * t + 1] = s0[3];
        sc[g * C + tile * 8 + 8 + 2 * t] = s1[0];       sc[g * C + tile * 8 + 9 + 2 * t] = s1[1];
        sc[(g + 8) * C + tile * 8 + 8 + 2 * t] = s1[2]; sc[(g + 8) * C + tile * 8 + 9 + 2 * t] = s1[3];
      }
    }
  } else
  // each thread owns a candidate: its key row is read once per group of 16 query rows and
  // meets the rows (broadcast from shared memory) in 16 independent accumulators
  for (int j = threadIdx.x; j < C; j += blockDim.x) {
    const T* kr = k0 + (int64_t) max(cand[j], 0) * D;
    for (int r0 = 0; r0 < bs; r0 += 16) {
      float acc[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) acc[r] = 0.f;
      for (int d = 0; d < D; d += 8) {
        float kv[8];
        if constexpr (sizeof(T) == 2) {
          const uint4 x = ldg128(kr + d);
          kv[0] = bf16_lo(x.x); kv[1] = bf16_hi(x.x); kv[2] = bf16_lo(x.y); kv[3] = bf16_hi(x.y);
          kv[4] = bf16_lo(x.z); kv[5] = bf16_hi(x.z); kv[6] = bf16_lo(x.w); kv[7] = bf16_hi(x.w);
        } else {
          const float4 x = __ldg(reinterpret_cast<const float4*>(kr + d)), y = __ldg(reinterpret_cast<const float4*>(kr + d + 4));
          kv[0] = x.x; kv[1] = x.y; kv[2] = x.z; kv[3] = x.w; kv[4] = y.x; kv[5] = y.y; kv[6] = y.z; kv[7] = y.w;
        }
#pragma unroll
        for (int r = 0; r < 16; ++r) {
          if (r0 + r < bs) {
            const float* qr = qs + (r0 + r) * D + d;
#pragma unroll
            for (int u = 0; u < 8; ++u) acc[r] = fmaf(qr[u], kv[u], acc[r]);
          }
        }
      }
#pragma unroll
      for (int r = 0; r < 16; ++r)
        if (r0 + r < bs) sc[(r0 + r) * C + j] = acc[r];
    }
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  if (C <= 32 * kRefineSlots) {
    if (C <= 128 && topk <= 32) refine_select_sorted4(sc, cand, C, bs, topk, idx_out, idx64, bh * M + P * bs, warp, lane, nwarps);
    else if (C <= 128) refine_select_regs<4>(sc, cand, C, bs, topk, idx_out, idx64, bh * M + P * bs, warp, lane, nwarps);
    else refine_select_regs<kRefineSlots>(sc, cand, C, bs, topk, idx_out, idx64, bh * M + P * bs, warp, lane, nwarps);
    return;
  }
  for (int r = warp; r < bs; r += nwarps) {
    float* s = sc + r * C;
    for (int j = lane; j < C; j += 32) s[j] = cand[j] < 0 ? CUDART_NAN_F : nan_first(s[j]);
    __syncwarp();
    for (int t = 0; t < topk; ++t) {
      Cand best{-CUDART_INF_F, INT64_MAX};
      int bj = -1;
      for (int j = lane; j < C; j += 32) {
        const float v = s[j];           // NaN here = retired or a repeated parent's candidate
        if (better(v, cand[j], best.v, best.i)) { best.v = v; best.i = cand[j]; bj = j; }
      }
      const Cand w = warp_argmax(best);
      if (bj >= 0 && w.i == best.i && w.v == best.v) s[bj] = CUDART_NAN_F;  // candidates are distinct blocks: one owner
      if (lane == 0) {
        const int64_t o = (bh * M + P * bs + r) * topk + t;
        if (idx64) reinterpret_cast<int64_t*>(idx_out)[o] = w.i;
        else reinterpret_cast<int32_t*>(idx_out)[o] = (int32_t) w.i;
      }
      __syncwarp();
    }
  }
}

}  // namespace llsa

using namespace llsa;

extern "C" int llsa_coarse_topk(const LlsaTensor* pq, const LlsaTensor* pk, const LlsaTensor* idx, int topk, void* stream) {
  LLSA_REQUIRE(pq && pk && idx && pq->ptr && pk->ptr && idx->ptr, LLSA_ERR_NULL, "coarse_topk: null tensor");
  LLSA_REQUIRE(pq->ndim == 4 && pk->ndim == 4, LLSA_ERR_SHAPE, "coarse_topk: pq, pk must be [B,H,M,D]");
  const int64_t B = pq->shape[0], H = pq->shape[1], M = pq->shape[2], D = pq->shape[3], n = pk->shape[2];
  LLSA_REQUIRE(is_float_dtype(pq->dtype) && pk->dtype == pq->dtype, LLSA_ERR_DTYPE, "coarse_topk: pq/pk must both be f32 or bf16");
  LLSA_REQUIRE(is_index_dtype(idx->dtype), LLSA_ERR_DTYPE, "coarse_topk: idx must be i32 or i64");
  LLSA_REQUIRE(topk >= 1 && topk <= kMaxTopk && topk <= n, LLSA_ERR_ARG, "coarse_topk: topk=%d must be in 1..min(%d, n=%lld)", topk, kMaxTopk, (long long) n);
  LLSA_REQUIRE(D % 8 == 0 && D <= 512, LLSA_ERR_SHAPE, "coarse_topk: D=%lld must be a multiple of 8, at most 512", (long long) D);
  const int64_t sq[4] = {B, H, M, D}, sk[4] = {B, H, n, D}, si[4] = {B, H, M, topk};
  int rc;
  if ((rc = check_contig(pq, "pq", pq->dtype, 4, sq))) return rc;
  if ((rc = check_contig(pk, "pk", pq->dtype, 4, sk))) return rc;
  if ((rc = check_contig(idx, "idx", idx->dtype, 4, si))) return rc;
  if (B * H * M == 0) return LLSA_OK;
  const size_t smem = (size_t) kCoarseRows * (D + kCoarseChunk) * 4 + (size_t) kCoarseRows * kMaxTopk * (4 + 8) * 2;
  dim3 grid((unsigned) ((M + kCoarseRows - 1) / kCoarseRows), (unsigned) (B * H));
  cudaStream_t st = (cudaStream_t) stream;
  if (pq->dtype == LLSA_F32) {
    LLSA_SMEM_LIMIT((coarse_topk_kernel<float>), smem);
    coarse_topk_kernel<float><<<grid, kCoarseThreads, smem, st>>>((const float*) pq->ptr, (const float*) pk->ptr, idx->ptr,
                                                                   idx->dtype == LLSA_I64, M, n, (int) D, topk);
  } else if (D == 64 && topk <= kCmTop && n % kCmKeys == 0 && n >= topk && ((uintptr_t) pq->ptr % 32) == 0 && ((uintptr_t) pk->ptr % 16) == 0 &&
             n * 64 < (int64_t) 1 << 31) {
    coarse_topk_mma_kernel<<<dim3((unsigned) ((M + kCmRows - 1) / kCmRows), (unsigned) (B * H)), 128, 0, st>>>(
        (const __nv_bfloat16*) pq->ptr, (const __nv_bfloat16*) pk->ptr, idx->ptr, idx->dtype == LLSA_I64, M, n, topk);
  } else {
    LLSA_SMEM_LIMIT((coarse_topk_kernel<__nv_bfloat16>), smem);
    coarse_topk_kernel<__nv_bfloat16><<<grid, kCoarseThreads, smem, st>>>((const __nv_bfloat16*) pq->ptr, (const __nv_bfloat16*) pk->ptr,
                                                                           idx->ptr, idx->dtype == LLSA_I64, M, n, (int) D, topk);
  }
  LLSA_LAUNCH_OK("coarse_topk_kernel");
  return LLSA_OK;
}

extern "C" int llsa_refine_topk(const LlsaTensor* pq1, const LlsaTensor* pk1, const LlsaTensor* p_idx, const LlsaTensor* idx, int topk,
                                int p_topk, int block_size, void* stream) {
  LLSA_REQUIRE(pq1 && pk1 && p_idx && idx && pq1->ptr && pk1->ptr && p_idx->ptr && idx->ptr, LLSA_ERR_NULL, "refine_topk: null tensor");
  LLSA_REQUIRE(pq1->ndim == 4 && pk1->ndim == 4, LLSA_ERR_SHAPE, "refine_topk: pq1, pk1 must be [B,H,M,D]");
  const int64_t B = pq1->shape[0], H = pq1->shape[1], M = pq1->shape[2], D = pq1->shape[3], Mk = pk1->shape[2];
  const int bs = block_size;
  LLSA_REQUIRE(is_float_dtype(pq1->dtype) && pk1->dtype == pq1->dtype, LLSA_ERR_DTYPE, "refine_topk: pq1/pk1 must both be f32 or bf16");
  LLSA_REQUIRE(is_index_dtype(idx->dtype) && is_index_dtype(p_idx->dtype), LLSA_ERR_DTYPE, "refine_topk: index tensors must be i32 or i64");
  LLSA_REQUIRE(bs >= 1 && M % bs == 0 && Mk % bs == 0, LLSA_ERR_ARG, "refine_topk: M=%lld / Mk=%lld not divisible by block size %d", (long long) M,
               (long long) Mk, bs);
  LLSA_REQUIRE(p_topk >= 1 && topk >= 1 && topk <= p_topk * bs && p_topk <= Mk / bs, LLSA_ERR_ARG, "refine_topk: bad topk=%d / p_topk=%d", topk, p_topk);
  LLSA_REQUIRE(D % 8 == 0, LLSA_ERR_SHAPE, "refine_topk: D=%lld must be a multiple of 8", (long long) D);
  const size_t smem = ((size_t) bs * D + (size_t) bs * p_topk * bs + (size_t) p_topk * bs) * 4;
  LLSA_REQUIRE(smem <= 200 * 1024, LLSA_ERR_ARG, "refine_topk: bs*p_topk too large");
  const int64_t sq[4] = {B, H, M, D}, sk[4] = {B, H, Mk, D}, sp[4] = {B, H, M / bs, p_topk}, si[4] = {B, H, M, topk};
  int rc;
  if ((rc = check_contig(pq1, "pq1", pq1->dtype, 4, sq))) return rc;
  if ((rc = check_contig(pk1, "pk1", pq1->dtype, 4, sk))) return rc;
  if ((rc = check_contig(p_idx, "p_idx", p_idx->dtype, 4, sp))) return rc;
  if ((rc = check_contig(idx, "idx", idx->dtype, 4, si))) return rc;
  if (B * H * M == 0) return LLSA_OK;
  dim3 grid((unsigned) (M / bs), (unsigned) (B * H));
  cudaStream_t st = (cudaStream_t) stream;
  if (pq1->dtype == LLSA_F32) {
    LLSA_SMEM_LIMIT((refine_topk_kernel<float, false>), smem);
    refine_topk_kernel<float, false><<<grid, 128, smem, st>>>((const float*) pq1->ptr, (const float*) pk1->ptr, make_idx(p_idx), idx->ptr,
                                                              idx->dtype == LLSA_I64, M, Mk, (int) D, topk, p_topk, bs, FusedCoarse{});
  } else if (D == 64 && bs == 16 && p_topk % 2 == 0 && ((uintptr_t) pq1->ptr % 32) == 0 && ((uintptr_t) pk1->ptr % 32) == 0) {
    LLSA_SMEM_LIMIT((refine_topk_kernel<__nv_bfloat16, true>), smem);
    refine_topk_kernel<__nv_bfloat16, true><<<grid, 128, smem, st>>>((const __nv_bfloat16*) pq1->ptr, (const __nv_bfloat16*) pk1->ptr,
                                                                     make_idx(p_idx), idx->ptr, idx->dtype == LLSA_I64, M, Mk, (int) D, topk, p_topk, bs, FusedCoarse{});
  } else {
    LLSA_SMEM_LIMIT((refine_topk_kernel<__nv_bfloat16, false>), smem);
    refine_topk_kernel<__nv_bfloat16, false><<<grid, 128, smem, st>>>((const __nv_bfloat16*) pq1->ptr, (const __nv_bfloat16*) pk1->ptr,
                                                                      make_idx(p_idx), idx->ptr, idx->dtype == LLSA_I64, M, Mk, (int) D, topk, p_topk, bs, FusedCoarse{});
  }
  LLSA_LAUNCH_OK("refine_topk_kernel");
  return LLSA_OK;
}

extern "C" int llsa_select_two_level(const LlsaTensor* pq1, const LlsaTensor* pk1, const LlsaTensor* pq2, const LlsaTensor* pk2,
                                     const LlsaTensor* p_idx, const LlsaTensor* idx, int topk, int p_topk, int block_size, void* stream) {
  LLSA_REQUIRE(pq1 && pk1 && pq2 && pk2 && p_idx && idx, LLSA_ERR_NULL, "select_two_level: null tensor");
  // the fused form covers the benchmark class: bf16, D = 64, block 16, exactly 64 level-2 keys, at most 8 parents per row
  const bool fusable = pq1->ptr && pk1->ptr && pq2->ptr && pk2->ptr && p_idx->ptr && idx->ptr && pq1->dtype == LLSA_BF16 && pq1->ndim == 4 &&
                       pk2->ndim == 4 && pq1->shape[3] == 64 && block_size == 16 && pk2->shape[2] == 64 && p_topk >= 2 && p_topk <= kCmTop &&
                       p_topk % 2 == 0 && ((uintptr_t) pq1->ptr % 32) == 0 && ((uintptr_t) pk1->ptr % 32) == 0 &&
                       ((uintptr_t) pq2->ptr % 32) == 0 && ((uintptr_t) pk2->ptr % 32) == 0;
  if (!fusable) {
    int rc = llsa_coarse_topk(pq2, pk2, p_idx, p_topk, stream);
    if (rc) return rc;
    return llsa_refine_topk(pq1, pk1, p_idx, idx, topk, p_topk, block_size, stream);
  }
  const int64_t B = pq1->shape[0], H = pq1->shape[1], M = pq1->shape[2], D = 64, Mk = pk1->shape[2];
  const int bs = block_size;
  LLSA_REQUIRE(pk1->dtype == LLSA_BF16 && pq2->dtype == LLSA_BF16 && pk2->dtype == LLSA_BF16, LLSA_ERR_DTYPE, "select_two_level: all pooled tensors must be bf16");
  LLSA_REQUIRE(is_index_dtype(idx->dtype) && is_index_dtype(p_idx->dtype), LLSA_ERR_DTYPE, "select_two_level: index tensors must be i32 or i64");
  LLSA_REQUIRE(M % bs == 0 && Mk == 64 * bs, LLSA_ERR_SHAPE, "select_two_level: M=%lld / Mk=%lld do not fit 64 level-2 keys", (long long) M, (long long) Mk);
  LLSA_REQUIRE(topk >= 1 && topk <= p_topk * bs, LLSA_ERR_ARG, "select_two_level: bad topk=%d / p_topk=%d", topk, p_topk);
  const int64_t sq[4] = {B, H, M, D}, sk[4] = {B, H, Mk, D}, sq2[4] = {B, H, M / bs, D}, sk2[4] = {B, H, 64, D}, sp[4] = {B, H, M / bs, p_topk},
                si[4] = {B, H, M, topk};
  int rc;
  if ((rc = check_contig(pq1, "pq1", LLSA_BF16, 4, sq))) return rc;
  if ((rc = check_contig(pk1, "pk1", LLSA_BF16, 4, sk))) return rc;
  if ((rc = check_contig(pq2, "pq2", LLSA_BF16, 4, sq2))) return rc;
  if ((rc = check_contig(pk2, "pk2", LLSA_BF16, 4, sk2))) return rc;
  if ((rc = check_contig(p_idx, "p_idx", p_idx->dtype, 4, sp))) return rc;
  if ((rc = check_contig(idx, "idx", idx->dtype, 4, si))) return rc;
  if (B * H * M == 0) return LLSA_OK;
  const size_t smem = ((size_t) bs * D + (size_t) bs * p_topk * bs + (size_t) p_topk * bs) * 4;
  FusedCoarse f;
  f.pq2 = (const __nv_bfloat16*) pq2->ptr;
  f.pk2 = (const __nv_bfloat16*) pk2->ptr;
  f.pidx_out = p_idx->ptr;
  f.pidx64 = p_idx->dtype == LLSA_I64;
  LLSA_SMEM_LIMIT((refine_topk_kernel<__nv_bfloat16, true, true>), smem);
  refine_topk_kernel<__nv_bfloat16, true, true><<<dim3((unsigned) (M / bs), (unsigned) (B * H)), 128, smem, (cudaStream_t) stream>>>(
      (const __nv_bfloat16*) pq1->ptr, (const __nv_bfloat16*) pk1->ptr, IdxView{nullptr, 0}, idx->ptr, idx->dtype == LLSA_I64, M, Mk, (int) D, topk,
      p_topk, bs, f);
  LLSA_LAUNCH_OK("refine_topk_kernel<fused>");
  return LLSA_OK;
}
