// Block-sparse LLSA backward on the tensor cores (bf16, D = 64, 16-token blocks).
// Reference: sparse_indices_attn_res_scatter_bwd_v2 (sparse_attention_res_1.py:403-471)
// and sparse_indices_attn_res_scatter_2_2_bwd_v2 (sparse_attention_res_2.py:578-681).
//
// Three kernels on mma.sync.m16n8k16 with the operand fragments of mma_frag.cuh:
//   attn_dq_mma_kernel     one warp per query block: delta = rowsum(o*do) (the
//                          reference's separate _attn_bwd_preprocess pass), then
//                          S, dP and dQ over the fine, pooled-1 and pooled-2 keys.
//                          Pooled K/V tiles are shared by the CTA through shared
//                          memory (cp.async), fine blocks stream from global memory.
//   attn_dkv_pooled_kernel one CTA per group of 16 query blocks (= one parent):
//                          the group's 256 rows of Q and dO (+ lse, delta) are
//                          staged once in shared memory; the warps share out the
//                          pooled key tiles the group attends to, run the transposed
//                          products S^T, dP^T, dV += P^T.dO, dK += dS^T.Q over the
//                          16 query blocks and add the 16x64 results into fp32
//                          accumulators (one red.add per element and group).
//   attn_dq_fine_kernel    the same for the fine blocks alone (the pooled keys then run on
//                          tcgen05); both dQ kernels leave P and dS of every (query block,
//                          selected block) pair in a scratch tensor for the next kernel.
//   attn_dkv_fine_ring_kernel  the CSR of a head is cut into equal windows of 128 entries
//                          (one CTA, 32 entries per warp) so every warp runs the same
//                          number of steps however skewed the fan-in is; an entry is
//                          dV += P^T.dO, dK += dS^T.Q with P, dS read back; tiles of
//                          buckets that straddle a range meet in shared memory / a
//                          global partial tensor (no atomics), and
//   attn_dkv_finish_ld_kernel sums the window partials; every store folds in the pooling
//                          backward (dk += (dpk[j] + dpk2[j/16]/16)/16), one bf16 store.
// The reference multiplies k by scale into new tensors first (res_1.py:420-422);
// here scale rides in the exp2 argument and in the epilogues.
#include <type_traits>

#include "attn.cuh"
#include "mma_frag.cuh"

namespace llsa {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float rowfrag_dot(const RowFrag& x, const RowFrag& y) {
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    acc = fmaf(bf16_lo(x.r[i]), bf16_lo(y.r[i]), acc);
    acc = fmaf(bf16_hi(x.r[i]), bf16_hi(y.r[i]), acc);
  }
  return acc;
}

struct DqRow {
  float L0, L1, delta0, delta1;   // lse (log2 domain) and delta of rows g and g+8
};

// dS (bf16, as A registers) of one 16-key block from its S and dP accumulators
__device__ __forceinline__ void dq_ds(float (&s0)[4], float (&s1)[4], const float (&p0)[4], const float (&p1)[4], const DqRow& r, float sl2,
                                      float lw, uint32_t (&da)[4]) {
  // ds = w * exp(s*scale - lse) * (dp - delta)
  s0[0] = fast_exp2(fmaf(s0[0], sl2, lw - r.L0)) * (p0[0] - r.delta0);
  s0[1] = fast_exp2(fmaf(s0[1], sl2, lw - r.L0)) * (p0[1] - r.delta0);
  s0[2] = fast_exp2(fmaf(s0[2], sl2, lw - r.L1)) * (p0[2] - r.delta1);
  s0[3] = fast_exp2(fmaf(s0[3], sl2, lw - r.L1)) * (p0[3] - r.delta1);
  s1[0] = fast_exp2(fmaf(s1[0], sl2, lw - r.L0)) * (p1[0] - r.delta0);
  s1[1] = fast_exp2(fmaf(s1[1], sl2, lw - r.L0)) * (p1[1] - r.delta0);
  s1[2] = fast_exp2(fmaf(s1[2], sl2, lw - r.L1)) * (p1[2] - r.delta1);
  s1[3] = fast_exp2(fmaf(s1[3], sl2, lw - r.L1)) * (p1[3] - r.delta1);
  da[0] = pack_bf16(s0[0], s0[1]); da[1] = pack_bf16(s0[2], s0[3]); da[2] = pack_bf16(s1[0], s1[1]); da[3] = pack_bf16(s1[2], s1[3]);
}

// The same for a fine block (weight 1), returning P (bf16) as well: both go to the dK/dV stage.
__device__ __forceinline__ void dq_p_ds(float (&s0)[4], float (&s1)[4], const float (&p0)[4], const float (&p1)[4], const DqRow& r, float sl2,
                                        uint32_t (&pa)[4], uint32_t (&da)[4]) {
  s0[0] = fast_exp2(fmaf(s0[0], sl2, -r.L0)); s0[1] = fast_exp2(fmaf(s0[1], sl2, -r.L0));
  s0[2] = fast_exp2(fmaf(s0[2], sl2, -r.L1)); s0[3] = fast_exp2(fmaf(s0[3], sl2, -r.L1));
  s1[0] = fast_exp2(fmaf(s1[0], sl2, -r.L0)); s1[1] = fast_exp2(fmaf(s1[1], sl2, -r.L0));
  s1[2] = fast_exp2(fmaf(s1[2], sl2, -r.L1)); s1[3] = fast_exp2(fmaf(s1[3], sl2, -r.L1));
  pa[0] = pack_bf16(s0[0], s0[1]); pa[1] = pack_bf16(s0[2], s0[3]); pa[2] = pack_bf16(s1[0], s1[1]); pa[3] = pack_bf16(s1[2], s1[3]);
  da[0] = pack_bf16(s0[0] * (p0[0] - r.delta0), s0[1] * (p0[1] - r.delta0));
  da[1] = pack_bf16(s0[2] * (p0[2] - r.delta1), s0[3] * (p0[3] - r.delta1));
  da[2] = pack_bf16(s1[0] * (p1[0] - r.delta0), s1[1] * (p1[1] - r.delta0));
  da[3] = pack_bf16(s1[2] * (p1[2] - r.delta1), s1[3] * (p1[3] - r.delta1));
}

// Hands P and dS of a (query block, selected block) pair to the dK/dV stage.  That stage multiplies their transposes
// (rows = keys) from the left: dV += P^T.dO, dK += dS^T.Q.  The A operand of those products holds, in lane (g,t),
// (key g, queries 2t,2t+1), (key g+8, same), (key g, queries 8+2t,9+2t), (key g+8, same); the registers here hold
// (query g, keys 2t,2t+1), (query g+8, ..), (query g, keys 8+2t,..), (query g+8, ..): each is an 8x8 matrix spread over
// the warp, and transposing the four (movmatrix) and swapping the middle two gives exactly the A operand.  One uint4 per
// lane and matrix: 1 KB per pair, written and later read in full 512-byte rows.
__device__ __forceinline__ void store_pds(uint4* dst, const uint32_t (&pa)[4], const uint32_t (&da)[4], int lane) {
  uint4 p, d;
  p.x = movmatrix_trans(pa[0]); p.y = movmatrix_trans(pa[2]); p.z = movmatrix_trans(pa[1]); p.w = movmatrix_trans(pa[3]);
  d.x = movmatrix_trans(da[0]); d.y = movmatrix_trans(da[2]); d.z = movmatrix_trans(da[1]); d.w = movmatrix_trans(da[3]);
  dst[lane] = p;
  dst[32 + lane] = d;
}

struct GlobalKV {
  const bf16* k;
  const bf16* v;
  int64_t ks, vs;
  float lw;
};

__device__ __forceinline__ GlobalKV global_kv(const AttnP<bf16>& a, int64_t b, int64_t h, int64_t bh, int64_t qb, int gi, int my_fine,
                                              int n_smem_tiles, float lw1, float lw2) {
  GlobalKV r;
  if (gi < a.topk) {
    const int64_t j = __shfl_sync(0xffffffffu, my_fine, gi);
    r.k = a.k.row(b, h, j * kBS); r.v = a.v.row(b, h, j * kBS); r.ks = a.k.sn; r.vs = a.v.sn; r.lw = 0.f;
  } else {
    const int ip = n_smem_tiles + gi - a.topk;
    if (ip < a.p1_blocks) {
      const int64_t off = (bh * a.n1 + p1_block(a, bh, qb, ip) * kBS) * kD;
      r.k = a.pk + off; r.v = a.pv + off; r.lw = lw1;
    } else {
      const int64_t off = (bh * a.n2 + (int64_t) (ip - a.p1_blocks) * kBS) * kD;
      r.k = a.pk2 + off; r.v = a.pv2 + off; r.lw = lw2;
    }
    r.ks = r.vs = kD;
  }
  return r;
}

__device__ __forceinline__ void stage_pooled_tiles_bwd(const AttnP<bf16>& a, int64_t bh, int64_t qb0, int n_tiles, bf16* sk, bf16* sv) {
  for (int c = threadIdx.x; c < n_tiles * kBS * 8; c += blockDim.x) {
    const int tile = c >> 7, row = (c >> 3) & 15, ch = (c & 7) * 8;
    const bf16 *gk, *gv;
    if (tile < a.p1_blocks) {
      const int64_t off = (bh * a.n1 + p1_block(a, bh, qb0, tile) * kBS + row) * kD + ch;
      gk = a.pk + off; gv = a.pv + off;
    } else {
      const int64_t off = (bh * a.n2 + (int64_t) (tile - a.p1_blocks) * kBS + row) * kD + ch;
      gk = a.pk2 + off; gv = a.pv2 + off;
    }
    const int so = (tile * kBS + row) * kSmemPitch + ch;
    cp_async16(sk + so, gk);
    cp_async16(sv + so, gv);
  }
  cp_async_commit();
}

template <int NW>
__global__ void __launch_bounds__(NW * 32, 4) attn_dq_mma_kernel(AttnP<bf16> a, int n_smem_tiles) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sk = reinterpret_cast<bf16*>(smem_raw);
  bf16* sv = sk + n_smem_tiles * kBS * kSmemPitch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t qb0 = (int64_t) blockIdx.x * NW, qb = qb0 + warp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  stage_pooled_tiles_bwd(a, bh, qb0, n_smem_tiles, sk, sv);

  const int my_fine = lane < a.topk ? (int) fine_block(a, bh, qb, lane) : 0;
  const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
  const float sl2 = a.scale * kLog2e;

  RowFrag qlo, qhi, dlo, dhi;
  load_rowfrag(qlo, a.q.row(b, h, qb * kBS + g), t);
  load_rowfrag(qhi, a.q.row(b, h, qb * kBS + g + 8), t);
  load_rowfrag(dlo, a.d_o.row(b, h, qb * kBS + g), t);
  load_rowfrag(dhi, a.d_o.row(b, h, qb * kBS + g + 8), t);
  DqRow row;
  {
    RowFrag olo, ohi;
    load_rowfrag(olo, a.o_in.row(b, h, qb * kBS + g), t);
    load_rowfrag(ohi, a.o_in.row(b, h, qb * kBS + g + 8), t);
    row.delta0 = quad_sum(rowfrag_dot(olo, dlo));
    row.delta1 = quad_sum(rowfrag_dot(ohi, dhi));
  }
  const int64_t rbase = bh * a.Nq + qb * kBS;
  if (t == 0) { a.delta[rbase + g] = row.delta0; a.delta[rbase + g + 8] = row.delta1; }
  row.L0 = a.lse[rbase + g] * kLog2e;
  row.L1 = a.lse[rbase + g + 8] * kLog2e;

  float dq[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) dq[j][0] = dq[j][1] = dq[j][2] = dq[j][3] = 0.f;

  const int n_pooled = a.p1_blocks + a.p2_blocks;
  const int n_glob = a.topk + (n_pooled - n_smem_tiles);
  {
    GlobalKV r = global_kv(a, b, h, bh, qb, 0, my_fine, n_smem_tiles, lw1, lw2);
    RowFrag k0, k1, v0, v1;
    load_rowfrag(k0, r.k + (int64_t) g * r.ks, t);
    load_rowfrag(k1, r.k + (int64_t) (g + 8) * r.ks, t);
    load_rowfrag(v0, r.v + (int64_t) g * r.vs, t);
    load_rowfrag(v1, r.v + (int64_t) (g + 8) * r.vs, t);
    for (int gi = 0; gi < n_glob; ++gi) {
      const float lw = r.lw;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
      mma_rows_x_keys(s0, s1, qlo, qhi, k0, k1);
      mma_rows_x_keys(p0, p1, dlo, dhi, v0, v1);
      uint32_t tk0[8], tk1[8];   // K transposed in registers: the B operand of dQ += dS.K, no second load
#pragma unroll
      for (int i = 0; i < 8; ++i) { tk0[i] = movmatrix_trans(k0.r[i]); tk1[i] = movmatrix_trans(k1.r[i]); }
      if (gi + 1 < n_glob) {
        r = global_kv(a, b, h, bh, qb, gi + 1, my_fine, n_smem_tiles, lw1, lw2);
        load_rowfrag(k0, r.k + (int64_t) g * r.ks, t);
        load_rowfrag(k1, r.k + (int64_t) (g + 8) * r.ks, t);
        load_rowfrag(v0, r.v + (int64_t) g * r.vs, t);
        load_rowfrag(v1, r.v + (int64_t) (g + 8) * r.vs, t);
      }
      uint32_t da[4];
      if (gi < a.topk && a.pds) {           // a fine block: P and dS also go to the dK/dV stage
        uint32_t pa[4];
        dq_p_ds(s0, s1, p0, p1, row, sl2, pa, da);
        store_pds(a.pds + ((bh * a.nq1 + qb) * a.topk + gi) * 64, pa, da, lane);
      } else {
        dq_ds(s0, s1, p0, p1, row, sl2, lw, da);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) mma_bf16_16816(dq[i], da[0], da[1], da[2], da[3], tk0[i], tk1[i]);
    }
  }
  cp_async_wait_all();
  __syncthreads();
  for (int ip = 0; ip < n_smem_tiles; ++ip) {
    const bf16* tk = sk + ip * kBS * kSmemPitch;
    const bf16* tv = sv + ip * kBS * kSmemPitch;
    RowFrag k0, k1, v0, v1;
    load_rowfrag_smem(k0, tk + g * kSmemPitch, t);
    load_rowfrag_smem(k1, tk + (g + 8) * kSmemPitch, t);
    load_rowfrag_smem(v0, tv + g * kSmemPitch, t);
    load_rowfrag_smem(v1, tv + (g + 8) * kSmemPitch, t);
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
    mma_rows_x_keys(s0, s1, qlo, qhi, k0, k1);
    mma_rows_x_keys(p0, p1, dlo, dhi, v0, v1);
    uint32_t da[4];
    dq_ds(s0, s1, p0, p1, row, sl2, ip < a.p1_blocks ? lw1 : lw2, da);
    mma_x_rowfrag_t(dq, da[0], da[1], da[2], da[3], k0, k1);
  }
  store_acc_row_t<0>(a.dq.row(b, h, qb * kBS + g), dq, t, a.scale);
  store_acc_row_t<1>(a.dq.row(b, h, qb * kBS + g + 8), dq, t, a.scale);
}

// Fine blocks only (the pooled keys are on the tcgen05 kernel): the selected K / V blocks go through a per-warp
// cp.async ring in shared memory, two blocks ahead, instead of being held in registers one block ahead.
constexpr int kDqStages = 3;

template <int NW>
__global__ void __launch_bounds__(NW * 32, 4) attn_dq_fine_kernel(AttnP<bf16> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  bf16* ring = reinterpret_cast<bf16*>(smem_raw) + warp * (kDqStages * 2 * kRingTileElems);
  const int64_t qb = (int64_t) blockIdx.x * NW + warp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int my_fine = lane < a.topk ? (int) fine_block(a, bh, qb, lane) : 0;
  const float sl2 = a.scale * kLog2e;
  const int n_glob = a.topk;
  // a lane copies the same four 16-byte chunks of every K tile and of every V tile: offsets computed once
  int off_k[4], off_v[4], off_s[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 4 + (lane >> 3), c = lane & 7;
    off_k[i] = r * (int) a.k.sn + c * 8;
    off_v[i] = r * (int) a.v.sn + c * 8;
    off_s[i] = r * 64 + ((c ^ (r & 7)) << 3);
  }
  const bf16* kb0 = a.k.row(b, h, 0);
  const bf16* vb0 = a.v.row(b, h, 0);
  const int64_t kblk = (int64_t) kBS * a.k.sn, vblk = (int64_t) kBS * a.v.sn;
  auto issue = [&](int i) {
    const int64_t j = __shfl_sync(0xffffffffu, my_fine, i);
    bf16* stage = ring + (i % kDqStages) * 2 * kRingTileElems;
    const bf16* kp = kb0 + j * kblk;
    const bf16* vp = vb0 + j * vblk;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      cp_async16(stage + off_s[u], kp + off_k[u]);
      cp_async16(stage + kRingTileElems + off_s[u], vp + off_v[u]);
    }
  };
#pragma unroll
  for (int s = 0; s < kDqStages - 1; ++s) {
    if (s < n_glob) issue(s);
    cp_async_commit();
  }
  RowFrag qlo, qhi, dlo, dhi;
  load_rowfrag(qlo, a.q.row(b, h, qb * kBS + g), t);
  load_rowfrag(qhi, a.q.row(b, h, qb * kBS + g + 8), t);
  load_rowfrag(dlo, a.d_o.row(b, h, qb * kBS + g), t);
  load_rowfrag(dhi, a.d_o.row(b, h, qb * kBS + g + 8), t);
  DqRow row;
  {
    RowFrag olo, ohi;
    load_rowfrag(olo, a.o_in.row(b, h, qb * kBS + g), t);
    load_rowfrag(ohi, a.o_in.row(b, h, qb * kBS + g + 8), t);
    row.delta0 = quad_sum(rowfrag_dot(olo, dlo));
    row.delta1 = quad_sum(rowfrag_dot(ohi, dhi));
  }
  const int64_t rbase = bh * a.Nq + qb * kBS;
  if (t == 0) { a.delta[rbase + g] = row.delta0; a.delta[rbase + g + 8] = row.delta1; }
  row.L0 = a.lse[rbase + g] * kLog2e;
  row.L1 = a.lse[rbase + g + 8] * kLog2e;
  float dq[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) dq[j][0] = dq[j][1] = dq[j][2] = dq[j][3] = 0.f;
  for (int gi = 0; gi < n_glob; ++gi) {
    cp_async_wait_group<kDqStages - 2>();       // block gi has landed (this lane's chunks) ...
    __syncwarp();                               // ... and everybody else's; the stage read last time is free
    if (gi + kDqStages - 1 < n_glob) issue(gi + kDqStages - 1);
    cp_async_commit();
    const bf16* tk = ring + (gi % kDqStages) * 2 * kRingTileElems;
    RowFrag k0, k1, v0, v1;
    load_rowfrag_ring(k0, tk, g, t);
    load_rowfrag_ring(k1, tk, g + 8, t);
    load_rowfrag_ring(v0, tk + kRingTileElems, g, t);
    load_rowfrag_ring(v1, tk + kRingTileElems, g + 8, t);
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
    mma_rows_x_keys(s0, s1, qlo, qhi, k0, k1);
    mma_rows_x_keys(p0, p1, dlo, dhi, v0, v1);
    uint32_t da[4];
    if (a.pds) {                            // P and dS also go to the dK/dV stage
      uint32_t pa[4];
      dq_p_ds(s0, s1, p0, p1, row, sl2, pa, da);
      store_pds(a.pds + ((bh * a.nq1 + qb) * a.topk + gi) * 64, pa, da, lane);
    } else {
      dq_ds(s0, s1, p0, p1, row, sl2, 0.f, da);
    }
    mma_x_rowfrag_t(dq, da[0], da[1], da[2], da[3], k0, k1);      // K transposed in registers (movmatrix)
  }
  store_acc_row_t<0>(a.dq.row(b, h, qb * kBS + g), dq, t, a.scale);
  store_acc_row_t<1>(a.dq.row(b, h, qb * kBS + g + 8), dq, t, a.scale);
}

// P^T and dS^T (bf16, as A registers) of one (key tile) x (query block) pair from the
// transposed accumulators: rows = keys (g, g+8), columns = query rows (tile 0: 0..7, tile 1: 8..15).
__device__ __forceinline__ void dkv_p_ds(float (&s0)[4], float (&s1)[4], float (&e0)[4], float (&e1)[4], float2 la, float2 lb, float2 da,
                                         float2 db, float sl2, float lw, uint32_t (&pa)[4], uint32_t (&ea)[4]) {
  const float a0 = lw - la.x * kLog2e, a1 = lw - la.y * kLog2e, b0 = lw - lb.x * kLog2e, b1 = lw - lb.y * kLog2e;
  // c0: (key g, row 2t)  c1: (key g, row 2t+1)  c2: (key g+8, row 2t)  c3: (key g+8, row 2t+1)
  s0[0] = fast_exp2(fmaf(s0[0], sl2, a0)); s0[1] = fast_exp2(fmaf(s0[1], sl2, a1));
  s0[2] = fast_exp2(fmaf(s0[2], sl2, a0)); s0[3] = fast_exp2(fmaf(s0[3], sl2, a1));
  s1[0] = fast_exp2(fmaf(s1[0], sl2, b0)); s1[1] = fast_exp2(fmaf(s1[1], sl2, b1));
  s1[2] = fast_exp2(fmaf(s1[2], sl2, b0)); s1[3] = fast_exp2(fmaf(s1[3], sl2, b1));
  e0[0] = s0[0] * (e0[0] - da.x); e0[1] = s0[1] * (e0[1] - da.y); e0[2] = s0[2] * (e0[2] - da.x); e0[3] = s0[3] * (e0[3] - da.y);
  e1[0] = s1[0] * (e1[0] - db.x); e1[1] = s1[1] * (e1[1] - db.y); e1[2] = s1[2] * (e1[2] - db.x); e1[3] = s1[3] * (e1[3] - db.y);
  pa[0] = pack_bf16(s0[0], s0[1]); pa[1] = pack_bf16(s0[2], s0[3]); pa[2] = pack_bf16(s1[0], s1[1]); pa[3] = pack_bf16(s1[2], s1[3]);
  ea[0] = pack_bf16(e0[0], e0[1]); ea[1] = pack_bf16(e0[2], e0[3]); ea[2] = pack_bf16(e1[0], e1[1]); ea[3] = pack_bf16(e1[2], e1[3]);
}

template <int NW>
__global__ void __launch_bounds__(NW * 32, 1) attn_dkv_pooled_kernel(AttnP<bf16> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sq = reinterpret_cast<bf16*>(smem_raw);              // [256][kSmemPitch]
  bf16* sd = sq + kBS * kBS * kSmemPitch;                    // [256][kSmemPitch]
  float* sl = reinterpret_cast<float*>(sd + kBS * kBS * kSmemPitch);   // lse [256]
  float* sdel = sl + kBS * kBS;                                        // delta [256]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const float sl2 = a.scale * kLog2e;
  // stage the group's 256 rows of Q and dO
  const int64_t row0 = grp * kBS * kBS;
  for (int c = threadIdx.x; c < kBS * kBS * 8; c += blockDim.x) {
    const int r = c >> 3, ch = (c & 7) * 8;
    cp_async16(sq + r * kSmemPitch + ch, a.q.row(b, h, row0 + r) + ch);
    cp_async16(sd + r * kSmemPitch + ch, a.d_o.row(b, h, row0 + r) + ch);
  }
  cp_async_commit();
  for (int r = threadIdx.x; r < kBS * kBS; r += blockDim.x) {
    sl[r] = a.lse[bh * a.Nq + row0 + r];
    sdel[r] = a.delta[bh * a.Nq + row0 + r];
  }
  cp_async_wait_all();
  __syncthreads();

  const int ntiles = a.p1_blocks + a.p2_blocks;
  for (int i = warp; i < ntiles; i += NW) {
    const bf16 *kp, *vp;
    float *gk, *gv;
    float lw;
    if (i < a.p1_blocks) {
      const int64_t off = (bh * a.n1 + p1_block(a, bh, grp * kBS, i) * kBS) * kD;
      kp = a.pk + off; vp = a.pv + off; gk = a.dpk + off; gv = a.dpv + off; lw = log2f(a.kvw1);
    } else {
      const int64_t off = (bh * a.n2 + (int64_t) (i - a.p1_blocks) * kBS) * kD;
      kp = a.pk2 + off; vp = a.pv2 + off; gk = a.dpk2 + off; gv = a.dpv2 + off; lw = log2f(a.kvw2);
    }
    RowFrag ka, kb, va, vb;
    load_rowfrag(ka, kp + g * kD, t);
    load_rowfrag(kb, kp + (g + 8) * kD, t);
    load_rowfrag(va, vp + g * kD, t);
    load_rowfrag(vb, vp + (g + 8) * kD, t);
    float dk[8][4], dv[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j) dk[j][0] = dk[j][1] = dk[j][2] = dk[j][3] = dv[j][0] = dv[j][1] = dv[j][2] = dv[j][3] = 0.f;
#pragma unroll 1
    for (int qi = 0; qi < kBS; ++qi) {
      const bf16* tq = sq + qi * kBS * kSmemPitch;
      const bf16* td = sd + qi * kBS * kSmemPitch;
      float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, e0[4] = {0.f, 0.f, 0.f, 0.f}, e1[4] = {0.f, 0.f, 0.f, 0.f};
      RowFrag q0, q1, d0, d1;
      load_rowfrag_smem(q0, tq + g * kSmemPitch, t);
      load_rowfrag_smem(q1, tq + (g + 8) * kSmemPitch, t);
      mma_rows_x_keys(s0, s1, ka, kb, q0, q1);
      load_rowfrag_smem(d0, td + g * kSmemPitch, t);
      load_rowfrag_smem(d1, td + (g + 8) * kSmemPitch, t);
      mma_rows_x_keys(e0, e1, va, vb, d0, d1);
      const float2 la = *reinterpret_cast<const float2*>(sl + qi * kBS + 2 * t), lb = *reinterpret_cast<const float2*>(sl + qi * kBS + 8 + 2 * t);
      const float2 da = *reinterpret_cast<const float2*>(sdel + qi * kBS + 2 * t), db = *reinterpret_cast<const float2*>(sdel + qi * kBS + 8 + 2 * t);
      uint32_t pa[4], ea[4];
      dkv_p_ds(s0, s1, e0, e1, la, lb, da, db, sl2, lw, pa, ea);
      // the same tiles, transposed in registers, are the B operands of dV and dK
      mma_x_rowfrag_t(dv, pa[0], pa[1], pa[2], pa[3], d0, d1);
      mma_x_rowfrag_t(dk, ea[0], ea[1], ea[2], ea[3], q0, q1);
    }
    // a lane owns channels [16t, 16t+16) of key rows g and g+8: four 128-bit reductions per row
    red_acc_row_t<0>(gk + g * kD, dk, t, a.scale);
    red_acc_row_t<1>(gk + (g + 8) * kD, dk, t, a.scale);
    red_acc_row_t<0>(gv + g * kD, dv, t, 1.f);
    red_acc_row_t<1>(gv + (g + 8) * kD, dv, t, 1.f);
  }
}

// ---- fine dK/dV: ranges of the CSR entry list, whatever the fan-in ------------------------------
// The CSR of a head lists, bucket after bucket (KV block after KV block), the query blocks that selected each KV
// block.  Fan-in is very uneven (0 ... >150 on correlated inputs), so the work is cut by ENTRIES, not by buckets: the
// index transpose cuts the list into ranges of nominally kRangeEntries entries, one per warp, moving a cut that would
// fall inside a bucket of at most kRangeEntries entries to that bucket's start.  Most buckets are therefore finished
// by one warp; longer ones are cut at multiples of kRangeEntries and their pieces meet in shared memory (same CTA) or
// in the `partial` scratch (summed in window order by the finish kernel).  No atomics: bit-reproducible.
constexpr int kTileFloats = 64 * 32;            // a parked dK + dV tile pair: 64 accumulators x 32 lanes (8 KB)

__device__ __forceinline__ int64_t csr_off(const AttnP<bf16>& a, int64_t bh, int64_t j) {
  const int64_t o = bh * (a.n1 + 1) + j;
  return a.off64 ? reinterpret_cast<const int64_t*>(a.offsets)[o] : (int64_t) reinterpret_cast<const int32_t*>(a.offsets)[o];
}

// A parked dK + dV tile pair is [16 accumulator quads][32 lanes] float4: every access of a warp is one 128-bit
// instruction over 512 contiguous bytes.  (A warp gets about eight loads per memory round trip, however many it has issued:
// the same tile as 64 32-bit loads cost the finish kernel eight round trips per piece in a clock trace.)
__device__ __forceinline__ void tile_to_mem(float* s, const float (&dk)[8][4], const float (&dv)[8][4], int lane) {
  float4* s4 = reinterpret_cast<float4*>(s) + lane;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    s4[u * 32] = make_float4(dk[u][0], dk[u][1], dk[u][2], dk[u][3]);
    s4[(8 + u) * 32] = make_float4(dv[u][0], dv[u][1], dv[u][2], dv[u][3]);
  }
}
__device__ __forceinline__ void tile_add_mem(const float* s, float (&dk)[8][4], float (&dv)[8][4], int lane) {
  const float4* s4 = reinterpret_cast<const float4*>(s) + lane;
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    const float4 x = s4[u * 32], y = s4[(8 + u) * 32];
    dk[u][0] += x.x; dk[u][1] += x.y; dk[u][2] += x.z; dk[u][3] += x.w;
    dv[u][0] += y.x; dv[u][1] += y.y; dv[u][2] += y.z; dv[u][3] += y.w;
  }
}
// The same from global memory with all 16 loads in flight before the first add: for the finish kernel, whose warps do
// little else than wait for these loads.
__device__ __forceinline__ void tile_add_mem_batched(const float* s, float (&dk)[8][4], float (&dv)[8][4], int lane) {
  const float4* s4 = reinterpret_cast<const float4*>(s) + lane;
  float4 x[8], y[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) { x[u] = __ldcg(s4 + u * 32); y[u] = __ldcg(s4 + (8 + u) * 32); }
#pragma unroll
  for (int u = 0; u < 8; ++u) {
    dk[u][0] += x[u].x; dk[u][1] += x[u].y; dk[u][2] += x[u].z; dk[u][3] += x[u].w;
    dv[u][0] += y[u].x; dv[u][1] += y[u].y; dv[u][2] += y[u].z; dv[u][3] += y[u].w;
  }
}
__device__ __forceinline__ void tile_zero(float (&dk)[8][4], float (&dv)[8][4]) {
#pragma unroll
  for (int u = 0; u < 8; ++u) dk[u][0] = dk[u][1] = dk[u][2] = dk[u][3] = dv[u][0] = dv[u][1] = dv[u][2] = dv[u][3] = 0.f;
}

// ---- fine dK/dV kernel ------------------------------------------------------------------------------
// dV_j += P^T.dO and dK_j += dS^T.Q over the query blocks that selected KV block j (reference:
// sparse_attention_res_2.py:371-415, the dK/dV half of _attn_bwd_res_dqkv).  P and dS are NOT recomputed here: the dQ
// stage has left them, already transposed into A-operand registers, in `pds` (store_pds), so an entry costs two
// 512-byte loads, the Q and dO tiles of its query block and 16 MMAs; K, V, lse and delta are not touched.
//   * The Q / dO tiles come through a per-warp cp.async ring of kRingFineStages stages, three entries ahead, and are
//     read with ldmatrix.trans (the B operand of a contraction over the tile's 16 rows).
//   * The P^T / dS^T registers of the entry three ahead are requested with plain 128-bit loads into a rotating set
//     of register buffers (two CTAs of four warps per SM leave 255 registers per thread).
//   * A warp owns one range of the entry list, a CTA four consecutive ranges (its window).  The index transpose cuts
//     the ranges so that a bucket of up to kRangeEntries entries is never split and hands over each range's first
//     bucket, so a warp starts without a search.  A longer bucket is cut at multiples of kRangeEntries: a warp parks
//     the tile of a bucket it shares with EARLIER warps in its shared-memory slot; the tile it shares with later warps
//     stays in its accumulators until the CTA has synchronised and is then completed from their slots; pieces of
//     buckets that straddle windows go to the `partial` scratch and attn_dkv_finish_ld_kernel adds them in window order.
//   * The pooled-gradient rows a finished tile folds in (the pooling backward) are requested into registers when
//     the bucket begins and parked in shared memory right before the store.
// Accumulator layout (ldmatrix): tile u holds channels 8u + 2t, 8u + 2t + 1 of keys g (c0, c1) and g + 8 (c2, c3).
constexpr int kRingWarps = 4;                   // warps per CTA, each on its own range; two CTAs per SM
constexpr int kRingFineStages = 4;
constexpr int kRingFineStageBytes = 2 * kRingTileElems * (int) sizeof(bf16);           // Q tile, dO tile
constexpr int kRingFoldBytes = 4 * 64 * (int) sizeof(float);                           // per warp: dpk, dpv, dpk2, dpv2 rows of the bucket

// Pooling-backward fold and scale for the ldmatrix accumulator layout: afterwards dk / dv hold the final fp32 values.
// The four gradient rows of KV block j (64 fp32 each) arrive with two 128-bit loads per lane -- lanes 0..15 the 16 quads
// of the key rows, lanes 16..31 of the value rows, level 1 and level 2 -- so that a warp can have the next block's rows
// under way (8 registers) while it finishes this one.
struct FoldRows { float4 e, f; };
__device__ __forceinline__ FoldRows dkv_fold_rows_load(const AttnP<bf16>& a, int64_t bh, int64_t j, int lane) {
  FoldRows r;
  r.e = r.f = make_float4(0.f, 0.f, 0.f, 0.f);
  if (a.fold) {
    const int half = lane >> 4, q = lane & 15;
    r.e = __ldcg(reinterpret_cast<const float4*>((half ? a.dpv : a.dpk) + (bh * a.n1 + j) * kD + 4 * q));
    if (a.two_level) r.f = __ldcg(reinterpret_cast<const float4*>((half ? a.dpv2 : a.dpk2) + (bh * a.n2 + j / kBS) * kD + 4 * q));
  }
  return r;
}
__device__ __forceinline__ void dkv_fine_fold_apply(const AttnP<bf16>& a, const FoldRows& r, float (&dk)[8][4], float (&dv)[8][4], int lane) {
  if (a.fold) {
    const int t = lane & 3;
    float4 e = r.e;
    if (a.two_level) { e.x += r.f.x * (1.f / kBS); e.y += r.f.y * (1.f / kBS); e.z += r.f.z * (1.f / kBS); e.w += r.f.w * (1.f / kBS); }
    const bool hi = (t & 1) != 0;                 // channels 8u + 2t, 8u + 2t + 1: quad 2u + t/2, its first or second pair
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int src = 2 * u + (t >> 1);
      const float kx0 = __shfl_sync(0xffffffffu, e.x, src), ky0 = __shfl_sync(0xffffffffu, e.y, src);
      const float kx1 = __shfl_sync(0xffffffffu, e.z, src), ky1 = __shfl_sync(0xffffffffu, e.w, src);
      const float vx0 = __shfl_sync(0xffffffffu, e.x, 16 + src), vy0 = __shfl_sync(0xffffffffu, e.y, 16 + src);
      const float vx1 = __shfl_sync(0xffffffffu, e.z, 16 + src), vy1 = __shfl_sync(0xffffffffu, e.w, 16 + src);
      const float2 ek = make_float2(hi ? kx1 : kx0, hi ? ky1 : ky0), ev = make_float2(hi ? vx1 : vx0, hi ? vy1 : vy0);
      dk[u][0] = dk[u][0] * a.scale + ek.x * (1.f / kBS); dk[u][1] = dk[u][1] * a.scale + ek.y * (1.f / kBS);
      dk[u][2] = dk[u][2] * a.scale + ek.x * (1.f / kBS); dk[u][3] = dk[u][3] * a.scale + ek.y * (1.f / kBS);
      dv[u][0] += ev.x * (1.f / kBS); dv[u][1] += ev.y * (1.f / kBS); dv[u][2] += ev.x * (1.f / kBS); dv[u][3] += ev.y * (1.f / kBS);
    }
  } else {
#pragma unroll
    for (int u = 0; u < 8; ++u) { dk[u][0] *= a.scale; dk[u][1] *= a.scale; dk[u][2] *= a.scale; dk[u][3] *= a.scale; }
  }
}

// The same from this warp's copy of the four gradient rows in shared memory ([dpk | dpv | dpk2 | dpv2] x 64 fp32, fetched with
// cp.async when the bucket began); sa_fold already includes the lane's 8t bytes.
__device__ __forceinline__ void dkv_fine_fold_smem(const AttnP<bf16>& a, uint32_t sa_fold, float (&dk)[8][4], float (&dv)[8][4]) {
  if (a.fold) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      float2 ek, ev;
      if (u == 0) { ek = lds64f<0>(sa_fold); ev = lds64f<256>(sa_fold); }
      if (u == 1) { ek = lds64f<32>(sa_fold); ev = lds64f<256 + 32>(sa_fold); }
      if (u == 2) { ek = lds64f<64>(sa_fold); ev = lds64f<256 + 64>(sa_fold); }
      if (u == 3) { ek = lds64f<96>(sa_fold); ev = lds64f<256 + 96>(sa_fold); }
      if (u == 4) { ek = lds64f<128>(sa_fold); ev = lds64f<256 + 128>(sa_fold); }
      if (u == 5) { ek = lds64f<160>(sa_fold); ev = lds64f<256 + 160>(sa_fold); }
      if (u == 6) { ek = lds64f<192>(sa_fold); ev = lds64f<256 + 192>(sa_fold); }
      if (u == 7) { ek = lds64f<224>(sa_fold); ev = lds64f<256 + 224>(sa_fold); }
      if (a.two_level) {
        float2 fk, fv;
        if (u == 0) { fk = lds64f<512>(sa_fold); fv = lds64f<768>(sa_fold); }
        if (u == 1) { fk = lds64f<512 + 32>(sa_fold); fv = lds64f<768 + 32>(sa_fold); }
        if (u == 2) { fk = lds64f<512 + 64>(sa_fold); fv = lds64f<768 + 64>(sa_fold); }
        if (u == 3) { fk = lds64f<512 + 96>(sa_fold); fv = lds64f<768 + 96>(sa_fold); }
        if (u == 4) { fk = lds64f<512 + 128>(sa_fold); fv = lds64f<768 + 128>(sa_fold); }
        if (u == 5) { fk = lds64f<512 + 160>(sa_fold); fv = lds64f<768 + 160>(sa_fold); }
        if (u == 6) { fk = lds64f<512 + 192>(sa_fold); fv = lds64f<768 + 192>(sa_fold); }
        if (u == 7) { fk = lds64f<512 + 224>(sa_fold); fv = lds64f<768 + 224>(sa_fold); }
        ek.x += fk.x * (1.f / kBS); ek.y += fk.y * (1.f / kBS); ev.x += fv.x * (1.f / kBS); ev.y += fv.y * (1.f / kBS);
      }
      dk[u][0] = dk[u][0] * a.scale + ek.x * (1.f / kBS); dk[u][1] = dk[u][1] * a.scale + ek.y * (1.f / kBS);
      dk[u][2] = dk[u][2] * a.scale + ek.x * (1.f / kBS); dk[u][3] = dk[u][3] * a.scale + ek.y * (1.f / kBS);
      dv[u][0] += ev.x * (1.f / kBS); dv[u][1] += ev.y * (1.f / kBS); dv[u][2] += ev.x * (1.f / kBS); dv[u][3] += ev.y * (1.f / kBS);
    }
  } else {
#pragma unroll
    for (int u = 0; u < 8; ++u) { dk[u][0] *= a.scale; dk[u][1] *= a.scale; dk[u][2] *= a.scale; dk[u][3] *= a.scale; }
  }
}

// The staging half of the store below: dk / dv already hold the final fp32 values.
template <int SB>
__device__ __forceinline__ void dkv_tile_store_staged(const AttnP<bf16>& a, int64_t b, int64_t h, int64_t j, float (&dk)[8][4], float (&dv)[8][4],
                                                      const uint32_t (&sa_m)[4], uint32_t sa_cp0, uint32_t sa_cp1, int lane) {
  constexpr int TB = kRingTileElems * (int) sizeof(bf16);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    stsm_x4<SB>(sa_m[c], pack_bf16(dk[2 * c][0], dk[2 * c][1]), pack_bf16(dk[2 * c][2], dk[2 * c][3]),
                pack_bf16(dk[2 * c + 1][0], dk[2 * c + 1][1]), pack_bf16(dk[2 * c + 1][2], dk[2 * c + 1][3]));
    stsm_x4<SB + TB>(sa_m[c], pack_bf16(dv[2 * c][0], dv[2 * c][1]), pack_bf16(dv[2 * c][2], dv[2 * c][3]),
                     pack_bf16(dv[2 * c + 1][0], dv[2 * c + 1][1]), pack_bf16(dv[2 * c + 1][2], dv[2 * c + 1][3]));
  }
  __syncwarp();
  bf16* kp = a.dk.row(b, h, j * kBS + (lane >> 3)) + (lane & 7) * 8;
  bf16* vp = a.dv.row(b, h, j * kBS + (lane >> 3)) + (lane & 7) * 8;
  const int64_t ks = 4 * a.dk.sn, vs = 4 * a.dv.sn;
  uint4 x;
  lds128<SB>(x.x, x.y, x.z, x.w, sa_cp0);             *reinterpret_cast<uint4*>(kp) = x;
  lds128<SB + 512>(x.x, x.y, x.z, x.w, sa_cp1);       *reinterpret_cast<uint4*>(kp + ks) = x;
  lds128<SB + 1024>(x.x, x.y, x.z, x.w, sa_cp0);      *reinterpret_cast<uint4*>(kp + 2 * ks) = x;
  lds128<SB + 1536>(x.x, x.y, x.z, x.w, sa_cp1);      *reinterpret_cast<uint4*>(kp + 3 * ks) = x;
  lds128<SB + TB>(x.x, x.y, x.z, x.w, sa_cp0);        *reinterpret_cast<uint4*>(vp) = x;
  lds128<SB + TB + 512>(x.x, x.y, x.z, x.w, sa_cp1);  *reinterpret_cast<uint4*>(vp + vs) = x;
  lds128<SB + TB + 1024>(x.x, x.y, x.z, x.w, sa_cp0); *reinterpret_cast<uint4*>(vp + 2 * vs) = x;
  lds128<SB + TB + 1536>(x.x, x.y, x.z, x.w, sa_cp1); *reinterpret_cast<uint4*>(vp + 3 * vs) = x;
  __syncwarp();
}


// Store of a finished tile through a free ring stage at byte offset SB: stmatrix writes the bf16 tile in the ring's swizzled row
// layout (the ldmatrix addresses sa_m), every lane reads back four 16-byte chunks per tensor (the cp.async addresses sa_cp0 /
// sa_cp1) and eight lanes write one whole 128-byte row: full sectors, 8 store instructions instead of 32.
template <int SB>
__device__ __forceinline__ void dkv_fine_store_staged(const AttnP<bf16>& a, int64_t b, int64_t h, int64_t j, float (&dk)[8][4],
                                                      float (&dv)[8][4], const uint32_t (&sa_m)[4], uint32_t sa_cp0, uint32_t sa_cp1,
                                                      uint32_t sa_fold, int lane) {
  dkv_fine_fold_smem(a, sa_fold, dk, dv);
  dkv_tile_store_staged<SB>(a, b, h, j, dk, dv, sa_m, sa_cp0, sa_cp1, lane);
}
__global__ void __launch_bounds__(kRingWarps * 32, 2) attn_dkv_fine_ring_kernel(AttnP<bf16> a, float* __restrict__ partial) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // the swizzle arithmetic below works on absolute shared addresses: start at a 128-byte boundary (the launch adds 128 bytes)
  unsigned char* smem = smem_raw + ((128u - ((uint32_t) __cvta_generic_to_shared(smem_raw) & 127u)) & 127u);
  float* slots = reinterpret_cast<float*>(smem);            // [kRingWarps][kTileFloats]: tile of the bucket a warp shares with earlier warps
  __shared__ int s_head_bucket[kRingWarps];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = lane & 3;
  // per warp: the ring stages, then its copy of the pooled-gradient rows the current bucket folds in (4 rows x 256 bytes)
  constexpr int kWarpBytes = kRingFineStages * kRingFineStageBytes + kRingFoldBytes;
  constexpr int kFoldOff = kRingFineStages * kRingFineStageBytes;
  unsigned char* ring = smem + kRingWarps * kTileFloats * sizeof(float) + warp * kWarpBytes;
  const int64_t bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int E = (int) (a.nq1 * a.topk), n1 = (int) a.n1;
  const int R = (E + a.range_entries - 1) / a.range_entries;
  // entries the CSR really holds: fewer than E when the transpose dropped out-of-range indices; ranges and offsets handed in
  // by a caller are not trusted further than these clamps and the bounds on the bucket walk below
  const int E_used = (int) min((int64_t) E, max((int64_t) 0, csr_off(a, bh, n1)));
  auto cut = [&](int r) { return r < R ? min(max(__ldcg(&a.ranges[bh * R + r].x), 0), E_used) : E_used; };
  const int r = blockIdx.x * kRingWarps + warp;           // this warp's range; the CTA's window is its four ranges
  const int cb = cut(blockIdx.x * kRingWarps), ce = max(cut((blockIdx.x + 1) * kRingWarps), cb);
  const int rb = min(max(cut(r), cb), ce), re = min(max(cut(r + 1), rb), ce);
  const int32_t* fl = a.flat + bh * (int64_t) E;
  const int32_t* pr = a.pairs + bh * (int64_t) E;
  if (threadIdx.x < kRingWarps) s_head_bucket[threadIdx.x] = -1;
  __syncthreads();

  // Per-lane shared addresses, computed once (the ring is 128-byte aligned, so the chunk index of an address is its bits 4..6
  // and a swizzle partner is one XOR away):
  //   sa_cp0 / sa_cp1  where this lane's cp.async chunks of tile rows (lane/8) + {0, 8} / + {4, 12} land
  //   sa_m[c]          ldmatrix.trans row address for output channels 16c..16c+15
  const uint32_t ring_sa = (uint32_t) __cvta_generic_to_shared(ring);
  const uint32_t sa_t8 = ring_sa + 8 * t, sa_l16 = ring_sa + lane * 16;      // + immediates: gradient rows
  const uint32_t sa_fold = sa_t8 + kFoldOff;
  const uint32_t sa_cp0 = ring_sa + (lane >> 3) * 128 + (((lane & 7) ^ (lane >> 3)) << 4), sa_cp1 = sa_cp0 ^ 64;
  uint32_t sa_m[4];
  {
    const int lr = (lane & 7) + ((lane >> 3) & 1) * 8;
    const uint32_t base = ring_sa + lr * 128 + (((lane >> 4) ^ (lane & 7)) << 4);
#pragma unroll
    for (int c = 0; c < 4; ++c) sa_m[c] = base ^ (c << 5);
  }
  float dk[8][4], dv[8][4];
  int tail_j = -1;                          // bucket whose tile is still in dk / dv after the loop
  if (rb < re) {
    const int n = min(re - rb, 4 * 32);     // entries of this warp: 1..127 for ranges cut by the transpose kernel
    // lane i: query block and pair number of entries rb + i, rb + 32 + i, ... (clamped: nothing is read outside the tensors);
    // requested first, they arrive while the bucket offsets below are being fetched
    int my_qb[4] = {0, 0, 0, 0}, my_pair[4] = {0, 0, 0, 0};
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (lane + 32 * u < n) {
        my_qb[u] = __ldcg(fl + rb + 32 * u + lane);
        my_pair[u] = __ldcg(pr + rb + 32 * u + lane);
      }
    // first bucket of the range (handed over by the transpose kernel; clamped, and moved on if it does not hold rb)
    int j = min(max(__ldcg(&a.ranges[bh * R + r].y), 0), n1 - 1);
    int bo = (int) csr_off(a, bh, j), nxt = (int) csr_off(a, bh, j + 1);
    while (nxt <= rb && j + 1 < n1) { ++j; bo = nxt; nxt = (int) csr_off(a, bh, j + 1); }
    int nxt2 = j + 2 <= n1 ? (int) csr_off(a, bh, j + 2) : 0x7fffffff;      // one bucket ahead: no load to wait for at a switch
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      my_qb[u] = my_qb[u] < 0 ? 0 : (my_qb[u] >= (int) a.nq1 ? (int) a.nq1 - 1 : my_qb[u]);
      my_pair[u] = my_pair[u] < 0 ? 0 : (my_pair[u] >= E ? E - 1 : my_pair[u]);
    }
    // the pooled-gradient rows the bucket's store folds in: lanes 0..15 hold the dpk row, lanes 16..31 the dpv row (16 bytes each)
    uint4 f1 = make_uint4(0u, 0u, 0u, 0u), f2 = make_uint4(0u, 0u, 0u, 0u);
    auto load_fold = [&](int jj) {
      if (a.fold) {
        f1 = __ldcg(reinterpret_cast<const uint4*>((lane < 16 ? a.dpk : a.dpv) + (bh * a.n1 + jj) * kD + (lane & 15) * 4));
        if (a.two_level) f2 = __ldcg(reinterpret_cast<const uint4*>((lane < 16 ? a.dpk2 : a.dpv2) + (bh * a.n2 + jj / kBS) * kD + (lane & 15) * 4));
      }
    };
    auto park_fold = [&]() {
      if (a.fold) {
        sts128<kFoldOff>(sa_l16, f1);
        if (a.two_level) sts128<kFoldOff + 512>(sa_l16, f2);
      }
      __syncwarp();
    };
    // global side: row (lane/8), chunk (lane%8) of block 0; a block is qblk / dblk bytes further, four rows qstep / dstep bytes
    const char* q_lane = reinterpret_cast<const char*>(a.q.row(b, h, lane >> 3) + (lane & 7) * 8);
    const char* d_lane = reinterpret_cast<const char*>(a.d_o.row(b, h, lane >> 3) + (lane & 7) * 8);
    const int qblk = (int) (kBS * a.q.sn * sizeof(bf16)), dblk = (int) (kBS * a.d_o.sn * sizeof(bf16));
    const int qstep = (int) (4 * a.q.sn * sizeof(bf16)), dstep = (int) (4 * a.d_o.sn * sizeof(bf16));
    // the P / dS registers of the whole range come from HBM (the hand-over does not fit the L2): every lane pulls its own
    // entries' 1 KB towards L2 now, so that the loads three entries ahead find them there
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (lane + 32 * u < n) {
        const char* pf = reinterpret_cast<const char*>(a.pds + (bh * (int64_t) E + my_pair[u]) * 64);
#pragma unroll
        for (int l = 0; l < 8; ++l) asm volatile("prefetch.global.L2 [%0];" ::"l"(pf + 128 * l));
      }
    const uint4* pds_lane = a.pds + bh * (int64_t) E * 64 + lane;
    uint4 pP[kRingFineStages], pD[kRingFineStages];       // P^T / dS^T registers of the entries in flight
    // The request for entry i goes out in four parts (PART 0..3) so that the entry loop can put a part between two groups of
    // products: address arithmetic and copies of the entry three ahead then run while the tensor pipe works on this one.
    const char* qp_i = q_lane;
    const char* dp_i = d_lane;
    auto issue_part = [&](auto stage_tag, auto part_tag, int i) {
      constexpr int ST = decltype(stage_tag)::value, PART = decltype(part_tag)::value;
      constexpr int SB = ST * kRingFineStageBytes, TB = kRingTileElems * (int) sizeof(bf16);
      if (PART == 0) {
        const int u = i >> 5;
        const int qb = __shfl_sync(0xffffffffu, u == 0 ? my_qb[0] : (u == 1 ? my_qb[1] : (u == 2 ? my_qb[2] : my_qb[3])), i & 31);
        const int pair = __shfl_sync(0xffffffffu, u == 0 ? my_pair[0] : (u == 1 ? my_pair[1] : (u == 2 ? my_pair[2] : my_pair[3])), i & 31);
        qp_i = q_lane + (int64_t) qb * qblk;
        dp_i = d_lane + (int64_t) qb * dblk;
        const uint4* pp = pds_lane + (int64_t) pair * 64;
        pP[ST] = __ldcg(pp);
        pD[ST] = __ldcg(pp + 32);
      } else if (PART == 1) {
        cp_async16_sa<SB>(sa_cp0, qp_i);
        cp_async16_sa<SB + 512>(sa_cp1, qp_i + qstep);
        cp_async16_sa<SB + 1024>(sa_cp0, qp_i + 2 * qstep);
        cp_async16_sa<SB + 1536>(sa_cp1, qp_i + 3 * qstep);
      } else if (PART == 2) {
        cp_async16_sa<SB + TB>(sa_cp0, dp_i);
        cp_async16_sa<SB + TB + 512>(sa_cp1, dp_i + dstep);
      } else {
        cp_async16_sa<SB + TB + 1024>(sa_cp0, dp_i + 2 * dstep);
        cp_async16_sa<SB + TB + 1536>(sa_cp1, dp_i + 3 * dstep);
      }
    };
    auto issue = [&](auto stage_tag, int i) {
      issue_part(stage_tag, std::integral_constant<int, 0>{}, i);
      issue_part(stage_tag, std::integral_constant<int, 1>{}, i);
      issue_part(stage_tag, std::integral_constant<int, 2>{}, i);
      issue_part(stage_tag, std::integral_constant<int, 3>{}, i);
    };
    static_assert(kRingFineStages == 4, "the entry loop below is unrolled over four stages");
    if (0 < n) issue(std::integral_constant<int, 0>{}, 0);
    cp_async_commit();
    if (1 < n) issue(std::integral_constant<int, 1>{}, 1);
    cp_async_commit();
    if (2 < n) issue(std::integral_constant<int, 2>{}, 2);
    cp_async_commit();
    load_fold(j);
    tile_zero(dk, dv);
    // one entry; the ring stage is a template argument so that every shared-memory offset below is an immediate
    auto entry = [&](auto stage_tag, int i) {
      constexpr int S = decltype(stage_tag)::value, SF = (S + kRingFineStages - 1) % kRingFineStages;    // SF: the stage read an entry ago
      constexpr int SB = S * kRingFineStageBytes, TB = kRingTileElems * (int) sizeof(bf16);
      const int e = rb + i;
      cp_async_wait_group<kRingFineStages - 2>();     // entry i has landed (this lane's chunks) ...
      __syncwarp();                                   // ... and everybody else's; stage SF is free
      if (e >= nxt && j + 1 < n1) {                   // next non-empty bucket; stage SF stages the store before it is refilled
        if (bo >= rb) {
          park_fold();
          dkv_fine_store_staged<SF * kRingFineStageBytes>(a, b, h, j, dk, dv, sa_m, sa_cp0, sa_cp1, sa_fold, lane);
        } else {
          tile_to_mem(slots + warp * kTileFloats, dk, dv, lane);   // began in an earlier warp's range
          if (lane == 0) s_head_bucket[warp] = j;
        }
        ++j; bo = nxt; nxt = nxt2;
        while (nxt <= e && j + 1 < n1) { ++j; bo = nxt; nxt = (int) csr_off(a, bh, j + 1); }      // empty buckets
        nxt2 = j + 2 <= n1 ? (int) csr_off(a, bh, j + 2) : 0x7fffffff;
        load_fold(j);
        tile_zero(dk, dv);
      }
      const uint4 P = pP[S], D = pD[S];
      const bool more = i + kRingFineStages - 1 < n;
      constexpr auto sf_tag = std::integral_constant<int, SF>{};
      // all eight operand loads first (a product issued right behind its own load would wait out the load's latency), then
      // the sixteen products in four groups with a part of the next request between them
      uint32_t bd[4][4], bq[4][4];
#pragma unroll
      for (int c = 0; c < 4; ++c) ldsm_x4_trans<SB + TB>(bd[c][0], bd[c][1], bd[c][2], bd[c][3], sa_m[c]);
#pragma unroll
      for (int c = 0; c < 4; ++c) ldsm_x4_trans<SB>(bq[c][0], bq[c][1], bq[c][2], bq[c][3], sa_m[c]);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        mma_bf16_16816(dv[2 * c], P.x, P.y, P.z, P.w, bd[c][0], bd[c][1]);
        mma_bf16_16816(dv[2 * c + 1], P.x, P.y, P.z, P.w, bd[c][2], bd[c][3]);
      }
      if (more) issue_part(sf_tag, std::integral_constant<int, 0>{}, i + kRingFineStages - 1);
#pragma unroll
      for (int c = 2; c < 4; ++c) {
        mma_bf16_16816(dv[2 * c], P.x, P.y, P.z, P.w, bd[c][0], bd[c][1]);
        mma_bf16_16816(dv[2 * c + 1], P.x, P.y, P.z, P.w, bd[c][2], bd[c][3]);
      }
      if (more) issue_part(sf_tag, std::integral_constant<int, 1>{}, i + kRingFineStages - 1);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        mma_bf16_16816(dk[2 * c], D.x, D.y, D.z, D.w, bq[c][0], bq[c][1]);
        mma_bf16_16816(dk[2 * c + 1], D.x, D.y, D.z, D.w, bq[c][2], bq[c][3]);
      }
      if (more) issue_part(sf_tag, std::integral_constant<int, 2>{}, i + kRingFineStages - 1);
#pragma unroll
      for (int c = 2; c < 4; ++c) {
        mma_bf16_16816(dk[2 * c], D.x, D.y, D.z, D.w, bq[c][0], bq[c][1]);
        mma_bf16_16816(dk[2 * c + 1], D.x, D.y, D.z, D.w, bq[c][2], bq[c][3]);
      }
      if (more) issue_part(sf_tag, std::integral_constant<int, 3>{}, i + kRingFineStages - 1);
      cp_async_commit();
    };
    for (int i = 0; i < n; i += 4) {
      entry(std::integral_constant<int, 0>{}, i);
      if (i + 1 < n) entry(std::integral_constant<int, 1>{}, i + 1);
      if (i + 2 < n) entry(std::integral_constant<int, 2>{}, i + 2);
      if (i + 3 < n) entry(std::integral_constant<int, 3>{}, i + 3);
    }
    cp_async_wait_all();
    __syncwarp();
    park_fold();                            // the last bucket's gradient rows, for whichever path below stores it
    // the last bucket of the range (the ring is idle by now)
    if (bo >= rb && nxt <= re) {
      dkv_fine_store_staged<0>(a, b, h, j, dk, dv, sa_m, sa_cp0, sa_cp1, sa_fold, lane);
    } else if (bo < rb) {                   // the whole range lies inside one bucket that began earlier
      tile_to_mem(slots + warp * kTileFloats, dk, dv, lane);
      if (lane == 0) s_head_bucket[warp] = j;
    } else {
      tail_j = j;                           // continues in later warps (or windows): completed below
    }
  }
  __syncthreads();
  if (tail_j >= 0) {
    for (int w = warp + 1; w < kRingWarps && s_head_bucket[w] == tail_j; ++w) tile_add_mem(slots + w * kTileFloats, dk, dv, lane);
    if ((int) csr_off(a, bh, tail_j + 1) <= ce) {
      dkv_fine_store_staged<0>(a, b, h, tail_j, dk, dv, sa_m, sa_cp0, sa_cp1, sa_fold, lane);
    } else {                                // runs on into the next window: this window's tail slot
      tile_to_mem(partial + ((bh * gridDim.x + blockIdx.x) * 2 + 1) * (int64_t) kTileFloats, dk, dv, lane);
    }
  }
  if (warp == 0 && s_head_bucket[0] >= 0) { // began in an earlier window: this window's head slot
    const int j0 = s_head_bucket[0];
    tile_zero(dk, dv);
    for (int w = 0; w < kRingWarps && s_head_bucket[w] == j0; ++w) tile_add_mem(slots + w * kTileFloats, dk, dv, lane);
    tile_to_mem(partial + ((bh * gridDim.x + blockIdx.x) * 2 + 0) * (int64_t) kTileFloats, dk, dv, lane);
  }
}

constexpr int kFinishPerWarp = 8;
// One warp per eight KV blocks: blocks nobody selected get their pooling-backward term alone, blocks whose bucket was cut
// across windows of the main kernel get the sum of their pieces, in window order.
__global__ void __launch_bounds__(128) attn_dkv_finish_ld_kernel(AttnP<bf16> a, const float* __restrict__ partial, int n_windows) {
  __shared__ __align__(1024) unsigned char s_stage[4][2 * kRingTileElems * sizeof(bf16)];      // per warp: a dK and a dV tile on their way out
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = lane & 3;
  const int64_t j0 = ((int64_t) blockIdx.x * 4 + warp) * kFinishPerWarp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  if (j0 >= a.n1) return;
  // a warp looks at eight consecutive buckets at once (lane i: offsets of bucket j0 + i) and works only on those that need it:
  // most buckets were finished by one warp of the main kernel
  const int64_t jl = j0 + lane < a.n1 ? j0 + lane : a.n1 - 1;
  // offsets are clamped to [0, E] and to each other: a malformed CSR cannot send the range arithmetic below outside `partial`
  const int64_t E = a.nq1 * a.topk;
  const int my_bo = lane < kFinishPerWarp ? (int) min(E, max((int64_t) 0, csr_off(a, bh, jl))) : 0;
  const int my_be = lane < kFinishPerWarp ? (int) min(E, max((int64_t) my_bo, csr_off(a, bh, jl + 1))) : 1;
  const int range = a.range_entries, window = kRingWarps * range;       // nominal entries per warp / per CTA of the main kernel
  const bool need = lane < kFinishPerWarp && j0 + lane < a.n1 && (my_be == my_bo || (my_be - my_bo > range && my_bo / window != (my_be - 1) / window));
  unsigned todo = __ballot_sync(0xffffffffu, need);
  if (!todo) return;
  const uint32_t st_sa = (uint32_t) __cvta_generic_to_shared(s_stage[warp]);
  const uint32_t sa_cp0 = st_sa + (lane >> 3) * 128 + (((lane & 7) ^ (lane >> 3)) << 4), sa_cp1 = sa_cp0 ^ 64;
  uint32_t sa_m[4];
  {
    const uint32_t base = st_sa + ((lane & 7) + ((lane >> 3) & 1) * 8) * 128 + (((lane >> 4) ^ (lane & 7)) << 4);
#pragma unroll
    for (int c = 0; c < 4; ++c) sa_m[c] = base ^ (c << 5);
  }
  // pieces of the split buckets: towards L2 now (two of a piece's 64 lines per lane), they are read a few microseconds later
  for (unsigned m = todo; m; m &= m - 1) {
    const int l = __ffs((int) m) - 1;
    const int bo = __shfl_sync(0xffffffffu, my_bo, l), be = __shfl_sync(0xffffffffu, my_be, l);
    if (be > bo) {
      const int c_first = bo / window, c_last = min((be - 1) / window, n_windows - 1);
      for (int c = c_first; c <= c_last; ++c) {
        const char* pf = reinterpret_cast<const char*>(partial + ((bh * n_windows + c) * 2 + (c == c_first ? 1 : 0)) * (int64_t) kTileFloats);
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pf + 128 * lane));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(pf + 128 * (32 + lane)));
      }
    }
  }
  // the gradient rows of the next bucket are requested before this one is finished
  FoldRows rows = dkv_fold_rows_load(a, bh, j0 + __ffs((int) todo) - 1, lane);
  while (todo) {
    const int l = __ffs((int) todo) - 1;
    todo &= todo - 1;
    const FoldRows mine = rows;
    if (todo) rows = dkv_fold_rows_load(a, bh, j0 + __ffs((int) todo) - 1, lane);
    const int bo = __shfl_sync(0xffffffffu, my_bo, l), be = __shfl_sync(0xffffffffu, my_be, l);
    const int64_t j = j0 + l;
    float dk[8][4], dv[8][4];
    tile_zero(dk, dv);
    if (be > bo) {
      // a bucket of more than `range` entries is cut at multiples of `range` only, so its pieces by windows lie
      // between multiples of `window`: the first is the tail of the window that holds entry bo, every later one a head
      const int c_first = bo / window, c_last = min((be - 1) / window, n_windows - 1);
      for (int c = c_first; c <= c_last; ++c)
        tile_add_mem_batched(partial + ((bh * n_windows + c) * 2 + (c == c_first ? 1 : 0)) * (int64_t) kTileFloats, dk, dv, lane);
    }
    dkv_fine_fold_apply(a, mine, dk, dv, lane);
    dkv_tile_store_staged<0>(a, b, h, j, dk, dv, sa_m, sa_cp0, sa_cp1, lane);
  }
}

int zero_pooled_acc(const LlsaAttnArgs* g, cudaStream_t st);

int launch_attn_bwd_mma(const LlsaAttnArgs* g, cudaStream_t st) {
  if (!mma_path_ok(g, true)) {
    note_scalar_path();
    return launch_attn_bwd_generic(g, st);
  }
  AttnP<bf16> a = build_attn_params<bf16>(g, true);
  const unsigned BH = (unsigned) (g->q->shape[0] * a.H);
  const int mask = g->stage_mask ? g->stage_mask : 7;
  // pooled keys on tcgen05 (attn_pooled_bwd_tc.cu): the dQ kernel then covers the fine blocks only and the
  // tensor-core kernel adds the pooled part of dq and produces the pooled-key gradients
  const bool tc = pooled_bwd_tc_ok(a) && !g->no_tcgen05;
  // long pooled key lists: the pooled part of dQ on the key-loop tcgen05 kernel (the pooled dK/dV stay on mma.sync)
  const bool loop_dq = !tc && pooled_dq_loop_tc_keys(a) > 0 && !g->no_tcgen05;
  if (mask & 1) {
    int rc = zero_pooled_acc(g, st);
    if (rc) return rc;
    constexpr int NWQ = 4;
    AttnP<bf16> aq = a;
    if (tc || loop_dq) aq.p1_blocks = aq.p2_blocks = 0;
    const int n_all = aq.p1_blocks + aq.p2_blocks;
    const int n_smem = n_all < 12 ? n_all : 12;   // 12 tiles = 54 KB of K+V, three CTAs per SM
    const size_t smem = (size_t) n_smem * kBS * kSmemPitch * sizeof(bf16) * 2;
    if (n_all == 0) {
      const size_t ring = (size_t) NWQ * kDqStages * 2 * kRingTileElems * sizeof(bf16);
      LLSA_SMEM_LIMIT((attn_dq_fine_kernel<NWQ>), ring);
      attn_dq_fine_kernel<NWQ><<<dim3((unsigned) (a.nq1 / NWQ), BH), NWQ * 32, ring, st>>>(aq);
      LLSA_LAUNCH_OK("attn_dq_fine_kernel");
    } else {
      LLSA_SMEM_LIMIT((attn_dq_mma_kernel<NWQ>), smem);
      attn_dq_mma_kernel<NWQ><<<dim3((unsigned) (a.nq1 / NWQ), BH), NWQ * 32, smem, st>>>(aq, n_smem);
      LLSA_LAUNCH_OK("attn_dq_mma_kernel");
    }
  }
  if ((mask & 2) && tc) {
    int rc = launch_attn_bwd_pooled_tc(g, a, BH, st);
    if (rc) return rc;
  } else if ((mask & 2) && a.p1_blocks + a.p2_blocks > 0) {
    if (loop_dq) {
      int rc = launch_attn_dq_pooled_loop_tc(g, a, BH, st);
      if (rc) return rc;
    }
    // the keys every query attends to (level 1 of one level, level 2 of two levels) on the key-major tcgen05 kernel; what is
    // left for the mma.sync kernel is the gathered level-1 part of the two-level form
    const int dense_level = loop_dq ? pooled_dkv_loop_tc_level(a) : 0;
    AttnP<bf16> ap = a;
    if (dense_level) {
      int rc = launch_attn_dkv_pooled_loop_tc(g, a, BH, st);
      if (rc) return rc;
      if (dense_level == 1) ap.p1_blocks = 0; else ap.p2_blocks = 0;
    }
    if (ap.p1_blocks + ap.p2_blocks > 0) {
      constexpr int NWP = 8;
      const size_t smem = (size_t) 2 * kBS * kBS * kSmemPitch * sizeof(bf16) + 2 * kBS * kBS * sizeof(float);
      LLSA_SMEM_LIMIT((attn_dkv_pooled_kernel<NWP>), smem);
      attn_dkv_pooled_kernel<NWP><<<dim3((unsigned) (a.nq1 / kBS), BH), NWP * 32, smem, st>>>(ap);
      LLSA_LAUNCH_OK("attn_dkv_pooled_kernel");
    }
  }
  if (mask & 4) {
    const int64_t E = a.nq1 * a.topk;
    const int n_ranges = (int) ((E + a.range_entries - 1) / a.range_entries), n_windows = (n_ranges + kRingWarps - 1) / kRingWarps;
    float* partial = (float*) g->dkv_partial->ptr;
    const size_t smem = (size_t) kRingWarps * (kTileFloats * sizeof(float) + kRingFineStages * kRingFineStageBytes + kRingFoldBytes) + 128;   // per warp: slot, ring, gradient rows
    LLSA_SMEM_LIMIT((attn_dkv_fine_ring_kernel), smem);
    attn_dkv_fine_ring_kernel<<<dim3((unsigned) n_windows, BH), kRingWarps * 32, smem, st>>>(a, partial);
    LLSA_LAUNCH_OK("attn_dkv_fine_ring_kernel");
    attn_dkv_finish_ld_kernel<<<dim3((unsigned) ((a.n1 + 4 * kFinishPerWarp - 1) / (4 * kFinishPerWarp)), BH), 128, 0, st>>>(a, partial, n_windows);
    LLSA_LAUNCH_OK("attn_dkv_finish_ld_kernel");
  }
  return LLSA_OK;
}

}  // namespace llsa
