// Block-sparse LLSA backward on the tensor cores (bf16, D = 64, 16-token blocks).
// Reference: sparse_indices_attn_res_scatter_bwd_v2 (sparse_attention_res_1.py:403-471)
// and sparse_indices_attn_res_scatter_2_2_bwd_v2 (sparse_attention_res_2.py:578-681).
//
// Three kernels, all with register-direct operand fragments (mma_frag.cuh):
//   attn_dq_mma_kernel     one warp per query block: delta = rowsum(o*do) (the
//                          reference's separate _attn_bwd_preprocess pass), then
//                          S, dP and dQ over the fine, pooled-1 and pooled-2 keys.
//   attn_dkv_pooled_kernel one CTA per group of 16 query blocks (= one parent):
//                          its warps share out the pooled key tiles the group
//                          attends to, run the transposed products S^T, dP^T,
//                          dV += P^T.dO, dK += dS^T.Q over the group's 256 rows and
//                          add the 16x64 results into fp32 accumulators.
//   attn_dkv_fine_kernel   one CTA per KV block: its warps share out the block's
//                          CSR list of query blocks, partial sums meet in shared
//                          memory, and the epilogue folds in the pooling backward
//                          (dk += (dpk[j] + dpk2[j/16]/16)/16) before one bf16 store.
// The reference multiplies k by scale into new tensors first (res_1.py:420-422);
// here scale rides in the exp2 argument and in the epilogues.
#include "attn.cuh"
#include "mma_frag.cuh"

namespace llsa {

constexpr float kLog2e = 1.4426950408889634f;

struct BwdBlockRef {
  const bf16* k;
  const bf16* v;
  int64_t ks, vs;
  float lw;
};

__device__ __forceinline__ BwdBlockRef resolve_bwd_block(const AttnP<bf16>& a, int64_t b, int64_t h, int64_t bh, int i, int my_fine, int my_p1,
                                                         float lw1, float lw2) {
  BwdBlockRef r;
  if (i < a.topk) {
    const int64_t j = __shfl_sync(0xffffffffu, my_fine, i);
    r.k = a.k.row(b, h, j * kBS); r.v = a.v.row(b, h, j * kBS); r.ks = a.k.sn; r.vs = a.v.sn; r.lw = 0.f;
  } else if (i < a.topk + a.p1_blocks) {
    const int ii = i - a.topk;
    const int64_t j = a.two_level ? (int64_t) __shfl_sync(0xffffffffu, my_p1, ii) : (int64_t) ii;
    r.k = a.pk + (bh * a.n1 + j * kBS) * kD; r.v = a.pv + (bh * a.n1 + j * kBS) * kD; r.ks = r.vs = kD; r.lw = lw1;
  } else {
    const int64_t j = i - a.topk - a.p1_blocks;
    r.k = a.pk2 + (bh * a.n2 + j * kBS) * kD; r.v = a.pv2 + (bh * a.n2 + j * kBS) * kD; r.ks = r.vs = kD; r.lw = lw2;
  }
  return r;
}

__device__ __forceinline__ float rowfrag_dot(const RowFrag& x, const RowFrag& y) {
  float acc = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    acc = fmaf(bf16_lo(x.r[i]), bf16_lo(y.r[i]), acc);
    acc = fmaf(bf16_hi(x.r[i]), bf16_hi(y.r[i]), acc);
  }
  return acc;
}

template <int NW>
__global__ void __launch_bounds__(NW * 32) attn_dq_mma_kernel(AttnP<bf16> a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t qb = (int64_t) blockIdx.x * NW + warp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  if (qb >= a.n1) return;
  const int my_fine = lane < a.topk ? (int) fine_block(a, bh, qb, lane) : 0;
  const int my_p1 = (a.two_level && lane < a.topk_p) ? (int) p1_block(a, bh, qb, lane) : 0;
  const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
  const float sl2 = a.scale * kLog2e;

  RowFrag qlo, qhi, dlo, dhi;
  load_rowfrag(qlo, a.q.row(b, h, qb * kBS + g), t);
  load_rowfrag(qhi, a.q.row(b, h, qb * kBS + g + 8), t);
  load_rowfrag(dlo, a.d_o.row(b, h, qb * kBS + g), t);
  load_rowfrag(dhi, a.d_o.row(b, h, qb * kBS + g + 8), t);
  float delta0, delta1;
  {
    RowFrag olo, ohi;
    load_rowfrag(olo, a.o_in.row(b, h, qb * kBS + g), t);
    load_rowfrag(ohi, a.o_in.row(b, h, qb * kBS + g + 8), t);
    delta0 = quad_sum(rowfrag_dot(olo, dlo));
    delta1 = quad_sum(rowfrag_dot(ohi, dhi));
  }
  const int64_t rbase = bh * a.N + qb * kBS;
  if (t == 0) { a.delta[rbase + g] = delta0; a.delta[rbase + g + 8] = delta1; }
  const float L0 = a.lse[rbase + g] * kLog2e, L1 = a.lse[rbase + g + 8] * kLog2e;

  float dq[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) dq[j][0] = dq[j][1] = dq[j][2] = dq[j][3] = 0.f;

  const int nblk = a.topk + a.p1_blocks + a.p2_blocks;
  BwdBlockRef r = resolve_bwd_block(a, b, h, bh, 0, my_fine, my_p1, lw1, lw2);
  RowFrag k0, k1, v0, v1;
  load_rowfrag(k0, r.k + (int64_t) g * r.ks, t);
  load_rowfrag(k1, r.k + (int64_t) (g + 8) * r.ks, t);
  load_rowfrag(v0, r.v + (int64_t) g * r.vs, t);
  load_rowfrag(v1, r.v + (int64_t) (g + 8) * r.vs, t);
  for (int i = 0; i < nblk; ++i) {
    ColFrag kc;
    load_colfrag(kc, r.k, r.ks, g, t);
    const float lw = r.lw;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, p0[4] = {0.f, 0.f, 0.f, 0.f}, p1[4] = {0.f, 0.f, 0.f, 0.f};
    mma_rows_x_keys(s0, s1, qlo, qhi, k0, k1);
    mma_rows_x_keys(p0, p1, dlo, dhi, v0, v1);
    if (i + 1 < nblk) {
      r = resolve_bwd_block(a, b, h, bh, i + 1, my_fine, my_p1, lw1, lw2);
      load_rowfrag(k0, r.k + (int64_t) g * r.ks, t);
      load_rowfrag(k1, r.k + (int64_t) (g + 8) * r.ks, t);
      load_rowfrag(v0, r.v + (int64_t) g * r.vs, t);
      load_rowfrag(v1, r.v + (int64_t) (g + 8) * r.vs, t);
    }
    // ds = w * exp(s*scale - lse) * (dp - delta)
    s0[0] = fast_exp2(fmaf(s0[0], sl2, lw - L0)) * (p0[0] - delta0);
    s0[1] = fast_exp2(fmaf(s0[1], sl2, lw - L0)) * (p0[1] - delta0);
    s0[2] = fast_exp2(fmaf(s0[2], sl2, lw - L1)) * (p0[2] - delta1);
    s0[3] = fast_exp2(fmaf(s0[3], sl2, lw - L1)) * (p0[3] - delta1);
    s1[0] = fast_exp2(fmaf(s1[0], sl2, lw - L0)) * (p1[0] - delta0);
    s1[1] = fast_exp2(fmaf(s1[1], sl2, lw - L0)) * (p1[1] - delta0);
    s1[2] = fast_exp2(fmaf(s1[2], sl2, lw - L1)) * (p1[2] - delta1);
    s1[3] = fast_exp2(fmaf(s1[3], sl2, lw - L1)) * (p1[3] - delta1);
    mma_x_cols(dq, pack_bf16(s0[0], s0[1]), pack_bf16(s0[2], s0[3]), pack_bf16(s1[0], s1[1]), pack_bf16(s1[2], s1[3]), kc);
  }
  store_acc_row<0>(a.dq.row(b, h, qb * kBS + g), dq, t, a.scale);
  store_acc_row<1>(a.dq.row(b, h, qb * kBS + g + 8), dq, t, a.scale);
}

// One (key tile) x (query block) step of the dK/dV side.  ka/kb, va/vb: the key
// tile's rows g / g+8 as the A operand.  Accumulates dV += P^T.dO, dK += dS^T.Q (unscaled).
__device__ __forceinline__ void dkv_step(const AttnP<bf16>& a, int64_t b, int64_t h, int64_t bh, int64_t qb, const RowFrag& ka, const RowFrag& kb,
                                         const RowFrag& va, const RowFrag& vb, float lw, float sl2, int g, int t, float (&dk)[8][4],
                                         float (&dv)[8][4]) {
  const bf16* qp = a.q.row(b, h, qb * kBS);
  const bf16* dp = a.d_o.row(b, h, qb * kBS);
  RowFrag q0, q1, d0, d1;
  load_rowfrag(q0, qp + (int64_t) g * a.q.sn, t);
  load_rowfrag(q1, qp + (int64_t) (g + 8) * a.q.sn, t);
  load_rowfrag(d0, dp + (int64_t) g * a.d_o.sn, t);
  load_rowfrag(d1, dp + (int64_t) (g + 8) * a.d_o.sn, t);
  ColFrag qc, dc;
  load_colfrag(qc, qp, a.q.sn, g, t);
  load_colfrag(dc, dp, a.d_o.sn, g, t);
  const int64_t rbase = bh * a.N + qb * kBS;
  const float2 la = *reinterpret_cast<const float2*>(a.lse + rbase + 2 * t);        // query rows 2t, 2t+1
  const float2 lb = *reinterpret_cast<const float2*>(a.lse + rbase + 8 + 2 * t);    // query rows 8+2t, 9+2t
  const float2 da = *reinterpret_cast<const float2*>(a.delta + rbase + 2 * t);
  const float2 db = *reinterpret_cast<const float2*>(a.delta + rbase + 8 + 2 * t);
  // transposed tiles: rows = keys (g, g+8), columns = query rows (tile 0: 0..7, tile 1: 8..15)
  float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f}, e0[4] = {0.f, 0.f, 0.f, 0.f}, e1[4] = {0.f, 0.f, 0.f, 0.f};
  mma_rows_x_keys(s0, s1, ka, kb, q0, q1);
  mma_rows_x_keys(e0, e1, va, vb, d0, d1);
  const float a0 = lw - la.x * kLog2e, a1 = lw - la.y * kLog2e, b0 = lw - lb.x * kLog2e, b1 = lw - lb.y * kLog2e;
  // c0: (key g, row 2t)  c1: (key g, row 2t+1)  c2: (key g+8, row 2t)  c3: (key g+8, row 2t+1)
  s0[0] = fast_exp2(fmaf(s0[0], sl2, a0)); s0[1] = fast_exp2(fmaf(s0[1], sl2, a1));
  s0[2] = fast_exp2(fmaf(s0[2], sl2, a0)); s0[3] = fast_exp2(fmaf(s0[3], sl2, a1));
  s1[0] = fast_exp2(fmaf(s1[0], sl2, b0)); s1[1] = fast_exp2(fmaf(s1[1], sl2, b1));
  s1[2] = fast_exp2(fmaf(s1[2], sl2, b0)); s1[3] = fast_exp2(fmaf(s1[3], sl2, b1));
  e0[0] = s0[0] * (e0[0] - da.x); e0[1] = s0[1] * (e0[1] - da.y); e0[2] = s0[2] * (e0[2] - da.x); e0[3] = s0[3] * (e0[3] - da.y);
  e1[0] = s1[0] * (e1[0] - db.x); e1[1] = s1[1] * (e1[1] - db.y); e1[2] = s1[2] * (e1[2] - db.x); e1[3] = s1[3] * (e1[3] - db.y);
  mma_x_cols(dv, pack_bf16(s0[0], s0[1]), pack_bf16(s0[2], s0[3]), pack_bf16(s1[0], s1[1]), pack_bf16(s1[2], s1[3]), dc);
  mma_x_cols(dk, pack_bf16(e0[0], e0[1]), pack_bf16(e0[2], e0[3]), pack_bf16(e1[0], e1[1]), pack_bf16(e1[2], e1[3]), qc);
}

template <int NW>
__global__ void __launch_bounds__(NW * 32) attn_dkv_pooled_kernel(AttnP<bf16> a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t grp = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const float sl2 = a.scale * kLog2e;
  const int ntiles = a.p1_blocks + a.p2_blocks;
  for (int i = warp; i < ntiles; i += NW) {
    const bf16 *kp, *vp;
    float *gk, *gv;
    float lw;
    if (i < a.p1_blocks) {
      const int64_t j = p1_block(a, bh, grp * kBS, i);
      const int64_t off = (bh * a.n1 + j * kBS) * kD;
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
    for (int qi = 0; qi < kBS; ++qi) dkv_step(a, b, h, bh, grp * kBS + qi, ka, kb, va, vb, lw, sl2, g, t, dk, dv);
    // accumulator tile j: channels 16t + j (c0, c2) and 16t + 8 + j (c1, c3); rows g (c0, c1) and g + 8 (c2, c3)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      atomicAdd(gk + g * kD + 16 * t + j, dk[j][0] * a.scale);
      atomicAdd(gk + g * kD + 16 * t + 8 + j, dk[j][1] * a.scale);
      atomicAdd(gk + (g + 8) * kD + 16 * t + j, dk[j][2] * a.scale);
      atomicAdd(gk + (g + 8) * kD + 16 * t + 8 + j, dk[j][3] * a.scale);
      atomicAdd(gv + g * kD + 16 * t + j, dv[j][0]);
      atomicAdd(gv + g * kD + 16 * t + 8 + j, dv[j][1]);
      atomicAdd(gv + (g + 8) * kD + 16 * t + j, dv[j][2]);
      atomicAdd(gv + (g + 8) * kD + 16 * t + 8 + j, dv[j][3]);
    }
  }
}

template <int NW>
__global__ void __launch_bounds__(NW * 32) attn_dkv_fine_kernel(AttnP<bf16> a) {
  __shared__ float red[NW - 1][64][32];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t j = blockIdx.x, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const float sl2 = a.scale * kLog2e;
  int64_t list0, list1;
  if (a.off64) {
    list0 = reinterpret_cast<const int64_t*>(a.offsets)[bh * (a.n1 + 1) + j];
    list1 = reinterpret_cast<const int64_t*>(a.offsets)[bh * (a.n1 + 1) + j + 1];
  } else {
    list0 = reinterpret_cast<const int32_t*>(a.offsets)[bh * (a.n1 + 1) + j];
    list1 = reinterpret_cast<const int32_t*>(a.offsets)[bh * (a.n1 + 1) + j + 1];
  }
  float dk[8][4], dv[8][4];
#pragma unroll
  for (int u = 0; u < 8; ++u) dk[u][0] = dk[u][1] = dk[u][2] = dk[u][3] = dv[u][0] = dv[u][1] = dv[u][2] = dv[u][3] = 0.f;
  if (list0 + warp < list1) {
    const bf16* kp = a.k.row(b, h, j * kBS);
    const bf16* vp = a.v.row(b, h, j * kBS);
    RowFrag ka, kb, va, vb;
    load_rowfrag(ka, kp + (int64_t) g * a.k.sn, t);
    load_rowfrag(kb, kp + (int64_t) (g + 8) * a.k.sn, t);
    load_rowfrag(va, vp + (int64_t) g * a.v.sn, t);
    load_rowfrag(vb, vp + (int64_t) (g + 8) * a.v.sn, t);
    const int32_t* fl = a.flat + bh * a.n1 * a.topk;
    for (int64_t it = list0 + warp; it < list1; it += NW) {
      int64_t qb = fl[it];
      qb = qb < 0 ? 0 : (qb >= a.n1 ? a.n1 - 1 : qb);
      dkv_step(a, b, h, bh, qb, ka, kb, va, vb, 0.f, sl2, g, t, dk, dv);
    }
  }
  // partial sums of warps 1..NW-1 meet in shared memory; warp 0 adds them up and stores
  if (warp > 0) {
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        red[warp - 1][u * 4 + c][lane] = dk[u][c];
        red[warp - 1][32 + u * 4 + c][lane] = dv[u][c];
      }
  }
  __syncthreads();
  if (warp == 0) {
#pragma unroll
    for (int w = 0; w < NW - 1; ++w)
#pragma unroll
      for (int u = 0; u < 8; ++u)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          dk[u][c] += red[w][u * 4 + c][lane];
          dv[u][c] += red[w][32 + u * 4 + c][lane];
        }
    float ek[2][8], ev[2][8];   // pooling-backward term for channels 16t + {0..7} and 16t + 8 + {0..7}
#pragma unroll
    for (int u = 0; u < 8; ++u) ek[0][u] = ek[1][u] = ev[0][u] = ev[1][u] = 0.f;
    if (a.fold) {
      const float* g1k = a.dpk + (bh * a.n1 + j) * kD + 16 * t;
      const float* g1v = a.dpv + (bh * a.n1 + j) * kD + 16 * t;
#pragma unroll
      for (int u = 0; u < 8; ++u) { ek[0][u] = g1k[u]; ek[1][u] = g1k[8 + u]; ev[0][u] = g1v[u]; ev[1][u] = g1v[8 + u]; }
      if (a.two_level) {
        const float* g2k = a.dpk2 + (bh * a.n2 + j / kBS) * kD + 16 * t;
        const float* g2v = a.dpv2 + (bh * a.n2 + j / kBS) * kD + 16 * t;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          ek[0][u] += g2k[u] * (1.f / kBS); ek[1][u] += g2k[8 + u] * (1.f / kBS);
          ev[0][u] += g2v[u] * (1.f / kBS); ev[1][u] += g2v[8 + u] * (1.f / kBS);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      dk[u][0] = dk[u][0] * a.scale + ek[0][u] * (1.f / kBS); dk[u][1] = dk[u][1] * a.scale + ek[1][u] * (1.f / kBS);
      dk[u][2] = dk[u][2] * a.scale + ek[0][u] * (1.f / kBS); dk[u][3] = dk[u][3] * a.scale + ek[1][u] * (1.f / kBS);
      dv[u][0] += ev[0][u] * (1.f / kBS); dv[u][1] += ev[1][u] * (1.f / kBS);
      dv[u][2] += ev[0][u] * (1.f / kBS); dv[u][3] += ev[1][u] * (1.f / kBS);
    }
    store_acc_row<0>(a.dk.row(b, h, j * kBS + g), dk, t, 1.f);
    store_acc_row<1>(a.dk.row(b, h, j * kBS + g + 8), dk, t, 1.f);
    store_acc_row<0>(a.dv.row(b, h, j * kBS + g), dv, t, 1.f);
    store_acc_row<1>(a.dv.row(b, h, j * kBS + g + 8), dv, t, 1.f);
  }
}

int zero_pooled_acc(const LlsaAttnArgs* g, cudaStream_t st);

int launch_attn_bwd_mma(const LlsaAttnArgs* g, cudaStream_t st) {
  if (g->topk > 32 || (g->pk2 && g->topk_p > 32)) return launch_attn_bwd_generic(g, st);
  AttnP<bf16> a = build_attn_params<bf16>(g, true);
  const unsigned BH = (unsigned) (g->q->shape[0] * a.H);
  const int mask = g->stage_mask ? g->stage_mask : 7;
  if (mask & 1) {
    int rc = zero_pooled_acc(g, st);
    if (rc) return rc;
    constexpr int NWQ = 4;
    attn_dq_mma_kernel<NWQ><<<dim3((unsigned) ((a.n1 + NWQ - 1) / NWQ), BH), NWQ * 32, 0, st>>>(a);
    LLSA_LAUNCH_OK("attn_dq_mma_kernel");
  }
  if ((mask & 2) && a.p1_blocks + a.p2_blocks > 0) {
    constexpr int NWP = 4;
    attn_dkv_pooled_kernel<NWP><<<dim3((unsigned) (a.n1 / kBS), BH), NWP * 32, 0, st>>>(a);
    LLSA_LAUNCH_OK("attn_dkv_pooled_kernel");
  }
  if (mask & 4) {
    constexpr int NWF = 4;
    attn_dkv_fine_kernel<NWF><<<dim3((unsigned) a.n1, BH), NWF * 32, 0, st>>>(a);
    LLSA_LAUNCH_OK("attn_dkv_fine_kernel");
  }
  return LLSA_OK;
}

}  // namespace llsa
