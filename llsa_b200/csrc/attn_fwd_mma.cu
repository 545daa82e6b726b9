// Block-sparse LLSA forward on the tensor cores (bf16, D = 64, 16-token blocks).
// Reference: _sparse_indices_attn_res_fwd (sparse_attention_res_1.py:9-120) and
// _sparse_indices_attn_res_2_2_fwd (sparse_attention_res_2.py:9-163).
//
// One warp owns one 16-row query block (the m16 of mma.sync.m16n8k16); a CTA of
// NW warps owns NW consecutive query blocks, which always share their parent
// block, so the pooled keys the parent selected are fetched from L2 once per
// CTA and served from L1 afterwards.  Key/value blocks go from global memory
// straight into mma operand registers (mma_frag.cuh) -- no shared memory.
// The softmax runs online over chunks of 32 keys (two blocks) in the exp2
// domain; a pooled key's weight enters as +log2(weight) on its logit, which is
// what `l += l_ij * W; acc += P.V * W` in the reference amounts to.
#include "attn.cuh"
#include "mma_frag.cuh"

namespace llsa {

struct BlockRef {
  const bf16* k;
  const bf16* v;
  int64_t ks, vs;
  float lw;  // log2 of the token weight
};

// Resolves key block i of the list [fine | pooled-1 | pooled-2]; i is warp-uniform.
// my_fine / my_p1: lane i holds the i-th selected fine block / parent block index.
__device__ __forceinline__ BlockRef resolve_block(const AttnP<bf16>& a, int64_t b, int64_t h, int64_t bh, int i, int my_fine, int my_p1,
                                                  float lw1, float lw2) {
  BlockRef r;
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

template <int NW>
__global__ void __launch_bounds__(NW * 32) attn_fwd_mma_kernel(AttnP<bf16> a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t qb = (int64_t) blockIdx.x * NW + warp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  if (qb >= a.n1) return;
  const int my_fine = lane < a.topk ? (int) fine_block(a, bh, qb, lane) : 0;
  const int my_p1 = (a.two_level && lane < a.topk_p) ? (int) p1_block(a, bh, qb, lane) : 0;
  const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
  const float sl2 = a.scale * 1.4426950408889634f;

  RowFrag qlo, qhi;
  load_rowfrag(qlo, a.q.row(b, h, qb * kBS + g), t);
  load_rowfrag(qhi, a.q.row(b, h, qb * kBS + g + 8), t);

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

  const int nchunks = (a.topk + a.p1_blocks + a.p2_blocks) >> 1;
  RowFrag k00, k01, k10, k11;   // block 0 keys g / g+8, block 1 keys g / g+8
  ColFrag v0, v1;
  BlockRef r0 = resolve_block(a, b, h, bh, 0, my_fine, my_p1, lw1, lw2);
  BlockRef r1 = resolve_block(a, b, h, bh, 1, my_fine, my_p1, lw1, lw2);
  load_rowfrag(k00, r0.k + (int64_t) g * r0.ks, t);
  load_rowfrag(k01, r0.k + (int64_t) (g + 8) * r0.ks, t);
  load_rowfrag(k10, r1.k + (int64_t) g * r1.ks, t);
  load_rowfrag(k11, r1.k + (int64_t) (g + 8) * r1.ks, t);
  load_colfrag(v0, r0.v, r0.vs, g, t);
  load_colfrag(v1, r1.v, r1.vs, g, t);

  for (int c = 0; c < nchunks; ++c) {
    float s[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    mma_rows_x_keys(s[0], s[1], qlo, qhi, k00, k01);
    mma_rows_x_keys(s[2], s[3], qlo, qhi, k10, k11);
    const float lw = r0.lw;
    const bool more = c + 1 < nchunks;
    if (more) {  // next chunk's keys: the registers are free as soon as the products above have issued
      r0 = resolve_block(a, b, h, bh, 2 * c + 2, my_fine, my_p1, lw1, lw2);
      r1 = resolve_block(a, b, h, bh, 2 * c + 3, my_fine, my_p1, lw1, lw2);
      load_rowfrag(k00, r0.k + (int64_t) g * r0.ks, t);
      load_rowfrag(k01, r0.k + (int64_t) (g + 8) * r0.ks, t);
      load_rowfrag(k10, r1.k + (int64_t) g * r1.ks, t);
      load_rowfrag(k11, r1.k + (int64_t) (g + 8) * r1.ks, t);
    }
    // logits in the exp2 domain
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = fmaf(s[j][0], sl2, lw); s[j][1] = fmaf(s[j][1], sl2, lw);
      s[j][2] = fmaf(s[j][2], sl2, lw); s[j][3] = fmaf(s[j][3], sl2, lw);
      mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
      mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    const float mn0 = fmaxf(m0, quad_max(mx0)), mn1 = fmaxf(m1, quad_max(mx1));
    const float al0 = fast_exp2(m0 - mn0), al1 = fast_exp2(m1 - mn1);
    m0 = mn0; m1 = mn1;
    float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      s[j][0] = fast_exp2(s[j][0] - mn0); s[j][1] = fast_exp2(s[j][1] - mn0);
      s[j][2] = fast_exp2(s[j][2] - mn1); s[j][3] = fast_exp2(s[j][3] - mn1);
      sum0 += s[j][0] + s[j][1];
      sum1 += s[j][2] + s[j][3];
    }
    l0 = l0 * al0 + sum0;   // per-lane partial sums; reduced over the quad at the end
    l1 = l1 * al1 + sum1;
#pragma unroll
    for (int j = 0; j < 8; ++j) { o[j][0] *= al0; o[j][1] *= al0; o[j][2] *= al1; o[j][3] *= al1; }
    // P (bf16) as the A operand: C tiles (2j, 2j+1) of S are the k16 halves of block j
    mma_x_cols(o, pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]), pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3]), v0);
    mma_x_cols(o, pack_bf16(s[2][0], s[2][1]), pack_bf16(s[2][2], s[2][3]), pack_bf16(s[3][0], s[3][1]), pack_bf16(s[3][2], s[3][3]), v1);
    if (more) {
      load_colfrag(v0, r0.v, r0.vs, g, t);
      load_colfrag(v1, r1.v, r1.vs, g, t);
    }
  }
  l0 = quad_sum(l0);
  l1 = quad_sum(l1);
  store_acc_row<0>(a.o.row(b, h, qb * kBS + g), o, t, 1.f / l0);
  store_acc_row<1>(a.o.row(b, h, qb * kBS + g + 8), o, t, 1.f / l1);
  if (t == 0) {
    a.lse[bh * a.N + qb * kBS + g] = (m0 + log2f(l0)) * 0.6931471805599453f;
    a.lse[bh * a.N + qb * kBS + g + 8] = (m1 + log2f(l1)) * 0.6931471805599453f;
  }
}

int launch_attn_fwd_mma(const LlsaAttnArgs* g, cudaStream_t st) {
  if (g->topk > 32 || (g->pk2 && g->topk_p > 32)) return launch_attn_fwd_generic(g, st);
  AttnP<bf16> a = build_attn_params<bf16>(g, false);
  constexpr int NW = 4;
  dim3 grid((unsigned) ((a.n1 + NW - 1) / NW), (unsigned) (g->q->shape[0] * a.H));
  attn_fwd_mma_kernel<NW><<<grid, NW * 32, 0, st>>>(a);
  LLSA_LAUNCH_OK("attn_fwd_mma_kernel");
  return LLSA_OK;
}

}  // namespace llsa
