// Block-sparse LLSA forward on the tensor cores (bf16, D = 64, 16-token blocks).
// Reference: _sparse_indices_attn_res_fwd (sparse_attention_res_1.py:9-120) and
// _sparse_indices_attn_res_2_2_fwd (sparse_attention_res_2.py:9-163).
//
// One warp owns one 16-row query block (the m16 of mma.sync.m16n8k16); a CTA of
// NW warps owns NW consecutive query blocks, which always share their parent
// block and therefore the same pooled keys.
//   * Pooled key/value tiles (the children of the parent's selected level-2
//     blocks and the level-2 keys; all level-1 keys in the one-level form) are
//     copied once per CTA into shared memory with cp.async while the fine stage
//     runs, then read by every warp as conflict-free 128-bit fragments.  Tiles
//     beyond the shared-memory budget are streamed like fine blocks.
//   * Fine key/value blocks are private to a query block: they go from global
//     memory straight into mma operand registers (mma_frag.cuh) with the next
//     block's loads in flight behind the current block's math.
// The softmax runs online, one 16-key block at a time, in the exp2 domain; a
// pooled key's weight enters as +log2(weight) on its logit, which is what
// `l += l_ij * W; acc += P.V * W` in the reference amounts to.
#include <type_traits>

#include "attn.cuh"
#include "mma_frag.cuh"

namespace llsa {

struct FwdState {
  float o[8][4];
  float m0, m1, l0, l1;
};

// First half of a 16-key block: S = Q.K^T and the online-softmax update; returns P (bf16) as the
// four A registers of the P.V product.  The key fragments are dead afterwards.
__device__ __forceinline__ void fwd_scores(FwdState& st, const RowFrag& qlo, const RowFrag& qhi, const RowFrag& k0, const RowFrag& k1,
                                           float sl2, float lw, uint32_t (&pa)[4]) {
  float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
  mma_rows_x_keys(s0, s1, qlo, qhi, k0, k1);
#pragma unroll
  for (int c = 0; c < 4; ++c) { s0[c] = fmaf(s0[c], sl2, lw); s1[c] = fmaf(s1[c], sl2, lw); }
  const float mn0 = fmaxf(st.m0, quad_max(fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]))));
  const float mn1 = fmaxf(st.m1, quad_max(fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]))));
  const float al0 = fast_exp2(st.m0 - mn0), al1 = fast_exp2(st.m1 - mn1);
  st.m0 = mn0; st.m1 = mn1;
  s0[0] = fast_exp2(s0[0] - mn0); s0[1] = fast_exp2(s0[1] - mn0); s1[0] = fast_exp2(s1[0] - mn0); s1[1] = fast_exp2(s1[1] - mn0);
  s0[2] = fast_exp2(s0[2] - mn1); s0[3] = fast_exp2(s0[3] - mn1); s1[2] = fast_exp2(s1[2] - mn1); s1[3] = fast_exp2(s1[3] - mn1);
  st.l0 = st.l0 * al0 + (s0[0] + s0[1] + s1[0] + s1[1]);   // per-lane partial sums; reduced over the quad at the end
  st.l1 = st.l1 * al1 + (s0[2] + s0[3] + s1[2] + s1[3]);
#pragma unroll
  for (int j = 0; j < 8; ++j) { st.o[j][0] *= al0; st.o[j][1] *= al0; st.o[j][2] *= al1; st.o[j][3] *= al1; }
  // the two C tiles of S are the k16 halves of the A operand
  pa[0] = pack_bf16(s0[0], s0[1]); pa[1] = pack_bf16(s0[2], s0[3]); pa[2] = pack_bf16(s1[0], s1[1]); pa[3] = pack_bf16(s1[2], s1[3]);
}

struct GlobalBlock {
  const bf16* k;
  const bf16* v;
  int64_t ks, vs;
  float lw;
};

// Block gi of the list streamed from global memory: the fine blocks, then the pooled tiles that
// did not fit in shared memory.  gi is warp-uniform; lane i of my_fine holds fine block i.
__device__ __forceinline__ GlobalBlock global_block(const AttnP<bf16>& a, int64_t b, int64_t h, int64_t bh, int64_t qb, int gi, int my_fine,
                                                    int n_smem_tiles, float lw1, float lw2) {
  GlobalBlock r;
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

// Copies pooled tiles 0..n_tiles-1 of the query group of `qb0` into shared memory (K and V), asynchronously.
__device__ __forceinline__ void stage_pooled_tiles(const AttnP<bf16>& a, int64_t bh, int64_t qb0, int n_tiles, bf16* sk, bf16* sv) {
  for (int c = threadIdx.x; c < n_tiles * kBS * 8; c += blockDim.x) {
    const int tile = c >> 7, row = (c >> 3) & 15, ch = (c & 7) * 8;
    int64_t off;
    const bf16 *gk, *gv;
    if (tile < a.p1_blocks) {
      off = (bh * a.n1 + p1_block(a, bh, qb0, tile) * kBS + row) * kD + ch;
      gk = a.pk + off; gv = a.pv + off;
    } else {
      off = (bh * a.n2 + (int64_t) (tile - a.p1_blocks) * kBS + row) * kD + ch;
      gk = a.pk2 + off; gv = a.pv2 + off;
    }
    const int so = (tile * kBS + row) * kSmemPitch + ch;
    cp_async16(sk + so, gk);
    cp_async16(sv + so, gv);
  }
  cp_async_commit();
}

template <int NW>
__global__ void __launch_bounds__(NW * 32, 2) attn_fwd_mma_kernel(AttnP<bf16> a, int n_smem_tiles) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* sk = reinterpret_cast<bf16*>(smem_raw);
  bf16* sv = sk + n_smem_tiles * kBS * kSmemPitch;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const int64_t qb0 = (int64_t) blockIdx.x * NW, qb = qb0 + warp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  stage_pooled_tiles(a, bh, qb0, n_smem_tiles, sk, sv);

  const int my_fine = lane < a.topk ? (int) fine_block(a, bh, qb, lane) : 0;
  const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
  const float sl2 = a.scale * 1.4426950408889634f;
  RowFrag qlo, qhi;
  load_rowfrag(qlo, a.q.row(b, h, qb * kBS + g), t);
  load_rowfrag(qhi, a.q.row(b, h, qb * kBS + g + 8), t);

  FwdState st;
#pragma unroll
  for (int j = 0; j < 8; ++j) st.o[j][0] = st.o[j][1] = st.o[j][2] = st.o[j][3] = 0.f;
  st.m0 = st.m1 = -INFINITY;
  st.l0 = st.l1 = 0.f;

  // ---- blocks streamed from global memory, next block's loads in flight behind the math
  const int n_pooled = a.p1_blocks + a.p2_blocks;
  const int n_glob = a.topk + (n_pooled - n_smem_tiles);
  {
    RowFrag k0, k1;
    ColFrag v;
    GlobalBlock r = global_block(a, b, h, bh, qb, 0, my_fine, n_smem_tiles, lw1, lw2);
    load_rowfrag(k0, r.k + (int64_t) g * r.ks, t);
    load_rowfrag(k1, r.k + (int64_t) (g + 8) * r.ks, t);
    load_colfrag(v, r.v, r.vs, g, t);
    for (int gi = 0; gi < n_glob; ++gi) {
      if (gi + 2 < n_glob) {   // two blocks ahead: K rows (lanes 0..15) and V rows (lanes 16..31) towards L1
        const GlobalBlock f = global_block(a, b, h, bh, qb, gi + 2, my_fine, n_smem_tiles, lw1, lw2);
        if (lane < 16) prefetch_tile_rows(f.k, f.ks, lane);
        else prefetch_tile_rows(f.v, f.vs, lane - 16);
      }
      uint32_t pa[4];
      fwd_scores(st, qlo, qhi, k0, k1, sl2, r.lw, pa);
      const bool more = gi + 1 < n_glob;
      if (more) {   // the key registers are free: start the next block's keys
        r = global_block(a, b, h, bh, qb, gi + 1, my_fine, n_smem_tiles, lw1, lw2);
        load_rowfrag(k0, r.k + (int64_t) g * r.ks, t);
        load_rowfrag(k1, r.k + (int64_t) (g + 8) * r.ks, t);
      }
      mma_x_cols(st.o, pa[0], pa[1], pa[2], pa[3], v);
      if (more) load_colfrag(v, r.v, r.vs, g, t);
    }
  }
  // ---- pooled tiles shared by the CTA
  cp_async_wait_all();
  __syncthreads();
  for (int ip = 0; ip < n_smem_tiles; ++ip) {
    RowFrag k0, k1;
    ColFrag v;
    const bf16* tk = sk + ip * kBS * kSmemPitch;
    load_rowfrag_smem(k0, tk + g * kSmemPitch, t);
    load_rowfrag_smem(k1, tk + (g + 8) * kSmemPitch, t);
    load_colfrag_smem(v, sv + ip * kBS * kSmemPitch, g, t);
    uint32_t pa[4];
    fwd_scores(st, qlo, qhi, k0, k1, sl2, ip < a.p1_blocks ? lw1 : lw2, pa);
    mma_x_cols(st.o, pa[0], pa[1], pa[2], pa[3], v);
  }

  const float l0 = quad_sum(st.l0), l1 = quad_sum(st.l1);
  store_acc_row<0>(a.o.row(b, h, qb * kBS + g), st.o, t, 1.f / l0);
  store_acc_row<1>(a.o.row(b, h, qb * kBS + g + 8), st.o, t, 1.f / l1);
  if (t == 0) {
    a.lse[bh * a.Nq + qb * kBS + g] = (st.m0 + log2f(l0)) * 0.6931471805599453f;
    a.lse[bh * a.Nq + qb * kBS + g + 8] = (st.m1 + log2f(l1)) * 0.6931471805599453f;
  }
}

// Fine stage alone (the pooled stages then run on tcgen05, attn_pooled_tc.cu, and merge into the
// o / lse written here).  Every selected K/V block costs a full L2/HBM round trip, far longer
// than the 16 MMAs it feeds, so each warp keeps kFineStages-1 blocks in flight with cp.async
// into its own ring of shared-memory stages (mma_frag.cuh) and reads the fragments from there.
constexpr int kFineStages = 3;

template <int NW>
__global__ void __launch_bounds__(NW * 32, 2) attn_fwd_fine_kernel(AttnP<bf16> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  bf16* ring = reinterpret_cast<bf16*>(smem_raw) + warp * (kFineStages * 2 * kRingTileElems);
  const int64_t qb = (int64_t) blockIdx.x * NW + warp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int my_fine = lane < a.topk ? (int) fine_block(a, bh, qb, lane) : 0;
  const float sl2 = a.scale * 1.4426950408889634f;
  const int n_glob = a.topk;
  // A lane copies the same four 16-byte chunks of every K tile and of every V tile (chunk = 4 i + lane / 8 -> row, lane % 8 ->
  // column): their global and shared-memory offsets are computed once, a block costs two base pointers and eight adds.
  int off_k[4], off_v[4], off_s[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = i * 4 + (lane >> 3), c = lane & 7;
    off_k[i] = r * (int) a.k.sn + c * 8;
    off_v[i] = r * (int) a.v.sn + c * 8;
    off_s[i] = r * 64 + ((c ^ (r & 7)) << 3);
  }
  // fragment read offsets inside a ring tile (rows r and r + 8 share r & 7, so the second row is 8 * 64 elements further)
  const int rd_k[2] = {g * 64 + (((2 * t) ^ (g & 7)) << 3), g * 64 + (((2 * t + 1) ^ (g & 7)) << 3)};
  const int rd_v[2] = {(2 * t) * 64 + ((g ^ ((2 * t) & 7)) << 3), (2 * t + 1) * 64 + ((g ^ ((2 * t + 1) & 7)) << 3)};
  const bf16* kb0 = a.k.row(b, h, 0);
  const bf16* vb0 = a.v.row(b, h, 0);
  const int64_t kblk = (int64_t) kBS * a.k.sn, vblk = (int64_t) kBS * a.v.sn;
  auto issue = [&](int i) {
    const int64_t j = __shfl_sync(0xffffffffu, my_fine, i);
    bf16* stage = ring + (i % kFineStages) * 2 * kRingTileElems;
    const bf16* kp = kb0 + j * kblk;
    const bf16* vp = vb0 + j * vblk;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      cp_async16(stage + off_s[u], kp + off_k[u]);
      cp_async16(stage + kRingTileElems + off_s[u], vp + off_v[u]);
    }
  };
#pragma unroll
  for (int s = 0; s < kFineStages - 1; ++s) {
    if (s < n_glob) issue(s);
    cp_async_commit();
  }
  RowFrag qlo, qhi;
  load_rowfrag(qlo, a.q.row(b, h, qb * kBS + g), t);
  load_rowfrag(qhi, a.q.row(b, h, qb * kBS + g + 8), t);
  FwdState st;
#pragma unroll
  for (int j = 0; j < 8; ++j) st.o[j][0] = st.o[j][1] = st.o[j][2] = st.o[j][3] = 0.f;
  st.m0 = st.m1 = -INFINITY;
  st.l0 = st.l1 = 0.f;
  for (int gi = 0; gi < n_glob; ++gi) {
    cp_async_wait_group<kFineStages - 2>();     // block gi has landed (this lane's chunks) ...
    __syncwarp();                               // ... and everybody else's; the stage read last time is free
    if (gi + kFineStages - 1 < n_glob) issue(gi + kFineStages - 1);
    cp_async_commit();
    const bf16* tk = ring + (gi % kFineStages) * 2 * kRingTileElems;
    RowFrag k0, k1;
    {
      const uint4 x0 = *reinterpret_cast<const uint4*>(tk + rd_k[0]), x1 = *reinterpret_cast<const uint4*>(tk + rd_k[1]);
      const uint4 y0 = *reinterpret_cast<const uint4*>(tk + 8 * 64 + rd_k[0]), y1 = *reinterpret_cast<const uint4*>(tk + 8 * 64 + rd_k[1]);
      k0.r[0] = x0.x; k0.r[1] = x0.y; k0.r[2] = x0.z; k0.r[3] = x0.w; k0.r[4] = x1.x; k0.r[5] = x1.y; k0.r[6] = x1.z; k0.r[7] = x1.w;
      k1.r[0] = y0.x; k1.r[1] = y0.y; k1.r[2] = y0.z; k1.r[3] = y0.w; k1.r[4] = y1.x; k1.r[5] = y1.y; k1.r[6] = y1.z; k1.r[7] = y1.w;
    }
    uint32_t pa[4];
    fwd_scores(st, qlo, qhi, k0, k1, sl2, 0.f, pa);
    ColFrag v;
    v.row[0] = *reinterpret_cast<const uint4*>(tk + kRingTileElems + rd_v[0]);
    v.row[1] = *reinterpret_cast<const uint4*>(tk + kRingTileElems + rd_v[1]);
    v.row[2] = *reinterpret_cast<const uint4*>(tk + kRingTileElems + 8 * 64 + rd_v[0]);
    v.row[3] = *reinterpret_cast<const uint4*>(tk + kRingTileElems + 8 * 64 + rd_v[1]);
    mma_x_cols(st.o, pa[0], pa[1], pa[2], pa[3], v);
  }
  const float l0 = quad_sum(st.l0), l1 = quad_sum(st.l1);
  store_acc_row<0>(a.o.row(b, h, qb * kBS + g), st.o, t, 1.f / l0);
  store_acc_row<1>(a.o.row(b, h, qb * kBS + g + 8), st.o, t, 1.f / l1);
  if (t == 0) {
    a.lse[bh * a.Nq + qb * kBS + g] = (st.m0 + log2f(l0)) * 0.6931471805599453f;
    a.lse[bh * a.Nq + qb * kBS + g + 8] = (st.m1 + log2f(l1)) * 0.6931471805599453f;
  }
}

// ---- eight fine blocks, second form ----------------------------------------------------------------
// The kernel above spends most of its issue slots around the MMAs: an online-softmax update (maximum, rescale of the 16x64
// output) per 16-key block, byte permutes for the V operand, run-time ring addresses.  This form, for top-8, takes the blocks in
// two halves of four: the four S tiles of a half are computed first, the softmax statistics are updated once per half, and P.V
// follows with V read by ldmatrix.trans.  The sixteen K / V tiles go through a per-warp ring of six 2 KB stages in the order
// K0..K3 V0..V3 K4..K7 V4..V7, five tiles ahead; the loop is unrolled over the tiles so that every shared-memory offset is an
// immediate.  The output leaves through stmatrix into a free stage and 128-bit row stores.
constexpr int kF8Stages = 6;
constexpr int kF8TileBytes = kRingTileElems * (int) sizeof(bf16);

template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}

template <int NW>
__global__ void __launch_bounds__(NW * 32, 2) attn_fwd_fine8_kernel(AttnP<bf16> a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  // the swizzle arithmetic works on absolute shared addresses: start at a 128-byte boundary (the launch adds 128 bytes)
  const uint32_t smem_sa = ((uint32_t) __cvta_generic_to_shared(smem_raw) + 127u) & ~127u;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t ring_sa = smem_sa + warp * (kF8Stages * kF8TileBytes);
  const uint32_t sa_cp0 = ring_sa + (lane >> 3) * 128 + (((lane & 7) ^ (lane >> 3)) << 4), sa_cp1 = sa_cp0 ^ 64;
  const uint32_t sa_f0 = ring_sa + g * 128 + (((2 * t) ^ g) << 4), sa_f1 = sa_f0 ^ 16;
  const uint32_t sa_m = ring_sa + ((lane & 7) + ((lane >> 3) & 1) * 8) * 128 + (((lane >> 4) ^ (lane & 7)) << 4);
  const int64_t qb = (int64_t) blockIdx.x * NW + warp, bh = blockIdx.y, b = bh / a.H, h = bh % a.H;
  const int my_fine = lane < 8 ? (int) fine_block(a, bh, qb, lane) : 0;
  const float sl2 = a.scale * 1.4426950408889634f;
  const char* k_lane = reinterpret_cast<const char*>(a.k.row(b, h, lane >> 3) + (lane & 7) * 8);
  const char* v_lane = reinterpret_cast<const char*>(a.v.row(b, h, lane >> 3) + (lane & 7) * 8);
  const int kblk = (int) (kBS * a.k.sn * sizeof(bf16)), vblk = (int) (kBS * a.v.sn * sizeof(bf16));
  // tile s of the sequence K0..K3 V0..V3 K4..K7 V4..V7
  auto issue = [&](auto s_tag) {
    constexpr int s = decltype(s_tag)::value, blk = (s / 8) * 4 + s % 4, ST = (s % kF8Stages) * kF8TileBytes;
    constexpr bool is_v = (s % 8) >= 4;
    const int j = __shfl_sync(0xffffffffu, my_fine, blk);
    const int blkb = is_v ? vblk : kblk;
    const char* p = (is_v ? v_lane : k_lane) + (int64_t) j * blkb;
    cp_async16_sa<ST>(sa_cp0, p);
    cp_async16_sa<ST + 512>(sa_cp1, p + (blkb >> 2));
    cp_async16_sa<ST + 1024>(sa_cp0, p + (blkb >> 1));
    cp_async16_sa<ST + 1536>(sa_cp1, p + 3 * (blkb >> 2));
  };
  static_for<0, kF8Stages - 1>([&](auto s_tag) {
    issue(s_tag);
    cp_async_commit();
  });
  RowFrag qlo, qhi;
  load_rowfrag(qlo, a.q.row(b, h, qb * kBS + g), t);
  load_rowfrag(qhi, a.q.row(b, h, qb * kBS + g + 8), t);
  float o[8][4], sc[4][2][4];
  uint32_t pa[4][4];
  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  static_for<0, 16>([&](auto s_tag) {
    constexpr int s = decltype(s_tag)::value, half = s / 8, i = s % 4, ST = (s % kF8Stages) * kF8TileBytes;
    constexpr bool is_v = (s % 8) >= 4;
    cp_async_wait_group<kF8Stages - 2>();       // tile s has landed (this lane's chunks) ...
    __syncwarp();                               // ... and everybody else's; the stage read last time is free
    if constexpr (s + kF8Stages - 1 < 16) issue(std::integral_constant<int, s + kF8Stages - 1>{});
    cp_async_commit();
    if constexpr (!is_v) {
      half_rows_x_keys<ST, true>(sc[i][0], sc[i][1], qlo, qhi, sa_f0);
      half_rows_x_keys<ST, false>(sc[i][0], sc[i][1], qlo, qhi, sa_f1);
      if constexpr (i == 3) {                   // the half's four S tiles are complete: one softmax update for 64 keys
        float x0 = -INFINITY, x1 = -INFINITY;
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            x0 = fmax3(x0, sc[u][n][0], sc[u][n][1]);
            x1 = fmax3(x1, sc[u][n][2], sc[u][n][3]);
          }
        const float mn0 = fmaxf(m0, quad_max(x0) * sl2), mn1 = fmaxf(m1, quad_max(x1) * sl2);
        if constexpr (half > 0) {
          const float al0 = fast_exp2(m0 - mn0), al1 = fast_exp2(m1 - mn1);
          l0 *= al0; l1 *= al1;
#pragma unroll
          for (int u = 0; u < 8; ++u) { o[u][0] *= al0; o[u][1] *= al0; o[u][2] *= al1; o[u][3] *= al1; }
        }
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            sc[u][n][0] = fast_exp2(fmaf(sc[u][n][0], sl2, -mn0)); sc[u][n][1] = fast_exp2(fmaf(sc[u][n][1], sl2, -mn0));
            sc[u][n][2] = fast_exp2(fmaf(sc[u][n][2], sl2, -mn1)); sc[u][n][3] = fast_exp2(fmaf(sc[u][n][3], sl2, -mn1));
            l0 += sc[u][n][0] + sc[u][n][1];    // per-lane partial sums; reduced over the quad at the end
            l1 += sc[u][n][2] + sc[u][n][3];
          }
          // the two C tiles of S are the k16 halves of the A operand
          pa[u][0] = pack_bf16(sc[u][0][0], sc[u][0][1]); pa[u][1] = pack_bf16(sc[u][0][2], sc[u][0][3]);
          pa[u][2] = pack_bf16(sc[u][1][0], sc[u][1][1]); pa[u][3] = pack_bf16(sc[u][1][2], sc[u][1][3]);
        }
      }
    } else {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r0, r1, r2, r3;
        ldsm_x4_trans<ST>(r0, r1, r2, r3, sa_m ^ (c << 5));
        if constexpr (s == 4) {                 // first product: no accumulator input
          mma_bf16_16816_z(o[2 * c], pa[i][0], pa[i][1], pa[i][2], pa[i][3], r0, r1);
          mma_bf16_16816_z(o[2 * c + 1], pa[i][0], pa[i][1], pa[i][2], pa[i][3], r2, r3);
        } else {
          mma_bf16_16816(o[2 * c], pa[i][0], pa[i][1], pa[i][2], pa[i][3], r0, r1);
          mma_bf16_16816(o[2 * c + 1], pa[i][0], pa[i][1], pa[i][2], pa[i][3], r2, r3);
        }
      }
    }
  });
  l0 = quad_sum(l0); l1 = quad_sum(l1);
  const float i0 = 1.f / l0, i1 = 1.f / l1;
  if (t == 0) {
    a.lse[bh * a.Nq + qb * kBS + g] = (m0 + log2f(l0)) * 0.6931471805599453f;
    a.lse[bh * a.Nq + qb * kBS + g + 8] = (m1 + log2f(l1)) * 0.6931471805599453f;
  }
  // accumulator tile u holds channels 8u + 2t, 8u + 2t + 1 of rows g (c0, c1) and g + 8 (c2, c3): through stage 0 to whole rows
  __syncwarp();
#pragma unroll
  for (int c = 0; c < 4; ++c)
    stsm_x4<0>(sa_m ^ (c << 5), pack_bf16(o[2 * c][0] * i0, o[2 * c][1] * i0), pack_bf16(o[2 * c][2] * i1, o[2 * c][3] * i1),
               pack_bf16(o[2 * c + 1][0] * i0, o[2 * c + 1][1] * i0), pack_bf16(o[2 * c + 1][2] * i1, o[2 * c + 1][3] * i1));
  __syncwarp();
  bf16* op = a.o.row(b, h, qb * kBS + (lane >> 3)) + (lane & 7) * 8;
  const int64_t os = 4 * a.o.sn;
  uint4 x;
  lds128<0>(x.x, x.y, x.z, x.w, sa_cp0);    *reinterpret_cast<uint4*>(op) = x;
  lds128<512>(x.x, x.y, x.z, x.w, sa_cp1);  *reinterpret_cast<uint4*>(op + os) = x;
  lds128<1024>(x.x, x.y, x.z, x.w, sa_cp0); *reinterpret_cast<uint4*>(op + 2 * os) = x;
  lds128<1536>(x.x, x.y, x.z, x.w, sa_cp1); *reinterpret_cast<uint4*>(op + 3 * os) = x;
}

// A bf16 call whose operands miss the tensor-core kernels' limits still runs, on the scalar kernels and many times
// slower: the call succeeds, and the thread's error string says why so that a caller who wonders can find out.
void note_scalar_path() {
  set_error("note: bf16 operands ran on the scalar kernels (the tensor-core kernels need 32-byte aligned rows, "
            "batch/head/token strides that are multiples of 16 elements, and top-k <= 32)");
}

bool mma_path_ok(const LlsaAttnArgs* g, bool bwd) {
  if (g->topk > 32 || (g->pk2 && g->topk_p > 32)) return false;
  // 256-bit fragment loads need 32-byte aligned rows
  const LlsaTensor* ts[8] = {g->q, g->k, g->v, g->o, bwd ? g->d_o : nullptr, bwd ? g->dq : nullptr, bwd ? g->dk : nullptr, bwd ? g->dv : nullptr};
  for (const LlsaTensor* t : ts) {
    if (!t) continue;
    if ((uintptr_t) t->ptr % 32) return false;
    for (int i = 0; i < 3; ++i)
      if (t->shape[i] != 1 && t->stride[i] % 16) return false;
  }
  return ((uintptr_t) g->pk->ptr % 32) == 0 && ((uintptr_t) g->pv->ptr % 32) == 0 &&
         (!g->pk2 || (((uintptr_t) g->pk2->ptr % 32) == 0 && ((uintptr_t) g->pv2->ptr % 32) == 0));
}

int pooled_smem_tiles(int n_pooled) { return n_pooled < 20 ? n_pooled : 20; }   // 20 tiles = 90 KB of K+V, two CTAs per SM

int launch_attn_fwd_mma(const LlsaAttnArgs* g, cudaStream_t st) {
  if (!mma_path_ok(g, false)) {
    note_scalar_path();
    return launch_attn_fwd_generic(g, st);
  }
  AttnP<bf16> a = build_attn_params<bf16>(g, false);
  constexpr int NW = 8;
  const int64_t BH = g->q->shape[0] * a.H;
  const bool loop_tc = pooled_loop_tc_keys(a) > 0;
  if ((pooled_tc_keys(a) || loop_tc) && !g->no_tcgen05) {
    // fine blocks on mma.sync (o and lse of the fine part alone), pooled keys on tcgen05, merged there
    if (a.topk == 8) {
      const size_t ring = (size_t) NW * kF8Stages * kF8TileBytes + 128;
      LLSA_SMEM_LIMIT((attn_fwd_fine8_kernel<NW>), ring);
      attn_fwd_fine8_kernel<NW><<<dim3((unsigned) (a.nq1 / NW), (unsigned) BH), NW * 32, ring, st>>>(a);
      LLSA_LAUNCH_OK("attn_fwd_fine8_kernel");
    } else {
      const size_t ring = (size_t) NW * kFineStages * 2 * kRingTileElems * sizeof(bf16);
      LLSA_SMEM_LIMIT((attn_fwd_fine_kernel<NW>), ring);
      attn_fwd_fine_kernel<NW><<<dim3((unsigned) (a.nq1 / NW), (unsigned) BH), NW * 32, ring, st>>>(a);
      LLSA_LAUNCH_OK("attn_fwd_fine_kernel");
    }
    return loop_tc ? launch_attn_fwd_pooled_loop_tc(g, a, BH, st) : launch_attn_fwd_pooled_tc(g, a, BH, st);
  }
  const int n_smem = pooled_smem_tiles(a.p1_blocks + a.p2_blocks);
  const size_t smem = (size_t) n_smem * kBS * kSmemPitch * sizeof(bf16) * 2;
  LLSA_SMEM_LIMIT((attn_fwd_mma_kernel<NW>), smem);
  dim3 grid((unsigned) (a.nq1 / NW), (unsigned) (g->q->shape[0] * a.H));
  attn_fwd_mma_kernel<NW><<<grid, NW * 32, smem, st>>>(a, n_smem);
  LLSA_LAUNCH_OK("attn_fwd_mma_kernel");
  return LLSA_OK;
}

}  // namespace llsa
