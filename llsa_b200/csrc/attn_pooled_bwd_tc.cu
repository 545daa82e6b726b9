// Pooled stages of the LLSA backward (two-level form) on tcgen05 tensor cores with TMEM accumulators.
// Replaces, for the pooled keys, the dQ half of _attn_bwd_res_dqkv (sparse_attention_res_2.py:287-415)
// and the dPK/dPV kernels _attn_bwd_res_dpkv1_sparse (:492-575) and _attn_bwd_res_dpkv2 (:418-489).
//
// A tile is 128 consecutive query rows; all of them attend to the same 192 pooled keys: the 128
// level-1 children of the parent's selected level-2 blocks (key tiles 0, 1) and the 64 level-2 keys
// (key tile 2; the kernel is used when exactly 64 exist).  Per tile, five GEMMs:
//     S  = Q  . PK^T        [128 x 192], K = 64      operands in shared memory (K-major both)
//     dP = dO . PV^T        [128 x 192], K = 64
//     dQ = dS . PK          [128 x 64],  K = 192     dS K-major, PK MN-major (the same copy of PK)
//     dPV = P^T  . dO       [192 x 64],  K = 128     P MN-major (rows = queries), dO MN-major
//     dPK = dS^T . Q        [192 x 64],  K = 128
// with P = exp(S*scale + ln w - lse) and dS = P * (dP - delta) * scale computed by the softmax warps
// between the first two and the last three.  The 64 level-2 keys would need an M = 64 product; instead
// P(tile 2) and dS(tile 2) are laid out next to each other and used as ONE M = 128 operand, so that
// [P2 | dS2]^T . dO holds dPV2 in TMEM lanes 0..63 and [P2 | dS2]^T . Q holds dPK2 in lanes 64..127.
//
// TMEM columns: S, then dP, share [0,192) (the softmax warps keep P in registers between the two);
// dQ [192,256); dPV1 [256,320); dPK1 [320,384); [P2|dS2]^T.dO [384,448); [P2|dS2]^T.Q [448,512).
// The level-1 results accumulate in TMEM over the two tiles of a parent, the level-2 results over all
// tiles of a head that the CTA walks, so the fp32 reductions to global memory happen once per parent /
// once per head and CTA instead of once per tile.
//
// One persistent CTA per SM walks a contiguous range of tiles (the two tiles of a parent share their
// level-1 keys, all tiles of a head share the level-2 keys: those are loaded only when they change).
//   warp 12, one lane: TMA producer (Q, dO double-buffered; pooled keys single-buffered)
//   warp 13, one lane: tcgen05.mma issuer.  tcgen05.mma operations execute in issue order, so S of the
//                      next tile is issued as soon as dP of this tile has been read, ahead of this
//                      tile's three output products.
//   warps 0-11       : three softmax warpgroups; group g owns key tile g (64 keys), thread r of a
//                      group owns query row r = TMEM lane r.  Afterwards group 0 adds dQ to the fine
//                      part already in dq, group 1 adds dPV1 / dPK1 and group 2 the level-2 results to
//                      the fp32 pooled-gradient accumulators (red.global.add.v4.f32).
// Every mbarrier wait is bounded; a wait that expires raises a CTA-wide abort flag, every role leaves
// its loop, the host-visible status word is set and TMEM is freed.
#include <string.h>

#include "attn.cuh"
#include "mma_frag.cuh"
#include "tc05.cuh"
#include "tma.cuh"

namespace llsa {

namespace {

constexpr int kRows = 128;
constexpr int kThreads = 448;         // 12 softmax warps + producer warp + MMA warp
constexpr int kTile = kRows * 64;     // elements of a [128 x 64] bf16 tile (16 KB)
constexpr float kLog2eF = 1.4426950408889634f;

struct BwdMaps {
  CUtensorMap q, d_o;          // [B,H,Nq,64] 4-D, box 128 rows
  CUtensorMap pk1, pv1;        // [BH*n1, 64], box 16 rows
  CUtensorMap pk2, pv2;        // [BH*n2, 64], box 64 rows
};

struct BwdBars {
  uint64_t full[2], mma_done[2], s_ready, s_consumed, dp_ready, pds_ready, out_ready;
};

constexpr uint32_t kColDQ = 192, kColPV1 = 256, kColPK1 = 320, kColX = 384, kColY = 448;

__device__ __forceinline__ bool bw_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < 400000; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_pooled_tc_kernel(AttnP<bf16> a, const __grid_constant__ BwdMaps maps, int n_tiles, int tiles_per_head, int* __restrict__ status) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ BwdBars bars;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  bf16* base = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  bf16* sQ = base;                      // [2][128][64]
  bf16* sDO = sQ + 2 * kTile;           // [2][128][64]
  bf16* sK1 = sDO + 2 * kTile;          // [128][64] level-1 keys of the parent
  bf16* sV1 = sK1 + kTile;
  bf16* sK2 = sV1 + kTile;              // [64][64] level-2 keys of the head
  bf16* sV2 = sK2 + kTile / 2;
  bf16* sP = sV2 + kTile / 2;           // P tiles 0, 1, 2, then dS tiles 2, 0, 1 (tile = [128 rows][64 keys])
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &s_abort;

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars.full[i], 1);
      tc::mbar_init(&bars.mma_done[i], 1);
    }
    tc::mbar_init(&bars.s_ready, 1);
    tc::mbar_init(&bars.dp_ready, 1);
    tc::mbar_init(&bars.out_ready, 1);
    tc::mbar_init(&bars.s_consumed, 12);     // one arrival per softmax warp
    tc::mbar_init(&bars.pds_ready, 12);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&s_tmem, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem;
  // contiguous tile range of this CTA
  const int t_begin = (int) ((int64_t) n_tiles * blockIdx.x / gridDim.x), t_end = (int) ((int64_t) n_tiles * (blockIdx.x + 1) / gridDim.x);
  const int n_my = t_end - t_begin;

  if (warp == 12) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      for (int i = 0; i < n_my; ++i) {
        const int tile = t_begin + i, s = i & 1;
        const int64_t bh = tile / tiles_per_head, row0 = (int64_t) (tile % tiles_per_head) * kRows;
        const bool new_parent = i == 0 || (tile >> 1) != ((tile - 1) >> 1);
        const bool new_head = i == 0 || bh != (tile - 1) / tiles_per_head;
        if (i >= 2 && !bw_wait(&bars.mma_done[s], ((i - 2) >> 1) & 1, abort_flag)) break;          // stage s is free
        if (i >= 1 && new_parent && !bw_wait(&bars.mma_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag)) break;   // key buffers are free
        tma::expect_tx(&bars.full[s], 2u * kTile * 2 + (new_parent ? 2u * kTile * 2 : 0u) + (new_head ? (uint32_t) kTile * 2 : 0u));
        tma::load_4d(sQ + s * kTile, &maps.q, &bars.full[s], 0, (int) row0, (int) (bh % a.H), (int) (bh / a.H));
        tma::load_4d(sDO + s * kTile, &maps.d_o, &bars.full[s], 0, (int) row0, (int) (bh % a.H), (int) (bh / a.H));
        if (new_parent) {
          for (int j = 0; j < 8; ++j) {
            const int r = (int) (bh * a.n1 + p1_block(a, bh, row0 / kBS, j) * kBS);
            tma::load_2d(sK1 + j * kBS * 64, &maps.pk1, &bars.full[s], 0, r);
            tma::load_2d(sV1 + j * kBS * 64, &maps.pv1, &bars.full[s], 0, r);
          }
        }
        if (new_head) {
          tma::load_2d(sK2, &maps.pk2, &bars.full[s], 0, (int) (bh * a.n2));
          tma::load_2d(sV2, &maps.pv2, &bars.full[s], 0, (int) (bh * a.n2));
        }
      }
    }
  } else if (warp == 13) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t id_s128 = tc::instr_desc(128, 128, 0, 0), id_s64 = tc::instr_desc(128, 64, 0, 0);
      const uint32_t id_dq = tc::instr_desc(128, 64, 0, 1), id_kv = tc::instr_desc(128, 64, 1, 1);
      const uint32_t k1a = tc::smem_u32(sK1), v1a = tc::smem_u32(sV1), k2a = tc::smem_u32(sK2), v2a = tc::smem_u32(sV2);
      const uint32_t pa = tc::smem_u32(sP), dsa2 = pa + 3 * kTile * 2, dsa0 = dsa2 + kTile * 2;
      auto issue_s = [&](int i) -> bool {          // S(i) = Q . [PK1 ; PK2]^T into columns [0,192)
        const int s = i & 1;
        if (!bw_wait(&bars.full[s], (i >> 1) & 1, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t qa = tc::smem_u32(sQ + s * kTile);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {      // K-major operands: 32 bytes per k-step inside the swizzled 128-byte row
          const uint64_t dq_ = tc::smem_desc(qa + ks * 32, 16, 1024);
          tc::umma_ss(tmem + 0, dq_, tc::smem_desc(k1a + ks * 32, 16, 1024), id_s128, ks > 0);
          tc::umma_ss(tmem + 128, dq_, tc::smem_desc(k2a + ks * 32, 16, 1024), id_s64, ks > 0);
        }
        tc::umma_commit(&bars.s_ready);
        return true;
      };
      bool ok = n_my > 0 && issue_s(0);
      for (int i = 0; ok && i < n_my; ++i) {
        const int s = i & 1, tile = t_begin + i;
        const uint32_t qa = tc::smem_u32(sQ + s * kTile), doa = tc::smem_u32(sDO + s * kTile);
        // dP(i) = dO . [PV1 ; PV2]^T over the columns of S once every softmax warp has read S
        if (!bw_wait(&bars.s_consumed, i & 1, abort_flag)) break;
        tc::fence_after_sync();
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t dd_ = tc::smem_desc(doa + ks * 32, 16, 1024);
          tc::umma_ss(tmem + 0, dd_, tc::smem_desc(v1a + ks * 32, 16, 1024), id_s128, ks > 0);
          tc::umma_ss(tmem + 128, dd_, tc::smem_desc(v2a + ks * 32, 16, 1024), id_s64, ks > 0);
        }
        tc::umma_commit(&bars.dp_ready);
        if (!bw_wait(&bars.pds_ready, i & 1, abort_flag)) break;
        tc::fence_after_sync();
        // the next tile's S goes first when it uses the same level-1 keys (their buffer is reloaded only after
        // this tile's products have completed, which a new parent's S would wait for)
        const bool next_same_parent = i + 1 < n_my && ((tile + 1) >> 1) == (tile >> 1);
        if (next_same_parent && !issue_s(i + 1)) break;
        // dQ = dS . PK: 12 k-steps of 16 keys; dS tile kt = ks / 4 (memory order 2, 0, 1), PK rows 16 ks .. 16 ks + 15
        for (int ks = 0; ks < 12; ++ks) {
          const int kt = ks >> 2;
          const uint32_t da = (kt == 2 ? dsa2 : dsa0 + kt * kTile * 2) + (ks & 3) * 32;
          const uint32_t kb = ks < 8 ? k1a + ks * 2048 : k2a + (ks - 8) * 2048;
          tc::umma_ss(tmem + kColDQ, tc::smem_desc(da, 16, 1024), tc::smem_desc(kb, 1024, 1024), id_dq, ks > 0);
        }
        // transposed products, K = 128 query rows in 8 k-steps of 16 rows (2048 bytes); the A operand spans two
        // 64-key tiles 16 KB apart (leading-dimension byte offset).  Level-1 results accumulate over the tiles of
        // a parent, level-2 results over the tiles of a head.
        const uint32_t acc1 = (i > 0 && (tile & 1)) ? 1u : 0u;
        const uint32_t acc2 = (i > 0 && (tile % tiles_per_head) != 0) ? 1u : 0u;
        for (int ks = 0; ks < 8; ++ks) {
          const uint64_t bdo = tc::smem_desc(doa + ks * 2048, 1024, 1024), bq = tc::smem_desc(qa + ks * 2048, 1024, 1024);
          const uint64_t ap2 = tc::smem_desc(pa + 2 * kTile * 2 + ks * 2048, kTile * 2, 1024);
          tc::umma_ss(tmem + kColPV1, tc::smem_desc(pa + ks * 2048, kTile * 2, 1024), bdo, id_kv, acc1 | (ks > 0));
          tc::umma_ss(tmem + kColPK1, tc::smem_desc(dsa0 + ks * 2048, kTile * 2, 1024), bq, id_kv, acc1 | (ks > 0));
          tc::umma_ss(tmem + kColX, ap2, bdo, id_kv, acc2 | (ks > 0));
          tc::umma_ss(tmem + kColY, ap2, bq, id_kv, acc2 | (ks > 0));
        }
        tc::umma_commit(&bars.out_ready);
        tc::umma_commit(&bars.mma_done[s]);
        if (!next_same_parent && i + 1 < n_my && !issue_s(i + 1)) break;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax / dS, then the drains; thread = query row
    const int wg = warp >> 2, r = (warp & 3) * 32 + lane;
    const float sl2 = a.scale * kLog2eF;
    const float lw = log2f(wg < 2 ? a.w1 : a.w2);
    const uint32_t t_row = tmem + ((uint32_t) ((warp & 3) * 32) << 16);
    bf16* myP = sP + wg * kTile;
    bf16* myDS = sP + (wg == 2 ? 3 : 4 + wg) * kTile;
    float va[32], vb[32];
    uint4 dqv[8];
    // group 0: dq row of `tile` = fine part (already in memory, fetched into dqv) + pooled part (TMEM)
    auto load_dq = [&](int tile) {
      const int64_t bh = tile / tiles_per_head, row = (int64_t) (tile % tiles_per_head) * kRows + r;
      const bf16* p = a.dq.row(bh / a.H, bh % a.H, row);
#pragma unroll
      for (int q = 0; q < 8; ++q) dqv[q] = *reinterpret_cast<const uint4*>(p + 8 * q);
    };
    auto drain_dq = [&](int tile) {
      const int64_t bh = tile / tiles_per_head, row = (int64_t) (tile % tiles_per_head) * kRows + r;
      bf16* dqrow = a.dq.row(bh / a.H, bh % a.H, row);
      tc::tmem_ld32_async(t_row + kColDQ, va);
      tc::tmem_ld32_async(t_row + kColDQ + 32, vb);
      tc::tmem_ld_wait(va);
      tc::tmem_ld_wait(vb);
      auto add_store = [&](const float (&v)[32], int c0) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const uint4 f = dqv[(c0 >> 3) + q];
          uint4 w;
          w.x = pack_bf16(bf16_lo(f.x) + v[8 * q], bf16_hi(f.x) + v[8 * q + 1]);
          w.y = pack_bf16(bf16_lo(f.y) + v[8 * q + 2], bf16_hi(f.y) + v[8 * q + 3]);
          w.z = pack_bf16(bf16_lo(f.z) + v[8 * q + 4], bf16_hi(f.z) + v[8 * q + 5]);
          w.w = pack_bf16(bf16_lo(f.w) + v[8 * q + 6], bf16_hi(f.w) + v[8 * q + 7]);
          *reinterpret_cast<uint4*>(dqrow + c0 + 8 * q) = w;
        }
      };
      add_store(va, 0);
      add_store(vb, 32);
    };
    // groups 1, 2: TMEM lane r = pooled key r of the tile's key set, added to the fp32 accumulators in global memory
    auto drain_cols = [&](float* dst, uint32_t col, float mul) {
      tc::tmem_ld32_async(t_row + col, va);
      tc::tmem_ld32_async(t_row + col + 32, vb);
      tc::tmem_ld_wait(va);
      tc::tmem_ld_wait(vb);
#pragma unroll
      for (int q = 0; q < 8; ++q) red_add_v4(dst + 4 * q, va[4 * q] * mul, va[4 * q + 1] * mul, va[4 * q + 2] * mul, va[4 * q + 3] * mul);
#pragma unroll
      for (int q = 0; q < 8; ++q) red_add_v4(dst + 32 + 4 * q, vb[4 * q] * mul, vb[4 * q + 1] * mul, vb[4 * q + 2] * mul, vb[4 * q + 3] * mul);
    };
    bool pending = false;        // the previous tile's products have not been waited for yet
    for (int i = 0; i < n_my; ++i) {
      const int tile = t_begin + i;
      const int64_t bh = tile / tiles_per_head, row0 = (int64_t) (tile % tiles_per_head) * kRows, row = row0 + r;
      const float off = lw - a.lse[bh * a.Nq + row] * kLog2eF;
      const float dls = a.delta[bh * a.Nq + row] * a.scale;
      if (pending && wg == 0) load_dq(tile - 1);
      bool ok = __all_sync(0xffffffffu, bw_wait(&bars.s_ready, i & 1, abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      uint32_t pk[32];          // this row's 64 probabilities, bf16 pairs, kept for dS
      tc::tmem_ld32_async(t_row + wg * 64, va);
      tc::tmem_ld32_async(t_row + wg * 64 + 32, vb);
      tc::tmem_ld_wait(va);
      tc::tmem_ld_wait(vb);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        pk[j] = pack_bf16(fast_exp2(fmaf(va[2 * j], sl2, off)), fast_exp2(fmaf(va[2 * j + 1], sl2, off)));
        pk[16 + j] = pack_bf16(fast_exp2(fmaf(vb[2 * j], sl2, off)), fast_exp2(fmaf(vb[2 * j + 1], sl2, off)));
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.s_consumed);
      if (pending) {
        // the previous tile's products still read its P / dS tiles: wait for them before overwriting (and finish its dq)
        ok = __all_sync(0xffffffffu, bw_wait(&bars.out_ready, (i - 1) & 1, abort_flag));
        tc::fence_after_sync();
        if (!ok) break;
        if (wg == 0) drain_dq(tile - 1);
        pending = false;
      }
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<uint4*>(myP + tc::swz(r, q)) = make_uint4(pk[4 * q], pk[4 * q + 1], pk[4 * q + 2], pk[4 * q + 3]);
      ok = __all_sync(0xffffffffu, bw_wait(&bars.dp_ready, i & 1, abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      tc::tmem_ld32_async(t_row + wg * 64, va);
      tc::tmem_ld32_async(t_row + wg * 64 + 32, vb);
      tc::tmem_ld_wait(va);
      tc::tmem_ld_wait(vb);
      auto ds_store = [&](const float (&v)[32], int half) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 w;
          uint32_t* wp = reinterpret_cast<uint32_t*>(&w);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const uint32_t p2 = pk[half * 16 + 4 * q + e];
            wp[e] = pack_bf16(bf16_lo(p2) * fmaf(v[8 * q + 2 * e], a.scale, -dls), bf16_hi(p2) * fmaf(v[8 * q + 2 * e + 1], a.scale, -dls));
          }
          *reinterpret_cast<uint4*>(myDS + tc::swz(r, half * 4 + q)) = w;
        }
      };
      ds_store(va, 0);
      ds_store(vb, 1);
      tc::fence_async_smem();          // P, dS must be visible to the tensor core's (async proxy) reads
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.pds_ready);
      // A tile that ends its parent inside this CTA's range is finished at once (the next tile's S has to wait for
      // new keys anyway); otherwise the wait moves behind the next tile's exponentials.
      const bool last = i == n_my - 1;
      if (!((tile & 1) || last)) { pending = true; continue; }
      if (wg == 0) load_dq(tile);
      ok = __all_sync(0xffffffffu, bw_wait(&bars.out_ready, i & 1, abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      if (wg == 0) {
        drain_dq(tile);
      } else if (wg == 1) {
        const int64_t key = p1_block(a, bh, row0 / kBS, r >> 4) * kBS + (r & 15);
        drain_cols(a.dpv + (bh * a.n1 + key) * kD, kColPV1, a.kvw1 / a.w1);
        drain_cols(a.dpk + (bh * a.n1 + key) * kD, kColPK1, a.kvw1 / a.w1);
      } else if (last || (tile + 1) % tiles_per_head == 0) {
        // lanes 0..63: level-2 key r, dPV2 in [P2|dS2]^T.dO; lanes 64..127: level-2 key r - 64, dPK2 in [P2|dS2]^T.Q
        if (r < 64) drain_cols(a.dpv2 + (bh * a.n2 + r) * kD, kColX, a.kvw2 / a.w2);
        else drain_cols(a.dpk2 + (bh * a.n2 + (r - 64)) * kD, kColY, a.kvw2 / a.w2);
      }
      tc::fence_before_sync();      // the TMEM reads above are ordered before this warp's next barrier arrival
    }
  }
  tc::fence_before_sync();
  __syncthreads();
  if (tid == 0 && s_abort && status) *status = 1;
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
}

}  // namespace

// True when the tcgen05 pooled backward can take this problem: two levels, 8 selected parents (128 level-1
// pooled keys per row), exactly 64 level-2 keys, whole 128-row tiles.
bool pooled_bwd_tc_ok(const AttnP<bf16>& a) {
  return a.two_level && a.p1_blocks == 8 && a.p2_blocks == 4 && a.n2 == 64 && a.Nq % 256 == 0;
}

int launch_attn_bwd_pooled_tc(const LlsaAttnArgs* g, const AttnP<bf16>& a, int64_t BH, cudaStream_t st) {
  BwdMaps maps;
  memset(&maps, 0, sizeof(maps));
  int rc;
  if ((rc = tma::make_map_bhnd(&maps.q, g->q, kRows))) return rc;
  if ((rc = tma::make_map_bhnd(&maps.d_o, g->d_o, kRows))) return rc;
  if ((rc = tma::make_map_rows(&maps.pk1, a.pk, (uint64_t) BH * a.n1, kBS))) return rc;
  if ((rc = tma::make_map_rows(&maps.pv1, a.pv, (uint64_t) BH * a.n1, kBS))) return rc;
  if ((rc = tma::make_map_rows(&maps.pk2, a.pk2, (uint64_t) BH * a.n2, 64))) return rc;
  if ((rc = tma::make_map_rows(&maps.pv2, a.pv2, (uint64_t) BH * a.n2, 64))) return rc;
  const int tiles_per_head = (int) (a.Nq / kRows), n_tiles = (int) (BH * tiles_per_head);
  int dev = 0, sms = 148;
  LLSA_CUDA_OK(cudaGetDevice(&dev));
  LLSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = n_tiles < sms ? n_tiles : sms;
  const size_t smem = 1024 + (size_t) 13 * kTile * sizeof(bf16);     // Q, dO x 2, K1, V1, K2 + V2, P x 3, dS x 3
  LLSA_CUDA_OK(cudaFuncSetAttribute(attn_bwd_pooled_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
  attn_bwd_pooled_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, n_tiles, tiles_per_head, nullptr);
  LLSA_LAUNCH_OK("attn_bwd_pooled_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
