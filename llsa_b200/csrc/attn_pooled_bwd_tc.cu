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
// P(tile 2) and dS(tile 2) are laid out next to each other and used as ONE M = 128 operand against
// [Q | dO] (N = 128): the result holds dPK2 in TMEM lanes 64..127 of its first 64 columns and dPV2 in
// lanes 0..63 of its last 64.
//
// TMEM columns: S, then dP, share [0,192) (the softmax warps keep P in registers between the two);
// dQ [192,256); dPV1 [256,320); dPK1 [320,384); [P2|dS2]^T.[Q|dO] [384,512).
// The level-1 results accumulate in TMEM over the two tiles of a parent, the level-2 results over all
// tiles of a head that the CTA walks, so the fp32 reductions to global memory (whose rate at the L2
// is what bounds them) happen once per parent / once per head and CTA, and a warpgroup of their own
// issues them while the others are already on the next tile.
//
// One persistent CTA per SM walks a contiguous range of tiles.
//   warps 0-11        : three softmax warpgroups; group g owns key tile g (64 keys), thread r of a
//                       group owns query row r = TMEM lane r.  Group 0 also adds dQ to the fine part
//                       already in dq (through shared memory, so that global rows are touched whole).
//   warps 12-15       : drain warpgroup: at the end of a parent adds dPV1 / dPK1 (TMEM lane = pooled
//                       key) to the fp32 pooled-gradient accumulators with red.global.add.v4.f32, at
//                       the end of a head the level-2 results.
//   warp 16, one lane : TMA producer (Q, dO and the level-1 keys double-buffered; level-1 values
//                       reloaded as soon as dP of the parent's last tile has read them)
//   warp 17, one lane : tcgen05.mma issuer for S, dP and dQ.  Its operations execute in issue order, so S of
//                       the next tile is issued as soon as dP of this tile has been read, ahead of dQ.
//   warp 18, one lane : tcgen05.mma issuer for the three transposed products (accumulators and operands no
//                       instruction of warp 17 writes; ordered against it by the barriers only).
// Every mbarrier wait is bounded; a wait that expires raises a CTA-wide abort flag, every role leaves
// its loop, the host-visible status word is set and TMEM is freed.
#include <string.h>

#include <type_traits>

#include "attn.cuh"
#include "mma_frag.cuh"
#include "tc05.cuh"
#include "tma.cuh"

namespace llsa {

namespace {

constexpr int kRows = 128;
constexpr int kThreads = 608;         // 12 softmax warps + 4 drain warps + producer warp + two MMA warps
constexpr int kTile = kRows * 64;     // elements of a [128 x 64] bf16 tile (16 KB)
constexpr float kLog2eF = 1.4426950408889634f;
constexpr uint32_t kColDQ = 192, kColPV1 = 256, kColPK1 = 320, kColYX = 384, kColY = 384, kColX = 448;

struct BwdMaps {
  CUtensorMap q, d_o;          // [B,H,Nq,64] 4-D, box 128 rows
  CUtensorMap pk1, pv1;        // [BH*n1, 64], box 16 rows
  CUtensorMap pk2, pv2;        // [BH*n2, 64], box 64 rows
};

// Phases: full / mma_done / v_free alternate between two barriers by tile parity; the others complete once per
// tile (acc_free: once per parent).
struct BwdBars {
  uint64_t full[2], mma_done[2], v_free[2], s_ready, s_consumed, dp_ready, pds_ready, out_ready, dq_free, acc_free;
};

__global__ void __launch_bounds__(kThreads, 1)
attn_bwd_pooled_tc_kernel(AttnP<bf16> a, const __grid_constant__ BwdMaps maps, int n_tiles, int tiles_per_head) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ BwdBars bars;
  __shared__ uint32_t s_tmem;
  __shared__ tc::WaitCtl s_ctl;
  bf16* base = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  bf16* sQ = base;                      // [2][128][64]
  bf16* sDO = sQ + 2 * kTile;           // [2][128][64]
  bf16* sK1 = sDO + 2 * kTile;          // [2][128][64] level-1 keys, buffer = parity of the parent
  bf16* sK2 = sK1 + 2 * kTile;          // [64][64] level-2 keys of the head
  bf16* sV1 = sK2 + kTile / 2;          // [128][64] level-1 values, then
  bf16* sV2 = sV1 + kTile;              // [64][64] level-2 values: 192 contiguous rows
  bf16* sP = sV2 + kTile / 2;           // P tiles 0, 1, 2, then dS tiles 2, 0, 1 (tile = [128 rows][64 keys])
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile tc::WaitCtl* abort_flag = &s_ctl;

  if (tid == 0) {
    s_ctl.abort = 0;
    s_ctl.limit = a.wait_limit > 0 ? a.wait_limit : tc::kWaitPolls;
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars.full[i], 1);
      tc::mbar_init(&bars.mma_done[i], 2);
      tc::mbar_init(&bars.v_free[i], 1);
    }
    tc::mbar_init(&bars.s_ready, 1);
    tc::mbar_init(&bars.dp_ready, 1);
    tc::mbar_init(&bars.out_ready, 2);        // one commit per MMA-issuing thread
    tc::mbar_init(&bars.s_consumed, 12);     // one arrival per softmax warp
    tc::mbar_init(&bars.pds_ready, 12);
    tc::mbar_init(&bars.dq_free, 4);         // one arrival per drain warp
    tc::mbar_init(&bars.acc_free, 4);
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

  if (warp == 16) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      for (int i = 0; i < n_my; ++i) {
        const int tile = t_begin + i, s = i & 1;
        const int bh = tile / tiles_per_head, row0 = (tile % tiles_per_head) * kRows;
        const bool new_parent = i == 0 || (tile >> 1) != ((tile - 1) >> 1);
        const bool new_head = i == 0 || bh != (tile - 1) / tiles_per_head;
        int krow[8];                      // rows of the parent's 8 selected level-1 key blocks: independent loads, ahead of the waits
        if (new_parent) {
#pragma unroll
          for (int j = 0; j < 8; ++j) krow[j] = (int) ((int64_t) bh * a.n1 + p1_block(a, bh, row0 / kBS, j) * kBS);
        }
        // stage s (and the level-1 key buffer of the parent two back) is free once every product of tile i - 2 has completed
        if (i >= 2 && !tc::bounded_wait(&bars.mma_done[s], ((i - 2) >> 1) & 1, abort_flag)) break;
        // the level-2 buffers are free once every product of the previous tile has completed
        if (i >= 1 && new_head && !tc::bounded_wait(&bars.mma_done[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag)) break;
        tma::expect_tx(&bars.full[s], 2u * kTile * 2 + (new_parent ? 2u * kTile * 2 : 0u) + (new_head ? (uint32_t) kTile * 2 : 0u));
        tma::load_4d(sQ + s * kTile, &maps.q, &bars.full[s], 0, row0, bh % a.H, bh / a.H);
        tma::load_4d(sDO + s * kTile, &maps.d_o, &bars.full[s], 0, row0, bh % a.H, bh / a.H);
        if (new_head) {
          tma::load_2d(sK2, &maps.pk2, &bars.full[s], 0, (int) ((int64_t) bh * a.n2));
          tma::load_2d(sV2, &maps.pv2, &bars.full[s], 0, (int) ((int64_t) bh * a.n2));
        }
        if (new_parent) {
          bf16* k1 = sK1 + ((tile >> 1) & 1) * kTile;
#pragma unroll
          for (int j = 0; j < 8; ++j) tma::load_2d(k1 + j * kBS * 64, &maps.pk1, &bars.full[s], 0, krow[j]);
          // the level-1 values are last read by dP of the previous tile.  New parents come every other tile, so one of
          // the two v_free barriers is waited on at each of its phases and the other never.
          if (i >= 1 && !tc::bounded_wait(&bars.v_free[(i - 1) & 1], ((i - 1) >> 1) & 1, abort_flag)) break;
#pragma unroll
          for (int j = 0; j < 8; ++j) tma::load_2d(sV1 + j * kBS * 64, &maps.pv1, &bars.full[s], 0, krow[j]);
        }
      }
    }
  } else if (warp == 17) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t id_s128 = tc::instr_desc(128, 128, 0, 0), id_s64 = tc::instr_desc(128, 64, 0, 0), id_s192 = tc::instr_desc(128, 192, 0, 0);
      const uint32_t id_dq = tc::instr_desc(128, 64, 0, 1), id_kv = tc::instr_desc(128, 64, 1, 1), id_kv2 = tc::instr_desc(128, 128, 1, 1);
      // Shared-memory descriptors as (low word, high word).  The high word (stride between 8-row groups = 1024 bytes,
      // descriptor version, 128-byte swizzle) is the same for every operand here; the low word holds the address
      // (>> 4, 14 bits: addresses stay below 2^18) and the leading-dimension byte offset, so a k-step is one 32-bit add:
      // K-major operand: 32 bytes (2 units) per k-step of 16 channels inside the swizzled 128-byte row;
      // MN-major operand: 16 rows = 2048 bytes (128 units) per k-step.
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      // Every operand sits at a compile-time offset from the 1024-byte aligned base, and the address field counts 16-byte
      // units below 2^14, so each low word is `sb` plus a constant: one live register instead of twenty.
      const uint32_t sb = (tc::smem_u32(base) >> 4) & 0x3FFFu;
      constexpr uint32_t kU = (uint32_t) (kTile * 2) >> 4;          // 16-byte units of one [128 x 64] tile
      auto lo = [sb](uint32_t units, uint32_t lbo_bytes) { return sb + units + ((lbo_bytes >> 4) << 16); };
      constexpr uint32_t kStage = kU;                                // one 16 KB buffer further
      constexpr uint32_t kT = kTile * 2;                             // bytes of a tile
      constexpr uint32_t uQ = 0, uDO = 2 * kU, uK1 = 4 * kU, uK2 = 6 * kU, uV1 = 6 * kU + kU / 2, uP = 8 * kU;
      const uint32_t lK2_k = lo(uK2, 16), lK2_m = lo(uK2, 1024), lV_k = lo(uV1, 16);                // [V1;V2] as N = 192 rows
      const uint32_t lDS_k0 = lo(uP + 4 * kU, 16), lDS_k1 = lo(uP + 5 * kU, 16), lDS_k2 = lo(uP + 3 * kU, 16);
      const uint32_t lP1_m = lo(uP, kT), lDS1_m = lo(uP + 4 * kU, kT), lP2_m = lo(uP + 2 * kU, kT);   // M = 128 over two tiles
      const uint32_t lQ_k0 = lo(uQ, 16), lDO_k0 = lo(uDO, 16), lQ_m0 = lo(uQ, 1024), lDO_m0 = lo(uDO, 1024);
      const uint32_t lQDO_m0 = lo(uQ, 2 * kT);                       // N = 128: channels of Q, then of dO (32 KB further)
      const uint32_t lK1_k0 = lo(uK1, 16), lK1_m0 = lo(uK1, 1024);
      auto issue_s = [&](int i) -> bool {          // S(i) = Q . [PK1 ; PK2]^T into columns [0,192)
        const int s = i & 1;
        if (!tc::bounded_wait(&bars.full[s], (i >> 1) & 1, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t q_ = lQ_k0 + s * kStage, k1_ = lK1_k0 + (((t_begin + i) >> 1) & 1) * kStage;
        tc::umma_ss_lh<0>(tmem, q_, hi, k1_, hi, id_s128);
        tc::umma_ss_lh<0>(tmem + 128, q_, hi, lK2_k, hi, id_s64);
#pragma unroll
        for (int ks = 1; ks < 4; ++ks) {
          tc::umma_ss_lh<1>(tmem, q_ + 2 * ks, hi, k1_ + 2 * ks, hi, id_s128);
          tc::umma_ss_lh<1>(tmem + 128, q_ + 2 * ks, hi, lK2_k + 2 * ks, hi, id_s64);
        }
        tc::umma_commit(&bars.s_ready);
        return true;
      };
      bool ok = n_my > 0 && issue_s(0);
      for (int i = 0; ok && i < n_my; ++i) {
        const int s = i & 1, tile = t_begin + i;
        // dP(i) = dO . [PV1 ; PV2]^T over the columns of S once every softmax warp has read S
        if (!tc::bounded_wait(&bars.s_consumed, i & 1, abort_flag)) break;
        tc::fence_after_sync();
        {
          const uint32_t d_ = lDO_k0 + s * kStage;
          tc::umma_ss_lh<0>(tmem, d_, hi, lV_k, hi, id_s192);
#pragma unroll
          for (int ks = 1; ks < 4; ++ks) tc::umma_ss_lh<1>(tmem, d_ + 2 * ks, hi, lV_k + 2 * ks, hi, id_s192);
        }
        tc::umma_commit(&bars.dp_ready);
        tc::umma_commit(&bars.v_free[s]);
        if (!tc::bounded_wait(&bars.pds_ready, i & 1, abort_flag)) break;
        tc::fence_after_sync();
        // The next tile's S goes ahead of this tile's output products, unless it belongs to a new head: the level-2
        // buffers are reloaded only after these products have completed.
        const bool next_early = i + 1 < n_my && (tile + 1) % tiles_per_head != 0;
        if (next_early && !issue_s(i + 1)) break;
        // dQ = dS . [PK1 ; PK2]: 12 k-steps of 16 keys, dS tile ks / 4; its columns are free once the drain warps have read
        // the previous tile's dQ
        if (i > 0 && !tc::bounded_wait(&bars.dq_free, (i - 1) & 1, abort_flag)) break;
        tc::fence_after_sync();
        {
          const uint32_t k1_ = lK1_m0 + ((tile >> 1) & 1) * kStage;
          tc::umma_ss_lh<0>(tmem + kColDQ, lDS_k0, hi, k1_, hi, id_dq);
#pragma unroll
          for (int ks = 1; ks < 4; ++ks) tc::umma_ss_lh<1>(tmem + kColDQ, lDS_k0 + 2 * ks, hi, k1_ + 128 * ks, hi, id_dq);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) tc::umma_ss_lh<1>(tmem + kColDQ, lDS_k1 + 2 * ks, hi, k1_ + 128 * (4 + ks), hi, id_dq);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) tc::umma_ss_lh<1>(tmem + kColDQ, lDS_k2 + 2 * ks, hi, lK2_m + 128 * ks, hi, id_dq);
        }
        tc::umma_commit(&bars.out_ready);           // this thread's half: S, dP, dQ of the tile
        tc::umma_commit(&bars.mma_done[s]);
        if (!next_early && i + 1 < n_my && !issue_s(i + 1)) break;
      }
    }
  } else if (warp == 18) {
    // ---------------------------------------------------------------- second MMA issuer: the three transposed products
    // One thread issues a tcgen05.mma of these shapes every 56-90 cycles here, the pipe takes one every 48-64: the tile's 48
    // instructions are dealt to two threads in two warps.  This one's 24 write accumulators nobody else's instructions
    // touch and read P / dS, Q and dO only, so nothing orders the two threads but the barriers: out_ready and mma_done
    // count one commit of each.
    if (lane == 0) {
      const uint32_t id_kv = tc::instr_desc(128, 64, 1, 1), id_kv2 = tc::instr_desc(128, 128, 1, 1);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      const uint32_t sb = (tc::smem_u32(base) >> 4) & 0x3FFFu;
      constexpr uint32_t kU = (uint32_t) (kTile * 2) >> 4, kStage = kU, kT = kTile * 2;
      auto lo = [sb](uint32_t units, uint32_t lbo_bytes) { return sb + units + ((lbo_bytes >> 4) << 16); };
      constexpr uint32_t uQ = 0, uDO = 2 * kU, uP = 8 * kU;
      const uint32_t lP1_m = lo(uP, kT), lDS1_m = lo(uP + 4 * kU, kT), lP2_m = lo(uP + 2 * kU, kT);   // M = 128 over two tiles
      const uint32_t lQ_m0 = lo(uQ, 1024), lDO_m0 = lo(uDO, 1024), lQDO_m0 = lo(uQ, 2 * kT);
      int parents_done = 0;
      for (int i = 0; i < n_my; ++i) {
        const int s = i & 1, tile = t_begin + i;
        if (!tc::bounded_wait(&bars.pds_ready, i & 1, abort_flag)) break;
        tc::fence_after_sync();
        // transposed products, K = 128 query rows in 8 k-steps.  Level-1 results accumulate over the tiles of a
        // parent, level-2 results over the tiles of a head; a fresh start waits for the drain warps to have read
        // the previous parent's results.
        const uint32_t acc1 = (i > 0 && (tile & 1)) ? 1u : 0u;
        const uint32_t acc2 = (i > 0 && (tile % tiles_per_head) != 0) ? 1u : 0u;
        if (!acc1 && parents_done > 0 && !tc::bounded_wait(&bars.acc_free, (parents_done - 1) & 1, abort_flag)) break;
        tc::fence_after_sync();
        {
          const uint32_t do_ = lDO_m0 + s * kStage, q_ = lQ_m0 + s * kStage, qdo_ = lQDO_m0 + s * kStage;
          tc::umma_ss_lh(tmem + kColPV1, lP1_m, hi, do_, hi, id_kv, acc1);
          tc::umma_ss_lh(tmem + kColPK1, lDS1_m, hi, q_, hi, id_kv, acc1);
          tc::umma_ss_lh(tmem + kColYX, lP2_m, hi, qdo_, hi, id_kv2, acc2);
#pragma unroll
          for (int ks = 1; ks < 8; ++ks) {
            tc::umma_ss_lh<1>(tmem + kColPV1, lP1_m + 128 * ks, hi, do_ + 128 * ks, hi, id_kv);
            tc::umma_ss_lh<1>(tmem + kColPK1, lDS1_m + 128 * ks, hi, q_ + 128 * ks, hi, id_kv);
            tc::umma_ss_lh<1>(tmem + kColYX, lP2_m + 128 * ks, hi, qdo_ + 128 * ks, hi, id_kv2);
          }
        }
        tc::umma_commit(&bars.out_ready);
        tc::umma_commit(&bars.mma_done[s]);
        if ((tile & 1) || i == n_my - 1) ++parents_done;
      }
    }
  } else if (warp >= 12) {
    // ---------------------------------------------------------------- drain warpgroup
    const int qd = warp & 3, r = qd * 32 + lane;
    const uint32_t t_row = tmem + ((uint32_t) (qd * 32) << 16);
    float va[16];
    auto red_cols = [&](float* dst, uint32_t col, float mul) {      // 64 columns of this lane -> dst[0..63]
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tc::tmem_ld16(t_row + col + 16 * c, va);
#pragma unroll
        for (int q = 0; q < 4; ++q) red_add_v4(dst + 16 * c + 4 * q, va[4 * q] * mul, va[4 * q + 1] * mul, va[4 * q + 2] * mul, va[4 * q + 3] * mul);
      }
    };
    for (int i = 0; i < n_my; ++i) {
      const int tile = t_begin + i;
      const int bh = tile / tiles_per_head, row0 = (tile % tiles_per_head) * kRows;
      const bool parent_end = (tile & 1) || i == n_my - 1;
      // every tile: dq row r of the tile = fine part (already in memory) + pooled part (TMEM lane r = query row r)
      bf16* dqrow = a.dq.row(bh / a.H, bh % a.H, row0 + r);
      uint4 old[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) old[q] = *reinterpret_cast<const uint4*>(dqrow + 8 * q);
      const int64_t key = parent_end ? p1_block(a, bh, row0 / kBS, r >> 4) * kBS + (r & 15) : 0;
      const bool ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.out_ready, i & 1, abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tc::tmem_ld16(t_row + kColDQ + 16 * c, va);
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const uint4 f = old[2 * c + q];
          uint4 w;
          w.x = pack_bf16(bf16_lo(f.x) + va[8 * q], bf16_hi(f.x) + va[8 * q + 1]);
          w.y = pack_bf16(bf16_lo(f.y) + va[8 * q + 2], bf16_hi(f.y) + va[8 * q + 3]);
          w.z = pack_bf16(bf16_lo(f.z) + va[8 * q + 4], bf16_hi(f.z) + va[8 * q + 5]);
          w.w = pack_bf16(bf16_lo(f.w) + va[8 * q + 6], bf16_hi(f.w) + va[8 * q + 7]);
          *reinterpret_cast<uint4*>(dqrow + 16 * c + 8 * q) = w;
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.dq_free);
      if (!parent_end) continue;
      // end of a parent: TMEM lane r = level-1 pooled key r of the parent
      red_cols(a.dpv + ((int64_t) bh * a.n1 + key) * kD, kColPV1, a.kvw1 / a.w1);
      red_cols(a.dpk + ((int64_t) bh * a.n1 + key) * kD, kColPK1, a.kvw1 / a.w1);
      if (i == n_my - 1 || (tile + 1) % tiles_per_head == 0) {
        // level-2 keys: dPK2 of key r - 64 in lanes 64..127 of the first 64 columns, dPV2 of key r in lanes 0..63 of the last 64
        if (qd < 2) red_cols(a.dpv2 + ((int64_t) bh * a.n2 + r) * kD, kColX, a.kvw2 / a.w2);
        else red_cols(a.dpk2 + ((int64_t) bh * a.n2 + (r - 64)) * kD, kColY, a.kvw2 / a.w2);
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.acc_free);
    }
  } else {
    // ---------------------------------------------------------------- softmax / dS; thread = query row
    const int wg = warp >> 2, qd = warp & 3, r = qd * 32 + lane;
    const float sl2 = a.scale * kLog2eF;
    const float lw = log2f(wg < 2 ? a.w1 : a.w2);
    const uint32_t t_row = tmem + ((uint32_t) (qd * 32) << 16);
    // this thread's row in its P tile and its dS tile: start of the row with the swizzle of chunk 0 applied
    const uint32_t myP = tc::smem_u32(sP + wg * kTile + tc::swz(r, 0));
    const uint32_t myDS = tc::smem_u32(sP + (wg == 2 ? 3 : 4 + wg) * kTile + tc::swz(r, 0));
    float lse_n = 0.f, delta_n = 0.f;
    if (n_my > 0) {
      const int bh = t_begin / tiles_per_head, row = (t_begin % tiles_per_head) * kRows + r;
      lse_n = a.lse[(int64_t) bh * a.Nq + row];
      delta_n = a.delta[(int64_t) bh * a.Nq + row];
    }
    bool ok = true;
    for (int i = 0; i < n_my; ++i) {
      const int tile = t_begin + i;
      const float off = lw - lse_n * kLog2eF;
      const float dls = delta_n * a.scale;
      ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.s_ready, i & 1, abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      uint32_t pk[32];          // this row's 64 probabilities, bf16 pairs, kept for dS
      float vh[16];             // 16 columns at a time: the row's registers stay below the point where loop invariants spill
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        tc::tmem_ld16(t_row + wg * 64 + 16 * c, vh);
#pragma unroll
        for (int j = 0; j < 8; ++j) pk[8 * c + j] = pack_bf16(fast_exp2(fmaf(vh[2 * j], sl2, off)), fast_exp2(fmaf(vh[2 * j + 1], sl2, off)));
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.s_consumed);
      if (i > 0) {
        // the previous tile's products read its P / dS tiles: wait for them before overwriting
        ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.out_ready, (i - 1) & 1, abort_flag));
        tc::fence_after_sync();
        if (!ok) break;
      }
      tc::sts128_xor<0>(myP, pk[0], pk[1], pk[2], pk[3]);
      tc::sts128_xor<16>(myP, pk[4], pk[5], pk[6], pk[7]);
      tc::sts128_xor<32>(myP, pk[8], pk[9], pk[10], pk[11]);
      tc::sts128_xor<48>(myP, pk[12], pk[13], pk[14], pk[15]);
      tc::sts128_xor<64>(myP, pk[16], pk[17], pk[18], pk[19]);
      tc::sts128_xor<80>(myP, pk[20], pk[21], pk[22], pk[23]);
      tc::sts128_xor<96>(myP, pk[24], pk[25], pk[26], pk[27]);
      tc::sts128_xor<112>(myP, pk[28], pk[29], pk[30], pk[31]);
      ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.dp_ready, i & 1, abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      if (i + 1 < n_my) {        // next tile's log-sum-exp and delta: in flight during the dS arithmetic
        const int bhn = (tile + 1) / tiles_per_head, rown = ((tile + 1) % tiles_per_head) * kRows + r;
        lse_n = a.lse[(int64_t) bhn * a.Nq + rown];
        delta_n = a.delta[(int64_t) bhn * a.Nq + rown];
      }
      auto ds_chunk = [&](auto tag, int c) {          // dS of columns [16c, 16c+16): two 16-byte chunks of the row
        constexpr int C = decltype(tag)::value;
        uint32_t w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const uint32_t p2 = pk[8 * C + e];
          w[e] = pack_bf16(bf16_lo(p2) * fmaf(vh[2 * e], a.scale, -dls), bf16_hi(p2) * fmaf(vh[2 * e + 1], a.scale, -dls));
        }
        tc::sts128_xor<32 * C>(myDS, w[0], w[1], w[2], w[3]);
        tc::sts128_xor<32 * C + 16>(myDS, w[4], w[5], w[6], w[7]);
      };
      tc::tmem_ld16(t_row + wg * 64, vh);
      ds_chunk(std::integral_constant<int, 0>{}, 0);
      tc::tmem_ld16(t_row + wg * 64 + 16, vh);
      ds_chunk(std::integral_constant<int, 1>{}, 1);
      tc::tmem_ld16(t_row + wg * 64 + 32, vh);
      ds_chunk(std::integral_constant<int, 2>{}, 2);
      tc::tmem_ld16(t_row + wg * 64 + 48, vh);
      ds_chunk(std::integral_constant<int, 3>{}, 3);
      tc::fence_async_smem();          // P, dS must be visible to the tensor core's (async proxy) reads
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.pds_ready);
    }
  }
  if (abort_flag->abort) tc::abort_drain();
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag->abort && a.status) atomicOr(a.status, (int) LLSA_DEV_WAIT_EXPIRED);
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
  const size_t smem = 1024 + (size_t) 14 * kTile * sizeof(bf16);     // Q, dO x 2, K1 x 2, V1, K2 + V2, P x 3, dS x 3
  LLSA_SMEM_LIMIT((attn_bwd_pooled_tc_kernel), smem);
  attn_bwd_pooled_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, n_tiles, tiles_per_head);
  LLSA_LAUNCH_OK("attn_bwd_pooled_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
