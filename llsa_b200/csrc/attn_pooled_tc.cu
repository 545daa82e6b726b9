// Pooled stages of the LLSA forward on the 5th-generation tensor cores: TMA loads,
// tcgen05.mma with accumulators in tensor memory (TMEM), warp-specialised and persistent.
//
// Every query row of a parent block attends to the SAME pooled keys: the children of the
// level-2 blocks its parent selected plus all level-2 keys (two levels), or all level-1
// keys (one level) -- sparse_attention_res_2.py:94-149, sparse_attention_res_1.py:85-106.
// That part of the attention is a dense [128 query rows] x [NP pooled keys] problem per
// tile, the shape tcgen05.mma is made for; the private 16-row fine blocks stay on
// mma.sync (attn_fwd_mma.cu: attn_fwd_fine_kernel) and the two parts are merged here
// through their log-sum-exp.
//
// attn_fwd_pooled_tc_kernel: one persistent CTA per SM walks tiles of 128 query rows.
//   warp 8, one lane : TMA producer.  Per tile: Q [128x64], pooled K [NPx64], pooled V [NPx64]
//                      as 128-byte swizzled tiles into one of three stages (mbarrier expect_tx).
//   warp 9, one lane : MMA issuer.  S = Q.PK^T (M=128, N=NP, K=64, both operands from shared
//                      memory) into TMEM buffer (tile & 1), two tiles ahead of the P.PV product;
//                      O_p = P.PV (M=128, N=64, K=NP) with P read from TENSOR MEMORY (it overwrites
//                      the first NP/2 columns of S as packed bf16 pairs) and PV from shared memory.
//   warps 0-3, 4-7   : two softmax warpgroups, tiles alternate between them so that one group's
//                      TMEM / MMA / global latencies hide behind the other's arithmetic.  Thread r
//                      of a group owns query row r = TMEM lane r: reads its NP scores (tcgen05.ld),
//                      softmax in the exp2 domain with +log2(weight) per key class, writes P back
//                      (tcgen05.st); later reads its O_p row, merges it with the fine part (o, lse
//                      written by the fine kernel for this row, fetched at the top of the tile)
//                      and stores the final o and lse.
// tcgen05.mma operations of one thread execute in issue order, which is what lets S of tile i+2
// reuse the buffer of tile i right behind P.PV of tile i without a barrier.
// All mbarrier waits are bounded; a wait that expires raises a CTA-wide abort flag, every
// role leaves its loop, lse of the unfinished rows is poisoned with NaN and TMEM is freed.
#include <string.h>

#include "attn.cuh"
#include "mma_frag.cuh"
#include "tc05.cuh"
#include "tma.cuh"

namespace llsa {

constexpr int kTcRows = 128;
constexpr int kTcStages = 3;
constexpr int kTcThreads = 352;       // 2 x 4 softmax warps + Q/key producer warp + MMA warp + value producer warp

struct TcMaps {
  CUtensorMap q;      // [B,H,N,64] 4-D, box 128 rows
  CUtensorMap pk1;    // [BH*n1, 64], box 16 rows
  CUtensorMap pv1;
  CUtensorMap pk2;    // [BH*n2, 64], box 64 rows (two levels only)
  CUtensorMap pv2;
};

struct TcBars {
  // a stage's [Q | pooled keys] part and its [pooled values] part fill and drain separately: Q and the keys are free again as soon
  // as S = Q.PK^T has executed, two tiles before the values (free after O = P.PV), so their refill runs that much further ahead
  uint64_t full_k[kTcStages], empty_k[kTcStages], full_v[kTcStages], empty_v[kTcStages], s_ready[2], p_head[2], p_ready[2], o_ready[2];
};

__global__ void __launch_bounds__(kTcThreads, 1)
attn_fwd_pooled_tc_kernel(AttnP<bf16> a, const __grid_constant__ TcMaps maps, int p1_keys, int np, int n_tiles, int tiles_per_head) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ TcBars bars;
  __shared__ uint32_t s_tmem;
  __shared__ tc::WaitCtl s_ctl;
  bf16* base = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const int stage_elems = kTcRows * 64 + 2 * np * 64;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile tc::WaitCtl* abort_flag = &s_ctl;

  if (tid == 0) {
    s_ctl.abort = 0;
    s_ctl.limit = a.wait_limit > 0 ? a.wait_limit : tc::kWaitPolls;
    for (int i = 0; i < kTcStages; ++i) {
      tc::mbar_init(&bars.full_k[i], 1);
      tc::mbar_init(&bars.empty_k[i], 1);
      tc::mbar_init(&bars.full_v[i], 1);
      tc::mbar_init(&bars.empty_v[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars.s_ready[i], 1);
      tc::mbar_init(&bars.o_ready[i], 1);
      tc::mbar_init(&bars.p_ready[i], 4);       // one arrival per softmax warp
      tc::mbar_init(&bars.p_head[i], 4);        // P of all but the last 64 keys is written (np > 64)
    }
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&s_tmem, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int n_my = (n_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x;

  if (warp == 8 || warp == 10) {
    // ---------------------------------------------------------------- TMA producers: warp 8 Q + pooled keys, warp 10 pooled values
    // One lane per copy: lane j < n_p1 fetches its block index and issues the copy of level-1 block j, the next lanes the 64-row
    // level-2 boxes, lane 31 the Q tile.  A single lane doing all of them pays one index round trip per block, back to back
    // (the copies' asm statements order memory accesses), which is longer than the tile period.
    const bool vals = warp == 10;
    const uint32_t bytes = (uint32_t) (vals ? np * 64 : kTcRows * 64 + np * 64) * 2;
    const CUtensorMap* m1 = vals ? &maps.pv1 : &maps.pk1;
    const CUtensorMap* m2 = vals ? &maps.pv2 : &maps.pk2;
    const int n_p1 = p1_keys / kBS, n_p2 = (np - p1_keys) / 64;
    for (int i = 0; i < n_my; ++i) {
      const int tile = blockIdx.x + i * gridDim.x, s = i % kTcStages, u = i / kTcStages;
      const int64_t bh = tile / tiles_per_head, row0 = (int64_t) (tile % tiles_per_head) * kTcRows;
      uint64_t* full = vals ? &bars.full_v[s] : &bars.full_k[s];
      int ok = 1;
      if (lane == 0) {
        ok = tc::bounded_wait(vals ? &bars.empty_v[s] : &bars.empty_k[s], (u & 1) ^ 1, abort_flag) ? 1 : 0;
        if (ok) tma::expect_tx(full, bytes);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      bf16* sQ = base + s * stage_elems;
      bf16* dst = sQ + kTcRows * 64 + (vals ? np * 64 : 0);
      if (lane < n_p1) {
        tma::load_2d(dst + lane * kBS * 64, m1, full, 0, (int) (bh * a.n1 + p1_block(a, bh, row0 / kBS, lane) * kBS));
      } else if (lane < n_p1 + n_p2) {
        const int j = lane - n_p1;
        tma::load_2d(dst + (p1_keys + j * 64) * 64, m2, full, 0, (int) (bh * a.n2 + j * 64));
      } else if (lane == 31 && !vals) {
        tma::load_4d(sQ, &maps.q, full, 0, (int) row0, (int) (bh % a.H), (int) (bh / a.H));
      }
      __syncwarp();
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc::instr_desc(kTcRows, np, 0, 0), idesc_o = tc::instr_desc(kTcRows, 64, 0, 1);
      auto issue_s = [&](int i) -> bool {          // S(i) = Q.PK^T into TMEM buffer i & 1
        const int s = i % kTcStages, u = i / kTcStages, b = i & 1;
        if (!tc::bounded_wait(&bars.full_k[s], u & 1, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t qa = tc::smem_u32(base + s * stage_elems), ka = qa + kTcRows * 128;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          tc::umma_ss(tmem + b * 256, tc::smem_desc(qa + ks * 32, 16, 1024), tc::smem_desc(ka + ks * 32, 16, 1024), idesc_s, ks > 0);
        tc::umma_commit(&bars.s_ready[b]);
        tc::umma_commit(&bars.empty_k[s]);          // Q and the keys of this stage are free once S has executed
        return true;
      };
      bool ok = n_my > 0 && issue_s(0);
      if (ok && n_my > 1) ok = issue_s(1);
      for (int i = 0; ok && i < n_my; ++i) {
        const int s = i % kTcStages, b = i & 1;
        // O = P.PV starts on the keys whose P is already written while the softmax warps finish the last 64
        const int ks_head = np > 64 ? (np - 64) / 16 : 0;
        if (ks_head && !tc::bounded_wait(&bars.p_head[b], (i >> 1) & 1, abort_flag)) break;
        if (!tc::bounded_wait(&bars.full_v[s], (i / kTcStages) & 1, abort_flag)) break;
        tc::fence_after_sync();
        const uint32_t va = tc::smem_u32(base + s * stage_elems) + (kTcRows + np) * 128;
        for (int ks = 0; ks < ks_head; ++ks)       // P: 16 keys = 8 packed columns per k-step; PV: 16 key rows = 2048 bytes
          tc::umma_ts(tmem + b * 256 + np, tmem + b * 256 + ks * 8, tc::smem_desc(va + ks * 2048, 1024, 1024), idesc_o, ks > 0);
        if (!tc::bounded_wait(&bars.p_ready[b], (i >> 1) & 1, abort_flag)) break;
        tc::fence_after_sync();
        for (int ks = ks_head; ks < np / 16; ++ks)
          tc::umma_ts(tmem + b * 256 + np, tmem + b * 256 + ks * 8, tc::smem_desc(va + ks * 2048, 1024, 1024), idesc_o, ks > 0);
        tc::umma_commit(&bars.o_ready[b]);
        tc::umma_commit(&bars.empty_v[s]);
        if (i + 2 < n_my && !issue_s(i + 2)) break;
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue, thread = query row
    const int wg = warp >> 2, r_tile = (warp & 3) * 32 + lane;
    const float sl2 = a.scale * 1.4426950408889634f;
    const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
    const uint32_t t_s = tmem + wg * 256 + ((uint32_t) ((warp & 3) * 32) << 16), t_o = t_s + np;
    for (int i = wg; i < n_my; i += 2) {
      const int tile = blockIdx.x + i * gridDim.x, u = i >> 1;
      const int64_t bh = tile / tiles_per_head, row = (int64_t) (tile % tiles_per_head) * kTcRows + r_tile;
      const int64_t b = bh / a.H, h = bh % a.H;
      // the fine part of this row: requested now, consumed in the epilogue
      bf16* orow = a.o.row(b, h, row);
      uint4 of[8];
#pragma unroll
      for (int q = 0; q < 8; ++q) of[q] = *reinterpret_cast<const uint4*>(orow + 8 * q);
      const float lse_f = a.lse[bh * a.Nq + row];
      // `ok` is kept warp-uniform: the TMEM accesses below are warp-wide instructions
      bool ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.s_ready[wg], u & 1, abort_flag));
      tc::fence_after_sync();
      float mx = 0.f, lsum = 0.f;
      float va[32], vb[32];
      if (ok) {
        float m1 = -INFINITY, m2 = -INFINITY;
        auto chunk_max = [&](const float (&v)[32], int c0) {
          float m = fmaxf(v[0], v[1]);
#pragma unroll
          for (int j = 2; j < 32; j += 2) m = fmax3(m, v[j], v[j + 1]);
          if (c0 < p1_keys) m1 = fmaxf(m1, m); else m2 = fmaxf(m2, m);
        };
        tc::tmem_ld32_async(t_s, va);
        tc::tmem_ld_wait(va);
        for (int c0 = 0; c0 < np; c0 += 64) {        // chunk c0+32 is in flight while chunk c0 is reduced
          tc::tmem_ld32_async(t_s + c0 + 32, vb);
          chunk_max(va, c0);
          tc::tmem_ld_wait(vb);
          if (c0 + 64 < np) tc::tmem_ld32_async(t_s + c0 + 64, va);
          chunk_max(vb, c0 + 32);
          if (c0 + 64 < np) tc::tmem_ld_wait(va);
        }
        mx = fmaxf(fmaf(m1, sl2, lw1), fmaf(m2, sl2, lw2));
        auto chunk_exp = [&](const float (&v)[32], int c0) {
          const float off = (c0 < p1_keys ? lw1 : lw2) - mx;
          uint32_t pk[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float e0 = fast_exp2(fmaf(v[2 * j], sl2, off)), e1 = fast_exp2(fmaf(v[2 * j + 1], sl2, off));
            lsum += e0 + e1;
            pk[j] = pack_bf16(e0, e1);
          }
          tc::tmem_st16(t_s + (c0 >> 1), pk);       // P columns [c0/2, c0/2+16): scores read long before
        };
        tc::tmem_ld32_async(t_s, va);
        tc::tmem_ld_wait(va);
        for (int c0 = 0; c0 < np; c0 += 64) {
          tc::tmem_ld32_async(t_s + c0 + 32, vb);
          chunk_exp(va, c0);
          tc::tmem_ld_wait(vb);
          if (c0 + 64 < np) tc::tmem_ld32_async(t_s + c0 + 64, va);
          chunk_exp(vb, c0 + 32);
          if (c0 + 64 < np) tc::tmem_ld_wait(va);
          if (c0 + 128 == np) {                     // everything but the last 64 keys: the MMA warp may start O = P.PV
            tc::tmem_st_wait();
            tc::fence_before_sync();
            __syncwarp();
            if (lane == 0) tma::mbar_arrive(&bars.p_head[wg]);
          }
        }
        tc::tmem_st_wait();
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(&bars.p_ready[wg]);
        ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.o_ready[wg], u & 1, abort_flag));
        tc::fence_after_sync();
      }
      float lse_out = __int_as_float(0x7fc00000);               // NaN unless everything completed
      if (ok) {
        tc::tmem_ld32_async(t_o, va);
        tc::tmem_ld32_async(t_o + 32, vb);
        const float Lf = lse_f * 1.4426950408889634f;            // fine part, log2 domain
        const float Lp = mx + log2f(lsum);
        const float Lm = fmaxf(Lf, Lp);
        const float ef = fast_exp2(Lf - Lm), ep = fast_exp2(Lp - Lm);
        const float inv = 1.f / (ef + ep);
        const float wf = ef * inv, wp = ep * inv / lsum;
        lse_out = (Lm + log2f(ef + ep)) * 0.6931471805599453f;
        tc::tmem_ld_wait(va);
        tc::tmem_ld_wait(vb);
        auto merge = [&](const float (&v)[32], int c0) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 f = of[(c0 >> 3) + q];
            uint4 w;
            w.x = pack_bf16(bf16_lo(f.x) * wf + v[8 * q] * wp, bf16_hi(f.x) * wf + v[8 * q + 1] * wp);
            w.y = pack_bf16(bf16_lo(f.y) * wf + v[8 * q + 2] * wp, bf16_hi(f.y) * wf + v[8 * q + 3] * wp);
            w.z = pack_bf16(bf16_lo(f.z) * wf + v[8 * q + 4] * wp, bf16_hi(f.z) * wf + v[8 * q + 5] * wp);
            w.w = pack_bf16(bf16_lo(f.w) * wf + v[8 * q + 6] * wp, bf16_hi(f.w) * wf + v[8 * q + 7] * wp);
            *reinterpret_cast<uint4*>(orow + c0 + 8 * q) = w;
          }
        };
        merge(va, 0);
        merge(vb, 32);
      }
      a.lse[bh * a.Nq + row] = lse_out;
      if (!ok) break;
    }
  }
  if (abort_flag->abort) tc::abort_drain();
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag->abort && a.status) atomicOr(a.status, (int) LLSA_DEV_WAIT_EXPIRED);
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
}

// Number of pooled keys per query row if the tcgen05 kernel can take this problem, else 0.
int pooled_tc_keys(const AttnP<bf16>& a) {
  const int p1_keys = a.p1_blocks * kBS, np = (a.p1_blocks + a.p2_blocks) * kBS;
  if (np < 64 || np > 192 || np % 64 || p1_keys % 32 || (np - p1_keys) % 64) return 0;
  if (a.Nq % kTcRows) return 0;
  return np;
}

int launch_attn_fwd_pooled_tc(const LlsaAttnArgs* g, const AttnP<bf16>& a, int64_t BH, cudaStream_t st) {
  const int np = pooled_tc_keys(a), p1_keys = a.p1_blocks * kBS;
  TcMaps maps;
  memset(&maps, 0, sizeof(maps));
  int rc;
  if ((rc = tma::make_map_bhnd(&maps.q, g->q, kTcRows))) return rc;
  if ((rc = tma::make_map_rows(&maps.pk1, a.pk, (uint64_t) BH * a.n1, kBS))) return rc;
  if ((rc = tma::make_map_rows(&maps.pv1, a.pv, (uint64_t) BH * a.n1, kBS))) return rc;
  if (a.two_level) {
    if ((rc = tma::make_map_rows(&maps.pk2, a.pk2, (uint64_t) BH * a.n2, 64))) return rc;
    if ((rc = tma::make_map_rows(&maps.pv2, a.pv2, (uint64_t) BH * a.n2, 64))) return rc;
  }
  const int tiles_per_head = (int) (a.Nq / kTcRows), n_tiles = (int) (BH * tiles_per_head);
  int dev = 0, sms = 148;
  LLSA_CUDA_OK(cudaGetDevice(&dev));
  LLSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = n_tiles < sms ? n_tiles : sms;
  const size_t smem = 1024 + (size_t) kTcStages * (kTcRows * 64 + 2 * np * 64) * sizeof(bf16);
  LLSA_SMEM_LIMIT((attn_fwd_pooled_tc_kernel), smem);
  attn_fwd_pooled_tc_kernel<<<grid, kTcThreads, smem, st>>>(a, maps, p1_keys, np, n_tiles, tiles_per_head);
  LLSA_LAUNCH_OK("attn_fwd_pooled_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
