// Pooled part of dQ on tcgen05 for LONG pooled key lists (llsa_l1 at any N; llsa_l2 with more than 64 level-2
// keys): the query-major half of _attn_bwd_res_dqkv (sparse_attention_res_1.py:225-281,
// sparse_attention_res_2.py:287-415) restricted to the pooled keys, with a key loop over 64-key chunks.
//
// Per tile of 128 query rows and per chunk c of its pooled keys:
//     S  = Q  . K_c^T   [128 x 64]  (K = 64 channels)        shared-memory operands
//     dP = dO . V_c^T   [128 x 64]
//     dS = exp2(S*scale*log2e + log2 w - lse) * (dP - delta) * scale      softmax warps, thread = query row
//     dQ += dS . K_c    [128 x 64]  (K = 64 keys)             dS read from TENSOR MEMORY (packed bf16 over S), K_c MN-major
// The final log-sum-exp is known in the backward, so one pass over the chunks suffices.  dQ accumulates in TMEM over
// all chunks of the tile and is then added to the fine part already in dq.
// TMEM columns: three buffers, chunk number n of the CTA (counted over all its tiles) uses buffer n mod 3: S at 128 b,
// dP at 128 b + 64; dQ at [384, 448).
// Roles (one persistent CTA per SM, 11 warps): warp 8 lane 0 = TMA producer (Q, dO per tile, 2 stages; K and V
// chunks in rings of 8: a stage is refilled four chunks before it is needed), warp 9 lane 0 issues S and dP, warp 10 lane 0 issues dQ, warps 0-3 / 4-7 = two softmax
// warpgroups on alternating chunks; in the epilogue group w handles dQ columns [32 w, 32 w + 32).
// Two issuing threads because one is the pace of the kernel: with the waits, commits and fences around twelve
// instructions per chunk a single thread needed 1,400 cycles per chunk against 576 of tensor-pipe time.  The two run
// independently (S / dP of the next tile start while dQ of this one is still being issued); a buffer goes back to the
// S / dP thread through buf_free, committed behind the dQ instructions that read its dS.
// Every mbarrier wait is bounded (abort flag; the kernel then ends early and frees its TMEM; dq is left partial).
#include <string.h>

#include "attn.cuh"
#include "mma_frag.cuh"
#include "tc05.cuh"
#include "tma.cuh"

namespace llsa {

namespace {

constexpr int kRows = 128;
constexpr int kCk = 64;                      // keys per chunk
constexpr int kTile = kRows * 64;            // elements of a [128 x 64] bf16 tile (16 KB)
constexpr int kChunkElems = kCk * 64;        // elements of a key chunk (8 KB)
constexpr int kStages = 8;
constexpr int kThreads = 352;
constexpr float kLog2eF = 1.4426950408889634f;
constexpr int kBufs = 3;
constexpr uint32_t kColDQ = 384;

struct DqMaps {
  CUtensorMap q, d_o;         // [B,H,Nq,64] 4-D, box 128 rows
  CUtensorMap kg, vg;         // gathered level-1 keys / values (two levels): [BH*n1, 64], box 16 rows
  CUtensorMap kc, vc;         // contiguous pooled keys / values: [BH*n, 64], box 64 rows
};

struct DqBars {
  uint64_t q_full[2], q_empty[2], k_full[kStages], k_empty[kStages], v_full[kStages], v_empty[kStages];
  uint64_t sdp_ready[kBufs], ds_ready[kBufs], buf_free[kBufs], dq_ready, dq_free;
};

// jobs: 64-key chunks per tile (even); gathered: number of leading chunks that are gathered level-1 blocks (0 or 2);
// n_c: rows per head of the contiguous pooled tensor.
__global__ void __launch_bounds__(kThreads, 1)
attn_dq_pooled_loop_tc_kernel(AttnP<bf16> a, const __grid_constant__ DqMaps maps, int jobs, int gathered, int64_t n_c, int n_tiles,
                              int tiles_per_head) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ DqBars bars;
  __shared__ uint32_t s_tmem;
  __shared__ tc::WaitCtl s_ctl;
  bf16* base = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  bf16* sQ = base;                          // [2][128][64]
  bf16* sDO = sQ + 2 * kTile;               // [2][128][64]
  bf16* sK = sDO + 2 * kTile;               // [kStages][64][64]
  bf16* sV = sK + kStages * kChunkElems;    // [kStages][64][64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile tc::WaitCtl* abort_flag = &s_ctl;

  if (tid == 0) {
    s_ctl.abort = 0;
    s_ctl.limit = a.wait_limit > 0 ? a.wait_limit : tc::kWaitPolls;
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars.q_full[i], 1);
      tc::mbar_init(&bars.q_empty[i], 1);
    }
    for (int i = 0; i < kBufs; ++i) {
      tc::mbar_init(&bars.sdp_ready[i], 1);
      tc::mbar_init(&bars.ds_ready[i], 4);        // one arrival per warp of the group
      tc::mbar_init(&bars.buf_free[i], 1);
    }
    for (int i = 0; i < kStages; ++i) {
      tc::mbar_init(&bars.k_full[i], 1); tc::mbar_init(&bars.k_empty[i], 1);
      tc::mbar_init(&bars.v_full[i], 1); tc::mbar_init(&bars.v_empty[i], 1);
    }
    tc::mbar_init(&bars.dq_ready, 1);
    tc::mbar_init(&bars.dq_free, 8);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&s_tmem, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int n_my = (n_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x;

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int cj = 0;                                   // chunks loaded so far
      for (int i = 0; i < n_my; ++i) {
        const int tile = blockIdx.x + i * gridDim.x, qs = i & 1;
        const int bh = tile / tiles_per_head, row0 = (tile % tiles_per_head) * kRows;
        if (!tc::bounded_wait(&bars.q_empty[qs], ((i >> 1) & 1) ^ 1, abort_flag)) break;
        tma::expect_tx(&bars.q_full[qs], 2 * kTile * 2);
        tma::load_4d(sQ + qs * kTile, &maps.q, &bars.q_full[qs], 0, row0, bh % a.H, bh / a.H);
        tma::load_4d(sDO + qs * kTile, &maps.d_o, &bars.q_full[qs], 0, row0, bh % a.H, bh / a.H);
        int krow[8];
        if (gathered) {
#pragma unroll
          for (int j = 0; j < 8; ++j) krow[j] = (int) ((int64_t) bh * a.n1 + p1_block(a, bh, row0 / kBS, j) * kBS);
        }
        bool ok = true;
        for (int j = 0; ok && j < jobs; ++j, ++cj) {
          const int st = cj % kStages;
          const uint32_t par = ((cj / kStages) & 1) ^ 1;
          const int crow = (int) ((int64_t) bh * n_c + (int64_t) (j - gathered) * kCk);
          if (!(ok = tc::bounded_wait(&bars.k_empty[st], par, abort_flag))) break;
          tma::expect_tx(&bars.k_full[st], kChunkElems * 2);
          if (j < gathered) {
#pragma unroll
            for (int b4 = 0; b4 < 4; ++b4)
              tma::load_2d(sK + st * kChunkElems + b4 * kBS * 64, &maps.kg, &bars.k_full[st], 0, j == 0 ? krow[b4] : krow[4 + b4]);
          } else {
            tma::load_2d(sK + st * kChunkElems, &maps.kc, &bars.k_full[st], 0, crow);
          }
          if (!(ok = tc::bounded_wait(&bars.v_empty[st], par, abort_flag))) break;
          tma::expect_tx(&bars.v_full[st], kChunkElems * 2);
          if (j < gathered) {
#pragma unroll
            for (int b4 = 0; b4 < 4; ++b4)
              tma::load_2d(sV + st * kChunkElems + b4 * kBS * 64, &maps.vg, &bars.v_full[st], 0, j == 0 ? krow[b4] : krow[4 + b4]);
          } else {
            tma::load_2d(sV + st * kChunkElems, &maps.vc, &bars.v_full[st], 0, crow);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer 1: S and dP
    if (lane == 0) {
      const uint32_t id_s = tc::instr_desc(kRows, kCk, 0, 0);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      auto lo = [](const void* p, uint32_t lbo_bytes) { return ((tc::smem_u32(p) >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16); };
      constexpr uint32_t kQStage = (uint32_t) (kTile * 2) >> 4, kCStage = (uint32_t) (kChunkElems * 2) >> 4;
      const uint32_t lQ = lo(sQ, 16), lDO = lo(sDO, 16), lK = lo(sK, 16), lV = lo(sV, 16);
      int cj = 0, st = 0, buf = 0;                  // chunks issued so far; ring stage and buffer of the next one
      uint32_t par = 0, bph = 0;                    // phase parities of the ring stage and of the buffer
      bool ok = true;
      for (int i = 0; ok && i < n_my; ++i) {
        const int qs = i & 1;
        if (!(ok = tc::bounded_wait(&bars.q_full[qs], (i >> 1) & 1, abort_flag))) break;
        const uint32_t q_ = lQ + qs * kQStage, o_ = lDO + qs * kQStage;
        for (int j = 0; j < jobs; ++j) {
          // the buffer's previous chunk (three back): its dQ instructions have read dS
          if (cj >= kBufs && !(ok = tc::bounded_wait(&bars.buf_free[buf], bph ^ 1, abort_flag))) break;
          if (!(ok = tc::bounded_wait(&bars.k_full[st], par, abort_flag))) break;
          if (!(ok = tc::bounded_wait(&bars.v_full[st], par, abort_flag))) break;
          tc::fence_after_sync();
          const uint32_t d = tmem + buf * 128;
          const uint32_t k_ = lK + st * kCStage, v_ = lV + st * kCStage;
          tc::umma_ss_lh<0>(d, q_, hi, k_, hi, id_s);
          tc::umma_ss_lh<0>(d + 64, o_, hi, v_, hi, id_s);
#pragma unroll
          for (int s4 = 1; s4 < 4; ++s4) {
            tc::umma_ss_lh<1>(d, q_ + 2 * s4, hi, k_ + 2 * s4, hi, id_s);
            tc::umma_ss_lh<1>(d + 64, o_ + 2 * s4, hi, v_ + 2 * s4, hi, id_s);
          }
          tc::umma_commit(&bars.sdp_ready[buf]);
          tc::umma_commit(&bars.v_empty[st]);        // the values are not needed again
          ++cj;
          if (++st == kStages) { st = 0; par ^= 1; }
          if (++buf == kBufs) { buf = 0; bph ^= 1; }
        }
        if (!ok) break;
        tc::umma_commit(&bars.q_empty[qs]);
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- MMA issuer 2: dQ (+)= dS(chunk, TMEM) . K chunk
    if (lane == 0) {
      const uint32_t id_dq = tc::instr_desc(kRows, 64, 0, 1);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      constexpr uint32_t kCStage = (uint32_t) (kChunkElems * 2) >> 4;
      const uint32_t lKm = ((tc::smem_u32(sK) >> 4) & 0x3FFFu) | ((1024u >> 4) << 16);
      int st = 0, buf = 0;
      uint32_t bph = 0;
      bool ok = true;
      for (int i = 0; ok && i < n_my; ++i) {
        for (int j = 0; j < jobs; ++j) {
          if (!(ok = tc::bounded_wait(&bars.ds_ready[buf], bph, abort_flag))) break;
          if (j == 0 && i > 0 && !(ok = tc::bounded_wait(&bars.dq_free, (i - 1) & 1, abort_flag))) break;     // previous tile's dQ has been read
          tc::fence_after_sync();
          const uint64_t kdesc = ((uint64_t) hi << 32) | (uint64_t) (lKm + st * kCStage);       // 16 key rows = 2048 bytes per k-step
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4)
            tc::umma_ts(tmem + kColDQ, tmem + buf * 128 + s4 * 8, kdesc + 128 * s4, id_dq, (j > 0 || s4 > 0) ? 1u : 0u);
          tc::umma_commit(&bars.k_empty[st]);
          tc::umma_commit(&bars.buf_free[buf]);
          if (++st == kStages) st = 0;
          if (++buf == kBufs) { buf = 0; bph ^= 1; }
        }
        if (!ok) break;
        tc::umma_commit(&bars.dq_ready);
      }
    }
  } else {
    // ---------------------------------------------------------------- dS, then the dq update; thread = query row
    const int wg = warp >> 2, qd = warp & 3, r = qd * 32 + lane;
    const float sl2 = a.scale * kLog2eF;
    const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
    const uint32_t t_lane = tmem + ((uint32_t) (qd * 32) << 16);
    int buf = wg;                          // this group takes every other chunk: buffer and phase parity of its next one
    uint32_t bph = 0;
    const uint32_t t_dq = tmem + kColDQ + wg * 32 + ((uint32_t) (qd * 32) << 16);
    float vs[32], vd[32];
    for (int i = 0; i < n_my; ++i) {
      const int tile = blockIdx.x + i * gridDim.x;
      const int bh = tile / tiles_per_head, row = (tile % tiles_per_head) * kRows + r;
      const float L = a.lse[(int64_t) bh * a.Nq + row] * kLog2eF;
      const float dls = a.delta[(int64_t) bh * a.Nq + row] * a.scale;
      bf16* dqrow = a.dq.row(bh / a.H, bh % a.H, row) + wg * 32;
      uint4 old[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) old[q4] = *reinterpret_cast<const uint4*>(dqrow + 8 * q4);
      bool ok = true;
      for (int j = wg; j < jobs; j += 2) {
        const float off = ((gathered ? (j < gathered) : !a.two_level) ? lw1 : lw2) - L;
        ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.sdp_ready[buf], bph, abort_flag));
        tc::fence_after_sync();
        if (!ok) break;
        const uint32_t t_b = t_lane + buf * 128;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          tc::tmem_ld32_async(t_b + 32 * half, vs);
          tc::tmem_ld32_async(t_b + 64 + 32 * half, vd);
          tc::tmem_ld_wait(vs);
          tc::tmem_ld_wait(vd);
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float p0 = fast_exp2(fmaf(vs[2 * e], sl2, off)), p1 = fast_exp2(fmaf(vs[2 * e + 1], sl2, off));
            pk[e] = pack_bf16(p0 * fmaf(vd[2 * e], a.scale, -dls), p1 * fmaf(vd[2 * e + 1], a.scale, -dls));
          }
          tc::tmem_st16(t_b + 16 * half, pk);          // dS columns [16 half, 16 half + 16) over S columns read before
        }
        tc::tmem_st_wait();
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(&bars.ds_ready[buf]);
        buf += 2;
        if (buf >= kBufs) { buf -= kBufs; bph ^= 1; }
      }
      if (!ok) break;
      ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.dq_ready, (uint32_t) (i & 1), abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      tc::tmem_ld32_async(t_dq, vs);
      tc::tmem_ld_wait(vs);
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        const uint4 f = old[q4];
        uint4 w;
        w.x = pack_bf16(bf16_lo(f.x) + vs[8 * q4], bf16_hi(f.x) + vs[8 * q4 + 1]);
        w.y = pack_bf16(bf16_lo(f.y) + vs[8 * q4 + 2], bf16_hi(f.y) + vs[8 * q4 + 3]);
        w.z = pack_bf16(bf16_lo(f.z) + vs[8 * q4 + 4], bf16_hi(f.z) + vs[8 * q4 + 5]);
        w.w = pack_bf16(bf16_lo(f.w) + vs[8 * q4 + 6], bf16_hi(f.w) + vs[8 * q4 + 7]);
        *reinterpret_cast<uint4*>(dqrow + 8 * q4) = w;
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.dq_free);
    }
  }
  if (abort_flag->abort) tc::abort_drain();
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag->abort && a.status) atomicOr(a.status, (int) LLSA_DEV_WAIT_EXPIRED);
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
}

}  // namespace

// Pooled keys per row if the key-loop dQ kernel applies (a multiple of 128 beyond what the single-shot backward takes).
int pooled_dq_loop_tc_keys(const AttnP<bf16>& a) {
  const int64_t np = (int64_t) (a.p1_blocks + a.p2_blocks) * kBS;
  if (np <= 192 || np % 128 || a.Nq % kRows) return 0;
  if (a.two_level && (a.p1_blocks != 8 || a.p2_blocks == 0)) return 0;
  return (int) np;
}

int launch_attn_dq_pooled_loop_tc(const LlsaAttnArgs* g, const AttnP<bf16>& a, int64_t BH, cudaStream_t st) {
  const int np = pooled_dq_loop_tc_keys(a);
  DqMaps maps;
  memset(&maps, 0, sizeof(maps));
  int rc;
  if ((rc = tma::make_map_bhnd(&maps.q, g->q, kRows))) return rc;
  if ((rc = tma::make_map_bhnd(&maps.d_o, g->d_o, kRows))) return rc;
  const int gathered = a.two_level ? 2 : 0;
  const int64_t n_c = a.two_level ? a.n2 : a.n1;
  if (gathered) {
    if ((rc = tma::make_map_rows(&maps.kg, a.pk, (uint64_t) BH * a.n1, kBS))) return rc;
    if ((rc = tma::make_map_rows(&maps.vg, a.pv, (uint64_t) BH * a.n1, kBS))) return rc;
  }
  if ((rc = tma::make_map_rows(&maps.kc, a.two_level ? a.pk2 : a.pk, (uint64_t) BH * n_c, kCk))) return rc;
  if ((rc = tma::make_map_rows(&maps.vc, a.two_level ? a.pv2 : a.pv, (uint64_t) BH * n_c, kCk))) return rc;
  const int tiles_per_head = (int) (a.Nq / kRows), n_tiles = (int) (BH * tiles_per_head);
  int dev = 0, sms = 148;
  LLSA_CUDA_OK(cudaGetDevice(&dev));
  LLSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = n_tiles < sms ? n_tiles : sms;
  const size_t smem = 1024 + (size_t) (4 * kTile + 2 * kStages * kChunkElems) * sizeof(bf16);
  LLSA_SMEM_LIMIT((attn_dq_pooled_loop_tc_kernel), smem);
  attn_dq_pooled_loop_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, np / kCk, gathered, n_c, n_tiles, tiles_per_head);
  LLSA_LAUNCH_OK("attn_dq_pooled_loop_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
