// Pooled stages of the LLSA forward on tcgen05 for LONG pooled key lists: a key loop over 128-key chunks.
//
// attn_pooled_tc.cu keeps all pooled keys of a tile in tensor memory at once and therefore stops at 192 keys.
// Here a tile of 128 query rows walks its pooled keys chunk by chunk:
//   one level  (sparse_attention_res_1.py:85-106): ALL N/16 level-1 pooled keys, weight token_weight;
//   two levels (sparse_attention_res_2.py:94-149): chunk 0 = the 128 level-1 children of the parent's selected
//              level-2 blocks (gathered, weight token_weight), then ALL N/256 level-2 keys (weight token_weight_2).
// Two passes over the chunks make the softmax exact without rescaling an accumulator that lives in TMEM:
//   pass 1: S = Q.K_c^T per chunk, row maxima only;
//   pass 2: S again, P = exp2(S*scale*log2e + log2 w - max) written back into TMEM over S (packed bf16) and used as
//           the A operand of O += P.V_c; row sums on the side.
// With a `redo` byte per query row from the caller the first pass is dropped: the pooled part only ever meets the fine
// part through their log-sum-exp, so the fine part's log-sum-exp (already known per row) serves as the reference of the
// exponentials, P = exp2(S' - lse_fine).  Anything below 2^-126 of the fine part's weight is irrelevant, and bf16 / fp32
// hold anything up to 2^127 times it; a row whose pooled keys outweigh its fine keys by more than that (its row sum
// passes 1e30, or is NaN) is left untouched and marked in `redo`, and a second launch of the two-pass form redoes
// exactly the marked rows (it scans its tiles' marks first and returns at once when there are none).
// Roles (one persistent CTA per SM, 11 warps):
//   warp 8, one lane : TMA producer: Q per tile (2 stages), K chunks (ring of 4; every chunk is loaded in both
//                      passes), V chunks (ring of 4, pass 2 only)
//   warp 9, one lane : issues S of every "job" (a chunk of a pass).  Job number n, counted over all tiles of the CTA,
//                      uses S buffer n mod 3 (TMEM columns [128 b, 128 b + 128)); O lives in [384,448).
//   warp 10, one lane: issues O += P.V of the pass-2 jobs and hands every job's buffer back to warp 9 (buf_free,
//                      committed behind the instructions that read P).  Two issuing threads because one, with its waits,
//                      commits and fences, was the pace of the kernel: 2,050 cycles per job against 780 of pipe time.
//   warps 0-3 / 4-7  : two softmax warpgroups, group w owns the jobs n = w (mod 2); thread r owns query row r
//                      (TMEM lane r).  Row maxima and row sums of the two groups meet in shared memory (an
//                      mbarrier with one arrival per softmax warp, so that this wait is bounded too).  Epilogue: group w merges O columns [32w, 32w+32)
//                      with the fine part (o, lse written by the fine kernel) and stores them.
// Every mbarrier wait is bounded; a wait that expires raises a CTA-wide abort flag, every role leaves its loops,
// lse of the unfinished rows is poisoned with NaN and TMEM is freed.
#include <string.h>

#include "attn.cuh"
#include "mma_frag.cuh"
#include "tc05.cuh"
#include "tma.cuh"

namespace llsa {

namespace {

constexpr int kRows = 128;
constexpr int kChunk = 128;                 // keys per chunk
constexpr int kTile = kRows * 64;           // elements of a [128 x 64] bf16 tile (16 KB)
constexpr int kKStages = 4, kVStages = 4;
constexpr int kThreads = 352;
constexpr int kBufs = 3;
constexpr float kLog2eF = 1.4426950408889634f;
constexpr uint32_t kColO = 384;

struct LoopMaps {
  CUtensorMap q;              // [B,H,Nq,64] 4-D, box 128 rows
  CUtensorMap kg, vg;         // gathered level-1 keys / values (two levels): [BH*n1, 64], box 16 rows
  CUtensorMap kc, vc;         // contiguous pooled keys / values: [BH*n, 64], box 128 rows
};

struct LoopBars {
  uint64_t q_full[2], q_empty[2], k_full[kKStages], k_empty[kKStages], v_full[kVStages], v_empty[kVStages];
  uint64_t s_ready[kBufs], wg_done[kBufs], buf_free[kBufs], o_ready, o_free, xchg;
};

// n_chunks: chunks per tile; gathered: chunk 0 is the gathered level-1 set (two levels); n_c: rows per head of the
// contiguous pooled tensor.
__global__ void __launch_bounds__(kThreads, 1)
attn_fwd_pooled_loop_tc_kernel(AttnP<bf16> a, const __grid_constant__ LoopMaps maps, int n_chunks, int gathered, int64_t n_c, int n_tiles,
                               int tiles_per_head, int n_pass, unsigned char* redo) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ LoopBars bars;
  __shared__ uint32_t s_tmem;
  __shared__ tc::WaitCtl s_ctl;
  __shared__ float s_part[2][2][kRows];     // [exchange parity][group][row]: row maxima, then row sums
  bf16* base = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  bf16* sQ = base;                          // [2][128][64]
  bf16* sK = sQ + 2 * kTile;                // [kKStages][128][64]
  bf16* sV = sK + kKStages * kTile;         // [kVStages][128][64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile tc::WaitCtl* abort_flag = &s_ctl;
  const int n_my = (n_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x;
  if (n_pass == 2 && redo) {
    // the second launch: anything to redo in this CTA's tiles?  (a tile's 128 marks are 32 words)
    int any = 0;
    if (warp == 0)
      for (int i = 0; i < n_my; ++i) any |= (int) reinterpret_cast<const uint32_t*>(redo)[(int64_t) (blockIdx.x + i * gridDim.x) * (kRows / 4) + lane];
    if (!__syncthreads_or(any)) return;
  }

  if (tid == 0) {
    s_ctl.abort = 0;
    s_ctl.limit = a.wait_limit > 0 ? a.wait_limit : tc::kWaitPolls;
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars.q_full[i], 1);
      tc::mbar_init(&bars.q_empty[i], 1);
    }
    for (int i = 0; i < kBufs; ++i) {
      tc::mbar_init(&bars.s_ready[i], 1);
      tc::mbar_init(&bars.wg_done[i], 4);         // one arrival per warp of the group
      tc::mbar_init(&bars.buf_free[i], 1);
    }
    for (int i = 0; i < kKStages; ++i) { tc::mbar_init(&bars.k_full[i], 1); tc::mbar_init(&bars.k_empty[i], 1); }
    for (int i = 0; i < kVStages; ++i) { tc::mbar_init(&bars.v_full[i], 1); tc::mbar_init(&bars.v_empty[i], 1); }
    tc::mbar_init(&bars.o_ready, 1);
    tc::mbar_init(&bars.o_free, 8);
    tc::mbar_init(&bars.xchg, 8);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&s_tmem, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem;
  // jobs per tile; job j of tile i has the CTA-wide number i * jobs + j, which picks the S buffer (mod 3) and the softmax
  // group (mod 2; with one pass and an odd chunk count the parity of a tile's first job alternates)
  const int jobs = n_pass * n_chunks, first_p2 = jobs - n_chunks;

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int kjob = 0, vjob = 0;
      for (int i = 0; i < n_my; ++i) {
        const int tile = blockIdx.x + i * gridDim.x, qs = i & 1;
        const int bh = tile / tiles_per_head, row0 = (tile % tiles_per_head) * kRows;
        if (!tc::bounded_wait(&bars.q_empty[qs], ((i >> 1) & 1) ^ 1, abort_flag)) break;
        tma::expect_tx(&bars.q_full[qs], kTile * 2);
        tma::load_4d(sQ + qs * kTile, &maps.q, &bars.q_full[qs], 0, row0, bh % a.H, bh / a.H);
        int krow[8];
        if (gathered) {
#pragma unroll
          for (int j = 0; j < 8; ++j) krow[j] = (int) ((int64_t) bh * a.n1 + p1_block(a, bh, row0 / kBS, j) * kBS);
        }
        bool ok = true;
        for (int j = 0; ok && j < jobs; ++j) {
          const int c = j % n_chunks, pass = j >= first_p2;
          const int crow = (int) ((int64_t) bh * n_c + (int64_t) (c - gathered) * kChunk);      // contiguous chunk
          const int ks = kjob % kKStages;
          if (!(ok = tc::bounded_wait(&bars.k_empty[ks], ((kjob / kKStages) & 1) ^ 1, abort_flag))) break;
          tma::expect_tx(&bars.k_full[ks], kTile * 2);
          if (gathered && c == 0) {
#pragma unroll
            for (int b8 = 0; b8 < 8; ++b8) tma::load_2d(sK + ks * kTile + b8 * kBS * 64, &maps.kg, &bars.k_full[ks], 0, krow[b8]);
          } else {
            tma::load_2d(sK + ks * kTile, &maps.kc, &bars.k_full[ks], 0, crow);
          }
          ++kjob;
          if (pass == 1) {
            const int vs = vjob % kVStages;
            if (!(ok = tc::bounded_wait(&bars.v_empty[vs], ((vjob / kVStages) & 1) ^ 1, abort_flag))) break;
            tma::expect_tx(&bars.v_full[vs], kTile * 2);
            if (gathered && c == 0) {
#pragma unroll
              for (int b8 = 0; b8 < 8; ++b8) tma::load_2d(sV + vs * kTile + b8 * kBS * 64, &maps.vg, &bars.v_full[vs], 0, krow[b8]);
            } else {
              tma::load_2d(sV + vs * kTile, &maps.vc, &bars.v_full[vs], 0, crow);
            }
            ++vjob;
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer 1: S of every job
    if (lane == 0) {
      const uint32_t id_s = tc::instr_desc(kRows, kChunk, 0, 0);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      auto lo = [](const void* p, uint32_t lbo_bytes) { return ((tc::smem_u32(p) >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16); };
      constexpr uint32_t kStage = (uint32_t) (kTile * 2) >> 4;
      const uint32_t lQ = lo(sQ, 16), lK = lo(sK, 16);
      int n = 0, ks = 0, buf = 0;                   // jobs issued so far; K ring stage and S buffer of the next one
      uint32_t kph = 0, bph = 0;                    // their phase parities
      bool ok = true;
      for (int i = 0; ok && i < n_my; ++i) {
        const int qs = i & 1;
        if (!(ok = tc::bounded_wait(&bars.q_full[qs], (i >> 1) & 1, abort_flag))) break;
        const uint32_t q_ = lQ + qs * kStage;
        for (int j = 0; j < jobs; ++j, ++n) {
          // the buffer's previous job (three back): its group has read S and, in pass 2, P.V has read P
          if (n >= kBufs && !(ok = tc::bounded_wait(&bars.buf_free[buf], bph ^ 1, abort_flag))) break;
          if (!(ok = tc::bounded_wait(&bars.k_full[ks], kph, abort_flag))) break;
          tc::fence_after_sync();
          const uint32_t k_ = lK + ks * kStage, d = tmem + buf * kChunk;
          tc::umma_ss_lh<0>(d, q_, hi, k_, hi, id_s);
#pragma unroll
          for (int s4 = 1; s4 < 4; ++s4) tc::umma_ss_lh<1>(d, q_ + 2 * s4, hi, k_ + 2 * s4, hi, id_s);
          tc::umma_commit(&bars.s_ready[buf]);
          tc::umma_commit(&bars.k_empty[ks]);
          if (++ks == kKStages) { ks = 0; kph ^= 1; }
          if (++buf == kBufs) { buf = 0; bph ^= 1; }
        }
        if (!ok) break;
        tc::umma_commit(&bars.q_empty[qs]);
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- MMA issuer 2: O (+)= P(job, TMEM) . V chunk
    if (lane == 0) {
      const uint32_t id_o = tc::instr_desc(kRows, 64, 0, 1);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      constexpr uint32_t kStage = (uint32_t) (kTile * 2) >> 4;
      const uint32_t lV = ((tc::smem_u32(sV) >> 4) & 0x3FFFu) | ((1024u >> 4) << 16);
      int vs = 0, buf = 0;
      uint32_t vph = 0, bph = 0;
      bool ok = true;
      for (int i = 0; ok && i < n_my; ++i) {
        for (int j = 0; j < jobs; ++j) {
          if (!(ok = tc::bounded_wait(&bars.wg_done[buf], bph, abort_flag))) break;
          if (j >= first_p2) {
            const int c = j - first_p2;
            if (!(ok = tc::bounded_wait(&bars.v_full[vs], vph, abort_flag))) break;
            if (c == 0 && i > 0 && !(ok = tc::bounded_wait(&bars.o_free, (i - 1) & 1, abort_flag))) break;      // previous tile's O has been read
            tc::fence_after_sync();
            const uint64_t vdesc = ((uint64_t) hi << 32) | (uint64_t) (lV + vs * kStage);
#pragma unroll
            for (int s8 = 0; s8 < 8; ++s8)       // P: 16 keys = 8 packed columns per k-step; V: 16 key rows = 2048 bytes
              tc::umma_ts(tmem + kColO, tmem + buf * kChunk + s8 * 8, vdesc + 128 * s8, id_o, (c > 0 || s8 > 0) ? 1u : 0u);
            tc::umma_commit(&bars.v_empty[vs]);
            if (++vs == kVStages) { vs = 0; vph ^= 1; }
          }
          tc::umma_commit(&bars.buf_free[buf]);
          if (++buf == kBufs) { buf = 0; bph ^= 1; }
        }
        if (!ok) break;
        tc::umma_commit(&bars.o_ready);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue, thread = query row
    const int wg = warp >> 2, qd = warp & 3, r = qd * 32 + lane;
    const float sl2 = a.scale * kLog2eF;
    const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
    const uint32_t t_lane = tmem + ((uint32_t) (qd * 32) << 16);
    const uint32_t t_o = t_lane + kColO + wg * 32;
    int buf = wg;                          // S buffer of this group's next job (it takes every other job of the CTA) and
    uint32_t bph = 0;                      // the phase parity of that buffer's barriers
    uint32_t n_x = 0;                      // exchanges so far
    float va[32];
    // Both groups publish a per-row value and read the other group's.  The buffer alternates with the exchange count:
    // a buffer is rewritten two exchanges later, after every thread has passed the barrier in between.
    auto exchange = [&](float mine, float& other) -> bool {
      s_part[n_x & 1][wg][r] = mine;
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.xchg);
      const bool ok_ = __all_sync(0xffffffffu, tc::bounded_wait(&bars.xchg, n_x & 1, abort_flag));
      other = s_part[n_x & 1][wg ^ 1][r];
      ++n_x;
      return ok_;
    };
    for (int i = 0; i < n_my; ++i) {
      const int tile = blockIdx.x + i * gridDim.x;
      const int bh = tile / tiles_per_head, row = (tile % tiles_per_head) * kRows + r;
      bf16* orow = a.o.row(bh / a.H, bh % a.H, row) + wg * 32;
      // the fine part of this row (this group's 32 channels): requested now, consumed in the epilogue
      uint4 of[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) of[q4] = *reinterpret_cast<const uint4*>(orow + 8 * q4);
      const float lse_f = a.lse[(int64_t) bh * a.Nq + row];
      // one pass: the fine part's log-sum-exp is the reference of the exponentials
      float mx = n_pass == 1 ? lse_f * kLog2eF : -INFINITY, lsum = 0.f;
      bool ok = true;
      for (int j = (int) ((wg - (int64_t) i * jobs) & 1); j < jobs; j += 2) {
        const int c = j % n_chunks, pass = j >= first_p2;
        const float lw = (gathered ? (c == 0) : !a.two_level) ? lw1 : lw2;
        if (n_pass == 2 && pass == 1 && j - 2 < first_p2) {
          // first pass-2 job of this group: exchange the row maxima of the two groups
          float other;
          if (!(ok = exchange(mx, other))) break;
          mx = fmaxf(mx, other);
        }
        ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.s_ready[buf], bph, abort_flag));
        tc::fence_after_sync();
        if (!ok) break;
        const uint32_t t_s = t_lane + buf * kChunk;
        if (pass == 0) {
          float m = -INFINITY;
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            tc::tmem_ld32_async(t_s + 32 * q4, va);
            tc::tmem_ld_wait(va);
#pragma unroll
            for (int e = 0; e < 32; e += 2) m = fmax3(m, va[e], va[e + 1]);
          }
          mx = fmaxf(mx, fmaf(m, sl2, lw));
        } else {
          const float off = lw - mx;
#pragma unroll 1          // unrolled, the four quarters' registers overlap and 18 of them spill (to L2: L1 is 28 KB here)
          for (int q4 = 0; q4 < 4; ++q4) {
            tc::tmem_ld32_async(t_s + 32 * q4, va);
            tc::tmem_ld_wait(va);
            uint32_t pk[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float e0 = fast_exp2(fmaf(va[2 * e], sl2, off)), e1 = fast_exp2(fmaf(va[2 * e + 1], sl2, off));
              lsum += e0 + e1;
              pk[e] = pack_bf16(e0, e1);
            }
            tc::tmem_st16(t_s + 16 * q4, pk);          // P columns [16 q4, 16 q4 + 16): scores read before
          }
          tc::tmem_st_wait();
        }
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(&bars.wg_done[buf]);
        buf += 2;
        if (buf >= kBufs) { buf -= kBufs; bph ^= 1; }
      }
      float lse_out = __int_as_float(0x7fc00000);               // NaN unless everything completed
      if (ok) {
        float other;
        ok = exchange(lsum, other);
        lsum = wg == 0 ? lsum + other : other + lsum;          // the same order in both groups: identical bits
      }
      // does this launch own the row?  One pass: unless its sum left the safe range (then the mark hands it to the
      // second launch).  Second launch: only the marked rows.
      bool mine = true;
      if (redo) {
        if (n_pass == 1) {
          mine = lsum < 1e30f;                                  // false for NaN too
          if (wg == 0 && ok) redo[(int64_t) bh * a.Nq + row] = mine ? 0 : 1;
        } else {
          mine = redo[(int64_t) bh * a.Nq + row] != 0;
        }
      }
      if (ok) {
        ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.o_ready, (uint32_t) (i & 1), abort_flag));
        tc::fence_after_sync();
      }
      if (ok) {
        tc::tmem_ld32_async(t_o, va);
        const float Lf = lse_f * kLog2eF;                        // fine part, log2 domain
        const float Lp = mx + log2f(lsum);
        const float Lm = fmaxf(Lf, Lp);
        const float ef = fast_exp2(Lf - Lm), ep = fast_exp2(Lp - Lm);
        const float inv = 1.f / (ef + ep);
        const float wf = ef * inv, wp = lsum > 0.f ? ep * inv / lsum : 0.f;      // every exponential may have underflowed
        lse_out = (Lm + log2f(ef + ep)) * 0.6931471805599453f;
        tc::tmem_ld_wait(va);
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {
          const uint4 f = of[q4];
          uint4 w;
          w.x = pack_bf16(bf16_lo(f.x) * wf + va[8 * q4] * wp, bf16_hi(f.x) * wf + va[8 * q4 + 1] * wp);
          w.y = pack_bf16(bf16_lo(f.y) * wf + va[8 * q4 + 2] * wp, bf16_hi(f.y) * wf + va[8 * q4 + 3] * wp);
          w.z = pack_bf16(bf16_lo(f.z) * wf + va[8 * q4 + 4] * wp, bf16_hi(f.z) * wf + va[8 * q4 + 5] * wp);
          w.w = pack_bf16(bf16_lo(f.w) * wf + va[8 * q4 + 6] * wp, bf16_hi(f.w) * wf + va[8 * q4 + 7] * wp);
          if (mine) *reinterpret_cast<uint4*>(orow + 8 * q4) = w;
        }
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(&bars.o_free);
      }
      // both groups read the fine lse above; group 0 replaces it only after both have (second exchange barrier)
      if (wg == 0 && mine) a.lse[(int64_t) bh * a.Nq + row] = lse_out;
      if (!ok) break;
    }
  }
  if (abort_flag->abort) tc::abort_drain();
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag->abort && a.status) atomicOr(a.status, (int) LLSA_DEV_WAIT_EXPIRED);
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
}

}  // namespace

// Pooled keys per row if the key-loop kernel applies (a multiple of 128, more than the 192 the single-shot kernel
// holds), else 0.
int pooled_loop_tc_keys(const AttnP<bf16>& a) {
  const int64_t np = (int64_t) (a.p1_blocks + a.p2_blocks) * kBS;
  if (np <= 192 || np % kChunk || a.Nq % kRows) return 0;
  if (a.two_level && a.p1_blocks != 8) return 0;         // the gathered chunk is exactly 8 blocks
  if (a.two_level && a.p2_blocks == 0) return 0;
  return (int) np;
}

int launch_attn_fwd_pooled_loop_tc(const LlsaAttnArgs* g, const AttnP<bf16>& a, int64_t BH, cudaStream_t st) {
  const int np = pooled_loop_tc_keys(a);
  LoopMaps maps;
  memset(&maps, 0, sizeof(maps));
  int rc;
  if ((rc = tma::make_map_bhnd(&maps.q, g->q, kRows))) return rc;
  const int gathered = a.two_level ? 1 : 0;
  const int64_t n_c = a.two_level ? a.n2 : a.n1;
  if (gathered) {
    if ((rc = tma::make_map_rows(&maps.kg, a.pk, (uint64_t) BH * a.n1, kBS))) return rc;
    if ((rc = tma::make_map_rows(&maps.vg, a.pv, (uint64_t) BH * a.n1, kBS))) return rc;
  }
  if ((rc = tma::make_map_rows(&maps.kc, a.two_level ? a.pk2 : a.pk, (uint64_t) BH * n_c, kChunk))) return rc;
  if ((rc = tma::make_map_rows(&maps.vc, a.two_level ? a.pv2 : a.pv, (uint64_t) BH * n_c, kChunk))) return rc;
  const int tiles_per_head = (int) (a.Nq / kRows), n_tiles = (int) (BH * tiles_per_head);
  int dev = 0, sms = 148;
  LLSA_CUDA_OK(cudaGetDevice(&dev));
  LLSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int grid = n_tiles < sms ? n_tiles : sms;
  const size_t smem = 1024 + (size_t) (2 + kKStages + kVStages) * kTile * sizeof(bf16);
  LLSA_SMEM_LIMIT((attn_fwd_pooled_loop_tc_kernel), smem);
  unsigned char* redo = g->fwd_redo ? reinterpret_cast<unsigned char*>(g->fwd_redo->ptr) : nullptr;
  if (redo) {        // one pass with the fine part's log-sum-exp as reference, then the two-pass form for the rows it marked
    attn_fwd_pooled_loop_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, np / kChunk, gathered, n_c, n_tiles, tiles_per_head, 1, redo);
    LLSA_LAUNCH_OK("attn_fwd_pooled_loop_tc_kernel");
  }
  attn_fwd_pooled_loop_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, np / kChunk, gathered, n_c, n_tiles, tiles_per_head, 2, redo);
  LLSA_LAUNCH_OK("attn_fwd_pooled_loop_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
