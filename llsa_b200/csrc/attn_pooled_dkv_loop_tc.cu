// Pooled-key gradients on tcgen05 for the keys that EVERY query attends to: all level-1 pooled keys of the
// one-level form (sparse_attention_res_1.py:362-400) and all level-2 keys of the two-level form
// (_attn_bwd_res_dpkv2, sparse_attention_res_2.py:418-489) -- the key-major half of the pooled backward, with a
// loop over the queries.
//
// A work unit is (head, chunk of 128 pooled keys) and a range of the head's query rows, walked 64 at a time (a job):
//     S^T  = K_c . Q_t^T   [128 keys x 64 queries]  (K = 64 channels)   shared-memory operands
//     dP^T = V_c . dO_t^T  [128 x 64]
//     P^T  = exp2(S^T*scale*log2e + log2 w - lse[q]),  dS^T = P^T * (dP^T - delta[q]) * scale     thread = key row;
//            lse and delta of the 64 query columns sit in shared memory next to the Q / dO tile
//     dV_c += P^T  . dO_t  [128 x 64]  (K = 64 queries)   P^T, dS^T read from TENSOR MEMORY (packed bf16, written over
//     dK_c += dS^T . Q_t                                   S^T / dP^T), dO_t / Q_t as MN-major operands (the same tiles)
// dK_c, dV_c accumulate in TMEM over the unit's query range and are then written to the fp32 pooled-gradient
// accumulators (scaled by kv_weight / token_weight, the reference's weighting of the pooled dK/dV side): plain stores if
// the unit covers all queries of its head, reductions otherwise.
// Work split: all (head, chunk, job) triples in that order form one flat list that is cut into gridDim.x equal pieces,
// one per CTA; a piece is one to a few units (it changes unit where it crosses a chunk boundary).
// TMEM columns: three buffers, job number n of the CTA uses buffer n mod 3: S^T at 128 b, dP^T at 128 b + 64; dV at
// [384,448), dK at [448,512).
// Roles (one persistent CTA per SM, 11 warps): warp 8 lane 0 = TMA producer (K_c, V_c per unit; Q_t, dO_t, lse, delta per
// job in a ring of 8), warp 9 lane 0 issues S^T and dP^T, warp 10 lane 0 issues dV and dK (one issuing thread, with its
// waits, commits and fences, is slower than the tensor pipe), warps 0-3 / 4-7 = two softmax warpgroups on alternating
// jobs; at the end of a unit group 0 writes dV, group 1 writes dK.  Every mbarrier wait is bounded (abort flag, TMEM freed).
#include <string.h>

#include "attn.cuh"
#include "mma_frag.cuh"
#include "tc05.cuh"
#include "tma.cuh"

namespace llsa {

namespace {

constexpr int kKeys = 128;                   // keys per unit (MMA M)
constexpr int kQ = 64;                       // query rows per job (MMA N)
constexpr int kKeyTile = kKeys * 64;         // elements of the K / V chunk (16 KB)
constexpr int kQTile = kQ * 64;              // elements of a Q / dO job tile (8 KB)
constexpr int kStages = 8;
constexpr int kThreads = 352;
constexpr int kBufs = 3;
constexpr float kLog2eF = 1.4426950408889634f;
constexpr uint32_t kColDV = 384, kColDK = 448;

struct KvMaps {
  CUtensorMap q, d_o;         // [B,H,Nq,64] 4-D, box 64 rows
  CUtensorMap k, v;           // contiguous pooled keys / values [BH*n, 64], box 128 rows
};

struct KvBars {
  uint64_t kv_full, kv_empty, q_full[kStages], q_empty[kStages], sdp_ready[kBufs], pds_ready[kBufs], buf_free[kBufs], acc_ready, acc_free;
};

// A CTA's piece of the flat job list, walked unit by unit.
struct Piece {
  int64_t f, f_end;           // next flat job, end of the piece
  int jobs_all;               // jobs per (head, chunk): query rows / 64
  int unit, job0, n;          // current unit: (head, chunk) number, first job, job count
  __device__ Piece(int64_t total, int jobs_all_) : jobs_all(jobs_all_), unit(0), job0(0), n(0) {
    f = total * blockIdx.x / gridDim.x;
    f_end = total * (blockIdx.x + 1) / gridDim.x;
  }
  __device__ bool next() {
    f += n;
    if (f >= f_end) return false;
    unit = (int) (f / jobs_all);
    job0 = (int) (f - (int64_t) unit * jobs_all);
    const int64_t left = f_end - f;
    n = left < jobs_all - job0 ? (int) left : jobs_all - job0;
    return true;
  }
};

// n_keys: pooled keys per head (a multiple of 128); jobs_all: 64-row query jobs per head; n_base: heads x key chunks.
__global__ void __launch_bounds__(kThreads, 1)
attn_dkv_pooled_loop_tc_kernel(AttnP<bf16> a, const __grid_constant__ KvMaps maps, float* __restrict__ dpk, float* __restrict__ dpv,
                               int64_t n_keys, int jobs_all, int n_base, float lw_log2, float out_mul) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ KvBars bars;
  __shared__ uint32_t s_tmem;
  __shared__ tc::WaitCtl s_ctl;
  __shared__ __align__(16) float s_lse[kStages][kQ], s_delta[kStages][kQ];
  bf16* base = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  bf16* sK = base;                           // [128][64]
  bf16* sV = sK + kKeyTile;                  // [128][64]
  bf16* sQ = sV + kKeyTile;                  // [kStages][64][64]
  bf16* sDO = sQ + kStages * kQTile;         // [kStages][64][64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile tc::WaitCtl* abort_flag = &s_ctl;

  if (tid == 0) {
    s_ctl.abort = 0;
    s_ctl.limit = a.wait_limit > 0 ? a.wait_limit : tc::kWaitPolls;
    tc::mbar_init(&bars.kv_full, 1);
    tc::mbar_init(&bars.kv_empty, 1);
    for (int i = 0; i < kStages; ++i) { tc::mbar_init(&bars.q_full[i], 1); tc::mbar_init(&bars.q_empty[i], 1); }
    for (int i = 0; i < kBufs; ++i) {
      tc::mbar_init(&bars.sdp_ready[i], 1);
      tc::mbar_init(&bars.pds_ready[i], 4);
      tc::mbar_init(&bars.buf_free[i], 1);
    }
    tc::mbar_init(&bars.acc_ready, 1);
    tc::mbar_init(&bars.acc_free, 8);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&s_tmem, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int chunks_per_head = (int) (n_keys / kKeys);
  Piece pc((int64_t) n_base * jobs_all, jobs_all);

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int cj = 0;
      bool ok = true;
      for (int i = 0; ok && pc.next(); ++i) {
        const int bh = pc.unit / chunks_per_head, c = pc.unit % chunks_per_head;
        if (!tc::bounded_wait(&bars.kv_empty, (i & 1) ^ 1, abort_flag)) break;
        tma::expect_tx(&bars.kv_full, 2 * kKeyTile * 2);
        tma::load_2d(sK, &maps.k, &bars.kv_full, 0, (int) ((int64_t) bh * n_keys + (int64_t) c * kKeys));
        tma::load_2d(sV, &maps.v, &bars.kv_full, 0, (int) ((int64_t) bh * n_keys + (int64_t) c * kKeys));
        for (int j = 0; j < pc.n; ++j, ++cj) {
          const int st = cj & (kStages - 1);
          if (!(ok = tc::bounded_wait(&bars.q_empty[st], ((cj / kStages) & 1) ^ 1, abort_flag))) break;
          tma::expect_tx(&bars.q_full[st], 2 * kQTile * 2 + 2 * kQ * 4);
          const int qrow = (pc.job0 + j) * kQ;
          tma::load_4d(sQ + st * kQTile, &maps.q, &bars.q_full[st], 0, qrow, bh % a.H, bh / a.H);
          tma::load_4d(sDO + st * kQTile, &maps.d_o, &bars.q_full[st], 0, qrow, bh % a.H, bh / a.H);
          tma::load_bulk(s_lse[st], a.lse + (int64_t) bh * a.Nq + qrow, kQ * 4, &bars.q_full[st]);
          tma::load_bulk(s_delta[st], a.delta + (int64_t) bh * a.Nq + qrow, kQ * 4, &bars.q_full[st]);
        }
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer 1: S^T and dP^T of every job
    if (lane == 0) {
      const uint32_t id_s = tc::instr_desc(kKeys, kQ, 0, 0);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      auto lo = [](const void* p, uint32_t lbo_bytes) { return ((tc::smem_u32(p) >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16); };
      constexpr uint32_t kQStage = (uint32_t) (kQTile * 2) >> 4;
      const uint32_t lK = lo(sK, 16), lV = lo(sV, 16), lQ = lo(sQ, 16), lDO = lo(sDO, 16);
      int cj = 0, buf = 0;                          // jobs issued so far by this CTA; buffer of the next one
      uint32_t bph = 0;                             // phase parity of that buffer's barriers
      bool ok = true;
      for (int i = 0; ok && pc.next(); ++i) {
        if (!(ok = tc::bounded_wait(&bars.kv_full, i & 1, abort_flag))) break;
        for (int j = 0; j < pc.n; ++j, ++cj) {
          const int st = cj & (kStages - 1);
          // the buffer's previous job (three back): the dV / dK instructions that read its P^T / dS^T have completed
          if (cj >= kBufs && !(ok = tc::bounded_wait(&bars.buf_free[buf], bph ^ 1, abort_flag))) break;
          if (!(ok = tc::bounded_wait(&bars.q_full[st], (cj / kStages) & 1, abort_flag))) break;
          tc::fence_after_sync();
          const uint32_t d = tmem + buf * 128, q_ = lQ + st * kQStage, o_ = lDO + st * kQStage;
          tc::umma_ss_lh<0>(d, lK, hi, q_, hi, id_s);
          tc::umma_ss_lh<0>(d + 64, lV, hi, o_, hi, id_s);
#pragma unroll
          for (int s4 = 1; s4 < 4; ++s4) {
            tc::umma_ss_lh<1>(d, lK + 2 * s4, hi, q_ + 2 * s4, hi, id_s);
            tc::umma_ss_lh<1>(d + 64, lV + 2 * s4, hi, o_ + 2 * s4, hi, id_s);
          }
          tc::umma_commit(&bars.sdp_ready[buf]);
          if (++buf == kBufs) { buf = 0; bph ^= 1; }
        }
        if (!ok) break;
        tc::umma_commit(&bars.kv_empty);             // the key chunk is only read by these products
      }
    }
  } else if (warp == 10) {
    // ---------------------------------------------------------------- MMA issuer 2: dV (+)= P^T . dO_t, dK (+)= dS^T . Q_t
    if (lane == 0) {
      const uint32_t id_o = tc::instr_desc(kKeys, 64, 0, 1);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      auto lo = [](const void* p, uint32_t lbo_bytes) { return ((tc::smem_u32(p) >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16); };
      constexpr uint32_t kQStage = (uint32_t) (kQTile * 2) >> 4;
      const uint32_t lQm = lo(sQ, 1024), lDOm = lo(sDO, 1024);
      int cj = 0, buf = 0;
      uint32_t bph = 0;
      bool ok = true;
      for (int i = 0; ok && pc.next(); ++i) {
        for (int j = 0; j < pc.n; ++j, ++cj) {
          const int st = cj & (kStages - 1);
          if (!(ok = tc::bounded_wait(&bars.pds_ready[buf], bph, abort_flag))) break;
          if (j == 0 && i > 0 && !(ok = tc::bounded_wait(&bars.acc_free, (i - 1) & 1, abort_flag))) break;    // previous unit's results have been read
          tc::fence_after_sync();
          // 4 k-steps of 16 query rows (2048 bytes of the MN-major dO / Q tile)
          const uint64_t dodesc = ((uint64_t) hi << 32) | (uint64_t) (lDOm + st * kQStage), qdesc = ((uint64_t) hi << 32) | (uint64_t) (lQm + st * kQStage);
          const uint32_t b = tmem + buf * 128;
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const uint32_t acc = (j > 0 || s4 > 0) ? 1u : 0u;
            tc::umma_ts(tmem + kColDV, b + s4 * 8, dodesc + 128 * s4, id_o, acc);
            tc::umma_ts(tmem + kColDK, b + 64 + s4 * 8, qdesc + 128 * s4, id_o, acc);
          }
          tc::umma_commit(&bars.q_empty[st]);
          tc::umma_commit(&bars.buf_free[buf]);
          if (++buf == kBufs) { buf = 0; bph ^= 1; }
        }
        if (!ok) break;
        tc::umma_commit(&bars.acc_ready);
      }
    }
  } else {
    // ---------------------------------------------------------------- P^T / dS^T, then the results; thread = key row
    const int wg = warp >> 2, qd = warp & 3, r = qd * 32 + lane;
    const float sl2 = a.scale * kLog2eF;
    const uint32_t t_lane = tmem + ((uint32_t) (qd * 32) << 16);
    const uint32_t t_acc = t_lane + (wg == 0 ? kColDV : kColDK);
    int jn = wg, jc = 0;                          // this group's next job and the unit's first job, both numbered over the CTA
    int buf = wg;                                 // buffer of job jn and the phase parity of its barriers
    uint32_t bph = 0;
    float vs[32], vd[32];
    bool ok = true;
    for (int i = 0; ok && pc.next(); ++i) {
      const int bh = pc.unit / chunks_per_head, c = pc.unit % chunks_per_head;
      for (; jn < jc + pc.n; jn += 2) {
        const int st = jn & (kStages - 1);
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
          uint32_t pp[16], pd[16];
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4) {           // 4 query columns at a time: their lse / delta are broadcast reads
            const float4 l4 = *reinterpret_cast<const float4*>(&s_lse[st][32 * half + 4 * q4]);
            const float4 d4 = *reinterpret_cast<const float4*>(&s_delta[st][32 * half + 4 * q4]);
            const float p0 = fast_exp2(fmaf(vs[4 * q4], sl2, fmaf(l4.x, -kLog2eF, lw_log2)));
            const float p1 = fast_exp2(fmaf(vs[4 * q4 + 1], sl2, fmaf(l4.y, -kLog2eF, lw_log2)));
            const float p2 = fast_exp2(fmaf(vs[4 * q4 + 2], sl2, fmaf(l4.z, -kLog2eF, lw_log2)));
            const float p3 = fast_exp2(fmaf(vs[4 * q4 + 3], sl2, fmaf(l4.w, -kLog2eF, lw_log2)));
            pp[2 * q4] = pack_bf16(p0, p1);
            pp[2 * q4 + 1] = pack_bf16(p2, p3);
            pd[2 * q4] = pack_bf16(p0 * ((vd[4 * q4] - d4.x) * a.scale), p1 * ((vd[4 * q4 + 1] - d4.y) * a.scale));
            pd[2 * q4 + 1] = pack_bf16(p2 * ((vd[4 * q4 + 2] - d4.z) * a.scale), p3 * ((vd[4 * q4 + 3] - d4.w) * a.scale));
          }
          tc::tmem_st16(t_b + 16 * half, pp);            // P^T over S^T columns read before
          tc::tmem_st16(t_b + 64 + 16 * half, pd);       // dS^T over dP^T columns read before
        }
        tc::tmem_st_wait();
        tc::fence_before_sync();
        __syncwarp();
        if (lane == 0) tma::mbar_arrive(&bars.pds_ready[buf]);
        buf += 2;
        if (buf >= kBufs) { buf -= kBufs; bph ^= 1; }
      }
      if (!ok) break;
      jc += pc.n;
      ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.acc_ready, (uint32_t) (i & 1), abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      float* dst = (wg == 0 ? dpv : dpk) + ((int64_t) bh * n_keys + (int64_t) c * kKeys + r) * kD;
      const bool whole = pc.n == jobs_all;           // the unit saw every query of its head: nobody else adds to these rows
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        tc::tmem_ld32_async(t_acc + 32 * half, vs);
        tc::tmem_ld_wait(vs);
        if (whole) {
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            *reinterpret_cast<float4*>(dst + 32 * half + 4 * q4) = make_float4(vs[4 * q4] * out_mul, vs[4 * q4 + 1] * out_mul, vs[4 * q4 + 2] * out_mul, vs[4 * q4 + 3] * out_mul);
        } else {
#pragma unroll
          for (int q4 = 0; q4 < 8; ++q4)
            red_add_v4(dst + 32 * half + 4 * q4, vs[4 * q4] * out_mul, vs[4 * q4 + 1] * out_mul, vs[4 * q4 + 2] * out_mul, vs[4 * q4 + 3] * out_mul);
        }
      }
      tc::fence_before_sync();
      __syncwarp();
      if (lane == 0) tma::mbar_arrive(&bars.acc_free);
    }
  }
  if (abort_flag->abort) tc::abort_drain();
  tc::fence_before_sync();
  __syncthreads();
  if (threadIdx.x == 0 && abort_flag->abort && a.status) atomicOr(a.status, (int) LLSA_DEV_WAIT_EXPIRED);
  if (warp == 0) tc::tmem_dealloc(tmem, 512);
}

}  // namespace

// The pooled keys that every query attends to -- all level-1 keys of the one-level form, all level-2 keys of the two-level
// form: the key-major tcgen05 kernel applies when their count is a multiple of 128 and the query rows come in pairs of
// 64-row jobs.  Returns the pooling level it would handle (1 or 2), else 0.
int pooled_dkv_loop_tc_level(const AttnP<bf16>& a) {
  if (a.Nq % (2 * kQ)) return 0;
  if (!a.two_level) return (a.p1_blocks > 0 && a.n1 % kKeys == 0) ? 1 : 0;
  return (a.p2_blocks > 0 && a.n2 % kKeys == 0) ? 2 : 0;
}

int launch_attn_dkv_pooled_loop_tc(const LlsaAttnArgs* g, const AttnP<bf16>& a, int64_t BH, cudaStream_t st) {
  const int level = pooled_dkv_loop_tc_level(a);
  KvMaps maps;
  memset(&maps, 0, sizeof(maps));
  int rc;
  if ((rc = tma::make_map_bhnd(&maps.q, g->q, kQ))) return rc;
  if ((rc = tma::make_map_bhnd(&maps.d_o, g->d_o, kQ))) return rc;
  const int64_t n_keys = level == 1 ? a.n1 : a.n2;
  if ((rc = tma::make_map_rows(&maps.k, level == 1 ? a.pk : a.pk2, (uint64_t) BH * n_keys, kKeys))) return rc;
  if ((rc = tma::make_map_rows(&maps.v, level == 1 ? a.pv : a.pv2, (uint64_t) BH * n_keys, kKeys))) return rc;
  int dev = 0, sms = 148;
  LLSA_CUDA_OK(cudaGetDevice(&dev));
  LLSA_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  // one CTA per SM, each with an equal piece of the flat (head, chunk, job) list
  const int jobs_all = (int) (a.Nq / kQ), n_base = (int) (BH * (n_keys / kKeys));
  const int64_t total = (int64_t) n_base * jobs_all;
  const int grid = total < sms ? (int) total : sms;
  const size_t smem = 1024 + (size_t) (2 * kKeyTile + 2 * kStages * kQTile) * sizeof(bf16);
  LLSA_SMEM_LIMIT((attn_dkv_pooled_loop_tc_kernel), smem);
  if (level == 1)
    attn_dkv_pooled_loop_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, a.dpk, a.dpv, n_keys, jobs_all, n_base, log2f(a.w1),
                                                                 a.kvw1 / a.w1);
  else
    attn_dkv_pooled_loop_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, a.dpk2, a.dpv2, n_keys, jobs_all, n_base, log2f(a.w2),
                                                                 a.kvw2 / a.w2);
  LLSA_LAUNCH_OK("attn_dkv_pooled_loop_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
