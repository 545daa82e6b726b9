// Pooled-key gradients on tcgen05 for the keys that EVERY query attends to: all level-1 pooled keys of the
// one-level form (sparse_attention_res_1.py:362-400) and all level-2 keys of the two-level form
// (_attn_bwd_res_dpkv2, sparse_attention_res_2.py:418-489) -- the key-major half of the pooled backward, with a
// loop over the queries.
//
// A work unit is (head, chunk of 128 pooled keys); it walks all query rows of the head 64 at a time:
//     S^T  = K_c . Q_t^T   [128 keys x 64 queries]  (K = 64 channels)   shared-memory operands
//     dP^T = V_c . dO_t^T  [128 x 64]
//     P^T  = exp2(S^T*scale*log2e + log2 w - lse[q]),  dS^T = P^T * (dP^T - delta[q]) * scale     thread = key row;
//            lse and delta of the 64 query columns sit in shared memory next to the Q / dO tile
//     dV_c += P^T  . dO_t  [128 x 64]  (K = 64 queries)   P^T, dS^T read from TENSOR MEMORY (packed bf16, written over
//     dK_c += dS^T . Q_t                                   S^T / dP^T), dO_t / Q_t as MN-major operands (the same tiles)
// dK_c, dV_c accumulate in TMEM over the whole query loop; the unit owns its keys, so the results are plain stores
// into the fp32 pooled-gradient accumulators (scaled by kv_weight / token_weight, the reference's weighting of the
// pooled dK/dV side).
// TMEM columns: buffer b (job parity): S^T at 128 b, dP^T at 128 b + 64; dV at [256,320), dK at [320,384).
// Roles (one persistent CTA per SM, 10 warps): warp 8 lane 0 = TMA producer (K_c, V_c per unit; Q_t, dO_t, lse, delta per
// job in a ring of 4), warp 9 lane 0 = MMA issuer, warps 0-3 / 4-7 = two softmax warpgroups on alternating jobs; at the
// end of a unit group 0 stores dV, group 1 stores dK.  Every mbarrier wait is bounded (abort flag, TMEM freed).
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
constexpr int kStages = 4;
constexpr int kThreads = 320;
constexpr float kLog2eF = 1.4426950408889634f;
constexpr uint32_t kColDV = 256, kColDK = 320;

struct KvMaps {
  CUtensorMap q, d_o;         // [B,H,Nq,64] 4-D, box 64 rows
  CUtensorMap k, v;           // contiguous pooled keys / values [BH*n, 64], box 128 rows
};

struct KvBars {
  uint64_t kv_full, kv_empty, q_full[kStages], q_empty[kStages], sdp_ready[2], pds_ready[2], acc_ready, acc_free;
};

// n_keys: pooled keys per head (a multiple of 128); jobs: 64-row query jobs per unit (even); splits: units per (head, key chunk),
// each walking its own range of the queries (with more than one, the results are added with reductions instead of stored);
// units = BH * n_keys / 128 * splits.
__global__ void __launch_bounds__(kThreads, 1)
attn_dkv_pooled_loop_tc_kernel(AttnP<bf16> a, const __grid_constant__ KvMaps maps, float* __restrict__ dpk, float* __restrict__ dpv,
                               int64_t n_keys, int jobs, int splits, int n_units, float lw_log2, float out_mul) {
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
    for (int i = 0; i < 2; ++i) { tc::mbar_init(&bars.sdp_ready[i], 1); tc::mbar_init(&bars.pds_ready[i], 4); }
    tc::mbar_init(&bars.acc_ready, 1);
    tc::mbar_init(&bars.acc_free, 8);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&s_tmem, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int n_my = (n_units - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x;
  const int chunks_per_head = (int) (n_keys / kKeys);

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      int cj = 0;
      for (int i = 0; i < n_my; ++i) {
        const int unit = blockIdx.x + i * gridDim.x, sp = unit % splits;
        const int bh = unit / splits / chunks_per_head, c = unit / splits % chunks_per_head;
        if (!tc::bounded_wait(&bars.kv_empty, (i & 1) ^ 1, abort_flag)) break;
        tma::expect_tx(&bars.kv_full, 2 * kKeyTile * 2);
        tma::load_2d(sK, &maps.k, &bars.kv_full, 0, (int) ((int64_t) bh * n_keys + (int64_t) c * kKeys));
        tma::load_2d(sV, &maps.v, &bars.kv_full, 0, (int) ((int64_t) bh * n_keys + (int64_t) c * kKeys));
        bool ok = true;
        for (int j = 0; ok && j < jobs; ++j, ++cj) {
          const int st = cj % kStages;
          if (!(ok = tc::bounded_wait(&bars.q_empty[st], ((cj / kStages) & 1) ^ 1, abort_flag))) break;
          tma::expect_tx(&bars.q_full[st], 2 * kQTile * 2 + 2 * kQ * 4);
          const int qrow = (sp * jobs + j) * kQ;
          tma::load_4d(sQ + st * kQTile, &maps.q, &bars.q_full[st], 0, qrow, bh % a.H, bh / a.H);
          tma::load_4d(sDO + st * kQTile, &maps.d_o, &bars.q_full[st], 0, qrow, bh % a.H, bh / a.H);
          tma::load_bulk(s_lse[st], a.lse + (int64_t) bh * a.Nq + qrow, kQ * 4, &bars.q_full[st]);
          tma::load_bulk(s_delta[st], a.delta + (int64_t) bh * a.Nq + qrow, kQ * 4, &bars.q_full[st]);
        }
        if (!ok) break;
      }
    }
  } else if (warp == 9) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t id_s = tc::instr_desc(kKeys, kQ, 0, 0), id_o = tc::instr_desc(kKeys, 64, 0, 1);
      const uint32_t hi = (uint32_t) (tc::smem_desc(0, 0, 1024) >> 32);
      auto lo = [](const void* p, uint32_t lbo_bytes) { return ((tc::smem_u32(p) >> 4) & 0x3FFFu) | (((lbo_bytes >> 4) & 0x3FFFu) << 16); };
      constexpr uint32_t kQStage = (uint32_t) (kQTile * 2) >> 4;
      const uint32_t lK = lo(sK, 16), lV = lo(sV, 16), lQ = lo(sQ, 16), lDO = lo(sDO, 16), lQm = lo(sQ, 1024), lDOm = lo(sDO, 1024);
      int cj = 0;
      int64_t J = 0;
      bool ok = true;
      for (int i = 0; ok && i < n_my; ++i) {
        if (!(ok = tc::bounded_wait(&bars.kv_full, i & 1, abort_flag))) break;
        tc::fence_after_sync();
        const int cj0 = cj;
        auto issue_sdp = [&](int j) -> bool {        // S^T and dP^T of job j into buffer j & 1
          const int st = cj % kStages;
          if (!tc::bounded_wait(&bars.q_full[st], (cj / kStages) & 1, abort_flag)) return false;
          tc::fence_after_sync();
          const uint32_t d = tmem + (j & 1) * 128, q_ = lQ + st * kQStage, o_ = lDO + st * kQStage;
          tc::umma_ss_lh<0>(d, lK, hi, q_, hi, id_s);
          tc::umma_ss_lh<0>(d + 64, lV, hi, o_, hi, id_s);
#pragma unroll
          for (int s4 = 1; s4 < 4; ++s4) {
            tc::umma_ss_lh<1>(d, lK + 2 * s4, hi, q_ + 2 * s4, hi, id_s);
            tc::umma_ss_lh<1>(d + 64, lV + 2 * s4, hi, o_ + 2 * s4, hi, id_s);
          }
          tc::umma_commit(&bars.sdp_ready[j & 1]);
          ++cj;
          return true;
        };
        auto issue_out = [&](int j) -> bool {        // dV (+)= P^T . dO_t, dK (+)= dS^T . Q_t: 4 k-steps of 16 query rows (2048 bytes)
          const int st = (cj0 + j) % kStages;
          if (j == 0 && i > 0 && !tc::bounded_wait(&bars.acc_free, (i - 1) & 1, abort_flag)) return false;    // previous unit's results have been read
          tc::fence_after_sync();
          const uint64_t dodesc = ((uint64_t) hi << 32) | (uint64_t) (lDOm + st * kQStage), qdesc = ((uint64_t) hi << 32) | (uint64_t) (lQm + st * kQStage);
          const uint32_t b = tmem + (j & 1) * 128;
#pragma unroll
          for (int s4 = 0; s4 < 4; ++s4) {
            const uint32_t acc = (j > 0 || s4 > 0) ? 1u : 0u;
            tc::umma_ts(tmem + kColDV, b + s4 * 8, dodesc + 128 * s4, id_o, acc);
            tc::umma_ts(tmem + kColDK, b + 64 + s4 * 8, qdesc + 128 * s4, id_o, acc);
          }
          tc::umma_commit(&bars.q_empty[st]);
          return true;
        };
        for (int j = 0; ok && j < jobs; ++j) {
          if (j >= 2) {
            const int64_t Jp = J + j - 2;
            if (!(ok = tc::bounded_wait(&bars.pds_ready[j & 1], (uint32_t) ((Jp >> 1) & 1), abort_flag))) break;
            tc::fence_after_sync();
            if (!(ok = issue_out(j - 2))) break;
          }
          ok = issue_sdp(j);
        }
        if (!ok) break;
        for (int j = jobs - 2; ok && j < jobs; ++j) {
          const int64_t Jp = J + j;
          if (!(ok = tc::bounded_wait(&bars.pds_ready[j & 1], (uint32_t) ((Jp >> 1) & 1), abort_flag))) break;
          tc::fence_after_sync();
          ok = issue_out(j);
        }
        if (!ok) break;
        tc::umma_commit(&bars.acc_ready);
        tc::umma_commit(&bars.kv_empty);
        J += jobs;
      }
    }
  } else {
    // ---------------------------------------------------------------- P^T / dS^T, then the stores; thread = key row
    const int wg = warp >> 2, qd = warp & 3, r = qd * 32 + lane;
    const float sl2 = a.scale * kLog2eF;
    const uint32_t t_b = tmem + wg * 128 + ((uint32_t) (qd * 32) << 16);
    const uint32_t t_acc = tmem + (wg == 0 ? kColDV : kColDK) + ((uint32_t) (qd * 32) << 16);
    int64_t Jw = 0;
    int cj = wg;                                  // ring position of this group's next job
    float vs[32], vd[32];
    for (int i = 0; i < n_my; ++i) {
      const int unit = blockIdx.x + i * gridDim.x;
      const int bh = unit / splits / chunks_per_head, c = unit / splits % chunks_per_head;
      bool ok = true;
      for (int j = wg; j < jobs; j += 2, cj += 2) {
        const int st = cj % kStages;
        ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.sdp_ready[wg], (uint32_t) (Jw & 1), abort_flag));
        tc::fence_after_sync();
        if (!ok) break;
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
        if (lane == 0) tma::mbar_arrive(&bars.pds_ready[wg]);
        ++Jw;
      }
      if (!ok) break;
      ok = __all_sync(0xffffffffu, tc::bounded_wait(&bars.acc_ready, (uint32_t) (i & 1), abort_flag));
      tc::fence_after_sync();
      if (!ok) break;
      float* dst = (wg == 0 ? dpv : dpk) + ((int64_t) bh * n_keys + (int64_t) c * kKeys + r) * kD;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        tc::tmem_ld32_async(t_acc + 32 * half, vs);
        tc::tmem_ld_wait(vs);
        if (splits == 1) {
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
  // enough units for two rounds over the SMs: split the query range (an even number of 64-row jobs per unit)
  const int jobs_all = (int) (a.Nq / kQ), base_units = (int) (BH * (n_keys / kKeys));
  int splits = 1;
  while (base_units * splits < 2 * sms && jobs_all % (4 * splits) == 0 && jobs_all / (2 * splits) >= 16) splits *= 2;
  const int n_units = base_units * splits, jobs = jobs_all / splits;
  const int grid = n_units < sms ? n_units : sms;
  const size_t smem = 1024 + (size_t) (2 * kKeyTile + 2 * kStages * kQTile) * sizeof(bf16);
  LLSA_SMEM_LIMIT((attn_dkv_pooled_loop_tc_kernel), smem);
  if (level == 1)
    attn_dkv_pooled_loop_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, a.dpk, a.dpv, n_keys, jobs, splits, n_units, log2f(a.w1),
                                                                 a.kvw1 / a.w1);
  else
    attn_dkv_pooled_loop_tc_kernel<<<grid, kThreads, smem, st>>>(a, maps, a.dpk2, a.dpv2, n_keys, jobs, splits, n_units, log2f(a.w2),
                                                                 a.kvw2 / a.w2);
  LLSA_LAUNCH_OK("attn_dkv_pooled_loop_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
