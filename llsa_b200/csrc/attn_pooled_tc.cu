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
//   warp 4, one lane : TMA producer.  Per tile: Q [128x64], pooled K [NPx64], pooled V [NPx64]
//                      as 128-byte swizzled tiles into one of two stages (mbarrier expect_tx).
//   warp 5, one lane : MMA issuer.  S = Q.PK^T (M=128, N=NP, K=64) into one of two TMEM buffers,
//                      issued one tile ahead; O_p = P.PV (M=128, N=64, K=NP) when P is ready.
//   warps 0-3        : thread r owns query row r = TMEM lane r.  Reads its NP scores
//                      (tcgen05.ld), softmax in the exp2 domain with +log2(weight) per key
//                      class, writes P (bf16) as a K-major tile; later reads its O_p row,
//                      merges it with the fine part (o, lse written by the fine kernel for
//                      this row) and stores the final o and lse.
// All mbarrier waits are bounded; a wait that expires raises a CTA-wide abort flag, every
// role leaves its loop, lse of the unfinished rows is poisoned with NaN and TMEM is freed.
#include <string.h>

#include "attn.cuh"
#include "mma_frag.cuh"
#include "tc05.cuh"
#include "tma.cuh"

namespace llsa {

constexpr int kTcRows = 128;
constexpr int kTcThreads = 192;       // 4 softmax warps + producer warp + MMA warp

struct TcMaps {
  CUtensorMap q;      // [B,H,N,64] 4-D, box 128 rows
  CUtensorMap pk1;    // [BH*n1, 64], box 16 rows
  CUtensorMap pv1;
  CUtensorMap pk2;    // [BH*n2, 64], box 64 rows (two levels only)
  CUtensorMap pv2;
};

struct TcBars {
  uint64_t full[2], empty[2], s_ready[2], o_ready[2], tmem_free[2], p_ready, p_free;
};

__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  for (int i = 0; i < 400000; ++i) {
    if (tc::mbar_try_wait(bar, parity)) return true;
    if ((i & 1023) == 1023 && *abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

__global__ void __launch_bounds__(kTcThreads, 1)
attn_fwd_pooled_tc_kernel(AttnP<bf16> a, const __grid_constant__ TcMaps maps, int p1_keys, int np, int n_tiles, int tiles_per_head) {
  extern __shared__ unsigned char smem_dyn[];
  __shared__ TcBars bars;
  __shared__ uint32_t s_tmem;
  __shared__ int s_abort;
  bf16* base = reinterpret_cast<bf16*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const int stage_elems = kTcRows * 64 + 2 * np * 64;
  bf16* sP = base + 2 * stage_elems;               // [np/64][128][64]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  volatile int* abort_flag = &s_abort;

  if (tid == 0) {
    s_abort = 0;
    for (int i = 0; i < 2; ++i) {
      tc::mbar_init(&bars.full[i], 1);
      tc::mbar_init(&bars.empty[i], 1);
      tc::mbar_init(&bars.s_ready[i], 1);
      tc::mbar_init(&bars.o_ready[i], 1);
      tc::mbar_init(&bars.tmem_free[i], kTcRows);
    }
    tc::mbar_init(&bars.p_ready, kTcRows);
    tc::mbar_init(&bars.p_free, 1);
    tc::fence_mbar_init();
  }
  if (warp == 0) tc::tmem_alloc(&s_tmem, 512);
  tc::fence_before_sync();
  __syncthreads();
  tc::fence_after_sync();
  const uint32_t tmem = s_tmem;
  const int n_my = (n_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x;

  if (warp == 4) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      const uint32_t bytes = (uint32_t) stage_elems * 2;
      for (int i = 0; i < n_my; ++i) {
        const int tile = blockIdx.x + i * gridDim.x, s = i & 1, u = i >> 1;
        const int64_t bh = tile / tiles_per_head, row0 = (int64_t) (tile % tiles_per_head) * kTcRows;
        if (!tc_wait(&bars.empty[s], (u & 1) ^ 1, abort_flag)) break;
        bf16* sQ = base + s * stage_elems;
        bf16* sK = sQ + kTcRows * 64;
        bf16* sV = sK + np * 64;
        tma::expect_tx(&bars.full[s], bytes);
        tma::load_4d(sQ, &maps.q, &bars.full[s], 0, (int) row0, (int) (bh % a.H), (int) (bh / a.H));
        const int n_p1 = p1_keys / kBS;
        for (int j = 0; j < n_p1; ++j) {
          const int r = (int) (bh * a.n1 + p1_block(a, bh, row0 / kBS, j) * kBS);
          tma::load_2d(sK + j * kBS * 64, &maps.pk1, &bars.full[s], 0, r);
          tma::load_2d(sV + j * kBS * 64, &maps.pv1, &bars.full[s], 0, r);
        }
        for (int j = 0; j < (np - p1_keys) / 64; ++j) {
          const int r = (int) (bh * a.n2 + j * 64);
          tma::load_2d(sK + (p1_keys + j * 64) * 64, &maps.pk2, &bars.full[s], 0, r);
          tma::load_2d(sV + (p1_keys + j * 64) * 64, &maps.pv2, &bars.full[s], 0, r);
        }
      }
    }
  } else if (warp == 5) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = tc::instr_desc(kTcRows, np, 0, 0), idesc_o = tc::instr_desc(kTcRows, 64, 0, 1);
      auto issue_s = [&](int i) -> bool {          // S(i) = Q.PK^T into TMEM buffer i & 1
        const int s = i & 1, u = i >> 1;
        if (!tc_wait(&bars.full[s], u & 1, abort_flag)) return false;
        if (!tc_wait(&bars.tmem_free[s], (u & 1) ^ 1, abort_flag)) return false;
        tc::fence_after_sync();
        const uint32_t qa = tc::smem_u32(base + s * stage_elems), ka = qa + kTcRows * 128;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          tc::umma_ss(tmem + s * 256, tc::smem_desc(qa + ks * 32, 16, 1024), tc::smem_desc(ka + ks * 32, 16, 1024), idesc_s, ks > 0);
        tc::umma_commit(&bars.s_ready[s]);
        return true;
      };
      bool ok = n_my > 0 && issue_s(0);
      for (int i = 0; ok && i < n_my; ++i) {
        const int s = i & 1;
        if (i + 1 < n_my && !issue_s(i + 1)) break;
        if (!tc_wait(&bars.p_ready, i & 1, abort_flag)) break;
        tc::fence_after_sync();
        const uint32_t va = tc::smem_u32(base + s * stage_elems) + (kTcRows + np) * 128;
        for (int ks = 0; ks < np / 16; ++ks) {
          const uint32_t pa = tc::smem_u32(sP) + (ks >> 2) * (kTcRows * 128) + (ks & 3) * 32;   // K-major A, 64 keys per K-block
          tc::umma_ss(tmem + s * 256 + np, tc::smem_desc(pa, 16, 1024), tc::smem_desc(va + ks * 2048, 1024, 1024), idesc_o, ks > 0);
        }
        tc::umma_commit(&bars.o_ready[s]);
        tc::umma_commit(&bars.p_free);
        tc::umma_commit(&bars.empty[s]);
      }
    }
  } else {
    // ---------------------------------------------------------------- softmax + epilogue, thread = query row
    const float sl2 = a.scale * 1.4426950408889634f;
    const float lw1 = log2f(a.w1), lw2 = log2f(a.w2);
    const uint32_t lane_addr = (uint32_t) (warp * 32) << 16;
    for (int i = 0; i < n_my; ++i) {
      const int tile = blockIdx.x + i * gridDim.x, s = i & 1, u = i >> 1;
      const int64_t bh = tile / tiles_per_head, row = (int64_t) (tile % tiles_per_head) * kTcRows + tid;
      const int64_t b = bh / a.H, h = bh % a.H;
      // `ok` is kept warp-uniform: the TMEM loads below are warp-wide instructions
      bool ok = __all_sync(0xffffffffu, tc_wait(&bars.s_ready[s], u & 1, abort_flag));
      tc::fence_after_sync();
      const uint32_t t_s = tmem + s * 256 + lane_addr, t_o = t_s + np;
      float mx = -INFINITY, lsum = 0.f;
      if (ok) {
        for (int c0 = 0; c0 < np; c0 += 32) {
          float v[32];
          tc::tmem_ld32(t_s + c0, v);
          const float lw = c0 < p1_keys ? lw1 : lw2;
#pragma unroll
          for (int j = 0; j < 32; ++j) mx = fmaxf(mx, fmaf(v[j], sl2, lw));
        }
        ok = __all_sync(0xffffffffu, tc_wait(&bars.p_free, (i & 1) ^ 1, abort_flag));      // the previous tile's P.PV has consumed sP
      }
      if (ok) {
        for (int c0 = 0; c0 < np; c0 += 32) {
          float v[32];
          tc::tmem_ld32(t_s + c0, v);
          const float lw = c0 < p1_keys ? lw1 : lw2;
#pragma unroll
          for (int j = 0; j < 32; ++j) { v[j] = fast_exp2(fmaf(v[j], sl2, lw) - mx); lsum += v[j]; }
          bf16* pt = sP + (c0 >> 6) * (kTcRows * 64);          // K-block of 64 keys
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 w;
            w.x = pack_bf16(v[8 * q], v[8 * q + 1]); w.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
            w.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]); w.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
            *reinterpret_cast<uint4*>(pt + tc::swz(tid, ((c0 & 63) >> 3) + q)) = w;
          }
        }
        tc::fence_async_smem();          // P must be visible to the tensor core's (async proxy) reads
        tc::fence_before_sync();
        tma::mbar_arrive(&bars.p_ready);
        ok = __all_sync(0xffffffffu, tc_wait(&bars.o_ready[s], u & 1, abort_flag));
        tc::fence_after_sync();
      }
      float lse_out = __int_as_float(0x7fc00000);               // NaN unless everything completed
      if (ok) {
        const float Lf = a.lse[bh * a.Nq + row] * 1.4426950408889634f;    // fine part, log2 domain
        const float Lp = mx + log2f(lsum);
        const float Lm = fmaxf(Lf, Lp);
        const float ef = fast_exp2(Lf - Lm), ep = fast_exp2(Lp - Lm);
        const float inv = 1.f / (ef + ep);
        const float wf = ef * inv, wp = ep * inv / lsum;
        bf16* orow = a.o.row(b, h, row);
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 32) {
          float v[32];
          tc::tmem_ld32(t_o + c0, v);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const uint4 f = *reinterpret_cast<const uint4*>(orow + c0 + 8 * q);
            uint4 w;
            w.x = pack_bf16(bf16_lo(f.x) * wf + v[8 * q] * wp, bf16_hi(f.x) * wf + v[8 * q + 1] * wp);
            w.y = pack_bf16(bf16_lo(f.y) * wf + v[8 * q + 2] * wp, bf16_hi(f.y) * wf + v[8 * q + 3] * wp);
            w.z = pack_bf16(bf16_lo(f.z) * wf + v[8 * q + 4] * wp, bf16_hi(f.z) * wf + v[8 * q + 5] * wp);
            w.w = pack_bf16(bf16_lo(f.w) * wf + v[8 * q + 6] * wp, bf16_hi(f.w) * wf + v[8 * q + 7] * wp);
            *reinterpret_cast<uint4*>(orow + c0 + 8 * q) = w;
          }
        }
        lse_out = (Lm + log2f(ef + ep)) * 0.6931471805599453f;
        tc::fence_before_sync();
        tma::mbar_arrive(&bars.tmem_free[s]);                    // this row's S / O columns may be overwritten
      }
      a.lse[bh * a.Nq + row] = lse_out;
      if (!ok) break;
    }
  }
  tc::fence_before_sync();
  __syncthreads();
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
  const size_t smem = 1024 + (size_t) (2 * (kTcRows * 64 + 2 * np * 64) + (np / 64) * kTcRows * 64) * sizeof(bf16);
  LLSA_CUDA_OK(cudaFuncSetAttribute(attn_fwd_pooled_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
  attn_fwd_pooled_tc_kernel<<<grid, kTcThreads, smem, st>>>(a, maps, p1_keys, np, n_tiles, tiles_per_head);
  LLSA_LAUNCH_OK("attn_fwd_pooled_tc_kernel");
  return LLSA_OK;
}

}  // namespace llsa
