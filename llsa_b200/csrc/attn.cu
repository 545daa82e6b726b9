// Argument validation and dispatch of the attention entry points.
#include <string.h>

#include "attn.cuh"

namespace llsa {

static int check_attn_args(const LlsaAttnArgs* g, bool bwd) {
  LLSA_REQUIRE(g, LLSA_ERR_NULL, "attn: null argument block");
  LLSA_REQUIRE(g->q && g->k && g->v && g->pk && g->pv && g->indices && g->o && g->lse, LLSA_ERR_NULL, "attn: a required tensor is null");
  LLSA_REQUIRE(g->q->ndim == 4, LLSA_ERR_SHAPE, "attn: q must be [B,H,N,D]");
  const int dt = g->q->dtype;
  LLSA_REQUIRE(is_float_dtype(dt), LLSA_ERR_DTYPE, "attn: q must be f32 or bf16");
  LLSA_REQUIRE(g->k->ndim == 4, LLSA_ERR_SHAPE, "attn: k must be [B,H,N,D]");
  // Nq query tokens attend to N key tokens; Nq < N when q is a shard of the sequence (both multiples of 256)
  const int64_t B = g->q->shape[0], H = g->q->shape[1], Nq = g->q->shape[2], D = g->q->shape[3], N = g->k->shape[2];
  LLSA_REQUIRE(D == kD, LLSA_ERR_SHAPE, "attn: head dim %lld unsupported (only 64)", (long long) D);
  LLSA_REQUIRE(g->block_size == kBS, LLSA_ERR_ARG, "attn: block size %d unsupported (only 16)", g->block_size);
  LLSA_REQUIRE(N >= 256 && N % 256 == 0, LLSA_ERR_SHAPE, "attn: N=%lld must be a positive multiple of 256", (long long) N);
  LLSA_REQUIRE(Nq >= 256 && Nq % 256 == 0, LLSA_ERR_SHAPE, "attn: query length %lld must be a positive multiple of 256", (long long) Nq);
  const int64_t n1 = N / kBS, n2 = n1 / kBS, nq1 = Nq / kBS, nq2 = nq1 / kBS;
  const bool two = g->pk2 != nullptr;
  LLSA_REQUIRE(g->topk >= 2 && g->topk % 2 == 0 && g->topk <= n1 && g->topk <= 64, LLSA_ERR_ARG,
               "attn: topk=%d must be even, in 2..min(64, N/16)", g->topk);
  int rc;
  if ((rc = check_bhnd(g->q, "q", dt, B, H, Nq, D))) return rc;
  if ((rc = check_bhnd(g->k, "k", dt, B, H, N, D))) return rc;
  if ((rc = check_bhnd(g->v, "v", dt, B, H, N, D))) return rc;
  if ((rc = check_bhnd(g->o, "o", dt, B, H, Nq, D))) return rc;
  const int64_t s1[4] = {B, H, n1, D}, s2[4] = {B, H, n2, D}, sl[3] = {B, H, Nq}, si[4] = {B, H, nq1, g->topk};
  if ((rc = check_contig(g->pk, "pk", dt, 4, s1))) return rc;
  if ((rc = check_contig(g->pv, "pv", dt, 4, s1))) return rc;
  if ((rc = check_contig(g->lse, "lse", LLSA_F32, 3, sl))) return rc;
  LLSA_REQUIRE(is_index_dtype(g->indices->dtype), LLSA_ERR_DTYPE, "attn: indices must be i32 or i64");
  if ((rc = check_contig(g->indices, "indices", g->indices->dtype, 4, si))) return rc;
  if (two) {
    LLSA_REQUIRE(g->pv2 && g->p_indices, LLSA_ERR_NULL, "attn: pv2 / p_indices missing for the two-level form");
    LLSA_REQUIRE(g->topk_p >= 2 && g->topk_p % 2 == 0 && g->topk_p <= n2 && g->topk_p <= 64, LLSA_ERR_ARG,
                 "attn: topk_p=%d must be even, in 2..min(64, N/256)", g->topk_p);
    LLSA_REQUIRE(n2 < 64 || n2 % 32 == 0, LLSA_ERR_SHAPE, "attn: N/256=%lld must be a multiple of 32", (long long) n2);
    const int64_t sp[4] = {B, H, nq2, g->topk_p};
    if ((rc = check_contig(g->pk2, "pk2", dt, 4, s2))) return rc;
    if ((rc = check_contig(g->pv2, "pv2", dt, 4, s2))) return rc;
    LLSA_REQUIRE(is_index_dtype(g->p_indices->dtype), LLSA_ERR_DTYPE, "attn: p_indices must be i32 or i64");
    if ((rc = check_contig(g->p_indices, "p_indices", g->p_indices->dtype, 4, sp))) return rc;
  } else {
    LLSA_REQUIRE(n1 < 64 || n1 % 32 == 0, LLSA_ERR_SHAPE, "attn: N/16=%lld must be a multiple of 32", (long long) n1);
  }
  if (!bwd && g->fwd_redo) {
    int64_t have = 1;
    for (int i = 0; i < g->fwd_redo->ndim; ++i) have *= g->fwd_redo->shape[i];
    LLSA_REQUIRE(g->fwd_redo->ptr && g->fwd_redo->dtype == LLSA_I32 && is_contiguous(g->fwd_redo) && have * 4 >= B * H * Nq &&
                     ((uintptr_t) g->fwd_redo->ptr % 4) == 0,
                 LLSA_ERR_WORKSPACE, "attn_fwd: fwd_redo must be a contiguous I32 tensor of at least B*H*N/4 = %lld elements", (long long) ((B * H * Nq + 3) / 4));
  }
  if (bwd) {
    LLSA_REQUIRE(g->d_o && g->dq && g->dk && g->dv && g->offsets && g->flat && g->delta && g->dpk_acc && g->dpv_acc, LLSA_ERR_NULL,
                 "attn_bwd: a required tensor is null");
    if ((rc = check_bhnd(g->d_o, "d_o", dt, B, H, Nq, D))) return rc;
    if ((rc = check_bhnd(g->dq, "dq", dt, B, H, Nq, D))) return rc;
    if ((rc = check_bhnd(g->dk, "dk", dt, B, H, N, D))) return rc;
    if ((rc = check_bhnd(g->dv, "dv", dt, B, H, N, D))) return rc;
    const int64_t so[3] = {B, H, n1 + 1}, sf[3] = {B, H, nq1 * g->topk};
    LLSA_REQUIRE(is_index_dtype(g->offsets->dtype), LLSA_ERR_DTYPE, "attn_bwd: offsets must be i32 or i64");
    if ((rc = check_contig(g->offsets, "offsets", g->offsets->dtype, 3, so))) return rc;
    if ((rc = check_contig(g->flat, "flat", LLSA_I32, 3, sf))) return rc;
    if ((rc = check_contig(g->delta, "delta", LLSA_F32, 3, sl))) return rc;
    if ((rc = check_contig(g->dpk_acc, "dpk_acc", LLSA_F32, 4, s1))) return rc;
    if ((rc = check_contig(g->dpv_acc, "dpv_acc", LLSA_F32, 4, s1))) return rc;
    if (dt == LLSA_BF16 && !g->force_generic) {
      LLSA_REQUIRE(g->dkv_partial, LLSA_ERR_WORKSPACE, "attn_bwd: dkv_partial scratch missing");
      const int64_t need = llsa_attn_bwd_partial_elems(B, H, Nq, g->topk);
      LLSA_REQUIRE(g->dkv_partial->ptr && g->dkv_partial->dtype == LLSA_F32 && g->dkv_partial->ndim == 4 && is_contiguous(g->dkv_partial) &&
                       g->dkv_partial->shape[0] * g->dkv_partial->shape[1] * g->dkv_partial->shape[2] * g->dkv_partial->shape[3] >= need,
                   LLSA_ERR_WORKSPACE, "attn_bwd: dkv_partial must be a contiguous F32 tensor of at least %lld elements", (long long) need);
    }
    if (dt == LLSA_BF16 && !g->force_generic) {
      // P / dS hand-over between the dQ stage and the dK/dV stage of the tensor-core path
      const int64_t need = B * H * nq1 * g->topk * 256;
      LLSA_REQUIRE(g->fine_pds && g->fine_pds->ptr && g->fine_pds->dtype == LLSA_F32 && is_contiguous(g->fine_pds), LLSA_ERR_WORKSPACE,
                   "attn_bwd: fine_pds scratch missing (a contiguous F32 tensor of llsa_attn_bwd_pds_elems() elements)");
      int64_t have = 1;
      for (int i = 0; i < g->fine_pds->ndim; ++i) have *= g->fine_pds->shape[i];
      LLSA_REQUIRE(have >= need && ((uintptr_t) g->fine_pds->ptr % 16) == 0, LLSA_ERR_WORKSPACE,
                   "attn_bwd: fine_pds holds %lld elements, %lld needed", (long long) have, (long long) need);
      LLSA_REQUIRE(g->flat_pairs && g->flat_ranges, LLSA_ERR_WORKSPACE, "attn_bwd: flat_pairs / flat_ranges missing (llsa_transpose_indices_pairs)");
      if ((rc = check_contig(g->flat_pairs, "flat_pairs", LLSA_I32, 3, sf))) return rc;
      LLSA_REQUIRE(g->flat_ranges->ndim == 4 && range_entries_of(nq1 * g->topk, g->flat_ranges->shape[2]) > 0, LLSA_ERR_SHAPE,
                   "attn_bwd: flat_ranges must be the [B,H,R,2] ranges tensor of llsa_transpose_indices_pairs");
      const int64_t sr[4] = {B, H, g->flat_ranges->shape[2], 2};
      if ((rc = check_contig(g->flat_ranges, "flat_ranges", LLSA_I32, 4, sr))) return rc;
    }
    if (two) {
      LLSA_REQUIRE(g->dpk2_acc && g->dpv2_acc, LLSA_ERR_NULL, "attn_bwd: dpk2_acc / dpv2_acc missing");
      if ((rc = check_contig(g->dpk2_acc, "dpk2_acc", LLSA_F32, 4, s2))) return rc;
      if ((rc = check_contig(g->dpv2_acc, "dpv2_acc", LLSA_F32, 4, s2))) return rc;
    }
  }
  return LLSA_OK;
}

}  // namespace llsa

using namespace llsa;

extern "C" int64_t llsa_attn_bwd_partial_elems(int64_t B, int64_t H, int64_t Nq, int32_t topk) {
  if (B <= 0 || H <= 0 || Nq <= 0 || topk <= 0) return 0;
  const int64_t ranges = (Nq / kBS * topk + kRangeEntriesSmall - 1) / kRangeEntriesSmall;     // sized for the smaller of the two range sizes
  return B * H * ((ranges + 3) / 4) * 4096;          // a head and a tail tile (2048 floats each) per CTA of four ranges
}

extern "C" int64_t llsa_attn_bwd_pds_elems(int64_t B, int64_t H, int64_t Nq, int32_t topk) {
  if (B <= 0 || H <= 0 || Nq <= 0 || topk <= 0) return 0;
  return B * H * (Nq / kBS) * topk * 256;
}

extern "C" int llsa_attn_fwd(const LlsaAttnArgs* args, void* stream) {
  int rc = check_attn_args(args, false);
  if (rc) return rc;
  if (args->q->shape[0] * args->q->shape[1] == 0) return LLSA_OK;
  cudaStream_t st = (cudaStream_t) stream;
  if (args->q->dtype == LLSA_BF16 && !args->force_generic) return launch_attn_fwd_mma(args, st);
  return launch_attn_fwd_generic(args, st);
}

extern "C" int llsa_attn_bwd(const LlsaAttnArgs* args, void* stream) {
  int rc = check_attn_args(args, true);
  if (rc) return rc;
  if (args->q->shape[0] * args->q->shape[1] == 0) return LLSA_OK;
  cudaStream_t st = (cudaStream_t) stream;
  if (args->q->dtype == LLSA_BF16 && !args->force_generic) return launch_attn_bwd_mma(args, st);
  return launch_attn_bwd_generic(args, st);
}
