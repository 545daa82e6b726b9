// Parameters shared by the attention kernels (forward, dQ side, dK/dV side).
//
// Key sets a query row attends to (reference: sparse_attention_res_1.py:54-106,
// sparse_attention_res_2.py:60-149); all sets come in blocks of 16 keys:
//   fine    : the topk selected 16-token blocks of the row's query block, weight 1
//   pooled-1: one level  -> ALL level-1 pooled keys;
//             two levels -> the 16 children of each of the topk_p level-2 blocks
//             selected by the row's PARENT query block; weight token_weight
//   pooled-2: two levels only -> ALL level-2 pooled keys; weight token_weight_2
// A pooled stage with fewer than 64 keys is skipped, as the reference's forward
// loops do (res_1.py:85, res_2.py:127).
#pragma once
#include "common.cuh"

namespace llsa {

constexpr int kBS = 16;   // tokens per block
constexpr int kD = 64;    // head dim

template <typename T>
struct AttnP {
  View<const T> q, k, v, d_o, o_in;
  View<T> o, dq, dk, dv;
  const T* pk;   // contiguous [BH, n1, D]
  const T* pv;
  const T* pk2;  // contiguous [BH, n2, D] or nullptr
  const T* pv2;
  IdxView idx, pidx;
  float* lse;    // [BH, Nq]
  float* delta;  // [BH, Nq]
  float* dpk;    // fp32 accumulators [BH, n1, D]
  float* dpv;
  float* dpk2;   // [BH, n2, D]
  float* dpv2;
  const void* offsets;  // CSR of idx: [BH, n1+1]
  int off64;
  const int32_t* flat;  // [BH, nq1*topk]
  const int32_t* pairs; // [BH, nq1*topk]: position qb*topk + slot of each CSR entry inside the head's index list, or nullptr
  int range_entries;    // nominal entries per work range (32, or 16 for small problems)
  const int2* ranges;   // [BH, ceil(nq1*topk / 32)]: (first entry, its bucket) of every work range of the fine dK/dV kernel, or nullptr
  uint4* pds;           // [BH*nq1*topk][2][32]: P^T and dS^T (bf16) of every (query block, selected block) pair as the
                        // A-operand registers of the dK/dV products, one uint4 per lane; nullptr: not handed over
  int32_t* status;      // device status word (LlsaDeviceStatus bits) or nullptr
  int wait_limit;       // polls before a bounded mbarrier wait gives up (0: the kernels' default)
  int H;
  int64_t N, n1, n2;      // KEY side: tokens, 16-token blocks, 256-token blocks of k / v
  int64_t Nq, nq1, nq2;   // QUERY side: the same counts for q (equal to the key side unless q is a shard of the sequence)
  int topk, topk_p;
  int two_level;
  int p1_blocks;   // pooled-1 key blocks per query row (0 when the stage is skipped)
  int p2_blocks;   // pooled-2 key blocks per query row
  float w1, w2;    // token weights (forward and dQ side)
  float kvw1, kvw2;  // weights on the pooled dK/dV side
  float scale;     // 1/sqrt(D)
  int fold;        // fold the pooling backward into dk/dv
};

// Block index (in units of 16 keys) of pooled-1 block `i` (0 <= i < p1_blocks)
// for query block `qb` of head `bh`.
template <typename T>
__device__ __forceinline__ int64_t p1_block(const AttnP<T>& a, int64_t bh, int64_t qb, int i) {
  if (!a.two_level) return i;
  int64_t p = a.pidx.at((bh * a.nq2 + qb / kBS) * a.topk_p + i);
  return p < 0 ? 0 : (p >= a.n2 ? a.n2 - 1 : p);
}

template <typename T>
__device__ __forceinline__ int64_t fine_block(const AttnP<T>& a, int64_t bh, int64_t qb, int i) {
  int64_t j = a.idx.at((bh * a.nq1 + qb) * a.topk + i);
  return j < 0 ? 0 : (j >= a.n1 ? a.n1 - 1 : j);
}

int build_attn_params_check(const LlsaAttnArgs* g, bool bwd);

template <typename T>
AttnP<T> build_attn_params(const LlsaAttnArgs* g, bool bwd);

void note_scalar_path();                             // leaves a note in the thread's error string: bf16 operands on the scalar kernels
bool mma_path_ok(const LlsaAttnArgs* g, bool bwd);   // operands meet the tensor-core kernels' alignment / top-k limits
int pooled_smem_tiles(int n_pooled);                 // pooled key tiles a CTA keeps in shared memory
int pooled_tc_keys(const AttnP<__nv_bfloat16>& a);   // pooled keys per row if the tcgen05 pooled kernels apply, else 0
int launch_attn_fwd_pooled_tc(const LlsaAttnArgs* g, const AttnP<__nv_bfloat16>& a, int64_t BH, cudaStream_t st);
int pooled_loop_tc_keys(const AttnP<__nv_bfloat16>& a);   // pooled keys per row if the key-loop tcgen05 forward applies, else 0
int launch_attn_fwd_pooled_loop_tc(const LlsaAttnArgs* g, const AttnP<__nv_bfloat16>& a, int64_t BH, cudaStream_t st);
int pooled_dq_loop_tc_keys(const AttnP<__nv_bfloat16>& a);  // pooled keys per row if the key-loop tcgen05 dQ kernel applies, else 0
int launch_attn_dq_pooled_loop_tc(const LlsaAttnArgs* g, const AttnP<__nv_bfloat16>& a, int64_t BH, cudaStream_t st);
int pooled_dkv_loop_tc_level(const AttnP<__nv_bfloat16>& a);  // pooling level (1 or 2) the key-major tcgen05 pooled dK/dV kernel would take, else 0
int launch_attn_dkv_pooled_loop_tc(const LlsaAttnArgs* g, const AttnP<__nv_bfloat16>& a, int64_t BH, cudaStream_t st);
bool pooled_bwd_tc_ok(const AttnP<__nv_bfloat16>& a);  // the tcgen05 pooled backward applies (two levels, 128 + 64 pooled keys)
int launch_attn_bwd_pooled_tc(const LlsaAttnArgs* g, const AttnP<__nv_bfloat16>& a, int64_t BH, cudaStream_t st);
int launch_attn_fwd_generic(const LlsaAttnArgs* g, cudaStream_t st);
int launch_attn_bwd_generic(const LlsaAttnArgs* g, cudaStream_t st);
int launch_attn_fwd_mma(const LlsaAttnArgs* g, cudaStream_t st);
int launch_attn_bwd_mma(const LlsaAttnArgs* g, cudaStream_t st);

template <typename T>
inline AttnP<T> build_attn_params(const LlsaAttnArgs* g, bool bwd) {
  AttnP<T> a;
  memset(&a, 0, sizeof(a));
  a.q = make_view<const T>(g->q);
  a.k = make_view<const T>(g->k);
  a.v = make_view<const T>(g->v);
  a.pk = (const T*) g->pk->ptr;
  a.pv = (const T*) g->pv->ptr;
  a.two_level = g->pk2 != nullptr;
  if (a.two_level) {
    a.pk2 = (const T*) g->pk2->ptr;
    a.pv2 = (const T*) g->pv2->ptr;
    a.pidx = make_idx(g->p_indices);
  }
  a.idx = make_idx(g->indices);
  a.lse = (float*) g->lse->ptr;
  a.H = (int) g->q->shape[1];
  a.N = g->k->shape[2];
  a.n1 = a.N / kBS;
  a.n2 = a.n1 / kBS;
  a.Nq = g->q->shape[2];
  a.nq1 = a.Nq / kBS;
  a.nq2 = a.nq1 / kBS;
  a.topk = g->topk;
  a.topk_p = g->topk_p;
  a.w1 = g->token_weight;
  a.w2 = g->token_weight_2;
  a.scale = 0.125f;
  a.status = g->status;
  a.wait_limit = g->wait_limit;
  if (a.two_level) {
    a.p1_blocks = a.topk_p;
    a.p2_blocks = a.n2 >= 64 ? (int) (a.n2 / kBS) : 0;
  } else {
    a.p1_blocks = a.n1 >= 64 ? (int) (a.n1 / kBS) : 0;
    a.p2_blocks = 0;
  }
  if (!bwd) {
    a.o = make_view<T>(g->o);
  } else {
    a.o_in = make_view<const T>(g->o);
    a.d_o = make_view<const T>(g->d_o);
    a.dq = make_view<T>(g->dq);
    a.dk = make_view<T>(g->dk);
    a.dv = make_view<T>(g->dv);
    a.delta = (float*) g->delta->ptr;
    a.dpk = (float*) g->dpk_acc->ptr;
    a.dpv = (float*) g->dpv_acc->ptr;
    if (a.two_level) {
      a.dpk2 = (float*) g->dpk2_acc->ptr;
      a.dpv2 = (float*) g->dpv2_acc->ptr;
    }
    a.offsets = g->offsets->ptr;
    a.off64 = g->offsets->dtype == LLSA_I64;
    a.flat = (const int32_t*) g->flat->ptr;
    a.pairs = g->flat_pairs ? (const int32_t*) g->flat_pairs->ptr : nullptr;
    a.pds = g->fine_pds ? (uint4*) g->fine_pds->ptr : nullptr;
    a.ranges = g->flat_ranges ? (const int2*) g->flat_ranges->ptr : nullptr;
    a.range_entries = g->flat_ranges ? range_entries_of(a.nq1 * a.topk, g->flat_ranges->shape[2]) : kRangeEntries;
    a.kvw1 = g->kv_weight;
    a.kvw2 = g->kv_weight_2;
    a.fold = g->fold_pool_bwd;
  }
  return a;
}

}  // namespace llsa
