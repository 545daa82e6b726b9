/* llsa_b200 -- C ABI of the B200 (sm_100a) implementation of the LLSA
 * (log-linear sparse attention) hot path.
 *
 * Every entry point replaces one kernel group of the reference
 * (SingleZombie/LLSA, all Triton/Python); the reference file:line each one
 * stands in for is given beside it.  A Python caller binds these with ctypes
 * (llsa_b200/_lib.py); any other host language binds them the same way.
 *
 * Rules that hold for every function:
 *   - the caller owns all memory: inputs, outputs and scratch are device
 *     pointers passed in; unless stated otherwise nothing is allocated or freed
 *     here and no state is kept between calls;
 *   - work is enqueued on `stream` (a cudaStream_t passed as void*; NULL = the
 *     legacy default stream) and the call returns without synchronising;
 *   - the return value is 0 on success or a LLSA_ERR_* code; nothing throws.
 *     llsa_last_error_string() describes the last failure on this thread;
 *   - tensors are described by LlsaTensor: up to 4 dims, strides in ELEMENTS.
 *     Attention tensors are [B,H,N,D] with stride[3]==1 and 16-byte aligned
 *     rows; any batch/head/token strides are accepted (the model passes
 *     [B,H,N,D] views of [B,N,H,D] storage).
 */
#ifndef LLSA_B200_H_
#define LLSA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum LlsaDtype { LLSA_F32 = 0, LLSA_BF16 = 1, LLSA_I32 = 2, LLSA_I64 = 3 };

enum LlsaStatus {
  LLSA_OK = 0,
  LLSA_ERR_NULL = 1,        /* a required pointer is NULL                         */
  LLSA_ERR_DTYPE = 2,       /* unsupported or mismatching element types           */
  LLSA_ERR_SHAPE = 3,       /* shapes inconsistent or outside the supported set   */
  LLSA_ERR_STRIDE = 4,      /* innermost stride != 1, or rows not 16-byte aligned */
  LLSA_ERR_ARG = 5,         /* bad scalar argument (topk, block size, ...)        */
  LLSA_ERR_WORKSPACE = 6,   /* scratch buffer missing or too small                */
  LLSA_ERR_CUDA = 7,        /* a CUDA runtime call or kernel launch failed        */
  LLSA_ERR_DEVICE_CHECK = 8 /* a kernel set the caller's device status word: an out-of-range
                               index, or a bounded wait inside a kernel that ran out      */
};

/* Bits a kernel may set in a device status word (LlsaAttnArgs.status, the `status`
 * argument of the transpose).  The host reads the word after synchronising;
 * llsa_status_check() turns it into a return code. */
enum LlsaDeviceStatus {
  LLSA_DEV_BAD_INDEX = 1,    /* a block index outside [0, n) was met (and skipped or clamped) */
  LLSA_DEV_WAIT_EXPIRED = 2  /* a bounded wait on an mbarrier gave up; the CTA left its tiles
                                unfinished and the call's outputs are not valid               */
};

typedef struct LlsaTensor {
  void* ptr;
  int32_t dtype; /* LlsaDtype */
  int32_t ndim;
  int64_t shape[4];
  int64_t stride[4]; /* in elements */
} LlsaTensor;

int llsa_version(void);
const char* llsa_last_error_string(void);
/* LLSA_OK for a status word of 0, else LLSA_ERR_DEVICE_CHECK with the error string naming the bits
 * (`status_word` is the value the caller copied back from the device). */
int llsa_status_check(int32_t status_word);

/* ---- pooling: src/llsa/kernel/triton/mean_pool.py --------------------------
 * y[b,h,s,:] = (sum_{t<k} x[b,h,s*k+t,:]) / k with the sum accumulated
 * sequentially in x's dtype (mean_pool.py:26-30).  y is contiguous [B,H,S/k,C].
 * Replaces mean_pool1d / MeanPool1dFunction_BHSC.forward (mean_pool.py:129-148). */
int llsa_mean_pool_fwd(const LlsaTensor* x, const LlsaTensor* y, int k, void* stream);
/* dx[b,h,s*k+t,:] = dy[b,h,s,:] / k.  Replaces MeanPool1dFunction_BHSC.backward
 * (mean_pool.py:150-165). */
int llsa_mean_pool_bwd(const LlsaTensor* dy, const LlsaTensor* dx, int k, void* stream);
/* All pyramid levels of up to 3 tensors (q, k, v) in one pass over HBM:
 * y1[i] = pool(x[i], bs) and, when y2 != NULL, y2[i] = pool(y1[i], bs).  Replaces
 * the 3 (llsa_l1) or 6 (llsa_l2) mean_pool1d launches of
 * torch_op/flash_sparse_attention_res_1.py:42-44 and ..._res_2.py:49-55. */
int llsa_pool_pyramid_fwd(int n_tensors, const LlsaTensor* x, const LlsaTensor* y1, const LlsaTensor* y2,
                          int block_size, void* stream);
/* The same pass with the 2-D RoPE apply fused in front (north-star item "fused 2D RoPE apply on Q/K ahead of
 * pooling"): tensors whose bit is set in rope_mask (bit i = x[i]) are rotated by the [N,C] table `freq` (even
 * columns sin, odd columns cos; same dtype as x) exactly as llsa_rope_fwd does, the rotated rows are written to
 * xr[i] (x's shape, any strides) and the pyramid is pooled from the rotated values; the other tensors are pooled
 * as they are and their xr entry is ignored.  Replaces my_rope_fn on q and k (rope_dit_transformer_2d.py:232-238)
 * followed by the mean_pool1d launches, saving one read of q and k. */
int llsa_rope_pool_pyramid_fwd(int n_tensors, const LlsaTensor* x, const LlsaTensor* freq, int rope_mask, const LlsaTensor* xr,
                               const LlsaTensor* y1, const LlsaTensor* y2, int block_size, void* stream);

/* The same pass with the attention block's q / k RMSNorm fused in front of the rotation as well
 * (models/rope_dit_transformer_2d.py:215-238: norm_q / norm_k, then my_rope_fn, then llsa_l1 / llsa_l2 pools): tensors
 * whose bit is set in norm_mask are normalised over their C channels, y = T((x * rsqrt(mean(x^2) + eps)) * w) in fp32
 * with w = norm_weight[i] (F32 [C]; a NULL entry means ones), then rotated if their rope_mask bit is set (freq may be
 * NULL when rope_mask is 0), written to xr[i] and pooled.  One read of q and k instead of three.  The arithmetic is
 * that of llsa_rms_norm_fwd followed by llsa_rope_fwd and llsa_pool_pyramid_fwd, bit for bit. */
int llsa_rms_rope_pool_pyramid_fwd(int n_tensors, const LlsaTensor* x, const LlsaTensor* const* norm_weight, int norm_mask, float eps,
                                   const LlsaTensor* freq, int rope_mask, const LlsaTensor* xr, const LlsaTensor* y1,
                                   const LlsaTensor* y2, int block_size, void* stream);
/* RMSNorm over the last dimension of a [B,H,S,C] tensor (any batch/head/token strides), the q / k normalisation of the
 * reference's attention block (diffusers' RMSNorm as used at rope_dit_transformer_2d.py:215-218): fp32 sum of squares in
 * a fixed order, y = T((x * rsqrt(mean + eps)) * weight).  weight: F32 [C] or NULL (ones). */
int llsa_rms_norm_fwd(const LlsaTensor* x, const LlsaTensor* weight, float eps, const LlsaTensor* y, void* stream);

/* ---- RoPE: src/llsa/kernel/triton/rope.py ---------------------------------
 * Interleaved-pair rotation by a [S,D] table whose even columns are sin and odd
 * columns cos (rope.py:28-50); y has x's shape, any strides.  Replaces
 * MyRopeFunction.forward (rope.py:100-124) / .backward (rope.py:126-146). */
int llsa_rope_fwd(const LlsaTensor* x, const LlsaTensor* freq, const LlsaTensor* y, void* stream);
int llsa_rope_bwd(const LlsaTensor* dy, const LlsaTensor* freq, const LlsaTensor* dx, void* stream);

/* ---- selection: src/llsa/kernel/triton/topk.py ----------------------------
 * Coarse: idx[b,h,i,:] = top-`topk` columns of round_dtype(pq[b,h,i,:] . pk[b,h,:,:]^T),
 * descending, ties -> smallest index.  idx is I32 or I64 [B,H,M,topk].  Replaces
 * gen_sparse_indices (topk.py:6-9: torch.matmul + torch.topk). */
int llsa_coarse_topk(const LlsaTensor* pq, const LlsaTensor* pk, const LlsaTensor* idx, int topk, void* stream);
/* Refine: for level-1 query block i with parent P = i / bs the candidates are
 * the children p*bs .. p*bs+bs-1 of p in p_idx[b,h,P,:]; fp32 scores, top-`topk`,
 * descending, ties -> smallest block index.  Replaces compute_topk_indices_sparse
 * + _topk_indices_lastdim_k8_kernel (topk.py:102-197). */
int llsa_refine_topk(const LlsaTensor* pq1, const LlsaTensor* pk1, const LlsaTensor* p_idx, const LlsaTensor* idx,
                     int topk, int p_topk, int block_size, void* stream);

/* Both selections of the two-level operator in one launch where the shape allows it (bf16, D = 64, block 16, exactly 64
 * level-2 keys, p_topk <= 8): every CTA of the refine kernel first selects its own level-2 query block's parents, with the
 * arithmetic and tie rule of llsa_coarse_topk, writes them to p_idx and goes on to the refine step; otherwise the two
 * entry points above are called one after the other.  Outputs are those of llsa_coarse_topk(pq2, pk2) followed by
 * llsa_refine_topk, bit for bit.  Replaces gen_sparse_indices + compute_topk_indices_sparse as called at
 * torch_op/flash_sparse_attention_res_2.py:14-16. */
int llsa_select_two_level(const LlsaTensor* pq1, const LlsaTensor* pk1, const LlsaTensor* pq2, const LlsaTensor* pk2,
                          const LlsaTensor* p_idx, const LlsaTensor* idx, int topk, int p_topk, int block_size, void* stream);

/* ---- index transpose: src/llsa/kernel/triton/indices_transpose.py ---------
 * Query-major lists idx [B,H,M,T] (I32/I64, values in [0,n_kv)) -> KV-major CSR:
 * offsets [B,H,n_kv+1] (I32 or I64) and flat [B,H,M*T] (I32), each bucket in
 * ascending query order (a stable counting sort without atomics).  `scratch`
 * is llsa_transpose_scratch_bytes() bytes of device memory (may be NULL when
 * that returns 0); `status` is one int32 on the device, set non-zero if an
 * index is out of range (may be NULL).  Replaces transpose_indices =
 * _count_k_major + torch.cumsum + _k_major_indices (indices_transpose.py:6-109). */
size_t llsa_transpose_scratch_bytes(int64_t B, int64_t H, int64_t M, int64_t T, int64_t n_kv);
int llsa_transpose_indices(const LlsaTensor* idx, const LlsaTensor* offsets, const LlsaTensor* flat, int64_t n_kv,
                           void* scratch, size_t scratch_bytes, int32_t* status, void* stream);
/* The same transpose with two more lists for llsa_attn_bwd (the reference has the plain list only,
 * indices_transpose.py:70-78):
 *   pairs  [B,H,M*T] (I32): in the order of `flat`, the position m*T + t of each entry inside its head's idx
 *          (flat = pairs / T); finds what the query-major stage left for each (query block, selected block) pair;
 *   ranges [B,H,ceil(M*T/S),2] (I32), S = llsa_transpose_range_entries(B,H,M,T) (32, or 16 for problems too small to fill
 *          the GPU with 32; the tensor's length tells the library which): the entry list cut into the work ranges of
 *          the dK/dV kernel, (first entry, bucket of that entry) per range.  Range r nominally starts at entry S r;
 *          where that entry lies inside a bucket of at most S entries the range starts at the bucket's first entry
 *          instead, so that only longer buckets are ever split (at multiples of S).  Range r ends where r+1 starts. */
int llsa_transpose_range_entries(int64_t B, int64_t H, int64_t M, int64_t T);
int llsa_transpose_indices_pairs(const LlsaTensor* idx, const LlsaTensor* offsets, const LlsaTensor* flat, const LlsaTensor* pairs,
                                 const LlsaTensor* ranges, int64_t n_kv, void* scratch, size_t scratch_bytes, int32_t* status,
                                 void* stream);

/* The same transpose for hosts that cannot provide device scratch.  This entry
 * point has no counterpart in the reference: it exists for callers that never
 * get to call cudaMalloc themselves -- a process that handed the whole device to
 * its own memory arena at start-up, or a plugin runtime that only passes input
 * and output buffers across its boundary -- and that still need the
 * long-sequence case, where llsa_transpose_indices asks for scratch.
 *   - It allocates nothing.  The count table [B*H][32][n_kv] of 16-bit counters
 *     lives in an 8 MiB array built into the library, resident on every GPU that
 *     loads the library until the process exits.  B*H*32*n_kv*2 bytes must fit
 *     in those 8 MiB (e.g. B*H = 6 with n_kv = 16384, or B*H = 48 with
 *     n_kv = 2048); larger problems are refused with LLSA_ERR_WORKSPACE and must
 *     use llsa_transpose_indices with caller scratch.
 *   - The first call on a device looks up the array's device address (with that
 *     device current) and caches it; make that first call before any stream
 *     capture is started on the device.
 *   - All calls share the one array and it keeps the previous call's contents;
 *     the kernel clears the part it uses before counting.  Two calls whose
 *     kernels overlap on the GPU (different streams, or different threads on the
 *     same device) race on it: issue them on one stream or order them yourself.
 * Inputs and outputs are exactly those of llsa_transpose_indices. */
int llsa_transpose_indices_noalloc(const LlsaTensor* idx, const LlsaTensor* offsets, const LlsaTensor* flat, int64_t n_kv,
                                   int32_t* status, void* stream);

/* ---- attention ------------------------------------------------------------ */
typedef struct LlsaAttnArgs {
  /* forward operands */
  const LlsaTensor* q;   /* [B,H,N,D] */
  const LlsaTensor* k;
  const LlsaTensor* v;
  const LlsaTensor* pk;  /* [B,H,N/bs,D] contiguous rows */
  const LlsaTensor* pv;
  const LlsaTensor* pk2; /* [B,H,N/bs^2,D]; NULL selects the one-level form   */
  const LlsaTensor* pv2;
  const LlsaTensor* indices;   /* I32/I64 [B,H,N/bs,topk]                      */
  const LlsaTensor* p_indices; /* I32/I64 [B,H,N/bs^2,topk_p]; NULL for one level */
  const LlsaTensor* o;   /* out (fwd) / in (bwd): q's shape, any strides       */
  const LlsaTensor* lse; /* F32 [B,H,N] contiguous: out (fwd) / in (bwd)       */
  int32_t topk, topk_p, block_size;
  float token_weight, token_weight_2;
  /* backward only */
  const LlsaTensor* d_o;       /* upstream gradient, any strides               */
  const LlsaTensor* dq;        /* outputs, dtype of q                          */
  const LlsaTensor* dk;
  const LlsaTensor* dv;
  const LlsaTensor* offsets;   /* CSR of `indices`   (llsa_transpose_indices)  */
  const LlsaTensor* flat;
  const LlsaTensor* delta;     /* F32 [B,H,N] scratch                           */
  const LlsaTensor* dpk_acc;   /* F32 [B,H,N/bs,D] scratch+output: gradient of pk */
  const LlsaTensor* dpv_acc;
  const LlsaTensor* dpk2_acc;  /* F32 [B,H,N/bs^2,D]; NULL for one level        */
  const LlsaTensor* dpv2_acc;
  int32_t fold_pool_bwd;       /* 1: dk,dv include the pooling backward of the pooled-key
                                  gradients (what k.grad holds after llsa_l1/llsa_l2);
                                  0: dk,dv are the fine-token terms only         */
  float kv_weight, kv_weight_2;/* weights on the pooled dK/dV side; the reference's
                                  one-level backward uses 1 here (sparse_attention_res_1.py:389) */
  int32_t force_generic;       /* 1: use the plain FFMA kernels for any dtype   */
  int32_t stage_mask;          /* backward only; 0 = everything.  Otherwise a bit set of
                                  1: zero the *_acc tensors + delta + dq,  2: pooled-key
                                  gradients (and the pooled part of dq where the tcgen05
                                  kernels apply),  4: dk, dv -- to be issued in this order
                                  (lets a caller time the kernels separately, or build the CSR
                                  on another stream while 1 and 2 run) */
  const LlsaTensor* dkv_partial; /* backward, bf16 tensors only: F32 scratch
                                  of llsa_attn_bwd_partial_elems() elements for dK/dV tiles of KV
                                  blocks whose list of query blocks is split over several CTAs (not
                                  read before it is written; may be NULL for f32 tensors) */
  const LlsaTensor* fine_pds;  /* backward, bf16 tensors only: F32-typed scratch of
                                  llsa_attn_bwd_pds_elems() elements.  The dQ stage (stage_mask 1)
                                  leaves P and dS (bf16) of every (query block, selected block) pair
                                  here and the dK/dV stage (stage_mask 4) reads them instead of
                                  recomputing both from q, k, v, lse and delta */
  const LlsaTensor* flat_pairs;/* backward, bf16 tensors only: I32 [B,H,N/16*topk], the `pairs` list of
                                  llsa_transpose_indices_pairs for the same CSR as offsets / flat */
  const LlsaTensor* flat_ranges;/* backward, bf16 tensors only: I32 [B,H,ceil(N/16*topk/S),2], the `ranges`
                                  list of the same call */
  int32_t no_tcgen05;          /* 1: keep the pooled-key stages on the mma.sync kernels (the form used
                                  for shapes the tcgen05 kernels do not cover); for cross-checks */
  int32_t wait_limit;          /* 0: default.  Otherwise the number of polls after which a bounded
                                  mbarrier wait inside the tcgen05 kernels gives up (tests use a tiny
                                  value to exercise the give-up path; the kernel then returns
                                  normally with LLSA_DEV_WAIT_EXPIRED in *status) */
  int32_t* status;             /* device int32 or NULL: kernels OR LlsaDeviceStatus bits into it; the
                                  caller zeroes it, and reads it back after synchronising */
  const LlsaTensor* fwd_redo;  /* forward, optional: I32 scratch of at least B*H*N/4 elements (one byte per
                                  query row; not read before it is written).  With it, a pooled stage
                                  that walks a long pooled key list (more than 192 pooled keys per row)
                                  makes ONE pass over the keys with the fine part's log-sum-exp as the
                                  reference of its exponentials, marks here the rows whose pooled keys
                                  outweigh the fine ones by more than 1e30, and a second launch redoes
                                  exactly those rows with the exact two-pass form.  NULL: two passes for
                                  every row.  Same results either way up to rounding */
} LlsaAttnArgs;

/* Forward: o, lse.  One level (pk2 == NULL) replaces sparse_indices_attn_res_fwd
 * (sparse_attention_res_1.py:9-150); two levels replaces
 * sparse_indices_attn_res_2_2_fwd (sparse_attention_res_2.py:9-199). */
int llsa_attn_fwd(const LlsaAttnArgs* args, void* stream);
/* Backward: dq, dk, dv (+ pooled-key gradients in the *_acc tensors, which this
 * call zero-fills first).  Replaces sparse_indices_attn_res_scatter_bwd_v2
 * (sparse_attention_res_1.py:403-471) / ..._scatter_2_2_bwd_v2
 * (sparse_attention_res_2.py:578-681) and, with fold_pool_bwd, the
 * MeanPool1dFunction_BHSC.backward calls autograd runs after them. */
int llsa_attn_bwd(const LlsaAttnArgs* args, void* stream);
/* Element count of the F32 scratch tensor LlsaAttnArgs.dkv_partial that llsa_attn_bwd needs for bf16 tensors with
 * Nq query rows per (b,h) and `topk` selected blocks per query block (the caller allocates it; any 4-D contiguous
 * shape with at least this many elements is accepted).  The library itself never allocates device memory. */
int64_t llsa_attn_bwd_partial_elems(int64_t B, int64_t H, int64_t Nq, int32_t topk);
/* Element count (4-byte elements) of LlsaAttnArgs.fine_pds: 1 KB per (query block, selected block) pair. */
int64_t llsa_attn_bwd_pds_elems(int64_t B, int64_t H, int64_t Nq, int32_t topk);

#ifdef __cplusplus
}
#endif
#endif /* LLSA_B200_H_ */
