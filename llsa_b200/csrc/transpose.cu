// KV-block -> query-block index transpose used by the backward pass
// (reference: src/llsa/kernel/triton/indices_transpose.py).
//
// The reference builds the CSR with a global-atomic histogram, a cumsum and a
// second pass that claims slots with atomics, which leaves the order inside a
// bucket to chance (indices_transpose.py:23-27, :70-78).  Here one CTA per (b,h)
// runs a stable counting sort WITHOUT atomics:
//   1. the E = M*T entries are cut into W contiguous segments, one per warp; a
//      warp walks its segment 32 entries at a time, groups equal keys with
//      __match_any_sync and lets the lowest lane of each group add the group size
//      to the warp's own row of a [W][n_kv] count table;
//   2. every key's column of the table is turned into exclusive prefixes over the
//      segments and the column totals are scanned across keys -> offsets;
//   3. the warps walk their segments again; an entry lands at
//      offsets[key] + (count in earlier segments) + (count earlier in this segment)
//      + (rank inside its match group).
// Entries keep their original relative order, so every bucket lists its query
// blocks in ascending order and the output is bit-reproducible.
#include <mutex>

#include "common.cuh"

namespace llsa {

struct TransposeArgs {
  IdxView idx;      // [BH, M*T]
  void* offsets;    // [BH, n_kv+1]
  int off64;
  int32_t* flat;    // [BH, M*T]
  int32_t* pairs;   // [BH, M*T] or nullptr: entry position m*T + t in the order of `flat`
  int2* ranges;     // [BH, ceil(M*T / range_entries)] or nullptr: (first entry, its bucket) of the work ranges cut for the dK/dV kernel
  int range_entries;
  int64_t E;        // entries per head
  int T;
  int64_t n_kv;
  uint16_t* gtab;   // global table [BH][W][n_kv] or nullptr (shared memory)
  int32_t* status;
};

__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& block_total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  int inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int s = lane < nw ? warp_sums[lane] : 0;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, s, o);
      if (lane >= o) s += t;
    }
    warp_sums[lane] = s;  // inclusive over warps
  }
  __syncthreads();
  const int before = warp > 0 ? warp_sums[warp - 1] : 0;
  block_total = warp_sums[nw - 1];
  const int excl = before + inc - v;
  __syncthreads();  // warp_sums is reused by the next call
  return excl;
}

__global__ void __launch_bounds__(1024) transpose_kernel(TransposeArgs a) {
  extern __shared__ unsigned char smraw[];
  __shared__ int warp_sums[32];
  const int W = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t bh = blockIdx.x, n = a.n_kv, E = a.E;
  int* base = reinterpret_cast<int*>(smraw);                                        // [n_kv]
  uint16_t* tab = a.gtab ? a.gtab + bh * W * n : reinterpret_cast<uint16_t*>(base + n);  // [W][n_kv]

  for (int64_t i = threadIdx.x; i < (int64_t) W * n; i += blockDim.x) tab[i] = 0;
  __syncthreads();

  int64_t L = (E + W - 1) / W;
  L = (L + 31) / 32 * 32;
  const int64_t seg0 = min(E, warp * L), seg1 = min(E, seg0 + L);
  uint16_t* mytab = tab + (int64_t) warp * n;
  const unsigned lt_mask = (1u << lane) - 1u;

  // ---- 1: per-segment histograms
  for (int64_t e0 = seg0; e0 < seg1; e0 += 32) {
    const int64_t e = e0 + lane;
    bool valid = e < seg1;
    int64_t key = valid ? a.idx.at(bh * E + e) : -1;
    if (valid && (key < 0 || key >= n)) {
      if (a.status) atomicOr(a.status, (int) LLSA_DEV_BAD_INDEX);
      valid = false;
    }
    const unsigned act = __ballot_sync(0xffffffffu, valid);
    if (valid) {
      const unsigned peers = __match_any_sync(act, (int) key);
      if ((peers & lt_mask) == 0) mytab[key] = (uint16_t) (mytab[key] + __popc(peers));
    }
    __syncwarp();
  }
  __syncthreads();

  // ---- 2: per-key prefix over segments, then scan of the totals over keys
  int carry = 0;
  for (int64_t j0 = 0; j0 < n; j0 += blockDim.x) {
    const int64_t j = j0 + threadIdx.x;
    int run = 0;
    if (j < n) {
      for (int s = 0; s < W; ++s) {
        const int c = tab[(int64_t) s * n + j];
        tab[(int64_t) s * n + j] = (uint16_t) run;
        run += c;
      }
      // the prefixes are 16-bit: a key listed more than 65535 times in one head (possible only when rows repeat a key)
      // cannot be placed; the fill below then skips what would fall outside and the status word says so
      if (run > 65535 && a.status) atomicOr(a.status, (int) LLSA_DEV_BAD_INDEX);
    }
    int total;
    const int excl = block_exclusive_scan(run, warp_sums, total);
    if (j < n) {
      base[j] = carry + excl;
      if (a.off64) reinterpret_cast<int64_t*>(a.offsets)[bh * (n + 1) + j] = carry + excl;
      else reinterpret_cast<int32_t*>(a.offsets)[bh * (n + 1) + j] = carry + excl;
    }
    carry += total;
  }
  if (threadIdx.x == 0) {
    if (a.off64) reinterpret_cast<int64_t*>(a.offsets)[bh * (n + 1) + n] = carry;
    else reinterpret_cast<int32_t*>(a.offsets)[bh * (n + 1) + n] = carry;
  }
  __syncthreads();
  // ranges that lie wholly behind the last entry (entries were dropped, or E is not a multiple of the range size) are empty
  if (a.ranges) {
    const int64_t R = (E + a.range_entries - 1) / a.range_entries;
    for (int64_t r = threadIdx.x; r < R; r += blockDim.x)
      if (r * a.range_entries >= carry) a.ranges[bh * R + r] = make_int2(carry, (int) n - 1);
  }

  // ---- 3: stable fill
  const int total_entries = carry;          // every thread ran the same scan: entries that were kept
  for (int64_t e0 = seg0; e0 < seg1; e0 += 32) {
    const int64_t e = e0 + lane;
    bool valid = e < seg1;
    int64_t key = valid ? a.idx.at(bh * E + e) : -1;
    if (valid && (key < 0 || key >= n)) valid = false;
    const unsigned act = __ballot_sync(0xffffffffu, valid);
    unsigned peers = 0;
    int seen = 0;
    if (valid) {
      peers = __match_any_sync(act, (int) key);
      seen = mytab[key];
      const int pos = base[key] + seen + __popc(peers & lt_mask);
      if (pos < E) {
        a.flat[bh * E + pos] = (int32_t) (e / a.T);
        if (a.pairs) a.pairs[bh * E + pos] = (int32_t) e;
        // Work ranges of the dK/dV kernel: nominally S = range_entries entries each, but a bucket of at most S entries is
        // never cut -- the range that would begin inside it begins at the bucket's first entry instead (ranges then hold
        // 1 .. 2 S - 1 entries); only longer buckets are cut, at multiples of S.  The entry that lands on such a multiple knows
        // its bucket and that bucket's extent.
        if (a.ranges && pos % a.range_entries == 0) {
          const int S = a.range_entries, b0 = base[key], b1 = key + 1 < n ? base[key + 1] : total_entries;
          a.ranges[bh * ((E + S - 1) / S) + pos / S] = make_int2(b1 - b0 <= S ? b0 : pos, (int) key);
        }
      }
    }
    __syncwarp();
    if (valid && (peers & lt_mask) == 0) mytab[key] = (uint16_t) (seen + __popc(peers));
    __syncwarp();
  }
}

// Chooses the warp count W and where the [W][n_kv] count table lives.  Returns
// W (8, 16 or 32); *global is set when the table does not fit in shared memory
// or the segments would overflow the 16-bit counters with fewer warps.
static int plan_transpose(int64_t n_kv, int64_t E, size_t* smem, bool* global) {
  const size_t limit = 200 * 1024;
  for (int W = 32; W >= 8; W >>= 1) {
    const size_t need = (size_t) n_kv * 4 + (size_t) W * n_kv * 2;
    if (need <= limit && (E + W - 1) / W + 32 <= 65535) {
      *smem = need;
      *global = false;
      return W;
    }
  }
  *smem = (size_t) n_kv * 4;
  *global = true;
  return 32;
}

}  // namespace llsa

using namespace llsa;

extern "C" int llsa_transpose_range_entries(int64_t B, int64_t H, int64_t M, int64_t T) {
  const int64_t ranges = B * H * ((M * T + kRangeEntries - 1) / kRangeEntries);
  return ranges < 2 * 148 * 8 * 2 ? kRangeEntriesSmall : kRangeEntries;      // fewer than two rounds of the dK/dV kernel's resident warps
}

extern "C" size_t llsa_transpose_scratch_bytes(int64_t B, int64_t H, int64_t M, int64_t T, int64_t n_kv) {
  size_t smem;
  bool global;
  plan_transpose(n_kv, M * T, &smem, &global);
  return global ? (size_t) B * H * 32 * n_kv * 2 : 0;
}

static int transpose_impl(const LlsaTensor* idx, const LlsaTensor* offsets, const LlsaTensor* flat, const LlsaTensor* pairs,
                          const LlsaTensor* ranges, int64_t n_kv, void* scratch, size_t scratch_bytes, int32_t* status, void* stream) {
  LLSA_REQUIRE(idx && offsets && flat && idx->ptr && offsets->ptr && flat->ptr, LLSA_ERR_NULL, "transpose_indices: null tensor");
  LLSA_REQUIRE(idx->ndim == 4, LLSA_ERR_SHAPE, "transpose_indices: idx must be [B,H,M,T]");
  const int64_t B = idx->shape[0], H = idx->shape[1], M = idx->shape[2], T = idx->shape[3];
  LLSA_REQUIRE(is_index_dtype(idx->dtype) && is_index_dtype(offsets->dtype) && flat->dtype == LLSA_I32, LLSA_ERR_DTYPE,
               "transpose_indices: idx/offsets must be i32 or i64, flat i32");
  LLSA_REQUIRE(n_kv >= 1 && n_kv < (1ll << 31) && T >= 1, LLSA_ERR_ARG, "transpose_indices: bad n_kv=%lld", (long long) n_kv);
  const int64_t E = M * T;
  LLSA_REQUIRE(E <= 32ll * 65504, LLSA_ERR_SHAPE, "transpose_indices: M*T=%lld exceeds the supported %lld", (long long) E, 32ll * 65504);
  const int64_t si[4] = {B, H, M, T}, so[3] = {B, H, n_kv + 1}, sf[3] = {B, H, E};
  int rc;
  if ((rc = check_contig(idx, "idx", idx->dtype, 4, si))) return rc;
  if ((rc = check_contig(offsets, "offsets", offsets->dtype, 3, so))) return rc;
  if ((rc = check_contig(flat, "flat", LLSA_I32, 3, sf))) return rc;
  if (pairs && (rc = check_contig(pairs, "pairs", LLSA_I32, 3, sf))) return rc;
  int S = kRangeEntries;
  if (ranges) {
    LLSA_REQUIRE(ranges->ndim == 4, LLSA_ERR_SHAPE, "transpose_indices_pairs: ranges must be [B,H,R,2]");
    S = range_entries_of(E, ranges->shape[2]);
    LLSA_REQUIRE(S > 0, LLSA_ERR_SHAPE, "transpose_indices_pairs: ranges holds %lld ranges; expected ceil(%lld / %d) or ceil(%lld / %d)",
                 (long long) ranges->shape[2], (long long) E, kRangeEntries, (long long) E, kRangeEntriesSmall);
    const int64_t sr[4] = {B, H, (E + S - 1) / S, 2};
    if ((rc = check_contig(ranges, "ranges", LLSA_I32, 4, sr))) return rc;
  }
  // the per-key prefixes over the segments are 16-bit: with distinct keys inside a row a key occurs at most M times per head
  LLSA_REQUIRE(M <= 65535, LLSA_ERR_SHAPE, "transpose_indices: M=%lld query blocks per head exceed the supported 65535", (long long) M);
  if (B * H == 0) return LLSA_OK;
  size_t smem;
  bool global;
  const int W = plan_transpose(n_kv, E, &smem, &global);
  LLSA_REQUIRE(smem <= 200 * 1024, LLSA_ERR_SHAPE, "transpose_indices: n_kv=%lld too large", (long long) n_kv);
  TransposeArgs a;
  a.idx = make_idx(idx);
  a.offsets = offsets->ptr;
  a.off64 = offsets->dtype == LLSA_I64;
  a.flat = (int32_t*) flat->ptr;
  a.pairs = pairs ? (int32_t*) pairs->ptr : nullptr;
  a.ranges = ranges ? (int2*) ranges->ptr : nullptr;
  a.range_entries = S;
  a.E = E;
  a.T = (int) T;
  a.n_kv = n_kv;
  a.gtab = nullptr;
  a.status = status;
  if (global) {
    const size_t need = (size_t) B * H * 32 * n_kv * 2;
    LLSA_REQUIRE(scratch && scratch_bytes >= need, LLSA_ERR_WORKSPACE, "transpose_indices: needs %zu bytes of scratch", need);
    a.gtab = (uint16_t*) scratch;
  }
  // a segment holds at most 65535 entries, so the 16-bit counters cannot overflow
  LLSA_SMEM_LIMIT((transpose_kernel), smem);
  transpose_kernel<<<(unsigned) (B * H), W * 32, smem, (cudaStream_t) stream>>>(a);
  LLSA_LAUNCH_OK("transpose_kernel");
  return LLSA_OK;
}

extern "C" int llsa_transpose_indices(const LlsaTensor* idx, const LlsaTensor* offsets, const LlsaTensor* flat, int64_t n_kv,
                                      void* scratch, size_t scratch_bytes, int32_t* status, void* stream) {
  return transpose_impl(idx, offsets, flat, nullptr, nullptr, n_kv, scratch, scratch_bytes, status, stream);
}

extern "C" int llsa_transpose_indices_pairs(const LlsaTensor* idx, const LlsaTensor* offsets, const LlsaTensor* flat, const LlsaTensor* pairs,
                                            const LlsaTensor* ranges, int64_t n_kv, void* scratch, size_t scratch_bytes, int32_t* status,
                                            void* stream) {
  LLSA_REQUIRE(pairs && pairs->ptr && ranges && ranges->ptr, LLSA_ERR_NULL, "transpose_indices_pairs: null pairs / ranges tensor");
  return transpose_impl(idx, offsets, flat, pairs, ranges, n_kv, scratch, scratch_bytes, status, stream);
}

// ---------------------------------------------------------------------------
// llsa_transpose_indices_noalloc: the same index transpose for callers that
// cannot hand over a scratch buffer.
//
// Some hosts of this library never get to call cudaMalloc themselves: a
// serving or training process that gave the whole device to its own memory
// arena at start-up, or a plugin runtime that only passes input and output
// buffers across its boundary.  For the long-sequence shapes (n_kv above a few
// thousand KV blocks) llsa_transpose_indices needs B*H*32*n_kv*2 bytes of
// device scratch for its count table; here that table lives in a fixed array
// inside the library image instead.  Every GPU that loads the library carries
// the array (kNoAllocScratchBytes) until the process exits.
//
// The array's name is only a host-side handle: its device address is looked up
// once per device with cudaGetSymbolAddress (with that device current) and the
// address -- not the symbol -- is what the kernel receives.
namespace llsa {

constexpr size_t kNoAllocScratchBytes = 8u << 20;   // 8 MiB: e.g. B*H = 6 heads of 262144 tokens (n_kv = 16384)
static __device__ __align__(256) unsigned char g_transpose_scratch[kNoAllocScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_scratch_addr[kMaxDevices];   // device address of g_transpose_scratch, per device ordinal
static bool g_scratch_ready[kMaxDevices];
static std::mutex g_scratch_mutex;

// Device address of the static scratch on the CURRENT device (looked up on first use there).
static int noalloc_scratch(void** out) {
  int dev = -1;
  LLSA_CUDA_OK(cudaGetDevice(&dev));
  LLSA_REQUIRE(dev >= 0 && dev < kMaxDevices, LLSA_ERR_ARG, "transpose_indices_noalloc: device ordinal %d unsupported", dev);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ready[dev]) {
    void* p = nullptr;
    LLSA_CUDA_OK(cudaGetSymbolAddress(&p, g_transpose_scratch));
    LLSA_REQUIRE(p != nullptr, LLSA_ERR_CUDA, "transpose_indices_noalloc: no device address for the static scratch");
    g_scratch_addr[dev] = p;
    g_scratch_ready[dev] = true;
  }
  *out = g_scratch_addr[dev];
  return LLSA_OK;
}

}  // namespace llsa

extern "C" int llsa_transpose_indices_noalloc(const LlsaTensor* idx, const LlsaTensor* offsets, const LlsaTensor* flat, int64_t n_kv,
                                              int32_t* status, void* stream) {
  LLSA_REQUIRE(idx && offsets && flat && idx->ptr && offsets->ptr && flat->ptr, LLSA_ERR_NULL, "transpose_indices_noalloc: null tensor");
  LLSA_REQUIRE(idx->ndim == 4, LLSA_ERR_SHAPE, "transpose_indices_noalloc: idx must be [B,H,M,T]");
  const int64_t B = idx->shape[0], H = idx->shape[1], M = idx->shape[2], T = idx->shape[3];
  LLSA_REQUIRE(is_index_dtype(idx->dtype) && is_index_dtype(offsets->dtype) && flat->dtype == LLSA_I32, LLSA_ERR_DTYPE,
               "transpose_indices_noalloc: idx/offsets must be i32 or i64, flat i32");
  LLSA_REQUIRE(n_kv >= 1 && n_kv < (1ll << 31) && T >= 1, LLSA_ERR_ARG, "transpose_indices_noalloc: bad n_kv=%lld", (long long) n_kv);
  const int64_t E = M * T;
  LLSA_REQUIRE(E <= 32ll * 65504, LLSA_ERR_SHAPE, "transpose_indices_noalloc: M*T=%lld exceeds the supported %lld", (long long) E,
               32ll * 65504);
  const int64_t si[4] = {B, H, M, T}, so[3] = {B, H, n_kv + 1}, sf[3] = {B, H, E};
  int rc;
  if ((rc = check_contig(idx, "idx", idx->dtype, 4, si))) return rc;
  if ((rc = check_contig(offsets, "offsets", offsets->dtype, 3, so))) return rc;
  if ((rc = check_contig(flat, "flat", LLSA_I32, 3, sf))) return rc;
  // the count table [B*H][32 warps][n_kv] of 16-bit counters always goes to the static array
  const size_t need = (size_t) B * H * 32 * (size_t) n_kv * 2;
  LLSA_REQUIRE(need <= kNoAllocScratchBytes, LLSA_ERR_WORKSPACE,
               "transpose_indices_noalloc: B*H*n_kv = %lld needs %zu bytes of count table, the built-in scratch holds %zu "
               "(use llsa_transpose_indices with caller scratch)", (long long) (B * H * n_kv), need, (size_t) kNoAllocScratchBytes);
  const size_t smem = (size_t) n_kv * 4;   // per-key bases stay in shared memory
  LLSA_REQUIRE(smem <= 200 * 1024, LLSA_ERR_SHAPE, "transpose_indices_noalloc: n_kv=%lld too large", (long long) n_kv);
  LLSA_REQUIRE(M <= 65535, LLSA_ERR_SHAPE, "transpose_indices_noalloc: M=%lld query blocks per head exceed the supported 65535", (long long) M);
  if (B * H == 0) return LLSA_OK;
  void* tab = nullptr;
  if ((rc = noalloc_scratch(&tab))) return rc;
  TransposeArgs a;
  a.idx = make_idx(idx);
  a.offsets = offsets->ptr;
  a.off64 = offsets->dtype == LLSA_I64;
  a.flat = (int32_t*) flat->ptr;
  a.pairs = nullptr;
  a.ranges = nullptr;
  a.range_entries = kRangeEntries;
  a.E = E;
  a.T = (int) T;
  a.n_kv = n_kv;
  a.gtab = (uint16_t*) tab;     // the kernel zero-fills the part of the table it uses before counting
  a.status = status;
  LLSA_SMEM_LIMIT((transpose_kernel), smem);
  transpose_kernel<<<(unsigned) (B * H), 32 * 32, smem, (cudaStream_t) stream>>>(a);
  LLSA_LAUNCH_OK("transpose_kernel");
  return LLSA_OK;
}
