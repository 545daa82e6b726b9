// Register-direct operand fragments for mma.sync.m16n8k16 (bf16 in, fp32 out).
//
// Every tile the attention kernels multiply is 16 rows x 64 channels of bf16 with
// 128-byte rows.  Instead of staging tiles in shared memory and reading them back
// with ldmatrix, each lane loads its mma operand registers straight from global
// memory (L1/L2) with 128-bit loads, using the freedom to PERMUTE the contraction
// index: an m16n8k16 product only needs A and B to agree on which physical
// element sits at which logical k.
//
// Lane numbering: g = lane / 4 (0..7), t = lane % 4.
//
// * RowFrag -- "channel-contraction" layout, for products that sum over the 64
//   channels (S = Q.K^T, dP = dO.V^T).  Lane (g,t) holds, for row g of the tile,
//   the 16 channels [16t, 16t+16): ONE 256-bit load; the four lanes of a quad
//   cover the whole 128-byte row.  k-step s (0..3) uses registers r[2s]
//   (logical k = 2t,2t+1) and r[2s+1] (logical k = 2t+8,2t+9).
//   The same struct is the A operand (rows g and g+8 -> two RowFrags) and the B
//   operand (key n = g -> one RowFrag per 8 keys).
//
// * ColFrag -- "row-contraction" layout, for products that sum over the 16 rows
//   of the tile (O += P.V, dQ += dS.K, dV += P^T.dO, dK += dS^T.Q).  Lane (g,t)
//   loads channels [8g, 8g+8) of rows 2t, 2t+1, 2t+8, 2t+9 (four 128-bit loads,
//   eight lanes cover a whole 128-byte row) and builds the B registers of output
//   n-tile j with two byte permutes: n = g of tile j is channel 8g + j.
//   Consequently accumulator tile j holds channels 16t + j (c0/c2) and
//   16t + 8 + j (c1/c3): after the 8 tiles a lane owns the 16 CONSECUTIVE
//   channels [16t, 16t+16) of rows g and g+8, which it stores with 128-bit stores.
#pragma once
#include "common.cuh"

namespace llsa {

using bf16 = __nv_bfloat16;

struct RowFrag {
  uint32_t r[8];
};

// One 256-bit load (sm_100): lane (g,t) takes channels [16t, 16t+16) of its row, so the
// four lanes of a quad read one whole 128-byte row and a warp-wide load touches 8 lines.
// `row` must be 32-byte aligned.
__device__ __forceinline__ void load_rowfrag(RowFrag& f, const bf16* row, int t) {
  asm volatile("ld.global.ca.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(f.r[0]), "=r"(f.r[1]), "=r"(f.r[2]), "=r"(f.r[3]), "=r"(f.r[4]), "=r"(f.r[5]), "=r"(f.r[6]), "=r"(f.r[7])
               : "l"(row + 16 * t));
}

// The same load without an L1 allocation (L2 only): for kernels whose small L1 must keep other lines
__device__ __forceinline__ void load_rowfrag_cg(RowFrag& f, const bf16* row, int t) {
  asm volatile("ld.global.cg.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(f.r[0]), "=r"(f.r[1]), "=r"(f.r[2]), "=r"(f.r[3]), "=r"(f.r[4]), "=r"(f.r[5]), "=r"(f.r[6]), "=r"(f.r[7])
               : "l"(row + 16 * t));
}

// The same fragment from a shared-memory tile (rows padded to kSmemPitch elements).
constexpr int kSmemPitch = 72;   // 144 bytes: consecutive rows shift by 4 banks -> conflict-free 128-bit reads
__device__ __forceinline__ void load_rowfrag_smem(RowFrag& f, const bf16* row, int t) {
  const uint4 a = *reinterpret_cast<const uint4*>(row + 16 * t), b = *reinterpret_cast<const uint4*>(row + 16 * t + 8);
  f.r[0] = a.x; f.r[1] = a.y; f.r[2] = a.z; f.r[3] = a.w;
  f.r[4] = b.x; f.r[5] = b.y; f.r[6] = b.z; f.r[7] = b.w;
}

struct ColFrag {
  uint4 row[4];  // rows 2t, 2t+1, 2t+8, 2t+9; channels 8g..8g+7
};

__device__ __forceinline__ void load_colfrag(ColFrag& f, const bf16* tile, int64_t stride, int g, int t) {
  const bf16* p = tile + 8 * g;
  f.row[0] = ldg128(p + (int64_t) (2 * t) * stride);
  f.row[1] = ldg128(p + (int64_t) (2 * t + 1) * stride);
  f.row[2] = ldg128(p + (int64_t) (2 * t + 8) * stride);
  f.row[3] = ldg128(p + (int64_t) (2 * t + 9) * stride);
}

__device__ __forceinline__ void load_colfrag_smem(ColFrag& f, const bf16* tile, int g, int t) {
  const bf16* p = tile + 8 * g;
  f.row[0] = *reinterpret_cast<const uint4*>(p + (2 * t) * kSmemPitch);
  f.row[1] = *reinterpret_cast<const uint4*>(p + (2 * t + 1) * kSmemPitch);
  f.row[2] = *reinterpret_cast<const uint4*>(p + (2 * t + 8) * kSmemPitch);
  f.row[3] = *reinterpret_cast<const uint4*>(p + (2 * t + 9) * kSmemPitch);
}

// 16 bytes global -> shared without passing through registers
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = (uint32_t) __cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void cp_async_wait_group() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// ---- per-warp gather ring ------------------------------------------------------------------
// Gathered 16x64 tiles (selected K/V blocks, or the Q/dO blocks of a CSR entry) have a
// latency of well over a thousand cycles from L2/HBM; registers can hold one tile ahead at
// most.  Each warp therefore owns a small ring of stages in shared memory that it fills with
// cp.async several tiles ahead and drains with 128-bit ld.shared.  A stage holds two tiles of
// 2 KB (16 rows x 128 B, no padding); the 16-byte chunk c of row r sits at chunk c ^ (r & 7),
// which makes both fragment read patterns bank-conflict free.
constexpr int kRingTileElems = 16 * 64;          // one tile, in bf16 elements

// The 32 lanes copy two tiles (A rows: a + r*sa, B rows: b + r*sb) into one stage: 8 chunks per lane.
__device__ __forceinline__ void ring_issue(bf16* stage, const bf16* a, int64_t sa, const bf16* b, int64_t sb, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int idx = i * 32 + lane, tile = idx >> 7, r = (idx >> 3) & 15, c = idx & 7;
    const bf16* src = (tile ? b + (int64_t) r * sb : a + (int64_t) r * sa) + c * 8;
    cp_async16(stage + tile * kRingTileElems + r * 64 + ((c ^ (r & 7)) << 3), src);
  }
}

__device__ __forceinline__ void load_rowfrag_ring(RowFrag& f, const bf16* tile, int r, int t) {
  const bf16* row = tile + r * 64;
  const uint4 a = *reinterpret_cast<const uint4*>(row + (((2 * t) ^ (r & 7)) << 3));
  const uint4 b = *reinterpret_cast<const uint4*>(row + (((2 * t + 1) ^ (r & 7)) << 3));
  f.r[0] = a.x; f.r[1] = a.y; f.r[2] = a.z; f.r[3] = a.w;
  f.r[4] = b.x; f.r[5] = b.y; f.r[6] = b.z; f.r[7] = b.w;
}

__device__ __forceinline__ void load_colfrag_ring(ColFrag& f, const bf16* tile, int g, int t) {
  const int r0 = 2 * t, r1 = 2 * t + 1, r2 = 2 * t + 8, r3 = 2 * t + 9;
  f.row[0] = *reinterpret_cast<const uint4*>(tile + r0 * 64 + ((g ^ (r0 & 7)) << 3));
  f.row[1] = *reinterpret_cast<const uint4*>(tile + r1 * 64 + ((g ^ (r1 & 7)) << 3));
  f.row[2] = *reinterpret_cast<const uint4*>(tile + r2 * 64 + ((g ^ (r2 & 7)) << 3));
  f.row[3] = *reinterpret_cast<const uint4*>(tile + r3 * 64 + ((g ^ (r3 & 7)) << 3));
}

// Shared-memory accesses as [32-bit shared address + compile-time offset]: the per-lane part of every address is computed
// once per kernel, the stage / tile / row part is an immediate, and the entry loop spends no integer instruction on them.
template <int IMM>
__device__ __forceinline__ void ldsm_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t sa) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(sa), "n"(IMM));
}
template <int IMM>
__device__ __forceinline__ void lds128(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, uint32_t sa) {
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4+%5];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(sa), "n"(IMM));
}
template <int IMM>
__device__ __forceinline__ void sts128(uint32_t sa, const uint4& v) {
  asm volatile("st.shared.v4.b32 [%0+%1], {%2,%3,%4,%5};" ::"r"(sa), "n"(IMM), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
template <int IMM>
__device__ __forceinline__ float2 lds64f(uint32_t sa) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2+%3];" : "=f"(v.x), "=f"(v.y) : "r"(sa), "n"(IMM));
  return v;
}
template <int IMM>
__device__ __forceinline__ void cp_async16_sa(uint32_t sa, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0+%1], [%2], 16;" ::"r"(sa), "n"(IMM), "l"(gsrc) : "memory");
}
// RowFrag of tile row (g or g+8: ROWOFF) from a swizzled ring tile: chunks 2t and 2t+1 of the row sit at sa0 / sa1
template <int IMM>
__device__ __forceinline__ void rowfrag_sa(RowFrag& f, uint32_t sa0, uint32_t sa1) {
  lds128<IMM>(f.r[0], f.r[1], f.r[2], f.r[3], sa0);
  lds128<IMM>(f.r[4], f.r[5], f.r[6], f.r[7], sa1);
}
template <int IMM>
__device__ __forceinline__ void stsm_x4(uint32_t sa, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0+%1], {%2,%3,%4,%5};" ::"r"(sa), "n"(IMM), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}

// D = A.B (no accumulator input: the zero is the hardware zero register, not sixteen moves per entry)
__device__ __forceinline__ void mma_bf16_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
// Half of mma_rows_x_keys straight from a ring tile at byte offset IMM: the 128-bit chunk at `sa` (row g) and at sa + 1024 (row g + 8)
// carries k-steps 0, 1 (FIRST, which also initialises the accumulators) or 2, 3 of the channel contraction.
template <int IMM, bool FIRST>
__device__ __forceinline__ void half_rows_x_keys(float (&s0)[4], float (&s1)[4], const RowFrag& alo, const RowFrag& ahi, uint32_t sa) {
  uint32_t x0[4], x1[4];
  lds128<IMM>(x0[0], x0[1], x0[2], x0[3], sa);
  lds128<IMM + 1024>(x1[0], x1[1], x1[2], x1[3], sa);
  constexpr int o = FIRST ? 0 : 4;
  if (FIRST) {
    mma_bf16_16816_z(s0, alo.r[0], ahi.r[0], alo.r[1], ahi.r[1], x0[0], x0[1]);
    mma_bf16_16816_z(s1, alo.r[0], ahi.r[0], alo.r[1], ahi.r[1], x1[0], x1[1]);
  } else {
    mma_bf16_16816(s0, alo.r[o], ahi.r[o], alo.r[o + 1], ahi.r[o + 1], x0[0], x0[1]);
    mma_bf16_16816(s1, alo.r[o], ahi.r[o], alo.r[o + 1], ahi.r[o + 1], x1[0], x1[1]);
  }
  mma_bf16_16816(s0, alo.r[o + 2], ahi.r[o + 2], alo.r[o + 3], ahi.r[o + 3], x0[2], x0[3]);
  mma_bf16_16816(s1, alo.r[o + 2], ahi.r[o + 2], alo.r[o + 3], ahi.r[o + 3], x1[2], x1[3]);
}

__device__ __forceinline__ void mma_rows_x_keys_z(float (&s0)[4], float (&s1)[4], const RowFrag& alo, const RowFrag& ahi, const RowFrag& k0,
                                                  const RowFrag& k1) {
  mma_bf16_16816_z(s0, alo.r[0], ahi.r[0], alo.r[1], ahi.r[1], k0.r[0], k0.r[1]);
  mma_bf16_16816_z(s1, alo.r[0], ahi.r[0], alo.r[1], ahi.r[1], k1.r[0], k1.r[1]);
#pragma unroll
  for (int s = 1; s < 4; ++s) {
    mma_bf16_16816(s0, alo.r[2 * s], ahi.r[2 * s], alo.r[2 * s + 1], ahi.r[2 * s + 1], k0.r[2 * s], k0.r[2 * s + 1]);
    mma_bf16_16816(s1, alo.r[2 * s], ahi.r[2 * s], alo.r[2 * s + 1], ahi.r[2 * s + 1], k1.r[2 * s], k1.r[2 * s + 1]);
  }
}

// Pulls the 16 rows of a tile (128 bytes each) towards L1 without using registers:
// lanes 0..15 of `lane16` each touch one row.
__device__ __forceinline__ void prefetch_tile_rows(const bf16* tile, int64_t stride, int lane16) {
  asm volatile("prefetch.global.L1 [%0];" ::"l"(tile + (int64_t) lane16 * stride));
}

__device__ __forceinline__ uint32_t u4_get(const uint4& v, int m) { return m == 0 ? v.x : (m == 1 ? v.y : (m == 2 ? v.z : v.w)); }

// B registers of output tile j (compile-time j under full unrolling)
__device__ __forceinline__ void colfrag_b(const ColFrag& f, int j, uint32_t& b0, uint32_t& b1) {
  const int m = j >> 1;
  const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
  b0 = __byte_perm(u4_get(f.row[0], m), u4_get(f.row[1], m), sel);
  b1 = __byte_perm(u4_get(f.row[2], m), u4_get(f.row[3], m), sel);
}

// acc[0..1] (16 x 16 keys, two n-tiles) += A(rows g / g+8) . B(keys)^T over the 64 channels
__device__ __forceinline__ void mma_rows_x_keys(float (&s0)[4], float (&s1)[4], const RowFrag& alo, const RowFrag& ahi, const RowFrag& k0,
                                                const RowFrag& k1) {
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    mma_bf16_16816(s0, alo.r[2 * s], ahi.r[2 * s], alo.r[2 * s + 1], ahi.r[2 * s + 1], k0.r[2 * s], k0.r[2 * s + 1]);
    mma_bf16_16816(s1, alo.r[2 * s], ahi.r[2 * s], alo.r[2 * s + 1], ahi.r[2 * s + 1], k1.r[2 * s], k1.r[2 * s + 1]);
  }
}

// acc (16 x 64, eight n-tiles) += A(16 x 16, given as the four A registers) . tile(16 rows x 64 channels)
__device__ __forceinline__ void mma_x_cols(float (&acc)[8][4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, const ColFrag& f) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint32_t b0, b1;
    colfrag_b(f, j, b0, b1);
    mma_bf16_16816(acc[j], a0, a1, a2, a3, b0, b1);
  }
}

// ---- row-contraction operand from a RowFrag pair, without a second load ------------------------
// movmatrix transposes the 8x8 b16 matrix a warp holds one register per lane.  Register i of a
// RowFrag is the matrix M_i[row][c] = tile[row][16*(c/2) + 2i + c%2]; transposed, lane (g,t)
// holds tile[rows 2t,2t+1][channel 16*(g/2) + 2i + g%2]: exactly a B register whose n-slot g is
// that channel.  With `lo` = rows 0..7 and `hi` = rows 8..15 of the tile this gives b0 / b1 of
// output tile i, whose accumulators c0,c1 (c2,c3) are channels 16t + 2i, 16t + 2i + 1 of rows
// g (g + 8): again 16 consecutive channels per lane, in the order acc[0][0], acc[0][1], acc[1][0] ...
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

// acc (16 x 64) += A(16 x 16 as four A registers) . tile(16 rows x 64 channels given as its RowFrag pair)
__device__ __forceinline__ void mma_x_rowfrag_t(float (&acc)[8][4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, const RowFrag& lo,
                                                const RowFrag& hi) {
#pragma unroll
  for (int i = 0; i < 8; ++i) mma_bf16_16816(acc[i], a0, a1, a2, a3, movmatrix_trans(lo.r[i]), movmatrix_trans(hi.r[i]));
}

// Channel of accumulator acc[u][e] (e = 0/1, or 2/3 for row g+8) inside the lane's 16 channels, for
// tiles produced by mma_x_rowfrag_t: 2u + e.  Stores one row (ROW 0: c0/c1, ROW 1: c2/c3) as bf16.
template <int ROW>
__device__ __forceinline__ void store_acc_row_t(bf16* row, const float (&acc)[8][4], int t, float mul) {
  constexpr int lo = ROW * 2, hi = ROW * 2 + 1;
  uint4 x, y;
  x.x = pack_bf16(acc[0][lo] * mul, acc[0][hi] * mul); x.y = pack_bf16(acc[1][lo] * mul, acc[1][hi] * mul);
  x.z = pack_bf16(acc[2][lo] * mul, acc[2][hi] * mul); x.w = pack_bf16(acc[3][lo] * mul, acc[3][hi] * mul);
  y.x = pack_bf16(acc[4][lo] * mul, acc[4][hi] * mul); y.y = pack_bf16(acc[5][lo] * mul, acc[5][hi] * mul);
  y.z = pack_bf16(acc[6][lo] * mul, acc[6][hi] * mul); y.w = pack_bf16(acc[7][lo] * mul, acc[7][hi] * mul);
  *reinterpret_cast<uint4*>(row + 16 * t) = x;
  *reinterpret_cast<uint4*>(row + 16 * t + 8) = y;
}

// max of three in one instruction (sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float quad_max(float v) {
  v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
  return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// Stores the 16 consecutive channels [16t, 16t+16) a lane owns for one row (ROW 0: c0/c1, ROW 1: c2/c3)
template <int ROW>
__device__ __forceinline__ void store_acc_row(bf16* row, const float (&acc)[8][4], int t, float mul) {
  constexpr int lo = ROW * 2, hi = ROW * 2 + 1;
  uint4 x, y;
  x.x = pack_bf16(acc[0][lo] * mul, acc[1][lo] * mul); x.y = pack_bf16(acc[2][lo] * mul, acc[3][lo] * mul);
  x.z = pack_bf16(acc[4][lo] * mul, acc[5][lo] * mul); x.w = pack_bf16(acc[6][lo] * mul, acc[7][lo] * mul);
  y.x = pack_bf16(acc[0][hi] * mul, acc[1][hi] * mul); y.y = pack_bf16(acc[2][hi] * mul, acc[3][hi] * mul);
  y.z = pack_bf16(acc[4][hi] * mul, acc[5][hi] * mul); y.w = pack_bf16(acc[6][hi] * mul, acc[7][hi] * mul);
  *reinterpret_cast<uint4*>(row + 16 * t) = x;
  *reinterpret_cast<uint4*>(row + 16 * t + 8) = y;
}

__device__ __forceinline__ void red_add_v4(float* p, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// Adds the same 16 channels of one row into an fp32 row in global memory with four 128-bit reductions
template <int ROW>
__device__ __forceinline__ void red_acc_row(float* row, const float (&acc)[8][4], int t, float mul) {
  constexpr int lo = ROW * 2, hi = ROW * 2 + 1;
  float* p = row + 16 * t;
  red_add_v4(p, acc[0][lo] * mul, acc[1][lo] * mul, acc[2][lo] * mul, acc[3][lo] * mul);
  red_add_v4(p + 4, acc[4][lo] * mul, acc[5][lo] * mul, acc[6][lo] * mul, acc[7][lo] * mul);
  red_add_v4(p + 8, acc[0][hi] * mul, acc[1][hi] * mul, acc[2][hi] * mul, acc[3][hi] * mul);
  red_add_v4(p + 12, acc[4][hi] * mul, acc[5][hi] * mul, acc[6][hi] * mul, acc[7][hi] * mul);
}

// The same for tiles produced by mma_x_rowfrag_t (acc[u][e] = channel 16t + 2u + e)
template <int ROW>
__device__ __forceinline__ void red_acc_row_t(float* row, const float (&acc)[8][4], int t, float mul) {
  constexpr int lo = ROW * 2, hi = ROW * 2 + 1;
  float* p = row + 16 * t;
#pragma unroll
  for (int u = 0; u < 8; u += 2)
    red_add_v4(p + 2 * u, acc[u][lo] * mul, acc[u][hi] * mul, acc[u + 1][lo] * mul, acc[u + 1][hi] * mul);
}

}  // namespace llsa
