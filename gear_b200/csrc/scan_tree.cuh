// The fixed addition tree of the level-2 cumulative table, one 512-value block per warp.
//
// It is written once here because three kernels must produce the same bits: the scan
// (scan.cu), the rescan of touched partitions (update.cu) and the sampling kernel that rebuilds
// a partition's entries on the fly instead of reading a stored table (sample_gather.cu).
//
//   chunk = 4 consecutive values: s0=x0, s1=s0+x1, s2=s1+x2, s3=s2+x3; T=s3
//   group = 4 consecutive chunks: g0=T0, g1=g0+T1, g2=g1+T2, g3=g2+T3
//   block = 32 consecutive groups (512 values): I = Hillis-Steele inclusive scan of g3 over
//           the groups; E = I of group q-1 (0 for q=0); block total = I of group 31
//   part  = 8 consecutive blocks: X(0)=0, X(w+1) = X(w) + total(w); X(8) is the partition's
//           AGGREGATE, the number level 1 is built from
//   chunk offset O = X + E for a group's first chunk, (X + E) + g(i-1) for its chunk i=1..3
//   value = O + s_j, then a running maximum over the partition (max is exact, so its order is
//           free) makes the table monotone.
//
// Data layout in the warp: lane l holds the float4 (= chunk) 32k + l of the block for
// k = 0..3, the ones it can fetch without a bank conflict.  The step to "four consecutive
// chunks per lane", which makes one shuffle scan per block enough, goes through a 128-float
// exchange area in shared memory that is private to the warp.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace gearb {
namespace tree {

constexpr unsigned kAll = 0xffffffffu;
constexpr int kBlockValues = 512;

__device__ __forceinline__ float hs_sum(float v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float t = __shfl_up_sync(kAll, v, d);
    if (lane >= d) v = __fadd_rn(t, v);
  }
  return v;
}
__device__ __forceinline__ float hs_max(float v, int lane) {
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float t = __shfl_up_sync(kAll, v, d);
    if (lane >= d) v = fmaxf(t, v);
  }
  return v;
}

// What a lane keeps of its block between the first pass and the second.
struct Group {
  float g0, g1, g2;  // running sums of the lane's four consecutive chunk totals (g3 is scanned)
  float E;           // sum of the groups before this lane's group
  float total;       // block total (the same in every lane)
};

// A priority is bad when its sign bit is set (negative, or -0.0) or it is NaN.  The check is
// folded into `bits`: the OR of all bit patterns seen, plus the sign bit when a block total is
// NaN (a NaN anywhere in a block survives into its total).  Bad <=> bits >> 31.
__device__ __forceinline__ void note_bits(const float4 (&x)[4], unsigned &bits) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    bits |= __float_as_uint(x[k].x) | __float_as_uint(x[k].y);
    bits |= __float_as_uint(x[k].z) | __float_as_uint(x[k].w);
  }
}
__device__ __forceinline__ void note_total(float total, unsigned &bits) {
  if (!(total == total)) bits |= 0x80000000u;
}

// First pass: chunk sums sv[k][0..3] of the lane's four chunks, group sums, scan over the block.
__device__ __forceinline__ Group block_sums(const float4 (&x)[4], float *xs, int lane, float (&sv)[4][4],
                                            unsigned &bits) {
  note_bits(x, bits);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    sv[k][0] = x[k].x;
    sv[k][1] = __fadd_rn(sv[k][0], x[k].y);
    sv[k][2] = __fadd_rn(sv[k][1], x[k].z);
    sv[k][3] = __fadd_rn(sv[k][2], x[k].w);
    xs[k * 32 + lane] = sv[k][3];
  }
  __syncwarp();
  const float4 t4 = reinterpret_cast<const float4 *>(xs)[lane];
  Group g;
  g.g0 = t4.x;
  g.g1 = __fadd_rn(g.g0, t4.y);
  g.g2 = __fadd_rn(g.g1, t4.z);
  const float g3 = __fadd_rn(g.g2, t4.w);
  const float I = hs_sum(g3, lane);
  const float up = __shfl_up_sync(kAll, I, 1);
  g.E = lane == 0 ? 0.f : up;
  g.total = __shfl_sync(kAll, I, 31);
  note_total(g.total, bits);
  return g;
}

// The block total alone (every lane gets it).  The last element of a Hillis-Steele scan is the
// balanced tree (lower half + upper half at every level), which a butterfly reduction computes
// in the lane that is the upper half at every level: lane 31.
__device__ __forceinline__ float block_total(const float4 (&x)[4], float *xs, int lane, unsigned &bits) {
  note_bits(x, bits);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    xs[k * 32 + lane] = __fadd_rn(__fadd_rn(__fadd_rn(x[k].x, x[k].y), x[k].z), x[k].w);
  __syncwarp();
  const float4 t4 = reinterpret_cast<const float4 *>(xs)[lane];
  float v = __fadd_rn(__fadd_rn(__fadd_rn(t4.x, t4.y), t4.z), t4.w);
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const float o = __shfl_xor_sync(kAll, v, d);
    v = (lane & d) ? __fadd_rn(o, v) : __fadd_rn(v, o);  // lower + upper either way
  }
  const float total = __shfl_sync(kAll, v, 31);
  note_total(total, bits);
  __syncwarp();  // the exchange area may be rewritten by the caller's next block
  return total;
}

// Second pass, given the block's offset X: makes sv the block's values (all of them, or with
// only_tops just sv[k][3]) and returns in top[k] the largest VALID value of each chunk.  e0 is
// the global index of the block's first value, n the number of priorities.
__device__ __forceinline__ void block_values(float X, const Group &g, float *xs, int lane, float (&sv)[4][4],
                                             float (&top)[4], bool only_tops, int64_t e0, int64_t n) {
  const float b0 = __fadd_rn(X, g.E);
  reinterpret_cast<float4 *>(xs)[lane] =
      make_float4(b0, __fadd_rn(b0, g.g0), __fadd_rn(b0, g.g1), __fadd_rn(b0, g.g2));
  __syncwarp();
  const bool whole = e0 + kBlockValues <= n;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float off = xs[k * 32 + lane];
    // An entry before which its chunk holds only zeros (running sum still 0) counts as 0: it takes
    // no part in any maximum and so repeats the running maximum before it bit for bit -- the
    // chunk's offset can be an ulp above the previous chunk's last value, and an entry of weight
    // zero must never be the first one greater than a variate.
    if (!only_tops || !whole) {
#pragma unroll
      for (int j = 0; j < 4; ++j) sv[k][j] = sv[k][j] == 0.f ? 0.f : __fadd_rn(off, sv[k][j]);
    } else {
      sv[k][3] = sv[k][3] == 0.f ? 0.f : __fadd_rn(off, sv[k][3]);
    }
    top[k] = sv[k][3];  // sums of non-negative terms do not decrease inside a chunk
    if (!whole) {       // entries past n take no part in any maximum (and are never stored)
      const int64_t e = e0 + (k * 32 + lane) * 4;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (e + j >= n) sv[k][j] = 0.f;
      top[k] = fmaxf(fmaxf(sv[k][0], sv[k][1]), fmaxf(sv[k][2], sv[k][3]));
    }
  }
}

// Largest value of the block (every lane gets it).
__device__ __forceinline__ float block_max(const float (&top)[4]) {
  float m = fmaxf(fmaxf(top[0], top[1]), fmaxf(top[2], top[3]));
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) m = fmaxf(m, __shfl_xor_sync(kAll, m, d));
  return m;
}

// Running maximum inside the block, the same two-step shape as the sums: leaves in xs[c] the
// largest value of the block BEFORE chunk c (0 for the first) and returns the block's largest.
// The caller combines xs[32k + lane] with the maximum of the blocks before this one.
__device__ __forceinline__ float block_prefix_max(const float (&top)[4], float *xs, int lane) {
#pragma unroll
  for (int k = 0; k < 4; ++k) xs[k * 32 + lane] = top[k];
  __syncwarp();
  const float4 m4 = reinterpret_cast<const float4 *>(xs)[lane];
  const float m0 = m4.x;
  const float m1 = fmaxf(m0, m4.y);
  const float m2 = fmaxf(m1, m4.z);
  const float m3 = fmaxf(m2, m4.w);
  const float M = hs_max(m3, lane);
  const float up = __shfl_up_sync(kAll, M, 1);
  const float pm0 = lane == 0 ? 0.f : up;
  reinterpret_cast<float4 *>(xs)[lane] = make_float4(pm0, fmaxf(pm0, m0), fmaxf(pm0, m1), fmaxf(pm0, m2));
  __syncwarp();
  return __shfl_sync(kAll, M, 31);
}

}  // namespace tree
}  // namespace gearb
