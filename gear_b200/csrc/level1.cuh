// Level 1 of the cumulative table from the per-partition aggregates, by one CTA.
//
//   l1[0] = 0, l1[p+1] = l1[p] + (double)aggregate(p), DEFINED as the in-order float64 sum.
//
// Float64 arithmetic is the scarce resource here (a B200 SM retires about two float64
// operations per clock: a TwoSum-checked parallel scan of 24,415 aggregates took 77 us on one
// SM), so the sums are formed in INTEGER arithmetic: the aggregates are float32, i.e. 24-bit
// integers times a power of two; on the common scale 2^(emin-150) of the smallest non-zero
// aggregate every prefix sum is an exact 64-bit integer, and it is turned into a float64 with
// shifts.  While every prefix sum fits 53 significant bits, the in-order float64 sum never
// rounds either and is that same number, bit for bit.  If the aggregates span too many binary
// orders for 64 bits, a prefix needs more than 53 bits, or an aggregate is not finite, thread 0
// repeats the sum strictly in order in float64 (GEARB_ST_L1_RESUMMED).
// Used by the scan's last CTA (scan.cu) and by the incremental update (update.cu).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "gear_b200.h"

namespace gearb {
namespace level1 {

// biased exponent with denormals counted as exponent 1, and the 24-bit significand
__device__ __forceinline__ unsigned expo(unsigned bits) {
  const unsigned e = (bits >> 23) & 0xffu;
  return e ? e : 1u;
}
__device__ __forceinline__ unsigned long long signif(unsigned bits) {
  return (bits & 0x7fffffu) | (((bits >> 23) & 0xffu) ? 0x800000u : 0u);
}

// The aggregate with bit pattern b (not +-0) as an integer on the scale 2^(emin - 150).
__device__ __forceinline__ unsigned long long scaled(unsigned b, unsigned emin) {
  return signif(b) << (expo(b) - emin);
}
// acc * 2^(emin - 150) as the bit pattern of a float64, exact or flagged.
__device__ __forceinline__ unsigned long long double_bits(unsigned long long acc, unsigned emin, bool &inexact) {
  if (!acc) return 0ull;
  const int top = 63 - __clzll(acc);  // index of the leading one
  unsigned long long frac;
  if (top > 52) {
    inexact |= (acc & ((1ull << (top - 52)) - 1ull)) != 0ull;
    frac = acc >> (top - 52);
  } else {
    frac = acc << (52 - top);
  }
  const unsigned long long biased = static_cast<unsigned long long>(top + static_cast<int>(emin) - 150 + 1023);
  return (biased << 52) | (frac & ((1ull << 52) - 1ull));
}
// nparts aggregates below 2^(24 + emax - emin) must sum below 2^63; exponent 255 stands for
// infinity, NaN or a negative aggregate.
__device__ __forceinline__ bool too_wide(unsigned emin, unsigned emax, unsigned nparts) {
  return emax >= 255u || (emax - emin) + 24u + (32u - __clz(nparts)) > 63u;
}
__device__ __forceinline__ void note_exponent(unsigned b, unsigned &emin, unsigned &emax) {
  if (b << 1) {  // not +-0
    const unsigned e = (b >> 31) ? 255u : expo(b);
    emin = min(emin, e);
    emax = max(emax, e);
  }
}
// Strictly in-order float64 sum by one thread: the definition itself, for the rare inputs the
// integer route cannot take.
__device__ inline void in_order(const float *agg, unsigned nparts, double *l1, int32_t *status,
                                double *mirror = nullptr) {
  double s = 0.0;
  if (l1) __stcg(&l1[0], 0.0);
  if (mirror) mirror[0] = 0.0;
  for (unsigned q = 0; q < nparts; ++q) {
    s = __dadd_rn(s, static_cast<double>(__ldcg(agg + q)));
    if (l1) __stcg(&l1[q + 1], s);
    if (mirror) mirror[q + 1] = s;
  }
  atomicOr(reinterpret_cast<unsigned *>(status), GEARB_ST_L1_RESUMMED);
}

constexpr int kTile = 16384;  // aggregates per shared-memory tile (64 KiB)

// Tile `t` of the aggregates into shared memory: 16-byte asynchronous copies, all of a thread's
// copies in flight at once (the array is padded to a multiple of 256 bytes, so the last copy of
// the last tile stays inside it).
__device__ __forceinline__ void load_tile(const float *agg, unsigned first, unsigned count, float *tile) {
  const unsigned quads = (count + 3u) / 4u;
  for (unsigned i = threadIdx.x; i < quads; i += blockDim.x) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(tile + 4 * i));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(agg + first + 4 * i) : "memory");
  }
  asm volatile("cp.async.wait_all;" ::: "memory");
  __syncthreads();
}

// Every thread of the CTA calls this (blockDim.x a multiple of 32, at most 1024).  `tile` is
// kTile floats of shared memory, 16-byte aligned, that nothing else uses meanwhile.  Each
// thread works on a contiguous run of the tile; the run length is odd, which spreads the
// threads' accesses over all banks.
// l1 (global memory) and mirror (nparts + 1 doubles of this CTA's shared memory) each receive
// the result when not null: a kernel whose CTAs all need level 1 lets every CTA build its own
// copy in shared memory and one of them write the global one.
__device__ inline void build(const float *agg, unsigned nparts, double *l1, int32_t *status, float *tile,
                             double *mirror = nullptr) {
  __shared__ unsigned long long warp_tot[32];
  __shared__ unsigned warp_emin[32], warp_emax[32];
  __shared__ unsigned long long tile_total;
  __shared__ int fallback;
  const unsigned kAll = 0xffffffffu;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
  if (tid == 0) fallback = 0;
  const unsigned ntiles = (nparts + kTile - 1) / kTile;

  // ---- exponent range of the non-zero aggregates
  unsigned emin = 0xffffffffu, emax = 0u;
  for (unsigned t = 0; t < ntiles; ++t) {
    const unsigned first = t * kTile, count = min(static_cast<unsigned>(kTile), nparts - first);
    load_tile(agg, first, count, tile);
    const unsigned run = ((count + blockDim.x - 1) / blockDim.x) | 1u;
    const unsigned lo = min(count, tid * run), hi = min(count, lo + run);
#pragma unroll 8
    for (unsigned q = lo; q < hi; ++q) {
      note_exponent(__float_as_uint(tile[q]), emin, emax);
    }
    if (ntiles > 1) __syncthreads();  // the tile is overwritten by the next one
  }
  emin = __reduce_min_sync(kAll, emin);
  emax = __reduce_max_sync(kAll, emax);
  if (lane == 0) {
    warp_emin[warp] = emin;
    warp_emax[warp] = emax;
  }
  __syncthreads();
  emin = 0xffffffffu;
  emax = 0u;
  for (int w = 0; w < nwarps; ++w) {
    emin = min(emin, warp_emin[w]);
    emax = max(emax, warp_emax[w]);
  }
  if (emax == 0u) emin = 1u;  // all zero
  const bool wide = too_wide(emin, emax, nparts);

  bool inexact = false;
  if (!wide) {
    unsigned long long carry = 0ull;  // sum of the tiles before this one
    for (unsigned t = 0; t < ntiles; ++t) {
      const unsigned first = t * kTile, count = min(static_cast<unsigned>(kTile), nparts - first);
      if (ntiles > 1) load_tile(agg, first, count, tile);  // a single tile is still there
      const unsigned run = ((count + blockDim.x - 1) / blockDim.x) | 1u;
      const unsigned lo = min(count, tid * run), hi = min(count, lo + run);
      unsigned long long sum = 0ull;
#pragma unroll 8
      for (unsigned q = lo; q < hi; ++q) {
        const unsigned b = __float_as_uint(tile[q]);
        if (b << 1) sum += scaled(b, emin);
      }
      unsigned long long incl = sum;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const unsigned long long o = __shfl_up_sync(kAll, incl, d);
        if (lane >= d) incl += o;
      }
      if (lane == 31) warp_tot[warp] = incl;
      __syncthreads();
      if (warp == 0) {
        unsigned long long w = lane < nwarps ? warp_tot[lane] : 0ull;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
          const unsigned long long o = __shfl_up_sync(kAll, w, d);
          if (lane >= d) w += o;
        }
        const unsigned long long before = __shfl_up_sync(kAll, w, 1);
        if (lane == 31) tile_total = w;  // lanes past the last warp hold zeros: this is the tile's sum
        warp_tot[lane] = lane == 0 ? 0ull : before;  // exclusive: the warps before this one
      }
      __syncthreads();
      const unsigned long long up = __shfl_up_sync(kAll, incl, 1);
      unsigned long long acc = carry + warp_tot[warp] + (lane == 0 ? 0ull : up);
#pragma unroll 4
      for (unsigned q = lo; q < hi; ++q) {
        const unsigned b = __float_as_uint(tile[q]);
        if (b << 1) acc += scaled(b, emin);
        const unsigned long long dbits = double_bits(acc, emin, inexact);
        if (l1) __stcg(reinterpret_cast<unsigned long long *>(l1) + first + q + 1, dbits);
        if (mirror) mirror[first + q + 1] = __longlong_as_double(static_cast<long long>(dbits));
      }
      carry += tile_total;
      __syncthreads();  // warp_tot and the tile are reused
    }
    if (tid == 0) {
      if (l1) __stcg(&l1[0], 0.0);
      if (mirror) mirror[0] = 0.0;
    }
  }
  if (wide || inexact) atomicOr(&fallback, 1);
  __syncthreads();
  if (fallback && tid == 0) in_order(agg, nparts, l1, status, mirror);
  if (mirror) __syncthreads();
}

}  // namespace level1
}  // namespace gearb
