// Warp-cooperative "first entry greater than v" over a sorted array, 256-fold per round.
#pragma once
#include <cstdint>

namespace gearb {

struct LoadReadOnly {  // data that no kernel running now writes
  template <typename T>
  __device__ __forceinline__ T operator()(const T *p) const { return __ldg(p); }
};
struct LoadL2 {  // data written earlier in this same kernel by other CTAs (made visible by a fence + flag)
  template <typename T>
  __device__ __forceinline__ T operator()(const T *p) const { return __ldcg(p); }
};
struct LoadPlain {  // shared memory, or anything else an ordinary load serves
  template <typename T>
  __device__ __forceinline__ T operator()(const T *p) const { return *p; }
};

// First q in [lo, hi] with a[q] > v, given a[hi] > v.  Slot s of a round probes
// lo + (s+1)*step - 1 (clamped to hi); lane l takes slots l, l+32, ..., so that the probes of a
// round with step 1 are consecutive across the lanes.  Eight probes per lane and round, all in
// flight together.
template <typename T, typename Load>
__device__ __forceinline__ int64_t warp_upper_bound(const T *a, int64_t lo, int64_t hi, T v, int lane, Load ld) {
  constexpr unsigned kAll = 0xffffffffu;
  constexpr int kPer = 8;
  for (;;) {
    const int64_t width = hi - lo + 1;
    if (width <= 32) {  // one probe per lane finishes it
      int64_t q = lo + lane;
      if (q > hi) q = hi;
      const unsigned m = __ballot_sync(kAll, ld(a + q) > v);  // never 0: a[hi] > v
      return lo + (__ffs(m) - 1);
    }
    const int64_t step = (width + 32 * kPer - 1) / (32 * kPer);
    T x[kPer];
#pragma unroll
    for (int k = 0; k < kPer; ++k) {
      int64_t q = lo + (static_cast<int64_t>(k * 32 + lane) + 1) * step - 1;
      if (q > hi) q = hi;
      x[k] = ld(a + q);
    }
    int first = 32 * kPer - 1;  // the last slot probes hi, whose entry is greater
#pragma unroll
    for (int k = kPer - 1; k >= 0; --k) {
      const unsigned m = __ballot_sync(kAll, x[k] > v);
      if (m) first = k * 32 + __ffs(m) - 1;
    }
    int64_t qf = lo + (static_cast<int64_t>(first) + 1) * step - 1;
    if (qf > hi) qf = hi;
    if (first > 0) lo = lo + static_cast<int64_t>(first) * step;  // one past the previous slot's probe
    hi = qf;
    if (step == 1 || lo >= hi) return hi;
  }
}

}  // namespace gearb
