// Prioritized sample + gather in one launch.
//
// The reference does this in four steps with the host in between: sample
// (gear/sampler/global_sampler.py:93-152), partition (offline_loader.py:123-140),
// read the timesteps on the host (:168-177) and one fused_subcopy launch per
// column (:178-203).  Here one CTA serves one request end to end:
//   1. the whole CTA searches the two-level cumulative table for the request's
//      variate, 128 probes per round (two or three rounds per level);
//   2. the flat step index is decoded to GEAR's (trajectory, timestep, length);
//   3. the CTA's four warps copy the request's slots of every subscribed column.
// Results are identical to search_kernel + decode_kernel + gather_kernel run one
// after the other; only the launches and the index round trip through HBM go.
#include "common.h"
#include "device_copy.cuh"

namespace gearb {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr unsigned kFull = 0xffffffffu;

// First q in [lo, hi] with a[q] > v, given a[hi] > v; all kThreads threads take part.
template <typename T>
__device__ __forceinline__ int64_t block_upper_bound(const T *a, int64_t lo, int64_t hi, T v,
                                                     unsigned (*masks)[kWarps], int &round) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (;;) {
    const int64_t width = hi - lo + 1;
    const int64_t step = (width + kThreads - 1) / kThreads;
    int64_t q = lo + (tid + 1) * step - 1;
    if (q > hi) q = hi;
    const unsigned m = __ballot_sync(kFull, __ldg(a + q) > v);
    unsigned(&slot)[kWarps] = masks[round & 1];
    ++round;
    if (lane == 0) slot[warp] = m;
    __syncthreads();
    int first = kThreads - 1;  // the last thread probes hi, which is known to be greater
#pragma unroll
    for (int w = kWarps - 1; w >= 0; --w) {
      const unsigned mw = slot[w];
      if (mw) first = w * 32 + __ffs(mw) - 1;
    }
    int64_t qf = lo + (first + 1) * step - 1;
    if (qf > hi) qf = hi;
    if (first > 0) lo = lo + first * step;
    hi = qf;
    if (step == 1 || lo >= hi) return hi;
  }
}

struct SampleArgs {
  const float *cdf;
  const double *l1;
  const double *u;
  const int64_t *lengths;  // per-trajectory lengths or null
  int64_t *out_flat, *out_idx, *out_ts, *out_len;  // each may be null
  int64_t n, nparts, index_offset;
  int flags;
};

__global__ void __launch_bounds__(kThreads, 8)
sample_gather_kernel(const __grid_constant__ GatherParams P, const SampleArgs a) {
  __shared__ unsigned masks[2][kWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned flags = 0;
  int near_count = 0;
  int round = 0;
  const double total = __ldg(a.l1 + a.nparts);

  for (int64_t g = blockIdx.x; g < P.n; g += gridDim.x) {
    int64_t flat;
    if (!(total > 0.0)) {
      flat = a.n - 1;  // nothing selectable: defined as the last index
    } else {
      double v = __ldg(a.u + g);
      if (a.flags & GEARB_SEARCH_SCALE) v = __dmul_rn(v, total);
      if (!(v >= 0.0)) v = 0.0;
      if (!(v < total)) v = __longlong_as_double(__double_as_longlong(total) - 1);
      const int64_t p = block_upper_bound<double>(a.l1 + 1, 0, a.nparts - 1, v, masks, round);
      const int64_t base = p * GEARB_PART;
      const int64_t valid = (a.n - base < GEARB_PART) ? (a.n - base) : GEARB_PART;
      float r = __double2float_rn(__dsub_rn(v, __ldg(a.l1 + p)));
      const float last = __ldg(a.cdf + base + valid - 1);
      if (!(r < last)) r = __uint_as_float(__float_as_uint(last) - 1u);
      const int64_t j = block_upper_bound<float>(a.cdf + base, 0, valid - 1, r, masks, round);
      flat = base + j;
      if (threadIdx.x == 0 && P.status) {
        bool near = __uint_as_float(__float_as_uint(r) + 1u) >= __ldg(a.cdf + flat);
        if (j > 0 && r == __ldg(a.cdf + flat - 1)) near = true;
        near_count += near;
      }
    }
    const int64_t t = flat / P.T;
    const int64_t ts = flat - t * P.T;
    const int64_t len = a.lengths ? __ldg(a.lengths + t) : P.T;
    if (threadIdx.x == 0) {
      if (a.out_flat) a.out_flat[g] = flat;
      if (a.out_idx) a.out_idx[g] = t + a.index_offset;
      if (a.out_ts) a.out_ts[g] = ts;
      if (a.out_len) a.out_len[g] = len;
    }
    for (int q = warp; q < P.chunks_per_request; q += kWarps) {
      const int c = dev::column_of_piece(P, q);
      dev::gather_piece(P, P.cols[c], q - P.cols[c].chunk_first, g, t, ts, len, lane, flags);
    }
  }
  if (P.status) {
    if (flags && lane == 0) atomicOr(reinterpret_cast<unsigned *>(P.status), flags);
    if (near_count) atomicAdd(P.status + 1, near_count);
  }
}

}  // namespace

int launch_sample_gather(const GatherParams &p, const float *cdf, const double *l1, int64_t n,
                         const double *u, int flags, const int64_t *lengths, int64_t index_offset,
                         int64_t *out_flat, int64_t *out_idx, int64_t *out_ts, int64_t *out_len,
                         cudaStream_t stream) {
  GEARB_REQUIRE(n > 0, "sample_gather: the priority table is empty");
  if (p.n == 0) return GEARB_OK;
  GEARB_REQUIRE(cdf && l1 && u, "sample_gather: null pointer argument");
  SampleArgs a;
  a.cdf = cdf; a.l1 = l1; a.u = u; a.lengths = lengths;
  a.out_flat = out_flat; a.out_idx = out_idx; a.out_ts = out_ts; a.out_len = out_len;
  a.n = n; a.nparts = (n + GEARB_PART - 1) / GEARB_PART;
  a.index_offset = index_offset;
  a.flags = flags;
  int64_t grid = p.n;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (grid > cap) grid = cap;
  sample_gather_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(p, a);
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

}  // namespace gearb
