// Incremental priority update: write m new priorities, rescan only the partitions they fall
// into, and rebuild the float64 partition offsets.
//
// In prioritized replay a training step changes the priorities of the batch it just used
// (the reference's Indexset::set_weight, include/index/set.h:245-247, and its
// WeightUpdateRequestArray, src/index/request.cc:41-75, are that interface on the host).  A full
// rescan moves 8 bytes per priority; an update of m entries touches at most m partitions of
// 4096, so this path moves m x 32 KiB plus 8 bytes per partition for level 1 -- 34 MB instead
// of 800 MB for m = 1024 at 1e8 priorities.
//
// The results are bit-identical to a full scan of the updated priorities: a rescanned partition
// goes through the same addition tree as scan_kernel (scan.cu), and level 1 is the same
// in-order float64 sum (computed in parallel with every addition checked for exactness, and
// re-done strictly in order if one of them rounded).
//
//   mark_kernel     priorities[idx[i]] = value[i]; each touched partition enters a list once
//   rescan_kernel   one CTA per listed partition: load, scan, store cdf and the aggregate word
//   level1_kernel   one CTA: offsets from all aggregate words; clears the list for the next call
#include "common.h"
#include "scan_tree.cuh"

namespace gearb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPart = GEARB_PART;
constexpr unsigned kFull = 0xffffffffu;
static_assert(kWarps * tree::kBlockValues == kPart, "one warp per block of the partition");

__device__ __forceinline__ double checked_add(double a, double b, bool &inexact) {
  const double s = __dadd_rn(a, b);
  const double bb = __dsub_rn(s, a);
  const double err = __dadd_rn(__dsub_rn(a, __dsub_rn(s, bb)), __dsub_rn(b, bb));
  inexact |= (err != 0.0);
  return s;
}

__global__ void mark_kernel(float *prio, int64_t n, const int64_t *idx, const float *val, int64_t m,
                            unsigned *dirty, unsigned *list, unsigned *count, int32_t *status) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= m) return;
  const int64_t k = idx[i];
  if (k < 0 || k >= n) {
    atomicOr(reinterpret_cast<unsigned *>(status), GEARB_ST_BAD_REQUEST);
    return;
  }
  const float v = val[i];
  if (!(v >= 0.f)) atomicOr(reinterpret_cast<unsigned *>(status), GEARB_ST_BAD_PRIORITY);
  prio[k] = v;  // two updates of one index in a batch: one of them wins, as with any scatter
  const unsigned p = static_cast<unsigned>(k / kPart);
  if (atomicExch(&dirty[p], 1u) == 0u) list[atomicAdd(count, 1u)] = p;
}

// Same tree as the compute warps of scan_kernel (scan_tree.cuh): warp w scans block w.
// cdf == nullptr: the table is kept without its level-2 entries, only the aggregate is redone.
__global__ void __launch_bounds__(kThreads) rescan_kernel(const float *prio, int64_t n, float *cdf,
                                                          unsigned long long *aggw, const unsigned *list,
                                                          const unsigned *count, unsigned *dirty) {
  __shared__ float wt[kWarps], wm[kWarps];
  __shared__ __align__(16) float xs_all[kWarps][128];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float *xs = xs_all[warp];
  const unsigned total = *count;
  bool bad = false;  // priorities were checked when they were written (mark_kernel)
  for (unsigned li = blockIdx.x; li < total; li += gridDim.x) {
    const unsigned p = list[li];
    const int64_t base = static_cast<int64_t>(p) * kPart;
    const int64_t e0 = base + warp * tree::kBlockValues;
    float4 x[4];
    float sv[4][4], top[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int64_t e = e0 + (k * 32 + lane) * 4;
      if (e + 4 <= n) {
        x[k] = *reinterpret_cast<const float4 *>(prio + e);
      } else {
        x[k].x = (e + 0 < n) ? prio[e + 0] : 0.f;
        x[k].y = (e + 1 < n) ? prio[e + 1] : 0.f;
        x[k].z = (e + 2 < n) ? prio[e + 2] : 0.f;
        x[k].w = (e + 3 < n) ? prio[e + 3] : 0.f;
      }
    }
    const tree::Group g = tree::block_sums(x, xs, lane, sv, bad);
    if (lane == 0) wt[warp] = g.total;
    __syncthreads();
    float X = 0.f;
    for (int w = 0; w < warp; ++w) X = __fadd_rn(X, wt[w]);
    tree::block_values(X, g, xs, lane, sv, top, cdf == nullptr, e0, n);
    float G = 0.f, run;
    if (cdf == nullptr) {
      run = tree::block_max(top);
      if (lane == 0) wm[warp] = run;
      __syncthreads();
      for (int w = 0; w < warp; ++w) G = fmaxf(G, wm[w]);
    } else {
      run = tree::block_prefix_max(top, xs, lane);
      if (lane == 0) wm[warp] = run;
      __syncthreads();
      for (int w = 0; w < warp; ++w) G = fmaxf(G, wm[w]);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float m = fmaxf(G, xs[k * 32 + lane]);
        const int64_t e = e0 + (k * 32 + lane) * 4;
        if (e + 4 <= n) {
          *reinterpret_cast<float4 *>(cdf + e) =
              make_float4(fmaxf(sv[k][0], m), fmaxf(sv[k][1], m), fmaxf(sv[k][2], m), fmaxf(sv[k][3], m));
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (e + j < n) cdf[e + j] = fmaxf(sv[k][j], m);
        }
      }
    }
    if (tid == kThreads - 1) {
      // only the float bits are read back (level1_kernel, and scan_kernel's in-order rebuild)
      aggw[p] = static_cast<unsigned long long>(__float_as_uint(fmaxf(G, run)));
      dirty[p] = 0u;
    }
    __syncthreads();  // wt / wm are reused by the next listed partition
  }
}

// l1[0] = 0, l1[p+1] = l1[p] + aggregate(p), in order.  Computed as: each thread sums a run of
// consecutive aggregates, a block-wide scan joins the runs; every addition is checked, and if
// any rounded thread 0 repeats the whole sum strictly in order (then grouping matters).
__global__ void __launch_bounds__(1024) level1_kernel(const unsigned long long *aggw, unsigned nparts, double *l1,
                                                      unsigned *count, int32_t *status) {
  __shared__ double warp_tot[32];
  __shared__ int any_inexact;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid == 0) any_inexact = 0;
  const unsigned per = (nparts + 1023) / 1024;
  const unsigned lo = min(nparts, tid * per), hi = min(nparts, lo + per);
  bool inexact = false;
  double run = 0.0;
  for (unsigned q = lo; q < hi; ++q)
    run = checked_add(run, static_cast<double>(__uint_as_float(static_cast<unsigned>(aggw[q]))), inexact);
  double incl = run;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const double t = __shfl_up_sync(kFull, incl, d);
    if (lane >= d) incl = checked_add(t, incl, inexact);
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    double w = warp_tot[lane];
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const double t = __shfl_up_sync(kFull, w, d);
      if (lane >= d) w = checked_add(t, w, inexact);
    }
    warp_tot[lane] = w;
  }
  __syncthreads();
  // exclusive offset of this thread's run: warps before this one + lanes before this one
  const double up = __shfl_up_sync(kFull, incl, 1);
  const double excl = checked_add(warp == 0 ? 0.0 : warp_tot[warp - 1], lane == 0 ? 0.0 : up, inexact);
  double acc = excl;
  for (unsigned q = lo; q < hi; ++q) {
    acc = checked_add(acc, static_cast<double>(__uint_as_float(static_cast<unsigned>(aggw[q]))), inexact);
    l1[q + 1] = acc;
  }
  if (inexact) atomicOr(&any_inexact, 1);
  __syncthreads();
  if (tid == 0) {
    l1[0] = 0.0;
    if (any_inexact) {
      double a = 0.0;
      for (unsigned q = 0; q < nparts; ++q) {
        a = __dadd_rn(a, static_cast<double>(__uint_as_float(static_cast<unsigned>(aggw[q]))));
        l1[q + 1] = a;
      }
      atomicOr(reinterpret_cast<unsigned *>(status), GEARB_ST_L1_RESUMMED);
    }
    *count = 0u;
  }
}

}  // namespace

// upd: dirty flags (4 B per partition) | list (4 B per partition) | count (4 B, padded)
int64_t update_scratch_bytes(int64_t n) {
  const int64_t nparts = (n + kPart - 1) / kPart;
  return ((nparts * 4 + 255) & ~int64_t(255)) * 2 + 256;
}

int launch_update(float *prio, int64_t n, float *cdf, double *l1, unsigned long long *aggw, void *upd,
                  const int64_t *idx, const float *val, int64_t m, int32_t *status, cudaStream_t stream) {
  GEARB_REQUIRE(n > 0 && m >= 0, "update: bad sizes");
  if (m == 0) return GEARB_OK;
  GEARB_REQUIRE(prio && l1 && aggw && upd && idx && val && status, "update: null pointer argument");  // cdf may be null
  const int64_t nparts = (n + kPart - 1) / kPart;
  const int64_t seg = (nparts * 4 + 255) & ~int64_t(255);
  unsigned *dirty = reinterpret_cast<unsigned *>(upd);
  unsigned *list = reinterpret_cast<unsigned *>(static_cast<char *>(upd) + seg);
  unsigned *count = reinterpret_cast<unsigned *>(static_cast<char *>(upd) + 2 * seg);
  mark_kernel<<<static_cast<unsigned>((m + 255) / 256), 256, 0, stream>>>(prio, n, idx, val, m, dirty, list, count,
                                                                        status);
  GEARB_CUDA(cudaGetLastError());
  int64_t grid = m < nparts ? m : nparts;  // at most that many partitions are listed
  const int64_t cap = static_cast<int64_t>(sm_count()) * 8;
  if (grid > cap) grid = cap;
  rescan_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(prio, n, cdf, aggw, list, count, dirty);
  GEARB_CUDA(cudaGetLastError());
  level1_kernel<<<1, 1024, 0, stream>>>(aggw, static_cast<unsigned>(nparts), l1, count, status);
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

}  // namespace gearb
