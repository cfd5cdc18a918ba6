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
//   launch_level1   (level1.cu) offsets from all aggregates; clears the list for the next call
#include "common.h"
#include "scan_tree.cuh"

namespace gearb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kPart = GEARB_PART;
static_assert(kWarps * tree::kBlockValues == kPart, "one warp per block of the partition");

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
  if ((__float_as_uint(v) >> 31) || !(v == v))  // sign bit set (negative or -0.0) or NaN
    atomicOr(reinterpret_cast<unsigned *>(status), GEARB_ST_BAD_PRIORITY);
  prio[k] = v;  // two updates of one index in a batch: one of them wins, as with any scatter
  const unsigned p = static_cast<unsigned>(k / kPart);
  if (atomicExch(&dirty[p], 1u) == 0u) list[atomicAdd(count, 1u)] = p;
}

// Same tree as the compute warps of scan_kernel (scan_tree.cuh): warp w scans block w.
// cdf == nullptr: the table is kept without its level-2 entries, only the aggregate is redone.
__global__ void __launch_bounds__(kThreads) rescan_kernel(const float *prio, int64_t n, float *cdf,
                                                          float *aggw, float *blkw, const unsigned *list,
                                                          const unsigned *count, unsigned *dirty) {
  __shared__ float wt[kWarps], wm[kWarps];
  __shared__ __align__(16) float xs_all[kWarps][128];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  float *xs = xs_all[warp];
  const unsigned total = *count;
  unsigned bits = 0;  // priorities were checked when they were written (mark_kernel)
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
    const tree::Group g = tree::block_sums(x, xs, lane, sv, bits);
    if (lane == 0) {
      wt[warp] = g.total;
      if (blkw) blkw[static_cast<int64_t>(p) * kWarps + warp] = g.total;  // the partition's block totals follow it
    }
    __syncthreads();
    float X = 0.f;
    for (int w = 0; w < warp; ++w) X = __fadd_rn(X, wt[w]);
    if (cdf != nullptr) {
      tree::block_values(X, g, xs, lane, sv, top, false, e0, n);
      const float run = tree::block_prefix_max(top, xs, lane);
      if (lane == 0) wm[warp] = run;
      __syncthreads();
      float G = 0.f;
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
      aggw[p] = __fadd_rn(X, g.total);  // aggregate X(8)
      dirty[p] = 0u;
    }
    __syncthreads();  // wt / wm are reused by the next listed partition
  }
}

}  // namespace

// upd: dirty flags (4 B per partition) | list (4 B per partition) | count (4 B, padded)
int64_t update_scratch_bytes(int64_t n) {
  const int64_t nparts = (n + kPart - 1) / kPart;
  return ((nparts * 4 + 255) & ~int64_t(255)) * 2 + 256;
}

int launch_update(float *prio, int64_t n, float *cdf, double *l1, float *aggw, float *blkw, ScanHeader *hdr,
                  void *upd, const int64_t *idx, const float *val, int64_t m, int32_t *status, cudaStream_t stream) {
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
  rescan_kernel<<<static_cast<unsigned>(grid), kThreads, 0, stream>>>(prio, n, cdf, aggw, blkw, list, count, dirty);
  GEARB_CUDA(cudaGetLastError());
  // l1 from all aggregates (level1.cu); the list of touched partitions is cleared for the next call
  {
    int rc = launch_level1(aggw, nparts, l1, count, status, stream, hdr, false);
    if (rc != GEARB_OK) return rc;
  }
  return GEARB_OK;
}

}  // namespace gearb
