// Level 1 of the cumulative table as its own small launch, spread over a thread-block cluster.
//
// The integer route of level1.cuh costs about 70 instructions per aggregate, and one SM needs
// 25 us for config 3's 24,415 aggregates -- a third of the scan it follows.  Eight CTAs of one
// cluster each take an eighth of the array; what they must tell each other (the exponent
// range, the sums of the ranks before, whether anything was inexact) travels through
// distributed shared memory between three cluster barriers.  The kernel is launched with
// programmatic stream serialisation behind the scan, and lets the kernel behind it start early
// in the same way.
#include <cooperative_groups.h>

#include "common.h"
#include "level1.cuh"

namespace cg = cooperative_groups;

namespace gearb {
namespace {

constexpr int kClusterCtas = 8;
constexpr int kClusterThreads = 512;

struct Shared {
  unsigned long long warp_tot[32];
  unsigned warp_emin[32], warp_emax[32];
  unsigned long long total;  // this CTA's sum, read by the ranks after it
  unsigned emin, emax;       // this CTA's exponent range, read by every rank
  int bad;                   // this CTA met a prefix sum that does not fit a float64
};

__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(kClusterThreads)
    level1_cluster_kernel(const float *agg, unsigned nparts, double *l1, unsigned *clear_word, int32_t *status) {
  extern __shared__ float4 tile4[];  // level1::kTile floats
  __shared__ Shared sh;
  float *tile = reinterpret_cast<float *>(tile4);
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  const unsigned kAll = 0xffffffffu;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kClusterThreads / 32;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the aggregates come from the kernel before

  // this rank's share: a multiple of four aggregates, so that its 16-byte copies stay aligned
  const unsigned per = ((nparts + kClusterCtas - 1) / kClusterCtas + 3u) & ~3u;
  const unsigned first = min(nparts, rank * per), count = min(per, nparts - first);
  level1::load_tile(agg, first, count, tile);
  const unsigned run = ((count + kClusterThreads - 1) / kClusterThreads) | 1u;
  const unsigned lo = min(count, tid * run), hi = min(count, lo + run);

  // ---- exponent range of the non-zero aggregates, over the whole cluster
  unsigned emin = 0xffffffffu, emax = 0u;
#pragma unroll 4
  for (unsigned q = lo; q < hi; ++q) level1::note_exponent(__float_as_uint(tile[q]), emin, emax);
  emin = __reduce_min_sync(kAll, emin);
  emax = __reduce_max_sync(kAll, emax);
  if (lane == 0) {
    sh.warp_emin[warp] = emin;
    sh.warp_emax[warp] = emax;
  }
  __syncthreads();
  if (tid == 0) {
    unsigned a = 0xffffffffu, b = 0u;
    for (int w = 0; w < nwarps; ++w) {
      a = min(a, sh.warp_emin[w]);
      b = max(b, sh.warp_emax[w]);
    }
    sh.emin = a;
    sh.emax = b;
    sh.bad = 0;
  }
  cluster.sync();
  emin = 0xffffffffu;
  emax = 0u;
  for (unsigned r = 0; r < kClusterCtas; ++r) {
    const Shared *peer = cluster.map_shared_rank(&sh, r);
    emin = min(emin, peer->emin);
    emax = max(emax, peer->emax);
  }
  if (emax == 0u) emin = 1u;  // all zero
  const bool wide = level1::too_wide(emin, emax, nparts);  // the same verdict in every thread of the cluster

  // ---- sums inside this rank's share
  unsigned long long sum = 0ull;
  if (!wide) {
#pragma unroll 4
    for (unsigned q = lo; q < hi; ++q) {
      const unsigned b = __float_as_uint(tile[q]);
      if (b << 1) sum += level1::scaled(b, emin);
    }
  }
  unsigned long long incl = sum;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const unsigned long long o = __shfl_up_sync(kAll, incl, d);
    if (lane >= d) incl += o;
  }
  if (lane == 31) sh.warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    unsigned long long w = lane < nwarps ? sh.warp_tot[lane] : 0ull;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const unsigned long long o = __shfl_up_sync(kAll, w, d);
      if (lane >= d) w += o;
    }
    const unsigned long long before = __shfl_up_sync(kAll, w, 1);
    if (lane == 31) sh.total = w;  // lanes past the last warp hold zeros: this is the share's sum
    sh.warp_tot[lane] = lane == 0 ? 0ull : before;  // exclusive: the warps before this one
  }
  cluster.sync();

  // ---- offsets out: the ranks before this one, the warps before this one, the lanes before this one
  bool inexact = false;
  if (!wide) {
    unsigned long long acc = 0ull;
    for (unsigned r = 0; r < rank; ++r) acc += cluster.map_shared_rank(&sh, r)->total;
    const unsigned long long up = __shfl_up_sync(kAll, incl, 1);
    acc += sh.warp_tot[warp] + (lane == 0 ? 0ull : up);
#pragma unroll 4
    for (unsigned q = lo; q < hi; ++q) {
      const unsigned b = __float_as_uint(tile[q]);
      if (b << 1) acc += level1::scaled(b, emin);
      __stcg(reinterpret_cast<unsigned long long *>(l1) + first + q + 1, level1::double_bits(acc, emin, inexact));
    }
    if (rank == 0 && tid == 0) __stcg(&l1[0], 0.0);
  }
  if (inexact) atomicOr(&sh.bad, 1);
  cluster.sync();
  bool redo = wide;
  for (unsigned r = 0; r < kClusterCtas; ++r) redo |= cluster.map_shared_rank(&sh, r)->bad != 0;
  cluster.sync();  // nobody leaves while a peer may still read its shared memory
  if (rank == 0 && tid == 0) {
    if (redo) level1::in_order(agg, nparts, l1, status);
    if (clear_word) *clear_word = 0u;
  }
}

// One CTA, any size: the tiles are walked in sequence (level1::build).
__global__ void __launch_bounds__(1024)
    level1_single_kernel(const float *agg, unsigned nparts, double *l1, unsigned *clear_word, int32_t *status) {
  extern __shared__ float4 tile4[];
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
  level1::build(agg, nparts, l1, status, reinterpret_cast<float *>(tile4));
  if (threadIdx.x == 0 && clear_word) *clear_word = 0u;
}

}  // namespace

// l1 from the aggregates of `nparts` partitions; `clear_word`, when given, is zeroed at the end
// (the incremental update's list counter).
int launch_level1(const float *agg, int64_t nparts, double *l1, unsigned *clear_word, int32_t *status,
                  cudaStream_t stream) {
  constexpr int kTileBytes = level1::kTile * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    GEARB_CUDA(cudaFuncSetAttribute(level1_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileBytes));
    GEARB_CUDA(cudaFuncSetAttribute(level1_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileBytes));
    attr_set = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.dynamicSmemBytes = kTileBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const unsigned np = static_cast<unsigned>(nparts);
  if (nparts <= static_cast<int64_t>(kClusterCtas) * (level1::kTile - 4)) {
    cfg.gridDim = dim3(kClusterCtas);
    cfg.blockDim = dim3(kClusterThreads);
    GEARB_CUDA(cudaLaunchKernelEx(&cfg, level1_cluster_kernel, agg, np, l1, clear_word, status));
  } else {
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    GEARB_CUDA(cudaLaunchKernelEx(&cfg, level1_single_kernel, agg, np, l1, clear_word, status));
  }
  return GEARB_OK;
}

}  // namespace gearb
