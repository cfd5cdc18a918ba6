// Level 1 of the cumulative table as its own small launch, spread over a thread-block cluster.
//
// The integer route of level1.cuh costs about 70 instructions per aggregate, and one SM needs
// 25 us for config 3's 24,415 aggregates -- a third of the scan it follows.  Eight CTAs of one
// cluster each take an eighth of the array.  The exponent range comes with the aggregates (the
// scan leaves it in its header); the sums of the ranks before a rank travel through eight words
// of that header behind ONE cluster barrier; the last rank to finish does the clean-up.  The kernel is launched with
// programmatic stream serialisation behind the scan, and lets the kernel behind it be scheduled
// once it has read everything it needs.
#include <cooperative_groups.h>

#include "common.h"
#include "level1.cuh"

namespace cg = cooperative_groups;

namespace gearb {
namespace {

constexpr int kClusterCtas = 8;
constexpr int kClusterThreads = 512;

// Words of the scan header (common.h: ScanHeader::pad) that this kernel and the scan share.
constexpr int kPadEminInv = 1;  // max over non-zero aggregates of 256 - exponent (0: none seen)
constexpr int kPadEmax = 2;     // max exponent
constexpr int kPadBad = 3;      // some rank met a prefix sum that does not fit a float64
constexpr int kPadDone = 4;     // ranks that have finished
constexpr int kPadTotals = 9;   // 8 x 64-bit: the sum of every rank's share (8-byte aligned in the header)

struct Shared {
  unsigned long long warp_tot[32];
  unsigned warp_emin[32], warp_emax[32];
  unsigned emin, emax;
};

// have_range: the scan that produced the aggregates also left their exponent range in the
// header; otherwise (aggregates touched by an incremental update) the cluster finds it first.
__global__ void __cluster_dims__(kClusterCtas, 1, 1) __launch_bounds__(kClusterThreads)
    level1_cluster_kernel(const float *agg, unsigned nparts, double *l1, unsigned *clear_word, int32_t *status,
                          ScanHeader *hdr, int have_range, double *sb, int after_next,
                          const __grid_constant__ PublishTail pub) {
  extern __shared__ float4 tile4[];  // level1::kTile floats
  __shared__ Shared sh;
  float *tile = reinterpret_cast<float *>(tile4);
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  const unsigned kAll = 0xffffffffu;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = kClusterThreads / 32;
  unsigned long long *totals = reinterpret_cast<unsigned long long *>(&hdr->pad[kPadTotals]);

  // The aggregates come from the kernel before -- or, when this launch sits behind the NEXT scan
  // (after_next), from a scan that was complete before that one began: then there is nothing to
  // wait for yet, and what follows this launch may be staged at once (it waits for this grid).
  if (!after_next) asm volatile("griddepcontrol.wait;" ::: "memory");
  else asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  // this rank's share: a multiple of four aggregates, so that its 16-byte copies stay aligned
  const unsigned per = ((nparts + kClusterCtas - 1) / kClusterCtas + 3u) & ~3u;
  const unsigned first = min(nparts, rank * per), count = min(per, nparts - first);
  level1::load_tile(agg, first, count, tile);
  const unsigned run = ((count + kClusterThreads - 1) / kClusterThreads) | 1u;
  const unsigned lo = min(count, tid * run), hi = min(count, lo + run);

  // ---- exponent range of the non-zero aggregates, over the whole table
  unsigned emin = 0xffffffffu, emax = 0u;
  if (have_range) {
    const unsigned inv = __ldcg(&hdr->pad[kPadEminInv]);
    emax = __ldcg(&hdr->pad[kPadEmax]);
    emin = inv ? 256u - inv : 0xffffffffu;
  } else {
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
    }
    cluster.sync();
    emin = 0xffffffffu;
    emax = 0u;
    for (unsigned r = 0; r < kClusterCtas; ++r) {
      const Shared *peer = cluster.map_shared_rank(&sh, r);
      emin = min(emin, peer->emin);
      emax = max(emax, peer->emax);
    }
    cluster.sync();  // nobody's shared memory is read by a peer after this point
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
    if (lane == 31) __stcg(&totals[rank], w);  // lanes past the last warp hold zeros: the share's sum
    sh.warp_tot[lane] = lane == 0 ? 0ull : before;  // exclusive: the warps before this one
  }
  cluster.sync();  // every rank's sum is in global memory (the barrier orders it for the cluster)

  // ---- offsets out: the ranks before this one, the warps before this one, the lanes before this one
  bool inexact = false;
  if (!wide) {
    unsigned long long acc = 0ull;
    for (unsigned r = 0; r < rank; ++r) acc += __ldcg(&totals[r]);
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
  // ---- last rank out: the in-order repeat if anyone needs it, and the header's words back to zero
  if (__syncthreads_or(inexact) && tid == 0) atomicOr(&hdr->pad[kPadBad], 1u);
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(&hdr->pad[kPadDone], 1u) == kClusterCtas - 1) {
      __threadfence();
      if (wide || atomicOr(&hdr->pad[kPadBad], 0u)) level1::in_order(agg, nparts, l1, status);
      // Behind the next scan: that scan ends only after the sampling launch before it, the one
      // reader of the exponent range and of the superblock sums besides this launch, has ended.
      if (after_next) asm volatile("griddepcontrol.wait;" ::: "memory");
      if (sb) {
        const unsigned nsb = (nparts + GEARB_SUPER_PARTS - 1) / GEARB_SUPER_PARTS;
        for (unsigned k = 0; k < nsb; ++k) sb[k] = 0.0;
      }
      hdr->pad[kPadEminInv] = 0u;
      hdr->pad[kPadEmax] = 0u;
      hdr->pad[kPadBad] = 0u;
      hdr->pad[kPadDone] = 0u;
      if (clear_word) *clear_word = 0u;
      if (pub.world > 0) {
        // The table is complete (every rank's fence came before its count above): this shard's
        // total, then -- behind ONE fence at system scope -- the step's number, into every
        // rank's mailbox.  The pull launches wait for that number with acquire loads.
        const unsigned slot = static_cast<unsigned>(pub.epoch & 1u);
        const double t = __ldcg(l1 + nparts);
        for (int j = 0; j < pub.world; ++j) {
          double *tot = reinterpret_cast<double *>(pub.box[j]) + slot * GEARB_MAX_SHARDS + pub.rank;
          asm volatile("st.relaxed.sys.global.f64 [%0], %1;" ::"l"(tot), "d"(t) : "memory");
        }
        __threadfence_system();
        for (int j = 0; j < pub.world; ++j) {
          unsigned long long *ep = reinterpret_cast<unsigned long long *>(static_cast<char *>(pub.box[j]) +
                                                                          2 * GEARB_MAX_SHARDS * 8) +
                                   slot * GEARB_MAX_SHARDS + pub.rank;
          asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(ep), "l"(pub.epoch) : "memory");
        }
      }
    }
    // Everything this launch reads has been read (by the last rank too, had it to repeat the sum
    // in order): the launch behind it may be scheduled.  If that is the next scan of the same
    // table it overwrites the aggregates; it touches the header's exponent-range words only
    // after this whole grid has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  }
}

// One CTA, any size: the tiles are walked in sequence (level1::build).
__global__ void __launch_bounds__(1024)
    level1_single_kernel(const float *agg, unsigned nparts, double *l1, unsigned *clear_word, int32_t *status,
                         ScanHeader *hdr, double *sb) {
  extern __shared__ float4 tile4[];
  asm volatile("griddepcontrol.wait;" ::: "memory");  // dependents start when this grid is done
  level1::build(agg, nparts, l1, status, reinterpret_cast<float *>(tile4));
  if (sb) {
    const unsigned nsb = (nparts + GEARB_SUPER_PARTS - 1) / GEARB_SUPER_PARTS;
    for (unsigned k = threadIdx.x; k < nsb; k += blockDim.x) sb[k] = 0.0;
  }
  if (threadIdx.x == 0) {
    hdr->pad[kPadEminInv] = 0u;  // left by the scan, not used here
    hdr->pad[kPadEmax] = 0u;
    if (clear_word) *clear_word = 0u;
  }
}

}  // namespace

// l1 from the aggregates of `nparts` partitions; `clear_word`, when given, is zeroed at the end
// (the incremental update's list counter).  hdr: the header of the scratch block the aggregates
// live in; have_range: the scan that wrote them left their exponent range there.
bool level1_can_follow_next_scan(int64_t nparts) {
  return nparts <= static_cast<int64_t>(kClusterCtas) * (level1::kTile - 4);
}

int launch_level1(const float *agg, int64_t nparts, double *l1, unsigned *clear_word, int32_t *status,
                  cudaStream_t stream, ScanHeader *hdr, bool have_range, double *sb, bool after_next,
                  const PublishTail *publish) {
  GEARB_REQUIRE(!after_next || level1_can_follow_next_scan(nparts), "level1: table too large to follow the next scan");
  GEARB_REQUIRE(!publish || (level1_can_follow_next_scan(nparts) && !after_next),
                "level1: publishing from this launch needs the cluster kernel in its usual place");
  const PublishTail none = PublishTail();
  constexpr int kTileBytes = level1::kTile * sizeof(float);
  {
    int rc = per_device_once(kOnceLevel1, [](int *) -> int {  // function attributes are per device
      GEARB_CUDA(cudaFuncSetAttribute(level1_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileBytes));
      GEARB_CUDA(cudaFuncSetAttribute(level1_single_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTileBytes));
      return GEARB_OK;
    }, nullptr);
    if (rc != GEARB_OK) return rc;
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
    // only the rank's share is staged: a small footprint lets the CTAs sit beside a running scan
    const unsigned per = ((np + kClusterCtas - 1) / kClusterCtas + 3u) & ~3u;
    cfg.dynamicSmemBytes = per * 4u < 1024u ? 1024u : per * 4u;
    GEARB_CUDA(cudaLaunchKernelEx(&cfg, level1_cluster_kernel, agg, np, l1, clear_word, status, hdr,
                                  static_cast<int>(have_range), sb, static_cast<int>(after_next),
                                  publish ? *publish : none));
  } else {
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(1024);
    GEARB_CUDA(cudaLaunchKernelEx(&cfg, level1_single_kernel, agg, np, l1, clear_word, status, hdr, sb));
  }
  return GEARB_OK;
}

}  // namespace gearb
