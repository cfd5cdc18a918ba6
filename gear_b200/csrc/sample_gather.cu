// Prioritized sample + gather in one launch.
//
// The reference does this in four steps with the host in between: sample
// (gear/sampler/global_sampler.py:93-152), partition (offline_loader.py:123-140),
// read the timesteps on the host (:168-177) and one fused_subcopy launch per
// column (:178-203).  Here one CTA of four warps serves one request end to end:
//   1. the CTA searches the two-level cumulative table for the request's variate,
//      256 probes per round (two per thread), two rounds per level; the probe
//      loads of a level's first round do not depend on the value they are compared
//      with, so they are issued together with the load of that value;
//   2. the flat step index is decoded to GEAR's (trajectory, timestep, length);
//   3. the request's columns are staged in shared memory by bulk asynchronous copies that
//      are all in flight at once (when they fit and the table is in HBM), and the four warps
//      realign them into the destination slots; larger requests are copied directly.
// Results are identical to search_kernel + decode_kernel + gather_kernel run one
// after the other; only the launches and the index round trip through HBM go.
//
// The kernel is launched with programmatic stream serialisation: its CTAs may be
// scheduled while the kernel before it in the stream (normally the scan) drains,
// and wait in griddepcontrol.wait until that kernel's results are visible.
#include <cstdlib>

#include "common.h"
#include "device_copy.cuh"
#include "scan_tree.cuh"

namespace gearb {
namespace {

constexpr int kThreads = 128;
constexpr int kWarps = kThreads / 32;
constexpr int kSlots = 2 * kThreads;  // probes per round
constexpr unsigned kFull = 0xffffffffu;
#ifndef GEARB_SG_RING_SLOTS
#define GEARB_SG_RING_SLOTS 3
#endif
#ifndef GEARB_SG_RING_CTAS
#define GEARB_SG_RING_CTAS 4
#endif
constexpr int kRingSlots = GEARB_SG_RING_SLOTS;  // per-warp ring of bulk copies for large requests
constexpr int kRingSlotBytes = GEARB_SG_PIECE + 128;  // one piece plus the 16-byte blocks around a misaligned one
constexpr unsigned kWaitLimit = 1u << 20;  // mbarrier polls before a staged copy is declared lost
// Polls of a peer's epoch word before the peer is declared absent: about four seconds, far beyond the
// skew between ranks of one job (host jitter included), short enough to come back from a dead peer.
constexpr unsigned kPeerWaitLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_addr(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_addr(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// 1-D bulk asynchronous copy global -> this CTA's shared memory; completes on `bar`.
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src, unsigned bytes, uint64_t *bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_addr(dst_smem)),
      "l"(src), "r"(bytes), "r"(smem_addr(bar))
      : "memory");
}

// Build with -DGEARB_SG_TIMING to record, per CTA, the SM clock at the phases of its first
// request (a tuning aid; the array is read back with gearb_debug_sg_times).
#ifdef GEARB_SG_TIMING
__device__ unsigned long long g_sg_times[8192][10];
#define GEARB_STAMP(i)                                                                         \
  do {                                                                                         \
    if (threadIdx.x == 0 && blockIdx.x < 8192 && it == static_cast<int64_t>(blockIdx.x))        \
      g_sg_times[blockIdx.x][i] = clock64();                                                   \
  } while (0)
#else
#define GEARB_STAMP(i) do { } while (0)
#endif

struct Range {
  int64_t lo, hi;  // the answer (first index whose entry is greater) lies in [lo, hi]
  int64_t step;
};

__device__ __forceinline__ void probe_positions(const Range &r, int64_t &q0, int64_t &q1, int64_t &step) {
  const int64_t width = r.hi - r.lo + 1;
  step = (width + kSlots - 1) / kSlots;
  q0 = r.lo + (static_cast<int64_t>(threadIdx.x) + 1) * step - 1;
  q1 = r.lo + (static_cast<int64_t>(threadIdx.x) + kThreads + 1) * step - 1;
  if (q0 > r.hi) q0 = r.hi;
  if (q1 > r.hi) q1 = r.hi;
}

// Narrow [lo, hi] to the slot of the first probe that compared greater.  Returns that slot.
// Slot s probes lo + (s+1)*step - 1 (clamped); slot kSlots-1 always probes hi, whose entry is
// known to be greater.
__device__ __forceinline__ int resolve(Range &r, int64_t step, bool gt0, bool gt1, unsigned (*masks)[2 * kWarps],
                                       int &round) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned m0 = __ballot_sync(kFull, gt0), m1 = __ballot_sync(kFull, gt1);
  unsigned *slot = masks[round & 1];
  ++round;
  if (lane == 0) {
    slot[warp] = m0;
    slot[kWarps + warp] = m1;
  }
  __syncthreads();
  int first = kSlots - 1;
#pragma unroll
  for (int w = 2 * kWarps - 1; w >= 0; --w) {
    const unsigned mw = slot[w];
    if (mw) first = w * 32 + __ffs(mw) - 1;
  }
  int64_t qf = r.lo + (static_cast<int64_t>(first) + 1) * step - 1;
  if (qf > r.hi) qf = r.hi;
  if (first > 0) r.lo = r.lo + static_cast<int64_t>(first) * step;
  r.hi = qf;
  return first;
}

struct SampleArgs {
  const float *cdf;   // level-2 table, or null when it is rebuilt from `prio` on the fly
  const float *prio;  // the priorities the level-1 table was built from (only when cdf is null)
  const float *blk;   // with prio: the eight block totals of every partition, as the scan left them (or null)
  const double *l1;
  const double *u;
  const int64_t *lengths;  // per-trajectory lengths or null
  int64_t *out_flat, *out_idx, *out_ts, *out_len;  // each may be null
  int64_t n, nparts, index_offset;
  int64_t u_stride;     // request g reads u[g * u_stride]
  int64_t flat_offset;  // added to out_flat
  int flags;
  double mul, sub;  // GEARB_SEARCH_AFFINE: variate -> variate * mul - sub (global draw -> this shard)
  // Level 1 not built yet (its launch follows the next scan): the partition and its offset come
  // from the superblock sums and the aggregates the scan left (local kLazy instances only).
  const double *sb;       // null: l1 is valid
  const float *agg;       // one aggregate per partition
  const unsigned *range;  // two words: 256 - smallest exponent among the aggregates (0: none), largest exponent
};

// Sharded table read in place: every request is routed to the shard that owns its variate, and
// that shard's cumulative table and trajectory table are read through peer pointers (another
// GPU's memory mapped into this process, or other allocations of this GPU).
struct PeerArgs {
  int world;             // 0: not sharded
  int self;              // the shard that lives in this GPU's own memory, or -1
  const double *totals;  // float64[world], total priority of every shard (device memory)
  // When the totals arrive in a mailbox that the peers write directly (publish_kernel), the words
  // they set to the step's epoch AFTER their total; null: `totals` is complete at launch.
  const unsigned long long *epochs;
  unsigned long long epoch;
  const float *cdf[GEARB_MAX_SHARDS];   // stored level-2 tables (instances without kLazy)
  const float *prio[GEARB_MAX_SHARDS];  // priorities and block totals (instances with kLazy)
  const float *blk[GEARB_MAX_SHARDS];
  const double *l1[GEARB_MAX_SHARDS];   // the owner's level 1, or a copy of it in this GPU's memory
  const uint8_t *table[GEARB_MAX_SHARDS];
};

// How a request's bytes travel, one kernel instance each.  Resident CTAs per SM: the ring's
// shared memory (50.7 KB per CTA) allows four anyway, so that instance may use more registers.
enum { kStaged = 0, kRing = 1, kDirect = 2 };

constexpr int kLazyBytes = GEARB_PART * 4 + kWarps * 512;  // a partition of priorities + exchange areas

// Cumulative tables that another GPU rewrites every step are read past the L1 cache (a line that
// an earlier kernel left there would be stale); a table of this GPU is read-only while the kernel
// runs, and the non-coherent path is the cheaper one.
template <bool kRemote, typename T>
__device__ __forceinline__ T ldt(const T *p) {
  if constexpr (kRemote) return __ldcg(p);
  else return __ldg(p);
}

// Destination slot of request g of this launch (GatherParams::slot_*).
__device__ __forceinline__ int64_t dst_slot(const GatherParams &P, int64_t g) {
  if (P.slot_mod == 0) return g;
  const int64_t q = P.slot_lo + g;
  if (P.slot_mod < 0) return (q >= P.slot_base[0] && q < P.slot_base[1]) ? q - P.slot_base[0] : P.slot_base[2] + g;
  return P.slot_base[q % P.slot_mod] + q / P.slot_mod;
}

// kLazy: there is no stored level-2 table.  The scan left the eight block totals of every
// partition; they say which 512-value block holds the request's entry, and one warp rebuilds
// that block with the scan's own addition tree (2 KiB of priorities straight into registers).
// A variate so close to a block boundary that rounding could put the entry on either side of it
// (within 2^-17 of the partition's aggregate; the tree's sums of one set of terms differ by at
// most 42 ulp), or in a ragged last partition, takes the long way: the whole partition (one
// 16 KiB bulk copy) rebuilt in shared memory and searched.  Both ways give the stored table's
// answer bit for bit.
// Superblock sums per thread when level 1 comes from them: tables of up to
// kThreads * kSuperPerThread superblocks (131,072 partitions) can do without a level-1 table.
constexpr int kSuperPerThread = 8;

// Exclusive prefix of one float64 per thread over the CTA (kThreads threads) and the CTA's sum.
// Plain float64 additions: the callers use it where every partial sum is exact.
__device__ __forceinline__ double cta_exclusive_sum(double x, double &before, int lane, int warp, double *warp_tot,
                                                    double *total_slot) {
  double incl = x;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const double o = __shfl_up_sync(kFull, incl, d);
    if (lane >= d) incl = __dadd_rn(incl, o);
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  double wbase = 0.0, all = 0.0;
#pragma unroll
  for (int w = 0; w < kWarps; ++w) {
    if (w < warp) wbase = __dadd_rn(wbase, warp_tot[w]);
    all = __dadd_rn(all, warp_tot[w]);
  }
  before = __dadd_rn(wbase, __dsub_rn(incl, x));
  (void)total_slot;
  __syncthreads();  // warp_tot may be written again
  return all;
}

template <bool kPeers, int kPath, bool kLazy>
__global__ void __launch_bounds__(kThreads, kPath == kStaged ? 7 : (kPath == kRing ? GEARB_SG_RING_CTAS : 5))
sample_gather_kernel(const __grid_constant__ GatherParams P, const __grid_constant__ SampleArgs a,
                     const __grid_constant__ PeerArgs peers) {
  extern __shared__ __align__(128) uint8_t stage[];  // P.stage_bytes of staging area
  __shared__ unsigned masks[2][2 * kWarps];
  __shared__ float vals[kSlots];
  __shared__ uint64_t stage_bar;
  __shared__ uint64_t ring_bar[kWarps][kRingSlots];
  __shared__ float blk_total[8], blk_max[8];
  __shared__ int warp_best[kWarps];
  __shared__ float warp_lo[kWarps];
  __shared__ int fast_j;
  __shared__ double dsum_warp[kWarps];  // level 1 from the superblock sums: warp totals,
  __shared__ double dsum_total[1];      // the total (or the offset of the pick),
  __shared__ int dsum_pick[1];          // and the superblock / partition picked
  __shared__ int plan_bytes[GEARB_MAX_COLUMNS];     // staged path: clipped bytes of every column of the request
  __shared__ unsigned plan_mis[GEARB_MAX_COLUMNS];  // ... and how far its first byte sits inside a 16-byte block
  unsigned ring_it = 0;  // pieces this warp has pushed through its ring so far
  bool ring_dead = false;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  unsigned flags = 0, stage_parity = 0;
  int round = 0;
#ifdef GEARB_SG_TIMING
  {
    const int64_t it = blockIdx.x;
    GEARB_STAMP(0);
    if (threadIdx.x == 0 && blockIdx.x < 8192) {
      unsigned long long gt;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt));
      g_sg_times[blockIdx.x][8] = gt;
    }
  }
#endif
  if (threadIdx.x == 0) {
    mbar_init(&stage_bar, 1);
    for (int w = 0; w < kWarps; ++w)
      for (int r = 0; r < kRingSlots; ++r) mbar_init(&ring_bar[w][r], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  // Everything this kernel reads may have been written by the kernel before it in the stream.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // A scan launched right behind this kernel may start while it runs (it only reads the
  // priorities and writes its own scratch, the block totals of the OTHER parity, or the other of
  // two alternating tables; it waits for this grid before it lets level 1 go).  The trigger comes
  // after the wait, so whatever starts early behind this kernel finds everything before this
  // kernel complete.  With peers, not before they are known to have finished their previous step
  // (further down): they may still be reading what that scan overwrites.
  if (!(kPeers && peers.epochs)) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (kPeers && peers.epochs) {
    // The shard totals are written into this GPU's mailbox by the peers themselves: wait (with a
    // limit) until every rank's word carries this step's epoch; its total was written before it.
    // A CTA whose wait runs out leaves the epoch in status word 2, and every CTA looks there
    // first: giving up costs the launch one wait, not one per wave of CTAs.
    if (warp == 0) {
      bool ok = true;
      const unsigned ep32 = static_cast<unsigned>(peers.epoch);
      unsigned *gave_up = P.status ? reinterpret_cast<unsigned *>(P.status) + 2 : nullptr;
      if (lane < peers.world) {
        unsigned polls = 0;
        for (;;) {
          unsigned long long seen;
          asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(seen) : "l"(peers.epochs + lane) : "memory");
          if (seen >= peers.epoch) break;
          if ((polls & 63u) == 0u && gave_up && __ldcg(gave_up) == ep32) {
            ok = false;
            break;
          }
          if (++polls > kPeerWaitLimit) {
            ok = false;
            if (gave_up) atomicExch(gave_up, ep32);
            break;
          }
          __nanosleep(polls < 4096u ? 100 : 1000);
        }
      }
      if (!__all_sync(kFull, ok) && lane == 0) masks[0][0] = 0xdeadu;
      else if (lane == 0) masks[0][0] = 0u;
    }
    __syncthreads();
    const bool late = masks[0][0] == 0xdeadu;
    __syncthreads();  // masks is reused by the search
    if (late) {  // a peer never published: report, touch nothing
      if (threadIdx.x == 0 && P.status) atomicOr(reinterpret_cast<unsigned *>(P.status), GEARB_ST_SCAN_ABORTED);
      return;
    }
    // What the peers wrote before their epoch word is read below through ordinary loads and
    // through bulk copies (the asynchronous proxy): order both behind the acquire above.
    asm volatile("fence.proxy.async;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");  // every peer is past its previous step
  }

  // Level 1 not built yet: the prefix of the superblock sums is the same for every request this
  // CTA serves, so it is formed once (kept in registers: the sums of this thread's superblocks
  // and of all before them).
  const bool from_sums = !kPeers && a.sb != nullptr;  // the same in every thread of the grid
  double sum_before = 0.0, sums_total = 0.0;
  double sum_run[kSuperPerThread];
  bool sums_exact = true;
  if (from_sums) {
    // Every sum of aggregates is exact in float64 -- and therefore the in-order sum that level 1
    // is defined as, whatever the order -- when the exponents of the aggregates span little enough.
    // (the sums are fetched beside the range words that say whether they may be used)
    const int nsb = static_cast<int>((a.nparts + GEARB_SUPER_PARTS - 1) / GEARB_SUPER_PARTS);
#pragma unroll
    for (int k = 0; k < kSuperPerThread; ++k) {
      const int q = static_cast<int>(threadIdx.x) * kSuperPerThread + k;
      sum_run[k] = q < nsb ? __ldcg(a.sb + q) : 0.0;
    }
    const unsigned inv = __ldcg(a.range), emax = __ldcg(a.range + 1);
    const unsigned emin = inv ? 256u - inv : 1u;
    sums_exact = emax == 0u || (emax < 255u && (emax - emin) + 24u + (32u - __clz(static_cast<unsigned>(a.nparts))) <= 53u);
    if (sums_exact) {
      double run = 0.0;
#pragma unroll
      for (int k = 0; k < kSuperPerThread; ++k) {
        run = __dadd_rn(run, sum_run[k]);
        sum_run[k] = run;
      }
      sums_total = cta_exclusive_sum(run, sum_before, lane, warp, dsum_warp, dsum_total);
    } else {
      if (threadIdx.x == 0) {  // the definition itself, by one thread: rare tables only
        double acc = 0.0;
        for (int64_t q = 0; q < a.nparts; ++q) acc = __dadd_rn(acc, static_cast<double>(__ldcg(a.agg + q)));
        *dsum_total = acc;
      }
      __syncthreads();
      sums_total = *dsum_total;
      __syncthreads();
    }
  }

  for (int64_t it = blockIdx.x; it < P.n; it += gridDim.x) {
    GEARB_STAMP(1);
    // Sharded: the two ends of the (ascending) slice first, where the requests for other shards
    // are when slices are contiguous -- they take longest and should not start last.
    const int64_t g = kPeers ? ((it & 1) ? P.n - 1 - (it >> 1) : (it >> 1)) : it;
    const int64_t gd = dst_slot(P, g);
    // ---- which shard: sharded tables route the request by the shard totals first
    const float *cdf = a.cdf;
    const float *prio = a.prio;
    const float *blk = a.blk;
    const double *l1 = a.l1;
    const uint8_t *table = P.table;
    double v = __ldg(a.u + g * a.u_stride);
    int owner = 0;
    if (kPeers) {
      // In-order float64 prefix of the shard totals, as the host router computes it
      // (route() in gear_b200/sharded.py): shard j owns prefix[j] <= v < prefix[j+1].
      double gtotal = 0.0;
      for (int j = 0; j < peers.world; ++j) gtotal = __dadd_rn(gtotal, __ldcg(peers.totals + j));
      v = __dmul_rn(v, gtotal);
      if (!(v >= 0.0)) v = 0.0;
      if (!(v < gtotal)) v = __longlong_as_double(__double_as_longlong(gtotal) - 1);
      double acc = 0.0, before = 0.0;
      owner = peers.world - 1;
      for (int j = 0; j < peers.world; ++j) {
        before = acc;
        acc = __dadd_rn(before, __ldcg(peers.totals + j));
        if (acc > v) {
          owner = j;
          break;
        }
      }
      v = __dsub_rn(v, before);
      cdf = peers.cdf[owner];
      prio = peers.prio[owner];
      blk = peers.blk[owner];
      l1 = peers.l1[owner];
      table = peers.table[owner];
    }

    // ---- level 1
    Range r1{0, a.nparts - 1, 0};
    int64_t q0 = 0, q1 = 0, step = 1;
    double p0 = 0.0, p1 = 0.0, total;
    if (from_sums) {
      total = sums_total;
    } else {
      // first round: the probes and the variate travel together
      probe_positions(r1, q0, q1, step);
      p0 = ldt<kPeers>(l1 + 1 + q0);
      p1 = ldt<kPeers>(l1 + 1 + q1);
      total = ldt<kPeers>(l1 + a.nparts);
    }
    int64_t flat;
    if (!(total > 0.0)) {
      flat = a.n - 1;  // nothing selectable: defined as the last index
    } else {
      if (a.flags & GEARB_SEARCH_SCALE) v = __dmul_rn(v, total);
      if (a.flags & GEARB_SEARCH_AFFINE) {
        // global draw -> this shard: clamp into [0, mul) as the router does, then shift
        v = __dmul_rn(v, a.mul);
        if (!(v >= 0.0)) v = 0.0;
        if (!(v < a.mul)) v = __longlong_as_double(__double_as_longlong(a.mul) - 1);
        v = __dsub_rn(v, a.sub);
      }
      if (!(v >= 0.0)) v = 0.0;
      if (!(v < total)) v = __longlong_as_double(__double_as_longlong(total) - 1);
      double off_sums = 0.0;
      if (from_sums && sums_exact) {
        // the superblock whose half-open range of sums holds v (exactly one thread finds it) ...
#pragma unroll
        for (int k = 0; k < kSuperPerThread; ++k) {
          const double lo = __dadd_rn(sum_before, k ? sum_run[k - 1] : 0.0), hi = __dadd_rn(sum_before, sum_run[k]);
          if (lo <= v && v < hi) {
            *dsum_pick = static_cast<int>(threadIdx.x) * kSuperPerThread + k;
            *dsum_total = lo;
          }
        }
        __syncthreads();
        const int64_t first = static_cast<int64_t>(*dsum_pick) * GEARB_SUPER_PARTS;
        const double base_sum = *dsum_total;
        __syncthreads();
        // ... then the partition inside it, one aggregate per thread
        static_assert(kThreads == GEARB_SUPER_PARTS, "one partition of a superblock per thread");
        const int64_t q = first + threadIdx.x;
        const double x = q < a.nparts ? static_cast<double>(__ldcg(a.agg + q)) : 0.0;
        double before;
        cta_exclusive_sum(x, before, lane, warp, dsum_warp, dsum_total);
        const double lo = __dadd_rn(base_sum, before), hi = __dadd_rn(lo, x);
        __syncthreads();  // everybody has read the total slot
        if (lo <= v && v < hi) {
          *dsum_pick = static_cast<int>(threadIdx.x);
          *dsum_total = lo;
        }
        __syncthreads();
        r1.hi = first + *dsum_pick;
        off_sums = *dsum_total;
        __syncthreads();
      } else if (from_sums) {
        if (threadIdx.x == 0) {
          double acc = 0.0, before = 0.0;
          int64_t q = 0;
          for (; q < a.nparts; ++q) {
            before = acc;
            acc = __dadd_rn(acc, static_cast<double>(__ldcg(a.agg + q)));
            if (acc > v) break;
          }
          *dsum_pick = static_cast<int>(q < a.nparts ? q : a.nparts - 1);
          *dsum_total = before;
        }
        __syncthreads();
        r1.hi = *dsum_pick;
        off_sums = *dsum_total;
        __syncthreads();
      } else {
        for (;;) {
          resolve(r1, step, p0 > v, p1 > v, masks, round);
          if (step == 1 || r1.lo >= r1.hi) break;
          probe_positions(r1, q0, q1, step);
          p0 = ldt<kPeers>(l1 + 1 + q0);
          p1 = ldt<kPeers>(l1 + 1 + q1);
        }
      }
      const int64_t p = r1.hi;
      GEARB_STAMP(2);

      const int64_t base = p * GEARB_PART;
      const int64_t valid = (a.n - base < GEARB_PART) ? (a.n - base) : GEARB_PART;
      if (!kLazy) {
        // ---- level 2, first round: probes, the partition's offset and its last entry together
        const float *cp = cdf + base;
        Range r2{0, valid - 1, 0};
        probe_positions(r2, q0, q1, step);
        float c0 = ldt<kPeers>(cp + q0), c1 = ldt<kPeers>(cp + q1);
        const double off = from_sums ? off_sums : ldt<kPeers>(l1 + p);
        const float last = ldt<kPeers>(cp + valid - 1);
        float r = __double2float_rn(__dsub_rn(v, off));
        if (!(r < last)) r = __uint_as_float(__float_as_uint(last) - 1u);
        int first;
        for (;;) {
          if (step == 1) {  // keep the last round's entries: the boundary check below reads two of them
            vals[threadIdx.x] = c0;
            vals[threadIdx.x + kThreads] = c1;
          }
          first = resolve(r2, step, c0 > r, c1 > r, masks, round);
          if (step == 1 || r2.lo >= r2.hi) break;
          probe_positions(r2, q0, q1, step);
          c0 = ldt<kPeers>(cp + q0);
          c1 = ldt<kPeers>(cp + q1);
        }
        const int64_t j = r2.hi;
        flat = base + j;

        // ---- variates within one ulp of a boundary of the chosen entry
        if (P.status && threadIdx.x == 0) {
          // After a round with step 1, slot `first` held cdf[j] and slot `first-1` held cdf[j-1].
          float hi_v, lo_v = 0.f;
          if (step == 1) {
            hi_v = vals[first];
            if (first > 0) lo_v = vals[first - 1];
            else if (j > 0) lo_v = ldt<kPeers>(cp + j - 1);
          } else {
            hi_v = ldt<kPeers>(cp + j);
            if (j > 0) lo_v = ldt<kPeers>(cp + j - 1);
          }
          const bool near = (__uint_as_float(__float_as_uint(r) + 1u) >= hi_v) || (j > 0 && r == lo_v);
          if (near) atomicAdd(P.status + 1, 1);
        }
      } else {
        // ---- level 2 rebuilt from the priorities
        float *pv = reinterpret_cast<float *>(stage);
        float4 *pv4 = reinterpret_cast<float4 *>(stage);
        float *xs = pv + GEARB_PART + warp * 128;
        const float *src = prio + base;
        const double off = from_sums ? off_sums : ldt<kPeers>(l1 + p);
        const float r_raw = __double2float_rn(__dsub_rn(v, off));

        // -- the short way: the block totals say which block holds the entry
        bool fast = false;
        int wsel = 0;
        float Xsel = 0.f;
        if (blk != nullptr && valid == GEARB_PART) {
          const float4 b0 = ldt<kPeers>(reinterpret_cast<const float4 *>(blk + p * 8));
          const float4 b1 = ldt<kPeers>(reinterpret_cast<const float4 *>(blk + p * 8) + 1);
          float X[9];
          X[0] = 0.f;
          X[1] = __fadd_rn(X[0], b0.x); X[2] = __fadd_rn(X[1], b0.y);
          X[3] = __fadd_rn(X[2], b0.z); X[4] = __fadd_rn(X[3], b0.w);
          X[5] = __fadd_rn(X[4], b1.x); X[6] = __fadd_rn(X[5], b1.y);
          X[7] = __fadd_rn(X[6], b1.z); X[8] = __fadd_rn(X[7], b1.w);
          const float delta = X[8] * 7.62939453125e-06f;  // 2^-17 of the aggregate: 128 ulp or more
          int w = 8;
#pragma unroll
          for (int k = 7; k >= 0; --k)
            if (X[k + 1] > r_raw) w = k;
          if (w < 8) {
            float Xlo = 0.f, Xhi = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k)
              if (k == w) {
                Xlo = X[k];
                Xhi = X[k + 1];
              }
            // every value of the blocks before w lies below r, and block w has one above it
            fast = (w == 0 || r_raw > Xlo + delta) && (r_raw < Xhi - delta);
            wsel = w;
            Xsel = Xlo;
          }
        }
        int j = -1;
        GEARB_STAMP(3);
        if (fast) {
          if (warp == 0) {
            const float4 *src4 = reinterpret_cast<const float4 *>(src + wsel * tree::kBlockValues);
            float4 x[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) x[k] = ldt<kPeers>(src4 + k * 32 + lane);
            unsigned bits = 0;  // ignored: the scan has already reported bad priorities
            float sv[4][4], top[4];
            const tree::Group gq = tree::block_sums(x, xs, lane, sv, bits);
            tree::block_values(Xsel, gq, xs, lane, sv, top, false, base + wsel * tree::kBlockValues, a.n);
            int best = tree::kBlockValues;
#pragma unroll
            for (int k = 3; k >= 0; --k)
#pragma unroll
              for (int q = 3; q >= 0; --q)
                if (sv[k][q] > r_raw) best = (k * 32 + lane) * 4 + q;
            best = __reduce_min_sync(kFull, best);
            // the entry itself (it exceeds everything before it) and the largest value before it in the
            // block; the blocks before this one stay below r by the margin, so they cannot tie with it
            float hi_v = 0.f, inner = 0.f;
#pragma unroll
            for (int k = 0; k < 4; ++k)
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const int e = (k * 32 + lane) * 4 + q;
                if (e == best) hi_v = sv[k][q];
                if (e < best) inner = fmaxf(inner, sv[k][q]);
              }
            hi_v = __uint_as_float(__reduce_max_sync(kFull, __float_as_uint(hi_v)));
            inner = __uint_as_float(__reduce_max_sync(kFull, __float_as_uint(inner)));
            if (lane == 0) {
              fast_j = best < tree::kBlockValues ? wsel * tree::kBlockValues + best : -1;
              if (P.status && best < tree::kBlockValues) {
                const bool near =
                    (__uint_as_float(__float_as_uint(r_raw) + 1u) >= hi_v) || (best > 0 && r_raw == inner);
                if (near) atomicAdd(P.status + 1, 1);
              }
            }
          }
          __syncthreads();
          j = fast_j;
          __syncthreads();  // fast_j and warp 0's exchange area are free again
        }
        if (j < 0) {
          // -- the long way: the whole partition
          if (valid == GEARB_PART) {
            if (threadIdx.x == 0) {
              mbar_arrive_expect_tx(&stage_bar, GEARB_PART * 4);
              bulk_load(pv, src, GEARB_PART * 4, &stage_bar);
            }
          } else {  // the ragged last partition: by hand, zeros past the end
            for (int e = threadIdx.x; e < GEARB_PART; e += kThreads) pv[e] = e < valid ? ldt<kPeers>(src + e) : 0.f;
            __syncthreads();
            if (threadIdx.x == 0) mbar_arrive(&stage_bar);
          }
          unsigned polls = 0;
          bool ok;
          while (!(ok = mbar_try_wait(&stage_bar, stage_parity)))
            if (++polls > kWaitLimit) break;
          stage_parity ^= 1u;
          if (__syncthreads_or(!ok)) {
            if (threadIdx.x == 0 && P.status) atomicOr(reinterpret_cast<unsigned *>(P.status), GEARB_ST_SCAN_ABORTED);
            break;
          }
          unsigned bits = 0;  // ignored: the scan has already reported bad priorities
          float sv[4][4], top[4];
          float4 x[4];
          // first pass: block totals (warp w: blocks w and w + 4)
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            const int b = warp + h * kWarps;
#pragma unroll
            for (int k = 0; k < 4; ++k) x[k] = pv4[(b * 4 + k) * 32 + lane];
            const float bt = tree::block_total(x, xs, lane, bits);
            if (lane == 0) blk_total[b] = bt;
          }
          __syncthreads();
          // second pass: values, written back over the priorities; block maxima
#pragma unroll 1
          for (int h = 0; h < 2; ++h) {
            const int b = warp + h * kWarps;
#pragma unroll
            for (int k = 0; k < 4; ++k) x[k] = pv4[(b * 4 + k) * 32 + lane];
            const tree::Group gq = tree::block_sums(x, xs, lane, sv, bits);
            float X = 0.f;
            for (int w = 0; w < b; ++w) X = __fadd_rn(X, blk_total[w]);
            tree::block_values(X, gq, xs, lane, sv, top, false, base + b * tree::kBlockValues, a.n);
#pragma unroll
            for (int k = 0; k < 4; ++k)
              pv4[(b * 4 + k) * 32 + lane] = make_float4(sv[k][0], sv[k][1], sv[k][2], sv[k][3]);
            const float m = tree::block_max(top);
            if (lane == 0) blk_max[b] = m;
          }
          __syncthreads();
          float last = 0.f;
#pragma unroll
          for (int w = 0; w < 8; ++w) last = fmaxf(last, blk_max[w]);
          float r = r_raw;
          if (!(r < last)) r = __uint_as_float(__float_as_uint(last) - 1u);
          // The stored table would be the running maximum of these values; its first entry above r
          // is the first VALUE above r, because the maximum passes r exactly where a value does.
          int best = GEARB_PART;
#pragma unroll 8
          for (int i = GEARB_PART / kThreads - 1; i >= 0; --i) {
            const int e = i * kThreads + threadIdx.x;
            if (pv[e] > r) best = e;
          }
          best = __reduce_min_sync(kFull, best);
          if (lane == 0) warp_best[warp] = best;
          __syncthreads();
          j = warp_best[0];
#pragma unroll
          for (int w = 1; w < kWarps; ++w) j = min(j, warp_best[w]);
          if (j >= valid) j = static_cast<int>(valid) - 1;  // cannot happen while r < last; keeps the index in range
          if (P.status) {
            // ---- variates within one ulp of a boundary of the chosen entry: the entry itself is
            // value j (it exceeds everything before it); its predecessor is the largest value before j
            float lo = 0.f;
#pragma unroll 8
            for (int i = 0; i < GEARB_PART / kThreads; ++i) {
              const int e = i * kThreads + threadIdx.x;
              if (e < j) lo = fmaxf(lo, pv[e]);
            }
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) lo = fmaxf(lo, __shfl_xor_sync(kFull, lo, d));
            if (lane == 0) warp_lo[warp] = lo;
            __syncthreads();
            if (threadIdx.x == 0) {
              float lo_v = 0.f;
              for (int w = 0; w < kWarps; ++w) lo_v = fmaxf(lo_v, warp_lo[w]);
              const float hi_v = pv[j];
              const bool near = (__uint_as_float(__float_as_uint(r) + 1u) >= hi_v) || (j > 0 && r == lo_v);
              if (near) atomicAdd(P.status + 1, 1);
            }
          }
          __syncthreads();  // the partition's values are dead: the gather may reuse the area
        }
        flat = base + j;
      }
    }
    GEARB_STAMP(4);

    // ---- decode
    int64_t t, ts;
    if (((static_cast<uint64_t>(flat) | static_cast<uint64_t>(P.T)) >> 32) == 0) {
      const unsigned f32 = static_cast<unsigned>(flat), T32 = static_cast<unsigned>(P.T);
      const unsigned tq = f32 / T32;
      t = tq;
      ts = f32 - tq * T32;
    } else {
      t = flat / P.T;
      ts = flat - t * P.T;
    }
    const int64_t len = a.lengths ? __ldg(a.lengths + t) : P.T;
    if (threadIdx.x == 0) {
      // sharded: global ids, shard `owner` holds steps [owner*n, (owner+1)*n)
      if (a.out_flat) a.out_flat[gd] = flat + a.flat_offset + (kPeers ? owner * a.n : 0);
      if (a.out_idx) a.out_idx[gd] = t + a.index_offset + (kPeers ? owner * P.capacity : 0);
      if (a.out_ts) a.out_ts[gd] = ts;
      if (a.out_len) a.out_len[gd] = len;
    }

    // ---- gather
    if (kPath == kStaged) {
      // Staged: lane c of the first warp clips column c and starts its bulk asynchronous copy
      // (the 16-byte blocks that cover the clipped segment) into shared memory, so every column
      // of the request is described and in flight at once; then the warps realign from shared
      // memory to the destination.
      if (warp == 0) {
        unsigned cover = 0;
        uintptr_t src = 0;
        if (lane < P.ncols) {
          int64_t start, bytes;
          dev::clip_segment(P, P.cols[lane], t, ts, len, start, bytes, flags);
          if (bytes > 0) {
            src = reinterpret_cast<uintptr_t>(dev::segment_src(P, P.cols[lane], t, start, table));
            cover = static_cast<unsigned>(((src & 15u) + bytes + 15) & ~int64_t(15));
          }
          plan_bytes[lane] = static_cast<int>(bytes);
          plan_mis[lane] = static_cast<unsigned>(src & 15u);
        }
        const unsigned total_tx = __reduce_add_sync(kFull, cover);
        if (lane == 0) {
          if (total_tx) mbar_arrive_expect_tx(&stage_bar, total_tx);
          else mbar_arrive(&stage_bar);
        }
        __syncwarp();
        if (cover)
          bulk_load(stage + P.cols[lane].stage_off, reinterpret_cast<const void *>(src & ~uintptr_t(15)), cover,
                    &stage_bar);
      }
      GEARB_STAMP(5);
      unsigned polls = 0;
      bool ok;
      while (!(ok = mbar_try_wait(&stage_bar, stage_parity)))
        if (++polls > kWaitLimit) break;
      stage_parity ^= 1u;
      GEARB_STAMP(6);
      if (__syncthreads_or(!ok)) {  // a copy never landed: report, do not touch the staging area
        if (threadIdx.x == 0 && P.status) atomicOr(reinterpret_cast<unsigned *>(P.status), GEARB_ST_SCAN_ABORTED);
        break;
      }
      for (int q = warp; q < P.chunks_per_request; q += kWarps) {
        const int c = dev::column_of_piece(P, q);
        const GatherColumn &col = P.cols[c];
        dev::copy_piece<true>(P, col, q - col.chunk_first, gd, stage + col.stage_off + plan_mis[c], plan_bytes[c], lane);
      }
      __syncthreads();  // the staging area is free for the next request
      GEARB_STAMP(7);
    } else if (kPath == kRing && !(kPeers && owner == peers.self)) {
      // Ring: a request too large to stage whole.  Each warp streams its pieces (4 KiB of a
      // slot each) through a private ring of bulk asynchronous copies that runs kRingSlots - 1
      // pieces ahead of the copy-out, so the loads in flight do not depend on registers.  Works
      // the same from HBM, from a peer's memory and from mapped host memory.  (Requests that a
      // sharded table routes to this GPU's own shard take the direct path below: from local HBM
      // plain loads are faster.)
      uint8_t *ring = stage + static_cast<size_t>(warp) * kRingSlots * kRingSlotBytes;
      const int npieces =
          (!ring_dead && warp < P.chunks_per_request) ? (P.chunks_per_request - warp + kWarps - 1) / kWarps : 0;
      auto describe = [&](int k, dev::PieceInfo &pi, uintptr_t &src) {
        const int q = warp + k * kWarps;
        const int c = dev::column_of_piece(P, q);
        const GatherColumn &col = P.cols[c];
        int64_t start, bytes;
        dev::clip_segment(P, col, t, ts, len, start, bytes, flags);
        pi = dev::piece_info(P, col, q - col.chunk_first, gd, bytes);
        src = reinterpret_cast<uintptr_t>(dev::segment_src(P, col, t, start, table)) + static_cast<uintptr_t>(pi.seg_off);
      };
      auto issue = [&](int k) {  // lane 0
        dev::PieceInfo pi;
        uintptr_t src;
        describe(k, pi, src);
        const unsigned s_ = (ring_it + k) % kRingSlots;
        if (pi.len > 0) {
          const unsigned cover = static_cast<unsigned>(((src & 15u) + pi.len + 15) & ~15u);
          mbar_arrive_expect_tx(&ring_bar[warp][s_], cover);
          bulk_load(ring + s_ * kRingSlotBytes, reinterpret_cast<const void *>(src & ~uintptr_t(15)), cover,
                    &ring_bar[warp][s_]);
        } else {
          mbar_arrive(&ring_bar[warp][s_]);
        }
      };
      if (lane == 0)
        for (int k = 0; k < kRingSlots && k < npieces; ++k) issue(k);
      bool lost = false;
      for (int k = 0; k < npieces; ++k) {
        const unsigned itr = ring_it + k, s_ = itr % kRingSlots, parity = (itr / kRingSlots) & 1u;
        unsigned polls = 0;
        bool ok;
        while (!(ok = mbar_try_wait(&ring_bar[warp][s_], parity)))
          if (++polls > kWaitLimit) break;
        if (!__all_sync(kFull, ok)) {
          lost = true;
          break;
        }
        dev::PieceInfo pi;
        uintptr_t src;
        describe(k, pi, src);
        if (pi.len > 0) dev::warp_copy_t<true>(pi.dst, ring + s_ * kRingSlotBytes + (src & 15u), pi.len, lane);
        if (pi.zero_a_len) dev::warp_zero(pi.zero_a, pi.zero_a_len, lane);
        if (pi.zero_b_len) dev::warp_zero(pi.zero_b, pi.zero_b_len, lane);
        __syncwarp();
        if (lane == 0 && k + kRingSlots < npieces) issue(k + kRingSlots);
      }
      ring_it += npieces;
      if (lost) {
        // Copies may still be in flight into this warp's ring: it copies nothing from now on,
        // but keeps walking the loop, whose search rounds contain CTA-wide barriers.
        if (lane == 0 && P.status) atomicOr(reinterpret_cast<unsigned *>(P.status), GEARB_ST_SCAN_ABORTED);
        ring_dead = true;
      }
    } else {
      // Direct: the request's pieces, column by column, dealt to the four warps.
      for (int q = warp; q < P.chunks_per_request; q += kWarps) {
        const int c = dev::column_of_piece(P, q);
        dev::gather_piece(P, P.cols[c], q - P.cols[c].chunk_first, gd, t, ts, len, lane, flags, table);
      }
    }
  }
  flags = __reduce_or_sync(kFull, flags);  // any lane may have clipped a column
  if (P.status && flags && lane == 0) atomicOr(reinterpret_cast<unsigned *>(P.status), flags);
}

}  // namespace

namespace {
using Kernel = void (*)(const GatherParams, const SampleArgs, const PeerArgs);
// [peers][lazy][path]
const Kernel kInstances[2][2][3] = {
    {{sample_gather_kernel<false, kStaged, false>, sample_gather_kernel<false, kRing, false>,
      sample_gather_kernel<false, kDirect, false>},
     {sample_gather_kernel<false, kStaged, true>, sample_gather_kernel<false, kRing, true>,
      sample_gather_kernel<false, kDirect, true>}},
    {{sample_gather_kernel<true, kStaged, false>, sample_gather_kernel<true, kRing, false>,
      sample_gather_kernel<true, kDirect, false>},
     {sample_gather_kernel<true, kStaged, true>, sample_gather_kernel<true, kRing, true>,
      sample_gather_kernel<true, kDirect, true>}}};
constexpr size_t kRingBytes = static_cast<size_t>(kWarps) * kRingSlots * kRingSlotBytes;

int launch_any(const GatherParams &p, const SampleArgs &a, const PeerArgs &peers, cudaStream_t stream, int width = 0) {
  int64_t grid = p.n;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (grid > cap) grid = cap;
  // A table whose level 1 is still owed is a table that is rescanned every step: the next scan
  // starts while this launch runs.  With few CTAs per SM (each striding over the requests) this
  // launch fits beside that scan's CTAs -- shared memory and registers both -- so the scan runs at
  // full width from its start; the full grid would keep it out until this launch drains.
  // Measured at 1024 requests and 1e8 priorities: totals-only scans, 2 per SM: 73.5 us per step
  // against 84; storing scans on two tables in turn, 4 per SM: 139 against 143.
  if (width > 0 && grid > static_cast<int64_t>(sm_count()) * width) grid = static_cast<int64_t>(sm_count()) * width;
#ifdef GEARB_TUNE_ENV  // tuning builds only: a smaller grid (the CTAs stride over the requests)
  if (const char *e = getenv("GEARB_TUNE_SG_GRID")) grid = atoi(e) > 0 && atoi(e) < grid ? atoi(e) : grid;
#endif

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kThreads);
  {
    int rc = per_device_once(kOnceSampleGather, [](int *) -> int {  // function attributes are per device
      for (int pe = 0; pe < 2; ++pe)
        for (int lz = 0; lz < 2; ++lz)
          GEARB_CUDA(cudaFuncSetAttribute(kInstances[pe][lz][kRing], cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          static_cast<int>(kRingBytes > static_cast<size_t>(kLazyBytes) ? kRingBytes : kLazyBytes)));
      return GEARB_OK;
    }, nullptr);
    if (rc != GEARB_OK) return rc;
  }
  const int path = p.stage_bytes > 0 ? kStaged : (p.ring ? kRing : kDirect);
  const bool lazy = a.cdf == nullptr;
  size_t smem = path == kStaged ? static_cast<size_t>(p.stage_bytes) : (path == kRing ? kRingBytes : 0);
  if (lazy && smem < static_cast<size_t>(kLazyBytes)) smem = kLazyBytes;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GEARB_CUDA(cudaLaunchKernelEx(&cfg, kInstances[peers.world > 0][lazy][path], p, a, peers));
  return GEARB_OK;
}
}  // namespace

int launch_sample_gather(const GatherParams &p, const float *cdf, const double *l1, int64_t n,
                         const double *u, int flags, const int64_t *lengths, int64_t index_offset,
                         int64_t *out_flat, int64_t *out_idx, int64_t *out_ts, int64_t *out_len,
                         cudaStream_t stream, double mul, double sub, const float *lazy_prio,
                         const float *lazy_blk, const DrawLayout &lay, const Level1Sums *sums) {
  GEARB_REQUIRE(n > 0, "sample_gather: the priority table is empty");
  GEARB_REQUIRE(!sums || (sums->sb && sums->agg && sums->range &&
                          (n + GEARB_PART - 1) / GEARB_PART <= int64_t(kThreads) * kSuperPerThread * GEARB_SUPER_PARTS),
                "sample_gather: level 1 from the scan's sums: null pointer or too many partitions");
  if (p.n == 0) return GEARB_OK;
  GEARB_REQUIRE((cdf || lazy_prio) && l1 && u, "sample_gather: null pointer argument");
  GEARB_REQUIRE(!lazy_prio || (reinterpret_cast<uintptr_t>(lazy_prio) & 15) == 0,
                "sample_gather: the priorities must be 16-byte aligned");
  SampleArgs a = {};
  a.cdf = lazy_prio ? nullptr : cdf; a.prio = lazy_prio; a.blk = lazy_prio ? lazy_blk : nullptr;
  a.l1 = l1; a.u = u; a.lengths = lengths;
  a.out_flat = out_flat; a.out_idx = out_idx; a.out_ts = out_ts; a.out_len = out_len;
  a.n = n; a.nparts = (n + GEARB_PART - 1) / GEARB_PART;
  a.index_offset = index_offset;
  a.u_stride = lay.u_stride;
  a.flat_offset = lay.flat_offset;
  a.flags = flags;
  a.mul = mul;
  a.sub = sub;
  if (sums) {
    a.sb = sums->sb;
    a.agg = sums->agg;
    a.range = sums->range;
  }
  PeerArgs peers = {};
  return launch_any(p, a, peers, stream, sums ? sums->ctas_per_sm : 0);
}

namespace {
struct Mailboxes {
  void *box[GEARB_MAX_SHARDS];
};
constexpr int kPublishThreads = 256;
// One rank's level 1 (optionally) and total into every rank's mailbox, then the epoch.
//   header of a mailbox:   totals[2 slots][GEARB_MAX_SHARDS] f64 | epochs[2][GEARB_MAX_SHARDS] u64
//   behind the header:     level-1 copies [2 slots][GEARB_MAX_SHARDS] of l1_stride bytes each
// Slot epoch & 1 is used.  With copy_l1 the CTAs first spread this rank's level 1 over the other
// ranks' mailboxes with ordinary stores; the last CTA to finish (a counter in this rank's own
// memory) then writes the total and, with release semantics at system scope, the epoch word the
// pull launches of the other ranks wait for.
__global__ void __launch_bounds__(kPublishThreads)
    publish_kernel(const double *l1, unsigned nparts, Mailboxes m, int world, int rank, unsigned long long epoch,
                   int copy_l1, long long l1_stride, unsigned *counter, const float *blk, long long blk_base,
                   long long blk_stride) {
  __shared__ int is_last;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // level 1 comes from the launch before
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned slot = static_cast<unsigned>(epoch & 1u);
  if (copy_l1) {
    const unsigned count = nparts + 1u;
    for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x) {
      const double v = __ldcg(l1 + i);
      for (int j = 0; j < world; ++j) {
        if (j == rank) continue;
        double *dst = reinterpret_cast<double *>(static_cast<char *>(m.box[j]) + GEARB_MAILBOX_BYTES +
                                                 (static_cast<long long>(slot) * GEARB_MAX_SHARDS + rank) * l1_stride);
        dst[i] = v;
      }
    }
    if (blk) {  // the eight block totals of every partition travel too: 32 bytes per partition, as two float4
      const unsigned quads = nparts * 2u;
      for (unsigned i = blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += gridDim.x * blockDim.x) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(blk) + i);
        for (int j = 0; j < world; ++j) {
          if (j == rank) continue;
          float4 *dst = reinterpret_cast<float4 *>(static_cast<char *>(m.box[j]) + blk_base +
                                                   (static_cast<long long>(slot) * GEARB_MAX_SHARDS + rank) * blk_stride);
          dst[i] = v;
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      is_last = atomicAdd(counter, 1u) == gridDim.x - 1;
      __threadfence_system();
    }
    __syncthreads();
    if (!is_last) return;
    if (threadIdx.x == 0) *counter = 0u;
  } else if (blockIdx.x != 0) {
    return;
  }
  const int j = threadIdx.x;
  if (j >= world) return;
  char *box = static_cast<char *>(m.box[j]);
  double *tot = reinterpret_cast<double *>(box) + slot * GEARB_MAX_SHARDS + rank;
  unsigned long long *ep =
      reinterpret_cast<unsigned long long *>(box + 2 * GEARB_MAX_SHARDS * 8) + slot * GEARB_MAX_SHARDS + rank;
  const double t = __ldcg(l1 + nparts);
  asm volatile("st.relaxed.sys.global.f64 [%0], %1;" ::"l"(tot), "d"(t) : "memory");
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(ep), "l"(epoch) : "memory");
}
}  // namespace

#ifdef GEARB_SG_TIMING
extern "C" __attribute__((visibility("default"))) int gearb_debug_sg_times(unsigned long long *out, int rows) {
  return cudaMemcpyFromSymbol(out, g_sg_times, sizeof(unsigned long long) * 10 * rows) == cudaSuccess ? 0 : 2;
}
#endif

int64_t mailbox_l1_stride(int64_t n) {
  const int64_t nparts = (n + GEARB_PART - 1) / GEARB_PART;
  return ((nparts + 1) * 8 + 255) & ~int64_t(255);
}
int64_t mailbox_blk_stride(int64_t n) {
  const int64_t nparts = (n + GEARB_PART - 1) / GEARB_PART;
  return (nparts * 32 + 255) & ~int64_t(255);
}
int64_t mailbox_blk_base(int64_t n) { return GEARB_MAILBOX_BYTES + 2 * GEARB_MAX_SHARDS * mailbox_l1_stride(n); }

int launch_publish(const double *l1, int64_t nparts, int world, int rank, void *const *mailboxes,
                   unsigned long long epoch, int copy_l1, unsigned *counter, cudaStream_t stream, const float *blk) {
  GEARB_REQUIRE(world >= 1 && world <= GEARB_MAX_SHARDS && rank >= 0 && rank < world, "publish: bad rank or world");
  GEARB_REQUIRE(l1 && mailboxes && epoch > 0, "publish: null argument or epoch 0");
  GEARB_REQUIRE(!copy_l1 || counter, "publish: the level-1 copy needs a counter word");
  Mailboxes m = {};
  for (int j = 0; j < world; ++j) {
    GEARB_REQUIRE(mailboxes[j], "publish: null mailbox for rank %d", j);
    m.box[j] = mailboxes[j];
  }
  cudaLaunchConfig_t cfg = {};
  int64_t grid = 1;
  if (copy_l1 && world > 1) {
    grid = ((blk ? nparts * 2 : nparts + 1) + kPublishThreads - 1) / kPublishThreads;
    if (grid > 32) grid = 32;
  }
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(kPublishThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const long long stride = mailbox_l1_stride(nparts * GEARB_PART);
  GEARB_CUDA(cudaLaunchKernelEx(&cfg, publish_kernel, l1, static_cast<unsigned>(nparts), m, world, rank, epoch,
                                (copy_l1 && world > 1) ? 1 : 0, stride, counter,
                                (copy_l1 && world > 1) ? blk : nullptr,
                                static_cast<long long>(mailbox_blk_base(nparts * GEARB_PART)),
                                static_cast<long long>(mailbox_blk_stride(nparts * GEARB_PART))));
  return GEARB_OK;
}

int launch_pull(const GatherParams &p, int world, int self, const double *totals, const void *const *peer_cdf,
                const void *const *peer_prio, const void *const *peer_blk, const void *const *peer_l1,
                const void *const *peer_table, int64_t n, const double *u, int64_t *out_flat, int64_t *out_idx,
                int64_t *out_ts, cudaStream_t stream, const void *mailbox, unsigned long long epoch,
                const DrawLayout &lay) {
  GEARB_REQUIRE(n > 0, "pull: the priority table is empty");
  GEARB_REQUIRE(world >= 1 && world <= GEARB_MAX_SHARDS, "pull: %d shards, at most %d", world, GEARB_MAX_SHARDS);
  if (p.n == 0) return GEARB_OK;
  GEARB_REQUIRE((totals || mailbox) && (peer_cdf || peer_prio) && peer_l1 && peer_table && u,
                "pull: null pointer argument");
  PeerArgs peers = {};
  peers.world = world;
  peers.self = self;
  peers.totals = totals;
  if (mailbox) {  // totals and epoch words of the step's slot in this rank's mailbox
    GEARB_REQUIRE(epoch > 0, "pull: epoch 0 with a mailbox");
    const char *box = static_cast<const char *>(mailbox);
    const unsigned slot = static_cast<unsigned>(epoch & 1u);
    peers.totals = reinterpret_cast<const double *>(box) + slot * GEARB_MAX_SHARDS;
    peers.epochs = reinterpret_cast<const unsigned long long *>(box + 2 * GEARB_MAX_SHARDS * 8) + slot * GEARB_MAX_SHARDS;
    peers.epoch = epoch;
  }
  const bool lazy = peer_cdf == nullptr;
  for (int j = 0; j < world; ++j) {
    GEARB_REQUIRE(peer_l1[j] && peer_table[j], "pull: null pointer for shard %d", j);
    if (lazy) {
      GEARB_REQUIRE(peer_prio[j], "pull: null priorities for shard %d", j);
      GEARB_REQUIRE((reinterpret_cast<uintptr_t>(peer_prio[j]) & 15) == 0, "pull: priorities must be 16-byte aligned");
      peers.prio[j] = static_cast<const float *>(peer_prio[j]);
      peers.blk[j] = peer_blk ? static_cast<const float *>(peer_blk[j]) : nullptr;
    } else {
      GEARB_REQUIRE(peer_cdf[j], "pull: null level-2 table for shard %d", j);
      peers.cdf[j] = static_cast<const float *>(peer_cdf[j]);
    }
    peers.l1[j] = static_cast<const double *>(peer_l1[j]);
    peers.table[j] = static_cast<const uint8_t *>(peer_table[j]);
  }
  SampleArgs a = {};
  a.cdf = lazy ? nullptr : peers.cdf[0];
  a.prio = lazy ? peers.prio[0] : nullptr;
  a.l1 = peers.l1[0]; a.u = u;
  a.out_flat = out_flat; a.out_idx = out_idx; a.out_ts = out_ts;
  a.n = n; a.nparts = (n + GEARB_PART - 1) / GEARB_PART;
  a.u_stride = lay.u_stride;
  a.flat_offset = lay.flat_offset;
  a.mul = 1.0;
  return launch_any(p, a, peers, stream);
}

}  // namespace gearb
