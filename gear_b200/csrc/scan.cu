// Single-pass construction of the two-level cumulative priority table.
//
// Stands where the reference's launch_prefix_sum / launch_sum would be
// (src/cuda/one_dim_prefix_sum.cu:125-273, src/cuda/one_dim_sum.cu:22-99).
// The reference kernel is unfinished and has no caller; what is kept from it is
// the shape of the addition tree (four values per thread in sequence, :40-49; a
// Hillis-Steele shuffle scan over the lanes of a warp, :23-28; a second pass over
// warp totals, :192-201).  Its partition descriptors with a status word for a
// look-back (one_dim_prefix_sum.cuh:5-10) are not used: see level 1 below.
//
// Level 2 (cdf): each 4096-entry partition is scanned on its own, in float32, with the
// fixed tree written out in scan_tree.cuh (chunks of 4 in sequence, groups of 4 chunk totals
// in sequence, one Hillis-Steele shuffle scan over the 32 groups of a 512-value block, the
// 8 blocks of the partition in sequence, then a running maximum), so the values do not
// depend on scheduling.  Warp w of the CTA scans block w.
// Level 1 (l1): float64 exclusive offsets of the partitions, defined as the in-order sum of
// the partitions' aggregates (the eight block totals of a partition added in sequence).  This
// kernel leaves every partition's aggregate in global memory; a second, small launch
// (level1.cu) turns the aggregates into l1 (tables of at most 1024 partitions take
// small_scan_kernel below, whose last CTA does it on the spot).  An earlier version chained the offsets through a
// decoupled look-back while streaming: at 6 TB/s the look-back could not keep up with the
// partitions (37 of 105 us at 1e8 priorities), the separate launch costs a few us.
//
// Execution: a persistent, warp-specialised CTA of 9 warps.
//   warp 8 (loader)    takes tickets (a group of up to 4 consecutive partitions
//                      each), and stages one partition (16 KiB) per ring slot in
//                      shared memory with a bulk asynchronous copy that signals
//                      an mbarrier;
//   warps 0-7 (compute) wait for a slot, pull it into registers, free the slot,
//                      scan, and store the cdf with 16-byte streaming stores (or, in
//                      the totals-only instance, keep just the block totals).
// Every wait is bounded; a wait that runs out raises a flag instead of hanging.
//
// HBM traffic: 4 B read + 4 B written per priority, plus ~16 B per partition; the
// totals-only instance (cdf == nullptr) writes nothing per priority.
#include <cstdlib>
#include <mutex>

#include "common.h"
#include "level1.cuh"
#include "warp_search.cuh"
#include "scan_tree.cuh"

namespace gearb {
namespace {

constexpr int kComputeWarps = 8;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kThreads = kComputeThreads + 32;  // + loader warp
constexpr int kTilesPerWarp = 4;
constexpr int kPart = kComputeWarps * kTilesPerWarp * 128;
static_assert(kPart == GEARB_PART, "partition size is part of the ABI");
// Three ring slots and (below) at most three CTAs per SM: 162 KB of the SM's shared memory and
// two thirds of its registers.  Four slots, or a fourth CTA, move no more bytes per second (144 KB
// in flight per SM is three times what the latency-bandwidth product asks for), but they leave
// no room for the sampling launch of the step before, which otherwise runs beside this kernel's
// first third: with 1024 requests a step of scan + draw takes 73.5 us this way against 76.4.
#ifndef GEARB_SCAN_STAGES
#define GEARB_SCAN_STAGES 3
#endif
constexpr int kMaxCtasPerSm = 3;
#ifndef GEARB_SCAN_GROUP
#define GEARB_SCAN_GROUP 4
#endif
constexpr int kStages = GEARB_SCAN_STAGES;   // ring slots of one partition each
constexpr int kGroupMax = GEARB_SCAN_GROUP;  // partitions per ticket
constexpr unsigned kSpinLimit = 1u << 20;  // polls of a shared-memory word / mbarrier before giving up

constexpr unsigned kFull = 0xffffffffu;

// ---- small PTX wrappers -------------------------------------------------------
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
__device__ __forceinline__ void named_barrier_compute() {
  asm volatile("bar.sync 1, %0;" ::"n"(kComputeThreads) : "memory");
}
// Same barrier, but every thread also learns whether any of them raised `flag`.
__device__ __forceinline__ bool named_barrier_compute_or(bool flag) {
  unsigned r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r)
      : "r"(static_cast<unsigned>(flag)), "n"(kComputeThreads)
      : "memory");
  return r != 0;
}
struct ScanArgs {
  const float *prio;
  float *cdf;
  double *l1;
  ScanHeader *hdr;
  float *aggw;               // per partition: its aggregate
  float *blkw;               // per partition: its eight block totals (or null: not wanted)
  double *sb;                // per superblock of kSuperParts partitions: the sum of their aggregates (or null)
  int32_t *status;
  int64_t n;
  unsigned nparts;
  unsigned group;    // partitions per ticket (1, 2 or 4) for the first `nbig` tickets;
  unsigned nbig;     // the tickets after them hold one partition each, which evens out the finish
  unsigned ngroups;  // tickets
  int inline_level1;  // the last CTA builds l1 itself (small tables)
};

struct __align__(128) Smem {
  float4 stage[kStages][kPart / 4];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int stage_part[kStages];         // partition staged in the slot, -1 = no more work
  float wt[2][kComputeWarps];      // block totals, double-buffered by iteration parity
  float wm[2][kComputeWarps];      // block maxima
  alignas(16) float xs[kComputeWarps][128];    // per-warp exchange area: one float per chunk of the warp's block
  volatile unsigned abort;         // a bounded wait ran out somewhere in this CTA
  unsigned emin, emax;             // exponent range of the aggregates this CTA produced
};

// The status word is the caller's and accumulates; the header's word belongs to this launch
// alone (its last CTA reads and clears it), so an abort of an earlier launch -- or one that
// another kernel reported through the same status word -- does not make this one skip level 1.
__device__ __forceinline__ void raise_abort(Smem &sm, const ScanArgs &a) {
  sm.abort = 1u;
  atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_SCAN_ABORTED);
  atomicExch(&a.hdr->aborted, 1u);
}

// ------------------------------------------------------------------ loader warp
__device__ void loader_warp(Smem &sm, const ScanArgs &a, int lane) {
  unsigned it = 0;
  bool stop = false;
  // The ticket after the current one is requested before the current one is served, so the
  // round trip of the atomic is hidden behind a group of partitions' worth of copies.
  unsigned ahead = 0;
  if (lane == 0) ahead = atomicAdd(&a.hdr->ticket, 1u);
  while (!stop) {
    const unsigned t = __shfl_sync(kFull, ahead, 0);
    if (lane == 0 && t < a.ngroups) ahead = atomicAdd(&a.hdr->ticket, 1u);
    const bool last = t >= a.ngroups;
    const unsigned first = t < a.nbig ? t * a.group : a.nbig * a.group + (t - a.nbig);
    const unsigned count = (last || t >= a.nbig) ? 1u : a.group;
    for (unsigned k = 0; k < count && !stop; ++k, ++it) {
      const unsigned s = it % kStages;
      const unsigned parity = ((it / kStages) & 1u) ^ 1u;
      unsigned spins = 0;
      bool ok = false;
      while (!(ok = mbar_try_wait(&sm.empty[s], parity))) {
        if (++spins > kSpinLimit || sm.abort) break;
      }
      if (!__all_sync(kFull, ok)) {
        if (lane == 0 && !sm.abort) raise_abort(sm, a);
        stop = true;
        break;
      }
      if (last) {
        if (lane == 0) {
          sm.stage_part[s] = -1;
          mbar_arrive(&sm.full[s]);
        }
        stop = true;
        break;
      }
      const unsigned p = first + k;
      const int64_t base = static_cast<int64_t>(p) * kPart;
      const int64_t valid = (a.n - base < kPart) ? (a.n - base) : kPart;
      const unsigned bulk_bytes = static_cast<unsigned>((valid * 4) & ~int64_t(15));
      if (valid < kPart) {
        // Ragged last partition: the part a bulk copy cannot express is filled by hand.
        float *st = reinterpret_cast<float *>(sm.stage[s]);
        for (int e = static_cast<int>(bulk_bytes / 4) + lane; e < kPart; e += 32)
          st[e] = (e < valid) ? a.prio[base + e] : 0.f;
        __syncwarp();
      }
      if (lane == 0) {
        sm.stage_part[s] = static_cast<int>(p);
        if (bulk_bytes) {
          mbar_arrive_expect_tx(&sm.full[s], bulk_bytes);
          bulk_load(sm.stage[s], a.prio + base, bulk_bytes, &sm.full[s]);
        } else {
          mbar_arrive(&sm.full[s]);
        }
      }
    }
  }
}

// One partition's aggregate to its word in global memory (read back by the last CTA).
// The exponent range of the aggregates is collected on the way for the level-1 launch.
// With a.sb the aggregate is also added to its superblock's sum: float64 additions in whatever
// order the CTAs arrive, which is the in-order sum whenever no addition rounds -- the consumer
// (the sampling kernel's level-1 lookup without a level-1 table) checks the exponent range for
// that before it trusts the sums.
__device__ __forceinline__ void hand_over(const ScanArgs &a, int part, float agg, unsigned &emin, unsigned &emax) {
  a.aggw[part] = agg;
  if (a.sb) atomicAdd(a.sb + (part / GEARB_SUPER_PARTS), static_cast<double>(agg));
  level1::note_exponent(__float_as_uint(agg), emin, emax);
}
// The partition's eight block totals, for a sampling kernel that rebuilds single blocks of the
// level-2 table from the priorities (sample_gather.cu).
__device__ __forceinline__ void hand_over_blocks(const ScanArgs &a, int part, const float *wt) {
  if (a.blkw == nullptr) return;
  float4 *dst = reinterpret_cast<float4 *>(a.blkw + static_cast<int64_t>(part) * kComputeWarps);
  dst[0] = make_float4(wt[0], wt[1], wt[2], wt[3]);
  dst[1] = make_float4(wt[4], wt[5], wt[6], wt[7]);
}

// ----------------------------------------------------------------- compute warps
// Warp w scans block w (512 values) of the staged partition.  Lane l holds chunk 32k + l of
// the block for k = 0..3 (the float4 it can fetch without a bank conflict); the step from
// "one chunk per lane and tile" to "four consecutive chunks per lane" -- which makes one
// shuffle scan per block enough -- goes through a 512-byte exchange area in shared memory.
// kStore = false: only the partition's last (largest) entry is produced, nothing is stored.
template <bool kStore>
__device__ void compute_warps(Smem &sm, const ScanArgs &a, int warp, int lane) {
  unsigned bits = 0;  // OR of the bit patterns seen: the sign bit ends up set if a priority was bad
  unsigned emin = 0xffffffffu, emax = 0u;  // exponent range of the aggregates this CTA produced (warp 7, lane 0)
  float *xs = sm.xs[warp];
  for (unsigned it = 0;; ++it) {
    const unsigned s = it % kStages;
    const unsigned parity = (it / kStages) & 1u;
    unsigned spins = 0;
    bool ok = false;
    while (!(ok = mbar_try_wait(&sm.full[s], parity))) {
      if (++spins > kSpinLimit || sm.abort) break;
    }
    // A warp that has to leave (its wait ran out, or the loader posted the end marker) still
    // walks, on zeros, to the first barrier below, which doubles as a vote: either every
    // compute warp goes on or every one leaves, so no warp is ever left alone in a barrier.
    const bool lost = !__all_sync(kFull, ok);
    if (lost && lane == 0 && !sm.abort) raise_abort(sm, a);
    const int part_raw = lost ? -1 : sm.stage_part[s];  // -1: the loader has no more work
    const bool leave = part_raw < 0;
    const int part = leave ? 0 : part_raw;
    float4 x[kTilesPerWarp];
#pragma unroll
    for (int k = 0; k < kTilesPerWarp; ++k)
      x[k] = leave ? make_float4(0.f, 0.f, 0.f, 0.f) : sm.stage[s][(warp * kTilesPerWarp + k) * 32 + lane];
    __syncwarp();
    if (lane == 0 && !leave) mbar_arrive(&sm.empty[s]);
    const int buf = it & 1;

    if (!kStore) {
      // ---- totals only: the block totals are all the partition's aggregate needs
      const float total = tree::block_total(x, xs, lane, bits);
      if (lane == 0) sm.wt[buf][warp] = total;
      if (named_barrier_compute_or(leave)) break;
      if (warp == kComputeWarps - 1 && lane == 0) {
        float X = 0.f;
#pragma unroll
        for (int w = 0; w < kComputeWarps; ++w) X = __fadd_rn(X, sm.wt[buf][w]);
        hand_over(a, part, X, emin, emax);
        hand_over_blocks(a, part, sm.wt[buf]);
      }
      continue;  // wt[buf] is next written two rounds on, behind the next round's barrier
    }

    const int64_t base = static_cast<int64_t>(part) * kPart;
    const int64_t e0 = base + warp * tree::kBlockValues;  // this warp's block
    float sv[kTilesPerWarp][4], top[kTilesPerWarp];

    // ---- first pass: sums inside the block; block totals meet in shared memory
    const tree::Group g = tree::block_sums(x, xs, lane, sv, bits);
    if (lane == 0) sm.wt[buf][warp] = g.total;
    if (named_barrier_compute_or(leave)) break;

    // ---- offset of this warp's block: the totals of the blocks before it, in sequence
    float X = 0.f;
    for (int w = 0; w < warp; ++w) X = __fadd_rn(X, sm.wt[buf][w]);
    // the last warp also knows the partition's aggregate X(8): hand it over
    if (warp == kComputeWarps - 1 && lane == 0) {
      hand_over(a, part, __fadd_rn(X, g.total), emin, emax);
      hand_over_blocks(a, part, sm.wt[buf]);
    }

    // ---- second pass: values, then the running maximum block by block
    tree::block_values(X, g, xs, lane, sv, top, false, e0, a.n);
    const float run = tree::block_prefix_max(top, xs, lane);
    if (lane == 0) sm.wm[buf][warp] = run;
    named_barrier_compute();
    float G = 0.f;
    for (int w = 0; w < warp; ++w) G = fmaxf(G, sm.wm[buf][w]);

    // ---- store
    if (e0 + tree::kBlockValues <= a.n) {
      float4 *dst = reinterpret_cast<float4 *>(a.cdf + e0);
#pragma unroll
      for (int k = 0; k < kTilesPerWarp; ++k) {
        const float m = fmaxf(G, xs[k * 32 + lane]);
        __stcs(dst + k * 32 + lane,
               make_float4(fmaxf(sv[k][0], m), fmaxf(sv[k][1], m), fmaxf(sv[k][2], m), fmaxf(sv[k][3], m)));
      }
    } else {
#pragma unroll
      for (int k = 0; k < kTilesPerWarp; ++k) {
        const float m = fmaxf(G, xs[k * 32 + lane]);
        const int64_t e = e0 + (k * 32 + lane) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (e + j < a.n) a.cdf[e + j] = fmaxf(sv[k][j], m);
      }
    }
  }
  if (__any_sync(kFull, (bits >> 31) != 0) && lane == 0)
    atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_BAD_PRIORITY);
  if (warp == kComputeWarps - 1 && lane == 0) {  // published at the very end of the kernel
    sm.emin = emin;
    sm.emax = emax;
  }
}

// Last CTA out: the header is re-armed for the next launch.
__device__ void finish_launch(Smem &sm, const ScanArgs &a, int tid) {
  __shared__ int is_last;
  if (tid == 0) {
    __threadfence();  // this CTA's aggregates before its count
    const unsigned d = atomicAdd(&a.hdr->done, 1u);
    is_last = d == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  // after an abort of THIS launch some aggregates are stale and copies may still land in the
  // ring: leave l1 alone (every CTA raised its flag before it counted itself done)
  const unsigned aborted = __ldcg(&a.hdr->aborted);
  (void)aborted;  // after an abort the status word says that the tables are not valid
  if (tid == 0) {
    a.hdr->ticket = 0u;
    a.hdr->done = 0u;
    a.hdr->aborted = 0u;
    __threadfence();
  }
}

template <bool kStore>
__global__ void __launch_bounds__(kThreads, kMaxCtasPerSm) scan_kernel(const ScanArgs a) {
  extern __shared__ unsigned char smem_raw[];
  Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // A kernel launched behind this one with programmatic stream serialisation may be scheduled
  // as this grid drains; it still waits (griddepcontrol.wait) for this grid to complete.
  // (Two scans of one sampler never run side by side: the level-1 launch between them lets its
  // successor go only at its end, and the host does not overlap two scans in a row.)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kComputeWarps);
    }
    sm.abort = 0;
    sm.emin = 0xffffffffu;
    sm.emax = 0u;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp < kComputeWarps) compute_warps<kStore>(sm, a, warp, lane);
  else loader_warp(sm, a, lane);

  __syncthreads();
  // This grid may have been started while the kernel before it in the stream was still running
  // (programmatic stream serialisation): it only read the priorities and wrote its own scratch
  // (and, if the caller allowed that for the storing instance, its own level-2 table) so far.  What follows it (level 1) overwrites l1, which that kernel may be reading,
  // so this grid must not complete before that one has.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // Only now, with everything before this launch complete (a level-1 launch of an earlier scan
  // clears these words at its end), the exponent range goes to the header for the level-1
  // launch behind this one (level1.cu).
  if (tid == 0 && sm.emax != 0u) {
    atomicMax(&a.hdr->pad[1], 256u - sm.emin);
    atomicMax(&a.hdr->pad[2], sm.emax);
  }
  // Bulk copies still in flight into this CTA's shared memory (only after an abort) must land
  // before the CTA retires.
  if (sm.abort && tid == 0) {
    for (int s = 0; s < kStages; ++s)
      for (unsigned par = 0; par < 2; ++par) {
        unsigned spins = 0;
        while (!mbar_try_wait(&sm.full[s], par) && ++spins < 4096u) {}
      }
  }

  finish_launch(sm, a, tid);
}


// ---------------------------------------------------------------------------------------------
// Tables of at most kSmallParts partitions: one CTA per partition, no tickets, no staging ring.
// A table this small sits in L2 and the whole scan is a chain of a few dependent steps (load,
// tree, aggregate, count, level 1 by the last CTA), so what counts is the length of that chain:
// the persistent kernel above would add a ticket round trip and a bulk copy to it.  The tree is
// the same code (scan_tree.cuh), the results the same bits.
// The kernel lets the launch behind it be scheduled at once (it still waits for this grid where
// it says so) and is itself never launched to overlap what is before it, so two scans of one
// sampler cannot share the CTA counter.
constexpr int kSmallParts = 1024;
constexpr int kSmallThreads = kComputeThreads;

// One partition by one CTA of kSmallThreads threads: warp w scans block w.  On return (after a
// barrier) wt[] holds the eight block totals; the level-2 entries are stored when kStore.
template <bool kStore>
__device__ __forceinline__ void small_partition(const ScanArgs &a, int part, float (*xs_all)[128], float *wt,
                                                float *wm) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int64_t base = static_cast<int64_t>(part) * kPart;
  const int64_t e0 = base + warp * tree::kBlockValues;
  float *xs = xs_all[warp];
  unsigned bits = 0;
  float4 x[kTilesPerWarp];
#pragma unroll
  for (int k = 0; k < kTilesPerWarp; ++k) {
    const int64_t e = e0 + (k * 32 + lane) * 4;
    if (e + 4 <= a.n) {
      x[k] = __ldg(reinterpret_cast<const float4 *>(a.prio + e));
    } else {
      x[k].x = e + 0 < a.n ? __ldg(a.prio + e + 0) : 0.f;
      x[k].y = e + 1 < a.n ? __ldg(a.prio + e + 1) : 0.f;
      x[k].z = e + 2 < a.n ? __ldg(a.prio + e + 2) : 0.f;
      x[k].w = e + 3 < a.n ? __ldg(a.prio + e + 3) : 0.f;
    }
  }
  if (!kStore) {
    const float total = tree::block_total(x, xs, lane, bits);
    if (lane == 0) wt[warp] = total;
    __syncthreads();
  } else {
    float sv[kTilesPerWarp][4], top[kTilesPerWarp];
    const tree::Group g = tree::block_sums(x, xs, lane, sv, bits);
    if (lane == 0) wt[warp] = g.total;
    __syncthreads();
    float X = 0.f;
    for (int w = 0; w < warp; ++w) X = __fadd_rn(X, wt[w]);
    tree::block_values(X, g, xs, lane, sv, top, false, e0, a.n);
    const float run = tree::block_prefix_max(top, xs, lane);
    if (lane == 0) wm[warp] = run;
    __syncthreads();
    float G = 0.f;
    for (int w = 0; w < warp; ++w) G = fmaxf(G, wm[w]);
    if (e0 + tree::kBlockValues <= a.n) {
      float4 *dst = reinterpret_cast<float4 *>(a.cdf + e0);
#pragma unroll
      for (int k = 0; k < kTilesPerWarp; ++k) {
        const float m = fmaxf(G, xs[k * 32 + lane]);
        dst[k * 32 + lane] = make_float4(fmaxf(sv[k][0], m), fmaxf(sv[k][1], m), fmaxf(sv[k][2], m), fmaxf(sv[k][3], m));
      }
    } else {
#pragma unroll
      for (int k = 0; k < kTilesPerWarp; ++k) {
        const float m = fmaxf(G, xs[k * 32 + lane]);
        const int64_t e = e0 + (k * 32 + lane) * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (e + j < a.n) a.cdf[e + j] = fmaxf(sv[k][j], m);
      }
    }
  }
  if (__any_sync(kFull, (bits >> 31) != 0) && lane == 0)
    atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_BAD_PRIORITY);
}

template <bool kStore>
__global__ void __launch_bounds__(kSmallThreads) small_scan_kernel(const ScanArgs a) {
  __shared__ __align__(16) float xs_all[kComputeWarps][128];
  __shared__ float wt[kComputeWarps], wm[kComputeWarps];
  __shared__ __align__(16) float tile[kSmallParts];
  __shared__ int is_last;
  const int tid = threadIdx.x;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int part = blockIdx.x;
  small_partition<kStore>(a, part, xs_all, wt, wm);
  if (tid == 0) {
    float X = 0.f;
#pragma unroll
    for (int w = 0; w < kComputeWarps; ++w) X = __fadd_rn(X, wt[w]);  // the aggregate: block totals in sequence
    a.aggw[part] = X;
    hand_over_blocks(a, part, wt);
    // This grid was launched to start only after everything before it in the stream, but the
    // instruction costs nothing and keeps "no output before the predecessor is done" explicit.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    __threadfence();
    is_last = atomicAdd(&a.hdr->done, 1u) == gridDim.x - 1;
    __threadfence();
  }
  __syncthreads();
  if (!is_last) return;
  if (a.inline_level1) level1::build(a.aggw, a.nparts, a.l1, a.status, tile);
  if (tid == 0) {
    a.hdr->done = 0u;
    __threadfence();
  }
}

// ---------------------------------------------------------------------------------------------
// Scan and draw in ONE launch, for tables small enough that every partition's CTA is resident at
// once (a cooperative launch guarantees that, and refuses the launch otherwise): the place of
// "prefix sum, then torch.multinomial" (gear/sampler/global_sampler.py:154-176) when the table
// changes before every draw.  Two launches cost a second launch latency and a second ramp-up on
// top of a chain that is only a few memory round trips long; here the chain is
//   load partition -> tree -> store -> count in -> [all CTAs counted] -> level 1, built by every
//   CTA into its own shared memory -> level-1 search there -> two rounds into the level-2 table.
// The wait in the middle has an iteration limit; a CTA that runs into it raises
// GEARB_ST_SCAN_ABORTED, skips its draws and leaves.  Results are the bits of the two launches.
struct DrawArgs {
  const double *u;
  int64_t *out;
  int64_t b;
  int flags;
};

__global__ void __launch_bounds__(kSmallThreads) small_scan_search_kernel(const ScanArgs a, const DrawArgs d) {
  __shared__ __align__(16) float xs_all[kComputeWarps][128];
  __shared__ float wt[kComputeWarps], wm[kComputeWarps];
  __shared__ __align__(16) float tile[kSmallParts];
  __shared__ __align__(16) double l1s[kSmallParts + 1];
  __shared__ int gave_up;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int part = blockIdx.x;
  // this warp's first variate travels while the partition is scanned
  const int64_t w_first = static_cast<int64_t>(part) * kComputeWarps + warp;
  double u_next = w_first < d.b ? __ldg(d.u + w_first) : 0.0;
  small_partition<true>(a, part, xs_all, wt, wm);
  __syncthreads();  // every thread's level-2 stores before thread 0's fence and count
  if (tid == 0) {
    float X = 0.f;
#pragma unroll
    for (int w = 0; w < kComputeWarps; ++w) X = __fadd_rn(X, wt[w]);
    a.aggw[part] = X;
    hand_over_blocks(a, part, wt);
    __threadfence();
    atomicAdd(&a.hdr->done, 1u);
    unsigned seen = 0, spins = 0;
    do {
      asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(&a.hdr->done) : "memory");
    } while (seen < gridDim.x && ++spins < (1u << 22));
    gave_up = seen < gridDim.x;
    if (gave_up) atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_SCAN_ABORTED);
    // The counters are cleared by whoever leaves the wait last: nobody reads `done` after that.
    if (atomicAdd(&a.hdr->ticket, 1u) == gridDim.x - 1) {
      a.hdr->done = 0u;
      a.hdr->ticket = 0u;
      __threadfence();
    }
  }
  __syncthreads();
  if (gave_up) return;
  level1::build(a.aggw, a.nparts, part == 0 ? a.l1 : nullptr, a.status, tile, l1s);

  const double total = l1s[a.nparts];
  const int64_t w_stride = static_cast<int64_t>(gridDim.x) * kComputeWarps;
  for (int64_t w = w_first; w < d.b; w += w_stride) {
    double v = u_next;
    if (w + w_stride < d.b) u_next = __ldg(d.u + w + w_stride);
    if (!(total > 0.0)) {  // no selectable entry at all: defined as the last index
      if (lane == 0) d.out[w] = a.n - 1;
      continue;
    }
    if (d.flags & GEARB_SEARCH_SCALE) v = __dmul_rn(v, total);
    if (!(v >= 0.0)) v = 0.0;
    if (!(v < total)) v = __longlong_as_double(__double_as_longlong(total) - 1);
    const int64_t p = warp_upper_bound<double>(l1s + 1, 0, static_cast<int64_t>(a.nparts) - 1, v, lane, LoadPlain());
    const int64_t base = p * kPart;
    const int64_t valid = (a.n - base < kPart) ? (a.n - base) : kPart;
    // Level 2 in two rounds of loads.  Round 1: 256 probes at a fixed stride, eight per lane, whose
    // addresses do not depend on the residual -- they travel at once, and the last of them IS
    // the partition's last entry, which clamps the residual.  Round 2: the <= 16 entries between
    // two probes plus the one before them, one per lane, which also are the two entries the
    // boundary check wants.  "First entry greater than r", as warp_upper_bound finds it.
    const float *cp = a.cdf + base;
    const int64_t st = (valid + 255) / 256;
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      int64_t q = (static_cast<int64_t>(k * 32 + lane) + 1) * st - 1;
      if (q > valid - 1) q = valid - 1;
      x[k] = __ldcg(cp + q);
    }
    const float last = __shfl_sync(kFull, x[7], 31);  // slot 255 probes the last valid entry
    float r = __double2float_rn(__dsub_rn(v, l1s[p]));
    if (!(r < last)) r = __uint_as_float(__float_as_uint(last) - 1u);
    int first = 255;
#pragma unroll
    for (int k = 7; k >= 0; --k) {
      const unsigned m = __ballot_sync(kFull, x[k] > r);
      if (m) first = k * 32 + __ffs(m) - 1;
    }
    const int64_t lo = static_cast<int64_t>(first) * st;  // one past the previous slot's probe
    int64_t hi = lo + st - 1;
    if (hi > valid - 1) hi = valid - 1;
    const int width = static_cast<int>(hi - lo + 1);  // 1..16
    const int64_t qe = lo - 1 + lane;                 // lane 0: the entry before the range
    const float y = (qe >= 0 && lane <= width) ? __ldcg(cp + qe) : 0.f;
    const unsigned m2 = __ballot_sync(kFull, lane >= 1 && lane <= width && y > r);  // never 0: cp[hi] > r
    const int pick = __ffs(m2) - 1;
    const int64_t j = lo + pick - 1;
    const float edge = __shfl_sync(kFull, y, pick);
    const float lo_b = __shfl_sync(kFull, y, pick - 1);
    const int64_t flat = base + j;
    if (lane == 0) {
      d.out[w] = flat;
      bool near = __uint_as_float(__float_as_uint(r) + 1u) >= edge;
      if (j > 0 && r == lo_b) near = true;
      if (near) atomicAdd(a.status + 1, 1);
    }
  }
}

inline int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }
constexpr size_t kSmemBytes = sizeof(Smem) + 128;

}  // namespace

// Scratch layout: header (256 B) | partition aggregates (float32 each).
int64_t scan_scratch_bytes(int64_t n) {
  const int64_t nparts = (n + kPart - 1) / kPart;
  return static_cast<int64_t>(sizeof(ScanHeader)) + align256(nparts * 4);
}

int launch_scan(const float *prio, int64_t n, float *cdf, double *l1, void *scratch,
                int64_t scratch_bytes, int32_t *status, int fresh, cudaStream_t stream, bool level1,
                bool overlap_previous, float *blkw, double *sb, const PublishTail *publish) {
  GEARB_REQUIRE(n > 0, "scan: n must be positive (got %lld)", (long long)n);
  GEARB_REQUIRE(prio && l1 && scratch && status, "scan: null pointer argument");  // cdf may be null
  GEARB_REQUIRE((reinterpret_cast<uintptr_t>(prio) & 15) == 0 &&
                    (reinterpret_cast<uintptr_t>(cdf) & 15) == 0,
                "scan: priorities and cdf must be 16-byte aligned");
  GEARB_REQUIRE((reinterpret_cast<uintptr_t>(l1) & 7) == 0 &&
                    (reinterpret_cast<uintptr_t>(scratch) & 255) == 0,
                "scan: l1 must be 8-byte and scratch 256-byte aligned");
  const int64_t nparts = (n + kPart - 1) / kPart;
  GEARB_REQUIRE(nparts < (int64_t(1) << 30), "scan: too many partitions");
  GEARB_REQUIRE(scratch_bytes >= scan_scratch_bytes(n), "scan: scratch too small (%lld < %lld)",
                (long long)scratch_bytes, (long long)scan_scratch_bytes(n));
  char *sc = static_cast<char *>(scratch);
  if (fresh) {
    // the header's ticket and CTA counters must start at zero
    GEARB_CUDA(cudaMemsetAsync(sc, 0, sizeof(ScanHeader), stream));
  }

  ScanArgs a;
  a.prio = prio;
  a.cdf = cdf;  // null: only level 1 and the aggregates are produced
  a.l1 = l1;
  a.hdr = reinterpret_cast<ScanHeader *>(sc);
  a.aggw = reinterpret_cast<float *>(sc + sizeof(ScanHeader));
  a.blkw = blkw;
  a.sb = nparts > kSmallParts ? sb : nullptr;  // small tables have their level 1 at once
  a.status = status;
  a.n = n;
  a.nparts = static_cast<unsigned>(nparts);

  // Function attributes and occupancy belong to a device: set up once per device, not per process.
  int packed = 0;  // resident CTAs per SM: storing instance in the high half, totals-only in the low
  {
    int rc = per_device_once(kOnceScan, [](int *value) -> int {
      GEARB_CUDA(cudaFuncSetAttribute(scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kSmemBytes)));
      GEARB_CUDA(cudaFuncSetAttribute(scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      static_cast<int>(kSmemBytes)));
      int st = 0, tot = 0;
      GEARB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&st, scan_kernel<true>, kThreads, kSmemBytes));
      GEARB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&tot, scan_kernel<false>, kThreads, kSmemBytes));
      st = st > kMaxCtasPerSm ? kMaxCtasPerSm : st;
      tot = tot > kMaxCtasPerSm ? kMaxCtasPerSm : tot;
      *value = ((st > 0 ? st : 1) << 16) | (tot > 0 ? tot : 1);
      return GEARB_OK;
    }, &packed);
    if (rc != GEARB_OK) return rc;
  }
  if (nparts <= kSmallParts) {
    // one CTA per partition; never launched to overlap its predecessor (see small_scan_kernel)
    a.inline_level1 = level1;
    a.group = a.nbig = a.ngroups = 0;
    if (a.cdf) small_scan_kernel<true><<<static_cast<unsigned>(nparts), kSmallThreads, 0, stream>>>(a);
    else small_scan_kernel<false><<<static_cast<unsigned>(nparts), kSmallThreads, 0, stream>>>(a);
    GEARB_CUDA(cudaGetLastError());
    return GEARB_OK;
  }
  const size_t smem_bytes = kSmemBytes;
  int ctas_per_sm = cdf != nullptr ? (packed >> 16) : (packed & 0xffff);
#ifdef GEARB_TUNE_ENV  // tuning builds only: resident CTAs per SM from the environment
  if (const char *e = getenv("GEARB_TUNE_SCAN_CTAS")) ctas_per_sm = atoi(e) > 0 && atoi(e) < ctas_per_sm ? atoi(e) : ctas_per_sm;
#endif
  const int64_t resident = static_cast<int64_t>(sm_count()) * ctas_per_sm;
  // Group partitions per ticket only when there is enough work to keep every CTA busy.
  a.group = nparts >= resident * kGroupMax * 2 ? kGroupMax : (nparts >= resident * 4 ? 2 : 1);
  // The last stretch (about two partitions per resident CTA) goes out one partition per ticket.
  const int64_t tail = resident * 2 < nparts ? resident * 2 : nparts;
  a.nbig = static_cast<unsigned>((nparts - tail) / a.group);
  a.ngroups = static_cast<unsigned>(a.nbig + (nparts - static_cast<int64_t>(a.nbig) * a.group));

  a.inline_level1 = 0;  // small tables took the other kernel above
  int64_t grid = resident;
  if (grid > a.ngroups) grid = a.ngroups;
  {
    // The launch may overlap the end of the kernel before it in the stream only when the caller
    // says so: that kernel must read nothing this launch writes (its level-2 table; l1 is written
    // by the level-1 launch behind this one, which waits for everything before it).
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap_previous ? 1 : 0;
    if (a.cdf) GEARB_CUDA(cudaLaunchKernelEx(&cfg, scan_kernel<true>, a));
    else GEARB_CUDA(cudaLaunchKernelEx(&cfg, scan_kernel<false>, a));
  }
  // level 1 from the aggregates: a second, small launch (level1.cu), unless the last CTA did it
  return (a.inline_level1 || !level1) ? GEARB_OK
                                       : launch_level1(a.aggw, nparts, l1, nullptr, status, stream, a.hdr, true, a.sb, false, publish);
}

int launch_scan_search(const float *prio, int64_t n, float *cdf, double *l1, void *scratch, int64_t scratch_bytes,
                       int32_t *status, float *blkw, const double *u, int64_t b, int flags, int64_t *out,
                       cudaStream_t stream, int *fused) {
  GEARB_REQUIRE(n > 0 && b >= 0, "scan_search: n must be positive and b non-negative");
  GEARB_REQUIRE(prio && cdf && l1 && scratch && status && fused && (b == 0 || (u && out)),
                "scan_search: null pointer argument");
  GEARB_REQUIRE((reinterpret_cast<uintptr_t>(prio) & 15) == 0 && (reinterpret_cast<uintptr_t>(cdf) & 15) == 0,
                "scan_search: priorities and cdf must be 16-byte aligned");
  GEARB_REQUIRE((flags & ~GEARB_SEARCH_SCALE) == 0, "scan_search: unknown flag");
  GEARB_REQUIRE(scratch_bytes >= scan_scratch_bytes(n), "scan_search: scratch too small");
  const int64_t nparts = (n + kPart - 1) / kPart;
  int resident = 0;  // CTAs of the fused kernel that one device holds at once
  int rc = per_device_once(kOnceScanSearch, [](int *value) -> int {
    int per_sm = 0, coop = 0, dev = 0;
    GEARB_CUDA(cudaGetDevice(&dev));
    GEARB_CUDA(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev));
    GEARB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, small_scan_search_kernel, kSmallThreads, 0));
    *value = coop ? per_sm * sm_count() : 0;
    return GEARB_OK;
  }, &resident);
  if (rc != GEARB_OK) return rc;
  *fused = nparts <= kSmallParts && nparts <= resident;
  if (!*fused) return GEARB_OK;
  char *sc = static_cast<char *>(scratch);
  ScanArgs a;
  a.prio = prio;
  a.cdf = cdf;
  a.l1 = l1;
  a.hdr = reinterpret_cast<ScanHeader *>(sc);
  a.aggw = reinterpret_cast<float *>(sc + sizeof(ScanHeader));
  a.blkw = blkw;
  a.sb = nullptr;
  a.status = status;
  a.n = n;
  a.nparts = static_cast<unsigned>(nparts);
  a.group = a.nbig = a.ngroups = 0;
  a.inline_level1 = 1;
  DrawArgs d;
  d.u = u;
  d.out = out;
  d.b = b;
  d.flags = flags;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(nparts));
  cfg.blockDim = dim3(kSmallThreads);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident together, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GEARB_CUDA(cudaLaunchKernelEx(&cfg, small_scan_search_kernel, a, d));
  return GEARB_OK;
}

// ---------------------------------------------------------------------------------------
// Scratch that lives in the library image, for gearb_scan_static.
//
// kStaticMaxN priorities need kStaticScratchBytes of scratch; every device that loads this
// library reserves that much global memory until the process exits.
constexpr int64_t kStaticMaxN = int64_t(1) << 28;  // 268,435,456 priorities = 65,536 partitions
constexpr int64_t kStaticParts = kStaticMaxN / kPart;
constexpr int64_t kStaticScratchBytes = sizeof(ScanHeader) + kStaticParts * 4;  // 262,400 B

// In host code this name is only a handle for the symbol, not a device address: the address
// each device gave the array is asked for with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScratchBytes];

int64_t static_scan_max_n() { return kStaticMaxN; }

// Where a scratch block keeps its per-partition aggregate words.
float *scan_aggregate_words(void *scratch) {
  return reinterpret_cast<float *>(static_cast<char *>(scratch) + sizeof(ScanHeader));
}

int launch_scan_static(const float *prio, int64_t n, float *cdf, double *l1, int32_t *status,
                       cudaStream_t stream) {
  GEARB_REQUIRE(n > 0, "scan_static: n must be positive (got %lld)", (long long)n);
  if (n > kStaticMaxN)
    return fail(GEARB_ERR_UNSUPPORTED,
                "scan_static: %lld priorities exceed the built-in scratch (at most %lld); use gearb_scan "
                "with caller-provided scratch",
                (long long)n, (long long)kStaticMaxN);
  // One-time set-up per device, with that device current: ask the runtime where this device
  // keeps the array.  No allocation happens here or anywhere else on this path.
  constexpr int kMaxDevices = 64;
  static void *scratch_of_device[kMaxDevices] = {};
  static std::mutex mu;
  int dev = 0;
  GEARB_CUDA(cudaGetDevice(&dev));
  GEARB_REQUIRE(dev >= 0 && dev < kMaxDevices, "scan_static: device ordinal %d not supported", dev);
  void *scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!scratch_of_device[dev]) {
      void *ptr = nullptr;
      GEARB_CUDA(cudaGetSymbolAddress(&ptr, g_static_scan_scratch));
      scratch_of_device[dev] = ptr;
    }
    scratch = scratch_of_device[dev];
  }
  // The array starts zeroed when the module is loaded and every launch leaves its header
  // re-armed (ticket and CTA counter back at zero), so nothing has to be cleared between calls.
  return launch_scan(prio, n, cdf, l1, scratch, kStaticScratchBytes, status, /*fresh=*/0, stream);
}

}  // namespace gearb
