// Single-pass construction of the two-level cumulative priority table.
//
// Stands where the reference's launch_prefix_sum / launch_sum would be
// (src/cuda/one_dim_prefix_sum.cu:125-273, src/cuda/one_dim_sum.cu:22-99).
// The reference kernel is unfinished and has no caller; what is kept from it is
// the shape of the addition tree (four values per thread in sequence, :40-49; a
// Hillis-Steele shuffle scan over the lanes of a warp, :23-28; a second scan
// pass over warp totals, :192-201; partition descriptors with a status word for the
// look-back, one_dim_prefix_sum.cuh:5-10).
//
// Level 2 (cdf): each 4096-entry partition is scanned on its own, in float32, with the
// fixed tree written out in scan_tree.cuh (chunks of 4 in sequence, groups of 4 chunk totals
// in sequence, one Hillis-Steele shuffle scan over the 32 groups of a 512-value block, the
// 8 blocks of the partition in sequence, then a running maximum), so the values do not
// depend on scheduling.  Warp w of the CTA scans block w.
// Level 1 (l1): float64 exclusive offsets of the partitions, defined as the
// in-order sum of the partitions' last cdf entries.  They come out of a
// decoupled look-back over published aggregates.  The look-back adds in a
// timing-dependent grouping, so every float64 addition is checked with TwoSum;
// while all of them are exact the result equals the in-order sum bit for bit.
// If one is inexact (or a bounded wait gives up) the last CTA to finish
// recomputes l1 strictly in order from the per-partition aggregates.
//
// Execution: a persistent, warp-specialised CTA of 10 warps.
//   warp 8 (loader)    takes tickets (a group of up to 4 consecutive partitions
//                      each), and stages one partition (16 KiB) per ring slot in
//                      shared memory with a bulk asynchronous copy that signals
//                      an mbarrier;
//   warps 0-7 (compute) wait for a slot, pull it into registers, free the slot,
//                      scan, and store the cdf with 16-byte streaming stores (or, in
//                      the totals-only instance, keep just the partition's last entry);
//   warp 9 (look-back) receives each partition's aggregate through a small ring
//                      in shared memory, chains the aggregates of a group in
//                      order, publishes one descriptor per group and looks back
//                      over earlier groups while the other warps keep streaming.
// Descriptors carry their own validity: each 64-bit word is (tag << 32 | half of
// a float64), so a reader needs no fence and one 32-byte read per predecessor.
// Every wait is bounded; a wait that runs out raises a flag instead of hanging.
//
// HBM traffic: 4 B read + 4 B written per priority, plus ~16 B per partition; the
// totals-only instance (cdf == nullptr) writes nothing per priority.
#include <mutex>

#include "common.h"
#include "scan_tree.cuh"

namespace gearb {
namespace {

constexpr int kComputeWarps = 8;
constexpr int kComputeThreads = kComputeWarps * 32;
constexpr int kThreads = kComputeThreads + 64;  // + loader warp + look-back warp
constexpr int kTilesPerWarp = 4;
constexpr int kPart = kComputeWarps * kTilesPerWarp * 128;
static_assert(kPart == GEARB_PART, "partition size is part of the ABI");
#ifndef GEARB_SCAN_STAGES
#define GEARB_SCAN_STAGES 4
#endif
#ifndef GEARB_SCAN_GROUP
#define GEARB_SCAN_GROUP 4
#endif
constexpr int kStages = GEARB_SCAN_STAGES;   // ring slots of one partition each
constexpr int kGroupMax = GEARB_SCAN_GROUP;  // partitions per ticket
constexpr int kRing = 16;    // aggregate ring entries (compute -> look-back)
#ifndef GEARB_SCAN_SUPER
#define GEARB_SCAN_SUPER 32
#endif
constexpr int kSuper = GEARB_SCAN_SUPER;  // partitions per look-back descriptor (at most 32: one lane each)

constexpr unsigned kSpinLimit = 1u << 20;  // polls of a shared-memory word / mbarrier before giving up
constexpr unsigned kLookLimit = 1u << 17;  // polls (x ~100 ns) of a predecessor descriptor

constexpr unsigned kHdrRebuild = 1u;  // header flag: level 1 must be re-summed in order
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
__device__ __forceinline__ void st_u64(unsigned long long *p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void ld_desc(const unsigned long long *p, unsigned long long w[4]) {
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(w[0]), "=l"(w[1]) : "l"(p) : "memory");
  asm volatile("ld.relaxed.gpu.global.v2.u64 {%0,%1}, [%2];" : "=l"(w[2]), "=l"(w[3]) : "l"(p + 2) : "memory");
}
__device__ __forceinline__ unsigned long long ld_u64_relaxed(const unsigned long long *p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_u32_relaxed(const unsigned *p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// s = a + b in float64; raises `inexact` when the addition rounded.
__device__ __forceinline__ double checked_add(double a, double b, bool &inexact) {
  const double s = __dadd_rn(a, b);
  const double bb = __dsub_rn(s, a);
  const double err = __dadd_rn(__dsub_rn(a, __dsub_rn(s, bb)), __dsub_rn(b, bb));
  inexact |= (err != 0.0);
  return s;
}

// A float64 split over two self-validating 64-bit words.
__device__ __forceinline__ void publish(unsigned long long *two_words, double v, unsigned tag) {
  const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(v));
  const unsigned long long t = static_cast<unsigned long long>(tag) << 32;
  st_u64(two_words, t | (bits >> 32));
  st_u64(two_words + 1, t | (bits & 0xffffffffull));
}
__device__ __forceinline__ bool decode(unsigned long long hi, unsigned long long lo, unsigned tag, double &v) {
  if (static_cast<unsigned>(hi >> 32) != tag || static_cast<unsigned>(lo >> 32) != tag) return false;
  v = __longlong_as_double(static_cast<long long>(((hi & 0xffffffffull) << 32) | (lo & 0xffffffffull)));
  return true;
}

struct ScanArgs {
  const float *prio;
  float *cdf;
  double *l1;
  ScanHeader *hdr;
  unsigned *gcount;          // per super-group: partitions finished (returns to 0 by itself)
  unsigned long long *desc;  // per super-group: {agg hi, agg lo, prefix hi, prefix lo}
  unsigned long long *aggw;  // per partition: (tag << 32) | bits of the float32 aggregate
  int32_t *status;
  int64_t n;
  unsigned nparts;
  unsigned group;    // partitions per ticket (1, 2 or 4: divides kSuper) for the first `nbig` tickets;
  unsigned nbig;     // the tickets after them hold one partition each, which evens out the finish
  unsigned ngroups;  // tickets
  unsigned nsuper;   // super-groups of kSuper partitions
};

struct __align__(128) Smem {
  float4 stage[kStages][kPart / 4];
  uint64_t full[kStages];
  uint64_t empty[kStages];
  int stage_part[kStages];         // partition staged in the slot, -1 = no more work
  float wt[2][kComputeWarps];      // block totals, double-buffered by iteration parity
  float wm[2][kComputeWarps];      // block maxima
  alignas(16) float xs[kComputeWarps][128];    // per-warp exchange area: one float per chunk of the warp's block
  volatile int ring_part[kRing];   // aggregate ring: partition id (-1 = end)
  volatile float ring_agg[kRing];
  volatile unsigned ring_head;     // entries produced
  volatile unsigned ring_tail;     // entries consumed
  volatile unsigned abort;         // a bounded wait ran out somewhere in this CTA
};

__device__ __forceinline__ void raise_abort(Smem &sm, const ScanArgs &a) {
  sm.abort = 1u;
  atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_SCAN_ABORTED);
}

// ------------------------------------------------------------------ loader warp
__device__ void loader_warp(Smem &sm, const ScanArgs &a, int lane) {
  unsigned it = 0;
  bool stop = false;
  // The ticket after the current one is requested before the current one is served, so the
  // round trip of the atomic is hidden behind four partitions' worth of copies.
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

// One partition's aggregate from the compute warps to the look-back warp.
__device__ __forceinline__ void hand_over(Smem &sm, int part, float agg) {
  const unsigned h = sm.ring_head;
  unsigned sp = 0;
  while (h - sm.ring_tail >= kRing) {
    if (++sp > kSpinLimit || sm.abort) break;
  }
  sm.ring_part[h % kRing] = part;
  sm.ring_agg[h % kRing] = agg;
  __threadfence_block();
  sm.ring_head = h + 1;
}

// ----------------------------------------------------------------- compute warps
// Warp w scans block w (512 values) of the staged partition.  Lane l holds chunk 32k + l of
// the block for k = 0..3 (the float4 it can fetch without a bank conflict); the step from
// "one chunk per lane and tile" to "four consecutive chunks per lane" -- which makes one
// shuffle scan per block enough -- goes through a 512-byte exchange area in shared memory.
// kStore = false: only the partition's last (largest) entry is produced, nothing is stored.
template <bool kStore>
__device__ void compute_warps(Smem &sm, const ScanArgs &a, int warp, int lane) {
  bool bad = false;
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

    const int64_t base = static_cast<int64_t>(part) * kPart;
    const int64_t e0 = base + warp * tree::kBlockValues;  // this warp's block
    const int buf = it & 1;
    float sv[kTilesPerWarp][4], top[kTilesPerWarp];

    // ---- first pass: sums inside the block; block totals meet in shared memory
    const tree::Group g = tree::block_sums(x, xs, lane, sv, bad);
    if (lane == 0) sm.wt[buf][warp] = g.total;
    if (named_barrier_compute_or(leave)) break;

    // ---- offset of this warp's block: the totals of the blocks before it, in sequence
    float X = 0.f;
    for (int w = 0; w < warp; ++w) X = __fadd_rn(X, sm.wt[buf][w]);

    // ---- second pass: values (kStore) or only each chunk's largest one
    tree::block_values(X, g, xs, lane, sv, top, !kStore, e0, a.n);

    if (!kStore) {
      // ---- the partition's largest entry is all that is needed
      const float m = tree::block_max(top);
      if (lane == 0) sm.wm[buf][warp] = m;
      named_barrier_compute();
      if (warp == kComputeWarps - 1 && lane == 0) {
        float G = 0.f;
        for (int w = 0; w < kComputeWarps; ++w) G = fmaxf(G, sm.wm[buf][w]);
        hand_over(sm, part, G);
      }
      continue;
    }

    // ---- running maximum, block by block
    const float run = tree::block_prefix_max(top, xs, lane);
    if (lane == 0) sm.wm[buf][warp] = run;
    named_barrier_compute();
    float G = 0.f;
    for (int w = 0; w < warp; ++w) G = fmaxf(G, sm.wm[buf][w]);
    // the last warp knows the partition's last (= largest) entry
    if (warp == kComputeWarps - 1 && lane == 0) hand_over(sm, part, fmaxf(G, run));

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
  if (warp == kComputeWarps - 1 && lane == 0) {  // tell the look-back warp there is no more
    const unsigned h = sm.ring_head;
    unsigned sp = 0;
    while (h - sm.ring_tail >= kRing && ++sp < kSpinLimit && !sm.abort) {}
    sm.ring_part[h % kRing] = -1;
    __threadfence_block();
    sm.ring_head = h + 1;
  }
  if (__any_sync(kFull, bad) && lane == 0)
    atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_BAD_PRIORITY);
}

// --------------------------------------------------------------- look-back warp
// Two levels keep the look-back cheap.  A ticket (up to 4 partitions) only publishes its
// partitions' aggregates and bumps the counter of its super-group (16 partitions); the warp
// whose bump completes the super-group chains the 16 aggregates in order, publishes ONE
// descriptor and looks back over earlier super-groups.  The number of look-back
// participants, and with it the time the prefix needs to travel down the table, drops 4x
// against one look-back per ticket.
// The warp that completed group g: chain its aggregates, publish, look back, write l1.
__device__ void finish_group(const ScanArgs &a, unsigned g, unsigned epoch, int lane) {
  const unsigned tagA = (epoch << 2) | 1u, tagP = (epoch << 2) | 2u;
  const unsigned first = g * kSuper;
  const unsigned in_group = min(static_cast<unsigned>(kSuper), a.nparts - first);
  bool inexact = false;
  // The counter says every partition of the group has issued its aggregate; the words carry
  // their own tag, so poll (normally zero times) until each one is visible.
  double incl = 0.0;
  bool late = false;
  if (lane < static_cast<int>(in_group)) {
    unsigned polls = 0;
    for (;;) {
      const unsigned long long w = ld_u64_relaxed(&a.aggw[first + lane]);
      if (static_cast<unsigned>(w >> 32) == tagA) {
        incl = static_cast<double>(__uint_as_float(static_cast<unsigned>(w)));
        break;
      }
      if (++polls > kLookLimit) {
        late = true;
        break;
      }
      __nanosleep(32);
    }
  }
  if (__any_sync(kFull, late)) {
    if (lane == 0) {
      atomicOr(&a.hdr->pad[0], kHdrRebuild);
      atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_SCAN_ABORTED);
    }
    return;
  }
  // inclusive in-order sums of the group's aggregates (shuffle scan; exact => order-free)
#pragma unroll
  for (int d = 1; d < kSuper; d <<= 1) {
    const double t = __shfl_up_sync(kFull, incl, d);
    if (lane >= d) incl = checked_add(t, incl, inexact);
  }
  const double gsum = __shfl_sync(kFull, incl, in_group - 1);
  unsigned long long *mine = a.desc + static_cast<size_t>(g) * 4;
  double excl = 0.0;
  bool gave_up = false;
  if (g > 0) {
    if (lane == 0) publish(mine, gsum, tagA);
    long long j = static_cast<long long>(g) - 1;
    for (;;) {
      const long long q = j - lane;
      double val = 0.0;
      int kind = 2;  // 2 = prefix known, 1 = aggregate known, 0 = nothing yet; "group -1" has prefix 0
      unsigned polls = 0;
      for (;;) {
        if (q >= 0) {
          unsigned long long w[4];
          ld_desc(a.desc + static_cast<size_t>(q) * 4, w);
          kind = decode(w[2], w[3], tagP, val) ? 2 : (decode(w[0], w[1], tagA, val) ? 1 : 0);
        }
        if (__all_sync(kFull, kind != 0)) break;
        ++polls;
        const bool quit =
            polls > kLookLimit || ((polls & 31u) == 0 && (ld_u32_relaxed(&a.hdr->pad[0]) & kHdrRebuild));
        if (__any_sync(kFull, quit)) {
          gave_up = true;
          break;
        }
        __nanosleep(64);
      }
      if (gave_up) break;
      const unsigned pmask = __ballot_sync(kFull, kind == 2);
      const int fp = pmask ? (__ffs(pmask) - 1) : 32;
      if (lane > fp) val = 0.0;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const double o = __shfl_down_sync(kFull, val, d);
        val = checked_add(val, o, inexact);
      }
      const double wsum = __shfl_sync(kFull, val, 0);
      excl = checked_add(excl, wsum, inexact);
      if (pmask) break;
      j -= 32;
    }
  }
  if (gave_up) {
    // Nothing to publish; later groups find the rebuild flag and stop waiting too.
    if (lane == 0) {
      const unsigned old = atomicOr(&a.hdr->pad[0], kHdrRebuild);
      if (!(old & kHdrRebuild)) atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_LOOKBACK_TIMEOUT);
    }
    return;
  }
  if (lane == 0) publish(mine + 2, checked_add(excl, gsum, inexact), tagP);
  if (lane < static_cast<int>(in_group)) __stcg(&a.l1[first + lane + 1], checked_add(excl, incl, inexact));
  if (g == 0 && lane == 0) __stcg(&a.l1[0], 0.0);
  if (__any_sync(kFull, inexact) && lane == 0) atomicOr(&a.hdr->pad[0], kHdrRebuild);
}


__device__ void lookback_warp(Smem &sm, const ScanArgs &a, unsigned epoch, int lane) {
  const unsigned tagA = (epoch << 2) | 1u;
  unsigned have = 0;  // partitions of the current ticket seen so far
  for (;;) {
    // ---- pop one aggregate
    const unsigned tl = sm.ring_tail;
    unsigned spins = 0;
    bool ok = true;
    while (sm.ring_head == tl) {
      if (++spins > kSpinLimit || sm.abort) {
        ok = false;
        break;
      }
      __nanosleep(20);
    }
    if (!__all_sync(kFull, ok)) {
      if (lane == 0 && !sm.abort) raise_abort(sm, a);
      break;
    }
    const int part = sm.ring_part[tl % kRing];
    const float aggf = sm.ring_agg[tl % kRing];
    __syncwarp();
    if (lane == 0) sm.ring_tail = tl + 1;
    if (part < 0) break;

    // The aggregate word validates itself (tag + float bits in one 64-bit store): no fence.
    if (lane == 0)
      st_u64(&a.aggw[part], (static_cast<unsigned long long>(tagA) << 32) | __float_as_uint(aggf));
    const bool big = static_cast<unsigned>(part) < a.nbig * a.group;
    const unsigned k = big ? static_cast<unsigned>(part) % a.group : 0u;
    if (k != have) {  // aggregates of a ticket arrive in order; anything else is a logic error
      if (lane == 0) raise_abort(sm, a);
      break;
    }
    have = k + 1;
    const unsigned in_ticket = big ? a.group : 1u;
    if (have < in_ticket) continue;
    have = 0;
#ifdef GEARB_SCAN_NO_LOOKBACK  // timing experiment only: level 1 is left unwritten
    continue;
#endif
    const unsigned sg = static_cast<unsigned>(part) / kSuper;
    const unsigned in_super = min(static_cast<unsigned>(kSuper), a.nparts - sg * kSuper);
    unsigned arrived = 0;
    if (lane == 0) arrived = atomicAdd(&a.gcount[sg], in_ticket) + in_ticket;
    arrived = __shfl_sync(kFull, arrived, 0);
    if (arrived == in_super) {
      if (lane == 0) a.gcount[sg] = 0u;  // last one to touch it: ready for the next launch
      finish_group(a, sg, epoch, lane);
    }
  }
}

// Last CTA out: rebuild level 1 in order if asked, then re-arm the header for the next launch.
__device__ void finish_launch(const ScanArgs &a, unsigned epoch, int tid) {
  if (tid == 0) {
    __threadfence();
    const unsigned d = atomicAdd(&a.hdr->done, 1u);
    if (d == gridDim.x - 1) {
      __threadfence();
      const unsigned flags = atomicOr(&a.hdr->pad[0], 0u);
      if (flags & kHdrRebuild) {
        double acc = 0.0;
        __stcg(&a.l1[0], 0.0);
        for (unsigned q = 0; q < a.nparts; ++q) {
          acc = __dadd_rn(acc, static_cast<double>(__uint_as_float(static_cast<unsigned>(__ldcg(&a.aggw[q])))));
          __stcg(&a.l1[q + 1], acc);
        }
        atomicOr(reinterpret_cast<unsigned *>(a.status), GEARB_ST_L1_RESUMMED);
      }
      if (atomicOr(reinterpret_cast<unsigned *>(a.status), 0u) & GEARB_ST_SCAN_ABORTED)
        for (unsigned g = 0; g < a.nsuper; ++g) a.gcount[g] = 0u;  // counters may be left half-way
      a.hdr->pad[0] = 0u;
      a.hdr->ticket = 0u;
      a.hdr->done = 0u;
      a.hdr->epoch = epoch + 1u;
      __threadfence();
    }
  }
}

template <bool kStore>
__global__ void __launch_bounds__(kThreads, 3) scan_kernel(const ScanArgs a) {
  extern __shared__ unsigned char smem_raw[];
  Smem &sm = *reinterpret_cast<Smem *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned epoch = ld_u32_relaxed(&a.hdr->epoch);
  // A kernel launched behind this one with programmatic stream serialisation may be scheduled
  // as this grid drains; it still waits (griddepcontrol.wait) for this grid to complete.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sm.full[s], 1);
      mbar_init(&sm.empty[s], kComputeWarps);
    }
    sm.ring_head = 0;
    sm.ring_tail = 0;
    sm.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncthreads();

  if (warp < kComputeWarps) compute_warps<kStore>(sm, a, warp, lane);
  else if (warp == kComputeWarps) loader_warp(sm, a, lane);
  else lookback_warp(sm, a, epoch, lane);

  __syncthreads();
  // Bulk copies still in flight into this CTA's shared memory (only after an abort) must land
  // before the CTA retires.
  if (sm.abort && tid == 0) {
    for (int s = 0; s < kStages; ++s)
      for (unsigned par = 0; par < 2; ++par) {
        unsigned spins = 0;
        while (!mbar_try_wait(&sm.full[s], par) && ++spins < 4096u) {}
      }
  }

  finish_launch(a, epoch, tid);
}

inline int64_t align256(int64_t v) { return (v + 255) & ~int64_t(255); }

}  // namespace

// Scratch layout: header | super-group counters (4 B) | super-group descriptors (32 B) |
// partition aggregate words (8 B).
int64_t scan_scratch_bytes(int64_t n) {
  const int64_t nparts = (n + kPart - 1) / kPart;
  const int64_t nsuper = (nparts + kSuper - 1) / kSuper;
  return static_cast<int64_t>(sizeof(ScanHeader)) + align256(nsuper * 4) + align256(nsuper * 32) +
         align256(nparts * 8);
}

int launch_scan(const float *prio, int64_t n, float *cdf, double *l1, void *scratch,
                int64_t scratch_bytes, int32_t *status, int fresh, cudaStream_t stream, int64_t layout_n) {
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
  const int64_t nsuper = (nparts + kSuper - 1) / kSuper;
  // A scratch block that serves calls of different sizes keeps ONE layout (that of layout_n):
  // the counters of a larger call must never land on words a smaller call used for something else.
  if (layout_n < n) layout_n = n;
  const int64_t lay_parts = (layout_n + kPart - 1) / kPart;
  const int64_t lay_super = (lay_parts + kSuper - 1) / kSuper;
  GEARB_REQUIRE(scratch_bytes >= scan_scratch_bytes(layout_n), "scan: scratch too small for its layout");
  const int64_t off_desc = sizeof(ScanHeader) + align256(lay_super * 4);
  const int64_t off_agg = off_desc + align256(lay_super * 32);
  if (fresh) {
    // Everything must start at zero: the epoch restarts at 0, so a stale tagged word could
    // otherwise pass for a fresh one.
    GEARB_CUDA(cudaMemsetAsync(sc, 0, static_cast<size_t>(scan_scratch_bytes(layout_n)), stream));
  }

  ScanArgs a;
  a.prio = prio;
  a.cdf = cdf;  // null: only level 1 and the aggregates are produced
  a.l1 = l1;
  a.hdr = reinterpret_cast<ScanHeader *>(sc);
  a.gcount = reinterpret_cast<unsigned *>(sc + sizeof(ScanHeader));
  a.desc = reinterpret_cast<unsigned long long *>(sc + off_desc);
  a.aggw = reinterpret_cast<unsigned long long *>(sc + off_agg);
  a.nsuper = static_cast<unsigned>(nsuper);
  a.status = status;
  a.n = n;
  a.nparts = static_cast<unsigned>(nparts);

  const size_t smem_bytes = sizeof(Smem) + 128;
  static int ctas_per_sm = 0;
  if (ctas_per_sm == 0) {
    GEARB_CUDA(cudaFuncSetAttribute(scan_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem_bytes)));
    GEARB_CUDA(cudaFuncSetAttribute(scan_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    static_cast<int>(smem_bytes)));
    int v = 0;
    GEARB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, scan_kernel<true>, kThreads, smem_bytes));
    ctas_per_sm = v > 0 ? v : 1;
  }
  const int64_t resident = static_cast<int64_t>(sm_count()) * ctas_per_sm;
  // Group partitions per ticket only when there is enough work to keep every CTA busy.
  a.group = nparts >= resident * kGroupMax * 2 ? kGroupMax : (nparts >= resident * 4 ? 2 : 1);
  // The last stretch (about two partitions per resident CTA) goes out one partition per ticket.
  const int64_t tail = resident * 2 < nparts ? resident * 2 : nparts;
  a.nbig = static_cast<unsigned>((nparts - tail) / a.group);
  a.ngroups = static_cast<unsigned>(a.nbig + (nparts - static_cast<int64_t>(a.nbig) * a.group));

  int64_t grid = resident;
  if (grid > a.ngroups) grid = a.ngroups;
  if (a.cdf) scan_kernel<true><<<static_cast<unsigned>(grid), kThreads, smem_bytes, stream>>>(a);
  else scan_kernel<false><<<static_cast<unsigned>(grid), kThreads, smem_bytes, stream>>>(a);
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

// ---------------------------------------------------------------------------------------
// Scratch that lives in the library image, for gearb_scan_static.
//
// kStaticMaxN priorities need kStaticScratchBytes of scratch; every device that loads this
// library reserves that much global memory until the process exits.
constexpr int64_t kStaticMaxN = int64_t(1) << 28;  // 268,435,456 priorities = 65,536 partitions
constexpr int64_t kStaticParts = kStaticMaxN / kPart;
constexpr int64_t kStaticSuper = kStaticParts / kSuper;
constexpr int64_t kStaticScratchBytes =
    sizeof(ScanHeader) + kStaticSuper * 4 + kStaticSuper * 32 + kStaticParts * 8;  // 672,000 B
static_assert(kStaticSuper * 4 % 256 == 0 && kStaticSuper * 32 % 256 == 0 && kStaticParts * 8 % 256 == 0,
              "the static scratch uses the same 256-byte aligned layout as scan_scratch_bytes()");

// In host code this name is only a handle for the symbol, not a device address: the address
// each device gave the array is asked for with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_static_scan_scratch[kStaticScratchBytes];

int64_t static_scan_max_n() { return kStaticMaxN; }

// Where a scratch block laid out for layout_n priorities keeps its per-partition aggregate words.
unsigned long long *scan_aggregate_words(void *scratch, int64_t layout_n) {
  const int64_t lay_parts = (layout_n + kPart - 1) / kPart;
  const int64_t lay_super = (lay_parts + kSuper - 1) / kSuper;
  return reinterpret_cast<unsigned long long *>(static_cast<char *>(scratch) + sizeof(ScanHeader) +
                                                align256(lay_super * 4) + align256(lay_super * 32));
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
  // The array starts zeroed when the module is loaded and every launch leaves it re-armed
  // (ticket and counters back at zero, epoch advanced, older words invalid by their tag), so
  // nothing has to be cleared between calls.
  return launch_scan(prio, n, cdf, l1, scratch, kStaticScratchBytes, status, /*fresh=*/0, stream, kStaticMaxN);
}

}  // namespace gearb
