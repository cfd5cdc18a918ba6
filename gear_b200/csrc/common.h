// Shared host-side helpers of libgear_b200: error text, CUDA checks, launch
// parameter structs exchanged between the C ABI layer and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "gear_b200.h"

namespace gearb {

// Thread-local text of the last failure; returned by gearb_last_error().
std::string &last_error();
int fail(int code, const char *fmt, ...);

#define GEARB_CUDA(expr)                                                              \
  do {                                                                                \
    cudaError_t e__ = (expr);                                                         \
    if (e__ != cudaSuccess)                                                           \
      return ::gearb::fail(GEARB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,            \
                           cudaGetErrorString(e__), __FILE__, __LINE__);              \
  } while (0)

#define GEARB_REQUIRE(cond, ...)                                                      \
  do {                                                                                \
    if (!(cond)) return ::gearb::fail(GEARB_ERR_INVALID, __VA_ARGS__);                \
  } while (0)

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// NVTX range around the host side of an entry point, so that the launches of a step can be told
// apart in a timeline (scan, level 1, sample + gather, publish, pull, all-to-all, update).  Costs a
// few nanoseconds when no tool is attached.
struct TraceRange {
  explicit TraceRange(const char *name);
  ~TraceRange();
  TraceRange(const TraceRange &) = delete;
  TraceRange &operator=(const TraceRange &) = delete;
};

// Number of SMs of the current device (cached per device).
int sm_count();

// Runs `setup` the first time it is called with `slot` on the current device (function
// attributes and occupancy figures are per device) and hands back the int it produced then.
// Thread-safe; slots are small integers, one per call site.
enum { kOnceScan = 0, kOnceLevel1 = 1, kOnceSampleGather = 2, kOnceSmallScan = 3, kOnceScanSearch = 4, kOnceSlots = 8 };
int per_device_once(int slot, int (*setup)(int *value), int *value);

// ---- scan ------------------------------------------------------------------
// First block of the scan scratch (the rest is laid out in scan.cu).
struct ScanHeader {
  unsigned int ticket;  // next ticket (group of partitions) to hand out
  unsigned int done;    // CTAs that have finished
  unsigned int aborted; // a bounded wait of the launch in flight ran out; cleared by its last CTA
  unsigned int pad[61];  // pad[1..24]: words shared with the level-1 launch (level1.cu)
};
static_assert(sizeof(ScanHeader) == 256, "header is one 256-byte block");
// Words of ScanHeader::pad beyond those the level-1 launch uses (level1.cu: 1-4, 9-24).
enum { kPadPublish = 30 };  // CTA counter of the publish launch

struct PublishTail;
int64_t scan_scratch_bytes(int64_t n);
// fresh != 0: scratch contents are unknown, clear them first (one memset).
// level1 == false: only the partitions' aggregates (and the cdf) are produced; the caller
// follows up with launch_level1 on scan_aggregate_words(scratch).  overlap_previous: the scan may
// start while the kernel before it in the stream finishes (that kernel must not read the cdf of
// this call; l1 is written by the level-1 launch, which waits for everything before it).
int launch_scan(const float *prio, int64_t n, float *cdf, double *l1, void *scratch,
                int64_t scratch_bytes, int32_t *status, int fresh, cudaStream_t stream,
                bool level1 = true, bool overlap_previous = false, float *blkw = nullptr, double *sb = nullptr,
                const PublishTail *publish = nullptr);
// sb (tables of more than 1024 partitions): one float64 per GEARB_SUPER_PARTS partitions, zero before
// the launch, receives the sums of their aggregates; the level-1 launch for this scan gets the
// same pointer and zeroes the words again at its end.
#define GEARB_SUPER_PARTS 128
// Bytes per piece of a request's column in the fused launches' ring of bulk copies.
#ifndef GEARB_SG_PIECE
#define GEARB_SG_PIECE 4096
#endif
int64_t static_scan_max_n();
int launch_scan_static(const float *prio, int64_t n, float *cdf, double *l1, int32_t *status,
                       cudaStream_t stream);
float *scan_aggregate_words(void *scratch);
// sb: superblock sums to zero at the end (or null).  after_next: the launch sits BEHIND the next
// scan in the stream instead of in front of it (that scan works in the other scratch block, and
// began only when the one whose aggregates these are was complete): it starts at once, works
// beside that scan, and waits for it only before its clean-up -- so whatever follows finds both
// complete, and nothing that still reads the header words or the sums can be running.
bool level1_can_follow_next_scan(int64_t nparts);
// A rank's total and the step's number into every rank's mailbox, done by the level-1 launch
// itself at its end (the place of a separate publish launch without a level-1 copy).
struct PublishTail {
  void *box[GEARB_MAX_SHARDS];
  int world = 0;  // 0: nothing to publish
  int rank = 0;
  unsigned long long epoch = 0;
};
int launch_level1(const float *agg, int64_t nparts, double *l1, unsigned *clear_word, int32_t *status,
                  cudaStream_t stream, ScanHeader *hdr, bool have_range, double *sb = nullptr,
                  bool after_next = false, const PublishTail *publish = nullptr);
int64_t update_scratch_bytes(int64_t n);
int launch_update(float *prio, int64_t n, float *cdf, double *l1, float *aggw, float *blkw, ScanHeader *hdr,
                  void *upd, const int64_t *idx, const float *val, int64_t m, int32_t *status, cudaStream_t stream);
// Scan (level-2 table stored, level 1, block totals) and draw in one cooperative launch; *fused = 0
// and nothing launched when the table has more partitions than CTAs can be resident at once.
int launch_scan_search(const float *prio, int64_t n, float *cdf, double *l1, void *scratch, int64_t scratch_bytes,
                       int32_t *status, float *blkw, const double *u, int64_t b, int flags, int64_t *out,
                       cudaStream_t stream, int *fused);
int launch_search(const float *cdf, const double *l1, int64_t n, const double *u, int64_t b,
                  int flags, int64_t *out, int32_t *status, cudaStream_t stream);
int launch_uniform(int64_t n, const double *u01, int64_t b, int64_t *out, cudaStream_t stream);
int launch_decode(const int64_t *flat, int64_t b, int64_t T, const int64_t *lengths,
                  int64_t index_offset, int64_t *idx, int64_t *ts, int64_t *len,
                  cudaStream_t stream);

// ---- gather ----------------------------------------------------------------
struct GatherColumn {
  int64_t col_offset;  // byte offset of the column inside one trajectory (accu * T)
  uint8_t *dst;        // [n, pat_length * row] bytes
  int32_t row;         // bytes per timestep
  int32_t pat_offset;  // SubscribePattern::offset
  int32_t pat_length;  // SubscribePattern::length
  int32_t pad_head;    // 1 when PadOption::kHead
  int32_t chunk_first; // first chunk id of this column inside a request
  int32_t chunk_count; // chunks this column's slot is cut into
  int32_t stage_off;   // byte offset of this column's staging area in shared memory
  int32_t reserved;
};

struct GatherParams {
  const uint8_t *table;
  const int64_t *idx, *ts, *len;
  int64_t n;
  int64_t traj_stride;
  int64_t capacity;  // trajectories in the table (bounds check)
  int64_t T;         // trajectory_length (length clamp)
  int32_t *status;   // may be null
  int32_t ncols;
  int32_t chunks_per_request;
  int32_t chunk_bytes;
  int32_t zero_fill;
  int32_t stage_bytes;  // > 0: a request's columns fit this much shared memory and the table is in HBM
  int32_t ring;         // 1: larger requests stream through per-warp rings of bulk copies
  // Where request g of a launch lands in the destinations (sample_gather only).  Position
  // q = slot_lo + g of the global batch goes to
  //   slot_mod == 0:  slot g;
  //   slot_mod  > 1:  slot_base[q % slot_mod] + q / slot_mod -- an owner that serves a run of a batch
  //                   dealt round-robin to slot_mod requesters groups its answers by requester;
  //   slot_mod == -1: q - slot_base[0] when slot_base[0] <= q < slot_base[1] (the owner's own
  //                   contiguous slice: straight into its final place), else slot_base[2] + g.
  int32_t slot_mod;
  int64_t slot_lo;
  int64_t slot_base[GEARB_MAX_SHARDS];
  GatherColumn cols[GEARB_MAX_COLUMNS];
};

// How the sampling kernels address their variates and number their results.
struct DrawLayout {
  int64_t u_stride = 1;     // request g reads variate u[g * u_stride]
  int64_t flat_offset = 0;  // added to every flat step index written to out_flat
};

// What a scan leaves besides level 1, enough to find a variate's partition and its offset
// before the level-1 table exists: the sums of the aggregates of every GEARB_SUPER_PARTS
// partitions, the aggregates, and the two header words with their exponent range.
struct Level1Sums {
  const double *sb;
  const float *agg;
  const unsigned *range;
  int ctas_per_sm;  // > 0: a scan is expected to start under this launch; it leaves room with this many CTAs per SM
};

int launch_gather(const GatherParams &p, cudaStream_t stream);
// sums (with lazy_prio, local tables): l1 has not been built yet, see Level1Sums.
// lazy_prio / lazy_blk: the table was built without its level-2 entries; the kernel rebuilds what a
// request needs from the priorities and the per-block totals the scan left (8 floats per partition).
int launch_sample_gather(const GatherParams &p, const float *cdf, const double *l1, int64_t n,
                         const double *u, int flags, const int64_t *lengths, int64_t index_offset,
                         int64_t *out_flat, int64_t *out_idx, int64_t *out_ts, int64_t *out_len,
                         cudaStream_t stream, double mul = 1.0, double sub = 0.0,
                         const float *lazy_prio = nullptr, const float *lazy_blk = nullptr,
                         const DrawLayout &lay = DrawLayout(), const Level1Sums *sums = nullptr);
// Per shard: either its stored level-2 table (peer_cdf) or its priorities and block totals
// (peer_prio, peer_blk; peer_cdf null).  peer_l1 may point at local copies of the peers' level 1.
int launch_pull(const GatherParams &p, int world, int self, const double *totals, const void *const *peer_cdf,
                const void *const *peer_prio, const void *const *peer_blk, const void *const *peer_l1,
                const void *const *peer_table, int64_t n, const double *u, int64_t *out_flat, int64_t *out_idx,
                int64_t *out_ts, cudaStream_t stream, const void *mailbox, unsigned long long epoch,
                const DrawLayout &lay);
// Mailbox layout (one per rank, GEARB_MAILBOX_BYTES of header, then optional level-1 copies).
// behind the level-1 copies: copies of the block totals [2 slots][GEARB_MAX_SHARDS] of blk_stride bytes each
int64_t mailbox_l1_stride(int64_t n);
int64_t mailbox_blk_stride(int64_t n);
int64_t mailbox_blk_base(int64_t n);
// blk (with copy_l1): the rank's block totals of the step travel with its level 1.
int launch_publish(const double *l1, int64_t nparts, int world, int rank, void *const *mailboxes,
                   unsigned long long epoch, int copy_l1, unsigned *counter, cudaStream_t stream,
                   const float *blk = nullptr);
int launch_vcopy(const uint8_t *src, uint8_t *dst, const int64_t *src_off,
                 const int64_t *dst_off, const int64_t *lengths, int64_t fixed_length,
                 int64_t n, int64_t max_length, cudaStream_t stream);

int launch_fill(void *dst, int64_t count, int kind, uint64_t seed, uint64_t stream_id, double a,
                double b, cudaStream_t stream);

}  // namespace gearb
