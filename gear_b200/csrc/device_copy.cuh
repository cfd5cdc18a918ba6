// Device-side building blocks of the gather kernels: a warp-wide byte copy that
// accepts any alignment on either side, and the per-request addressing of
// CpuTrajectoryStorageHandler::sub (src/storage/handler.cc:78-131 of the
// reference) applied to one 2 KiB piece of one column's slot.
#pragma once

#include "common.h"

namespace gearb {
namespace dev {

__device__ __forceinline__ uint4 ld_nc(const uint4 *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// Bytes [sh, sh+16) of the 32-byte pair (a,b); sh in 1..15.
__device__ __forceinline__ uint4 shift_pair(const uint4 &a, const uint4 &b, unsigned ws,
                                            unsigned bs) {
  uint4 o;
  switch (ws) {
    case 0:
      o.x = __funnelshift_r(a.x, a.y, bs); o.y = __funnelshift_r(a.y, a.z, bs);
      o.z = __funnelshift_r(a.z, a.w, bs); o.w = __funnelshift_r(a.w, b.x, bs);
      break;
    case 1:
      o.x = __funnelshift_r(a.y, a.z, bs); o.y = __funnelshift_r(a.z, a.w, bs);
      o.z = __funnelshift_r(a.w, b.x, bs); o.w = __funnelshift_r(b.x, b.y, bs);
      break;
    case 2:
      o.x = __funnelshift_r(a.z, a.w, bs); o.y = __funnelshift_r(a.w, b.x, bs);
      o.z = __funnelshift_r(b.x, b.y, bs); o.w = __funnelshift_r(b.y, b.z, bs);
      break;
    default:
      o.x = __funnelshift_r(a.w, b.x, bs); o.y = __funnelshift_r(b.x, b.y, bs);
      o.z = __funnelshift_r(b.y, b.z, bs); o.w = __funnelshift_r(b.z, b.w, bs);
      break;
  }
  return o;
}

template <bool kSmemSrc>
__device__ __forceinline__ uint4 load16(const uint4 *p) {
  if constexpr (kSmemSrc) return *p;  // staged in shared memory: an ordinary load
  else return ld_nc(p);
}

// One warp copies nbytes from s to d; any alignment on either side.
// Reads touch only 16-byte aligned blocks that contain at least one source byte.
// kSmemSrc: the source was staged in shared memory.
template <bool kSmemSrc>
__device__ __forceinline__ void warp_copy_t(uint8_t *d, const uint8_t *s, int nbytes, int lane) {
  // Loads in flight per lane: global sources need several to cover the latency, shared ones do not.
  constexpr int kUnroll = kSmemSrc ? 1 : 4;
  int head = static_cast<int>((16u - (reinterpret_cast<uintptr_t>(d) & 15u)) & 15u);
  if (head > nbytes) head = nbytes;
  if (lane < head) d[lane] = s[lane];
  d += head;
  s += head;
  nbytes -= head;
  const int nvec = nbytes >> 4;
  const unsigned sh = static_cast<unsigned>(reinterpret_cast<uintptr_t>(s) & 15u);
  uint4 *dv = reinterpret_cast<uint4 *>(d);
  if (sh == 0) {
    const uint4 *sv = reinterpret_cast<const uint4 *>(s);
    for (int v0 = lane; v0 < nvec; v0 += 32 * kUnroll) {
      uint4 r[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v0 + 32 * u < nvec) r[u] = load16<kSmemSrc>(sv + v0 + 32 * u);
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v0 + 32 * u < nvec) dv[v0 + 32 * u] = r[u];
    }
  } else {
    const uint4 *sv = reinterpret_cast<const uint4 *>(s - sh);
    const unsigned ws = sh >> 2, bs = (sh & 3u) * 8u;
    for (int v0 = lane; v0 < nvec; v0 += 32 * kUnroll) {
      uint4 a[kUnroll], b[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v0 + 32 * u < nvec) {
          a[u] = load16<kSmemSrc>(sv + v0 + 32 * u);
          b[u] = load16<kSmemSrc>(sv + v0 + 32 * u + 1);
        }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u)
        if (v0 + 32 * u < nvec) dv[v0 + 32 * u] = shift_pair(a[u], b[u], ws, bs);
    }
  }
  const int done = nvec << 4;
  const int tail = nbytes - done;
  if (lane < tail) d[done + lane] = s[done + lane];
}

__device__ __forceinline__ void warp_copy(uint8_t *d, const uint8_t *s, int nbytes, int lane) {
  warp_copy_t<false>(d, s, nbytes, lane);
}

__device__ __forceinline__ void warp_zero(uint8_t *d, int nbytes, int lane) {
  int head = static_cast<int>((16u - (reinterpret_cast<uintptr_t>(d) & 15u)) & 15u);
  if (head > nbytes) head = nbytes;
  if (lane < head) d[lane] = 0;
  d += head;
  nbytes -= head;
  const int nvec = nbytes >> 4;
  uint4 *dv = reinterpret_cast<uint4 *>(d);
  const uint4 z = make_uint4(0, 0, 0, 0);
  for (int v = lane; v < nvec; v += 32) dv[v] = z;
  const int done = nvec << 4;
  if (lane < nbytes - done) d[done + lane] = 0;
}


// The clipped segment of column `col` for request (idx, ts, len): first timestep and byte
// count, the addressing of CpuTrajectoryStorageHandler::sub (handler.cc:104-115).
__device__ __forceinline__ void clip_segment(const GatherParams &P, const GatherColumn &col, int64_t idx,
                                             int64_t ts, int64_t len, int64_t &start, int64_t &bytes,
                                             unsigned &flags) {
  bytes = 0;
  start = 0;
  if (idx < 0 || idx >= P.capacity) {
    flags |= GEARB_ST_BAD_REQUEST;
    return;
  }
  if (len > P.T) {
    len = P.T;
    flags |= GEARB_ST_LEN_CLAMPED;
  }
  start = ts + col.pat_offset;
  if (start < 0) start = 0;
  int64_t end = start + col.pat_length;
  if (end > len) end = len;
  const int64_t steps = end - start;
  bytes = steps > 0 ? steps * static_cast<int64_t>(col.row) : 0;
}

// One warp handles piece `cq` of request g's slot of column `col`: copies the part of the
// segment (`bytes` bytes starting at `data`) that falls into the piece and, when asked,
// zero-fills the padding that falls into it.
template <bool kSmemSrc>
__device__ __forceinline__ void copy_piece(const GatherParams &P, const GatherColumn &col, int cq, int64_t g,
                                           const uint8_t *data, int64_t bytes, int lane) {
  const int64_t slot = static_cast<int64_t>(col.row) * col.pat_length;
  const int64_t data_off = col.pad_head ? slot - bytes : 0;
  const int64_t c0 = static_cast<int64_t>(cq) * P.chunk_bytes;
  int64_t c1 = c0 + P.chunk_bytes;
  if (c1 > slot) c1 = slot;
  uint8_t *dslot = col.dst + g * slot;
  const int64_t lo = c0 > data_off ? c0 : data_off;
  const int64_t hi = c1 < data_off + bytes ? c1 : data_off + bytes;
  if (hi > lo) warp_copy_t<kSmemSrc>(dslot + lo, data + (lo - data_off), static_cast<int>(hi - lo), lane);
  if (P.zero_fill) {
    // padding before the data (head padding) and after it (tail padding)
    const int64_t z1 = c1 < data_off ? c1 : data_off;
    if (z1 > c0) warp_zero(dslot + c0, static_cast<int>(z1 - c0), lane);
    const int64_t z0 = c0 > data_off + bytes ? c0 : data_off + bytes;
    if (c1 > z0) warp_zero(dslot + z0, static_cast<int>(c1 - z0), lane);
  }
}

// What piece `cq` of request g's slot of column `col` consists of: `len` data bytes going to
// `dst` (their offset inside the clipped segment is `seg_off`), and up to two runs of padding.
struct PieceInfo {
  uint8_t *dst;
  int64_t seg_off;
  int len;
  uint8_t *zero_a, *zero_b;
  int zero_a_len, zero_b_len;
};

__device__ __forceinline__ PieceInfo piece_info(const GatherParams &P, const GatherColumn &col, int cq, int64_t g,
                                                int64_t bytes) {
  const int64_t slot = static_cast<int64_t>(col.row) * col.pat_length;
  const int64_t data_off = col.pad_head ? slot - bytes : 0;
  const int64_t c0 = static_cast<int64_t>(cq) * P.chunk_bytes;
  int64_t c1 = c0 + P.chunk_bytes;
  if (c1 > slot) c1 = slot;
  uint8_t *dslot = col.dst + g * slot;
  const int64_t lo = c0 > data_off ? c0 : data_off;
  const int64_t hi = c1 < data_off + bytes ? c1 : data_off + bytes;
  PieceInfo pi;
  pi.dst = dslot + lo;
  pi.seg_off = lo - data_off;
  pi.len = hi > lo ? static_cast<int>(hi - lo) : 0;
  const int64_t z1 = c1 < data_off ? c1 : data_off;
  pi.zero_a = dslot + c0;
  pi.zero_a_len = (P.zero_fill && z1 > c0) ? static_cast<int>(z1 - c0) : 0;
  const int64_t z0 = c0 > data_off + bytes ? c0 : data_off + bytes;
  pi.zero_b = dslot + z0;
  pi.zero_b_len = (P.zero_fill && c1 > z0) ? static_cast<int>(c1 - z0) : 0;
  return pi;
}

// Address of the segment's first byte in the table.
// `table` is the base of the table that holds trajectory idx: P.table, or a peer shard's.
__device__ __forceinline__ const uint8_t *segment_src(const GatherParams &P, const GatherColumn &col, int64_t idx,
                                                      int64_t start, const uint8_t *table) {
  return table + idx * P.traj_stride + col.col_offset + start * static_cast<int64_t>(col.row);
}

// Straight from the table (HBM or mapped host memory) to the destination.
__device__ __forceinline__ void gather_piece(const GatherParams &P, const GatherColumn &col, int cq,
                                             int64_t g, int64_t idx, int64_t ts, int64_t len, int lane,
                                             unsigned &flags, const uint8_t *table) {
  int64_t start, bytes;
  clip_segment(P, col, idx, ts, len, start, bytes, flags);
  copy_piece<false>(P, col, cq, g, bytes > 0 ? segment_src(P, col, idx, start, table) : table, bytes, lane);
}

// Column that owns piece q of a request (pieces are numbered column by column).
__device__ __forceinline__ int column_of_piece(const GatherParams &P, int q) {
  int c = 0;
  while (c + 1 < P.ncols && q >= P.cols[c + 1].chunk_first) ++c;
  return c;
}

}  // namespace dev
}  // namespace gearb
