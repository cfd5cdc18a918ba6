// Trajectory-segment gather.
//
// gather_kernel is the fused multi-column form of the reference's
// fused_subcopy_collect (src/cuda/copy.cu:91-134): per request g and subscribed
// column it clips [ts+offset, ts+offset+length) to [0, len), and moves the
// clipped rows from  table + idx*trajectory_stride + column_offset + start*row
// to  dst + g*slot (+ slot - bytes when padding at the head), the addressing of
// CpuTrajectoryStorageHandler::sub (src/storage/handler.cc:78-131).
// vcopy_kernel is the generic offset-list form (vary_/fix_stride_copy_collect,
// src/cuda/copy.cu:12-89).
//
// Differences in HOW, not in WHAT:
//  * all subscribed columns of a batch go in one launch;
//  * one warp moves one 2 KiB piece of a slot with 16-byte accesses that are
//    consecutive across the lanes (the reference gives each thread its own 64
//    bytes, so a warp's 16-byte loads sit 64 bytes apart);
//  * source and destination may have any byte alignment: stores are aligned to
//    the destination, and a misaligned source is read as two aligned 16-byte
//    blocks that are funnel-shifted together (the reference casts both sides to
//    float4 and is only defined for 16-byte aligned addresses);
//  * all offsets are 64-bit (the reference's kernel parameters are int);
//  * a trajectory index outside the table is skipped and reported through the
//    status word instead of being dereferenced.
// The source pointer may be HBM or pinned mapped host memory; the code is the same.
#include "common.h"

namespace gearb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;
constexpr int kUnroll = 4;

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

// One warp copies nbytes from s to d; any alignment on either side.
// Reads touch only 16-byte aligned blocks that contain at least one source byte.
__device__ __forceinline__ void warp_copy(uint8_t *d, const uint8_t *s, int nbytes, int lane) {
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
        if (v0 + 32 * u < nvec) r[u] = ld_nc(sv + v0 + 32 * u);
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
          a[u] = ld_nc(sv + v0 + 32 * u);
          b[u] = ld_nc(sv + v0 + 32 * u + 1);
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

__global__ void __launch_bounds__(kThreads) gather_kernel(const __grid_constant__ GatherParams P) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;
  const int64_t items = P.n * P.chunks_per_request;
  unsigned flags = 0;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
       item < items; item += warps_total) {
    const int64_t g = item / P.chunks_per_request;
    const int q = static_cast<int>(item - g * P.chunks_per_request);
    int c = 0;
    while (c + 1 < P.ncols && q >= P.cols[c + 1].chunk_first) ++c;
    const GatherColumn &col = P.cols[c];
    const int cq = q - col.chunk_first;

    const int64_t idx = __ldg(P.idx + g), ts = __ldg(P.ts + g);
    int64_t len = __ldg(P.len + g);
    const int64_t row = col.row;
    const int64_t slot = row * col.pat_length;
    int64_t bytes = 0, start = 0;
    if (idx < 0 || idx >= P.capacity) {
      flags |= GEARB_ST_BAD_REQUEST;
    } else {
      if (len > P.T) {
        len = P.T;
        flags |= GEARB_ST_LEN_CLAMPED;
      }
      start = ts + col.pat_offset;
      if (start < 0) start = 0;
      int64_t end = start + col.pat_length;
      if (end > len) end = len;
      const int64_t steps = end - start;
      bytes = steps > 0 ? steps * row : 0;
    }
    const int64_t data_off = col.pad_head ? slot - bytes : 0;
    const int64_t c0 = static_cast<int64_t>(cq) * P.chunk_bytes;
    int64_t c1 = c0 + P.chunk_bytes;
    if (c1 > slot) c1 = slot;
    uint8_t *dslot = col.dst + g * slot;

    const int64_t lo = c0 > data_off ? c0 : data_off;
    const int64_t hi = c1 < data_off + bytes ? c1 : data_off + bytes;
    if (hi > lo) {
      const uint8_t *src = P.table + idx * P.traj_stride + col.col_offset + start * row;
      warp_copy(dslot + lo, src + (lo - data_off), static_cast<int>(hi - lo), lane);
    }
    if (P.zero_fill) {
      // padding before the data (head padding) and after it (tail padding)
      const int64_t z1 = c1 < data_off ? c1 : data_off;
      if (z1 > c0) warp_zero(dslot + c0, static_cast<int>(z1 - c0), lane);
      const int64_t z0 = c0 > data_off + bytes ? c0 : data_off + bytes;
      if (c1 > z0) warp_zero(dslot + z0, static_cast<int>(c1 - z0), lane);
    }
  }
  if (flags && P.status && lane == 0) atomicOr(reinterpret_cast<unsigned *>(P.status), flags);
}

struct VcopyArgs {
  const uint8_t *src;
  uint8_t *dst;
  const int64_t *src_off, *dst_off, *lengths;
  int64_t fixed_length;  // used when lengths == nullptr
  int64_t n;
  int32_t chunks_per_slice;
  int32_t chunk_bytes;
};

__global__ void __launch_bounds__(kThreads) vcopy_kernel(const VcopyArgs a) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;
  const int64_t items = a.n * a.chunks_per_slice;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
       item < items; item += warps_total) {
    const int64_t g = item / a.chunks_per_slice;
    const int64_t c0 = (item - g * a.chunks_per_slice) * a.chunk_bytes;
    const int64_t length = a.lengths ? __ldg(a.lengths + g) : a.fixed_length;
    int64_t c1 = c0 + a.chunk_bytes;
    if (c1 > length) c1 = length;
    if (c1 > c0)
      warp_copy(a.dst + __ldg(a.dst_off + g) + c0, a.src + __ldg(a.src_off + g) + c0,
                static_cast<int>(c1 - c0), lane);
  }
}

int grid_for(int64_t items) {
  int64_t blocks = (items + kWarpsPerBlock - 1) / kWarpsPerBlock;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 64;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace

int launch_gather(const GatherParams &p, cudaStream_t stream) {
  if (p.n == 0 || p.ncols == 0) return GEARB_OK;
  const int64_t items = p.n * p.chunks_per_request;
  gather_kernel<<<grid_for(items), kThreads, 0, stream>>>(p);
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

int launch_vcopy(const uint8_t *src, uint8_t *dst, const int64_t *src_off,
                 const int64_t *dst_off, const int64_t *lengths, int64_t fixed_length, int64_t n,
                 int64_t max_length, cudaStream_t stream) {
  GEARB_REQUIRE(n >= 0 && max_length >= 0, "vcopy: negative count or length");
  if (n == 0 || max_length == 0) return GEARB_OK;
  GEARB_REQUIRE(src && dst && src_off && dst_off, "vcopy: null pointer argument");
  VcopyArgs a;
  a.src = src; a.dst = dst; a.src_off = src_off; a.dst_off = dst_off; a.lengths = lengths;
  a.fixed_length = fixed_length; a.n = n;
  a.chunk_bytes = 2048;
  const int64_t cps = (max_length + a.chunk_bytes - 1) / a.chunk_bytes;
  GEARB_REQUIRE(cps < (int64_t(1) << 31), "vcopy: max_length too large");
  a.chunks_per_slice = static_cast<int32_t>(cps);
  vcopy_kernel<<<grid_for(n * cps), kThreads, 0, stream>>>(a);
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

}  // namespace gearb
