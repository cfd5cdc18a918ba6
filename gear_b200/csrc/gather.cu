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
#include "device_copy.cuh"

namespace gearb {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;
using dev::warp_copy;

__global__ void __launch_bounds__(kThreads) gather_kernel(const __grid_constant__ GatherParams P) {
  const int lane = threadIdx.x & 31;
  const int64_t warps_total = static_cast<int64_t>(gridDim.x) * kWarpsPerBlock;
  const int64_t items = P.n * P.chunks_per_request;
  unsigned flags = 0;
  for (int64_t item = static_cast<int64_t>(blockIdx.x) * kWarpsPerBlock + (threadIdx.x >> 5);
       item < items; item += warps_total) {
    const int64_t g = item / P.chunks_per_request;
    const int q = static_cast<int>(item - g * P.chunks_per_request);
    const int c = dev::column_of_piece(P, q);
    dev::gather_piece(P, P.cols[c], q - P.cols[c].chunk_first, g, __ldg(P.idx + g), __ldg(P.ts + g),
                      __ldg(P.len + g), lane, flags, P.table);
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
