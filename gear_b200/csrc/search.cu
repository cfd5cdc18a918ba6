// Batched draws on caller-supplied variates.
//
// search_kernel: prioritized draw through the two-level cumulative table -- the
// place torch.multinomial has in the reference (gear/sampler/global_sampler.py:170),
// restated so that it consumes external variates: "first entry greater than the
// variate" at both levels (zero priorities repeat their predecessor's entry and
// are never selected; "weight = 0 indicates unselectable", src/index/server.cc:147).
// uniform_kernel: floor(u*n), the place of torch.randint (global_sampler.py:121-129).
// decode: flat step index -> GEAR's (trajectory, timestep, length) request triple.
//
// One warp serves one variate and narrows the range 256-fold per round (eight probes per
// lane, all in flight together), so a draw costs about four dependent memory round trips
// instead of ~27: level 1 of a table of up to 256 partitions in one, level 2 in two.
#include "common.h"
#include "warp_search.cuh"

namespace gearb {
namespace {

constexpr int kThreads = 256;

struct SearchArgs {
  const float *cdf;
  const double *l1;
  const double *u;
  int64_t *out;
  int32_t *status;
  int64_t n, b, nparts;
  int flags;
  // optional fused decode
  int64_t T, index_offset;
  const int64_t *lengths;
  int64_t *idx, *ts, *len;
};

__global__ void __launch_bounds__(kThreads) search_kernel(const SearchArgs a) {
  // Launched with programmatic stream serialisation: the grid may be scheduled while the scan
  // before it drains (a small table's scan says so at its start), and waits here until that
  // scan's tables are complete and visible.  What is launched behind this kernel may be
  // scheduled from here on; it finds everything before this kernel complete.
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane = threadIdx.x & 31;
  const int64_t w = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
  if (w >= a.b) return;

  const double total = __ldg(a.l1 + a.nparts);
  if (!(total > 0.0)) {  // no selectable entry at all: defined as the last index
    if (lane == 0) {
      const int64_t flat = a.n - 1;
      a.out[w] = flat;
      if (a.idx) {
        const int64_t t = flat / a.T;
        a.idx[w] = t + a.index_offset;
        a.ts[w] = flat - t * a.T;
        a.len[w] = a.lengths ? __ldg(a.lengths + t) : a.T;
      }
    }
    return;
  }
  double v = __ldg(a.u + w);
  if (a.flags & GEARB_SEARCH_SCALE) v = __dmul_rn(v, total);
  if (!(v >= 0.0)) v = 0.0;
  if (!(v < total)) v = __longlong_as_double(__double_as_longlong(total) - 1);  // next below total

  // level 1: partition p with l1[p] <= v < l1[p+1]
  const int64_t p = warp_upper_bound<double>(a.l1 + 1, 0, a.nparts - 1, v, lane, LoadReadOnly());
  const int64_t base = p * GEARB_PART;
  const int64_t valid = (a.n - base < GEARB_PART) ? (a.n - base) : GEARB_PART;
  float r = __double2float_rn(__dsub_rn(v, __ldg(a.l1 + p)));
  const float last = __ldg(a.cdf + base + valid - 1);
  if (!(r < last)) r = __uint_as_float(__float_as_uint(last) - 1u);  // next below last (> 0)

  // level 2: first entry of the partition greater than r
  const int64_t j = warp_upper_bound<float>(a.cdf + base, 0, valid - 1, r, lane, LoadReadOnly());
  const int64_t flat = base + j;

  if (lane == 0) {
    a.out[w] = flat;
    if (a.idx) {
      const int64_t t = flat / a.T;
      a.idx[w] = t + a.index_offset;
      a.ts[w] = flat - t * a.T;
      a.len[w] = a.lengths ? __ldg(a.lengths + t) : a.T;
    }
    if (a.status) {
      const float hi_b = __ldg(a.cdf + flat);
      bool near = __uint_as_float(__float_as_uint(r) + 1u) >= hi_b;  // r >= 0: bits+1 is next above
      if (j > 0 && r == __ldg(a.cdf + flat - 1)) near = true;
      if (near) atomicAdd(a.status + 1, 1);
    }
  }
}

__global__ void uniform_kernel(int64_t n, const double *u01, int64_t b, int64_t *out) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= b) return;
  double v = u01[i];
  if (!(v >= 0.0)) v = 0.0;
  int64_t k = static_cast<int64_t>(floor(__dmul_rn(v, static_cast<double>(n))));
  if (k >= n) k = n - 1;
  out[i] = k;
}

__global__ void decode_kernel(const int64_t *flat, int64_t b, int64_t T, const int64_t *lengths,
                              int64_t index_offset, int64_t *idx, int64_t *ts, int64_t *len) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= b) return;
  const int64_t f = flat[i];
  const int64_t t = f / T;
  idx[i] = t + index_offset;
  ts[i] = f - t * T;
  len[i] = lengths ? lengths[t] : T;
}

}  // namespace

int launch_search_ex(const float *cdf, const double *l1, int64_t n, const double *u, int64_t b,
                     int flags, int64_t *out, int32_t *status, int64_t T, const int64_t *lengths,
                     int64_t index_offset, int64_t *idx, int64_t *ts, int64_t *len,
                     cudaStream_t stream) {
  GEARB_REQUIRE(n > 0 && b >= 0, "search: n must be positive and b non-negative");
  if (b == 0) return GEARB_OK;
  GEARB_REQUIRE(cdf && l1 && u && out, "search: null pointer argument");
  GEARB_REQUIRE(!idx || (ts && len && T > 0), "search: decode needs idx, ts, len and T > 0");
  SearchArgs a;
  a.cdf = cdf; a.l1 = l1; a.u = u; a.out = out; a.status = status;
  a.n = n; a.b = b; a.nparts = (n + GEARB_PART - 1) / GEARB_PART;
  a.flags = flags;
  a.T = T; a.index_offset = index_offset; a.lengths = lengths;
  a.idx = idx; a.ts = ts; a.len = len;
  const int64_t blocks = (b * 32 + kThreads - 1) / kThreads;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(blocks));
  cfg.blockDim = dim3(kThreads);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  GEARB_CUDA(cudaLaunchKernelEx(&cfg, search_kernel, a));
  return GEARB_OK;
}

int launch_search(const float *cdf, const double *l1, int64_t n, const double *u, int64_t b,
                  int flags, int64_t *out, int32_t *status, cudaStream_t stream) {
  return launch_search_ex(cdf, l1, n, u, b, flags, out, status, 0, nullptr, 0, nullptr, nullptr,
                          nullptr, stream);
}

int launch_uniform(int64_t n, const double *u01, int64_t b, int64_t *out, cudaStream_t stream) {
  GEARB_REQUIRE(n > 0 && b >= 0, "sample_uniform: n must be positive and b non-negative");
  if (b == 0) return GEARB_OK;
  GEARB_REQUIRE(u01 && out, "sample_uniform: null pointer argument");
  uniform_kernel<<<static_cast<unsigned>((b + 255) / 256), 256, 0, stream>>>(n, u01, b, out);
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

int launch_decode(const int64_t *flat, int64_t b, int64_t T, const int64_t *lengths,
                  int64_t index_offset, int64_t *idx, int64_t *ts, int64_t *len,
                  cudaStream_t stream) {
  GEARB_REQUIRE(T > 0 && b >= 0, "decode: trajectory_length must be positive");
  if (b == 0) return GEARB_OK;
  GEARB_REQUIRE(flat && idx && ts && len, "decode: null pointer argument");
  decode_kernel<<<static_cast<unsigned>((b + 255) / 256), 256, 0, stream>>>(
      flat, b, T, lengths, index_offset, idx, ts, len);
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

}  // namespace gearb
