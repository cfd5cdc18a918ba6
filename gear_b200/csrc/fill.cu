// Device-side Philox4x32-10 fills for synthetic benchmark tables.
//
// The reference has no generator: its example converts a downloaded D4RL file
// (examples/offline/single-node/create.py:12-17).  Benchmark tables here are
// seeded synthetic data of the same shapes, and the largest ones (18.9 GB,
// 131 GB) are written directly in HBM by these kernels.
//
// Conventions (shared with the CPU checker so integer kinds match bit for bit):
//   32-bit word i  = lane (i & 3) of Philox block (i >> 2)        (U32, I32_RANGE, U8)
//   U[0,1) double i = 53 bits of block i: (w0 << 21) ^ (w1 >> 11) (U01_F64, F32_UNIFORM)
//   N(0,1) value i  = Box-Muller on the doubles of blocks 2i and 2i+1, in float64
// Float kinds go through CUDA's log/cos/exp and agree with a host libm only to
// rounding, not bit for bit.
#include "common.h"

namespace gearb {
namespace {

struct Block { uint32_t w[4]; };

__device__ __forceinline__ Block philox(uint64_t seed, uint64_t stream, uint64_t counter) {
  uint32_t c0 = static_cast<uint32_t>(counter), c1 = static_cast<uint32_t>(counter >> 32);
  uint32_t c2 = static_cast<uint32_t>(stream), c3 = static_cast<uint32_t>(stream >> 32);
  uint32_t k0 = static_cast<uint32_t>(seed), k1 = static_cast<uint32_t>(seed >> 32);
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t h0 = __umulhi(0xD2511F53u, c0), l0 = 0xD2511F53u * c0;
    const uint32_t h1 = __umulhi(0xCD9E8D57u, c2), l1 = 0xCD9E8D57u * c2;
    const uint32_t n0 = h1 ^ c1 ^ k0, n2 = h0 ^ c3 ^ k1;
    c0 = n0; c1 = l1; c2 = n2; c3 = l0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  Block b;
  b.w[0] = c0; b.w[1] = c1; b.w[2] = c2; b.w[3] = c3;
  return b;
}

__device__ __forceinline__ double u01(uint64_t seed, uint64_t stream, uint64_t i) {
  const Block b = philox(seed, stream, i);
  const uint64_t bits = ((static_cast<uint64_t>(b.w[0]) << 21) ^ (b.w[1] >> 11)) & ((1ull << 53) - 1);
  return static_cast<double>(bits) * (1.0 / 9007199254740992.0);
}

__device__ __forceinline__ double normal(uint64_t seed, uint64_t stream, uint64_t i) {
  const double u1 = 1.0 - u01(seed, stream, 2 * i);
  const double u2 = u01(seed, stream, 2 * i + 1);
  return sqrt(-2.0 * log(u1)) * cos(2.0 * 3.141592653589793 * u2);
}

// One Philox block per unit: 4 words / 16 bytes.
__global__ void fill_words(void *dst, int64_t count, int kind, uint64_t seed, uint64_t stream,
                           int64_t lo, uint64_t span) {
  const int64_t units = (kind == GEARB_FILL_U8) ? (count + 15) / 16 : (count + 3) / 4;
  for (int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < units;
       u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const Block b = philox(seed, stream, static_cast<uint64_t>(u));
    if (kind == GEARB_FILL_U8) {
      uint8_t *p = static_cast<uint8_t *>(dst) + u * 16;
      if (u * 16 + 16 <= count && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        *reinterpret_cast<uint4 *>(p) = make_uint4(b.w[0], b.w[1], b.w[2], b.w[3]);
      } else {
        for (int k = 0; k < 16 && u * 16 + k < count; ++k)
          p[k] = static_cast<uint8_t>(b.w[k >> 2] >> (8 * (k & 3)));
      }
    } else {
      uint32_t *p = static_cast<uint32_t *>(dst) + u * 4;
      uint32_t o[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        o[k] = (kind == GEARB_FILL_U32)
                   ? b.w[k]
                   : static_cast<uint32_t>(static_cast<int32_t>(
                         lo + static_cast<int64_t>((static_cast<uint64_t>(b.w[k]) * span) >> 32)));
      if (u * 4 + 4 <= count && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
        *reinterpret_cast<uint4 *>(p) = make_uint4(o[0], o[1], o[2], o[3]);
      } else {
        for (int k = 0; k < 4 && u * 4 + k < count; ++k) p[k] = o[k];
      }
    }
  }
}

__global__ void fill_real(void *dst, int64_t count, int kind, uint64_t seed, uint64_t stream,
                          double a, double b) {
  for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const uint64_t e = static_cast<uint64_t>(i);
    switch (kind) {
      case GEARB_FILL_F32_NORMAL:
        static_cast<float *>(dst)[i] = static_cast<float>(normal(seed, stream, e));
        break;
      case GEARB_FILL_F32_LOGNORMAL:
        static_cast<float *>(dst)[i] =
            static_cast<float>(exp(static_cast<double>(static_cast<float>(normal(seed, stream, e)))));
        break;
      case GEARB_FILL_F32_UNIFORM:
        static_cast<float *>(dst)[i] =
            static_cast<float>(__dadd_rn(a, __dmul_rn(b - a, u01(seed, stream, e))));
        break;
      default:  // GEARB_FILL_U01_F64
        static_cast<double *>(dst)[i] = u01(seed, stream, e);
        break;
    }
  }
}

}  // namespace

int launch_fill(void *dst, int64_t count, int kind, uint64_t seed, uint64_t stream_id, double a,
                double b, cudaStream_t stream) {
  GEARB_REQUIRE(count >= 0, "fill: negative count");
  if (count == 0) return GEARB_OK;
  GEARB_REQUIRE(dst != nullptr, "fill: null destination");
  const int threads = 256;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (kind == GEARB_FILL_U32 || kind == GEARB_FILL_I32_RANGE || kind == GEARB_FILL_U8) {
    const int64_t units = (kind == GEARB_FILL_U8) ? (count + 15) / 16 : (count + 3) / 4;
    int64_t blocks = (units + threads - 1) / threads;
    if (blocks > cap) blocks = cap;
    const int64_t lo = static_cast<int64_t>(a);
    const int64_t hi = static_cast<int64_t>(b);
    GEARB_REQUIRE(kind != GEARB_FILL_I32_RANGE || (hi > lo && hi - lo <= 0xffffffffll),
                  "fill: empty or oversized integer range");
    fill_words<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
        dst, count, kind, seed, stream_id, lo, static_cast<uint64_t>(hi - lo));
  } else if (kind == GEARB_FILL_F32_NORMAL || kind == GEARB_FILL_F32_LOGNORMAL ||
             kind == GEARB_FILL_F32_UNIFORM || kind == GEARB_FILL_U01_F64) {
    int64_t blocks = (count + threads - 1) / threads;
    if (blocks > cap) blocks = cap;
    fill_real<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(dst, count, kind, seed,
                                                                     stream_id, a, b);
  } else {
    return fail(GEARB_ERR_INVALID, "fill: unknown kind %d", kind);
  }
  GEARB_CUDA(cudaGetLastError());
  return GEARB_OK;
}

}  // namespace gearb
