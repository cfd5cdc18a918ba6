// ref_shim.cc -- C entry points around the REFERENCE's own host classes.
//
// TEST INFRASTRUCTURE ONLY.  This file contains no logic of the path: it builds
// the reference's TableSpec / TrajectoryTable / CpuTrajectoryStorageHandler
// (src/storage/specs.cc, table.cc, handler.cc of bigrl-team/gear, compiled from
// where they lie by oracle/Makefile into oracle/_ref/) and forwards to
// CpuTrajectoryStorageHandler::sub (handler.cc:78-131).  It is used to
//   * pin the C restatement in gear_oracle.c to the reference's real code, and
//   * time the reference's CPU path (sub + a host memcpy per request; the
//     reference has no host copy loop of its own, its copy is the GPU kernel
//     vary_stride_copy_collect, src/cuda/copy.cu:47-89) on the host cores.
// The table is never connected (no shared memory, no CUDA call): sub() only
// needs the strides, as the reference's own tests/test_sub.py:12 notes.
#include <chrono>
#include <cstring>
#include <stdexcept>
#include <thread>
#include <vector>

#include "storage/handler.h"

using gear::common::DataType;
using gear::common::Int64Span;
using gear::common::Range;
using gear::storage::ColumnSpec;
using gear::storage::CpuTrajectoryStorageHandler;
using gear::storage::SubscribePattern;
using gear::storage::TableSpec;
using gear::storage::TrajectoryTable;

// handler.cc references the GPU launcher; it is never called from here.
namespace gear::cuda {
void launch_fused_subcopy_collect(void *, void *, int, int64_t *, int64_t *, int64_t *, bool,
                                  int64_t, int64_t, int, int, int, int) {
  throw std::runtime_error("GPU launcher is not part of the CPU reference build");
}
}  // namespace gear::cuda

namespace {
struct Ref {
  TrajectoryTable *table;
  CpuTrajectoryStorageHandler *handler;
  std::vector<int64_t> row_bytes;
};
}  // namespace

extern "C" {

void *gearref_create(const int64_t *row_bytes, int ncols, int64_t T, int64_t capacity) {
  std::vector<ColumnSpec> cols;
  for (int c = 0; c < ncols; ++c)
    cols.emplace_back(std::vector<size_t>{static_cast<size_t>(row_bytes[c])}, DataType::kByte, "");
  TableSpec spec(0, 1, static_cast<size_t>(T), static_cast<size_t>(capacity), static_cast<size_t>(ncols), cols);
  auto *r = new Ref();
  r->table = new TrajectoryTable(spec, 0, false);
  r->handler = new CpuTrajectoryStorageHandler(r->table, static_cast<size_t>(capacity), Range(0, 0),
                                               Range(0, static_cast<size_t>(capacity)));
  r->row_bytes.assign(row_bytes, row_bytes + ncols);
  return r;
}

// pad: 0 inactive, 1 head, 2 tail (SubscribePattern::PadOption order).
void gearref_set(void *h, int column, int offset, int64_t length, int pad) {
  auto *r = static_cast<Ref *>(h);
  auto opt = pad == 1   ? SubscribePattern::PadOption::kHead
             : pad == 2 ? SubscribePattern::PadOption::kTail
                        : SubscribePattern::PadOption::kInactive;
  r->handler->set({static_cast<size_t>(column)}, {SubscribePattern(offset, static_cast<size_t>(length), opt)});
}

int64_t gearref_sub(void *h, int64_t *idx, int64_t *ts, int64_t *len, int64_t n, int column,
                    int64_t *src_off, int64_t *dst_off, int64_t *copy_len) {
  auto *r = static_cast<Ref *>(h);
  try {
    return r->handler->sub(Int64Span(idx, n), Int64Span(ts, n), Int64Span(len, n),
                           static_cast<size_t>(column), Int64Span(src_off, n), Int64Span(dst_off, n),
                           Int64Span(copy_len, n));
  } catch (const std::exception &) {
    return -1;
  }
}

// Timed CPU path: `iters` batches; each batch runs sub() for every listed column
// and memcpy's each request, requests striped over `threads` host threads.
// Returns seconds for all iterations.
double gearref_time_gather(void *h, const uint8_t *table, int64_t *idx, int64_t *ts, int64_t *len,
                           int64_t n, const int *columns, int ncols, uint8_t *const *dst, int threads,
                           int iters) {
  auto *r = static_cast<Ref *>(h);
  if (threads < 1) threads = 1;
  auto work = [&](int t) {
    const int64_t lo = n * t / threads, hi = n * (t + 1) / threads, m = hi - lo;
    std::vector<int64_t> s(m), d(m), b(m);
    for (int c = 0; c < ncols; ++c) {
      const int64_t slot = r->handler->sub(Int64Span(idx + lo, m), Int64Span(ts + lo, m), Int64Span(len + lo, m),
                                           static_cast<size_t>(columns[c]), Int64Span(s.data(), m),
                                           Int64Span(d.data(), m), Int64Span(b.data(), m));
      uint8_t *base = dst[c] + lo * slot;  // sub() numbers the stripe's requests from 0
      for (int64_t i = 0; i < m; ++i)
        if (b[i] > 0) std::memcpy(base + d[i], table + s[i], static_cast<size_t>(b[i]));
    }
  };
  const auto t0 = std::chrono::steady_clock::now();
  for (int it = 0; it < iters; ++it) {
    std::vector<std::thread> pool;
    for (int t = 1; t < threads; ++t) pool.emplace_back(work, t);
    work(0);
    for (auto &th : pool) th.join();
  }
  return std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
}

void gearref_destroy(void *h) {
  auto *r = static_cast<Ref *>(h);
  delete r->handler;
  delete r->table;
  delete r;
}

}  // extern "C"
