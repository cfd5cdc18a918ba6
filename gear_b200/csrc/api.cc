// Host side of libgear_b200: the objects behind the C ABI (trajectory table,
// storage handler, index set, sampler) and the extern "C" entry points.
//
// These mirror, in behaviour and not in code, the reference's host classes:
//   TrajectoryTable             src/storage/table.cc
//   CpuTrajectoryStorageHandler src/storage/handler.cc
//   SharedMemory / CudaUVMemory src/memory/shared_memory.cc, cuda_uvm.cc
//   CudaMemory                  src/memory/cuda_memory.cc
//   Indexset / StatusTableShard include/index/set.h
// with 64-bit sizes everywhere and status codes instead of assert/exit.
#include <errno.h>
#include <sys/ipc.h>
#include <sys/shm.h>

#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <optional>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "common.h"

namespace gearb {

TraceRange::TraceRange(const char *name) { nvtxRangePushA(name); }
TraceRange::~TraceRange() { nvtxRangePop(); }

std::string &last_error() {
  static thread_local std::string e;
  return e;
}

int fail(int code, const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  last_error() = buf;
  return code;
}

int sm_count() {
  constexpr int kMaxDevices = 64;
  static int cache[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 1;
  if (dev >= 0 && dev < kMaxDevices && cache[dev] > 0) return cache[dev];
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 1;
  if (dev >= 0 && dev < kMaxDevices) cache[dev] = n;
  return n;
}

int per_device_once(int slot, int (*setup)(int *value), int *value) {
  constexpr int kMaxDevices = 64;
  static std::mutex mu;
  static bool done[kOnceSlots][kMaxDevices] = {};
  static int vals[kOnceSlots][kMaxDevices] = {};
  int dev = 0;
  GEARB_CUDA(cudaGetDevice(&dev));
  GEARB_REQUIRE(slot >= 0 && slot < kOnceSlots && dev >= 0 && dev < kMaxDevices,
                "device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!done[slot][dev]) {
    int v = 0;
    const int rc = setup(&v);
    if (rc != GEARB_OK) return rc;
    vals[slot][dev] = v;
    done[slot][dev] = true;
  }
  if (value) *value = vals[slot][dev];
  return GEARB_OK;
}

static bool have_cuda_device() {
  static int state = -1;
  if (state < 0) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) (void)cudaGetLastError();
    state = (e == cudaSuccess && n > 0) ? 1 : 0;
  }
  return state == 1;
}

static inline int64_t round_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

// A block of host memory the GPU can read in place: a System-V segment that is
// registered with CUDA (SharedMemory, shared_memory.cc:35-63), or
// cudaHostAlloc(Mapped|Portable) memory (CudaUVMemory, cuda_uvm.cc:29-32).
// Without a CUDA device (CPU-only hosts) it degrades to plain memory so that
// the host-side logic stays usable.
struct HostBlock {
  void *addr = nullptr;
  void *dev_alias = nullptr;
  int64_t size = 0;
  int shmid = -1;
  bool is_shm = false, creator = false, registered = false, cuda_alloc = false;

  int alloc(int64_t bytes, int key, bool create) {
    if (addr) return GEARB_OK;
    size = bytes;
    const size_t sz = static_cast<size_t>(bytes > 0 ? bytes : 1);
    if (key != 0) {
      shmid = create ? shmget(key, sz, IPC_CREAT | 0777) : shmget(key, sz, 0666);
      if (shmid == -1)
        return fail(GEARB_ERR_STATE, "shmget(key=%d, size=%zu, create=%d) failed: errno %d", key, sz,
                    (int)create, errno);
      void *p = shmat(shmid, nullptr, 0);
      if (p == reinterpret_cast<void *>(-1))
        return fail(GEARB_ERR_STATE, "shmat(key=%d) failed: errno %d", key, errno);
      addr = p;
      is_shm = true;
      creator = create;
      if (have_cuda_device()) {
        cudaError_t e = cudaHostRegister(addr, sz, cudaHostRegisterMapped | cudaHostRegisterPortable);
        if (e != cudaSuccess) {
          (void)cudaGetLastError();
          release();
          return fail(GEARB_ERR_CUDA, "cudaHostRegister(%zu bytes) failed: %s", sz,
                      cudaGetErrorString(e));
        }
        registered = true;
      }
    } else if (have_cuda_device()) {
      cudaError_t e = cudaHostAlloc(&addr, sz, cudaHostAllocMapped | cudaHostAllocPortable);
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        addr = nullptr;
        return fail(GEARB_ERR_NOMEM, "cudaHostAlloc(%zu bytes) failed: %s", sz, cudaGetErrorString(e));
      }
      cuda_alloc = true;
      std::memset(addr, 0, sz);
    } else {
      if (posix_memalign(&addr, 256, round_up(static_cast<int64_t>(sz), 256)) != 0) {
        addr = nullptr;
        return fail(GEARB_ERR_NOMEM, "host allocation of %zu bytes failed", sz);
      }
      std::memset(addr, 0, sz);
    }
    if (registered || cuda_alloc) {
      if (cudaHostGetDevicePointer(&dev_alias, addr, 0) != cudaSuccess) {
        (void)cudaGetLastError();
        dev_alias = nullptr;
      }
    }
    return GEARB_OK;
  }

  void release() {
    if (!addr) return;
    if (registered) (void)cudaHostUnregister(addr);
    if (is_shm) {
      shmdt(addr);
      if (creator && shmid != -1) shmctl(shmid, IPC_RMID, nullptr);
    } else if (cuda_alloc) {
      (void)cudaFreeHost(addr);
    } else {
      std::free(addr);
    }
    addr = dev_alias = nullptr;
    registered = cuda_alloc = is_shm = false;
  }
  ~HostBlock() { release(); }
};

struct Pattern {
  int32_t offset;
  int64_t length;
  int32_t pad;
};

}  // namespace gearb

using namespace gearb;

struct gearb_table {
  std::vector<int64_t> row_bytes, accu;
  int64_t T = 0, capacity = 0, traj_stride = 0, nbytes = 0;
  int residency = 0, shm_key = 0;
  bool create = true, connected = false;
  HostBlock host;
  void *hbm = nullptr;
  int hbm_device = -1;

  const uint8_t *device_base() const {
    if (hbm) return static_cast<const uint8_t *>(hbm);
    return static_cast<const uint8_t *>(host.dev_alias);
  }
};

struct gearb_handler {
  gearb_table *table = nullptr;
  int64_t global_capacity = 0, w_lb = 0, w_hb = 0, r_lb = 0, r_hb = 0;
  std::vector<std::optional<Pattern>> patterns;
};

struct gearb_indexset {
  int64_t global_capacity = 0, local_capacity = 0, index_offset = 0;
  HostBlock mem;
  int64_t *timesteps = nullptr;
  float *weights = nullptr;
};

struct gearb_sampler {
  int64_t n = 0, nparts = 0, scratch_bytes = 0;
  int device = 0;
  float *cdf = nullptr;
  double *l1s[2] = {nullptr, nullptr};  // level 1 of the last scan and of the one before it, like blk below
  void *scratches[2] = {nullptr, nullptr};  // header + aggregates of the last scan and of the one before it
  double *sb[2] = {nullptr, nullptr};       // superblock sums, zero except between a scan_totals and its level-1 launch
  void *upd = nullptr;  // dirty flags + list of touched partitions for incremental updates
  int32_t *status = nullptr;
  const float *lazy_prio = nullptr;  // set by scan_totals: level 2 is rebuilt from these on demand
  // Block totals (eight per partition) of the last scan and of the one before it: a scan writes
  // the buffer the previous one did not, so a scan that starts while a sampling launch is still
  // reading (this GPU's, or a peer's in the pull mode) never overwrites what that launch reads.
  float *blk[2] = {nullptr, nullptr};
  int slot = 0;        // buffer the last scan wrote
  int next_slot = -1;  // chosen by the caller for the next scan, or -1: the other one
  int take_slot() {
    slot = next_slot >= 0 ? next_slot : (slot ^ 1);
    next_slot = -1;
    return slot;
  }
  double *l1() const { return l1s[slot]; }
  void *scratch() const { return scratches[slot]; }
  // A totals-only scan of a table of more than 1024 partitions leaves level 1 for later: the
  // sampling launch behind it finds partitions through the superblock sums, and the level-1
  // launch goes behind the NEXT scan, beside which it runs (the two work in different slots).
  // Every other consumer of level 1 has it launched first (settle()).
  bool l1_owed = false;
  int owed_slot = 0;
  cudaStream_t owed_stream = nullptr;  // for the entry points that take no stream
  bool drawn_since_scan = false;
  bool last_scan_may_start_early = false;
  int settle(cudaStream_t stream, bool after_next = false) {
    if (!l1_owed) return GEARB_OK;
    l1_owed = false;
    return launch_level1(scan_aggregate_words(scratches[owed_slot]), nparts, l1s[owed_slot], nullptr, status, stream,
                         static_cast<ScanHeader *>(scratches[owed_slot]), true, sb[owed_slot], after_next);
  }
  // A scan may begin while the launch before it in the stream is still finishing -- but never
  // beside an earlier scan of the same sampler: they share the scratch block.  Every launch that
  // reads the tables waits for the scan before it to complete before it lets its own successor
  // go, so one such launch between two scans is enough; two scans in a row are not overlapped.
  bool scan_unconsumed = false;
  bool may_overlap() {
    const bool ok = !scan_unconsumed;
    scan_unconsumed = true;
    return ok;
  }
};

extern "C" {

const char *gearb_last_error(void) { return last_error().c_str(); }
int gearb_version(void) { return 100; }

int gearb_init(int device) {
  GEARB_CUDA(cudaSetDevice(device));
  GEARB_CUDA(cudaFree(nullptr));  // force context creation, like the first runtime call would
  return GEARB_OK;
}

int gearb_device_count(int *count) {
  GEARB_REQUIRE(count, "device_count: null argument");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    n = 0;
  }
  *count = n;
  return GEARB_OK;
}

/* ------------------------------ table ---------------------------------- */
int gearb_table_create(const int64_t *row_bytes, int ncols, int64_t trajectory_length,
                       int64_t capacity, int residency, int shm_key, int create,
                       gearb_table **out) {
  GEARB_REQUIRE(out && row_bytes, "table_create: null argument");
  GEARB_REQUIRE(ncols > 0 && ncols <= GEARB_MAX_COLUMNS, "table_create: %d columns (1..%d supported)",
                ncols, GEARB_MAX_COLUMNS);
  GEARB_REQUIRE(trajectory_length > 0 && capacity > 0,
                "table_create: trajectory_length and capacity must be positive");
  GEARB_REQUIRE((residency & (GEARB_RES_HOST | GEARB_RES_HBM)) != 0 &&
                    (residency & ~(GEARB_RES_HOST | GEARB_RES_HBM)) == 0,
                "table_create: residency must combine GEARB_RES_HOST / GEARB_RES_HBM");
  auto *t = new gearb_table();
  t->row_bytes.assign(row_bytes, row_bytes + ncols);
  t->accu.resize(ncols + 1);
  int64_t sum = 0;
  for (int c = 0; c < ncols; ++c) {
    if (row_bytes[c] <= 0 || row_bytes[c] > (int64_t(1) << 30)) {
      delete t;
      return fail(GEARB_ERR_INVALID, "table_create: column %d has row size %lld", c,
                  (long long)row_bytes[c]);
    }
    t->accu[c] = sum;
    sum += row_bytes[c];
  }
  t->accu[ncols] = sum;
  t->T = trajectory_length;
  t->capacity = capacity;
  t->traj_stride = sum * trajectory_length;
  t->nbytes = t->traj_stride * capacity;
  t->residency = residency;
  t->shm_key = shm_key;
  t->create = create != 0;
  *out = t;
  return GEARB_OK;
}

int gearb_table_connect(gearb_table *t, int64_t *nbytes) {
  GEARB_REQUIRE(t, "table_connect: null table");
  if (!t->connected) {
    if (t->residency & GEARB_RES_HOST) {
      int rc = t->host.alloc(t->nbytes, t->shm_key, t->create);
      if (rc != GEARB_OK) return rc;
    }
    if ((t->residency & GEARB_RES_HBM) && !t->hbm) {
      GEARB_CUDA(cudaGetDevice(&t->hbm_device));
      cudaError_t e = cudaMalloc(&t->hbm, static_cast<size_t>(round_up(t->nbytes, 256)));
      if (e != cudaSuccess) {
        (void)cudaGetLastError();
        t->hbm = nullptr;
        return fail(GEARB_ERR_NOMEM, "cudaMalloc(%lld bytes) for the HBM table failed: %s",
                    (long long)t->nbytes, cudaGetErrorString(e));
      }
      if (!(t->residency & GEARB_RES_HOST)) GEARB_CUDA(cudaMemset(t->hbm, 0, static_cast<size_t>(t->nbytes)));
    }
    t->connected = true;
  }
  if (nbytes) *nbytes = t->nbytes;
  return GEARB_OK;
}

int gearb_table_destroy(gearb_table *t) {
  if (!t) return GEARB_OK;
  if (t->hbm) (void)cudaFree(t->hbm);
  delete t;
  return GEARB_OK;
}

int gearb_table_layout(const gearb_table *t, int64_t *trajectory_stride, int64_t *nbytes,
                       int64_t *accu) {
  GEARB_REQUIRE(t, "table_layout: null table");
  if (trajectory_stride) *trajectory_stride = t->traj_stride;
  if (nbytes) *nbytes = t->nbytes;
  if (accu) std::memcpy(accu, t->accu.data(), t->accu.size() * sizeof(int64_t));
  return GEARB_OK;
}

void *gearb_table_host_ptr(const gearb_table *t) { return t ? t->host.addr : nullptr; }
void *gearb_table_device_ptr(const gearb_table *t) {
  return t ? const_cast<uint8_t *>(t->device_base()) : nullptr;
}

int gearb_table_upload(gearb_table *t, void *stream) {
  TraceRange trace("gearb:table_upload");
  GEARB_REQUIRE(t && t->connected, "table_upload: table is not connected");
  GEARB_REQUIRE(t->host.addr, "table_upload: table has no host copy");
  if (!t->hbm) {
    GEARB_CUDA(cudaGetDevice(&t->hbm_device));
    cudaError_t e = cudaMalloc(&t->hbm, static_cast<size_t>(round_up(t->nbytes, 256)));
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      t->hbm = nullptr;
      return fail(GEARB_ERR_NOMEM, "cudaMalloc(%lld bytes) for the HBM table failed: %s",
                  (long long)t->nbytes, cudaGetErrorString(e));
    }
    t->residency |= GEARB_RES_HBM;
  }
  GEARB_CUDA(cudaMemcpyAsync(t->hbm, t->host.addr, static_cast<size_t>(t->nbytes),
                             cudaMemcpyHostToDevice, as_stream(stream)));
  return GEARB_OK;
}

int gearb_table_upload_range(gearb_table *t, int64_t offset, int64_t bytes, void *stream) {
  GEARB_REQUIRE(t && t->connected, "table_upload_range: table is not connected");
  GEARB_REQUIRE(t->host.addr && t->hbm, "table_upload_range: the table needs a host copy and an uploaded device copy");
  GEARB_REQUIRE(offset >= 0 && bytes >= 0 && offset + bytes <= t->nbytes,
                "table_upload_range: range [%lld, +%lld) outside the table (%lld bytes)", (long long)offset,
                (long long)bytes, (long long)t->nbytes);
  if (bytes == 0) return GEARB_OK;
  GEARB_CUDA(cudaMemcpyAsync(static_cast<char *>(t->hbm) + offset, static_cast<const char *>(t->host.addr) + offset,
                             static_cast<size_t>(bytes), cudaMemcpyHostToDevice, as_stream(stream)));
  return GEARB_OK;
}

int gearb_table_write(gearb_table *t, int64_t offset, const void *src, int64_t bytes, void *stream) {
  GEARB_REQUIRE(t && t->connected, "table_write: table is not connected");
  GEARB_REQUIRE(offset >= 0 && bytes >= 0 && offset + bytes <= t->nbytes,
                "table_write: range [%lld, +%lld) outside the table (%lld bytes)", (long long)offset,
                (long long)bytes, (long long)t->nbytes);
  if (bytes == 0) return GEARB_OK;
  GEARB_REQUIRE(src, "table_write: null source");
  if (t->host.addr) std::memcpy(static_cast<char *>(t->host.addr) + offset, src, static_cast<size_t>(bytes));
  if (t->hbm)
    GEARB_CUDA(cudaMemcpyAsync(static_cast<char *>(t->hbm) + offset, src, static_cast<size_t>(bytes),
                               cudaMemcpyDefault, as_stream(stream)));
  return GEARB_OK;
}

int gearb_table_read(const gearb_table *t, int64_t offset, void *dst, int64_t bytes) {
  GEARB_REQUIRE(t && t->connected, "table_read: table is not connected");
  GEARB_REQUIRE(offset >= 0 && bytes >= 0 && offset + bytes <= t->nbytes,
                "table_read: range outside the table");
  if (bytes == 0) return GEARB_OK;
  GEARB_REQUIRE(dst, "table_read: null destination");
  if (t->hbm) {
    GEARB_CUDA(cudaMemcpy(dst, static_cast<const char *>(t->hbm) + offset, static_cast<size_t>(bytes),
                          cudaMemcpyDefault));
  } else {
    std::memcpy(dst, static_cast<const char *>(t->host.addr) + offset, static_cast<size_t>(bytes));
  }
  return GEARB_OK;
}

/* ------------------------------ handler -------------------------------- */
int gearb_handler_create(gearb_table *t, int64_t global_capacity, int64_t w_lb, int64_t w_hb,
                         int64_t r_lb, int64_t r_hb, gearb_handler **out) {
  GEARB_REQUIRE(t && out, "handler_create: null argument");
  auto *h = new gearb_handler();
  h->table = t;
  h->global_capacity = global_capacity;
  h->w_lb = w_lb; h->w_hb = w_hb; h->r_lb = r_lb; h->r_hb = r_hb;
  h->patterns.resize(t->row_bytes.size());
  *out = h;
  return GEARB_OK;
}

int gearb_handler_destroy(gearb_handler *h) {
  delete h;
  return GEARB_OK;
}

int gearb_handler_set(gearb_handler *h, const int64_t *cids, int n, const int32_t *offsets,
                      const int64_t *lengths, const int32_t *pads) {
  GEARB_REQUIRE(h && (n == 0 || (cids && offsets && lengths && pads)), "handler_set: null argument");
  for (int i = 0; i < n; ++i) {
    GEARB_REQUIRE(cids[i] >= 0 && cids[i] < (int64_t)h->patterns.size(),
                  "handler_set: column id %lld out of range", (long long)cids[i]);
    GEARB_REQUIRE(lengths[i] >= 0 && lengths[i] < (int64_t(1) << 31),
                  "handler_set: pattern length %lld out of range", (long long)lengths[i]);
    GEARB_REQUIRE(pads[i] >= GEARB_PAD_INACTIVE && pads[i] <= GEARB_PAD_TAIL,
                  "handler_set: unknown pad option %d", pads[i]);
  }
  for (int i = 0; i < n; ++i) h->patterns[cids[i]] = Pattern{offsets[i], lengths[i], pads[i]};
  return GEARB_OK;
}

static int pattern_of(const gearb_handler *h, int column, const Pattern **out) {
  GEARB_REQUIRE(h, "null handler");
  GEARB_REQUIRE(column >= 0 && column < (int)h->patterns.size(), "column id %d out of range", column);
  if (!h->patterns[column].has_value())
    return fail(GEARB_ERR_STATE, "Subscribing a column without setting its SubscribePattern.");
  *out = &*h->patterns[column];
  return GEARB_OK;
}

int gearb_handler_sub(const gearb_handler *h, const int64_t *idx, const int64_t *ts,
                      const int64_t *len, int64_t n, int column, int64_t *src_off,
                      int64_t *dst_off, int64_t *copy_len, int64_t *slot_bytes) {
  const Pattern *pat = nullptr;
  int rc = pattern_of(h, column, &pat);
  if (rc != GEARB_OK) return rc;
  GEARB_REQUIRE(n == 0 || (idx && ts && len && src_off && dst_off && copy_len),
                "handler_sub: null argument");
  const gearb_table *t = h->table;
  const int64_t row = t->row_bytes[column];
  const int64_t column_ofst = t->accu[column] * t->T;
  const int64_t slot = pat->length * row;
  for (int64_t i = 0; i < n; ++i) {
    int64_t start = ts[i] + pat->offset;
    if (start < 0) start = 0;
    int64_t end = start + pat->length;
    if (end > len[i]) end = len[i];
    int64_t bytes = (end - start) * row;
    if (bytes < 0) bytes = 0;
    copy_len[i] = bytes;
    src_off[i] = idx[i] * t->traj_stride + column_ofst + start * row;
    dst_off[i] = slot * i + (pat->pad == GEARB_PAD_HEAD ? slot - bytes : 0);
  }
  if (slot_bytes) *slot_bytes = slot;
  return GEARB_OK;
}

// Fills the launch parameters shared by the gather kernels from the handler's patterns.
static int build_gather_params(gearb_handler *h, const int32_t *columns, int ncols, int64_t n,
                               void *const *dst, int zero_fill, int32_t *status, GatherParams &p,
                               int piece_bytes = 2048, bool staged_pieces = true) {
  GEARB_REQUIRE(h && h->table, "gather: null handler");
  GEARB_REQUIRE(ncols >= 0 && ncols <= GEARB_MAX_COLUMNS, "gather: %d columns", ncols);
  GEARB_REQUIRE(n >= 0, "gather: negative request count");
  GEARB_REQUIRE(ncols == 0 || (columns && dst), "gather: null argument");
  const gearb_table *t = h->table;
  if (!t->connected || !t->device_base())
    return fail(GEARB_ERR_STATE, "gather: the table has no device-visible copy (connect it first)");
  p = GatherParams{};
  p.table = t->device_base();
  p.n = n;
  p.traj_stride = t->traj_stride;
  p.capacity = t->capacity;
  p.T = t->T;
  p.status = status;
  p.zero_fill = zero_fill ? 1 : 0;
  p.chunk_bytes = piece_bytes;
  int64_t chunks = 0, stage = 0;
  int used = 0;
  for (int i = 0; i < ncols; ++i) {
    const Pattern *pat = nullptr;
    int rc = pattern_of(h, columns[i], &pat);
    if (rc != GEARB_OK) return rc;
    GEARB_REQUIRE(dst[i], "gather: null destination for column %d", columns[i]);
    const int64_t row = t->row_bytes[columns[i]];
    const int64_t slot = row * pat->length;
    if (slot == 0) continue;
    GatherColumn &c = p.cols[used++];
    c.col_offset = t->accu[columns[i]] * t->T;
    c.dst = static_cast<uint8_t *>(dst[i]);
    c.row = static_cast<int32_t>(row);
    c.pat_offset = pat->offset;
    c.pat_length = static_cast<int32_t>(pat->length);
    c.pad_head = pat->pad == GEARB_PAD_HEAD;
    c.chunk_first = static_cast<int32_t>(chunks);
    c.stage_off = static_cast<int32_t>(stage < (int64_t(1) << 30) ? stage : 0);
    stage += round_up(slot + 32, 128);  // covering 16-byte blocks of a misaligned segment fit
    const int64_t cc = (slot + p.chunk_bytes - 1) / p.chunk_bytes;
    c.chunk_count = static_cast<int32_t>(cc);
    chunks += cc;
    GEARB_REQUIRE(chunks < (int64_t(1) << 30), "gather: request too large");
  }
  p.ncols = used;
  p.chunks_per_request = static_cast<int32_t>(chunks);
  // Small requests from an HBM table are staged through shared memory by the fused kernel, which
  // copies them out in pieces of 1 KiB so that its four warps get equal shares.
  p.stage_bytes = (t->hbm && stage > 0 && stage <= 24 * 1024) ? static_cast<int32_t>(stage) : 0;
  if (p.stage_bytes > 0 && piece_bytes == GEARB_SG_PIECE && staged_pieces)  // the fused launches ask for 4 KiB pieces
    return build_gather_params(h, columns, ncols, n, dst, zero_fill, status, p, 1024, false);
  // Larger requests: from mapped host memory they stream through per-warp rings of bulk copies
  // (measured on config 4: 51.3 GB/s = 0.92 of the host-to-device copy peak, against 32.0 GB/s with
  // plain loads); from HBM plain 16-byte loads are faster (3.6 against 2.6 TB/s on 64 KiB requests).
  static const char *force = getenv("GEARB_GATHER_PATH");  // tuning knob: "ring" or "direct"
  const bool want_ring = force ? (force[0] == 'r') : (t->hbm == nullptr);
  p.ring = (p.stage_bytes == 0 && want_ring) ? 1 : 0;
  return GEARB_OK;
}

int gearb_handler_gather(gearb_handler *h, const int32_t *columns, int ncols, const int64_t *idx,
                         const int64_t *ts, const int64_t *len, int64_t n, void *const *dst,
                         int zero_fill, int32_t *status, void *stream) {
  TraceRange trace("gearb:gather");
  GatherParams p;
  int rc = build_gather_params(h, columns, ncols, n, dst, zero_fill, status, p);
  if (rc != GEARB_OK) return rc;
  if (n == 0 || p.ncols == 0) return GEARB_OK;
  GEARB_REQUIRE(idx && ts && len, "gather: null request arrays");
  p.idx = idx; p.ts = ts; p.len = len;
  return launch_gather(p, as_stream(stream));
}

int gearb_handler_subcopy(gearb_handler *h, const int64_t *idx, const int64_t *ts,
                          const int64_t *len, int64_t n, int column, void *dst, int32_t *status,
                          void *stream) {
  const int32_t col = column;
  void *d = dst;
  return gearb_handler_gather(h, &col, 1, idx, ts, len, n, &d, 0, status, stream);
}

int gearb_handler_view(const gearb_handler *h, int64_t index, int column, void **host_ptr,
                       int64_t *bytes) {
  GEARB_REQUIRE(h && h->table && host_ptr && bytes, "handler_view: null argument");
  const gearb_table *t = h->table;
  GEARB_REQUIRE(column >= 0 && column < (int)t->row_bytes.size(), "handler_view: column %d out of range",
                column);
  GEARB_REQUIRE(index >= 0 && index < t->capacity, "handler_view: trajectory %lld out of range",
                (long long)index);
  if (!t->host.addr) return fail(GEARB_ERR_STATE, "handler_view: the table has no host copy");
  *host_ptr = static_cast<char *>(t->host.addr) + index * t->traj_stride + t->accu[column] * t->T;
  *bytes = t->row_bytes[column] * t->T;
  return GEARB_OK;
}

int gearb_vcopy(const void *src, void *dst, const int64_t *src_off, const int64_t *dst_off,
                const int64_t *lengths, int64_t n, int64_t max_length, void *stream) {
  TraceRange trace("gearb:vcopy");
  GEARB_REQUIRE(lengths || n == 0, "vcopy: null lengths");
  return launch_vcopy(static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), src_off, dst_off,
                      lengths, 0, n, max_length, as_stream(stream));
}

int gearb_copy(const void *src, void *dst, const int64_t *src_off, const int64_t *dst_off, int64_t n,
               int64_t length, void *stream) {
  TraceRange trace("gearb:copy");
  return launch_vcopy(static_cast<const uint8_t *>(src), static_cast<uint8_t *>(dst), src_off, dst_off,
                      nullptr, length, n, length, as_stream(stream));
}

/* ------------------------------ index set ------------------------------ */
int gearb_indexset_create(int64_t global_capacity, int64_t local_capacity, int64_t index_offset,
                          int shared, int shm_key, int create, gearb_indexset **out) {
  GEARB_REQUIRE(out, "indexset_create: null argument");
  GEARB_REQUIRE(local_capacity > 0 && global_capacity >= local_capacity && index_offset >= 0,
                "indexset_create: bad capacities");
  auto *s = new gearb_indexset();
  s->global_capacity = global_capacity;
  s->local_capacity = local_capacity;
  s->index_offset = index_offset;
  const int64_t ts_bytes = round_up(local_capacity * 8, 128);
  const int64_t w_bytes = round_up(local_capacity * 4, 128);
  int rc = s->mem.alloc(ts_bytes + w_bytes, shared ? shm_key : 0, create != 0);
  if (rc != GEARB_OK) {
    delete s;
    return rc;
  }
  s->timesteps = static_cast<int64_t *>(s->mem.addr);
  s->weights = reinterpret_cast<float *>(static_cast<char *>(s->mem.addr) + ts_bytes);
  *out = s;
  return GEARB_OK;
}

int gearb_indexset_destroy(gearb_indexset *s) {
  delete s;
  return GEARB_OK;
}
int64_t *gearb_indexset_timesteps(const gearb_indexset *s) { return s ? s->timesteps : nullptr; }
float *gearb_indexset_weights(const gearb_indexset *s) { return s ? s->weights : nullptr; }

/* ------------------------------ sampling ------------------------------- */
int64_t gearb_scan_scratch_bytes(int64_t n) { return n > 0 ? scan_scratch_bytes(n) : 0; }

int gearb_scan(const float *priorities, int64_t n, float *cdf, double *l1, void *scratch,
               int64_t scratch_bytes, int32_t *status, void *stream) {
  TraceRange trace("gearb:scan");
  return launch_scan(priorities, n, cdf, l1, scratch, scratch_bytes, status, 1, as_stream(stream));
}

int gearb_scan_static(const float *priorities, int64_t n, float *cdf, double *l1, int32_t *status,
                      void *stream) {
  TraceRange trace("gearb:scan");
  return launch_scan_static(priorities, n, cdf, l1, status, as_stream(stream));
}

int64_t gearb_scan_static_max_n(void) { return static_scan_max_n(); }

int gearb_search(const float *cdf, const double *l1, int64_t n, const double *variates, int64_t b,
                 int flags, int64_t *out_index, int32_t *status, void *stream) {
  TraceRange trace("gearb:search");
  return launch_search(cdf, l1, n, variates, b, flags, out_index, status, as_stream(stream));
}

int gearb_sample_uniform(int64_t n, const double *u01, int64_t b, int64_t *out_index, void *stream) {
  return launch_uniform(n, u01, b, out_index, as_stream(stream));
}

int gearb_decode(const int64_t *flat, int64_t b, int64_t trajectory_length, const int64_t *lengths,
                 int64_t index_offset, int64_t *idx, int64_t *ts, int64_t *len, void *stream) {
  return launch_decode(flat, b, trajectory_length, lengths, index_offset, idx, ts, len,
                       as_stream(stream));
}

int gearb_sampler_create(int64_t n, gearb_sampler **out) {
  GEARB_REQUIRE(out && n > 0, "sampler_create: n must be positive");
  auto *s = new gearb_sampler();
  s->n = n;
  s->nparts = (n + GEARB_PART - 1) / GEARB_PART;
  s->scratch_bytes = scan_scratch_bytes(n);
  cudaError_t e = cudaGetDevice(&s->device);
  if (e == cudaSuccess) e = cudaMalloc(&s->cdf, static_cast<size_t>(round_up(n * 4, 256)));
  if (e == cudaSuccess) e = cudaMalloc(&s->l1s[0], static_cast<size_t>(round_up((s->nparts + 1) * 8, 256)));
  if (e == cudaSuccess) e = cudaMalloc(&s->l1s[1], static_cast<size_t>(round_up((s->nparts + 1) * 8, 256)));
  const size_t sb_bytes = static_cast<size_t>(round_up((s->nparts / GEARB_SUPER_PARTS + 1) * 8, 256));
  for (int k = 0; k < 2; ++k) {
    if (e == cudaSuccess) e = cudaMalloc(&s->scratches[k], static_cast<size_t>(s->scratch_bytes));
    if (e == cudaSuccess) e = cudaMemset(s->scratches[k], 0, static_cast<size_t>(s->scratch_bytes));
    if (e == cudaSuccess) e = cudaMalloc(&s->sb[k], sb_bytes);
    if (e == cudaSuccess) e = cudaMemset(s->sb[k], 0, sb_bytes);
  }
  if (e == cudaSuccess) e = cudaMalloc(&s->upd, static_cast<size_t>(update_scratch_bytes(n)));
  if (e == cudaSuccess) e = cudaMemset(s->upd, 0, static_cast<size_t>(update_scratch_bytes(n)));
  if (e == cudaSuccess) e = cudaMalloc(&s->blk[0], static_cast<size_t>(round_up(s->nparts * 32, 256)));
  if (e == cudaSuccess) e = cudaMalloc(&s->blk[1], static_cast<size_t>(round_up(s->nparts * 32, 256)));
  if (e == cudaSuccess) e = cudaMalloc(&s->status, 256);
  if (e == cudaSuccess) e = cudaMemset(s->status, 0, 256);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    gearb_sampler_destroy(s);
    return fail(GEARB_ERR_NOMEM, "sampler_create(%lld): %s", (long long)n, cudaGetErrorString(e));
  }
  *out = s;
  return GEARB_OK;
}

int gearb_sampler_destroy(gearb_sampler *s) {
  if (!s) return GEARB_OK;
  if (s->cdf) (void)cudaFree(s->cdf);
  if (s->l1s[0]) (void)cudaFree(s->l1s[0]);
  if (s->l1s[1]) (void)cudaFree(s->l1s[1]);
  for (int k = 0; k < 2; ++k) {
    if (s->scratches[k]) (void)cudaFree(s->scratches[k]);
    if (s->sb[k]) (void)cudaFree(s->sb[k]);
  }
  if (s->upd) (void)cudaFree(s->upd);
  if (s->blk[0]) (void)cudaFree(s->blk[0]);
  if (s->blk[1]) (void)cudaFree(s->blk[1]);
  if (s->status) (void)cudaFree(s->status);
  delete s;
  return GEARB_OK;
}

int gearb_sampler_scan_partitions(gearb_sampler *s, const float *priorities, int store, void *stream) {
  TraceRange trace("gearb:scan_partitions");
  GEARB_REQUIRE(s, "sampler_scan_partitions: null sampler");
  int rc0 = s->settle(as_stream(stream));
  if (rc0 != GEARB_OK) return rc0;
  const int slot = s->take_slot();
  int rc = launch_scan(priorities, s->n, store ? s->cdf : nullptr, s->l1s[slot], s->scratch(), s->scratch_bytes, s->status,
                       0, as_stream(stream), /*level1=*/false, /*overlap_previous=*/s->may_overlap() && !store,
                       s->blk[slot]);
  if (rc == GEARB_OK) s->lazy_prio = store ? nullptr : priorities;
  return rc;
}

int gearb_sampler_scan_level1(gearb_sampler *s, void *stream) {
  TraceRange trace("gearb:level1");
  GEARB_REQUIRE(s, "sampler_scan_level1: null sampler");
  const bool was_owed_here = s->l1_owed && s->owed_slot == s->slot;
  int rc0 = s->settle(as_stream(stream));
  if (rc0 != GEARB_OK || was_owed_here) return rc0;  // that WAS this table's level-1 launch
  s->scan_unconsumed = false;  // this launch waits for the scan before it (see may_overlap)
  return launch_level1(scan_aggregate_words(s->scratch()), s->nparts, s->l1(), nullptr, s->status,
                       as_stream(stream), static_cast<ScanHeader *>(s->scratch()),
                       /*have_range=*/s->nparts > 1024);  // only the streaming kernel leaves the exponent range
}

// The three whole-table scans.  Level 1 of a table of more than 1024 partitions is left owing
// (see gearb_sampler::settle): a sampling launch that follows does without it, everything else
// has it launched first.  Not when the caller pinned the slot: then peers read this table.
static int scan_whole(gearb_sampler *s, const float *priorities, cudaStream_t stream, bool store, bool may_start_early) {
  const int before = s->slot;
  const bool pinned = s->next_slot >= 0;
  const int slot = s->take_slot();
  const bool owe = !pinned && s->nparts > 1024 && level1_can_follow_next_scan(s->nparts);
  if (s->l1_owed && (s->owed_slot == slot || !owe)) {  // the old order: level 1 in front of this scan
    int rc0 = s->settle(stream);
    if (rc0 != GEARB_OK) return rc0;
  }
  const bool overlap = s->may_overlap() && may_start_early && slot != before;
  int rc = launch_scan(priorities, s->n, store ? s->cdf : nullptr, s->l1s[slot], s->scratch(), s->scratch_bytes,
                       s->status, 0, stream, /*level1=*/!owe, overlap, s->blk[slot], owe ? s->sb[slot] : nullptr);
  if (rc != GEARB_OK) return rc;
  s->lazy_prio = store ? nullptr : priorities;
  s->last_scan_may_start_early = may_start_early;
  rc = s->settle(stream, /*after_next=*/true);  // what the previous scan owes goes behind this one and runs beside it
  if (owe) {
    s->l1_owed = true;
    s->owed_slot = slot;
    s->owed_stream = stream;
    s->drawn_since_scan = false;
  }
  return rc;
}

int gearb_sampler_scan_totals(gearb_sampler *s, const float *priorities, void *stream) {
  TraceRange trace("gearb:scan_totals");
  GEARB_REQUIRE(s, "sampler_scan_totals: null sampler");
  // The launch may begin while the one before it in the stream is finishing -- a sampling launch
  // that reads the level 1 and block totals of the OTHER slot.
  return scan_whole(s, priorities, as_stream(stream), /*store=*/false, /*may_start_early=*/true);
}

int gearb_sampler_scan_alternate(gearb_sampler *s, const float *priorities, void *stream) {
  TraceRange trace("gearb:scan");
  GEARB_REQUIRE(s, "sampler_scan_alternate: null sampler");
  return scan_whole(s, priorities, as_stream(stream), /*store=*/true, /*may_start_early=*/true);
}

int gearb_sampler_scan(gearb_sampler *s, const float *priorities, void *stream) {
  TraceRange trace("gearb:scan");
  GEARB_REQUIRE(s, "sampler_scan: null sampler");
  s->scan_unconsumed = true;  // never beside the launch before it: that launch may read this table's level 2
  return scan_whole(s, priorities, as_stream(stream), /*store=*/true, /*may_start_early=*/false);
}

int gearb_sampler_scan_search(gearb_sampler *s, const float *priorities, const double *variates, int64_t b,
                              int flags, int64_t *out_index, void *stream) {
  TraceRange trace("gearb:scan_search");
  GEARB_REQUIRE(s, "sampler_scan_search: null sampler");
  {
    int rc0 = s->settle(as_stream(stream));
    if (rc0 != GEARB_OK) return rc0;
  }
  s->lazy_prio = nullptr;
  const int slot = s->take_slot();
  int fused = 0;
  int rc = launch_scan_search(priorities, s->n, s->cdf, s->l1s[slot], s->scratch(), s->scratch_bytes, s->status,
                              s->blk[slot], variates, b, flags, out_index, as_stream(stream), &fused);
  if (rc != GEARB_OK) return rc;
  s->scan_unconsumed = false;  // in either form the draw comes after the scan
  if (fused) return GEARB_OK;
  rc = launch_scan(priorities, s->n, s->cdf, s->l1s[slot], s->scratch(), s->scratch_bytes, s->status, 0,
                   as_stream(stream), true, false, s->blk[slot]);
  if (rc != GEARB_OK) return rc;
  return launch_search(s->cdf, s->l1s[slot], s->n, variates, b, flags, out_index, s->status, as_stream(stream));
}

int gearb_sampler_update(gearb_sampler *s, float *priorities, const int64_t *idx, const float *values, int64_t m,
                         void *stream) {
  TraceRange trace("gearb:update");
  GEARB_REQUIRE(s, "sampler_update: null sampler");
  {
    int rc0 = s->settle(as_stream(stream));
    if (rc0 != GEARB_OK) return rc0;
  }
  s->scan_unconsumed = false;  // this launch waits for the scan before it (see may_overlap)
  GEARB_REQUIRE(!s->lazy_prio || s->lazy_prio == priorities,
                "sampler_update: not the array the table was built from");
  return launch_update(priorities, s->n, s->lazy_prio ? nullptr : s->cdf, s->l1(), scan_aggregate_words(s->scratch()),
                       s->blk[s->slot], static_cast<ScanHeader *>(s->scratch()), s->upd, idx,
                       values, m, s->status, as_stream(stream));
}

int gearb_sampler_search(gearb_sampler *s, const double *variates, int64_t b, int flags,
                         int64_t *out_index, void *stream) {
  TraceRange trace("gearb:search");
  GEARB_REQUIRE(s, "sampler_search: null sampler");
  {
    int rc0 = s->settle(as_stream(stream));
    if (rc0 != GEARB_OK) return rc0;
  }
  s->scan_unconsumed = false;  // this launch waits for the scan before it (see may_overlap)
  if (s->lazy_prio) return fail(GEARB_ERR_STATE, "sampler_search: the table was built without its level-2 entries");
  return launch_search(s->cdf, s->l1(), s->n, variates, b, flags, out_index, s->status,
                       as_stream(stream));
}

int gearb_sampler_sample_gather_affine(gearb_sampler *s, gearb_handler *h, const double *variates, int64_t b,
                                       double mul, double sub, const int64_t *lengths, int64_t index_offset,
                                       const int32_t *columns, int ncols, void *const *dst, int zero_fill,
                                       int64_t *out_flat, int64_t *out_idx, int64_t *out_ts, int64_t *out_len,
                                       int64_t flat_offset, int slot_mod, int64_t slot_lo, const int64_t *slot_base,
                                       void *stream) {
  TraceRange trace("gearb:sample_gather(owner)");
  GEARB_REQUIRE(s, "sample_gather: null sampler");
  {
    int rc0 = s->settle(as_stream(stream));
    if (rc0 != GEARB_OK) return rc0;
  }
  s->scan_unconsumed = false;  // this launch waits for the scan before it (see may_overlap)
  GEARB_REQUIRE(slot_mod >= -1 && slot_mod <= GEARB_MAX_SHARDS && (slot_mod == 0 || slot_mod == 1 || slot_base),
                "sample_gather: bad slot map");
  GatherParams p;
  int rc = build_gather_params(h, columns, ncols, b, dst, zero_fill, s->status, p, GEARB_SG_PIECE);
  if (rc != GEARB_OK) return rc;
  if (slot_mod > 1 || slot_mod == -1) {
    p.slot_mod = slot_mod;
    p.slot_lo = slot_lo;
    for (int q = 0; q < (slot_mod > 1 ? slot_mod : 3); ++q) p.slot_base[q] = slot_base[q];
  }
  GEARB_REQUIRE(s->n <= h->table->capacity * h->table->T,
                "sample_gather: %lld priorities but the table holds only %lld steps", (long long)s->n,
                (long long)(h->table->capacity * h->table->T));
  DrawLayout lay;
  lay.flat_offset = flat_offset;
  return launch_sample_gather(p, s->cdf, s->l1(), s->n, variates, GEARB_SEARCH_AFFINE, lengths, index_offset,
                              out_flat, out_idx, out_ts, out_len, as_stream(stream), mul, sub, s->lazy_prio,
                              s->blk[s->slot], lay);
}

int gearb_sampler_sample_gather(gearb_sampler *s, gearb_handler *h, const double *variates, int64_t b,
                                int flags, const int64_t *lengths, int64_t index_offset,
                                const int32_t *columns, int ncols, void *const *dst, int zero_fill,
                                int64_t *out_flat, int64_t *out_idx, int64_t *out_ts, int64_t *out_len,
                                void *stream) {
  TraceRange trace("gearb:sample_gather");
  GEARB_REQUIRE(s, "sample_gather: null sampler");
  s->scan_unconsumed = false;  // this launch waits for the scan before it (see may_overlap)
  GEARB_REQUIRE((flags & ~GEARB_SEARCH_SCALE) == 0, "sample_gather: unknown flag");
  GatherParams p;
  int rc = build_gather_params(h, columns, ncols, b, dst, zero_fill, s->status, p, GEARB_SG_PIECE);
  if (rc != GEARB_OK) return rc;
  GEARB_REQUIRE(s->n <= h->table->capacity * h->table->T,
                "sample_gather: %lld priorities but the table holds only %lld steps", (long long)s->n,
                (long long)(h->table->capacity * h->table->T));
  // Level 1 still owed for this very table: the launch finds partitions through what the scan
  // left (the level-1 launch follows the next scan, or the next call that needs the table).
  // Only for the first draw after the scan: a second draw from one table says that no scan is
  // about to follow, so the table is completed and the launch takes its full width again.
  Level1Sums sums;
  const bool from_sums = s->l1_owed && s->owed_slot == s->slot && !s->drawn_since_scan;
  s->drawn_since_scan = true;
  if (from_sums) {
    sums.sb = s->sb[s->slot];
    sums.agg = scan_aggregate_words(s->scratch());
    sums.range = &static_cast<ScanHeader *>(s->scratch())->pad[1];
    // the scan expected behind this launch: a totals-only one fits beside two of its CTAs per
    // SM, a storing one of the other of two tables beside four; a storing scan of THIS table
    // cannot start before the launch has ended, so the launch keeps its full width
    sums.ctas_per_sm = s->lazy_prio ? 2 : (s->last_scan_may_start_early ? 4 : 0);
  } else {
    rc = s->settle(as_stream(stream));
    if (rc != GEARB_OK) return rc;
  }
  return launch_sample_gather(p, s->cdf, s->l1(), s->n, variates, flags, lengths, index_offset, out_flat,
                              out_idx, out_ts, out_len, as_stream(stream), 1.0, 0.0, s->lazy_prio,
                              s->blk[s->slot], DrawLayout(), from_sums ? &sums : nullptr);
}

int gearb_ipc_export(const void *device_ptr, void *handle64) {
  GEARB_REQUIRE(device_ptr && handle64, "ipc_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == GEARB_IPC_HANDLE_BYTES, "handle size");
  cudaIpcMemHandle_t hd;
  GEARB_CUDA(cudaIpcGetMemHandle(&hd, const_cast<void *>(device_ptr)));
  memcpy(handle64, &hd, sizeof(hd));
  return GEARB_OK;
}

int gearb_ipc_open(const void *handle64, void **device_ptr) {
  GEARB_REQUIRE(device_ptr && handle64, "ipc_open: null argument");
  cudaIpcMemHandle_t hd;
  memcpy(&hd, handle64, sizeof(hd));
  GEARB_CUDA(cudaIpcOpenMemHandle(device_ptr, hd, cudaIpcMemLazyEnablePeerAccess));
  return GEARB_OK;
}

int gearb_ipc_close(void *device_ptr) {
  GEARB_REQUIRE(device_ptr, "ipc_close: null argument");
  GEARB_CUDA(cudaIpcCloseMemHandle(device_ptr));
  return GEARB_OK;
}

int gearb_device_alloc(int64_t bytes, void **ptr) {
  GEARB_REQUIRE(ptr && bytes > 0, "device_alloc: bad argument");
  cudaError_t e = cudaMalloc(ptr, static_cast<size_t>(bytes));
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return fail(GEARB_ERR_NOMEM, "cudaMalloc(%lld bytes) failed: %s", (long long)bytes, cudaGetErrorString(e));
  }
  GEARB_CUDA(cudaMemset(*ptr, 0, static_cast<size_t>(bytes)));
  return GEARB_OK;
}

int gearb_device_free(void *ptr) {
  if (ptr) GEARB_CUDA(cudaFree(ptr));
  return GEARB_OK;
}

int64_t gearb_mailbox_bytes(int64_t n) {
  return n > 0 ? mailbox_blk_base(n) + 2 * GEARB_MAX_SHARDS * mailbox_blk_stride(n) : GEARB_MAILBOX_BYTES;
}

int64_t gearb_mailbox_l1_offset(int64_t n, uint64_t epoch, int shard) {
  if (n <= 0 || shard < 0 || shard >= GEARB_MAX_SHARDS) return -1;
  return GEARB_MAILBOX_BYTES +
         (static_cast<int64_t>(epoch & 1u) * GEARB_MAX_SHARDS + shard) * mailbox_l1_stride(n);
}

int64_t gearb_mailbox_blk_offset(int64_t n, uint64_t epoch, int shard) {
  if (n <= 0 || shard < 0 || shard >= GEARB_MAX_SHARDS) return -1;
  return mailbox_blk_base(n) + (static_cast<int64_t>(epoch & 1u) * GEARB_MAX_SHARDS + shard) * mailbox_blk_stride(n);
}

int gearb_sampler_publish(gearb_sampler *s, int world, int rank, void *const *mailboxes, uint64_t epoch,
                          int copy_l1, void *stream) {
  TraceRange trace("gearb:publish");
  GEARB_REQUIRE(s, "publish: null sampler");
  {
    int rc0 = s->settle(as_stream(stream));
    if (rc0 != GEARB_OK) return rc0;
  }
  s->scan_unconsumed = false;  // this launch waits for the scan before it (see may_overlap)
  unsigned *counter = &static_cast<ScanHeader *>(s->scratch())->pad[kPadPublish];
  // with the level-1 copy, a table without stored level 2 also sends its block totals of this step
  return launch_publish(s->l1(), s->nparts, world, rank, mailboxes, epoch, copy_l1, counter, as_stream(stream),
                        (copy_l1 && s->lazy_prio) ? s->blk[s->slot] : nullptr);
}

int gearb_sampler_scan_totals_publish(gearb_sampler *s, const float *priorities, int world, int rank,
                                      void *const *mailboxes, uint64_t epoch, void *stream) {
  TraceRange trace("gearb:scan_totals+publish");
  GEARB_REQUIRE(s && mailboxes, "scan_totals_publish: null argument");
  GEARB_REQUIRE(world >= 1 && world <= GEARB_MAX_SHARDS && rank >= 0 && rank < world && epoch > 0,
                "scan_totals_publish: bad rank, world or epoch");
  int rc = s->settle(as_stream(stream));  // peers read this table's level 1: nothing is left owing here
  if (rc != GEARB_OK) return rc;
  const int before = s->slot;
  const int slot = s->take_slot();
  PublishTail tail;
  tail.world = world;
  tail.rank = rank;
  tail.epoch = epoch;
  for (int j = 0; j < world; ++j) {
    GEARB_REQUIRE(mailboxes[j], "scan_totals_publish: null mailbox for rank %d", j);
    tail.box[j] = mailboxes[j];
  }
  // Tables whose level 1 is its own launch let that launch write the mailboxes at its end; the
  // others (at most 1024 partitions: level 1 by the scan's last CTA) take the publish launch.
  const bool in_level1 = s->nparts > 1024 && level1_can_follow_next_scan(s->nparts);
  rc = launch_scan(priorities, s->n, nullptr, s->l1s[slot], s->scratch(), s->scratch_bytes, s->status, 0,
                   as_stream(stream), true, /*overlap_previous=*/s->may_overlap() && slot != before, s->blk[slot],
                   nullptr, in_level1 ? &tail : nullptr);
  if (rc != GEARB_OK) return rc;
  s->lazy_prio = priorities;
  s->scan_unconsumed = false;  // the level-1 launch behind the scan waits for it
  if (in_level1) return GEARB_OK;
  unsigned *counter = &static_cast<ScanHeader *>(s->scratch())->pad[kPadPublish];
  return launch_publish(s->l1(), s->nparts, world, rank, mailboxes, epoch, 0, counter, as_stream(stream));
}

int gearb_sampler_publish_total(gearb_sampler *s, int world, int rank, void *const *mailboxes, uint64_t epoch,
                                void *stream) {
  return gearb_sampler_publish(s, world, rank, mailboxes, epoch, 0, stream);
}

int gearb_sampler_pull_ex(gearb_sampler *s, gearb_handler *h, const gearb_pull_args *a, void *stream) {
  TraceRange trace("gearb:pull");
  GEARB_REQUIRE(s && a, "pull: null sampler or arguments");
  {
    int rc0 = s->settle(as_stream(stream));
    if (rc0 != GEARB_OK) return rc0;
  }
  s->scan_unconsumed = false;  // this launch waits for the scan before it (see may_overlap)
  GEARB_REQUIRE(a->cdf || a->prio, "pull: neither level-2 tables nor priorities were given");
  GEARB_REQUIRE(a->totals || a->mailbox, "pull: neither totals nor a mailbox were given");
  GatherParams p;
  int rc = build_gather_params(h, a->columns, a->ncols, a->b, a->dst, a->zero_fill, s->status, p, GEARB_SG_PIECE);
  if (rc != GEARB_OK) return rc;
  GEARB_REQUIRE(s->n <= h->table->capacity * h->table->T,
                "pull: %lld priorities but a shard holds only %lld steps", (long long)s->n,
                (long long)(h->table->capacity * h->table->T));
  GEARB_REQUIRE(h->table->hbm, "pull: the shards must be in device memory");
  if (p.stage_bytes == 0) p.ring = a->ring ? 1 : 0;
  DrawLayout lay;
  lay.u_stride = a->variate_stride > 0 ? a->variate_stride : 1;
  return launch_pull(p, a->world, a->self, a->mailbox ? nullptr : a->totals, a->cdf, a->cdf ? nullptr : a->prio,
                     a->cdf ? nullptr : a->blk, a->l1, a->table, s->n, a->variates, a->out_flat, a->out_idx,
                     a->out_ts, as_stream(stream), a->mailbox, a->epoch, lay);
}

int gearb_sampler_pull_mailbox(gearb_sampler *s, gearb_handler *h, int world, int self, const void *mailbox,
                               uint64_t epoch, const void *const *cdf, const void *const *l1,
                               const void *const *table, const double *variates, int64_t b, const int32_t *columns,
                               int ncols, void *const *dst, int zero_fill, int ring, int64_t *out_flat,
                               int64_t *out_idx, int64_t *out_ts, void *stream) {
  GEARB_REQUIRE(mailbox && cdf, "pull: null mailbox or level-2 tables");
  gearb_pull_args a = {};
  a.world = world; a.self = self; a.mailbox = mailbox; a.epoch = epoch; a.cdf = cdf; a.l1 = l1; a.table = table;
  a.variates = variates; a.b = b; a.variate_stride = 1; a.columns = columns; a.ncols = ncols; a.dst = dst;
  a.zero_fill = zero_fill; a.ring = ring; a.out_flat = out_flat; a.out_idx = out_idx; a.out_ts = out_ts;
  return gearb_sampler_pull_ex(s, h, &a, stream);
}

int gearb_sampler_pull(gearb_sampler *s, gearb_handler *h, int world, int self, const double *totals,
                       const void *const *cdf, const void *const *l1, const void *const *table,
                       const double *variates, int64_t b, const int32_t *columns, int ncols,
                       void *const *dst, int zero_fill, int ring, int64_t *out_flat, int64_t *out_idx,
                       int64_t *out_ts, void *stream) {
  GEARB_REQUIRE(totals && cdf, "pull: null totals or level-2 tables");
  gearb_pull_args a = {};
  a.world = world; a.self = self; a.totals = totals; a.cdf = cdf; a.l1 = l1; a.table = table;
  a.variates = variates; a.b = b; a.variate_stride = 1; a.columns = columns; a.ncols = ncols; a.dst = dst;
  a.zero_fill = zero_fill; a.ring = ring; a.out_flat = out_flat; a.out_idx = out_idx; a.out_ts = out_ts;
  return gearb_sampler_pull_ex(s, h, &a, stream);
}

int gearb_sampler_select_slot(gearb_sampler *s, int slot) {
  GEARB_REQUIRE(s && (slot == 0 || slot == 1), "sampler_select_slot: slot must be 0 or 1");
  s->next_slot = slot;
  return GEARB_OK;
}

int gearb_sampler_level1_buffers(const gearb_sampler *s, double **slot0, double **slot1) {
  GEARB_REQUIRE(s, "sampler_level1_buffers: null sampler");
  if (slot0) *slot0 = s->l1s[0];
  if (slot1) *slot1 = s->l1s[1];
  return GEARB_OK;
}

int gearb_sampler_block_totals(const gearb_sampler *s, float **slot0, float **slot1, int *current) {
  GEARB_REQUIRE(s, "sampler_block_totals: null sampler");
  if (slot0) *slot0 = s->blk[0];
  if (slot1) *slot1 = s->blk[1];
  if (current) *current = s->slot;
  return GEARB_OK;
}

int gearb_sampler_clear_status(gearb_sampler *s, void *stream) {
  GEARB_REQUIRE(s, "sampler_clear_status: null sampler");
  GEARB_CUDA(cudaMemsetAsync(s->status, 0, sizeof(int32_t) * GEARB_STATUS_WORDS, as_stream(stream)));
  return GEARB_OK;
}

int gearb_sampler_buffers(const gearb_sampler *cs, float **cdf, double **l1, int32_t **status) {
  GEARB_REQUIRE(cs, "sampler_buffers: null sampler");
  gearb_sampler *s = const_cast<gearb_sampler *>(cs);
  if (l1) {  // whoever asks for the table gets it launched, on the stream of the scan that owes it
    int rc0 = s->settle(s->owed_stream);
    if (rc0 != GEARB_OK) return rc0;
  }
  if (cdf) *cdf = s->cdf;
  if (l1) *l1 = s->l1();
  if (status) *status = s->status;
  return GEARB_OK;
}

int gearb_sampler_result(gearb_sampler *s, void *stream, double *total, int32_t *status) {
  GEARB_REQUIRE(s, "sampler_result: null sampler");
  {
    int rc0 = s->settle(as_stream(stream));
    if (rc0 != GEARB_OK) return rc0;
  }
  GEARB_CUDA(cudaStreamSynchronize(as_stream(stream)));
  if (total)
    GEARB_CUDA(cudaMemcpy(total, s->l1() + s->nparts, sizeof(double), cudaMemcpyDeviceToHost));
  int32_t st[GEARB_STATUS_WORDS];
  GEARB_CUDA(cudaMemcpy(st, s->status, sizeof(st), cudaMemcpyDeviceToHost));
  if (status) std::memcpy(status, st, sizeof(st));
  if (st[0] & GEARB_ST_SCAN_ABORTED)
    return fail(GEARB_ERR_TIMEOUT, "a bounded wait on the device ran out (status 0x%x): the tables and the last "
                "batch are not valid; gearb_sampler_clear_status re-arms the status word", st[0]);
  return GEARB_OK;
}

/* ------------------------------ fill ----------------------------------- */
int gearb_fill(void *dst, int64_t count, int kind, uint64_t seed, uint64_t stream_id, double a,
               double b, void *stream) {
  return launch_fill(dst, count, kind, seed, stream_id, a, b, as_stream(stream));
}

}  // extern "C"
