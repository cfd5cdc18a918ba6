// Online trajectory ingestion: the hand-off between simulator processes, which fill trajectories
// of the table, and the trainer process, which samples them.
//
// Stands where the reference's SharedMemoryIndexServer / SharedMemoryIndexClient are
// (src/index/server.cc:115-190, src/index/client.cc:30-91, include/index/sim_status.h:7-17,
// include/circular_buffer.h): one 64-byte status slot per simulator in a System-V segment, an
// ownership word that is passed back and forth with release / acquire ordering, a FIFO of
// trajectory indices that are free to be (over)written, and per-trajectory weight / length
// arrays that a committed trajectory updates.  The protocol is the reference's:
//
//   simulator                               trainer (one scan over all slots)
//   ---------                               -------
//   owns the slot, no trajectory:           owns the slot:
//     ask for one (terminated, alloc)   ->    running trajectory -> an inference request, slot
//   owns the slot, has a trajectory:           handed back by callback() once it is answered
//     step ... writeback(terminated?)   ->    finished trajectory -> its index to the back of the
//                                              FIFO, (index, length, weight) recorded as an update
//                                             allocation wanted -> front of the FIFO, recorded with
//                                              weight 0 (not selectable while it is being written)
//
// What differs: every wait takes a time limit and returns a status code (the reference spins
// until the Python signal handler fires), the updates of one scan come back de-duplicated and
// in order (the device-side incremental update, gearb_sampler_update, wants one writer per
// index), the whole server state is one flat byte image, and nothing aborts.
#include <errno.h>
#include <sys/ipc.h>
#include <sys/shm.h>
#include <time.h>

#include <atomic>
#include <cstring>
#include <new>
#include <thread>
#include <vector>

#include "common.h"

namespace {

struct alignas(64) Slot {
  std::atomic<uint32_t> owner;  // 0: the simulator's turn, 1: the trainer's
  // guarded by `owner`
  uint8_t terminated, want_alloc, valid, reserved;
  int64_t tindex;
  int64_t timestep;
  double weight;
};
static_assert(sizeof(Slot) == 64, "one slot per cache line");

struct Segment {
  void *addr = nullptr;
  int shmid = -1;
  bool creator = false;
  int attach(int key, size_t bytes, bool create) {
    shmid = create ? shmget(key, bytes, IPC_CREAT | 0777) : shmget(key, bytes, 0666);
    if (shmid == -1)
      return gearb::fail(GEARB_ERR_STATE, "shmget(key=%d, size=%zu, create=%d) failed: errno %d", key, bytes,
                         (int)create, errno);
    void *p = shmat(shmid, nullptr, 0);
    if (p == reinterpret_cast<void *>(-1)) return gearb::fail(GEARB_ERR_STATE, "shmat(key=%d) failed: errno %d", key, errno);
    addr = p;
    creator = create;
    return GEARB_OK;
  }
  ~Segment() {
    if (!addr) return;
    shmdt(addr);
    if (creator && shmid != -1) shmctl(shmid, IPC_RMID, nullptr);
  }
};

double now_ms() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

}  // namespace

struct gearb_ingest_server {
  int key = 0, num_clients = 0;
  int64_t capacity = 0, index_offset = 0;
  Segment seg;
  Slot *slots = nullptr;
  std::vector<float> weights;
  std::vector<int64_t> timesteps;
  // FIFO of free trajectory indices (global ids, index_offset included)
  std::vector<int64_t> ring;
  int64_t head = 0, count = 0;
  std::vector<int64_t> slot_of_update;  // per local index: position in this scan's update list, or -1

  bool pop(int64_t &v) {
    if (count == 0) return false;
    v = ring[head];
    head = (head + 1) % capacity;
    --count;
    return true;
  }
  bool push(int64_t v) {
    if (count == capacity) return false;
    ring[(head + count) % capacity] = v;
    ++count;
    return true;
  }
};

struct gearb_ingest_client {
  int rank = 0, num_clients = 0;
  Segment seg;
  Slot *slot = nullptr;
  bool on_the_fly = false;
  int64_t tindex = 0, timestep = 0;
};

using namespace gearb;

extern "C" {

int gearb_ingest_server_create(int shm_key, int num_clients, int64_t index_offset, int64_t capacity,
                               gearb_ingest_server **out) {
  GEARB_REQUIRE(out && shm_key != 0 && num_clients > 0 && capacity > 0 && index_offset >= 0,
                "ingest_server_create: bad argument");
  auto *s = new (std::nothrow) gearb_ingest_server();
  if (!s) return fail(GEARB_ERR_NOMEM, "ingest_server_create: out of memory");
  s->key = shm_key;
  s->num_clients = num_clients;
  s->capacity = capacity;
  s->index_offset = index_offset;
  int rc = s->seg.attach(shm_key, sizeof(Slot) * static_cast<size_t>(num_clients), true);
  if (rc != GEARB_OK) {
    delete s;
    return rc;
  }
  s->slots = static_cast<Slot *>(s->seg.addr);
  for (int i = 0; i < num_clients; ++i) {
    Slot *q = new (s->slots + i) Slot();
    q->terminated = q->want_alloc = q->valid = q->reserved = 0;
    q->tindex = q->timestep = 0;
    q->weight = 0.0;
    q->owner.store(0, std::memory_order_release);
  }
  s->weights.assign(static_cast<size_t>(capacity), 0.f);
  s->timesteps.assign(static_cast<size_t>(capacity), 0);
  s->ring.resize(static_cast<size_t>(capacity));
  for (int64_t i = 0; i < capacity; ++i) s->ring[i] = i + index_offset;  // server.cc:62-64
  s->count = capacity;
  s->slot_of_update.assign(static_cast<size_t>(capacity), -1);
  *out = s;
  return GEARB_OK;
}

int gearb_ingest_server_destroy(gearb_ingest_server *s) {
  delete s;
  return GEARB_OK;
}

/* One pass over the simulators' slots (SharedMemoryIndexServer::scan, server.cc:115-170).
 * Inference requests (slot, trajectory, timestep) of running trajectories and the updates
 * (trajectory, length, weight) of committed or freshly allocated ones are appended to the
 * caller's arrays; an index appears at most once among the updates, with its latest values. */
int gearb_ingest_server_scan(gearb_ingest_server *s, int32_t *infer_src, int64_t *infer_idx, int64_t *infer_ts,
                             int64_t infer_cap, int64_t *n_infer, int64_t *upd_idx, int64_t *upd_ts, float *upd_w,
                             int64_t upd_cap, int64_t *n_upd) {
  GEARB_REQUIRE(s && n_infer && n_upd, "ingest_server_scan: null argument");
  GEARB_REQUIRE(infer_cap >= s->num_clients && infer_src && infer_idx && infer_ts,
                "ingest_server_scan: room for one inference request per simulator is required");
  GEARB_REQUIRE(upd_cap >= 2 * static_cast<int64_t>(s->num_clients) && upd_idx && upd_ts && upd_w,
                "ingest_server_scan: room for two updates per simulator is required");
  int64_t ni = 0, nu = 0;
  auto record = [&](int64_t gidx, int64_t ts, float w) {
    const int64_t local = gidx - s->index_offset;
    int64_t &pos = s->slot_of_update[static_cast<size_t>(local)];
    if (pos < 0) pos = nu++;
    upd_idx[pos] = gidx;
    upd_ts[pos] = ts;
    upd_w[pos] = w;
  };
  int bad = 0;
  for (int i = 0; i < s->num_clients; ++i) {
    Slot *q = s->slots + i;
    if (q->owner.load(std::memory_order_acquire) != 1u) continue;
    if (!q->terminated) {
      if (q->valid) {
        infer_src[ni] = i;
        infer_idx[ni] = q->tindex;
        infer_ts[ni] = q->timestep;
        ++ni;
      } else {
        ++bad;  // a running slot without a trajectory: left with the trainer, reported below
      }
      continue;
    }
    if (q->valid) {  // a finished trajectory: it becomes selectable, its index goes to the back of the FIFO
      const int64_t local = q->tindex - s->index_offset;
      if (local >= 0 && local < s->capacity) {
        s->push(q->tindex);
        record(q->tindex, q->timestep, static_cast<float>(q->weight));
      } else {
        ++bad;
      }
      q->valid = 0;
    }
    if (q->want_alloc) {
      int64_t fresh = 0;
      if (s->pop(fresh)) {
        q->want_alloc = 0;
        q->terminated = 0;
        q->tindex = fresh;
        q->timestep = 0;
        q->weight = 0.0;
        q->valid = 1;
        record(fresh, 0, 0.f);  // weight 0: not selectable while it is being written (server.cc:147)
        q->owner.store(0, std::memory_order_release);
      }  // else: nothing free; the slot stays with the trainer until a later scan
    } else {
      q->owner.store(0, std::memory_order_release);
    }
  }
  for (int64_t k = 0; k < nu; ++k) s->slot_of_update[static_cast<size_t>(upd_idx[k] - s->index_offset)] = -1;
  *n_infer = ni;
  *n_upd = nu;
  if (bad) return fail(GEARB_ERR_STATE, "ingest_server_scan: %d slot(s) in an invalid state (running without a "
                       "trajectory, or an index outside this shard)", bad);
  return GEARB_OK;
}

/* SharedMemoryIndexServer::update (server.cc:172-177): the updates into the weight / length arrays. */
int gearb_ingest_server_update(gearb_ingest_server *s, const int64_t *upd_idx, const int64_t *upd_ts,
                               const float *upd_w, int64_t n) {
  GEARB_REQUIRE(s && (n == 0 || (upd_idx && upd_ts && upd_w)), "ingest_server_update: null argument");
  for (int64_t k = 0; k < n; ++k) {
    const int64_t local = upd_idx[k] - s->index_offset;
    GEARB_REQUIRE(local >= 0 && local < s->capacity, "ingest_server_update: index %lld outside this shard",
                  (long long)upd_idx[k]);
    s->weights[static_cast<size_t>(local)] = upd_w[k];
    s->timesteps[static_cast<size_t>(local)] = upd_ts[k];
  }
  return GEARB_OK;
}

/* SharedMemoryIndexServer::callback (server.cc:179-188): answered slots go back to their simulators. */
int gearb_ingest_server_callback(gearb_ingest_server *s, const int32_t *srcs, int64_t n) {
  GEARB_REQUIRE(s && (n == 0 || srcs), "ingest_server_callback: null argument");
  for (int64_t k = 0; k < n; ++k) {
    GEARB_REQUIRE(srcs[k] >= 0 && srcs[k] < s->num_clients, "ingest_server_callback: slot %d out of range", srcs[k]);
    s->slots[srcs[k]].owner.store(0, std::memory_order_release);
  }
  return GEARB_OK;
}

float *gearb_ingest_server_weights(gearb_ingest_server *s) { return s ? s->weights.data() : nullptr; }
int64_t *gearb_ingest_server_timesteps(gearb_ingest_server *s) { return s ? s->timesteps.data() : nullptr; }
int64_t gearb_ingest_server_free_count(const gearb_ingest_server *s) { return s ? s->count : 0; }

/* The whole server as one byte image (SharedMemoryIndexServerState, include/index/server.h:20-52):
 * header | slots | weights | lengths | FIFO in order.  get with buf == NULL returns the size. */
int64_t gearb_ingest_server_get_state(const gearb_ingest_server *s, void *buf, int64_t cap) {
  if (!s) return -1;
  const int64_t hdr[6] = {s->capacity, s->num_clients, s->index_offset, s->key, s->count, 0x6EA2};
  const int64_t need = static_cast<int64_t>(sizeof(hdr)) + 64 * s->num_clients + 12 * s->capacity + 8 * s->count;
  if (!buf) return need;
  if (cap < need) return -1;
  char *p = static_cast<char *>(buf);
  std::memcpy(p, hdr, sizeof(hdr)); p += sizeof(hdr);
  std::memcpy(p, s->slots, 64 * static_cast<size_t>(s->num_clients)); p += 64 * s->num_clients;
  std::memcpy(p, s->weights.data(), 4 * static_cast<size_t>(s->capacity)); p += 4 * s->capacity;
  std::memcpy(p, s->timesteps.data(), 8 * static_cast<size_t>(s->capacity)); p += 8 * s->capacity;
  for (int64_t k = 0; k < s->count; ++k) {
    const int64_t v = s->ring[(s->head + k) % s->capacity];
    std::memcpy(p, &v, 8); p += 8;
  }
  return need;
}

int gearb_ingest_server_set_state(gearb_ingest_server *s, const void *buf, int64_t bytes) {
  GEARB_REQUIRE(s && buf && bytes >= 48, "ingest_server_set_state: bad argument");
  int64_t hdr[6];
  std::memcpy(hdr, buf, sizeof(hdr));
  // the reference refuses a state of another shape (server.cc:204-209)
  GEARB_REQUIRE(hdr[5] == 0x6EA2 && hdr[0] == s->capacity && hdr[1] == s->num_clients && hdr[3] == s->key,
                "Can not rebuild SharedMemoryIndexServer from State, key, capacity or num_clients mismatch");
  GEARB_REQUIRE(hdr[4] >= 0 && hdr[4] <= s->capacity &&
                    bytes == 48 + 64 * s->num_clients + 12 * s->capacity + 8 * hdr[4],
                "ingest_server_set_state: truncated state");
  s->index_offset = hdr[2];
  const char *p = static_cast<const char *>(buf) + sizeof(hdr);
  std::memcpy(static_cast<void *>(s->slots), p, 64 * static_cast<size_t>(s->num_clients)); p += 64 * s->num_clients;
  std::memcpy(s->weights.data(), p, 4 * static_cast<size_t>(s->capacity)); p += 4 * s->capacity;
  std::memcpy(s->timesteps.data(), p, 8 * static_cast<size_t>(s->capacity)); p += 8 * s->capacity;
  s->head = 0;
  s->count = hdr[4];
  std::memcpy(s->ring.data(), p, 8 * static_cast<size_t>(s->count));
  return GEARB_OK;
}

/* ------------------------------------------------------------------ simulator side */
int gearb_ingest_client_create(int shm_key, int client_rank, int num_clients, gearb_ingest_client **out) {
  GEARB_REQUIRE(out && shm_key != 0 && num_clients > 0 && client_rank >= 0 && client_rank < num_clients,
                "ingest_client_create: bad argument");
  auto *c = new (std::nothrow) gearb_ingest_client();
  if (!c) return fail(GEARB_ERR_NOMEM, "ingest_client_create: out of memory");
  c->rank = client_rank;
  c->num_clients = num_clients;
  int rc = c->seg.attach(shm_key, sizeof(Slot) * static_cast<size_t>(num_clients), false);
  if (rc != GEARB_OK) {  // the server has not created the segment yet: callers retry (client.cc:19-27)
    delete c;
    return rc;
  }
  c->slot = static_cast<Slot *>(c->seg.addr) + client_rank;
  *out = c;
  return GEARB_OK;
}

int gearb_ingest_client_destroy(gearb_ingest_client *c) {
  delete c;
  return GEARB_OK;
}

static int wait_for_turn(gearb_ingest_client *c, double deadline) {
  unsigned spins = 0;
  while (c->slot->owner.load(std::memory_order_acquire) != 0u) {
    if (++spins < 64) {
      std::this_thread::yield();
    } else {
      if (now_ms() > deadline) return fail(GEARB_ERR_TIMEOUT, "ingest client %d: the trainer kept the slot", c->rank);
      timespec nap = {0, 50000};
      nanosleep(&nap, nullptr);
    }
  }
  return GEARB_OK;
}

/* SharedMemoryIndexClient::acquire (client.cc:30-50): returns once this simulator holds a
 * trajectory to fill (asking the trainer for one first if it has none), or GEARB_ERR_TIMEOUT. */
int gearb_ingest_client_acquire(gearb_ingest_client *c, int64_t timeout_ms, int64_t *tindex) {
  GEARB_REQUIRE(c && timeout_ms >= 0, "ingest_client_acquire: bad argument");
  const double deadline = now_ms() + static_cast<double>(timeout_ms);
  for (;;) {
    int rc = wait_for_turn(c, deadline);
    if (rc != GEARB_OK) return rc;
    if (!c->slot->valid) {  // no trajectory: ask for one and give the slot to the trainer
      c->slot->terminated = 1;
      c->slot->want_alloc = 1;
      c->slot->owner.store(1, std::memory_order_release);
      continue;
    }
    c->on_the_fly = true;
    c->tindex = c->slot->tindex;
    c->timestep = 0;
    if (tindex) *tindex = c->tindex;
    return GEARB_OK;
  }
}

/* SharedMemoryIndexClient::wait (client.cc:52-63). */
int gearb_ingest_client_wait(gearb_ingest_client *c, int64_t timeout_ms) {
  GEARB_REQUIRE(c && timeout_ms >= 0, "ingest_client_wait: bad argument");
  return wait_for_turn(c, now_ms() + static_cast<double>(timeout_ms));
}

/* SharedMemoryIndexClient::release (client.cc:28). */
int gearb_ingest_client_release(gearb_ingest_client *c) {
  GEARB_REQUIRE(c, "ingest_client_release: null client");
  c->slot->owner.store(1, std::memory_order_release);
  return GEARB_OK;
}

/* SharedMemoryIndexClient::step_inc (client.cc:97-102): the timestep just written, then one more. */
int64_t gearb_ingest_client_step(gearb_ingest_client *c) {
  if (!c) return 0;
  c->timestep += 1;
  return c->on_the_fly ? c->timestep - 1 : 0;
}

/* SharedMemoryIndexClient::writeback (client.cc:76-91), with the weight the finished trajectory
 * is to be sampled with: hands the slot to the trainer.  Returns the number of steps written. */
int64_t gearb_ingest_client_writeback(gearb_ingest_client *c, int terminated, int alloc_new, double weight) {
  if (!c || !c->on_the_fly) return 0;
  c->slot->terminated = terminated ? 1 : 0;
  c->slot->timestep = c->timestep;
  c->slot->want_alloc = alloc_new ? 1 : 0;
  c->slot->weight = weight;
  c->on_the_fly = !terminated;
  c->slot->owner.store(1, std::memory_order_release);
  return c->timestep;
}

/* get_index / get_timestep / get_status_unsafe (client.cc:65-74,93-95): out[0..6] = owner, terminated,
 * alloc, valid, tindex, timestep, on_the_fly; *weight = the slot's weight. */
int gearb_ingest_client_status(const gearb_ingest_client *c, int64_t *out7, double *weight) {
  GEARB_REQUIRE(c && out7, "ingest_client_status: null argument");
  out7[0] = c->slot->owner.load(std::memory_order_relaxed);
  out7[1] = c->slot->terminated;
  out7[2] = c->slot->want_alloc;
  out7[3] = c->slot->valid;
  out7[4] = c->on_the_fly ? c->tindex : 0;
  out7[5] = c->on_the_fly ? c->timestep : 0;
  out7[6] = c->on_the_fly;
  if (weight) *weight = c->slot->weight;
  return GEARB_OK;
}

}  // extern "C"
