// NCCL communicator behind the C ABI.
//
// Stands where the reference's NcclCommunicator is (src/nccl_comm.cc:4-102): unique id,
// ncclCommInitRank, send / recv / all-reduce on the caller's stream -- plus the collective
// the reference declares and leaves empty, group_exchange (src/nccl_comm.cc:83-86): a
// variable-count all-to-all made of grouped ncclSend / ncclRecv, which is what replaces the
// one-NCCL-call-per-segment loops of subsend / subrecv (src/storage/handler.cc:178-191,208-220).
//
// NCCL is not linked: its entry points are looked up in the process at first use
// (dlopen("libnccl.so.2")), so the library loads on hosts without NCCL and, inside a PyTorch
// process, shares the NCCL that PyTorch already loaded instead of bringing a second copy.
// Failures are status codes (the reference's NCCL_CHECK calls exit(), include/nccl_comm.h:51-59).
#include <dlfcn.h>
#include <nccl.h>

#include <cstring>
#include <mutex>

#include "common.h"

namespace {

struct Nccl {
  void *handle = nullptr;
  decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
  decltype(&ncclCommInitRank) CommInitRank = nullptr;
  decltype(&ncclCommDestroy) CommDestroy = nullptr;
  decltype(&ncclCommCuDevice) CommCuDevice = nullptr;
  decltype(&ncclGetErrorString) GetErrorString = nullptr;
  decltype(&ncclGroupStart) GroupStart = nullptr;
  decltype(&ncclGroupEnd) GroupEnd = nullptr;
  decltype(&ncclSend) Send = nullptr;
  decltype(&ncclRecv) Recv = nullptr;
  decltype(&ncclAllReduce) AllReduce = nullptr;
  decltype(&ncclAllGather) AllGather = nullptr;
  bool ok = false;
};

Nccl &nccl() {
  static Nccl n;
  static std::once_flag once;
  std::call_once(once, [] {
    const char *names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char *name : names) {
      n.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (n.handle) break;
    }
    if (!n.handle) return;
#define GEARB_SYM(field, sym) n.field = reinterpret_cast<decltype(n.field)>(dlsym(n.handle, #sym))
    GEARB_SYM(GetUniqueId, ncclGetUniqueId);
    GEARB_SYM(CommInitRank, ncclCommInitRank);
    GEARB_SYM(CommDestroy, ncclCommDestroy);
    GEARB_SYM(CommCuDevice, ncclCommCuDevice);
    GEARB_SYM(GetErrorString, ncclGetErrorString);
    GEARB_SYM(GroupStart, ncclGroupStart);
    GEARB_SYM(GroupEnd, ncclGroupEnd);
    GEARB_SYM(Send, ncclSend);
    GEARB_SYM(Recv, ncclRecv);
    GEARB_SYM(AllReduce, ncclAllReduce);
    GEARB_SYM(AllGather, ncclAllGather);
#undef GEARB_SYM
    n.ok = n.GetUniqueId && n.CommInitRank && n.CommDestroy && n.CommCuDevice && n.GetErrorString &&
           n.GroupStart && n.GroupEnd && n.Send && n.Recv && n.AllReduce && n.AllGather;
  });
  return n;
}

int need_nccl() {
  if (!nccl().ok) return gearb::fail(GEARB_ERR_NCCL, "NCCL is not available in this process (libnccl.so.2 not found)");
  return GEARB_OK;
}

#define GEARB_NCCL(expr)                                                                   \
  do {                                                                                     \
    ncclResult_t r__ = (expr);                                                             \
    if (r__ != ncclSuccess)                                                                \
      return ::gearb::fail(GEARB_ERR_NCCL, "%s failed: %s", #expr, nccl().GetErrorString(r__)); \
  } while (0)

}  // namespace

struct gearb_comm {
  ncclComm_t comm = nullptr;
  int rank = 0, world = 1;
};

using namespace gearb;

extern "C" {

int gearb_comm_unique_id(char *id128) {
  GEARB_REQUIRE(id128, "comm_unique_id: null argument");
  int rc = need_nccl();
  if (rc) return rc;
  static_assert(sizeof(ncclUniqueId) == 128, "the id travels as 128 bytes, like create_nccl_id");
  ncclUniqueId id;
  GEARB_NCCL(nccl().GetUniqueId(&id));
  std::memcpy(id128, id.internal, 128);
  return GEARB_OK;
}

int gearb_comm_create(int rank, int world, const char *id128, gearb_comm **out) {
  GEARB_REQUIRE(out && id128, "comm_create: null argument");
  GEARB_REQUIRE(world >= 1 && rank >= 0 && rank < world, "comm_create: rank %d of %d", rank, world);
  int rc = need_nccl();
  if (rc) return rc;
  ncclUniqueId id;
  std::memcpy(id.internal, id128, 128);
  auto *c = new gearb_comm();
  c->rank = rank;
  c->world = world;
  ncclResult_t r = nccl().CommInitRank(&c->comm, world, id, rank);
  if (r != ncclSuccess) {
    delete c;
    return fail(GEARB_ERR_NCCL, "ncclCommInitRank(rank %d of %d) failed: %s", rank, world,
                nccl().GetErrorString(r));
  }
  *out = c;
  return GEARB_OK;
}

int gearb_comm_destroy(gearb_comm *c) {
  if (!c) return GEARB_OK;
  if (c->comm && nccl().ok) nccl().CommDestroy(c->comm);
  delete c;
  return GEARB_OK;
}

int gearb_comm_info(const gearb_comm *c, int *rank, int *world, int *device) {
  GEARB_REQUIRE(c, "comm_info: null communicator");
  if (rank) *rank = c->rank;
  if (world) *world = c->world;
  if (device) GEARB_NCCL(nccl().CommCuDevice(c->comm, device));
  return GEARB_OK;
}

int gearb_comm_send(gearb_comm *c, const void *buf, int64_t bytes, int peer, void *stream) {
  GEARB_REQUIRE(c && (buf || bytes == 0) && bytes >= 0, "comm_send: bad argument");
  GEARB_NCCL(nccl().Send(buf, static_cast<size_t>(bytes), ncclUint8, peer, c->comm, as_stream(stream)));
  return GEARB_OK;
}

int gearb_comm_recv(gearb_comm *c, void *buf, int64_t bytes, int peer, void *stream) {
  GEARB_REQUIRE(c && (buf || bytes == 0) && bytes >= 0, "comm_recv: bad argument");
  GEARB_NCCL(nccl().Recv(buf, static_cast<size_t>(bytes), ncclUint8, peer, c->comm, as_stream(stream)));
  return GEARB_OK;
}

int gearb_comm_allreduce_sum(gearb_comm *c, void *buf, int64_t count, int dtype, void *stream) {
  GEARB_REQUIRE(c && buf && count >= 0, "comm_allreduce_sum: bad argument");
  ncclDataType_t t;
  switch (dtype) {
    case GEARB_DT_F32: t = ncclFloat32; break;
    case GEARB_DT_F64: t = ncclFloat64; break;
    case GEARB_DT_I64: t = ncclInt64; break;
    case GEARB_DT_F16: t = ncclFloat16; break;
    default: return fail(GEARB_ERR_INVALID, "comm_allreduce_sum: unsupported dtype %d", dtype);
  }
  GEARB_NCCL(nccl().AllReduce(buf, buf, static_cast<size_t>(count), t, ncclSum, c->comm, as_stream(stream)));
  return GEARB_OK;
}

int gearb_comm_allgather(gearb_comm *c, const void *send, void *recv, int64_t bytes_per_rank, void *stream) {
  GEARB_REQUIRE(c && send && recv && bytes_per_rank >= 0, "comm_allgather: bad argument");
  GEARB_NCCL(nccl().AllGather(send, recv, static_cast<size_t>(bytes_per_rank), ncclUint8, c->comm,
                              as_stream(stream)));
  return GEARB_OK;
}

int gearb_comm_alltoallv(gearb_comm *c, int nbuf, const void *const *send, const int64_t *send_off,
                         const int64_t *send_bytes, void *const *recv, const int64_t *recv_off,
                         const int64_t *recv_bytes, void *stream) {
  TraceRange trace("gearb:alltoallv");
  GEARB_REQUIRE(c && nbuf >= 0, "comm_alltoallv: bad argument");
  if (nbuf == 0) return GEARB_OK;
  GEARB_REQUIRE(send && recv && send_off && send_bytes && recv_off && recv_bytes, "comm_alltoallv: null argument");
  const int W = c->world;
  cudaStream_t s = as_stream(stream);
  // The part addressed to this rank itself never enters NCCL.
  for (int b = 0; b < nbuf; ++b) {
    const int64_t k = static_cast<int64_t>(b) * W + c->rank;
    GEARB_REQUIRE(send_bytes[k] == recv_bytes[k], "comm_alltoallv: self send/recv sizes differ");
    if (send_bytes[k] > 0)
      GEARB_CUDA(cudaMemcpyAsync(static_cast<char *>(recv[b]) + recv_off[k],
                                 static_cast<const char *>(send[b]) + send_off[k],
                                 static_cast<size_t>(send_bytes[k]), cudaMemcpyDeviceToDevice, s));
  }
  if (W == 1) return GEARB_OK;
  GEARB_NCCL(nccl().GroupStart());
  for (int b = 0; b < nbuf; ++b)
    for (int peer = 0; peer < W; ++peer) {
      if (peer == c->rank) continue;
      const int64_t k = static_cast<int64_t>(b) * W + peer;
      if (send_bytes[k] > 0) {
        ncclResult_t r = nccl().Send(static_cast<const char *>(send[b]) + send_off[k],
                                     static_cast<size_t>(send_bytes[k]), ncclUint8, peer, c->comm, s);
        if (r != ncclSuccess) {
          nccl().GroupEnd();
          return fail(GEARB_ERR_NCCL, "ncclSend to %d failed: %s", peer, nccl().GetErrorString(r));
        }
      }
      if (recv_bytes[k] > 0) {
        ncclResult_t r = nccl().Recv(static_cast<char *>(recv[b]) + recv_off[k],
                                     static_cast<size_t>(recv_bytes[k]), ncclUint8, peer, c->comm, s);
        if (r != ncclSuccess) {
          nccl().GroupEnd();
          return fail(GEARB_ERR_NCCL, "ncclRecv from %d failed: %s", peer, nccl().GetErrorString(r));
        }
      }
    }
  GEARB_NCCL(nccl().GroupEnd());
  return GEARB_OK;
}

}  // extern "C"
