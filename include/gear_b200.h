/*
 * gear_b200.h -- C ABI of the B200-native replay sample + gather engine.
 *
 * Every entry point returns a status code (GEARB_OK == 0), never throws and
 * never aborts; gearb_last_error() gives the text for the calling thread's last
 * failure.  Device work is enqueued on the caller's stream and returns
 * asynchronously, like the reference launchers (which use the c10 current
 * stream, src/cuda/copy.cu:169,202,236).  `stream` is a cudaStream_t passed as
 * void*; NULL is the legacy default stream.
 *
 * Each declaration cites the interface of bigrl-team/gear it stands in for
 * (paths relative to that tree).
 */
#ifndef GEAR_B200_H_
#define GEAR_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* ---- status codes ------------------------------------------------------- */
#define GEARB_OK 0
#define GEARB_ERR_INVALID 1     /* bad argument (reference: std::runtime_error)  */
#define GEARB_ERR_CUDA 2        /* CUDA runtime failure (reference: assert(0))   */
#define GEARB_ERR_NOMEM 3
#define GEARB_ERR_STATE 4       /* object not connected / pattern not set        */
#define GEARB_ERR_TIMEOUT 5     /* a bounded device-side wait ran out (gearb_sampler_result) */
#define GEARB_ERR_NCCL 6        /* NCCL failure (reference: exit())              */
#define GEARB_ERR_UNSUPPORTED 7

/* Bits of the device status word written by the kernels (status[0]).        */
#define GEARB_ST_L1_RESUMMED 0x2      /* scan: a float64 partial sum was inexact; level-1 was rebuilt in order */
#define GEARB_ST_BAD_PRIORITY 0x4     /* scan: a priority had its sign bit set (negative, -0.0) or was NaN */
#define GEARB_ST_BAD_REQUEST 0x8      /* gather: trajectory index outside the table, request skipped */
#define GEARB_ST_LEN_CLAMPED 0x10     /* gather: a length beyond trajectory_length was clamped */
#define GEARB_ST_SCAN_ABORTED 0x20    /* a bounded wait inside a kernel ran out (a lost copy, a peer that never
                                         published): the tables or the batch of that launch are NOT valid */
/* status[1] = number of variates that landed within one float32 ulp of a
 * cumulative-priority boundary (search), accumulated until cleared.
 * status[2] = low 32 bits of the epoch at which a pull launch last gave up waiting for its peers.
 * The words accumulate; gearb_sampler_clear_status zeroes them.               */
#define GEARB_STATUS_WORDS 4

/* ---- constants of the cumulative-priority table ------------------------- */
#define GEARB_PART 4096 /* priorities per level-2 partition */

/* ---- residency of a trajectory table ------------------------------------ */
#define GEARB_RES_HOST 1 /* pinned, device-mapped host memory (zero-copy reads) */
#define GEARB_RES_HBM 2  /* device memory                                       */

/* ---- pad options, same numbering as SubscribePattern::PadOption
 *      (include/storage/handler.h:21) ------------------------------------- */
#define GEARB_PAD_INACTIVE 0
#define GEARB_PAD_HEAD 1
#define GEARB_PAD_TAIL 2

#define GEARB_MAX_COLUMNS 16
#define GEARB_MAX_SHARDS 16 /* shards one pull launch can address */

typedef struct gearb_table gearb_table;
typedef struct gearb_handler gearb_handler;
typedef struct gearb_indexset gearb_indexset;
typedef struct gearb_sampler gearb_sampler;
typedef struct gearb_comm gearb_comm;

const char *gearb_last_error(void);
int gearb_version(void);

/* gear::cuda::init, src/cuda/init.cu:6-13 (bound as libgear.core.init). */
int gearb_init(int device);
/* Device count as print_environ reports it, src/env.cc:55-58. */
int gearb_device_count(int *count);

/* ======================= trajectory table =============================== */
/* TrajectoryTable::TrajectoryTable, src/storage/table.cc:8-25, with
 * ColumnSpec::size (src/storage/specs.cc:10-14) already applied by the caller:
 * row_bytes[c] is the byte size of one timestep of column c.  Layout is
 * [trajectory][column][timestep][element].  shm_key != 0 places the host copy
 * in a System-V segment like SharedMemory (src/memory/shared_memory.cc:35-63);
 * shm_key == 0 uses cudaHostAlloc(Mapped|Portable) like CudaUVMemory
 * (src/memory/cuda_uvm.cc:29-32).  Nothing is allocated until connect.      */
int gearb_table_create(const int64_t *row_bytes, int ncols, int64_t trajectory_length,
                       int64_t capacity, int residency, int shm_key, int create,
                       gearb_table **out);
/* TrajectoryTable::connect, src/storage/table.cc:27: returns the table size in
 * *nbytes, or fails with GEARB_ERR_STATE when the segment is not there yet
 * (the Python layer maps that to the reference's -1 and retries).            */
int gearb_table_connect(gearb_table *t, int64_t *nbytes);
int gearb_table_destroy(gearb_table *t);
/* Strides the constructor derives (table.cc:10-24): accu has ncols+1 entries. */
int gearb_table_layout(const gearb_table *t, int64_t *trajectory_stride, int64_t *nbytes,
                       int64_t *accu);
/* TrajectoryTable::get_address, src/storage/table.cc:37 (host pointer, NULL
 * for an HBM-only table) and its device-visible counterpart.                 */
void *gearb_table_host_ptr(const gearb_table *t);
void *gearb_table_device_ptr(const gearb_table *t);
/* Copy the host image to the HBM copy (allocating it on first use): the
 * HBM-resident table the reference only declares
 * (CudaTrajectoryStorageHandler, include/storage/handler.h:89-102).          */
int gearb_table_upload(gearb_table *t, void *stream);
/* One byte range of the host copy into the device copy (after gearb_table_upload): what a
 * trainer does with a trajectory that a simulator process has finished writing into the
 * shared-memory side of the table (the reference's trainer reads that memory in place,
 * src/memory/shared_memory.cc:59-61; a device-resident table has to be told).             */
int gearb_table_upload_range(gearb_table *t, int64_t offset, int64_t bytes, void *stream);
/* Byte-range write/read against every resident copy (Uint8Span::copy on a
 * handler view, include/common/span.h:73-79).                                */
int gearb_table_write(gearb_table *t, int64_t offset, const void *src, int64_t bytes,
                      void *stream);
int gearb_table_read(const gearb_table *t, int64_t offset, void *dst, int64_t bytes);

/* ======================= storage handler ================================ */
/* get_cpu_handler, src/storage/pybind.cc:157-164 /
 * CpuTrajectoryStorageHandler ctor, src/storage/handler.cc:42-49.  The handler
 * borrows the table (non-owning), as in the reference.                       */
int gearb_handler_create(gearb_table *t, int64_t global_capacity, int64_t w_lb, int64_t w_hb,
                         int64_t r_lb, int64_t r_hb, gearb_handler **out);
int gearb_handler_destroy(gearb_handler *h);
/* CpuTrajectoryStorageHandler::set, src/storage/handler.cc:51-60. */
int gearb_handler_set(gearb_handler *h, const int64_t *cids, int n, const int32_t *offsets,
                      const int64_t *lengths, const int32_t *pads);
/* CpuTrajectoryStorageHandler::sub, src/storage/handler.cc:78-131: host-side
 * offset arithmetic into three caller arrays; *slot_bytes = length*row.      */
int gearb_handler_sub(const gearb_handler *h, const int64_t *idx, const int64_t *ts,
                      const int64_t *len, int64_t n, int column, int64_t *src_off,
                      int64_t *dst_off, int64_t *copy_len, int64_t *slot_bytes);
/* CpuTrajectoryStorageHandler::fused_subcopy, src/storage/handler.cc:133-154 +
 * launch_fused_subcopy_collect, include/kernel_launchers.h:30-41: idx/ts/len
 * are int64 device arrays, dst is the caller's [n, length, *shape] device
 * buffer.  Bytes outside the clipped segment are left untouched (the
 * reference's loader pre-zeroes dst).                                        */
int gearb_handler_subcopy(gearb_handler *h, const int64_t *idx, const int64_t *ts,
                          const int64_t *len, int64_t n, int column, void *dst,
                          int32_t *status, void *stream);
/* All subscribed columns of a batch in ONE launch (replaces the loader's
 * per-column Python loop, gear/loader/offline_loader.py:178-203).
 * zero_fill != 0 also writes the padding of every slot, so dst may be
 * uninitialised memory.                                                      */
int gearb_handler_gather(gearb_handler *h, const int32_t *columns, int ncols,
                         const int64_t *idx, const int64_t *ts, const int64_t *len, int64_t n,
                         void *const *dst, int zero_fill, int32_t *status, void *stream);
/* CpuTrajectoryStorageHandler::view / raw, src/storage/handler.cc:223-241. */
int gearb_handler_view(const gearb_handler *h, int64_t index, int column, void **host_ptr,
                       int64_t *bytes);

/* launch_vary_stride_copy_collect / launch_fix_stride_copy_collect,
 * include/kernel_launchers.h:17-28 (libgear.core.vcopy / copy): generic
 * offset-list gathers with arbitrary byte alignment.                         */
int gearb_vcopy(const void *src, void *dst, const int64_t *src_off, const int64_t *dst_off,
                const int64_t *lengths, int64_t n, int64_t max_length, void *stream);
int gearb_copy(const void *src, void *dst, const int64_t *src_off, const int64_t *dst_off,
               int64_t n, int64_t length, void *stream);

/* ======================= index set ====================================== */
/* Indexset / StatusTableShard, include/index/set.h:35-69,191-251: one block
 * holding int64 timesteps then float32 weights at a 128-byte aligned offset. */
int gearb_indexset_create(int64_t global_capacity, int64_t local_capacity, int64_t index_offset,
                          int shared, int shm_key, int create, gearb_indexset **out);
int gearb_indexset_destroy(gearb_indexset *s);
int64_t *gearb_indexset_timesteps(const gearb_indexset *s);
float *gearb_indexset_weights(const gearb_indexset *s);

/* ======================= priority sampling ============================== */
/* Two-level cumulative table over n float32 priorities: cdf[n] (partition-
 * local inclusive float32 sums in a fixed order) and l1[nparts+1] (float64
 * exclusive partition offsets; l1[nparts] is the total).  Replaces
 * launch_prefix_sum and launch_sum, include/kernel_launchers.h:13-15
 * (src/cuda/one_dim_prefix_sum.cu, src/cuda/one_dim_sum.cu).                 */
int64_t gearb_scan_scratch_bytes(int64_t n);
int gearb_scan(const float *priorities, int64_t n, float *cdf, double *l1, void *scratch,
               int64_t scratch_bytes, int32_t *status, void *stream);
/* gearb_scan without any allocation by anyone: the scratch is an array inside the
 * library image (262,400 bytes of device memory on every GPU that loads the library,
 * held until the process exits), enough for n <= gearb_scan_static_max_n() =
 * 268,435,456 priorities; a larger n is refused with GEARB_ERR_UNSUPPORTED.
 * No counterpart in the reference -- it is for callers that must not, or cannot,
 * allocate device memory when they need a scan: code on a latency-critical path, where
 * cudaMalloc would stall every stream of the device; a process whose device memory has
 * all been handed to another allocator (a framework's caching pool), where a late
 * cudaMalloc can simply fail; a plain C caller that does not want to own and size a
 * scratch buffer.  Inputs and outputs are still the caller's.  Results are identical to
 * gearb_scan's.  The first call on a device looks up the array's address on that
 * device (a host-side query, with that device current); make that first call before
 * starting any stream capture.  All calls on a device share the one array: calls whose
 * kernels overlap on the GPU (two streams, two threads) race and give wrong tables --
 * serialise them, or use gearb_scan with separate scratch.                          */
int gearb_scan_static(const float *priorities, int64_t n, float *cdf, double *l1, int32_t *status,
                      void *stream);
int64_t gearb_scan_static_max_n(void);
/* Batched search on caller-supplied float64 variates (stands where
 * torch.multinomial is called, gear/sampler/global_sampler.py:170).
 * flags: GEARB_SEARCH_SCALE -> variates are U[0,1) and are multiplied by the
 * total on the device; otherwise they are U[0,total).                        */
#define GEARB_SEARCH_SCALE 1
#define GEARB_SEARCH_AFFINE 2 /* internal to gearb_sampler_sample_gather_affine */
int gearb_search(const float *cdf, const double *l1, int64_t n, const double *variates,
                 int64_t b, int flags, int64_t *out_index, int32_t *status, void *stream);
/* Uniform draw floor(u*n) on U[0,1) variates (stands where torch.randint is
 * called, gear/sampler/global_sampler.py:121-129).                           */
int gearb_sample_uniform(int64_t n, const double *u01, int64_t b, int64_t *out_index,
                         void *stream);
/* Flat step index -> (trajectory, timestep, length) request triple;
 * lengths == NULL means every trajectory has trajectory_length steps.        */
int gearb_decode(const int64_t *flat, int64_t b, int64_t trajectory_length,
                 const int64_t *lengths, int64_t index_offset, int64_t *idx, int64_t *ts,
                 int64_t *len, void *stream);

/* Sampler object: owns cdf, l1, scratch and a status word on the current
 * device, so that repeated scans need no allocation and no clearing.  All calls on one sampler
 * are expected on one stream.  After any of the three whole-table scans of a table of more than
 * 1024 partitions, the launch that writes l1 is issued lazily -- behind the next scan, beside
 * which it runs, or in front of the first call that needs l1 (see gearb_sampler_scan_totals);
 * the first gearb_sampler_sample_gather behind a scan does not need it.                      */
int gearb_sampler_create(int64_t n, gearb_sampler **out);
int gearb_sampler_destroy(gearb_sampler *s);
int gearb_sampler_scan(gearb_sampler *s, const float *priorities, void *stream);
/* The same scan without storing the level-2 table: only the partition offsets (l1) and the
 * total are produced, so the scan reads 4 bytes per priority and writes next to nothing.
 * gearb_sampler_sample_gather then rebuilds the one partition each request falls into from
 * `priorities` (16 KiB per request, the scan's own addition tree), with the same result bit
 * for bit.  `priorities` must stay unchanged (except through gearb_sampler_update) until the
 * last such call.  gearb_sampler_search and gearb_sampler_pull need the stored table and
 * return GEARB_ERR_STATE until the next gearb_sampler_scan.
 * For a table of more than 1024 partitions the call leaves l1 owing: the first
 * gearb_sampler_sample_gather behind it finds its partitions through sums the scan left, and
 * the launch that writes l1 is issued behind the NEXT gearb_sampler_scan_totals (beside which it
 * runs) or in front of the next call of any other kind on this sampler -- gearb_sampler_result
 * and gearb_sampler_buffers included, so a caller never sees an incomplete l1.  All calls on one
 * sampler are expected on one stream.                                                      */
int gearb_sampler_scan_totals(gearb_sampler *s, const float *priorities, void *stream);
/* gearb_sampler_scan for one of two samplers that are used in turn: the launch may start while
 * the launch before it in the stream is still finishing, which is only correct when that launch
 * does not read THIS sampler's tables (it reads the other one's).  It still completes after it.
 * Which launches may overlap: gearb_sampler_scan_totals and this call may begin while the launch
 * directly before them in the stream (a sampling or pull launch, a level-1 launch) is still
 * running; they never run beside an earlier scan of the same sampler, and a table of at most
 * 1024 partitions (4,194,304 priorities) is always scanned strictly after everything before it.  */
int gearb_sampler_scan_alternate(gearb_sampler *s, const float *priorities, void *stream);
/* The two launches of a scan, separately, for callers that want to put something between
 * them (an event, work of their own): first the pass over the priorities that leaves one
 * aggregate per partition (store != 0: and the level-2 table), then the small launch that
 * turns the aggregates into l1.  Together they equal gearb_sampler_scan (store != 0) or
 * gearb_sampler_scan_totals (store == 0).                                                */
int gearb_sampler_scan_partitions(gearb_sampler *s, const float *priorities, int store, void *stream);
int gearb_sampler_scan_level1(gearb_sampler *s, void *stream);
/* Every scan of a sampler also leaves the eight 512-value block totals of each partition, from
 * which a sampling launch on a table without stored level-2 entries rebuilds only the block a
 * request falls into.  There are two such buffers -- and two level-1 tables -- and a scan writes
 * the slot the previous scan did not (so that a scan never overwrites what a launch still
 * running -- on this GPU, or on a peer in the pull mode -- is reading).  select_slot fixes the
 * slot (0 or 1) of the NEXT scan, for ranks that must agree on it without talking (pull mode:
 * slot = epoch & 1) or for callers that want fixed addresses (then a scan waits for everything
 * before it in the stream); block_totals returns both buffers and the slot the last scan wrote. */
int gearb_sampler_select_slot(gearb_sampler *s, int slot);
int gearb_sampler_block_totals(const gearb_sampler *s, float **slot0, float **slot1, int *current);
/* The level-1 table is kept twice in the same way (gearb_sampler_buffers returns the one of
 * the last scan): the addresses of both, for peers that map them.                          */
int gearb_sampler_level1_buffers(const gearb_sampler *s, double **slot0, double **slot1);
/* Scan, then draw, as one call: the prefix sum and the torch.multinomial call behind it
 * (gear/sampler/global_sampler.py:154-176) for a table that changes before every draw.  Tables of
 * up to 1024 partitions whose CTAs fit on the device together take ONE cooperative launch (the
 * chain is a few memory round trips long; a second launch would double it); larger ones take the
 * scan's and the search's launches.  Tables, status words and indices are those of
 * gearb_sampler_scan followed by gearb_sampler_search, bit for bit.                          */
int gearb_sampler_scan_search(gearb_sampler *s, const float *priorities, const double *variates, int64_t b,
                              int flags, int64_t *out_index, void *stream);
/* Incremental update after a gearb_sampler_scan of the same array: priorities[idx[i]] =
 * values[i] for i < m (idx, values: device arrays), then only the partitions that were touched
 * are rescanned and the partition offsets rebuilt.  The table afterwards is bit-identical to a
 * full scan of the updated priorities.  Host counterparts in the reference: Indexset::set_weight,
 * include/index/set.h:245-247; WeightUpdateRequestArray, src/index/request.cc:41-75.         */
int gearb_sampler_update(gearb_sampler *s, float *priorities, const int64_t *idx, const float *values,
                         int64_t m, void *stream);
int gearb_sampler_search(gearb_sampler *s, const double *variates, int64_t b, int flags,
                         int64_t *out_index, void *stream);
/* Prioritized sample + gather of a whole batch in ONE launch: search each
 * variate, decode the flat step index i to (trajectory i / T, timestep i % T,
 * length lengths[trajectory] or T), and gather every listed column of the
 * handler's table -- the loader's fused_iterate (gear/loader/offline_loader.py:155-204)
 * without its host round trips.  out_* may each be NULL; out_idx gets
 * trajectory + index_offset.                                                 */
int gearb_sampler_sample_gather(gearb_sampler *s, gearb_handler *h, const double *variates,
                                int64_t b, int flags, const int64_t *lengths, int64_t index_offset,
                                const int32_t *columns, int ncols, void *const *dst, int zero_fill,
                                int64_t *out_flat, int64_t *out_idx, int64_t *out_ts,
                                int64_t *out_len, void *stream);
/* The same for one shard of a sharded table: a variate u of the GLOBAL draw becomes
 * u * mul - sub before the search (mul = total priority of all shards, sub = total of the
 * shards before this one), clamped into this shard's range.  Stands where an owner answers
 * the requests of its peers, CpuTrajectoryStorageHandler::subsend, src/storage/handler.cc:160-193.
 * flat_offset is added to out_flat (the shard's first global step id).  The b requests are
 * positions [slot_lo, slot_lo + b) of a global batch.  slot_mod > 1: the batch is dealt
 * round-robin to slot_mod requesters; the request at position q lands in slot
 * slot_base[q % slot_mod] + q / slot_mod of dst and out_*, which groups an owner's answers by
 * requester.  slot_mod == -1: the batch is cut into contiguous slices; positions
 * slot_base[0] <= q < slot_base[1] (the owner's own slice) land in slot q - slot_base[0], the
 * others in slot slot_base[2] + i, so that one buffer holds the owner's finished slice followed
 * by what it sends away.  slot_mod 0 or 1: request i lands in slot i.                     */
int gearb_sampler_sample_gather_affine(gearb_sampler *s, gearb_handler *h, const double *variates,
                                       int64_t b, double mul, double sub, const int64_t *lengths,
                                       int64_t index_offset, const int32_t *columns, int ncols,
                                       void *const *dst, int zero_fill, int64_t *out_flat,
                                       int64_t *out_idx, int64_t *out_ts, int64_t *out_len,
                                       int64_t flat_offset, int slot_mod, int64_t slot_lo,
                                       const int64_t *slot_base, void *stream);
int gearb_sampler_buffers(const gearb_sampler *s, float **cdf, double **l1, int32_t **status);
/* Synchronises `stream`, then returns total and the status words.  When GEARB_ST_SCAN_ABORTED is
 * set in them the outputs are still filled in and the call returns GEARB_ERR_TIMEOUT.       */
int gearb_sampler_result(gearb_sampler *s, void *stream, double *total, int32_t *status);
/* Zeroes the sampler's status words on `stream` (they accumulate otherwise).               */
int gearb_sampler_clear_status(gearb_sampler *s, void *stream);

/* ======================= communication ================================== */
/* create_nccl_id, src/nccl_comm.cc:4-10: 128 bytes to hand to every rank.       */
int gearb_comm_unique_id(char *id128);
/* NcclCommunicator::NcclCommunicator, src/nccl_comm.cc:12-17 (ncclCommInitRank on
 * the current device); CpuTrajectoryStorageHandler::connect, handler.cc:156-158. */
int gearb_comm_create(int rank, int world, const char *id128, gearb_comm **out);
int gearb_comm_destroy(gearb_comm *c);
/* get_rank / get_size / get_device, src/nccl_comm.cc:23-31. */
int gearb_comm_info(const gearb_comm *c, int *rank, int *world, int *device);
/* NcclCommunicator::send / recv, src/nccl_comm.cc:33-47, counted in bytes. */
int gearb_comm_send(gearb_comm *c, const void *buf, int64_t bytes, int peer, void *stream);
int gearb_comm_recv(gearb_comm *c, void *buf, int64_t bytes, int peer, void *stream);
/* NcclCommunicator::allreduce (ncclSum, in place), src/nccl_comm.cc:49-55. */
#define GEARB_DT_F32 0
#define GEARB_DT_F64 1
#define GEARB_DT_I64 2
#define GEARB_DT_F16 3
int gearb_comm_allreduce_sum(gearb_comm *c, void *buf, int64_t count, int dtype, void *stream);
int gearb_comm_allgather(gearb_comm *c, const void *send, void *recv, int64_t bytes_per_rank,
                         void *stream);
/* The exchange the reference declares and leaves empty (group_exchange,
 * src/nccl_comm.cc:83-86), standing in for the per-segment ncclSend / ncclRecv
 * loops of subsend / subrecv (src/storage/handler.cc:178-191,208-220): for each of
 * nbuf buffer pairs b and each peer p, send_bytes[b*W+p] bytes at send[b] +
 * send_off[b*W+p] go to p and recv_bytes[b*W+p] bytes from p land at recv[b] +
 * recv_off[b*W+p], all in one NCCL group.  The block a rank addresses to itself is a
 * device copy.                                                                  */
int gearb_comm_alltoallv(gearb_comm *c, int nbuf, const void *const *send, const int64_t *send_off,
                         const int64_t *send_bytes, void *const *recv, const int64_t *recv_off,
                         const int64_t *recv_bytes, void *stream);

/* ---- sharded table read in place over NVLink ------------------------------
 * Between GPUs of one box the reference moves every segment with its own ncclSend /
 * ncclRecv pair (subsend / subrecv, src/storage/handler.cc:160-222).  Here a shard's
 * table and cumulative-priority tables can instead be mapped into the peers' address
 * space, and the REQUESTER searches and gathers from the owner's memory with ordinary
 * and bulk loads: no send buffer, no exchange step.                           */
#define GEARB_IPC_HANDLE_BYTES 64
/* Handle of a device allocation of this process (table, cdf, l1 as returned by
 * gearb_table_device_ptr / gearb_sampler_buffers) to pass to the other ranks.   */
int gearb_ipc_export(const void *device_ptr, void *handle64);
/* Map another rank's allocation; the pointer is valid on the current device.    */
int gearb_ipc_open(const void *handle64, void **device_ptr);
int gearb_ipc_close(void *device_ptr);
/* One rank's slice of a global batch, pulled from `world` equal shards: request g
 * scales its variate in [0,1) by the sum of totals[] (float64[world] in device memory,
 * each shard's total priority, e.g. from gearb_comm_allgather), finds the owning
 * shard j by the in-order prefix of totals[], searches cdf[j] / l1[j] with the
 * remainder and gathers the listed columns from table[j] into dst.  Every shard has
 * the layout of `h`'s table and `s`'s number of priorities; entry `self` of the
 * pointer arrays is memory of this GPU (-1: none is).  ring != 0 streams large requests
 * from other GPUs through rings of bulk copies in shared memory (faster over NVLink);
 * requests of shard `self` and ring == 0 use plain 16-byte loads.  out_flat gets the global step id
 * j * n + i, out_idx the global trajectory j * capacity + i / T.  The caller orders
 * this launch after all shards' scans and the next scan after all peers' pulls
 * (a collective on the same stream does both).                                  */
int gearb_sampler_pull(gearb_sampler *s, gearb_handler *h, int world, int self, const double *totals,
                       const void *const *cdf, const void *const *l1, const void *const *table,
                       const double *variates, int64_t b, const int32_t *columns, int ncols,
                       void *const *dst, int zero_fill, int ring, int64_t *out_flat, int64_t *out_idx,
                       int64_t *out_ts, void *stream);

/* The all-gather of the shard totals without a collective: every rank writes its total
 * straight into every rank's MAILBOX (a zero-initialised device allocation of
 * GEARB_MAILBOX_BYTES per rank, e.g. from gearb_device_alloc, exported to the peers with
 * gearb_ipc_export) followed by the step's epoch; the pull launch waits, with a limit, until
 * all `world` epoch words of its own mailbox have reached the epoch (GEARB_ST_SCAN_ABORTED if
 * one never does).  Epochs count steps from 1; slot epoch & 1 of the mailbox is used, so a
 * rank may be one step ahead of its peers but not two -- which the waiting itself ensures.
 * No counterpart in the reference (its totals never leave rank 0, gear/sampler/global_sampler.py:105-152). */
#define GEARB_MAILBOX_BYTES (2 * GEARB_MAX_SHARDS * 16)
int gearb_device_alloc(int64_t bytes, void **ptr); /* cudaMalloc, zeroed */
int gearb_device_free(void *ptr);
int gearb_sampler_publish_total(gearb_sampler *s, int world, int rank, void *const *mailboxes, uint64_t epoch,
                                void *stream);
/* A mailbox may also carry copies of the peers' level-1 tables, so that a pull launch searches
 * level 1 in its own GPU's memory instead of the owner's: gearb_mailbox_bytes(n) is the size of
 * such a mailbox for shards of n priorities (the header above plus two slots of GEARB_MAX_SHARDS
 * copies), gearb_mailbox_l1_offset(n, epoch, shard) the byte offset of shard's copy for that
 * epoch.  gearb_sampler_publish with copy_l1 != 0 writes this rank's level 1 into every other
 * rank's mailbox before the total and the epoch.                                          */
int64_t gearb_mailbox_bytes(int64_t n);
int64_t gearb_mailbox_l1_offset(int64_t n, uint64_t epoch, int shard);
/* With copy_l1 a sampler scanned by gearb_sampler_scan_totals also sends its block totals (32 bytes
 * per partition): gearb_mailbox_blk_offset is where shard's copy for that epoch lies, to be passed
 * as that shard's `blk` to gearb_sampler_pull_ex.  gearb_mailbox_bytes covers both kinds.      */
int64_t gearb_mailbox_blk_offset(int64_t n, uint64_t epoch, int shard);
int gearb_sampler_publish(gearb_sampler *s, int world, int rank, void *const *mailboxes, uint64_t epoch,
                          int copy_l1, void *stream);
/* gearb_sampler_scan_totals followed by gearb_sampler_publish (without the level-1 copy) as one
 * call: for tables of more than 1024 partitions the launch that builds level 1 writes the total
 * and the epoch into the mailboxes at its end, which saves the publish launch of every step.  */
int gearb_sampler_scan_totals_publish(gearb_sampler *s, const float *priorities, int world, int rank,
                                      void *const *mailboxes, uint64_t epoch, void *stream);
/* The general form of gearb_sampler_pull / gearb_sampler_pull_mailbox.  Per shard either its
 * stored level-2 table (cdf) or, with cdf == NULL, its priorities and block totals (prio, blk:
 * the slot of the step, see gearb_sampler_select_slot) -- then the shards may have been scanned
 * with gearb_sampler_scan_totals, which reads half as much.  l1[j] may point at a copy of shard
 * j's level 1 in this GPU's memory (a mailbox).  Request g of the launch uses variate
 * variates[g * variate_stride].  Either totals or mailbox + epoch.                          */
typedef struct gearb_pull_args {
  int world, self;
  const double *totals;
  const void *mailbox;
  uint64_t epoch;
  const void *const *cdf;
  const void *const *prio;
  const void *const *blk;
  const void *const *l1;
  const void *const *table;
  const double *variates;
  int64_t b;
  int64_t variate_stride;
  const int32_t *columns;
  int ncols;
  void *const *dst;
  int zero_fill;
  int ring;
  int64_t *out_flat, *out_idx, *out_ts;
} gearb_pull_args;
int gearb_sampler_pull_ex(gearb_sampler *s, gearb_handler *h, const gearb_pull_args *args, void *stream);
/* gearb_sampler_pull with the totals taken from this rank's mailbox at `epoch`. */
int gearb_sampler_pull_mailbox(gearb_sampler *s, gearb_handler *h, int world, int self, const void *mailbox,
                               uint64_t epoch, const void *const *cdf, const void *const *l1,
                               const void *const *table, const double *variates, int64_t b,
                               const int32_t *columns, int ncols, void *const *dst, int zero_fill, int ring,
                               int64_t *out_flat, int64_t *out_idx, int64_t *out_ts, void *stream);

/* ======================= online ingestion =============================== */
/* The hand-off between simulator processes that fill trajectories and the trainer that samples
 * them: SharedMemoryIndexServer / SharedMemoryIndexClient (src/index/server.cc, src/index/client.cc),
 * one 64-byte status slot per simulator in a System-V segment (include/index/sim_status.h:7-17)
 * and a FIFO of free trajectory indices (include/circular_buffer.h).  Host code only; what a scan
 * reports goes to the device through gearb_sampler_update.  Every wait takes a limit in
 * milliseconds and comes back with GEARB_ERR_TIMEOUT when it runs out.                      */
typedef struct gearb_ingest_server gearb_ingest_server;
typedef struct gearb_ingest_client gearb_ingest_client;
/* SharedMemoryIndexServer::SharedMemoryIndexServer + connect, server.cc:49-110. */
int gearb_ingest_server_create(int shm_key, int num_clients, int64_t index_offset, int64_t capacity,
                               gearb_ingest_server **out);
int gearb_ingest_server_destroy(gearb_ingest_server *s);
/* SharedMemoryIndexServer::scan, server.cc:115-170.  infer_*: room for num_clients entries,
 * upd_*: room for 2 * num_clients; an index appears once among the updates.               */
int gearb_ingest_server_scan(gearb_ingest_server *s, int32_t *infer_src, int64_t *infer_idx, int64_t *infer_ts,
                             int64_t infer_cap, int64_t *n_infer, int64_t *upd_idx, int64_t *upd_ts, float *upd_w,
                             int64_t upd_cap, int64_t *n_upd);
/* SharedMemoryIndexServer::update / callback, server.cc:172-188. */
int gearb_ingest_server_update(gearb_ingest_server *s, const int64_t *upd_idx, const int64_t *upd_ts,
                               const float *upd_w, int64_t n);
int gearb_ingest_server_callback(gearb_ingest_server *s, const int32_t *srcs, int64_t n);
/* get_weights / get_timesteps, server.cc:190-192; free entries of the FIFO. */
float *gearb_ingest_server_weights(gearb_ingest_server *s);
int64_t *gearb_ingest_server_timesteps(gearb_ingest_server *s);
int64_t gearb_ingest_server_free_count(const gearb_ingest_server *s);
/* get_state / set_state, server.cc:196-246, as one byte image; get with buf == NULL returns its size. */
int64_t gearb_ingest_server_get_state(const gearb_ingest_server *s, void *buf, int64_t cap);
int gearb_ingest_server_set_state(gearb_ingest_server *s, const void *buf, int64_t bytes);
/* SharedMemoryIndexClient, src/index/client.cc:9-105.  create attaches the server's segment
 * (GEARB_ERR_STATE while it does not exist).                                               */
int gearb_ingest_client_create(int shm_key, int client_rank, int num_clients, gearb_ingest_client **out);
int gearb_ingest_client_destroy(gearb_ingest_client *c);
int gearb_ingest_client_acquire(gearb_ingest_client *c, int64_t timeout_ms, int64_t *tindex);
int gearb_ingest_client_wait(gearb_ingest_client *c, int64_t timeout_ms);
int gearb_ingest_client_release(gearb_ingest_client *c);
int64_t gearb_ingest_client_step(gearb_ingest_client *c);
int64_t gearb_ingest_client_writeback(gearb_ingest_client *c, int terminated, int alloc_new, double weight);
int gearb_ingest_client_status(const gearb_ingest_client *c, int64_t *out7, double *weight);

/* ======================= synthetic data ================================= */
/* Device-side Philox4x32-10 fills for benchmark tables that are too large to
 * stage through the host.  kind selects the distribution.                   */
#define GEARB_FILL_U32 0         /* raw 32-bit words                          */
#define GEARB_FILL_F32_NORMAL 1  /* N(0,1) float32 (Box-Muller)               */
#define GEARB_FILL_F32_UNIFORM 2 /* U(a,b) float32                            */
#define GEARB_FILL_F32_LOGNORMAL 3
#define GEARB_FILL_I32_RANGE 4   /* int32 uniform in [a,b)                    */
#define GEARB_FILL_U8 5          /* uniform bytes                             */
#define GEARB_FILL_U01_F64 6     /* U[0,1) float64 from 53 bits               */
int gearb_fill(void *dst, int64_t count, int kind, uint64_t seed, uint64_t stream_id,
               double a, double b, void *stream);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* GEAR_B200_H_ */
