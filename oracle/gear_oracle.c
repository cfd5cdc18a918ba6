/*
 * gear_oracle.c -- CPU restatement of GEAR's replay sample + gather path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the CUDA path is compared
 * against; nothing in the shipped library links, loads or calls it.
 *
 * Every function cites the reference file:line (paths relative to the
 * bigrl-team/gear tree) whose behaviour it restates.  Build with
 *     gcc -O2 -ffp-contract=off -fno-fast-math -fPIC -shared
 * so that every float/double addition below is a single IEEE-754
 * round-to-nearest operation in the written order.
 *
 * Parity pins:
 *   - gather addressing: validated against the reference's own compiled
 *     CpuTrajectoryStorageHandler::sub (oracle/_ref) on randomised requests,
 *     and against the reference's tests/test_copy.py case.
 *   - prioritized / uniform draw: PARITY UNPINNED.  The reference delegates the
 *     arithmetic to torch.multinomial / torch.randint (third-party, torch
 *     1.13.0+cu117 per requirements.txt:1) and its own prefix-sum kernel has no
 *     caller and no test; this file fixes the reduction tree that kernel
 *     sketches (src/cuda/one_dim_prefix_sum.cu:40-49,23-28,192-201) as the
 *     definition both sides implement.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GEARO_PART 4096  /* priorities per partition (level-2 scan unit)   */
#define GEARO_BLOCK 512  /* values per block of 32 groups of 16             */
#define GEARO_BLOCKS 8   /* blocks per partition                            */

/* ------------------------------------------------------------------------- */
/* Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1,2,3",
 * SC'11) -- the published algorithm, written out here so that seeded synthetic
 * tables, priorities and variates are identical on host and device.          */
static inline void philox_round(uint32_t c[4], uint32_t k0, uint32_t k1) {
  const uint64_t p0 = (uint64_t)0xD2511F53u * c[0];
  const uint64_t p1 = (uint64_t)0xCD9E8D57u * c[2];
  const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0;
  const uint32_t n1 = (uint32_t)p1;
  const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1;
  const uint32_t n3 = (uint32_t)p0;
  c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
}

void gearo_philox4x32(uint64_t seed, uint64_t stream, uint64_t counter,
                      uint32_t out[4]) {
  uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32),
                   (uint32_t)stream, (uint32_t)(stream >> 32)};
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) {
    philox_round(c, k0, k1);
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
  memcpy(out, c, sizeof(uint32_t) * 4);
}

/* n raw 32-bit words: word i = lane (i & 3) of block (i >> 2). */
void gearo_philox_u32(uint64_t seed, uint64_t stream, uint64_t first,
                      int64_t n, uint32_t *out) {
  for (int64_t i = 0; i < n; ++i) {
    uint64_t g = first + (uint64_t)i;
    uint32_t b[4];
    gearo_philox4x32(seed, stream, g >> 2, b);
    out[i] = b[g & 3];
  }
}

/* Uniform double in [0,1) from 53 random bits: element i uses block i. */
void gearo_philox_u01(uint64_t seed, uint64_t stream, uint64_t first,
                      int64_t n, double *out) {
  for (int64_t i = 0; i < n; ++i) {
    uint32_t b[4];
    gearo_philox4x32(seed, stream, first + (uint64_t)i, b);
    uint64_t bits = (((uint64_t)b[0]) << 21) ^ (uint64_t)(b[1] >> 11);
    out[i] = (double)(bits & ((1ull << 53) - 1)) * (1.0 / 9007199254740992.0);
  }
}

/* ------------------------------------------------------------------------- */
/* Table layout.  Restates TrajectoryTable's constructor
 * (src/storage/table.cc:8-25): a column's row is `row_bytes[c]` bytes
 * (ColumnSpec::size, src/storage/specs.cc:10-14); accu[c] is the exclusive
 * prefix of the row sizes; one trajectory occupies sum(row_bytes) * T bytes and
 * inside it column c starts at accu[c] * T.  64-bit throughout (the reference
 * seeds std::accumulate with an int, table.cc:14-16).                        */
int64_t gearo_table_layout(const int64_t *row_bytes, int ncols, int64_t T,
                           int64_t *accu /* ncols+1 */) {
  int64_t sum = 0;
  for (int c = 0; c < ncols; ++c) {
    accu[c] = sum;
    sum += row_bytes[c];
  }
  accu[ncols] = sum;
  return sum * T; /* trajectory stride in bytes */
}

/* Addressing of one subscribed column.  Restates
 * CpuTrajectoryStorageHandler::sub (src/storage/handler.cc:78-131) line by
 * line in meaning: clip [ts+offset, ts+offset+length) to [0, len), convert to
 * bytes, place at the head or the tail of the request's slot.
 * pad_head != 0 corresponds to PadOption::kHead; tail and inactive place the
 * data at the start of the slot (handler.cc:117-120).                        */
int64_t gearo_sub(const int64_t *idx, const int64_t *ts, const int64_t *len,
                  int64_t n, int64_t traj_stride, int64_t col_accu, int64_t T,
                  int64_t row, int32_t pat_offset, int64_t pat_length,
                  int pad_head, int64_t *src_off, int64_t *dst_off,
                  int64_t *copy_len) {
  const int64_t column_ofst = col_accu * T;
  const int64_t slot = pat_length * row;
  for (int64_t i = 0; i < n; ++i) {
    int64_t base = idx[i] * traj_stride + column_ofst;
    int64_t start = ts[i] + (int64_t)pat_offset;
    if (start < 0) start = 0;
    int64_t end = start + pat_length;
    if (end > len[i]) end = len[i];
    start *= row;
    end *= row;
    int64_t bytes = end - start;
    if (bytes < 0) bytes = 0;
    int64_t d = pad_head ? slot - bytes : 0;
    copy_len[i] = bytes;
    src_off[i] = base + start;
    dst_off[i] = d + slot * i;
  }
  return slot;
}

/* The effect of vary_stride_copy_collect (src/cuda/copy.cu:47-89) for offsets
 * produced by gearo_sub: slice i moves copy_len[i] bytes.  The destination is
 * whatever the caller prepared (the reference's loader passes torch.zeros,
 * gear/loader/offline_loader.py:181-189).                                    */
void gearo_vcopy(const uint8_t *src, uint8_t *dst, int64_t n,
                 const int64_t *src_off, const int64_t *dst_off,
                 const int64_t *copy_len) {
  for (int64_t i = 0; i < n; ++i)
    if (copy_len[i] > 0) memcpy(dst + dst_off[i], src + src_off[i], (size_t)copy_len[i]);
}

/* The fused form: addressing + copy in one pass, i.e. what
 * fused_subcopy_collect (src/cuda/copy.cu:91-134) intends, with the clipped
 * length clamped at zero the way handler.cc:115 does (the kernel itself returns
 * without copying when the byte count is negative, copy.cu:116-117).
 * zero_fill != 0 additionally writes zeros to the unused part of every slot. */
void gearo_fused_subcopy(const uint8_t *table, uint8_t *dst, const int64_t *idx,
                         const int64_t *ts, const int64_t *len, int64_t n,
                         int64_t traj_stride, int64_t col_accu, int64_t T,
                         int64_t row, int32_t pat_offset, int64_t pat_length,
                         int pad_head, int zero_fill) {
  const int64_t slot = pat_length * row;
  for (int64_t i = 0; i < n; ++i) {
    int64_t s, d, b;
    gearo_sub(idx + i, ts + i, len + i, 1, traj_stride, col_accu, T, row,
              pat_offset, pat_length, pad_head, &s, &d, &b);
    d += slot * i; /* gearo_sub saw the request as slot 0 */
    if (zero_fill) {
      uint8_t *slot0 = dst + slot * i;
      if (pad_head) memset(slot0, 0, (size_t)(slot - b));
      else memset(slot0 + b, 0, (size_t)(slot - b));
    }
    if (b > 0) memcpy(dst + d, table + s, (size_t)b);
  }
}

/* ------------------------------------------------------------------------- */
/* Two-level cumulative priority table.
 *
 * Level 2: for each partition of GEARO_PART priorities, a partition-local
 * inclusive float32 scan with this fixed addition tree (the shape sketched by
 * the reference's unfinished kernel: four values per thread added in sequence,
 * src/cuda/one_dim_prefix_sum.cu:40-49; Hillis-Steele shuffle scan over the 32
 * lanes of a warp, :23-28; a second pass over the warp totals, :192-201):
 *
 *   chunk = 4 consecutive values: s0=x0, s1=s0+x1, s2=s1+x2, s3=s2+x3; T=s3
 *   group = 4 consecutive chunks: g0=T0, g1=g0+T1, g2=g1+T2, g3=g2+T3
 *   block = 32 consecutive groups (512 values):
 *           I = Hillis-Steele inclusive scan of g3 over the groups (d=1,2,4,8,16)
 *           E = I of group q-1 (0 for q=0); block total = I of group 31
 *   part  = 8 consecutive blocks: X(0)=0, X(w+1) = X(w) + total(w)
 *   chunk offset O = X(w) + E(q) for the group's first chunk, (X(w) + E(q)) + g(i-1)
 *           for its chunk i = 1..3
 *   value = O + s_j
 *
 * followed by a running maximum over the partition, which removes the one-ulp
 * inversions a tree-shaped float scan can leave between chunks, so that the
 * stored table is non-decreasing and "first entry greater than r" is well
 * defined for any search order.  Entries past n count as zero.
 * One exception keeps "a zero priority repeats its predecessor's entry" exact:
 * inside a chunk that holds for zeros (s_j = s_(j-1)), but a chunk that BEGINS
 * with zeros would give them the chunk's offset O, which can be an ulp above
 * the previous chunk's last value (two roundings of the same sum) -- and an
 * entry of weight zero could then be the first one greater than r.  Entries
 * with s_j = 0 therefore take no part in the maximum (their value counts as
 * 0) and so repeat the running maximum before them.
 *
 * Level 1: l1[0]=0, l1[p+1] = l1[p] + (double)aggregate(p), added in partition order in
 * float64, where aggregate(p) = X(8) is the partition's eight block totals added in sequence
 * (it can differ from the partition's last cdf entry by an ulp; the search pulls a variate
 * that lands on or above the last entry just below it).  total = l1[nparts].
 *
 * The sum of the reference's one_dimension_sum (src/cuda/one_dim_sum.cu:22-74)
 * is folded into this: `total` replaces it, without the atomicAdd whose order
 * is not reproducible (:72-74).                                             */
static void hs_scan32(float v[32]) {
  for (int d = 1; d < 32; d <<= 1) {
    float nv[32];
    for (int l = 0; l < 32; ++l) nv[l] = (l >= d) ? (v[l - d] + v[l]) : v[l];
    memcpy(v, nv, sizeof(nv));
  }
}

static float scan_partition(const float *x, int64_t valid, float *out) {
  /* x: up to GEARO_PART inputs (valid of them real), out: GEARO_PART values.
   * Returns the partition's aggregate: its block totals added in sequence.   */
  float s[GEARO_PART];               /* running sums inside each chunk           */
  float gprev[GEARO_PART / 4];       /* g(i-1) of every chunk (unused for i = 0) */
  float E[GEARO_PART / 16];          /* exclusive offset of every group          */
  float Y[GEARO_BLOCKS];
  for (int w = 0; w < GEARO_BLOCKS; ++w) {
    float I[32];
    for (int q = 0; q < 32; ++q) {
      float g = 0.0f;
      for (int i = 0; i < 4; ++i) {
        const int e = w * GEARO_BLOCK + 16 * q + 4 * i;
        float acc = 0.0f;
        for (int j = 0; j < 4; ++j) {
          const float a = (e + j < valid) ? x[e + j] : 0.0f;
          acc = (j == 0) ? a : acc + a;
          s[e + j] = acc;
        }
        gprev[e / 4] = g;
        g = (i == 0) ? acc : g + acc;
      }
      I[q] = g;
    }
    hs_scan32(I);
    Y[w] = I[31];
    for (int q = 0; q < 32; ++q) E[w * 32 + q] = (q == 0) ? 0.0f : I[q - 1];
  }
  float run = 0.0f, X = 0.0f;
  for (int w = 0; w < GEARO_BLOCKS; ++w) {
    if (w > 0) X = X + Y[w - 1];
    for (int q = 0; q < 32; ++q) {
      const float b = X + E[w * 32 + q];
      for (int i = 0; i < 4; ++i) {
        const int e0 = w * GEARO_BLOCK + 16 * q + 4 * i;
        const float off = (i == 0) ? b : b + gprev[e0 / 4];
        for (int j = 0; j < 4; ++j) {
          /* an entry before which its chunk holds only zeros takes no part in the maximum:
           * it repeats what came before it, bit for bit (see the comment above)           */
          const float v = (s[e0 + j] == 0.0f) ? 0.0f : off + s[e0 + j];
          if (v > run) run = v;
          out[e0 + j] = run;
        }
      }
    }
  }
  return X + Y[GEARO_BLOCKS - 1];
}

/* Returns 0, or 1 when a priority has its sign bit set (negative, or -0.0) or is NaN (the
 * table is then meaningless; the CUDA path raises the same flag).            */
int gearo_scan(const float *prio, int64_t n, float *cdf, double *l1 /* nparts+1 */,
               double *total) {
  const int64_t nparts = (n + GEARO_PART - 1) / GEARO_PART;
  int bad = 0;
  float buf[GEARO_PART];
  double acc = 0.0;
  l1[0] = 0.0;
  for (int64_t p = 0; p < nparts; ++p) {
    const int64_t lo = p * GEARO_PART;
    const int64_t valid = (n - lo < GEARO_PART) ? (n - lo) : GEARO_PART;
    for (int64_t i = 0; i < valid; ++i)
      if (signbit(prio[lo + i]) || isnan(prio[lo + i])) bad = 1;
    const float agg = scan_partition(prio + lo, valid, buf);
    memcpy(cdf + lo, buf, (size_t)valid * sizeof(float));
    acc = acc + (double)agg;
    l1[p + 1] = acc;
  }
  *total = acc;
  return bad;
}

/* Batched search on caller-supplied variates.  For variate u in [0,total):
 *   p  = partition with l1[p] <= u < l1[p+1]
 *   r  = (float)(u - l1[p]), pulled just below the partition's last entry if
 *        rounding put it on or above it
 *   j  = number of entries of partition p that are <= r   (searchsorted right)
 * A zero priority repeats its predecessor's entry and can therefore never be
 * the first entry greater than r ("weight = 0 indicates unselectable",
 * src/index/server.cc:147).  scale != 0 multiplies u by total first (u is then
 * a U[0,1) variate).  near[i], when given, is set when r is within one float32
 * ulp of either boundary of the chosen entry, i.e. when another rounding of
 * the same sums could have picked a neighbour.                               */
void gearo_search(const float *cdf, const double *l1, int64_t n,
                  const double *u, int64_t b, int scale, int64_t *out,
                  uint8_t *near) {
  const int64_t nparts = (n + GEARO_PART - 1) / GEARO_PART;
  const double total = l1[nparts];
  for (int64_t i = 0; i < b; ++i) {
    if (!(total > 0.0)) { /* nothing selectable: defined as the last index */
      out[i] = n - 1;
      if (near) near[i] = 0;
      continue;
    }
    double v = u[i];
    if (scale) v = v * total;
    if (!(v >= 0.0)) v = 0.0;
    if (!(v < total)) v = nextafter(total, 0.0);
    /* upper bound over l1[1..nparts] */
    int64_t lo = 0, hi = nparts;
    while (lo < hi) {
      int64_t mid = (lo + hi) >> 1;
      if (l1[mid + 1] <= v) lo = mid + 1; else hi = mid;
    }
    int64_t p = lo;
    if (p >= nparts) p = nparts - 1;
    const int64_t base = p * GEARO_PART;
    const int64_t valid = (n - base < GEARO_PART) ? (n - base) : GEARO_PART;
    float r = (float)(v - l1[p]);
    const float last = cdf[base + valid - 1];
    if (!(r < last)) r = nextafterf(last, 0.0f);
    int64_t a = 0, z = valid;
    while (a < z) {
      int64_t mid = (a + z) >> 1;
      if (cdf[base + mid] <= r) a = mid + 1; else z = mid;
    }
    if (a >= valid) a = valid - 1;
    out[i] = base + a;
    if (near) {
      const float hi_b = cdf[base + a];
      int flag = nextafterf(r, INFINITY) >= hi_b;
      if (a > 0 && r == cdf[base + a - 1]) flag = 1;
      near[i] = (uint8_t)flag;
    }
  }
}

/* Uniform draw over n items on U[0,1) variates: floor(u*n), clamped.  The
 * reference's UniformSampler draws torch.randint(0, n)
 * (gear/sampler/global_sampler.py:121-129); with the variate supplied by the
 * caller the draw is this one multiplication.                                */
void gearo_uniform(const double *u01, int64_t b, int64_t n, int64_t *out) {
  for (int64_t i = 0; i < b; ++i) {
    double v = u01[i];
    if (!(v >= 0.0)) v = 0.0;
    int64_t k = (int64_t)floor(v * (double)n);
    if (k >= n) k = n - 1;
    out[i] = k;
  }
}

/* Flat step index -> GEAR's request triple (trajectory, timestep, length):
 * idx = i / T, ts = i % T, len = lengths[idx] (or T when lengths is NULL).   */
void gearo_decode(const int64_t *flat, int64_t b, int64_t T,
                  const int64_t *lengths, int64_t index_offset, int64_t *idx,
                  int64_t *ts, int64_t *len) {
  for (int64_t i = 0; i < b; ++i) {
    int64_t t = flat[i] / T;
    idx[i] = t + index_offset;
    ts[i] = flat[i] % T;
    len[i] = lengths ? lengths[t] : T;
  }
}

/* Independent high-precision answer used only to COUNT index flips: a float64
 * running sum over all priorities in index order and searchsorted(right).     */
void gearo_search_f64(const float *prio, int64_t n, const double *u, int64_t b,
                      double scale_total, int64_t *out, double *cdf64_scratch) {
  double acc = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    acc += (double)prio[i];
    cdf64_scratch[i] = acc;
  }
  for (int64_t i = 0; i < b; ++i) {
    double v = u[i];
    if (scale_total > 0.0) v = v * scale_total;
    if (!(v < acc)) v = nextafter(acc, 0.0);
    int64_t lo = 0, hi = n;
    while (lo < hi) {
      int64_t mid = (lo + hi) >> 1;
      if (cdf64_scratch[mid] <= v) lo = mid + 1; else hi = mid;
    }
    out[i] = lo < n ? lo : n - 1;
  }
}

/* ------------------------------------------------------------------------- */
/* Ownership of a global trajectory id under block sharding: rank g / cap
 * (gear/loader/offline_loader.py:131-137).                                   */
void gearo_owner(const int64_t *gidx, int64_t b, int64_t cap_per_rank,
                 int32_t *owner, int64_t *local) {
  for (int64_t i = 0; i < b; ++i) {
    owner[i] = (int32_t)(gidx[i] / cap_per_rank);
    local[i] = gidx[i] % cap_per_rank;
  }
}

/* Peer visiting order of a rank: rotation that starts at (W - rank) % W
 * (gear/loader/offline_loader.py:142-153).                                   */
void gearo_comm_order(int rank, int world, int32_t *order) {
  order[0] = (world - rank) % world;
  for (int i = 1; i < world; ++i) order[i] = (order[i - 1] + 1) % world;
}
