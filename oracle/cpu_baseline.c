/*
 * cpu_baseline.c -- multi-threaded drivers around the CPU restatement, used only
 * to TIME the CPU path on the host cores (the reported baseline) and by tests
 * that check the threaded drivers against the sequential functions.
 *
 * TEST / BENCHMARK INFRASTRUCTURE ONLY; nothing in the shipped library uses it.
 *
 * The arithmetic is gear_oracle.c's: partitions of the cumulative table are
 * independent, so they are striped over threads and level 1 is summed in order
 * afterwards; gather requests are independent and are striped the same way.
 */
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define GEARO_PART 4096

int gearo_scan(const float *prio, int64_t n, float *cdf, double *l1, double *total);
void gearo_fused_subcopy(const uint8_t *table, uint8_t *dst, const int64_t *idx, const int64_t *ts,
                         const int64_t *len, int64_t n, int64_t traj_stride, int64_t col_accu, int64_t T,
                         int64_t row, int32_t pat_offset, int64_t pat_length, int pad_head, int zero_fill);

typedef struct {
  const float *prio;
  float *cdf;
  double *agg; /* aggregate of every partition */
  int64_t n, p0, p1;
  int bad;
} scan_job;

static void *scan_worker(void *arg) {
  scan_job *j = (scan_job *)arg;
  double l1[2], total;
  for (int64_t p = j->p0; p < j->p1; ++p) {
    const int64_t lo = p * GEARO_PART;
    const int64_t valid = (j->n - lo < GEARO_PART) ? (j->n - lo) : GEARO_PART;
    j->bad |= gearo_scan(j->prio + lo, valid, j->cdf + lo, l1, &total);
    j->agg[p] = l1[1];
  }
  return NULL;
}

/* Same result as gearo_scan, partitions striped over `threads` host threads. */
int gearo_scan_mt(const float *prio, int64_t n, float *cdf, double *l1, double *total, int threads) {
  const int64_t nparts = (n + GEARO_PART - 1) / GEARO_PART;
  if (threads < 1) threads = 1;
  if (threads > nparts) threads = (int)nparts;
  double *agg = (double *)malloc(sizeof(double) * (size_t)nparts);
  scan_job *jobs = (scan_job *)calloc((size_t)threads, sizeof(scan_job));
  pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
  for (int t = 0; t < threads; ++t) {
    jobs[t].prio = prio; jobs[t].cdf = cdf; jobs[t].agg = agg; jobs[t].n = n;
    jobs[t].p0 = nparts * t / threads; jobs[t].p1 = nparts * (t + 1) / threads;
    if (t > 0) pthread_create(&tid[t], NULL, scan_worker, &jobs[t]);
  }
  scan_worker(&jobs[0]);
  int bad = jobs[0].bad;
  for (int t = 1; t < threads; ++t) {
    pthread_join(tid[t], NULL);
    bad |= jobs[t].bad;
  }
  double acc = 0.0;
  l1[0] = 0.0;
  for (int64_t p = 0; p < nparts; ++p) {
    acc = acc + agg[p];
    l1[p + 1] = acc;
  }
  *total = acc;
  free(agg); free(jobs); free(tid);
  return bad;
}

typedef struct {
  const uint8_t *table;
  uint8_t *const *dst;
  const int64_t *idx, *ts, *len;
  int64_t r0, r1, traj_stride, T;
  const int64_t *col_accu, *row, *pat_length;
  const int32_t *pat_offset, *pad_head;
  int ncols;
} gather_job;

static void *gather_worker(void *arg) {
  gather_job *j = (gather_job *)arg;
  const int64_t m = j->r1 - j->r0;
  for (int c = 0; c < j->ncols; ++c) {
    const int64_t slot = j->pat_length[c] * j->row[c];
    gearo_fused_subcopy(j->table, j->dst[c] + j->r0 * slot, j->idx + j->r0, j->ts + j->r0, j->len + j->r0, m,
                        j->traj_stride, j->col_accu[c], j->T, j->row[c], j->pat_offset[c], j->pat_length[c],
                        j->pad_head[c], 1);
  }
  return NULL;
}

/* All listed columns of a batch, requests striped over `threads` host threads. */
void gearo_gather_mt(const uint8_t *table, uint8_t *const *dst, const int64_t *idx, const int64_t *ts,
                     const int64_t *len, int64_t n, int64_t traj_stride, int64_t T, int ncols,
                     const int64_t *col_accu, const int64_t *row, const int32_t *pat_offset,
                     const int64_t *pat_length, const int32_t *pad_head, int threads) {
  if (threads < 1) threads = 1;
  if (threads > n) threads = n > 0 ? (int)n : 1;
  gather_job *jobs = (gather_job *)calloc((size_t)threads, sizeof(gather_job));
  pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
  for (int t = 0; t < threads; ++t) {
    gather_job *j = &jobs[t];
    j->table = table; j->dst = dst; j->idx = idx; j->ts = ts; j->len = len;
    j->r0 = n * t / threads; j->r1 = n * (t + 1) / threads;
    j->traj_stride = traj_stride; j->T = T; j->ncols = ncols;
    j->col_accu = col_accu; j->row = row; j->pat_offset = pat_offset; j->pat_length = pat_length;
    j->pad_head = pad_head;
    if (t > 0) pthread_create(&tid[t], NULL, gather_worker, j);
  }
  gather_worker(&jobs[0]);
  for (int t = 1; t < threads; ++t) pthread_join(tid[t], NULL);
  free(jobs); free(tid);
}

/* ------------------------------------------------------------------------------------------
 * The plain way to draw on a CPU, timed beside the tree port above: a flat running sum of the
 * priorities in float64 (chunks summed by the threads, then offset by the chunks before them)
 * and one upper_bound per variate.  Its indices may differ from the two-level table's by the
 * flips that a different summation order causes; it is a timing baseline, not a checker.
 * cum must hold n doubles.  Returns the total. */
typedef struct {
  const float *prio;
  double *cum;
  int64_t lo, hi;
  double sum, offset;
} cumsum_job;

static void *cumsum_pass1(void *arg) {
  cumsum_job *j = (cumsum_job *)arg;
  double s = 0.0;
  for (int64_t i = j->lo; i < j->hi; ++i) {
    s += (double)j->prio[i];
    j->cum[i] = s;
  }
  j->sum = s;
  return NULL;
}

static void *cumsum_pass2(void *arg) {
  cumsum_job *j = (cumsum_job *)arg;
  const double o = j->offset;
  if (o != 0.0)
    for (int64_t i = j->lo; i < j->hi; ++i) j->cum[i] += o;
  return NULL;
}

double gearo_plain_cumsum_mt(const float *prio, int64_t n, double *cum, int threads) {
  if (threads < 1) threads = 1;
  if (threads > n) threads = n > 0 ? (int)n : 1;
  cumsum_job *jobs = (cumsum_job *)calloc((size_t)threads, sizeof(cumsum_job));
  pthread_t *tid = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)threads);
  for (int pass = 0; pass < 2; ++pass) {
    if (pass == 1) {
      double acc = 0.0;
      for (int t = 0; t < threads; ++t) {
        jobs[t].offset = acc;
        acc += jobs[t].sum;
      }
    }
    for (int t = 0; t < threads; ++t) {
      jobs[t].prio = prio; jobs[t].cum = cum;
      jobs[t].lo = n * t / threads; jobs[t].hi = n * (t + 1) / threads;
      if (t > 0) pthread_create(&tid[t], NULL, pass == 0 ? cumsum_pass1 : cumsum_pass2, &jobs[t]);
    }
    (pass == 0 ? cumsum_pass1 : cumsum_pass2)(&jobs[0]);
    for (int t = 1; t < threads; ++t) pthread_join(tid[t], NULL);
  }
  const double total = n > 0 ? cum[n - 1] : 0.0;
  free(jobs); free(tid);
  return total;
}

/* First index whose running sum exceeds u * total (scale != 0) or u. */
void gearo_plain_upper_bound(const double *cum, int64_t n, const double *u, int64_t b, int scale, int64_t *out) {
  const double total = n > 0 ? cum[n - 1] : 0.0;
  for (int64_t k = 0; k < b; ++k) {
    const double v = scale ? u[k] * total : u[k];
    int64_t lo = 0, hi = n - 1;
    while (lo < hi) {
      const int64_t mid = lo + (hi - lo) / 2;
      if (cum[mid] > v) hi = mid;
      else lo = mid + 1;
    }
    out[k] = lo;
  }
}
