/* CPU oracle for the stick relayout, in plain C.  TEST INFRASTRUCTURE ONLY:
 * it is linked or loaded by the tests, the smoke check and the benchmark's
 * CPU-baseline leg, never by the product path.
 *
 * Restates the element walk the reference's host<->device copy describes to
 * its data-conversion engine: get_device_stride_info
 * (torch_spyre/csrc/spyre_mem.cpp:213-244) emits, per device dim, a size, a
 * source stride and a destination stride; the engine visits every index of
 * that iteration space and moves one element.  Here the same iteration space
 * is derived from a SpyreTensorLayout (device_size / device_strides / dim_map,
 * torch_spyre/csrc/spyre_tensor_impl.cpp:39-74) and the host strides.
 *
 * Parity status: layout metadata pinned by the reference's golden vectors; the
 * byte image itself is pinned by no reference test ("parity unpinned"), it is
 * defined as that layout with zero pad lanes and unchanged element bits.
 *
 * Elements are moved as opaque 2-byte (or 1/4-byte) words.
 */
#include <pthread.h>
#include <stdint.h>
#include <string.h>

#define ORACLE_MAX_DIMS 8

/* For each device dim d: the host stride it advances by.  The innermost
 * device dim mapped to a host dim advances by that host stride; each further
 * device dim of the same host dim (moving outwards) advances by the product
 * of the inner ones' sizes times the host stride. */
static void host_steps(const int64_t *dev_size, const int32_t *dim_map, int ndev,
                       const int64_t *host_strides, int64_t *step) {
  for (int d = ndev - 1; d >= 0; --d) {
    int64_t mult = 1;
    for (int e = ndev - 1; e > d; --e)
      if (dim_map[e] == dim_map[d]) mult *= dev_size[e];
    step[d] = mult * host_strides[dim_map[d]];
  }
}

/* Host index (along dim_map[d]) that device coordinate c[] corresponds to. */
static int in_bounds(const int64_t *dev_size, const int32_t *dim_map, int ndev,
                     const int64_t *host_size, const int64_t *c) {
  for (int d = 0; d < ndev; ++d) {
    int first = 1;
    for (int e = 0; e < d; ++e)
      if (dim_map[e] == dim_map[d]) first = 0;
    if (!first) continue;
    int64_t idx = 0;
    for (int e = d; e < ndev; ++e)
      if (dim_map[e] == dim_map[d]) idx = idx * dev_size[e] + c[e];
    if (idx >= host_size[dim_map[d]]) return 0;
  }
  return 1;
}

typedef struct {
  void *dev, *host;
  int to_device, elem_bytes, ndev;
  const int64_t *host_size, *dev_size, *dev_strides;
  const int32_t *dim_map;
  int64_t step[ORACLE_MAX_DIMS];
  int64_t row_begin, row_end;
} walk_job;

/* Rows = every device coordinate except the innermost one. */
static void *walk_rows(void *arg) {
  const walk_job *job = (const walk_job *)arg;
  void *dev = job->dev, *host = job->host;
  const int to_device = job->to_device, elem_bytes = job->elem_bytes, ndev = job->ndev;
  const int64_t *host_size = job->host_size, *dev_size = job->dev_size;
  const int64_t *dev_strides = job->dev_strides, *step = job->step;
  const int32_t *dim_map = job->dim_map;
  const int last = ndev - 1;
  const int64_t n_last = dev_size[last];
  const int hd_last = dim_map[last];
  for (int64_t r = job->row_begin; r < job->row_end; ++r) {
    int64_t c[ORACLE_MAX_DIMS];
    int64_t rem = r;
    for (int d = last - 1; d >= 0; --d) {
      c[d] = rem % dev_size[d];
      rem /= dev_size[d];
    }
    c[last] = 0;
    int64_t doff = 0, hoff = 0;
    for (int d = 0; d < last; ++d) {
      doff += c[d] * dev_strides[d];
      hoff += c[d] * step[d];
    }
    /* how many innermost positions are inside the host tensor */
    int64_t valid = 0;
    if (in_bounds(dev_size, dim_map, ndev, host_size, c)) {
      int64_t outer_idx = 0;
      for (int e = 0; e < last; ++e)
        if (dim_map[e] == hd_last) outer_idx = outer_idx * dev_size[e] + c[e];
      int64_t left = host_size[hd_last] - outer_idx * n_last;
      valid = left < 0 ? 0 : (left > n_last ? n_last : left);
    }
    char *dp = (char *)dev + doff * elem_bytes;
    char *hp = (char *)host + hoff * elem_bytes;
    const int64_t ds = dev_strides[last] * elem_bytes, hs = step[last] * elem_bytes;
    if (to_device) {
      if (ds == elem_bytes && hs == elem_bytes) {
        memcpy(dp, hp, (size_t)(valid * elem_bytes));
        memset(dp + valid * elem_bytes, 0, (size_t)((n_last - valid) * elem_bytes));
      } else {
        for (int64_t j = 0; j < n_last; ++j) {
          if (j < valid) memcpy(dp + j * ds, hp + j * hs, (size_t)elem_bytes);
          else memset(dp + j * ds, 0, (size_t)elem_bytes);
        }
      }
    } else {
      if (ds == elem_bytes && hs == elem_bytes) memcpy(hp, dp, (size_t)(valid * elem_bytes));
      else
        for (int64_t j = 0; j < valid; ++j) memcpy(hp + j * hs, dp + j * ds, (size_t)elem_bytes);
    }
  }
  return 0;
}

#define ORACLE_MAX_THREADS 256

static void walk(void *dev, void *host, int to_device, int elem_bytes,
                 const int64_t *host_size, const int64_t *host_strides,
                 const int64_t *dev_size, const int64_t *dev_strides,
                 const int32_t *dim_map, int ndev, int nthreads) {
  walk_job jobs[ORACLE_MAX_THREADS];
  pthread_t tid[ORACLE_MAX_THREADS];
  int64_t rows = 1;
  for (int d = 0; d < ndev - 1; ++d) rows *= dev_size[d];
  if (nthreads < 1) nthreads = 1;
  if (nthreads > ORACLE_MAX_THREADS) nthreads = ORACLE_MAX_THREADS;
  if (nthreads > rows) nthreads = rows > 0 ? (int)rows : 1;
  for (int t = 0; t < nthreads; ++t) {
    walk_job *j = &jobs[t];
    j->dev = dev; j->host = host; j->to_device = to_device; j->elem_bytes = elem_bytes;
    j->ndev = ndev; j->host_size = host_size; j->dev_size = dev_size;
    j->dev_strides = dev_strides; j->dim_map = dim_map;
    host_steps(dev_size, dim_map, ndev, host_strides, j->step);
    j->row_begin = rows * t / nthreads;
    j->row_end = rows * (t + 1) / nthreads;
  }
  for (int t = 1; t < nthreads; ++t) pthread_create(&tid[t], 0, walk_rows, &jobs[t]);
  walk_rows(&jobs[0]);
  for (int t = 1; t < nthreads; ++t) pthread_join(tid[t], 0);
}

int oracle_to_sticks(const void *host, void *dev, int elem_bytes,
                     const int64_t *host_size, const int64_t *host_strides, int rank,
                     const int64_t *dev_size, const int64_t *dev_strides,
                     const int32_t *dim_map, int ndev, int nthreads) {
  if (ndev > ORACLE_MAX_DIMS || rank > ORACLE_MAX_DIMS || ndev < 1) return -1;
  walk(dev, (void *)host, 1, elem_bytes, host_size, host_strides, dev_size, dev_strides,
       dim_map, ndev, nthreads);
  return 0;
}

int oracle_from_sticks(const void *dev, void *host, int elem_bytes,
                       const int64_t *host_size, const int64_t *host_strides, int rank,
                       const int64_t *dev_size, const int64_t *dev_strides,
                       const int32_t *dim_map, int ndev, int nthreads) {
  if (ndev > ORACLE_MAX_DIMS || rank > ORACLE_MAX_DIMS || ndev < 1) return -1;
  walk((void *)dev, host, 0, elem_bytes, host_size, host_strides, dev_size, dev_strides,
       dim_map, ndev, nthreads);
  return 0;
}
