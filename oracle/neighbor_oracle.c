/*
 * TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT PATH.
 *
 * Plain-C restatement, on the CPU, of what the reference's CUDA neighbour
 * search computes.  It exists to check the sm_100a kernels bit for bit and is
 * imported only by tests, the smoke check and the CPU-baseline leg of the
 * benchmark.  Nothing under pytorch_cluster_b200/ may call it.
 *
 * What is restated (paths are relative to the reference checkout):
 *   - segment pointers      torch_cluster/knn.py:74-79 (bucketize, right=False)
 *   - segment lookup        csrc/cuda/utils.cuh:11-19
 *   - squared-L2 distance   csrc/cuda/knn_cuda.cu:61-64, radius_cuda.cu:28-31
 *   - cosine distance       csrc/cuda/knn_cuda.cu:9-28, 55-59
 *   - k-best insertion      csrc/cuda/knn_cuda.cu:44-50, 67-77 (strict '>')
 *   - radius scan           csrc/cuda/radius_cuda.cu:26-41 (strict '<', first
 *                           max_num_neighbors hits in ascending x order)
 *   - r*r narrowing         csrc/cuda/radius_cuda.cu:90
 *   - nearest               csrc/cuda/nearest_cuda.cu:9-61 (1024-thread stride and
 *                           tree reduction: their tie order is restated, see below)
 *   - farthest point sampling  csrc/cuda/fps_cuda.cu:9-68
 *
 * Rounding policy.  nvcc contracts `acc += d*d` into one fused multiply-add by
 * default, so the reference CUDA kernels accumulate acc = fma(d, d, acc) in the
 * tensor's scalar type, starting from 0, in ascending feature order.  `fused`
 * = 1 restates exactly that.  `fused` = 0 restates the reference's CPU
 * arithmetic instead (nanoflann L2_Adaptor, csrc/cpu/utils/nanoflann.hpp:383-408):
 * separately rounded multiplies and adds, in groups of four features
 * (d0*d0 + d1*d1 + d2*d2 + d3*d3 added to the running sum) with a sequential
 * tail.  The file must be compiled with -ffp-contract=off so that only the
 * explicit fma()/fmaf() calls fuse.
 *
 * 16-bit inputs (`*_r16`).  The reference instantiates the same kernels for
 * c10::Half (knn_cuda.cu:125, radius_cuda.cu:84-85) and c10::BFloat16 (radius
 * only).  Those types are not part of the reference checkout: they come from its
 * dependency PyTorch (here 2.11.0; torch/headeronly/util/Half.h and BFloat16.h),
 * whose published definition is: every arithmetic operator converts both
 * operands to float, operates in float and narrows the result to the 16-bit type
 * with round-to-nearest-even; comparisons convert to float; double op Half
 * yields double.  The `*_r16` functions restate the kernels under that
 * definition on float arrays holding 16-bit-representable values.  They are
 * pinned on the GPU against the reference's own CUDA kernels compiled for
 * sm_100a (tests/test_gpu_reference_cuda.py) and, on the CPU, by the reference's
 * half-precision known-answer tests.
 *
 * Parity pin: checked in tests/test_oracle.py against the reference's own
 * known-answer tests (test/test_knn.py, test/test_radius.py, README examples)
 * and against outputs of the reference's compiled CPU path (oracle/_ref, and
 * the fixtures under tests/golden that were generated with it).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#if defined(__x86_64__) && defined(__GNUC__)
#define HOT __attribute__((target_clones("fma", "default")))
#else
#define HOT
#endif

/* ptr[i] = number of entries of the sorted batch vector that are < i,
 * i = 0..num_segments (torch.bucketize(arange(B+1), batch), knn.py:77-79). */
void oracle_segment_ptr(const int64_t *batch, int64_t n, int64_t num_segments,
                        int64_t *ptr) {
  int64_t j = 0;
  for (int64_t i = 0; i <= num_segments; i++) {
    while (j < n && batch[j] < i)
      j++;
    ptr[i] = j;
  }
}

/* First i with ptr[i+1] > idx, else num_segments-1 (utils.cuh:11-19). */
static int64_t segment_of(int64_t idx, const int64_t *ptr, int64_t num_segments) {
  for (int64_t i = 0; i < num_segments; i++)
    if (ptr[i + 1] > idx)
      return i;
  return num_segments - 1;
}

#define DEFINE_ORACLE(T, SUFFIX, FMA, SQRT)                                     \
  static inline T sqdist_##SUFFIX(const T *a, const T *b, int64_t dim,         \
                                  int fused) {                                  \
    if (fused) {                                                                \
      T acc = 0;                                                                \
      for (int64_t d = 0; d < dim; d++) {                                       \
        T diff = a[d] - b[d];                                                   \
        acc = FMA(diff, diff, acc);                                             \
      }                                                                         \
      return acc;                                                               \
    }                                                                           \
    /* non-fused: a = query side, b = point side, as nanoflann evaluates */     \
    T result = 0;                                                      \
    int64_t d = 0;                                                              \
    for (; d + 3 < dim; d += 4) {                                               \
      T d0 = a[d] - b[d], d1 = a[d + 1] - b[d + 1];                    \
      T d2 = a[d + 2] - b[d + 2], d3 = a[d + 3] - b[d + 3];            \
      T p0 = d0 * d0, p1 = d1 * d1, p2 = d2 * d2, p3 = d3 * d3;        \
      T s = p0 + p1;                                                   \
      s = s + p2;                                                               \
      s = s + p3;                                                               \
      result = result + s;                                                      \
    }                                                                           \
    for (; d < dim; d++) {                                                      \
      T d0 = a[d] - b[d];                                              \
      T p0 = d0 * d0;                                                  \
      result = result + p0;                                                     \
    }                                                                           \
    return result;                                                              \
  }                                                                             \
                                                                                \
  static inline T cosdist_##SUFFIX(const T *xr, const T *yr, int64_t dim) {    \
    T dot = 0, nx = 0, ny = 0;                                                  \
    for (int64_t d = 0; d < dim; d++)                                           \
      dot = FMA(xr[d], yr[d], dot);                                             \
    for (int64_t d = 0; d < dim; d++)                                           \
      nx = FMA(xr[d], xr[d], nx);                                               \
    for (int64_t d = 0; d < dim; d++)                                           \
      ny = FMA(yr[d], yr[d], ny);                                               \
    T q = dot / (SQRT(nx) * SQRT(ny));                                          \
    return (T)(1. - (double)q);                                                 \
  }                                                                             \
                                                                                \
  /* out_col / out_dist: [m*k], -1 / 1e10 where fewer than k were found.        \
   * Returns the number of valid (non -1) slots. */                             \
  HOT int64_t oracle_knn_##SUFFIX(                                              \
      const T *x, const T *y, const int64_t *ptr_x, const int64_t *ptr_y,       \
      int64_t num_segments, int64_t n, int64_t m, int64_t dim, int64_t k,       \
      int cosine, int fused, int64_t *out_col, T *out_dist) {                   \
    (void)n;                                                                    \
    int64_t valid = 0;                                                          \
    _Pragma("omp parallel for schedule(dynamic, 64) reduction(+ : valid)")      \
    for (int64_t n_y = 0; n_y < m; n_y++) {                                     \
      const int64_t b = segment_of(n_y, ptr_y, num_segments);                   \
      T *best_dist = out_dist + n_y * k;                                        \
      int64_t *best_idx = out_col + n_y * k;                                    \
      for (int64_t e = 0; e < k; e++) {                                         \
        best_dist[e] = (T)1e10;                                                 \
        best_idx[e] = -1;                                                       \
      }                                                                         \
      for (int64_t n_x = ptr_x[b]; n_x < ptr_x[b + 1]; n_x++) {                 \
        T tmp = cosine ? cosdist_##SUFFIX(x + n_x * dim, y + n_y * dim, dim)    \
                       : sqdist_##SUFFIX(x + n_x * dim, y + n_y * dim, dim,     \
                                         fused);                                \
        /* the list is ascending, so "no slot is > tmp" == "last is not" */     \
        if (!(best_dist[k - 1] > tmp))                                          \
          continue;                                                             \
        int64_t e1 = 0;                                                         \
        while (!(best_dist[e1] > tmp))                                          \
          e1++;                                                                 \
        for (int64_t e2 = k - 1; e2 > e1; e2--) {                               \
          best_dist[e2] = best_dist[e2 - 1];                                    \
          best_idx[e2] = best_idx[e2 - 1];                                      \
        }                                                                       \
        best_dist[e1] = tmp;                                                    \
        best_idx[e1] = n_x;                                                     \
      }                                                                         \
      for (int64_t e = 0; e < k; e++)                                           \
        valid += best_idx[e] >= 0;                                              \
    }                                                                           \
    return valid;                                                               \
  }                                                                             \
                                                                                \
  /* Pass 1 (out_col == NULL): counts[n_y] = number of edges kept for n_y.      \
   * Pass 2: out_col[offsets[n_y] + j] = j-th kept x index (ascending).         \
   * Returns the total number of edges. */                                      \
  HOT int64_t oracle_radius_##SUFFIX(                                           \
      const T *x, const T *y, const int64_t *ptr_x, const int64_t *ptr_y,       \
      int64_t num_segments, int64_t n, int64_t m, int64_t dim, double r,        \
      int64_t max_num_neighbors, int ignore_same_index, int fused,              \
      int64_t *counts, const int64_t *offsets, int64_t *out_col) {              \
    (void)n;                                                                    \
    const T r2 = (T)(r * r);                                                    \
    int64_t total = 0;                                                          \
    _Pragma("omp parallel for schedule(dynamic, 64) reduction(+ : total)")      \
    for (int64_t n_y = 0; n_y < m; n_y++) {                                     \
      const int64_t b = segment_of(n_y, ptr_y, num_segments);                   \
      int64_t count = 0;                                                        \
      for (int64_t n_x = ptr_x[b]; n_x < ptr_x[b + 1]; n_x++) {                 \
        if (count >= max_num_neighbors)                                         \
          break;                                                                \
        T dist = fused ? sqdist_##SUFFIX(x + n_x * dim, y + n_y * dim, dim, 1)  \
                       : sqdist_##SUFFIX(y + n_y * dim, x + n_x * dim, dim, 0); \
        if (dist < r2 && !(ignore_same_index && n_y == n_x)) {                  \
          if (out_col)                                                          \
            out_col[offsets[n_y] + count] = n_x;                                \
          count++;                                                              \
        }                                                                       \
      }                                                                         \
      if (counts)                                                               \
        counts[n_y] = count;                                                    \
      total += count;                                                           \
    }                                                                           \
    return total;                                                               \
  }

DEFINE_ORACLE(float, f32, fmaf, sqrtf)
DEFINE_ORACLE(double, f64, fma, sqrt)


/* ---- 16-bit inputs: float arithmetic, every result narrowed to fp16 (kind 1) or bf16 (kind 2) ---- */

static inline float round_f16(float v) { return (float)(_Float16)v; }

static inline float round_bf16(float v) {
  uint32_t u;
  memcpy(&u, &v, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) {
    u = 0x7fc00000u; /* NaN stays NaN */
  } else {
    u += 0x7fffu + ((u >> 16) & 1u); /* round to nearest, ties to even */
    u &= 0xffff0000u;
  }
  memcpy(&v, &u, 4);
  return v;
}

static inline float r16(float v, int kind) { return kind == 1 ? round_f16(v) : round_bf16(v); }

/* `acc += (a - b) * (a - b)` with Half / BFloat16 operands (knn_cuda.cu:61-64) */
static inline float sqdist_r16(const float *a, const float *b, int64_t dim, int kind) {
  float acc = 0;
  for (int64_t d = 0; d < dim; d++) {
    float diff = r16(a[d] - b[d], kind);
    float prod = r16(diff * diff, kind);
    acc = r16(acc + prod, kind);
  }
  return acc;
}

/* knn_cuda.cu:9-28, 55-59 with Half operands; `1. - q` is formed in double and narrowed
 * through float (the 16-bit types construct from float) */
static inline float cosdist_r16(const float *xr, const float *yr, int64_t dim, int kind) {
  float dot = 0, nx = 0, ny = 0;
  for (int64_t d = 0; d < dim; d++)
    dot = r16(dot + r16(xr[d] * yr[d], kind), kind);
  for (int64_t d = 0; d < dim; d++)
    nx = r16(nx + r16(xr[d] * xr[d], kind), kind);
  for (int64_t d = 0; d < dim; d++)
    ny = r16(ny + r16(yr[d] * yr[d], kind), kind);
  nx = r16(sqrtf(nx), kind);
  ny = r16(sqrtf(ny), kind);
  float den = r16(nx * ny, kind);
  float q = r16(dot / den, kind);
  return r16((float)(1. - (double)q), kind);
}

int64_t oracle_knn_r16(const float *x, const float *y, const int64_t *ptr_x, const int64_t *ptr_y,
                       int64_t num_segments, int64_t n, int64_t m, int64_t dim, int64_t k, int cosine,
                       int kind, int64_t *out_col, float *out_dist) {
  (void)n;
  int64_t valid = 0;
  const float init = r16(1e10f, kind); /* `best_dist[e] = 1e10` narrows: +inf for fp16 */
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : valid)
  for (int64_t n_y = 0; n_y < m; n_y++) {
    const int64_t b = segment_of(n_y, ptr_y, num_segments);
    float *best_dist = out_dist + n_y * k;
    int64_t *best_idx = out_col + n_y * k;
    for (int64_t e = 0; e < k; e++) {
      best_dist[e] = init;
      best_idx[e] = -1;
    }
    for (int64_t n_x = ptr_x[b]; n_x < ptr_x[b + 1]; n_x++) {
      float tmp = cosine ? cosdist_r16(x + n_x * dim, y + n_y * dim, dim, kind)
                         : sqdist_r16(x + n_x * dim, y + n_y * dim, dim, kind);
      if (!(best_dist[k - 1] > tmp))
        continue;
      int64_t e1 = 0;
      while (!(best_dist[e1] > tmp))
        e1++;
      for (int64_t e2 = k - 1; e2 > e1; e2--) {
        best_dist[e2] = best_dist[e2 - 1];
        best_idx[e2] = best_idx[e2 - 1];
      }
      best_dist[e1] = tmp;
      best_idx[e1] = n_x;
    }
    for (int64_t e = 0; e < k; e++)
      valid += best_idx[e] >= 0;
  }
  return valid;
}

int64_t oracle_radius_r16(const float *x, const float *y, const int64_t *ptr_x, const int64_t *ptr_y,
                          int64_t num_segments, int64_t n, int64_t m, int64_t dim, double r,
                          int64_t max_num_neighbors, int ignore_same_index, int kind, int64_t *counts,
                          const int64_t *offsets, int64_t *out_col) {
  (void)n;
  const float r2 = r16((float)(r * r), kind); /* radius_cuda.cu:90: double -> float -> 16-bit */
  int64_t total = 0;
#pragma omp parallel for schedule(dynamic, 64) reduction(+ : total)
  for (int64_t n_y = 0; n_y < m; n_y++) {
    const int64_t b = segment_of(n_y, ptr_y, num_segments);
    int64_t count = 0;
    for (int64_t n_x = ptr_x[b]; n_x < ptr_x[b + 1]; n_x++) {
      if (count >= max_num_neighbors)
        break;
      float dist = sqdist_r16(x + n_x * dim, y + n_y * dim, dim, kind);
      if (dist < r2 && !(ignore_same_index && n_y == n_x)) {
        if (out_col)
          out_col[offsets[n_y] + count] = n_x;
        count++;
      }
    }
    if (counts)
      counts[n_y] = count;
    total += count;
  }
  return total;
}


/* ---- nearest and farthest point sampling ------------------------------------------------------
 * Both reference kernels stride THREADS threads over a segment, keep each thread's first strict
 * optimum and then reduce over threads keeping the lower thread on equal values.  Assuming each
 * reduction round reads the values of the round before (the reference's shared-memory updates
 * are not double buffered; values it may mix are equal-distance entries only), the winner among
 * equal optima is the entry with the smallest ((index - segment start) mod THREADS, index).
 * policy: 0 = float with fused multiply-add (nvcc's contraction), 1 = fp16, 2 = bf16 rounding of
 * every operation; the double variants always fuse. */

static inline float sqd_policy_f32(const float *a, const float *b, int64_t dim, int policy) {
  if (policy != 0)
    return sqdist_r16(a, b, dim, policy);
  float acc = 0;
  for (int64_t d = 0; d < dim; d++) {
    float diff = a[d] - b[d];
    acc = fmaf(diff, diff, acc);
  }
  return acc;
}

static inline double sqd_f64(const double *a, const double *b, int64_t dim) {
  double acc = 0;
  for (int64_t d = 0; d < dim; d++) {
    double diff = a[d] - b[d];
    acc = fma(diff, diff, acc);
  }
  return acc;
}

static inline int tie_before(int64_t i, int64_t j, int64_t lo, int64_t threads) {
  int64_t a = (i - lo) % threads, b = (j - lo) % threads;
  return a < b || (a == b && i < j);
}

#define DEFINE_NEAREST_FPS(T, SUFFIX, DIST, INIT_NEAREST, INIT_FPS)                               \
  /* nearest_cuda.cu:9-61: out[n_x] = nearest y of the same segment */                           \
  void oracle_nearest_##SUFFIX(const T *x, const T *y, const int64_t *ptr_x, const int64_t *ptr_y, \
                               int64_t num_segments, int64_t n, int64_t dim, int policy,         \
                               int64_t *out) {                                                   \
    (void)policy;                                                                                \
    _Pragma("omp parallel for schedule(dynamic, 64)")                                            \
    for (int64_t n_x = 0; n_x < n; n_x++) {                                                      \
      int64_t b = 0;                                                                             \
      for (; b < num_segments; b++)                                                              \
        if (n_x >= ptr_x[b] && n_x < ptr_x[b + 1])                                               \
          break;                                                                                 \
      const T init = INIT_NEAREST;                                                               \
      T best = init;                                                                             \
      int64_t best_idx = 0;                                                                      \
      int found = 0;                                                                             \
      for (int64_t n_y = ptr_y[b]; n_y < ptr_y[b + 1]; n_y++) {                                  \
        T dist = DIST(x + n_x * dim, y + n_y * dim, dim, policy);                                \
        if (!(dist < init))                                                                      \
          continue;                                                                              \
        if (!found || dist < best ||                                                             \
            (dist == best && tie_before(n_y, best_idx, ptr_y[b], 1024))) {                       \
          best = dist;                                                                           \
          best_idx = n_y;                                                                        \
          found = 1;                                                                             \
        }                                                                                        \
      }                                                                                          \
      out[n_x] = best_idx;                                                                       \
    }                                                                                            \
  }                                                                                              \
                                                                                                 \
  /* fps_cuda.cu:9-68; start may be NULL (all zero); dist: scratch [n] */                        \
  void oracle_fps_##SUFFIX(const T *src, const int64_t *ptr, const int64_t *out_ptr,             \
                           const int64_t *start, int64_t num_segments, int64_t dim, int policy,  \
                           T *dist, int64_t *out) {                                              \
    (void)policy;                                                                                \
    _Pragma("omp parallel for schedule(dynamic, 1)")                                             \
    for (int64_t b = 0; b < num_segments; b++) {                                                 \
      const int64_t lo = ptr[b], hi = ptr[b + 1];                                                \
      if (hi <= lo || out_ptr[b + 1] <= out_ptr[b])                                              \
        continue;                                                                                \
      for (int64_t p = lo; p < hi; p++)                                                          \
        dist[p] = INIT_FPS;                                                                      \
      out[out_ptr[b]] = lo + (start ? start[b] : 0);                                             \
      for (int64_t m = out_ptr[b] + 1; m < out_ptr[b + 1]; m++) {                                \
        const int64_t old = out[m - 1];                                                          \
        T best = (T)-1;                                                                          \
        int64_t best_idx = 0;                                                                    \
        for (int64_t p = lo; p < hi; p++) {                                                      \
          T dd = DIST(src + old * dim, src + p * dim, dim, policy);                              \
          /* min() of the CUDA math library: a NaN operand is ignored */                         \
          dd = (dist[p] != dist[p]) ? dd : ((dd != dd) ? dist[p] : (dd < dist[p] ? dd : dist[p])); \
          dist[p] = dd;                                                                          \
          if (dd > best || (dd == best && dd > (T)-1 && tie_before(p, best_idx, lo, 256))) {     \
            best = dd;                                                                           \
            best_idx = p;                                                                        \
          }                                                                                      \
        }                                                                                        \
        out[m] = best_idx;                                                                       \
      }                                                                                          \
    }                                                                                            \
  }

#define DIST_F64(a, b, dim, policy) sqd_f64(a, b, dim)
DEFINE_NEAREST_FPS(float, f32, sqd_policy_f32, (policy ? r16(1e38f, policy) : 1e38f),
                   (policy ? r16(5e4f, policy) : 5e4f))
DEFINE_NEAREST_FPS(double, f64, DIST_F64, 1e38, 5e4)
