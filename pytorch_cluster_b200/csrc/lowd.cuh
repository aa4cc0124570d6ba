// Brute-force scan machinery for low-dimensional points (1 <= DIM <= 8), shared by the kNN and
// radius kernels.
//
// Work mapping.  A CTA owns a tile of consecutive query rows; each of its 8 warps owns up to QW
// of those queries for the whole scan.  The points of the queries' segment stream through
// shared memory in chunks (cp.async, double buffered, one plane per feature so that every
// lane-strided read is bank-conflict free).  Per step a warp takes 32 * R points — lane l holds
// points l, l + 32, ... in registers — and runs each of its queries (broadcast from shared
// memory) against them.  Distances are accumulated exactly as the reference's CUDA kernels do:
// acc = fma(x_d - y_d, x_d - y_d, acc) over ascending d in the data type
// (csrc/cuda/knn_cuda.cu:61-64, csrc/cuda/radius_cuda.cu:28-31); for fp32 two points are
// processed per instruction with the packed f32x2 forms of sm_100 (same rounding per element).
#pragma once

#include "common.cuh"

namespace b200c {

template <typename T, int DIM>
struct LowD {
  static constexpr int R = sizeof(T) == 4 ? 8 : 4;  // points per lane per step
  static constexpr int STEP = 32 * R;               // points per warp step
  // chunk: about 12 KB per buffer, at most 1024 points, a whole number of steps
  static constexpr int XC_FIT = 12288 / (DIM * (int)sizeof(T));
  static constexpr int XC_RAW = XC_FIT < 1024 ? XC_FIT : 1024;
  static constexpr int XC = (XC_RAW / STEP) > 0 ? (XC_RAW / STEP) * STEP : STEP;
  static constexpr int XP = XC + 4;  // plane stride (elements)
  static constexpr int PLANES_ELEMS = DIM * XP;
  // query record, in elements of T: fp32 keeps (-q_d, -q_d) pairs so a record feeds the packed
  // instructions without moves; the last element is the query's current bound.
  static constexpr int REC_USED = sizeof(T) == 4 ? 2 * DIM + 1 : DIM + 1;
  static constexpr int REC_ALIGN = 16 / (int)sizeof(T);
  static constexpr int REC = (REC_USED + REC_ALIGN - 1) / REC_ALIGN * REC_ALIGN;
};

// Stage `npts` points starting at row `first` of x (row-major [*, DIM]) into feature planes,
// and pad up to the next multiple of STEP with +inf (an infinite coordinate gives an infinite
// or NaN distance, which no strict "<" accepts).
template <typename T, int DIM>
__device__ __forceinline__ void stage_chunk(T *planes, const T *__restrict__ x, int64_t first,
                                            int npts, int tid) {
  using C = LowD<T, DIM>;
  const T *src = x + first * DIM;
  const int total = npts * DIM;
  for (int f = tid; f < total; f += CTA_THREADS) {
    int p = f / DIM, d = f - p * DIM;
    cp_async_elem(&planes[d * C::XP + p], src + f);
  }
  const int padded = (npts + C::STEP - 1) / C::STEP * C::STEP;
  for (int f = total + tid; f < padded * DIM; f += CTA_THREADS) {
    int p = f / DIM, d = f - p * DIM;
    planes[d * C::XP + p] = pos_inf<T>();
  }
  cp_async_commit();
}

// The R points a lane holds for one step.
template <typename T, int DIM>
struct LanePoints;

template <int DIM>
struct LanePoints<float, DIM> {
  using C = LowD<float, DIM>;
  float2 v[DIM][C::R / 2];

  __device__ __forceinline__ void load(const float *planes, int p0) {
#pragma unroll
    for (int d = 0; d < DIM; ++d)
#pragma unroll
      for (int h = 0; h < C::R / 2; ++h)
        v[d][h] = make_float2(planes[d * C::XP + p0 + 64 * h], planes[d * C::XP + p0 + 64 * h + 32]);
  }

  // rec: the query record in shared memory.  out[r] = squared distance to point p0 + 32 r.
  __device__ __forceinline__ float dists(const float *rec, float (&out)[C::R]) const {
    float4 w[C::REC / 4];
#pragma unroll
    for (int i = 0; i < C::REC / 4; ++i) w[i] = reinterpret_cast<const float4 *>(rec)[i];
    const float *f = reinterpret_cast<const float *>(w);
#pragma unroll
    for (int h = 0; h < C::R / 2; ++h) {
      float2 diff = __fadd2_rn(v[0][h], make_float2(f[0], f[1]));
      float2 acc = __fmul2_rn(diff, diff);
#pragma unroll
      for (int d = 1; d < DIM; ++d) {
        diff = __fadd2_rn(v[d][h], make_float2(f[2 * d], f[2 * d + 1]));
        acc = __ffma2_rn(diff, diff, acc);
      }
      out[2 * h] = acc.x;
      out[2 * h + 1] = acc.y;
    }
    return f[2 * DIM];
  }

  __device__ __forceinline__ static void write_rec(float *rec, const float *__restrict__ yrow,
                                                   float bound) {
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
      float q = -yrow[d];
      rec[2 * d] = q;
      rec[2 * d + 1] = q;
    }
    rec[2 * DIM] = bound;
  }
  __device__ __forceinline__ static float *bound_ptr(float *rec) { return rec + 2 * DIM; }
};

template <int DIM>
struct LanePoints<double, DIM> {
  using C = LowD<double, DIM>;
  double v[DIM][C::R];

  __device__ __forceinline__ void load(const double *planes, int p0) {
#pragma unroll
    for (int d = 0; d < DIM; ++d)
#pragma unroll
      for (int r = 0; r < C::R; ++r) v[d][r] = planes[d * C::XP + p0 + 32 * r];
  }

  __device__ __forceinline__ double dists(const double *rec, double (&out)[C::R]) const {
    double2 w[C::REC / 2];
#pragma unroll
    for (int i = 0; i < C::REC / 2; ++i) w[i] = reinterpret_cast<const double2 *>(rec)[i];
    const double *f = reinterpret_cast<const double *>(w);
#pragma unroll
    for (int r = 0; r < C::R; ++r) {
      double diff = __dadd_rn(v[0][r], f[0]);
      double acc = __dmul_rn(diff, diff);
#pragma unroll
      for (int d = 1; d < DIM; ++d) {
        diff = __dadd_rn(v[d][r], f[d]);
        acc = __fma_rn(diff, diff, acc);
      }
      out[r] = acc;
    }
    return f[DIM];
  }

  __device__ __forceinline__ static void write_rec(double *rec, const double *__restrict__ yrow,
                                                   double bound) {
#pragma unroll
    for (int d = 0; d < DIM; ++d) rec[d] = -yrow[d];
    rec[DIM] = bound;
  }
  __device__ __forceinline__ static double *bound_ptr(double *rec) { return rec + DIM; }
};

// Squared distance between two rows with the reference's operation order (used for the single
// "same index" pair of the radius count).
template <typename T, int DIM>
__device__ __forceinline__ T row_sqdist(const T *__restrict__ a, const T *__restrict__ b) {
  T acc = 0;
#pragma unroll
  for (int d = 0; d < DIM; ++d) {
    T diff = a[d] - b[d];
    if constexpr (sizeof(T) == 4)
      acc = __fmaf_rn(diff, diff, acc);
    else
      acc = __fma_rn(diff, diff, acc);
  }
  return acc;
}

}  // namespace b200c
