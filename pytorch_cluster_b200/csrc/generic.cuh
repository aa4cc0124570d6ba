// Exact brute-force kernels for any feature dimension (used above 8 features, for cosine
// distance, and wherever the tensor-core candidate path does not apply).
//
// Same ownership as the low-dimensional scan: a CTA owns 32 consecutive query rows, each warp 4
// of them for the whole scan.  Points stream through shared memory in blocks of 256 points x 16
// features (cp.async, double buffered, one plane per feature); a lane owns points l and l + 32 of
// each group of 64 and keeps the 4 x 4 x 2 running distances of its (group, query, point)
// triples in registers while the feature blocks go by.  A pair's accumulator therefore sees its
// features in ascending order, one fused multiply-add each: acc = fma(x_d - y_d, x_d - y_d, acc)
// for squared L2 (csrc/cuda/knn_cuda.cu:61-64) or acc = fma(x_d, y_d, acc) for the dot product
// of the cosine distance (knn_cuda.cu:9-18), which is then finished as
// 1 - dot / (|x| * |y|) with norms = sqrt of the same sequential sum (knn_cuda.cu:20-27, 55-59).
#pragma once

#include "common.cuh"
#include "select.cuh"

namespace b200c {

enum GenMode { GEN_KNN = 0, GEN_RADIUS_COUNT = 1, GEN_RADIUS_FILL = 2, GEN_NEAREST = 3 };

template <typename T>
struct GenD {
  static constexpr int R = 2;            // points per lane per group
  static constexpr int GROUP = 64;       // points per group (32 lanes x R)
  static constexpr int NSUB = 4;         // groups per staged block
  static constexpr int XC = GROUP * NSUB;
  static constexpr int NR = NSUB * R;    // candidates per lane per block
  static constexpr int DC = 16;          // features per staged block
  static constexpr int XP = XC + 2;      // plane stride: two rows of 16 features hit 32 banks
  static constexpr int QW = 4;
  static constexpr int TQ = QW * WARPS_PER_CTA;
  static constexpr int STAGE_ELEMS = DC * XP + TQ * DC;  // point planes + query block
};

template <typename T, int KP>
struct GenSmem {
  using G = GenD<T>;
  static constexpr size_t STAGE_BYTES = 2 * (size_t)G::STAGE_ELEMS * sizeof(T);
  static constexpr size_t OFF_KEYS = (STAGE_BYTES + 15) / 16 * 16;
  static constexpr size_t KEYS_BYTES = KP > 0 ? (size_t)G::TQ * 2 * KP * sizeof(Key<T>) : 0;
  static constexpr size_t OFF_CNT = OFF_KEYS + KEYS_BYTES;  // kNN: queue fill per query
  static constexpr size_t SMEM_BYTES = OFF_CNT + (KP > 0 ? (size_t)G::TQ * sizeof(int) : 0);
};

// Stage features [d0, d0 + DC) of points [first, first + XC) and of the CTA's query rows.
// Out-of-range points and features are zero (they add exactly nothing to an accumulator;
// out-of-range points are masked by index later).
template <typename T>
__device__ __forceinline__ void stage_block(T *stage, const T *__restrict__ x, const T *__restrict__ y,
                                            int64_t first, int npts, int d0, int dim, int64_t q_lo,
                                            int64_t q_hi, int tid) {
  using G = GenD<T>;
  const int dn = dim - d0 < G::DC ? dim - d0 : G::DC;
  for (int f = tid; f < G::XC * G::DC; f += CTA_THREADS) {
    const int p = f / G::DC, d = f % G::DC;
    T *dst = &stage[d * G::XP + p];
    if (p < npts && d < dn)
      cp_async_elem(dst, x + (first + p) * dim + d0 + d);
    else
      *dst = (T)0;
  }
  T *qs = stage + G::DC * G::XP;
  for (int f = tid; f < G::TQ * G::DC; f += CTA_THREADS) {
    const int s = f / G::DC, d = f % G::DC;
    const int64_t row = q_lo + (s / G::QW) + (int64_t)(s % G::QW) * WARPS_PER_CTA;
    if (row < q_hi && d < dn)
      cp_async_elem(&qs[f], y + row * dim + d0 + d);
    else
      qs[f] = (T)0;
  }
  cp_async_commit();
}

template <typename T>
__device__ __forceinline__ T fma_rn(T a, T b, T c) {
  if constexpr (sizeof(T) == 4)
    return __fmaf_rn(a, b, c);
  else
    return __fma_rn(a, b, c);
}

// The reference's nearest kernel (csrc/cuda/nearest_cuda.cu:31-60) strides 1024 threads over the
// points of a segment; a thread keeps the first strict minimum of its stride and the tree
// reduction keeps the lower thread on equal distances.  Its winner among equal minima is
// therefore the point with the smallest ((index - segment start) mod 1024, index).
constexpr int NEAREST_STRIDE = 1024;

template <typename T>
__device__ __forceinline__ bool nearest_better(T d, int64_t i, T bd, int64_t bi, int64_t seg_lo) {
  if (d < bd) return true;
  if (!(d == bd)) return false;
  const int64_t a = (i - seg_lo) & (NEAREST_STRIDE - 1), b = (bi - seg_lo) & (NEAREST_STRIDE - 1);
  return a < b || (a == b && i < bi);
}

// MODE GEN_KNN:          out_row/out_col padded [m*k], counts, num_valid; `bound0` unused.
// MODE GEN_NEAREST:      out_col[q] = the nearest point of q's segment (0 when no point is closer
//                        than 1e38, as in the reference); the kernel's "x" are the points searched
//                        (the reference's y) and its "y" the rows assigned (the reference's x).
// MODE GEN_RADIUS_COUNT: counts.   MODE GEN_RADIUS_FILL: offsets -> out_row/out_col.
// COSINE only with GEN_KNN; norms_x / norms_y hold |row| as the reference computes it.
// RND: rounding of every operation result for 16-bit inputs widened to float (see rnd16).
template <typename T, int MODE, int KP, bool COSINE, int RND = 0>
__global__ void __launch_bounds__(CTA_THREADS)
generic_kernel(const T *__restrict__ x, const T *__restrict__ y, const int64_t *__restrict__ ptr_x,
               const int64_t *__restrict__ ptr_y, int num_segments, int64_t n, int64_t m, int dim, int k,
               T r2, int64_t max_nn, int ignore_same, const T *__restrict__ norms_x,
               const T *__restrict__ norms_y, const int64_t *__restrict__ offsets,
               int64_t *__restrict__ out_row, int64_t *__restrict__ out_col, int32_t *__restrict__ counts,
               unsigned long long *__restrict__ num_valid, int64_t query_base) {
  using G = GenD<T>;
  using S = GenSmem<T, KP>;
  using K = Key<T>;
  constexpr int QW = G::QW, TQ = G::TQ, NSUB = G::NSUB, R = G::R, NR = G::NR;

  extern __shared__ __align__(16) unsigned char smem[];
  T *stage = reinterpret_cast<T *>(smem);
  K *keys_all = reinterpret_cast<K *>(smem + S::OFF_KEYS);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  K *my_keys = keys_all + (size_t)warp * QW * 2 * (KP > 0 ? KP : 1);
  int *my_cnt = reinterpret_cast<int *>(smem + S::OFF_CNT) + warp * QW;
  const bool may_stop_early = max_nn < (int64_t)(1 << 20);

  const int64_t tile_lo = (int64_t)blockIdx.x * TQ;
  const int64_t tile_hi = tile_lo + TQ < m ? tile_lo + TQ : m;
  const int b_first = segment_of(ptr_y, num_segments, tile_lo);
  const int b_last = segment_of(ptr_y, num_segments, tile_hi - 1);
  const int nd = (dim + G::DC - 1) / G::DC;
  int my_valid = 0;

  for (int b = b_first; b <= b_last; ++b) {
    int64_t y_lo, y_hi, x_lo, x_hi;
    segment_rows(ptr_y, num_segments, m, b, y_lo, y_hi);
    const int64_t q_lo = y_lo > tile_lo ? y_lo : tile_lo;
    const int64_t q_hi = y_hi < tile_hi ? y_hi : tile_hi;
    if (q_lo >= q_hi) continue;
    segment_points(ptr_x, n, b, x_lo, x_hi);

    const int nq_tile = (int)(q_hi - q_lo);
    const int nq = nq_tile > warp ? (nq_tile - warp + WARPS_PER_CTA - 1) / WARPS_PER_CTA : 0;

    // per-query state in registers (query loops are fully unrolled)
    T bound[QW];      // kNN: current k-th distance; radius: r2
    T ny[QW];         // cosine: |y_q|
    int cnt[QW];      // count: lane's hits; fill: hits so far
    int64_t base[QW];
    int limit[QW];
#pragma unroll
    for (int qi = 0; qi < QW; ++qi) {
      bound[qi] = MODE == GEN_KNN ? rnd16<RND>((T)1e10) : (MODE == GEN_NEAREST ? rnd16<RND>((T)1e38) : r2);
      ny[qi] = (T)1;
      cnt[qi] = 0;
      base[qi] = 0;
      limit[qi] = 0;
      if (qi < nq) {
        const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
        if constexpr (COSINE) ny[qi] = norms_y[q];
        if constexpr (MODE == GEN_KNN) {
          knn_reset<T, KP>(my_keys + qi * 2 * KP, lane);
          if (lane == 0) my_cnt[qi] = 0;
        }
        if constexpr (MODE == GEN_RADIUS_FILL) {
          base[qi] = offsets[q];
          limit[qi] = (int)(offsets[q + 1] - base[qi]);
        }
      }
    }
    __syncwarp();
    bool active = nq > 0;
    if constexpr (MODE == GEN_RADIUS_FILL) {
      bool todo = false;
#pragma unroll
      for (int qi = 0; qi < QW; ++qi) todo |= limit[qi] > 0;
      active = active && todo;
    }

    const int64_t nx = x_hi > x_lo ? x_hi - x_lo : 0;
    const int nchunks = (int)((nx + G::XC - 1) / G::XC);
    const int nsteps = nchunks * nd;  // (point block, feature block) pairs, feature block fastest
    if (nsteps > 0) {
      const int npts0 = nx < G::XC ? (int)nx : G::XC;
      stage_block<T>(stage, x, y, x_lo, npts0, 0, dim, q_lo, q_hi, tid);
    }

    // nearest: every lane's best so far per query; `bound` holds the distance, admissible only below 1e38
    int64_t near_idx[QW];
    bool near_found[QW];
#pragma unroll
    for (int qi = 0; qi < QW; ++qi) {
      near_idx[qi] = 0;
      near_found[qi] = false;
    }

    T acc[NSUB][QW][R];
    for (int t = 0; t < nsteps; ++t) {
      const int c = t / nd, j = t - c * nd;
      const int64_t first = x_lo + (int64_t)c * G::XC;
      if (t + 1 < nsteps) {
        const int c1 = (t + 1) / nd, j1 = (t + 1) - c1 * nd;
        const int64_t nfirst = x_lo + (int64_t)c1 * G::XC;
        const int nn = (x_hi - nfirst) < G::XC ? (int)(x_hi - nfirst) : G::XC;
        stage_block<T>(stage + ((t + 1) & 1) * G::STAGE_ELEMS, x, y, nfirst, nn, j1 * G::DC, dim, q_lo,
                       q_hi, tid);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (active) {
        const T *xs = stage + (t & 1) * G::STAGE_ELEMS;
        const T *qs = xs + G::DC * G::XP + warp * QW * G::DC;
        if (j == 0) {
#pragma unroll
          for (int s = 0; s < NSUB; ++s)
#pragma unroll
            for (int qi = 0; qi < QW; ++qi)
#pragma unroll
              for (int r = 0; r < R; ++r) acc[s][qi][r] = (T)0;
        }
#pragma unroll
        for (int s = 0; s < NSUB; ++s) {
#pragma unroll
          for (int d4 = 0; d4 < G::DC; d4 += 4) {
            T xv[R][4];
#pragma unroll
            for (int dd = 0; dd < 4; ++dd)
#pragma unroll
              for (int r = 0; r < R; ++r) xv[r][dd] = xs[(d4 + dd) * G::XP + s * G::GROUP + 32 * r + lane];
#pragma unroll
            for (int qi = 0; qi < QW; ++qi) {
              T qv[4];
              if constexpr (sizeof(T) == 4) {
                const float4 t4 = *reinterpret_cast<const float4 *>(qs + qi * G::DC + d4);
                qv[0] = t4.x; qv[1] = t4.y; qv[2] = t4.z; qv[3] = t4.w;
              } else {
                const double2 a2 = *reinterpret_cast<const double2 *>(qs + qi * G::DC + d4);
                const double2 b2 = *reinterpret_cast<const double2 *>(qs + qi * G::DC + d4 + 2);
                qv[0] = a2.x; qv[1] = a2.y; qv[2] = b2.x; qv[3] = b2.y;
              }
#pragma unroll
              for (int dd = 0; dd < 4; ++dd)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                  if constexpr (COSINE)
                    acc[s][qi][r] = dot_accumulate<RND>(xv[r][dd], qv[dd], acc[s][qi][r]);
                  else
                    acc[s][qi][r] = sq_accumulate<RND>(xv[r][dd], qv[dd], acc[s][qi][r]);
                }
            }
          }
        }

        if (j == nd - 1) {
          // all features seen: finish the distances of this point block and hand them over
          const int64_t idx0 = first + lane;
          T nxv[NR];
          if constexpr (COSINE) {
#pragma unroll
            for (int i = 0; i < NR; ++i) {
              const int64_t idx = idx0 + 32 * i;
              nxv[i] = idx < x_hi ? norms_x[idx] : (T)1;
            }
          }
#pragma unroll
          for (int qi = 0; qi < QW; ++qi) {
            if (qi < nq) {
              T dist[NR];
#pragma unroll
              for (int s = 0; s < NSUB; ++s)
#pragma unroll
                for (int r = 0; r < R; ++r) {
                  const int i = s * R + r;
                  T d = acc[s][qi][r];
                  if constexpr (COSINE) d = cosine_finish<RND>(d, nxv[i], ny[qi]);
                  dist[i] = (idx0 + 32 * i) < x_hi ? d : pos_inf<T>();
                }
              const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
              if constexpr (MODE == GEN_RADIUS_COUNT) {
#pragma unroll
                for (int i = 0; i < NR; ++i) cnt[qi] += dist[i] < bound[qi] ? 1 : 0;
              } else if constexpr (MODE == GEN_NEAREST) {
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                  // strict "<" against the initial 1e38 (nearest_cuda.cu:31, 41), the full order after
                  const bool take = near_found[qi] ? nearest_better(dist[i], idx0 + 32 * i, bound[qi], near_idx[qi], x_lo)
                                                   : dist[i] < bound[qi];
                  if (take) {
                    bound[qi] = dist[i];
                    near_idx[qi] = idx0 + 32 * i;
                    near_found[qi] = true;
                  }
                }
              } else {
                const T dmin = min_of(dist);
                if (__any_sync(FULL_MASK, dmin < bound[qi])) {
                  if constexpr (MODE == GEN_KNN)
                    knn_offer<T, KP, NR, !COSINE>(my_keys + qi * 2 * KP, my_cnt + qi, bound[qi], dist,
                                                  (uint32_t)idx0, k, lane);
                  else
                    radius_fill_offer<T, NR>(dist, bound[qi], idx0, q, q + query_base, ignore_same != 0, cnt[qi], limit[qi],
                                             base[qi], out_row, out_col, lane);
                }
              }
            }
          }
          if constexpr (MODE == GEN_RADIUS_FILL) {
            bool todo = false;
#pragma unroll
            for (int qi = 0; qi < QW; ++qi) todo |= cnt[qi] < limit[qi];
            active = todo;
          } else if (MODE == GEN_RADIUS_COUNT && may_stop_early) {
            bool todo = false;
#pragma unroll
            for (int qi = 0; qi < QW; ++qi) {
              if (qi < nq) {
                int tot = cnt[qi];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(FULL_MASK, tot, o);
                todo |= (int64_t)tot - (ignore_same ? 1 : 0) < max_nn;
              }
            }
            active = todo;
          }
        }
      }
      __syncthreads();
    }

#pragma unroll
    for (int qi = 0; qi < QW; ++qi) {
      if (qi < nq) {
        const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
        if constexpr (MODE == GEN_KNN) {
          const int valid = knn_finish<T, KP>(my_keys + qi * 2 * KP, my_cnt[qi], k, q, out_row, out_col, lane);
          if (lane == 0) {
            counts[q] = valid;
            my_valid += valid;
          }
        } else if constexpr (MODE == GEN_NEAREST) {
          T bd = bound[qi];
          int64_t bi = near_idx[qi];
          bool bf = near_found[qi];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) {
            const T od = __shfl_xor_sync(FULL_MASK, bd, o);
            const int64_t oi = __shfl_xor_sync(FULL_MASK, bi, o);
            const bool of = __shfl_xor_sync(FULL_MASK, (int)bf, o) != 0;
            if (of && (!bf || nearest_better(od, oi, bd, bi, x_lo))) {
              bd = od;
              bi = oi;
              bf = true;
            }
          }
          if (lane == 0) out_col[q] = bf ? bi : 0;
        } else if constexpr (MODE == GEN_RADIUS_COUNT) {
          int tot = cnt[qi];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(FULL_MASK, tot, o);
          if (lane == 0) {
            int64_t c = tot;
            const int64_t same = q + query_base;  // the x row with the query's own row number
            if (ignore_same && same >= x_lo && same < x_hi) {
              T a = 0;
              for (int d = 0; d < dim; ++d) a = sq_accumulate<RND>(x[same * dim + d], y[q * dim + d], a);
              if (a < r2) c -= 1;
            }
            counts[q] = (int32_t)(c < max_nn ? c : max_nn);
          }
        }
      }
    }
    __syncthreads();
  }
  if constexpr (MODE == GEN_KNN) {
    if (lane == 0 && my_valid) atomicAdd(num_valid, (unsigned long long)my_valid);
  }
}

// |row| for the cosine distance: sqrt of the sequential fused sum of squares
// (csrc/cuda/knn_cuda.cu:20-27).  One thread per row.
template <typename T, int RND = 0>
__global__ void row_norms_kernel(const T *__restrict__ a, int64_t rows, int dim, T *__restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  T s = 0;
  for (int d = 0; d < dim; ++d) {
    const T v = a[i * dim + d];
    s = dot_accumulate<RND>(v, v, s);
  }
  out[i] = rnd16<RND>(sqrt(s));
}

}  // namespace b200c
