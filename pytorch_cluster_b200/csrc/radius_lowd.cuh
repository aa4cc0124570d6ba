// Fixed-radius search for low-dimensional points: count pass and ordered fill pass.
//
// Both passes use the scan of lowd.cuh; the count pass keeps one counter per (lane, query) in
// registers and needs no warp communication in its inner loop, the fill pass appends through
// radius_fill_offer (select.cuh).
#pragma once

#include "lowd.cuh"
#include "select.cuh"

namespace b200c {

template <typename T, int DIM>
struct RadiusLowD {
  using C = LowD<T, DIM>;
  static constexpr int QW = 8;
  static constexpr int TQ = QW * WARPS_PER_CTA;
  static constexpr size_t PLANES_BYTES = 2 * (size_t)C::PLANES_ELEMS * sizeof(T);
  static constexpr size_t OFF_REC = (PLANES_BYTES + 15) / 16 * 16;
  static constexpr size_t SMEM_BYTES = OFF_REC + (size_t)TQ * C::REC * sizeof(T);
};

// FILL == false: counts[q] = min(max_nn, hits(q)).
// FILL == true : edge rows written at offsets[q] .. offsets[q + 1].
template <typename T, int DIM, bool FILL>
__global__ void __launch_bounds__(CTA_THREADS)
radius_lowd_kernel(const T *__restrict__ x, const T *__restrict__ y,
                   const int64_t *__restrict__ ptr_x, const int64_t *__restrict__ ptr_y,
                   int num_segments, int64_t n, int64_t m, T r2, int64_t max_nn, int ignore_same,
                   int32_t *__restrict__ counts, const int64_t *__restrict__ offsets,
                   int64_t *__restrict__ out_row, int64_t *__restrict__ out_col) {
  using Cfg = RadiusLowD<T, DIM>;
  using C = LowD<T, DIM>;
  constexpr int QW = Cfg::QW, TQ = Cfg::TQ, R = C::R;

  extern __shared__ __align__(16) unsigned char smem[];
  T *planes = reinterpret_cast<T *>(smem);
  T *recs = reinterpret_cast<T *>(smem + Cfg::OFF_REC);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T *my_recs = recs + warp * QW * C::REC;
  const bool may_stop_early = max_nn < (int64_t)(1 << 20);

  const int64_t tile_lo = (int64_t)blockIdx.x * TQ;
  const int64_t tile_hi = tile_lo + TQ < m ? tile_lo + TQ : m;
  const int b_first = segment_of(ptr_y, num_segments, tile_lo);
  const int b_last = segment_of(ptr_y, num_segments, tile_hi - 1);

  for (int b = b_first; b <= b_last; ++b) {
    int64_t y_lo, y_hi, x_lo, x_hi;
    segment_rows(ptr_y, num_segments, m, b, y_lo, y_hi);
    const int64_t q_lo = y_lo > tile_lo ? y_lo : tile_lo;
    const int64_t q_hi = y_hi < tile_hi ? y_hi : tile_hi;
    if (q_lo >= q_hi) continue;
    segment_points(ptr_x, n, b, x_lo, x_hi);

    const int nq_tile = (int)(q_hi - q_lo);
    const int nq = nq_tile > warp ? (nq_tile - warp + WARPS_PER_CTA - 1) / WARPS_PER_CTA : 0;

    // per-query state, all in registers (the query loops below are fully unrolled)
    int cnt[QW];        // count pass: this lane's hits; fill pass: hits of the query so far
    int64_t base[QW];   // fill pass: offsets[q]
    int limit[QW];      // fill pass: number of edges to write
#pragma unroll
    for (int qi = 0; qi < QW; ++qi) {
      cnt[qi] = 0;
      base[qi] = 0;
      limit[qi] = 0;
      if (qi < nq) {
        const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
        if (lane == 0) LanePoints<T, DIM>::write_rec(my_recs + qi * C::REC, y + q * DIM, r2);
        if constexpr (FILL) {
          base[qi] = offsets[q];
          limit[qi] = (int)(offsets[q + 1] - base[qi]);
        }
      }
    }
    __syncwarp();
    bool active = nq > 0;
    if constexpr (FILL) {
      bool todo = false;
#pragma unroll
      for (int qi = 0; qi < QW; ++qi) todo |= limit[qi] > 0;
      active = active && todo;
    }

    const int64_t nx = x_hi > x_lo ? x_hi - x_lo : 0;
    const int nchunks = (int)((nx + C::XC - 1) / C::XC);
    if (nchunks > 0) {
      const int npts0 = nx < C::XC ? (int)nx : C::XC;
      stage_chunk<T, DIM>(planes, x, x_lo, npts0, tid);
    }
    for (int c = 0; c < nchunks; ++c) {
      const int64_t first = x_lo + (int64_t)c * C::XC;
      const int npts = (x_hi - first) < C::XC ? (int)(x_hi - first) : C::XC;
      if (c + 1 < nchunks) {
        const int64_t nfirst = first + C::XC;
        const int nn = (x_hi - nfirst) < C::XC ? (int)(x_hi - nfirst) : C::XC;
        stage_chunk<T, DIM>(planes + ((c + 1) & 1) * C::PLANES_ELEMS, x, nfirst, nn, tid);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      const T *buf = planes + (c & 1) * C::PLANES_ELEMS;
      const int nsub = (npts + C::STEP - 1) / C::STEP;
      if (active) {
        for (int sub = 0; sub < nsub; ++sub) {
          LanePoints<T, DIM> pts;
          pts.load(buf, sub * C::STEP + lane);
          const int64_t idx0 = first + sub * C::STEP + lane;
#pragma unroll
          for (int qi = 0; qi < QW; ++qi) {
            if (qi < nq) {
              T dist[R];
              const T bound = pts.dists(my_recs + qi * C::REC, dist);
              if constexpr (!FILL) {
#pragma unroll
                for (int r = 0; r < R; ++r) cnt[qi] += dist[r] < bound ? 1 : 0;
              } else {
                const T dmin = min_of(dist);
                if (__any_sync(FULL_MASK, dmin < bound)) {
                  const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
                  radius_fill_offer<T, R>(dist, bound, idx0, q, ignore_same != 0, cnt[qi], limit[qi], base[qi],
                                          out_row, out_col, lane);
                }
              }
            }
          }
        }
        // a warp whose queries all reached their quota has nothing left to find
        if constexpr (FILL) {
          bool todo = false;
#pragma unroll
          for (int qi = 0; qi < QW; ++qi) todo |= cnt[qi] < limit[qi];
          active = todo;
        } else if (may_stop_early) {
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
      __syncthreads();
    }

    if constexpr (!FILL) {
#pragma unroll
      for (int qi = 0; qi < QW; ++qi) {
        if (qi < nq) {
          const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
          int tot = cnt[qi];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(FULL_MASK, tot, o);
          if (lane == 0) {
            int64_t c = tot;
            if (ignore_same && q >= x_lo && q < x_hi &&
                row_sqdist<T, DIM>(x + q * DIM, y + q * DIM) < r2)
              c -= 1;
            counts[q] = (int32_t)(c < max_nn ? c : max_nn);
          }
        }
      }
    }
    __syncthreads();
  }
}

}  // namespace b200c
