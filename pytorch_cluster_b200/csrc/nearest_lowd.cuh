// Nearest point assignment for low-dimensional points (1 <= DIM <= 8): the scan of lowd.cuh with
// a lane-private running minimum.
//
// A warp owns up to 8 rows to assign for the whole scan; lane l sees points l, l + 32, ... of
// every 256-point step and keeps, per row, the best (distance, index) among the points it has
// seen.  A step costs the distances, a min tree and one compare; only a lane whose minimum
// reaches its current best goes through its 8 distances.  The 32 partial results of a row meet
// in one shuffle reduction after the scan.  Order among equal minima is the reference's
// (csrc/cuda/nearest_cuda.cu:31-60, see nearest_better in generic.cuh).
#pragma once

#include "generic.cuh"
#include "launchers.h"
#include "lowd.cuh"

namespace b200c {

template <typename T, int DIM>
struct NearestLowD {
  using C = LowD<T, DIM>;
  static constexpr int QW = 8;
  static constexpr int TQ = QW * WARPS_PER_CTA;
  static constexpr size_t PLANES_BYTES = 2 * (size_t)C::PLANES_ELEMS * sizeof(T);
  static constexpr size_t OFF_REC = (PLANES_BYTES + 15) / 16 * 16;
  static constexpr size_t SMEM_BYTES = OFF_REC + (size_t)TQ * C::REC * sizeof(T);
};

// pts / ptr_p: the points searched (the reference's y); rows / ptr_r: the rows assigned (its x).
template <typename T, int DIM>
__global__ void __launch_bounds__(CTA_THREADS, 2)
nearest_lowd_kernel(const T *__restrict__ pts, const T *__restrict__ rows, const int64_t *__restrict__ ptr_p,
                    const int64_t *__restrict__ ptr_r, int num_segments, int64_t n_pts, int64_t n_rows,
                    int64_t *__restrict__ out) {
  using Cfg = NearestLowD<T, DIM>;
  using C = LowD<T, DIM>;
  constexpr int QW = Cfg::QW, TQ = Cfg::TQ, R = C::R;

  extern __shared__ __align__(16) unsigned char smem_nearest[];
  T *planes = reinterpret_cast<T *>(smem_nearest);
  T *recs = reinterpret_cast<T *>(smem_nearest + Cfg::OFF_REC);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T *my_recs = recs + warp * QW * C::REC;

  const int64_t tile_lo = (int64_t)blockIdx.x * TQ;
  const int64_t tile_hi = tile_lo + TQ < n_rows ? tile_lo + TQ : n_rows;
  const int b_first = segment_of(ptr_r, num_segments, tile_lo);
  const int b_last = segment_of(ptr_r, num_segments, tile_hi - 1);

  for (int b = b_first; b <= b_last; ++b) {
    int64_t r_lo, r_hi, p_lo, p_hi;
    segment_rows(ptr_r, num_segments, n_rows, b, r_lo, r_hi);
    const int64_t q_lo = r_lo > tile_lo ? r_lo : tile_lo;
    const int64_t q_hi = r_hi < tile_hi ? r_hi : tile_hi;
    if (q_lo >= q_hi) continue;
    segment_points(ptr_p, n_pts, b, p_lo, p_hi);

    const int nq_tile = (int)(q_hi - q_lo);
    const int nq = nq_tile > warp ? (nq_tile - warp + WARPS_PER_CTA - 1) / WARPS_PER_CTA : 0;

    const T init = (T)1e38;  // only distances below it compete (nearest_cuda.cu:31, 41)
    T best[QW];
    int best_rel[QW];  // offset from the segment's first point; -1: nothing admissible seen yet
#pragma unroll
    for (int qi = 0; qi < QW; ++qi) {
      best[qi] = init;
      best_rel[qi] = -1;
      if (lane == 0) {
        const int64_t q = qi < nq ? q_lo + warp + (int64_t)qi * WARPS_PER_CTA : q_lo;
        LanePoints<T, DIM>::write_rec(my_recs + qi * C::REC, rows + q * DIM, init);
      }
    }
    __syncwarp();

    const int64_t np = p_hi > p_lo ? p_hi - p_lo : 0;
    const int nchunks = (int)((np + C::XC - 1) / C::XC);
    if (nchunks > 0) {
      const int npts0 = np < C::XC ? (int)np : C::XC;
      stage_chunk<T, DIM>(planes, pts, p_lo, npts0, tid);
    }
    for (int c = 0; c < nchunks; ++c) {
      const int64_t first = p_lo + (int64_t)c * C::XC;
      const int npts = (p_hi - first) < C::XC ? (int)(p_hi - first) : C::XC;
      if (c + 1 < nchunks) {
        const int64_t nfirst = first + C::XC;
        const int nn = (p_hi - nfirst) < C::XC ? (int)(p_hi - nfirst) : C::XC;
        stage_chunk<T, DIM>(planes + ((c + 1) & 1) * C::PLANES_ELEMS, pts, nfirst, nn, tid);
        cp_async_wait<1>();
      } else {
        cp_async_wait<0>();
      }
      __syncthreads();
      if (nq > 0) {
        const T *buf = planes + (c & 1) * C::PLANES_ELEMS;
        const int nsub = (npts + C::STEP - 1) / C::STEP;
        for (int sub = 0; sub < nsub; ++sub) {
          LanePoints<T, DIM> lp;
          lp.load(buf, sub * C::STEP + lane);
          const int rel0 = c * C::XC + sub * C::STEP + lane;
#pragma unroll
          for (int qi = 0; qi < QW; ++qi) {
            T dist[R];
            lp.dists(my_recs + qi * C::REC, dist);
            const T dmin = min_of(dist);
            if (dmin < best[qi]) {
              // the 8 points of a step lie in one 1024-aligned block of the segment, where the
              // reference's order among equal distances is the index order: first strict minimum
#pragma unroll
              for (int r = 0; r < R; ++r) {
                const bool take = dist[r] < best[qi];
                best[qi] = take ? dist[r] : best[qi];
                best_rel[qi] = take ? rel0 + 32 * r : best_rel[qi];
              }
            } else if (dmin == best[qi] && best_rel[qi] >= 0) {
              // equal to the best of an earlier step: the full order decides (rare)
#pragma unroll
              for (int r = 0; r < R; ++r) {
                if (nearest_better(dist[r], (int64_t)(rel0 + 32 * r), best[qi], (int64_t)best_rel[qi], (int64_t)0)) {
                  best[qi] = dist[r];
                  best_rel[qi] = rel0 + 32 * r;
                }
              }
            }
          }
        }
      }
      __syncthreads();
    }

#pragma unroll
    for (int qi = 0; qi < QW; ++qi) {
      if (qi < nq) {
        T bd = best[qi];
        int bi = best_rel[qi];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          const T od = __shfl_xor_sync(FULL_MASK, bd, o);
          const int oi = __shfl_xor_sync(FULL_MASK, bi, o);
          if (oi >= 0 && (bi < 0 || nearest_better(od, (int64_t)oi, bd, (int64_t)bi, (int64_t)0))) {
            bd = od;
            bi = oi;
          }
        }
        if (lane == 0) out[q_lo + warp + (int64_t)qi * WARPS_PER_CTA] = bi < 0 ? 0 : p_lo + bi;
      }
    }
    __syncthreads();
  }
}

template <typename T, int DIM>
static int launch_nearest_lowd_one(const KnnArgs &a) {
  using Cfg = NearestLowD<T, DIM>;
  auto kern = nearest_lowd_kernel<T, DIM>;
  static unsigned long long configured = 0ull;  // devices on which the shared-memory opt-in is done
  B200C_CUDA(opt_in_shared_memory(kern, Cfg::SMEM_BYTES, configured));
  const int64_t tiles = (a.m + Cfg::TQ - 1) / Cfg::TQ;
  if (tiles > 0x7fffffffLL) {
    set_error("too many row tiles");
    return B200C_ERR_INVALID;
  }
  kern<<<(unsigned)tiles, CTA_THREADS, Cfg::SMEM_BYTES, a.stream>>>((const T *)a.x, (const T *)a.y, a.ptr_x, a.ptr_y,
                                                                   a.num_segments, a.n, a.m, a.out_col);
  B200C_LAUNCH_CHECK("nearest_lowd_kernel");
  return B200C_OK;
}

// a.x / a.ptr_x: the points searched; a.y / a.ptr_y: the rows assigned; a.out_col [a.m]
template <typename T>
static int launch_nearest_lowd(const KnnArgs &a) {
  switch (a.dim) {
    case 1: return launch_nearest_lowd_one<T, 1>(a);
    case 2: return launch_nearest_lowd_one<T, 2>(a);
    case 3: return launch_nearest_lowd_one<T, 3>(a);
    case 4: return launch_nearest_lowd_one<T, 4>(a);
    case 5: return launch_nearest_lowd_one<T, 5>(a);
    case 6: return launch_nearest_lowd_one<T, 6>(a);
    case 7: return launch_nearest_lowd_one<T, 7>(a);
    case 8: return launch_nearest_lowd_one<T, 8>(a);
  }
  set_error("low-dimensional nearest kernel called with dim=%d", a.dim);
  return B200C_ERR_INVALID;
}

}  // namespace b200c
