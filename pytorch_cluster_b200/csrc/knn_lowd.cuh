// k nearest neighbours for low-dimensional points (1 <= DIM <= 8): the scan of lowd.cuh feeding the
// threshold-first selection of select.cuh.
#pragma once

#include "lowd.cuh"
#include "select.cuh"

namespace b200c {

template <typename T, int DIM, int KP>
struct KnnLowD {
  using C = LowD<T, DIM>;
  using K = Key<T>;
  static constexpr int QCAP = KP;                      // queue capacity
  static constexpr int QW = KP == 32 ? 8 : (KP == 64 ? 4 : 2);  // queries per warp
  static constexpr int TQ = QW * WARPS_PER_CTA;        // queries per CTA
  static constexpr size_t PLANES_BYTES = 2 * (size_t)C::PLANES_ELEMS * sizeof(T);
  static constexpr size_t REC_BYTES = (size_t)TQ * C::REC * sizeof(T);
  static constexpr size_t KEYS_BYTES = (size_t)TQ * (KP + QCAP) * sizeof(K);
  static constexpr size_t CNT_BYTES = (size_t)TQ * sizeof(int);
  static constexpr size_t align16(size_t v) { return (v + 15) / 16 * 16; }
  static constexpr size_t OFF_REC = align16(PLANES_BYTES);
  static constexpr size_t OFF_KEYS = align16(OFF_REC + REC_BYTES);
  static constexpr size_t OFF_CNT = align16(OFF_KEYS + KEYS_BYTES);
  static constexpr size_t SMEM_BYTES = OFF_CNT + CNT_BYTES;
};

template <typename T, int DIM, int KP>
__global__ void __launch_bounds__(CTA_THREADS, KP == 32 ? 3 : 2)
knn_lowd_kernel(const T *__restrict__ x, const T *__restrict__ y, const int64_t *__restrict__ ptr_x,
                const int64_t *__restrict__ ptr_y, int num_segments, int64_t n, int64_t m, int k,
                int64_t *__restrict__ out_row, int64_t *__restrict__ out_col,
                int32_t *__restrict__ counts, unsigned long long *__restrict__ num_valid,
                int64_t *__restrict__ graph_out, int64_t graph_row_stride, int64_t graph_index_base, int graph_s2t,
                int *__restrict__ graph_irregular) {
  using Cfg = KnnLowD<T, DIM, KP>;
  using C = LowD<T, DIM>;
  using K = Key<T>;
  constexpr int QW = Cfg::QW, TQ = Cfg::TQ, R = C::R;

  extern __shared__ __align__(16) unsigned char smem[];
  T *planes = reinterpret_cast<T *>(smem);
  T *recs = reinterpret_cast<T *>(smem + Cfg::OFF_REC);
  K *keys_all = reinterpret_cast<K *>(smem + Cfg::OFF_KEYS);
  int *cnt_all = reinterpret_cast<int *>(smem + Cfg::OFF_CNT);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T *my_recs = recs + warp * QW * C::REC;
  K *my_keys = keys_all + (size_t)warp * QW * (KP + Cfg::QCAP);
  int *my_cnt = cnt_all + warp * QW;

  const int64_t tile_lo = (int64_t)blockIdx.x * TQ;
  const int64_t tile_hi = tile_lo + TQ < m ? tile_lo + TQ : m;
  const int b_first = segment_of(ptr_y, num_segments, tile_lo);
  const int b_last = segment_of(ptr_y, num_segments, tile_hi - 1);
  int my_valid = 0, my_irregular = 0;

  for (int b = b_first; b <= b_last; ++b) {
    int64_t y_lo, y_hi, x_lo, x_hi;
    segment_rows(ptr_y, num_segments, m, b, y_lo, y_hi);
    const int64_t q_lo = y_lo > tile_lo ? y_lo : tile_lo;
    const int64_t q_hi = y_hi < tile_hi ? y_hi : tile_hi;
    if (q_lo >= q_hi) continue;  // uniform for the CTA
    segment_points(ptr_x, n, b, x_lo, x_hi);

    // queries of this warp: rows q_lo + warp, q_lo + warp + 8, ...
    const int nq_tile = (int)(q_hi - q_lo);
    const int nq = nq_tile > warp ? (nq_tile - warp + WARPS_PER_CTA - 1) / WARPS_PER_CTA : 0;
    for (int qi = 0; qi < nq; ++qi) {
      const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
      if (lane == 0) {
        LanePoints<T, DIM>::write_rec(my_recs + qi * C::REC, y + q * DIM, (T)1e10);
        my_cnt[qi] = 0;
      }
      knn_reset<T, KP>(my_keys + qi * (KP + Cfg::QCAP), lane);
    }
    __syncwarp();

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
      if (nq > 0) {
        for (int sub = 0; sub < nsub; ++sub) {
          LanePoints<T, DIM> pts;
          pts.load(buf, sub * C::STEP + lane);
          const uint32_t idx0 = (uint32_t)(first + sub * C::STEP + lane);
          for (int qi = 0; qi < nq; ++qi) {
            T *rec = my_recs + qi * C::REC;
            T dist[R];
            T bound = pts.dists(rec, dist);
            const T dmin = min_of(dist);
            if (__any_sync(FULL_MASK, dmin < bound)) {
              const T before = bound;
              knn_offer<T, KP, R, true>(my_keys + qi * (KP + Cfg::QCAP), my_cnt + qi, bound, dist, idx0, k, lane);
              if (bound != before) {
                if (lane == 0) *LanePoints<T, DIM>::bound_ptr(rec) = bound;
                __syncwarp();
              }
            }
          }
        }
      }
      __syncthreads();
    }

    // final merge and output
    for (int qi = 0; qi < nq; ++qi) {
      const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
      if (graph_out != nullptr) {
        if (!knn_finish_graph<T, KP>(my_keys + qi * (KP + Cfg::QCAP), my_cnt[qi], k, q, graph_row_stride,
                                     graph_index_base, graph_out, graph_s2t != 0, lane))
          ++my_irregular;
        continue;
      }
      const int valid = knn_finish<T, KP>(my_keys + qi * (KP + Cfg::QCAP), my_cnt[qi], k, q, out_row, out_col, lane);
      if (lane == 0) {
        counts[q] = valid;
        my_valid += valid;
      }
    }
    __syncthreads();  // the planes are restaged by the next segment
  }

  if (lane == 0 && my_valid) atomicAdd(num_valid, (unsigned long long)my_valid);
  if (lane == 0 && my_irregular) atomicAdd(graph_irregular, my_irregular);
}

}  // namespace b200c
