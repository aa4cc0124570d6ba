// Consumers of candidate distances, shared by the low-dimensional and the general kernels.
//
// kNN: threshold-first selection.  Every query keeps, in shared memory, a sorted list of its best
// KP >= k candidates and a queue of KP pending ones, plus its current bound (the k-th best
// distance; 1e10 while fewer than k are known — the reference's initial value,
// csrc/cuda/knn_cuda.cu:48).  Only a distance strictly below the bound is queued (ballot +
// prefix popcount); a full queue is merged into the list by a warp-wide bitonic network
// (shuffles for KP == 32, shared memory above).  Keys order by (distance, index) and the
// scan advances through x in ascending order, so the final list equals the reference's
// insertion result: its strict '>' keeps the lower index on ties (knn_cuda.cu:67-77).
//
// Radius: the hits of 32 consecutive points form a ballot; a lane's output slot is the query's
// running total plus the popcount of the lower lanes — "append in ascending x order, stop at
// max_num_neighbors" (csrc/cuda/radius_cuda.cu:33-40) without atomics, because one warp owns a
// query for the whole scan.
#pragma once

#include "common.cuh"

namespace b200c {

// Merge the first `cnt` queued keys of a query into its sorted list; returns the new bound.
template <typename T, int KP>
__device__ __forceinline__ T knn_merge(Key<T> *keys /* [KP list | KP queue] */, int cnt, int k,
                                       int lane) {
  using K = Key<T>;
  __syncwarp();
  K kth;
  if constexpr (KP == 32) {
    K lk = keys[lane];
    K qk = lane < cnt ? keys[32 + lane] : K::empty();
    qk = warp_sort32(qk, lane);
    K rq = qk.shfl(31 - lane);
    K mn = key_min(lk, rq);
    mn = warp_bitonic_merge32(mn, lane);
    keys[lane] = mn;
    kth = mn.shfl(k - 1);
  } else {
    for (int i = cnt + lane; i < KP; i += 32) keys[KP + i] = K::empty();
    warp_sort_shared(keys, 2 * KP, lane);
    kth = keys[k - 1];
  }
  __syncwarp();
  return kth.is_empty() ? (T)1e10 : kth.dist();
}

template <typename T, int KP>
__device__ __forceinline__ void knn_reset(Key<T> *keys, int lane) {
  for (int i = lane; i < KP; i += 32) keys[i] = Key<T>::empty();
}

// Offer NR candidates per lane to one query: candidate r of lane l has distance dist[r] and
// index idx0 + 32 r (idx0 already includes the lane).  `cnt` (queue fill) and `bound` are
// warp-uniform and updated in place.  Must be called by the whole warp.
template <typename T, int KP, int NR>
__device__ __forceinline__ void knn_offer(Key<T> *keys, int &cnt, T &bound, const T (&dist)[NR],
                                          uint32_t idx0, int k, int lane) {
  using K = Key<T>;
  const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    bool hit = dist[r] < bound;
    unsigned mask = __ballot_sync(FULL_MASK, hit);
    if (mask) {
      int nh = __popc(mask);
      if (cnt + nh > KP) {
        bound = knn_merge<T, KP>(keys, cnt, k, lane);
        cnt = 0;
        hit = dist[r] < bound;
        mask = __ballot_sync(FULL_MASK, hit);
        nh = __popc(mask);
      }
      if (hit) keys[KP + cnt + __popc(mask & lt_mask)] = K::make(dist[r], idx0 + 32u * r);
      cnt += nh;
    }
  }
}

// Final merge and padded output of one query (row q): slots q*k .. q*k+k-1.  Returns the number
// of valid slots (warp-uniform).
template <typename T, int KP>
__device__ __forceinline__ int knn_finish(Key<T> *keys, int cnt, int k, int64_t q,
                                          int64_t *__restrict__ out_row, int64_t *__restrict__ out_col,
                                          int lane) {
  if (cnt > 0) knn_merge<T, KP>(keys, cnt, k, lane);
  int valid = 0;
  for (int e = lane; e < k; e += 32) {
    Key<T> key = keys[e];
    bool ok = !key.is_empty();
    out_row[q * k + e] = q;
    out_col[q * k + e] = ok ? (int64_t)key.index() : (int64_t)-1;
    valid += ok;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) valid += __shfl_xor_sync(FULL_MASK, valid, o);
  return valid;
}

// Ordered append of radius hits.  `run` = hits of the query so far (warp-uniform).
template <typename T, int NR>
__device__ __forceinline__ void radius_fill_offer(const T (&dist)[NR], T r2, int64_t idx0, int64_t q,
                                                  bool ignore_same, int &run, int limit, int64_t base,
                                                  int64_t *__restrict__ out_row,
                                                  int64_t *__restrict__ out_col, int lane) {
  const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int64_t idx = idx0 + 32 * r;
    const bool hit = dist[r] < r2 && !(ignore_same && idx == q);
    const unsigned mask = __ballot_sync(FULL_MASK, hit);
    if (mask) {
      const int pos = run + __popc(mask & lt_mask);
      if (hit && pos < limit) {
        out_row[base + pos] = q;
        out_col[base + pos] = idx;
      }
      run += __popc(mask);
    }
  }
}

template <typename T, int N>
__device__ __forceinline__ T min_of(const T (&a)[N]) {
  // fmin ignores a NaN operand, so one NaN distance cannot hide a hit next to it
  T m = a[0];
#pragma unroll
  for (int i = 1; i < N; ++i) m = fmin(m, a[i]);
  return m;
}

}  // namespace b200c
