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
// index idx0 + 32 r (idx0 already includes the lane).  `cnt_s` is the query's queue fill in
// shared memory, `bound` its current bound (warp-uniform, updated in place).  Must be called by
// the whole warp.  NONNEG promises dist >= 0 (squared L2), which enables the cold-start shortcut.
//
// Fast path: lanes count their own hits, one warp reduction tells whether they fit into the
// queue, and each hitting lane reserves its slots with one shared-memory atomic (the queue is
// unordered; order is restored by the keys when it is merged).
// Cold start (nothing known yet, more hits than the queue holds): the k-th smallest of the 32
// per-lane minima is an upper bound of the k-th smallest of all 32 NR candidates, so it is used
// as a first filter instead of merging group after group.
//
// knn_offer_at is the general form: `index_of(r)` gives the x index of the lane's candidate r;
// knn_offer is the common case index_of(r) = idx0 + 32 r.
template <typename T, int KP, int NR, bool NONNEG, typename IndexOf>
__device__ __forceinline__ void knn_offer_at(Key<T> *keys, int *cnt_s, T &bound, const T (&dist)[NR],
                                             IndexOf index_of, int k, int lane) {
  using K = Key<T>;
  int cnt = *cnt_s;
  T limit = bound;  // candidates must be < limit
  int nl = 0;
#pragma unroll
  for (int r = 0; r < NR; ++r) nl += dist[r] < limit ? 1 : 0;
  int tot = __reduce_add_sync(FULL_MASK, nl);

  if (cnt + tot > KP) {
    if (cnt > 0) {
      bound = knn_merge<T, KP>(keys, cnt, k, lane);
      cnt = 0;
      limit = bound;
    } else if (NONNEG && KP == 32 && sizeof(T) == 4) {
      // cold start on an empty queue
      float lmin = (float)dist[0];
#pragma unroll
      for (int r = 1; r < NR; ++r) lmin = fminf(lmin, (float)dist[r]);
      const uint32_t kth = __shfl_sync(FULL_MASK, warp_sort32_u32(__float_as_uint(lmin), lane), k - 1);
      // non-negative floats order like their bit patterns; NaN patterns sort above +inf
      if (kth < 0x7f800000u) {
        const float cap = __uint_as_float(kth + 1u);  // "<= kth" as a strict bound
        if (cap < (float)limit) limit = (T)cap;
      }
    }
    nl = 0;
#pragma unroll
    for (int r = 0; r < NR; ++r) nl += dist[r] < limit ? 1 : 0;
    tot = __reduce_add_sync(FULL_MASK, nl);
    if (cnt + tot > KP) {
      // still too many at once: go group by group, merging whenever the queue is full
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
          if (hit) keys[KP + cnt + __popc(mask & lt_mask)] = K::make(dist[r], index_of(r));
          cnt += nh;
        }
      }
      __syncwarp();
      if (lane == 0) *cnt_s = cnt;
      __syncwarp();
      return;
    }
    __syncwarp();
    if (lane == 0) *cnt_s = cnt;
    __syncwarp();
  }
  if (nl > 0) {
    int p = KP + atomicAdd(cnt_s, nl);
#pragma unroll
    for (int r = 0; r < NR; ++r) {
      if (dist[r] < limit) {
        keys[p] = K::make(dist[r], index_of(r));
        ++p;
      }
    }
  }
  __syncwarp();
}

template <typename T, int KP, int NR, bool NONNEG>
__device__ __forceinline__ void knn_offer(Key<T> *keys, int *cnt_s, T &bound, const T (&dist)[NR],
                                          uint32_t idx0, int k, int lane) {
  knn_offer_at<T, KP, NR, NONNEG>(keys, cnt_s, bound, dist, [idx0](int r) { return idx0 + 32u * (uint32_t)r; }, k,
                                  lane);
}

// Out-of-line form of knn_offer for hot loops that must stay small: the distances travel by
// value (registers), the new bound comes back as the result.
template <typename T, int NR>
struct DistPack {
  T v[NR];
};

template <typename T, int KP, int NR, bool NONNEG>
__device__ __noinline__ T knn_offer_call(Key<T> *keys, int *cnt_s, T bound, DistPack<T, NR> pack,
                                         uint32_t idx0, int k) {
  knn_offer<T, KP, NR, NONNEG>(keys, cnt_s, bound, pack.v, idx0, k, (int)(threadIdx.x & 31));
  return bound;
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

// knn_graph output of one query (row q) whose k1 = k + 1 best points include q itself: the k other
// ones, in order, at slots q*k .. q*k+k-1 of the two edge rows (row 0 = neighbour, row 1 = query
// when s2t, else the other way round; the rows lie row_stride apart; index_base is added to both) — the `row != col` mask and the flow swap of
// torch_cluster/knn.py:135-144 applied while the list is still in shared memory.  Returns false
// (and writes nothing) when the query has fewer than k1 points or q is not among them; such
// queries need the general path.
template <typename T, int KP>
__device__ __forceinline__ bool knn_finish_graph(Key<T> *keys, int cnt, int k1, int64_t q, int64_t row_stride,
                                                 int64_t index_base, int64_t *__restrict__ graph_out, bool s2t,
                                                 int lane) {
  if (cnt > 0) knn_merge<T, KP>(keys, cnt, k1, lane);
  int valid = 0, selfpos = -1;
  for (int e0 = 0; e0 < k1; e0 += 32) {
    const int e = e0 + lane;
    Key<T> key = e < k1 ? keys[e] : Key<T>::empty();
    const bool ok = !key.is_empty();
    const unsigned self_mask = __ballot_sync(FULL_MASK, ok && (int64_t)key.index() == q);
    if (self_mask != 0u && selfpos < 0) selfpos = e0 + __ffs(self_mask) - 1;
    valid += __popc(__ballot_sync(FULL_MASK, ok));
  }
  if (valid != k1 || selfpos < 0) return false;
  const int64_t k = k1 - 1;
  int64_t *row_nb = s2t ? graph_out : graph_out + row_stride;
  int64_t *row_q = s2t ? graph_out + row_stride : graph_out;
  for (int e = lane; e < k1; e += 32) {
    if (e == selfpos) continue;
    const int64_t slot = q * k + e - (e > selfpos ? 1 : 0);
    row_nb[slot] = index_base + (int64_t)keys[e].index();
    row_q[slot] = index_base + q;
  }
  return true;
}

// Ordered append of radius hits.  `run` = hits of the query so far (warp-uniform); `same` = the x
// row skipped when ignore_same (the query's own row number in x's numbering).
template <typename T, int NR>
__device__ __forceinline__ void radius_fill_offer(const T (&dist)[NR], T r2, int64_t idx0, int64_t q,
                                                  int64_t same, bool ignore_same, int &run, int limit, int64_t base,
                                                  int64_t *__restrict__ out_row,
                                                  int64_t *__restrict__ out_col, int lane) {
  const unsigned lt_mask = (1u << lane) - 1u;
#pragma unroll
  for (int r = 0; r < NR; ++r) {
    const int64_t idx = idx0 + 32 * r;
    const bool hit = dist[r] < r2 && !(ignore_same && idx == same);
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
