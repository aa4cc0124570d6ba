// Fixed-radius search for low-dimensional points (1 <= DIM <= 8).
//
// The scan of lowd.cuh without a single data-dependent branch in its inner loop: for every
// (query, group of 32 consecutive points) the warp's hit predicates become one ballot word, and
// lane 0 parks the 8 words of a step in shared memory.  After a chunk (1024 points = 32 words per
// query) the warp resolves the words of its queries, lane l taking word l:
//   COUNT   counts[q] += popc                      (pass 1 of count -> scan -> fill)
//   FILL    hits are written at offsets[q] + running total + (hits of lower lanes) + (lower bits)
//   DIRECT  as FILL, but into a row of `max_nn` int32 slots per query (one pass; a compaction
//           copy follows the scan) — used when that scratch is small enough
//   COUNT_MASK  as COUNT, and the words themselves go to a bit matrix in global memory (one row of
//           chunks x WORDS words per query), from which radius_mask_fill_kernel writes the edges
//           without evaluating a single distance again — for large neighbour caps
// Ballot words cover points in ascending index order and one warp owns a query for the whole
// scan, so "append in ascending x order, stop at max_num_neighbors"
// (csrc/cuda/radius_cuda.cu:33-40) needs no atomics.  A warp stops scanning once all its queries
// reached their quota, which is what makes truncation cheap.
#pragma once

#include "lowd.cuh"
#include "radius_compact.cuh"
#include "select.cuh"

namespace b200c {

enum RadiusMode { RADIUS_COUNT = 0, RADIUS_FILL = 1, RADIUS_DIRECT = 2, RADIUS_COUNT_MASK = 3 };

template <typename T, int DIM>
struct RadiusLowD {
  using C = LowD<T, DIM>;
  static constexpr int QW = 8;
  static constexpr int TQ = QW * WARPS_PER_CTA;
  static constexpr int WORDS = C::XC / 32;  // ballot words per query and chunk
  static_assert(WORDS <= 32, "one lane resolves one word");
  static constexpr size_t PLANES_BYTES = 2 * (size_t)C::PLANES_ELEMS * sizeof(T);
  static constexpr size_t OFF_REC = (PLANES_BYTES + 15) / 16 * 16;
  static constexpr size_t OFF_MASK = (OFF_REC + (size_t)TQ * C::REC * sizeof(T) + 15) / 16 * 16;
  static constexpr size_t SMEM_BYTES = OFF_MASK + (size_t)TQ * 32 * sizeof(uint32_t);
};

template <typename T, int DIM, int MODE>
__global__ void __launch_bounds__(CTA_THREADS, 3)
radius_lowd_kernel(const T *__restrict__ x, const T *__restrict__ y,
                   const int64_t *__restrict__ ptr_x, const int64_t *__restrict__ ptr_y,
                   int num_segments, int64_t n, int64_t m, T r2, int64_t max_nn, int ignore_same,
                   int32_t *__restrict__ counts, const int64_t *__restrict__ offsets,
                   int64_t *__restrict__ out_row, int64_t *__restrict__ out_col,
                   int32_t *__restrict__ direct_rows, const int64_t *__restrict__ mask_base,
                   uint32_t *__restrict__ mask_words, int64_t query_base) {
  using Cfg = RadiusLowD<T, DIM>;
  using C = LowD<T, DIM>;
  constexpr int QW = Cfg::QW, TQ = Cfg::TQ, R = C::R;
  constexpr int STEP_WORDS = C::STEP / 32;  // = R

  extern __shared__ __align__(16) unsigned char smem[];
  T *planes = reinterpret_cast<T *>(smem);
  T *recs = reinterpret_cast<T *>(smem + Cfg::OFF_REC);
  uint32_t *masks = reinterpret_cast<uint32_t *>(smem + Cfg::OFF_MASK);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  T *my_recs = recs + warp * QW * C::REC;
  uint32_t *my_masks = masks + warp * QW * 32;
  const unsigned lt_mask = (1u << lane) - 1u;
  const int quota_all = max_nn < 0x7fffffffLL ? (int)max_nn : 0x7fffffff;

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

    // per-query state in registers, warp-uniform (the query loops are fully unrolled)
    int run[QW];       // hits so far
    int quota[QW];     // hits to keep: max_nn (count/direct) or offsets[q+1]-offsets[q] (fill)
    int64_t base[QW];  // fill: offsets[q]; direct: q * max_nn
#pragma unroll
    for (int qi = 0; qi < QW; ++qi) {
      run[qi] = 0;
      quota[qi] = 0;
      base[qi] = 0;
      T *rec = my_recs + qi * C::REC;
      if (qi < nq) {
        const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
        if (lane == 0) LanePoints<T, DIM>::write_rec(rec, y + q * DIM, r2);
        if constexpr (MODE == RADIUS_FILL) {
          base[qi] = offsets[q];
          quota[qi] = (int)(offsets[q + 1] - base[qi]);
        } else {
          quota[qi] = quota_all;
          base[qi] = q * max_nn;
        }
      } else if (lane == 0) {
        // an unused slot: bound = -inf, no distance is below it
        LanePoints<T, DIM>::write_rec(rec, y + q_lo * DIM, -pos_inf<T>());
      }
    }
    __syncwarp();
    bool active = false;
#pragma unroll
    for (int qi = 0; qi < QW; ++qi) active |= run[qi] < quota[qi];

    const int64_t nx = x_hi > x_lo ? x_hi - x_lo : 0;
    const int nchunks = (int)((nx + C::XC - 1) / C::XC);
    // COUNT_MASK: the bit rows of this segment's queries start at mask_base[b]; a row has
    // nchunks * WORDS words
    const int64_t row_words = (int64_t)nchunks * Cfg::WORDS;
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
      if (active) {
        const T *buf = planes + (c & 1) * C::PLANES_ELEMS;
        const int nsub = (npts + C::STEP - 1) / C::STEP;
        // ---- scan: ballots only, no branches on the data ----
        for (int sub = 0; sub < nsub; ++sub) {
          LanePoints<T, DIM> pts;
          pts.load(buf, sub * C::STEP + lane);
#pragma unroll
          for (int qi = 0; qi < QW; ++qi) {
            T dist[R];
            const T bound = pts.dists(my_recs + qi * C::REC, dist);
            uint32_t w[R];
#pragma unroll
            for (int r = 0; r < R; ++r) w[r] = __ballot_sync(FULL_MASK, dist[r] < bound);
            if (lane == 0) {
              uint4 *dst = reinterpret_cast<uint4 *>(my_masks + qi * 32 + sub * STEP_WORDS);
#pragma unroll
              for (int v = 0; v < R / 4; ++v) dst[v] = make_uint4(w[4 * v], w[4 * v + 1], w[4 * v + 2], w[4 * v + 3]);
            }
          }
        }
        __syncwarp();
        // ---- resolve: lane l owns word l (points first + 32 l ... + 31) of each query ----
        const int nwords = nsub * STEP_WORDS;
        bool todo = false;
#pragma unroll
        for (int qi = 0; qi < QW; ++qi) {
          if (qi < nq && run[qi] < quota[qi]) {
            const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
            uint32_t word = lane < nwords ? my_masks[qi * 32 + lane] : 0u;
            if (ignore_same) {
              // the pair with equal row numbers is skipped; query_base is the row number of y's first
              // row in the set x indexes (non-zero when y is a slice of a larger query set)
              const int64_t rel = q + query_base - first;
              if (rel >= 0 && (rel >> 5) == lane) word &= ~(1u << (rel & 31));
            }
            const int mine = __popc(word);
            const int total = __reduce_add_sync(FULL_MASK, mine);
            if constexpr (MODE == RADIUS_COUNT_MASK) {
              if (lane < Cfg::WORDS)
                mask_words[mask_base[b] + (q - y_lo) * row_words + (int64_t)c * Cfg::WORDS + lane] = word;
            }
            if constexpr (MODE == RADIUS_FILL || MODE == RADIUS_DIRECT) {
              if (total > 0) {
                // hits of lower lanes: inclusive scan over the lanes, minus own
                int incl = mine;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                  const int t = __shfl_up_sync(FULL_MASK, incl, o);
                  if (lane >= o) incl += t;
                }
                int pos = run[qi] + incl - mine;
                const int64_t idx0 = first + 32 * lane;
                while (word != 0u && pos < quota[qi]) {
                  const int bit = __ffs(word) - 1;
                  word &= word - 1u;
                  if constexpr (MODE == RADIUS_FILL) {
                    out_row[base[qi] + pos] = q;
                    out_col[base[qi] + pos] = idx0 + bit;
                  } else {
                    direct_rows[base[qi] + pos] = (int32_t)(idx0 + bit);
                  }
                  ++pos;
                }
              }
            }
            run[qi] += total;
            todo |= run[qi] < quota[qi];
          }
        }
        active = todo;  // a warp whose queries all reached their quota has nothing left to find
        __syncwarp();
      }
      __syncthreads();
    }

    if constexpr (MODE != RADIUS_FILL) {
#pragma unroll
      for (int qi = 0; qi < QW; ++qi) {
        if (qi < nq && lane == 0) {
          const int64_t q = q_lo + warp + (int64_t)qi * WARPS_PER_CTA;
          counts[q] = run[qi] < quota[qi] ? run[qi] : quota[qi];
        }
      }
    }
    __syncthreads();
  }
}

// Edges from the bit matrix a COUNT_MASK pass left: one warp per query walks the query's row in
// blocks of 128 words (lane l: words 4 l .. 4 l + 3 in one 16-byte load), places every set bit at
// offsets[q] + (bits before it) and stops after counts[q] of them (the truncation rule of
// csrc/cuda/radius_cuda.cu:33-40; words of chunks the scan skipped after the query reached its quota are
// never needed).  The pass is bound by its instruction count, not by bytes in flight, so the loop over a
// lane's bits is kept to the minimum: 32-bit words, one store per bit (the point index); the query's own
// row number goes out separately, count times, by consecutive lanes.
static __global__ void radius_mask_fill_kernel(const uint32_t *__restrict__ mask_words,
                                               const int64_t *__restrict__ mask_base,
                                               const int64_t *__restrict__ ptr_x, const int64_t *__restrict__ ptr_y,
                                               int num_segments, int64_t n, int64_t m, int chunk_points,
                                               const int32_t *__restrict__ counts,
                                               const int64_t *__restrict__ offsets, int64_t *__restrict__ out_row,
                                               int64_t *__restrict__ out_col) {
  const int lane = threadIdx.x & 31;
  const int64_t q = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (q >= m) return;
  const int count = counts[q];
  if (count <= 0) return;
  const int b = segment_of(ptr_y, num_segments, q);
  int64_t y_lo, y_hi, x_lo, x_hi;
  segment_rows(ptr_y, num_segments, m, b, y_lo, y_hi);
  segment_points(ptr_x, n, b, x_lo, x_hi);
  const int64_t nx = x_hi > x_lo ? x_hi - x_lo : 0;
  const int chunk_words = chunk_points / 32;
  const int64_t row_words = (nx + chunk_points - 1) / chunk_points * chunk_words;
  const uint32_t *row = mask_words + mask_base[b] + (q - y_lo) * row_words;
  const int64_t o = offsets[q];
  // the query's own row number, count times: consecutive lanes, consecutive places (the bit loops below then
  // only place the point indices)
  for (int e = lane; e < count; e += 32) out_row[o + e] = q;
  int64_t *col = out_col + o;
  int run = 0;
  // 128 words (4096 points) per step: lane l takes words 4 l .. 4 l + 3 in one 16-byte load (a row holds a
  // whole number of chunks, i.e. a multiple of four words, and starts at such a multiple: the load is aligned
  // and either wholly inside the row or wholly past its end)
  for (int64_t w0 = 0; w0 < row_words && run < count; w0 += 128) {
    const int64_t w = w0 + 4 * lane;
    uint4 quad = make_uint4(0u, 0u, 0u, 0u);
    if (w < row_words) quad = *reinterpret_cast<const uint4 *>(row + w);
    const int mine = __popc(quad.x) + __popc(quad.y) + __popc(quad.z) + __popc(quad.w);
    // hits of lower lanes
    int incl = mine;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int t = __shfl_up_sync(FULL_MASK, incl, d);
      if (lane >= d) incl += t;
    }
    int pos = run + incl - mine;
    const int64_t idx0 = x_lo + w * 32;
    uint32_t words[4] = {quad.x, quad.y, quad.z, quad.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t word = words[j];
      const int64_t first = idx0 + 32 * j;
      while (word != 0u && pos < count) {
        const int bit = __ffs((int)word) - 1;
        word &= word - 1u;
        col[pos] = first + bit;
        ++pos;
      }
    }
    run += __shfl_sync(FULL_MASK, incl, 31);
  }
}

}  // namespace b200c
