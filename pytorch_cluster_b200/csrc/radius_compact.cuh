// The copy pass that follows a one-pass radius scan (radius_lowd.cuh, radius_screen.cuh).
#pragma once

#include "common.cuh"

namespace b200c {

// Compaction after a one-pass radius scan: copies the first counts[q] int32 slots of every query's row
// (row_stride slots) to offsets[q].. of the int64 edge rows.  A query with more hits than its row holds
// is left out (its edges are written by a second scan).  A warp takes four consecutive queries at a time and issues
// all their loads (counts, offsets, then up to eight slots per lane) before the first store, so that
// four times as many bytes are in flight per warp as with a query at a time.
static __global__ void radius_direct_compact_kernel(const int32_t *__restrict__ direct_rows,
                                             const int32_t *__restrict__ counts,
                                             const int64_t *__restrict__ offsets, int64_t m, int64_t row_stride,
                                             int64_t *__restrict__ out_row, int64_t *__restrict__ out_col) {
  constexpr int G = 4;
  const int lane = threadIdx.x & 31;
  const int64_t q0 = (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * G;
  if (q0 >= m) return;
  int c[G];
  int64_t o[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const bool in = q0 + g < m;
    c[g] = in ? counts[q0 + g] : 0;
    if (c[g] > row_stride) c[g] = 0;
    o[g] = in ? offsets[q0 + g] : 0;
  }
  int mx = 0;
#pragma unroll
  for (int g = 0; g < G; ++g) mx = c[g] > mx ? c[g] : mx;
  for (int e0 = 0; e0 < mx; e0 += 64) {
    int32_t v[G][2];
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int e = e0 + 32 * h + lane;
        v[g][h] = e < c[g] ? direct_rows[(q0 + g) * row_stride + e] : 0;
      }
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int e = e0 + 32 * h + lane;
        if (e < c[g]) {
          out_row[o[g] + e] = q0 + g;
          out_col[o[g] + e] = v[g][h];
        }
      }
  }
}

}  // namespace b200c
