// Fixed-radius search for fp32 points of up to 8 features with the screened scan of knn_spatial.cuh.
//
// Still every (query, point) pair of a segment is evaluated, and hits are kept "in ascending x order,
// the first max_num_neighbors of them" (csrc/cuda/radius_cuda.cu:33-40) — but nearly all pairs go through
// DIM fused multiply-adds and a share of a minimum instead of DIM subtractions, DIM multiply-adds, a
// compare and a vote:
//
//   * A small pass lays the points out chunk by chunk (256 points, segments padded to whole chunks, the
//     original order kept): coordinates relative to the segment's first point, their squared norms w,
//     the row numbers, the original coordinates.  One bulk asynchronous copy moves a chunk into a ring of
//     stages in shared memory (a copy warp issues them, mbarriers count them in and out; waits bounded).
//   * A thread block owns 64 consecutive queries, 8 per warp.  Per (query, chunk) a lane screens its 8
//     points with s = w - 2 p'.q' against c = r^2 - |q'|^2 + margin (the margin of knn_spatial.cuh with
//     r^2 as the bound).  Only when some lane's smallest s is at or below c (one vote) does the warp evaluate
//     the chunk for that query with the reference's arithmetic, fma(x_d - y_d, x_d - y_d, acc) over
//     ascending d on the original coordinates (csrc/cuda/radius_cuda.cu:28-32): hit bits by ballot — strictly
//     below (float)(r * r), and not the query's own row when that is to be skipped — placed in ascending
//     position (a chunk's points are consecutive rows), truncated at max_num_neighbors; a query that reached
//     it stops screening.  Segments whose centred norms are not finite are searched exactly throughout.
//
// The scan pays when hits are sparse — the screen of a (query, chunk) pair costs about half of its exact
// evaluation, and a pair with a hit costs both.  A caller can be sure of that from the sizes alone: a query
// keeps at most max_num_neighbors hits, so with segments of at least 2048 * max_num_neighbors points at most
// one (query, chunk) pair in eight can hold one.
//
// Pass 1 (count) parks up to `direct_cap` hits per query as int32 in the workspace and counts up to
// max_num_neighbors; pass 2 copies the parked hits to the edge rows (radius_direct_compact_kernel) and, when
// direct_cap < max_num_neighbors, scans again for exactly the queries that found more than direct_cap
// (thread blocks without such a query leave at once).
#pragma once

#include "knn_spatial.cuh"

namespace b200c {

constexpr int64_t RS_ERROR_WAIT = 1;              // *status when a bounded wait ran out
constexpr int64_t RS_ERROR_OVERLAP = 2;           // *status when the segment pointers of x overlap
enum RadiusScreenMode { RS_PASS_COUNT = 0, RS_PASS_FILL = 1 };

// Pieces of the workspace (radius_screen_carve); status comes first so that a caller can read it.
struct RadiusScreenView {
  int64_t *status;  // [1] 0, RS_ERROR_WAIT or RS_ERROR_OVERLAP
  int64_t *sptr;    // [B + 1] first padded position of every segment of x
  uint32_t *stat;   // [B] largest w of the segment (bits of a non-negative float; +inf: no screen)
  float *blob;      // [cap / 256][2 dim + 2][256]
  int32_t *direct;  // [m][direct_cap]
  int64_t cap;
  int direct_cap;
};

template <int DIM>
struct RadiusScreen {
  using KS = KnnSpatial<DIM, 32>;  // the chunk layout and the per-query screen record
  static constexpr int QW = 8;
  static constexpr int REC = KS::REC;
  static constexpr int QI = (DIM + 3) / 4 * 4;  // the query's own coordinates
  static constexpr size_t OFF_BAR = (size_t)KS_STAGES * KS::STAGE_BYTES;
  static constexpr size_t OFF_REC = OFF_BAR + 2 * KS_STAGES * 8;
  static constexpr size_t OFF_QI = OFF_REC + (size_t)KS_TILE * REC * 4;
  static constexpr size_t OFF_SKIP = OFF_QI + (size_t)KS_TILE * QI * 4;  // int64 [tile]: x row to skip, -1
  static constexpr size_t OFF_BASE = OFF_SKIP + (size_t)KS_TILE * 8;     // int64 [tile]: first output slot
  static constexpr size_t OFF_CNT = OFF_BASE + (size_t)KS_TILE * 8;      // int [tile] x 2: hits, quota
  static constexpr size_t SMEM_BYTES = OFF_CNT + (size_t)KS_TILE * 2 * 4;
};

struct RadiusScreenArgs {
  const float *x, *y;
  const int64_t *ptr_x, *ptr_y;
  int num_segments;
  int64_t n, m;
  float r2;
  int64_t max_nn;
  int ignore_same;
  int64_t query_base;
  int mode;
  int32_t *counts;
  const int64_t *offsets;
  int64_t *out_row, *out_col;
  RadiusScreenView v;
};

// ---- preparation -------------------------------------------------------------------------------------
// One thread block: padded first position of every segment, statistics and status reset.
static __global__ void __launch_bounds__(1024)
rs_layout_kernel(const int64_t *__restrict__ ptr_x, int segs, int64_t n, RadiusScreenView v) {
  __shared__ int64_t run[1024];
  const int t = threadIdx.x;
  const int per = (segs + 1023) / 1024;
  const int lo = t * per < segs ? t * per : segs;
  const int hi = lo + per < segs ? lo + per : segs;
  auto padded = [&](int b) {
    int64_t a, e;
    segment_points(ptr_x, n, b, a, e);
    const int64_t nb = e > a ? e - a : 0;
    return (nb + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
  };
  int64_t mine = 0;
  for (int b = lo; b < hi; ++b) mine += padded(b);
  run[t] = mine;
  __syncthreads();
  for (int o = 1; o < 1024; o <<= 1) {
    const int64_t add = t >= o ? run[t - o] : 0;
    __syncthreads();
    run[t] += add;
    __syncthreads();
  }
  // Overlapping segments (pointers that are not a partition of the rows) would not fit the arrays sized for
  // n rows: their padded sizes then add up to more than the capacity.  The layout is left empty and flagged.
  const bool overlap = run[1023] > v.cap;
  int64_t at = run[t] - mine;
  for (int b = lo; b < hi; ++b) {
    v.sptr[b] = overlap ? 0 : at;
    at += padded(b);
  }
  if (t == 1023) v.sptr[segs] = overlap ? 0 : run[t];
  for (int i = t; i < segs; i += 1024) v.stat[i] = 0u;
  if (t == 0) *v.status = overlap ? RS_ERROR_OVERLAP : 0;
}

// One thread block per chunk of the padded layout: the chunk's arrays, and the segment's largest w.
template <int DIM>
static __global__ void __launch_bounds__(SP_CHUNK)
rs_blob_kernel(const float *__restrict__ x, const int64_t *__restrict__ ptr_x, int segs, int64_t n, RadiusScreenView v) {
  using KS = KnnSpatial<DIM, 32>;
  __shared__ float red[SP_CHUNK / 32];
  const int64_t pos0 = (int64_t)blockIdx.x * SP_CHUNK;
  if (pos0 >= v.sptr[segs]) return;
  int b;
  {
    int lo = 0, hi = segs - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (v.sptr[mid + 1] > pos0)
        hi = mid;
      else
        lo = mid + 1;
    }
    b = lo;
  }
  int64_t x_lo, x_hi;
  segment_points(ptr_x, n, b, x_lo, x_hi);
  const int64_t row = x_lo + (pos0 - v.sptr[b]) + threadIdx.x;
  float *chunk = v.blob + (pos0 / SP_CHUNK) * KS::STAGE_ELEMS + threadIdx.x;
  const float inf = __int_as_float(0x7f800000);
  float w = 0.f;
  if (row < x_hi) {
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
      const float p = x[row * DIM + d];
      const float c = p - x[x_lo * DIM + d];
      chunk[(KS::P_ORG + d) * SP_CHUNK] = p;
      chunk[d * SP_CHUNK] = c;
      w = __fmaf_rn(c, c, w);
    }
    chunk[KS::P_W * SP_CHUNK] = w;
    chunk[KS::P_IDX * SP_CHUNK] = __int_as_float((int32_t)row);
  } else {
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
      chunk[(KS::P_ORG + d) * SP_CHUNK] = inf;
      chunk[d * SP_CHUNK] = inf;
    }
    chunk[KS::P_W * SP_CHUNK] = inf;
    chunk[KS::P_IDX * SP_CHUNK] = __int_as_float(-1);
  }
  // a NaN or huge w switches the segment's screen off
  float wm = (w < 1e30f) ? w : inf;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wm = fmaxf(wm, __shfl_xor_sync(FULL_MASK, wm, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = wm;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < SP_CHUNK / 32; ++i) m = fmaxf(m, red[i]);
    atomicMax(v.stat + b, __float_as_uint(m));  // non-negative floats order like their bits
  }
}

// ---- the scan ----------------------------------------------------------------------------------------
// Where a hit goes: pass 1 parks it in the query's row of the workspace, pass 2 writes the edge.
struct RsSink {
  int mode;
  int direct_cap;
  int32_t *direct;
  int64_t *out_row, *out_col;
  __device__ __forceinline__ void put(int64_t q, int64_t base, int pos, int quota, int64_t x_row) const {
    if (pos >= quota) return;
    if (mode == RS_PASS_COUNT) {
      if (pos < direct_cap) direct[q * direct_cap + pos] = (int32_t)x_row;
    } else {
      out_row[base + pos] = q;
      out_col[base + pos] = x_row;
    }
  }
};

// Whole-warp exact evaluation of a chunk for one query (no screen): hit bits by ballot, hits placed in
// ascending position.  Returns the number of hits.
template <int DIM>
__device__ __noinline__ int rs_chunk_exact(const float *buf, const float *qinfo, float r2, int64_t skip, int64_t q,
                                           int64_t base, int run, int quota, const RsSink sink) {
  using KS = KnnSpatial<DIM, 32>;
  const int lane = threadIdx.x & 31;
  const unsigned lt_mask = (1u << lane) - 1u;
  const int32_t *idx_plane = reinterpret_cast<const int32_t *>(buf + KS::P_IDX * SP_CHUNK);
  float qv[DIM];
#pragma unroll
  for (int d = 0; d < DIM; ++d) qv[d] = qinfo[d];
  int total = 0;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    // the lane's four consecutive points of this half: one 16-byte load per array
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
      const float4 o = *reinterpret_cast<const float4 *>(buf + (KS::P_ORG + d) * SP_CHUNK + h * 128 + 4 * lane);
      const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float diff = __fsub_rn(ov[j], qv[d]);
        acc[j] = __fmaf_rn(diff, diff, acc[j]);
      }
    }
    const int4 id4 = *reinterpret_cast<const int4 *>(idx_plane + h * 128 + 4 * lane);
    const int32_t id[4] = {id4.x, id4.y, id4.z, id4.w};
    bool hit[4];
    unsigned word[4];
    int below = 0;  // hits of lower lanes in this half
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      hit[j] = id[j] >= 0 && acc[j] < r2 && (int64_t)id[j] != skip;
      word[j] = __ballot_sync(FULL_MASK, hit[j]);
      below += __popc(word[j] & lt_mask);
    }
    int pos = run + total + below;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (hit[j]) {
        sink.put(q, base, pos, quota, (int64_t)id[j]);
        ++pos;
      }
      total += __popc(word[j]);
    }
  }
  return total;
}

template <int DIM>
__global__ void __launch_bounds__(KS_THREADS, DIM <= 4 ? KS_MINBLOCKS : 2)
radius_screen_kernel(const RadiusScreenArgs a) {
  using Cfg = RadiusScreen<DIM>;
  using KS = KnnSpatial<DIM, 32>;
  constexpr int QW = Cfg::QW, REC = Cfg::REC, QI = Cfg::QI;

  extern __shared__ __align__(128) unsigned char rs_smem_raw[];
  float *stages = reinterpret_cast<float *>(rs_smem_raw);
  uint64_t *full = reinterpret_cast<uint64_t *>(rs_smem_raw + Cfg::OFF_BAR);
  uint64_t *empty = full + KS_STAGES;
  float *recs = reinterpret_cast<float *>(rs_smem_raw + Cfg::OFF_REC);
  float *qinfos = reinterpret_cast<float *>(rs_smem_raw + Cfg::OFF_QI);
  int64_t *skips = reinterpret_cast<int64_t *>(rs_smem_raw + Cfg::OFF_SKIP);
  int64_t *bases = reinterpret_cast<int64_t *>(rs_smem_raw + Cfg::OFF_BASE);
  int *cnt_all = reinterpret_cast<int *>(rs_smem_raw + Cfg::OFF_CNT);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int segs = a.num_segments;
  const int64_t tile_lo = (int64_t)blockIdx.x * KS_TILE;
  const int64_t tile_hi = tile_lo + KS_TILE < a.m ? tile_lo + KS_TILE : a.m;
  const int direct_cap = a.v.direct_cap;

  // pass 2 is only for queries that found more hits than pass 1 could park
  if (a.mode == RS_PASS_FILL) {
    const bool mine = tid < KS_TILE && tile_lo + tid < tile_hi && a.counts[tile_lo + tid] > direct_cap;
    if (!__syncthreads_or(mine)) return;
  }

  if (tid == 0) {
    for (int s = 0; s < KS_STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ks_smem(full + s)) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ks_smem(empty + s)), "r"(KS_WARPS)
                   : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  const int b_first = segment_of(a.ptr_y, segs, tile_lo);
  const int b_last = segment_of(a.ptr_y, segs, tile_hi - 1);
  const bool producer = warp == KS_WARPS;
  bool failed = false;
  int step = 0;  // chunks of this thread block so far, over all its segments: slot and phase of the ring

  if (producer) {
    // ---- the copy warp: one lane walks the same (segment, chunk) sequence and keeps the ring full ----
    if (lane != 0) return;
    int issued = 0;
    for (int b = b_first; b <= b_last && !failed; ++b) {
      int64_t y_lo, y_hi;
      segment_rows(a.ptr_y, segs, a.m, b, y_lo, y_hi);
      if ((y_lo > tile_lo ? y_lo : tile_lo) >= (y_hi < tile_hi ? y_hi : tile_hi)) continue;
      const int64_t chunk0 = a.v.sptr[b] / SP_CHUNK;
      const int nch = (int)(a.v.sptr[b + 1] / SP_CHUNK - chunk0);
      for (int c = 0; c < nch; ++c, ++step) {
        const int slot = step % KS_STAGES;
        if (step >= KS_STAGES && !ks_wait(empty + slot, (unsigned)((step / KS_STAGES - 1) & 1))) {
          failed = true;
          break;
        }
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(ks_smem(full + slot)),
                     "r"(KS::STAGE_BYTES)
                     : "memory");
        ks_bulk_load(stages + slot * KS::STAGE_ELEMS, a.v.blob + (chunk0 + c) * KS::STAGE_ELEMS, KS::STAGE_BYTES,
                     full + slot);
        issued = step + 1;
      }
    }
    if (failed) {
      // a wait ran out: flag the result as invalid and let the copies already issued land
      for (int s = issued > KS_STAGES ? issued - KS_STAGES : 0; s < issued; ++s)
        (void)ks_wait(full + s % KS_STAGES, (unsigned)((s / KS_STAGES) & 1));
      atomicExch((unsigned long long *)a.v.status, (unsigned long long)RS_ERROR_WAIT);
    }
    return;
  }

  float *my_recs = recs + warp * QW * REC;
  float *my_qi = qinfos + warp * QW * QI;
  int64_t *my_skip = skips + warp * QW, *my_base = bases + warp * QW;
  int *my_run = cnt_all + warp * 2 * QW, *my_quota = my_run + QW;
  const int quota_all = a.max_nn < 0x7fffffffLL ? (int)a.max_nn : 0x7fffffff;
  const float ninf = -__int_as_float(0x7f800000);
  RsSink sink{a.mode, direct_cap, a.v.direct, a.out_row, a.out_col};

  for (int b = b_first; b <= b_last && !failed; ++b) {
    int64_t y_lo, y_hi, x_lo, x_hi;
    segment_rows(a.ptr_y, segs, a.m, b, y_lo, y_hi);
    const int64_t q_lo = y_lo > tile_lo ? y_lo : tile_lo;
    const int64_t q_hi = y_hi < tile_hi ? y_hi : tile_hi;
    if (q_lo >= q_hi) continue;
    segment_points(a.ptr_x, a.n, b, x_lo, x_hi);
    const int nch = (int)((a.v.sptr[b + 1] - a.v.sptr[b]) / SP_CHUNK);
    const float wmax = __uint_as_float(a.v.stat[b]);
    const bool screen = wmax < 1e30f;  // false also for NaN

    // ---- queries of this warp in this segment: q_lo + warp + 8 qi; lane qi prepares query qi ----
    const int nq_tile = (int)(q_hi - q_lo);
    const int nq = nq_tile > warp ? (nq_tile - warp + KS_WARPS - 1) / KS_WARPS : 0;
    __syncwarp();
    if (lane < QW) {
      float *rec = my_recs + lane * REC, *qi = my_qi + lane * QI;
      int quota = 0;
      if (lane < nq && nch > 0) {
        const int64_t q = q_lo + warp + (int64_t)lane * KS_WARPS;
        if (a.mode == RS_PASS_FILL) {
          const int found = a.counts[q];
          quota = found > direct_cap ? found : 0;
          my_base[lane] = a.offsets[q];
        } else {
          quota = quota_all;
          my_base[lane] = 0;
        }
        my_skip[lane] = a.ignore_same ? q + a.query_base : -1;
        float nq2 = 0.f;
#pragma unroll
        for (int d = 0; d < DIM; ++d) {
          const float v = a.y[q * DIM + d];
          const float qc = v - a.x[x_lo * DIM + d];
          qi[d] = v;
          rec[2 * d] = -2.f * qc;
          rec[2 * d + 1] = -2.f * qc;
          nq2 = __fmaf_rn(qc, qc, nq2);
        }
        rec[2 * DIM] = quota > 0 ? ((a.r2 - nq2) + KS_MARGIN * (a.r2 + nq2 + wmax)) + KS_MARGIN_ABS : ninf;
      } else {
#pragma unroll
        for (int d = 0; d < DIM; ++d) {
          qi[d] = 0.f;
          rec[2 * d] = 0.f;
          rec[2 * d + 1] = 0.f;
        }
        rec[2 * DIM] = ninf;  // nothing is at or below -inf
        my_skip[lane] = -1;
        my_base[lane] = 0;
      }
      my_run[lane] = 0;
      my_quota[lane] = quota;
    }
    __syncwarp();
    unsigned open = __ballot_sync(FULL_MASK, lane < QW && my_quota[lane] > 0);  // queries still collecting

    for (int c = 0; c < nch; ++c, ++step) {
      const int slot = step % KS_STAGES;
      if (!ks_wait(full + slot, (unsigned)((step / KS_STAGES) & 1))) {
        failed = true;
        break;
      }
      const float *buf = stages + slot * KS::STAGE_ELEMS;
      if (open != 0u && screen) {
        // the lane's 8 points as four pairs: (slot 0,1) (2,3) of the first run, (4,5) (6,7) of the second
        float2 pc[DIM][4], pw[4];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int d = 0; d < DIM; ++d) {
            const float4 v = *reinterpret_cast<const float4 *>(buf + d * SP_CHUNK + h * 128 + 4 * lane);
            pc[d][2 * h] = make_float2(v.x, v.y);
            pc[d][2 * h + 1] = make_float2(v.z, v.w);
          }
          const float4 v = *reinterpret_cast<const float4 *>(buf + KS::P_W * SP_CHUNK + h * 128 + 4 * lane);
          pw[2 * h] = make_float2(v.x, v.y);
          pw[2 * h + 1] = make_float2(v.z, v.w);
        }
        unsigned pass = 0u;  // queries with a screened point in this chunk
#pragma unroll
        for (int qi = 0; qi < QW; ++qi) {
          const float *rec = my_recs + qi * REC;
          float4 rv[REC / 4];
#pragma unroll
          for (int i = 0; i < REC / 4; ++i) rv[i] = reinterpret_cast<const float4 *>(rec)[i];
          const float *f = reinterpret_cast<const float *>(rv);
          float2 s[4];
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            s[h] = __ffma2_rn(pc[0][h], make_float2(f[0], f[1]), pw[h]);
#pragma unroll
            for (int d = 1; d < DIM; ++d) s[h] = __ffma2_rn(pc[d][h], make_float2(f[2 * d], f[2 * d + 1]), s[h]);
          }
          // fminf drops a NaN operand; eight NaN give NaN, which is below nothing
          const float m0 = fminf(fminf(s[0].x, s[0].y), s[1].x), m1 = fminf(fminf(s[1].y, s[2].x), s[2].y);
          const float m = fminf(fminf(m0, m1), fminf(s[3].x, s[3].y));
          if (__any_sync(FULL_MASK, m <= f[2 * DIM])) pass |= 1u << qi;
        }
        while (pass) {
          const int qi = __ffs(pass) - 1;
          pass &= pass - 1u;
          const int64_t q = q_lo + warp + (int64_t)qi * KS_WARPS;
          const int run = my_run[qi], quota = my_quota[qi];
          const int total = rs_chunk_exact<DIM>(buf, my_qi + qi * QI, a.r2, my_skip[qi], q, my_base[qi], run, quota,
                                                sink);
          __syncwarp();
          if (lane == 0) {
            my_run[qi] = run + total;
            if (run + total >= quota) my_recs[qi * REC + 2 * DIM] = ninf;  // the query has all it may keep
          }
          if (run + total >= quota) open &= ~(1u << qi);
        }
      } else if (open != 0u) {
        for (int qi = 0; qi < QW; ++qi) {
          if (!((open >> qi) & 1u)) continue;
          const int64_t q = q_lo + warp + (int64_t)qi * KS_WARPS;
          const int run = my_run[qi], quota = my_quota[qi];
          const int total = rs_chunk_exact<DIM>(buf, my_qi + qi * QI, a.r2, my_skip[qi], q, my_base[qi], run, quota,
                                                sink);
          __syncwarp();
          if (lane == 0) my_run[qi] = run + total;
          if (run + total >= quota) open &= ~(1u << qi);
        }
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(ks_smem(empty + slot)) : "memory");
    }
    if (failed) break;
    __syncwarp();
    if (a.mode == RS_PASS_COUNT && lane < nq) {
      const int64_t q = q_lo + warp + (int64_t)lane * KS_WARPS;
      const int found = nch > 0 ? my_run[lane] : 0;
      a.counts[q] = found < quota_all ? found : quota_all;
    }
  }
  if (failed && lane == 0) atomicExch((unsigned long long *)a.v.status, (unsigned long long)RS_ERROR_WAIT);
}

}  // namespace b200c
