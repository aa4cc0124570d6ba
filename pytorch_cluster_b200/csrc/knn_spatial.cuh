// k nearest neighbours of low-dimensional fp32 points over Morton-ordered copies (spatial.cuh).
//
// Still a brute-force search — every (query, point) pair of a segment is evaluated — but built so
// that nearly all pairs go through a loop of DIM fused multiply-adds and a share of a minimum:
//
//   * A thread block owns 64 consecutive queries of the sorted order (8 per warp) and starts its
//     scan at the chunk of 256 sorted points around them, then walks outwards, alternating sides.
//     After the first chunks every query's bound (its k-th best candidate so far) is at or close
//     to its final value.
//   * Per (query, chunk) a lane screens its 8 points with s = |p'|^2 - 2 p'.q' (p', q' relative to
//     the centre of the segment's bounding box; |p'|^2 comes with the sorted copy) against
//     c = bound - |q'|^2 + margin, the margin covering the rounding of both sides.  A lane whose
//     smallest s is at or below c — and only that lane, no vote — re-evaluates its screened points with
//     the reference's arithmetic, fma(x_d - y_d, x_d - y_d, acc) over ascending d on the original
//     coordinates (csrc/cuda/knn_cuda.cu:61-64), and appends those that beat the query's k-th best
//     (distance, index) key to the query's queue in shared memory.
//   * After every chunk the warp looks at its queries' queues: queued candidates are merged into
//     the sorted list (select.cuh), which tightens the bound; a queue that overflowed is rolled
//     back to its fill before the chunk and the chunk is offered again by the whole warp.
//     Selection ranks exact distances and original indices only, and keys order by (distance,
//     index), so the result is the reference's whatever the order of the scan.
//   * Chunks travel global -> shared memory as bulk asynchronous copies (one per array, issued by
//     one thread, completion counted by an mbarrier) through a ring of stages; warps release a
//     stage through a second mbarrier, so they drift apart by up to the ring's depth instead of
//     meeting at a block-wide barrier per chunk.  All waits are bounded.
//
// Margin.  With u = 2^-24 and D features, |s - (d - |q'|^2)| for real arithmetic d = |p - q|^2 is at
// most u ((2D + 8) bound + (5D + 5) |q'|^2 + (4D + 2) max|p'|^2) for every pair whose reference distance
// is at most `bound` (rounding of the centred copies, of |p'|^2, |q'|^2, the D-term chains and of
// the reference distance itself); the kernel uses 2^-17 (bound + |q'|^2 + max|p'|^2), at least
// twice that for D <= 8, plus a few steps of the subnormal grid, where rounding errors are absolute;
// the test is s <= c, so that a candidate at exactly the bound's distance (which wins with a lower
// index) passes even where the margin rounds to nothing.  Segments whose centred norms are not finite (or above 1e30) are
// searched without the screen.
#pragma once

#include "select.cuh"
#include "spatial.cuh"

namespace b200c {

constexpr int KS_STAGES = 4;
constexpr int KS_SPIN_LIMIT = 1 << 26;      // polls of a wait (about a second: see ks_wait)
constexpr unsigned KS_WAIT_NS = 20000u;     // suspend-time hint of one poll
constexpr int KS_WARPS = WARPS_PER_CTA;          // scanning warps per thread block
constexpr int KS_MINBLOCKS = 3;                  // thread blocks per SM the register budget is set for
constexpr int KS_TILE = 8 * KS_WARPS;            // queries per thread block
constexpr int KS_THREADS = 32 * (KS_WARPS + 1);  // the scanning warps and the warp that issues the copies
static_assert(KS_TILE == SP_TILE, "the sorted copies pad query segments to whole tiles of this size");
constexpr float KS_MARGIN = 7.62939453125e-6f;  // 2^-17
constexpr float KS_MARGIN_ABS = 2e-43f;         // about 140 steps of the subnormal grid: rounding there is absolute
constexpr unsigned long long KS_ERROR_COUNT = 1ull << 62;  // added to *num_valid when a wait ran out
constexpr int KS_ERROR_IRREGULAR = 1 << 30;                // added to *graph_irregular likewise

template <int DIM, int KP>
struct KnnSpatial {
  using K = Key<float>;
  static constexpr int R = SP_CHUNK / 32;  // points per lane per chunk
  static_assert(R == 8, "the lane layout below takes two float4 per array");
  static constexpr int QW = 8;
  // arrays of a staged chunk: centred coordinates, w, idx, original coordinates
  static constexpr int P_W = DIM, P_IDX = DIM + 1, P_ORG = DIM + 2, PLANES = 2 * DIM + 2;
  static constexpr int STAGE_ELEMS = PLANES * SP_CHUNK;
  static constexpr unsigned STAGE_BYTES = STAGE_ELEMS * 4u;
  static constexpr int REC = (2 * DIM + 1 + 3) / 4 * 4;  // (-2 q'_d) twice each, then c
  // per query: q_d, |q'|^2, then (8-byte aligned) the key of its k-th best candidate
  static constexpr int QI_KTH = (DIM + 1 + 1) / 2 * 2;
  static constexpr int QI = (QI_KTH + 2 + 3) / 4 * 4;
  static constexpr int QCAP = KP;
};

// Stages of the ring and thread blocks per SM of a variant.  Short segments (the rolled variant) spend
// much of their time outside the scan loop — selection code, instruction fetch — and gain more from a
// fourth resident thread block than from a deeper ring; up to three features that block fits with two
// stages (53 KB per block) and 56 registers.  Long segments and more features keep four stages and
// three blocks.  The 64-wide selection is bound by its key arrays to two blocks.
__host__ __device__ constexpr bool ks_four_blocks(int dim, int kp, bool rolled) { return kp == 32 && rolled && dim <= 3; }
__host__ __device__ constexpr int ks_stages(int dim, int kp, bool rolled) {
  return ks_four_blocks(dim, kp, rolled) ? 2 : KS_STAGES;
}
__host__ __device__ constexpr int ks_minblocks(int dim, int kp, bool rolled) {
  return kp == 32 ? (ks_four_blocks(dim, kp, rolled) ? KS_MINBLOCKS + 1 : KS_MINBLOCKS) : 2;
}

// Shared memory of a thread block: the ring's stages, its mbarriers, then the per-query state.
template <int DIM, int KP, int STAGES>
struct KnnSpatialLayout {
  using Cfg = KnnSpatial<DIM, KP>;
  static constexpr size_t OFF_BAR = (size_t)STAGES * Cfg::STAGE_BYTES;
  static constexpr size_t OFF_REC = OFF_BAR + 2 * STAGES * 8;
  static constexpr size_t OFF_QI = OFF_REC + (size_t)KS_TILE * Cfg::REC * 4;
  static constexpr size_t OFF_KEYS = OFF_QI + (size_t)KS_TILE * Cfg::QI * 4;
  static constexpr size_t OFF_CNT = OFF_KEYS + (size_t)KS_TILE * (KP + Cfg::QCAP) * sizeof(Key<float>);
  static constexpr size_t SMEM_BYTES = OFF_CNT + (size_t)KS_TILE * 2 * 4;  // fill, and fill before the chunk
};

__device__ __forceinline__ unsigned ks_smem(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }

// Waits for a phase of an mbarrier with a bounded number of polls.  A poll returns within about ten
// nanoseconds whatever its suspend-time hint (measured: some 14000 polls per thread block of the headline
// workload, which lives 130 us), so 2^26 polls are about a second.  A bound in cycles (clock64 every 256 polls)
// made the scans 2 % slower — the wait is inlined in the scan loop — and so did 128 ns of sleep between the
// polls of the copy warp, which waits nearly all the time (a stage is refilled later; the issue slots its
// spinning takes cost less).
__device__ __forceinline__ bool ks_wait(uint64_t *bar, unsigned parity) {
  unsigned done = 0;
  for (int it = 0; it < KS_SPIN_LIMIT && !done; ++it) {
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(ks_smem(bar)), "r"(parity), "r"(KS_WAIT_NS)
        : "memory");
  }
  return done != 0;
}

__device__ __forceinline__ void ks_bulk_load(void *smem_dst, const void *gmem_src, unsigned bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(
                   ks_smem(smem_dst)),
               "l"(gmem_src), "r"(bytes), "r"(ks_smem(bar))
               : "memory");
}

// Chunk visited at step i of a scan that starts at chunk `seed` of `n` and walks outwards.
__device__ __forceinline__ int ks_chunk_at(int i, int seed, int n) {
  const int left = seed, right = n - 1 - seed;
  const int both = left < right ? left : right;
  if (i <= 2 * both) return (i & 1) ? seed + ((i + 1) >> 1) : seed - (i >> 1);
  const int d = i - both;
  return left > right ? seed - d : seed + d;
}

// Position within its chunk of a lane's point r: two runs of four consecutive points.
__device__ __forceinline__ int ks_slot(int lane, int r) { return (r >> 2) * 128 + 4 * lane + (r & 3); }

// The key no admissible candidate reaches: distance 1e10, the reference's initial best distance
// (csrc/cuda/knn_cuda.cu:48) — candidates must be strictly below it.
__device__ __forceinline__ Key<float> ks_no_bound() { return Key<float>::make(1e10f, 0u); }

// Squared distance of the staged point at `slot` to the query, in the reference's arithmetic.
template <int DIM, int KP>
__device__ __forceinline__ float ks_exact(const float *buf, int slot, const float *qinfo) {
  using Cfg = KnnSpatial<DIM, KP>;
  float acc = 0.f;
#pragma unroll
  for (int d = 0; d < DIM; ++d) {
    const float diff = __fsub_rn(buf[(Cfg::P_ORG + d) * SP_CHUNK + slot], qinfo[d]);
    acc = __fmaf_rn(diff, diff, acc);
  }
  return acc;
}

// A lane found screen values below the query's threshold: its screened points are evaluated
// exactly and those beating the query's k-th key are appended to the queue.  No warp-wide
// operation — lanes without a passing point simply wait at the reconvergence point.  The fill
// counter may run past the queue's capacity; the caller notices and offers the chunk again.
template <int DIM, int KP>
__device__ __noinline__ void ks_push(float s0, float s1, float s2, float s3, float s4, float s5, float s6, float s7,
                                     const float *buf, const float *rec, const float *qinfo, Key<float> *queue,
                                     int *cnt_s) {
  using Cfg = KnnSpatial<DIM, KP>;
  using K = Key<float>;
  const int lane = threadIdx.x & 31;
  const float s[8] = {s0, s1, s2, s3, s4, s5, s6, s7};
  const float c = rec[2 * DIM];
  const uint64_t kth = *reinterpret_cast<const uint64_t *>(qinfo + Cfg::QI_KTH);
  const int32_t *idx_plane = reinterpret_cast<const int32_t *>(buf + Cfg::P_IDX * SP_CHUNK);
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    if (s[r] <= c) {
      const int slot = ks_slot(lane, r);
      const int32_t idx = idx_plane[slot];
      const float d = ks_exact<DIM, KP>(buf, slot, qinfo);
      const K key = K::make(d, (uint32_t)idx);
      // d < 1e10 is the reference's admission test (false for NaN, whatever its sign bit)
      if (idx >= 0 && d < 1e10f && key.v < kth) {
        const int pos = atomicAdd(cnt_s, 1);
        if (pos < Cfg::QCAP) queue[pos] = key;
      }
    }
  }
}

// One copy of the merge network for all its call sites (code size matters more than the call).
template <int KP>
__device__ __noinline__ void ks_merge(Key<float> *keys, int cnt, int k) {
  knn_merge<float, KP>(keys, cnt, k, (int)(threadIdx.x & 31));
}

// The query's bound after a merge: the key of its k-th best candidate (or "none yet"), and the
// screen threshold that goes with it.  Call by the whole warp after knn_merge.
template <int DIM, int KP>
__device__ __forceinline__ void ks_update_bound(const Key<float> *keys, float *rec, float *qinfo, float wmax, int k,
                                                int lane) {
  using Cfg = KnnSpatial<DIM, KP>;
  if (lane == 0) {
    Key<float> kth = keys[k - 1];
    if (!(kth.v < ks_no_bound().v)) kth = ks_no_bound();  // fewer than k known yet
    *reinterpret_cast<uint64_t *>(qinfo + Cfg::QI_KTH) = kth.v;
    const float bound = kth.dist(), nq2 = qinfo[DIM];
    rec[2 * DIM] = ((bound - nq2) + KS_MARGIN * (bound + nq2 + wmax)) + KS_MARGIN_ABS;
  }
  __syncwarp();
}

// Whole-warp offer of a chunk to one query, exact distances for every real point of the chunk (no
// screen): the first chunk of a scan, segments without a usable screen, and chunks whose
// lane-private pushes overflowed the queue.  Candidates are filtered by key against the query's
// k-th best; the queue is merged whenever it would overflow and once more at the end.
template <int DIM, int KP>
__device__ __noinline__ void ks_offer_chunk(const float *buf, float *rec, float *qinfo, Key<float> *keys, int *cnt_s,
                                            float wmax, int k) {
  using Cfg = KnnSpatial<DIM, KP>;
  using K = Key<float>;
  const int lane = threadIdx.x & 31;
  const unsigned lt_mask = (1u << lane) - 1u;
  const int32_t *idx_plane = reinterpret_cast<const int32_t *>(buf + Cfg::P_IDX * SP_CHUNK);
  uint64_t kth = *reinterpret_cast<const uint64_t *>(qinfo + Cfg::QI_KTH);
  int cnt = *cnt_s;
  // the lane's two runs of four consecutive points: one 16-byte load per array and run
  float qv[DIM];
#pragma unroll
  for (int d = 0; d < DIM; ++d) qv[d] = qinfo[d];
  K cand[8];
  uint32_t lane_min_word = 0xffffffffu;  // smallest distance word of the lane's candidates
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
      const float4 o = *reinterpret_cast<const float4 *>(buf + (Cfg::P_ORG + d) * SP_CHUNK + h * 128 + 4 * lane);
      const float ov[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float diff = __fsub_rn(ov[j], qv[d]);
        acc[j] = __fmaf_rn(diff, diff, acc[j]);
      }
    }
    const int4 id4 = *reinterpret_cast<const int4 *>(idx_plane + h * 128 + 4 * lane);
    const int32_t id[4] = {id4.x, id4.y, id4.z, id4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      // d < 1e10 is the reference's admission test (false for NaN, whatever its sign bit)
      const K c = (id[j] >= 0 && acc[j] < 1e10f) ? K::make(acc[j], (uint32_t)id[j]) : K::empty();
      cand[4 * h + j] = c;
      const uint32_t word = (uint32_t)(c.v >> 32);
      lane_min_word = word < lane_min_word ? word : lane_min_word;
    }
  }
  // Nothing known yet and far more candidates than the queue holds: the k-th smallest of the 32
  // lane minima is an upper bound of the k-th smallest key overall, so it filters first.
  if (KP == 32 && kth == ks_no_bound().v) {
    // non-negative floats order like their bit patterns; an empty key's distance word sorts last
    const uint32_t cap = __shfl_sync(FULL_MASK, warp_sort32_u32(lane_min_word, lane), k - 1);
    // every key with a distance word <= cap; fewer than k lanes with a candidate give an empty cap
    const uint64_t below = cap == 0xffffffffu ? ~0ull : ((uint64_t)cap + 1u) << 32;
    if (below < kth) kth = below;
  }
#pragma unroll
  for (int r = 0; r < 8; ++r) {
    bool hit = cand[r].v < kth;
    unsigned mask = __ballot_sync(FULL_MASK, hit);
    if (mask == 0u) continue;
    int nh = __popc(mask);
    if (cnt + nh > Cfg::QCAP) {
      ks_merge<KP>(keys, cnt, k);
      cnt = 0;
      const K nk = keys[k - 1];  // the k-th best so far (empty while fewer than k are known)
      if (nk.v < kth) kth = nk.v;
      hit = cand[r].v < kth;
      mask = __ballot_sync(FULL_MASK, hit);
      nh = __popc(mask);
    }
    if (hit) keys[KP + cnt + __popc(mask & lt_mask)] = cand[r];
    cnt += nh;
  }
  if (cnt > 0) ks_merge<KP>(keys, cnt, k);
  if (lane == 0) *cnt_s = 0;
  ks_update_bound<DIM, KP>(keys, rec, qinfo, wmax, k, lane);
}

// Arguments of one search.  Graph mode (graph_out != nullptr): the queries are the points themselves
// (yv == xv), k counts the self match, and the final edge rows are written (see knn_finish_graph).
struct KnnSpatialArgs {
  const float *y;      // [m, DIM] original query rows
  SpatialView xv, yv;  // sorted points (with coordinates) / sorted queries (order and keys)
  int num_segments;
  int k;
  int64_t *out_row, *out_col;
  int32_t *counts;
  unsigned long long *num_valid;
  int64_t *graph_out;
  int64_t graph_row_stride, graph_index_base;
  int graph_s2t;
  int *graph_irregular;
  // queue policy: during the first eager_steps scan steps any queued key is merged at once (the bound
  // is still falling fast); later only a queue holding lazy_fill keys is
  int eager_steps, lazy_fill;
  // x-split: thread blocks per query tile, and their lists ([padded query][part][KP] keys) when > 1
  int parts;
  Key<float> *part_keys;
};

// ROLLED: the loop over a warp's eight queries stays a loop; up to three features that variant also runs
// with two ring stages and four thread blocks per SM (ks_four_blocks).  Short segments spend much of their
// time in the selection code and gain from the extra resident warps; long segments live in the scan loop and
// want it unrolled.  Instruction fetch is this kernel's largest stall on short segments, so code size matters
// throughout: the merge network, the push and the chunk offer exist once (noinline), and loops over the
// warp's queries outside the scan stay rolled.
template <int DIM, int KP, bool ROLLED>
__global__ void __launch_bounds__(KS_THREADS, ks_minblocks(DIM, KP, ROLLED))
knn_spatial_kernel(const KnnSpatialArgs a) {
  using Cfg = KnnSpatial<DIM, KP>;
  using K = Key<float>;
  constexpr int QW = Cfg::QW, REC = Cfg::REC, QI = Cfg::QI;
  constexpr int STAGES = ks_stages(DIM, KP, ROLLED);
  using Lay = KnnSpatialLayout<DIM, KP, STAGES>;

  extern __shared__ __align__(128) unsigned char ks_smem_raw[];
  float *stages = reinterpret_cast<float *>(ks_smem_raw);
  uint64_t *full = reinterpret_cast<uint64_t *>(ks_smem_raw + Lay::OFF_BAR);
  uint64_t *empty = full + STAGES;
  float *recs = reinterpret_cast<float *>(ks_smem_raw + Lay::OFF_REC);
  float *qinfos = reinterpret_cast<float *>(ks_smem_raw + Lay::OFF_QI);
  K *keys_all = reinterpret_cast<K *>(ks_smem_raw + Lay::OFF_KEYS);
  int *cnt_all = reinterpret_cast<int *>(ks_smem_raw + Lay::OFF_CNT);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int segs = a.num_segments;
  // With parts > 1 the points of a tile's segment are shared out over `parts` thread blocks: block
  // `part` takes the scan steps part, part + parts, ... of the common outward order and leaves its
  // list for knn_spatial_merge_kernel.
  const int parts = a.parts, part = (int)(blockIdx.x % (unsigned)parts);
  const int64_t pos0 = (int64_t)(blockIdx.x / (unsigned)parts) * KS_TILE;  // first padded query position of this tile
  if (blockIdx.x == 0 && tid == 0 && (*a.xv.bad != 0 || *a.yv.bad != 0)) {
    // segment pointers that overlap: the ordering pass left its layout empty; the result is flagged invalid
    if (a.graph_out != nullptr)
      atomicAdd(a.graph_irregular, KS_ERROR_IRREGULAR);
    else
      atomicAdd(a.num_valid, KS_ERROR_COUNT);
  }
  if (pos0 >= a.yv.sptr[segs]) return;
  int b;
  {
    int lo = 0, hi = segs - 1;
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (a.yv.sptr[mid + 1] > pos0)
        hi = mid;
      else
        lo = mid + 1;
    }
    b = lo;
  }
  const int64_t xs_lo = a.xv.sptr[b];
  const int nch_all = (int)((a.xv.sptr[b + 1] - xs_lo) / SP_CHUNK);
  const int nch = nch_all > part ? (nch_all - part + parts - 1) / parts : 0;  // scan steps of this block
  const float wmax = __uint_as_float(a.xv.stat[2 * b]);
  const bool screen = wmax < 1e30f;  // false also for NaN

  const bool producer = warp == KS_WARPS;  // the ninth warp only moves chunks
  const int cwarp = producer ? 0 : warp;
  float *my_recs = recs + cwarp * QW * REC;
  float *my_qi = qinfos + cwarp * QW * QI;
  K *my_keys = keys_all + (size_t)cwarp * QW * (KP + Cfg::QCAP);
  int *my_cnt = cnt_all + cwarp * 2 * QW;  // [QW] queue fill, [QW] fill before the current chunk
  int *my_mark = my_cnt + QW;

  // ---- queries of this warp: padded positions pos0 + warp + 8 qi; lane qi prepares query qi ----
  int64_t my_row = -1;  // lane qi < QW: original row of query qi, -1 for padding
  if (lane < QW && !producer) {
    my_row = a.yv.idx[pos0 + warp + KS_WARPS * lane];
    float *rec = my_recs + lane * REC, *qi = my_qi + lane * QI;
    const float *box = a.xv.box + (int64_t)b * 2 * DIM;
    if (my_row >= 0) {
      float nq2 = 0.f;
#pragma unroll
      for (int d = 0; d < DIM; ++d) {
        const float q = a.y[my_row * DIM + d];
        const float qc = q - (0.5f * box[d] + 0.5f * box[DIM + d]);
        qi[d] = q;
        rec[2 * d] = -2.f * qc;
        rec[2 * d + 1] = -2.f * qc;
        nq2 = __fmaf_rn(qc, qc, nq2);
      }
      qi[DIM] = nq2;
      *reinterpret_cast<uint64_t *>(qi + Cfg::QI_KTH) = ks_no_bound().v;
      rec[2 * DIM] = ((1e10f - nq2) + KS_MARGIN * (1e10f + nq2 + wmax)) + KS_MARGIN_ABS;
    } else {
#pragma unroll
      for (int d = 0; d < DIM; ++d) {
        qi[d] = 0.f;
        rec[2 * d] = 0.f;
        rec[2 * d + 1] = 0.f;
      }
      qi[DIM] = 0.f;
      *reinterpret_cast<uint64_t *>(qi + Cfg::QI_KTH) = 0ull;  // no key is below it
      rec[2 * DIM] = -__int_as_float(0x7f800000);              // nothing is below -inf
    }
    my_cnt[lane] = 0;
    my_mark[lane] = 0;
  }
  const unsigned valid_mask = __ballot_sync(FULL_MASK, lane < QW && my_row >= 0);
  if (!producer) {
#pragma unroll 1
    for (int qi = 0; qi < QW; ++qi) knn_reset<float, KP>(my_keys + qi * (KP + Cfg::QCAP), lane);
  }

  // ---- first chunk: the one around the tile's queries ----
  int seed = 0;
  if (nch_all > 0) {
    if (a.yv.idx == a.xv.idx) {
      seed = (int)((pos0 - xs_lo) / SP_CHUNK);  // the queries are these points
    } else {
      // the sorted points are bisected for the key of the tile's middle query
      uint32_t key = a.yv.key[pos0 + KS_TILE / 2];
      if (key == 0xffffffffu) key = a.yv.key[pos0];
      const uint32_t *xk = a.xv.key + xs_lo;
      int lo = 0, hi = nch_all * SP_CHUNK;
      while (lo < hi) {
        const int m2 = (lo + hi) >> 1;
        if (xk[m2] < key)
          lo = m2 + 1;
        else
          hi = m2;
      }
      seed = lo / SP_CHUNK;
    }
    if (seed > nch_all - 1) seed = nch_all - 1;
  }

  // ---- stage ring ----
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(ks_smem(full + s)) : "memory");
      asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(ks_smem(empty + s)), "r"(KS_WARPS)
                   : "memory");
    }
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
  }
  __syncthreads();

  auto issue = [&](int step) {  // thread 0: bulk copies of the chunk of scan step `step`
    const int slot = step % STAGES;
    const int64_t pos = xs_lo + (int64_t)ks_chunk_at(part + step * parts, seed, nch_all) * SP_CHUNK;
    float *dst = stages + slot * Cfg::STAGE_ELEMS;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(ks_smem(full + slot)),
                 "r"(Cfg::STAGE_BYTES)
                 : "memory");
    // the chunk's arrays lie back to back in the sorted copy, in the order of the stage: one copy
    ks_bulk_load(dst, a.xv.blob + (pos / SP_CHUNK) * Cfg::STAGE_ELEMS, Cfg::STAGE_BYTES, full + slot);
  };

  bool failed = false;
  if (producer) {
    // ---- the copy warp: one lane keeps the ring full; a slot is refilled once all scanning warps
    // have released it ----
    if (lane == 0) {
      int issued = 0;
      for (int step = 0; step < nch && !failed; ++step) {
        if (step >= STAGES && !ks_wait(empty + step % STAGES, (unsigned)((step / STAGES - 1) & 1))) {
          failed = true;
          break;
        }
        issue(step);
        issued = step + 1;
      }
      if (failed) {
        // a wait ran out: flag the result as invalid and let the copies already issued land
        for (int s = issued > STAGES ? issued - STAGES : 0; s < issued; ++s)
          (void)ks_wait(full + s % STAGES, (unsigned)((s / STAGES) & 1));
        if (a.graph_out != nullptr)
          atomicAdd(a.graph_irregular, KS_ERROR_IRREGULAR);
        else
          atomicAdd(a.num_valid, KS_ERROR_COUNT);
      }
    }
    return;
  }

  for (int step = 0; step < nch; ++step) {
    const int slot = step % STAGES;
    if (!ks_wait(full + slot, (unsigned)((step / STAGES) & 1))) {
      failed = true;
      break;
    }
    const float *buf = stages + slot * Cfg::STAGE_ELEMS;

    if (screen && step > 0) {
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
        const float4 v = *reinterpret_cast<const float4 *>(buf + Cfg::P_W * SP_CHUNK + h * 128 + 4 * lane);
        pw[2 * h] = make_float2(v.x, v.y);
        pw[2 * h + 1] = make_float2(v.z, v.w);
      }
      auto screen_query = [&](int qi) {
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
        if (m <= f[2 * DIM])
          ks_push<DIM, KP>(s[0].x, s[0].y, s[1].x, s[1].y, s[2].x, s[2].y, s[3].x, s[3].y, buf, rec, my_qi + qi * QI,
                           my_keys + qi * (KP + Cfg::QCAP) + KP, my_cnt + qi);
      };
      // The loop over the warp's queries only notes — one vote per query — which of them have a point at or
      // below their threshold in this chunk; those are screened again afterwards with the push attached.  The
      // loop that does the bulk of the work then holds no call, no convergence bracket and no screen values
      // that outlive their minimum (long segments: 2.43 -> 2.20 ms on 8 x (131072 points, 8192 queries);
      // clouds of 4096 / 8192 points: 1.5 % / 5 % faster, of 2048 points 2 % slower).
      auto note_query = [&](int qi) -> bool {
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
        const float m0 = fminf(fminf(s[0].x, s[0].y), s[1].x), m1 = fminf(fminf(s[1].y, s[2].x), s[2].y);
        const float m = fminf(fminf(m0, m1), fminf(s[3].x, s[3].y));
        return __any_sync(FULL_MASK, m <= f[2 * DIM]) != 0;
      };
      unsigned noted = 0u;
      if constexpr (ROLLED) {
#pragma unroll 1
        for (int qi = 0; qi < QW; ++qi)
          if (note_query(qi)) noted |= 1u << qi;
      } else {
#pragma unroll
        for (int qi = 0; qi < QW; ++qi)
          if (note_query(qi)) noted |= 1u << qi;
      }
      // no noted query: no queue has changed in this chunk, and long segments (where that is the rule) skip the
      // look at the queues; on short ones the extra test costs more than it saves (measured: 3 % either way)
      const bool pushed = ROLLED || noted != 0u;
      while (noted) {
        const int qi = __ffs(noted) - 1;
        noted &= noted - 1u;
        screen_query(qi);
      }
      __syncwarp();
      // the queues after this chunk: overflowed ones are rolled back and the chunk offered again by
      // the whole warp; filled ones are merged, which tightens the bound
      const int fill = (pushed && lane < QW) ? my_cnt[lane] : 0;
      const int want = step < a.eager_steps ? 1 : a.lazy_fill;
      unsigned todo = pushed ? __ballot_sync(FULL_MASK, fill >= want) : 0u;
      const unsigned over = pushed ? __ballot_sync(FULL_MASK, fill > Cfg::QCAP) : 0u;
      while (todo) {
        const int qi = __ffs(todo) - 1;
        todo &= todo - 1u;
        K *keys = my_keys + qi * (KP + Cfg::QCAP);
        if ((over >> qi) & 1u) {
          if (lane == 0) my_cnt[qi] = my_mark[qi];
          __syncwarp();
          ks_offer_chunk<DIM, KP>(buf, my_recs + qi * REC, my_qi + qi * QI, keys, my_cnt + qi, wmax, a.k);
        } else {
          ks_merge<KP>(keys, my_cnt[qi], a.k);
          if (lane == 0) my_cnt[qi] = 0;
          ks_update_bound<DIM, KP>(keys, my_recs + qi * REC, my_qi + qi * QI, wmax, a.k, lane);
        }
      }
      if (pushed && lane < QW) my_mark[lane] = my_cnt[lane];
    } else {
      for (int qi = 0; qi < QW; ++qi)
        if ((valid_mask >> qi) & 1u)
          ks_offer_chunk<DIM, KP>(buf, my_recs + qi * REC, my_qi + qi * QI, my_keys + qi * (KP + Cfg::QCAP),
                                  my_cnt + qi, wmax, a.k);
    }
    __syncwarp();
    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(ks_smem(empty + slot)) : "memory");
  }

  if (failed) {
    // a wait of this warp ran out: nothing of its queries is written, the result is flagged invalid
    if (lane == 0) {
      if (a.graph_out != nullptr)
        atomicAdd(a.graph_irregular, KS_ERROR_IRREGULAR);
      else
        atomicAdd(a.num_valid, KS_ERROR_COUNT);
    }
    return;
  }

  // ---- output ----
  if (parts > 1) {
    // this block's list of every query, sorted, KP keys each, for the merge kernel
#pragma unroll 1
    for (int qi = 0; qi < QW; ++qi) {
      K *keys = my_keys + qi * (KP + Cfg::QCAP);
      if (my_cnt[qi] > 0) ks_merge<KP>(keys, my_cnt[qi], a.k);
      K *dst = a.part_keys + ((pos0 + warp + KS_WARPS * qi) * parts + part) * KP;
      for (int e = lane; e < KP; e += 32) dst[e] = keys[e];
    }
    return;
  }
  // A loop, and the last merge through the shared copy of the network: the kernel's code stays small
  // (with this loop unrolled and the merges inline, eight more copies of the network, the scan of
  // clouds of 4096 points took 0.544 ms instead of 0.471 ms — instruction fetch).
  int my_valid = 0, my_irregular = 0;
#pragma unroll 1
  for (int qi = 0; qi < QW; ++qi) {
    const int64_t q = __shfl_sync(FULL_MASK, my_row, qi);
    if (q < 0) continue;  // warp-uniform
    K *keys = my_keys + qi * (KP + Cfg::QCAP);
    if (my_cnt[qi] > 0) ks_merge<KP>(keys, my_cnt[qi], a.k);
    if (a.graph_out != nullptr) {
      if (!knn_finish_graph<float, KP>(keys, 0, a.k, q, a.graph_row_stride, a.graph_index_base, a.graph_out,
                                       a.graph_s2t != 0, lane))
        ++my_irregular;
      continue;
    }
    const int valid = knn_finish<float, KP>(keys, 0, a.k, q, a.out_row, a.out_col, lane);
    if (lane == 0) {
      a.counts[q] = valid;
      my_valid += valid;
    }
  }
  if (lane == 0 && my_valid) atomicAdd(a.num_valid, (unsigned long long)my_valid);
  if (lane == 0 && my_irregular) atomicAdd(a.graph_irregular, my_irregular);
}

// Merges the `parts` lists of every query that an x-split scan left and writes the output as the scan
// kernel itself would have: one warp per padded query position.
template <int KP>
__global__ void __launch_bounds__(CTA_THREADS)
knn_spatial_merge_kernel(const KnnSpatialArgs a, int64_t padded_queries) {
  using K = Key<float>;
  __shared__ K keys_s[WARPS_PER_CTA][2 * KP];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t qpos = (int64_t)blockIdx.x * WARPS_PER_CTA + warp;
  int my_valid = 0, my_irregular = 0;
  if (qpos < padded_queries && qpos < a.yv.sptr[a.num_segments]) {
    const int64_t q = a.yv.idx[qpos];
    if (q >= 0) {
      K *keys = keys_s[warp];
      const K *src = a.part_keys + qpos * a.parts * KP;
      for (int e = lane; e < KP; e += 32) keys[e] = src[e];
      for (int p = 1; p < a.parts; ++p) {
        for (int e = lane; e < KP; e += 32) keys[KP + e] = src[(int64_t)p * KP + e];
        knn_merge<float, KP>(keys, KP, a.k, lane);  // empty keys sort to the end
      }
      __syncwarp();
      if (a.graph_out != nullptr) {
        if (!knn_finish_graph<float, KP>(keys, 0, a.k, q, a.graph_row_stride, a.graph_index_base, a.graph_out,
                                         a.graph_s2t != 0, lane))
          ++my_irregular;
      } else {
        const int valid = knn_finish<float, KP>(keys, 0, a.k, q, a.out_row, a.out_col, lane);
        if (lane == 0) {
          a.counts[q] = valid;
          my_valid = valid;
        }
      }
    }
  }
  if (lane == 0 && my_valid) atomicAdd(a.num_valid, (unsigned long long)my_valid);
  if (lane == 0 && my_irregular) atomicAdd(a.graph_irregular, my_irregular);
}

}  // namespace b200c
