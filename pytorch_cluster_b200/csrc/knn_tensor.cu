// Feature-space kNN (fp32, 32 <= D <= 128, D % 8 == 0, k <= 32): tensor-core candidates, exact re-rank.
//
// Stage 1, knn_tensor_candidates_kernel — tcgen05 / TMEM.  A CTA of 512 threads owns 128 query rows.
// The query tile and a ring of two 128-point tiles of the queries' segment are laid out in shared
// memory in the K-major, 128-byte-swizzled operand layout of the 5th-generation tensor cores (rows
// of 32 tf32 values = 128 bytes, 16-byte chunk c of row r stored at chunk c ^ (r & 7); cp.async, 16
// bytes per copy, coalesced on the global side and conflict-free on the shared side).  One thread
// issues D / 8 `tcgen05.mma.cta_group::1.kind::tf32` instructions (M = 128, N = 128, K = 8) per tile
// that accumulate S = Q X^T into one of two 128-column accumulators in tensor memory;
// `tcgen05.commit` signals that accumulator's mbarrier.  The loop is software-pipelined: while the
// tensor core works on tile s, the threads read back tile s - 1 from the other accumulator with
// `tcgen05.ld.32x32b` (four threads per query row, 32 columns each) and the copies of tile s + 1
// are in flight.  From S the approximate distance a = |x|^2 - 2 S + |q|^2 (or 1 - S on
// pre-normalised rows for cosine) costs one FFMA per pair.  The segment is swept twice:
//   pass A keeps, per query, the minimum of a over groups of points (at most 64 groups, 16 per
//          thread).  The k-th smallest of those minima, T, is an upper bound of the k-th smallest
//          approximate distance: k different points lie at or below it.
//   pass B records every point with a <= T + 2 E as a candidate of that query (two lists per
//          query, each filled by one thread from the front and by another from the back), E being a bound of |a - d_exact| for
//          tf32 operands (each truncated to 10 mantissa bits: |dS| <= 2^-9 |x||q|).  If d_k is the
//          exact k-th distance, then d_k <= T + E, so every true neighbour (d <= d_k) has
//          a <= T + 2 E: no neighbour is lost.
// Stage 2, knn_rerank_kernel — one warp per query evaluates its candidates exactly as the
// reference does (sequential fused multiply-adds over ascending features,
// csrc/cuda/knn_cuda.cu:9-28, 55-64) and selects the k best by (distance, index) with the
// selection of select.cuh.  A query whose candidate list overflowed (or whose segment is too
// short to give k group minima) is searched exhaustively by its warp instead.  Only exact
// distances are compared, so the result equals the exact kernels' bit for bit.
//
// Every wait on the mbarrier is bounded; on expiry the CTA raises an error flag and the re-rank
// kernel searches every query exhaustively instead of trusting the candidate lists.
#include "common.cuh"
#include "launchers.h"
#include "select.cuh"

namespace b200c {

constexpr int TC_M = 128;        // queries per CTA = TMEM lanes
constexpr int TC_N = 128;        // points per tile = TMEM columns
constexpr int TC_PARTS = 4;      // threads per query row: each reads back 32 of a tile's 128 columns
constexpr int TC_COLS = TC_N / TC_PARTS;
constexpr int TC_GH = 16;        // group minima kept per thread: 64 per query
constexpr int TC_CAP = 128;      // candidates kept per query: two lists of 64, each filled from both ends
constexpr int TC_THREADS = TC_M * TC_PARTS;
constexpr int TC_SPIN_LIMIT = 1 << 22;
// Point tiles held in shared memory.  The kernel also runs with 4 (they fit up to 64 features), but three
// tiles of look-ahead measured slower than one on 16 x 2048 x 64 (148 us against 129 us): the step is
// not waiting for its copies.
constexpr int TC_RING = 2;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Shared-memory matrix descriptor, K-major, 128-byte swizzle: start address, stride byte offset
// 1024 (8 rows of 128 bytes), leading byte offset unused, descriptor version 1, layout type 2.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3fffu);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024u >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

__device__ __forceinline__ void cp_async_16(void *smem_dst, const void *gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}

// Rows [row0, row0 + 128) of src ([*, dim] row-major) into the swizzled operand layout: features
// [32 a, 32 a + 32) of all rows form "atom" a (128 rows x 128 bytes = 16 KiB); inside an atom the
// 16-byte chunk c of row r sits at r * 128 + ((c ^ (r & 7)) * 16).  Rows >= row_end are zero.
// Consecutive threads copy consecutive chunks of a row (coalesced 16-byte loads).  When the
// number of chunks per row divides the thread count (dim = 32, 64, 128) a thread keeps its chunk
// and walks down the rows in steps that are multiples of 8, so its swizzle term is constant and
// the addresses advance by constants; other dims pay an integer division per copy.
__device__ __forceinline__ void stage_operand(unsigned char *dst, const float *__restrict__ src, int64_t row0,
                                              int64_t row_end, int dim, int tid) {
  const int chunks = dim >> 2;  // 16-byte chunks per row
  if ((chunks & (chunks - 1)) == 0) {
    const int ch = tid & (chunks - 1);
    const int r0 = tid / chunks;            // chunks is a power of two: a shift
    const int rstep = TC_THREADS / chunks;  // 32, 16 or 8
    unsigned char *d = dst + (ch >> 3) * 16384 + r0 * 128 + (((ch & 7) ^ (r0 & 7)) << 4);
    const float *g = src + (row0 + r0) * dim + ch * 4;
    int64_t row = row0 + r0;
    for (int r = r0; r < TC_M; r += rstep) {
      if (row < row_end)
        cp_async_16(d, g);
      else
        *reinterpret_cast<float4 *>(d) = make_float4(0.f, 0.f, 0.f, 0.f);
      d += rstep * 128;
      g += (int64_t)rstep * dim;
      row += rstep;
    }
    return;
  }
  for (int p = tid; p < TC_M * chunks; p += TC_THREADS) {
    const int row = p / chunks, ch = p - row * chunks;
    unsigned char *d = dst + (ch >> 3) * 16384 + row * 128 + (((ch & 7) ^ (row & 7)) << 4);
    const int64_t g = row0 + row;
    if (g < row_end)
      cp_async_16(d, src + g * dim + ch * 4);
    else
      *reinterpret_cast<float4 *>(d) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Waits for phase `parity` of the mbarrier with a bounded number of polls.
__device__ __forceinline__ bool mbar_wait(uint64_t *mbar, uint32_t parity) {
  uint32_t done = 0;
  for (int it = 0; it < TC_SPIN_LIMIT && !done; ++it) {
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
        : "=r"(done)
        : "r"(smem_u32(mbar)), "r"(parity)
        : "memory");
  }
  return done != 0;
}

__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,"
      "%28,%29,%30,%31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
        "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
        "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Ascending bitonic sort of 64 values held in registers (all indices are compile-time constants).
__device__ __forceinline__ void sort64(float (&v)[64]) {
#pragma unroll
  for (int size = 2; size <= 64; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
#pragma unroll
      for (int i = 0; i < 64; ++i) {
        const int l = i ^ stride;
        if (l > i) {
          const float lo = fminf(v[i], v[l]), hi = fmaxf(v[i], v[l]);
          const bool asc = (i & size) == 0;
          v[i] = asc ? lo : hi;
          v[l] = asc ? hi : lo;
        }
      }
    }
  }
}

// Group minima of a CTA: 64 per query row, row r's entry c stored at r * 64 + (c ^ (r & 31)), so that
// both the writers (consecutive rows, same c) and the readers (one row, consecutive c) hit 32
// different banks.
__device__ __forceinline__ int gmin_slot(int row, int c) { return row * 64 + (c ^ (row & 31)); }

// Ascending merge of a bitonic sequence of 32-bit values held one per lane.
__device__ __forceinline__ uint32_t warp_bitonic_merge32_u32(uint32_t v, int lane) {
#pragma unroll
  for (int stride = 16; stride > 0; stride >>= 1) {
    const uint32_t o = __shfl_xor_sync(FULL_MASK, v, stride);
    v = ((o < v) == ((lane & stride) == 0)) ? o : v;
  }
  return v;
}

struct TensorArgs {
  const float *xa, *ya;        // operands of the product: x, y (L2) or their normalised copies (cosine)
  const float *sq_x, *sq_y;    // L2: |row|^2 ; cosine: unused
  const float *xmax;           // L2: largest |x| over all rows (one float)
  const int64_t *ptr_x, *ptr_y;
  int num_segments;
  int64_t n, m;
  int dim, k;
  int32_t *cand;               // [m, TC_CAP]
  int32_t *cand_count;         // [m]; four 8-bit counts: list A front, A back, list B front, B back
  int *error_flag;
};

template <bool COSINE>
__global__ void __launch_bounds__(TC_THREADS, 1) knn_tensor_candidates_kernel(TensorArgs a) {
  // The 128-byte swizzle works on absolute shared-memory address bits, so the operand tiles must
  // start on a 1024-byte boundary.  The declared alignment of an extern array is shared by every
  // kernel of the translation unit that names it, so the base is aligned by hand instead (the
  // launch reserves 1024 bytes of slack).
  extern __shared__ unsigned char smem_tensor_raw[];
  unsigned char *smem = smem_tensor_raw + ((1024u - (smem_u32(smem_tensor_raw) & 1023u)) & 1023u);
  const int dim = a.dim;
  const uint32_t tile_bytes = (uint32_t)((dim + 31) >> 5) * 16384u;  // whole atoms of 32 features
  unsigned char *sQ = smem;
  constexpr int ring = TC_RING, ahead = ring - 1, sqx_slots = ring + 1;
  unsigned char *sX = smem + tile_bytes;                                      // ring of point tiles
  float *s_sqx = reinterpret_cast<float *>(smem + (1 + ring) * tile_bytes);   // |x|^2 per column, ring + 1 tiles
  float *gmin = s_sqx + sqx_slots * TC_N;                                     // [TC_M][64] group minima, see gmin_slot
  __shared__ __align__(8) uint64_t mbar[2];
  __shared__ uint32_t tmem_base_s;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int row = tid & (TC_M - 1);  // the query this thread reads back (TMEM lane)
  const int part = tid >> 7;         // which 32 of a tile's 128 columns it reads
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[0])));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar[1])));
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)),
                 "r"(2 * TC_N));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_base_s;
  // a warp reaches the 32 TMEM lanes of its quarter (warp index mod 4)
  const uint32_t my_taddr = tmem + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(part * TC_COLS);
  // D = f32, A = B = tf32, both K-major, N >> 3 at bit 17, M >> 4 at bit 24
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(TC_N >> 3) << 17) |
                         ((uint32_t)(TC_M >> 4) << 24);
  uint32_t phase0 = 0u, phase1 = 0u;  // parity of the next completion of each accumulator's mbarrier
  bool ok = true, failed = false;

  const int64_t tile_lo = (int64_t)blockIdx.x * TC_M;
  const int64_t tile_hi = tile_lo + TC_M < a.m ? tile_lo + TC_M : a.m;
  const int b_first = segment_of(a.ptr_y, a.num_segments, tile_lo);
  const int b_last = segment_of(a.ptr_y, a.num_segments, tile_hi - 1);
  const float xmax = COSINE ? 1.f : *a.xmax;

  for (int b = b_first; b <= b_last && !failed; ++b) {
    int64_t y_lo, y_hi, x_lo, x_hi;
    segment_rows(a.ptr_y, a.num_segments, a.m, b, y_lo, y_hi);
    const int64_t q_lo = y_lo > tile_lo ? y_lo : tile_lo;
    const int64_t q_hi = y_hi < tile_hi ? y_hi : tile_hi;
    if (q_lo >= q_hi) continue;
    segment_points(a.ptr_x, a.n, b, x_lo, x_hi);
    const int64_t nx = x_hi > x_lo ? x_hi - x_lo : 0;
    const int64_t q = q_lo + row;
    const bool have_q = q < q_hi;
    if (nx == 0) continue;  // the candidate counts were zeroed before the launch

    // A thread meets 32 columns of every tile; it groups that stream into at most TC_GH groups of
    // `gs` columns (a multiple of 32).  The four threads of a query hold at most 64 group minima.
    const int ntiles = (int)((nx + TC_N - 1) / TC_N);
    const int64_t own = (int64_t)ntiles * TC_COLS;
    const int gs = (int)(((own + TC_GH - 1) / TC_GH + 31) / 32 * 32);

    // Everything is compared in "shifted" form a' = bias_x + scale * S, i.e. the approximate distance
    // minus the query's own constant (|q|^2 for L2, 1 for cosine): bias_x = |x|^2 or 0, +inf for
    // columns past the segment's end; scale = -2 or -1.  err bounds |a' - (d_exact - constant)|.
    const float scale = COSINE ? -1.f : -2.f;
    float err = 0.00390625f * 1.05f + 1e-6f;  // cosine: 2 * 2^-9 on unit vectors, plus slack
    if (!COSINE && have_q) {
      const float qsq = a.sq_y[q];
      err = 0.00390625f * 1.05f * sqrtf(qsq) * xmax + 4e-6f * (xmax * xmax + qsq);
    }

    // Software pipeline over the 2 * ntiles steps (pass A then pass B over the same tiles): in
    // iteration s the tensor core works on step s while the threads read back step s - 1 and the
    // copies of steps s + 1 .. s + ring - 1 are in flight.  Point tile of step s: ring slot
    // s % ring; accumulator: TMEM columns (s & 1) * 128 ..; |x|^2 of its columns: slot
    // s % (ring + 1).  Every iteration commits exactly one copy group (possibly empty), so that
    // "all but the newest ring - 2 groups" always means "step s has landed".
    const int nsteps = 2 * ntiles;
    auto stage_step = [&](int step) {
      if (step < nsteps) {
        const int t1 = step < ntiles ? step : step - ntiles;
        const int64_t p1 = x_lo + (int64_t)t1 * TC_N;
        stage_operand(sX + (uint32_t)(step % ring) * tile_bytes, a.xa, p1, x_hi, dim, tid);
        if (tid < TC_N)
          s_sqx[(step % sqx_slots) * TC_N + tid] =
              p1 + tid < x_hi ? (COSINE ? 0.f : a.sq_x[p1 + tid]) : pos_inf<float>();
      }
      asm volatile("cp.async.commit_group;\n" ::: "memory");
    };
    stage_operand(sQ, a.ya, q_lo, q_hi, dim, tid);  // joins the first point tile's copy group
    for (int step = 0; step < ahead; ++step) stage_step(step);

    float thr = 0.f, run_min = pos_inf<float>();
    int group = 0, in_group = 0, ncand = 0;
    for (int s = 0; s <= nsteps; ++s) {
      if (s < nsteps) {
        if constexpr (ahead == 1)
          asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        else
          asm volatile("cp.async.wait_group 2;\n" ::: "memory");
        static_assert(ahead == 1 || ahead == 3, "the wait above names the number of groups that may stay in flight");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> tensor-core reads
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      // step s is in place; everyone has finished reading the accumulator of step s - 2; and one
      // decision for the whole CTA if some wait ran out
      if (__syncthreads_or(!ok)) {
        failed = true;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (s < nsteps && tid == 0) {
        const uint32_t sx = smem_u32(sX) + (uint32_t)(s % ring) * tile_bytes;
        const uint32_t acc = tmem + (uint32_t)(s & 1) * TC_N;
        for (int ks = 0; ks < (dim >> 3); ++ks) {
          const uint32_t off = (uint32_t)(ks >> 2) * 16384u + (uint32_t)(ks & 3) * 32u;
          const uint64_t da = umma_desc_sw128(smem_u32(sQ) + off);
          const uint64_t db = umma_desc_sw128(sx + off);
          const uint32_t accumulate = ks > 0 ? 1u : 0u;
          asm volatile(
              "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
              "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n}"
              ::"r"(acc), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
              : "memory");
        }
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     ::"r"(smem_u32(&mbar[s & 1]))
                     : "memory");
      }
      if (s >= 1) {
        const int pb = (s - 1) & 1;
        // step s - 1 is complete: its tile may be overwritten.  One answer per warp: the read-back
        // below is a warp-wide instruction
        ok = __all_sync(FULL_MASK, mbar_wait(&mbar[pb], pb ? phase1 : phase0));
        if (pb)
          phase1 ^= 1u;
        else
          phase0 ^= 1u;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      // the slot of step s - 1 is free again: it takes step s + ring - 1
      if (ok) stage_step(s + ahead);
      if (s >= 1 && ok) {
        // read back step s - 1: this thread's 32 columns of its query's row
        const int e = s - 1;
        const int pass = e >= ntiles ? 1 : 0;
        const int t = e - pass * ntiles;
        const int64_t p0 = x_lo + (int64_t)t * TC_N + part * TC_COLS;
        const float *sqx = s_sqx + (e % sqx_slots) * TC_N + part * TC_COLS;
        uint32_t v[32];
        tmem_load32(my_taddr + (uint32_t)(e & 1) * TC_N, v);
        constexpr int c0 = 0;
        if (p0 < x_hi) {  // else: a block past the segment's end
          if (pass == 0) {
            // four independent chains, so that the minimum does not wait on itself
            float m0 = run_min, m1 = pos_inf<float>(), m2 = m1, m3 = m1;
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const float4 bx = *reinterpret_cast<const float4 *>(sqx + c0 + 4 * j4);
              m0 = fminf(m0, __fmaf_rn(scale, __uint_as_float(v[4 * j4 + 0]), bx.x));
              m1 = fminf(m1, __fmaf_rn(scale, __uint_as_float(v[4 * j4 + 1]), bx.y));
              m2 = fminf(m2, __fmaf_rn(scale, __uint_as_float(v[4 * j4 + 2]), bx.z));
              m3 = fminf(m3, __fmaf_rn(scale, __uint_as_float(v[4 * j4 + 3]), bx.w));
            }
            run_min = fminf(fminf(m0, m1), fminf(m2, m3));
            in_group += 32;
            if (in_group >= gs) {
              gmin[gmin_slot(row, part * TC_GH + group)] = run_min;
              ++group;
              run_min = pos_inf<float>();
              in_group = 0;
            }
          } else {
            // one bit per column that passes, without branches; the few set bits are walked after
            uint32_t hits = 0u;
#pragma unroll
            for (int j4 = 0; j4 < 8; ++j4) {
              const float4 bx = *reinterpret_cast<const float4 *>(sqx + c0 + 4 * j4);
              hits |= (__fmaf_rn(scale, __uint_as_float(v[4 * j4 + 0]), bx.x) <= thr ? 1u : 0u) << (4 * j4 + 0);
              hits |= (__fmaf_rn(scale, __uint_as_float(v[4 * j4 + 1]), bx.y) <= thr ? 1u : 0u) << (4 * j4 + 1);
              hits |= (__fmaf_rn(scale, __uint_as_float(v[4 * j4 + 2]), bx.z) <= thr ? 1u : 0u) << (4 * j4 + 2);
              hits |= (__fmaf_rn(scale, __uint_as_float(v[4 * j4 + 3]), bx.w) <= thr ? 1u : 0u) << (4 * j4 + 3);
            }
            while (hits != 0u) {
              const int j = __ffs(hits) - 1;
              hits &= hits - 1u;
              // threads 0 and 1 of a query share the first half of its list, 2 and 3 the second;
              // one fills its half from the front, the other from the back: no atomics, no
              // waiting on the stores
              if (ncand < TC_CAP / 2 && have_q)
                a.cand[q * TC_CAP + (part >> 1) * (TC_CAP / 2) + ((part & 1) ? TC_CAP / 2 - 1 - ncand : ncand)] =
                    (int32_t)(p0 + c0 + j);
              ++ncand;
            }
          }
        }
      }
      if (s == ntiles) {
        // pass A is read back: the k-th smallest of the query's group minima (this thread's and
        // its partner's) bounds the k-th smallest approximate distance — k different points lie
        // at or below it
        if (in_group > 0) gmin[gmin_slot(row, part * TC_GH + group++)] = run_min;
        for (int g = group; g < TC_GH; ++g) gmin[gmin_slot(row, part * TC_GH + g)] = pos_inf<float>();
        __syncthreads();
        // every warp selects for 8 rows: 64 values as two per lane, two warp sorts, the 32 smallest
        // of both by one bitonic merge (k <= 32), compared as order-preserving integers
        const int lane = tid & 31;
        for (int r = warp * (TC_M / (TC_THREADS / 32)); r < (warp + 1) * (TC_M / (TC_THREADS / 32)); ++r) {
          uint32_t lo = warp_sort32_u32(ordered_bits(gmin[gmin_slot(r, lane)]), lane);
          const uint32_t hi = warp_sort32_u32(ordered_bits(gmin[gmin_slot(r, lane + 32)]), lane);
          const uint32_t rev = __shfl_sync(FULL_MASK, hi, 31 - lane);
          lo = warp_bitonic_merge32_u32(rev < lo ? rev : lo, lane);
          const uint32_t kb = __shfl_sync(FULL_MASK, lo, a.k - 1);
          if (lane == 0) gmin[r * 64] = from_ordered_bits(kb);  // the row's minima are consumed: reuse its first word
        }
        __syncthreads();
        const float kth = gmin[row * 64];
        thr = kth + 2.f * err;
        // NaN, infinite, or fewer than k non-empty groups (their minima are +inf): keep every real
        // column; padding columns are +inf and still fail the comparison
        if (!(thr < 3.0e38f)) thr = 3.0e38f;
      }
    }
    // the four counts of a query in one word (zeroed before the launch), 8 bits each; a count
    // beyond a list's capacity is stored as capacity + 1, so that the pair's sum still says "overflow"
    if (have_q && !failed) {
      const int c = ncand < TC_CAP / 2 + 1 ? ncand : TC_CAP / 2 + 1;
      atomicAdd(&a.cand_count[q], c << (8 * part));
    }
    __syncthreads();  // every read-back of this segment is done before the buffers are restaged
  }
  if (failed && tid == 0) *a.error_flag = 1;

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * TC_N));
}

// ---- exact re-rank: one warp per query ---------------------------------------------------------------------
constexpr int RR_WARPS = 4;

template <bool COSINE>
__global__ void __launch_bounds__(RR_WARPS * 32)
knn_rerank_kernel(const float *__restrict__ x, const float *__restrict__ y, const int64_t *__restrict__ ptr_x,
                  const int64_t *__restrict__ ptr_y, int num_segments, int64_t n, int64_t m, int dim, int k,
                  const float *__restrict__ norms_x, const float *__restrict__ norms_y,
                  const int32_t *__restrict__ cand, const int32_t *__restrict__ cand_count,
                  const int *__restrict__ error_flag, int64_t *__restrict__ out_row, int64_t *__restrict__ out_col,
                  int32_t *__restrict__ counts, unsigned long long *__restrict__ num_valid,
                  int64_t *__restrict__ graph_out, int64_t graph_row_stride, int64_t graph_index_base, int graph_s2t,
                  int *__restrict__ graph_irregular) {
  // graph_out != nullptr: knn_graph output (see knn_finish_graph in select.cuh) instead of the padded rows:
  // the k - 1 neighbours other than the query itself straight into the final edge rows; queries that do not
  // have that shape are counted in *graph_irregular and write nothing.
  using K = Key<float>;
  constexpr int KP = 32;
  extern __shared__ __align__(16) unsigned char smem_rerank[];
  unsigned char *smem = smem_rerank;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // per warp: query row (dim floats, padded to 4), 2 * KP keys, queue fill
  const int qstride = (dim + 3) & ~3;
  float *my_q = reinterpret_cast<float *>(smem) + warp * qstride;
  K *my_keys = reinterpret_cast<K *>(smem + (size_t)RR_WARPS * qstride * 4) + warp * 2 * KP;
  int *my_cnt = reinterpret_cast<int *>(smem + (size_t)RR_WARPS * qstride * 4 + (size_t)RR_WARPS * 2 * KP * sizeof(K)) + warp;

  const int64_t q = (int64_t)blockIdx.x * RR_WARPS + warp;
  if (q >= m) return;
  const int b = segment_of(ptr_y, num_segments, q);
  int64_t x_lo, x_hi;
  segment_points(ptr_x, n, b, x_lo, x_hi);

  for (int d = lane; d < dim; d += 32) my_q[d] = y[q * dim + d];
  knn_reset<float, KP>(my_keys, lane);
  if (lane == 0) *my_cnt = 0;
  __syncwarp();
  const float ny = COSINE ? norms_y[q] : 1.f;
  const bool vec4 = (dim & 3) == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;  // rows are whole float4s

  // candidate row: two lists of TC_CAP / 2 slots, each filled from its front and from its back
  const int packed = cand_count[q];
  const int c0 = packed & 0xff, c1 = (packed >> 8) & 0xff, c2 = (packed >> 16) & 0xff, c3 = (packed >> 24) & 0xff;
  const int nc = c0 + c1 + c2 + c3;
  const bool exhaustive = *error_flag != 0 || c0 + c1 > TC_CAP / 2 || c2 + c3 > TC_CAP / 2;
  const int64_t total = exhaustive ? (x_hi > x_lo ? x_hi - x_lo : 0) : nc;
  // exact distance of point `idx` to the query, with the reference's operation order
  auto exact_dist = [&](uint32_t idx) -> float {
    float acc = 0.f;
    if (vec4) {
      const float4 *row = reinterpret_cast<const float4 *>(x + (size_t)idx * dim);
      for (int d4 = 0; d4 < (dim >> 2); ++d4) {
        const float4 xv = row[d4];
        const float4 qv = *reinterpret_cast<const float4 *>(my_q + 4 * d4);
        if (COSINE) {
          acc = __fmaf_rn(xv.x, qv.x, acc);
          acc = __fmaf_rn(xv.y, qv.y, acc);
          acc = __fmaf_rn(xv.z, qv.z, acc);
          acc = __fmaf_rn(xv.w, qv.w, acc);
        } else {
          float df = xv.x - qv.x;
          acc = __fmaf_rn(df, df, acc);
          df = xv.y - qv.y;
          acc = __fmaf_rn(df, df, acc);
          df = xv.z - qv.z;
          acc = __fmaf_rn(df, df, acc);
          df = xv.w - qv.w;
          acc = __fmaf_rn(df, df, acc);
        }
      }
    } else {
      const float *row = x + (size_t)idx * dim;
      for (int d = 0; d < dim; ++d) {
        if (COSINE) {
          acc = __fmaf_rn(row[d], my_q[d], acc);
        } else {
          const float df = row[d] - my_q[d];
          acc = __fmaf_rn(df, df, acc);
        }
      }
    }
    return COSINE ? 1.f - acc / (norms_x[idx] * ny) : acc;
  };
  auto cand_at = [&](int i) -> uint32_t {
    int slot = i;
    if (i >= c0 + c1 + c2)
      slot = TC_CAP - 1 - (i - c0 - c1 - c2);
    else if (i >= c0 + c1)
      slot = TC_CAP / 2 + (i - c0 - c1);
    else if (i >= c0)
      slot = TC_CAP / 2 - 1 - (i - c0);
    return (uint32_t)cand[q * TC_CAP + slot];
  };

  if (!exhaustive && total <= 64) {
    // The usual case, at most two candidates per lane: two warp sorts and a merge in registers,
    // without the queue in shared memory.  Only distances below 1e10 are admissible, as everywhere.
    K k0 = K::empty(), k1 = K::empty();
    if (lane < total) {
      const uint32_t idx = cand_at(lane);
      const float d = exact_dist(idx);
      if (d < 1e10f) k0 = K::make(d, idx);
    }
    if (lane + 32 < total) {
      const uint32_t idx = cand_at(lane + 32);
      const float d = exact_dist(idx);
      if (d < 1e10f) k1 = K::make(d, idx);
    }
    k0 = warp_sort32(k0, lane);
    if (total > 32) {
      k1 = warp_sort32(k1, lane);
      // the 32 smallest of both: element i of one against element 31 - i of the other is bitonic
      k0 = key_min(k0, k1.shfl(31 - lane));
      k0 = warp_bitonic_merge32(k0, lane);
    }
    const bool okk = lane < k && !k0.is_empty();
    if (graph_out != nullptr) {
      // lane e holds the e-th best: all k present and the query itself among them, else irregular
      const unsigned present = __ballot_sync(FULL_MASK, okk);
      const unsigned self = __ballot_sync(FULL_MASK, okk && (int64_t)k0.index() == q);
      if (__popc(present) != k || self == 0u) {
        if (lane == 0) atomicAdd(graph_irregular, 1);
        return;
      }
      const int selfpos = __ffs(self) - 1;
      if (lane < k && lane != selfpos) {
        const int64_t slot = q * (k - 1) + lane - (lane > selfpos ? 1 : 0);
        int64_t *row_nb = graph_s2t ? graph_out : graph_out + graph_row_stride;
        int64_t *row_q = graph_s2t ? graph_out + graph_row_stride : graph_out;
        row_nb[slot] = graph_index_base + (int64_t)k0.index();
        row_q[slot] = graph_index_base + q;
      }
      return;
    }
    if (lane < k) {
      out_row[q * k + lane] = q;
      out_col[q * k + lane] = okk ? (int64_t)k0.index() : (int64_t)-1;
    }
    const int valid = __popc(__ballot_sync(FULL_MASK, okk));
    if (lane == 0) {
      counts[q] = valid;
      if (valid) atomicAdd(num_valid, (unsigned long long)valid);
    }
    return;
  }

  float bound = 1e10f;
  for (int64_t base = 0; base < total; base += 32) {
    const int64_t i = base + lane;
    float dist[1] = {pos_inf<float>()};
    uint32_t idx = 0;
    if (i < total) {
      idx = exhaustive ? (uint32_t)(x_lo + i) : cand_at((int)i);
      dist[0] = exact_dist(idx);
    }
    if (__any_sync(FULL_MASK, dist[0] < bound)) {
      // candidate r = 0 of lane l is offered with index idx0 + 32 * 0; pass the lane's own index
      using K1 = Key<float>;
      const bool hit = dist[0] < bound;
      const unsigned mask = __ballot_sync(FULL_MASK, hit);
      int cnt = *my_cnt;
      const int nh = __popc(mask);
      if (cnt + nh > KP) {
        bound = knn_merge<float, KP>(my_keys, cnt, k, lane);
        cnt = 0;
      }
      const bool hit2 = dist[0] < bound;
      const unsigned mask2 = __ballot_sync(FULL_MASK, hit2);
      if (hit2) my_keys[KP + cnt + __popc(mask2 & ((1u << lane) - 1u))] = K1::make(dist[0], idx);
      cnt += __popc(mask2);
      __syncwarp();
      if (lane == 0) *my_cnt = cnt;
      __syncwarp();
    }
  }
  if (graph_out != nullptr) {
    if (!knn_finish_graph<float, KP>(my_keys, *my_cnt, k, q, graph_row_stride, graph_index_base, graph_out,
                                     graph_s2t != 0, lane) &&
        lane == 0)
      atomicAdd(graph_irregular, 1);
    return;
  }
  const int valid = knn_finish<float, KP>(my_keys, *my_cnt, k, q, out_row, out_col, lane);
  if (lane == 0) {
    counts[q] = valid;
    if (valid) atomicAdd(num_valid, (unsigned long long)valid);
  }
}

// |row|^2 (sequential fused sum), optional largest |row| (float bits, atomicMax) and optional normalised copy.
__global__ void tensor_prep_kernel(const float *__restrict__ a, int64_t rows, int dim, float *__restrict__ sq,
                                   unsigned *__restrict__ max_bits, float *__restrict__ normalised) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows) return;
  float s = 0.f;
  for (int d = 0; d < dim; ++d) {
    const float v = a[i * dim + d];
    s = __fmaf_rn(v, v, s);
  }
  if (sq) sq[i] = s;
  const float nrm = sqrtf(s);
  if (max_bits && nrm == nrm) atomicMax(max_bits, __float_as_uint(nrm));  // nrm >= 0: bits order like values
  if (normalised)
    for (int d = 0; d < dim; ++d) normalised[i * dim + d] = a[i * dim + d] / nrm;
}

// query tile + ring of point tiles + |x|^2 ring + group minima + alignment slack
size_t knn_tensor_smem_bytes(int dim, int ring) {
  return (size_t)(1 + ring) * ((dim + 31) / 32) * 16384 + (size_t)(ring + 1) * TC_N * 4 + (size_t)TC_GH * TC_THREADS * 4 +
         1024;
}

static size_t al256(size_t v) { return (v + 255) / 256 * 256; }

// workspace: [sq_x n][sq_y m][xmax + error flag 256][cand m*CAP][cand_count m]
//            cosine adds [norms_x n][norms_y m][xhat n*dim][yhat m*dim]
size_t knn_tensor_workspace_bytes(int64_t n, int64_t m, int dim, int cosine) {
  size_t b = al256((size_t)n * 4) + al256((size_t)m * 4) + 256 + al256((size_t)m * TC_CAP * 4) + al256((size_t)m * 4);
  if (cosine) b += al256((size_t)n * 4) + al256((size_t)m * 4) + al256((size_t)n * dim * 4) + al256((size_t)m * dim * 4);
  return b;
}

bool knn_tensor_applicable(int64_t n, int64_t m, int dim, int k, int64_t num_segments, const void *x, const void *y) {
  if (dim < 32 || dim > 128 || (dim & 7) || k > 32 || m < 1 || n < 1) return false;
  if (((uintptr_t)x | (uintptr_t)y) & 15) return false;
  return n / num_segments >= 32 * (int64_t)k;  // enough points per segment for k group minima, on average
}

// Exact re-rank of candidate lists ([m, 128] int32 + counts); shared with the low-dimensional screen.
int launch_knn_rerank_f32(const KnnArgs &a, const int32_t *cand, const int32_t *cand_count, const int *error_flag,
                          const float *norms_x, const float *norms_y) {
  const int qstride = (a.dim + 3) & ~3;
  const size_t rr_smem = (size_t)RR_WARPS * qstride * 4 + (size_t)RR_WARPS * 64 * sizeof(Key<float>) + RR_WARPS * 4;
  const unsigned rr_ctas = (unsigned)((a.m + RR_WARPS - 1) / RR_WARPS);
  if (a.cosine)
    knn_rerank_kernel<true><<<rr_ctas, RR_WARPS * 32, rr_smem, a.stream>>>(
        (const float *)a.x, (const float *)a.y, a.ptr_x, a.ptr_y, a.num_segments, a.n, a.m, a.dim, a.k, norms_x,
        norms_y, cand, cand_count, error_flag, a.out_row, a.out_col, a.counts, a.num_valid, a.graph_out,
        a.graph_row_stride, a.graph_index_base, a.graph_s2t, a.graph_irregular);
  else
    knn_rerank_kernel<false><<<rr_ctas, RR_WARPS * 32, rr_smem, a.stream>>>(
        (const float *)a.x, (const float *)a.y, a.ptr_x, a.ptr_y, a.num_segments, a.n, a.m, a.dim, a.k, nullptr,
        nullptr, cand, cand_count, error_flag, a.out_row, a.out_col, a.counts, a.num_valid, a.graph_out,
        a.graph_row_stride, a.graph_index_base, a.graph_s2t, a.graph_irregular);
  B200C_LAUNCH_CHECK("knn_rerank_kernel");
  return B200C_OK;
}

int launch_knn_tensor_f32(const KnnArgs &a, void *workspace) {
  char *ws = (char *)workspace;
  float *sq_x = (float *)ws; ws += al256((size_t)a.n * 4);
  float *sq_y = (float *)ws; ws += al256((size_t)a.m * 4);
  float *xmax = (float *)ws;
  int *error_flag = (int *)(ws + 128); ws += 256;
  int32_t *cand = (int32_t *)ws; ws += al256((size_t)a.m * TC_CAP * 4);
  int32_t *cand_count = (int32_t *)ws; ws += al256((size_t)a.m * 4);
  float *norms_x = nullptr, *norms_y = nullptr, *xhat = nullptr, *yhat = nullptr;
  if (a.cosine) {
    norms_x = (float *)ws; ws += al256((size_t)a.n * 4);
    norms_y = (float *)ws; ws += al256((size_t)a.m * 4);
    xhat = (float *)ws; ws += al256((size_t)a.n * a.dim * 4);
    yhat = (float *)ws; ws += al256((size_t)a.m * a.dim * 4);
  }
  B200C_CUDA(cudaMemsetAsync(xmax, 0, 256, a.stream));
  B200C_CUDA(cudaMemsetAsync(cand_count, 0, (size_t)a.m * 4, a.stream));  // the two threads of a query add their counts
  const int threads = 128;
  tensor_prep_kernel<<<(unsigned)((a.n + threads - 1) / threads), threads, 0, a.stream>>>(
      (const float *)a.x, a.n, a.dim, sq_x, (unsigned *)xmax, xhat);
  B200C_LAUNCH_CHECK("tensor_prep_kernel");
  const bool self = a.x == a.y && a.n == a.m;  // x searched in itself (knn_graph): one set of norms serves both
  if (self) {
    sq_y = sq_x;
    yhat = xhat;
  } else {
    tensor_prep_kernel<<<(unsigned)((a.m + threads - 1) / threads), threads, 0, a.stream>>>(
        (const float *)a.y, a.m, a.dim, sq_y, nullptr, yhat);
    B200C_LAUNCH_CHECK("tensor_prep_kernel");
  }
  if (a.cosine) {
    int st = launch_row_norms_f32(a.x, a.n, a.dim, norms_x, a.stream);
    if (st != B200C_OK) return st;
    if (self) {
      norms_y = norms_x;
    } else {
      st = launch_row_norms_f32(a.y, a.m, a.dim, norms_y, a.stream);
      if (st != B200C_OK) return st;
    }
  }

  TensorArgs t{a.cosine ? xhat : (const float *)a.x, a.cosine ? yhat : (const float *)a.y, sq_x, sq_y, xmax,
               a.ptr_x, a.ptr_y, a.num_segments, a.n, a.m, a.dim, a.k, cand, cand_count, error_flag};
  const size_t smem = knn_tensor_smem_bytes(a.dim, TC_RING);
  const unsigned ctas = (unsigned)((a.m + TC_M - 1) / TC_M);
  // the opt-in covers the largest tile set (128 features) once per device and kernel
  const size_t smem_most = knn_tensor_smem_bytes(128, TC_RING);
  static unsigned long long configured_cosine = 0ull, configured_l2 = 0ull;
  if (a.cosine) {
    B200C_CUDA(opt_in_shared_memory(knn_tensor_candidates_kernel<true>, smem_most, configured_cosine));
    knn_tensor_candidates_kernel<true><<<ctas, TC_THREADS, smem, a.stream>>>(t);
  } else {
    B200C_CUDA(opt_in_shared_memory(knn_tensor_candidates_kernel<false>, smem_most, configured_l2));
    knn_tensor_candidates_kernel<false><<<ctas, TC_THREADS, smem, a.stream>>>(t);
  }
  B200C_LAUNCH_CHECK("knn_tensor_candidates_kernel");

  return launch_knn_rerank_f32(a, cand, cand_count, error_flag, norms_x, norms_y);
}

}  // namespace b200c
