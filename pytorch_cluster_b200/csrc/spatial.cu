// Morton-ordered copies of low-dimensional fp32 point sets (see spatial.cuh): segment layout,
// bounding boxes, keys, a sort of (key, row) pairs — a bitonic network in shared memory for segments
// of up to SP_SORT_BLOCK points, a bucket sort with sampled splitters above (bitonic exchange passes
// through global memory for the very largest) — and the sorted arrays.
// All passes are HBM- or latency-bound and small next to the scan they prepare: 32 bytes are read
// and about 60 written per point.
#include "launchers.h"
#include "spatial.cuh"

namespace b200c {

constexpr int SP_THREADS = 1024;

static size_t sp_align(size_t v) { return (v + 255) / 256 * 256; }

static int64_t view_cap(int64_t rows, int64_t segs) {
  const int64_t raw = rows + segs * (SP_CHUNK - 1);
  return (raw + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
}
static int64_t pairs_small_cap(int64_t rows) { return (2 * rows + SP_SORT_BLOCK - 1) / SP_SORT_BLOCK * SP_SORT_BLOCK; }

size_t spatial_view_carve(SpatialView *v, void *workspace, int64_t rows, int dim, int64_t segs, bool points) {
  char *p = (char *)workspace;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char *r = p ? p + off : nullptr;
    off += sp_align(bytes);
    return r;
  };
  const int64_t cap = view_cap(rows, segs);
  SpatialView t{};
  t.cap = cap;
  t.idx = (int32_t *)take((size_t)cap * 4);
  t.key = (uint32_t *)take((size_t)cap * 4);
  t.sptr = (int64_t *)take((size_t)(segs + 1) * 8);
  t.pptr = (int64_t *)take((size_t)(segs + 1) * 8);
  t.lptr = (int64_t *)take((size_t)(segs + 1) * 8);
  t.box = (float *)take((size_t)segs * 2 * dim * 4);
  t.stat = (uint32_t *)take((size_t)segs * 2 * 4);
  t.pairs_cap = pairs_small_cap(rows) + 2 * rows + SP_SORT_BLOCK;
  t.pairs = (uint64_t *)take((size_t)t.pairs_cap * 8);
  if (points) t.blob = (float *)take((size_t)cap * (2 * dim + 2) * 4);
  const int64_t large_blocks = 2 * rows / SP_SORT_BLOCK + 2;
  t.pairs2 = (uint64_t *)take((size_t)rows * 8);
  t.split = (uint64_t *)take((size_t)large_blocks * SP_MAX_BUCKETS * 8);
  t.bcount = (int32_t *)take((size_t)large_blocks * SP_MAX_BUCKETS * 4);
  t.boffset = (int32_t *)take((size_t)large_blocks * (SP_MAX_BUCKETS + 1) * 4);
  t.bcursor = (int32_t *)take((size_t)large_blocks * SP_MAX_BUCKETS * 4);
  t.table_cap = rows / SP_BUCKET_TARGET + rows / SP_SORT_BLOCK + 2 * large_blocks + 8;
  t.table = (int32_t *)take((size_t)t.table_cap * 4 * 4);
  t.table_count = (int32_t *)take(4);
  t.bad = (int32_t *)take(4);
  if (v) *v = t;
  return off;
}

size_t spatial_view_bytes(int64_t rows, int dim, int64_t segs, bool points) {
  return spatial_view_carve(nullptr, nullptr, rows, dim, segs, points);
}

// ---- helpers ----------------------------------------------------------------------------------------
__device__ __forceinline__ int64_t pow2_ceil(int64_t v) {
  int64_t p = 1;
  while (p < v) p <<= 1;
  return p;
}

__device__ __forceinline__ void seg_rows_clamped(const int64_t *__restrict__ ptr, int64_t rows, int b, int64_t &lo,
                                                 int64_t &hi) {
  if (ptr == nullptr) {
    lo = 0;
    hi = rows;
    return;
  }
  lo = ptr[b];
  hi = ptr[b + 1];
  if (lo < 0) lo = 0;
  if (hi > rows) hi = rows;
  if (hi < lo) hi = lo;
}

// Bits per feature of the Morton key (at most 30 bits in all).
__host__ __device__ constexpr int morton_bits(int dim) { return dim == 1 ? 30 : (dim == 2 ? 15 : 30 / dim); }

template <int DIM>
__device__ __forceinline__ uint32_t morton_key(const float *p, const float *lo, const float *scale) {
  constexpr int BITS = morton_bits(DIM);
  uint32_t cell[DIM];
#pragma unroll
  for (int d = 0; d < DIM; ++d) {
    // fmaxf / fminf drop a NaN operand: NaN and out-of-box values land in a border cell
    const float t = fminf(fmaxf((p[d] - lo[d]) * scale[d], 0.f), (float)((1u << BITS) - 1u));
    cell[d] = (uint32_t)t;
  }
  uint32_t key = 0;
#pragma unroll
  for (int bit = 0; bit < BITS; ++bit)
#pragma unroll
    for (int d = 0; d < DIM; ++d) key |= ((cell[d] >> bit) & 1u) << (bit * DIM + d);
  return key;
}

template <int DIM>
__device__ __forceinline__ void box_scale(const float *box, float *lo, float *scale, float *centre) {
  constexpr int BITS = morton_bits(DIM);
#pragma unroll
  for (int d = 0; d < DIM; ++d) {
    const float a = box[d], b = box[DIM + d];
    lo[d] = a;
    const float ext = b - a;
    scale[d] = (ext > 0.f && ext < 3.0e38f) ? (float)(1u << BITS) / ext : 0.f;
    centre[d] = 0.5f * a + 0.5f * b;
  }
}

__device__ __forceinline__ void atomic_min_float(float *addr, float v) {
  int *ia = reinterpret_cast<int *>(addr);
  int old = *ia;
  while (v < __int_as_float(old)) {
    const int seen = atomicCAS(ia, old, __float_as_int(v));
    if (seen == old) break;
    old = seen;
  }
}
__device__ __forceinline__ void atomic_max_float(float *addr, float v) {
  int *ia = reinterpret_cast<int *>(addr);
  int old = *ia;
  while (v > __int_as_float(old)) {
    const int seen = atomicCAS(ia, old, __float_as_int(v));
    if (seen == old) break;
    old = seen;
  }
}

// ---- layout: one thread block -----------------------------------------------------------------------------
// sptr: padded first position of every segment (multiples of SP_CHUNK).  pptr: first (key, row) pair
// of every segment in the sort scratch; segments of up to SP_SORT_BLOCK points lie back to back in
// [0, small_cap), larger ones — whole numbers of sort blocks — from small_cap on.  lptr: number of
// sort blocks of the large segments before each segment.  Also resets boxes and statistics.
__global__ void __launch_bounds__(SP_THREADS)
sp_layout_kernel(const int64_t *__restrict__ ptr, int segs, int64_t rows, int64_t small_cap, int dim,
                 int64_t *__restrict__ sptr, int64_t *__restrict__ pptr, int64_t *__restrict__ lptr,
                 float *__restrict__ box, uint32_t *__restrict__ stat, int reset_box,
                 int32_t *__restrict__ table_count, int32_t *__restrict__ bad) {
  __shared__ int64_t run[4][SP_THREADS];
  const int t = threadIdx.x;
  if (t == 0) *table_count = 0;
  const int per = (segs + SP_THREADS - 1) / SP_THREADS;
  const int lo = t * per < segs ? t * per : segs;
  const int hi = lo + per < segs ? lo + per : segs;
  int64_t s3 = 0;  // rows of this thread's segments: the sizes of segments that do not overlap add up to <= rows
  auto sizes = [&](int b, int64_t &padded, int64_t &small, int64_t &large) {
    int64_t a, e;
    seg_rows_clamped(ptr, rows, b, a, e);
    const int64_t nb = e - a;
    padded = (nb + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
    const int64_t p2 = nb > 0 ? pow2_ceil(nb) : 0;
    small = p2 <= SP_SORT_BLOCK ? p2 : 0;
    large = p2 <= SP_SORT_BLOCK ? 0 : p2;
  };
  int64_t s0 = 0, s1 = 0, s2 = 0;
  for (int b = lo; b < hi; ++b) {
    int64_t p, s, l;
    sizes(b, p, s, l);
    s0 += p;
    s1 += s;
    s2 += l;
    int64_t a, e;
    seg_rows_clamped(ptr, rows, b, a, e);
    s3 += e - a;
  }
  run[0][t] = s0;
  run[1][t] = s1;
  run[2][t] = s2;
  run[3][t] = s3;
  __syncthreads();
  for (int o = 1; o < SP_THREADS; o <<= 1) {
    int64_t a0 = 0, a1 = 0, a2 = 0, a3 = 0;
    if (t >= o) {
      a0 = run[0][t - o];
      a1 = run[1][t - o];
      a2 = run[2][t - o];
      a3 = run[3][t - o];
    }
    __syncthreads();
    run[0][t] += a0;
    run[1][t] += a1;
    run[2][t] += a2;
    run[3][t] += a3;
    __syncthreads();
  }
  // Overlapping segments (pointers that are not a partition of the rows) would not fit the arrays sized for
  // `rows` rows: the layout is left empty — every kernel after this one finds nothing to do — and flagged.
  const bool overlap = run[3][SP_THREADS - 1] > rows;
  if (t == 0) *bad = overlap ? 1 : 0;
  if (overlap) {
    for (int b = t; b <= segs; b += SP_THREADS) {
      sptr[b] = 0;
      pptr[b] = 0;
      lptr[b] = 0;
    }
    for (int i = t; i < segs * 2; i += SP_THREADS) stat[i] = 0u;
    return;
  }
  int64_t r0 = run[0][t] - s0, r1 = run[1][t] - s1, r2 = run[2][t] - s2;
  for (int b = lo; b < hi; ++b) {
    int64_t p, s, l;
    sizes(b, p, s, l);
    sptr[b] = r0;
    pptr[b] = l > 0 ? small_cap + r2 : r1;
    lptr[b] = r2 / SP_SORT_BLOCK;
    r0 += p;
    r1 += s;
    r2 += l;
  }
  if (t == SP_THREADS - 1) {
    sptr[segs] = run[0][t];
    pptr[segs] = small_cap + run[2][t];
    lptr[segs] = run[2][t] / SP_SORT_BLOCK;
  }
  for (int i = t; i < segs * 2; i += SP_THREADS) stat[i] = 0u;
  if (reset_box) {
    const float inf = __int_as_float(0x7f800000);
    for (int i = t; i < segs * 2 * dim; i += SP_THREADS) box[i] = (i % (2 * dim)) < dim ? inf : -inf;
  }
}

// ---- bitonic network on 64-bit pairs in shared memory ----------------------------------------------------
// a[0 .. count): count a power of two; base = position of a[0] within its segment (directions follow
// the segment-wide network).  Runs the merges of sizes first_size .. last_size; for sizes above
// count only the strides below count (the exchanges that stay inside this block).
__device__ __forceinline__ void smem_bitonic(uint64_t *a, int count, int64_t base, int64_t first_size,
                                             int64_t last_size, int tid, int nthreads) {
  for (int64_t size = first_size; size <= last_size; size <<= 1) {
    int stride = (int)((size >> 1) < (int64_t)(count >> 1) ? (size >> 1) : (count >> 1));
    for (; stride > 0; stride >>= 1) {
      __syncthreads();
      for (int c = tid; c < (count >> 1); c += nthreads) {
        const int i = 2 * c - (c & (stride - 1));
        const int j = i + stride;
        const bool asc = ((base + i) & size) == 0;
        const uint64_t x = a[i], y = a[j];
        if ((y < x) == asc) {
          a[i] = y;
          a[j] = x;
        }
      }
    }
  }
  __syncthreads();
}

// ---- the same network, sixteen keys per thread in registers ------------------------------------------------
// For blocks of 1024 keys and more.  A pass loads, per thread, groups of 2^NB keys whose indices
// differ in NB consecutive bits, runs the NB exchange steps of those strides in registers and stores
// the keys back: a merge of size 2^s costs ceil(s / 4) passes over shared memory instead of s, and an
// exchange a compare and two selects per word instead of two loads and two stores.  Keys live at
// padded positions i + i / 16 so that a thread's run of 16 consecutive keys (the passes over the
// lowest four bits) does not meet the other lanes' runs in the same banks.
__device__ __forceinline__ int sp_pad(int i) { return i + (i >> 4); }
constexpr int SP_SORT_SMEM_KEYS = SP_SORT_BLOCK + SP_SORT_BLOCK / 16;

__device__ __forceinline__ void sp_exchange(uint64_t &x, uint64_t &y, bool asc) {
  const bool swap = (y < x) == asc;
  const uint64_t lo = swap ? y : x, hi = swap ? x : y;
  x = lo;
  y = hi;
}

template <int NB>
__device__ __forceinline__ void bitonic_pass(uint64_t *a, int count, int lowbit, int64_t base, int size_log, int tid,
                                             int nthreads) {
  constexpr int G = 1 << NB;
  const int groups = count >> NB;
  for (int g = tid; g < groups; g += nthreads) {
    const int low = g & ((1 << lowbit) - 1);
    const int i0 = ((g >> lowbit) << (lowbit + NB)) | low;
    const bool asc = (((base + i0) >> size_log) & 1) == 0;
    uint64_t v[G];
#pragma unroll
    for (int j = 0; j < G; ++j) v[j] = a[sp_pad(i0 | (j << lowbit))];
#pragma unroll
    for (int b = NB - 1; b >= 0; --b)
#pragma unroll
      for (int j = 0; j < G; ++j)
        if (!(j & (1 << b))) sp_exchange(v[j], v[j | (1 << b)], asc);
#pragma unroll
    for (int j = 0; j < G; ++j) a[sp_pad(i0 | (j << lowbit))] = v[j];
  }
}

// Merges of sizes 2, 4, 8, 16 of every run of 16 consecutive keys in one pass.
__device__ __forceinline__ void bitonic_first16(uint64_t *a, int count, int64_t base, int tid, int nthreads) {
  for (int g = tid; g < (count >> 4); g += nthreads) {
    const int i0 = g << 4;
    const bool asc16 = (((base + i0) >> 4) & 1) == 0;
    uint64_t v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = a[sp_pad(i0 | j)];
#pragma unroll
    for (int s = 1; s <= 4; ++s)
#pragma unroll
      for (int b = s - 1; b >= 0; --b)
#pragma unroll
        for (int j = 0; j < 16; ++j)
          if (!(j & (1 << b))) sp_exchange(v[j], v[j | (1 << b)], s < 4 ? ((j >> s) & 1) == 0 : asc16);
#pragma unroll
    for (int j = 0; j < 16; ++j) a[sp_pad(i0 | j)] = v[j];
  }
}

// a: 2^p keys at padded positions (4 <= p), base as in smem_bitonic.  Runs the merges of sizes
// 2^first_log .. 2^last_log (first_log == 1: from scratch); of a merge larger than the block only the
// strides inside it.
__device__ __forceinline__ void smem_bitonic_blocked(uint64_t *a, int p, int64_t base, int first_log, int last_log,
                                                     int tid, int nthreads) {
  const int count = 1 << p;
  int s = first_log;
  if (s == 1) {
    __syncthreads();
    bitonic_first16(a, count, base, tid, nthreads);
    s = 5;
  }
  for (; s <= last_log; ++s) {
    int top = (s < p ? s : p) - 1;  // highest stride bit inside the block
    const int rem = (top + 1) & 3;
    __syncthreads();
    if (rem == 1) bitonic_pass<1>(a, count, top, base, s, tid, nthreads);
    if (rem == 2) bitonic_pass<2>(a, count, top - 1, base, s, tid, nthreads);
    if (rem == 3) bitonic_pass<3>(a, count, top - 2, base, s, tid, nthreads);
    top -= rem;
    for (; top >= 3; top -= 4) {
      __syncthreads();
      bitonic_pass<4>(a, count, top - 3, base, s, tid, nthreads);
    }
  }
  __syncthreads();
}

// ---- sorted arrays of one position -----------------------------------------------------------------------
template <int DIM>
__device__ __forceinline__ float emit_position(const SpatialView &v, const float *__restrict__ pts, int64_t x_lo,
                                               int64_t pos, uint64_t pair, bool valid, bool points,
                                               const float *centre) {
  float wv = 0.f;
  // the position's slot in its chunk's block of 2 DIM + 2 arrays
  float *chunk = points ? v.blob + (pos / SP_CHUNK) * ((2 * DIM + 2) * SP_CHUNK) + (pos % SP_CHUNK) : nullptr;
  if (valid) {
    const int64_t row = x_lo + (int64_t)(uint32_t)pair;
    v.idx[pos] = (int32_t)row;
    v.key[pos] = (uint32_t)(pair >> 32);
    if (points) {
      float acc = 0.f;
#pragma unroll
      for (int d = 0; d < DIM; ++d) {
        const float p = pts[row * DIM + d];
        const float c = p - centre[d];
        chunk[(DIM + 2 + d) * SP_CHUNK] = p;
        chunk[d * SP_CHUNK] = c;
        acc = __fmaf_rn(c, c, acc);
      }
      chunk[DIM * SP_CHUNK] = acc;
      chunk[(DIM + 1) * SP_CHUNK] = __int_as_float((int32_t)row);
      wv = acc;
    }
  } else {
    const float inf = __int_as_float(0x7f800000);
    v.idx[pos] = -1;
    v.key[pos] = 0xffffffffu;
    if (points) {
#pragma unroll
      for (int d = 0; d < DIM; ++d) {
        chunk[(DIM + 2 + d) * SP_CHUNK] = inf;
        chunk[d * SP_CHUNK] = inf;
      }
      chunk[DIM * SP_CHUNK] = inf;
      chunk[(DIM + 1) * SP_CHUNK] = __int_as_float(-1);
    }
  }
  return wv;
}

// largest w of a block -> stat[b][0]; a NaN or infinite w becomes +inf (the scan then treats the
// whole segment without its screen)
__device__ __forceinline__ void publish_wmax(float wmax, bool bad, uint32_t *stat_b, float *red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (bad) wmax = __int_as_float(0x7f800000);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(FULL_MASK, wmax, o));
  if (lane == 0) red[warp] = wmax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = 0.f;
    for (int i = 0; i < (int)(blockDim.x >> 5); ++i) m = fmaxf(m, red[i]);
    atomicMax(stat_b, __float_as_uint(m));  // non-negative floats order like their bits
  }
  __syncthreads();
}

// ---- segments of up to SP_SORT_BLOCK points: everything in one thread block -------------------------------
template <int DIM>
__global__ void __launch_bounds__(SP_THREADS)
sp_small_kernel(const float *__restrict__ pts, const int64_t *__restrict__ ptr, int segs, int64_t rows,
                const float *__restrict__ box_from, int points, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  extern __shared__ __align__(16) unsigned char sp_smem[];
  uint64_t *pairs = reinterpret_cast<uint64_t *>(sp_smem);
  __shared__ float red[2 * SP_MAX_DIM][32];
  __shared__ float box_s[2 * SP_MAX_DIM];
  const int b = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int nb = (int)((x_hi - x_lo) < (int64_t)SP_SORT_BLOCK + 1 ? (x_hi - x_lo) : (int64_t)SP_SORT_BLOCK + 1);
  if (nb == 0 || nb > SP_SORT_BLOCK) return;  // empty, or one for the multi-block path
  const int p2 = (int)pow2_ceil(nb);
  const float inf = __int_as_float(0x7f800000);

  if (box_from == nullptr) {
    float mn[DIM], mx[DIM];
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
      mn[d] = inf;
      mx[d] = -inf;
    }
    for (int i = tid; i < nb; i += SP_THREADS) {
#pragma unroll
      for (int d = 0; d < DIM; ++d) {
        const float p = pts[(x_lo + i) * DIM + d];
        mn[d] = fminf(mn[d], p);
        mx[d] = fmaxf(mx[d], p);
      }
    }
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        mn[d] = fminf(mn[d], __shfl_xor_sync(FULL_MASK, mn[d], o));
        mx[d] = fmaxf(mx[d], __shfl_xor_sync(FULL_MASK, mx[d], o));
      }
      if (lane == 0) {
        red[d][warp] = mn[d];
        red[DIM + d][warp] = mx[d];
      }
    }
    __syncthreads();
    if (tid < 2 * DIM) {
      float m = red[tid][0];
      for (int i = 1; i < SP_THREADS / 32; ++i) m = tid < DIM ? fminf(m, red[tid][i]) : fmaxf(m, red[tid][i]);
      box_s[tid] = m;
      v.box[(int64_t)b * 2 * DIM + tid] = m;
    }
  } else if (tid < 2 * DIM) {
    box_s[tid] = box_from[(int64_t)b * 2 * DIM + tid];
  }
  __syncthreads();
  float lo[DIM], scale[DIM], centre[DIM];
  box_scale<DIM>(box_s, lo, scale, centre);

  const bool blocked = p2 >= 1024;  // sixteen keys per thread, padded positions
  for (int i = tid; i < p2; i += SP_THREADS) {
    uint64_t pair = ~0ull;
    if (i < nb) {
      float p[DIM];
#pragma unroll
      for (int d = 0; d < DIM; ++d) p[d] = pts[(x_lo + i) * DIM + d];
      pair = ((uint64_t)morton_key<DIM>(p, lo, scale) << 32) | (uint32_t)i;
    }
    pairs[blocked ? sp_pad(i) : i] = pair;
  }
  if (blocked) {
    int plog = 10;
    while ((1 << plog) < p2) ++plog;
    smem_bitonic_blocked(pairs, plog, 0, 1, plog, tid, SP_THREADS);
  } else if (p2 > 1) {
    smem_bitonic(pairs, p2, 0, 2, p2, tid, SP_THREADS);
  } else {
    __syncthreads();
  }

  const int64_t s_lo = v.sptr[b];
  const int padded = (nb + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
  float wmax = 0.f;
  bool bad = false;
  for (int j = tid; j < padded; j += SP_THREADS) {
    const float wv = emit_position<DIM>(v, pts, x_lo, s_lo + j, j < nb ? pairs[blocked ? sp_pad(j) : j] : 0ull, j < nb,
                                        points != 0, centre);
    bad |= !(wv < 1e30f);
    wmax = fmaxf(wmax, wv);
  }
  if (points) publish_wmax(wmax, bad, v.stat + 2 * b, &red[0][0]);
}

// ---- larger segments: the same steps as separate kernels over (part, segment) grids ----------------------
__device__ __forceinline__ bool large_segment(const SpatialView &v, int b) { return v.lptr[b + 1] > v.lptr[b]; }

template <int DIM>
__global__ void __launch_bounds__(SP_THREADS)
sp_box_kernel(const float *__restrict__ pts, const int64_t *__restrict__ ptr, int64_t rows, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  __shared__ float red[2 * SP_MAX_DIM][32];
  const int b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (!large_segment(v, b)) return;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const float inf = __int_as_float(0x7f800000);
  float mn[DIM], mx[DIM];
#pragma unroll
  for (int d = 0; d < DIM; ++d) {
    mn[d] = inf;
    mx[d] = -inf;
  }
  for (int64_t i = x_lo + (int64_t)blockIdx.x * SP_THREADS + tid; i < x_hi; i += (int64_t)gridDim.x * SP_THREADS) {
#pragma unroll
    for (int d = 0; d < DIM; ++d) {
      const float p = pts[i * DIM + d];
      mn[d] = fminf(mn[d], p);
      mx[d] = fmaxf(mx[d], p);
    }
  }
#pragma unroll
  for (int d = 0; d < DIM; ++d) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mn[d] = fminf(mn[d], __shfl_xor_sync(FULL_MASK, mn[d], o));
      mx[d] = fmaxf(mx[d], __shfl_xor_sync(FULL_MASK, mx[d], o));
    }
    if (lane == 0) {
      red[d][warp] = mn[d];
      red[DIM + d][warp] = mx[d];
    }
  }
  __syncthreads();
  if (tid < 2 * DIM) {
    float m = red[tid][0];
    for (int i = 1; i < SP_THREADS / 32; ++i) m = tid < DIM ? fminf(m, red[tid][i]) : fmaxf(m, red[tid][i]);
    if (tid < DIM)
      atomic_min_float(&v.box[(int64_t)b * 2 * DIM + tid], m);
    else
      atomic_max_float(&v.box[(int64_t)b * 2 * DIM + tid], m);
  }
}

template <int DIM>
__global__ void __launch_bounds__(SP_THREADS)
sp_keys_kernel(const float *__restrict__ pts, const int64_t *__restrict__ ptr, int64_t rows,
               const float *__restrict__ box, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  const int b = blockIdx.y;
  if (!large_segment(v, b)) return;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int64_t nb = x_hi - x_lo, p2 = (v.lptr[b + 1] - v.lptr[b]) * SP_SORT_BLOCK;
  float lo[DIM], scale[DIM], centre[DIM];
  box_scale<DIM>(box + (int64_t)b * 2 * DIM, lo, scale, centre);
  uint64_t *dst = v.pairs + v.pptr[b];
  for (int64_t i = (int64_t)blockIdx.x * SP_THREADS + threadIdx.x; i < p2; i += (int64_t)gridDim.x * SP_THREADS) {
    uint64_t pair = ~0ull;
    if (i < nb) {
      float p[DIM];
#pragma unroll
      for (int d = 0; d < DIM; ++d) p[d] = pts[(x_lo + i) * DIM + d];
      pair = ((uint64_t)morton_key<DIM>(p, lo, scale) << 32) | (uint32_t)i;
    }
    dst[i] = pair;
  }
}

// First segment whose sort blocks include block j of the large region.
__device__ __forceinline__ int segment_of_block(const int64_t *__restrict__ lptr, int segs, int64_t j) {
  int lo = 0, hi = segs - 1;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (lptr[mid + 1] > j)
      hi = mid;
    else
      lo = mid + 1;
  }
  return lo;
}

// One sort block in shared memory.  size == 0: the full sort of the block (merges 2 .. SP_SORT_BLOCK);
// size > SP_SORT_BLOCK: the block-local tail (strides below SP_SORT_BLOCK) of the merge of that size.
__global__ void __launch_bounds__(SP_THREADS)
sp_sort_block_kernel(SpatialView v, int segs, int64_t size) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  extern __shared__ __align__(16) unsigned char sp_smem[];
  uint64_t *a = reinterpret_cast<uint64_t *>(sp_smem);
  const int64_t j = blockIdx.x;
  if (j >= v.lptr[segs]) return;
  const int b = segment_of_block(v.lptr, segs, j);
  const int64_t jb = j - v.lptr[b], p2 = (v.lptr[b + 1] - v.lptr[b]) * SP_SORT_BLOCK;
  if (size > p2) return;
  uint64_t *g = v.pairs + v.pptr[b] + jb * SP_SORT_BLOCK;
  constexpr int PLOG = 14;
  static_assert((1 << PLOG) == SP_SORT_BLOCK, "block size and its logarithm");
  for (int i = threadIdx.x; i < SP_SORT_BLOCK; i += SP_THREADS) a[sp_pad(i)] = g[i];
  if (size == 0) {
    smem_bitonic_blocked(a, PLOG, jb * SP_SORT_BLOCK, 1, PLOG, threadIdx.x, SP_THREADS);
  } else {
    int slog = PLOG;
    while (((int64_t)1 << slog) < size) ++slog;
    smem_bitonic_blocked(a, PLOG, jb * SP_SORT_BLOCK, slog, slog, threadIdx.x, SP_THREADS);
  }
  for (int i = threadIdx.x; i < SP_SORT_BLOCK; i += SP_THREADS) g[i] = a[sp_pad(i)];
}

// One exchange step (stride >= SP_SORT_BLOCK) of the merge of `size` over all large segments.
__global__ void sp_sort_global_kernel(SpatialView v, int segs, int64_t size, int64_t stride) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  const int64_t t = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // exchange number over the large region
  const int64_t total = v.lptr[segs] * (SP_SORT_BLOCK / 2);
  if (t >= total) return;
  const int b = segment_of_block(v.lptr, segs, t / (SP_SORT_BLOCK / 2));
  const int64_t p2 = (v.lptr[b + 1] - v.lptr[b]) * SP_SORT_BLOCK;
  if (size > p2) return;
  const int64_t c = t - v.lptr[b] * (SP_SORT_BLOCK / 2);
  const int64_t i = 2 * c - (c & (stride - 1)), j = i + stride;
  uint64_t *g = v.pairs + v.pptr[b];
  const bool asc = (i & size) == 0;
  const uint64_t x = g[i], y = g[j];
  if ((y < x) == asc) {
    g[i] = y;
    g[j] = x;
  }
}

template <int DIM>
__global__ void __launch_bounds__(SP_THREADS)
sp_emit_kernel(const float *__restrict__ pts, const int64_t *__restrict__ ptr, int64_t rows,
               const float *__restrict__ box, int points, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  __shared__ float red[32];
  const int b = blockIdx.y;
  if (!large_segment(v, b)) return;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int64_t nb = x_hi - x_lo, padded = (nb + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
  float lo[DIM], scale[DIM], centre[DIM];
  box_scale<DIM>(box + (int64_t)b * 2 * DIM, lo, scale, centre);
  const uint64_t *src = v.pairs + v.pptr[b];
  const int64_t s_lo = v.sptr[b];
  float wmax = 0.f;
  bool bad = false;
  for (int64_t j = (int64_t)blockIdx.x * SP_THREADS + threadIdx.x; j < padded; j += (int64_t)gridDim.x * SP_THREADS) {
    const float wv = emit_position<DIM>(v, pts, x_lo, s_lo + j, j < nb ? src[j] : 0ull, j < nb, points != 0, centre);
    bad |= !(wv < 1e30f);
    wmax = fmaxf(wmax, wv);
  }
  if (points) publish_wmax(wmax, bad, v.stat + 2 * b, red);
}

// ---- bucket sort of the segments above one sort block (up to SP_BUCKET_MAX_ROWS points) ---------------------
// Instead of log^2 exchange passes over the whole segment: a sample of its (key, row) pairs is sorted by
// one thread block and gives up to 255 splitters; every pair is counted into, then scattered to, the
// bucket between two splitters (pairs are unique, so even equal keys spread evenly); each bucket — about
// 4096 pairs — is sorted in shared memory by its own thread block, which also writes the sorted copy.
// Six launches whatever the size, and as many blocks at work as there are buckets.  A bucket that comes out
// larger than a sort block (a sample that misled) is cut into pieces that are sorted on their own: the
// order is then not quite the Morton order, which costs the scan time, never correctness.
constexpr int SP_SAMPLE = 8192;

__device__ __forceinline__ int bucket_count_of(int64_t nb) {
  const int64_t want = (nb + SP_BUCKET_TARGET - 1) / SP_BUCKET_TARGET;
  return (int)(want < 2 ? 2 : (want > SP_MAX_BUCKETS ? SP_MAX_BUCKETS : want));
}

// bucket of a pair: number of splitters <= pair
__device__ __forceinline__ int bucket_of(const uint64_t *split_s, int nsplit, uint64_t pair) {
  int lo = 0, hi = nsplit;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (split_s[mid] <= pair)
      lo = mid + 1;
    else
      hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(SP_THREADS)
sp_sample_kernel(const int64_t *__restrict__ ptr, int64_t rows, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  extern __shared__ __align__(16) unsigned char sp_smem[];
  uint64_t *a = reinterpret_cast<uint64_t *>(sp_smem);
  const int b = blockIdx.x, tid = threadIdx.x;
  if (!large_segment(v, b)) return;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int64_t nb = x_hi - x_lo;
  const uint64_t *src = v.pairs + v.pptr[b];
  // 32 samples per bucket (a power of two between 1024 and SP_SAMPLE): one pair from every stretch of
  // nb / samples pairs, at a position that varies from stretch to stretch
  const int nbk = bucket_count_of(nb);
  int slog = 10;
  while ((1 << slog) < 32 * nbk && (1 << slog) < SP_SAMPLE) ++slog;
  const int samples = 1 << slog;
  for (int i = tid; i < samples; i += SP_THREADS) {
    const int64_t lo = nb * i / samples, hi = nb * (i + 1) / samples;
    const int64_t span = hi > lo ? hi - lo : 1;
    a[sp_pad(i)] = src[lo + (int64_t)((uint32_t)i * 2654435761u % (uint64_t)span)];
  }
  smem_bitonic_blocked(a, slog, 0, 1, slog, tid, SP_THREADS);
  const int64_t li = v.lptr[b];
  for (int j = tid; j < SP_MAX_BUCKETS; j += SP_THREADS) {
    if (j < nbk - 1) v.split[li * SP_MAX_BUCKETS + j] = a[sp_pad((int)((int64_t)(j + 1) * samples / nbk))];
    v.bcount[li * SP_MAX_BUCKETS + j] = 0;
  }
}

__global__ void __launch_bounds__(SP_THREADS)
sp_count_kernel(const int64_t *__restrict__ ptr, int64_t rows, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  __shared__ uint64_t split_s[SP_MAX_BUCKETS];
  __shared__ int hist[SP_MAX_BUCKETS];
  const int b = blockIdx.y, tid = threadIdx.x;
  if (!large_segment(v, b)) return;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int64_t nb = x_hi - x_lo, li = v.lptr[b];
  const int nbk = bucket_count_of(nb);
  for (int j = tid; j < SP_MAX_BUCKETS; j += SP_THREADS) {
    if (j < nbk - 1) split_s[j] = v.split[li * SP_MAX_BUCKETS + j];
    hist[j] = 0;
  }
  __syncthreads();
  const uint64_t *src = v.pairs + v.pptr[b];
  for (int64_t i = (int64_t)blockIdx.x * SP_THREADS + tid; i < nb; i += (int64_t)gridDim.x * SP_THREADS)
    atomicAdd(&hist[bucket_of(split_s, nbk - 1, src[i])], 1);
  __syncthreads();
  for (int j = tid; j < nbk; j += SP_THREADS)
    if (hist[j]) atomicAdd(&v.bcount[li * SP_MAX_BUCKETS + j], hist[j]);
}

// One block per segment: bucket offsets, scatter cursors, and the segment's entries of the bucket table.
__global__ void __launch_bounds__(SP_MAX_BUCKETS)
sp_offsets_kernel(const int64_t *__restrict__ ptr, int64_t rows, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  __shared__ int scan[SP_MAX_BUCKETS], entries[SP_MAX_BUCKETS];
  __shared__ int table_base;
  const int b = blockIdx.x, t = threadIdx.x;
  if (!large_segment(v, b)) return;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int64_t nb = x_hi - x_lo, li = v.lptr[b];
  const int nbk = bucket_count_of(nb);
  const int mine = t < nbk ? v.bcount[li * SP_MAX_BUCKETS + t] : 0;
  const int pieces = (mine + SP_SORT_BLOCK - 1) / SP_SORT_BLOCK;  // 0 for an empty bucket, 1 as a rule
  scan[t] = mine;
  entries[t] = pieces;
  __syncthreads();
  for (int o = 1; o < SP_MAX_BUCKETS; o <<= 1) {
    const int a0 = t >= o ? scan[t - o] : 0, a1 = t >= o ? entries[t - o] : 0;
    __syncthreads();
    scan[t] += a0;
    entries[t] += a1;
    __syncthreads();
  }
  if (t == SP_MAX_BUCKETS - 1) table_base = atomicAdd(v.table_count, entries[t]);
  __syncthreads();
  const int start = scan[t] - mine;
  if (t < nbk) {
    v.boffset[li * (SP_MAX_BUCKETS + 1) + t] = start;
    v.bcursor[li * SP_MAX_BUCKETS + t] = start;
  }
  if (t == 0) v.boffset[li * (SP_MAX_BUCKETS + 1) + nbk] = (int)nb;
  int e = table_base + entries[t] - pieces;
  for (int p = 0; p < pieces; ++p, ++e) {
    if (e >= v.table_cap) break;  // cannot happen: the table is sized for every bucket and every piece
    const int first = start + p * SP_SORT_BLOCK;
    const int size = mine - p * SP_SORT_BLOCK < SP_SORT_BLOCK ? mine - p * SP_SORT_BLOCK : SP_SORT_BLOCK;
    v.table[4 * e + 0] = b;
    v.table[4 * e + 1] = first;
    v.table[4 * e + 2] = size;
    v.table[4 * e + 3] = first + size == nb ? 1 : 0;
  }
}

// Scatter with one global atomic per (thread block, bucket): a block takes stretches of 4096 pairs, ranks
// them within their buckets in shared memory, reserves a range of every bucket, then writes.
__global__ void __launch_bounds__(SP_THREADS)
sp_scatter_kernel(const int64_t *__restrict__ ptr, int64_t rows, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  __shared__ uint64_t split_s[SP_MAX_BUCKETS];
  __shared__ int hist[SP_MAX_BUCKETS], base[SP_MAX_BUCKETS];
  constexpr int PER = 4;
  const int b = blockIdx.y, tid = threadIdx.x;
  if (!large_segment(v, b)) return;
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int64_t nb = x_hi - x_lo, li = v.lptr[b];
  const int nbk = bucket_count_of(nb);
  for (int j = tid; j < nbk - 1; j += SP_THREADS) split_s[j] = v.split[li * SP_MAX_BUCKETS + j];
  const uint64_t *src = v.pairs + v.pptr[b];
  uint64_t *dst = v.pairs2 + x_lo;  // a segment's scattered pairs take the place of its rows
  for (int64_t t0 = (int64_t)blockIdx.x * (SP_THREADS * PER); t0 < nb; t0 += (int64_t)gridDim.x * (SP_THREADS * PER)) {
    for (int j = tid; j < SP_MAX_BUCKETS; j += SP_THREADS) hist[j] = 0;
    __syncthreads();
    uint64_t pair[PER];
    int bucket[PER], rank[PER];
#pragma unroll
    for (int u = 0; u < PER; ++u) {
      const int64_t i = t0 + u * SP_THREADS + tid;
      bucket[u] = -1;
      if (i < nb) {
        pair[u] = src[i];
        bucket[u] = bucket_of(split_s, nbk - 1, pair[u]);
        rank[u] = atomicAdd(&hist[bucket[u]], 1);
      }
    }
    __syncthreads();
    for (int j = tid; j < nbk; j += SP_THREADS)
      base[j] = hist[j] ? atomicAdd(&v.bcursor[li * SP_MAX_BUCKETS + j], hist[j]) : 0;
    __syncthreads();
#pragma unroll
    for (int u = 0; u < PER; ++u)
      if (bucket[u] >= 0) dst[base[bucket[u]] + rank[u]] = pair[u];
    __syncthreads();
  }
}

// One block per entry of the bucket table: sort the bucket in shared memory, write its part of the sorted copy.
template <int DIM>
__global__ void __launch_bounds__(SP_THREADS)
sp_bucket_sort_kernel(const float *__restrict__ pts, const int64_t *__restrict__ ptr, int64_t rows,
                      const float *__restrict__ box, int points, SpatialView v) {
  if (*v.bad) return;  // overlapping segments: see sp_layout_kernel
  extern __shared__ __align__(16) unsigned char sp_smem[];
  uint64_t *a = reinterpret_cast<uint64_t *>(sp_smem);
  __shared__ float red[32];
  const int e = blockIdx.x, tid = threadIdx.x;
  if (e >= *v.table_count || e >= v.table_cap) return;
  const int b = v.table[4 * e], first = v.table[4 * e + 1], size = v.table[4 * e + 2], last = v.table[4 * e + 3];
  int64_t x_lo, x_hi;
  seg_rows_clamped(ptr, rows, b, x_lo, x_hi);
  const int64_t nb = x_hi - x_lo;
  const uint64_t *src = v.pairs2 + x_lo + first;
  int plog = 0;
  while ((1 << plog) < size) ++plog;
  const int p2 = 1 << plog;
  const bool blocked = p2 >= 1024;
  for (int i = tid; i < p2; i += SP_THREADS) a[blocked ? sp_pad(i) : i] = i < size ? src[i] : ~0ull;
  if (blocked)
    smem_bitonic_blocked(a, plog, 0, 1, plog, tid, SP_THREADS);
  else if (p2 > 1)
    smem_bitonic(a, p2, 0, 2, p2, tid, SP_THREADS);
  else
    __syncthreads();
  float lo[DIM], scale[DIM], centre[DIM];
  box_scale<DIM>(box + (int64_t)b * 2 * DIM, lo, scale, centre);
  const int64_t s_lo = v.sptr[b];
  float wmax = 0.f;
  bool bad = false;
  for (int j = tid; j < size; j += SP_THREADS) {
    const float wv = emit_position<DIM>(v, pts, x_lo, s_lo + first + j, a[blocked ? sp_pad(j) : j], true, points != 0, centre);
    bad |= !(wv < 1e30f);
    wmax = fmaxf(wmax, wv);
  }
  if (last) {
    const int64_t padded = (nb + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
    for (int64_t j = nb + tid; j < padded; j += SP_THREADS)
      (void)emit_position<DIM>(v, pts, x_lo, s_lo + j, 0ull, false, points != 0, centre);
  }
  if (points) publish_wmax(wmax, bad, v.stat + 2 * b, red);
}

// ---- host side -------------------------------------------------------------------------------------------
template <int DIM>
static int spatial_sort_dim(const float *pts, const int64_t *ptr, int64_t segs, int64_t rows, const float *box_from,
                            bool points, int64_t max_segment_rows, SpatialView *v, cudaStream_t stream) {
  const size_t sort_smem = (size_t)SP_SORT_SMEM_KEYS * 8;
  static unsigned long long done_small = 0ull, done_block = 0ull;
  B200C_CUDA(opt_in_shared_memory(sp_small_kernel<DIM>, sort_smem, done_small));
  sp_layout_kernel<<<1, SP_THREADS, 0, stream>>>(ptr, (int)segs, rows, pairs_small_cap(rows), DIM, v->sptr, v->pptr,
                                                 v->lptr, v->box, v->stat, box_from == nullptr ? 1 : 0, v->table_count, v->bad);
  B200C_LAUNCH_CHECK("sp_layout_kernel");
  sp_small_kernel<DIM><<<(unsigned)segs, SP_THREADS, sort_smem, stream>>>(pts, ptr, (int)segs, rows, box_from,
                                                                           points ? 1 : 0, *v);
  B200C_LAUNCH_CHECK("sp_small_kernel");
  if (max_segment_rows <= SP_SORT_BLOCK) return B200C_OK;

  // segments above one sort block: at most rows / SP_SORT_BLOCK of them exist
  B200C_CUDA(opt_in_shared_memory(sp_sort_block_kernel, sort_smem, done_block));
  const float *box = box_from ? box_from : v->box;
  const int64_t parts64 = (rows / segs + 4 * SP_THREADS - 1) / (4 * SP_THREADS);
  const unsigned parts = (unsigned)(parts64 < 1 ? 1 : (parts64 > 64 ? 64 : parts64));
  const dim3 grid(parts, (unsigned)segs);
  if (box_from == nullptr) {
    sp_box_kernel<DIM><<<grid, SP_THREADS, 0, stream>>>(pts, ptr, rows, *v);
    B200C_LAUNCH_CHECK("sp_box_kernel");
  }
  sp_keys_kernel<DIM><<<grid, SP_THREADS, 0, stream>>>(pts, ptr, rows, box, *v);
  B200C_LAUNCH_CHECK("sp_keys_kernel");
  if (max_segment_rows <= SP_BUCKET_MAX_ROWS) {
    static unsigned long long done_sample = 0ull, done_bucket = 0ull;
    B200C_CUDA(opt_in_shared_memory(sp_sample_kernel, sort_smem, done_sample));
    B200C_CUDA(opt_in_shared_memory(sp_bucket_sort_kernel<DIM>, sort_smem, done_bucket));
    sp_sample_kernel<<<(unsigned)segs, SP_THREADS, sort_smem, stream>>>(ptr, rows, *v);
    B200C_LAUNCH_CHECK("sp_sample_kernel");
    sp_count_kernel<<<grid, SP_THREADS, 0, stream>>>(ptr, rows, *v);
    B200C_LAUNCH_CHECK("sp_count_kernel");
    sp_offsets_kernel<<<(unsigned)segs, SP_MAX_BUCKETS, 0, stream>>>(ptr, rows, *v);
    B200C_LAUNCH_CHECK("sp_offsets_kernel");
    sp_scatter_kernel<<<grid, SP_THREADS, 0, stream>>>(ptr, rows, *v);
    B200C_LAUNCH_CHECK("sp_scatter_kernel");
    sp_bucket_sort_kernel<DIM><<<(unsigned)v->table_cap, SP_THREADS, sort_smem, stream>>>(pts, ptr, rows, box,
                                                                                        points ? 1 : 0, *v);
    B200C_LAUNCH_CHECK("sp_bucket_sort_kernel");
    return B200C_OK;
  }
  const int64_t max_blocks = 2 * rows / SP_SORT_BLOCK + 1;  // padded sizes are below twice the row counts
  sp_sort_block_kernel<<<(unsigned)max_blocks, SP_THREADS, sort_smem, stream>>>(*v, (int)segs, 0);
  B200C_LAUNCH_CHECK("sp_sort_block_kernel");
  int64_t top = SP_SORT_BLOCK;
  while (top < max_segment_rows) top <<= 1;
  const int64_t exchanges = max_blocks * (SP_SORT_BLOCK / 2);
  for (int64_t size = 2 * SP_SORT_BLOCK; size <= top; size <<= 1) {
    for (int64_t stride = size >> 1; stride >= SP_SORT_BLOCK; stride >>= 1) {
      sp_sort_global_kernel<<<(unsigned)((exchanges + 255) / 256), 256, 0, stream>>>(*v, (int)segs, size, stride);
      B200C_LAUNCH_CHECK("sp_sort_global_kernel");
    }
    sp_sort_block_kernel<<<(unsigned)max_blocks, SP_THREADS, sort_smem, stream>>>(*v, (int)segs, size);
    B200C_LAUNCH_CHECK("sp_sort_block_kernel");
  }
  sp_emit_kernel<DIM><<<grid, SP_THREADS, 0, stream>>>(pts, ptr, rows, box, points ? 1 : 0, *v);
  B200C_LAUNCH_CHECK("sp_emit_kernel");
  return B200C_OK;
}

int launch_spatial_sort(const float *pts, const int64_t *ptr, int64_t segs, int64_t rows, int dim,
                        const float *box_from, bool points, int64_t max_segment_rows, SpatialView *v,
                        cudaStream_t stream) {
  if (max_segment_rows <= 0 || max_segment_rows > rows) max_segment_rows = rows;
  switch (dim) {
    case 1: return spatial_sort_dim<1>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
    case 2: return spatial_sort_dim<2>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
    case 3: return spatial_sort_dim<3>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
    case 4: return spatial_sort_dim<4>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
    case 5: return spatial_sort_dim<5>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
    case 6: return spatial_sort_dim<6>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
    case 7: return spatial_sort_dim<7>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
    case 8: return spatial_sort_dim<8>(pts, ptr, segs, rows, box_from, points, max_segment_rows, v, stream);
  }
  set_error("spatial sort called with dim=%d", dim);
  return B200C_ERR_INVALID;
}

}  // namespace b200c
