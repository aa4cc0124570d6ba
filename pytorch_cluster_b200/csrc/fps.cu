// Farthest point sampling — replaces fps_kernel + the launch in fps_cuda
// (csrc/cuda/fps_cuda.cu:9-68, 70-112).
//
// The algorithm is sequential per segment: sample m is the point whose distance to the samples
// 0..m-1 is largest, so every sample costs one pass over the segment's running minimum distances
// plus an arg-max reduction, and the reduction's latency bounds the step.  One CTA of 1024
// threads owns a segment.  The reference re-reads the coordinates and the running distances from
// global memory in every step; here both live in shared memory for the whole call when the
// segment fits (up to ~14 000 three-dimensional fp32 points in 200 KB; one plane per feature, so
// lane-strided reads are conflict free), and only larger segments fall back to global memory / L2
// with the running distances in the caller's workspace.  For fp32 points of up to 8 features a
// segment of up to 8192 (DIM <= 3) or 4096 points additionally keeps its coordinates and running
// distances in registers (thread t owns points t, t + 1024, ...; shared memory only serves the
// broadcast of the newest sample's coordinates), candidates travel as 64-bit keys
// (distance bits << 32 | inverted tie rank) and a step is: 3 broadcast loads, 8 distance updates
// per thread, two REDUX instructions per warp, one __syncthreads, and the same two REDUX again
// on the 32 partial keys in every warp (double buffered, so one barrier per step).
//
// Semantics kept (fps_cuda.cu:32-66): running distance starts at 5e4 and is min(previous, new)
// with fmin semantics; new = sum over features of (old_d - p_d)^2 accumulated in order (fused for
// float / double, every operation rounded for the 16-bit types); a candidate must be > -1 (NaN
// never is; none: index 0); among equal maxima the reference's 256-thread stride and "keep the
// lower thread on ties" reduction pick the smallest ((index - segment start) mod 256, index).
#include <cstdint>
#include "common.cuh"
#include "launchers.h"

namespace b200c {

constexpr int FPS_THREADS = 1024;
constexpr int FPS_REF_STRIDE = 256;  // THREADS of the reference kernel: defines its tie order
constexpr size_t FPS_SMEM_BUDGET = 200 * 1024;

template <typename T>
__device__ __forceinline__ bool fps_better(T d, int64_t i, T bd, int64_t bi, int64_t seg_lo) {
  if (d > bd) return true;
  if (!(d == bd)) return false;
  const int64_t a = (i - seg_lo) & (FPS_REF_STRIDE - 1), b = (bi - seg_lo) & (FPS_REF_STRIDE - 1);
  return a < b || (a == b && i < bi);
}

template <typename T>
__device__ __forceinline__ T fmin_t(T a, T b) {
  if constexpr (sizeof(T) == 4)
    return fminf(a, b);
  else
    return fmin(a, b);
}

// Maximum of 64-bit keys over a warp as two 32-bit REDUX steps: high words first, then the low
// words of the lanes that hold the maximal high word.
__device__ __forceinline__ void warp_max_key(uint32_t &hi, uint32_t &lo) {
  const uint32_t mh = __reduce_max_sync(FULL_MASK, hi);
  const uint32_t ml = __reduce_max_sync(FULL_MASK, hi == mh ? lo : 0u);
  hi = mh;
  lo = ml;
}

// DIM > 0: compile-time feature count with the register-resident path for segments of up to
// FPS_THREADS * PT points (fp32 without 16-bit rounding only); DIM == 0: run-time feature count.
template <typename T, int RND, int DIM, int PT>
__global__ void __launch_bounds__(FPS_THREADS, 1)
fps_kernel(const T *__restrict__ src, const int64_t *__restrict__ ptr, const int64_t *__restrict__ out_ptr,
           const int64_t *__restrict__ start, int dim, T *__restrict__ dist_global, int64_t *__restrict__ out,
           int64_t chip_capacity, int64_t skip_above) {
  extern __shared__ __align__(16) unsigned char smem_fps[];
  __shared__ T part_d[2][32];
  __shared__ int64_t part_i[2][32];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int b = blockIdx.x;
  const int64_t seg_lo = ptr[b], seg_hi = ptr[b + 1];
  const int64_t npts = seg_hi - seg_lo;
  const int64_t o_lo = out_ptr[b], o_hi = out_ptr[b + 1];
  if (npts <= 0 || o_hi <= o_lo || npts > skip_above) return;  // larger segments: the caller runs fps_multi_kernel

  if constexpr (DIM > 0 && RND == 0 && sizeof(T) == 4) {
    if (npts <= (int64_t)FPS_THREADS * PT) {
      __shared__ uint2 part_key[2][32];
      const int n = (int)npts;
      const int plane = (n + 3) / 4 * 4;
      float *planes = reinterpret_cast<float *>(smem_fps);
      for (int f = tid; f < n * DIM; f += FPS_THREADS) {
        const int p = f / DIM, d = f - p * DIM;
        planes[d * plane + p] = src[seg_lo * DIM + f];
      }
      __syncthreads();
      // keys: distance bits << 32 | 0xffffffff - ((offset mod 256) << 24 | offset); 0 = "no point"
      float c[PT][DIM], dmin[PT];
      uint32_t valid_mask = 0u;
#pragma unroll
      for (int j = 0; j < PT; ++j) {
        const int rel = tid + j * FPS_THREADS;
        const bool valid = rel < n;
#pragma unroll
        for (int d = 0; d < DIM; ++d) c[j][d] = valid ? planes[d * plane + rel] : 0.f;
        dmin[j] = 5e4f;
        valid_mask |= valid ? 1u << j : 0u;
      }
      int old_rel = (int)(start != nullptr ? start[b] : 0);
      if (tid == 0) out[o_lo] = seg_lo + old_rel;
      for (int64_t m = o_lo + 1; m < o_hi; ++m) {
        const int buf = (int)(m & 1);
        float q[DIM];
#pragma unroll
        for (int d = 0; d < DIM; ++d) q[d] = planes[d * plane + old_rel];
        // A thread's points t, t + 1024, ... share (offset mod 256), so among them the reference's
        // order of equal distances is the index order: keep the first strict maximum, without
        // branches.  Slots past the segment's end come last and hold bits 0, so they never replace
        // a real point.
        uint32_t hi = 0u;
        int jbest = 0;
#pragma unroll
        for (int j = 0; j < PT; ++j) {
          float dd = 0.f;
#pragma unroll
          for (int d = 0; d < DIM; ++d) dd = sq_accumulate<0>(q[d], c[j][d], dd);
          dd = fminf(dmin[j], dd);
          dmin[j] = dd;
          // dd >= 0 here (a NaN sum is dropped by fminf), so its bit pattern orders like its value
          const uint32_t bits = valid_mask & (1u << j) ? __float_as_uint(dd) : 0u;
          jbest = bits > hi ? j : jbest;
          hi = bits > hi ? bits : hi;
        }
        const int rel_best = tid + jbest * FPS_THREADS;
        uint32_t lo = tid < n ? 0xffffffffu - ((uint32_t)(rel_best & (FPS_REF_STRIDE - 1)) << 24 | (uint32_t)rel_best) : 0u;
        warp_max_key(hi, lo);
        if (lane == 0) part_key[buf][warp] = make_uint2(hi, lo);
        __syncthreads();
        const uint2 pk = part_key[buf][lane];
        hi = pk.x;
        lo = pk.y;
        warp_max_key(hi, lo);
        old_rel = (int)((0xffffffffu - lo) & 0x00ffffffu);
        if (tid == 0) out[m] = seg_lo + old_rel;
      }
      return;
    }
  }

  // where coordinates and running distances live
  const bool on_chip = npts <= chip_capacity;
  const T *coords;
  int64_t pstride, dstride;
  T *dist;
  if (on_chip) {
    const int64_t plane = (npts + 3) / 4 * 4;
    T *planes = reinterpret_cast<T *>(smem_fps);
    dist = planes + (int64_t)dim * plane;
    for (int64_t f = tid; f < npts * dim; f += FPS_THREADS) {
      const int64_t p = f / dim;
      const int d = (int)(f - p * dim);
      planes[d * plane + p] = src[seg_lo * dim + f];
    }
    coords = planes;
    pstride = 1;
    dstride = plane;
  } else {
    coords = src + seg_lo * dim;
    pstride = dim;
    dstride = 1;
    dist = dist_global + seg_lo;
  }
  const T init = rnd16<RND>((T)5e4);
  for (int64_t p = tid; p < npts; p += FPS_THREADS) dist[p] = init;

  int64_t old = seg_lo + (start != nullptr ? start[b] : 0);
  if (tid == 0) out[o_lo] = old;
  __syncthreads();

  for (int64_t m = o_lo + 1; m < o_hi; ++m) {
    const int buf = (int)(m & 1);
    const T *q = coords + (old - seg_lo) * pstride;
    T best = (T)-1;
    int64_t best_idx = 0;
    for (int64_t p = tid; p < npts; p += FPS_THREADS) {
      const T *c = coords + p * pstride;
      T dd = (T)0;
      for (int d = 0; d < dim; ++d) dd = sq_accumulate<RND>(q[d * dstride], c[d * dstride], dd);
      dd = fmin_t(dist[p], dd);
      dist[p] = dd;
      if (fps_better(dd, seg_lo + p, best, best_idx, seg_lo)) {
        best = dd;
        best_idx = seg_lo + p;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const T od = __shfl_xor_sync(FULL_MASK, best, o);
      const int64_t oi = __shfl_xor_sync(FULL_MASK, best_idx, o);
      if (fps_better(od, oi, best, best_idx, seg_lo)) {
        best = od;
        best_idx = oi;
      }
    }
    if (lane == 0) {
      part_d[buf][warp] = best;
      part_i[buf][warp] = best_idx;
    }
    __syncthreads();
    best = part_d[buf][lane];
    best_idx = part_i[buf][lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const T od = __shfl_xor_sync(FULL_MASK, best, o);
      const int64_t oi = __shfl_xor_sync(FULL_MASK, best_idx, o);
      if (fps_better(od, oi, best, best_idx, seg_lo)) {
        best = od;
        best_idx = oi;
      }
    }
    // no candidate above -1 anywhere (all distances NaN): the reference's untouched index 0
    old = best > (T)-1 ? best_idx : 0;
    if (tid == 0) out[m] = old;
  }
}

// ---- one large segment on many SMs ------------------------------------------------------------------
// A segment too large for one CTA's registers is spread over G CTAs of one cooperative launch (all
// resident at once, one per SM): CTA g keeps points [g * 1024 * PT, (g + 1) * 1024 * PT) of the
// segment in registers.  A step: every CTA finds its best key as above and publishes it, with the
// coordinates of that point, in a slot of a double-buffered array in global memory; a counter in
// global memory serves as the barrier (arrive: fence + atomic add; wait: bounded polling for
// G * step); then every CTA reads the G slots, reduces them the same way and continues with the
// winner's coordinates.  Two slot arrays suffice: a CTA can write step s + 2 only after all CTAs
// arrived at step s + 1, i.e. after they read step s.  On a timeout the kernel sets an error flag
// and returns; the host then reports the failure.
struct FpsSlot {
  unsigned long long key;  // distance bits << 32 | 0xffffffff - ((offset mod 256) << 24 | offset); 0 = none
  float c[8];              // coordinates of that point
  unsigned long long pad;
};

constexpr int FPS_MULTI_SPIN_LIMIT = 1 << 20;  // polls of an L2 word: well under a second; co-residency is guaranteed by the cooperative launch, this is a safety net

template <int DIM, int PT>
__global__ void __launch_bounds__(FPS_THREADS, 1)
fps_multi_kernel(const float *__restrict__ src, int64_t seg_lo, int64_t npts, int64_t start_offset, int64_t count,
                 int64_t *__restrict__ out, FpsSlot *__restrict__ slots /* [2][gridDim.x] */,
                 unsigned *__restrict__ counter, int *__restrict__ error_flag) {
  __shared__ uint2 part_key[32];
  __shared__ float q_s[8];
  __shared__ int winner_s;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = blockIdx.x, G = gridDim.x;
  const int64_t cta_lo = (int64_t)g * FPS_THREADS * PT;  // first point (segment-relative) of this CTA

  float c[PT][DIM], dmin[PT];
  uint32_t valid_mask = 0u;
#pragma unroll
  for (int j = 0; j < PT; ++j) {
    const int64_t rel = cta_lo + tid + (int64_t)j * FPS_THREADS;
    const bool valid = rel < npts;
#pragma unroll
    for (int d = 0; d < DIM; ++d) c[j][d] = valid ? src[(seg_lo + rel) * DIM + d] : 0.f;
    dmin[j] = 5e4f;
    valid_mask |= valid ? 1u << j : 0u;
  }
  float q[DIM];
#pragma unroll
  for (int d = 0; d < DIM; ++d) q[d] = src[(seg_lo + start_offset) * DIM + d];
  if (g == 0 && tid == 0) out[0] = seg_lo + start_offset;

  for (int64_t m = 1; m < count; ++m) {
    const int buf = (int)(m & 1);
    // local best: first strict maximum per thread (see fps_kernel), then the CTA's maximum key
    uint32_t hi = 0u;
    int jbest = 0;
#pragma unroll
    for (int j = 0; j < PT; ++j) {
      float dd = 0.f;
#pragma unroll
      for (int d = 0; d < DIM; ++d) dd = sq_accumulate<0>(q[d], c[j][d], dd);
      dd = fminf(dmin[j], dd);
      dmin[j] = dd;
      const uint32_t bits = valid_mask & (1u << j) ? __float_as_uint(dd) : 0u;
      jbest = bits > hi ? j : jbest;
      hi = bits > hi ? bits : hi;
    }
    const int64_t rel_best = cta_lo + tid + (int64_t)jbest * FPS_THREADS;
    uint32_t lo = (valid_mask & 1u)
                      ? 0xffffffffu - ((uint32_t)(rel_best & (FPS_REF_STRIDE - 1)) << 24 | (uint32_t)rel_best)
                      : 0u;
    const uint32_t my_hi = hi, my_lo = lo;
    warp_max_key(hi, lo);
    if (lane == 0) part_key[warp] = make_uint2(hi, lo);
    __syncthreads();
    {
      const uint2 pk = part_key[lane];
      hi = pk.x;
      lo = pk.y;
      warp_max_key(hi, lo);
    }
    // the thread that owns the CTA's best point publishes key and coordinates (keys are unique: the
    // low word encodes the point), then the CTA arrives at the step's barrier
    if (my_hi == hi && my_lo == lo && lo != 0u) {
      FpsSlot *slot = slots + (size_t)buf * G + g;
#pragma unroll
      for (int d = 0; d < DIM; ++d) {
        float v = c[0][d];
#pragma unroll
        for (int j = 1; j < PT; ++j) v = jbest == j ? c[j][d] : v;
        slot->c[d] = v;
      }
      slot->key = ((unsigned long long)hi << 32) | lo;
      __threadfence();
      atomicAdd(counter, 1u);
    } else if (lo == 0u && tid == 0) {
      // a CTA without points cannot occur (the grid covers the segment), but it must not stall the others
      slots[(size_t)buf * G + g].key = 0ull;
      __threadfence();
      atomicAdd(counter, 1u);
    }
    // wait for all G arrivals of this step (bounded), then pick the winner among the G slots
    if (tid == 0) {
      const unsigned want = (unsigned)((unsigned long long)G * (unsigned long long)m);
      int ok = 0;
      for (int it = 0; it < FPS_MULTI_SPIN_LIMIT; ++it) {
        const unsigned seen = *reinterpret_cast<volatile unsigned *>(counter);
        if ((int)(seen - want) >= 0) {
          ok = 1;
          break;
        }
      }
      __threadfence();
      winner_s = ok ? 0 : -1;
    }
    __syncthreads();
    if (winner_s < 0) {
      if (tid == 0) *error_flag = 1;
      return;
    }
    unsigned long long key = 0ull;
    if (tid < G) key = __ldcg(&slots[(size_t)buf * G + tid].key);
    hi = (uint32_t)(key >> 32);
    lo = (uint32_t)key;
    const uint32_t slot_hi = hi, slot_lo = lo;
    warp_max_key(hi, lo);
    __syncthreads();  // part_key is reused
    if (lane == 0) part_key[warp] = make_uint2(hi, lo);
    __syncthreads();
    {
      const uint2 pk = part_key[lane];
      hi = pk.x;
      lo = pk.y;
      warp_max_key(hi, lo);
    }
    if (tid < G && slot_hi == hi && slot_lo == lo && lo != 0u) {
      const FpsSlot *slot = slots + (size_t)buf * G + tid;
#pragma unroll
      for (int d = 0; d < DIM; ++d) q_s[d] = __ldcg(&slot->c[d]);
    }
    __syncthreads();
#pragma unroll
    for (int d = 0; d < DIM; ++d) q[d] = q_s[d];
    const int64_t old_rel = (int64_t)((0xffffffffu - lo) & 0x00ffffffu);
    if (g == 0 && tid == 0) out[m] = seg_lo + (lo != 0u ? old_rel : -seg_lo);
  }
}

template <typename T, int RND, int DIM = 0, int PT = 1>
static int launch_fps_t(const void *src, const int64_t *ptr, const int64_t *out_ptr, const int64_t *start,
                        int64_t num_segments, int dim, void *dist, int64_t *out, cudaStream_t stream,
                        int64_t skip_above) {
  auto kern = fps_kernel<T, RND, DIM, PT>;
  static unsigned long long configured = 0ull;  // devices on which the shared-memory opt-in is done
  B200C_CUDA(opt_in_shared_memory(kern, FPS_SMEM_BUDGET, configured));
  // points of (dim + 1) values each, planes padded to 4 elements
  const int64_t capacity = (int64_t)(FPS_SMEM_BUDGET / sizeof(T) - 4 * (size_t)dim) / (dim + 1);
  kern<<<(unsigned)num_segments, FPS_THREADS, FPS_SMEM_BUDGET, stream>>>(
      (const T *)src, ptr, out_ptr, start, dim, (T *)dist, out, capacity > 0 ? capacity : 0, skip_above);
  B200C_LAUNCH_CHECK("fps_kernel");
  return B200C_OK;
}

}  // namespace b200c

using namespace b200c;

static size_t fps_align256(size_t v) { return (v + 255) / 256 * 256; }

extern "C" size_t b200c_fps_workspace_bytes(int64_t n, int64_t dim, int dtype) {
  if (n < 0 || dim < 1) return 0;
  const bool h = dtype == B200C_F16 || dtype == B200C_BF16;
  const size_t elem = dtype == B200C_F64 ? 8 : 4;
  return fps_align256((size_t)n * elem) + (h ? fps_align256((size_t)n * dim * 4) : 0);
}

static int fps_impl(const void *src, const int64_t *ptr, const int64_t *out_ptr, const int64_t *start,
                    int64_t num_segments, int64_t n, int64_t dim, int dtype, int64_t *out, void *workspace,
                    size_t workspace_bytes, b200c_stream_t stream_, int64_t skip_above) {
  cudaStream_t stream = (cudaStream_t)stream_;
  B200C_CHECK_ARG(n >= 0 && dim >= 1 && dim <= 0x7fffffffLL / 4, "Input mismatch");
  B200C_CHECK_ARG(num_segments >= 0 && num_segments <= 0x7fffffffLL, "Input mismatch");
  B200C_CHECK_ARG(dtype >= B200C_F32 && dtype <= B200C_BF16, "unsupported dtype");
  if (num_segments == 0 || n == 0) return B200C_OK;
  B200C_CHECK_ARG(src && ptr && out_ptr && out, "null pointer");
  int dev = 0, major = 0;
  B200C_CUDA(cudaGetDevice(&dev));
  B200C_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) {
    set_error("device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
    return B200C_ERR_DEVICE;
  }
  const size_t need = b200c_fps_workspace_bytes(n, dim, dtype);
  if (workspace == nullptr || workspace_bytes < need) {
    set_error("fps workspace too small: %zu < %zu", workspace_bytes, need);
    return B200C_ERR_WORKSPACE;
  }
  void *dist = workspace;
  if (dtype == B200C_F16 || dtype == B200C_BF16) {
    float *wide = (float *)((char *)workspace + fps_align256((size_t)n * 4));
    int st = launch_widen16(src, n * dim, dtype, wide, stream);
    if (st != B200C_OK) return st;
    return dtype == B200C_F16
               ? launch_fps_t<float, 1>(wide, ptr, out_ptr, start, num_segments, (int)dim, dist, out, stream, skip_above)
               : launch_fps_t<float, 2>(wide, ptr, out_ptr, start, num_segments, (int)dim, dist, out, stream, skip_above);
  }
  if (dtype == B200C_F64)
    return launch_fps_t<double, 0>(src, ptr, out_ptr, start, num_segments, (int)dim, dist, out, stream, skip_above);
  switch (dim) {
    case 1: return launch_fps_t<float, 0, 1, 8>(src, ptr, out_ptr, start, num_segments, 1, dist, out, stream, skip_above);
    case 2: return launch_fps_t<float, 0, 2, 8>(src, ptr, out_ptr, start, num_segments, 2, dist, out, stream, skip_above);
    case 3: return launch_fps_t<float, 0, 3, 8>(src, ptr, out_ptr, start, num_segments, 3, dist, out, stream, skip_above);
    case 4: return launch_fps_t<float, 0, 4, 4>(src, ptr, out_ptr, start, num_segments, 4, dist, out, stream, skip_above);
    case 5: return launch_fps_t<float, 0, 5, 4>(src, ptr, out_ptr, start, num_segments, 5, dist, out, stream, skip_above);
    case 6: return launch_fps_t<float, 0, 6, 4>(src, ptr, out_ptr, start, num_segments, 6, dist, out, stream, skip_above);
    case 7: return launch_fps_t<float, 0, 7, 4>(src, ptr, out_ptr, start, num_segments, 7, dist, out, stream, skip_above);
    case 8: return launch_fps_t<float, 0, 8, 4>(src, ptr, out_ptr, start, num_segments, 8, dist, out, stream, skip_above);
  }
  return launch_fps_t<float, 0>(src, ptr, out_ptr, start, num_segments, (int)dim, dist, out, stream, skip_above);
}

extern "C" int b200c_fps(const void *src, const int64_t *ptr, const int64_t *out_ptr, const int64_t *start,
                         int64_t num_segments, int64_t n, int64_t dim, int dtype, int64_t *out, void *workspace,
                         size_t workspace_bytes, b200c_stream_t stream) {
  return fps_impl(src, ptr, out_ptr, start, num_segments, n, dim, dtype, out, workspace, workspace_bytes, stream,
                  INT64_MAX);
}

extern "C" int b200c_fps_up_to(const void *src, const int64_t *ptr, const int64_t *out_ptr, const int64_t *start,
                               int64_t num_segments, int64_t n, int64_t dim, int dtype, int64_t max_segment_points,
                               int64_t *out, void *workspace, size_t workspace_bytes, b200c_stream_t stream) {
  return fps_impl(src, ptr, out_ptr, start, num_segments, n, dim, dtype, out, workspace, workspace_bytes, stream,
                  max_segment_points);
}

// ---- one large segment on many SMs ----

static int fps_multi_points_per_cta(int64_t dim) { return FPS_THREADS * (dim <= 3 ? 8 : 4); }

extern "C" int64_t b200c_fps_large_segment_max_points(int64_t dim, int dtype) {
  if (dtype != B200C_F32 || dim < 1 || dim > 8) return 0;
  int dev = 0, sms = 0, coop = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev) != cudaSuccess || !coop) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  // one CTA per SM (1024 threads holding their points in registers), at most the 256 CTAs the
  // exchange slots in the workspace are laid out for
  const int64_t ctas = sms < 256 ? sms : 256;
  const int64_t cap = ctas * fps_multi_points_per_cta(dim);
  return cap < (1 << 24) ? cap : (1 << 24);  // offsets travel in 24 bits of the key
}

extern "C" size_t b200c_fps_large_segment_workspace_bytes(void) { return 2 * 256 * sizeof(FpsSlot) + 512; }

template <int DIM, int PT>
static int launch_fps_multi(const float *src, int64_t seg_lo, int64_t npts, int64_t start_offset, int64_t count,
                            int64_t *out, void *workspace, int32_t *status, cudaStream_t stream) {
  const int G = (int)((npts + (int64_t)FPS_THREADS * PT - 1) / ((int64_t)FPS_THREADS * PT));
  // all G CTAs must be resident together: what this context can hold (fewer SMs than the device
  // has under MPS or a green context) decides, not the device's SM count alone
  int dev = 0, sms = 0, per_sm = 0;
  B200C_CUDA(cudaGetDevice(&dev));
  B200C_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  B200C_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fps_multi_kernel<DIM, PT>, FPS_THREADS, 0));
  if (G > 256 || G > FPS_THREADS || (int64_t)G > (int64_t)per_sm * sms) {
    set_error("fps: %d thread blocks cannot be resident together on this device (%d x %d)", G, per_sm, sms);
    return B200C_ERR_UNSUPPORTED;
  }
  FpsSlot *slots = (FpsSlot *)workspace;
  unsigned *counter = (unsigned *)((char *)workspace + 2 * 256 * sizeof(FpsSlot));
  B200C_CUDA(cudaMemsetAsync(counter, 0, 256, stream));
  int *error_flag = (int *)status;
  void *args[] = {(void *)&src, (void *)&seg_lo, (void *)&npts, (void *)&start_offset, (void *)&count,
                  (void *)&out, (void *)&slots, (void *)&counter, (void *)&error_flag};
  // cooperative: all G CTAs are resident at once or the launch is refused
  const cudaError_t le = cudaLaunchCooperativeKernel((const void *)fps_multi_kernel<DIM, PT>, dim3(G),
                                                     dim3(FPS_THREADS), args, 0, stream);
  if (le != cudaSuccess) {
    (void)cudaGetLastError();  // a refused launch leaves nothing enqueued; the caller may use b200c_fps
    set_error("cooperative launch of fps_multi_kernel refused: %s", cudaGetErrorString(le));
    return B200C_ERR_UNSUPPORTED;
  }
  return B200C_OK;
}

extern "C" int b200c_fps_large_segment(const void *src, int64_t seg_lo, int64_t seg_points, int64_t start_offset,
                                       int64_t count, int64_t dim, int dtype, int64_t *out, void *workspace,
                                       size_t workspace_bytes, int32_t *status, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  B200C_CHECK_ARG(src && out && status, "null pointer");
  B200C_CHECK_ARG(seg_lo >= 0 && seg_points >= 1 && count >= 1 && start_offset >= 0 && start_offset < seg_points,
                  "Input mismatch");
  const int64_t cap = b200c_fps_large_segment_max_points(dim, dtype);
  if (cap == 0 || seg_points > cap) {
    set_error("b200c_fps_large_segment covers fp32 segments of up to %lld points with up to 8 features", (long long)cap);
    return B200C_ERR_UNSUPPORTED;
  }
  if (workspace == nullptr || workspace_bytes < b200c_fps_large_segment_workspace_bytes()) {
    set_error("fps workspace too small");
    return B200C_ERR_WORKSPACE;
  }
  const float *s = (const float *)src;
  switch (dim) {
    case 1: return launch_fps_multi<1, 8>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
    case 2: return launch_fps_multi<2, 8>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
    case 3: return launch_fps_multi<3, 8>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
    case 4: return launch_fps_multi<4, 4>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
    case 5: return launch_fps_multi<5, 4>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
    case 6: return launch_fps_multi<6, 4>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
    case 7: return launch_fps_multi<7, 4>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
    default: return launch_fps_multi<8, 4>(s, seg_lo, seg_points, start_offset, count, out, workspace, status, stream);
  }
}
