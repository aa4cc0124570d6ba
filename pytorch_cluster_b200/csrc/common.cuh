// Shared device/host helpers of the sm_100a neighbour-graph kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

#include "b200_cluster.h"

namespace b200c {

constexpr unsigned FULL_MASK = 0xffffffffu;
constexpr int WARPS_PER_CTA = 8;
constexpr int CTA_THREADS = WARPS_PER_CTA * 32;

// ---- host side: status + error text ---------------------------------------------------------
void set_error(const char *fmt, ...);

#define B200C_CHECK_ARG(cond, msg)                                              \
  do {                                                                          \
    if (!(cond)) {                                                              \
      ::b200c::set_error("%s (%s)", msg, #cond);                                \
      return B200C_ERR_INVALID;                                                 \
    }                                                                           \
  } while (0)

#define B200C_CUDA(call)                                                        \
  do {                                                                          \
    cudaError_t e__ = (call);                                                   \
    if (e__ != cudaSuccess) {                                                   \
      ::b200c::set_error("%s failed: %s", #call, cudaGetErrorString(e__));      \
      return B200C_ERR_CUDA;                                                    \
    }                                                                           \
  } while (0)

// Opt a kernel in to `bytes` of dynamic shared memory on the current device.  The attribute belongs
// to the (function, device) pair, so it is set once per device: `done` is the caller's bit mask of
// devices already configured (one static per kernel instantiation; a lost update only repeats an
// idempotent call).
template <typename Kern>
static inline cudaError_t opt_in_shared_memory(Kern kern, size_t bytes, unsigned long long &done) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && ((done >> dev) & 1ull)) return cudaSuccess;
  e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess && dev < 64) done |= 1ull << dev;
  return e;
}

#define B200C_LAUNCH_CHECK(name)                                                \
  do {                                                                          \
    cudaError_t e__ = cudaGetLastError();                                       \
    if (e__ != cudaSuccess) {                                                   \
      ::b200c::set_error("launch of %s failed: %s", name,                       \
                         cudaGetErrorString(e__));                              \
      return B200C_ERR_CUDA;                                                    \
    }                                                                           \
  } while (0)

// ---- segment lookup ---------------------------------------------------------------------------
// First i in [0, num_segments) with ptr[i + 1] > row, else num_segments - 1: the rule of the
// reference's linear scan (csrc/cuda/utils.cuh:11-19), found by bisection.  ptr == nullptr
// stands for a single segment.
__device__ __forceinline__ int segment_of(const int64_t *__restrict__ ptr, int num_segments,
                                          int64_t row) {
  if (ptr == nullptr) return 0;
  int lo = 0, hi = num_segments - 1;  // answer in [lo, hi]
  while (lo < hi) {
    int mid = (lo + hi) >> 1;
    if (ptr[mid + 1] > row)
      hi = mid;
    else
      lo = mid + 1;
  }
  return lo;
}

// Row range [lo, hi) of y that the reference assigns to segment b (rows before ptr[0] fall into
// the first segment that has an end beyond them, rows at or past ptr[B] into the last one).
__device__ __forceinline__ void segment_rows(const int64_t *__restrict__ ptr, int num_segments,
                                             int64_t total, int b, int64_t &lo, int64_t &hi) {
  if (ptr == nullptr) {
    lo = 0;
    hi = total;
    return;
  }
  lo = ptr[b];
  hi = (b == num_segments - 1) ? total : ptr[b + 1];
}

__device__ __forceinline__ void segment_points(const int64_t *__restrict__ ptr, int64_t total,
                                               int b, int64_t &lo, int64_t &hi) {
  if (ptr == nullptr) {
    lo = 0;
    hi = total;
    return;
  }
  lo = ptr[b];
  hi = ptr[b + 1];
  if (lo < 0) lo = 0;
  if (hi > total) hi = total;
}

// ---- order-preserving keys -------------------------------------------------------------------
// Unsigned integers whose order equals the floating-point order of the value (negative values
// included); NaN never reaches a key.
__device__ __forceinline__ uint32_t ordered_bits(float v) {
  uint32_t b = __float_as_uint(v);
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float from_ordered_bits(uint32_t o) {
  uint32_t b = (o & 0x80000000u) ? (o & 0x7fffffffu) : ~o;
  return __uint_as_float(b);
}
__device__ __forceinline__ uint64_t ordered_bits(double v) {
  uint64_t b = (uint64_t)__double_as_longlong(v);
  return (b & 0x8000000000000000ull) ? ~b : (b | 0x8000000000000000ull);
}
__device__ __forceinline__ double from_ordered_bits(uint64_t o) {
  uint64_t b = (o & 0x8000000000000000ull) ? (o & 0x7fffffffffffffffull) : ~o;
  return __longlong_as_double((long long)b);
}

// A candidate (distance, x index) that sorts by distance, then index.
template <typename T>
struct Key;

template <>
struct Key<float> {
  uint64_t v;  // ordered distance bits in the high word, index in the low word
  __device__ __forceinline__ static Key make(float d, uint32_t idx) {
    return Key{((uint64_t)ordered_bits(d) << 32) | idx};
  }
  __device__ __forceinline__ static Key empty() { return Key{~0ull}; }
  __device__ __forceinline__ bool is_empty() const { return v == ~0ull; }
  __device__ __forceinline__ float dist() const { return from_ordered_bits((uint32_t)(v >> 32)); }
  __device__ __forceinline__ uint32_t index() const { return (uint32_t)v; }
  __device__ __forceinline__ bool less(const Key &o) const { return v < o.v; }
  __device__ __forceinline__ Key shfl_xor(int m) const {
    return Key{__shfl_xor_sync(FULL_MASK, v, m)};
  }
  __device__ __forceinline__ Key shfl(int src) const { return Key{__shfl_sync(FULL_MASK, v, src)}; }
};

template <>
struct Key<double> {
  uint64_t hi;  // ordered distance bits
  uint32_t lo;  // index
  uint32_t pad_;
  __device__ __forceinline__ static Key make(double d, uint32_t idx) {
    return Key{ordered_bits(d), idx, 0u};
  }
  __device__ __forceinline__ static Key empty() { return Key{~0ull, ~0u, 0u}; }
  __device__ __forceinline__ bool is_empty() const { return hi == ~0ull && lo == ~0u; }
  __device__ __forceinline__ double dist() const { return from_ordered_bits(hi); }
  __device__ __forceinline__ uint32_t index() const { return lo; }
  __device__ __forceinline__ bool less(const Key &o) const {
    return hi < o.hi || (hi == o.hi && lo < o.lo);
  }
  __device__ __forceinline__ Key shfl_xor(int m) const {
    return Key{__shfl_xor_sync(FULL_MASK, hi, m), __shfl_xor_sync(FULL_MASK, lo, m), 0u};
  }
  __device__ __forceinline__ Key shfl(int src) const {
    return Key{__shfl_sync(FULL_MASK, hi, src), __shfl_sync(FULL_MASK, lo, src), 0u};
  }
};

template <typename K>
__device__ __forceinline__ K key_min(const K &a, const K &b) { return b.less(a) ? b : a; }
template <typename K>
__device__ __forceinline__ K key_max(const K &a, const K &b) { return b.less(a) ? a : b; }
// One compare per exchange: keep the smaller of (mine, other) when take_min, else the larger.
template <typename K>
__device__ __forceinline__ K key_pick(const K &mine, const K &other, bool take_min) {
  return (other.less(mine) == take_min) ? other : mine;
}

// Ascending bitonic sort of one key per lane.
template <typename K>
__device__ __forceinline__ K warp_sort32(K v, int lane) {
#pragma unroll
  for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      K o = v.shfl_xor(stride);
      bool lower = (lane & stride) == 0;
      bool asc = (lane & size) == 0;
      v = key_pick(v, o, lower == asc);
    }
  }
  return v;
}

// Ascending bitonic sort of one 32-bit value per lane.
__device__ __forceinline__ uint32_t warp_sort32_u32(uint32_t v, int lane) {
#pragma unroll
  for (int size = 2; size <= 32; size <<= 1) {
#pragma unroll
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      uint32_t o = __shfl_xor_sync(FULL_MASK, v, stride);
      bool take_min = ((lane & stride) == 0) == ((lane & size) == 0);
      v = ((o < v) == take_min) ? o : v;
    }
  }
  return v;
}

// Ascending merge of a bitonic sequence held one key per lane.
template <typename K>
__device__ __forceinline__ K warp_bitonic_merge32(K v, int lane) {
#pragma unroll
  for (int stride = 16; stride > 0; stride >>= 1) {
    K o = v.shfl_xor(stride);
    v = key_pick(v, o, (lane & stride) == 0);
  }
  return v;
}

// Ascending bitonic sort of `count` (a power of two, >= 64) keys in shared memory by one warp.
template <typename K>
__device__ __forceinline__ void warp_sort_shared(K *keys, int count, int lane) {
  for (int size = 2; size <= count; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      __syncwarp();
      for (int t = lane; t < (count >> 1); t += 32) {
        int i = 2 * t - (t & (stride - 1));
        int j = i + stride;
        bool asc = (i & size) == 0;
        K a = keys[i], b = keys[j];
        if (b.less(a) == asc) {
          keys[i] = b;
          keys[j] = a;
        }
      }
    }
  }
  __syncwarp();
}

// ---- cp.async (LDGSTS) ------------------------------------------------------------------------
__device__ __forceinline__ void cp_async_4(void *smem_dst, const void *gmem_src) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_8(void *smem_dst, const void *gmem_src) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}
template <typename T>
__device__ __forceinline__ void cp_async_elem(T *smem_dst, const T *gmem_src) {
  if constexpr (sizeof(T) == 4)
    cp_async_4(smem_dst, gmem_src);
  else
    cp_async_8(smem_dst, gmem_src);
}

// Arithmetic of 16-bit inputs.  The reference instantiates its kernels for c10::Half (and, for
// radius, c10::BFloat16), whose operators compute in float and round every single result back to
// the 16-bit type (torch/headeronly/util/Half.h: `operator+`, `operator*`, ... return
// static_cast<float>(a) op static_cast<float>(b), narrowed by __float2half / __float2bfloat16,
// round-to-nearest-even).  Here such inputs are widened to float once and every operation result is
// passed through rnd16<RND>: RND 0 = none (float / double data), 1 = fp16, 2 = bf16.
template <int RND, typename T>
__device__ __forceinline__ T rnd16(T v) {
  if constexpr (RND == 1) {
    return __half2float(__float2half_rn(v));
  } else if constexpr (RND == 2) {
    return __bfloat162float(__float2bfloat16_rn(v));
  } else {
    return v;
  }
}

// acc + diff^2 with diff = a - b, as the reference's `acc += (a - b) * (a - b)` evaluates it:
// one fused multiply-add for float / double (nvcc contracts the expression), three separately
// rounded operations for the 16-bit types.
template <int RND, typename T>
__device__ __forceinline__ T sq_accumulate(T a, T b, T acc) {
  if constexpr (RND == 0) {
    const T diff = a - b;
    if constexpr (sizeof(T) == 4)
      return __fmaf_rn(diff, diff, acc);
    else
      return __fma_rn(diff, diff, acc);
  } else {
    const float diff = rnd16<RND>(__fsub_rn(a, b));
    const float prod = rnd16<RND>(__fmul_rn(diff, diff));
    return rnd16<RND>(__fadd_rn(acc, prod));
  }
}

// acc + a * b (`result += a * b`, csrc/cuda/knn_cuda.cu:13-16), same policy.
template <int RND, typename T>
__device__ __forceinline__ T dot_accumulate(T a, T b, T acc) {
  if constexpr (RND == 0) {
    if constexpr (sizeof(T) == 4)
      return __fmaf_rn(a, b, acc);
    else
      return __fma_rn(a, b, acc);
  } else {
    return rnd16<RND>(__fadd_rn(acc, rnd16<RND>(__fmul_rn(a, b))));
  }
}

// 1 - dot / (|x| * |y|) (csrc/cuda/knn_cuda.cu:55-59).  For the 16-bit types the product, the
// quotient and the final difference (formed in double, narrowed through float) are each rounded.
template <int RND, typename T>
__device__ __forceinline__ T cosine_finish(T dot, T nx, T ny) {
  if constexpr (RND == 0) {
    return (T)1 - dot / (nx * ny);
  } else {
    const float den = rnd16<RND>(__fmul_rn(nx, ny));
    const float q = rnd16<RND>(__fdiv_rn(dot, den));
    return rnd16<RND>((float)(1.0 - (double)q));
  }
}

template <typename T>
__device__ __forceinline__ T pos_inf();
template <>
__device__ __forceinline__ float pos_inf<float>() { return __int_as_float(0x7f800000); }
template <>
__device__ __forceinline__ double pos_inf<double>() { return __longlong_as_double(0x7ff0000000000000ll); }

}  // namespace b200c
