// Small HBM-bound passes around the search kernels: segment pointers, the exclusive scan of the
// per-query edge counts, and the compaction of padded kNN output.
#include <type_traits>
#include <mutex>

#include "common.cuh"
#include "launchers.h"

namespace b200c {

// ---- segment pointers ----------------------------------------------------------------------------
// ptr[i] = lower_bound(batch, i): one thread per boundary bisects the sorted batch vector
// (torch.bucketize(arange(B + 1), batch), torch_cluster/knn.py:77-79).
__global__ void segment_ptr_kernel(const int64_t *__restrict__ batch, int64_t n, int64_t num_segments,
                                   int64_t *__restrict__ ptr) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i > num_segments) return;
  int64_t lo = 0, hi = n;
  while (lo < hi) {
    const int64_t mid = (lo + hi) >> 1;
    if (batch[mid] < i)
      lo = mid + 1;
    else
      hi = mid;
  }
  ptr[i] = lo;
}

// info[0] = batch[n - 1] + 1 (the ids are sorted, so the last is the largest), info[1] = rows of the
// longest run of equal ids.  The thread at the last row of a run bisects for the run's first row.
// With `unsorted` != nullptr also *unsorted = 1 if some entry is smaller than the one before it (the other two
// values mean nothing then).
__global__ void batch_info_kernel(const int64_t *__restrict__ batch, int64_t n, unsigned long long *__restrict__ info,
                                  unsigned long long *__restrict__ unsorted) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  unsigned long long best = 0;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const int64_t id = batch[i];
    if (unsorted != nullptr && i + 1 < n && batch[i + 1] < id) *unsorted = 1ull;
    if (i + 1 < n && batch[i + 1] == id) continue;
    int64_t lo = 0, hi = i;
    while (lo < hi) {
      const int64_t mid = (lo + hi) >> 1;
      if (batch[mid] < id)
        lo = mid + 1;
      else
        hi = mid;
    }
    const unsigned long long run = (unsigned long long)(i + 1 - lo);
    best = run > best ? run : best;
    if (i == n - 1) info[0] = (unsigned long long)(id + 1);
  }
  if (best) atomicMax(info + 1, best);
}

// ---- exclusive scan, int32 counts -> int64 offsets --------------------------------------------------
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ITEMS = 8;
constexpr int SCAN_TILE = SCAN_THREADS * SCAN_ITEMS;

__device__ __forceinline__ int64_t block_exclusive_scan(int64_t v, int64_t *total, int64_t *warp_sums) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int64_t inc = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int64_t t = __shfl_up_sync(FULL_MASK, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_sums[warp] = inc;
  __syncthreads();
  if (warp == 0) {
    int64_t w = lane < SCAN_THREADS / 32 ? warp_sums[lane] : 0;
    int64_t winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int64_t t = __shfl_up_sync(FULL_MASK, winc, o);
      if (lane >= o) winc += t;
    }
    if (lane < SCAN_THREADS / 32) warp_sums[lane] = winc - w;
    if (lane == SCAN_THREADS / 32 - 1) *total = winc;
  }
  __syncthreads();
  return inc - v + warp_sums[warp];
}

__global__ void __launch_bounds__(SCAN_THREADS)
scan_tile_sums_kernel(const int32_t *__restrict__ counts, int64_t m, int64_t *__restrict__ tile_sums) {
  __shared__ int64_t warp_sums[SCAN_THREADS / 32];
  const int64_t base = (int64_t)blockIdx.x * SCAN_TILE;
  int64_t s = 0;
#pragma unroll
  for (int i = 0; i < SCAN_ITEMS; ++i) {
    const int64_t j = base + (int64_t)i * SCAN_THREADS + threadIdx.x;
    if (j < m) s += counts[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
  if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    int64_t t = 0;
    for (int w = 0; w < SCAN_THREADS / 32; ++w) t += warp_sums[w];
    tile_sums[blockIdx.x] = t;
  }
}

// One CTA turns the tile sums into exclusive tile offsets (in place) and stores the grand total.
__global__ void __launch_bounds__(SCAN_THREADS)
scan_tile_offsets_kernel(int64_t *__restrict__ tile_sums, int64_t num_tiles, int64_t *__restrict__ total_out) {
  __shared__ int64_t warp_sums[SCAN_THREADS / 32];
  __shared__ int64_t block_total;
  int64_t carry = 0;
  for (int64_t base = 0; base < num_tiles; base += SCAN_THREADS) {
    const int64_t j = base + threadIdx.x;
    const int64_t v = j < num_tiles ? tile_sums[j] : 0;
    const int64_t ex = block_exclusive_scan(v, &block_total, warp_sums);
    if (j < num_tiles) tile_sums[j] = carry + ex;
    carry += block_total;
    __syncthreads();
  }
  if (threadIdx.x == 0) *total_out = carry;
}

__global__ void __launch_bounds__(SCAN_THREADS)
scan_apply_kernel(const int32_t *__restrict__ counts, int64_t m, const int64_t *__restrict__ tile_offsets,
                  int64_t *__restrict__ offsets) {
  __shared__ int64_t warp_sums[SCAN_THREADS / 32];
  __shared__ int64_t block_total;
  // thread t owns SCAN_ITEMS consecutive elements so that one block scan suffices
  const int64_t first = (int64_t)blockIdx.x * SCAN_TILE + (int64_t)threadIdx.x * SCAN_ITEMS;
  int32_t v[SCAN_ITEMS];
  int64_t s = 0;
#pragma unroll
  for (int i = 0; i < SCAN_ITEMS; ++i) {
    v[i] = first + i < m ? counts[first + i] : 0;
    s += v[i];
  }
  int64_t run = tile_offsets[blockIdx.x] + block_exclusive_scan(s, &block_total, warp_sums);
#pragma unroll
  for (int i = 0; i < SCAN_ITEMS; ++i) {
    if (first + i < m) offsets[first + i] = run;
    run += v[i];
  }
}

// ---- scratch of the workspace-free scan ---------------------------------------------------------------
// Partial sums of b200c_exclusive_scan_static: one per tile of 2048 rows, enough for
// B200C_SCAN_STATIC_MAX_ROWS rows.  Device code may name the array; host code may not (there the
// name is only a handle for cudaGetSymbolAddress), so the kernels receive its address as a pointer.
constexpr int64_t SCAN_STATIC_TILES = B200C_SCAN_STATIC_MAX_ROWS / SCAN_TILE;
static __device__ __align__(256) int64_t g_scan_static_tile_sums[SCAN_STATIC_TILES];

constexpr int SCAN_STATIC_MAX_DEVICES = 64;
static std::mutex g_scan_static_mutex;
static int64_t *g_scan_static_addr[SCAN_STATIC_MAX_DEVICES] = {};

// Device address of the array on the current device; looked up once per device.
static int scan_static_scratch(int64_t **out) {
  int dev = -1;
  B200C_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= SCAN_STATIC_MAX_DEVICES) {
    set_error("device ordinal %d is outside the range this entry point tracks (0..%d)", dev,
              SCAN_STATIC_MAX_DEVICES - 1);
    return B200C_ERR_INVALID;
  }
  std::lock_guard<std::mutex> lock(g_scan_static_mutex);
  if (g_scan_static_addr[dev] == nullptr) {
    void *addr = nullptr;
    B200C_CUDA(cudaGetSymbolAddress(&addr, g_scan_static_tile_sums));
    g_scan_static_addr[dev] = static_cast<int64_t *>(addr);
  }
  *out = g_scan_static_addr[dev];
  return B200C_OK;
}

// ---- compaction of padded kNN output ------------------------------------------------------------------
__global__ void knn_compact_kernel(const int64_t *__restrict__ col_padded, const int32_t *__restrict__ counts,
                                   const int64_t *__restrict__ offsets, int64_t m, int k,
                                   int64_t *__restrict__ out_row, int64_t *__restrict__ out_col) {
  const int64_t slot = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (slot >= m * k) return;
  const int64_t q = slot / k;
  const int e = (int)(slot - q * k);
  if (e < counts[q]) {
    const int64_t o = offsets[q] + e;
    out_row[o] = q;
    out_col[o] = col_padded[slot];
  }
}

// ---- knn_graph tail: drop self matches and padding, orient by flow -----------------------------------------
// kept[q] = number of valid slots of query q whose neighbour is not q itself (all valid ones when
// self loops are wanted).  One thread per query.
__global__ void knn_graph_tail_count_kernel(const int64_t *__restrict__ col_padded, const int32_t *__restrict__ counts,
                                            int64_t m, int k1, int drop_self, int32_t *__restrict__ kept) {
  const int64_t q = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (q >= m) return;
  const int c = counts[q];
  int n = c;
  if (drop_self)
    for (int e = 0; e < c; ++e) n -= col_padded[q * k1 + e] == q;
  kept[q] = n;
}

// One warp per query: its kept neighbours, in their stored order, to offsets[q]... of the output;
// row 0 holds the neighbour and row 1 the query for "source_to_target", the other way round otherwise.
__global__ void knn_graph_tail_write_kernel(const int64_t *__restrict__ col_padded, const int32_t *__restrict__ counts,
                                            const int64_t *__restrict__ offsets, int64_t m, int k1, int drop_self,
                                            int source_to_target, int64_t *__restrict__ out0,
                                            int64_t *__restrict__ out1) {
  const int lane = threadIdx.x & 31;
  const int64_t q = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  if (q >= m) return;
  const int c = counts[q];
  int64_t o = offsets[q];
  for (int base = 0; base < c; base += 32) {
    const int e = base + lane;
    const int64_t nb = e < c ? col_padded[q * k1 + e] : -1;
    const bool keep = e < c && !(drop_self && nb == q);
    const unsigned mask = __ballot_sync(FULL_MASK, keep);
    if (keep) {
      const int64_t pos = o + __popc(mask & ((1u << lane) - 1u));
      out0[pos] = source_to_target ? nb : q;
      out1[pos] = source_to_target ? q : nb;
    }
    o += __popc(mask);
  }
}

// fp16 / bf16 -> float, exact (every 16-bit value is a float value).  Grid-stride, 2 elements per
// 32-bit load where the element count allows it.
template <typename H>
__global__ void widen16_kernel(const H *__restrict__ src, int64_t elems, float *__restrict__ dst) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += stride) {
    if constexpr (sizeof(H) == 2 && std::is_same<H, __half>::value)
      dst[i] = __half2float(src[i]);
    else
      dst[i] = __bfloat162float(src[i]);
  }
}

// First bit-matrix word of every segment's rows for the bit-matrix radius search: the exclusive
// sum over segments of m_b * ceil(n_b / chunk) * (chunk / 32), formed from the device copies of the
// segment pointers.  One CTA: thread t sums a contiguous run of segments, the run totals are
// scanned in shared memory, then every thread writes its segments' bases.
constexpr int MASK_BASE_THREADS = 1024;
__global__ void __launch_bounds__(MASK_BASE_THREADS)
radius_mask_base_kernel(const int64_t *__restrict__ ptr_x, const int64_t *__restrict__ ptr_y, int num_segments,
                        int64_t n, int64_t m, int chunk, int64_t *__restrict__ base) {
  __shared__ int64_t run_total[MASK_BASE_THREADS];
  const int t = threadIdx.x;
  const int per = (num_segments + MASK_BASE_THREADS - 1) / MASK_BASE_THREADS;
  const int lo = t * per < num_segments ? t * per : num_segments;
  const int hi = lo + per < num_segments ? lo + per : num_segments;
  auto words_of = [&](int b) -> int64_t {
    const int64_t nb = ptr_x ? ptr_x[b + 1] - ptr_x[b] : n, mb = ptr_y ? ptr_y[b + 1] - ptr_y[b] : m;
    return (nb > 0 && mb > 0) ? mb * ((nb + chunk - 1) / chunk) * (chunk / 32) : 0;
  };
  int64_t sum = 0;
  for (int b = lo; b < hi; ++b) sum += words_of(b);
  run_total[t] = sum;
  __syncthreads();
  for (int o = 1; o < MASK_BASE_THREADS; o <<= 1) {
    const int64_t add = t >= o ? run_total[t - o] : 0;
    __syncthreads();
    run_total[t] += add;
    __syncthreads();
  }
  int64_t run = run_total[t] - sum;  // exclusive
  for (int b = lo; b < hi; ++b) {
    base[b] = run;
    run += words_of(b);
  }
}

// FP32 throughput probe: 16 independent chains of fused multiply-adds per thread, `iters` rounds.
constexpr int PROBE_CHAINS = 16, PROBE_THREADS = 256, PROBE_CTAS_PER_SM = 8;
__global__ void __launch_bounds__(PROBE_THREADS)
probe_fp32_kernel(int64_t iters, float seed, float *__restrict__ out) {
  float v[PROBE_CHAINS];
#pragma unroll
  for (int i = 0; i < PROBE_CHAINS; ++i) v[i] = seed + (float)(threadIdx.x + i);
  const float a = 1.0000001f, b = seed;
  for (int64_t it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < PROBE_CHAINS; ++i) v[i] = __fmaf_rn(v[i], a, b);
  }
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < PROBE_CHAINS; ++i) s += v[i];
  if (s == 12345.678f) out[0] = s;  // keeps the chains alive; practically never true
}

int launch_radius_mask_base(const int64_t *ptr_x, const int64_t *ptr_y, int num_segments, int64_t n, int64_t m,
                            int chunk, int64_t *base, cudaStream_t stream) {
  radius_mask_base_kernel<<<1, MASK_BASE_THREADS, 0, stream>>>(ptr_x, ptr_y, num_segments, n, m, chunk, base);
  B200C_LAUNCH_CHECK("radius_mask_base_kernel");
  return B200C_OK;
}

int launch_widen16(const void *src, int64_t elems, int dtype, float *dst, cudaStream_t stream) {
  if (elems == 0) return B200C_OK;
  const int64_t want = (elems + 255) / 256;
  const unsigned grid = (unsigned)(want < 148 * 16 ? want : 148 * 16);
  if (dtype == B200C_F16)
    widen16_kernel<__half><<<grid, 256, 0, stream>>>((const __half *)src, elems, dst);
  else
    widen16_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>((const __nv_bfloat16 *)src, elems, dst);
  B200C_LAUNCH_CHECK("widen16_kernel");
  return B200C_OK;
}

}  // namespace b200c

using namespace b200c;

extern "C" int b200c_segment_ptr(const int64_t *batch, int64_t n, int64_t num_segments, int64_t *ptr,
                                 b200c_stream_t stream) {
  B200C_CHECK_ARG(n >= 0 && num_segments >= 0, "Input mismatch");
  B200C_CHECK_ARG(ptr != nullptr && (batch != nullptr || n == 0), "null pointer");
  const int64_t total = num_segments + 1;
  const int threads = 128;
  segment_ptr_kernel<<<(unsigned)((total + threads - 1) / threads), threads, 0, (cudaStream_t)stream>>>(
      batch, n, num_segments, ptr);
  B200C_LAUNCH_CHECK("segment_ptr_kernel");
  return B200C_OK;
}

extern "C" int b200c_batch_info(const int64_t *batch, int64_t n, int64_t *info, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  B200C_CHECK_ARG(n >= 0 && info != nullptr && (batch != nullptr || n == 0), "Input mismatch");
  B200C_CUDA(cudaMemsetAsync(info, 0, 2 * sizeof(int64_t), stream));
  if (n == 0) return B200C_OK;
  const int64_t want = (n + 255) / 256;
  batch_info_kernel<<<(unsigned)(want < 148 * 8 ? want : 148 * 8), 256, 0, stream>>>(batch, n,
                                                                                  (unsigned long long *)info, nullptr);
  B200C_LAUNCH_CHECK("batch_info_kernel");
  return B200C_OK;
}

extern "C" int b200c_batch_check(const int64_t *batch, int64_t n, int64_t *info, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  B200C_CHECK_ARG(n >= 0 && info != nullptr && (batch != nullptr || n == 0), "Input mismatch");
  B200C_CUDA(cudaMemsetAsync(info, 0, 3 * sizeof(int64_t), stream));
  if (n == 0) return B200C_OK;
  const int64_t want = (n + 255) / 256;
  batch_info_kernel<<<(unsigned)(want < 148 * 8 ? want : 148 * 8), 256, 0, stream>>>(
      batch, n, (unsigned long long *)info, (unsigned long long *)info + 2);
  B200C_LAUNCH_CHECK("batch_info_kernel");
  return B200C_OK;
}

__global__ void segment_mismatch_kernel(const int64_t *__restrict__ ptr_x, const int64_t *__restrict__ ptr_y,
                                        int64_t num_segments, int32_t *__restrict__ flag) {
  const int64_t b = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= num_segments) return;
  if ((ptr_x[b + 1] > ptr_x[b]) != (ptr_y[b + 1] > ptr_y[b])) *flag = 1;
}

extern "C" int b200c_segment_mismatch(const int64_t *ptr_x, const int64_t *ptr_y, int64_t num_segments,
                                      int32_t *flag, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  B200C_CHECK_ARG(num_segments >= 0 && flag != nullptr && ((ptr_x != nullptr && ptr_y != nullptr) || num_segments == 0),
                  "Input mismatch");
  B200C_CUDA(cudaMemsetAsync(flag, 0, sizeof(int32_t), stream));
  if (num_segments == 0) return B200C_OK;
  segment_mismatch_kernel<<<(unsigned)((num_segments + 255) / 256), 256, 0, stream>>>(ptr_x, ptr_y, num_segments, flag);
  B200C_LAUNCH_CHECK("segment_mismatch_kernel");
  return B200C_OK;
}

extern "C" int b200c_probe_fp32(int64_t iters, float *scratch, double *flops, b200c_stream_t stream) {
  B200C_CHECK_ARG(iters >= 1 && scratch != nullptr && flops != nullptr, "Input mismatch");
  int dev = 0, sms = 0;
  B200C_CUDA(cudaGetDevice(&dev));
  B200C_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int ctas = sms * PROBE_CTAS_PER_SM;
  probe_fp32_kernel<<<ctas, PROBE_THREADS, 0, (cudaStream_t)stream>>>(iters, 0.5f, scratch);
  B200C_LAUNCH_CHECK("probe_fp32_kernel");
  *flops = 2.0 * (double)iters * PROBE_CHAINS * PROBE_THREADS * (double)ctas;
  return B200C_OK;
}

extern "C" size_t b200c_scan_workspace_bytes(int64_t m) {
  const int64_t tiles = m > 0 ? (m + SCAN_TILE - 1) / SCAN_TILE : 1;
  return (size_t)tiles * sizeof(int64_t);
}

extern "C" int b200c_exclusive_scan(const int32_t *counts, int64_t m, int64_t *offsets, void *workspace,
                                    size_t workspace_bytes, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  B200C_CHECK_ARG(m >= 0, "Input mismatch");
  B200C_CHECK_ARG(offsets != nullptr, "null pointer");
  if (m == 0) {
    B200C_CUDA(cudaMemsetAsync(offsets, 0, sizeof(int64_t), stream));
    return B200C_OK;
  }
  B200C_CHECK_ARG(counts != nullptr && workspace != nullptr, "null pointer");
  if (workspace_bytes < b200c_scan_workspace_bytes(m)) {
    set_error("scan workspace too small: %zu < %zu", workspace_bytes, b200c_scan_workspace_bytes(m));
    return B200C_ERR_WORKSPACE;
  }
  const int64_t tiles = (m + SCAN_TILE - 1) / SCAN_TILE;
  int64_t *tile_sums = (int64_t *)workspace;
  scan_tile_sums_kernel<<<(unsigned)tiles, SCAN_THREADS, 0, stream>>>(counts, m, tile_sums);
  B200C_LAUNCH_CHECK("scan_tile_sums_kernel");
  scan_tile_offsets_kernel<<<1, SCAN_THREADS, 0, stream>>>(tile_sums, tiles, offsets + m);
  B200C_LAUNCH_CHECK("scan_tile_offsets_kernel");
  scan_apply_kernel<<<(unsigned)tiles, SCAN_THREADS, 0, stream>>>(counts, m, tile_sums, offsets);
  B200C_LAUNCH_CHECK("scan_apply_kernel");
  return B200C_OK;
}

extern "C" int b200c_knn_graph_tail_count(const int64_t *edge_padded, const int32_t *counts, int64_t m, int64_t k,
                                          int drop_self, int32_t *kept, b200c_stream_t stream) {
  B200C_CHECK_ARG(m >= 0 && k >= 1 && k <= B200C_MAX_K, "Input mismatch");
  if (m == 0) return B200C_OK;
  B200C_CHECK_ARG(edge_padded && counts && kept, "null pointer");
  knn_graph_tail_count_kernel<<<(unsigned)((m + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      edge_padded + m * k, counts, m, (int)k, drop_self, kept);
  B200C_LAUNCH_CHECK("knn_graph_tail_count_kernel");
  return B200C_OK;
}

extern "C" int b200c_knn_graph_tail_write(const int64_t *edge_padded, const int32_t *counts, const int64_t *offsets,
                                          int64_t m, int64_t k, int drop_self, int source_to_target,
                                          int64_t num_edges, int64_t *edge_index, b200c_stream_t stream) {
  B200C_CHECK_ARG(m >= 0 && k >= 1 && k <= B200C_MAX_K && num_edges >= 0, "Input mismatch");
  if (m == 0 || num_edges == 0) return B200C_OK;
  B200C_CHECK_ARG(edge_padded && counts && offsets && edge_index, "null pointer");
  const int64_t threads = m * 32;
  knn_graph_tail_write_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      edge_padded + m * k, counts, offsets, m, (int)k, drop_self, source_to_target, edge_index,
      edge_index + num_edges);
  B200C_LAUNCH_CHECK("knn_graph_tail_write_kernel");
  return B200C_OK;
}

// The scan of b200c_exclusive_scan with its partial sums in the library's own fixed array, for
// callers without an allocator (see include/b200_cluster.h).  Allocates nothing.
extern "C" int b200c_exclusive_scan_static(const int32_t *counts, int64_t m, int64_t *offsets,
                                           b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  B200C_CHECK_ARG(m >= 0, "Input mismatch");
  if (m > (int64_t)B200C_SCAN_STATIC_MAX_ROWS) {
    set_error("b200c_exclusive_scan_static handles at most %lld rows (its scratch is a fixed 64 KiB array); "
              "got %lld - use b200c_exclusive_scan with a caller-provided workspace",
              (long long)B200C_SCAN_STATIC_MAX_ROWS, (long long)m);
    return B200C_ERR_WORKSPACE;
  }
  B200C_CHECK_ARG(offsets != nullptr, "null pointer");
  if (m == 0) {
    B200C_CUDA(cudaMemsetAsync(offsets, 0, sizeof(int64_t), stream));
    return B200C_OK;
  }
  B200C_CHECK_ARG(counts != nullptr, "null pointer");
  int64_t *tile_sums = nullptr;
  const int st = scan_static_scratch(&tile_sums);
  if (st != B200C_OK) return st;
  const int64_t tiles = (m + SCAN_TILE - 1) / SCAN_TILE;
  scan_tile_sums_kernel<<<(unsigned)tiles, SCAN_THREADS, 0, stream>>>(counts, m, tile_sums);
  B200C_LAUNCH_CHECK("scan_tile_sums_kernel");
  scan_tile_offsets_kernel<<<1, SCAN_THREADS, 0, stream>>>(tile_sums, tiles, offsets + m);
  B200C_LAUNCH_CHECK("scan_tile_offsets_kernel");
  scan_apply_kernel<<<(unsigned)tiles, SCAN_THREADS, 0, stream>>>(counts, m, tile_sums, offsets);
  B200C_LAUNCH_CHECK("scan_apply_kernel");
  return B200C_OK;
}

extern "C" int b200c_knn_compact(const int64_t *edge_padded, const int32_t *counts, const int64_t *offsets,
                                 int64_t m, int64_t k, int64_t num_edges, int64_t *edge_index,
                                 b200c_stream_t stream) {
  B200C_CHECK_ARG(m >= 0 && k >= 1 && k <= B200C_MAX_K && num_edges >= 0, "Input mismatch");
  if (m == 0 || num_edges == 0) return B200C_OK;
  B200C_CHECK_ARG(edge_padded && counts && offsets && edge_index, "null pointer");
  const int64_t slots = m * k;
  const int threads = 256;
  knn_compact_kernel<<<(unsigned)((slots + threads - 1) / threads), threads, 0, (cudaStream_t)stream>>>(
      edge_padded + slots, counts, offsets, m, (int)k, edge_index, edge_index + num_edges);
  B200C_LAUNCH_CHECK("knn_compact_kernel");
  return B200C_OK;
}
