// extern "C" entry points: argument checks (the reference's "Input mismatch" rules,
// csrc/cuda/knn_cuda.cu:91-114 and csrc/cuda/radius_cuda.cu:50-73, as far as they can be
// checked on raw pointers) and kernel selection.
#include <cstdarg>
#include <cstdio>

#include "common.cuh"
#include "launchers.h"
#include "spatial.cuh"

namespace b200c {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

// The kernels are built for sm_100a only; refuse other devices with a clear message instead of
// a launch failure.
static int check_device() {
  static thread_local int checked_device = -1;
  int dev = 0;
  B200C_CUDA(cudaGetDevice(&dev));
  if (dev == checked_device) return B200C_OK;
  int major = 0;
  B200C_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
  if (major != 10) {
    set_error("device %d has compute capability %d.x; this library is built for sm_100a only", dev, major);
    return B200C_ERR_DEVICE;
  }
  checked_device = dev;
  return B200C_OK;
}

static int check_common(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                        int64_t num_segments, int64_t n, int64_t m, int64_t dim, int dtype) {
  B200C_CHECK_ARG(x != nullptr && y != nullptr, "x and y must be CUDA tensors");
  B200C_CHECK_ARG(n >= 0 && m >= 0 && dim >= 1, "Input mismatch");
  B200C_CHECK_ARG(n <= 0x7fffffffLL && m <= 0x7fffffffLL, "more than 2^31-1 rows are not supported");
  B200C_CHECK_ARG(dtype == B200C_F32 || dtype == B200C_F64 || dtype == B200C_F16 || dtype == B200C_BF16,
                  "unsupported dtype");
  B200C_CHECK_ARG((ptr_x == nullptr) == (ptr_y == nullptr), "Input mismatch");
  B200C_CHECK_ARG(ptr_x == nullptr ? num_segments == 1 : (num_segments >= 1 && num_segments <= 0x7fffffffLL),
                  "Input mismatch");
  return B200C_OK;
}

}  // namespace b200c

using namespace b200c;

extern "C" int b200c_version(void) { return 100; }

extern "C" const char *b200c_last_error(void) { return g_error; }

static size_t align256(size_t v) { return (v + 255) / 256 * 256; }
static bool is16(int dtype) { return dtype == B200C_F16 || dtype == B200C_BF16; }

// float copies of 16-bit x and y at the front of a workspace
static size_t widen_bytes(int64_t n, int64_t m, int64_t dim, int dtype) {
  return is16(dtype) ? align256((size_t)n * dim * 4) + align256((size_t)m * dim * 4) : 0;
}

static int widen_inputs(const void *&x, const void *&y, int64_t n, int64_t m, int64_t dim, int dtype,
                        void *workspace, bool convert, cudaStream_t stream) {
  float *x32 = (float *)workspace;
  float *y32 = (float *)((char *)workspace + align256((size_t)n * dim * 4));
  if (convert) {
    int st = launch_widen16(x, n * dim, dtype, x32, stream);
    if (st != B200C_OK) return st;
    if ((st = launch_widen16(y, m * dim, dtype, y32, stream)) != B200C_OK) return st;
  }
  x = x32;
  y = y32;
  return B200C_OK;
}

extern "C" size_t b200c_knn_workspace_bytes(int64_t n, int64_t m, int64_t dim, int64_t k, int dtype, int cosine,
                                            int64_t num_segments) {
  const size_t elem = dtype == B200C_F64 ? 8 : 4;
  // 16-bit types: float copies; cosine: |row| of every x and y row
  const size_t exact = widen_bytes(n, m, dim, dtype) +
                       (cosine ? align256((size_t)n * elem) + align256((size_t)m * elem) : 0);
  // Morton-ordered copies for the low-dimensional fp32 scan (x == y cannot be known here: both copies)
  if (dtype == B200C_F32 && !cosine && knn_spatial_applicable(n, m, (int)dim, (int)k, num_segments))
    return knn_spatial_workspace_bytes(n, m, (int)dim, num_segments, false);
  // tensor-core candidate path: norms, candidate lists (and normalised copies for cosine)
  if (dtype == B200C_F32 && num_segments >= 1 &&
      knn_tensor_applicable(n, m, (int)dim, (int)k, num_segments, nullptr, nullptr)) {
    const size_t tensor = knn_tensor_workspace_bytes(n, m, (int)dim, cosine);
    return tensor > exact ? tensor : exact;
  }
  return exact;
}

extern "C" int b200c_knn(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                         int64_t num_segments, int64_t n, int64_t m, int64_t dim, int64_t k, int dtype,
                         int cosine, int64_t *edge_padded, int32_t *counts, int64_t *num_valid,
                         int64_t max_segment_rows, void *workspace, size_t workspace_bytes, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int st = check_common(x, y, ptr_x, ptr_y, num_segments, n, m, dim, dtype);
  if (st != B200C_OK) return st;
  B200C_CHECK_ARG(k >= 1, "`k` needs to be positive");
  B200C_CHECK_ARG(k <= B200C_MAX_K, "`k` needs to smaller than or equal to 100");
  B200C_CHECK_ARG(edge_padded && counts && num_valid, "null output pointer");
  if ((st = check_device()) != B200C_OK) return st;
  B200C_CUDA(cudaMemsetAsync(num_valid, 0, sizeof(int64_t), stream));
  if (m == 0) return B200C_OK;

  B200C_CHECK_ARG(dim <= 0x7fffffffLL / 4, "Input mismatch");
  // required: the norms of the exact cosine kernel; the larger size b200c_knn_workspace_bytes may
  // report also enables the tensor-core candidate path and is optional
  const size_t elem_bytes = dtype == B200C_F64 ? 8 : 4;
  const size_t wide = widen_bytes(n, m, dim, dtype);
  const size_t need = wide + (cosine ? align256((size_t)n * elem_bytes) + align256((size_t)m * elem_bytes) : 0);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need)) {
    set_error("kNN workspace too small: %zu < %zu", workspace_bytes, need);
    return B200C_ERR_WORKSPACE;
  }
  KnnArgs a{x, y, ptr_x, ptr_y, (int)num_segments, n, m, (int)dim, (int)k, cosine, nullptr, nullptr,
            edge_padded, edge_padded + m * k, counts, (unsigned long long *)num_valid, stream};
  if (is16(dtype)) {
    // exact general-dimension kernels on float copies, every operation rounded to the 16-bit type
    if ((st = widen_inputs(a.x, a.y, n, m, dim, dtype, workspace, true, stream)) != B200C_OK) return st;
    const bool h = dtype == B200C_F16;
    if (cosine) {
      char *ws = (char *)workspace + wide;
      a.norms_x = ws;
      a.norms_y = ws + align256((size_t)n * 4);
      st = h ? launch_row_norms_f16(a.x, n, (int)dim, (void *)a.norms_x, stream)
             : launch_row_norms_bf16(a.x, n, (int)dim, (void *)a.norms_x, stream);
      if (st != B200C_OK) return st;
      st = h ? launch_row_norms_f16(a.y, m, (int)dim, (void *)a.norms_y, stream)
             : launch_row_norms_bf16(a.y, m, (int)dim, (void *)a.norms_y, stream);
      if (st != B200C_OK) return st;
    }
    return h ? launch_knn_generic_f16(a) : launch_knn_generic_bf16(a);
  }
  const bool f32 = dtype == B200C_F32;
  if (f32 && knn_tensor_applicable(n, m, (int)dim, (int)k, num_segments, x, y) &&
      workspace_bytes >= knn_tensor_workspace_bytes(n, m, (int)dim, cosine))
    return launch_knn_tensor_f32(a, workspace);
  if (cosine) {
    const size_t elem = f32 ? 4 : 8;
    char *ws = (char *)workspace;
    a.norms_x = ws;
    a.norms_y = ws + align256((size_t)n * elem);
    st = f32 ? launch_row_norms_f32(x, n, (int)dim, (void *)a.norms_x, stream)
             : launch_row_norms_f64(x, n, (int)dim, (void *)a.norms_x, stream);
    if (st != B200C_OK) return st;
    st = f32 ? launch_row_norms_f32(y, m, (int)dim, (void *)a.norms_y, stream)
             : launch_row_norms_f64(y, m, (int)dim, (void *)a.norms_y, stream);
    if (st != B200C_OK) return st;
    return f32 ? launch_knn_generic_f32(a) : launch_knn_generic_f64(a);
  }
  if (dim <= 8) {
    if (f32 && workspace != nullptr && knn_spatial_applicable(n, m, (int)dim, (int)k, num_segments) &&
        workspace_bytes >= knn_spatial_workspace_bytes(n, m, (int)dim, num_segments, x == y && ptr_x == ptr_y && n == m))
      return launch_knn_spatial_f32(a, workspace, max_segment_rows);
    return f32 ? launch_knn_lowd_f32(a) : launch_knn_lowd_f64(a);
  }
  return f32 ? launch_knn_generic_f32(a) : launch_knn_generic_f64(a);
}

// knn_graph of low-dimensional points in one kernel: see b200_cluster.h
static int knn_graph_common(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n, int64_t dim,
                            int64_t k, int dtype, int cosine, int source_to_target, int64_t index_base,
                            int64_t *edge_row0, int64_t row_stride, int32_t *irregular, int64_t max_segment_rows,
                            void *workspace, size_t workspace_bytes, cudaStream_t stream) {
  int st = check_common(x, x, ptr, ptr, num_segments, n, n, dim, dtype);
  if (st != B200C_OK) return st;
  B200C_CHECK_ARG(k >= 1, "`k` needs to be positive");
  B200C_CHECK_ARG(k + 1 <= B200C_MAX_K, "`k` needs to smaller than or equal to 100");
  B200C_CHECK_ARG(irregular != nullptr && (edge_row0 != nullptr || n == 0), "null output pointer");
  B200C_CHECK_ARG(index_base >= 0 && row_stride >= n * k, "Input mismatch");
  // feature vectors: the tensor-core candidate path with the re-rank writing the edge rows (fp32, workspace given)
  const bool features = dtype == B200C_F32 && dim > 8 && workspace != nullptr &&
                        knn_tensor_applicable(n, n, (int)dim, (int)(k + 1), num_segments, x, x) &&
                        workspace_bytes >= knn_tensor_workspace_bytes(n, n, (int)dim, cosine);
  if ((dim > 8 && !features) || (cosine && !features) || is16(dtype)) {
    set_error("b200c_knn_graph covers fp32 / fp64 points of up to 8 features, and fp32 feature vectors where the "
              "tensor-core path applies and its workspace is given; use b200c_knn and the tail entry points");
    return B200C_ERR_UNSUPPORTED;
  }
  if ((st = check_device()) != B200C_OK) return st;
  B200C_CUDA(cudaMemsetAsync(irregular, 0, sizeof(int32_t), stream));
  if (n == 0) return B200C_OK;
  KnnArgs a{x, x, ptr, ptr, (int)num_segments, n, n, (int)dim, (int)(k + 1), cosine, nullptr, nullptr,
            nullptr, nullptr, nullptr, nullptr, stream};
  a.graph_out = edge_row0;
  a.graph_row_stride = row_stride;
  a.graph_index_base = index_base;
  a.graph_s2t = source_to_target;
  a.graph_irregular = (int *)irregular;
  if (features) return launch_knn_tensor_f32(a, workspace);
  if (dtype == B200C_F32 && workspace != nullptr && knn_spatial_applicable(n, n, (int)dim, (int)(k + 1), num_segments) &&
      workspace_bytes >= knn_spatial_workspace_bytes(n, n, (int)dim, num_segments, true))
    return launch_knn_spatial_f32(a, workspace, max_segment_rows);
  return dtype == B200C_F32 ? launch_knn_lowd_f32(a) : launch_knn_lowd_f64(a);
}

extern "C" int b200c_knn_graph_part(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n, int64_t dim,
                                    int64_t k, int dtype, int source_to_target, int64_t index_base,
                                    int64_t *edge_row0, int64_t row_stride, int32_t *irregular,
                                    int64_t max_segment_rows, void *workspace, size_t workspace_bytes,
                                    b200c_stream_t stream) {
  return knn_graph_common(x, ptr, num_segments, n, dim, k, dtype, 0, source_to_target, index_base, edge_row0, row_stride,
                          irregular, max_segment_rows, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" size_t b200c_knn_graph_cosine_workspace_bytes(int64_t n, int64_t dim, int64_t k, int64_t num_segments) {
  if (n >= 1 && dim > 8 && num_segments >= 1 &&
      knn_tensor_applicable(n, n, (int)dim, (int)(k + 1), num_segments, nullptr, nullptr))
    return knn_tensor_workspace_bytes(n, n, (int)dim, 1);
  return 0;
}

extern "C" int b200c_knn_graph_cosine(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n, int64_t dim,
                                      int64_t k, int source_to_target, int64_t *edge_index, int32_t *irregular,
                                      void *workspace, size_t workspace_bytes, b200c_stream_t stream) {
  return knn_graph_common(x, ptr, num_segments, n, dim, k, B200C_F32, 1, source_to_target, 0, edge_index, n * k,
                          irregular, 0, workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" size_t b200c_knn_graph_workspace_bytes(int64_t n, int64_t dim, int64_t k, int dtype, int64_t num_segments) {
  if (dtype == B200C_F32 && knn_spatial_applicable(n, n, (int)dim, (int)(k + 1), num_segments))
    return knn_spatial_workspace_bytes(n, n, (int)dim, num_segments, true);
  if (dtype == B200C_F32 && dim > 8 && num_segments >= 1 &&
      knn_tensor_applicable(n, n, (int)dim, (int)(k + 1), num_segments, nullptr, nullptr))
    return knn_tensor_workspace_bytes(n, n, (int)dim, 0);
  return 0;
}

extern "C" int b200c_knn_graph(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n, int64_t dim,
                               int64_t k, int dtype, int source_to_target, int64_t *edge_index, int32_t *irregular,
                               int64_t max_segment_rows, void *workspace, size_t workspace_bytes,
                               b200c_stream_t stream) {
  return b200c_knn_graph_part(x, ptr, num_segments, n, dim, k, dtype, source_to_target, 0, edge_index, n * k,
                              irregular, max_segment_rows, workspace, workspace_bytes, stream);
}

extern "C" int b200c_profile_knn_scan(int enable) { return knn_spatial_scan_timing(enable); }
extern "C" float b200c_profile_knn_scan_ms(void) { return knn_spatial_last_scan_ms(); }

// The ordering pass of the Morton-ordered scan on its own: see b200_cluster.h
extern "C" size_t b200c_morton_order_workspace_bytes(int64_t n, int64_t dim, int64_t num_segments) {
  if (n < 0 || dim < 1 || dim > SP_MAX_DIM || num_segments < 1) return 0;
  return spatial_view_bytes(n, (int)dim, num_segments, false);
}

extern "C" int64_t b200c_morton_order_rows(int64_t n, int64_t num_segments) {
  if (n < 0 || num_segments < 1) return 0;
  const int64_t raw = n + num_segments * (SP_CHUNK - 1);
  return (raw + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
}

extern "C" int b200c_morton_order(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n, int64_t dim,
                                  int64_t max_segment_rows, int32_t *order, uint32_t *keys, int64_t *first,
                                  void *workspace, size_t workspace_bytes, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int st = check_common(x, x, ptr, ptr, num_segments, n, n, dim, B200C_F32);
  if (st != B200C_OK) return st;
  B200C_CHECK_ARG(dim <= SP_MAX_DIM, "the Morton order covers up to 8 features");
  B200C_CHECK_ARG(order != nullptr && keys != nullptr && first != nullptr, "null output pointer");
  const size_t need = b200c_morton_order_workspace_bytes(n, dim, num_segments);
  if (workspace == nullptr || workspace_bytes < need) {
    set_error("Morton order workspace too small: %zu < %zu", workspace_bytes, need);
    return B200C_ERR_WORKSPACE;
  }
  if ((st = check_device()) != B200C_OK) return st;
  SpatialView v;
  spatial_view_carve(&v, workspace, n, (int)dim, num_segments, false);
  if ((st = launch_spatial_sort((const float *)x, ptr, num_segments, n, (int)dim, nullptr, false, max_segment_rows, &v,
                                stream)) != B200C_OK)
    return st;
  const int64_t rows = b200c_morton_order_rows(n, num_segments);
  B200C_CUDA(cudaMemcpyAsync(order, v.idx, (size_t)rows * 4, cudaMemcpyDeviceToDevice, stream));
  B200C_CUDA(cudaMemcpyAsync(keys, v.key, (size_t)rows * 4, cudaMemcpyDeviceToDevice, stream));
  B200C_CUDA(cudaMemcpyAsync(first, v.sptr, (size_t)(num_segments + 1) * 8, cudaMemcpyDeviceToDevice, stream));
  return B200C_OK;
}

// One-pass mode keeps a row of max_num_neighbors int32 slots per query; it is used when that
// scratch is modest, i.e. for the small neighbour caps that are typical in practice.
static constexpr int64_t RADIUS_DIRECT_MAX_NN = 256;
static constexpr int64_t RADIUS_DIRECT_MAX_BYTES = 2ll << 30;

static size_t radius_direct_bytes(int64_t m, int64_t dim, int64_t max_num_neighbors) {
  if (m <= 0 || dim < 1 || dim > 8 || max_num_neighbors < 1 || max_num_neighbors > RADIUS_DIRECT_MAX_NN) return 0;
  const int64_t bytes = m * max_num_neighbors * 4;
  return bytes <= RADIUS_DIRECT_MAX_BYTES ? (size_t)bytes : 0;
}

extern "C" size_t b200c_radius_workspace_bytes(int64_t n, int64_t m, int64_t dim, int64_t max_num_neighbors,
                                               int dtype) {
  if (is16(dtype)) return n >= 0 && m >= 0 && dim >= 1 ? widen_bytes(n, m, dim, dtype) : 0;
  return radius_direct_bytes(m, dim, max_num_neighbors);
}

extern "C" size_t b200c_radius_screen_workspace_bytes(int64_t n, int64_t m, int64_t dim, int64_t max_num_neighbors,
                                                      int dtype, int64_t num_segments) {
  if (dtype != B200C_F32 || dim < 1 || dim > 8 || n < 0 || m < 0) return 0;
  return radius_screen_workspace_bytes(n, m, (int)dim, max_num_neighbors, num_segments);
}

static int radius_common(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                         int64_t num_segments, int64_t n, int64_t m, int64_t dim, double r,
                         int64_t max_num_neighbors, int ignore_same_index, int dtype, int32_t *counts,
                         const int64_t *offsets, int64_t *out_row, int64_t *out_col, bool fill,
                         void *workspace, size_t workspace_bytes, int64_t query_base, cudaStream_t stream) {
  int st = check_common(x, y, ptr_x, ptr_y, num_segments, n, m, dim, dtype);
  if (st != B200C_OK) return st;
  B200C_CHECK_ARG(max_num_neighbors >= 1, "max_num_neighbors must be positive");
  B200C_CHECK_ARG(query_base >= 0, "Input mismatch");
  if ((st = check_device()) != B200C_OK) return st;
  if (m == 0) return B200C_OK;
  if (is16(dtype)) {
    const size_t need = widen_bytes(n, m, dim, dtype);
    if (workspace == nullptr || workspace_bytes < need) {
      set_error("radius workspace too small for 16-bit inputs: %zu < %zu", workspace_bytes, need);
      return B200C_ERR_WORKSPACE;
    }
    // the count pass converts; the fill pass finds the copies where the count pass left them
    if ((st = widen_inputs(x, y, n, m, dim, dtype, workspace, !fill, stream)) != B200C_OK) return st;
    RadiusArgs a{x, y, ptr_x, ptr_y, (int)num_segments, n, m, (int)dim, r, max_num_neighbors,
                 ignore_same_index, counts, offsets, out_row, out_col, nullptr, stream};
    a.query_base = query_base;
    return dtype == B200C_F16 ? launch_radius_generic_f16(a, fill) : launch_radius_generic_bf16(a, fill);
  }
  if (dtype == B200C_F32 && dim <= 8 && workspace != nullptr) {
    // the screened scan, when the workspace has room for its chunk arrays (the same decision in both passes)
    const size_t need = radius_screen_workspace_bytes(n, m, (int)dim, max_num_neighbors, num_segments);
    if (need > 0 && workspace_bytes >= need) {
      RadiusArgs a{x, y, ptr_x, ptr_y, (int)num_segments, n, m, (int)dim, r, max_num_neighbors,
                   ignore_same_index, counts, offsets, out_row, out_col, nullptr, stream};
      a.query_base = query_base;
      return launch_radius_screen_f32(a, fill, workspace);
    }
  }
  const size_t direct_bytes = radius_direct_bytes(m, dim, max_num_neighbors);
  int32_t *direct = (direct_bytes > 0 && workspace != nullptr && workspace_bytes >= direct_bytes)
                        ? (int32_t *)workspace
                        : nullptr;
  RadiusArgs a{x, y, ptr_x, ptr_y, (int)num_segments, n, m, (int)dim, r, max_num_neighbors,
               ignore_same_index, counts, offsets, out_row, out_col, direct, stream};
  a.query_base = query_base;
  B200C_CHECK_ARG(dim <= 0x7fffffffLL / 4, "Input mismatch");
  if (dim <= 8) return dtype == B200C_F32 ? launch_radius_lowd_f32(a, fill) : launch_radius_lowd_f64(a, fill);
  return dtype == B200C_F32 ? launch_radius_generic_f32(a, fill) : launch_radius_generic_f64(a, fill);
}

extern "C" int b200c_radius_count_part(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                                       int64_t num_segments, int64_t n, int64_t m, int64_t dim, double r,
                                       int64_t max_num_neighbors, int ignore_same_index, int64_t query_index_base,
                                       int dtype, int32_t *counts, void *workspace, size_t workspace_bytes,
                                       b200c_stream_t stream) {
  B200C_CHECK_ARG(counts != nullptr || m == 0, "null output pointer");
  return radius_common(x, y, ptr_x, ptr_y, num_segments, n, m, dim, r, max_num_neighbors,
                       ignore_same_index, dtype, counts, nullptr, nullptr, nullptr, false, workspace,
                       workspace_bytes, query_index_base, (cudaStream_t)stream);
}

extern "C" int b200c_radius_count(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                                  int64_t num_segments, int64_t n, int64_t m, int64_t dim, double r,
                                  int64_t max_num_neighbors, int ignore_same_index, int dtype,
                                  int32_t *counts, void *workspace, size_t workspace_bytes,
                                  b200c_stream_t stream) {
  return b200c_radius_count_part(x, y, ptr_x, ptr_y, num_segments, n, m, dim, r, max_num_neighbors,
                                 ignore_same_index, 0, dtype, counts, workspace, workspace_bytes, stream);
}

extern "C" int b200c_radius_fill_part(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                                      int64_t num_segments, int64_t n, int64_t m, int64_t dim, double r,
                                      int64_t max_num_neighbors, int ignore_same_index, int64_t query_index_base,
                                      int swap_rows, int dtype, const int32_t *counts, const int64_t *offsets,
                                      int64_t num_edges, int64_t *edge_index, void *workspace,
                                      size_t workspace_bytes, b200c_stream_t stream) {
  B200C_CHECK_ARG(num_edges >= 0, "Input mismatch");
  if (num_edges == 0) return B200C_OK;
  B200C_CHECK_ARG(counts != nullptr && offsets != nullptr && edge_index != nullptr, "null pointer");
  int64_t *row_q = swap_rows ? edge_index + num_edges : edge_index;
  int64_t *row_x = swap_rows ? edge_index : edge_index + num_edges;
  return radius_common(x, y, ptr_x, ptr_y, num_segments, n, m, dim, r, max_num_neighbors,
                       ignore_same_index, dtype, (int32_t *)counts, offsets, row_q, row_x, true, workspace,
                       workspace_bytes, query_index_base, (cudaStream_t)stream);
}

extern "C" int b200c_radius_fill(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                                 int64_t num_segments, int64_t n, int64_t m, int64_t dim, double r,
                                 int64_t max_num_neighbors, int ignore_same_index, int dtype,
                                 const int32_t *counts, const int64_t *offsets, int64_t num_edges,
                                 int64_t *edge_index, void *workspace, size_t workspace_bytes,
                                 b200c_stream_t stream) {
  return b200c_radius_fill_part(x, y, ptr_x, ptr_y, num_segments, n, m, dim, r, max_num_neighbors,
                                ignore_same_index, 0, 0, dtype, counts, offsets, num_edges, edge_index, workspace,
                                workspace_bytes, stream);
}

// ---- radius with a bit matrix of hits (every pair evaluated once, for large neighbour caps) ----------

// First word of every segment's rows, from host copies of the segment pointers; returns the total number
// of words.  A query of segment b owns ceil(n_b / chunk) * (chunk / 32) words.
// The host copies must describe x and y exactly (start at 0, never decrease, end at n / m): the
// kernels derive the rows of a segment from the device copies with the reference's tolerant rule,
// and a layout sized from anything else would be overrun.  Returns -1 for pointers that do not.
static int64_t radius_mask_layout(const int64_t *px, const int64_t *py, int64_t segs, int64_t n, int64_t m, int chunk) {
  if (px != nullptr && (px[0] != 0 || py[0] != 0 || px[segs] != n || py[segs] != m)) return -1;
  int64_t total = 0;
  for (int64_t b = 0; b < segs; ++b) {
    const int64_t nb = px ? px[b + 1] - px[b] : n, mb = py ? py[b + 1] - py[b] : m;
    if (nb < 0 || mb < 0) return -1;
    if (nb > 0 && mb > 0) total += mb * ((nb + chunk - 1) / chunk) * (chunk / 32);
  }
  return total;
}

extern "C" size_t b200c_radius_mask_workspace_bytes(const int64_t *ptr_x_host, const int64_t *ptr_y_host,
                                                    int64_t num_segments, int64_t n, int64_t m, int64_t dim,
                                                    int dtype) {
  if (dim < 1 || dim > 8 || (dtype != B200C_F32 && dtype != B200C_F64) || num_segments < 1 || n <= 0 || m <= 0) return 0;
  if ((ptr_x_host == nullptr) != (ptr_y_host == nullptr) || (ptr_x_host == nullptr && num_segments != 1)) return 0;
  const int chunk = radius_lowd_chunk_points((int)dim, dtype);
  const int64_t words = radius_mask_layout(ptr_x_host, ptr_y_host, num_segments, n, m, chunk);
  return words > 0 ? align256((size_t)num_segments * 8) + (size_t)words * 4 : 0;
}

extern "C" int b200c_radius_count_masks_part(const void *x, const void *y, const int64_t *ptr_x,
                                             const int64_t *ptr_y, const int64_t *ptr_x_host,
                                             const int64_t *ptr_y_host, int64_t num_segments, int64_t n, int64_t m,
                                             int64_t dim, double r, int64_t max_num_neighbors, int ignore_same_index,
                                             int64_t query_index_base, int dtype, int32_t *counts, void *workspace,
                                             size_t workspace_bytes, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int st = check_common(x, y, ptr_x, ptr_y, num_segments, n, m, dim, dtype);
  if (st != B200C_OK) return st;
  B200C_CHECK_ARG(max_num_neighbors >= 1, "max_num_neighbors must be positive");
  B200C_CHECK_ARG(counts != nullptr || m == 0, "null output pointer");
  B200C_CHECK_ARG((ptr_x == nullptr) == (ptr_x_host == nullptr), "device and host segment pointers must come together");
  B200C_CHECK_ARG(query_index_base >= 0, "Input mismatch");
  const size_t need = b200c_radius_mask_workspace_bytes(ptr_x_host, ptr_y_host, num_segments, n, m, dim, dtype);
  if (need == 0) {
    set_error("the bit-matrix radius search covers fp32 / fp64 points of up to 8 features and needs host segment "
              "pointers that start at 0, never decrease and end at the row counts");
    return B200C_ERR_UNSUPPORTED;
  }
  if (workspace == nullptr || workspace_bytes < need) {
    set_error("radius mask workspace too small: %zu < %zu", workspace_bytes, need);
    return B200C_ERR_WORKSPACE;
  }
  if ((st = check_device()) != B200C_OK) return st;
  // the per-segment bases are formed on the device (no copy from pageable host memory, hence no
  // hidden synchronisation of the stream); the host copies above only sized the workspace
  if ((st = launch_radius_mask_base(ptr_x, ptr_y, (int)num_segments, n, m, radius_lowd_chunk_points((int)dim, dtype),
                                    (int64_t *)workspace, stream)) != B200C_OK)
    return st;
  RadiusArgs a{x, y, ptr_x, ptr_y, (int)num_segments, n, m, (int)dim, r, max_num_neighbors,
               ignore_same_index, counts, nullptr, nullptr, nullptr, nullptr, stream};
  a.mask_base = (const int64_t *)workspace;
  a.mask_words = (uint32_t *)((char *)workspace + align256((size_t)num_segments * 8));
  a.query_base = query_index_base;
  return dtype == B200C_F32 ? launch_radius_lowd_f32(a, false) : launch_radius_lowd_f64(a, false);
}

extern "C" int b200c_radius_count_masks(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                                        const int64_t *ptr_x_host, const int64_t *ptr_y_host, int64_t num_segments,
                                        int64_t n, int64_t m, int64_t dim, double r, int64_t max_num_neighbors,
                                        int ignore_same_index, int dtype, int32_t *counts, void *workspace,
                                        size_t workspace_bytes, b200c_stream_t stream) {
  return b200c_radius_count_masks_part(x, y, ptr_x, ptr_y, ptr_x_host, ptr_y_host, num_segments, n, m, dim, r,
                                       max_num_neighbors, ignore_same_index, 0, dtype, counts, workspace,
                                       workspace_bytes, stream);
}

extern "C" int b200c_radius_fill_masks_part(const int64_t *ptr_x, const int64_t *ptr_y, int64_t num_segments,
                                            int64_t n, int64_t m, int64_t dim, int swap_rows, int dtype,
                                            const int32_t *counts, const int64_t *offsets, int64_t num_edges,
                                            int64_t *edge_index, const void *workspace, b200c_stream_t stream_) {
  B200C_CHECK_ARG(num_edges >= 0 && n >= 0 && m >= 0 && dim >= 1 && dim <= 8, "Input mismatch");
  B200C_CHECK_ARG(dtype == B200C_F32 || dtype == B200C_F64, "unsupported dtype");
  B200C_CHECK_ARG((ptr_x == nullptr) == (ptr_y == nullptr), "Input mismatch");
  if (num_edges == 0 || m == 0) return B200C_OK;
  B200C_CHECK_ARG(counts != nullptr && offsets != nullptr && edge_index != nullptr && workspace != nullptr, "null pointer");
  int st = check_device();
  if (st != B200C_OK) return st;
  RadiusArgs a{nullptr, nullptr, ptr_x, ptr_y, (int)num_segments, n, m, (int)dim, 0.0, 0, 0, (int32_t *)counts, offsets,
               swap_rows ? edge_index + num_edges : edge_index, swap_rows ? edge_index : edge_index + num_edges,
               nullptr, (cudaStream_t)stream_};
  a.mask_base = (const int64_t *)workspace;
  a.mask_words = (uint32_t *)((char *)workspace + align256((size_t)num_segments * 8));
  return dtype == B200C_F32 ? launch_radius_lowd_f32(a, true) : launch_radius_lowd_f64(a, true);
}

extern "C" int b200c_radius_fill_masks(const int64_t *ptr_x, const int64_t *ptr_y, int64_t num_segments, int64_t n,
                                       int64_t m, int64_t dim, int dtype, const int32_t *counts,
                                       const int64_t *offsets, int64_t num_edges, int64_t *edge_index,
                                       const void *workspace, b200c_stream_t stream) {
  return b200c_radius_fill_masks_part(ptr_x, ptr_y, num_segments, n, m, dim, 0, dtype, counts, offsets, num_edges,
                                      edge_index, workspace, stream);
}

// ---- nearest ------------------------------------------------------------------------------------------

extern "C" size_t b200c_nearest_workspace_bytes(int64_t n, int64_t m, int64_t dim, int dtype) {
  return n >= 0 && m >= 0 && dim >= 1 ? widen_bytes(n, m, dim, dtype) : 0;
}

extern "C" int b200c_nearest(const void *x, const void *y, const int64_t *ptr_x, const int64_t *ptr_y,
                             int64_t num_segments, int64_t n, int64_t m, int64_t dim, int dtype, int64_t *out,
                             void *workspace, size_t workspace_bytes, b200c_stream_t stream_) {
  cudaStream_t stream = (cudaStream_t)stream_;
  int st = check_common(x, y, ptr_x, ptr_y, num_segments, n, m, dim, dtype);
  if (st != B200C_OK) return st;
  B200C_CHECK_ARG(out != nullptr || n == 0, "null output pointer");
  B200C_CHECK_ARG(dim <= 0x7fffffffLL / 4, "Input mismatch");
  if ((st = check_device()) != B200C_OK) return st;
  if (n == 0) return B200C_OK;
  if (is16(dtype)) {
    const size_t need = widen_bytes(n, m, dim, dtype);
    if (workspace == nullptr || workspace_bytes < need) {
      set_error("nearest workspace too small for 16-bit inputs: %zu < %zu", workspace_bytes, need);
      return B200C_ERR_WORKSPACE;
    }
    if ((st = widen_inputs(x, y, n, m, dim, dtype, workspace, true, stream)) != B200C_OK) return st;
  }
  // the kernel's "points" are y, its "queries" the rows of x
  KnnArgs a{y, x, ptr_y, ptr_x, (int)num_segments, m, n, (int)dim, 1, 0, nullptr, nullptr,
            nullptr, out, nullptr, nullptr, stream};
  switch (dtype) {
    case B200C_F32: return dim <= 8 ? launch_nearest_lowd_f32(a) : launch_nearest_generic_f32(a);
    case B200C_F64: return dim <= 8 ? launch_nearest_lowd_f64(a) : launch_nearest_generic_f64(a);
    case B200C_F16: return launch_nearest_generic_f16(a);
    default: return launch_nearest_generic_bf16(a);
  }
}
