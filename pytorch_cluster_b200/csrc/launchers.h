// Internal launch entry points (one per translation unit, so that the template instantiations
// compile in parallel).  Each returns a B200C_* status.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace b200c {

struct KnnArgs {
  const void *x, *y;
  const int64_t *ptr_x, *ptr_y;
  int num_segments;
  int64_t n, m;
  int dim, k;
  int cosine;
  const void *norms_x, *norms_y;  // cosine only: |row| of x and y
  int64_t *out_row, *out_col;
  int32_t *counts;
  unsigned long long *num_valid;
  cudaStream_t stream;
  // graph mode of the low-dimensional kernel (x searched in itself, k = neighbours + 1): final
  // [2, m * (k - 1)] edge rows without the self matches, and a count of queries that do not fit
  // that shape; the padded outputs above are then unused
  int64_t *graph_out = nullptr;     // row 0 of this call's slots
  int64_t graph_row_stride = 0;     // distance from a slot of row 0 to the same slot of row 1
  int64_t graph_index_base = 0;     // added to every index written (rows of a part of a larger x)
  int graph_s2t = 0;
  int *graph_irregular = nullptr;
};

struct RadiusArgs {
  const void *x, *y;
  const int64_t *ptr_x, *ptr_y;
  int num_segments;
  int64_t n, m;
  int dim;
  double r;
  int64_t max_nn;
  int ignore_same;
  int32_t *counts;          // count pass
  const int64_t *offsets;   // fill pass
  int64_t *out_row, *out_col;
  int32_t *direct_rows;     // one-pass mode: [m, max_nn] int32 scratch, else nullptr
  cudaStream_t stream;
  // bit-matrix mode: per-segment first word of the segment's rows, and the words
  const int64_t *mask_base = nullptr;
  uint32_t *mask_words = nullptr;
  // row number of y's first row in the numbering of x: `ignore_same` skips x row q + query_base
  int64_t query_base = 0;
};

int launch_knn_lowd_f32(const KnnArgs &a);
int launch_knn_lowd_f64(const KnnArgs &a);
int launch_radius_lowd_f32(const RadiusArgs &a, bool fill);
int launch_radius_lowd_f64(const RadiusArgs &a, bool fill);
// Screened scan for fp32 points of up to 8 features (radius_screen.cuh): workspace (0: not applicable), both passes.
size_t radius_screen_workspace_bytes(int64_t n, int64_t m, int dim, int64_t max_nn, int64_t num_segments);
int launch_radius_screen_f32(const RadiusArgs &a, bool fill, void *workspace);
int radius_lowd_chunk_points(int dim, int dtype);  // points per chunk of the low-dimensional scan: 32 x (mask words per chunk)
int launch_knn_generic_f32(const KnnArgs &a);
int launch_knn_generic_f64(const KnnArgs &a);
int launch_radius_generic_f32(const RadiusArgs &a, bool fill);
int launch_radius_generic_f64(const RadiusArgs &a, bool fill);
// 16-bit inputs, already widened to float (x, y of the argument structs point to the float copies)
int launch_knn_generic_f16(const KnnArgs &a);
int launch_knn_generic_bf16(const KnnArgs &a);
int launch_radius_generic_f16(const RadiusArgs &a, bool fill);
int launch_radius_generic_bf16(const RadiusArgs &a, bool fill);
int launch_row_norms_f16(const void *a, int64_t rows, int dim, void *out, cudaStream_t s);
int launch_row_norms_bf16(const void *a, int64_t rows, int dim, void *out, cudaStream_t s);
int launch_nearest_lowd_f32(const KnnArgs &a);
int launch_nearest_lowd_f64(const KnnArgs &a);
int launch_nearest_generic_f32(const KnnArgs &a);
int launch_nearest_generic_f64(const KnnArgs &a);
int launch_nearest_generic_f16(const KnnArgs &a);
int launch_nearest_generic_bf16(const KnnArgs &a);
int launch_radius_mask_base(const int64_t *ptr_x, const int64_t *ptr_y, int num_segments, int64_t n, int64_t m,
                            int chunk, int64_t *base, cudaStream_t stream);
int launch_widen16(const void *src, int64_t elems, int dtype, float *dst, cudaStream_t s);
int launch_row_norms_f32(const void *a, int64_t rows, int dim, void *out, cudaStream_t s);
int launch_row_norms_f64(const void *a, int64_t rows, int dim, void *out, cudaStream_t s);

// tensor-core candidate path (fp32, 32 <= dim <= 128, dim % 8 == 0, k <= 32)
bool knn_tensor_applicable(int64_t n, int64_t m, int dim, int k, int64_t num_segments, const void *x, const void *y);
size_t knn_tensor_workspace_bytes(int64_t n, int64_t m, int dim, int cosine);
int launch_knn_tensor_f32(const KnnArgs &a, void *workspace);
int launch_knn_rerank_f32(const KnnArgs &a, const int32_t *cand, const int32_t *cand_count, const int *error_flag,
                          const float *norms_x, const float *norms_y);

// Morton-ordered scan for fp32 points of up to 8 features (knn_spatial.cuh): applicable sizes, the
// workspace it needs (same_set: the queries are the points themselves, one sorted copy serves both),
// and the launch (sorting passes + scan).  max_segment_rows: upper bound of a segment's row count, 0 = unknown.
bool knn_spatial_applicable(int64_t n, int64_t m, int dim, int k, int64_t num_segments);
size_t knn_spatial_workspace_bytes(int64_t n, int64_t m, int dim, int64_t num_segments, bool same_set);
int launch_knn_spatial_f32(const KnnArgs &a, void *workspace, int64_t max_segment_rows);
int knn_spatial_scan_timing(int enable);  // record CUDA events around the scan kernel of later calls
float knn_spatial_last_scan_ms();         // duration of the last timed scan kernel (waits for it), -1 if none

}  // namespace b200c
