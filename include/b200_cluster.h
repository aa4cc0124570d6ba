/*
 * b200_cluster.h — C ABI of the sm_100a neighbour-graph kernels.
 *
 * This is the boundary a maintainer of torch_cluster would bind instead of the
 * reference's CUDA backend functions `knn_cuda` (csrc/cuda/knn_cuda.h:5-8) and
 * `radius_cuda` (csrc/cuda/radius_cuda.h:5-9).  Everything is plain pointers
 * and sizes: no torch types, no allocation inside (except where stated), all
 * work is enqueued on the caller's stream.  All pointers are DEVICE pointers
 * unless a parameter says otherwise.  Every function returns a B200C_* status;
 * b200c_last_error() gives the message of the calling thread's last failure.
 *
 * Conventions shared with the reference operators:
 *   x [n, dim], y [m, dim]   row-major, contiguous, dtype f32 or f64
 *   ptr_x, ptr_y [num_segments + 1]   int64 segment boundaries (CSR style);
 *                            NULL means one segment covering all rows
 *   edge rows                row 0 = query (y) index, row 1 = point (x) index,
 *                            global row numbers, ordered by query
 */
#ifndef B200_CLUSTER_H_
#define B200_CLUSTER_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *b200c_stream_t; /* a cudaStream_t */

enum {
  B200C_OK = 0,
  B200C_ERR_INVALID = 1,     /* bad argument ("Input mismatch" family)            */
  B200C_ERR_UNSUPPORTED = 2, /* valid in the reference, not built here             */
  B200C_ERR_CUDA = 3,        /* a CUDA runtime call or launch failed               */
  B200C_ERR_WORKSPACE = 4,   /* workspace too small / scratch limit exceeded       */
  B200C_ERR_DEVICE = 5       /* the GPU is not an sm_100 device                    */
};

/* Data types of x and y.  The 16-bit types follow the reference's instantiations for c10::Half
 * (knn, radius) and c10::BFloat16 (radius; csrc/cuda/knn_cuda.cu:125, csrc/cuda/radius_cuda.cu:84-85):
 * every operation result is rounded to the 16-bit type, so results equal the reference's for
 * such inputs and differ from a search on the widened values.  They need a workspace (below). */
enum { B200C_F32 = 0, B200C_F64 = 1, B200C_F16 = 2, B200C_BF16 = 3 };

/* Largest k accepted, as in the reference (csrc/cuda/knn_cuda.cu:98). */
#define B200C_MAX_K 100

int b200c_version(void);
const char *b200c_last_error(void);

/* Segment pointers from a sorted batch vector:
 *   ptr[i] = number of entries of batch[0..n) that are < i,  i = 0..num_segments.
 * Replaces `torch.bucketize(arange(B + 1), batch)` of torch_cluster/knn.py:77-79
 * and torch_cluster/radius.py:82-84. */
int b200c_segment_ptr(const int64_t *batch, int64_t n, int64_t num_segments,
                      int64_t *ptr, b200c_stream_t stream);

/* info[0] = number of segments (last id + 1), info[1] = rows of the largest segment of a sorted batch
 * vector (int64 [2], device).  The first replaces the `batch.max()` reduction of
 * torch_cluster/knn.py:62-69; the second is the max_segment_rows hint of b200c_knn. */
int b200c_batch_info(const int64_t *batch, int64_t n, int64_t *info, b200c_stream_t stream);

/* The two device-side checks of torch_cluster/nearest.py:60-87, one kernel each instead of a dozen tensor
 * operations.  b200c_batch_check: info (int64 [3], device) = b200c_batch_info's two values and info[2] = 1
 * if the batch vector is not sorted ("'batch_x' is not sorted", nearest.py:60-66).  b200c_segment_mismatch:
 * *flag (int32, device) = 1 if some segment is empty on one side and not on the other ("Some batch indices
 * occur in 'batch_x' that do not occur in 'batch_y'", nearest.py:81-87), else 0. */
int b200c_batch_check(const int64_t *batch, int64_t n, int64_t *info, b200c_stream_t stream);
int b200c_segment_mismatch(const int64_t *ptr_x, const int64_t *ptr_y, int64_t num_segments,
                           int32_t *flag, b200c_stream_t stream);

/* Exclusive prefix sum of per-query edge counts:
 *   offsets[0] = 0, offsets[i + 1] = offsets[i] + counts[i];  offsets[m] = E.
 * Replaces the mask + masked_select compaction of csrc/cuda/radius_cuda.cu:94-95
 * and csrc/cuda/knn_cuda.cu:133-134.  `workspace` needs
 * b200c_scan_workspace_bytes(m) bytes. */
size_t b200c_scan_workspace_bytes(int64_t m);
int b200c_exclusive_scan(const int32_t *counts, int64_t m, int64_t *offsets,
                         void *workspace, size_t workspace_bytes,
                         b200c_stream_t stream);

/* The same exclusive prefix sum for callers that cannot hand over a workspace.
 *
 * This entry point has no counterpart in the reference.  It exists for hosts that must not, or
 * cannot, allocate device memory around the call: a plugin living inside an application whose
 * GPU memory was planned and handed out up front, an inference loop with a "no allocation after
 * warm-up" rule (cudaMalloc and cudaFree synchronise the whole device), or a caller that simply
 * has no allocator of its own to carve the scratch from.  They still pass `counts` and `offsets`;
 * the per-tile partial sums that b200c_exclusive_scan keeps in its workspace live instead in a
 * fixed array inside the library: 8 bytes per 2048 rows, 64 KiB in total, resident on every GPU
 * that loads the library until the process exits.
 *
 *   - m may not exceed B200C_SCAN_STATIC_MAX_ROWS; larger inputs are refused with
 *     B200C_ERR_WORKSPACE and an explanatory message, nothing is launched.
 *   - No cudaMalloc, cudaFree or other allocating routine is called, ever.
 *   - The first call on each device looks up the device address of the array (one
 *     cudaGetSymbolAddress with that device current) and remembers it; make that first call
 *     outside of any stream capture.  Later calls only launch kernels.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left
 *     there.  Nothing in it has to start at zero: every partial sum a call reads was written by
 *     that same call first.  Two calls that overlap on the GPU (different streams, or different
 *     host threads) race on the array; run them one after the other. */
#define B200C_SCAN_STATIC_MAX_ROWS (1 << 24)
int b200c_exclusive_scan_static(const int32_t *counts, int64_t m, int64_t *offsets,
                                b200c_stream_t stream);

/* k nearest neighbours — replaces knn_kernel + knn_cuda
 * (csrc/cuda/knn_cuda.cu:30-84, 86-135).
 *
 * For every query row of y, the k points of x of the same segment with the
 * smallest distance, ascending by (distance, x index); distance is the squared
 * L2 norm accumulated as fma(d, d, acc) over ascending features, or, with
 * `cosine`, 1 - dot / (|x| * |y|) as the reference evaluates it.  Candidates
 * with distance >= 1e10 or NaN are never selected.
 *
 * Output (padded form): edge_padded is int64 [2, m * k]; slot q * k + e of row 0
 * holds q, of row 1 the e-th neighbour or -1 when the segment had fewer than k
 * admissible points.  counts[q] (int32 [m]) is the number of valid slots of q
 * and *num_valid (one int64) their total.  When *num_valid == m * k the padded
 * form already is the final edge_index; otherwise run b200c_exclusive_scan on
 * counts and b200c_knn_compact.
 *
 * workspace: b200c_knn_workspace_bytes(...) bytes (may be 0).  The cosine distance needs one (the
 * rows' norms) and so do the 16-bit types (float copies of x and y); for these the full reported
 * size is required.  For fp32 the full size additionally enables the faster paths — for features
 * (32 <= dim <= 128, dim % 8 == 0, k <= 32) the tensor-core candidate path, for up to 8 features
 * (k <= 64, segments of 1024 points and more on average) the scan over Morton-ordered copies of x
 * and y that the call builds in the workspace; without it the plain exact kernels run.  All paths
 * return the same arrays.
 *
 * max_segment_rows: an upper bound of the row count of any segment of x or y, 0 when unknown (then
 * n and m are taken).  It only limits how many sorting passes the Morton-ordered path enqueues.
 *
 * The Morton-ordered path moves its chunks with bulk asynchronous copies whose waits are
 * bounded; if one ever runs out, 2^62 is added to *num_valid and the output is not valid.  The same
 * happens for segment pointers that overlap (segment sizes that add up to more than the rows): the
 * sorted copies are sized for a partition of the rows, so the pass leaves them empty and flags the call —
 * search such inputs without the workspace. */
size_t b200c_knn_workspace_bytes(int64_t n, int64_t m, int64_t dim, int64_t k,
                                 int dtype, int cosine, int64_t num_segments);
int b200c_knn(const void *x, const void *y, const int64_t *ptr_x,
              const int64_t *ptr_y, int64_t num_segments, int64_t n, int64_t m,
              int64_t dim, int64_t k, int dtype, int cosine,
              int64_t *edge_padded, int32_t *counts, int64_t *num_valid,
              int64_t max_segment_rows, void *workspace, size_t workspace_bytes,
              b200c_stream_t stream);

/* The ordering pass of the Morton-ordered scan on its own (fp32, up to 8 features): every segment's rows
 * sorted by the Morton key of their cell in the segment's bounding box (ties by row).  No counterpart
 * in the reference, which scans points in input order.
 *   first [num_segments + 1]  (int64) first padded position of every segment, a multiple of 256;
 *                             first[num_segments] <= b200c_morton_order_rows(n, num_segments)
 *   order [rows]              (int32) the row of x at each position of a segment's range, -1 in the
 *                             padding between a segment's last row and the next multiple of 256
 *   keys  [rows]              (uint32) the row's Morton key, 0xffffffff in the padding
 * Positions at and after first[num_segments] are not written.  workspace:
 * b200c_morton_order_workspace_bytes(...) bytes; max_segment_rows as for b200c_knn. */
size_t b200c_morton_order_workspace_bytes(int64_t n, int64_t dim, int64_t num_segments);
int64_t b200c_morton_order_rows(int64_t n, int64_t num_segments);
int b200c_morton_order(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n,
                       int64_t dim, int64_t max_segment_rows, int32_t *order, uint32_t *keys,
                       int64_t *first, void *workspace, size_t workspace_bytes,
                       b200c_stream_t stream);

/* Measurement aids (no counterpart in the reference).
 * b200c_profile_knn_scan(1): later calls of the Morton-ordered kNN path record CUDA events around
 * their scan kernel on the call's stream; b200c_profile_knn_scan_ms() waits for the last such kernel
 * and returns its duration in milliseconds (-1 if none was recorded).  One call of the path launches
 * the ordering passes and the scan; a roofline figure wants the scan alone.  Not thread safe.
 * b200c_probe_fp32: a kernel of nothing but independent fused multiply-adds over the whole device
 * (scratch: one float, device); *flops (host) receives the operations it performs, so that a caller
 * timing it has the FP32 rate this device sustains beside the nominal one. */
int b200c_profile_knn_scan(int enable);
float b200c_profile_knn_scan_ms(void);
int b200c_probe_fp32(int64_t iters, float *scratch, double *flops, b200c_stream_t stream);

/* Drops the -1 slots: edge_index (int64 [2, num_edges]) receives, for each
 * query q, its counts[q] valid slots at offsets[q].. (csrc/cuda/knn_cuda.cu:133-134). */
int b200c_knn_compact(const int64_t *edge_padded, const int32_t *counts,
                      const int64_t *offsets, int64_t m, int64_t k,
                      int64_t num_edges, int64_t *edge_index,
                      b200c_stream_t stream);

/* The tail of knn_graph on the device — replaces the flow swap, the `row != col` mask, the boolean
 * gathers and the stack of torch_cluster/knn.py:135-144.  From the padded kNN result of x against
 * itself (edge_padded, counts as written by b200c_knn):
 *   b200c_knn_graph_tail_count   kept[q] = valid slots of q, minus those equal to q when drop_self
 *   (b200c_exclusive_scan of kept -> offsets, offsets[m] = E)
 *   b200c_knn_graph_tail_write   edge_index int64 [2, E]: per query, in stored order, the kept
 *                                neighbours; row 0 = neighbour, row 1 = query when source_to_target,
 *                                else row 0 = query, row 1 = neighbour. */
int b200c_knn_graph_tail_count(const int64_t *edge_padded, const int32_t *counts, int64_t m, int64_t k,
                               int drop_self, int32_t *kept, b200c_stream_t stream);
int b200c_knn_graph_tail_write(const int64_t *edge_padded, const int32_t *counts, const int64_t *offsets,
                               int64_t m, int64_t k, int drop_self, int source_to_target,
                               int64_t num_edges, int64_t *edge_index, b200c_stream_t stream);

/* knn_graph with loop = False in one call, for fp32 / fp64 points of up to 8 features (one kernel) — the
 * search for k + 1 neighbours of every row of x in x, the `row != col` mask and the flow swap of
 * torch_cluster/knn.py:131-144 without the padded intermediate.
 *
 * edge_index is int64 [2, n * k].  A query whose k + 1 nearest points exist and include itself
 * writes its k other neighbours, in order, at slots q*k..; row 0 = neighbour and row 1 = query
 * when source_to_target, else the other way round.  *irregular (one int32, device) receives the
 * number of queries that do not have that shape (segments of fewer than k + 1 points; rows
 * pushed out of their own list by k + 1 exact duplicates); their slots are left unwritten.  When
 * it is 0 the result is final, otherwise run b200c_knn and the tail entry points instead.
 * Returns B200C_ERR_UNSUPPORTED for the 16-bit types and for more than 8 features, except fp32
 * feature vectors for which b200c_knn_graph_workspace_bytes answers non-zero (32 to 128 features, a
 * multiple of 8, k + 1 <= 32, 16-byte aligned x) when that workspace is given: the exact re-rank of the
 * tensor-core candidates (see b200c_knn) then writes the edge rows itself.
 *
 * workspace (optional for up to 8 features): b200c_knn_graph_workspace_bytes(...) bytes enable the scan
 * over a Morton-ordered copy of x for fp32 (see b200c_knn; max_segment_rows as there).  Should one of
 * that path's bounded waits run out, or the segments overlap, 2^30 is added to *irregular. */
size_t b200c_knn_graph_workspace_bytes(int64_t n, int64_t dim, int64_t k, int dtype,
                                       int64_t num_segments);
int b200c_knn_graph(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n,
                    int64_t dim, int64_t k, int dtype, int source_to_target,
                    int64_t *edge_index, int32_t *irregular, int64_t max_segment_rows,
                    void *workspace, size_t workspace_bytes, b200c_stream_t stream);

/* The same for a part of a larger point set, so that a host can cut one knn_graph call into
 * groups of whole segments and overlap their copies with the search of the next group: x, ptr,
 * n describe the part (ptr starts at 0), index_base (the part's first row in the whole set) is
 * added to every index written, edge_row0 points to the part's first slot in row 0 of the whole
 * edge_index and row_stride is the distance to the same slot of row 1 (the whole set's n * k).
 * No counterpart in the reference, which has no host-buffer path. */
int b200c_knn_graph_part(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n,
                         int64_t dim, int64_t k, int dtype, int source_to_target,
                         int64_t index_base, int64_t *edge_row0, int64_t row_stride,
                         int32_t *irregular, int64_t max_segment_rows, void *workspace,
                         size_t workspace_bytes, b200c_stream_t stream);

/* The same for the cosine distance of the reference (csrc/cuda/knn_cuda.cu:9-28, 55-59) on fp32 feature
 * vectors: tensor-core candidates over the normalised rows, the exact re-rank — which evaluates
 * 1 - dot / (|x| |y|) as the reference does — writing the edge rows.  The workspace is required
 * (b200c_knn_graph_cosine_workspace_bytes; 0: not applicable, use b200c_knn with cosine = 1 and the tail
 * entry points).  The reference composes this case from `knn(..., cosine=True)` and the mask of
 * torch_cluster/knn.py:131-144. */
size_t b200c_knn_graph_cosine_workspace_bytes(int64_t n, int64_t dim, int64_t k,
                                              int64_t num_segments);
int b200c_knn_graph_cosine(const void *x, const int64_t *ptr, int64_t num_segments, int64_t n,
                           int64_t dim, int64_t k, int source_to_target, int64_t *edge_index,
                           int32_t *irregular, void *workspace, size_t workspace_bytes,
                           b200c_stream_t stream);

/* Fixed-radius search — replaces radius_kernel and its -1 padded output
 * (csrc/cuda/radius_cuda.cu:9-42, 75-95) by count -> exclusive scan -> fill.
 *
 * Pass 1, b200c_radius_count:
 *   counts[q] = min(max_num_neighbors, #{x in segment(q): dist < (T)(r * r),
 *                                        and not (ignore_same_index and x == q)}).
 * The comparison is strict and r * r is formed in double and narrowed to the
 * data type (csrc/cuda/radius_cuda.cu:33, 90).
 * Pass 2, b200c_radius_fill: writes, for each query q, its first counts[q] hits
 * in ascending x order at offsets[q].. of edge_index (int64 [2, num_edges];
 * row 0 = q, row 1 = x index) — the truncation rule of
 * csrc/cuda/radius_cuda.cu:33-40.  offsets is the exclusive scan of counts.
 *
 * Workspace: b200c_radius_workspace_bytes(n, m, dim, max_num_neighbors, dtype).
 * For fp32 / fp64 it is optional and non-zero when a one-pass mode applies (small
 * neighbour caps): pass 1 then also parks the hits in the workspace
 * (m * max_num_neighbors int32) and pass 2 only copies them, instead of scanning
 * the points a second time; with NULL / too few bytes both passes scan.  For the
 * 16-bit types it is required (pass 1 leaves float copies of x and y there for
 * pass 2).  Give both passes the same workspace, untouched in between. */
size_t b200c_radius_workspace_bytes(int64_t n, int64_t m, int64_t dim,
                                    int64_t max_num_neighbors, int dtype);
/* Workspace of the screened scan for fp32 points of up to 8 features (0: not applicable — other
 * types, tiny inputs, fewer than 512 points per segment on average).  Given at least this many bytes
 * (it is never less than b200c_radius_workspace_bytes asks for the same call), pass 1 first lays the
 * points out in chunks of 256 (coordinates relative to the segment's first point, their squared norms,
 * the original coordinates) and then screens every (query, chunk) pair with `dim` fused multiply-adds per
 * point against a threshold that covers the rounding of both sides; only chunks with a point at or below
 * it are evaluated again for that query with the reference's arithmetic (csrc/cuda/radius_cuda.cu:28-33),
 * so the result is the same.  Worth it when hits are sparse: a screened pair costs about half of an exact
 * one, a pair with a hit costs both.  Segments of at least 2048 * max_num_neighbors points guarantee that
 * (a query keeps at most max_num_neighbors hits), which is the rule torch_cluster::radius applies.
 * Pass 1 parks the hits (up to 64 per query for neighbour caps above 256), pass 2 copies them and scans
 * again only for queries that found more than were parked.  After pass 1 the first 8 bytes of the
 * workspace are a status word (int64): non-zero means that a bounded wait inside the scan ran out (1),
 * or that the segments of x overlap so far that their chunk arrays do not fit (2), and the counts are
 * invalid; read it together with the total of the counts before sizing the output. */
size_t b200c_radius_screen_workspace_bytes(int64_t n, int64_t m, int64_t dim,
                                           int64_t max_num_neighbors, int dtype,
                                           int64_t num_segments);
int b200c_radius_count(const void *x, const void *y, const int64_t *ptr_x,
                       const int64_t *ptr_y, int64_t num_segments, int64_t n,
                       int64_t m, int64_t dim, double r,
                       int64_t max_num_neighbors, int ignore_same_index,
                       int dtype, int32_t *counts, void *workspace,
                       size_t workspace_bytes, b200c_stream_t stream);
int b200c_radius_fill(const void *x, const void *y, const int64_t *ptr_x,
                      const int64_t *ptr_y, int64_t num_segments, int64_t n,
                      int64_t m, int64_t dim, double r,
                      int64_t max_num_neighbors, int ignore_same_index,
                      int dtype, const int32_t *counts, const int64_t *offsets,
                      int64_t num_edges, int64_t *edge_index, void *workspace,
                      size_t workspace_bytes, b200c_stream_t stream);

/* The same two passes for a y that is a slice of a larger query set whose row numbers x shares
 * (one point cloud searched in itself, its queries split over several GPUs): the pair skipped by
 * ignore_same_index is x row (q + query_index_base), q being the row of the slice — the global
 * row comparison of csrc/cuda/radius_cuda.cu:33 carried over to a slice.  The edge rows still
 * hold q, the row of the slice; the caller adds the base.  With swap_rows the fill pass writes
 * row 0 = x index, row 1 = q: the `source_to_target` orientation of radius_graph
 * (torch_cluster/radius.py:143-148) without a second pass over the result.  query_index_base = 0
 * and swap_rows = 0 give b200c_radius_count / b200c_radius_fill.  The slice form has no
 * counterpart in the reference, which has no multi-GPU path. */
int b200c_radius_count_part(const void *x, const void *y, const int64_t *ptr_x,
                            const int64_t *ptr_y, int64_t num_segments, int64_t n,
                            int64_t m, int64_t dim, double r, int64_t max_num_neighbors,
                            int ignore_same_index, int64_t query_index_base, int dtype,
                            int32_t *counts, void *workspace, size_t workspace_bytes,
                            b200c_stream_t stream);
int b200c_radius_fill_part(const void *x, const void *y, const int64_t *ptr_x,
                           const int64_t *ptr_y, int64_t num_segments, int64_t n,
                           int64_t m, int64_t dim, double r, int64_t max_num_neighbors,
                           int ignore_same_index, int64_t query_index_base, int swap_rows,
                           int dtype, const int32_t *counts, const int64_t *offsets,
                           int64_t num_edges, int64_t *edge_index, void *workspace,
                           size_t workspace_bytes, b200c_stream_t stream);

/* Fixed-radius search that evaluates every pair once, for neighbour caps too large for the one-pass
 * mode above (fp32 / fp64, up to 8 features): pass 1 counts like b200c_radius_count and also stores one
 * hit bit per (query, point) in a bit matrix in the workspace; pass 2 writes the edges from those bits
 * (an HBM-bound kernel) instead of scanning the points again.  Same results as count + fill.
 *
 * The matrix's size depends on the segment sizes, so the caller hands over host copies of the segment
 * pointers (ptr_x_host, ptr_y_host: int64 [num_segments + 1] in host memory, equal to the device
 * copies; NULL with ptr_x == NULL for one segment): b200c_radius_mask_workspace_bytes gives the size
 * (0 = not applicable, also for pointers that do not start at 0, decrease, or do not end at n / m),
 * pass 1 checks it.  Rows: a query of a segment with n_b points owns ceil(n_b / c) * c / 32 words, c being the
 * scan's chunk (1024 points for 3-D fp32).  No counterpart in the reference, which evaluates once but
 * pads its output to max_num_neighbors slots per query. */
size_t b200c_radius_mask_workspace_bytes(const int64_t *ptr_x_host, const int64_t *ptr_y_host,
                                         int64_t num_segments, int64_t n, int64_t m, int64_t dim,
                                         int dtype);
int b200c_radius_count_masks(const void *x, const void *y, const int64_t *ptr_x,
                             const int64_t *ptr_y, const int64_t *ptr_x_host,
                             const int64_t *ptr_y_host, int64_t num_segments, int64_t n,
                             int64_t m, int64_t dim, double r, int64_t max_num_neighbors,
                             int ignore_same_index, int dtype, int32_t *counts,
                             void *workspace, size_t workspace_bytes, b200c_stream_t stream);
/* b200c_radius_count_masks for a slice of a larger query set: see b200c_radius_count_part. */
int b200c_radius_count_masks_part(const void *x, const void *y, const int64_t *ptr_x,
                                  const int64_t *ptr_y, const int64_t *ptr_x_host,
                                  const int64_t *ptr_y_host, int64_t num_segments, int64_t n,
                                  int64_t m, int64_t dim, double r, int64_t max_num_neighbors,
                                  int ignore_same_index, int64_t query_index_base, int dtype,
                                  int32_t *counts, void *workspace, size_t workspace_bytes,
                                  b200c_stream_t stream);
int b200c_radius_fill_masks_part(const int64_t *ptr_x, const int64_t *ptr_y,
                                 int64_t num_segments, int64_t n, int64_t m, int64_t dim,
                                 int swap_rows, int dtype, const int32_t *counts,
                                 const int64_t *offsets, int64_t num_edges, int64_t *edge_index,
                                 const void *workspace, b200c_stream_t stream);
int b200c_radius_fill_masks(const int64_t *ptr_x, const int64_t *ptr_y, int64_t num_segments,
                            int64_t n, int64_t m, int64_t dim, int dtype,
                            const int32_t *counts, const int64_t *offsets, int64_t num_edges,
                            int64_t *edge_index, const void *workspace, b200c_stream_t stream);

/* Nearest point assignment — replaces nearest_kernel + nearest_cuda
 * (csrc/cuda/nearest_cuda.cu:9-61, 63-88).
 *
 * out[i] (int64 [n]) = the row of y, within the segment of x row i, with the smallest squared
 * distance to x[i].  As in the reference only distances below 1e38 compete (none: out[i] = 0),
 * NaN never wins, and among equal minima the reference's reduction order decides: the point with
 * the smallest ((index - segment start) mod 1024, index).
 * workspace: b200c_nearest_workspace_bytes(...) bytes, non-zero (and required) for the 16-bit
 * types only. */
size_t b200c_nearest_workspace_bytes(int64_t n, int64_t m, int64_t dim, int dtype);
int b200c_nearest(const void *x, const void *y, const int64_t *ptr_x,
                  const int64_t *ptr_y, int64_t num_segments, int64_t n, int64_t m,
                  int64_t dim, int dtype, int64_t *out, void *workspace,
                  size_t workspace_bytes, b200c_stream_t stream);

/* Farthest point sampling — replaces fps_kernel and its launch in fps_cuda
 * (csrc/cuda/fps_cuda.cu:9-68, 100-109).
 *
 * For every segment b (ptr [num_segments + 1]) writes out_ptr[b+1] - out_ptr[b] sample indices
 * (global rows of src) at out[out_ptr[b]..]: the first is ptr[b] + start[b] (start == NULL: 0),
 * each further one the point farthest from the samples so far, the running distance starting at
 * 5e4 as in the reference; among equal maxima the point with the smallest
 * ((index - segment start) mod 256, index) wins, which is what the reference's 256-thread
 * reduction yields.  out_ptr is the caller's (the reference derives it from ratio on the host
 * side, fps_cuda.cu:83-86).  Segments of up to 200 KB / ((dim + 1) * element size) points are
 * held in shared memory for the whole call; larger ones run from global memory.
 * workspace: b200c_fps_workspace_bytes(n, dim, dtype) bytes, required. */
size_t b200c_fps_workspace_bytes(int64_t n, int64_t dim, int dtype);
int b200c_fps(const void *src, const int64_t *ptr, const int64_t *out_ptr,
              const int64_t *start, int64_t num_segments, int64_t n, int64_t dim,
              int dtype, int64_t *out, void *workspace, size_t workspace_bytes,
              b200c_stream_t stream);

/* b200c_fps, leaving out the segments of more than max_segment_points points (their slots of
 * `out` stay unwritten): for callers that hand those to b200c_fps_large_segment. */
int b200c_fps_up_to(const void *src, const int64_t *ptr, const int64_t *out_ptr,
                    const int64_t *start, int64_t num_segments, int64_t n, int64_t dim,
                    int dtype, int64_t max_segment_points, int64_t *out, void *workspace,
                    size_t workspace_bytes, b200c_stream_t stream);

/* Farthest point sampling of ONE large segment spread over many SMs (fp32, up to 8 features, up to
 * b200c_fps_large_segment_max_points points: 8192 — or 4096 above 3 features — per SM): a
 * cooperative launch of one CTA per 8192 points, each holding its points in registers; per step
 * the CTAs publish their best candidate in global memory, meet at a counter (bounded polling) and
 * all continue with the overall winner.  The reference runs any segment on one thread block; this
 * entry point has no counterpart there.  Same results as b200c_fps.
 *
 * src: the whole point array; seg_lo / seg_points: the segment's rows; start_offset: first sample
 * relative to seg_lo; count >= 1 samples are written to out[0..count) (global row numbers).
 * *status (int32, device; zero it before) becomes 1 if a wait ran out — the samples are then not
 * valid.  workspace: b200c_fps_large_segment_workspace_bytes() bytes.  Calls on one device must
 * not overlap (every launch wants all its CTAs resident). */
int64_t b200c_fps_large_segment_max_points(int64_t dim, int dtype);
size_t b200c_fps_large_segment_workspace_bytes(void);
int b200c_fps_large_segment(const void *src, int64_t seg_lo, int64_t seg_points,
                            int64_t start_offset, int64_t count, int64_t dim, int dtype,
                            int64_t *out, void *workspace, size_t workspace_bytes,
                            int32_t *status, b200c_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_CLUSTER_H_ */
