// Spatially ordered copies of low-dimensional fp32 point sets, the input of the kNN scan of
// knn_spatial.cuh.
//
// Brute-force kNN evaluates every (query, point) pair whatever the order of the points, and its
// result does not depend on that order (candidates are ranked by (distance, original index)).
// The order decides how fast a query's bound — its k-th best distance so far — falls, and
// with it how often the scan has to leave its hit-free inner loop.  So each segment's points are
// sorted along a Morton curve of the segment's bounding box; queries sorted the same way then
// start their scan at the chunk of points around them and have their final bound after a few
// chunks.
//
// Layout of a sorted set ("view") in the caller's workspace, indexed by the padded sorted position p
// (every segment starts at a multiple of SP_CHUNK and is padded to one):
//   blob  [cap / SP_CHUNK][2 DIM + 2][SP_CHUNK]  per chunk of 256 positions, back to back so that one
//         bulk copy moves a chunk: DIM arrays of coordinates minus the centre of the segment's
//         bounding box (padding: +inf), the squared norms of those (padding: +inf), the original rows
//         as int32 (padding: -1), DIM arrays of original coordinates (read when a candidate is
//         re-evaluated exactly)
//   idx   [cap]       original row of the point, int32                            (padding: -1)
//   key   [cap]       Morton key, uint32                                (padding: 0xffffffff)
//   sptr  [B + 1]     first padded position of every segment, int64
//   box   [B][2 DIM]  bounding box (min, max per feature) of every segment's points
//   stat  [B][2]      largest w of the segment (float bits of a non-negative value), spare
#pragma once

#include "common.cuh"

namespace b200c {

constexpr int SP_CHUNK = 256;         // points per chunk of the scan: 32 lanes x 8 points
constexpr int SP_TILE = 64;           // queries per thread block of the scan
constexpr int SP_SORT_BLOCK = 16384;  // keys one thread block sorts in shared memory
constexpr int SP_MAX_DIM = 8;

struct SpatialView {
  float *blob;      // [cap / SP_CHUNK][2 dim + 2][SP_CHUNK], points only
  int32_t *idx;     // [cap]
  uint32_t *key;    // [cap]
  int64_t *sptr;    // [B + 1]
  float *box;       // [B][2 * dim]
  uint32_t *stat;   // [B][2]
  int64_t cap;      // positions allocated: rows + B * (SP_CHUNK - 1), rounded up to SP_CHUNK
  // scratch of the sort: 64-bit (key, local row) pairs, every segment padded to a power of two
  uint64_t *pairs;  // [pairs_cap]
  int64_t *pptr;    // [B + 1] first pair of every segment
  int64_t *lptr;    // [B + 1] sort blocks (SP_SORT_BLOCK pairs) of the segments above one block, before each segment
  int64_t pairs_cap;
  // bucket sort of the segments above one sort block: the pairs scattered into buckets (pairs2), per
  // such segment up to SP_MAX_BUCKETS - 1 splitters and bucket counts / offsets (indexed by the
  // segment's lptr), and the table of buckets to sort (segment, first position, size)
  uint64_t *pairs2;     // [rows]
  uint64_t *split;      // [large_blocks][SP_MAX_BUCKETS]
  int32_t *bcount;      // [large_blocks][SP_MAX_BUCKETS]
  int32_t *boffset;     // [large_blocks][SP_MAX_BUCKETS + 1]
  int32_t *bcursor;     // [large_blocks][SP_MAX_BUCKETS]
  int32_t *table;       // [table_cap][4]: segment, first position in the segment, size, last-of-segment flag
  int32_t *table_count; // [1]
  int32_t *bad;         // [1] non-zero: the segment pointers overlap (their sizes add up to more than the rows);
                        //     the layout is then empty and the scan flags its result
  int64_t table_cap;
};

constexpr int SP_MAX_BUCKETS = 256;
constexpr int SP_BUCKET_TARGET = 2048;          // points per bucket aimed at
constexpr int64_t SP_BUCKET_MAX_ROWS = 1 << 19; // segments up to this size take the bucket sort (256 buckets of 2048)

// Bytes of workspace one view needs (points: with coordinates; queries: order and keys only).
size_t spatial_view_bytes(int64_t rows, int dim, int64_t num_segments, bool points);
// Carves a view out of `workspace` (256-byte aligned pieces); returns the bytes used.
size_t spatial_view_carve(SpatialView *v, void *workspace, int64_t rows, int dim, int64_t num_segments, bool points);

// Sorts the rows of `pts` ([rows, dim] fp32, segments ptr / num_segments) into `v`.  box_from:
// nullptr to use the bounding boxes of these rows (written to v->box), else the boxes of another
// view (queries are keyed in the box of the points they are searched in).  points: also write the
// coordinate arrays.  max_segment_rows: an upper bound of any segment's row count (rows when
// unknown); it only limits how many sorting passes are enqueued.
int launch_spatial_sort(const float *pts, const int64_t *ptr, int64_t num_segments, int64_t rows, int dim,
                        const float *box_from, bool points, int64_t max_segment_rows, SpatialView *v,
                        cudaStream_t stream);

}  // namespace b200c
