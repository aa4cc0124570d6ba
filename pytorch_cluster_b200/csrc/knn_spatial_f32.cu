// Instantiations and host side of the Morton-ordered kNN scan (knn_spatial.cuh).
#include "knn_spatial.cuh"
#include "launchers.h"

namespace b200c {

template <int DIM, int KP, bool ROLLED>
static int launch_knn_spatial_one(const KnnSpatialArgs &a, int64_t tiles, cudaStream_t stream) {
  using Cfg = KnnSpatialLayout<DIM, KP, ks_stages(DIM, KP, ROLLED)>;
  auto kern = knn_spatial_kernel<DIM, KP, ROLLED>;
  static unsigned long long configured = 0ull;  // devices on which the shared-memory opt-in is done
  B200C_CUDA(opt_in_shared_memory(kern, Cfg::SMEM_BYTES, configured));
  kern<<<(unsigned)(tiles * a.parts), KS_THREADS, Cfg::SMEM_BYTES, stream>>>(a);
  B200C_LAUNCH_CHECK("knn_spatial_kernel");
  if (a.parts > 1) {
    const int64_t padded = tiles * KS_TILE;
    knn_spatial_merge_kernel<KP><<<(unsigned)((padded + WARPS_PER_CTA - 1) / WARPS_PER_CTA), CTA_THREADS, 0, stream>>>(
        a, padded);
    B200C_LAUNCH_CHECK("knn_spatial_merge_kernel");
  }
  return B200C_OK;
}

// Thread blocks per query tile.  One block per tile fills the device from about one block per SM on;
// below that the points of every tile's segment are shared out over three blocks (five for very few
// tiles), as long as each keeps a few dozen chunks to scan.  Odd counts: the scan alternates sides, and
// an even count would hand a block chunks of one side only (measured slower).
static int knn_spatial_parts(int64_t n, int64_t padded_queries, int64_t num_segments) {
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) (void)cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t tiles = padded_queries / KS_TILE;
  const int64_t chunks = n / num_segments / SP_CHUNK;  // of an average segment
  int parts = 1;
  if (tiles * 5 <= 2 * sms && chunks >= 5 * 32)
    parts = 5;
  else if (tiles * 5 <= 6 * sms && chunks >= 3 * 32)
    parts = 3;
  return parts < 1 ? 1 : parts;
}

static int64_t padded_rows(int64_t rows, int64_t segs) {
  const int64_t raw = rows + segs * (SP_CHUNK - 1);
  return (raw + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
}

template <int DIM>
static int launch_knn_spatial_dim(const KnnSpatialArgs &a, int64_t tiles, bool short_segments, cudaStream_t stream) {
  if (a.k > 32) return launch_knn_spatial_one<DIM, 64, true>(a, tiles, stream);
  return short_segments ? launch_knn_spatial_one<DIM, 32, true>(a, tiles, stream)
                        : launch_knn_spatial_one<DIM, 32, false>(a, tiles, stream);
}

// ---- optional timing of the scan kernel alone (for benchmarks: roofline figures want the kernel's
// own duration, and one call of the path launches the ordering passes as well) ----
static bool g_scan_timing = false;
static cudaEvent_t g_scan_begin = nullptr, g_scan_end = nullptr;

int knn_spatial_scan_timing(int enable) {
  if (enable && g_scan_begin == nullptr) {
    B200C_CUDA(cudaEventCreate(&g_scan_begin));
    B200C_CUDA(cudaEventCreate(&g_scan_end));
  }
  g_scan_timing = enable != 0;
  return B200C_OK;
}

float knn_spatial_last_scan_ms() {
  float ms = -1.f;
  if (g_scan_begin == nullptr || cudaEventSynchronize(g_scan_end) != cudaSuccess ||
      cudaEventElapsedTime(&ms, g_scan_begin, g_scan_end) != cudaSuccess)
    return -1.f;
  return ms;
}

bool knn_spatial_applicable(int64_t n, int64_t m, int dim, int k, int64_t num_segments) {
  // enough points per segment for the ordering to pay (a chunk is 256 points), and within the
  // instantiated selection widths
  return dim >= 1 && dim <= SP_MAX_DIM && k <= 64 && num_segments >= 1 && m >= 1 && n >= 2048 &&
         n / num_segments >= 1024 && n <= 0x7fffffffLL - (int64_t)num_segments * SP_CHUNK;
}

size_t knn_spatial_workspace_bytes(int64_t n, int64_t m, int dim, int64_t num_segments, bool same_set) {
  size_t bytes = spatial_view_bytes(n, dim, num_segments, true);
  if (!same_set) bytes += spatial_view_bytes(m, dim, num_segments, false);
  // lists of an x-split scan: at most 8 parts of 64 keys per padded query, and only for few queries
  const int64_t padded = padded_rows(same_set ? n : m, num_segments);
  const int parts = knn_spatial_parts(n, padded, num_segments);
  if (parts > 1) bytes += (size_t)padded * parts * 64 * sizeof(uint64_t) + 256;
  return bytes;
}

int launch_knn_spatial_f32(const KnnArgs &a, void *workspace, int64_t max_segment_rows) {
  const bool same_set = a.x == a.y && a.ptr_x == a.ptr_y && a.n == a.m;
  KnnSpatialArgs s{};
  size_t off = spatial_view_carve(&s.xv, workspace, a.n, a.dim, a.num_segments, true);
  int st = launch_spatial_sort((const float *)a.x, a.ptr_x, a.num_segments, a.n, a.dim, nullptr, true,
                               max_segment_rows, &s.xv, a.stream);
  if (st != B200C_OK) return st;
  int64_t padded_queries;
  if (same_set) {
    s.yv = s.xv;
    padded_queries = s.xv.cap;
  } else {
    spatial_view_carve(&s.yv, (char *)workspace + off, a.m, a.dim, a.num_segments, false);
    // queries are keyed in the boxes of the points they are searched in; their segments are padded
    // to chunks as well, which keeps every tile of 64 inside one segment
    st = launch_spatial_sort((const float *)a.y, a.ptr_y, a.num_segments, a.m, a.dim, s.xv.box, false, 0, &s.yv,
                             a.stream);
    if (st != B200C_OK) return st;
    padded_queries = s.yv.cap;
  }
  s.parts = knn_spatial_parts(a.n, padded_queries, a.num_segments);
  s.part_keys = nullptr;
  if (s.parts > 1) {
    if (!same_set) off += spatial_view_bytes(a.m, a.dim, a.num_segments, false);
    s.part_keys = (Key<float> *)((char *)workspace + (off + 255) / 256 * 256);
  }
  s.y = (const float *)a.y;
  s.num_segments = a.num_segments;
  s.k = a.k;
  s.out_row = a.out_row;
  s.out_col = a.out_col;
  s.counts = a.counts;
  s.num_valid = a.num_valid;
  s.graph_out = a.graph_out;
  s.graph_row_stride = a.graph_row_stride;
  s.graph_index_base = a.graph_index_base;
  s.graph_s2t = a.graph_s2t;
  s.graph_irregular = a.graph_irregular;
  s.eager_steps = 1;
  s.lazy_fill = a.k <= 32 ? 16 : 32;
  // rolled variant up to 16 chunks per segment on average (measured on 3-D clouds, k = 21: 0.378 against 0.402 ms
  // at 2048 points per cloud, 0.471 against 0.485 ms at 4096, 0.627 against 0.619 ms at 8192, 0.937 against
  // 0.898 ms at 16384)
  const bool short_segments = a.n / a.num_segments <= 16 * SP_CHUNK;
  const int64_t tiles = padded_queries / KS_TILE;  // an upper bound: blocks past the last segment leave at once
  if (g_scan_timing) B200C_CUDA(cudaEventRecord(g_scan_begin, a.stream));
  set_error("Morton-ordered kNN called with dim=%d", a.dim);
  st = B200C_ERR_INVALID;
  switch (a.dim) {
    case 1: st = launch_knn_spatial_dim<1>(s, tiles, short_segments, a.stream); break;
    case 2: st = launch_knn_spatial_dim<2>(s, tiles, short_segments, a.stream); break;
    case 3: st = launch_knn_spatial_dim<3>(s, tiles, short_segments, a.stream); break;
    case 4: st = launch_knn_spatial_dim<4>(s, tiles, short_segments, a.stream); break;
    case 5: st = launch_knn_spatial_dim<5>(s, tiles, short_segments, a.stream); break;
    case 6: st = launch_knn_spatial_dim<6>(s, tiles, short_segments, a.stream); break;
    case 7: st = launch_knn_spatial_dim<7>(s, tiles, short_segments, a.stream); break;
    case 8: st = launch_knn_spatial_dim<8>(s, tiles, short_segments, a.stream); break;
  }
  if (st == B200C_OK && g_scan_timing) B200C_CUDA(cudaEventRecord(g_scan_end, a.stream));
  return st;
}

}  // namespace b200c
