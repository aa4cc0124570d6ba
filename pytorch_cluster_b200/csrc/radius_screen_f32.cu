// Instantiations and host side of the screened radius scan (radius_screen.cuh).
#include "launchers.h"
#include "radius_compact.cuh"
#include "radius_screen.cuh"

namespace b200c {

static size_t rs_align(size_t v) { return (v + 255) / 256 * 256; }

// Slots per query that pass 1 parks hits in: the neighbour cap itself while that scratch stays
// modest, else a fixed 64 (queries that find more are scanned again by pass 2).
static constexpr int64_t RS_DIRECT_MAX_BYTES = 1ll << 30;
static constexpr int RS_DIRECT_FALLBACK = 64;

static int rs_direct_cap(int64_t m, int64_t max_nn) {
  if (max_nn <= 256 && m * max_nn * 4 <= RS_DIRECT_MAX_BYTES) return (int)max_nn;
  return max_nn < RS_DIRECT_FALLBACK ? (int)max_nn : RS_DIRECT_FALLBACK;
}

bool radius_screen_applicable(int64_t n, int64_t m, int dim, int64_t num_segments) {
  // enough points per segment for chunks of 256 to be mostly full; row numbers travel as int32
  return dim >= 1 && dim <= SP_MAX_DIM && num_segments >= 1 && m >= 1 && n >= 1024 && n / num_segments >= 512 &&
         n <= 0x7fffffffLL - (int64_t)num_segments * SP_CHUNK && m <= (1ll << 40);
}

static size_t radius_screen_carve(RadiusScreenView *v, void *workspace, int64_t n, int64_t m, int dim, int64_t max_nn,
                                  int64_t segs) {
  char *p = (char *)workspace;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    char *r = p ? p + off : nullptr;
    off += rs_align(bytes);
    return r;
  };
  RadiusScreenView t{};
  const int64_t raw = n + segs * (SP_CHUNK - 1);
  t.cap = (raw + SP_CHUNK - 1) / SP_CHUNK * SP_CHUNK;
  t.direct_cap = rs_direct_cap(m, max_nn);
  t.status = (int64_t *)take(8);
  t.sptr = (int64_t *)take((size_t)(segs + 1) * 8);
  t.stat = (uint32_t *)take((size_t)segs * 4);
  t.blob = (float *)take((size_t)t.cap * (2 * dim + 2) * 4);
  t.direct = (int32_t *)take((size_t)m * t.direct_cap * 4);
  if (v) *v = t;
  return off;
}

size_t radius_screen_workspace_bytes(int64_t n, int64_t m, int dim, int64_t max_nn, int64_t num_segments) {
  if (!radius_screen_applicable(n, m, dim, num_segments) || max_nn < 1) return 0;
  return radius_screen_carve(nullptr, nullptr, n, m, dim, max_nn, num_segments);
}

template <int DIM>
static int launch_radius_screen_dim(const RadiusScreenArgs &a, bool fill, cudaStream_t stream) {
  using Cfg = RadiusScreen<DIM>;
  auto kern = radius_screen_kernel<DIM>;
  static unsigned long long configured = 0ull;  // devices on which the shared-memory opt-in is done
  B200C_CUDA(opt_in_shared_memory(kern, Cfg::SMEM_BYTES, configured));
  const int64_t tiles = (a.m + KS_TILE - 1) / KS_TILE;
  if (tiles > 0x7fffffffLL) {
    set_error("too many query tiles");
    return B200C_ERR_INVALID;
  }
  if (!fill) {
    rs_layout_kernel<<<1, 1024, 0, stream>>>(a.ptr_x, a.num_segments, a.n, a.v);
    B200C_LAUNCH_CHECK("rs_layout_kernel");
    rs_blob_kernel<DIM><<<(unsigned)(a.v.cap / SP_CHUNK), SP_CHUNK, 0, stream>>>(a.x, a.ptr_x, a.num_segments, a.n, a.v);
    B200C_LAUNCH_CHECK("rs_blob_kernel");
    kern<<<(unsigned)tiles, KS_THREADS, Cfg::SMEM_BYTES, stream>>>(a);
    B200C_LAUNCH_CHECK("radius_screen_kernel");
    return B200C_OK;
  }
  const int64_t threads = (a.m + 3) / 4 * 32;  // a warp per four queries
  radius_direct_compact_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, stream>>>(
      a.v.direct, a.counts, a.offsets, a.m, (int64_t)a.v.direct_cap, a.out_row, a.out_col);
  B200C_LAUNCH_CHECK("radius_direct_compact_kernel");
  if ((int64_t)a.v.direct_cap < a.max_nn) {
    kern<<<(unsigned)tiles, KS_THREADS, Cfg::SMEM_BYTES, stream>>>(a);
    B200C_LAUNCH_CHECK("radius_screen_kernel");
  }
  return B200C_OK;
}

// Both passes of the radius search over `workspace` (radius_screen_workspace_bytes; the same, untouched
// in between, for both).  fill == false: layout, chunk arrays, scan (counts, parked hits).  fill == true:
// the copy of the parked hits and, for caps above the parked rows, the second scan.
int launch_radius_screen_f32(const RadiusArgs &r, bool fill, void *workspace) {
  RadiusScreenArgs a{};
  a.x = (const float *)r.x;
  a.y = (const float *)r.y;
  a.ptr_x = r.ptr_x;
  a.ptr_y = r.ptr_y;
  a.num_segments = r.num_segments;
  a.n = r.n;
  a.m = r.m;
  a.r2 = (float)(r.r * r.r);  // formed in double, narrowed once (csrc/cuda/radius_cuda.cu:90)
  a.max_nn = r.max_nn;
  a.ignore_same = r.ignore_same;
  a.query_base = r.query_base;
  a.mode = fill ? RS_PASS_FILL : RS_PASS_COUNT;
  a.counts = r.counts;
  a.offsets = r.offsets;
  a.out_row = r.out_row;
  a.out_col = r.out_col;
  (void)radius_screen_carve(&a.v, workspace, r.n, r.m, r.dim, r.max_nn, r.num_segments);
  switch (r.dim) {
    case 1: return launch_radius_screen_dim<1>(a, fill, r.stream);
    case 2: return launch_radius_screen_dim<2>(a, fill, r.stream);
    case 3: return launch_radius_screen_dim<3>(a, fill, r.stream);
    case 4: return launch_radius_screen_dim<4>(a, fill, r.stream);
    case 5: return launch_radius_screen_dim<5>(a, fill, r.stream);
    case 6: return launch_radius_screen_dim<6>(a, fill, r.stream);
    case 7: return launch_radius_screen_dim<7>(a, fill, r.stream);
    case 8: return launch_radius_screen_dim<8>(a, fill, r.stream);
  }
  set_error("screened radius scan called with dim=%d", r.dim);
  return B200C_ERR_INVALID;
}

}  // namespace b200c
