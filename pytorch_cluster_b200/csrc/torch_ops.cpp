// Torch operator layer: registers `torch_cluster::knn` and `torch_cluster::radius` with the
// schemas of the reference (csrc/knn.cpp:22-40, csrc/radius.cpp:22-39) and forwards to the C ABI
// of include/b200_cluster.h.  Host logic only: argument checks with the reference's messages
// (csrc/cuda/utils.cuh:5-9, csrc/cuda/knn_cuda.cu:91-114), output allocation through the ATen
// caching allocator, the caller's current stream, and one device-to-host read of the edge
// count where the output size depends on the data.  There is no CPU branch: a CPU tensor is an
// error here, not a fallback.
#include <algorithm>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <ATen/cuda/CUDAEvent.h>
#include <torch/script.h>
#include <nvtx3/nvToolsExt.h>

#include <vector>

#include "b200_cluster.h"
#include "b200_cluster_torch.h"

namespace {

#define CHECK_CUDA(x) TORCH_CHECK(x.device().is_cuda(), #x " must be CUDA tensor")
#define CHECK_INPUT(x) TORCH_CHECK(x, "Input mismatch")
#define CHECK_CONTIGUOUS(x) TORCH_CHECK(x.is_contiguous(), #x " must be contiguous")

// neighbour caps up to this use the one-pass mode of b200c_radius_count (when its scratch fits); above it,
// the bit-matrix mode when the matrix stays below the byte limit
constexpr int64_t kRadiusDirectCap = 256;
constexpr size_t kRadiusMaskMaxBytes = (size_t)8 << 30;

// A named range around an operator call, visible in Nsight Systems timelines (header-only NVTX:
// a no-op costing a few nanoseconds when no tool is attached).
struct OpRange {
  explicit OpRange(const char *name) { nvtxRangePushA(name); }
  ~OpRange() { nvtxRangePop(); }
  OpRange(const OpRange &) = delete;
  OpRange &operator=(const OpRange &) = delete;
};

void check_status(int status) {
  TORCH_CHECK(status == B200C_OK, "b200_cluster: ", b200c_last_error());
}

// float, double, and the 16-bit types with the reference's rounding of every operation to the
// 16-bit type (csrc/cuda/knn_cuda.cu:125, csrc/cuda/radius_cuda.cu:84-85).  kNN on bfloat16 is an
// extension: the reference dispatches it for radius only.
int dtype_code(const torch::Tensor &t) {
  switch (t.scalar_type()) {
    case at::kFloat: return B200C_F32;
    case at::kDouble: return B200C_F64;
    case at::kHalf: return B200C_F16;
    case at::kBFloat16: return B200C_BF16;
    default: TORCH_CHECK(false, "expected a floating point tensor, got ", t.scalar_type());
  }
  return -1;
}

struct Prepared {
  torch::Tensor x, y, ptr_x, ptr_y;
  const int64_t *px = nullptr, *py = nullptr;
  int64_t num_segments = 1;
  int dtype = B200C_F32;
};

Prepared prepare(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> ptr_x,
                 std::optional<torch::Tensor> ptr_y) {
  CHECK_CUDA(x);
  CHECK_CONTIGUOUS(x);
  CHECK_INPUT(x.dim() == 2);
  CHECK_CUDA(y);
  CHECK_CONTIGUOUS(y);
  CHECK_INPUT(y.dim() == 2);
  CHECK_INPUT(x.size(1) == y.size(1));
  CHECK_INPUT(x.get_device() == y.get_device());
  CHECK_INPUT(x.scalar_type() == y.scalar_type());

  Prepared p;
  p.x = x;
  p.y = y;
  p.dtype = dtype_code(x);

  if (ptr_x.has_value() || ptr_y.has_value()) {
    // a missing side defaults to one segment over all rows (csrc/cuda/knn_cuda.cu:100-112)
    const auto opts = x.options().dtype(torch::kLong);
    p.ptr_x = ptr_x.has_value() ? ptr_x.value() : torch::arange(0, x.size(0) + 1, x.size(0) > 0 ? x.size(0) : 1, opts);
    p.ptr_y = ptr_y.has_value() ? ptr_y.value() : torch::arange(0, y.size(0) + 1, y.size(0) > 0 ? y.size(0) : 1, opts);
    CHECK_CUDA(p.ptr_x);
    CHECK_INPUT(p.ptr_x.dim() == 1);
    CHECK_CUDA(p.ptr_y);
    CHECK_INPUT(p.ptr_y.dim() == 1);
    CHECK_INPUT(p.ptr_x.numel() == p.ptr_y.numel());
    CHECK_INPUT(p.ptr_x.numel() >= 2);
    TORCH_CHECK(p.ptr_x.scalar_type() == at::kLong && p.ptr_y.scalar_type() == at::kLong,
                "ptr_x and ptr_y must be int64 tensors");
    p.ptr_x = p.ptr_x.contiguous();
    p.ptr_y = p.ptr_y.contiguous();
    p.px = p.ptr_x.data_ptr<int64_t>();
    p.py = p.ptr_y.data_ptr<int64_t>();
    p.num_segments = p.ptr_x.numel() - 1;
  }
  return p;
}

}  // namespace

namespace {

// A bounded wait of the Morton-ordered scan ran out (see b200_cluster.h): never expected, never silent.
constexpr int64_t kKnnWaitError = (int64_t)1 << 62;
constexpr int32_t kGraphWaitError = 1 << 30;

// knn with a hint: max_segment_rows bounds the row count of every segment (0 = unknown); it saves
// empty sorting passes on inputs of many small segments.
torch::Tensor knn_hinted(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> ptr_x,
                         std::optional<torch::Tensor> ptr_y, int64_t k, bool cosine, int64_t max_segment_rows) {
  OpRange range("torch_cluster::knn");
  Prepared p = prepare(x, y, ptr_x, ptr_y);
  TORCH_CHECK(k <= B200C_MAX_K, "`k` needs to smaller than or equal to 100");
  TORCH_CHECK(k >= 1, "`k` needs to be positive");

  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const auto lopts = x.options().dtype(torch::kLong);
  const int64_t n = p.x.size(0), m = p.y.size(0), dim = p.x.size(1);
  if (m == 0) return torch::empty({2, 0}, lopts);

  auto padded = torch::empty({2, m * k}, lopts);
  auto counts = torch::empty({m}, x.options().dtype(torch::kInt));
  auto num_valid = torch::empty({1}, lopts);
  const size_t ws_bytes = b200c_knn_workspace_bytes(n, m, dim, k, p.dtype, cosine, p.num_segments);
  auto ws = torch::empty({(int64_t)ws_bytes}, x.options().dtype(torch::kByte));

  check_status(b200c_knn(p.x.data_ptr(), p.y.data_ptr(), p.px, p.py, p.num_segments, n, m, dim, k, p.dtype,
                         cosine ? 1 : 0, padded.data_ptr<int64_t>(), counts.data_ptr<int32_t>(),
                         num_valid.data_ptr<int64_t>(), max_segment_rows, ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                         stream.stream()));
  const int64_t total = num_valid.item<int64_t>();  // the one host sync: the output size
  TORCH_CHECK(total < kKnnWaitError, "b200_cluster: the kNN scan was abandoned (a bounded wait ran out, or segment pointers that overlap)");
  if (total == m * k) return padded;

  // some query had fewer than k admissible points: drop the -1 slots
  auto offsets = torch::empty({m + 1}, lopts);
  const size_t scan_bytes = b200c_scan_workspace_bytes(m);
  auto scan_ws = torch::empty({(int64_t)scan_bytes}, x.options().dtype(torch::kByte));
  check_status(b200c_exclusive_scan(counts.data_ptr<int32_t>(), m, offsets.data_ptr<int64_t>(),
                                    scan_ws.data_ptr(), scan_bytes, stream.stream()));
  auto out = torch::empty({2, total}, lopts);
  check_status(b200c_knn_compact(padded.data_ptr<int64_t>(), counts.data_ptr<int32_t>(),
                                 offsets.data_ptr<int64_t>(), m, k, total, out.data_ptr<int64_t>(),
                                 stream.stream()));
  return out;
}

}  // namespace

torch::Tensor knn(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> ptr_x,
                  std::optional<torch::Tensor> ptr_y, int64_t k, bool cosine, int64_t num_workers) {
  (void)num_workers;  // no effect on the GPU, as in the reference
  return knn_hinted(x, y, ptr_x, ptr_y, k, cosine, 0);
}

namespace {

// knn_graph in one operator: kNN of x in x, then self-match removal, padding removal and flow
// orientation on the device (torch_cluster/knn.py:131-144), with a single host sync for the size.
torch::Tensor knn_graph_edges(torch::Tensor x, std::optional<torch::Tensor> ptr, int64_t k, bool loop,
                              bool source_to_target, bool cosine, int64_t max_segment_rows) {
  OpRange range("torch_cluster::knn_graph_edges");
  const int64_t k1 = loop ? k : k + 1;
  Prepared p = prepare(x, x, ptr, ptr);
  TORCH_CHECK(k1 <= B200C_MAX_K, "`k` needs to smaller than or equal to 100");
  TORCH_CHECK(k >= 1, "`k` needs to be positive");

  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const auto lopts = x.options().dtype(torch::kLong);
  const auto iopts = x.options().dtype(torch::kInt);
  const int64_t n = p.x.size(0), dim = p.x.size(1);
  if (n == 0) return torch::empty({2, 0}, lopts);

  size_t gws_bytes = 0;
  if (!loop && cosine && p.dtype == B200C_F32)
    gws_bytes = b200c_knn_graph_cosine_workspace_bytes(n, dim, k, p.num_segments);
  else if (!loop && !cosine)
    gws_bytes = b200c_knn_graph_workspace_bytes(n, dim, k, p.dtype, p.num_segments);
  const bool aligned = (reinterpret_cast<uintptr_t>(p.x.data_ptr()) & 15) == 0;  // the tensor-core path's operand copies
  const bool features = dim > 8 && gws_bytes > 0 && aligned;
  if (!loop && (p.dtype == B200C_F32 || p.dtype == B200C_F64) && ((!cosine && dim <= 8) || features)) {
    // the usual shape (every row finds itself and k others) comes out of one kernel (low-dimensional points)
    // or of the re-rank of the tensor-core candidates (feature vectors); anything else is detected there and
    // takes the general route below
    auto out = torch::empty({2, n * k}, lopts);
    auto irregular = torch::empty({1}, iopts);
    auto gws = torch::empty({(int64_t)gws_bytes}, x.options().dtype(torch::kByte));
    if (cosine)
      check_status(b200c_knn_graph_cosine(p.x.data_ptr(), p.px, p.num_segments, n, dim, k, source_to_target ? 1 : 0,
                                          out.data_ptr<int64_t>(), irregular.data_ptr<int32_t>(), gws.data_ptr(),
                                          gws_bytes, stream.stream()));
    else
      check_status(b200c_knn_graph(p.x.data_ptr(), p.px, p.num_segments, n, dim, k, p.dtype, source_to_target ? 1 : 0,
                                   out.data_ptr<int64_t>(), irregular.data_ptr<int32_t>(), max_segment_rows,
                                   gws_bytes ? gws.data_ptr() : nullptr, gws_bytes, stream.stream()));
    const int32_t odd = irregular.item<int32_t>();  // the one host sync
    TORCH_CHECK(odd < kGraphWaitError, "b200_cluster: the kNN scan was abandoned (a bounded wait ran out, or segment pointers that overlap)");
    if (odd == 0) return out;
  }

  auto padded = torch::empty({2, n * k1}, lopts);
  auto counts = torch::empty({n}, iopts);
  auto num_valid = torch::empty({1}, lopts);
  const size_t ws_bytes = b200c_knn_workspace_bytes(n, n, dim, k1, p.dtype, cosine, p.num_segments);
  auto ws = torch::empty({(int64_t)ws_bytes}, x.options().dtype(torch::kByte));
  check_status(b200c_knn(p.x.data_ptr(), p.x.data_ptr(), p.px, p.px, p.num_segments, n, n, dim, k1, p.dtype,
                         cosine ? 1 : 0, padded.data_ptr<int64_t>(), counts.data_ptr<int32_t>(),
                         num_valid.data_ptr<int64_t>(), max_segment_rows, ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                         stream.stream()));
  auto kept = torch::empty({n}, iopts);
  check_status(b200c_knn_graph_tail_count(padded.data_ptr<int64_t>(), counts.data_ptr<int32_t>(), n, k1,
                                          loop ? 0 : 1, kept.data_ptr<int32_t>(), stream.stream()));
  auto offsets = torch::empty({n + 1}, lopts);
  const size_t scan_bytes = b200c_scan_workspace_bytes(n);
  auto scan_ws = torch::empty({(int64_t)scan_bytes}, x.options().dtype(torch::kByte));
  check_status(b200c_exclusive_scan(kept.data_ptr<int32_t>(), n, offsets.data_ptr<int64_t>(), scan_ws.data_ptr(),
                                    scan_bytes, stream.stream()));
  // the output size and the search's own count travel together: one host sync
  auto sizes = torch::stack({offsets[n], num_valid[0]}).cpu();
  const int64_t total = sizes[0].item<int64_t>();
  TORCH_CHECK(sizes[1].item<int64_t>() < kKnnWaitError, "b200_cluster: the kNN scan was abandoned (a bounded wait ran out, or segment pointers that overlap)");
  auto out = torch::empty({2, total}, lopts);
  check_status(b200c_knn_graph_tail_write(padded.data_ptr<int64_t>(), counts.data_ptr<int32_t>(),
                                          offsets.data_ptr<int64_t>(), n, k1, loop ? 0 : 1,
                                          source_to_target ? 1 : 0, total, out.data_ptr<int64_t>(),
                                          stream.stream()));
  return out;
}

// The radius search behind `radius` and `radius_graph`.  query_index_base: row number of y's first row
// in x's numbering, for `ignore_same_index` on a slice of the queries (multi-GPU); swap_rows: write
// row 0 = x index, row 1 = query, the `source_to_target` orientation of radius_graph
// (torch_cluster/radius.py:143-148), instead of stacking the rows again afterwards.
torch::Tensor radius_part(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> ptr_x,
                          std::optional<torch::Tensor> ptr_y, double r, int64_t max_num_neighbors,
                          bool ignore_same_index, int64_t query_index_base, bool swap_rows) {
  OpRange range("torch_cluster::radius");
  Prepared p = prepare(x, y, ptr_x, ptr_y);
  TORCH_CHECK(query_index_base >= 0, "Input mismatch");

  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const auto lopts = x.options().dtype(torch::kLong);
  const int64_t n = p.x.size(0), m = p.y.size(0), dim = p.x.size(1);
  if (m == 0 || max_num_neighbors <= 0) return torch::empty({2, 0}, lopts);

  auto counts = torch::empty({m}, x.options().dtype(torch::kInt));
  auto offsets = torch::empty({m + 1}, lopts);
  const size_t scan_bytes = b200c_scan_workspace_bytes(m);
  auto scan_ws = torch::empty({(int64_t)scan_bytes}, x.options().dtype(torch::kByte));
  const int same = ignore_same_index ? 1 : 0, swap = swap_rows ? 1 : 0;

  // Large neighbour caps on low-dimensional points: every pair is evaluated once, its hit bit kept in
  // a bit matrix from which the edges are written afterwards.  The matrix's size depends on the segment
  // sizes, so the segment pointers are read to the host (a second small sync of this call).  Pointers
  // that do not describe x and y exactly make the size query answer 0 and take the route below.
  // The screened scan pays when hits are sparse.  A query keeps at most max_num_neighbors of them, so with
  // segments of 2048 * max_num_neighbors points on average at most one (query, chunk of 256 points) pair in
  // eight can hold one: known from the sizes alone.
  const bool sparse_for_sure = max_num_neighbors <= (1 << 20) && n / p.num_segments >= 2048 * max_num_neighbors;
  const size_t screen_bytes =
      sparse_for_sure ? b200c_radius_screen_workspace_bytes(n, m, dim, max_num_neighbors, p.dtype, p.num_segments) : 0;
  if (screen_bytes == 0 && max_num_neighbors > kRadiusDirectCap && dim <= 8 &&
      (p.dtype == B200C_F32 || p.dtype == B200C_F64)) {
    torch::Tensor hx, hy;
    const int64_t *hpx = nullptr, *hpy = nullptr;
    if (p.px != nullptr) {
      hx = p.ptr_x.cpu();
      hy = p.ptr_y.cpu();
      hpx = hx.data_ptr<int64_t>();
      hpy = hy.data_ptr<int64_t>();
    }
    const size_t mask_bytes = b200c_radius_mask_workspace_bytes(hpx, hpy, p.num_segments, n, m, dim, p.dtype);
    if (mask_bytes > 0 && mask_bytes <= kRadiusMaskMaxBytes) {
      auto mask_ws = torch::empty({(int64_t)mask_bytes}, x.options().dtype(torch::kByte));
      check_status(b200c_radius_count_masks_part(p.x.data_ptr(), p.y.data_ptr(), p.px, p.py, hpx, hpy, p.num_segments,
                                                 n, m, dim, r, max_num_neighbors, same, query_index_base, p.dtype,
                                                 counts.data_ptr<int32_t>(), mask_ws.data_ptr(), mask_bytes,
                                                 stream.stream()));
      check_status(b200c_exclusive_scan(counts.data_ptr<int32_t>(), m, offsets.data_ptr<int64_t>(), scan_ws.data_ptr(),
                                        scan_bytes, stream.stream()));
      const int64_t total = offsets[m].item<int64_t>();  // the output size
      auto out = torch::empty({2, total}, lopts);
      check_status(b200c_radius_fill_masks_part(p.px, p.py, p.num_segments, n, m, dim, swap, p.dtype,
                                                counts.data_ptr<int32_t>(), offsets.data_ptr<int64_t>(), total,
                                                out.data_ptr<int64_t>(), mask_ws.data_ptr(), stream.stream()));
      return out;
    }
  }

  // small neighbour caps: one scan that also parks the hits, then a copy (see b200_cluster.h)
  const size_t ws_bytes = std::max(screen_bytes, b200c_radius_workspace_bytes(n, m, dim, max_num_neighbors, p.dtype));
  auto ws = torch::empty({(int64_t)ws_bytes}, x.options().dtype(torch::kByte));
  void *ws_ptr = ws_bytes ? ws.data_ptr() : nullptr;
  check_status(b200c_radius_count_part(p.x.data_ptr(), p.y.data_ptr(), p.px, p.py, p.num_segments, n, m, dim, r,
                                       max_num_neighbors, same, query_index_base, p.dtype,
                                       counts.data_ptr<int32_t>(), ws_ptr, ws_bytes, stream.stream()));
  check_status(b200c_exclusive_scan(counts.data_ptr<int32_t>(), m, offsets.data_ptr<int64_t>(),
                                    scan_ws.data_ptr(), scan_bytes, stream.stream()));
  int64_t total;
  if (screen_bytes > 0) {
    // the output size and the scan's status word (first 8 bytes of its workspace) travel together
    auto sizes = torch::stack({offsets[m], ws.narrow(0, 0, 8).view(torch::kLong)[0]}).cpu();
    TORCH_CHECK(sizes[1].item<int64_t>() == 0, "b200_cluster: the radius scan was abandoned (a bounded wait ran out, or segment pointers that overlap)");
    total = sizes[0].item<int64_t>();
  } else {
    total = offsets[m].item<int64_t>();  // the one host sync: the output size
  }
  auto out = torch::empty({2, total}, lopts);
  check_status(b200c_radius_fill_part(p.x.data_ptr(), p.y.data_ptr(), p.px, p.py, p.num_segments, n, m, dim, r,
                                      max_num_neighbors, same, query_index_base, swap, p.dtype,
                                      counts.data_ptr<int32_t>(), offsets.data_ptr<int64_t>(), total,
                                      out.data_ptr<int64_t>(), ws_ptr, ws_bytes, stream.stream()));
  return out;
}

}  // namespace

torch::Tensor radius(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> ptr_x,
                     std::optional<torch::Tensor> ptr_y, double r, int64_t max_num_neighbors,
                     int64_t num_workers, bool ignore_same_index) {
  (void)num_workers;  // no effect on the GPU, as in the reference
  return radius_part(x, y, ptr_x, ptr_y, r, max_num_neighbors, ignore_same_index, 0, false);
}

namespace {

// [number of segments, rows of the largest segment] of a sorted batch vector (one host sync): what the
// Python wrappers need to size the segment pointers (torch_cluster/knn.py:62-69 reads batch.max()),
// plus the hint that saves empty sorting passes.
std::vector<int64_t> batch_info(torch::Tensor batch) {
  CHECK_CUDA(batch);
  CHECK_INPUT(batch.dim() == 1);
  TORCH_CHECK(batch.scalar_type() == at::kLong, "batch must be an int64 tensor");
  if (batch.numel() == 0) return {0, 0};
  batch = batch.contiguous();
  c10::cuda::CUDAGuard guard(batch.device());
  auto info = torch::empty({2}, batch.options());
  check_status(b200c_batch_info(batch.data_ptr<int64_t>(), batch.numel(), info.data_ptr<int64_t>(),
                                at::cuda::getCurrentCUDAStream().stream()));
  auto host = info.cpu();
  return {host[0].item<int64_t>(), host[1].item<int64_t>()};
}

// [last id + 1, rows of the longest run of equal ids, 1 if some entry is smaller than the one before it]
// (one kernel, one host sync): for callers that must not assume a sorted vector (torch_cluster/fps.py:95-104
// counts members instead of bisecting) but want the cheap route when it is.
std::vector<int64_t> batch_check(torch::Tensor batch) {
  CHECK_CUDA(batch);
  CHECK_INPUT(batch.dim() == 1);
  TORCH_CHECK(batch.scalar_type() == at::kLong, "batch must be an int64 tensor");
  if (batch.numel() == 0) return {0, 0, 0};
  batch = batch.contiguous();
  c10::cuda::CUDAGuard guard(batch.device());
  auto info = torch::empty({3}, batch.options());
  check_status(b200c_batch_check(batch.data_ptr<int64_t>(), batch.numel(), info.data_ptr<int64_t>(),
                                 at::cuda::getCurrentCUDAStream().stream()));
  auto host = info.cpu();
  return {host[0].item<int64_t>(), host[1].item<int64_t>(), host[2].item<int64_t>()};
}

// Device-side construction of the segment pointers from a sorted batch vector
// (what torch_cluster/knn.py:77-79 does with torch.bucketize).
torch::Tensor segment_ptr(torch::Tensor batch, int64_t num_segments) {
  CHECK_CUDA(batch);
  CHECK_INPUT(batch.dim() == 1);
  TORCH_CHECK(batch.scalar_type() == at::kLong, "batch must be an int64 tensor");
  CHECK_INPUT(num_segments >= 0);
  batch = batch.contiguous();
  c10::cuda::CUDAGuard guard(batch.device());
  auto ptr = torch::empty({num_segments + 1}, batch.options());
  check_status(b200c_segment_ptr(batch.data_ptr<int64_t>(), batch.numel(), num_segments,
                                 ptr.data_ptr<int64_t>(), at::cuda::getCurrentCUDAStream().stream()));
  return ptr;
}

}  // namespace

// nearest: torch_cluster::nearest of csrc/nearest.cpp:22-36; host side of csrc/cuda/nearest_cuda.cu:63-88.
torch::Tensor nearest(torch::Tensor x, torch::Tensor y, torch::Tensor ptr_x, torch::Tensor ptr_y) {
  OpRange range("torch_cluster::nearest");
  CHECK_CUDA(x);
  CHECK_CUDA(y);
  CHECK_CUDA(ptr_x);
  CHECK_CUDA(ptr_y);
  c10::cuda::CUDAGuard guard(x.device());
  x = x.view({x.size(0), -1}).contiguous();
  y = y.view({y.size(0), -1}).contiguous();
  CHECK_INPUT(x.size(1) == y.size(1));
  CHECK_INPUT(x.scalar_type() == y.scalar_type());
  CHECK_INPUT(ptr_x.dim() == 1 && ptr_y.dim() == 1 && ptr_x.numel() == ptr_y.numel() && ptr_x.numel() >= 2);
  TORCH_CHECK(ptr_x.scalar_type() == at::kLong && ptr_y.scalar_type() == at::kLong,
              "ptr_x and ptr_y must be int64 tensors");
  ptr_x = ptr_x.contiguous();
  ptr_y = ptr_y.contiguous();
  const int dtype = dtype_code(x);
  const int64_t n = x.size(0), m = y.size(0), dim = x.size(1);
  auto out = torch::empty({n}, ptr_x.options());
  if (n == 0) return out;
  const size_t ws_bytes = b200c_nearest_workspace_bytes(n, m, dim, dtype);
  auto ws = torch::empty({(int64_t)ws_bytes}, x.options().dtype(torch::kByte));
  check_status(b200c_nearest(x.data_ptr(), y.data_ptr(), ptr_x.data_ptr<int64_t>(), ptr_y.data_ptr<int64_t>(),
                             ptr_x.numel() - 1, n, m, dim, dtype, out.data_ptr<int64_t>(),
                             ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                             at::cuda::getCurrentCUDAStream().stream()));
  return out;
}

namespace {

// `nearest` of torch_cluster/nearest.py:44-87 with its checks in one operator: both batch vectors sorted
// (ValueError otherwise), equally many examples on both sides, and every example that has rows in x has rows
// in y.  One host read before the search (segments and sortedness of both vectors, one kernel each) and one
// after it (the emptiness comparison, which the search does not depend on: rows of an example without a row
// in y are assigned 0).
torch::Tensor nearest_batched(torch::Tensor x, torch::Tensor y, std::optional<torch::Tensor> batch_x,
                              std::optional<torch::Tensor> batch_y) {
  CHECK_CUDA(x);
  CHECK_CUDA(y);
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  const auto lopts = x.options().dtype(torch::kLong);
  const int64_t n = x.size(0), m = y.size(0);
  auto info = torch::zeros({6}, lopts);
  torch::Tensor bx, by;
  if (batch_x.has_value()) {
    bx = batch_x.value().contiguous();
    CHECK_CUDA(bx);
    TORCH_CHECK(bx.scalar_type() == at::kLong && bx.dim() == 1, "batch_x must be a 1-D int64 tensor");
    TORCH_CHECK(bx.numel() == n || bx.numel() == 0, "x.size(0) == batch_x.numel()");
    check_status(b200c_batch_check(bx.data_ptr<int64_t>(), bx.numel(), info.data_ptr<int64_t>(), stream.stream()));
  }
  if (batch_y.has_value()) {
    by = batch_y.value().contiguous();
    CHECK_CUDA(by);
    TORCH_CHECK(by.scalar_type() == at::kLong && by.dim() == 1, "batch_y must be a 1-D int64 tensor");
    TORCH_CHECK(by.numel() == m || by.numel() == 0, "y.size(0) == batch_y.numel()");
    check_status(b200c_batch_check(by.data_ptr<int64_t>(), by.numel(), info.data_ptr<int64_t>() + 3, stream.stream()));
  }
  const auto seen = info.cpu();
  const int64_t *h = seen.data_ptr<int64_t>();
  TORCH_CHECK_VALUE(h[2] == 0, "'batch_x' is not sorted");
  TORCH_CHECK_VALUE(h[5] == 0, "'batch_y' is not sorted");
  auto whole = [&](int64_t rows) {
    auto ptr = torch::zeros({2}, lopts);
    ptr[1].fill_(rows);
    return ptr;
  };
  const int64_t segs_x = batch_x.has_value() ? std::max<int64_t>(h[0], 1) : 1;
  const int64_t segs_y = batch_y.has_value() ? std::max<int64_t>(h[3], 1) : 1;
  auto ptr_x = batch_x.has_value() ? segment_ptr(bx, segs_x) : whole(n);
  auto ptr_y = batch_y.has_value() ? segment_ptr(by, segs_y) : whole(m);
  TORCH_CHECK_VALUE(segs_x == segs_y, "Some batch indices occur in 'batch_x' that do not occur in 'batch_y'");
  auto flag = torch::empty({1}, x.options().dtype(torch::kInt));
  check_status(b200c_segment_mismatch(ptr_x.data_ptr<int64_t>(), ptr_y.data_ptr<int64_t>(), segs_x,
                                      flag.data_ptr<int32_t>(), stream.stream()));
  auto out = nearest(x, y, ptr_x, ptr_y);
  TORCH_CHECK_VALUE(flag.item<int32_t>() == 0, "Some batch indices occur in 'batch_x' that do not occur in 'batch_y'");
  return out;
}

}  // namespace

// Which segments of an fps call go where: `large` (more than per_cta points, at most multi_cap, at least
// one sample) are sampled by many SMs together, `oversize` (more than multi_cap) by one thread block from
// global memory in a call of their own; every other segment runs in the common call.
static void fps_classify_segments(const int64_t *ptr, const int64_t *out_ptr, int64_t segments, int64_t per_cta,
                                  int64_t multi_cap, std::vector<int64_t> *large, std::vector<int64_t> *oversize) {
  for (int64_t b = 0; b < segments; ++b) {
    const int64_t pts = ptr[b + 1] - ptr[b];
    if (out_ptr[b + 1] <= out_ptr[b]) continue;
    if (pts > per_cta && pts <= multi_cap) large->push_back(b);
    else if (pts > multi_cap) oversize->push_back(b);
  }
}

// The classification above on host tensors: -> int64 [segments], 0 = common call, 1 = large, 2 = oversize.
torch::Tensor fps_segment_classes(torch::Tensor ptr, torch::Tensor out_ptr, int64_t per_cta, int64_t multi_cap) {
  TORCH_CHECK(!ptr.is_cuda() && !out_ptr.is_cuda() && ptr.scalar_type() == at::kLong &&
                  out_ptr.scalar_type() == at::kLong && ptr.numel() == out_ptr.numel() && ptr.numel() >= 1,
              "fps_segment_classes expects two host int64 vectors of equal length");
  ptr = ptr.contiguous();
  out_ptr = out_ptr.contiguous();
  const int64_t segments = ptr.numel() - 1;
  std::vector<int64_t> large, oversize;
  fps_classify_segments(ptr.data_ptr<int64_t>(), out_ptr.data_ptr<int64_t>(), segments, per_cta, multi_cap, &large,
                        &oversize);
  auto cls = torch::zeros({segments}, torch::kLong);
  for (int64_t b : large) cls[b] = 1;
  for (int64_t b : oversize) cls[b] = 2;
  return cls;
}

// fps: torch_cluster::fps of csrc/fps.cpp:22-36; host side of csrc/cuda/fps_cuda.cu:70-112.  The
// per-segment sample counts are formed exactly as there (degree in ratio's dtype, times ratio,
// ceil, cumulative sum); one host read gives the output size.
torch::Tensor fps(torch::Tensor src, torch::Tensor ptr, torch::Tensor ratio, bool random_start) {
  OpRange range("torch_cluster::fps");
  CHECK_CUDA(src);
  CHECK_CUDA(ptr);
  CHECK_CUDA(ratio);
  CHECK_INPUT(ptr.dim() == 1);
  TORCH_CHECK(ptr.scalar_type() == at::kLong, "ptr must be an int64 tensor");
  c10::cuda::CUDAGuard guard(src.device());
  src = src.view({src.size(0), -1}).contiguous();
  ptr = ptr.contiguous();
  const int64_t batch_size = ptr.numel() - 1;
  const int dtype = dtype_code(src);

  auto deg = ptr.narrow(0, 1, batch_size) - ptr.narrow(0, 0, batch_size);
  auto out_ptr = deg.toType(ratio.scalar_type()) * ratio;
  out_ptr = out_ptr.ceil().toType(torch::kLong).cumsum(0);
  out_ptr = torch::cat({torch::zeros({1}, ptr.options()), out_ptr}, 0).contiguous();

  torch::Tensor start;
  const int64_t *start_ptr = nullptr;
  if (random_start) {
    start = torch::rand(batch_size, src.options());
    start = (start * deg.toType(ratio.scalar_type())).toType(torch::kLong).contiguous();
    start_ptr = start.data_ptr<int64_t>();
  }
  const int64_t total = batch_size > 0 ? out_ptr[-1].item<int64_t>() : 0;  // the one host sync
  auto out = torch::empty({total}, ptr.options());
  if (total == 0) return out;
  const int64_t n = src.size(0), dim = src.size(1);
  const size_t ws_bytes = b200c_fps_workspace_bytes(n, dim, dtype);
  auto ws = torch::empty({(int64_t)ws_bytes}, src.options().dtype(torch::kByte));
  auto stream = at::cuda::getCurrentCUDAStream();

  // Segments too large for one SM's registers are sampled by many SMs together, one launch each; whether
  // there are any is only known from the segment sizes, which are read to the host when the input is large
  // enough to hold one.
  const int64_t per_cta = dim <= 3 ? 8192 : 4096;
  const int64_t multi_cap = b200c_fps_large_segment_max_points(dim, dtype);
  if (multi_cap > 0 && n > per_cta) {
    auto hptr = ptr.cpu();
    auto hout = out_ptr.cpu();
    torch::Tensor hstart;
    if (random_start) hstart = start.cpu();
    const int64_t *hp = hptr.data_ptr<int64_t>(), *ho = hout.data_ptr<int64_t>();
    // large: sampled by many SMs together; oversize: beyond what those hold, one thread block each from
    // global memory like every small segment, but in a call of their own (b200c_fps_up_to skips them)
    std::vector<int64_t> large, oversize;
    fps_classify_segments(hp, ho, batch_size, per_cta, multi_cap, &large, &oversize);
    if (!large.empty()) {
      check_status(b200c_fps_up_to(src.data_ptr(), ptr.data_ptr<int64_t>(), out_ptr.data_ptr<int64_t>(), start_ptr,
                                   batch_size, n, dim, dtype, per_cta, out.data_ptr<int64_t>(), ws.data_ptr(), ws_bytes,
                                   stream.stream()));
      const size_t big_bytes = b200c_fps_large_segment_workspace_bytes();
      auto big_ws = torch::empty({(int64_t)big_bytes}, src.options().dtype(torch::kByte));
      auto status = torch::zeros({1}, src.options().dtype(torch::kInt));
      for (int64_t b : large) {
        const int st = b200c_fps_large_segment(src.data_ptr(), hp[b], hp[b + 1] - hp[b],
                                               random_start ? hstart.data_ptr<int64_t>()[b] : 0, ho[b + 1] - ho[b], dim,
                                               dtype, out.data_ptr<int64_t>() + ho[b], big_ws.data_ptr(), big_bytes,
                                               status.data_ptr<int32_t>(), stream.stream());
        if (st == B200C_ERR_UNSUPPORTED)
          oversize.push_back(b);  // e.g. a context with too few SMs for a cooperative launch: one block does it
        else
          check_status(st);
      }
      // a one-segment call per remaining segment: the pointer arrays are entered at b
      for (int64_t b : oversize)
        check_status(b200c_fps(src.data_ptr(), ptr.data_ptr<int64_t>() + b, out_ptr.data_ptr<int64_t>() + b,
                               start_ptr ? start_ptr + b : nullptr, 1, n, dim, dtype, out.data_ptr<int64_t>(),
                               ws.data_ptr(), ws_bytes, stream.stream()));
      TORCH_CHECK(status.item<int32_t>() == 0, "b200_cluster: a wait between the thread blocks of fps ran out");
      return out;
    }
  }
  check_status(b200c_fps(src.data_ptr(), ptr.data_ptr<int64_t>(), out_ptr.data_ptr<int64_t>(), start_ptr,
                         batch_size, n, dim, dtype, out.data_ptr<int64_t>(), ws.data_ptr(), ws_bytes,
                         stream.stream()));
  return out;
}

// fps with the segment boundaries as a host list: no device-to-host read of the boundaries is
// needed to find the segments that want the many-SM kernel.
torch::Tensor fps_ptr_list(torch::Tensor src, std::vector<int64_t> ptr, torch::Tensor ratio, bool random_start) {
  CHECK_CUDA(src);
  auto ptr_dev = torch::tensor(ptr, torch::TensorOptions().dtype(torch::kLong)).to(src.device());
  return fps(src, ptr_dev, ratio, random_start);
}

namespace {

// knn_graph from host memory to host memory for low-dimensional points (loop = False): the call is cut
// into groups of whole segments, one stream each, so that uploads and downloads of the other groups
// overlap the search of a group and the block scheduler keeps the SMs filled across the groups'
// kernels.  x: CPU [n, dim] (pinned for overlap); ptr: CPU int64 [B + 1]; out: CPU int64 [2, n * k]
// (pinned).  Returns the number of irregular queries (see b200c_knn_graph): 0 means `out` is final.
int64_t knn_graph_host(torch::Tensor x, torch::Tensor ptr, int64_t k, bool source_to_target, torch::Tensor out,
                       int64_t num_groups, int64_t device_index) {
  OpRange range("torch_cluster::knn_graph_host");
  TORCH_CHECK(!x.is_cuda() && !ptr.is_cuda() && !out.is_cuda(), "knn_graph_host expects host tensors");
  CHECK_CONTIGUOUS(x);
  CHECK_INPUT(x.dim() == 2 && ptr.dim() == 1 && ptr.numel() >= 2);
  TORCH_CHECK(ptr.scalar_type() == at::kLong && out.scalar_type() == at::kLong, "ptr and out must be int64 tensors");
  const int64_t n = x.size(0), dim = x.size(1), segs = ptr.numel() - 1, total = n * k;
  TORCH_CHECK(out.is_contiguous() && out.dim() == 2 && out.size(0) == 2 && out.size(1) == total,
              "out must be a contiguous [2, n * k] tensor");
  const int dtype = dtype_code(x);
  TORCH_CHECK(dtype == B200C_F32 || dtype == B200C_F64, "knn_graph_host covers float and double points");
  if (n == 0) return 0;
  const int64_t *p = ptr.data_ptr<int64_t>();
  TORCH_CHECK(p[0] == 0 && p[segs] == n, "Input mismatch");

  // groups of consecutive segments with about equal numbers of (query, point) pairs
  num_groups = std::max<int64_t>(1, std::min<int64_t>(num_groups, segs));
  double all = 0;
  for (int64_t b = 0; b < segs; ++b) all += (double)(p[b + 1] - p[b]) * (double)(p[b + 1] - p[b]);
  std::vector<int64_t> cut{0};
  double acc = 0;
  for (int64_t b = 0; b < segs; ++b) {
    acc += (double)(p[b + 1] - p[b]) * (double)(p[b + 1] - p[b]);
    if ((int64_t)cut.size() < num_groups && acc >= all * (double)cut.size() / (double)num_groups && b + 1 < segs)
      cut.push_back(b + 1);
  }
  cut.push_back(segs);
  const int64_t groups = (int64_t)cut.size() - 1;

  c10::cuda::CUDAGuard guard((c10::DeviceIndex)device_index);
  const auto dopts = torch::TensorOptions().device(torch::kCUDA, (c10::DeviceIndex)device_index);
  const size_t elem = dtype == B200C_F64 ? 8 : 4;
  auto x_dev = torch::empty({n, dim}, dopts.dtype(x.scalar_type()));
  auto edges_dev = torch::empty({2, total}, dopts.dtype(torch::kLong));
  auto flags_dev = torch::empty({groups}, dopts.dtype(torch::kInt));
  // every group's search may build a Morton-ordered copy of its points: one workspace per group
  std::vector<size_t> ws_off(groups + 1, 0);
  for (int64_t g = 0; g < groups; ++g) {
    const size_t need = b200c_knn_graph_workspace_bytes(p[cut[g + 1]] - p[cut[g]], dim, k, dtype, cut[g + 1] - cut[g]);
    ws_off[g + 1] = ws_off[g] + (need + 255) / 256 * 256;
  }
  auto ws_dev = torch::empty({(int64_t)ws_off[groups]}, dopts.dtype(torch::kByte));
  int64_t max_rows = 0;
  for (int64_t b = 0; b < segs; ++b) max_rows = std::max(max_rows, p[b + 1] - p[b]);
  auto ptr_dev = torch::empty({segs + groups}, dopts.dtype(torch::kLong));
  // every group's own pointers (starting at 0), back to back, and the flags coming back: pinned
  auto small = torch::empty({segs + groups + groups}, torch::TensorOptions().dtype(torch::kLong).pinned_memory(true));
  int64_t *local = small.data_ptr<int64_t>();
  int32_t *flags_host = reinterpret_cast<int32_t *>(local + segs + groups);
  int64_t off = 0;
  for (int64_t g = 0; g < groups; ++g)
    for (int64_t b = cut[g]; b <= cut[g + 1]; ++b) local[off++] = p[b] - p[cut[g]];

  auto current = at::cuda::getCurrentCUDAStream();
  C10_CUDA_CHECK(cudaMemcpyAsync(ptr_dev.data_ptr(), local, (size_t)off * 8, cudaMemcpyHostToDevice, current.stream()));
  at::cuda::CUDAEvent ready;
  ready.record(current);  // the buffers above, and the pointers, belong to the current stream
  std::vector<at::cuda::CUDAStream> streams;
  const char *xh = (const char *)x.data_ptr();
  char *xd = (char *)x_dev.data_ptr();
  int64_t *ed = edges_dev.data_ptr<int64_t>(), *oh = out.data_ptr<int64_t>();
  off = 0;
  try {
  for (int64_t g = 0; g < groups; ++g) {
    streams.push_back(at::cuda::getStreamFromPool(false, (c10::DeviceIndex)device_index));
    cudaStream_t st = streams.back().stream();
    ready.block(streams.back());
    const int64_t r0 = p[cut[g]], r1 = p[cut[g + 1]], nseg = cut[g + 1] - cut[g];
    C10_CUDA_CHECK(cudaMemcpyAsync(xd + r0 * dim * elem, xh + r0 * dim * elem, (size_t)(r1 - r0) * dim * elem,
                                   cudaMemcpyHostToDevice, st));
    check_status(b200c_knn_graph_part(xd + r0 * dim * elem, ptr_dev.data_ptr<int64_t>() + off, nseg, r1 - r0, dim, k,
                                      dtype, source_to_target ? 1 : 0, r0, ed + r0 * k, total,
                                      flags_dev.data_ptr<int32_t>() + g, max_rows,
                                      ws_off[g + 1] > ws_off[g] ? (char *)ws_dev.data_ptr() + ws_off[g] : nullptr,
                                      ws_off[g + 1] - ws_off[g], st));
    C10_CUDA_CHECK(cudaMemcpyAsync(oh + r0 * k, ed + r0 * k, (size_t)(r1 - r0) * k * 8, cudaMemcpyDeviceToHost, st));
    C10_CUDA_CHECK(cudaMemcpyAsync(oh + total + r0 * k, ed + total + r0 * k, (size_t)(r1 - r0) * k * 8,
                                   cudaMemcpyDeviceToHost, st));
    C10_CUDA_CHECK(cudaMemcpyAsync(flags_host + g, flags_dev.data_ptr<int32_t>() + g, 4, cudaMemcpyDeviceToHost, st));
    off += nseg + 1;
  }
  } catch (...) {
    // copies and kernels already enqueued still use x_dev, edges_dev, the pinned buffer and `out`:
    // let them finish before the buffers go back to their allocators
    for (auto &s : streams) (void)cudaStreamSynchronize(s.stream());
    throw;
  }
  for (auto &s : streams) s.synchronize();
  int64_t irregular = 0;
  for (int64_t g = 0; g < groups; ++g) irregular += flags_host[g];
  TORCH_CHECK(irregular < kGraphWaitError, "b200_cluster: the kNN scan was abandoned (a bounded wait ran out, or segment pointers that overlap)");
  return irregular;
}

}  // namespace

static auto registry = torch::RegisterOperators()
                           .op("torch_cluster::knn", &knn)
                           .op("torch_cluster::knn_hinted", &knn_hinted)
                           .op("torch_cluster::batch_info", &batch_info)
                           .op("torch_cluster::batch_check", &batch_check)
                           .op("torch_cluster::nearest_batched", &nearest_batched)
                           .op("torch_cluster::radius", &radius)
                           .op("torch_cluster::radius_part", &radius_part)
                           .op("torch_cluster::fps_ptr_list", &fps_ptr_list)
                           .op("torch_cluster::fps_segment_classes", &fps_segment_classes)
                           .op("torch_cluster::segment_ptr", &segment_ptr)
                           .op("torch_cluster::knn_graph_edges", &knn_graph_edges)
                           .op("torch_cluster::nearest", &nearest)
                           .op("torch_cluster::fps", &fps)
                           .op("torch_cluster::knn_graph_host", &knn_graph_host);
