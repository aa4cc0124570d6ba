// The exact kernels for fp16 inputs: data widened to float, every operation result rounded to the
// 16-bit type as the reference's c10::Half instantiation does.
#include "generic_inst.cuh"
namespace b200c {
int launch_knn_generic_f16(const KnnArgs &a) { return launch_knn_generic<float, 1>(a); }
int launch_radius_generic_f16(const RadiusArgs &a, bool fill) { return launch_radius_generic<float, 1>(a, fill); }
int launch_row_norms_f16(const void *a, int64_t rows, int dim, void *out, cudaStream_t s) {
  return launch_row_norms_t<float, 1>(a, rows, dim, out, s);
}
int launch_nearest_generic_f16(const KnnArgs &a) { return launch_nearest_generic<float, 1>(a); }
}  // namespace b200c
