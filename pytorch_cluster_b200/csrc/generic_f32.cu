#include "generic_inst.cuh"
namespace b200c {
int launch_knn_generic_f32(const KnnArgs &a) { return launch_knn_generic<float>(a); }
int launch_radius_generic_f32(const RadiusArgs &a, bool fill) { return launch_radius_generic<float>(a, fill); }
int launch_row_norms_f32(const void *a, int64_t rows, int dim, void *out, cudaStream_t s) {
  return launch_row_norms_t<float>(a, rows, dim, out, s);
}
int launch_nearest_generic_f32(const KnnArgs &a) { return launch_nearest_generic<float, 0>(a); }
}  // namespace b200c
