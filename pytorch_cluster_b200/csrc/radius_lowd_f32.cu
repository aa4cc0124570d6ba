#include "radius_lowd_inst.cuh"
namespace b200c {
int launch_radius_lowd_f32(const RadiusArgs &a, bool fill) { return launch_radius_lowd<float>(a, fill); }
int radius_lowd_chunk_points(int dim, int dtype) {
  return dtype == B200C_F64 ? radius_lowd_chunk_points_t<double>(dim) : radius_lowd_chunk_points_t<float>(dim);
}
}  // namespace b200c
