#include "nearest_lowd.cuh"
namespace b200c {
int launch_nearest_lowd_f32(const KnnArgs &a) { return launch_nearest_lowd<float>(a); }
int launch_nearest_lowd_f64(const KnnArgs &a) { return launch_nearest_lowd<double>(a); }
}  // namespace b200c
