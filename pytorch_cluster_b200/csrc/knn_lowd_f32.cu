#include "knn_lowd_inst.cuh"
namespace b200c {
int launch_knn_lowd_f32(const KnnArgs &a) { return launch_knn_lowd<float>(a); }
}  // namespace b200c
