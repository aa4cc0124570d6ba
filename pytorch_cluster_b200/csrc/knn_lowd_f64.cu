#include "knn_lowd_inst.cuh"
namespace b200c {
int launch_knn_lowd_f64(const KnnArgs &a) { return launch_knn_lowd<double>(a); }
}  // namespace b200c
