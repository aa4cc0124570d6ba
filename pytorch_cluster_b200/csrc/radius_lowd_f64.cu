#include "radius_lowd_inst.cuh"
namespace b200c {
int launch_radius_lowd_f64(const RadiusArgs &a, bool fill) { return launch_radius_lowd<double>(a, fill); }
}  // namespace b200c
