#include "radius_lowd_inst.cuh"
namespace b200c {
int launch_radius_lowd_f32(const RadiusArgs &a, bool fill) { return launch_radius_lowd<float>(a, fill); }
}  // namespace b200c
