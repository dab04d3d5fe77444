// Placeholders for tcgen05 stages that are not built yet.
#include "common.cuh"
namespace moba {
bool gate_sm100_supported(const moba_b200_problem&) { return false; }
int launch_gate_sm100(const moba_b200_problem&, const void*, const void*, const int32_t*, int32_t*, cudaStream_t) { return MOBA_B200_EUNSUPPORTED; }
}
