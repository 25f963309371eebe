// placeholder until the tcgen05 backward lands
#include "common.cuh"
namespace b200fa {
cudaError_t launch_bwd_sm100(const BwdParams&, int, cudaStream_t, int*) { return cudaErrorNotSupported; }
}
