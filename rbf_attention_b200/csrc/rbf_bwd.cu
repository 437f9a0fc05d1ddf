#include "common.cuh"
#include "launch.h"
namespace rbf {
cudaError_t launch_bwd_dkdv(const BwdArgs&, bool, int, bool, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_bwd_dq(const BwdArgs&, bool, int, bool, cudaStream_t) { return cudaErrorNotSupported; }
}
