// placeholder until the backward kernels land
#include "fal_launch.h"
namespace fal {
cudaError_t launch_bwd_prep(const BwdPrepParams&, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_bwd(int, bool, const CUtensorMap&, const CUtensorMap&, const CUtensorMap&,
                       const CUtensorMap&, const BwdParams&, int, cudaStream_t) { return cudaErrorNotSupported; }
cudaError_t launch_bwd_post(const BwdPostParams&, cudaStream_t) { return cudaErrorNotSupported; }
}
