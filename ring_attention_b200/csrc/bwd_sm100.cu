// placeholder until the tcgen05 backward lands
#include "common.cuh"
#include "host_util.h"
namespace ra {
const char* tc_bwd_unsupported_reason(const BwdParams&, int) { return "not built yet"; }
cudaError_t tc_bwd_block(const BwdParams&, cudaStream_t) { return cudaErrorNotSupported; }
}
