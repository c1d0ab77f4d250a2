// placeholder until the tcgen05 forward lands
#include "common.cuh"
#include "host_util.h"
namespace ra {
const char* tc_fwd_unsupported_reason(const FwdParams&, int) { return "not built yet"; }
cudaError_t tc_fwd_block(const FwdParams&, cudaStream_t) { return cudaErrorNotSupported; }
}
