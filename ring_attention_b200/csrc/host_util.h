// Host-side helpers shared between the C-ABI file and the ring schedule.
#pragma once
#include "common.cuh"

namespace ra {

int fail(int code, const char* fmt, ...);
int fail_cuda(cudaError_t e, const char* what);
int current_impl();
void set_last_impl(int impl);
int last_impl();

int check_shape(const ra_shape_t* s);
int check_tensor(const ra_tensor_t* t, const char* name);
int check_mod(const ra_score_mod_t* m, ModParams* out);

int run_fwd_block(const FwdParams& p, int dtype, cudaStream_t s);
int run_bwd_block(const BwdParams& p, int dtype, cudaStream_t s);

// tcgen05 family.  *_unsupported_reason returns NULL when the kernel takes the call,
// else a short text saying which condition failed.
const char* tc_fwd_unsupported_reason(const FwdParams& p, int dtype);
const char* tc_bwd_unsupported_reason(const BwdParams& p, int dtype);
cudaError_t tc_fwd_block(const FwdParams& p, cudaStream_t s);
cudaError_t tc_bwd_block(const BwdParams& p, cudaStream_t s);

}  // namespace ra
