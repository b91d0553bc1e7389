// Internal declarations shared by the translation units of librzlinear_b200.so.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#include "../../include/rzlinear_b200.h"
#include "rz_hash.h"

// Codes written to the device status word by bounded waits that gave up.
enum RzWaitCode {
    RZ_WAIT_NONE = 0,
    RZ_WAIT_SMEM_FULL = 1,
    RZ_WAIT_SMEM_EMPTY = 2,
    RZ_WAIT_TMEM_FULL = 3,
    RZ_WAIT_TMEM_EMPTY = 4,
    RZ_WAIT_STORE = 5,
    RZ_WAIT_SELFTEST = 6
};

struct RzLaunchCtx {
    const rz_problem *pb;
    RzHash hash;
    cudaStream_t stream;
};

// host helpers (rz_abi.cu)
int rz_record_cuda(cudaError_t e, const char *what);
void rz_count_launch(int n);
int *rz_device_status_word();  // device address of the status word of the current device

// SIMT family (rz_simt.cu)
int rz_simt_forward(const RzLaunchCtx &c, const void *X, const float *hashed, const float *bias, void *Y);
int rz_simt_backward_input(const RzLaunchCtx &c, const void *dY, const float *hashed, void *dX);
int rz_simt_backward_weight(const RzLaunchCtx &c, const void *X, const void *dY, float *dH);
int rz_simt_materialize(const RzLaunchCtx &c, const float *hashed, float *W);
int rz_elementwise_grad_prepare(const RzLaunchCtx &c, const void *dY, const void *Y, void *dYm, float *bias_grad);
int rz_simt_hash_indices(const RzLaunchCtx &c, int64_t *out);

// tcgen05 family (rz_tc.cu)
bool rz_tc_supported(const rz_problem *pb, int op);
size_t rz_tc_shadow_bytes(const rz_problem *pb);
int rz_tc_shadow_refresh(const RzLaunchCtx &c, const float *hashed, void *shadow);
int rz_tc_sgd_step(const RzLaunchCtx &c, float *hashed, const float *dH, float lr, void *shadow);
int rz_tc_sgd_momentum_step(const RzLaunchCtx &c, float *hashed, const float *dH, float *velocity, float lr, float momentum,
                            void *shadow);
int rz_tc_forward(const RzLaunchCtx &c, const void *X, const void *shadow, const float *bias, void *Y);
int rz_tc_backward_input(const RzLaunchCtx &c, const void *dY, const void *shadow, void *dX);
int rz_tc_backward_weight(const RzLaunchCtx &c, const void *X, const void *dY, float *dH);
int rz_tc_wait_selftest(long long limit_cycles, cudaStream_t stream);
