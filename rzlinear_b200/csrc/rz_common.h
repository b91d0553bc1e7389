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

// Where a device-side bounded wait reports that it gave up (filled by rz_wait_context):
//   status      sticky device word, read and cleared by rz_device_status(); while it is non-zero every bounded wait on
//               the device gives up at once, so the other roles of the failing kernel leave their loops too;
//   host_status host-mapped copy of it (NULL when the page could not be pinned) that the host looks at, without
//               synchronising, before every tensor-core launch: work after a failed kernel is refused
//               (RZ_ERR_PIPELINE) instead of continuing on partial results, until rz_device_status() has
//               acknowledged the failure and cleared both words.
struct RzWaitCtx {
    int *status;
    int *host_status;
    long long limit_cycles;
};

struct RzLaunchCtx {
    const rz_problem *pb;
    RzHash hash;
    cudaStream_t stream;
};

// host helpers (rz_abi.cu)
int rz_record_cuda(cudaError_t e, const char *what);
void rz_count_launch(int n);
// Fills `w` for a launch on the current device.  RZ_ERR_PIPELINE when an earlier kernel on this device reported a
// wait that gave up and rz_device_status() has not been called since.
int rz_wait_context(RzWaitCtx *w, long long limit_cycles);

// rz_linear_forward with a say on the scratch: `copies_suffice` lets a scratch that holds the shifted copies but not
// the split-contraction workspace through (the launch then runs whole contractions per block).
int rz_forward_with_scratch(const rz_problem *pb, const void *X, const float *hashed, void *shadow, size_t shadow_bytes,
                            const float *bias, void *Y, void *stream, bool copies_suffice);

// SIMT family (rz_simt.cu)
int rz_simt_forward(const RzLaunchCtx &c, const void *X, const float *hashed, const float *bias, void *Y);
int rz_simt_backward_input(const RzLaunchCtx &c, const void *dY, const float *hashed, void *dX);
int rz_simt_backward_weight(const RzLaunchCtx &c, const void *X, const void *dY, float *dH);
int rz_simt_materialize(const RzLaunchCtx &c, const float *hashed, float *W);
int rz_elementwise_grad_prepare(const RzLaunchCtx &c, const void *dY, const void *Y, void *dYm, float *bias_grad);
int rz_simt_hash_indices(const RzLaunchCtx &c, int64_t *out);

// tcgen05 family (rz_tc.cu)
bool rz_tc_supported(const rz_problem *pb, int op);
size_t rz_tc_shadow_bytes(const rz_problem *pb);          // shifted copies + workspace
size_t rz_tc_copies_bytes(const rz_problem *pb);          // the shifted copies alone
bool rz_tc_needs_workspace(const rz_problem *pb, int op); // the launch cannot run without its workspace (fp32 precision, long contraction)
void rz_tc_reload_env();
int rz_tc_shadow_refresh(const RzLaunchCtx &c, const float *hashed, void *shadow);
// velocity == NULL: plain SGD.  shadow == NULL: the hashed array alone is updated.
int rz_tc_sgd_step(const RzLaunchCtx &c, float *hashed, const float *dH, float *velocity, float lr, float momentum, void *shadow);
// `shadow_bytes`: size of the caller's scratch.  When it holds the copies but not the workspace the launch runs every
// block's whole contraction (no workspace needed) unless rz_tc_needs_workspace().
int rz_tc_forward(const RzLaunchCtx &c, const void *X, void *shadow, size_t shadow_bytes, const float *bias, void *Y);
int rz_tc_backward_input(const RzLaunchCtx &c, const void *dY, void *shadow, size_t shadow_bytes, void *dX);
int rz_tc_backward_weight(const RzLaunchCtx &c, const void *X, const void *dY, float *dH);
int rz_tc_wait_selftest(long long limit_cycles, cudaStream_t stream);
