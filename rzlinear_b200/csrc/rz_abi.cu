// C ABI of librzlinear_b200.so: argument validation, path selection and dispatch.
// Declarations and the reference interfaces they replace: include/rzlinear_b200.h.
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "rz_common.h"

namespace {

thread_local char g_cuda_error[256] = "";
std::atomic<uint64_t> g_launches{0};

// Device-side status word: 0, or (wait code << 8 | 1) once a bounded wait gave up.  Sticky until rz_device_status().
__device__ int g_rz_status_word = 0;

// Host copy of the status words, one int per device index, in a page of this library that is registered as
// mapped pinned memory the first time a tensor-core launch is prepared: a kernel whose wait gives up stores its
// code here too, and the host reads it (a plain load, no synchronisation) before it launches anything else.
constexpr int RZ_MAX_DEVICES = 64;
alignas(4096) int g_host_status[1024];
std::once_flag g_host_once;
bool g_host_registered = false;

struct DeviceAddrs {
    std::atomic<int *> status{nullptr};
    std::atomic<int *> host{nullptr};
};
DeviceAddrs g_addrs[RZ_MAX_DEVICES];

int validate(const rz_problem *pb)
{
    if (!pb) return RZ_ERR_NULL;
    if (pb->M <= 0 || pb->K <= 0 || pb->N <= 0 || pb->H <= 0 || pb->BK <= 0 || pb->BN <= 0) return RZ_ERR_SHAPE;
    const int64_t lim = (int64_t)1 << 31;
    if (pb->M >= lim || pb->K >= lim || pb->N >= lim || pb->H >= lim) return RZ_ERR_SHAPE;
    if ((int64_t)pb->BK * pb->BN >= lim) return RZ_ERR_SHAPE;
    if (pb->H <= (int64_t)pb->BK * pb->BN) return RZ_ERR_HASH_RANGE;
    if (pb->hash_mode != RZ_HASH_SINGLE && pb->hash_mode != RZ_HASH_TWO_LEVEL) return RZ_ERR_HASH_PARAM;
    if (pb->R[0] <= 0) return RZ_ERR_HASH_PARAM;
    for (int i = 0; i < 8; ++i)
        if (pb->R[i] < 0 || pb->R[i] >= lim) return RZ_ERR_HASH_PARAM;
    if (pb->io_dtype != RZ_F32 && pb->io_dtype != RZ_BF16) return RZ_ERR_DTYPE;
    if (pb->precision != RZ_PREC_FP32 && pb->precision != RZ_PREC_TF32 && pb->precision != RZ_PREC_BF16)
        return RZ_ERR_DTYPE;
    if (pb->precision == RZ_PREC_TF32 && pb->io_dtype != RZ_F32) return RZ_ERR_DTYPE;
    if (pb->precision == RZ_PREC_BF16 && pb->io_dtype != RZ_BF16) return RZ_ERR_DTYPE;
    if (pb->sm_reserve < 0 || pb->sm_reserve > 1024) return RZ_ERR_SHAPE;
    return RZ_OK;
}

RzHash make_hash(const rz_problem *pb)
{
    RzHash h;
    h.R0 = (uint64_t)pb->R[0];
    h.R1 = (uint64_t)pb->R[1];
    h.R2 = (uint64_t)pb->R[2];
    h.R3 = (uint64_t)pb->R[3];
    h.R4 = (uint64_t)pb->R[4];
    h.R5 = (uint64_t)pb->R[5];
    h.R7 = (uint64_t)pb->R[7];
    h.range = (uint64_t)(pb->H - (int64_t)pb->BK * pb->BN);
    h.BK = pb->BK;
    h.BN = pb->BN;
    h.two_level = pb->hash_mode == RZ_HASH_TWO_LEVEL;
    h.pad = 0;
    rz_hash_finish(h);
    return h;
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

bool use_tc(const rz_problem *pb, int op)
{
    if (pb->flags & RZ_FLAG_FORCE_SIMT) return false;
    if (pb->precision == RZ_PREC_FP32 && pb->io_dtype != RZ_F32) return false;   // fp32 math on bf16 data: FMA kernels
    return rz_tc_supported(pb, op);
}

RzLaunchCtx make_ctx(const rz_problem *pb, void *stream)
{
    RzLaunchCtx c;
    c.pb = pb;
    c.hash = make_hash(pb);
    c.stream = reinterpret_cast<cudaStream_t>(stream);
    return c;
}

}  // namespace

int rz_record_cuda(cudaError_t e, const char *what)
{
    if (e == cudaSuccess) return RZ_OK;
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s", what, cudaGetErrorString(e));
    return RZ_ERR_CUDA;
}

void rz_count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

int rz_wait_context(RzWaitCtx *w, long long limit_cycles)
{
    int dev = 0;
    int st = rz_record_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (st) return st;
    if (dev < 0 || dev >= RZ_MAX_DEVICES) return RZ_ERR_UNSUPPORTED;
    DeviceAddrs &a = g_addrs[dev];
    int *status = a.status.load(std::memory_order_acquire);
    if (!status) {   // first launch on this device: the addresses never change while the module is loaded
        st = rz_record_cuda(cudaGetSymbolAddress(reinterpret_cast<void **>(&status), g_rz_status_word), "status word address");
        if (st) return st;
        std::call_once(g_host_once, [] {
            g_host_registered = cudaHostRegister(g_host_status, sizeof(g_host_status),
                                                 cudaHostRegisterPortable | cudaHostRegisterMapped) == cudaSuccess;
            if (!g_host_registered) (void)cudaGetLastError();   // no host copy: rz_device_status() is the only report
        });
        int *host_dev = nullptr;
        if (g_host_registered &&
            cudaHostGetDevicePointer(reinterpret_cast<void **>(&host_dev), g_host_status + dev, 0) != cudaSuccess) {
            host_dev = nullptr;
            (void)cudaGetLastError();
        }
        a.host.store(host_dev, std::memory_order_relaxed);
        a.status.store(status, std::memory_order_release);
    }
    w->status = status;
    w->host_status = a.host.load(std::memory_order_relaxed);
    w->limit_cycles = limit_cycles;
    if (w->host_status && *reinterpret_cast<volatile int *>(&g_host_status[dev]) != 0) return RZ_ERR_PIPELINE;
    return RZ_OK;
}

int rz_forward_with_scratch(const rz_problem *pb, const void *X, const float *hashed, void *shadow, size_t shadow_bytes,
                            const float *bias, void *Y, void *stream, bool copies_suffice)
{
    int st = validate(pb);
    if (st) return st;
    if (!X || !hashed || !Y) return RZ_ERR_NULL;
    RzLaunchCtx c = make_ctx(pb, stream);
    if (use_tc(pb, RZ_OP_FORWARD)) {
        if (!shadow) return RZ_ERR_NULL;
        if (!aligned16(X) || !aligned16(Y) || (reinterpret_cast<uintptr_t>(shadow) & 255u)) return RZ_ERR_ALIGN;
        if (shadow_bytes < (copies_suffice ? rz_tc_copies_bytes(pb) : rz_tc_shadow_bytes(pb))) return RZ_ERR_SCRATCH;
        return rz_tc_forward(c, X, shadow, shadow_bytes, bias, Y);
    }
    return rz_simt_forward(c, X, hashed, bias, Y);
}

extern "C" {

int rz_version(void) { return 100; }

const char *rz_status_string(int status)
{
    switch (status) {
    case RZ_OK: return "ok";
    case RZ_ERR_NULL: return "a required pointer is NULL";
    case RZ_ERR_SHAPE: return "bad shape: a dimension is <= 0 or does not fit";
    case RZ_ERR_HASH_RANGE: return "hashed array too small: H must be larger than BK*BN";
    case RZ_ERR_DTYPE: return "unsupported io_dtype / precision combination";
    case RZ_ERR_ALIGN: return "pointer not 16-byte aligned";
    case RZ_ERR_HASH_PARAM: return "bad hash parameters (prime <= 0, negative or >= 2^31 random number, unknown mode)";
    case RZ_ERR_CUDA: return "CUDA call failed";
    case RZ_ERR_PIPELINE: return "device pipeline wait timed out (results since then are invalid; rz_device_status() clears it)";
    case RZ_ERR_UNSUPPORTED: return "problem not supported on the requested path";
    case RZ_ERR_TOO_LARGE: return "size exceeds the capacity of this entry point";
    case RZ_ERR_SCRATCH: return "scratch buffer smaller than rz_shadow_bytes() of this problem";
    default: return "unknown status";
    }
}

const char *rz_last_cuda_error(void) { return g_cuda_error; }

int rz_hash_indices_host(const rz_problem *pb, int64_t *out_host)
{
    int st = validate(pb);
    if (st) return st;
    if (!out_host) return RZ_ERR_NULL;
    RzHash h = make_hash(pb);
    const uint32_t nk = (uint32_t)((pb->K + pb->BK - 1) / pb->BK);
    const uint32_t nn = (uint32_t)((pb->N + pb->BN - 1) / pb->BN);
    for (uint32_t pk = 0; pk < nk; ++pk)
        for (uint32_t pn = 0; pn < nn; ++pn) out_host[(size_t)pk * nn + pn] = (int64_t)rz_tile_offset(h, pk, pn);
    return RZ_OK;
}

int rz_hash_indices_device(const rz_problem *pb, int64_t *out_dev, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (!out_dev) return RZ_ERR_NULL;
    return rz_simt_hash_indices(make_ctx(pb, stream), out_dev);
}

int rz_plan(const rz_problem *pb, int op)
{
    int st = validate(pb);
    if (st) return st;
    if (op < RZ_OP_FORWARD || op > RZ_OP_BACKWARD_WEIGHT) return RZ_ERR_UNSUPPORTED;
    return use_tc(pb, op) ? RZ_PATH_TCGEN05 : RZ_PATH_SIMT;
}

size_t rz_shadow_bytes(const rz_problem *pb)
{
    if (validate(pb)) return 0;
    if (!use_tc(pb, RZ_OP_FORWARD) && !use_tc(pb, RZ_OP_BACKWARD_INPUT)) return 0;
    return rz_tc_shadow_bytes(pb);
}

int rz_shadow_refresh(const rz_problem *pb, const float *hashed, void *shadow, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (rz_shadow_bytes(pb) == 0) return RZ_OK;
    if (!hashed || !shadow) return RZ_ERR_NULL;
    if (!aligned16(hashed) || (reinterpret_cast<uintptr_t>(shadow) & 255u)) return RZ_ERR_ALIGN;
    return rz_tc_shadow_refresh(make_ctx(pb, stream), hashed, shadow);
}

int rz_linear_forward(const rz_problem *pb, const void *X, const float *hashed, void *shadow, size_t shadow_bytes,
                      const float *bias, void *Y, void *stream)
{
    return rz_forward_with_scratch(pb, X, hashed, shadow, shadow_bytes, bias, Y, stream, false);
}

int rz_linear_backward_input(const rz_problem *pb, const void *dY, const float *hashed, void *shadow, size_t shadow_bytes,
                             void *dX, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (!dY || !hashed || !dX) return RZ_ERR_NULL;
    RzLaunchCtx c = make_ctx(pb, stream);
    if (use_tc(pb, RZ_OP_BACKWARD_INPUT)) {
        if (!shadow) return RZ_ERR_NULL;
        if (!aligned16(dY) || !aligned16(dX) || (reinterpret_cast<uintptr_t>(shadow) & 255u)) return RZ_ERR_ALIGN;
        if (shadow_bytes < rz_tc_shadow_bytes(pb)) return RZ_ERR_SCRATCH;
        return rz_tc_backward_input(c, dY, shadow, shadow_bytes, dX);
    }
    return rz_simt_backward_input(c, dY, hashed, dX);
}

int rz_linear_backward_weight(const rz_problem *pb, const void *X, const void *dY, float *dH, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (!X || !dY || !dH) return RZ_ERR_NULL;
    RzLaunchCtx c = make_ctx(pb, stream);
    if (!(pb->flags & RZ_FLAG_ACCUMULATE_DH)) {
        st = rz_record_cuda(cudaMemsetAsync(dH, 0, sizeof(float) * (size_t)pb->H, c.stream), "zero dH");
        if (st) return st;
    }
    if (use_tc(pb, RZ_OP_BACKWARD_WEIGHT)) {
        if (!aligned16(X) || !aligned16(dY) || !aligned16(dH)) return RZ_ERR_ALIGN;
        return rz_tc_backward_weight(c, X, dY, dH);
    }
    return rz_simt_backward_weight(c, X, dY, dH);
}

int rz_linear_materialize(const rz_problem *pb, const float *hashed, float *W, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (!hashed || !W) return RZ_ERR_NULL;
    return rz_simt_materialize(make_ctx(pb, stream), hashed, W);
}

int rz_grad_prepare(const rz_problem *pb, const void *dY, const void *Y, void *dYm, float *bias_grad, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (!dY || (Y && !dYm) || (!dYm && !bias_grad)) return RZ_ERR_NULL;
    return rz_elementwise_grad_prepare(make_ctx(pb, stream), dY, Y, dYm, bias_grad);
}

int rz_sgd_step(const rz_problem *pb, float *hashed, const float *dH, float lr, void *shadow, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (!hashed || !dH) return RZ_ERR_NULL;
    if (!aligned16(hashed) || !aligned16(dH)) return RZ_ERR_ALIGN;
    if (shadow && rz_shadow_bytes(pb) == 0) shadow = nullptr;
    if (shadow && (reinterpret_cast<uintptr_t>(shadow) & 255u)) return RZ_ERR_ALIGN;
    return rz_tc_sgd_step(make_ctx(pb, stream), hashed, dH, nullptr, lr, 0.f, shadow);
}

int rz_sgd_momentum_step(const rz_problem *pb, float *hashed, const float *dH, float *velocity, float lr, float momentum,
                         void *shadow, void *stream)
{
    int st = validate(pb);
    if (st) return st;
    if (!hashed || !dH || !velocity) return RZ_ERR_NULL;
    if (!aligned16(hashed) || !aligned16(dH) || !aligned16(velocity)) return RZ_ERR_ALIGN;
    if (shadow && rz_shadow_bytes(pb) == 0) shadow = nullptr;
    if (shadow && (reinterpret_cast<uintptr_t>(shadow) & 255u)) return RZ_ERR_ALIGN;
    return rz_tc_sgd_step(make_ctx(pb, stream), hashed, dH, velocity, lr, momentum, shadow);
}

int rz_device_status(int *out, int *detail)
{
    if (!out) return RZ_ERR_NULL;
    int word = 0;
    int st = rz_record_cuda(cudaDeviceSynchronize(), "device synchronize");
    if (st) return st;
    st = rz_record_cuda(cudaMemcpyFromSymbol(&word, g_rz_status_word, sizeof(int)), "read status word");
    if (st) return st;
    if (word != 0) {
        int zero = 0;
        st = rz_record_cuda(cudaMemcpyToSymbol(g_rz_status_word, &zero, sizeof(int)), "clear status word");
        if (st) return st;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < RZ_MAX_DEVICES)
        *reinterpret_cast<volatile int *>(&g_host_status[dev]) = 0;   // the device is idle: no kernel can be writing it
    *out = word ? RZ_ERR_PIPELINE : RZ_OK;
    if (detail) *detail = word >> 8;
    return RZ_OK;
}

int rz_selftest_bounded_wait(int64_t limit_cycles, void *stream)
{
    if (limit_cycles <= 0 || limit_cycles > 2000000000ll) return RZ_ERR_SHAPE;
    return rz_tc_wait_selftest((long long)limit_cycles, reinterpret_cast<cudaStream_t>(stream));
}

uint64_t rz_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void rz_reload_env(void) { rz_tc_reload_env(); }

}  // extern "C"
