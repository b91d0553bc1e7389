// rz_linear_forward_noalloc: the forward pass for callers that cannot hand the library any scratch.
//
// The tensor-core forward kernel does not read the fp32 hashed array directly; it reads a "shadow" of
// it (element-shifted copies in the compute type), which the ordinary entry point expects the caller
// to allocate.  Some callers have nothing to allocate with: a host runtime that has already given all
// of the GPU's memory to its own pool so that cudaMalloc fails, a foreign-function binding that only
// ever sees the pointers it was handed, or a latency-critical loop where the implicit device
// synchronisation of an allocation is not acceptable.  For them this entry point keeps the shadow in
// a fixed array that is part of the library image.
//
// Consequences of the fixed array, all of which the caller has to know:
//   * capacity: the shadow of the problem must fit RZ_NOALLOC_SCRATCH_BYTES (16 MiB), i.e.
//     H <= 2^20 elements for both the bf16 and the tf32 paths; larger problems are refused with
//     RZ_ERR_TOO_LARGE and nothing is launched;
//   * every GPU on which the library's module gets loaded holds those 16 MiB until the process exits;
//   * the first call on a device looks up the array's device address (once per device, with that
//     device current).  Make that first call before any stream capture begins;
//   * there is one array per device and every call rewrites it, so two calls whose kernels can overlap
//     on the GPU (different streams, no ordering between them) race on it.  Calls on one stream, or
//     ordered by events, are fine.  Nothing in the array has to start at zero: each call rewrites
//     every byte the kernel will read, including the padding past the end of the hashed array.
//
// The call itself performs no cudaMalloc / cudaFree and uses no allocating library routine.
#include "rz_common.h"

namespace {

static_assert(RZ_NOALLOC_SCRATCH_BYTES == ((size_t)16 << 20), "capacity documented in the header");
constexpr int RZ_NOALLOC_MAX_DEVICES = 64;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device pointer.
static __device__ __align__(256) unsigned char g_rz_noalloc_scratch[RZ_NOALLOC_SCRATCH_BYTES];

void *g_scratch_ptr[RZ_NOALLOC_MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device; resolved once per device.
int scratch_address(void **out)
{
    int dev = -1;
    int st = rz_record_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (st) return st;
    if (dev < 0 || dev >= RZ_NOALLOC_MAX_DEVICES) return RZ_ERR_UNSUPPORTED;
    if (!g_scratch_ptr[dev]) {
        void *ptr = nullptr;
        st = rz_record_cuda(cudaGetSymbolAddress(&ptr, g_rz_noalloc_scratch), "cudaGetSymbolAddress(noalloc scratch)");
        if (st) return st;
        if (!ptr) return RZ_ERR_CUDA;
        g_scratch_ptr[dev] = ptr;
    }
    *out = g_scratch_ptr[dev];
    return RZ_OK;
}

}  // namespace

extern "C" {

int rz_linear_forward_noalloc(const rz_problem *pb, const void *X, const float *hashed, const float *bias, void *Y,
                              void *stream)
{
    // Problems that take the FMA kernels need no scratch at all: same call as the ordinary entry point.
    const size_t need = rz_shadow_bytes(pb);
    if (need == 0) return rz_linear_forward(pb, X, hashed, nullptr, bias, Y, stream);
    if (need > RZ_NOALLOC_SCRATCH_BYTES) return RZ_ERR_TOO_LARGE;
    if (!X || !hashed || !Y) return RZ_ERR_NULL;
    void *scratch = nullptr;
    int st = scratch_address(&scratch);
    if (st) return st;
    st = rz_shadow_refresh(pb, hashed, scratch, stream);
    if (st) return st;
    return rz_linear_forward(pb, X, hashed, scratch, bias, Y, stream);
}

}  // extern "C"
