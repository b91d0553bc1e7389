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
//   * capacity: the shifted copies of the hashed array must fit RZ_NOALLOC_SCRATCH_BYTES (16 MiB):
//     8 copies x 2 bytes (bf16 path) or 4 copies x 4 bytes (tf32 / fp32 paths) per element, H rounded
//     up to a multiple of 64, i.e. H <= 2^20.  Shapes for which the ordinary entry point would also put
//     a split-contraction workspace into the scratch (small batches with long contractions) still run:
//     when the workspace does not fit next to the copies the launch does every block's whole
//     contraction instead (same result, fewer CTAs busy).  The one exception is fp32 precision with a
//     contraction longer than 2048, where the split is what bounds the rounding error: there copies
//     plus workspace must fit, else RZ_ERR_TOO_LARGE.  A refused call launches nothing;
//   * every GPU on which the library's module gets loaded holds those 16 MiB until the process exits;
//   * there is one array per device and every call rewrites it, so two calls whose kernels can overlap
//     on the GPU (different streams, no ordering between them) race on it.  Calls on one stream, or
//     ordered by events, are fine.  Nothing in the array has to start at zero: each call rewrites
//     every byte the kernel will read, including the padding past the end of the hashed array, and
//     zeroes the workspace part when it uses it.
//
// The call allocates no device memory: no cudaMalloc / cudaFree of a real pointer and no allocating library
// routine.  What does happen once, and belongs before any stream capture: the first call on a device looks up
// the array's device address (with that device current) and the library's status words, and pins one page of
// the library's own host data for the status copy; the first call of a host thread binds the device's primary
// context to it (a null cudaFree); the first launch of each kernel variant on a device sets that variant's
// shared-memory attribute and queries its occupancy.  A new shape can select a variant not used before, so warm
// up every shape that will be captured.
#include <atomic>

#include "rz_common.h"

namespace {

static_assert(RZ_NOALLOC_SCRATCH_BYTES == ((size_t)16 << 20), "capacity documented in the header");
constexpr int RZ_NOALLOC_MAX_DEVICES = 64;

// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device pointer.
static __device__ __align__(256) unsigned char g_rz_noalloc_scratch[RZ_NOALLOC_SCRATCH_BYTES];

std::atomic<void *> g_scratch_ptr[RZ_NOALLOC_MAX_DEVICES];

// Device address of the scratch array on the current device; resolved once per device.
int scratch_address(void **out)
{
    int dev = -1;
    int st = rz_record_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (st) return st;
    if (dev < 0 || dev >= RZ_NOALLOC_MAX_DEVICES) return RZ_ERR_UNSUPPORTED;
    void *ptr = g_scratch_ptr[dev].load(std::memory_order_acquire);
    if (!ptr) {
        st = rz_record_cuda(cudaGetSymbolAddress(&ptr, g_rz_noalloc_scratch), "cudaGetSymbolAddress(noalloc scratch)");
        if (st) return st;
        if (!ptr) return RZ_ERR_CUDA;
        g_scratch_ptr[dev].store(ptr, std::memory_order_release);   // (a second thread would store the same address)
    }
    *out = ptr;
    return RZ_OK;
}

}  // namespace

extern "C" {

int rz_linear_forward_noalloc(const rz_problem *pb, const void *X, const float *hashed, const float *bias, void *Y,
                              void *stream)
{
    // Problems that take the FMA kernels need no scratch at all: same call as the ordinary entry point.
    const size_t full = rz_shadow_bytes(pb);
    if (full == 0) return rz_linear_forward(pb, X, hashed, nullptr, 0, bias, Y, stream);
    if (rz_tc_copies_bytes(pb) > RZ_NOALLOC_SCRATCH_BYTES) return RZ_ERR_TOO_LARGE;
    if (full > RZ_NOALLOC_SCRATCH_BYTES && rz_tc_needs_workspace(pb, RZ_OP_FORWARD)) return RZ_ERR_TOO_LARGE;
    if (!X || !hashed || !Y) return RZ_ERR_NULL;
    void *scratch = nullptr;
    int st = scratch_address(&scratch);
    if (st) return st;
    st = rz_shadow_refresh(pb, hashed, scratch, stream);
    if (st) return st;
    return rz_forward_with_scratch(pb, X, hashed, scratch, RZ_NOALLOC_SCRATCH_BYTES, bias, Y, stream, true);
}

}  // extern "C"
