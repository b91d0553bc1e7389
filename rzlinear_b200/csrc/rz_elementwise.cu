// Backward-pass preparation for a layer whose bias and ReLU were fused into the forward kernel: one pass over
// the incoming gradient that masks it with the saved activation (dYm = dY where Y > 0) and sums its columns into
// the bias gradient.  HBM-bound: reads dY (and Y), writes dYm; 16-byte accesses, every warp on 512 contiguous
// bytes of a row, grid sized to a few CTAs per SM.
#include "rz_common.h"

namespace {

template <typename T> struct Vec;            // 16 bytes of T
template <> struct Vec<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4 &u, float *f)
    {
        f[0] = __uint_as_float(u.x), f[1] = __uint_as_float(u.y), f[2] = __uint_as_float(u.z), f[3] = __uint_as_float(u.w);
    }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4 &u, float *f)
    {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);            // low half = first element
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// 16 bytes of gradient with the elements whose activation is not positive cleared.  The sign test works on
// the raw bits (positive = sign bit clear and not zero), so nothing is converted and dYm keeps dY's bits.
template <typename T> __device__ __forceinline__ uint4 mask_positive(const uint4 &g, const uint4 &y);
template <> __device__ __forceinline__ uint4 mask_positive<float>(const uint4 &g, const uint4 &y)
{
    uint4 r;
    r.x = (__uint_as_float(y.x) > 0.f) ? g.x : 0u;
    r.y = (__uint_as_float(y.y) > 0.f) ? g.y : 0u;
    r.z = (__uint_as_float(y.z) > 0.f) ? g.z : 0u;
    r.w = (__uint_as_float(y.w) > 0.f) ? g.w : 0u;
    return r;
}
template <> __device__ __forceinline__ uint4 mask_positive<__nv_bfloat16>(const uint4 &g, const uint4 &y)
{
    const uint32_t gw[4] = {g.x, g.y, g.z, g.w}, yw[4] = {y.x, y.y, y.z, y.w};
    uint32_t r[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = (__uint_as_float(yw[i] << 16) > 0.f) ? 0x0000ffffu : 0u;
        const uint32_t hi = (__uint_as_float(yw[i] & 0xffff0000u) > 0.f) ? 0xffff0000u : 0u;
        r[i] = gw[i] & (lo | hi);
    }
    return make_uint4(r[0], r[1], r[2], r[3]);
}

// Vector path: N a multiple of the vector width and all pointers 16-byte aligned.  Thread = one 16-byte column
// group, walking rows blockIdx.y, blockIdx.y + gridDim.y, ...; four rows in flight per thread.
template <typename T>
__global__ void __launch_bounds__(256) rz_grad_prepare_kernel(const uint4 *__restrict__ dY, const uint4 *__restrict__ Y,
                                                              uint4 *__restrict__ dYm, float *__restrict__ bias_grad,
                                                              uint32_t M, uint32_t vec_per_row)
{
    constexpr int V = Vec<T>::N;
    const uint32_t cv = blockIdx.x * blockDim.x + threadIdx.x;
    if (cv >= vec_per_row) return;
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    constexpr int U = 4;
    const uint32_t stride = gridDim.y;
    uint32_t r = blockIdx.y;
    for (; r + (U - 1) * stride < M; r += U * stride) {
        uint4 g[U], y[U];
#pragma unroll
        for (int i = 0; i < U; ++i) {
            const size_t o = (size_t)(r + i * stride) * vec_per_row + cv;
            g[i] = __ldg(dY + o);
            if (Y) y[i] = __ldg(Y + o);
        }
#pragma unroll
        for (int i = 0; i < U; ++i) {
            if (Y) g[i] = mask_positive<T>(g[i], y[i]);
            if (dYm) dYm[(size_t)(r + i * stride) * vec_per_row + cv] = g[i];
            if (bias_grad) {
                float f[V];
                Vec<T>::unpack(g[i], f);
#pragma unroll
                for (int j = 0; j < V; ++j) acc[j] += f[j];
            }
        }
    }
    for (; r < M; r += stride) {
        const size_t o = (size_t)r * vec_per_row + cv;
        uint4 g = __ldg(dY + o);
        if (Y) g = mask_positive<T>(g, __ldg(Y + o));
        if (dYm) dYm[o] = g;
        if (bias_grad) {
            float f[V];
            Vec<T>::unpack(g, f);
#pragma unroll
            for (int j = 0; j < V; ++j) acc[j] += f[j];
        }
    }
    if (bias_grad) {
#pragma unroll
        for (int j = 0; j < V; ++j) atomicAdd(bias_grad + (size_t)cv * V + j, acc[j]);
    }
}

template <typename T> __device__ __forceinline__ float elem_f32(T v);
template <> __device__ __forceinline__ float elem_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float elem_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// Any N, any alignment: thread = one column.
template <typename T>
__global__ void __launch_bounds__(256) rz_grad_prepare_scalar_kernel(const T *__restrict__ dY, const T *__restrict__ Y,
                                                                     T *__restrict__ dYm, float *__restrict__ bias_grad,
                                                                     uint32_t M, uint32_t N)
{
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= N) return;
    float acc = 0.f;
    for (uint32_t r = blockIdx.y; r < M; r += gridDim.y) {
        const size_t o = (size_t)r * N + c;
        T g = dY[o];
        if (Y && !(elem_f32(Y[o]) > 0.f)) g = T(0.f);
        if (dYm) dYm[o] = g;
        acc += elem_f32(g);
    }
    if (bias_grad) atomicAdd(bias_grad + c, acc);
}

template <typename T>
int launch(const RzLaunchCtx &c, const void *dY, const void *Y, void *dYm, float *bias_grad)
{
    const uint32_t M = (uint32_t)c.pb->M, N = (uint32_t)c.pb->N;
    constexpr int V = Vec<T>::N;
    const uintptr_t bits = reinterpret_cast<uintptr_t>(dY) | reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(dYm);
    const bool vec = (N % V == 0) && (bits & 15u) == 0;
    if (bias_grad) {
        int st = rz_record_cuda(cudaMemsetAsync(bias_grad, 0, sizeof(float) * N, c.stream), "zero bias gradient");
        if (st) return st;
    }
    const uint32_t per_row = vec ? N / V : N;
    dim3 grid((per_row + 255) / 256, 1, 1);
    // about eight CTAs per SM in total, at least one row each
    uint32_t gy = (148u * 8u + grid.x - 1) / grid.x;
    if (gy > M) gy = M;
    if (gy > 65535u) gy = 65535u;
    grid.y = gy;
    if (vec)
        rz_grad_prepare_kernel<T><<<grid, 256, 0, c.stream>>>(static_cast<const uint4 *>(dY), static_cast<const uint4 *>(Y),
                                                               static_cast<uint4 *>(dYm), bias_grad, M, per_row);
    else
        rz_grad_prepare_scalar_kernel<T><<<grid, 256, 0, c.stream>>>(static_cast<const T *>(dY), static_cast<const T *>(Y),
                                                                      static_cast<T *>(dYm), bias_grad, M, N);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "gradient preparation launch");
}

}  // namespace

int rz_elementwise_grad_prepare(const RzLaunchCtx &c, const void *dY, const void *Y, void *dYm, float *bias_grad)
{
    if (c.pb->io_dtype == RZ_BF16) return launch<__nv_bfloat16>(c, dY, Y, dYm, bias_grad);
    return launch<float>(c, dY, Y, dYm, bias_grad);
}
