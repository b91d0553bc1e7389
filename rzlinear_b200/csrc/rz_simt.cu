// SIMT (fp32 FMA) kernels of the RzLinear path: forward, input gradient, hashed-weight gradient,
// materialise and the tile-offset dump.  They accept every shape, hash tile and alignment, compute
// in fp32 exactly like the reference with allow_tf32=False, and are what RZ_PREC_FP32 runs; the
// tensor-core kernels cover the tf32 / bf16 precisions for tile-aligned shapes.
//
// One CTA of 256 threads computes a TB x TB output block (128 x 128 with 8 x 8 outputs per thread when the
// output is large enough to fill the GPU with such blocks, 64 x 64 with 4 x 4 otherwise), walking the
// contraction in chunks of TC.  The next chunk is fetched into registers while the current one is multiplied
// out of shared memory (two buffers, one barrier per chunk).  Elements of the virtual weight are fetched
// straight from the hashed array (L2-resident); a thread recomputes a tile offset in registers only when it
// crosses into another hash tile.
#include "rz_common.h"

namespace {

constexpr int PAD = 4;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Per-thread memo of the last tile offset, so the 64-bit hash runs once per tile crossing.
struct TileMemo {
    uint32_t pk = 0xffffffffu, pn = 0xffffffffu;
    uint32_t k_lo = 0, n_lo = 0;
    uint64_t off = 0;
    __device__ __forceinline__ uint64_t index(const RzHash &h, uint32_t k, uint32_t n)
    {
        if (!(pk != 0xffffffffu && k - k_lo < (uint32_t)h.BK && n - n_lo < (uint32_t)h.BN)) {
            pk = k / (uint32_t)h.BK;
            pn = n / (uint32_t)h.BN;
            k_lo = pk * (uint32_t)h.BK;
            n_lo = pn * (uint32_t)h.BN;
            off = rz_tile_offset(h, pk, pn);
        }
        return off + (uint64_t)(k - k_lo) * (uint32_t)h.BN + (n - n_lo);
    }
};

// OP 0: out[m][n] = sum_k X[m][k] W[k][n]       (rows M, cols N, contraction K)
// OP 1: out[m][k] = sum_n dY[m][n] W[k][n]      (rows M, cols K, contraction N)
// OP 2: dH[idx(k,n)] += sum_m X[m][k] dY[m][n]  (rows K, cols N, contraction M, split over grid.z)
// TB: block edge (64 or 128).  A thread owns G x G groups of 4 x 4 outputs, G = TB / 64, the groups 64 apart, so
// that its shared-memory reads are 16-byte loads without bank conflicts.  TC * TB = 1024: four elements of either
// operand per thread and chunk.
template <int OP, typename T, int TB>
__global__ void __launch_bounds__(256)
rz_simt_kernel(const T *__restrict__ A, const T *__restrict__ B2, const float *__restrict__ hashed,
               const float *__restrict__ bias, void *__restrict__ out_, float *__restrict__ dH,
               RzHash hash, uint32_t M, uint32_t K, uint32_t N, float alpha, int relu, uint32_t chunk_per_split)
{
    constexpr int TC = 1024 / TB;   // contraction chunk: 16 (TB = 64) or 8 (TB = 128)
    constexpr int G = TB / 64;
    __shared__ __align__(16) float As[2][TC][TB + PAD];
    __shared__ __align__(16) float Bs[2][TC][TB + PAD];

    const uint32_t rows = (OP == 2) ? K : M;
    const uint32_t cols = (OP == 1) ? K : N;
    const uint32_t depth = (OP == 0) ? K : (OP == 1 ? N : M);

    const uint32_t r0 = blockIdx.y * TB;
    const uint32_t c0 = blockIdx.x * TB;
    const uint32_t tid = threadIdx.x;
    const uint32_t tx = tid % 16, ty = tid / 16;

    uint32_t d_begin = 0, d_end = depth;
    if (OP == 2) {
        d_begin = blockIdx.z * chunk_per_split;
        d_end = min(depth, d_begin + chunk_per_split);
    }

    float acc[4 * G][4 * G];
#pragma unroll
    for (int i = 0; i < 4 * G; ++i)
#pragma unroll
        for (int j = 0; j < 4 * G; ++j) acc[i][j] = 0.f;

    TileMemo memo;
    // where this thread's four elements of a chunk sit: along the contraction (x = block row / column, d4 = first
    // of four contraction steps) for operands stored contraction-contiguous, or along the block edge (dd = one
    // contraction step, e4 = first of four block rows / columns) for the others
    const uint32_t x_of = tid / (TC / 4), d4_of = (tid % (TC / 4)) * 4;
    const uint32_t dd_of = tid / (TB / 4), e4_of = (tid % (TB / 4)) * 4;
    float ra[4], rb[4];

    auto fetch = [&](uint32_t d0) {
        if (OP == 0 || OP == 1) {   // A is [M][depth] row-major, contiguous along the contraction
            const uint32_t ld = (OP == 0) ? K : N, r = r0 + x_of;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t d = d0 + d4_of + e;
                ra[e] = (r < rows && d < d_end) ? to_f32<T>(A[(size_t)r * ld + d]) : 0.f;
            }
        } else {                    // A(k, m) = X[m][k]: contiguous along the output row index k
            const uint32_t d = d0 + dd_of;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t r = r0 + e4_of + e;
                ra[e] = (r < rows && d < d_end) ? to_f32<T>(A[(size_t)d * K + r]) : 0.f;
            }
        }
        if (OP == 0) {              // B(k, n) = W[k][n]
            const uint32_t k = d0 + dd_of;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t n = c0 + e4_of + e;
                rb[e] = (k < d_end && n < cols) ? hashed[memo.index(hash, k, n)] : 0.f;
            }
        } else if (OP == 1) {       // B(n, k) = W[k][n]: contiguous along the contraction n
            const uint32_t k = c0 + x_of;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t n = d0 + d4_of + e;
                rb[e] = (k < cols && n < d_end) ? hashed[memo.index(hash, k, n)] : 0.f;
            }
        } else {                    // B(m, n) = dY[m][n]
            const uint32_t m = d0 + dd_of;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t n = c0 + e4_of + e;
                rb[e] = (m < d_end && n < cols) ? to_f32<T>(B2[(size_t)m * N + n]) : 0.f;
            }
        }
    };
    auto stash = [&](int buf) {
        if (OP == 0 || OP == 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) As[buf][d4_of + e][x_of] = ra[e];
        } else {
            *reinterpret_cast<float4 *>(&As[buf][dd_of][e4_of]) = make_float4(ra[0], ra[1], ra[2], ra[3]);
        }
        if (OP == 1) {
#pragma unroll
            for (int e = 0; e < 4; ++e) Bs[buf][d4_of + e][x_of] = rb[e];
        } else {
            *reinterpret_cast<float4 *>(&Bs[buf][dd_of][e4_of]) = make_float4(rb[0], rb[1], rb[2], rb[3]);
        }
    };

    int buf = 0;
    if (d_begin < d_end) {
        fetch(d_begin);
        stash(0);
    }
    __syncthreads();
    for (uint32_t d0 = d_begin; d0 < d_end; d0 += TC) {
        const bool more = d0 + TC < d_end;
        if (more) fetch(d0 + TC);   // in flight while this chunk is multiplied
#pragma unroll
        for (int dd = 0; dd < TC; ++dd) {
            float a[4 * G], b[4 * G];
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 av = *reinterpret_cast<const float4 *>(&As[buf][dd][g * 64 + ty * 4]);
                const float4 bv = *reinterpret_cast<const float4 *>(&Bs[buf][dd][g * 64 + tx * 4]);
                a[4 * g + 0] = av.x, a[4 * g + 1] = av.y, a[4 * g + 2] = av.z, a[4 * g + 3] = av.w;
                b[4 * g + 0] = bv.x, b[4 * g + 1] = bv.y, b[4 * g + 2] = bv.z, b[4 * g + 3] = bv.w;
            }
#pragma unroll
            for (int i = 0; i < 4 * G; ++i)
#pragma unroll
                for (int j = 0; j < 4 * G; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (more) stash(buf ^ 1);   // (the other buffer was last read before the previous barrier)
        __syncthreads();
        buf ^= 1;
    }

    // ---- epilogue: output (i, j) of the thread is block row (i / 4) * 64 + ty * 4 + i % 4, likewise its column ----
    if (OP == 2) {
        TileMemo em;
#pragma unroll
        for (int i = 0; i < 4 * G; ++i)
#pragma unroll
            for (int j = 0; j < 4 * G; ++j) {
                const uint32_t k = r0 + (i / 4) * 64 + ty * 4 + (i % 4), n = c0 + (j / 4) * 64 + tx * 4 + (j % 4);
                if (k < rows && n < cols) atomicAdd(dH + em.index(hash, k, n), acc[i][j] * alpha);
            }
    } else {
        T *out = reinterpret_cast<T *>(out_);
#pragma unroll
        for (int i = 0; i < 4 * G; ++i)
#pragma unroll
            for (int j = 0; j < 4 * G; ++j) {
                const uint32_t r = r0 + (i / 4) * 64 + ty * 4 + (i % 4), c = c0 + (j / 4) * 64 + tx * 4 + (j % 4);
                if (r < rows && c < cols) {
                    float v = acc[i][j] * alpha;
                    if (OP == 0) {
                        if (bias) v += bias[c];
                        if (relu) v = fmaxf(v, 0.f);
                    }
                    out[(size_t)r * cols + c] = from_f32<T>(v);
                }
            }
    }
}

__global__ void rz_materialize_kernel(const float *__restrict__ hashed, float *__restrict__ W, RzHash hash,
                                      uint32_t K, uint32_t N)
{
    // blockIdx.y strides over rows k, threads sweep n; consecutive threads read consecutive slice elements
    for (uint32_t k = blockIdx.y; k < K; k += gridDim.y) {
        TileMemo memo;
        for (uint32_t n = blockIdx.x * blockDim.x + threadIdx.x; n < N; n += gridDim.x * blockDim.x)
            W[(size_t)k * N + n] = hashed[memo.index(hash, k, n)];
    }
}

__global__ void rz_hash_indices_kernel(int64_t *__restrict__ out, RzHash hash, uint32_t nk, uint32_t nn)
{
    uint64_t t = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < (uint64_t)nk * nn) out[t] = (int64_t)rz_tile_offset(hash, (uint32_t)(t / nn), (uint32_t)(t % nn));
}

template <int OP, int TB>
int launch_block(const RzLaunchCtx &c, const void *A, const void *B2, const float *hashed, const float *bias,
                 void *out, float *dH)
{
    constexpr int TC = 1024 / TB;
    const rz_problem *pb = c.pb;
    const uint32_t M = (uint32_t)pb->M, K = (uint32_t)pb->K, N = (uint32_t)pb->N;
    const uint32_t rows = (OP == 2) ? K : M, cols = (OP == 1) ? K : N;
    dim3 grid((cols + TB - 1) / TB, (rows + TB - 1) / TB, 1);
    uint32_t chunk = 0;
    if (OP == 2) {
        // split the batch so that small tile grids still fill the GPU
        uint64_t tiles = (uint64_t)grid.x * grid.y;
        uint32_t splits = (uint32_t)((2 * 148 + tiles - 1) / tiles);
        uint32_t max_splits = (M + 255) / 256;
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
        chunk = (M + splits - 1) / splits;
        chunk = (chunk + TC - 1) / TC * TC;
        splits = (M + chunk - 1) / chunk;
        grid.z = splits;
    }
    if (grid.y > 65535u || grid.z > 65535u) return RZ_ERR_SHAPE;
    const int relu = (pb->flags & RZ_FLAG_RELU) ? 1 : 0;
    if (pb->io_dtype == RZ_F32)
        rz_simt_kernel<OP, float, TB><<<grid, 256, 0, c.stream>>>((const float *)A, (const float *)B2, hashed, bias, out, dH,
                                                                 c.hash, M, K, N, pb->alpha, relu, chunk);
    else
        rz_simt_kernel<OP, __nv_bfloat16, TB><<<grid, 256, 0, c.stream>>>((const __nv_bfloat16 *)A, (const __nv_bfloat16 *)B2,
                                                                         hashed, bias, out, dH, c.hash, M, K, N, pb->alpha,
                                                                         relu, chunk);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "simt launch");
}

template <int OP>
int launch(const RzLaunchCtx &c, const void *A, const void *B2, const float *hashed, const float *bias,
           void *out, float *dH)
{
    // 128 x 128 blocks (8 x 8 outputs per thread: twice the flops per shared-memory byte) once they fill the GPU
    const rz_problem *pb = c.pb;
    const uint64_t rows = (OP == 2) ? pb->K : pb->M, cols = (OP == 1) ? pb->K : pb->N;
    const uint64_t big_tiles = ((rows + 127) / 128) * ((cols + 127) / 128);
    if (big_tiles >= 148) return launch_block<OP, 128>(c, A, B2, hashed, bias, out, dH);
    return launch_block<OP, 64>(c, A, B2, hashed, bias, out, dH);
}

}  // namespace

int rz_simt_forward(const RzLaunchCtx &c, const void *X, const float *hashed, const float *bias, void *Y)
{
    return launch<0>(c, X, nullptr, hashed, bias, Y, nullptr);
}

int rz_simt_backward_input(const RzLaunchCtx &c, const void *dY, const float *hashed, void *dX)
{
    return launch<1>(c, dY, nullptr, hashed, nullptr, dX, nullptr);
}

int rz_simt_backward_weight(const RzLaunchCtx &c, const void *X, const void *dY, float *dH)
{
    return launch<2>(c, X, dY, nullptr, nullptr, nullptr, dH);
}

int rz_simt_materialize(const RzLaunchCtx &c, const float *hashed, float *W)
{
    const uint32_t K = (uint32_t)c.pb->K, N = (uint32_t)c.pb->N;
    dim3 grid((N + 255) / 256, K < 65535u ? K : 65535u, 1);
    if (grid.x > 64) grid.x = 64;
    rz_materialize_kernel<<<grid, 256, 0, c.stream>>>(hashed, W, c.hash, K, N);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "materialize launch");
}

int rz_simt_hash_indices(const RzLaunchCtx &c, int64_t *out)
{
    const uint32_t nk = (uint32_t)((c.pb->K + c.pb->BK - 1) / c.pb->BK);
    const uint32_t nn = (uint32_t)((c.pb->N + c.pb->BN - 1) / c.pb->BN);
    uint64_t total = (uint64_t)nk * nn;
    rz_hash_indices_kernel<<<(unsigned)((total + 255) / 256), 256, 0, c.stream>>>(out, c.hash, nk, nn);
    rz_count_launch(1);
    return rz_record_cuda(cudaGetLastError(), "hash indices launch");
}
