/*
 * rzlinear_b200 - C ABI of the B200 (sm_100a) RzLinear ROBE-Z compressed-matmul kernels.
 *
 * The library replaces the kernel launchers of the reference's python/rz_linear package
 * (apd10/RzLinear).  Paths cited below are relative to that repository.
 *
 * Conventions
 *   - Every pointer is a plain device pointer (host pointer where the name says "host");
 *     the caller owns every buffer, the library allocates nothing the caller sees.
 *   - `stream` is a cudaStream_t passed as void*; all launches are asynchronous on it.
 *   - Matrices are contiguous row-major: X[M,K], Y[M,N], dY[M,N], dX[M,K]; the hashed array and
 *     its gradient are fp32 [H].
 *   - Return value: RZ_OK (0) or a negative rz_status; rz_status_string() names it.
 *   - Virtual weight: W[k,n] = hashed[ offset(k / BK, n / BN) + (k % BK) * BN + (n % BN) ].
 */
#ifndef RZLINEAR_B200_H
#define RZLINEAR_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum rz_status {
    RZ_OK = 0,
    RZ_ERR_NULL = -1,          /* a required pointer is NULL */
    RZ_ERR_SHAPE = -2,         /* a dimension is <= 0 or too large */
    RZ_ERR_HASH_RANGE = -3,    /* H <= BK*BN (the reference asserts H > BK*BN) */
    RZ_ERR_DTYPE = -4,         /* unknown io_dtype / precision combination */
    RZ_ERR_ALIGN = -5,         /* a pointer is not aligned as the kernels need (16 bytes) */
    RZ_ERR_HASH_PARAM = -6,    /* R[0] (the prime) <= 0, a negative R, or unknown hash mode */
    RZ_ERR_CUDA = -7,          /* a CUDA runtime/driver call failed (see rz_last_cuda_error) */
    RZ_ERR_PIPELINE = -8,      /* a device-side bounded wait gave up: reported by rz_device_status, and returned by
                                  every tensor-core launch on that device until rz_device_status has been called */
    RZ_ERR_UNSUPPORTED = -9,   /* the requested path cannot run this problem */
    RZ_ERR_TOO_LARGE = -10,    /* size exceeds a fixed capacity of the entry point */
    RZ_ERR_SCRATCH = -11       /* the scratch buffer passed is smaller than rz_shadow_bytes() of the problem */
};

enum rz_hash_mode {
    /* ((pk*R3 + pn*R2 + R1) mod R0) mod (H - BK*BN)
       python/rz_linear/impl/RzLinearIdx.py:70-71, python/tests/test_rz_linear.py:26-27 */
    RZ_HASH_SINGLE = 0,
    /* ((((pk*R3+pn*R2+R1) mod R0)*R0 + ((pk*R7+pn*R5+R4) mod R0)) mod (H - BK*BN))
       python/rz_linear/impl/RzLinearForward.py:316,349; RzLinearBackward.py:369,686,716 */
    RZ_HASH_TWO_LEVEL = 1
};

enum rz_dtype { RZ_F32 = 0, RZ_BF16 = 1 };

enum rz_precision {
    RZ_PREC_FP32 = 0,  /* fp32-grade arithmetic (reference: allow_tf32=False): split tf32 operands on the
                          tensor cores for fp32 data and tile-aligned shapes, fp32 FMA kernels otherwise */
    RZ_PREC_TF32 = 1,  /* tf32 tensor cores, fp32 accumulate (reference: allow_tf32=True); io fp32 */
    RZ_PREC_BF16 = 2   /* bf16 tensor cores, fp32 accumulate; io bf16, hashed array fp32 */
};

enum rz_flags {
    RZ_FLAG_ACCUMULATE_DH = 1,  /* backward_weight adds into dH instead of zeroing it first */
    RZ_FLAG_FORCE_SIMT = 2,     /* never take the tensor-core path */
    RZ_FLAG_RELU = 4            /* forward: Y = max(0, X.W*alpha + bias) */
};

enum rz_op { RZ_OP_FORWARD = 0, RZ_OP_BACKWARD_INPUT = 1, RZ_OP_BACKWARD_WEIGHT = 2 };
enum rz_path { RZ_PATH_SIMT = 0, RZ_PATH_TCGEN05 = 1 };

typedef struct rz_problem {
    int64_t M, K, N, H;   /* X[M,K], virtual W[K,N], hashed[H] */
    int32_t BK, BN;       /* hash tile: part of the definition of the virtual matrix */
    int32_t hash_mode;    /* enum rz_hash_mode */
    int32_t io_dtype;     /* enum rz_dtype of X, Y, dY, dX */
    int32_t precision;    /* enum rz_precision */
    int32_t flags;        /* enum rz_flags, or-ed */
    int64_t R[8];         /* random numbers, R[0] = the prime (python/rz_linear/RzLinear.py:68-74) */
    float alpha;          /* init_factor (RzLinearForward.py:357, RzLinearBackward.py:371,727) */
    int32_t sm_reserve;   /* SMs the persistent tensor-core kernels leave idle (0 = use every SM): room for a
                             collective or another kernel that should run beside them.  No reference counterpart. */
} rz_problem;

int rz_version(void);
const char *rz_status_string(int status);
/* Text of the last CUDA error seen by this thread's last failing call ("" if none). */
const char *rz_last_cuda_error(void);

/* Tile offsets on the host, out[cdiv(K,BK) * cdiv(N,BN)] row-major over (pk, pn).
   Replaces the index arithmetic of RzLinearIdx.py:62-71 / RzLinearForward.py:316. */
int rz_hash_indices_host(const rz_problem *pb, int64_t *out_host);

/* The same offsets computed on the device by the routine the kernels use (device pointer out). */
int rz_hash_indices_device(const rz_problem *pb, int64_t *out_dev, void *stream);

/* Which kernel family would run `op` for this problem: RZ_PATH_SIMT or RZ_PATH_TCGEN05 (>= 0),
   or a negative status if the problem is invalid. */
int rz_plan(const rz_problem *pb, int op);

/* Scratch ("shadow") memory the tensor-core forward / input-gradient kernels read instead of
   the fp32 hashed array: element-shifted copies in the compute type so that every tile slice
   starts on a 16-byte boundary of one copy, followed (small batches, ragged last waves, fp32
   precision) by an fp32 workspace for partial sums of split contractions, which those launches write.
   rz_shadow_bytes() is 0 when the problem takes the SIMT path; it depends on M, the precision and
   sm_reserve as well as on H, so size a buffer that serves several problems for the largest of them.
   The caller allocates `shadow` (256-byte aligned), and refreshes it whenever `hashed` changes
   (rz_shadow_refresh, or rz_sgd_step which does both). */
size_t rz_shadow_bytes(const rz_problem *pb);
int rz_shadow_refresh(const rz_problem *pb, const float *hashed, void *shadow, void *stream);

/* Y = (X . W_virtual) * alpha (+ bias[N], fp32, may be NULL) (+ ReLU with RZ_FLAG_RELU).
   Replaces rz_linear_forward_tl, python/rz_linear/impl/RzLinearForward.py:6-85, and the separate
   bias add of python/rz_linear/RzLinear.py:93-94.  `shadow` may be NULL only on the SIMT path;
   `shadow_bytes` is the size of that buffer: RZ_ERR_SCRATCH if it is below rz_shadow_bytes(pb). */
int rz_linear_forward(const rz_problem *pb, const void *X, const float *hashed, void *shadow,
                      size_t shadow_bytes, const float *bias, void *Y, void *stream);

/* Forward pass for callers that cannot supply scratch memory.  No counterpart in the reference.
   Same result as rz_linear_forward, but the shadow copies live in a fixed 16 MiB array inside the
   library instead of a caller-allocated buffer, and the call allocates no device memory.  Meant for
   hosts that have no way to allocate at this point: all of HBM already belongs to their own pool,
   they sit behind a binding that only passes pointers, or they cannot afford the device-wide stall an
   allocation may cause.  Limits: the shifted copies (8 x 2 bytes per element on the bf16 path, 4 x 4
   on the tf32 / fp32 paths, H rounded up to 64) must fit RZ_NOALLOC_SCRATCH_BYTES, i.e. H <= 2^20,
   else RZ_ERR_TOO_LARGE.  A split-contraction workspace that does not fit beside the copies is done
   without (whole contractions per block) - except for fp32 precision with a contraction longer than
   2048, which needs it and is refused when copies + workspace exceed the array.  The array is
   rewritten by every call and shared by all callers on a device, so calls that may overlap on the GPU
   race (order them on one stream or with events).  One-time set-up that belongs before any stream
   capture: the first call on each device resolves the array's address; like every tensor-core launch
   it also runs the per-thread / per-kernel-variant first-use steps listed in INTEGRATION.md, so warm
   up each shape you are going to capture. */
#define RZ_NOALLOC_SCRATCH_BYTES ((size_t)16 << 20)
int rz_linear_forward_noalloc(const rz_problem *pb, const void *X, const float *hashed,
                              const float *bias, void *Y, void *stream);

/* dX = (dY . W_virtual^T) * alpha.
   Replaces rz_linear_backward_input_grad_tl, python/rz_linear/impl/RzLinearBackward.py:374-449. */
int rz_linear_backward_input(const rz_problem *pb, const void *dY, const float *hashed,
                             void *shadow, size_t shadow_bytes, void *dX, void *stream);

/* dH[offset(pk,pn) + r*BN + c] += (X^T . dY)[pk*BK + r, pn*BN + c] * alpha; dH is zeroed first
   unless RZ_FLAG_ACCUMULATE_DH.  Replaces rz_linear_backward_weight_grad_tl,
   python/rz_linear/impl/RzLinearBackward.py:23-97. */
int rz_linear_backward_weight(const rz_problem *pb, const void *X, const void *dY, float *dH,
                              void *stream);

/* W[K,N] (fp32) = gather of the hashed slices.
   Replaces rz_linear_idx_tl, python/rz_linear/impl/RzLinearIdx.py:6-45. */
int rz_linear_materialize(const rz_problem *pb, const float *hashed, float *W, void *stream);

/* Backward-pass preparation for a layer whose bias add and ReLU were fused into rz_linear_forward, in one pass
   over the incoming gradient dY[M,N]: with Y != NULL (the layer's saved output) dYm = dY where Y > 0, else 0;
   with bias_grad != NULL, bias_grad[n] = sum over m of the (masked) gradient, fp32 [N], zeroed first.  dYm may be
   NULL when Y is NULL (bias gradient only).  Replaces the separate torch ops of the reference's module
   (python/rz_linear/RzLinear.py:93-94 adds the bias outside the kernel, so autograd sums it there). */
int rz_grad_prepare(const rz_problem *pb, const void *dY, const void *Y, void *dYm, float *bias_grad,
                    void *stream);

/* hashed -= lr * dH; when shadow != NULL the shifted copies are rewritten by the same kernel, in the same
   pass over the array (one launch).  No counterpart in the reference (its optimiser step is torch's);
   used by the data-parallel step. */
int rz_sgd_step(const rz_problem *pb, float *hashed, const float *dH, float lr, void *shadow,
                void *stream);

/* Heavy-ball variant: velocity = momentum * velocity + dH; hashed -= lr * velocity (velocity fp32 [H], caller-owned);
   the shadow copies are rewritten in the same pass when shadow != NULL.  No counterpart in the reference. */
int rz_sgd_momentum_step(const rz_problem *pb, float *hashed, const float *dH, float *velocity, float lr,
                         float momentum, void *shadow, void *stream);

/* Reads and clears the device-side status word (synchronises the device).  *out = RZ_OK or
   RZ_ERR_PIPELINE; *detail (may be NULL) receives the code of the wait that gave up.  A kernel whose wait
   gives up leaves partial results; the library notices without synchronising (a host-mapped copy of the
   word) and from then on every tensor-core launch on that device returns RZ_ERR_PIPELINE, until this call
   has acknowledged the failure. */
int rz_device_status(int *out, int *detail);

/* Failure-detection self-test (no counterpart in the reference): launches a one-thread kernel that waits
   on a barrier nothing completes, with the same bounded wait the tensor-core pipelines use.  After at
   most `limit_cycles` SM cycles (1 .. 2e9) the wait gives up and the kernel returns; rz_device_status()
   then reports RZ_ERR_PIPELINE with detail 6, and the context stays usable. */
int rz_selftest_bounded_wait(int64_t limit_cycles, void *stream);

/* Number of kernels this library has launched in this process (all threads). */
uint64_t rz_launch_count(void);

/* Re-reads the RZ_TC_* bring-up knobs from the environment (they are read once, at the first launch). */
void rz_reload_env(void);

#ifdef __cplusplus
}
#endif
#endif /* RZLINEAR_B200_H */
