// ROBE-Z tile hash shared by the host entry points and every kernel.
//
// offset(pk, pn) is the start of tile (pk, pn)'s contiguous BK*BN slice in the hashed array.
// Single level  : ((pk*R3 + pn*R2 + R1) mod R0) mod (H - BK*BN)
//                 (reference: python/rz_linear/impl/RzLinearIdx.py:70-71)
// Two level     : ((((pk*R3+pn*R2+R1) mod R0)*R0 + ((pk*R7+pn*R5+R4) mod R0)) mod (H - BK*BN))
//                 (reference: python/rz_linear/impl/RzLinearForward.py:316,349)
// All operands are non-negative; with every R < 2^31 and tile coordinates < 2^31 every
// intermediate fits in 64 unsigned bits (two level: a*R0 + b < 2^62).
//
// The two moduli are fixed per call, so `v mod d` is computed exactly without a division:
// with m = floor((2^64 - 1) / d), q = floor(v * m / 2^64) is floor(v / d) or one less, hence
// r = v - q*d lies in [0, 2d) and one conditional subtraction finishes it.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define RZ_HD __host__ __device__ __forceinline__
#else
#define RZ_HD inline
#endif

struct RzHash {
    uint64_t R0, R1, R2, R3, R4, R5, R7;
    uint64_t range;    // H - BK*BN
    uint64_t m_R0;     // floor((2^64-1) / R0)
    uint64_t m_range;  // floor((2^64-1) / range)
    int32_t BK, BN;
    int32_t two_level;
    int32_t pad;
};

RZ_HD uint64_t rz_mulhi64(uint64_t a, uint64_t b)
{
#if defined(__CUDA_ARCH__)
    return __umul64hi(a, b);
#else
    return (uint64_t)(((unsigned __int128)a * (unsigned __int128)b) >> 64);
#endif
}

RZ_HD uint64_t rz_fastmod(uint64_t v, uint64_t d, uint64_t m)
{
    uint64_t r = v - rz_mulhi64(v, m) * d;
    return r >= d ? r - d : r;
}

inline void rz_hash_finish(RzHash &h)
{
    h.m_R0 = ~(uint64_t)0 / h.R0;
    h.m_range = ~(uint64_t)0 / h.range;
}

RZ_HD uint64_t rz_tile_offset(const RzHash &h, uint32_t pk, uint32_t pn)
{
    uint64_t a = rz_fastmod((uint64_t)pk * h.R3 + (uint64_t)pn * h.R2 + h.R1, h.R0, h.m_R0);
    if (h.two_level) {
        uint64_t b = rz_fastmod((uint64_t)pk * h.R7 + (uint64_t)pn * h.R5 + h.R4, h.R0, h.m_R0);
        a = a * h.R0 + b;
    }
    return rz_fastmod(a, h.range, h.m_range);
}
