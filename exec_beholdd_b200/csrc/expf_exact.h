// exp(x) for f32 computed the way the GNU C library's expf does (the algorithm published
// in Arm's optimized-routines and adopted by glibc 2.27+): reduce x*32/ln2 = k + r, look up
// 2^(k/32) in a 32-entry table, multiply by a cubic in r, all in double, then round once to
// f32. The reference's softmax calls the host libm's expf (Rust f32::exp), and the router's
// top-k ranks the resulting probabilities, so the device has to produce the same floats for
// its ranking to be the CPU's ranking. The same function is compiled for the host so that
// it can be compared with the host libm bit for bit (tests/test_expf_exact.py).
//
// Every operation is an individually rounded double multiply/add (no FMA contraction), so
// host and device agree exactly with each other.
#pragma once
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define BHD_HD __host__ __device__ __forceinline__
#else
#define BHD_HD static inline
#endif

#if defined(__CUDA_ARCH__)
#define BHD_DMUL(a, b) __dmul_rn((a), (b))
#define BHD_DADD(a, b) __dadd_rn((a), (b))
#else
#define BHD_DMUL(a, b) ((a) * (b))
#define BHD_DADD(a, b) ((a) + (b))
#endif

#if defined(__CUDA_ARCH__)
__device__ __constant__
#else
static const
#endif
uint64_t bhd_exp2_tab32[32] = {
    0x3ff0000000000000ull, 0x3fefd9b0d3158574ull, 0x3fefb5586cf9890full, 0x3fef9301d0125b51ull,
    0x3fef72b83c7d517bull, 0x3fef54873168b9aaull, 0x3fef387a6e756238ull, 0x3fef1e9df51fdee1ull,
    0x3fef06fe0a31b715ull, 0x3feef1a7373aa9cbull, 0x3feedea64c123422ull, 0x3feece086061892dull,
    0x3feebfdad5362a27ull, 0x3feeb42b569d4f82ull, 0x3feeab07dd485429ull, 0x3feea47eb03a5585ull,
    0x3feea09e667f3bcdull, 0x3fee9f75e8ec5f74ull, 0x3feea11473eb0187ull, 0x3feea589994cce13ull,
    0x3feeace5422aa0dbull, 0x3feeb737b0cdc5e5ull, 0x3feec49182a3f090ull, 0x3feed503b23e255dull,
    0x3feee89f995ad3adull, 0x3feeff76f2fb5e47ull, 0x3fef199bdd85529cull, 0x3fef3720dcef9069ull,
    0x3fef5818dcfba487ull, 0x3fef7c97337b9b5full, 0x3fefa4afa2a490daull, 0x3fefd0765b6e4540ull,
};

BHD_HD double bhd_u64_as_double(uint64_t u) {
#if defined(__CUDA_ARCH__)
    return __longlong_as_double((long long)u);
#else
    double d;
    memcpy(&d, &u, 8);
    return d;
#endif
}

BHD_HD uint64_t bhd_double_as_u64(double d) {
#if defined(__CUDA_ARCH__)
    return (uint64_t)__double_as_longlong(d);
#else
    uint64_t u;
    memcpy(&u, &d, 8);
    return u;
#endif
}

// Valid for finite x <= 0 down to the underflow threshold and for moderate positive x;
// softmax only ever passes x = v - max <= 0. Below about -103.97 the result is 0.
BHD_HD float bhd_expf_exact(float x) {
    if (x < -103.972076f) return 0.0f;  // x < log(2^-150): rounds to +0
    const double inv_ln2_n = 0x1.71547652b82fep+0 * 32.0;
    const double shift = 0x1.8p+52;
    const double c0 = 0x1.c6af84b912394p-5 / 32.0 / 32.0 / 32.0;
    const double c1 = 0x1.ebfce50fac4f3p-3 / 32.0 / 32.0;
    const double c2 = 0x1.62e42ff0c52d6p-1 / 32.0;
    const double xd = (double)x;
    double z = BHD_DMUL(inv_ln2_n, xd);
    double kd = BHD_DADD(z, shift);
    const uint64_t ki = bhd_double_as_u64(kd);
    kd = BHD_DADD(kd, -shift);
    const double r = BHD_DADD(z, -kd);
    uint64_t t = bhd_exp2_tab32[ki & 31];
    t += ki << (52 - 5);
    const double s = bhd_u64_as_double(t);
    z = BHD_DADD(BHD_DMUL(c0, r), c1);
    const double r2 = BHD_DMUL(r, r);
    double y = BHD_DADD(BHD_DMUL(c2, r), 1.0);
    y = BHD_DADD(BHD_DMUL(z, r2), y);
    y = BHD_DMUL(y, s);
    return (float)y;
}
