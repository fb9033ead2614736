// Elementary functions with one definition for host and device.
//
// The decoder's support ops need exp, log, sin and cos.  A CPU libm and the CUDA math library round
// differently in the last place, which is enough to change a greedy token now and then.  These versions
// use only IEEE-exact operations (add, multiply, fused multiply-add, conversions), each written out
// explicitly, so that a host compiler and nvcc produce bit-identical results; their error is about one
// unit in the last place, the same class as either library.  They are the arithmetic of the CUDA support
// kernels, and the CPU oracle's "device order" mode includes this header to reproduce them.
#pragma once
#include <math.h>
#include <stdint.h>
#include <string.h>

#if defined(__CUDACC__)
#define IT_HD __host__ __device__ __forceinline__
#else
#define IT_HD static inline
#endif
// The longer functions (IEEE division and square root expand to dozens of instructions on the device, the elementary
// functions to more) can be compiled as calls instead of inline copies: a translation unit that defines IT_MATH_OUTLINE
// before including this header gets one copy of each.  The operations, and so the results, are the same either way.
#if defined(__CUDACC__) && defined(IT_MATH_OUTLINE)
#define IT_HD_BIG static __host__ __device__ __noinline__
#else
#define IT_HD_BIG IT_HD
#endif

IT_HD float it_fma(float a, float b, float c) {
#if defined(__CUDA_ARCH__)
    return __fmaf_rn(a, b, c);
#else
    return fmaf(a, b, c);
#endif
}
IT_HD float it_mul(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fmul_rn(a, b);
#else
    volatile float r = a * b; return r;   // the oracle is built without contraction; volatile keeps it that way anywhere
#endif
}
IT_HD float it_add(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fadd_rn(a, b);
#else
    volatile float r = a + b; return r;
#endif
}
IT_HD float it_sub(float a, float b) { return it_add(a, -b); }
IT_HD_BIG float it_div(float a, float b) {
#if defined(__CUDA_ARCH__)
    return __fdiv_rn(a, b);
#else
    volatile float r = a / b; return r;
#endif
}
IT_HD_BIG float it_sqrt(float a) {
#if defined(__CUDA_ARCH__)
    return __fsqrt_rn(a);
#else
    return sqrtf(a);
#endif
}
IT_HD float it_bits_to_float(uint32_t u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f; memcpy(&f, &u, 4); return f;
#endif
}
IT_HD uint32_t it_float_to_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    uint32_t u; memcpy(&u, &f, 4); return u;
#endif
}

// exp(x).  n = round(x / ln 2), r = x - n ln 2 in two pieces, degree-6 polynomial, exact scaling by 2^n.
IT_HD_BIG float it_expf(float x) {
    if (!(x == x)) return x;
    if (x > 88.72283935546875f) return it_bits_to_float(0x7f800000u);
    if (x < -103.97208404541015625f) return 0.0f;
    const float n = rintf(it_mul(x, 1.44269502162933349609375f));
    float r = it_fma(n, -0.693145751953125f, x);
    r = it_fma(n, -1.42860682030941723212e-6f, r);
    float p = 1.9875691500e-4f;
    p = it_fma(p, r, 1.3981999507e-3f);
    p = it_fma(p, r, 8.3334519073e-3f);
    p = it_fma(p, r, 4.1665795894e-2f);
    p = it_fma(p, r, 1.6666665459e-1f);
    p = it_fma(p, r, 5.0000001201e-1f);
    p = it_fma(it_mul(p, r), r, r);
    p = it_add(p, 1.0f);
    const int ni = (int)n, n1 = ni / 2, n2 = ni - n1;    // two exact power-of-two factors keep subnormal results right
    const float s1 = it_bits_to_float((uint32_t)(n1 + 127) << 23), s2 = it_bits_to_float((uint32_t)(n2 + 127) << 23);
    return it_mul(it_mul(p, s1), s2);
}

// log(x) for finite x > 0 (normal numbers): x = m 2^e with m in [sqrt(1/2), sqrt(2)), polynomial in m - 1.
IT_HD_BIG float it_logf(float x) {
    uint32_t u = it_float_to_bits(x);
    int e = (int)(u >> 23) - 126;
    float m = it_bits_to_float((u & 0x007fffffu) | 0x3f000000u);   // m in [0.5, 1)
    if (m < 0.707106781186547524f) { e -= 1; m = it_sub(it_add(m, m), 1.0f); } else { m = it_sub(m, 1.0f); }
    const float z = it_mul(m, m);
    float p = 7.0376836292e-2f;
    p = it_fma(p, m, -1.1514610310e-1f);
    p = it_fma(p, m, 1.1676998740e-1f);
    p = it_fma(p, m, -1.2420140846e-1f);
    p = it_fma(p, m, 1.4249322787e-1f);
    p = it_fma(p, m, -1.6668057665e-1f);
    p = it_fma(p, m, 2.0000714765e-1f);
    p = it_fma(p, m, -2.4999993993e-1f);
    p = it_fma(p, m, 3.3333331174e-1f);
    float y = it_mul(it_mul(p, m), z);
    const float fe = (float)e;
    y = it_fma(fe, -2.12194440e-4f, y);
    y = it_fma(-0.5f, z, y);
    float r = it_add(m, y);
    r = it_fma(fe, 0.693359375f, r);
    return r;
}

// sin and cos of x for |x| up to about 1e5 (rope angles are position * scale <= context length).
IT_HD_BIG void it_sincosf(float x, float* s, float* c) {
    const float k = rintf(it_mul(x, 0.636619772367581343f));          // nearest multiple of pi/2
    float r = it_fma(k, -1.5703125f, x);                              // pi/2 in three pieces
    r = it_fma(k, -4.837512969970703125e-4f, r);
    r = it_fma(k, -7.54978995489188216e-8f, r);
    const float z = it_mul(r, r);
    float ps = -1.9515295891e-4f;
    ps = it_fma(ps, z, 8.3321608736e-3f);
    ps = it_fma(ps, z, -1.6666654611e-1f);
    const float sn = it_fma(it_mul(ps, z), r, r);
    float pc = 2.443315711809948e-5f;
    pc = it_fma(pc, z, -1.388731625493765e-3f);
    pc = it_fma(pc, z, 4.166664568298827e-2f);
    const float cs = it_add(it_fma(it_mul(pc, z), z, it_mul(-0.5f, z)), 1.0f);
    const int q = (int)k & 3;
    const float ss = (q & 1) ? cs : sn, cc = (q & 1) ? sn : cs;
    *s = (q & 2) ? -ss : ss;
    *c = ((q + 1) & 2) ? -cc : cc;
}

IT_HD float it_silu(float x) { return it_div(x, it_add(1.0f, it_expf(-x))); }          // x / (1 + exp(-x))
IT_HD float it_sigmoid(float x) { return it_div(1.0f, it_add(1.0f, it_expf(-x))); }    // 1 / (1 + exp(-x))
IT_HD float it_softplus(float x) { return x > 20.0f ? x : it_logf(it_add(1.0f, it_expf(x))); }
