// Pieces shared by the backward kernels of the pairwise L_p reductions: the odd functions phi of the coordinate
// difference, the coefficient modes, and the packed two-lane float32 arithmetic.
#pragma once
#include "common.cuh"
#include "packed_f32x2.cuh"

#include <math.h>

namespace tpw {
namespace {

enum Phi {
    PHI_SGN = 0,    // sgn(d)
    PHI_D = 1,      // d
    PHI_DABS = 2,   // d*|d|
    PHI_SGNPOW = 3, // sgn(d)*|d|^q
    PHI_ABSPOW = 4, // |d|^q
    PHI_Y = 5,      // the streamed operand itself (plain contraction)
    PHI_SGN_EQ = 6, // sgn(d) where |d| equals the auxiliary value, else 0
    // derivatives of symmetric two-argument terms with respect to the register-resident operand x
    PHI_CANBERRA = 7, // sgn(d)/n - sgn(x)|d|/n^2, n = |x| + |y| (0 where n == 0)
    PHI_CHI2 = 8,     // t^2 - 2t, t = d/(x + y) (0 where x + y == 0): d/dx of -(x - y)^2/(x + y)
    PHI_JS = 9        // log(2x/(x + y)) where x > 0, else -y/(x + y) (0 where x + y == 0)
};

enum CoefMode { COEF_G = 0, COEF_DIV_O = 1, COEF_DIV_O2 = 2, COEF_DIV_POW = 3, COEF_MUL = 4, COEF_ZERO_WHERE_O0 = 5 };

template <typename T> __device__ __forceinline__ void load4(T *dst, const T *src);
template <> __device__ __forceinline__ void load4<float>(float *dst, const float *src) {
    float4 v = *reinterpret_cast<const float4 *>(src);
    dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
}
template <> __device__ __forceinline__ void load4<double>(double *dst, const double *src) {
    double2 a = *reinterpret_cast<const double2 *>(src);
    double2 b = *reinterpret_cast<const double2 *>(src + 2);
    dst[0] = a.x; dst[1] = a.y; dst[2] = b.x; dst[3] = b.y;
}

__device__ __forceinline__ float b_abs(float v) { return fabsf(v); }
__device__ __forceinline__ double b_abs(double v) { return fabs(v); }
__device__ __forceinline__ float b_fma(float a, float b, float c) { return fmaf(a, b, c); }
__device__ __forceinline__ double b_fma(double a, double b, double c) { return fma(a, b, c); }
__device__ __forceinline__ float b_powabs(float a, float q) { return a == 0.f ? 0.f : exp2f(q * __log2f(a)); }
__device__ __forceinline__ double b_powabs(double a, double q) { return a == 0.0 ? 0.0 : pow(a, q); }
__device__ __forceinline__ float b_copysign(float a, float s) { return copysignf(a, s); }
__device__ __forceinline__ double b_copysign(double a, double s) { return copysign(a, s); }
// c * sgn(d) for d != 0: flip c's sign bit with d's (one logic operation)
__device__ __forceinline__ float b_copysign_of(float c, float d) {
    return __int_as_float(__float_as_int(c) ^ (__float_as_int(d) & 0x80000000));
}
__device__ __forceinline__ double b_copysign_of(double c, double d) { return d < 0.0 ? -c : c; }
// g / v for the coefficient tile: an approximate reciprocal (2 ulp) is far inside the fp32 parity
// tolerance and an order of magnitude cheaper than the IEEE sequence; fp64 keeps the exact divide
__device__ __forceinline__ float b_div(float g, float v) { return __fdividef(g, v); }
__device__ __forceinline__ double b_div(double g, double v) { return g / v; }
__device__ __forceinline__ float b_log(float v) {   // flush-to-zero MUFU logarithm; callers pass normal numbers or guard the result
    float l;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(fmaxf(v, 1.17549435e-38f)));
    return 0.693147181f * l;
}
__device__ __forceinline__ double b_log(double v) { return log(v); }
__device__ __forceinline__ float b_pow(float a, double q) { return powf(a, (float)q); }
__device__ __forceinline__ double b_pow(double a, double q) { return pow(a, q); }


template <typename T, int PHI> struct PackedPhi {
    static constexpr bool value = false;
};
template <> struct PackedPhi<float, PHI_DABS> { static constexpr bool value = true; };
template <> struct PackedPhi<float, PHI_D> { static constexpr bool value = true; };
template <> struct PackedPhi<float, PHI_Y> { static constexpr bool value = true; };

// acc += c * phi(x - y) on two adjacent features: the same operations, in the same order and rounding, as the scalar form
template <int PHI>
__device__ __forceinline__ f32x2 bwd_accumulate2(f32x2 acc, f32x2 x, f32x2 y, f32x2 c) {
    if (PHI == PHI_Y) return fma2(c, y, acc);
    const f32x2 d = sub2(x, y);
    if (PHI == PHI_D) return fma2(c, d, acc);
    // d |d| lane by lane: the scalar multiply takes |.| as an operand modifier, a packed one would need two logic
    // operations for it, and those occupy the same lanes as the arithmetic
    float lo, hi;
    unpack2(d, lo, hi);
    return fma2(c, pack2(lo * fabsf(lo), hi * fabsf(hi)), acc);
}

// acc += c * phi(x - y)
template <int PHI, typename T>
__device__ __forceinline__ void bwd_accumulate(T &acc, T x, T y, T c, T o, T q, int pspec) {
    if (PHI == PHI_Y) {
        acc = b_fma(c, y, acc);
        return;
    }
    if (PHI == PHI_CANBERRA) {
        // r (sgn(d) - sgn(x) |d| r), branch-free: a zero denominator selects r = 0, and the two signs are
        // copied onto r and |d| r^2 (zero where d, respectively x, is zero)
        const T n = b_abs(x) + b_abs(y), d = x - y;
        const T r = rcp_or_zero(n);
        const T t1 = d != T(0) ? b_copysign(r, d) : T(0);
        const T t2 = x != T(0) ? b_copysign(b_abs(d) * r * r, x) : T(0);
        acc = b_fma(c, t1 - t2, acc);
        return;
    }
    if (PHI == PHI_CHI2) {
        const T n = x + y;
        const T r = rcp_or_zero(n);
        const T t = (x - y) * r;
        acc = b_fma(c, t * (t - T(2)), acc);
        return;
    }
    if (PHI == PHI_JS) {
        // d/dx of x log(x/m) + y log(y/m), m = (x + y)/2, is log(x/m); the reference's branches
        // (OPS/cpu/sqjensenshannon_kernel.cpp:98-112) add up to log 2 at y == 0 and to -1 at x == 0 < y
        const T r = rcp_or_zero(x + y);
        // x/m = 1 + t, t = (x - y)/(x + y): exactly 1 for equal entries; where x is much smaller than y
        // the sum 1 + t cancels, and the quotient 2x/(x + y) keeps the relative accuracy the logarithm needs
        const T t = (x - y) * r;
        const T ratio = b_abs(t) < T(0.5) ? T(1) + t : T(2) * x * r;
        acc = b_fma(c, x > T(0) ? b_log(ratio) : -y * r, acc);
        return;
    }
    T d = x - y;
    if (PHI == PHI_D) {
        acc = b_fma(c, d, acc);
    } else if (PHI == PHI_DABS) {
        acc = b_fma(c, d * b_abs(d), acc);
    } else if (PHI == PHI_SGN) {
        if (d != T(0)) acc += b_copysign_of(c, d);
    } else if (PHI == PHI_SGNPOW) {
        acc = b_fma(c, b_copysign(pow_abs_spec(b_abs(d), q, pspec), d), acc);
    } else if (PHI == PHI_ABSPOW) {
        acc = b_fma(c, pow_abs_spec(b_abs(d), q, pspec), acc);
    } else if (PHI == PHI_SGN_EQ) {
        // c is already zero where o == 0, and |d| == o > 0 implies d != 0
        if (b_abs(d) == o) acc += b_copysign_of(c, d);
    }
}

// coefficient of a pair from the upstream gradient g and the auxiliary value o
template <typename T>
__device__ __forceinline__ T bwd_coefficient(int mode, T g, T o, double q) {
    switch (mode) {
        case COEF_DIV_O: return o == T(0) ? T(0) : b_div(g, o);
        case COEF_DIV_O2: return o == T(0) ? T(0) : b_div(g, o * o);
        case COEF_DIV_POW: return o == T(0) ? T(0) : b_div(g, b_pow(o, q));
        case COEF_MUL: return g * o;
        case COEF_ZERO_WHERE_O0: return o == T(0) ? T(0) : g;
        default: return g;
    }
}

} // namespace
} // namespace tpw
