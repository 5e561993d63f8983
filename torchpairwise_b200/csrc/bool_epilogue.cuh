// Contingency-table epilogue of the boolean metrics, shared by the popcount kernels (bool_popcount.cu) and the
// tensor-core count kernel (bool_tcgen05.cu): from the exact integers n11 = |x & y|, |x|, |y| and D to the requested
// metric with the float32 operation order of the reference's tensor compositions (OPS/pairwise_metrics.cpp:206-399),
// every *, +, -, / rounded separately, so that the float32 output is bit-identical whichever kernel counted.
#pragma once
#include "common.cuh"

namespace tpw {
namespace {

// int -> float for 0 <= v < 2^23.  The conversion instruction issues at a quarter of the arithmetic rate; placing
// the integer in the mantissa of 2^23 and subtracting 2^23 gives the same exact value with one logic operation and
// one add.  FAST is set by the few-words kernel, where the conversions are a large share of the work per pair.
template <bool FAST>
__device__ __forceinline__ float count_to_float(int v) {
    return FAST ? __int_as_float(0x4B000000 | v) - 8388608.f : (float)v;
}

// INV: -1 = decide per call from inv_d, 1 = D is a power of two and inv_d its reciprocal, 0 = divide.  A caller that
// knows which holds for a whole tile passes it as a constant: decided per element, the division sequence is
// if-converted and executed next to the multiplication for every element.
template <bool FAST = false, int INV = -1>
__device__ __forceinline__ float bool_epilogue(int metric, int n11, int a, int b, int D, float inv_d) {
    const int nxor_i = a + b - 2 * n11;
    const int nor_i = a + b - n11;
    const float fand = count_to_float<FAST>(n11), fxor = count_to_float<FAST>(nxor_i), f_or = count_to_float<FAST>(nor_i);
    const float feq = count_to_float<FAST>(D - nxor_i), fD = count_to_float<FAST>(D);
    switch (metric) {
        case TPW_BOOL_AND_SUM: return fand;
        case TPW_BOOL_OR_SUM: return f_or;
        case TPW_BOOL_XOR_SUM:
        case TPW_BOOL_NE_SUM: return fxor;
        case TPW_BOOL_EQ_SUM: return feq;
        // dividing by a power of two is exact, and so is multiplying by its reciprocal
        case TPW_BOOL_EQ_MEAN:
            if (INV == 1) return __fmul_rn(feq, inv_d);
            if (INV == 0) return __fdiv_rn(feq, fD);
            return inv_d != 0.f ? __fmul_rn(feq, inv_d) : __fdiv_rn(feq, fD);
        case TPW_BOOL_NE_MEAN:
            if (INV == 1) return __fmul_rn(fxor, inv_d);
            if (INV == 0) return __fdiv_rn(fxor, fD);
            return inv_d != 0.f ? __fmul_rn(fxor, inv_d) : __fdiv_rn(fxor, fD);
        case TPW_BOOL_JACCARD: return f_or != 0.f ? __fdiv_rn(fxor, f_or) : 0.f;
        case TPW_BOOL_KULSINSKI: return __fdiv_rn(__fadd_rn(__fsub_rn(fxor, fand), fD), __fadd_rn(fxor, fD));
        case TPW_BOOL_KULCZYNSKI1: return __fdiv_rn(fand, fxor);
        case TPW_BOOL_YULE: {
            const float half_r = __fmul_rn(count_to_float<FAST>(a - n11), count_to_float<FAST>(b - n11));
            const float den = __fadd_rn(__fmul_rn(fand, count_to_float<FAST>(D - nor_i)), half_r);
            return den != 0.f ? __fdiv_rn(__fmul_rn(2.f, half_r), den) : 0.f;
        }
        case TPW_BOOL_DICE: return __fdiv_rn(fxor, __fadd_rn(__fmul_rn(2.f, fand), fxor));
        case TPW_BOOL_ROGERSTANIMOTO:
        case TPW_BOOL_SOKALMICHENER: {
            const float r2 = __fmul_rn(2.f, fxor);
            return __fdiv_rn(r2, __fadd_rn(feq, r2));
        }
        case TPW_BOOL_RUSSELLRAO: return __fdiv_rn(__fsub_rn(fD, fand), fD);
        case TPW_BOOL_SOKALSNEATH: {
            const float r2 = __fmul_rn(2.f, fxor);
            return __fdiv_rn(r2, __fadd_rn(fand, r2));
        }
        default: return 0.f;
    }
}

} // namespace
} // namespace tpw
