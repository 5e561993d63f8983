// Register-blocked CUDA-core tile kernel for every "combine two features, reduce over D" forward
// of the pairwise path: the L_p family (|d|, |d|^2, |d|^3, |d|^p, max, min, each optionally
// weighted), the fp32/fp64 cross-term metrics (dot product with fused cosine / correlation /
// squared-norm epilogues) and the element-compare counts of non-boolean hamming.
//
// Layout.  A CTA of 256 threads owns a TILE x TILE block of outputs (TILE = 16*R, R = 8 for
// 4-byte types, 4 for 8-byte types).  Operand tiles are staged in shared memory exactly as the
// TMA engine writes a {128-byte, TILE-row} box with the 128-byte swizzle: row r lives at
// r*128 and its 16-byte chunk c at position c ^ (r & 7).  Thread (ti, tj) = (tid/16, tid%16)
// owns rows {ti + 16 r} of x1 and rows {tj + 16 r} of x2, so that within a quarter warp the
// eight x2 rows hit eight different chunk positions (conflict-free 128-bit shared loads) while
// the x1 address is a broadcast.  Aligned inputs are fed by TMA through a 3-stage mbarrier
// ring issued by one thread; anything else (feature count not a multiple of 16 bytes, odd base
// address) takes a guarded plain-load path into the same layout.
#include "lp_forward_kernel.cuh"

using namespace tpw;

extern "C" int tpw_lp_forward(int dtype, const void *x1, const void *x2, const void *w, void *out,
                              int64_t B, int64_t N1, int64_t N2, int64_t D,
                              double p, double out_exponent, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_lp_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_lp_forward: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && out, "tpw_lp_forward: NULL pointer");
    TPW_CHECK_ARG(D > 0, "tpw_lp_forward: D must be positive");
    TPW_CHECK_ARG(p > 0 || (isinf(p) && p < 0), "tpw_lp_forward: p must be positive or -inf (got %g)", p);
    TPW_CHECK_ARG(!isnan(p) && !isnan(out_exponent), "tpw_lp_forward: NaN exponent");
    FwdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2; P.w = w; P.out = out;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // few features: the streaming kernel of lp_small_d.cu, bound by the output write instead of tile set-up
    if (dtype == TPW_F32 && !w && lp_small_d_eligible(N1, N2, D, p)) return lp_small_d_forward(x1, x2, out, B, N1, N2, D, p, out_exponent, s);
    return dtype == TPW_F32 ? lp_forward_typed<float>(P, p, out_exponent, s)
                            : lp_forward_typed<double>(P, p, out_exponent, s);
}

extern "C" int tpw_dot_metric_forward_simt(int dtype, int epilogue, const void *x1, const void *x2, void *out,
                                           int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_dot_metric_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(epilogue >= TPW_DOT_LINEAR && epilogue <= TPW_DOT_EUCLIDEAN, "tpw_dot_metric_forward: bad epilogue %d", epilogue);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_dot_metric_forward: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && out, "tpw_dot_metric_forward: NULL pointer");
    TPW_CHECK_ARG(D > 0, "tpw_dot_metric_forward: D must be positive");
    FwdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2; P.out = out;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.epilogue = epilogue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == TPW_F32 ? launch_forward<float, float, K_DOT, false>(P, s)
                            : launch_forward<double, double, K_DOT, false>(P, s);
}

extern "C" int tpw_cmp_reduce_forward(int dtype, int op, int reduction, const void *x1, const void *x2, float *out,
                                      int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype >= TPW_F32 && dtype <= TPW_I64, "tpw_cmp_reduce_forward: bad dtype %d", dtype);
    TPW_CHECK_ARG(op == TPW_CMP_EQ || op == TPW_CMP_NE, "tpw_cmp_reduce_forward: bad op %d", op);
    TPW_CHECK_ARG(reduction == TPW_RED_SUM || reduction == TPW_RED_MEAN, "tpw_cmp_reduce_forward: bad reduction %d", reduction);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_cmp_reduce_forward: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && out, "tpw_cmp_reduce_forward: NULL pointer");
    TPW_CHECK_ARG(D > 0 && D <= (1 << 24), "tpw_cmp_reduce_forward: D must be in [1, 2^24] for exact float counts");
    FwdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2; P.out = out;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.epilogue = (op == TPW_CMP_EQ ? 1 : 0) | (reduction == TPW_RED_MEAN ? 2 : 0);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TPW_F32: return launch_forward<float, float, K_NE, false>(P, s);
        case TPW_F64: return launch_forward<double, float, K_NE, false>(P, s);
        case TPW_I32: return launch_forward<float, float, K_NE_BITS, false>(P, s);
        default: return launch_forward<double, float, K_NE_BITS, false>(P, s);
    }
}

extern "C" int tpw_pair_sum_forward(int dtype, int metric, const void *x1, const void *x2, void *out,
                                    int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_pair_sum_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(metric == TPW_PAIR_CANBERRA || metric == TPW_PAIR_ADDITIVE_CHI2, "tpw_pair_sum_forward: bad metric %d", metric);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_pair_sum_forward: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && out, "tpw_pair_sum_forward: NULL pointer");
    TPW_CHECK_ARG(D > 0, "tpw_pair_sum_forward: D must be positive");
    FwdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2; P.out = out;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (metric == TPW_PAIR_CANBERRA)
        return dtype == TPW_F32 ? launch_forward<float, float, K_CANBERRA, false>(P, s) : launch_forward<double, double, K_CANBERRA, false>(P, s);
    return dtype == TPW_F32 ? launch_forward<float, float, K_CHI2, false>(P, s) : launch_forward<double, double, K_CHI2, false>(P, s);
}

extern "C" int tpw_jensenshannon_forward(int dtype, const void *x1, const void *x2, void *out,
                                         int64_t B, int64_t N1, int64_t N2, int64_t D, double scale, int take_sqrt,
                                         tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_jensenshannon_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_jensenshannon_forward: negative size");
    TPW_CHECK_ARG(take_sqrt == 0 || take_sqrt == 1, "tpw_jensenshannon_forward: take_sqrt must be 0 or 1");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && out, "tpw_jensenshannon_forward: NULL pointer");
    TPW_CHECK_ARG(D > 0, "tpw_jensenshannon_forward: D must be positive");
    FwdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2; P.out = out;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.root_mode = take_sqrt;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32) {
        P.scale = scale * 0.69314718055994530942;   // the float kernel sums in units of log 2
        return launch_forward<float, float, K_JS, false>(P, s);
    }
    P.scale = scale;
    return launch_forward<double, double, K_JS, false>(P, s);
}
