// Fused epilogues of the CUDA-core forward tile kernel: the streaming row minimum and the radius
// mask.  Same tile, staging and accumulation as the stored-tile kernels; only what happens to a
// finished 128 x 128 tile differs, chosen at compile time.  Unweighted distances only.
#include "lp_forward_kernel.cuh"

namespace tpw {
namespace {

// keys -> (smallest distance, its x2 row); a row that saw no x2 row keeps +inf and index -1.
__global__ void rowmin_finish_kernel(const unsigned long long *__restrict__ keys, float *__restrict__ min_out,
                                     long long *__restrict__ arg_out, long long n) {
    const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t >= n) return;
    const unsigned long long key = keys[t];
    const bool none = key == ~0ull;
    if (min_out) min_out[t] = none ? __int_as_float(0x7f800000) : __uint_as_float((uint32_t)(key >> 32));
    if (arg_out) arg_out[t] = none ? -1ll : (long long)(uint32_t)key;
}

} // namespace
} // namespace tpw

using namespace tpw;

extern "C" int64_t tpw_lp_rowmin_scratch_bytes(int64_t B, int64_t N1) {
    if (B <= 0 || N1 <= 0) return 0;
    return B * N1 * (int64_t)sizeof(unsigned long long);
}

extern "C" int tpw_lp_rowmin_forward(int dtype, const void *x1, const void *x2, const void *w,
                                     float *min_out, int64_t *arg_out, void *scratch,
                                     int64_t B, int64_t N1, int64_t N2, int64_t D,
                                     double p, double out_exponent, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32, "tpw_lp_rowmin_forward: dtype must be TPW_F32 (the key packs a 32-bit distance)");
    TPW_CHECK_ARG(w == nullptr, "tpw_lp_rowmin_forward: weighted distances are not built for this epilogue (w must be NULL)");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_lp_rowmin_forward: negative size");
    if (B == 0 || N1 == 0) return TPW_OK;
    TPW_CHECK_ARG(scratch != nullptr && (min_out || arg_out), "tpw_lp_rowmin_forward: NULL pointer");
    TPW_CHECK_ARG(p > 0 && !isnan(p) && !isnan(out_exponent), "tpw_lp_rowmin_forward: p must be positive (got %g)", p);
    TPW_CHECK_ARG(N2 < (1ll << 32), "tpw_lp_rowmin_forward: N2 must fit 32 bits");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long n = B * N1;
    TPW_CUDA_OK(cudaMemsetAsync(scratch, 0xFF, (size_t)n * sizeof(unsigned long long), s));
    if (N2 > 0) {
        TPW_CHECK_ARG(x1 && x2, "tpw_lp_rowmin_forward: NULL pointer");
        TPW_CHECK_ARG(D > 0, "tpw_lp_rowmin_forward: D must be positive");
        FwdParams P;
        memset(&P, 0, sizeof(P));
        P.x1 = x1; P.x2 = x2; P.w = w; P.out = nullptr;
        P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
        P.rowmin_keys = static_cast<unsigned long long *>(scratch);
        // few features: x1 rows and their running minima in registers, x2 rows broadcast (lp_small_d.cu)
        int st = lp_small_d_rowmin_eligible(N1, N2, D, p)
                     ? lp_small_d_rowmin(x1, x2, static_cast<unsigned long long *>(scratch), B, N1, N2, D, p, out_exponent, s)
                     : lp_forward_typed<float, EPI_ROWMIN>(P, p, out_exponent, s);
        if (st != TPW_OK) return st;
    }
    rowmin_finish_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(static_cast<const unsigned long long *>(scratch), min_out,
                                                                     reinterpret_cast<long long *>(arg_out), n);
    TPW_LAUNCH_OK("rowmin_finish_kernel");
    return TPW_OK;
}

extern "C" int tpw_lp_radius_mask_forward(int dtype, const void *x1, const void *x2, const void *w, uint8_t *mask,
                                          int64_t B, int64_t N1, int64_t N2, int64_t D,
                                          double p, double out_exponent, double radius, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_lp_radius_mask_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(w == nullptr, "tpw_lp_radius_mask_forward: weighted distances are not built for this epilogue (w must be NULL)");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_lp_radius_mask_forward: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && mask, "tpw_lp_radius_mask_forward: NULL pointer");
    TPW_CHECK_ARG(D > 0, "tpw_lp_radius_mask_forward: D must be positive");
    TPW_CHECK_ARG(p > 0 && !isnan(p) && !isnan(out_exponent) && !isnan(radius), "tpw_lp_radius_mask_forward: p must be positive (got %g)", p);
    FwdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2; P.w = w; P.out = nullptr;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.mask_out = mask;
    P.threshold = radius;
    P.mask_vec = (N2 % 16 == 0 && aligned16(mask)) ? 1 : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // few features: the streaming kernel of lp_small_d.cu with the radius test as its epilogue
    if (dtype == TPW_F32 && lp_small_d_eligible(N1, N2, D, p)) return lp_small_d_mask(x1, x2, mask, B, N1, N2, D, p, out_exponent, radius, s);
    return dtype == TPW_F32 ? lp_forward_typed<float, EPI_MASK>(P, p, out_exponent, s) : lp_forward_typed<double, EPI_MASK>(P, p, out_exponent, s);
}

extern "C" int tpw_lp_pdist_forward(int dtype, const void *x, void *out, int64_t B, int64_t N, int64_t D,
                                    double p, double out_exponent, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_lp_pdist_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N >= 0 && D >= 0, "tpw_lp_pdist_forward: negative size");
    if (B == 0 || N < 2) return TPW_OK;
    TPW_CHECK_ARG(x && out, "tpw_lp_pdist_forward: NULL pointer");
    TPW_CHECK_ARG(D > 0, "tpw_lp_pdist_forward: D must be positive");
    TPW_CHECK_ARG(p > 0 && !isnan(p) && !isnan(out_exponent), "tpw_lp_pdist_forward: p must be positive (got %g)", p);
    FwdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x; P.x2 = x; P.w = nullptr; P.out = out;
    P.B = B; P.N1 = N; P.N2 = N; P.D = D;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == TPW_F32 ? lp_forward_typed<float, EPI_PDIST>(P, p, out_exponent, s) : lp_forward_typed<double, EPI_PDIST>(P, p, out_exponent, s);
}
