// Small memory-bound helpers of the pairwise path: the "safe divide" and its gradient, and the
// per-row mean-centering / L2 norm that cosine and correlation need before the contraction.
#include "common.cuh"

#include <math.h>

namespace tpw {
namespace {

constexpr int kThreads = 256;

template <typename T>
__global__ void prf_div_forward_kernel(const T *x, const T *y, T *out, long long n, int identity) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const T a = x[i], b = y[i];
        out[i] = b != T(0) ? a / b : (identity ? a : T(0));
    }
}

template <typename T>
__global__ void prf_div_backward_kernel(const T *g, const T *x, const T *y, T *gx, T *gy, long long n, int identity) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const T go = g[i], b = y[i];
        const bool nz = b != T(0);
        const T gs = nz ? go / b : (identity ? go : T(0));
        if (gx) gx[i] = gs;
        if (gy) gy[i] = nz ? -gs * x[i] / b : T(0);
    }
}

// One warp per row: mean or sum of squares by shuffle reduction, rows of any length.
template <typename T, bool CENTER>
__global__ void row_stat_kernel(const T *x, T *out, long long rows, long long D) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        const T *row = x + r * D;
        T s = T(0);
        for (long long k = lane; k < D; k += 32) {
            const T v = row[k];
            s += CENTER ? v : v * v;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (CENTER) {
            const T mean = s / (T)D;
            for (long long k = lane; k < D; k += 32) out[r * D + k] = row[k] - mean;
        } else if (lane == 0) {
            out[r] = (T)sqrt((double)s);
        }
    }
}


// Cosine-similarity backward, element-wise part.  S = M / (n1 n2^T) with the "identity" safe
// divide; upstream gradient Gs w.r.t. S.  Per element: dM = Gs/denom (Gs where denom == 0) and
// d(denom) = -dM*S (0 where denom == 0).  Rows: one warp per (b,i) writes dM and
// rowterm[i] = sum_j d(denom)*n2[j]; columns: one thread per (b,j) sums colterm[j] =
// sum_i d(denom)*n1[i] in ascending i.  `epilogue` says what `out` holds (S, or 1 - S).
template <typename T>
__device__ __forceinline__ void cosine_terms(T g, T o, T na, T nb, int epilogue, T &dm, T &dd) {
    const T S = epilogue == TPW_DOT_COSINE_SIM ? o : T(1) - o;
    const T gs = epilogue == TPW_DOT_COSINE_SIM ? g : -g;
    const T denom = na * nb;
    if (denom != T(0)) {
        dm = gs / denom;
        dd = -dm * S;
    } else {
        dm = gs;
        dd = T(0);
    }
}

template <typename T>
__global__ void cosine_prepare_rows_kernel(const T *g, const T *out, const T *n1, const T *n2, T *dM, T *rowterm,
                                           long long B, long long N1, long long N2, int epilogue) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < B * N1; r += nwarps) {
        const long long b = r / N1;
        const T na = n1[r];
        const T *nb = n2 + b * N2;
        T acc = T(0);
        for (long long j = lane; j < N2; j += 32) {
            T dm, dd;
            cosine_terms(g[r * N2 + j], out[r * N2 + j], na, nb[j], epilogue, dm, dd);
            dM[r * N2 + j] = dm;
            acc += dd * nb[j];
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) rowterm[r] = acc;
    }
}

template <typename T>
__global__ void cosine_prepare_cols_kernel(const T *g, const T *out, const T *n1, const T *n2, T *colterm,
                                           long long B, long long N1, long long N2, int epilogue) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * N2) return;
    const long long b = idx / N2, j = idx % N2;
    const T nb = n2[idx];
    T acc = T(0);
    for (long long i = 0; i < N1; ++i) {
        const long long e = (b * N1 + i) * N2 + j;
        T dm, dd;
        cosine_terms(g[e], out[e], n1[b * N1 + i], nb, epilogue, dm, dd);
        acc += dd * n1[b * N1 + i];
    }
    colterm[idx] = acc;
}

// g[r,k] += term[r] * x[r,k] / n[r]  (nothing where n[r] == 0): the row-norm part of the chain.
template <typename T>
__global__ void cosine_finish_kernel(T *g, const T *x, const T *n, const T *term, long long rows, long long D) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < rows * D; e += stride) {
        const long long r = e / D;
        const T nr = n[r];
        if (nr != T(0)) g[e] += term[r] * x[e] / nr;
    }
}

inline unsigned grid_for(long long n) {
    long long blocks = (n + kThreads - 1) / kThreads;
    const long long cap = (long long)sm_count() * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

} // namespace
} // namespace tpw

using namespace tpw;

extern "C" int tpw_prf_div_forward(int dtype, int mode, const void *x, const void *y, void *out,
                                   int64_t n, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_prf_div_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(mode == TPW_PRF_ZERO || mode == TPW_PRF_IDENTITY, "tpw_prf_div_forward: bad mode %d", mode);
    TPW_CHECK_ARG(n >= 0, "tpw_prf_div_forward: negative size");
    if (n == 0) return TPW_OK;
    TPW_CHECK_ARG(x && y && out, "tpw_prf_div_forward: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32)
        prf_div_forward_kernel<float><<<grid_for(n), kThreads, 0, s>>>((const float *)x, (const float *)y, (float *)out, n, mode == TPW_PRF_IDENTITY);
    else
        prf_div_forward_kernel<double><<<grid_for(n), kThreads, 0, s>>>((const double *)x, (const double *)y, (double *)out, n, mode == TPW_PRF_IDENTITY);
    TPW_LAUNCH_OK("prf_div_forward_kernel");
    return TPW_OK;
}

extern "C" int tpw_prf_div_backward(int dtype, int mode, const void *grad, const void *x, const void *y,
                                    void *grad_x, void *grad_y, int64_t n, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_prf_div_backward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(mode == TPW_PRF_ZERO || mode == TPW_PRF_IDENTITY, "tpw_prf_div_backward: bad mode %d", mode);
    TPW_CHECK_ARG(n >= 0, "tpw_prf_div_backward: negative size");
    if (n == 0 || (!grad_x && !grad_y)) return TPW_OK;
    TPW_CHECK_ARG(grad && x && y, "tpw_prf_div_backward: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32)
        prf_div_backward_kernel<float><<<grid_for(n), kThreads, 0, s>>>((const float *)grad, (const float *)x, (const float *)y,
                                                                        (float *)grad_x, (float *)grad_y, n, mode == TPW_PRF_IDENTITY);
    else
        prf_div_backward_kernel<double><<<grid_for(n), kThreads, 0, s>>>((const double *)grad, (const double *)x, (const double *)y,
                                                                         (double *)grad_x, (double *)grad_y, n, mode == TPW_PRF_IDENTITY);
    TPW_LAUNCH_OK("prf_div_backward_kernel");
    return TPW_OK;
}

extern "C" int tpw_row_center(int dtype, const void *x, void *out, int64_t rows, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_row_center: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(rows >= 0 && D >= 0, "tpw_row_center: negative size");
    if (rows == 0 || D == 0) return TPW_OK;
    TPW_CHECK_ARG(x && out, "tpw_row_center: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32) row_stat_kernel<float, true><<<grid_for(rows * 32), kThreads, 0, s>>>((const float *)x, (float *)out, rows, D);
    else row_stat_kernel<double, true><<<grid_for(rows * 32), kThreads, 0, s>>>((const double *)x, (double *)out, rows, D);
    TPW_LAUNCH_OK("row_stat_kernel");
    return TPW_OK;
}

extern "C" int tpw_row_norm(int dtype, const void *x, void *norm, int64_t rows, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_row_norm: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(rows >= 0 && D >= 0, "tpw_row_norm: negative size");
    if (rows == 0) return TPW_OK;
    TPW_CHECK_ARG(norm && (x || D == 0), "tpw_row_norm: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32) row_stat_kernel<float, false><<<grid_for(rows * 32), kThreads, 0, s>>>((const float *)x, (float *)norm, rows, D);
    else row_stat_kernel<double, false><<<grid_for(rows * 32), kThreads, 0, s>>>((const double *)x, (double *)norm, rows, D);
    TPW_LAUNCH_OK("row_stat_kernel");
    return TPW_OK;
}

// Dispatcher of the cross-term metrics: SIMT engine here, tensor-core engine in gemm_tcgen05.cu.
extern "C" int tpw_dot_metric_forward_simt(int dtype, int epilogue, const void *x1, const void *x2, void *out,
                                           int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

extern "C" int tpw_dot_metric_forward(int dtype, int epilogue, int engine,
                                      const void *x1, const void *x2, void *out,
                                      int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    if (engine == TPW_ENGINE_AUTO || engine == TPW_ENGINE_SIMT_FP32)
        return tpw_dot_metric_forward_simt(dtype, epilogue, x1, x2, out, B, N1, N2, D, stream);
    return fail(TPW_ERR_UNSUPPORTED, "tpw_dot_metric_forward: engine %d needs scratch; call tpw_dot_metric_forward_ws", engine);
}

extern "C" int tpw_cosine_backward_prepare(int dtype, int epilogue, const void *grad, const void *out,
                                           const void *norm1, const void *norm2,
                                           void *dM, void *rowterm, void *colterm,
                                           int64_t B, int64_t N1, int64_t N2, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_cosine_backward_prepare: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(epilogue == TPW_DOT_COSINE_SIM || epilogue == TPW_DOT_COSINE_DIST || epilogue == TPW_DOT_ONE_MINUS_SIM,
                  "tpw_cosine_backward_prepare: bad epilogue %d", epilogue);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0, "tpw_cosine_backward_prepare: negative size");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = dtype == TPW_F32 ? 4 : 8;
    if (B * N1 * N2 == 0) {
        if (rowterm && B * N1 > 0) TPW_CUDA_OK(cudaMemsetAsync(rowterm, 0, (size_t)(B * N1) * es, s));
        if (colterm && B * N2 > 0) TPW_CUDA_OK(cudaMemsetAsync(colterm, 0, (size_t)(B * N2) * es, s));
        return TPW_OK;
    }
    TPW_CHECK_ARG(grad && out && norm1 && norm2 && dM && rowterm && colterm, "tpw_cosine_backward_prepare: NULL pointer");
    const unsigned cblocks = (unsigned)((B * N2 + kThreads - 1) / kThreads);
    if (dtype == TPW_F32) {
        cosine_prepare_rows_kernel<float><<<grid_for(B * N1 * 32), kThreads, 0, s>>>(
            (const float *)grad, (const float *)out, (const float *)norm1, (const float *)norm2, (float *)dM, (float *)rowterm, B, N1, N2, epilogue);
        cosine_prepare_cols_kernel<float><<<cblocks, kThreads, 0, s>>>(
            (const float *)grad, (const float *)out, (const float *)norm1, (const float *)norm2, (float *)colterm, B, N1, N2, epilogue);
    } else {
        cosine_prepare_rows_kernel<double><<<grid_for(B * N1 * 32), kThreads, 0, s>>>(
            (const double *)grad, (const double *)out, (const double *)norm1, (const double *)norm2, (double *)dM, (double *)rowterm, B, N1, N2, epilogue);
        cosine_prepare_cols_kernel<double><<<cblocks, kThreads, 0, s>>>(
            (const double *)grad, (const double *)out, (const double *)norm1, (const double *)norm2, (double *)colterm, B, N1, N2, epilogue);
    }
    TPW_LAUNCH_OK("cosine_prepare kernels");
    return TPW_OK;
}

extern "C" int tpw_cosine_backward_finish(int dtype, void *grad_x, const void *x, const void *norm, const void *term,
                                          int64_t rows, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_cosine_backward_finish: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(rows >= 0 && D >= 0, "tpw_cosine_backward_finish: negative size");
    if (rows * D == 0) return TPW_OK;
    TPW_CHECK_ARG(grad_x && x && norm && term, "tpw_cosine_backward_finish: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32)
        cosine_finish_kernel<float><<<grid_for(rows * D), kThreads, 0, s>>>((float *)grad_x, (const float *)x, (const float *)norm, (const float *)term, rows, D);
    else
        cosine_finish_kernel<double><<<grid_for(rows * D), kThreads, 0, s>>>((double *)grad_x, (const double *)x, (const double *)norm, (const double *)term, rows, D);
    TPW_LAUNCH_OK("cosine_finish_kernel");
    return TPW_OK;
}
