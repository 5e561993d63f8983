// Haversine (great-circle) distance between (latitude, longitude) pairs in radians, and its backward.
//
//   a = sin^2((lat1 - lat2)/2) + cos(lat1) cos(lat2) sin^2((lon1 - lon2)/2),   out = 2 asin(sqrt(a))
//     = 2 atan2(sqrt(a), sqrt(1 - a))
//
// (OPS/cpu/haversine_kernel.cpp:12-27 and its CUDA twin).  D is 2, so the forward is bound by the output
// write and the backward by the read of the upstream gradient; no tile of operands is worth staging.
// Every point is reduced once to the sines and cosines of its two half angles; the differences then come
// from the subtraction formulas, sin((p - q)/2) = sin(p/2) cos(q/2) - cos(p/2) sin(q/2), whose two products
// are rounded separately so that a point against itself gives exactly 0, as the reference's sin(0) does.
// The backward runs one pass per gradient (rows of x1, rows of x2); each gradient element is summed by one
// thread group in a fixed order, so the result is deterministic (the reference serialises one thread per row).
#include "common.cuh"

#include <math.h>

namespace tpw {
namespace {

template <typename T> struct Half4 { T sa, ca, so, co, cl; };   // sin, cos of lat/2; sin, cos of lon/2; cos(lat)

__device__ __forceinline__ void t_sincos(float v, float *s, float *c) { sincosf(v, s, c); }
__device__ __forceinline__ void t_sincos(double v, double *s, double *c) { sincos(v, s, c); }
__device__ __forceinline__ float h_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double h_mul(double a, double b) { return __dmul_rn(a, b); }
// 2 asin(sqrt(a)) from a and its complement c = 1 - a.  double: 2 atan2(sqrt(a), sqrt(c)).  float: the smaller of
// the two (at most 1/2, where asin is well conditioned) goes through the approximate square root (one MUFU
// operation) and asin(x) = x + x z P(z), z = x^2, a degree-6 fit on [0, 1/2] with relative error 5e-8; the larger
// side is the complement to pi.  Branch-free, about a dozen operations instead of the library atan2f.
__device__ __forceinline__ double hav_dist(double a, double c) { return 2.0 * atan2(sqrt(a), sqrt(c)); }
__device__ __forceinline__ float hav_dist(float a, float c) {
    const float z = fminf(a, c);
    float x;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(x) : "f"(z));
    float p = 0.08603748f;
    p = fmaf(p, z, -0.05019181f);
    p = fmaf(p, z, 0.04930707f);
    p = fmaf(p, z, 0.02518522f);
    p = fmaf(p, z, 0.04510614f);
    p = fmaf(p, z, 0.07498478f);
    p = fmaf(p, z, 0.16666675f);
    const float r = 2.f * fmaf(x * z, p, x);
    return a <= c ? r : 3.14159265358979f - r;
}
// 1 / (sqrt(a) sqrt(c)), 0 where the product is 0
__device__ __forceinline__ double hav_rden(double a, double c) { const double d = sqrt(a) * sqrt(c); return d > 0.0 ? 1.0 / d : 0.0; }
__device__ __forceinline__ float hav_rden(float a, float c) { const float d = a * c; return d >= 1.17549435e-38f ? rsqrtf(d) : 0.f; }

template <typename T>
__device__ __forceinline__ Half4<T> half_angles(const T *p) {
    Half4<T> h;
    t_sincos(p[0] * T(0.5), &h.sa, &h.ca);
    t_sincos(p[1] * T(0.5), &h.so, &h.co);
    h.cl = h.ca * h.ca - h.sa * h.sa;
    return h;
}

// u = sin(dlat/2), v = sin(dlon/2), cc = cos(lat1) cos(lat2); returns a = u^2 + cc v^2 >= 0 and its complement
// 1 - a = cos^2(dlat/2) - cc v^2 >= 0, formed from the cosine of the half difference rather than by
// subtracting from 1, so that nearly antipodal pairs (a -> 1) keep their relative accuracy
template <typename T>
__device__ __forceinline__ T hav_a(const Half4<T> &p, const Half4<T> &q, T &u, T &v, T &cc, T &one_minus_a) {
    u = h_mul(p.sa, q.ca) - h_mul(p.ca, q.sa);
    v = h_mul(p.so, q.co) - h_mul(p.co, q.so);
    cc = p.cl * q.cl;
    const T cu = p.ca * q.ca + p.sa * q.sa;
    const T w = cc * v * v;
    const T a = u * u + w, c = cu * cu - w;
    one_minus_a = c < T(0) ? T(0) : c;
    return a < T(0) ? T(0) : a;
}

constexpr int FT = 256;   // threads per CTA
constexpr int FJ = 4;     // consecutive columns (x2 rows) per thread: one 128-bit store per output row
constexpr int FR = 64;    // x1 rows per CTA

template <typename T> struct Out4 { T v[FJ]; };
__device__ __forceinline__ void store_out4(float *dst, const Out4<float> &o) {
    __stcs(reinterpret_cast<float4 *>(dst), make_float4(o.v[0], o.v[1], o.v[2], o.v[3]));
}
__device__ __forceinline__ void store_out4(double *dst, const Out4<double> &o) {
    __stcs(reinterpret_cast<double2 *>(dst), make_double2(o.v[0], o.v[1]));
    __stcs(reinterpret_cast<double2 *>(dst) + 1, make_double2(o.v[2], o.v[3]));
}

template <typename T>
__global__ void __launch_bounds__(FT) haversine_forward_kernel(const T *x1, const T *x2, T *out, long long N1, long long N2,
                                                               long long tiles_i, long long tiles_j, int vec_store) {
    __shared__ Half4<T> rows[FR];
    const long long tile = blockIdx.x;
    const long long tj = tile % tiles_j, ti = (tile / tiles_j) % tiles_i, b = tile / (tiles_j * tiles_i);
    const long long i0 = ti * FR, j0 = (tj * FT + threadIdx.x) * FJ;
    if (threadIdx.x < FR && i0 + threadIdx.x < N1) rows[threadIdx.x] = half_angles(x1 + (b * N1 + i0 + threadIdx.x) * 2);
    Half4<T> q[FJ];
#pragma unroll
    for (int c = 0; c < FJ; ++c)
        if (j0 + c < N2) q[c] = half_angles(x2 + (b * N2 + j0 + c) * 2);
        else q[c] = Half4<T>{T(0), T(1), T(0), T(1), T(1)};
    __syncthreads();
    if (j0 >= N2) return;
    const int nr = (int)min((long long)FR, N1 - i0);
    T *o = out + (b * N1 + i0) * N2 + j0;
    const bool whole = vec_store && j0 + FJ <= N2;
    for (int r = 0; r < nr; ++r) {
        const Half4<T> p = rows[r];
        Out4<T> res;
#pragma unroll
        for (int c = 0; c < FJ; ++c) {
            T u, v, cc, cm;
            const T a = hav_a(p, q[c], u, v, cc, cm);
            res.v[c] = hav_dist(a, cm);
        }
        T *dst = o + (long long)r * N2;
        if (whole) store_out4(dst, res);
        else {
#pragma unroll
            for (int c = 0; c < FJ; ++c)
                if (j0 + c < N2) dst[c] = res.v[c];
        }
    }
}

// coefficient g / (sqrt(a) sqrt(1 - a)), nothing where the denominator is 0 (coincident or antipodal points;
// the reference divides by it)
template <typename T>
__device__ __forceinline__ T hav_coef(T g, T a, T one_minus_a) {
    return g * hav_rden(a, one_minus_a);
}

// d a / d lat_p and d a / d lon_p for the pair (p, q):
//   lat: sin(dlat)/2 - sin(lat_p) cos(lat_q) v^2,   lon: cos(lat_p) cos(lat_q) v cos(dlon/2)
template <typename T>
__device__ __forceinline__ void hav_grad_terms(const Half4<T> &p, const Half4<T> &q, T u, T v, T cc, T &dlat, T &dlon) {
    const T cu = p.ca * q.ca + p.sa * q.sa;                 // cos(dlat/2)
    const T cv = p.co * q.co + p.so * q.so;                 // cos(dlon/2)
    const T sin_p = T(2) * p.sa * p.ca, cos_q = q.cl;
    dlat = u * cu - sin_p * cos_q * v * v;
    dlon = cc * v * cv;
}

constexpr int BW = 8;     // grad_x1: rows per CTA, one warp each
constexpr int BC = 256;   // grad_x1: streamed x2 rows per step

template <typename T>
__global__ void __launch_bounds__(BW * 32) haversine_backward_x1_kernel(const T *grad, const T *x1, const T *x2, T *gx1,
                                                                       long long N1, long long N2, long long tiles_i) {
    __shared__ Half4<T> cols[BC];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long b = blockIdx.x / tiles_i, i = (blockIdx.x % tiles_i) * BW + warp;
    const bool live = i < N1;
    Half4<T> p;
    if (live) p = half_angles(x1 + (b * N1 + i) * 2);
    T slat = T(0), slon = T(0);
    for (long long j0 = 0; j0 < N2; j0 += BC) {
        __syncthreads();
        if (j0 + threadIdx.x < N2) cols[threadIdx.x] = half_angles(x2 + (b * N2 + j0 + threadIdx.x) * 2);
        __syncthreads();
        if (!live) continue;
        const int nc = (int)min((long long)BC, N2 - j0);
        const T *g = grad + (b * N1 + i) * N2 + j0;
#pragma unroll 4
        for (int c = lane; c < nc; c += 32) {   // several gradient loads in flight per lane
            T u, v, cc, dlat, dlon, om;
            const T a = hav_a(p, cols[c], u, v, cc, om);
            const T k = hav_coef(g[c], a, om);
            hav_grad_terms(p, cols[c], u, v, cc, dlat, dlon);
            slat += k * dlat;
            slon += k * dlon;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        slat += __shfl_xor_sync(0xffffffffu, slat, off);
        slon += __shfl_xor_sync(0xffffffffu, slon, off);
    }
    if (live && lane == 0) {
        gx1[(b * N1 + i) * 2] = slat;
        gx1[(b * N1 + i) * 2 + 1] = slon;
    }
}

constexpr int CW = 64;    // grad_x2: columns per CTA
constexpr int CG = 8;     // grad_x2: row groups per CTA (rows i = group, group + CG, ...)
constexpr int CR = 64;    // grad_x2: x1 rows staged per step

template <typename T>
__global__ void __launch_bounds__(CW * CG) haversine_backward_x2_kernel(const T *grad, const T *x1, const T *x2, T *gx2,
                                                                       long long N1, long long N2, long long tiles_j) {
    __shared__ Half4<T> rows[CR];
    __shared__ T part[CG][CW][2];
    const int col = threadIdx.x % CW, grp = threadIdx.x / CW;
    const long long b = blockIdx.x / tiles_j, j = (blockIdx.x % tiles_j) * CW + col;
    const bool live = j < N2;
    Half4<T> q;
    if (live) q = half_angles(x2 + (b * N2 + j) * 2);
    T slat = T(0), slon = T(0);
    for (long long i0 = 0; i0 < N1; i0 += CR) {
        __syncthreads();
        if (threadIdx.x < CR && i0 + threadIdx.x < N1) rows[threadIdx.x] = half_angles(x1 + (b * N1 + i0 + threadIdx.x) * 2);
        __syncthreads();
        if (!live) continue;
        const int nr = (int)min((long long)CR, N1 - i0);
#pragma unroll 4
        for (int r = grp; r < nr; r += CG) {   // several gradient loads in flight per thread
            T u, v, cc, dlat, dlon, om;
            // the pair seen from x2: u and v change sign, a and cc do not
            const T a = hav_a(q, rows[r], u, v, cc, om);
            const T k = hav_coef(grad[(b * N1 + i0 + r) * N2 + j], a, om);
            hav_grad_terms(q, rows[r], u, v, cc, dlat, dlon);
            slat += k * dlat;
            slon += k * dlon;
        }
    }
    part[grp][col][0] = slat;
    part[grp][col][1] = slon;
    __syncthreads();
    if (grp == 0 && live) {
        T a0 = T(0), a1 = T(0);
#pragma unroll
        for (int g = 0; g < CG; ++g) { a0 += part[g][col][0]; a1 += part[g][col][1]; }
        gx2[(b * N2 + j) * 2] = a0;
        gx2[(b * N2 + j) * 2 + 1] = a1;
    }
}

template <typename T>
int haversine_forward_typed(const void *x1, const void *x2, void *out, long long B, long long N1, long long N2, cudaStream_t s) {
    const long long ti = (N1 + FR - 1) / FR, tj = (N2 + FT * FJ - 1) / (FT * FJ), tiles = B * ti * tj;
    TPW_CHECK_ARG(tiles < (1ll << 31), "tpw_haversine_forward: too many tiles (%lld)", tiles);
    const int vec = (N2 % FJ == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) ? 1 : 0;
    haversine_forward_kernel<T><<<(unsigned)tiles, FT, 0, s>>>((const T *)x1, (const T *)x2, (T *)out, N1, N2, ti, tj, vec);
    TPW_LAUNCH_OK("haversine_forward_kernel");
    return TPW_OK;
}

template <typename T>
int haversine_backward_typed(const void *g, const void *x1, const void *x2, void *g1, void *g2, long long B, long long N1,
                             long long N2, cudaStream_t s) {
    if (g1) {
        const long long ti = (N1 + BW - 1) / BW;
        TPW_CHECK_ARG(B * ti < (1ll << 31), "tpw_haversine_backward: too many row groups");
        haversine_backward_x1_kernel<T><<<(unsigned)(B * ti), BW * 32, 0, s>>>((const T *)g, (const T *)x1, (const T *)x2, (T *)g1, N1, N2, ti);
        TPW_LAUNCH_OK("haversine_backward_x1_kernel");
    }
    if (g2) {
        const long long tj = (N2 + CW - 1) / CW;
        TPW_CHECK_ARG(B * tj < (1ll << 31), "tpw_haversine_backward: too many column groups");
        haversine_backward_x2_kernel<T><<<(unsigned)(B * tj), CW * CG, 0, s>>>((const T *)g, (const T *)x1, (const T *)x2, (T *)g2, N1, N2, tj);
        TPW_LAUNCH_OK("haversine_backward_x2_kernel");
    }
    return TPW_OK;
}

} // namespace
} // namespace tpw

using namespace tpw;

extern "C" int tpw_haversine_forward(int dtype, const void *x1, const void *x2, void *out,
                                     int64_t B, int64_t N1, int64_t N2, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_haversine_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0, "tpw_haversine_forward: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && out, "tpw_haversine_forward: NULL pointer");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == TPW_F32 ? haversine_forward_typed<float>(x1, x2, out, B, N1, N2, s)
                            : haversine_forward_typed<double>(x1, x2, out, B, N1, N2, s);
}

extern "C" int tpw_haversine_backward(int dtype, const void *grad, const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                                      int64_t B, int64_t N1, int64_t N2, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_haversine_backward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0, "tpw_haversine_backward: negative size");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = dtype == TPW_F32 ? 4 : 8;
    if (B == 0 || N1 == 0 || N2 == 0) {
        if (grad_x1 && B * N1 > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x1, 0, (size_t)(B * N1 * 2) * es, s));
        if (grad_x2 && B * N2 > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x2, 0, (size_t)(B * N2 * 2) * es, s));
        return TPW_OK;
    }
    TPW_CHECK_ARG(grad && x1 && x2 && (grad_x1 || grad_x2), "tpw_haversine_backward: NULL pointer");
    return dtype == TPW_F32 ? haversine_backward_typed<float>(grad, x1, x2, grad_x1, grad_x2, B, N1, N2, s)
                            : haversine_backward_typed<double>(grad, x1, x2, grad_x1, grad_x2, B, N1, N2, s);
}
