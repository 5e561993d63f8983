// Shared template of the CUDA-core forward tile kernel: included by lp_forward.cu (tiles stored to
// global memory) and lp_forward_fused.cu (row-minimum and radius-mask epilogues), so that the fused
// epilogues are separate instantiations and leave the code of the stored-tile kernels untouched.
#pragma once
#include "common.cuh"
#include "packed_f32x2.cuh"

#include <math.h>

namespace tpw {
namespace {

enum Kind {
    K_L1 = 0,     // sum |d|
    K_P2 = 1,     // sum d^2
    K_P3 = 2,     // sum |d|^3
    K_PGEN = 3,   // sum |d|^p via exp2/log2
    K_MAX = 4,    // max |d|
    K_MIN = 5,    // min |d| (padding masked)
    K_DOT = 6,    // sum x*y with row norms accumulated on the side
    K_NE = 7,     // count of x != y (IEEE compare)
    K_NE_BITS = 8, // count of differing bit patterns (integer payloads)
    K_CANBERRA = 9, // sum |x - y| / (|x| + |y|), terms with a zero denominator skipped
    K_CHI2 = 10,    // - sum (x - y)^2 / (x + y), terms with a zero denominator skipped
    K_JS = 11       // sum x log(x/m) + y log(y/m), m = (x + y)/2 (float: in units of log 2, scaled at the end)
};

struct FwdParams {
    const void *x1, *x2, *w;
    void *out;
    long long B, N1, N2, D;
    long long tiles_i, tiles_j;
    double p;            // exponent of K_PGEN
    int pow_spec;        // make_pow_spec(p): how the float kernel evaluates |d|^p
    double out_exponent; // finite kinds: out = sum ^ out_exponent
    int root_mode;       // 0 none, 1 sqrt, 2 cbrt, 3 pow(out_exponent)
    double scale;        // K_JS: factor applied to the finished sum (before the optional square root)
    int epilogue;        // K_DOT: tpw_dot_epilogue; K_NE*: bit0 = report equal count, bit1 = mean
    int vec_store;       // 4-byte outputs, N2 % 4 == 0, 16-byte aligned base: staged 128-bit stores
    int *status;
    // Non-NULL (fp32 L_p kinds only): the tile is not stored; every x1 row folds its smallest
    // finished value, packed as (float bits << 32 | x2 row), into keys[b * N1 + i] with atomicMin.
    unsigned long long *rowmin_keys;
    // Non-NULL (L_p kinds): the tile is not stored; one byte per pair, finished value <= threshold.
    unsigned char *mask_out;
    double threshold;
    int mask_vec;        // N2 % 16 == 0 and 16-byte aligned mask: staged 128-bit stores
};

template <typename T> struct Vec16;
template <> struct Vec16<float> { typedef float4 type; static const int N = 4; };
template <> struct Vec16<double> { typedef double2 type; static const int N = 2; };

template <typename T> __device__ __forceinline__ T t_abs(T v);
template <> __device__ __forceinline__ float t_abs<float>(float v) { return fabsf(v); }
template <> __device__ __forceinline__ double t_abs<double>(double v) { return fabs(v); }
template <typename T> __device__ __forceinline__ T t_fma(T a, T b, T c);
template <> __device__ __forceinline__ float t_fma<float>(float a, float b, float c) { return fmaf(a, b, c); }
template <> __device__ __forceinline__ double t_fma<double>(double a, double b, double c) { return fma(a, b, c); }
template <typename T> __device__ __forceinline__ T t_max(T a, T b);
template <> __device__ __forceinline__ float t_max<float>(float a, float b) { return fmaxf(a, b); }
template <> __device__ __forceinline__ double t_max<double>(double a, double b) { return fmax(a, b); }
template <typename T> __device__ __forceinline__ T t_min(T a, T b);
template <> __device__ __forceinline__ float t_min<float>(float a, float b) { return fminf(a, b); }
template <> __device__ __forceinline__ double t_min<double>(double a, double b) { return fmin(a, b); }
// |a|^p for a >= 0.  fp32: two MUFU operations; 0^p = exp2(-inf) = 0 for p > 0.
__device__ __forceinline__ float t_powabs(float a, float p) { return exp2f(p * __log2f(a)); }
__device__ __forceinline__ double t_powabs(double a, double p) { return pow(a, p); }
__device__ __forceinline__ float t_sqrt(float v) { return sqrtf(v); }
__device__ __forceinline__ double t_sqrt(double v) { return sqrt(v); }
__device__ __forceinline__ float t_cbrt(float v) { return cbrtf(v); }
__device__ __forceinline__ double t_cbrt(double v) { return cbrt(v); }
__device__ __forceinline__ float t_pow(float v, double e) { return powf(v, (float)e); }
__device__ __forceinline__ double t_pow(double v, double e) { return pow(v, e); }
// One relative-entropy term v log(v/m) given q = v/m: zero at v == 0, +inf for a negative v (the
// reference's CPU loop returns its upper bound there, OPS/cpu/rel_entr.h:9-18).  The float form is in
// units of log 2 (one MUFU lg2); the caller folds log 2 into the final scale.
__device__ __forceinline__ float rel_entr_term(float v, float q) {
    // the ratio is kept above the smallest normal number, so the flush-to-zero logarithm stays finite and a
    // zero entry gives 0 * finite = 0 without a branch
    float l;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(l) : "f"(fmaxf(q, 1.17549435e-38f)));
    return v >= 0.f ? v * l : __int_as_float(0x7f800000);
}
__device__ __forceinline__ double rel_entr_term(double v, double q) {
    return v > 0.0 ? v * log(q) : (v == 0.0 ? 0.0 : __longlong_as_double(0x7ff0000000000000ll));
}
__device__ __forceinline__ bool bits_differ(float a, float b) { return __float_as_int(a) != __float_as_int(b); }
__device__ __forceinline__ bool bits_differ(double a, double b) {
    return __double_as_longlong(a) != __double_as_longlong(b);
}

template <int KIND, bool WEIGHTED, typename T>
__device__ __forceinline__ void accumulate(T &acc, T x, T y, T w, T p, int pspec) {
    if (KIND == K_DOT) {
        acc = t_fma(x, y, acc);
    } else if (KIND == K_NE) {
        acc += (x != y) ? T(1) : T(0);
    } else if (KIND == K_NE_BITS) {
        acc += bits_differ(x, y) ? T(1) : T(0);
    } else if (KIND == K_CANBERRA) {
        // branch-free: a zero denominator (zero padding included) selects a zero reciprocal
        const T den = t_abs(x) + t_abs(y);
        const T r = rcp_or_zero(den);
        acc = t_fma(t_abs(x - y), r, acc);
    } else if (KIND == K_CHI2) {
        const T nom = x + y, d = x - y;
        const T r = rcp_or_zero(nom);
        acc = t_fma(-(d * d), r, acc);
    } else if (KIND == K_JS) {
        // x/m = 1 + t and y/m = 1 - t with t = (x - y)/(x + y): one reciprocal for both ratios, and equal
        // entries give exactly log 1 = 0, so that a row against itself sums to exactly 0 as in the
        // reference; zero padding gives two zero terms
        const T t = (x - y) * rcp_or_zero(x + y);
        acc += rel_entr_term(x, T(1) + t) + rel_entr_term(y, T(1) - t);
    } else {
        T d = x - y;
        if (KIND == K_L1) {
            acc = WEIGHTED ? t_fma(t_abs(d), w, acc) : acc + t_abs(d);
        } else if (KIND == K_P2) {
            acc = WEIGHTED ? t_fma(d * d, w, acc) : t_fma(d, d, acc);
        } else if (KIND == K_P3) {
            T a = t_abs(d);
            acc = WEIGHTED ? t_fma(a * a, a * w, acc) : t_fma(a * a, a, acc);
        } else if (KIND == K_PGEN) {
            T t = pow_abs_spec(t_abs(d), p, pspec);
            acc = WEIGHTED ? t_fma(t, w, acc) : acc + t;
        } else if (KIND == K_MAX) {
            acc = t_max(acc, WEIGHTED ? t_abs(d) * w : t_abs(d));
        } else if (KIND == K_MIN) {
            acc = t_min(acc, WEIGHTED ? t_abs(d) * w : t_abs(d));
        }
    }
}

template <typename T, typename OutT, int KIND>
__device__ __forceinline__ OutT finish(T acc, T n1, T n2, const FwdParams &P) {
    if (KIND == K_DOT) {
        switch (P.epilogue) {
            case TPW_DOT_LINEAR: return (OutT)acc;
            case TPW_DOT_SQEUCLIDEAN: return (OutT)t_max(n1 + n2 - T(2) * acc, T(0));
            case TPW_DOT_EUCLIDEAN: return (OutT)t_sqrt(t_max(n1 + n2 - T(2) * acc, T(0)));
            default: {
                T denom = t_sqrt(n1) * t_sqrt(n2);
                T s = denom != T(0) ? acc / denom : acc;
                if (P.epilogue == TPW_DOT_COSINE_SIM) return (OutT)s;
                T dist = T(1) - s;
                if (P.epilogue == TPW_DOT_COSINE_DIST) dist = t_min(t_max(dist, T(0)), T(2));
                return (OutT)dist;
            }
        }
    } else if (KIND == K_NE || KIND == K_NE_BITS) {
        float cnt = (float)acc;
        if (P.epilogue & 1) cnt = (float)P.D - cnt;
        if (P.epilogue & 2) cnt = __fdiv_rn(cnt, (float)P.D);
        return (OutT)cnt;
    } else if (KIND == K_MAX || KIND == K_MIN) {
        return (OutT)acc;
    } else if (KIND == K_JS) {
        const T v = acc * (T)P.scale;
        return (OutT)(P.root_mode == 1 ? t_sqrt(t_max(v, T(0))) : v);
    } else {
        return (OutT)acc; // the root of the finite-p kinds is applied to the whole register tile by apply_root
    }
}

// out = sum ^ out_exponent for the finite-p kinds, on the whole register tile with the (uniform)
// choice of root hoisted out of the per-element code, so that the epilogues below are root-free.
template <typename T, int R, int KIND>
__device__ __forceinline__ void apply_root(T (&acc)[R][R], const FwdParams &P) {
    if (KIND != K_L1 && KIND != K_P2 && KIND != K_P3 && KIND != K_PGEN) return;
    if (P.root_mode == 0) return;
    if (P.root_mode == 1) {
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
            for (int c = 0; c < R; ++c) acc[a][c] = t_sqrt(acc[a][c]);
    } else if (P.root_mode == 2) {
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
            for (int c = 0; c < R; ++c) acc[a][c] = t_cbrt(acc[a][c]);
    } else {
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
            for (int c = 0; c < R; ++c) acc[a][c] = t_pow(acc[a][c], P.out_exponent);
    }
}

// what the epilogue does with a finished tile
enum { EPI_STORE = 0, EPI_ROWMIN = 1, EPI_MASK = 2, EPI_PDIST = 3 };

constexpr int kThreads = 256;
constexpr int kStages = 3;

template <typename T, int R> struct FwdSmem {
    static constexpr int TILE = 16 * R;
    static constexpr int KC = 128 / (int)sizeof(T); // features per 128-byte chunk row
    static constexpr int TILE_BYTES = TILE * 128;
    // [stage][x tile | y tile] then weights, norms and barriers
    static constexpr int OFF_W = kStages * 2 * TILE_BYTES;
    static constexpr int OFF_NORM = OFF_W + kStages * 128;
    static constexpr int OFF_BAR = OFF_NORM + 2 * TILE * (int)sizeof(T);
    static constexpr int BYTES = OFF_BAR + kStages * 8;
    static constexpr int ALLOC = BYTES + 1024; // slack for the 1024-byte alignment of the swizzled tiles
};

// Guarded plain-load staging of one chunk (rows x 128 bytes) into the swizzled layout.
template <typename T, int TILE>
__device__ __forceinline__ void stage_rows_generic(unsigned char *tile, const T *base, long long row0,
                                                   long long nrows, long long D, long long k0) {
    constexpr int KC = 128 / (int)sizeof(T);
    constexpr int PER16 = 16 / (int)sizeof(T);
    for (int e = threadIdx.x; e < TILE * KC; e += kThreads) {
        int r = e / KC, kk = e % KC;
        long long row = row0 + r, k = k0 + kk;
        T v = (row < nrows && k < D) ? base[row * D + k] : T(0);
        *reinterpret_cast<T *>(tile + swz128(r, kk / PER16) + (kk % PER16) * sizeof(T)) = v;
    }
}

template <typename T, typename OutT, int R, int KIND, bool WEIGHTED, bool USE_TMA, bool PARTIAL, int EPI>
__global__ void __launch_bounds__(kThreads, (sizeof(T) == 4 ? 2 : 1))
lp_forward_kernel(const __grid_constant__ CUtensorMap map1, const __grid_constant__ CUtensorMap map2,
                  const FwdParams P) {
    typedef FwdSmem<T, R> S;
    typedef typename Vec16<T>::type V;
    constexpr int VN = Vec16<T>::N;
    constexpr int TILE = S::TILE;
    constexpr int KC = S::KC;

    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    T *wsm = reinterpret_cast<T *>(smem + S::OFF_W);
    T *norms = reinterpret_cast<T *>(smem + S::OFF_NORM);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + S::OFF_BAR);

    const int tid = threadIdx.x;
    const int ti = tid >> 4, tj = tid & 15;
    // Packed form of the unweighted float32 p = 3 tile (full 128-byte chunks by TMA): a thread owns rows
    // {32 a + 2 ti, 32 a + 2 ti + 1} and columns {32 c + 2 tj, 32 c + 2 tj + 1} instead of {ti + 16 a} and {tj + 16 c},
    // so that two rows and two columns are adjacent words of the transposed operand tiles and fill the two lanes of
    // the packed subtract / fused multiply-add without a register move.  Every pair still adds its features in
    // ascending order with the same roundings, so the results are the scalar tile's bit for bit.
    constexpr bool PK = (KIND == K_P3 && !WEIGHTED && sizeof(T) == 4 && USE_TMA && !PARTIAL && R == 8);
    auto row_of = [&](int a) -> int { return PK ? 32 * (a >> 1) + 2 * ti + (a & 1) : ti + 16 * a; };
    auto col_of = [&](int c) -> int { return PK ? 32 * (c >> 1) + 2 * tj + (c & 1) : tj + 16 * c; };

    long long tile = blockIdx.x;
    const long long tjx = tile % P.tiles_j;
    tile /= P.tiles_j;
    const long long tix = tile % P.tiles_i;
    const long long b = tile / P.tiles_i;
    const long long i0 = tix * TILE, j0 = tjx * TILE;

    if constexpr (EPI == EPI_PDIST) {
        // condensed self-distances: only pairs j > i are wanted, tiles that hold none do no work at all
        if (j0 + TILE - 1 <= i0) return;
    }

    const T *x1 = reinterpret_cast<const T *>(P.x1) + b * P.N1 * P.D;
    const T *x2 = reinterpret_cast<const T *>(P.x2) + b * P.N2 * P.D;
    const T *w = WEIGHTED ? reinterpret_cast<const T *>(P.w) + b * P.D : nullptr;

    const int nchunks = (int)((P.D + KC - 1) / KC);

    T acc[R][R];
#pragma unroll
    for (int a = 0; a < R; ++a)
#pragma unroll
        for (int c = 0; c < R; ++c) acc[a][c] = (KIND == K_MIN) ? T(INFINITY) : T(0);
    T nsq = T(0); // K_DOT: squared norm of the row this thread looks after
    // packed accumulators: pa[a][c] = pairs (2a, 2c) and (2a+1, 2c+1), pb[a][c] = pairs (2a, 2c+1) and (2a+1, 2c)
    f32x2 pa[PK ? R / 2 : 1][PK ? R / 2 : 1], pb[PK ? R / 2 : 1][PK ? R / 2 : 1];
    if constexpr (PK) {
#pragma unroll
        for (int a = 0; a < R / 2; ++a)
#pragma unroll
            for (int c = 0; c < R / 2; ++c) { pa[a][c] = 0ull; pb[a][c] = 0ull; }
    }

    if (USE_TMA) {
        if (tid == 0) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
            mbar_init_fence();
            tma_prefetch_descriptor(&map1);
            tma_prefetch_descriptor(&map2);
        }
        __syncthreads();
        if (tid == 0) {
            for (int c = 0; c < kStages - 1 && c < nchunks; ++c) {
                mbar_expect_tx(&full[c], 2 * S::TILE_BYTES);
                tma_load_3d(smem + (2 * c) * S::TILE_BYTES, &map1, &full[c], c * KC, (int)i0, (int)b);
                tma_load_3d(smem + (2 * c + 1) * S::TILE_BYTES, &map2, &full[c], c * KC, (int)j0, (int)b);
            }
        }
        if (WEIGHTED && tid < KC) {
            for (int c = 0; c < kStages - 1 && c < nchunks; ++c) {
                long long k = (long long)c * KC + tid;
                wsm[c * KC + tid] = k < P.D ? w[k] : T(0);
            }
        }
    }

    const T pexp = (T)P.p;
    const int pspec = P.pow_spec;
    int failed = 0;

    for (int t = 0; t < nchunks; ++t) {
        int stage;
        if (USE_TMA) {
            // Everyone has finished chunk t-1, so its stage may be refilled with chunk t+kStages-1.
            if (__syncthreads_or(failed)) {
                if (tid == 0) {
                    if (P.status) atomicCAS(P.status, 0, (1 << 16) | 1);
                    // chunks t and t + 1 were issued earlier and may still be landing: the CTA stays (bounded) until
                    // they have, so that no copy writes into shared memory the CTA has given back
                    for (int c = t; c < t + kStages - 1 && c < nchunks; ++c) mbar_wait_bounded(&full[c % kStages], (uint32_t)((c / kStages) & 1));
                }
                return;
            }
            const int nxt = t + kStages - 1;
            if (nxt < nchunks) {
                const int ns = nxt % kStages;
                if (tid == 0) {
                    mbar_expect_tx(&full[ns], 2 * S::TILE_BYTES);
                    tma_load_3d(smem + (2 * ns) * S::TILE_BYTES, &map1, &full[ns], nxt * KC, (int)i0, (int)b);
                    tma_load_3d(smem + (2 * ns + 1) * S::TILE_BYTES, &map2, &full[ns], nxt * KC, (int)j0, (int)b);
                }
                if (WEIGHTED && tid < KC) {
                    long long k = (long long)nxt * KC + tid;
                    wsm[ns * KC + tid] = k < P.D ? w[k] : T(0);
                }
            }
            stage = t % kStages;
            if (!mbar_wait_bounded(&full[stage], (uint32_t)((t / kStages) & 1))) failed = 1;
        } else {
            stage = 0;
            __syncthreads();
            stage_rows_generic<T, TILE>(smem, x1, i0, P.N1, P.D, (long long)t * KC);
            stage_rows_generic<T, TILE>(smem + S::TILE_BYTES, x2, j0, P.N2, P.D, (long long)t * KC);
            if (WEIGHTED && tid < KC) {
                long long k = (long long)t * KC + tid;
                wsm[tid] = k < P.D ? w[k] : T(0);
            }
            __syncthreads();
        }
        const unsigned char *xs = smem + (2 * stage) * S::TILE_BYTES;
        const unsigned char *ys = xs + S::TILE_BYTES;
        const T *wst = wsm + stage * KC;
        const uint32_t xrow = ti, yrow = tj; // (row + 16 r) & 7 == row & 7
        const long long kbase = (long long)t * KC;

        // Each trip handles one 16-byte group of features (4 floats / 2 doubles) against the whole
        // register tile.  PARTIAL instantiations (D not a multiple of the chunk) stop the last chunk at
        // the last group that holds real features -- the rest is zero fill -- which keeps small-D
        // shapes output-bound; the others keep a constant trip count.
        const long long kleft = P.D - kbase;
        const int cmax = (PARTIAL && kleft < KC) ? (int)((kleft + VN - 1) / VN) : 8;
        if constexpr (PK) {
            // transpose both operand tiles in place: [128 rows][32 features] (swizzled) -> [32 features][128 rows].
            // Consecutive lanes read consecutive rows of one 16-byte chunk (all banks) and write consecutive words.
            {
                const uint32_t trow = tid & 127u, th = tid >> 7;
                float4 xv[4], yv[4];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    xv[cc] = *reinterpret_cast<const float4 *>(xs + swz128(trow, th * 4 + cc));
                    yv[cc] = *reinterpret_cast<const float4 *>(ys + swz128(trow, th * 4 + cc));
                }
                __syncthreads();
                float *xw = reinterpret_cast<float *>(const_cast<unsigned char *>(xs)) + (th * 16) * 128 + trow;
                float *yw = reinterpret_cast<float *>(const_cast<unsigned char *>(ys)) + (th * 16) * 128 + trow;
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    xw[(cc * 4 + 0) * 128] = xv[cc].x; xw[(cc * 4 + 1) * 128] = xv[cc].y;
                    xw[(cc * 4 + 2) * 128] = xv[cc].z; xw[(cc * 4 + 3) * 128] = xv[cc].w;
                    yw[(cc * 4 + 0) * 128] = yv[cc].x; yw[(cc * 4 + 1) * 128] = yv[cc].y;
                    yw[(cc * 4 + 2) * 128] = yv[cc].z; yw[(cc * 4 + 3) * 128] = yv[cc].w;
                }
                __syncthreads();
            }
            const float *xt = reinterpret_cast<const float *>(xs) + 2 * ti;
            const float *yt = reinterpret_cast<const float *>(ys) + 2 * tj;
#pragma unroll 2
            for (int e = 0; e < 32; ++e) {
                f32x2 x2[R / 2], y2[R / 2], ys2[R / 2];
#pragma unroll
                for (int a = 0; a < R / 2; ++a) x2[a] = *reinterpret_cast<const f32x2 *>(xt + e * 128 + 32 * a);
#pragma unroll
                for (int c = 0; c < R / 2; ++c) {
                    y2[c] = *reinterpret_cast<const f32x2 *>(yt + e * 128 + 32 * c);
                    float lo, hi;
                    unpack2(y2[c], lo, hi);
                    ys2[c] = pack2(hi, lo);
                }
#pragma unroll
                for (int a = 0; a < R / 2; ++a)
#pragma unroll
                    for (int c = 0; c < R / 2; ++c) {
                        // |d|^3 = (d |d|) d: the scalar multiply takes |.| as an operand modifier
                        float lo, hi;
                        const f32x2 da = sub2(x2[a], y2[c]);
                        unpack2(da, lo, hi);
                        pa[a][c] = fma2(pack2(lo * fabsf(lo), hi * fabsf(hi)), da, pa[a][c]);
                        const f32x2 db = sub2(x2[a], ys2[c]);
                        unpack2(db, lo, hi);
                        pb[a][c] = fma2(pack2(lo * fabsf(lo), hi * fabsf(hi)), db, pb[a][c]);
                    }
            }
        } else {
#pragma unroll 1
        for (int c = 0; c < cmax; ++c) {
            V xa[R];
#pragma unroll
            for (int r = 0; r < R; ++r)
                xa[r] = *reinterpret_cast<const V *>(xs + (xrow + 16 * r) * 128u + ((c ^ (xrow & 7u)) << 4));
            T wv[VN];
#pragma unroll
            for (int e = 0; e < VN; ++e) wv[e] = WEIGHTED ? wst[c * VN + e] : T(1);
#pragma unroll
            for (int rj = 0; rj < R; ++rj) {
                V yb = *reinterpret_cast<const V *>(ys + (yrow + 16 * rj) * 128u + ((c ^ (yrow & 7u)) << 4));
                const T *ye = reinterpret_cast<const T *>(&yb);
#pragma unroll
                for (int ri = 0; ri < R; ++ri) {
                    const T *xe = reinterpret_cast<const T *>(&xa[ri]);
#pragma unroll
                    for (int e = 0; e < VN; ++e) {
                        if (KIND == K_MIN) {
                            // zero padding beyond D must not win the minimum
                            if (kbase + c * VN + e < P.D) accumulate<KIND, WEIGHTED, T>(acc[ri][rj], xe[e], ye[e], wv[e], pexp, pspec);
                        } else {
                            accumulate<KIND, WEIGHTED, T>(acc[ri][rj], xe[e], ye[e], wv[e], pexp, pspec);
                        }
                    }
                }
            }
        }
        }
        if (KIND == K_DOT && tid < 2 * TILE) {
            // thread t < TILE sums squares of x1 row t, thread TILE + t of x2 row t
            const unsigned char *rows = tid < TILE ? xs : ys;
            const uint32_t r = tid < TILE ? tid : tid - TILE;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                V v = *reinterpret_cast<const V *>(rows + swz128(r, c));
                const T *ve = reinterpret_cast<const T *>(&v);
#pragma unroll
                for (int e = 0; e < VN; ++e) nsq = t_fma(ve[e], ve[e], nsq);
            }
        }
    }
    if (USE_TMA) {
        if (__syncthreads_or(failed)) {
            if (tid == 0 && P.status) atomicCAS(P.status, 0, (1 << 16) | 2);
            return;
        }
    }

    if (KIND == K_DOT) {
        if (tid < 2 * TILE) norms[tid] = nsq;
        __syncthreads();
    }
    if constexpr (PK) {
#pragma unroll
        for (int a = 0; a < R / 2; ++a)
#pragma unroll
            for (int c = 0; c < R / 2; ++c) {
                float lo, hi;
                unpack2(pa[a][c], lo, hi);
                acc[2 * a][2 * c] = lo; acc[2 * a + 1][2 * c + 1] = hi;
                unpack2(pb[a][c], lo, hi);
                acc[2 * a][2 * c + 1] = lo; acc[2 * a + 1][2 * c] = hi;
            }
    }
    apply_root<T, R, KIND>(acc, P);

    if constexpr (EPI == EPI_ROWMIN) {
        static_assert(sizeof(T) == 4 && sizeof(OutT) == 4, "the row-minimum key packs a 32-bit distance");
        {
            // Streaming row minimum: distances are non-negative, so their float bit patterns order
            // like unsigned integers and the x2 row in the low word breaks ties towards the smaller
            // index. The 16 threads that share an x1 row sit in one half warp: four xor shuffles,
            // then one atomicMin per row and column tile. A NaN distance sorts above +inf.
            unsigned long long *keys = P.rowmin_keys + b * P.N1;
#pragma unroll
            for (int ri = 0; ri < R; ++ri) {
                unsigned long long best = ~0ull;
#pragma unroll
                for (int rj = 0; rj < R; ++rj) {
                    const long long j = j0 + col_of(rj);
                    const float v = (float)finish<T, OutT, KIND>(acc[ri][rj], T(0), T(0), P);
                    const unsigned long long key = ((unsigned long long)__float_as_uint(v) << 32) | (unsigned long long)(uint32_t)j;
                    if (j < P.N2 && key < best) best = key;
                }
#pragma unroll
                for (int off = 1; off < 16; off <<= 1) {
                    const unsigned long long other = __shfl_xor_sync(0xffffffffu, best, off);
                    best = other < best ? other : best;
                }
                const long long i = i0 + row_of(ri);
                if (tj == 0 && i < P.N1) atomicMin(keys + i, best);
            }
            return;
        }
    }

    if constexpr (EPI == EPI_MASK) {
        {
            // Radius test fused into the epilogue: a quarter of the bytes of the float matrix and no second pass.
            unsigned char *mout = P.mask_out + b * P.N1 * P.N2;
            const T thr = static_cast<T>(P.threshold);
            if (P.mask_vec) {
                constexpr int ROWB = TILE + 16;
                static_assert(TILE * ROWB <= kStages * 2 * S::TILE_BYTES, "mask staging tile must fit in the operand stages");
                __syncthreads();
#pragma unroll
                for (int ri = 0; ri < R; ++ri)
#pragma unroll
                    for (int rj = 0; rj < R; ++rj)
                        smem[(row_of(ri)) * ROWB + col_of(rj)] =
                            static_cast<T>(finish<T, OutT, KIND>(acc[ri][rj], T(0), T(0), P)) <= thr ? 1 : 0;
                __syncthreads();
                for (int idx = tid; idx < TILE * (TILE / 16); idx += kThreads) {
                    const int rr = idx / (TILE / 16), cc = idx % (TILE / 16);
                    const long long i = i0 + rr, j = j0 + cc * 16;
                    if (i < P.N1 && j < P.N2) // N2 % 16 == 0: a 16-byte group is entirely inside or outside
                        *reinterpret_cast<uint4 *>(mout + i * P.N2 + j) = *reinterpret_cast<const uint4 *>(smem + rr * ROWB + cc * 16);
                }
            } else {
#pragma unroll
                for (int ri = 0; ri < R; ++ri) {
                    const long long i = i0 + row_of(ri);
                    if (i >= P.N1) continue;
#pragma unroll
                    for (int rj = 0; rj < R; ++rj) {
                        const long long j = j0 + col_of(rj);
                        if (j < P.N2) mout[i * P.N2 + j] = static_cast<T>(finish<T, OutT, KIND>(acc[ri][rj], T(0), T(0), P)) <= thr ? 1 : 0;
                    }
                }
            }
            return;
        }
    }

    if constexpr (EPI == EPI_PDIST) {
        // row i of the condensed layout starts at i (2N - i - 1) / 2 and holds j = i + 1 .. N - 1
        const long long N = P.N1;
        OutT *cond = reinterpret_cast<OutT *>(P.out) + b * (N * (N - 1) / 2);
#pragma unroll
        for (int ri = 0; ri < R; ++ri) {
            const long long i = i0 + row_of(ri);
            if (i >= N) continue;
            OutT *crow = cond + i * (2 * N - i - 1) / 2 - i - 1;
#pragma unroll
            for (int rj = 0; rj < R; ++rj) {
                const long long j = j0 + col_of(rj);
                if (j > i && j < N) crow[j] = finish<T, OutT, KIND>(acc[ri][rj], T(0), T(0), P);
            }
        }
        return;
    }

    OutT *out = reinterpret_cast<OutT *>(P.out) + b * P.N1 * P.N2;
    if (sizeof(OutT) == 4 && P.vec_store) {
        // Full tiles of 4-byte outputs go through shared memory (the operand stages are free now):
        // every warp then writes whole 512-byte row segments with 128-bit stores.
        constexpr int ROWB = (TILE + 16) * 4; // 16 floats of padding: the two x1 rows a warp writes hit disjoint banks
        static_assert(TILE * ROWB <= kStages * 2 * S::TILE_BYTES, "staging tile must fit in the operand stages");
        __syncthreads();
#pragma unroll
        for (int ri = 0; ri < R; ++ri) {
            const T n1 = KIND == K_DOT ? norms[row_of(ri)] : T(0);
#pragma unroll
            for (int rj = 0; rj < R; ++rj) {
                const T n2 = KIND == K_DOT ? norms[TILE + col_of(rj)] : T(0);
                *reinterpret_cast<OutT *>(smem + (row_of(ri)) * ROWB + (col_of(rj)) * 4) =
                    finish<T, OutT, KIND>(acc[ri][rj], n1, n2, P);
            }
        }
        __syncthreads();
        const int warp = tid >> 5, lane = tid & 31;
        const long long jcol = j0 + lane * 4;
#pragma unroll 4
        for (int rr = warp; rr < TILE; rr += kThreads / 32) {
            const long long i = i0 + rr;
            if (i < P.N1 && jcol < P.N2) // N2 % 4 == 0: a float4 is entirely inside or entirely outside
                *reinterpret_cast<float4 *>(out + i * P.N2 + jcol) = *reinterpret_cast<const float4 *>(smem + rr * ROWB + lane * 16);
        }
        return;
    }
#pragma unroll
    for (int ri = 0; ri < R; ++ri) {
        const long long i = i0 + row_of(ri);
        if (i >= P.N1) continue;
        const T n1 = KIND == K_DOT ? norms[row_of(ri)] : T(0);
#pragma unroll
        for (int rj = 0; rj < R; ++rj) {
            const long long j = j0 + col_of(rj);
            if (j >= P.N2) continue;
            const T n2 = KIND == K_DOT ? norms[TILE + col_of(rj)] : T(0);
            out[i * P.N2 + j] = finish<T, OutT, KIND>(acc[ri][rj], n1, n2, P);
        }
    }
}

template <typename T, typename OutT, int KIND, bool WEIGHTED, int EPI = EPI_STORE>
int launch_forward(FwdParams P, cudaStream_t stream) {
    constexpr int R = sizeof(T) == 4 ? 8 : 4;
    typedef FwdSmem<T, R> S;
    P.tiles_i = (P.N1 + S::TILE - 1) / S::TILE;
    P.tiles_j = (P.N2 + S::TILE - 1) / S::TILE;
    const long long tiles = P.B * P.tiles_i * P.tiles_j;
    if (tiles <= 0) return TPW_OK;
    TPW_CHECK_ARG(tiles < (1ll << 31), "lp forward: too many tiles (%lld)", tiles);
    TPW_CHECK_ARG(P.N1 < (1ll << 31) && P.N2 < (1ll << 31) && P.B < (1ll << 31) && P.D < (1ll << 31),
                  "lp forward: a dimension exceeds 2^31-1");
    P.status = device_status_ptr();
    P.vec_store = (sizeof(OutT) == 4 && S::TILE == 128 && P.N2 % 4 == 0 && aligned16(P.out)) ? 1 : 0;

    const bool tma_ok = !tma_disabled() && aligned16(P.x1) && aligned16(P.x2) && (P.D * (long long)sizeof(T)) % 16 == 0 && P.D > 0;
    CUtensorMap m1, m2;
    memset(&m1, 0, sizeof(m1));
    memset(&m2, 0, sizeof(m2));
    if (tma_ok) {
        int st = make_tensor_map_3d(&m1, P.x1, sizeof(T), P.D, P.N1, P.B, S::KC, S::TILE, true);
        if (st != TPW_OK) return st;
        st = make_tensor_map_3d(&m2, P.x2, sizeof(T), P.D, P.N2, P.B, S::KC, S::TILE, true);
        if (st != TPW_OK) return st;
        if (P.D % S::KC == 0) {
            auto kern = lp_forward_kernel<T, OutT, R, KIND, WEIGHTED, true, false, EPI>;
            TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC));
            kern<<<(unsigned)tiles, kThreads, S::ALLOC, stream>>>(m1, m2, P);
        } else {
            auto kern = lp_forward_kernel<T, OutT, R, KIND, WEIGHTED, true, true, EPI>;
            TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC));
            kern<<<(unsigned)tiles, kThreads, S::ALLOC, stream>>>(m1, m2, P);
        }
    } else {
        auto kern = lp_forward_kernel<T, OutT, R, KIND, WEIGHTED, false, true, EPI>;
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC));
        kern<<<(unsigned)tiles, kThreads, S::ALLOC, stream>>>(m1, m2, P);
    }
    TPW_LAUNCH_OK("lp_forward_kernel");
    return TPW_OK;
}

template <typename T, int KIND, int EPI>
int launch_forward_w(const FwdParams &P, cudaStream_t stream) {
    if constexpr (EPI == EPI_STORE) {
        if (P.w) return launch_forward<T, T, KIND, true, EPI>(P, stream);
    }
    return launch_forward<T, T, KIND, false, EPI>(P, stream);
}

template <typename T, int EPI = EPI_STORE>
int lp_forward_typed(FwdParams P, double p, double out_exponent, cudaStream_t stream) {
    P.p = p;
    P.pow_spec = make_pow_spec(p);
    P.out_exponent = out_exponent;
    if (isinf(p)) {
        if constexpr (EPI == EPI_STORE) {
            if (p < 0) return launch_forward_w<T, K_MIN, EPI>(P, stream);
        }
        return launch_forward_w<T, K_MAX, EPI>(P, stream);
    }
    if (out_exponent == 1.0) P.root_mode = 0;
    else if (out_exponent == 0.5) P.root_mode = 1;
    else if (p == 3.0 && out_exponent == 1.0 / 3.0) P.root_mode = 2;
    else P.root_mode = 3;
    if (p == 1.0) return launch_forward_w<T, K_L1, EPI>(P, stream);
    if (p == 2.0) return launch_forward_w<T, K_P2, EPI>(P, stream);
    if (p == 3.0) return launch_forward_w<T, K_P3, EPI>(P, stream);
    return launch_forward_w<T, K_PGEN, EPI>(P, stream);
}

} // namespace
} // namespace tpw
