// L_p forward for few features (D <= 32, float32, unweighted, p in {1, 2, 3, +inf}): the output-bound shapes.
//
// With a handful of features the 128 x 128 register tile spends more on staging operands, barriers and the
// shared-memory epilogue than on arithmetic, and the kernel should be limited by the 4 bytes it writes per
// pair.  Here the roles are fixed instead: every lane keeps JL = 8, 4 or 2 consecutive x2 rows in registers (JL * DP <= 64
// values, DP = D rounded up to 4, 8, 16 or 32), loaded once per CTA; x1 rows pass through shared memory 128 at a
// time (four such tiles per CTA), and the warp walks over them: one broadcast shared load of an x1 row (DP / 4 128-bit loads), 2 * DP * JL arithmetic lane operations,
// and one JL-wide store, so that a warp writes 32 * JL consecutive outputs of one output row with full
// 128-byte lines and nothing is staged.  Features are accumulated in ascending order exactly as the tile
// kernel does, with the same operations; only the square root differs (approximate, within 1 ulp).
#include "common.cuh"

#include <math.h>
#include <stdlib.h>

namespace tpw {
namespace {

enum SmallKind { SK_L1 = 0, SK_P2 = 1, SK_P3 = 2, SK_MAX = 3 };

constexpr int SD_THREADS = 256;
constexpr int SD_ROWS = 128;   // x1 rows per shared-memory tile
constexpr int SD_TILES = 4;    // row tiles per CTA (the x2 registers are loaded once for all of them)

template <int KIND>
__device__ __forceinline__ void sd_acc(float &acc, float x, float y) {
    const float d = x - y;
    if (KIND == SK_L1) acc += fabsf(d);
    else if (KIND == SK_P2) acc = fmaf(d, d, acc);
    else if (KIND == SK_P3) { const float a = fabsf(d); acc = fmaf(a * a, a, acc); }
    else acc = fmaxf(acc, fabsf(d));
}

// root_mode: 0 none, 1 sqrt, 2 cbrt, 3 powf(exponent)
__device__ __forceinline__ float sd_root(float v, int root_mode, float exponent) {
    if (root_mode == 0) return v;
    if (root_mode == 1) {   // one MUFU operation (1 ulp, flush-to-zero): the IEEE sequence would cost as much as D = 8 features
        float r;
        asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
        return r;
    }
    if (root_mode == 2) return cbrtf(v);
    return powf(v, exponent);
}

// MASK: instead of the float matrix, one byte per pair: finished value <= threshold (the radius test), written as
// 4-byte groups so that a warp's store still covers 128 contiguous bytes.
template <int KIND, int DP, int JL, bool MASK>
__global__ void __launch_bounds__(SD_THREADS, 2)
lp_small_d_kernel(const float *__restrict__ x1, const float *__restrict__ x2, float *__restrict__ out,
                  unsigned char *__restrict__ mask, float threshold,
                  long long N1, long long N2, int D, long long tiles_i, long long tiles_j, int root_mode, float exponent,
                  int vec_store, int vec_load) {
    constexpr int COLS = SD_THREADS * JL;   // x2 rows per CTA
    __shared__ __align__(16) float rows[SD_ROWS * DP];
    const long long tile = blockIdx.x;
    const long long tj = tile % tiles_j, ti = (tile / tiles_j) % tiles_i, b = tile / (tiles_j * tiles_i);
    // A lane's columns come in groups of G = min(JL, 4) consecutive x2 rows, the groups of one warp side by side:
    // column(c) = jw + (c / G) * 32 G + lane * G + c % G, so that every store instruction of a warp covers
    // 32 * G consecutive outputs (full lines) however many groups a lane holds.
    constexpr int G = JL < 4 ? JL : 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long jw = tj * COLS + (long long)warp * (32 * JL);
    const long long j0 = jw + lane * G;                       // first column of this lane's first group
    const long long jlast = jw + (JL / G - 1) * (32 * G) + lane * G + G - 1;   // its last column

    // this lane's x2 rows -> registers, once for all row tiles of the CTA (zero padding contributes |0 - 0| = 0);
    // 128-bit loads when the rows are whole 16-byte groups
    float y[JL][DP];
    if (vec_load && jlast < N2) {
#pragma unroll
        for (int c = 0; c < JL; ++c) {
            const float4 *src = reinterpret_cast<const float4 *>(x2 + (b * N2 + j0 + (c / G) * (32 * G) + c % G) * DP);
#pragma unroll
            for (int k4 = 0; k4 < DP / 4; ++k4) {
                const float4 v = __ldg(src + k4);
                y[c][4 * k4] = v.x; y[c][4 * k4 + 1] = v.y; y[c][4 * k4 + 2] = v.z; y[c][4 * k4 + 3] = v.w;
            }
        }
    } else {
#pragma unroll
        for (int c = 0; c < JL; ++c) {
            const long long j = j0 + (c / G) * (32 * G) + c % G;
            const float *src = x2 + (b * N2 + (j < N2 ? j : 0)) * D;
#pragma unroll
            for (int k = 0; k < DP; ++k) y[c][k] = (j < N2 && k < D) ? src[k] : 0.f;
        }
    }

    for (int t = 0; t < SD_TILES; ++t) {
        const long long i0 = (ti * SD_TILES + t) * SD_ROWS;
        if (i0 >= N1) break;
        const int nr = (int)min((long long)SD_ROWS, N1 - i0);
        // x1 rows -> shared memory, zero beyond D and beyond the last row
        const float *x1b = x1 + (b * N1 + i0) * D;
        __syncthreads();
        if (vec_load) {
            const float4 *src = reinterpret_cast<const float4 *>(x1b);
            for (int e = threadIdx.x; e < SD_ROWS * DP / 4; e += SD_THREADS)
                reinterpret_cast<float4 *>(rows)[e] = e < nr * (DP / 4) ? __ldg(src + e) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
            for (int e = threadIdx.x; e < SD_ROWS * DP; e += SD_THREADS) {
                const int r = e / DP, k = e % DP;
                rows[e] = (r < nr && k < D) ? x1b[(long long)r * D + k] : 0.f;
            }
        }
        __syncthreads();
        if (j0 >= N2) continue;

        float *o = MASK ? nullptr : out + (b * N1 + i0) * N2 + j0;
        unsigned char *om = MASK ? mask + (b * N1 + i0) * N2 + j0 : nullptr;
        for (int r = 0; r < nr; ++r) {
            float acc[JL];
#pragma unroll
            for (int c = 0; c < JL; ++c) acc[c] = 0.f;
#pragma unroll
            for (int k4 = 0; k4 < DP; k4 += 4) {
                const float4 xv = *reinterpret_cast<const float4 *>(&rows[r * DP + k4]);
#pragma unroll
                for (int c = 0; c < JL; ++c) {
                    sd_acc<KIND>(acc[c], xv.x, y[c][k4]);
                    sd_acc<KIND>(acc[c], xv.y, y[c][k4 + 1]);
                    sd_acc<KIND>(acc[c], xv.z, y[c][k4 + 2]);
                    sd_acc<KIND>(acc[c], xv.w, y[c][k4 + 3]);
                }
            }
#pragma unroll
            for (int c = 0; c < JL; ++c) acc[c] = sd_root(acc[c], root_mode, exponent);
            if constexpr (MASK) {
                unsigned char *dm = om + (long long)r * N2;
                if (vec_store && jlast < N2) {
                    if constexpr (JL == 2) {
                        *reinterpret_cast<uchar2 *>(dm) = make_uchar2(acc[0] <= threshold, acc[1] <= threshold);
                    } else {
#pragma unroll
                        for (int c = 0; c < JL; c += 4)
                            *reinterpret_cast<uchar4 *>(dm + (c / 4) * 128) =
                                make_uchar4(acc[c] <= threshold, acc[c + 1] <= threshold, acc[c + 2] <= threshold, acc[c + 3] <= threshold);
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < JL; ++c)
                        if (j0 + (c / G) * (32 * G) + c % G < N2) dm[(c / G) * (32 * G) + c % G] = acc[c] <= threshold;
                }
                continue;
            }
            float *dst = o + (long long)r * N2;
            if (vec_store && jlast < N2) {
                if constexpr (JL == 2) {
                    __stcs(reinterpret_cast<float2 *>(dst), make_float2(acc[0], acc[1]));
                } else {
#pragma unroll
                    for (int c = 0; c < JL; c += 4)
                        __stcs(reinterpret_cast<float4 *>(dst + (c / 4) * 128), make_float4(acc[c], acc[c + 1], acc[c + 2], acc[c + 3]));
                }
            } else {
#pragma unroll
                for (int c = 0; c < JL; ++c)
                    if (j0 + (c / G) * (32 * G) + c % G < N2) dst[(c / G) * (32 * G) + c % G] = acc[c];
            }
        }
    }
}

template <int KIND, int DP, int JL, bool MASK>
int launch_small(const float *x1, const float *x2, float *out, unsigned char *mask, float threshold, long long B, long long N1,
                 long long N2, int D, int root_mode, float exponent, cudaStream_t s) {
    const long long ti = (N1 + SD_ROWS * SD_TILES - 1) / (SD_ROWS * SD_TILES), tj = (N2 + SD_THREADS * JL - 1) / (SD_THREADS * JL), tiles = B * ti * tj;
    TPW_CHECK_ARG(tiles < (1ll << 31), "lp forward (few features): too many tiles (%lld)", tiles);
    constexpr int G = JL < 4 ? JL : 4;
    const int vec = MASK ? ((N2 % G == 0 && reinterpret_cast<uintptr_t>(mask) % G == 0) ? 1 : 0)
                         : ((N2 % G == 0 && (reinterpret_cast<uintptr_t>(out) % (JL == 2 ? 8 : 16)) == 0) ? 1 : 0);
    const int vload = (D == DP && reinterpret_cast<uintptr_t>(x1) % 16 == 0 && reinterpret_cast<uintptr_t>(x2) % 16 == 0) ? 1 : 0;
    lp_small_d_kernel<KIND, DP, JL, MASK><<<(unsigned)tiles, SD_THREADS, 0, s>>>(x1, x2, out, mask, threshold, N1, N2, D, ti, tj, root_mode,
                                                                               exponent, vec, vload);
    TPW_LAUNCH_OK("lp_small_d_kernel");
    return TPW_OK;
}

template <int KIND, bool MASK>
int launch_small_d(const float *x1, const float *x2, float *out, unsigned char *mask, float threshold, long long B, long long N1,
                   long long N2, int D, int root_mode, float exponent, cudaStream_t s) {
    if (D <= 4) return launch_small<KIND, 4, 8, MASK>(x1, x2, out, mask, threshold, B, N1, N2, D, root_mode, exponent, s);
    if (D <= 8) return launch_small<KIND, 8, 8, MASK>(x1, x2, out, mask, threshold, B, N1, N2, D, root_mode, exponent, s);
    if (D <= 16) return launch_small<KIND, 16, 4, MASK>(x1, x2, out, mask, threshold, B, N1, N2, D, root_mode, exponent, s);
    return launch_small<KIND, 32, 2, MASK>(x1, x2, out, mask, threshold, B, N1, N2, D, root_mode, exponent, s);
}

template <bool MASK>
int small_d_dispatch(const void *x1, const void *x2, void *out, unsigned char *mask, double threshold, long long B, long long N1,
                     long long N2, long long D, double p, double out_exponent, cudaStream_t s) {
    int root_mode;
    if (isinf(p) || out_exponent == 1.0) root_mode = 0;
    else if (out_exponent == 0.5) root_mode = 1;
    else if (p == 3.0 && out_exponent == 1.0 / 3.0) root_mode = 2;
    else root_mode = 3;
    const float *a = (const float *)x1, *b = (const float *)x2;
    float *o = (float *)out;
    const float ex = (float)out_exponent, th = (float)threshold;
    if (isinf(p)) return launch_small_d<SK_MAX, MASK>(a, b, o, mask, th, B, N1, N2, (int)D, root_mode, ex, s);
    if (p == 1.0) return launch_small_d<SK_L1, MASK>(a, b, o, mask, th, B, N1, N2, (int)D, root_mode, ex, s);
    if (p == 2.0) return launch_small_d<SK_P2, MASK>(a, b, o, mask, th, B, N1, N2, (int)D, root_mode, ex, s);
    return launch_small_d<SK_P3, MASK>(a, b, o, mask, th, B, N1, N2, (int)D, root_mode, ex, s);
}

// ---- streaming row minimum on few features -------------------------------------------------------------------
// The roles are swapped: every lane keeps JL x1 rows in registers together with their running minimum (as the bit
// pattern of the non-negative sum, so that NaN ranks above +inf) and the column that gave it; x2 rows pass through
// shared memory 128 at a time and are read as broadcasts.  Nothing is written per pair and no shuffle is needed:
// per x2 row a lane spends DP / 4 shared loads, 2 * DP * JL arithmetic lane operations and three compare / select
// operations per x1 row.  A CTA covers 256 * JL x1 rows and a range of x2 rows; ranges are merged by one atomicMin
// per x1 row on the key (bits of the finished value << 32 | x2 row), the contract of the tile kernel's epilogue.
// DC <= DP: features actually combined (D = 2 and D = 3 skip the zero padding of the 4-wide shared-memory rows)
template <int KIND, int DP, int JL, int DC>
__global__ void __launch_bounds__(SD_THREADS, 2)
lp_small_d_rowmin_kernel(const float *__restrict__ x1, const float *__restrict__ x2, unsigned long long *__restrict__ keys,
                         long long N1, long long N2, int D, long long tiles_i, long long chunks_j, int tiles_per_chunk,
                         int root_mode, float exponent, int exact_sqrt) {
    __shared__ __align__(16) float cols[SD_ROWS * DP];
    const long long tile = blockIdx.x;
    const long long cj = tile % chunks_j, ti = (tile / chunks_j) % tiles_i, b = tile / (chunks_j * tiles_i);
    const long long i0 = ti * (SD_THREADS * JL) + threadIdx.x;   // this lane's rows: i0 + c * 256 (coalesced loads)
    float x[JL][DP];
    unsigned best[JL], bestj[JL];
#pragma unroll
    for (int c = 0; c < JL; ++c) {
        const long long i = i0 + (long long)c * SD_THREADS;
        const float *src = x1 + (b * N1 + (i < N1 ? i : 0)) * D;
#pragma unroll
        for (int k = 0; k < DP; ++k) x[c][k] = (i < N1 && k < D) ? src[k] : 0.f;
        best[c] = 0xFFFFFFFFu;
        bestj[c] = 0xFFFFFFFFu;
    }
    const long long jbeg = cj * tiles_per_chunk * SD_ROWS;
    for (int t = 0; t < tiles_per_chunk; ++t) {
        const long long j0 = jbeg + (long long)t * SD_ROWS;
        if (j0 >= N2) break;
        const int nc = (int)min((long long)SD_ROWS, N2 - j0);
        const float *x2b = x2 + (b * N2 + j0) * D;
        __syncthreads();
        for (int e = threadIdx.x; e < SD_ROWS * DP; e += SD_THREADS) {
            const int r = e / DP, k = e % DP;
            cols[e] = (r < nc && k < D) ? x2b[(long long)r * D + k] : 0.f;
        }
        __syncthreads();
        for (int r = 0; r < nc; ++r) {
            float acc[JL];
#pragma unroll
            for (int c = 0; c < JL; ++c) acc[c] = 0.f;
#pragma unroll
            for (int k4 = 0; k4 < DP; k4 += 4) {
                const float4 yv = *reinterpret_cast<const float4 *>(&cols[r * DP + k4]);
#pragma unroll
                for (int c = 0; c < JL; ++c) {
                    if (k4 < DC) sd_acc<KIND>(acc[c], x[c][k4], yv.x);
                    if (k4 + 1 < DC) sd_acc<KIND>(acc[c], x[c][k4 + 1], yv.y);
                    if (k4 + 2 < DC) sd_acc<KIND>(acc[c], x[c][k4 + 2], yv.z);
                    if (k4 + 3 < DC) sd_acc<KIND>(acc[c], x[c][k4 + 3], yv.w);
                }
            }
            const unsigned j = (unsigned)(j0 + r);
#pragma unroll
            for (int c = 0; c < JL; ++c) {
                const unsigned bits = __float_as_uint(acc[c]);
                const bool better = bits < best[c];   // strict: the first (smallest) column keeps an exact tie
                best[c] = better ? bits : best[c];
                bestj[c] = better ? j : bestj[c];
            }
        }
    }
#pragma unroll
    for (int c = 0; c < JL; ++c) {
        const long long i = i0 + (long long)c * SD_THREADS;
        if (i < N1 && bestj[c] != 0xFFFFFFFFu) {
            // monotone: the root of the minimum; the square root is the one the matrix-writing kernel of the same
            // problem uses, so that the row minimum equals the minimum of that matrix bit for bit
            const float m = __uint_as_float(best[c]);
            const float v = (root_mode == 1 && exact_sqrt) ? sqrtf(m) : sd_root(m, root_mode, exponent);
            atomicMin(&keys[b * N1 + i], ((unsigned long long)__float_as_uint(v) << 32) | bestj[c]);
        }
    }
}

template <int KIND, int DP, int JL, int DC = DP>
int launch_small_rowmin(const float *x1, const float *x2, unsigned long long *keys, long long B, long long N1, long long N2, int D,
                        int root_mode, float exponent, cudaStream_t s) {
    const long long ti = (N1 + SD_THREADS * JL - 1) / (SD_THREADS * JL);
    const long long col_tiles = (N2 + SD_ROWS - 1) / SD_ROWS;
    // x2 ranges of up to 8 tiles, shortened while the grid would leave SMs idle
    long long per = 8;
    while (per > 1 && B * ti * ((col_tiles + per - 1) / per) < 592) per /= 2;
    const long long cj = (col_tiles + per - 1) / per, tiles = B * ti * cj;
    TPW_CHECK_ARG(tiles < (1ll << 31), "lp row minimum (few features): too many tiles (%lld)", tiles);
    const int exact_sqrt = lp_small_d_eligible(N1, N2, D, 2.0) ? 0 : 1;
    lp_small_d_rowmin_kernel<KIND, DP, JL, DC><<<(unsigned)tiles, SD_THREADS, 0, s>>>(x1, x2, keys, N1, N2, D, ti, cj, (int)per, root_mode, exponent, exact_sqrt);
    TPW_LAUNCH_OK("lp_small_d_rowmin_kernel");
    return TPW_OK;
}

template <int KIND>
int launch_small_d_rowmin(const float *x1, const float *x2, unsigned long long *keys, long long B, long long N1, long long N2, int D,
                          int root_mode, float exponent, cudaStream_t s) {
    if (D <= 2) return launch_small_rowmin<KIND, 4, 8, 2>(x1, x2, keys, B, N1, N2, D, root_mode, exponent, s);
    if (D == 3) return launch_small_rowmin<KIND, 4, 8, 3>(x1, x2, keys, B, N1, N2, D, root_mode, exponent, s);
    if (D <= 4) return launch_small_rowmin<KIND, 4, 8>(x1, x2, keys, B, N1, N2, D, root_mode, exponent, s);
    if (D <= 8) return launch_small_rowmin<KIND, 8, 8>(x1, x2, keys, B, N1, N2, D, root_mode, exponent, s);
    if (D <= 16) return launch_small_rowmin<KIND, 16, 4>(x1, x2, keys, B, N1, N2, D, root_mode, exponent, s);
    return launch_small_rowmin<KIND, 32, 2>(x1, x2, keys, B, N1, N2, D, root_mode, exponent, s);
}

// ---- streaming k nearest rows on few features ------------------------------------------------------------------
// One x1 row per thread: its features and an ascending list of the K smallest keys (bits of the non-negative sum << 32
// | x2 row) stay in registers while the CTA walks over all of x2 through shared memory, 128 rows at a time.  A
// candidate costs the distance arithmetic and one comparison against the list's last key; the unrolled insertion
// (K compare-select pairs) runs only when some lane of the warp has a candidate below its bound, which happens about
// K ln(N2 / K) times per row.  No scratch, no atomics: a thread sees every x2 row of its batch.
constexpr int TK_THREADS = 64;

template <int KIND, int DP, int DC, int K>
__global__ void __launch_bounds__(TK_THREADS)
lp_small_d_topk_kernel(const float *__restrict__ x1, const float *__restrict__ x2, float *__restrict__ vals, long long *__restrict__ inds,
                       long long N1, long long N2, int D, long long tiles_i, int k_out, int root_mode, float exponent, int exact_sqrt) {
    __shared__ __align__(16) float cols[SD_ROWS * DP];
    const long long b = blockIdx.x / tiles_i, i = (blockIdx.x % tiles_i) * TK_THREADS + threadIdx.x;
    float x[DP];
    {
        const float *src = x1 + (b * N1 + (i < N1 ? i : 0)) * D;
#pragma unroll
        for (int k = 0; k < DP; ++k) x[k] = (i < N1 && k < D) ? src[k] : 0.f;
    }
    unsigned long long list[K];
#pragma unroll
    for (int t = 0; t < K; ++t) list[t] = ~0ull;
    for (long long j0 = 0; j0 < N2; j0 += SD_ROWS) {
        const int nc = (int)min((long long)SD_ROWS, N2 - j0);
        const float *x2b = x2 + (b * N2 + j0) * D;
        __syncthreads();
        for (int e = threadIdx.x; e < SD_ROWS * DP; e += TK_THREADS) {
            const int r = e / DP, k = e % DP;
            cols[e] = (r < nc && k < D) ? x2b[(long long)r * D + k] : 0.f;
        }
        __syncthreads();
#pragma unroll 4
        for (int r = 0; r < nc; ++r) {   // four candidates in flight: their shared loads and sums overlap, the filters follow
            float acc = 0.f;
#pragma unroll
            for (int k4 = 0; k4 < DP; k4 += 4) {
                const float4 yv = *reinterpret_cast<const float4 *>(&cols[r * DP + k4]);
                if (k4 < DC) sd_acc<KIND>(acc, x[k4], yv.x);
                if (k4 + 1 < DC) sd_acc<KIND>(acc, x[k4 + 1], yv.y);
                if (k4 + 2 < DC) sd_acc<KIND>(acc, x[k4 + 2], yv.z);
                if (k4 + 3 < DC) sd_acc<KIND>(acc, x[k4 + 3], yv.w);
            }
            // one 32-bit comparison per candidate; a value equal to the bound passes too, and the insertion below leaves
            // the list unchanged for a key that is not smaller than its last entry
            if (__float_as_uint(acc) <= (unsigned)(list[K - 1] >> 32)) {
                const unsigned long long key = ((unsigned long long)__float_as_uint(acc) << 32) | (unsigned)(j0 + r);
#pragma unroll
                for (int t = K - 1; t > 0; --t) {
                    const unsigned long long below = list[t - 1];
                    list[t] = key < below ? below : (key < list[t] ? key : list[t]);
                }
                list[0] = key < list[0] ? key : list[0];
            }
        }
    }
    if (i >= N1) return;
    float *vo = vals + (b * N1 + i) * k_out;
    long long *io = inds + (b * N1 + i) * k_out;
#pragma unroll
    for (int t = 0; t < K; ++t) {
        if (t < k_out) {
            const float m = __uint_as_float((unsigned)(list[t] >> 32));
            vo[t] = (root_mode == 1 && exact_sqrt) ? sqrtf(m) : sd_root(m, root_mode, exponent);
            io[t] = (long long)(unsigned)(list[t] & 0xFFFFFFFFull);
        }
    }
}

template <int KIND, int DP, int DC>
int launch_small_topk(const float *x1, const float *x2, float *vals, long long *inds, long long B, long long N1, long long N2, int D,
                      int k, int root_mode, float exponent, cudaStream_t s) {
    const long long ti = (N1 + TK_THREADS - 1) / TK_THREADS, tiles = B * ti;
    TPW_CHECK_ARG(tiles < (1ll << 31), "lp k nearest (few features): too many tiles (%lld)", tiles);
    const int ex = lp_small_d_eligible(N1, N2, D, 2.0) ? 0 : 1;
#define TPW_TOPK(KK) lp_small_d_topk_kernel<KIND, DP, DC, KK><<<(unsigned)tiles, TK_THREADS, 0, s>>>(x1, x2, vals, inds, N1, N2, D, ti, k, root_mode, exponent, ex)
    if (k <= 4) TPW_TOPK(4);
    else if (k <= 8) TPW_TOPK(8);
    else TPW_TOPK(16);
#undef TPW_TOPK
    TPW_LAUNCH_OK("lp_small_d_topk_kernel");
    return TPW_OK;
}

template <int KIND>
int launch_small_d_topk(const float *x1, const float *x2, float *vals, long long *inds, long long B, long long N1, long long N2, int D,
                        int k, int root_mode, float exponent, cudaStream_t s) {
    if (D <= 2) return launch_small_topk<KIND, 4, 2>(x1, x2, vals, inds, B, N1, N2, D, k, root_mode, exponent, s);
    if (D == 3) return launch_small_topk<KIND, 4, 3>(x1, x2, vals, inds, B, N1, N2, D, k, root_mode, exponent, s);
    if (D <= 4) return launch_small_topk<KIND, 4, 4>(x1, x2, vals, inds, B, N1, N2, D, k, root_mode, exponent, s);
    if (D <= 8) return launch_small_topk<KIND, 8, 8>(x1, x2, vals, inds, B, N1, N2, D, k, root_mode, exponent, s);
    return launch_small_topk<KIND, 16, 16>(x1, x2, vals, inds, B, N1, N2, D, k, root_mode, exponent, s);
}

} // namespace

// Whether the few-feature kernel serves this float32 problem: D <= 32, an exponent with a closed form, and
// enough output rows and columns for its fixed roles to pay (a CTA covers up to 512 x1 rows and 512 to 2048 x2
// rows; small problems stay on the tile kernel).
bool lp_small_d_eligible(long long N1, long long N2, long long D, double p) {
    if (getenv("TPW_DISABLE_SMALL_D")) return false;
    return D >= 1 && D <= 32 && N1 >= 128 && N2 >= 1024 && (p == 1.0 || p == 2.0 || p == 3.0 || (isinf(p) && p > 0));
}

int lp_small_d_forward(const void *x1, const void *x2, void *out, long long B, long long N1, long long N2, long long D,
                       double p, double out_exponent, cudaStream_t s) {
    return small_d_dispatch<false>(x1, x2, out, nullptr, 0.0, B, N1, N2, D, p, out_exponent, s);
}

// mask[b,i,j] = finished value <= radius, one byte per pair; same eligibility as the matrix-writing kernel
int lp_small_d_mask(const void *x1, const void *x2, unsigned char *mask, long long B, long long N1, long long N2, long long D,
                    double p, double out_exponent, double radius, cudaStream_t s) {
    return small_d_dispatch<true>(x1, x2, nullptr, mask, radius, B, N1, N2, D, p, out_exponent, s);
}

} // namespace tpw

namespace tpw {

// The row-minimum variant: same exponents, at least 2048 x1 rows (a CTA holds 512 to 2048 of them) and 128 x2 rows.
bool lp_small_d_rowmin_eligible(long long N1, long long N2, long long D, double p) {
    if (getenv("TPW_DISABLE_SMALL_D")) return false;
    return D >= 1 && D <= 32 && N1 >= 2048 && N2 >= 128 && (p == 1.0 || p == 2.0 || p == 3.0 || (isinf(p) && p > 0));
}

// keys: B * N1 64-bit keys already set to all ones
int lp_small_d_rowmin(const void *x1, const void *x2, unsigned long long *keys, long long B, long long N1, long long N2, long long D,
                      double p, double out_exponent, cudaStream_t s) {
    int root_mode;
    if (isinf(p) || out_exponent == 1.0) root_mode = 0;
    else if (out_exponent == 0.5) root_mode = 1;
    else if (p == 3.0 && out_exponent == 1.0 / 3.0) root_mode = 2;
    else root_mode = 3;
    const float *a = (const float *)x1, *b = (const float *)x2;
    const float ex = (float)out_exponent;
    if (isinf(p)) return launch_small_d_rowmin<SK_MAX>(a, b, keys, B, N1, N2, (int)D, root_mode, ex, s);
    if (p == 1.0) return launch_small_d_rowmin<SK_L1>(a, b, keys, B, N1, N2, (int)D, root_mode, ex, s);
    if (p == 2.0) return launch_small_d_rowmin<SK_P2>(a, b, keys, B, N1, N2, (int)D, root_mode, ex, s);
    return launch_small_d_rowmin<SK_P3>(a, b, keys, B, N1, N2, (int)D, root_mode, ex, s);
}

} // namespace tpw

namespace tpw {

int lp_small_d_topk(const void *x1, const void *x2, float *vals, long long *inds, long long B, long long N1, long long N2, long long D,
                    int k, double p, double out_exponent, cudaStream_t s) {
    int root_mode;
    if (isinf(p) || out_exponent == 1.0) root_mode = 0;
    else if (out_exponent == 0.5) root_mode = 1;
    else if (p == 3.0 && out_exponent == 1.0 / 3.0) root_mode = 2;
    else root_mode = 3;
    const float *a = (const float *)x1, *b = (const float *)x2;
    const float ex = (float)out_exponent;
    if (isinf(p)) return launch_small_d_topk<SK_MAX>(a, b, vals, inds, B, N1, N2, (int)D, k, root_mode, ex, s);
    if (p == 1.0) return launch_small_d_topk<SK_L1>(a, b, vals, inds, B, N1, N2, (int)D, k, root_mode, ex, s);
    if (p == 2.0) return launch_small_d_topk<SK_P2>(a, b, vals, inds, B, N1, N2, (int)D, k, root_mode, ex, s);
    return launch_small_d_topk<SK_P3>(a, b, vals, inds, B, N1, N2, (int)D, k, root_mode, ex, s);
}

} // namespace tpw

extern "C" int tpw_lp_topk_max_features() { return 16; }
extern "C" int tpw_lp_topk_max_k() { return 16; }

extern "C" int tpw_lp_topk_forward(int dtype, const void *x1, const void *x2, float *vals, int64_t *inds,
                                   int64_t B, int64_t N1, int64_t N2, int64_t D, int k, double p, double out_exponent,
                                   tpw_stream_t stream) {
    using namespace tpw;
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32, "tpw_lp_topk_forward: dtype must be TPW_F32");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_lp_topk_forward: negative size");
    TPW_CHECK_ARG(k >= 1 && k <= 16 && k <= N2, "tpw_lp_topk_forward: k must be in [1, min(16, N2)] (got %d)", k);
    TPW_CHECK_ARG(D >= 1 && D <= 16, "tpw_lp_topk_forward: D must be in [1, 16] (got %lld)", (long long)D);
    TPW_CHECK_ARG(p == 1.0 || p == 2.0 || p == 3.0 || (isinf(p) && p > 0), "tpw_lp_topk_forward: p must be 1, 2, 3 or +inf (got %g)", p);
    TPW_CHECK_ARG(!isnan(out_exponent), "tpw_lp_topk_forward: NaN exponent");
    TPW_CHECK_ARG(N2 < (1ll << 32), "tpw_lp_topk_forward: N2 must fit 32 bits");
    if (B == 0 || N1 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && vals && inds, "tpw_lp_topk_forward: NULL pointer");
    return lp_small_d_topk(x1, x2, vals, reinterpret_cast<long long *>(inds), B, N1, N2, D, k, p, out_exponent,
                           static_cast<cudaStream_t>(stream));
}
