// Directed Hausdorff distance between point sets, fused so that the [M1, M2] distance matrix is
// never written.
//
// Fast path (float32, D <= 16): a CTA of 256 threads owns 1024 points of x1 for one set pair;
// each thread keeps four of them in registers and streams the whole x2 cloud through shared
// memory (one broadcast 128-bit load per x2 point, two for D > 4, feeds four point pairs).  Only the running row
// minimum is kept in the hot loop.  Row minima are packed as (float bits << 32 | visiting
// position of m), reduced with warp shuffles, and merged across CTAs with one 64-bit atomicMax
// per warp: the float bits of a non-negative value order like the value, and the low word makes
// the LAST visited m win ties, which is the rule of the reference loop.  A finishing kernel then
// recomputes the single winning row to find the FIRST visited n reaching its minimum, and writes
// sqrt(max), m*, n*.
//
// Squared distances are accumulated coordinate by coordinate with separately rounded multiply and
// add (no FMA contraction), i.e. bit-for-bit what the reference's CPU loop computes, so the
// selected indices agree with it whenever they are determined at all.
//
// With caller-provided scratch the hot loop does not pay for that: it forms the squared distance
// with fused multiply-adds (3 subtractions, 1 multiplication, 2 fused multiply-adds and the minimum:
// 7 operations per point pair instead of 9), which is within a few units in the last place of the
// separately rounded value, and stores every row's approximate minimum.  The finishing kernel then
// re-evaluates, with the exact arithmetic, only the rows whose approximate minimum lies within that
// error of the largest one (usually one or two per set pair) and applies the tie rules to them, so
// values and indices are still bit-identical to the exact path.
//
// Any other dtype / feature count runs a plain one-CTA-per-set-pair kernel with the same rules.
#include "common.cuh"

#include <math.h>
#include <stdlib.h>

#include <atomic>

namespace tpw {
namespace {

constexpr int kThreads = 256;
constexpr int PM = 4;            // x1 points per thread
constexpr int CHUNK_VECS = 2048; // float4 slots staged per pass (32 KB): 2048 x2 points of up to 4 features, 1024 of up to 8

__device__ __forceinline__ float sqdist_exact(const float *a, const float *b, int D) {
    float d = 0.f;
    for (int k = 0; k < D; ++k) {
        const float diff = __fsub_rn(a[k], b[k]);
        d = __fadd_rn(d, __fmul_rn(diff, diff));
    }
    return d;
}
__device__ __forceinline__ double sqdist_exact(const double *a, const double *b, int D) {
    double d = 0.0;
    for (int k = 0; k < D; ++k) {
        const double diff = __dsub_rn(a[k], b[k]);
        d = __dadd_rn(d, __dmul_rn(diff, diff));
    }
    return d;
}

struct HdParams {
    const void *x1, *x2;
    const long long *order1, *order2;
    void *out;
    long long *idx1, *idx2;
    unsigned long long *keys;
    float *rowmins;   // [pairs, M1] approximate row minima (fused path only)
    long long B, N1, N2, M1, M2, D;
    long long mtiles;
};

// An upper bound on the relative difference between the fused and the separately rounded sum of up to 8 squares
// (each is within D roundings of the real sum, all terms non-negative), with room to spare; below kTiny the
// relative bound gives way to an absolute one (products that underflow).
constexpr float kFusedSlack = 3.8146973e-6f;   // 2^-18
constexpr float kTiny = 1e-35f;
// 9 to 16 squares: (3 D - 1) roundings of 2^-24 between the two sums stay below 2^-17
template <int D> __device__ __forceinline__ constexpr float fused_slack() { return D <= 8 ? kFusedSlack : 2.f * kFusedSlack; }
constexpr int kMaxFastD = 16;                  // widest point the streamed kernels are instantiated for

// keys[pair] = max over m of (bits(rowmin) << 32 | position(m)).  FUSED: the distance is formed with fused
// multiply-adds and every row's minimum is also stored for the refining kernel.
template <int D, bool FUSED>
__global__ void __launch_bounds__(kThreads)
hausdorff_rowmin_kernel(const HdParams P) {
    constexpr int V = (D + 3) / 4;           // float4 slots per x2 point
    constexpr int CHUNK = CHUNK_VECS / V;
    __shared__ float4 pts[CHUNK_VECS];
    const int tid = threadIdx.x;
    long long blk = blockIdx.x;
    const long long mt = blk % P.mtiles;
    blk /= P.mtiles;
    const long long pair = blk; // (b*N1 + i)*N2 + j
    const long long j = pair % P.N2;
    const long long bi = pair / P.N2;
    const long long b = bi / P.N1;
    const float *x1 = reinterpret_cast<const float *>(P.x1) + bi * P.M1 * D;
    const float *x2 = reinterpret_cast<const float *>(P.x2) + (b * P.N2 + j) * P.M2 * D;

    float px[PM][D];
    float rowmin[PM];
    long long mm[PM];
#pragma unroll
    for (int q = 0; q < PM; ++q) {
        mm[q] = mt * (kThreads * PM) + q * kThreads + tid;
        rowmin[q] = INFINITY;
#pragma unroll
        for (int k = 0; k < D; ++k) px[q][k] = mm[q] < P.M1 ? x1[mm[q] * D + k] : 0.f;
    }

    for (long long n0 = 0; n0 < P.M2; n0 += CHUNK) {
        const int cnt = (int)((P.M2 - n0) < CHUNK ? (P.M2 - n0) : CHUNK);
        __syncthreads();
        for (int e = tid; e < cnt; e += kThreads) {
            const float *s = x2 + (n0 + e) * D;
            float c[4 * V];
#pragma unroll
            for (int k = 0; k < 4 * V; ++k) c[k] = k < D ? s[k] : 0.f;
#pragma unroll
            for (int v = 0; v < V; ++v) pts[e * V + v] = make_float4(c[4 * v], c[4 * v + 1], c[4 * v + 2], c[4 * v + 3]);
        }
        __syncthreads();
#pragma unroll 4
        for (int e = 0; e < cnt; ++e) {
            float c[4 * V];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const float4 t = pts[e * V + v];
                c[4 * v] = t.x; c[4 * v + 1] = t.y; c[4 * v + 2] = t.z; c[4 * v + 3] = t.w;
            }
#pragma unroll
            for (int q = 0; q < PM; ++q) {
                float d = 0.f;
#pragma unroll
                for (int k = 0; k < D; ++k) {
                    const float diff = __fsub_rn(px[q][k], c[k]);
                    if (FUSED) d = k == 0 ? __fmul_rn(diff, diff) : __fmaf_rn(diff, diff, d);
                    else d = __fadd_rn(d, __fmul_rn(diff, diff));
                }
                rowmin[q] = fminf(rowmin[q], d);
            }
        }
    }

    unsigned long long key = 0ull;
#pragma unroll
    for (int q = 0; q < PM; ++q) {
        if (mm[q] < P.M1) {
            if (FUSED) P.rowmins[pair * P.M1 + mm[q]] = rowmin[q];
            const unsigned long long pos =
                (unsigned long long)(P.order1 ? P.order1[b * P.M1 + mm[q]] : mm[q]);
            const unsigned long long kq = ((unsigned long long)__float_as_uint(rowmin[q]) << 32) | (pos & 0xffffffffull);
            key = kq > key ? kq : key;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, key, off);
        key = other > key ? other : key;
    }
    if ((tid & 31) == 0) atomicMax(P.keys + pair, key);
}

// One CTA per set pair: decode the winning m, recompute its row, pick the first visited n.
template <int D>
__global__ void __launch_bounds__(kThreads)
hausdorff_finish_kernel(const HdParams P) {
    __shared__ unsigned long long best;
    __shared__ long long mstar_s;
    const int tid = threadIdx.x;
    const long long pair = blockIdx.x;
    const long long j = pair % P.N2;
    const long long bi = pair / P.N2;
    const long long b = bi / P.N1;
    const float *x1 = reinterpret_cast<const float *>(P.x1) + bi * P.M1 * D;
    const float *x2 = reinterpret_cast<const float *>(P.x2) + (b * P.N2 + j) * P.M2 * D;
    const unsigned long long key = P.keys[pair];
    const unsigned int pos = (unsigned int)(key & 0xffffffffull);
    if (tid == 0) {
        best = ~0ull;
        mstar_s = P.order1 ? -1 : (long long)pos;
    }
    __syncthreads();
    if (P.order1) {
        for (long long m = tid; m < P.M1; m += kThreads)
            if ((unsigned int)P.order1[b * P.M1 + m] == pos) mstar_s = m;
        __syncthreads();
    }
    const long long mstar = mstar_s;
    float a[D];
#pragma unroll
    for (int k = 0; k < D; ++k) a[k] = (mstar >= 0 && mstar < P.M1) ? x1[mstar * D + k] : 0.f;
    unsigned long long mine = ~0ull;
    for (long long n = tid; n < P.M2; n += kThreads) {
        float c[D];
#pragma unroll
        for (int k = 0; k < D; ++k) c[k] = x2[n * D + k];
        const float d = sqdist_exact(a, c, D);
        const unsigned long long p2 = (unsigned long long)(P.order2 ? P.order2[b * P.M2 + n] : n);
        const unsigned long long kq = ((unsigned long long)__float_as_uint(d) << 32) | (p2 & 0xffffffffull);
        mine = kq < mine ? kq : mine;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, off);
        mine = other < mine ? other : mine;
    }
    if ((tid & 31) == 0) atomicMin(&best, mine);
    __syncthreads();
    const unsigned int npos = (unsigned int)(best & 0xffffffffull);
    if (P.order2) {
        for (long long n = tid; n < P.M2; n += kThreads)
            if ((unsigned int)P.order2[b * P.M2 + n] == npos) P.idx2[pair] = n;
    } else if (tid == 0) {
        P.idx2[pair] = P.M2 > 0 ? (long long)npos : 0;
    }
    if (tid == 0) {
        const float cmax = __uint_as_float((unsigned int)(key >> 32));
        reinterpret_cast<float *>(P.out)[pair] = sqrtf(cmax);
        P.idx1[pair] = mstar >= 0 ? mstar : 0;
    }
}

// Fused path: one CTA per set pair.  Every row whose approximate minimum could be the exact maximum is re-evaluated with
// the separately rounded arithmetic by one warp (lanes over n, first visited n on ties); the largest exact minimum wins,
// the last visited m on ties.
template <int D>
__global__ void __launch_bounds__(kThreads)
hausdorff_refine_kernel(const HdParams P) {
    constexpr int kWarps = kThreads / 32;
    __shared__ unsigned long long s_row[kWarps], s_n[kWarps];
    __shared__ long long s_m[kWarps];
    __shared__ long long s_nstar;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const long long pair = blockIdx.x;
    const long long j = pair % P.N2;
    const long long bi = pair / P.N2;
    const long long b = bi / P.N1;
    const float *x1 = reinterpret_cast<const float *>(P.x1) + bi * P.M1 * D;
    const float *x2 = reinterpret_cast<const float *>(P.x2) + (b * P.N2 + j) * P.M2 * D;
    const float *rm = P.rowmins + pair * P.M1;
    const unsigned long long key = P.keys[pair];
    const float amax = __uint_as_float((unsigned int)(key >> 32));
    const unsigned int pos_max = (unsigned int)(key & 0xffffffffull);
    // An approximate minimum of exactly 0 means every difference squared to 0, in either arithmetic: all rows then
    // tie at 0 and the last visited one, which the key already names, wins.  Otherwise a row can hold the exact
    // maximum only if its approximate minimum is within the rounding slack of the largest approximate minimum.
    const bool all_zero = amax == 0.f;
    const float lower = amax * (1.f - fused_slack<D>()) - kTiny;

    unsigned long long wrow = 0ull, wn = ~0ull;   // best (bits(min) << 32 | position(m)) of this warp, its n key
    long long wm = -1;
    for (long long base = (long long)warp * 32; base < P.M1; base += kThreads) {
        const long long m = base + lane;
        unsigned int pos = 0;
        bool cand = false;
        if (m < P.M1) {
            pos = (unsigned int)(P.order1 ? P.order1[b * P.M1 + m] : m);
            cand = all_zero ? (pos == pos_max) : (rm[m] >= lower);
        }
        unsigned int todo = __ballot_sync(0xffffffffu, cand);
        while (todo) {
            const int src = __ffs(todo) - 1;
            todo &= todo - 1;
            const long long mc = base + src;
            const unsigned int posc = __shfl_sync(0xffffffffu, pos, src);
            float a[D];
#pragma unroll
            for (int k = 0; k < D; ++k) a[k] = x1[mc * D + k];
            unsigned long long mine = ~0ull;
            for (long long n = lane; n < P.M2; n += 32) {
                float c[D];
#pragma unroll
                for (int k = 0; k < D; ++k) c[k] = x2[n * D + k];
                const float d = sqdist_exact(a, c, D);
                if (d == d) {   // a NaN distance never lowers a minimum
                    const unsigned long long p2 = (unsigned long long)(P.order2 ? P.order2[b * P.M2 + n] : n);
                    const unsigned long long kq = ((unsigned long long)__float_as_uint(d) << 32) | (p2 & 0xffffffffull);
                    mine = kq < mine ? kq : mine;
                }
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                const unsigned long long other = __shfl_xor_sync(0xffffffffu, mine, off);
                mine = other < mine ? other : mine;
            }
            // a row without any comparable distance has the minimum +inf, as in the streaming kernel
            const unsigned int vbits = mine == ~0ull ? 0x7f800000u : (unsigned int)(mine >> 32);
            const unsigned long long rkey = ((unsigned long long)vbits << 32) | posc;
            if (wm < 0 || rkey > wrow) { wrow = rkey; wn = mine; wm = mc; }
        }
    }
    if (lane == 0) { s_row[warp] = wrow; s_n[warp] = wn; s_m[warp] = wm; }
    __syncthreads();
    int bw = -1;
    for (int w = 0; w < kWarps; ++w)
        if (s_m[w] >= 0 && (bw < 0 || s_row[w] > s_row[bw])) bw = w;
    if (bw < 0) {   // cannot happen for M1 > 0: the row the key names is always a candidate
        if (tid == 0) { reinterpret_cast<float *>(P.out)[pair] = sqrtf(amax); P.idx1[pair] = 0; P.idx2[pair] = 0; }
        return;
    }
    const unsigned int npos = (unsigned int)(s_n[bw] & 0xffffffffull);
    if (tid == 0) s_nstar = (P.order2 || s_n[bw] == ~0ull) ? 0 : (long long)npos;
    __syncthreads();
    if (P.order2 && s_n[bw] != ~0ull) {
        for (long long n = tid; n < P.M2; n += kThreads)
            if ((unsigned int)P.order2[b * P.M2 + n] == npos) s_nstar = n;
        __syncthreads();
    }
    if (tid == 0) {
        reinterpret_cast<float *>(P.out)[pair] = sqrtf(__uint_as_float((unsigned int)(s_row[bw] >> 32)));
        P.idx1[pair] = s_m[bw];
        P.idx2[pair] = s_nstar;
    }
}

// ---- float64, D <= 16: the same streaming design ------------------------------------------------------------------------
// A 64-bit distance leaves no room for the visiting position in a 64-bit key, so every row's exact minimum is stored
// (8 bytes per x1 point in the caller's scratch) and one CTA per set pair then scans them: largest minimum, last
// visited row on ties, and for that row the first visited x2 point that attains it.  Products and sums are rounded
// separately, as in the reference's CPU loop, so values and indices equal the one-CTA-per-pair kernel's bit for bit.
constexpr int PMD = 2;             // x1 points per thread
constexpr int CHUNK_D = 4096;      // doubles staged per pass (32 KB)

template <int D>
__global__ void __launch_bounds__(kThreads)
hausdorff_rowmin_f64_kernel(const HdParams P) {
    constexpr int CHUNK = CHUNK_D / D;
    __shared__ double pts[CHUNK_D];
    const int tid = threadIdx.x;
    long long blk = blockIdx.x;
    const long long mt = blk % P.mtiles;
    const long long pair = blk / P.mtiles;
    const long long j = pair % P.N2;
    const long long bi = pair / P.N2;
    const long long b = bi / P.N1;
    const double *x1 = reinterpret_cast<const double *>(P.x1) + bi * P.M1 * D;
    const double *x2 = reinterpret_cast<const double *>(P.x2) + (b * P.N2 + j) * P.M2 * D;
    double px[PMD][D], rowmin[PMD];
    long long mm[PMD];
#pragma unroll
    for (int q = 0; q < PMD; ++q) {
        mm[q] = mt * (kThreads * PMD) + q * kThreads + tid;
        rowmin[q] = INFINITY;
#pragma unroll
        for (int k = 0; k < D; ++k) px[q][k] = mm[q] < P.M1 ? x1[mm[q] * D + k] : 0.0;
    }
    for (long long n0 = 0; n0 < P.M2; n0 += CHUNK) {
        const int cnt = (int)((P.M2 - n0) < CHUNK ? (P.M2 - n0) : CHUNK);
        __syncthreads();
        for (int e = tid; e < cnt * D; e += kThreads) pts[e] = x2[n0 * D + e];
        __syncthreads();
#pragma unroll 2
        for (int e = 0; e < cnt; ++e) {
            double c[D];
#pragma unroll
            for (int k = 0; k < D; ++k) c[k] = pts[e * D + k];
#pragma unroll
            for (int q = 0; q < PMD; ++q) rowmin[q] = fmin(rowmin[q], sqdist_exact(px[q], c, D));
        }
    }
    double *rm = reinterpret_cast<double *>(P.rowmins) + pair * P.M1;
#pragma unroll
    for (int q = 0; q < PMD; ++q)
        if (mm[q] < P.M1) rm[mm[q]] = rowmin[q];
}

template <int D>
__global__ void __launch_bounds__(kThreads)
hausdorff_finish_f64_kernel(const HdParams P) {
    __shared__ double s_val[kThreads];
    __shared__ long long s_pos[kThreads], s_m[kThreads];
    __shared__ unsigned long long s_npos[kThreads];
    __shared__ long long s_nstar;
    const int tid = threadIdx.x;
    const long long pair = blockIdx.x;
    const long long j = pair % P.N2;
    const long long bi = pair / P.N2;
    const long long b = bi / P.N1;
    const double *x1 = reinterpret_cast<const double *>(P.x1) + bi * P.M1 * D;
    const double *x2 = reinterpret_cast<const double *>(P.x2) + (b * P.N2 + j) * P.M2 * D;
    const double *rm = reinterpret_cast<const double *>(P.rowmins) + pair * P.M1;
    // largest row minimum, the last visited row on ties
    double best = -1.0;
    long long best_pos = -1, best_m = 0;
    for (long long m = tid; m < P.M1; m += kThreads) {
        const double v = rm[m];
        const long long p1 = P.order1 ? P.order1[b * P.M1 + m] : m;
        if (v > best || (v == best && p1 > best_pos)) { best = v; best_pos = p1; best_m = m; }
    }
    s_val[tid] = best; s_pos[tid] = best_pos; s_m[tid] = best_m;
    __syncthreads();
    for (int off = kThreads / 2; off > 0; off >>= 1) {
        if (tid < off) {
            const double v = s_val[tid + off];
            const long long p = s_pos[tid + off];
            if (v > s_val[tid] || (v == s_val[tid] && p > s_pos[tid])) { s_val[tid] = v; s_pos[tid] = p; s_m[tid] = s_m[tid + off]; }
        }
        __syncthreads();
    }
    const long long mstar = s_m[0];
    const double cmax = s_pos[0] >= 0 ? s_val[0] : 0.0;
    // the first visited x2 point at the row's minimum distance
    double a[D];
#pragma unroll
    for (int k = 0; k < D; ++k) a[k] = x1[mstar * D + k];
    unsigned long long mine = ~0ull;     // visiting position of the best candidate of this thread
    long long mine_n = 0;
    for (long long n = tid; n < P.M2; n += kThreads) {
        double c[D];
#pragma unroll
        for (int k = 0; k < D; ++k) c[k] = x2[n * D + k];
        if (sqdist_exact(a, c, D) == cmax) {
            const unsigned long long p2 = (unsigned long long)(P.order2 ? P.order2[b * P.M2 + n] : n);
            if (p2 < mine) { mine = p2; mine_n = n; }
        }
    }
    s_npos[tid] = mine; s_pos[tid] = mine_n;
    __syncthreads();
    for (int off = kThreads / 2; off > 0; off >>= 1) {
        if (tid < off && s_npos[tid + off] < s_npos[tid]) { s_npos[tid] = s_npos[tid + off]; s_pos[tid] = s_pos[tid + off]; }
        __syncthreads();
    }
    if (tid == 0) {
        s_nstar = s_npos[0] == ~0ull ? 0 : s_pos[0];
        reinterpret_cast<double *>(P.out)[pair] = sqrt(cmax);
        P.idx1[pair] = mstar;
        P.idx2[pair] = s_nstar;
    }
}

template <int D>
int launch_f64(HdParams P, cudaStream_t s) {
    const long long pairs = P.B * P.N1 * P.N2;
    P.mtiles = (P.M1 + kThreads * PMD - 1) / (kThreads * PMD);
    const long long blocks = pairs * P.mtiles;
    TPW_CHECK_ARG(blocks < (1ll << 31), "hausdorff: too many blocks");
    hausdorff_rowmin_f64_kernel<D><<<(unsigned)blocks, kThreads, 0, s>>>(P);
    TPW_LAUNCH_OK("hausdorff_rowmin_f64_kernel");
    hausdorff_finish_f64_kernel<D><<<(unsigned)pairs, kThreads, 0, s>>>(P);
    TPW_LAUNCH_OK("hausdorff_finish_f64_kernel");
    return TPW_OK;
}

// Plain path: any dtype, any D.  One CTA per set pair; thread t scans rows m = t, t+256, ...
template <typename T>
__global__ void __launch_bounds__(kThreads)
hausdorff_plain_kernel(const HdParams P) {
    __shared__ T s_val[kThreads];
    __shared__ long long s_pos[kThreads], s_m[kThreads], s_n[kThreads];
    const int tid = threadIdx.x;
    const long long pair = blockIdx.x;
    const long long j = pair % P.N2;
    const long long bi = pair / P.N2;
    const long long b = bi / P.N1;
    const int D = (int)P.D;
    const T *x1 = reinterpret_cast<const T *>(P.x1) + bi * P.M1 * D;
    const T *x2 = reinterpret_cast<const T *>(P.x2) + (b * P.N2 + j) * P.M2 * D;

    T best = T(-1);
    long long best_pos = -1, best_m = 0, best_n = 0;
    for (long long m = tid; m < P.M1; m += kThreads) {
        T rowmin = T(INFINITY);
        long long rn = 0, rpos = 0x7fffffffffffffffll;
        for (long long n = 0; n < P.M2; ++n) {
            const T d = sqdist_exact(x1 + m * D, x2 + n * D, D);
            const long long p2 = P.order2 ? P.order2[b * P.M2 + n] : n;
            if (d < rowmin || (d == rowmin && p2 < rpos)) { rowmin = d; rn = n; rpos = p2; }
        }
        const long long p1 = P.order1 ? P.order1[b * P.M1 + m] : m;
        if (rowmin > best || (rowmin == best && p1 > best_pos)) { best = rowmin; best_pos = p1; best_m = m; best_n = rn; }
    }
    s_val[tid] = best; s_pos[tid] = best_pos; s_m[tid] = best_m; s_n[tid] = best_n;
    __syncthreads();
    for (int off = kThreads / 2; off > 0; off >>= 1) {
        if (tid < off) {
            const T v = s_val[tid + off];
            const long long p = s_pos[tid + off];
            if (v > s_val[tid] || (v == s_val[tid] && p > s_pos[tid])) {
                s_val[tid] = v; s_pos[tid] = p; s_m[tid] = s_m[tid + off]; s_n[tid] = s_n[tid + off];
            }
        }
        __syncthreads();
    }
    if (tid == 0) {
        const T cmax = s_pos[0] >= 0 ? s_val[0] : T(0);
        reinterpret_cast<T *>(P.out)[pair] = (T)sqrt((double)cmax);
        P.idx1[pair] = s_m[0];
        P.idx2[pair] = s_n[0];
    }
}

// grad_x1[b,i,m*,k] += g * (x1[m*] - x2[n*]) / out, one thread per (b,i,k), ascending j.
template <typename T, bool SIDE2>
__global__ void hausdorff_backward_kernel(const T *grad, const T *out, const long long *idx1, const long long *idx2,
                                          const T *x1, const T *x2, T *gx,
                                          long long B, long long N1, long long N2, long long M1, long long M2, long long D) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long NO = SIDE2 ? N2 : N1; // sets on the side that owns the gradient
    if (idx >= B * NO * D) return;
    const long long k = idx % D, s = (idx / D) % NO, b = idx / (D * NO);
    const long long NI = SIDE2 ? N1 : N2;
    for (long long t = 0; t < NI; ++t) {
        const long long i = SIDE2 ? t : s, j = SIDE2 ? s : t;
        const long long pair = (b * N1 + i) * N2 + j;
        const long long m = idx1[pair], n = idx2[pair];
        const T a = x1[((b * N1 + i) * M1 + m) * D + k];
        const T c = x2[((b * N2 + j) * M2 + n) * D + k];
        const T diff = SIDE2 ? c - a : a - c;
        T *dst = SIDE2 ? gx + ((b * N2 + j) * M2 + n) * D + k : gx + ((b * N1 + i) * M1 + m) * D + k;
        *dst += grad[pair] * diff / out[pair];
    }
}

// P.rowmins != NULL selects the fused hot loop with the refining kernel, NULL the exact hot loop.
template <int D>
int launch_fast(HdParams P, cudaStream_t s) {
    const long long pairs = P.B * P.N1 * P.N2;
    P.mtiles = (P.M1 + kThreads * PM - 1) / (kThreads * PM);
    const long long blocks = pairs * P.mtiles;
    TPW_CHECK_ARG(blocks < (1ll << 31), "hausdorff: too many blocks");
    TPW_CUDA_OK(cudaMemsetAsync(P.keys, 0, (size_t)pairs * sizeof(unsigned long long), s));
    if (P.rowmins) {
        hausdorff_rowmin_kernel<D, true><<<(unsigned)blocks, kThreads, 0, s>>>(P);
        TPW_LAUNCH_OK("hausdorff_rowmin_kernel");
        hausdorff_refine_kernel<D><<<(unsigned)pairs, kThreads, 0, s>>>(P);
        TPW_LAUNCH_OK("hausdorff_refine_kernel");
        return TPW_OK;
    }
    hausdorff_rowmin_kernel<D, false><<<(unsigned)blocks, kThreads, 0, s>>>(P);
    TPW_LAUNCH_OK("hausdorff_rowmin_kernel");
    hausdorff_finish_kernel<D><<<(unsigned)pairs, kThreads, 0, s>>>(P);
    TPW_LAUNCH_OK("hausdorff_finish_kernel");
    return TPW_OK;
}

} // namespace
} // namespace tpw

using namespace tpw;

// one 8-byte key per set pair, then 8 bytes per x1 point of every set pair (the row minima: approximate float32 values
// for the fused float32 loop, exact float64 values for the float64 path; the query does not know the dtype)
extern "C" int64_t tpw_hausdorff_scratch_bytes(int64_t B, int64_t N1, int64_t N2, int64_t M1) {
    if (B <= 0 || N1 <= 0 || N2 <= 0) return 0;
    const int64_t pairs = B * N1 * N2;
    return pairs * (int64_t)sizeof(unsigned long long) + (M1 > 0 ? pairs * M1 * 8 : 0);
}

extern "C" int tpw_hausdorff_forward(int dtype, const void *x1, const void *x2,
                                     const int64_t *order1, const int64_t *order2,
                                     void *out, int64_t *idx1, int64_t *idx2, void *scratch,
                                     int64_t B, int64_t N1, int64_t N2, int64_t M1, int64_t M2, int64_t D,
                                     tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_hausdorff_forward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && M1 >= 0 && M2 >= 0 && D >= 0, "tpw_hausdorff_forward: negative size");
    const long long pairs = B * N1 * N2;
    if (pairs == 0) return TPW_OK;
    TPW_CHECK_ARG(M1 > 0 && M2 > 0 && D > 0, "tpw_hausdorff_forward: empty point sets (M1=%lld, M2=%lld, D=%lld)",
                  (long long)M1, (long long)M2, (long long)D);
    TPW_CHECK_ARG(M1 < (1ll << 32) && M2 < (1ll << 32), "tpw_hausdorff_forward: more than 2^32 points per set");
    TPW_CHECK_ARG(x1 && x2 && out && idx1 && idx2, "tpw_hausdorff_forward: NULL pointer");
    TPW_CHECK_ARG(pairs < (1ll << 31), "tpw_hausdorff_forward: too many set pairs");
    HdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2;
    P.order1 = reinterpret_cast<const long long *>(order1);
    P.order2 = reinterpret_cast<const long long *>(order2);
    P.out = out;
    P.idx1 = reinterpret_cast<long long *>(idx1);
    P.idx2 = reinterpret_cast<long long *>(idx2);
    P.keys = reinterpret_cast<unsigned long long *>(scratch);
    P.B = B; P.N1 = N1; P.N2 = N2; P.M1 = M1; P.M2 = M2; P.D = D;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32 && D <= kMaxFastD) {
        TPW_CHECK_ARG(scratch != nullptr, "tpw_hausdorff_forward: scratch is NULL");
        TPW_CHECK_ARG((reinterpret_cast<uintptr_t>(scratch) & 7u) == 0, "tpw_hausdorff_forward: scratch must be 8-byte aligned");
        if (!getenv("TPW_HAUSDORFF_EXACT_LOOP")) P.rowmins = reinterpret_cast<float *>(P.keys + pairs);
        switch (D) {
            case 1: return launch_fast<1>(P, s);
            case 2: return launch_fast<2>(P, s);
            case 3: return launch_fast<3>(P, s);
            case 4: return launch_fast<4>(P, s);
            case 5: return launch_fast<5>(P, s);
            case 6: return launch_fast<6>(P, s);
            case 7: return launch_fast<7>(P, s);
            case 8: return launch_fast<8>(P, s);
            case 9: return launch_fast<9>(P, s);
            case 10: return launch_fast<10>(P, s);
            case 11: return launch_fast<11>(P, s);
            case 12: return launch_fast<12>(P, s);
            case 13: return launch_fast<13>(P, s);
            case 14: return launch_fast<14>(P, s);
            case 15: return launch_fast<15>(P, s);
            default: return launch_fast<16>(P, s);
        }
    }
    if (dtype == TPW_F64 && D <= kMaxFastD && scratch != nullptr && (reinterpret_cast<uintptr_t>(scratch) & 7u) == 0 &&
        !getenv("TPW_HAUSDORFF_PLAIN_F64")) {
        P.rowmins = reinterpret_cast<float *>(P.keys + pairs);   // used as double[pairs * M1]
        switch (D) {
            case 1: return launch_f64<1>(P, s);
            case 2: return launch_f64<2>(P, s);
            case 3: return launch_f64<3>(P, s);
            case 4: return launch_f64<4>(P, s);
            case 5: return launch_f64<5>(P, s);
            case 6: return launch_f64<6>(P, s);
            case 7: return launch_f64<7>(P, s);
            case 8: return launch_f64<8>(P, s);
            case 9: return launch_f64<9>(P, s);
            case 10: return launch_f64<10>(P, s);
            case 11: return launch_f64<11>(P, s);
            case 12: return launch_f64<12>(P, s);
            case 13: return launch_f64<13>(P, s);
            case 14: return launch_f64<14>(P, s);
            case 15: return launch_f64<15>(P, s);
            default: return launch_f64<16>(P, s);
        }
    }
    if (dtype == TPW_F32) hausdorff_plain_kernel<float><<<(unsigned)pairs, kThreads, 0, s>>>(P);
    else hausdorff_plain_kernel<double><<<(unsigned)pairs, kThreads, 0, s>>>(P);
    TPW_LAUNCH_OK("hausdorff_plain_kernel");
    return TPW_OK;
}

extern "C" int tpw_hausdorff_backward(int dtype, const void *grad, const void *out,
                                      const int64_t *idx1, const int64_t *idx2,
                                      const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                                      int64_t B, int64_t N1, int64_t N2, int64_t M1, int64_t M2, int64_t D,
                                      tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_hausdorff_backward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && M1 >= 0 && M2 >= 0 && D >= 0, "tpw_hausdorff_backward: negative size");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = dtype == TPW_F32 ? 4 : 8;
    if (grad_x1 && B * N1 * M1 * D > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x1, 0, (size_t)(B * N1 * M1 * D) * es, s));
    if (grad_x2 && B * N2 * M2 * D > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x2, 0, (size_t)(B * N2 * M2 * D) * es, s));
    if (B * N1 * N2 == 0 || M1 == 0 || M2 == 0 || D == 0) return TPW_OK;
    TPW_CHECK_ARG(grad && out && idx1 && idx2 && x1 && x2, "tpw_hausdorff_backward: NULL pointer");
    const int threads = 128;
    const long long *i1 = reinterpret_cast<const long long *>(idx1), *i2 = reinterpret_cast<const long long *>(idx2);
#define TPW_HD_BWD(T)                                                                                                   \
    do {                                                                                                                \
        if (grad_x1) {                                                                                                  \
            const long long n = B * N1 * D;                                                                             \
            hausdorff_backward_kernel<T, false><<<(unsigned)((n + threads - 1) / threads), threads, 0, s>>>(            \
                (const T *)grad, (const T *)out, i1, i2, (const T *)x1, (const T *)x2, (T *)grad_x1, B, N1, N2, M1, M2, D); \
        }                                                                                                               \
        if (grad_x2) {                                                                                                  \
            const long long n = B * N2 * D;                                                                             \
            hausdorff_backward_kernel<T, true><<<(unsigned)((n + threads - 1) / threads), threads, 0, s>>>(             \
                (const T *)grad, (const T *)out, i1, i2, (const T *)x1, (const T *)x2, (T *)grad_x2, B, N1, N2, M1, M2, D); \
        }                                                                                                               \
    } while (0)
    if (dtype == TPW_F32) TPW_HD_BWD(float); else TPW_HD_BWD(double);
#undef TPW_HD_BWD
    TPW_LAUNCH_OK("hausdorff_backward_kernel");
    return TPW_OK;
}


// ---- allocation-free variant ----------------------------------------------------------------------
// Some hosts of this library are not allowed to obtain device memory at call time: a serving
// process that hands the whole GPU to its own pool when it starts, a plug-in host that forbids
// allocation inside its compute callback, or a latency-critical loop that cannot afford the
// device-wide synchronisation cudaMalloc may imply.  tpw_hausdorff_forward needs 8 bytes of scratch
// per set pair from such a caller; this variant brings its own instead, in a fixed array that
// lives in the library's device image (every GPU that loads the library holds it until exit).
namespace tpw {
namespace {

constexpr long long kStaticMaxPairs = 65536; // 512 KiB of keys

static __device__ __align__(256) unsigned long long g_hausdorff_static_keys[kStaticMaxPairs];

// `g_hausdorff_static_keys` names a host-side shadow here, not device memory; the device address
// has to be asked for, once per device, while that device is current.  That first lookup may make the
// runtime load this library's device image on the device (memory for the image, the 512 KiB array
// included, and an implicit synchronisation): it belongs in the host's start-up, before the region in
// which nothing may allocate.  The slots are atomic (any host thread may be first; all store the same
// address).  A cudaDeviceReset invalidates the address: a host that resets a device must not call into
// this library on it again in the same process.
int resolve_static_keys(unsigned long long **ptr) {
    static std::atomic<unsigned long long *> cache[64];
    int dev = 0;
    TPW_CUDA_OK(cudaGetDevice(&dev));
    TPW_CHECK_ARG(dev >= 0 && dev < 64, "tpw_hausdorff_forward_static: device ordinal %d is out of range", dev);
    unsigned long long *cached = cache[dev].load(std::memory_order_acquire);
    if (!cached) {
        void *p = nullptr;
        TPW_CUDA_OK(cudaGetSymbolAddress(&p, g_hausdorff_static_keys));
        TPW_CHECK_ARG(p != nullptr, "tpw_hausdorff_forward_static: the scratch symbol resolved to NULL");
        cached = static_cast<unsigned long long *>(p);
        cache[dev].store(cached, std::memory_order_release);
    }
    *ptr = cached;
    return TPW_OK;
}

} // namespace
} // namespace tpw

extern "C" int64_t tpw_hausdorff_static_max_pairs(void) { return tpw::kStaticMaxPairs; }

extern "C" int tpw_hausdorff_forward_static(int dtype, const void *x1, const void *x2,
                                            const int64_t *order1, const int64_t *order2,
                                            void *out, int64_t *idx1, int64_t *idx2,
                                            int64_t B, int64_t N1, int64_t N2, int64_t M1, int64_t M2, int64_t D,
                                            tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_hausdorff_forward_static: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && M1 >= 0 && M2 >= 0 && D >= 0, "tpw_hausdorff_forward_static: negative size");
    const long long pairs = B * N1 * N2;
    if (pairs == 0) return TPW_OK;
    TPW_CHECK_ARG(pairs <= kStaticMaxPairs,
                  "tpw_hausdorff_forward_static: %lld set pairs exceed the built-in scratch of %lld; "
                  "use tpw_hausdorff_forward with caller-provided scratch", pairs, kStaticMaxPairs);
    TPW_CHECK_ARG(M1 > 0 && M2 > 0 && D > 0, "tpw_hausdorff_forward_static: empty point sets (M1=%lld, M2=%lld, D=%lld)",
                  (long long)M1, (long long)M2, (long long)D);
    TPW_CHECK_ARG(M1 < (1ll << 32) && M2 < (1ll << 32), "tpw_hausdorff_forward_static: more than 2^32 points per set");
    TPW_CHECK_ARG(x1 && x2 && out && idx1 && idx2, "tpw_hausdorff_forward_static: NULL pointer");
    HdParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1; P.x2 = x2;
    P.order1 = reinterpret_cast<const long long *>(order1);
    P.order2 = reinterpret_cast<const long long *>(order2);
    P.out = out;
    P.idx1 = reinterpret_cast<long long *>(idx1);
    P.idx2 = reinterpret_cast<long long *>(idx2);
    P.B = B; P.N1 = N1; P.N2 = N2; P.M1 = M1; P.M2 = M2; P.D = D;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (dtype == TPW_F32 && D <= kMaxFastD) {
        int st = resolve_static_keys(&P.keys);
        if (st != TPW_OK) return st;
        // launch_fast clears the first `pairs` keys on the stream before the kernels use them; without room for
        // the approximate row minima (P.rowmins stays NULL) it evaluates every point pair in the exact arithmetic
        switch (D) {
            case 1: return launch_fast<1>(P, s);
            case 2: return launch_fast<2>(P, s);
            case 3: return launch_fast<3>(P, s);
            case 4: return launch_fast<4>(P, s);
            case 5: return launch_fast<5>(P, s);
            case 6: return launch_fast<6>(P, s);
            case 7: return launch_fast<7>(P, s);
            case 8: return launch_fast<8>(P, s);
            case 9: return launch_fast<9>(P, s);
            case 10: return launch_fast<10>(P, s);
            case 11: return launch_fast<11>(P, s);
            case 12: return launch_fast<12>(P, s);
            case 13: return launch_fast<13>(P, s);
            case 14: return launch_fast<14>(P, s);
            case 15: return launch_fast<15>(P, s);
            default: return launch_fast<16>(P, s);
        }
    }
    // the one-CTA-per-pair kernel keeps its state in shared memory and needs no scratch at all
    if (dtype == TPW_F32) hausdorff_plain_kernel<float><<<(unsigned)pairs, kThreads, 0, s>>>(P);
    else hausdorff_plain_kernel<double><<<(unsigned)pairs, kThreads, 0, s>>>(P);
    TPW_LAUNCH_OK("hausdorff_plain_kernel");
    return TPW_OK;
}
