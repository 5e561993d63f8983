// Backward of the pairwise L_p reductions in ONE pass over the pairs (float32, CUDA cores).
//
//   grad_x1[b,i,k] =  post * w[b,k] * sum_j coef[b,i,j] * phi(x1[b,i,k] - x2[b,j,k])
//   grad_x2[b,j,k] = -post * w[b,k] * sum_i coef[b,i,j] * phi(x1[b,i,k] - x2[b,j,k])          (phi is odd)
//
// The two-launch form (lp_backward.cu) evaluates the difference and phi once per gradient, 3 operations per pair and
// feature in each launch.  Here a pair's term coef * phi is formed once and added to both sums: 4 operations.
//
// A CTA of 16 warps owns 256 rows i and 64 features k and walks over all rows j, 32 per stage (TMA, two-stage mbarrier
// ring: the x2 rows, and the 256 x 32 tiles of the upstream gradient and of the auxiliary matrix with the 128-byte
// swizzle).  Every stage the CTA turns the two tiles into a coefficient tile stored transposed, [32 rows j][256 rows
// i], so that the coefficients of two adjacent rows i for one j are one 8-byte word.  A warp owns four features; a
// thread holds 8 rows i (4 lane, 4 lane + 1, ..., and the same 128 rows further on) x 4 features of x1 and of the
// grad_x1 sums in registers for the whole walk, as packed pairs of adjacent ROWS, so the packed subtract and fused
// multiply-adds take their coefficient pair straight from the tile, and grad_x1 needs no exchange at all.  For
// grad_x2 a thread has the sum over its own 8 rows; it parks the four sums of each row j in a per-warp exchange
// buffer, per four rows j the 32 lanes' contributions to one (j, k) are added in a fixed order, and the CTA's sum over
// its 256 rows goes to a scratch array [B][row blocks][N2][D].  A second kernel adds the row blocks in ascending
// order: no float atomics, every sum in a fixed order, bit-reproducible from run to run.
#include "common.cuh"
#include "lp_backward_phi.cuh"

#include <stdlib.h>
#include <string.h>

namespace tpw {
namespace {

constexpr int OP_THREADS = 512;
constexpr int OP_R = 8;           // rows i per thread
constexpr int OP_ROWS = 256;      // rows i per CTA (32 lanes x 8)
constexpr int OP_FEAT = 64;       // features per CTA (16 warps x 4)
constexpr int OP_JT = 32;         // rows j per stage: one 128-byte row of the gradient tile
constexpr int OP_STAGES = 2;
constexpr int OP_G_BYTES = OP_ROWS * OP_JT * 4;        // 32 KB, swizzled
constexpr int OP_Y_BYTES = OP_JT * OP_FEAT * 4;        // 8 KB
constexpr int OP_STAGE_BYTES = 2 * OP_G_BYTES + OP_Y_BYTES;
constexpr int OP_OFF_CT = OP_STAGES * OP_STAGE_BYTES;  // coefficient tile [32 rows j][256 rows i]
constexpr int OP_CT_BYTES = OP_JT * OP_ROWS * 4;
constexpr int OP_RED_PITCH = 20;                        // floats per lane in the exchange buffer (16 + 4: conflict-free 16-byte stores)
constexpr int OP_RED_BYTES = 32 * OP_RED_PITCH * 4;    // per warp
constexpr int OP_OFF_RED = OP_OFF_CT + OP_CT_BYTES;
constexpr int OP_OFF_BAR = OP_OFF_RED + (OP_THREADS / 32) * OP_RED_BYTES;
constexpr int OP_SMEM = OP_OFF_BAR + OP_STAGES * 8;
constexpr int OP_ALLOC = OP_SMEM + 1024;                // the swizzled tiles need a 1024-byte aligned base

struct OnePassParams {
    const float *x1, *x2, *w;
    float *g1, *partial;
    long long B, N1, N2, D;
    long long b0, ib0;           // first batch and first row block of this launch
    long long nib, tiles_k;      // row blocks and feature tiles per batch in this launch
    float q;
    int pow_spec;
    float post;
    double qd;
    int *status;
};

// coef * phi(x - y) for the metrics whose phi has no packed form
template <int PHI>
__device__ __forceinline__ float onepass_term(float x, float y, float c, float q, int pspec) {
    const float d = x - y;
    if (PHI == PHI_SGN) return d != 0.f ? b_copysign_of(c, d) : 0.f;
    if (PHI == PHI_SGNPOW) return c * b_copysign(pow_abs_spec(fabsf(d), q, pspec), d);
    if (PHI == PHI_D) return c * d;
    return c * (d * fabsf(d));
}

// COEF: how the coefficient of a pair is formed from the gradient and the auxiliary tile (COEF_G: the gradient itself, no
// auxiliary tile is loaded); a compile-time constant, so that the coefficient pass holds one formula
template <int PHI, int COEF>
__global__ void __launch_bounds__(OP_THREADS, 1)
lp_backward_onepass_kernel(const __grid_constant__ CUtensorMap map_x2, const __grid_constant__ CUtensorMap map_grad,
                           const __grid_constant__ CUtensorMap map_aux, const OnePassParams P) {
    constexpr bool PACKED = (PHI == PHI_DABS || PHI == PHI_D);
    constexpr bool NEED_AUX = (COEF != COEF_G);
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + OP_OFF_BAR);
    float *ct = reinterpret_cast<float *>(smem + OP_OFF_CT);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int kofs = warp * 4;                           // this warp's four features inside the CTA's 64
    float *red = reinterpret_cast<float *>(smem + OP_OFF_RED + warp * OP_RED_BYTES);

    long long tile = blockIdx.x;
    const long long tkx = tile % P.tiles_k;
    tile /= P.tiles_k;
    const long long lib = tile % P.nib, lb = tile / P.nib;   // row block and batch inside this launch (the scratch slot)
    const long long ib = P.ib0 + lib, b = P.b0 + lb;
    const long long i0 = ib * OP_ROWS, k0 = tkx * OP_FEAT;
    const long long kk = k0 + kofs;
    const bool k_ok = kk < P.D;                          // D is a multiple of 4: four features are in or out together

    // x1 rows {i0 + 128 h + 4 lane + e} (h < 2, e < 4) and their sums, resident for the whole walk.  The packed form
    // pairs rows 2m and 2m + 1 of one feature: a pair's two coefficients then lie side by side in the coefficient tile.
    float xr[OP_R][4], acc[OP_R][4];
#pragma unroll
    for (int a = 0; a < OP_R; ++a) {
        const long long row = i0 + (a >> 2) * 128 + lane * 4 + (a & 3);
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row < P.N1 && k_ok) v = *reinterpret_cast<const float4 *>(P.x1 + (b * P.N1 + row) * P.D + kk);
        xr[a][0] = v.x; xr[a][1] = v.y; xr[a][2] = v.z; xr[a][3] = v.w;
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
    }
    f32x2 xr2[PACKED ? OP_R / 2 : 1][4], acc2[PACKED ? OP_R / 2 : 1][4];
    if constexpr (PACKED) {
#pragma unroll
        for (int m = 0; m < OP_R / 2; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                xr2[m][c] = pack2(xr[2 * m][c], xr[2 * m + 1][c]);
                acc2[m][c] = 0ull;
            }
    }

    const int nchunks = (int)((P.N2 + OP_JT - 1) / OP_JT);
    const uint32_t tx_bytes = OP_Y_BYTES + OP_G_BYTES + (NEED_AUX ? OP_G_BYTES : 0);
    auto issue = [&](int chunk) {
        unsigned char *base = smem + (chunk % OP_STAGES) * OP_STAGE_BYTES;
        uint64_t *bar = &full[chunk % OP_STAGES];
        const int j0 = chunk * OP_JT;
        mbar_expect_tx(bar, tx_bytes);
        tma_load_3d(base, &map_grad, bar, j0, (int)i0, (int)b);
        if (NEED_AUX) tma_load_3d(base + OP_G_BYTES, &map_aux, bar, j0, (int)i0, (int)b);
        tma_load_3d(base + 2 * OP_G_BYTES, &map_x2, bar, (int)k0, j0, (int)b);
    };
    if (tid == 0) {
#pragma unroll
        for (int s = 0; s < OP_STAGES; ++s) mbar_init(&full[s], 1);
        mbar_init_fence();
        tma_prefetch_descriptor(&map_x2);
        tma_prefetch_descriptor(&map_grad);
        if (NEED_AUX) tma_prefetch_descriptor(&map_aux);
    }
    __syncthreads();
    if (tid == 0) issue(0);

    float *part = P.partial + ((lb * P.nib + lib) * P.N2) * P.D;   // this CTA's [N2][D] slab of the scratch
    // after the exchange lanes 0-15 hold the sums of (row j, feature) = (lane >> 2, lane & 3)
    const int o_u = (lane >> 2) & 3;
    const long long okk = kk + (lane & 3);
    const int t_row = tid & 255, t_half = tid >> 8;       // the transposing pass: one row i, four 16-byte chunks of it
    int failed = 0;

    for (int t = 0; t < nchunks; ++t) {
        const int stage = t % OP_STAGES;
        unsigned char *base = smem + stage * OP_STAGE_BYTES;
        const float *ys = reinterpret_cast<const float *>(base + 2 * OP_G_BYTES);
        // every thread is done with the other buffer and with the coefficient tile: refill, then wait for this stage
        if (__syncthreads_or(failed)) {
            if (tid == 0) {
                if (P.status) atomicCAS(P.status, 0, (2 << 16) | 3);
                // this stage's copy was issued an iteration ago and may still be landing: the CTA stays until it has
                // (again with a bound), so that no copy writes into shared memory the CTA has given back
                mbar_wait_bounded(&full[stage], (uint32_t)((t / OP_STAGES) & 1));
            }
            return;
        }
        if (tid == 0 && t + 1 < nchunks) issue(t + 1);
        if (!mbar_wait_bounded(&full[stage], (uint32_t)((t / OP_STAGES) & 1))) failed = 1;

        // coefficients from the gradient and auxiliary tiles ([256 rows i][32 rows j], swizzled), written transposed:
        // consecutive lanes read consecutive rows of one chunk (all banks) and write consecutive words
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
            const uint32_t chunk = (uint32_t)(t_half * 4 + cc);
            const uint32_t off = swz128((uint32_t)t_row, chunk);
            float4 g = *reinterpret_cast<const float4 *>(base + off);
            if (NEED_AUX) {
                const float4 o = *reinterpret_cast<const float4 *>(base + OP_G_BYTES + off);
                g.x = bwd_coefficient<float>(COEF, g.x, o.x, P.qd);
                g.y = bwd_coefficient<float>(COEF, g.y, o.y, P.qd);
                g.z = bwd_coefficient<float>(COEF, g.z, o.z, P.qd);
                g.w = bwd_coefficient<float>(COEF, g.w, o.w, P.qd);
            }
            float *dst = ct + (chunk * 4) * OP_ROWS + t_row;
            dst[0] = g.x; dst[OP_ROWS] = g.y; dst[2 * OP_ROWS] = g.z; dst[3 * OP_ROWS] = g.w;
        }
        __syncthreads();

#pragma unroll 1
        for (int jg = 0; jg < OP_JT / 4; ++jg) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                float sj[4];
                const int j = jg * 4 + u;
                const float4 yv = *reinterpret_cast<const float4 *>(ys + j * OP_FEAT + kofs);
                const float y[4] = {yv.x, yv.y, yv.z, yv.w};
                if constexpr (PACKED) {
                    f32x2 y2[4], sj2[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        y2[c] = pack2(y[c], y[c]);
                        sj2[c] = 0ull;
                    }
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float4 cv = *reinterpret_cast<const float4 *>(ct + j * OP_ROWS + h * 128 + lane * 4);
                        const f32x2 c2[2] = {pack2(cv.x, cv.y), pack2(cv.z, cv.w)};
#pragma unroll
                        for (int r = 0; r < 2; ++r)
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                f32x2 t2 = sub2(xr2[h * 2 + r][c], y2[c]);
                                if (PHI == PHI_DABS) {
                                    float lo, hi;
                                    unpack2(t2, lo, hi);
                                    t2 = pack2(lo * fabsf(lo), hi * fabsf(hi));
                                }
                                acc2[h * 2 + r][c] = fma2(c2[r], t2, acc2[h * 2 + r][c]);
                                sj2[c] = fma2(c2[r], t2, sj2[c]);
                            }
                    }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        float lo, hi;
                        unpack2(sj2[c], lo, hi);
                        sj[c] = lo + hi;
                    }
                } else {
#pragma unroll
                    for (int c = 0; c < 4; ++c) sj[c] = 0.f;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const float4 cv = *reinterpret_cast<const float4 *>(ct + j * OP_ROWS + h * 128 + lane * 4);
                        const float cs[4] = {cv.x, cv.y, cv.z, cv.w};
#pragma unroll
                        for (int r = 0; r < 4; ++r)
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const float term = onepass_term<PHI>(xr[h * 4 + r][c], y[c], cs[r], P.q, P.pow_spec);
                                acc[h * 4 + r][c] += term;
                                sj[c] += term;
                            }
                    }
                }
                // parked in the exchange buffer right away (the previous group's reads ended with a warp barrier)
                *reinterpret_cast<float4 *>(red + lane * OP_RED_PITCH + u * 4) = make_float4(sj[0], sj[1], sj[2], sj[3]);
            }
            // exchange: every lane has written its sums of (4 rows j) x (4 features); lanes l and l + 16 then add the even
            // and the odd lanes' contributions to one (j, feature) in ascending order, and the two are added
            __syncwarp();
            float tot = 0.f;
            const float *src = red + (lane >> 4) * OP_RED_PITCH + (lane & 15);
#pragma unroll
            for (int g = 0; g < 16; ++g) tot += src[2 * g * OP_RED_PITCH];
            tot += __shfl_down_sync(0xffffffffu, tot, 16);
            __syncwarp();
            const long long j = (long long)t * OP_JT + jg * 4 + o_u;
            if (lane < 16 && j < P.N2 && okk < P.D) part[j * P.D + okk] = tot;
        }
    }
    if (__syncthreads_or(failed)) {
        if (tid == 0 && P.status) atomicCAS(P.status, 0, (2 << 16) | 4);
        return;
    }

    if constexpr (PACKED) {
#pragma unroll
        for (int m = 0; m < OP_R / 2; ++m)
#pragma unroll
            for (int c = 0; c < 4; ++c) unpack2(acc2[m][c], acc[2 * m][c], acc[2 * m + 1][c]);
    }
    if (k_ok) {
        float4 wv = make_float4(P.post, P.post, P.post, P.post);
        if (P.w) {
            const float4 ww = *reinterpret_cast<const float4 *>(P.w + b * P.D + kk);
            wv.x *= ww.x; wv.y *= ww.y; wv.z *= ww.z; wv.w *= ww.w;
        }
#pragma unroll
        for (int a = 0; a < OP_R; ++a) {
            const long long row = i0 + (a >> 2) * 128 + lane * 4 + (a & 3);
            if (row >= P.N1) continue;
            *reinterpret_cast<float4 *>(P.g1 + (b * P.N1 + row) * P.D + kk) =
                make_float4(acc[a][0] * wv.x, acc[a][1] * wv.y, acc[a][2] * wv.z, acc[a][3] * wv.w);
        }
    }
}

// grad_x2[b,j,k] (+)= -post * w[b,k] * sum over the launch's row blocks, ascending; four features per thread
__global__ void __launch_bounds__(256)
lp_backward_onepass_sum_kernel(const float *partial, float *g2, const float *w, long long nb, long long nib, long long b0,
                               long long N2, long long D, float post, int accumulate) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long per_batch = N2 * D / 4;
    if (idx >= nb * per_batch) return;
    const long long lb = idx / per_batch, e = idx % per_batch;
    const float4 *src = reinterpret_cast<const float4 *>(partial) + lb * nib * per_batch + e;
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (long long ib = 0; ib < nib; ++ib) {
        const float4 v = src[ib * per_batch];
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    const long long b = b0 + lb;
    const long long k = (e * 4) % D;
    s.x *= -post; s.y *= -post; s.z *= -post; s.w *= -post;
    if (w) {
        const float4 ww = *reinterpret_cast<const float4 *>(w + b * D + k);
        s.x *= ww.x; s.y *= ww.y; s.z *= ww.z; s.w *= ww.w;
    }
    float4 *dst = reinterpret_cast<float4 *>(g2) + b * per_batch + e;
    if (accumulate) {
        const float4 o = *dst;
        s.x += o.x; s.y += o.y; s.z += o.z; s.w += o.w;
    }
    *dst = s;
}

constexpr long long kScratchCap = 2ll << 30;

template <int PHI, int COEF>
int launch_onepass(OnePassParams P, const void *grad, const void *aux, float *g2, void *scratch, long long scratch_bytes,
                   cudaStream_t stream) {
    CUtensorMap mx, mg, ma;
    memset(&ma, 0, sizeof(ma));
    int st = make_tensor_map_3d(&mx, P.x2, 4, P.D, P.N2, P.B, OP_FEAT, OP_JT, false);
    if (st != TPW_OK) return st;
    st = make_tensor_map_3d(&mg, grad, 4, P.N2, P.N1, P.B, OP_JT, OP_ROWS, true);
    if (st != TPW_OK) return st;
    if (COEF != COEF_G) {
        st = make_tensor_map_3d(&ma, aux, 4, P.N2, P.N1, P.B, OP_JT, OP_ROWS, true);
        if (st != TPW_OK) return st;
    }
    auto kern = lp_backward_onepass_kernel<PHI, COEF>;
    TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, OP_ALLOC));
    const long long nblk = (P.N1 + OP_ROWS - 1) / OP_ROWS;
    const long long slab = P.N2 * P.D * 4;                    // bytes of scratch per (batch, row block)
    const long long slabs = scratch_bytes / slab;
    TPW_CHECK_ARG(slabs >= 1, "lp backward: the scratch holds no [N2, D] slab");
    P.partial = reinterpret_cast<float *>(scratch);
    P.tiles_k = (P.D + OP_FEAT - 1) / OP_FEAT;
    P.status = device_status_ptr();
    const long long bpl = slabs >= nblk ? (slabs / nblk < P.B ? slabs / nblk : P.B) : 1;   // batches per launch
    const long long ipl = slabs >= nblk ? nblk : slabs;                                     // row blocks per launch
    for (long long b0 = 0; b0 < P.B; b0 += bpl) {
        const long long nb = P.B - b0 < bpl ? P.B - b0 : bpl;
        for (long long ib0 = 0; ib0 < nblk; ib0 += ipl) {
            P.b0 = b0; P.ib0 = ib0;
            P.nib = nblk - ib0 < ipl ? nblk - ib0 : ipl;
            const long long ctas = nb * P.nib * P.tiles_k;
            TPW_CHECK_ARG(ctas < (1ll << 31), "lp backward: too many tiles (%lld)", ctas);
            kern<<<(unsigned)ctas, OP_THREADS, OP_ALLOC, stream>>>(mx, mg, ma, P);
            TPW_LAUNCH_OK("lp_backward_onepass_kernel");
            const long long n4 = nb * P.N2 * P.D / 4;
            lp_backward_onepass_sum_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, stream>>>(
                P.partial, g2, P.w, nb, P.nib, b0, P.N2, P.D, P.post, ib0 > 0 ? 1 : 0);
            TPW_LAUNCH_OK("lp_backward_onepass_sum_kernel");
        }
    }
    return TPW_OK;
}

} // namespace

// 0 where the one-pass kernel does not apply; otherwise the scratch it wants (at most 2 GiB: larger problems run as
// several launches over batch or row-block ranges)
long long lp_backward_onepass_scratch_bytes(int mode, long long B, long long N1, long long N2, long long D, double p) {
    if (getenv("TPW_DISABLE_ONEPASS_BWD") || tma_disabled()) return 0;
    if (mode != TPW_LP_BWD_CDIST && mode != TPW_LP_BWD_PPMINKOWSKI && mode != TPW_LP_BWD_WMINKOWSKI) return 0;
    if (!(p > 0) || isinf(p) || isnan(p)) return 0;
    if (B <= 0 || N1 < OP_ROWS || N2 < OP_JT || D < 16 || D % 4 != 0 || N2 % 4 != 0) return 0;
    if (B >= (1ll << 31) || N1 >= (1ll << 31) || N2 >= (1ll << 31) || D >= (1ll << 31)) return 0;
    const long long nblk = (N1 + OP_ROWS - 1) / OP_ROWS, tiles_k = (D + OP_FEAT - 1) / OP_FEAT;
    if (nblk * OP_ROWS * 4 > N1 * 5 || tiles_k * OP_FEAT * 4 > D * 5) return 0;   // more than a quarter of a tile idle
    if ((double)B * (double)N1 * (double)N2 * (double)D < 268435456.0) return 0;
    if (B * nblk * tiles_k * 2 < sm_count()) return 0;
    const long long slab = N2 * D * 4;
    if (slab > kScratchCap) return 0;
    const long long full = B * nblk * slab;
    if (full <= kScratchCap) return full;
    if (nblk * slab <= kScratchCap) return (kScratchCap / (nblk * slab)) * nblk * slab;
    return (kScratchCap / slab) * slab;
}

int lp_backward_onepass(int mode, const void *grad, const void *aux, const void *x1, const void *x2, const void *w,
                        void *grad_x1, void *grad_x2, long long B, long long N1, long long N2, long long D, double p,
                        void *scratch, long long scratch_bytes, cudaStream_t stream) {
    OnePassParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = reinterpret_cast<const float *>(x1);
    P.x2 = reinterpret_cast<const float *>(x2);
    P.g1 = reinterpret_cast<float *>(grad_x1);
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.qd = p - 1.0;
    P.q = (float)(p - 1.0);
    P.pow_spec = make_pow_spec(p - 1.0);
    P.post = 1.f;
    float *g2 = reinterpret_cast<float *>(grad_x2);
    switch (mode) {
        case TPW_LP_BWD_CDIST:
            if (p == 1.0) return launch_onepass<PHI_SGN, COEF_G>(P, grad, nullptr, g2, scratch, scratch_bytes, stream);
            if (p == 2.0) return launch_onepass<PHI_D, COEF_DIV_O>(P, grad, aux, g2, scratch, scratch_bytes, stream);
            if (p == 3.0) return launch_onepass<PHI_DABS, COEF_DIV_O2>(P, grad, aux, g2, scratch, scratch_bytes, stream);
            return launch_onepass<PHI_SGNPOW, COEF_DIV_POW>(P, grad, aux, g2, scratch, scratch_bytes, stream);
        case TPW_LP_BWD_PPMINKOWSKI:
            P.post = (float)p;
            if (p == 1.0) return launch_onepass<PHI_SGN, COEF_G>(P, grad, nullptr, g2, scratch, scratch_bytes, stream);
            if (p == 2.0) return launch_onepass<PHI_D, COEF_G>(P, grad, nullptr, g2, scratch, scratch_bytes, stream);
            if (p == 3.0) return launch_onepass<PHI_DABS, COEF_G>(P, grad, nullptr, g2, scratch, scratch_bytes, stream);
            return launch_onepass<PHI_SGNPOW, COEF_G>(P, grad, nullptr, g2, scratch, scratch_bytes, stream);
        case TPW_LP_BWD_WMINKOWSKI:
            P.w = reinterpret_cast<const float *>(w);
            if (p == 1.0) return launch_onepass<PHI_SGN, COEF_MUL>(P, grad, aux, g2, scratch, scratch_bytes, stream);
            if (p == 2.0) return launch_onepass<PHI_D, COEF_MUL>(P, grad, aux, g2, scratch, scratch_bytes, stream);
            if (p == 3.0) return launch_onepass<PHI_DABS, COEF_MUL>(P, grad, aux, g2, scratch, scratch_bytes, stream);
            return launch_onepass<PHI_SGNPOW, COEF_MUL>(P, grad, aux, g2, scratch, scratch_bytes, stream);
        default:
            return fail(TPW_ERR_INVALID, "lp backward: unknown mode %d", mode);
    }
}

} // namespace tpw
