// Backward of the pairwise L_p reductions on the CUDA cores.
//
//   grad_x1[b,i,k] = post * w[b,k] * sum_j coef[b,i,j] * phi(x1[b,i,k] - x2[b,j,k])
//   grad_x2[b,j,k] = post * w[b,k] * sum_i coef[b,i,j] * phi(x2[b,j,k] - x1[b,i,k])
//
// with coef derived on the fly from the upstream gradient g and an auxiliary [B,N1,N2] matrix
// (the forward output, or the S^(1/p-1) matrix of the weighted form), and phi an odd function of
// the coordinate difference chosen by p.  The two sums are two passes of ONE kernel: the "row"
// operand (x1 for grad_x1, x2 for grad_x2) sits in registers, the other operand and the
// coefficient tile are streamed through shared memory 32 rows at a time.  A CTA (512 threads for
// float, 4 rows x 8 features each) owns a 128-row x 128-feature block of the gradient and sums
// over the whole streamed dimension itself, so every gradient element is written once, without
// atomics, in a fixed order.
//
// Thread (tr, tk) = (tid/16, tid%16) owns rows {4tr + e} and features {64g + 4tk + e} (e < 4):
// 16-byte shared loads of the streamed operand are contiguous across a quarter warp and the
// coefficient loads are broadcasts.  Aligned problems are fed by TMA (three-stage
// mbarrier ring, one issuing thread); others use guarded plain loads into the same layout.
#include "common.cuh"
#include "lp_backward_phi.cuh"

#include <math.h>
#include <stdlib.h>

#include <type_traits>

namespace tpw {
namespace {


struct BwdParams {
    const void *rowop;  // [B, NR, D] operand held in registers
    const void *stream; // [B, NS, D] operand streamed through shared memory
    const void *grad;   // [B, N1, N2]
    const void *aux;    // [B, N1, N2] or NULL
    const void *w;      // [B, D] or NULL
    void *out;          // [B, NR, D]
    long long B, N1, N2, D, NR, NS;
    long long tiles_r, tiles_k;
    double q;           // exponent of PHI_SGNPOW / PHI_ABSPOW, and of COEF_DIV_POW
    int pow_spec;       // make_pow_spec(q): how the float kernels evaluate |d|^q
    double post;        // scalar applied to every result
    int coef_mode;
    int *status;
    const unsigned long long *only_if; // non-NULL: the kernel does nothing unless this device counter exceeds only_if_above
    unsigned long long only_if_above;
};

constexpr int kStages = 2;
constexpr int SC = 64; // streamed rows per stage


// RR rows x RK features per thread, NTHR threads: (NTHR/16)*RR rows by 16*RK features per CTA.
// float: 4 x 8 on 512 threads (128 x 128, 16 warps per SM for latency hiding at <= 128 registers);
// double: 4 x 4 on 256 threads (64 x 64).
template <typename T, int RR, int RK, int NTHR> struct BwdSmem {
    static constexpr int TR = (NTHR / 16) * RR;   // rows of the register operand per CTA
    static constexpr int TK = 16 * RK;            // features per CTA
    static constexpr int YS_BYTES = SC * TK * (int)sizeof(T);
    static constexpr int GS_BYTES = SC * TR * (int)sizeof(T);
    static constexpr int STAGE_BYTES = YS_BYTES + 2 * GS_BYTES; // streamed rows | grad tile | aux tile
    static constexpr int OFF_BAR = kStages * STAGE_BYTES;
    static constexpr int BYTES = OFF_BAR + kStages * 8;
    static constexpr int ALLOC = BYTES + 128;
};

// TRANS = false: the register operand is x1 (rows i), streamed rows are j; the coefficient tile is
// stored [TR rows i][SC] exactly as it lies in memory.  TRANS = true: register operand x2 (rows j),
// streamed rows are i; the coefficient tile is stored [SC][TR rows j], again as it lies in memory.
template <typename T, int RR, int RK, int NTHR, int PHI, bool NEED_AUX, bool TRANS, bool USE_TMA>
__global__ void __launch_bounds__(NTHR, 1)
lp_backward_kernel(const __grid_constant__ CUtensorMap map_stream, const __grid_constant__ CUtensorMap map_grad,
                   const __grid_constant__ CUtensorMap map_aux, const BwdParams P) {
    typedef BwdSmem<T, RR, RK, NTHR> S;
    if (P.only_if && *P.only_if <= P.only_if_above) return;
    constexpr int TR = S::TR, TK = S::TK, GK = RK / 4;
    constexpr int RSTRIDE = (NTHR / 16) * 4;      // distance between a thread's groups of four rows
    constexpr int kThreads = NTHR;
    constexpr bool AUX_IN_LOOP = (PHI == PHI_SGN_EQ);

    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + S::OFF_BAR);

    const int tid = threadIdx.x;
    const int tr = tid >> 4, tk = tid & 15;

    long long tile = blockIdx.x;
    const long long tkx = tile % P.tiles_k;
    tile /= P.tiles_k;
    const long long trx = tile % P.tiles_r;
    const long long b = tile / P.tiles_r;
    const long long r0 = trx * TR, k0 = tkx * TK;

    const T *rowop = reinterpret_cast<const T *>(P.rowop) + b * P.NR * P.D;
    const T *stream = reinterpret_cast<const T *>(P.stream) + b * P.NS * P.D;
    const T *grad = reinterpret_cast<const T *>(P.grad) + b * P.N1 * P.N2;
    const T *aux = NEED_AUX ? reinterpret_cast<const T *>(P.aux) + b * P.N1 * P.N2 : nullptr;

    // register operand: rows {RSTRIDE*g + 4tr + e}, features {64g + 4tk + e}
    T xr[RR][RK];
    if (PHI != PHI_Y) {
#pragma unroll
        for (int a = 0; a < RR; ++a) {
            const long long row = r0 + (a / 4) * RSTRIDE + tr * 4 + (a % 4);
#pragma unroll
            for (int c = 0; c < RK; ++c) {
                const long long k = k0 + (c / 4) * 64 + tk * 4 + (c % 4);
                xr[a][c] = (row < P.NR && k < P.D) ? rowop[row * P.D + k] : T(0);
            }
        }
    }
    T acc[RR][RK];
#pragma unroll
    for (int a = 0; a < RR; ++a)
#pragma unroll
        for (int c = 0; c < RK; ++c) acc[a][c] = T(0);
    constexpr bool PACKED = PackedPhi<T, PHI>::value;
    f32x2 acc2[PACKED ? RR : 1][PACKED ? RK / 2 : 1], xr2[PACKED ? RR : 1][PACKED ? RK / 2 : 1];
    if constexpr (PACKED) {
#pragma unroll
        for (int a = 0; a < RR; ++a)
#pragma unroll
            for (int c = 0; c < RK / 2; ++c) {
                acc2[a][c] = 0ull;
                xr2[a][c] = PHI != PHI_Y ? pack2(xr[a][2 * c], xr[a][2 * c + 1]) : 0ull;
            }
    }

    const int nchunks = (int)((P.NS + SC - 1) / SC);
    const uint32_t tx_bytes = S::YS_BYTES + S::GS_BYTES + (NEED_AUX ? S::GS_BYTES : 0);

    auto issue = [&](int chunk) {
        const int st = chunk % kStages;
        unsigned char *base = smem + st * S::STAGE_BYTES;
        const int s0 = chunk * SC;
        mbar_expect_tx(&full[st], tx_bytes);
        tma_load_3d(base, &map_stream, &full[st], (int)k0, s0, (int)b);
        if (!TRANS) {
            tma_load_3d(base + S::YS_BYTES, &map_grad, &full[st], s0, (int)r0, (int)b);
            if (NEED_AUX) tma_load_3d(base + S::YS_BYTES + S::GS_BYTES, &map_aux, &full[st], s0, (int)r0, (int)b);
        } else {
            tma_load_3d(base + S::YS_BYTES, &map_grad, &full[st], (int)r0, s0, (int)b);
            if (NEED_AUX) tma_load_3d(base + S::YS_BYTES + S::GS_BYTES, &map_aux, &full[st], (int)r0, s0, (int)b);
        }
    };

    if (USE_TMA) {
        if (tid == 0) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
            mbar_init_fence();
            tma_prefetch_descriptor(&map_stream);
            tma_prefetch_descriptor(&map_grad);
            if (NEED_AUX) tma_prefetch_descriptor(&map_aux);
        }
        __syncthreads();
        if (tid == 0)
            for (int c = 0; c < kStages - 1 && c < nchunks; ++c) issue(c);
    }

    const T q = (T)P.q;
    const int pspec = P.pow_spec;
    int failed = 0;

    for (int t = 0; t < nchunks; ++t) {
        const int stage = USE_TMA ? t % kStages : 0;
        unsigned char *base = smem + stage * S::STAGE_BYTES;
        T *ys = reinterpret_cast<T *>(base);
        T *gs = reinterpret_cast<T *>(base + S::YS_BYTES);
        T *as = reinterpret_cast<T *>(base + S::YS_BYTES + S::GS_BYTES);
        const long long s0 = (long long)t * SC;

        if (USE_TMA) {
            if (__syncthreads_or(failed)) {
                if (tid == 0) {
                    if (P.status) atomicCAS(P.status, 0, (2 << 16) | 1);
                    // the chunks issued earlier may still be landing: the CTA stays (bounded) until they have
                    for (int c = t; c < t + kStages - 1 && c < nchunks; ++c) mbar_wait_bounded(&full[c % kStages], (uint32_t)((c / kStages) & 1));
                }
                return;
            }
            if (tid == 0 && t + kStages - 1 < nchunks) issue(t + kStages - 1);
            if (!mbar_wait_bounded(&full[stage], (uint32_t)((t / kStages) & 1))) failed = 1;
        } else {
            __syncthreads();
            for (int e = tid; e < SC * TK; e += kThreads) {
                const int s = e / TK, kk = e % TK;
                const long long row = s0 + s, k = k0 + kk;
                ys[e] = (row < P.NS && k < P.D) ? stream[row * P.D + k] : T(0);
            }
            for (int e = tid; e < SC * TR; e += kThreads) {
                long long i, j;
                if (!TRANS) { i = r0 + e / SC; j = s0 + e % SC; }
                else        { i = s0 + e / TR; j = r0 + e % TR; }
                const bool ok = i < P.N1 && j < P.N2;
                gs[e] = ok ? grad[i * P.N2 + j] : T(0);
                if (NEED_AUX) as[e] = ok ? aux[i * P.N2 + j] : T(0);
            }
            __syncthreads();
        }

        if (NEED_AUX) {
            // coefficient tile in place: c = f(g, aux).  The formula is picked once per stage, outside the element loop:
            // picked per element, the compiler keeps every candidate formula in the loop body.
            auto coefficients = [&](auto mode_tag) {
                constexpr int MODE = decltype(mode_tag)::value;
                for (int e = tid; e < SC * TR; e += kThreads) gs[e] = bwd_coefficient<T>(MODE, gs[e], as[e], P.q);
            };
            switch (P.coef_mode) {
                case COEF_DIV_O: coefficients(std::integral_constant<int, COEF_DIV_O>{}); break;
                case COEF_DIV_O2: coefficients(std::integral_constant<int, COEF_DIV_O2>{}); break;
                case COEF_DIV_POW: coefficients(std::integral_constant<int, COEF_DIV_POW>{}); break;
                case COEF_MUL: coefficients(std::integral_constant<int, COEF_MUL>{}); break;
                case COEF_ZERO_WHERE_O0: coefficients(std::integral_constant<int, COEF_ZERO_WHERE_O0>{}); break;
                default: break;
            }
            __syncthreads();
        }

#pragma unroll 1
        for (int s = 0; s < SC; s += 4) {
            T cv[TRANS ? 1 : RR][4];
            T ov[(AUX_IN_LOOP && !TRANS) ? RR : 1][4];
            if (!TRANS) {
#pragma unroll
                for (int a = 0; a < RR; ++a) {
                    const int row = (a / 4) * RSTRIDE + tr * 4 + (a % 4);
                    load4<T>(cv[a], gs + row * SC + s);
                    if (AUX_IN_LOOP) load4<T>(ov[a], as + row * SC + s);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                T yv[RK];
#pragma unroll
                for (int g = 0; g < GK; ++g) load4<T>(&yv[g * 4], ys + (s + u) * TK + g * 64 + tk * 4);
                T ct[RR], ot[RR];
                if (TRANS) {
#pragma unroll
                    for (int g = 0; g < RR / 4; ++g) {
                        load4<T>(&ct[g * 4], gs + (s + u) * TR + g * RSTRIDE + tr * 4);
                        if (AUX_IN_LOOP) load4<T>(&ot[g * 4], as + (s + u) * TR + g * RSTRIDE + tr * 4);
                    }
                }
                if constexpr (PACKED) {
                    f32x2 yv2[RK / 2];
#pragma unroll
                    for (int kk = 0; kk < RK / 2; ++kk) yv2[kk] = pack2(yv[2 * kk], yv[2 * kk + 1]);
#pragma unroll
                    for (int a = 0; a < RR; ++a) {
                        const float c = TRANS ? ct[a] : cv[a][u];
                        const f32x2 c2 = pack2(c, c);
#pragma unroll
                        for (int kk = 0; kk < RK / 2; ++kk) acc2[a][kk] = bwd_accumulate2<PHI>(acc2[a][kk], xr2[a][kk], yv2[kk], c2);
                    }
                } else {
#pragma unroll
                    for (int a = 0; a < RR; ++a) {
                        const T c = TRANS ? ct[a] : cv[a][u];
                        const T o = AUX_IN_LOOP ? (TRANS ? ot[a] : ov[a][u]) : T(0);
#pragma unroll
                        for (int kk = 0; kk < RK; ++kk) bwd_accumulate<PHI, T>(acc[a][kk], xr[a][kk], yv[kk], c, o, q, pspec);
                    }
                }
            }
        }
    }
    if (USE_TMA) {
        if (__syncthreads_or(failed)) {
            if (tid == 0 && P.status) atomicCAS(P.status, 0, (2 << 16) | 2);
            return;
        }
    }

    if constexpr (PACKED) {
#pragma unroll
        for (int a = 0; a < RR; ++a)
#pragma unroll
            for (int c = 0; c < RK / 2; ++c) unpack2(acc2[a][c], acc[a][2 * c], acc[a][2 * c + 1]);
    }
    T *out = reinterpret_cast<T *>(P.out) + b * P.NR * P.D;
    const T *w = P.w ? reinterpret_cast<const T *>(P.w) + b * P.D : nullptr;
    const T post = (T)P.post;
#pragma unroll
    for (int a = 0; a < RR; ++a) {
        const long long row = r0 + (a / 4) * RSTRIDE + tr * 4 + (a % 4);
        if (row >= P.NR) continue;
#pragma unroll
        for (int c = 0; c < RK; ++c) {
            const long long k = k0 + (c / 4) * 64 + tk * 4 + (c % 4);
            if (k >= P.D) continue;
            T v = acc[a][c] * post;
            if (w) v *= w[k];
            out[row * P.D + k] = v;
        }
    }
}

// Few gradient blocks (a small problem, or few rows against many): the tile kernel would occupy a handful of SMs, one
// CTA per 128 x 128 gradient block walking over the whole streamed dimension.  Here every gradient element has a
// thread of its own that walks over the streamed rows in ascending order -- the same terms in the same order as the
// tile kernel adds them, so the results are bit-identical and deterministic.  A warp holds 32 consecutive features of
// one gradient row: the streamed operand is read in 128-byte segments, the coefficient is a broadcast.
template <typename T, int PHI, bool NEED_AUX, bool TRANS>
__global__ void __launch_bounds__(256) lp_backward_small_kernel(const BwdParams P) {
    if (P.only_if && *P.only_if <= P.only_if_above) return;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= P.B * P.NR * P.D) return;
    const long long k = idx % P.D, r = (idx / P.D) % P.NR, b = idx / (P.D * P.NR);
    const T *stream = reinterpret_cast<const T *>(P.stream) + b * P.NS * P.D + k;
    const T *grad = reinterpret_cast<const T *>(P.grad) + b * P.N1 * P.N2;
    const T *aux = NEED_AUX ? reinterpret_cast<const T *>(P.aux) + b * P.N1 * P.N2 : nullptr;
    const T x = PHI != PHI_Y ? reinterpret_cast<const T *>(P.rowop)[(b * P.NR + r) * P.D + k] : T(0);
    const long long g0 = TRANS ? r : r * P.N2, gstep = TRANS ? P.N2 : 1;   // g[i][j]: i = r (rows) or i = s (columns)
    const T q = (T)P.q;
    T acc = T(0);
    // eight streamed rows at a time: all their loads are issued before the first term is added (the terms are still
    // added in ascending order, so the sum keeps the tile kernel's bits); a walk that waits for each row's loads in
    // turn is bound by their latency
    // The coefficient formula is picked once, outside the walk (picked per element, every candidate stays in the loop).
    auto walk = [&](auto mode_tag) {
        constexpr int MODE = decltype(mode_tag)::value;
        constexpr int U = 8;
        long long s = 0;
        for (; s + U <= P.NS; s += U) {
            T g[U], o[U], y[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                g[u] = grad[g0 + (s + u) * gstep];
                o[u] = NEED_AUX ? aux[g0 + (s + u) * gstep] : T(0);
                y[u] = stream[(s + u) * P.D];
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const T c = NEED_AUX ? bwd_coefficient<T>(MODE, g[u], o[u], P.q) : g[u];
                bwd_accumulate<PHI, T>(acc, x, y[u], c, o[u], q, P.pow_spec);
            }
        }
        for (; s < P.NS; ++s) {
            const T g = grad[g0 + s * gstep];
            const T o = NEED_AUX ? aux[g0 + s * gstep] : T(0);
            const T c = NEED_AUX ? bwd_coefficient<T>(MODE, g, o, P.q) : g;
            bwd_accumulate<PHI, T>(acc, x, stream[s * P.D], c, o, q, P.pow_spec);
        }
    };
    if (!NEED_AUX) {
        walk(std::integral_constant<int, COEF_G>{});
    } else {
        switch (P.coef_mode) {
            case COEF_DIV_O: walk(std::integral_constant<int, COEF_DIV_O>{}); break;
            case COEF_DIV_O2: walk(std::integral_constant<int, COEF_DIV_O2>{}); break;
            case COEF_DIV_POW: walk(std::integral_constant<int, COEF_DIV_POW>{}); break;
            case COEF_MUL: walk(std::integral_constant<int, COEF_MUL>{}); break;
            case COEF_ZERO_WHERE_O0: walk(std::integral_constant<int, COEF_ZERO_WHERE_O0>{}); break;
            default: walk(std::integral_constant<int, COEF_G>{}); break;
        }
    }
    T v = acc * (T)P.post;
    if (P.w) v *= reinterpret_cast<const T *>(P.w)[b * P.D + k];
    reinterpret_cast<T *>(P.out)[idx] = v;
}

template <typename T, int PHI, bool NEED_AUX, bool TRANS>
int launch_backward(BwdParams P, cudaStream_t stream) {
    constexpr int RR = 4;
    constexpr int RK = sizeof(T) == 4 ? 8 : 4;
    constexpr int NTHR = sizeof(T) == 4 ? 512 : 256;
    typedef BwdSmem<T, RR, RK, NTHR> S;
    P.tiles_r = (P.NR + S::TR - 1) / S::TR;
    P.tiles_k = (P.D + S::TK - 1) / S::TK;
    const long long tiles = P.B * P.tiles_r * P.tiles_k;
    if (tiles <= 0) return TPW_OK;
    TPW_CHECK_ARG(tiles < (1ll << 31), "lp backward: too many tiles (%lld)", tiles);
    TPW_CHECK_ARG(P.N1 < (1ll << 31) && P.N2 < (1ll << 31) && P.B < (1ll << 31) && P.D < (1ll << 31),
                  "lp backward: a dimension exceeds 2^31-1");
    P.status = device_status_ptr();

    // fewer gradient blocks than a third of the SMs: one thread per gradient element instead (TPW_DISABLE_SMALL_BWD=1
    // keeps the tile kernel); the walk per thread is bounded so that a launch stays in the millisecond range
    if (tiles * 3 < sm_count() && P.NS <= 65536 && P.B * P.NR * P.D < (1ll << 31) * 256 && !getenv("TPW_DISABLE_SMALL_BWD")) {
        const long long n = P.B * P.NR * P.D;
        lp_backward_small_kernel<T, PHI, NEED_AUX, TRANS><<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(P);
        TPW_LAUNCH_OK("lp_backward_small_kernel");
        return TPW_OK;
    }

    bool tma_ok = !tma_disabled() && aligned16(P.stream) && aligned16(P.grad) && (!NEED_AUX || aligned16(P.aux)) &&
                  (P.D * (long long)sizeof(T)) % 16 == 0 && (P.N2 * (long long)sizeof(T)) % 16 == 0;
    CUtensorMap ms, mg, ma;
    memset(&ms, 0, sizeof(ms));
    memset(&mg, 0, sizeof(mg));
    memset(&ma, 0, sizeof(ma));
    if (tma_ok) {
        int st = make_tensor_map_3d(&ms, P.stream, sizeof(T), P.D, P.NS, P.B, S::TK, SC, false);
        if (st != TPW_OK) return st;
        const uint32_t gb0 = TRANS ? S::TR : SC, gb1 = TRANS ? SC : S::TR;
        st = make_tensor_map_3d(&mg, P.grad, sizeof(T), P.N2, P.N1, P.B, gb0, gb1, false);
        if (st != TPW_OK) return st;
        if (NEED_AUX) {
            st = make_tensor_map_3d(&ma, P.aux, sizeof(T), P.N2, P.N1, P.B, gb0, gb1, false);
            if (st != TPW_OK) return st;
        }
        auto kern = lp_backward_kernel<T, RR, RK, NTHR, PHI, NEED_AUX, TRANS, true>;
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC));
        kern<<<(unsigned)tiles, NTHR, S::ALLOC, stream>>>(ms, mg, ma, P);
    } else {
        auto kern = lp_backward_kernel<T, RR, RK, NTHR, PHI, NEED_AUX, TRANS, false>;
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::ALLOC));
        kern<<<(unsigned)tiles, NTHR, S::ALLOC, stream>>>(ms, mg, ma, P);
    }
    TPW_LAUNCH_OK("lp_backward_kernel");
    return TPW_OK;
}

// One side (grad_x1 when trans == false, grad_x2 when true).
template <typename T, int PHI, bool NEED_AUX>
int launch_side(const BwdParams &base, bool trans, const void *x1, const void *x2, void *out, cudaStream_t stream) {
    BwdParams P = base;
    P.out = out;
    if (!trans) {
        P.rowop = x1; P.stream = x2; P.NR = base.N1; P.NS = base.N2;
        return launch_backward<T, PHI, NEED_AUX, false>(P, stream);
    }
    P.rowop = x2; P.stream = x1; P.NR = base.N2; P.NS = base.N1;
    return launch_backward<T, PHI, NEED_AUX, true>(P, stream);
}

template <typename T, int PHI, bool NEED_AUX>
int launch_both(const BwdParams &base, const void *x1, const void *x2, void *g1, void *g2, cudaStream_t stream) {
    if (g1) {
        int st = launch_side<T, PHI, NEED_AUX>(base, false, x1, x2, g1, stream);
        if (st != TPW_OK) return st;
    }
    if (g2) {
        int st = launch_side<T, PHI, NEED_AUX>(base, true, x1, x2, g2, stream);
        if (st != TPW_OK) return st;
    }
    return TPW_OK;
}

template <typename T>
int lp_backward_typed(int mode, BwdParams P, const void *x1, const void *x2, void *g1, void *g2, double p,
                      cudaStream_t stream) {
    P.post = 1.0;
    P.q = p - 1.0;
    P.pow_spec = make_pow_spec(P.q);
    P.coef_mode = COEF_G;
    switch (mode) {
        case TPW_LP_BWD_MATMUL:
            P.aux = nullptr; P.w = nullptr;
            return launch_both<T, PHI_Y, false>(P, x1, x2, g1, g2, stream);
        case TPW_LP_BWD_CDIST:
            P.w = nullptr;
            if (isinf(p)) { P.coef_mode = COEF_ZERO_WHERE_O0; return launch_both<T, PHI_SGN_EQ, true>(P, x1, x2, g1, g2, stream); }
            if (p == 1.0) { P.aux = nullptr; return launch_both<T, PHI_SGN, false>(P, x1, x2, g1, g2, stream); }
            if (p == 2.0) { P.coef_mode = COEF_DIV_O; return launch_both<T, PHI_D, true>(P, x1, x2, g1, g2, stream); }
            if (p == 3.0) { P.coef_mode = COEF_DIV_O2; return launch_both<T, PHI_DABS, true>(P, x1, x2, g1, g2, stream); }
            P.coef_mode = COEF_DIV_POW;
            return launch_both<T, PHI_SGNPOW, true>(P, x1, x2, g1, g2, stream);
        case TPW_LP_BWD_PPMINKOWSKI:
            P.aux = nullptr; P.w = nullptr; P.post = p;
            if (p == 1.0) return launch_both<T, PHI_SGN, false>(P, x1, x2, g1, g2, stream);
            if (p == 2.0) return launch_both<T, PHI_D, false>(P, x1, x2, g1, g2, stream);
            if (p == 3.0) return launch_both<T, PHI_DABS, false>(P, x1, x2, g1, g2, stream);
            return launch_both<T, PHI_SGNPOW, false>(P, x1, x2, g1, g2, stream);
        case TPW_LP_BWD_WMINKOWSKI:
            P.coef_mode = COEF_MUL;
            if (p == 1.0) return launch_both<T, PHI_SGN, true>(P, x1, x2, g1, g2, stream);
            if (p == 2.0) return launch_both<T, PHI_D, true>(P, x1, x2, g1, g2, stream);
            if (p == 3.0) return launch_both<T, PHI_DABS, true>(P, x1, x2, g1, g2, stream);
            return launch_both<T, PHI_SGNPOW, true>(P, x1, x2, g1, g2, stream);
        default:
            return fail(TPW_ERR_INVALID, "tpw_lp_backward: unknown mode %d", mode);
    }
}

// grad_w[b,k] = (1/p) * sum_i scratch[b,i,k]; one thread per (b,k), ascending i.
template <typename T>
__global__ void column_sum_kernel(const T *scratch, T *grad_w, long long B, long long N1, long long D, double scale) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * D) return;
    const long long b = idx / D, k = idx % D;
    const T *col = scratch + b * N1 * D + k;
    T s = T(0);
    for (long long i = 0; i < N1; ++i) s += col[i * D];
    grad_w[idx] = s * (T)scale;
}

// Single-coordinate +-inf backward: one thread per pair, first extreme coordinate wins.
template <typename T, bool NEG>
__global__ void lp_inf_backward_kernel(const T *grad, const T *x1, const T *x2, const T *w, T *g1, T *g2, T *gw,
                                       long long B, long long N1, long long N2, long long D) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= B * N1 * N2) return;
    const long long j = idx % N2, i = (idx / N2) % N1, b = idx / (N2 * N1);
    const T *a = x1 + (b * N1 + i) * D, *c = x2 + (b * N2 + j) * D;
    const T *wb = w ? w + b * D : nullptr;
    T val = a[0] - c[0], fabs_val = b_abs(val), w_val = wb ? fabs_val * wb[0] : fabs_val;
    long long best = 0;
    for (long long k = 1; k < D; ++k) {
        const T tmp = a[k] - c[k], ft = b_abs(tmp), wt = wb ? ft * wb[k] : ft;
        if (NEG ? (wt < w_val) : (wt > w_val)) { val = tmp; fabs_val = ft; w_val = wt; best = k; }
    }
    const T sgn = (T)((T(0) < val) - (val < T(0)));
    const T g = grad[idx];
    const T scale = wb ? wb[best] : T(1);
    if (g1) atomicAdd(g1 + (b * N1 + i) * D + best, g * scale * sgn);
    if (g2) atomicAdd(g2 + (b * N2 + j) * D + best, g * scale * -sgn);
    if (gw && wb) atomicAdd(gw + b * D + best, g * fabs_val);
}

} // namespace
} // namespace tpw

using namespace tpw;

// The dense p = +inf backward of cdist in float32, run only when the device counter *only_if exceeds `above` (the
// fallback of chebyshev_backward.cu for data full of tied maxima).
int tpw::lp_backward_cdist_inf_if(const unsigned long long *only_if, unsigned long long above, const void *grad, const void *out, const void *x1, const void *x2,
                                  void *grad_x1, void *grad_x2, long long B, long long N1, long long N2, long long D,
                                  cudaStream_t stream) {
    BwdParams P;
    memset(&P, 0, sizeof(P));
    P.grad = grad; P.aux = out; P.w = nullptr;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.post = 1.0; P.q = 0.0; P.pow_spec = 0; P.coef_mode = COEF_ZERO_WHERE_O0;
    P.only_if = only_if; P.only_if_above = above;
    return launch_both<float, PHI_SGN_EQ, true>(P, x1, x2, grad_x1, grad_x2, stream);
}

extern "C" int tpw_lp_backward(int dtype, int mode, const void *grad, const void *aux,
                               const void *x1, const void *x2, const void *w,
                               void *grad_x1, void *grad_x2,
                               int64_t B, int64_t N1, int64_t N2, int64_t D,
                               double p, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_lp_backward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_lp_backward: negative size");
    if (B == 0 || D == 0 || (N1 == 0 && N2 == 0)) return TPW_OK;
    if (N1 == 0 || N2 == 0) {
        // empty sums: the gradient of the non-empty side is all zero (its inputs may be NULL)
        cudaStream_t s0 = static_cast<cudaStream_t>(stream);
        const size_t es0 = dtype == TPW_F32 ? 4 : 8;
        if (grad_x1 && N1 > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x1, 0, (size_t)(B * N1 * D) * es0, s0));
        if (grad_x2 && N2 > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x2, 0, (size_t)(B * N2 * D) * es0, s0));
        return TPW_OK;
    }
    TPW_CHECK_ARG(x1 && x2, "tpw_lp_backward: NULL input");
    TPW_CHECK_ARG(grad != nullptr, "tpw_lp_backward: grad is NULL");
    TPW_CHECK_ARG(!isnan(p), "tpw_lp_backward: p is NaN");
    if (mode != TPW_LP_BWD_MATMUL) {
        TPW_CHECK_ARG(p > 0, "tpw_lp_backward: p must be positive (got %g)", p);
        TPW_CHECK_ARG(!isinf(p) || mode == TPW_LP_BWD_CDIST,
                      "tpw_lp_backward: p = inf is only defined for TPW_LP_BWD_CDIST; use tpw_lp_inf_backward");
    }
    const bool needs_aux = (mode == TPW_LP_BWD_WMINKOWSKI) || (mode == TPW_LP_BWD_CDIST && p != 1.0);
    TPW_CHECK_ARG(!needs_aux || aux != nullptr, "tpw_lp_backward: this mode needs the auxiliary matrix");
    TPW_CHECK_ARG(mode != TPW_LP_BWD_WMINKOWSKI || w != nullptr, "tpw_lp_backward: weighted mode needs w");
    BwdParams P;
    memset(&P, 0, sizeof(P));
    P.grad = grad; P.aux = aux; P.w = w;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return dtype == TPW_F32 ? lp_backward_typed<float>(mode, P, x1, x2, grad_x1, grad_x2, p, s)
                            : lp_backward_typed<double>(mode, P, x1, x2, grad_x1, grad_x2, p, s);
}

extern "C" int64_t tpw_lp_backward_scratch_bytes(int dtype, int mode, int64_t B, int64_t N1, int64_t N2, int64_t D, double p) {
    if (dtype != TPW_F32) return 0;
    return lp_backward_onepass_scratch_bytes(mode, B, N1, N2, D, p);
}

extern "C" int tpw_lp_backward_ws(int dtype, int mode, const void *grad, const void *aux,
                                  const void *x1, const void *x2, const void *w,
                                  void *grad_x1, void *grad_x2,
                                  int64_t B, int64_t N1, int64_t N2, int64_t D,
                                  double p, void *scratch, int64_t scratch_bytes, tpw_stream_t stream) {
    const int64_t want = dtype == TPW_F32 && B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0 && !isnan(p)
                             ? lp_backward_onepass_scratch_bytes(mode, B, N1, N2, D, p) : 0;
    const bool needs_aux = (mode == TPW_LP_BWD_WMINKOWSKI) || (mode == TPW_LP_BWD_CDIST && p != 1.0);
    const bool usable = want > 0 && scratch != nullptr && scratch_bytes >= N2 * D * 4 && grad_x1 && grad_x2 && grad && x1 && x2 &&
                        (!needs_aux || aux) && (mode != TPW_LP_BWD_WMINKOWSKI || w) &&
                        aligned16(grad) && aligned16(x1) && aligned16(x2) && aligned16(grad_x1) && aligned16(grad_x2) &&
                        aligned16(scratch) && (!needs_aux || aligned16(aux)) && (!w || aligned16(w));
    if (!usable) return tpw_lp_backward(dtype, mode, grad, aux, x1, x2, w, grad_x1, grad_x2, B, N1, N2, D, p, stream);
    clear_error();
    return lp_backward_onepass(mode, grad, aux, x1, x2, w, grad_x1, grad_x2, B, N1, N2, D, p, scratch,
                               scratch_bytes < want ? scratch_bytes : want, static_cast<cudaStream_t>(stream));
}

extern "C" int tpw_wminkowski_backward_w(int dtype, const void *grad, const void *aux,
                                         const void *x1, const void *x2, void *grad_w, void *scratch,
                                         int64_t B, int64_t N1, int64_t N2, int64_t D,
                                         double p, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_wminkowski_backward_w: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_wminkowski_backward_w: negative size");
    if (B == 0 || D == 0) return TPW_OK;
    TPW_CHECK_ARG(grad_w != nullptr, "tpw_wminkowski_backward_w: grad_w is NULL");
    TPW_CHECK_ARG(p > 0 && !isinf(p), "tpw_wminkowski_backward_w: p must be finite and positive");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = dtype == TPW_F32 ? 4 : 8;
    if (N1 == 0 || N2 == 0) {
        TPW_CUDA_OK(cudaMemsetAsync(grad_w, 0, (size_t)(B * D) * es, s));
        return TPW_OK;
    }
    TPW_CHECK_ARG(grad && aux && x1 && x2 && scratch, "tpw_wminkowski_backward_w: NULL pointer");
    BwdParams P;
    memset(&P, 0, sizeof(P));
    P.grad = grad; P.aux = aux; P.w = nullptr;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.post = 1.0; P.q = p; P.pow_spec = make_pow_spec(p); P.coef_mode = COEF_MUL;
    int st = dtype == TPW_F32 ? launch_side<float, PHI_ABSPOW, true>(P, false, x1, x2, scratch, s)
                              : launch_side<double, PHI_ABSPOW, true>(P, false, x1, x2, scratch, s);
    if (st != TPW_OK) return st;
    const long long n = B * D;
    const int threads = 128;
    const unsigned blocks = (unsigned)((n + threads - 1) / threads);
    if (dtype == TPW_F32)
        column_sum_kernel<float><<<blocks, threads, 0, s>>>((const float *)scratch, (float *)grad_w, B, N1, D, 1.0 / p);
    else
        column_sum_kernel<double><<<blocks, threads, 0, s>>>((const double *)scratch, (double *)grad_w, B, N1, D, 1.0 / p);
    TPW_LAUNCH_OK("column_sum_kernel");
    return TPW_OK;
}

extern "C" int tpw_lp_inf_backward(int dtype, const void *grad, const void *x1, const void *x2, const void *w,
                                   void *grad_x1, void *grad_x2, void *grad_w,
                                   int64_t B, int64_t N1, int64_t N2, int64_t D,
                                   int negative, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_lp_inf_backward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_lp_inf_backward: negative size");
    const long long n = B * N1 * N2;
    if (n == 0) return TPW_OK;
    TPW_CHECK_ARG(D > 0, "tpw_lp_inf_backward: D must be positive");
    TPW_CHECK_ARG(grad && x1 && x2, "tpw_lp_inf_backward: NULL input");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int threads = 256;
    const long long blocks_ll = (n + threads - 1) / threads;
    TPW_CHECK_ARG(blocks_ll < (1ll << 31), "tpw_lp_inf_backward: too many pairs");
    const unsigned blocks = (unsigned)blocks_ll;
#define TPW_INF_LAUNCH(T, NEG)                                                                              \
    lp_inf_backward_kernel<T, NEG><<<blocks, threads, 0, s>>>((const T *)grad, (const T *)x1, (const T *)x2, \
                                                              (const T *)w, (T *)grad_x1, (T *)grad_x2,      \
                                                              (T *)grad_w, B, N1, N2, D)
    if (dtype == TPW_F32) {
        if (negative) TPW_INF_LAUNCH(float, true); else TPW_INF_LAUNCH(float, false);
    } else {
        if (negative) TPW_INF_LAUNCH(double, true); else TPW_INF_LAUNCH(double, false);
    }
#undef TPW_INF_LAUNCH
    TPW_LAUNCH_OK("lp_inf_backward_kernel");
    return TPW_OK;
}

extern "C" int tpw_pair_sum_backward(int dtype, int metric, const void *grad, const void *x1, const void *x2,
                                     void *grad_x1, void *grad_x2,
                                     int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_pair_sum_backward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(metric == TPW_PAIR_CANBERRA || metric == TPW_PAIR_ADDITIVE_CHI2, "tpw_pair_sum_backward: bad metric %d", metric);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_pair_sum_backward: negative size");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = dtype == TPW_F32 ? 4 : 8;
    if (B * D == 0 || N1 == 0 || N2 == 0) {
        if (grad_x1 && B * N1 * D > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x1, 0, (size_t)(B * N1 * D) * es, s));
        if (grad_x2 && B * N2 * D > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x2, 0, (size_t)(B * N2 * D) * es, s));
        return TPW_OK;
    }
    TPW_CHECK_ARG(grad && x1 && x2 && (grad_x1 || grad_x2), "tpw_pair_sum_backward: NULL pointer");
    BwdParams P;
    memset(&P, 0, sizeof(P));
    P.grad = grad; P.aux = nullptr; P.w = nullptr;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.post = 1.0; P.coef_mode = COEF_G;
    if (metric == TPW_PAIR_CANBERRA)
        return dtype == TPW_F32 ? launch_both<float, PHI_CANBERRA, false>(P, x1, x2, grad_x1, grad_x2, s)
                                : launch_both<double, PHI_CANBERRA, false>(P, x1, x2, grad_x1, grad_x2, s);
    return dtype == TPW_F32 ? launch_both<float, PHI_CHI2, false>(P, x1, x2, grad_x1, grad_x2, s)
                            : launch_both<double, PHI_CHI2, false>(P, x1, x2, grad_x1, grad_x2, s);
}

extern "C" int tpw_jensenshannon_backward(int dtype, const void *grad, const void *out, const void *x1, const void *x2,
                                          void *grad_x1, void *grad_x2,
                                          int64_t B, int64_t N1, int64_t N2, int64_t D, double scale, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(dtype == TPW_F32 || dtype == TPW_F64, "tpw_jensenshannon_backward: dtype must be TPW_F32 or TPW_F64");
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_jensenshannon_backward: negative size");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = dtype == TPW_F32 ? 4 : 8;
    if (B * D == 0 || N1 == 0 || N2 == 0) {
        if (grad_x1 && B * N1 * D > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x1, 0, (size_t)(B * N1 * D) * es, s));
        if (grad_x2 && B * N2 * D > 0) TPW_CUDA_OK(cudaMemsetAsync(grad_x2, 0, (size_t)(B * N2 * D) * es, s));
        return TPW_OK;
    }
    TPW_CHECK_ARG(grad && x1 && x2 && (grad_x1 || grad_x2), "tpw_jensenshannon_backward: NULL pointer");
    BwdParams P;
    memset(&P, 0, sizeof(P));
    P.grad = grad; P.aux = out; P.w = nullptr;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    if (out) {
        // out = sqrt(scale * sum): d out = scale / (2 out) d sum, nothing where out == 0
        P.post = 0.5 * scale; P.coef_mode = COEF_DIV_O;
        return dtype == TPW_F32 ? launch_both<float, PHI_JS, true>(P, x1, x2, grad_x1, grad_x2, s)
                                : launch_both<double, PHI_JS, true>(P, x1, x2, grad_x1, grad_x2, s);
    }
    P.post = scale; P.coef_mode = COEF_G;
    return dtype == TPW_F32 ? launch_both<float, PHI_JS, false>(P, x1, x2, grad_x1, grad_x2, s)
                            : launch_both<double, PHI_JS, false>(P, x1, x2, grad_x1, grad_x2, s);
}
