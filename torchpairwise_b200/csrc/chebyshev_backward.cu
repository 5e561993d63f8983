// Backward of the Chebyshev distance (cdist with p = +inf) for float32, in three kernels.
//
//   out[b,i,j] = max_k |x1[b,i,k] - x2[b,j,k]|
//   grad_x1[b,i,k] = sum_j g[b,i,j] * sgn(d) * [|d| == out]      (d = x1[b,i,k] - x2[b,j,k]; nothing where out == 0)
//   grad_x2[b,j,k] = -sum_i (same term)
//
// (ATen's cdist backward under OPS/pairwise_metrics.cpp:305: every coordinate that attains the maximum
// receives the gradient.)  The dense form evaluates the test for every (i, j, k) once per gradient.
// Here the attaining coordinate is found once per pair and both gradients are then scattered:
//
//   1. chebyshev_match_kernel: the forward tile (x1 / x2 chunks staged by TMA, 4 x 4 pairs per thread) re-forms
//      d and compares |d| with the saved output; a match adds 65536 + k to the pair's code and d to a side sum,
//      so that code >> 16 counts the attaining coordinates.  One coordinate: the pair's code becomes
//      k | sign << 31.  None (out == 0, NaN, padding): the pair is skipped.  Several (a tied maximum): the pair is
//      marked and counted in a device counter.
//   2. chebyshev_scatter_kernel (once per gradient): four threads per x1 row (x2 row), a quarter of the features
//      each, walk over the row's pairs in order and add +-g into their part of a shared-memory gradient block at
//      the coded coordinate; for a marked pair they walk over their features themselves.  Every gradient
//      element has one owner and a fixed order of additions: deterministic, no atomics.
//   3. Exact ties are rare in continuous data (a few hundred among the 2.7e8 pairs of 256 normal features) but
//      the rule in lattice-valued data.  When more than one pair in 32768 is marked, the scatter kernels return
//      at once and the dense kernel of lp_backward.cu, which otherwise returns at once, writes both gradients.
#include "common.cuh"

namespace tpw {
namespace {

constexpr int kThreads = 256;
constexpr int kStages = 3;
constexpr int RI = 4, RJ = 4;               // pairs per thread: 4 x1 rows by 4 x2 rows (three registers per pair)
constexpr int TI = 16 * RI, TJ = 16 * RJ;   // 64 x 64 pairs per CTA
constexpr int KC = 32;                      // features per staged chunk (128 bytes per row)
constexpr int XB = TI * 128, YB = TJ * 128; // bytes of one stage's x1 and x2 tiles
constexpr int STAGE = XB + YB;
constexpr int OFF_BAR = kStages * STAGE;
constexpr int MATCH_SMEM = OFF_BAR + kStages * 8 + 1024;
constexpr uint32_t kSkip = 0xffffffffu;   // no gradient from this pair
constexpr uint32_t kTied = 0xfffffffeu;   // several coordinates attain the maximum

// more marked pairs than this and the dense kernel takes over (the same rule on both sides of the hand-over)
__host__ __device__ inline unsigned long long tie_limit(long long pairs) { return (unsigned long long)(pairs >> 15) + 64ull; }

struct MatchParams {
    const float *x1, *x2, *out;
    uint32_t *code;
    unsigned long long *ties;
    long long B, N1, N2, D, tiles_i, tiles_j;
    int *status;
};

__device__ __forceinline__ float match_mask(float d, float o) {   // 1.0 where |d| == o, else 0.0
    float m;
    asm("set.eq.f32.f32 %0, %1, %2;" : "=f"(m) : "f"(fabsf(d)), "f"(o));
    return m;
}

template <int ROWS>
__device__ __forceinline__ void stage_rows_plain(unsigned char *tile, const float *base, long long row0, long long nrows,
                                                 long long D, long long k0) {
    for (int e = threadIdx.x; e < ROWS * KC; e += kThreads) {
        const int r = e / KC, kk = e % KC;
        const long long row = row0 + r, k = k0 + kk;
        const float v = (row < nrows && k < D) ? base[row * D + k] : 0.f;
        *reinterpret_cast<float *>(tile + swz128(r, kk / 4) + (kk % 4) * 4) = v;
    }
}

template <bool USE_TMA>
__global__ void __launch_bounds__(kThreads, 2)
chebyshev_match_kernel(const __grid_constant__ CUtensorMap map1, const __grid_constant__ CUtensorMap map2, const MatchParams P) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + OFF_BAR);

    const int tid = threadIdx.x;
    const int ti = tid >> 4, tj = tid & 15;
    long long tile = blockIdx.x;
    const long long tjx = tile % P.tiles_j;
    tile /= P.tiles_j;
    const long long tix = tile % P.tiles_i;
    const long long b = tile / P.tiles_i;
    const long long i0 = tix * TI, j0 = tjx * TJ;

    const float *x1 = P.x1 + b * P.N1 * P.D;
    const float *x2 = P.x2 + b * P.N2 * P.D;
    const float *out = P.out + b * P.N1 * P.N2;
    const int nchunks = (int)((P.D + KC - 1) / KC);

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
                mbar_expect_tx(&full[c], STAGE);
                tma_load_3d(smem + c * STAGE, &map1, &full[c], c * KC, (int)i0, (int)b);
                tma_load_3d(smem + c * STAGE + XB, &map2, &full[c], c * KC, (int)j0, (int)b);
            }
        }
    }

    // the saved maximum of every pair; -1 (never equal to an absolute value) where the pair does not exist or
    // the maximum is 0, in which case the gradient is defined as 0
    float o[RI][RJ];
    float acc[RI][RJ];   // sum of (65536 + k) over the attaining coordinates: exact in float32 up to 255 of them
    float sgn[RI][RJ];   // sum of d over the attaining coordinates
#pragma unroll
    for (int ri = 0; ri < RI; ++ri) {
        const long long i = i0 + ti + 16 * ri;
#pragma unroll
        for (int rj = 0; rj < RJ; ++rj) {
            const long long j = j0 + tj + 16 * rj;
            float v = -1.f;
            if (i < P.N1 && j < P.N2) {
                v = out[i * P.N2 + j];
                if (v == 0.f) v = -1.f;
            }
            o[ri][rj] = v;
            acc[ri][rj] = 0.f;
            sgn[ri][rj] = 0.f;
        }
    }

    int failed = 0;
    for (int t = 0; t < nchunks; ++t) {
        int stage;
        if (USE_TMA) {
            if (__syncthreads_or(failed)) {
                if (tid == 0) {
                    if (P.status) atomicCAS(P.status, 0, (9 << 16) | 1);
                    // the chunks issued earlier may still be landing: the CTA stays (bounded) until they have
                    for (int c = t; c < t + kStages - 1 && c < nchunks; ++c) mbar_wait_bounded(&full[c % kStages], (uint32_t)((c / kStages) & 1));
                }
                return;
            }
            const int nxt = t + kStages - 1;
            if (nxt < nchunks && tid == 0) {
                const int ns = nxt % kStages;
                mbar_expect_tx(&full[ns], STAGE);
                tma_load_3d(smem + ns * STAGE, &map1, &full[ns], nxt * KC, (int)i0, (int)b);
                tma_load_3d(smem + ns * STAGE + XB, &map2, &full[ns], nxt * KC, (int)j0, (int)b);
            }
            stage = t % kStages;
            if (!mbar_wait_bounded(&full[stage], (uint32_t)((t / kStages) & 1))) failed = 1;
        } else {
            stage = 0;
            __syncthreads();
            stage_rows_plain<TI>(smem, x1, i0, P.N1, P.D, (long long)t * KC);
            stage_rows_plain<TJ>(smem + XB, x2, j0, P.N2, P.D, (long long)t * KC);
            __syncthreads();
        }
        const unsigned char *xs = smem + stage * STAGE;
        const unsigned char *ys = xs + XB;
        const uint32_t xrow = ti, yrow = tj;      // (row + 16 r) & 7 == row & 7
        const long long kleft = P.D - (long long)t * KC;
        const int cmax = kleft < KC ? (int)((kleft + 3) / 4) : 8;
#pragma unroll 1
        for (int c = 0; c < cmax; ++c) {
            float kce[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) kce[e] = (float)(0x10000 + t * KC + c * 4 + e);
            float4 xa[RI];
#pragma unroll
            for (int r = 0; r < RI; ++r)
                xa[r] = *reinterpret_cast<const float4 *>(xs + (xrow + 16 * r) * 128u + ((c ^ (xrow & 7u)) << 4));
#pragma unroll
            for (int rj = 0; rj < RJ; ++rj) {
                const float4 yb = *reinterpret_cast<const float4 *>(ys + (yrow + 16 * rj) * 128u + ((c ^ (yrow & 7u)) << 4));
                const float *ye = reinterpret_cast<const float *>(&yb);
#pragma unroll
                for (int ri = 0; ri < RI; ++ri) {
                    const float *xe = reinterpret_cast<const float *>(&xa[ri]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        // four operations per element and no predicate registers: subtract, compare into 1.0 / 0.0 (the
                        // compare issues at half the rate of the others), and two fused multiply-adds that take the match
                        // as a factor.  Features past D are zero on both sides: |0| never equals a positive maximum.
                        const float d = xe[e] - ye[e];
                        const float m = match_mask(d, o[ri][rj]);
                        acc[ri][rj] = fmaf(m, kce[e], acc[ri][rj]);
                        sgn[ri][rj] = fmaf(m, d, sgn[ri][rj]);
                    }
                }
            }
        }
    }
    if (USE_TMA) {
        if (__syncthreads_or(failed)) {
            if (tid == 0 && P.status) atomicCAS(P.status, 0, (9 << 16) | 2);
            return;
        }
    }

    uint32_t *code = P.code + b * P.N1 * P.N2;
    int tied = 0;
#pragma unroll
    for (int ri = 0; ri < RI; ++ri) {
        const long long i = i0 + ti + 16 * ri;
#pragma unroll
        for (int rj = 0; rj < RJ; ++rj) {
            const long long j = j0 + tj + 16 * rj;
            // 0 * d is NaN for an infinite or NaN difference next to a real match: such pairs go the slow, exact way too
            const uint32_t a = (uint32_t)acc[ri][rj];
            const float sg = sgn[ri][rj];
            uint32_t cd = kSkip;
            if ((a >> 16) == 1u && sg == sg) cd = (a & 0xffffu) | (sg < 0.f ? 0x80000000u : 0u);
            else if (a != 0u) { cd = kTied; ++tied; }
            if (i < P.N1 && j < P.N2) code[i * P.N2 + j] = cd;
        }
    }
    const int total = __syncthreads_count(tied != 0) ? 1 : 0;
    if (total) {   // rare: let every thread with marked pairs add its own count
        if (tied) atomicAdd(P.ties, (unsigned long long)tied);
    }
}

// ---- scatter ---------------------------------------------------------------------------------------------------------
constexpr int SR = 128;          // gradient rows per CTA
constexpr int SQ = 4;            // threads per gradient row (all of them stage the pairs)
constexpr int WQ = 4;            // of which this many walk over the pairs, each owning SD / WQ of the CTA's features
constexpr int STHR = SR * SQ;    // 512 threads: sixteen warps keep the shared-memory read-modify-write chains overlapped
constexpr int SD = 256;          // features per CTA
constexpr int SP = 32;           // pairs per gradient row staged at a time
constexpr int ACC_STRIDE = SD + 1;
constexpr int SCATTER_SMEM = SR * ACC_STRIDE * 4 + 2 * SR * (SP + 1) * 4;

struct ScatterParams {
    const float *grad;
    const uint32_t *code;
    const unsigned long long *ties;
    const float *x1, *x2, *fwd;   // read for marked pairs only
    float *out;                   // [B, NR, D]
    long long B, N1, N2, D, NR, tiles_r, tiles_k;
};

// A pair whose maximum is attained by several coordinates: every one of them in [klo, khi) receives +-g (ascending k).
__device__ __noinline__ void scatter_tied(float *row, const float *a, const float *c, float o, float g, int k0, int klo, int khi,
                                          bool negate) {
    for (int k = klo; k < khi; ++k) {
        const float d = a[k0 + k] - c[k0 + k];
        if (fabsf(d) == o) row[k] += (d < 0.f) != negate ? -g : g;
    }
}

// COLS = false: grad_x1.  Thread (r, q) owns features [q * 64, q * 64 + 64) of x1 row r0 + r and walks over j in ascending
// order.  COLS = true: grad_x2, the same with x2 row r0 + r, i ascending and the sign flipped.  The pairs are staged 32
// per gradient row at a time through shared memory (whole 128-byte segments of g and of the codes from global memory,
// the next tile already in registers while the current one is applied); every thread of a row looks at all of the
// row's pairs and applies those whose coordinate falls in its quarter.
template <bool COLS>
__global__ void __launch_bounds__(STHR, 1) chebyshev_scatter_kernel(const ScatterParams P) {
    if (*P.ties > tie_limit(P.B * P.N1 * P.N2)) return;   // tied maxima everywhere: the dense kernel that follows writes this gradient
    extern __shared__ float sm[];
    float *accs = sm;
    float *gs = sm + SR * ACC_STRIDE;
    uint32_t *cs = reinterpret_cast<uint32_t *>(gs + SR * (SP + 1));
    const int tid = threadIdx.x;
    long long tile = blockIdx.x;
    const long long tk = tile % P.tiles_k;
    tile /= P.tiles_k;
    const long long tr = tile % P.tiles_r;
    const long long b = tile / P.tiles_r;
    const long long r0 = tr * SR;
    const int k0 = (int)(tk * SD);
    const int kn = (int)((P.D - k0) < SD ? (P.D - k0) : SD);
    for (int e = tid; e < SR * ACC_STRIDE; e += STHR) accs[e] = 0.f;
    const float *grad = P.grad + b * P.N1 * P.N2;
    const uint32_t *code = P.code + b * P.N1 * P.N2;
    const int r = tid % SR, q = tid / SR;        // a warp holds 32 consecutive rows of one quarter
    float *mine = accs + r * ACC_STRIDE;
    const long long NS = COLS ? P.N1 : P.N2;     // length of the walk

    // staging: element e = tid + u * STHR of a tile is (row e / SP, step e % SP) for rows and (step e / SR, column
    // e % SR) for columns, so that consecutive threads read consecutive addresses of g and code.  Everything that does
    // not depend on the tile is worked out once: a thread's step (column) is fixed, its rows (steps) advance by a
    // constant, so a tile costs it one pointer bump and one predicate per element.
    constexpr int PER = SR * SP / STHR;          // 8 elements of each array per thread
    constexpr int UR = COLS ? STHR / SR : STHR / SP;      // rows (steps) between a thread's consecutive elements
    const int fix = COLS ? tid % SR : tid % SP;           // column of the gradient row block / step inside the tile
    const int var0 = COLS ? tid / SR : tid / SP;          // first step / first row
    // offset of element u = 0 of tile s0 = 0, then per element and per tile
    const long long off0 = COLS ? (long long)var0 * P.N2 + r0 + fix : (r0 + var0) * P.N2 + fix;
    const long long off_u = (long long)UR * P.N2;
    const long long off_tile = COLS ? (long long)SP * P.N2 : (long long)SP;
    const bool fix_ok = COLS ? (r0 + fix < P.N2) : true;
    const long long var_end = COLS ? P.N1 : P.N1 - r0;    // rows: row index below this; columns: step s0 + step below this
    const int sm0 = COLS ? fix * (SP + 1) + var0 : var0 * (SP + 1) + fix;
    constexpr int sm_u = COLS ? UR : UR * (SP + 1);
    float gr[PER];
    uint32_t cr[PER];
    auto fetch = [&](long long s0) {
        const float *gp = grad + off0 + (s0 / SP) * off_tile;
        const uint32_t *cp = code + off0 + (s0 / SP) * off_tile;
        const bool tile_ok = COLS ? fix_ok : (s0 + fix < P.N2);
        const long long first = COLS ? s0 + var0 : (long long)var0;
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const bool ok = tile_ok && first + (long long)u * UR < var_end;
            gr[u] = ok ? __ldg(gp) : 0.f;
            cr[u] = ok ? __ldg(cp) : kSkip;
            gp += off_u;
            cp += off_u;
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            gs[sm0 + u * sm_u] = gr[u];
            cs[sm0 + u * sm_u] = cr[u];
        }
    };
    fetch(0);
    for (long long s0 = 0; s0 < NS; s0 += SP) {
        __syncthreads();                         // everyone is done with the previous tile
        stash();
        __syncthreads();
        if (s0 + SP < NS) fetch(s0 + SP);
        if (q < WQ) {
            // WQ walkers per gradient row, each owning SD / WQ features: a pair costs a walker a load, a subtract and an
            // unsigned compare unless its coordinate falls into the walker's range
            constexpr int WD = SD / WQ;
            const int kq = k0 + q * WD;
            const int kw = kn - q * WD < WD ? kn - q * WD : WD;     // features of this walker that exist (may be <= 0)
            float *wmine = mine + q * WD;
#pragma unroll 8
            for (int ss = 0; ss < SP; ++ss) {
                const uint32_t cd = cs[r * (SP + 1) + ss];
                if (cd < kTied) {
                    const int k = (int)(cd & 0xffffu) - kq;
                    if ((unsigned)k < (unsigned)(kw > 0 ? kw : 0)) {
                        const float g = gs[r * (SP + 1) + ss];
                        wmine[k] += __uint_as_float(__float_as_uint(g) ^ ((cd ^ (COLS ? 0x80000000u : 0u)) & 0x80000000u));
                    }
                } else if (cd == kTied && kw > 0) {
                    const long long i = COLS ? s0 + ss : r0 + r, j = COLS ? r0 + r : s0 + ss;
                    scatter_tied(wmine, P.x1 + (b * P.N1 + i) * P.D, P.x2 + (b * P.N2 + j) * P.D, P.fwd[(b * P.N1 + i) * P.N2 + j],
                                 gs[r * (SP + 1) + ss], kq, 0, kw, COLS);
                }
            }
        }
    }
    __syncthreads();
    float *out = P.out + b * P.NR * P.D;
    for (int rr = tid / 32; rr < SR; rr += STHR / 32) {
        const long long row = r0 + rr;
        if (row >= P.NR) break;
        for (int k = tid % 32; k < kn; k += 32) out[row * P.D + k0 + k] = accs[rr * ACC_STRIDE + k];
    }
}

constexpr long long kHeader = 256;   // the counter of marked pairs, padded so that the codes start on an aligned address

} // namespace
} // namespace tpw

using namespace tpw;

extern "C" int64_t tpw_chebyshev_backward_scratch_bytes(int dtype, int64_t B, int64_t N1, int64_t N2, int64_t D) {
    if (dtype != TPW_F32 || B <= 0 || N1 <= 0 || N2 <= 0 || D < 16 || D >= 65536) return 0;
    if (N1 >= (1ll << 31) || N2 >= (1ll << 31) || B >= (1ll << 31)) return 0;
    return kHeader + 4 * B * N1 * N2;
}

extern "C" int tpw_chebyshev_backward_ws(const void *grad, const void *out, const void *x1, const void *x2,
                                         void *grad_x1, void *grad_x2, void *scratch, int64_t scratch_bytes,
                                         int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    const int64_t need = tpw_chebyshev_backward_scratch_bytes(TPW_F32, B, N1, N2, D);
    TPW_CHECK_ARG(need > 0, "tpw_chebyshev_backward_ws: this problem is served by tpw_lp_backward (scratch query returned 0)");
    TPW_CHECK_ARG(scratch != nullptr && scratch_bytes >= need, "tpw_chebyshev_backward_ws: scratch too small (%lld < %lld)",
                  (long long)scratch_bytes, (long long)need);
    TPW_CHECK_ARG(aligned16(scratch), "tpw_chebyshev_backward_ws: scratch must be 16-byte aligned");
    TPW_CHECK_ARG(grad && out && x1 && x2, "tpw_chebyshev_backward_ws: NULL input");
    if (!grad_x1 && !grad_x2) return TPW_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long *ties = static_cast<unsigned long long *>(scratch);
    uint32_t *code = reinterpret_cast<uint32_t *>(static_cast<unsigned char *>(scratch) + kHeader);
    TPW_CUDA_OK(cudaMemsetAsync(ties, 0, kHeader, s));

    MatchParams M;
    memset(&M, 0, sizeof(M));
    M.x1 = static_cast<const float *>(x1); M.x2 = static_cast<const float *>(x2); M.out = static_cast<const float *>(out);
    M.code = code; M.ties = ties;
    M.B = B; M.N1 = N1; M.N2 = N2; M.D = D;
    M.tiles_i = (N1 + TI - 1) / TI; M.tiles_j = (N2 + TJ - 1) / TJ;
    M.status = device_status_ptr();
    const long long tiles = B * M.tiles_i * M.tiles_j;
    TPW_CHECK_ARG(tiles < (1ll << 31), "tpw_chebyshev_backward_ws: too many tiles (%lld)", tiles);
    const bool tma_ok = !tma_disabled() && aligned16(x1) && aligned16(x2) && (D * 4) % 16 == 0;
    CUtensorMap m1, m2;
    memset(&m1, 0, sizeof(m1));
    memset(&m2, 0, sizeof(m2));
    if (tma_ok) {
        int st = make_tensor_map_3d(&m1, x1, 4, D, N1, B, KC, TI, true);
        if (st != TPW_OK) return st;
        st = make_tensor_map_3d(&m2, x2, 4, D, N2, B, KC, TJ, true);
        if (st != TPW_OK) return st;
        TPW_CUDA_OK(cudaFuncSetAttribute(chebyshev_match_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, MATCH_SMEM));
        chebyshev_match_kernel<true><<<(unsigned)tiles, kThreads, MATCH_SMEM, s>>>(m1, m2, M);
    } else {
        TPW_CUDA_OK(cudaFuncSetAttribute(chebyshev_match_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, MATCH_SMEM));
        chebyshev_match_kernel<false><<<(unsigned)tiles, kThreads, MATCH_SMEM, s>>>(m1, m2, M);
    }
    TPW_LAUNCH_OK("chebyshev_match_kernel");

    ScatterParams S;
    memset(&S, 0, sizeof(S));
    S.grad = static_cast<const float *>(grad); S.code = code; S.ties = ties;
    S.x1 = M.x1; S.x2 = M.x2; S.fwd = M.out;
    S.B = B; S.N1 = N1; S.N2 = N2; S.D = D;
    S.tiles_k = (D + SD - 1) / SD;
    if (grad_x1) {
        S.out = static_cast<float *>(grad_x1); S.NR = N1; S.tiles_r = (N1 + SR - 1) / SR;
        const long long n = B * S.tiles_r * S.tiles_k;
        TPW_CHECK_ARG(n < (1ll << 31), "tpw_chebyshev_backward_ws: too many row blocks");
        TPW_CUDA_OK(cudaFuncSetAttribute(chebyshev_scatter_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCATTER_SMEM));
        chebyshev_scatter_kernel<false><<<(unsigned)n, STHR, SCATTER_SMEM, s>>>(S);
        TPW_LAUNCH_OK("chebyshev_scatter_kernel (grad_x1)");
    }
    if (grad_x2) {
        S.out = static_cast<float *>(grad_x2); S.NR = N2; S.tiles_r = (N2 + SR - 1) / SR;
        const long long n = B * S.tiles_r * S.tiles_k;
        TPW_CHECK_ARG(n < (1ll << 31), "tpw_chebyshev_backward_ws: too many row blocks");
        TPW_CUDA_OK(cudaFuncSetAttribute(chebyshev_scatter_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SCATTER_SMEM));
        chebyshev_scatter_kernel<true><<<(unsigned)n, STHR, SCATTER_SMEM, s>>>(S);
        TPW_LAUNCH_OK("chebyshev_scatter_kernel (grad_x2)");
    }
    // tied maxima everywhere: the dense kernel writes both gradients; otherwise it returns at once
    return lp_backward_cdist_inf_if(ties, tie_limit(B * N1 * N2), grad, out, x1, x2, grad_x1, grad_x2, B, N1, N2, D, s);
}
