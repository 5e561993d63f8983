// Boolean pairwise metrics on bit-packed rows.
//
// tpw_bitpack turns one-byte booleans into 32-bit words (bit t of word q = feature 32q + t) and
// records each row's population count.  The tile kernel then needs a single AND-popcount per word
// pair: with n11 = |x & y| and the row counts |x|, |y| every cell of the 2x2 contingency table
// is an exact integer, and the epilogue turns it into the requested metric with the float32
// operation order of the reference's tensor compositions (each *, +, -, / rounded separately, no
// FMA contraction), which makes the float32 output bit-identical.
//
// Tiling follows the CUDA-core L_p forward: 64 x 128 outputs per CTA of 256 threads, 4 x 8 per
// thread (two CTAs per SM), operand tiles of 64 / 128 rows x 32 words staged by TMA with the
// 128-byte swizzle (three-stage mbarrier ring), conflict-free 128-bit shared loads.  POPC issues at
// 16 lanes per clock per SM, a quarter of the logic rate, so eight AND words at a time go through
// a 7:3 carry-save adder tree (four 3-input logic pairs) and cost four POPCs instead of eight.
#include "common.cuh"
#include "bool_epilogue.cuh"

#include <stdlib.h>

namespace tpw {
namespace {

constexpr int kThreads = 256;
constexpr int kStages = 3;
constexpr int RI = 4, RJ = 8;
constexpr int TILE_I = 16 * RI;  // 64 rows of x1
constexpr int TILE_J = 16 * RJ;  // 128 rows of x2
constexpr int KC = 32; // words per 128-byte chunk row
constexpr int XT_BYTES = TILE_I * 128, YT_BYTES = TILE_J * 128;
constexpr int STAGE_BYTES = XT_BYTES + YT_BYTES;
constexpr int OFF_BAR = kStages * STAGE_BYTES;
constexpr int SMEM_BYTES = OFF_BAR + kStages * 8;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;

struct BoolParams {
    const uint32_t *x1, *x2;
    const int32_t *pop1, *pop2;
    float *out;
    long long B, N1, N2, D, W;
    long long tiles_i, tiles_j;
    int metric;
    int vec_store; // N2 % 4 == 0 and out 16-byte aligned: staged 128-bit stores
    float inv_d; // 1/D when D is a power of two (then x * inv_d == x / D exactly), else 0
    int *status;
};

// One row per warp: lane l tests byte 32q + l, the ballot is word q.
__global__ void bitpack_kernel(const uint8_t *__restrict__ src, uint32_t *__restrict__ words,
                               int32_t *__restrict__ row_pop, long long rows, long long D, long long W) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long row = warp; row < rows; row += nwarps) {
        const uint8_t *s = src + row * D;
        int pop = 0;
        for (long long q = 0; q < W; ++q) {
            const long long k = q * 32 + lane;
            const bool bit = (k < D) && (s[k] != 0);
            const uint32_t word = __ballot_sync(0xffffffffu, bit);
            if (lane == 0) words[row * W + q] = word;
            pop += __popc(word);
        }
        if (lane == 0) row_pop[row] = pop;
    }
}

// sum (weight 1) and carry (weight 2) of three bit-vectors
__device__ __forceinline__ void csa(uint32_t a, uint32_t b, uint32_t c, uint32_t &sum, uint32_t &carry) {
    sum = a ^ b ^ c;
    carry = (a & b) | (c & (a ^ b));
}

template <bool USE_TMA>
__global__ void __launch_bounds__(kThreads, 2)
bool_popcount_kernel(const __grid_constant__ CUtensorMap map1, const __grid_constant__ CUtensorMap map2,
                     const BoolParams P) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + OFF_BAR);

    const int tid = threadIdx.x;
    const uint32_t ti = tid >> 4, tj = tid & 15;
    long long tile = blockIdx.x;
    const long long tjx = tile % P.tiles_j;
    tile /= P.tiles_j;
    const long long tix = tile % P.tiles_i;
    const long long b = tile / P.tiles_i;
    const long long i0 = tix * TILE_I, j0 = tjx * TILE_J;
    const uint32_t *x1 = P.x1 + b * P.N1 * P.W;
    const uint32_t *x2 = P.x2 + b * P.N2 * P.W;
    const int nchunks = (int)((P.W + KC - 1) / KC);

    int acc[RI][RJ];
#pragma unroll
    for (int a = 0; a < RI; ++a)
#pragma unroll
        for (int c = 0; c < RJ; ++c) acc[a][c] = 0;

    auto issue = [&](int chunk) {
        const int st = chunk % kStages;
        mbar_expect_tx(&full[st], STAGE_BYTES);
        tma_load_3d(smem + st * STAGE_BYTES, &map1, &full[st], chunk * KC, (int)i0, (int)b);
        tma_load_3d(smem + st * STAGE_BYTES + XT_BYTES, &map2, &full[st], chunk * KC, (int)j0, (int)b);
    };

    if (USE_TMA) {
        if (tid == 0) {
#pragma unroll
            for (int s = 0; s < kStages; ++s) mbar_init(&full[s], 1);
            mbar_init_fence();
            tma_prefetch_descriptor(&map1);
            tma_prefetch_descriptor(&map2);
        }
        __syncthreads();
        if (tid == 0)
            for (int c = 0; c < kStages - 1 && c < nchunks; ++c) issue(c);
    }

    int failed = 0;
    for (int t = 0; t < nchunks; ++t) {
        int stage;
        if (USE_TMA) {
            if (__syncthreads_or(failed)) {
                if (tid == 0 && P.status) atomicCAS(P.status, 0, (3 << 16) | 1);
                return;
            }
            if (tid == 0 && t + kStages - 1 < nchunks) issue(t + kStages - 1);
            stage = t % kStages;
            if (!mbar_wait_bounded(&full[stage], (uint32_t)((t / kStages) & 1))) failed = 1;
        } else {
            stage = 0;
            __syncthreads();
            for (int e = tid; e < (TILE_I + TILE_J) * KC; e += kThreads) {
                const int which = e >= TILE_I * KC, el = which ? e - TILE_I * KC : e;
                const int r = el / KC, kk = el % KC;
                const long long row = (which ? j0 : i0) + r, q = (long long)t * KC + kk;
                const long long nrows = which ? P.N2 : P.N1;
                const uint32_t *src = which ? x2 : x1;
                const uint32_t v = (row < nrows && q < P.W) ? src[row * P.W + q] : 0u;
                *reinterpret_cast<uint32_t *>(smem + (which ? XT_BYTES : 0) + swz128(r, kk / 4) + (kk % 4) * 4) = v;
            }
            __syncthreads();
        }
        const unsigned char *xs = smem + stage * STAGE_BYTES;
        const unsigned char *ys = xs + XT_BYTES;
        // pairs of 16-byte groups that hold real words in this chunk (the rest is zero fill)
        const long long wleft = P.W - (long long)t * KC;
        const int cend = wleft >= KC ? 8 : (int)((wleft + 7) / 8) * 2;
#pragma unroll 1
        for (int c = 0; c < cend; c += 2) {
            uint4 xa[RI], xb[RI];
#pragma unroll
            for (int r = 0; r < RI; ++r) {
                xa[r] = *reinterpret_cast<const uint4 *>(xs + (ti + 16 * r) * 128u + ((c ^ (ti & 7u)) << 4));
                xb[r] = *reinterpret_cast<const uint4 *>(xs + (ti + 16 * r) * 128u + (((c + 1) ^ (ti & 7u)) << 4));
            }
#pragma unroll
            for (int rj = 0; rj < RJ; ++rj) {
                const uint4 ya = *reinterpret_cast<const uint4 *>(ys + (tj + 16 * rj) * 128u + ((c ^ (tj & 7u)) << 4));
                const uint4 yb = *reinterpret_cast<const uint4 *>(ys + (tj + 16 * rj) * 128u + (((c + 1) ^ (tj & 7u)) << 4));
#pragma unroll
                for (int ri = 0; ri < RI; ++ri) {
                    uint32_t s1, c1, s2, c2, s3, c3, s4, c4;
                    csa(xa[ri].x & ya.x, xa[ri].y & ya.y, xa[ri].z & ya.z, s1, c1);
                    csa(xa[ri].w & ya.w, xb[ri].x & yb.x, xb[ri].y & yb.y, s2, c2);
                    csa(s1, s2, xb[ri].z & yb.z, s3, c3);
                    csa(c1, c2, c3, s4, c4);
                    acc[ri][rj] += __popc(s3) + __popc(xb[ri].w & yb.w) + 2 * __popc(s4) + 4 * __popc(c4);
                }
            }
        }
    }
    if (USE_TMA) {
        if (__syncthreads_or(failed)) {
            if (tid == 0 && P.status) atomicCAS(P.status, 0, (3 << 16) | 2);
            return;
        }
    }

    float *out = P.out + b * P.N1 * P.N2;
    const int32_t *pop1 = P.pop1 + b * P.N1, *pop2 = P.pop2 + b * P.N2;
    if (P.vec_store) {
        // Stage the raw AND counts of the 64 x 128 tile in the (now idle) operand stages, then let
        // every warp turn whole 512-byte row segments into the metric and write them with 128-bit
        // stores.  The metric code exists four times per thread here instead of thirty-two times in
        // the register-tile order, which keeps the kernel inside the instruction cache.
        constexpr int ROWB = (TILE_J + 16) * 4;
        static_assert(TILE_I * ROWB <= kStages * STAGE_BYTES, "staging tile must fit in the operand stages");
        __syncthreads();
#pragma unroll
        for (int ri = 0; ri < RI; ++ri)
#pragma unroll
            for (int rj = 0; rj < RJ; ++rj)
                *reinterpret_cast<int *>(smem + (ti + 16 * ri) * ROWB + (tj + 16 * rj) * 4) = acc[ri][rj];
        __syncthreads();
        const int warp = tid >> 5, lane = tid & 31;
        const long long jcol = j0 + lane * 4;
        if (jcol < P.N2) { // N2 % 4 == 0: a group of four columns is entirely inside or entirely outside
            const int4 pbv = *reinterpret_cast<const int4 *>(pop2 + jcol);
            const int D = (int)P.D;
#pragma unroll 1
            for (int rr = warp; rr < TILE_I; rr += kThreads / 32) {
                const long long i = i0 + rr;
                if (i >= P.N1) break;
                const int pa = pop1[i];
                const int4 n = *reinterpret_cast<const int4 *>(smem + rr * ROWB + lane * 16);
                float4 o;
                o.x = bool_epilogue(P.metric, n.x, pa, pbv.x, D, P.inv_d);
                o.y = bool_epilogue(P.metric, n.y, pa, pbv.y, D, P.inv_d);
                o.z = bool_epilogue(P.metric, n.z, pa, pbv.z, D, P.inv_d);
                o.w = bool_epilogue(P.metric, n.w, pa, pbv.w, D, P.inv_d);
                *reinterpret_cast<float4 *>(out + i * P.N2 + jcol) = o;
            }
        }
        return;
    }
    int pb[RJ];
#pragma unroll
    for (int rj = 0; rj < RJ; ++rj) {
        const long long j = j0 + tj + 16 * rj;
        pb[rj] = j < P.N2 ? pop2[j] : 0;
    }
#pragma unroll
    for (int ri = 0; ri < RI; ++ri) {
        const long long i = i0 + ti + 16 * ri;
        if (i >= P.N1) continue;
        const int pa = pop1[i];
#pragma unroll
        for (int rj = 0; rj < RJ; ++rj) {
            const long long j = j0 + tj + 16 * rj;
            if (j >= P.N2) continue;
            out[i * P.N2 + j] = bool_epilogue(P.metric, acc[ri][rj], pa, pb[rj], (int)P.D, P.inv_d);
        }
    }
}

// ---- few words per row (D <= 128 bits): the output-bound shapes --------------------------------------------
// Same fixed roles as the few-feature L_p kernel: every lane keeps 8 x2 rows (their words and row counts) in
// registers, in two groups of 4 consecutive rows 128 apart so that each store instruction of a warp covers 512
// contiguous bytes; 128 x1 rows at a time sit in shared memory and are read as broadcasts.  Per pair: one AND and
// one POPC per word, the integer contingency counts, and the metric's float32 epilogue -- nothing is staged.
constexpr int FW_THREADS = 256, FW_ROWS = 128, FW_TILES = 4, FW_JL = 8;

// WN: words that carry features, ceil(D / 32), 1..4 (rows are stored with 4 words).  METRIC: compiled in for the two
// common metrics (jaccard, hamming), -1 = the launch's metric through the epilogue's switch.
template <int WN, int METRIC>
__global__ void __launch_bounds__(FW_THREADS, 2) bool_few_words_kernel(BoolParams P) {
    constexpr int COLS = FW_THREADS * FW_JL;
    __shared__ __align__(16) uint32_t xs[FW_ROWS * 4];
    __shared__ int xp[FW_ROWS];
    const long long tile = blockIdx.x;
    const long long tj = tile % P.tiles_j, ti = (tile / P.tiles_j) % P.tiles_i, b = tile / (P.tiles_j * P.tiles_i);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long jw = tj * COLS + (long long)warp * (32 * FW_JL);
    const long long j0 = jw + lane * 4, jlast = jw + 128 + lane * 4 + 3;
    uint32_t y[FW_JL][WN];
    int yp[FW_JL];
#pragma unroll
    for (int c = 0; c < FW_JL; ++c) {
        const long long j = j0 + (c >> 2) * 128 + (c & 3);
        if (j < P.N2) {
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(P.x2 + (b * P.N2 + j) * 4));
            const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int q = 0; q < WN; ++q) y[c][q] = w4[q];
            yp[c] = P.pop2[b * P.N2 + j];
        } else {
#pragma unroll
            for (int q = 0; q < WN; ++q) y[c][q] = 0u;
            yp[c] = 0;
        }
    }
    const int D = (int)P.D, metric = METRIC >= 0 ? METRIC : P.metric;
    const float inv_d = P.inv_d;
    for (int t = 0; t < FW_TILES; ++t) {
        const long long i0 = (ti * FW_TILES + t) * FW_ROWS;
        if (i0 >= P.N1) break;
        const int nr = (int)min((long long)FW_ROWS, P.N1 - i0);
        __syncthreads();
        if (threadIdx.x < FW_ROWS) {
            const bool in = threadIdx.x < nr;
            reinterpret_cast<uint4 *>(xs)[threadIdx.x] =
                in ? __ldg(reinterpret_cast<const uint4 *>(P.x1 + (b * P.N1 + i0 + threadIdx.x) * 4)) : make_uint4(0u, 0u, 0u, 0u);
            xp[threadIdx.x] = in ? P.pop1[b * P.N1 + i0 + threadIdx.x] : 0;
        }
        __syncthreads();
        if (j0 >= P.N2) continue;
        float *o = P.out + (b * P.N1 + i0) * P.N2 + j0;
        for (int r = 0; r < nr; ++r) {
            const uint4 xv = reinterpret_cast<const uint4 *>(xs)[r];
            const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
            const int a = xp[r];
            float res[FW_JL];
#pragma unroll
            for (int c = 0; c < FW_JL; ++c) {
                int n11 = 0;
#pragma unroll
                for (int q = 0; q < WN; ++q) n11 += __popc(xw[q] & y[c][q]);
                res[c] = bool_epilogue<true>(metric, n11, a, yp[c], D, inv_d);
            }
            float *dst = o + (long long)r * P.N2;
            if (P.vec_store && jlast < P.N2) {
                __stcs(reinterpret_cast<float4 *>(dst), make_float4(res[0], res[1], res[2], res[3]));
                __stcs(reinterpret_cast<float4 *>(dst + 128), make_float4(res[4], res[5], res[6], res[7]));
            } else {
#pragma unroll
                for (int c = 0; c < FW_JL; ++c)
                    if (j0 + (c >> 2) * 128 + (c & 3) < P.N2) dst[(c >> 2) * 128 + (c & 3)] = res[c];
            }
        }
    }
}

int launch_few_words(BoolParams P, cudaStream_t s) {
    P.tiles_i = (P.N1 + FW_ROWS * FW_TILES - 1) / (FW_ROWS * FW_TILES);
    P.tiles_j = (P.N2 + FW_THREADS * FW_JL - 1) / (FW_THREADS * FW_JL);
    const long long tiles = P.B * P.tiles_i * P.tiles_j;
    TPW_CHECK_ARG(tiles < (1ll << 31), "tpw_bool_metric_forward: too many tiles");
    const int wn = (int)((P.D + 31) / 32);
#define TPW_FEW_WORDS(M)                                                                                  \
    switch (wn) {                                                                                         \
        case 1: bool_few_words_kernel<1, M><<<(unsigned)tiles, FW_THREADS, 0, s>>>(P); break;            \
        case 2: bool_few_words_kernel<2, M><<<(unsigned)tiles, FW_THREADS, 0, s>>>(P); break;            \
        case 3: bool_few_words_kernel<3, M><<<(unsigned)tiles, FW_THREADS, 0, s>>>(P); break;            \
        default: bool_few_words_kernel<4, M><<<(unsigned)tiles, FW_THREADS, 0, s>>>(P); break;           \
    }
    if (P.metric == TPW_BOOL_JACCARD) { TPW_FEW_WORDS(TPW_BOOL_JACCARD) }
    else if (P.metric == TPW_BOOL_NE_MEAN) { TPW_FEW_WORDS(TPW_BOOL_NE_MEAN) }
    else { TPW_FEW_WORDS(-1) }
#undef TPW_FEW_WORDS
    TPW_LAUNCH_OK("bool_few_words_kernel");
    return TPW_OK;
}

} // namespace
} // namespace tpw

using namespace tpw;

extern "C" int tpw_bitpack(const uint8_t *src, uint32_t *words, int32_t *row_popcount,
                           int64_t rows, int64_t D, int64_t words_per_row, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(rows >= 0 && D >= 0, "tpw_bitpack: negative size");
    TPW_CHECK_ARG(words_per_row * 32 >= D, "tpw_bitpack: words_per_row (%lld) is too small for D = %lld",
                  (long long)words_per_row, (long long)D);
    if (rows == 0) return TPW_OK;
    TPW_CHECK_ARG(words && row_popcount && (src || D == 0), "tpw_bitpack: NULL pointer");
    TPW_CHECK_ARG(words_per_row > 0, "tpw_bitpack: words_per_row must be positive");
    const int threads = 256;
    long long blocks = (rows * 32 + threads - 1) / threads;
    const long long cap = (long long)sm_count() * 32;
    if (blocks > cap) blocks = cap;
    bitpack_kernel<<<(unsigned)blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(src, words, row_popcount, rows, D,
                                                                                         words_per_row);
    TPW_LAUNCH_OK("bitpack_kernel");
    return TPW_OK;
}

extern "C" int tpw_bool_metric_forward(int metric, const uint32_t *x1_words, const uint32_t *x2_words,
                                       const int32_t *x1_popcount, const int32_t *x2_popcount, float *out,
                                       int64_t B, int64_t N1, int64_t N2, int64_t D, int64_t words_per_row,
                                       tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(metric >= 0 && metric < TPW_BOOL_METRIC_COUNT, "tpw_bool_metric_forward: unknown metric %d", metric);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_bool_metric_forward: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(D > 0 && D <= (1 << 24), "tpw_bool_metric_forward: D must be in [1, 2^24] (exact float32 counts)");
    TPW_CHECK_ARG(words_per_row * 32 >= D, "tpw_bool_metric_forward: words_per_row too small");
    TPW_CHECK_ARG(x1_words && x2_words && x1_popcount && x2_popcount && out, "tpw_bool_metric_forward: NULL pointer");
    BoolParams P;
    memset(&P, 0, sizeof(P));
    P.x1 = x1_words; P.x2 = x2_words; P.pop1 = x1_popcount; P.pop2 = x2_popcount; P.out = out;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D; P.W = words_per_row;
    P.metric = metric;
    P.vec_store = (N2 % 4 == 0 && aligned16(out) && aligned16(x2_popcount)) ? 1 : 0;
    P.inv_d = (D & (D - 1)) == 0 ? 1.0f / (float)D : 0.f;
    // few words per row on enough rows and columns: the streaming kernel (TPW_DISABLE_SMALL_D=1 keeps the tile kernel)
    if (D <= 128 && words_per_row == 4 && N1 >= 128 && N2 >= 2048 && aligned16(x1_words) && aligned16(x2_words) &&
        !getenv("TPW_DISABLE_SMALL_D")) {
        P.vec_store = (N2 % 4 == 0 && aligned16(out)) ? 1 : 0;
        return launch_few_words(P, static_cast<cudaStream_t>(stream));
    }
    P.tiles_i = (N1 + TILE_I - 1) / TILE_I;
    P.tiles_j = (N2 + TILE_J - 1) / TILE_J;
    const long long tiles = B * P.tiles_i * P.tiles_j;
    TPW_CHECK_ARG(tiles < (1ll << 31), "tpw_bool_metric_forward: too many tiles");
    TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && B < (1ll << 31) && words_per_row < (1ll << 31),
                  "tpw_bool_metric_forward: a dimension exceeds 2^31-1");
    P.status = device_status_ptr();
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool tma_ok = !tma_disabled() && aligned16(x1_words) && aligned16(x2_words) && words_per_row % 4 == 0;
    CUtensorMap m1, m2;
    memset(&m1, 0, sizeof(m1));
    memset(&m2, 0, sizeof(m2));
    if (tma_ok) {
        int st = make_tensor_map_3d(&m1, x1_words, 4, words_per_row, N1, B, KC, TILE_I, true);
        if (st != TPW_OK) return st;
        st = make_tensor_map_3d(&m2, x2_words, 4, words_per_row, N2, B, KC, TILE_J, true);
        if (st != TPW_OK) return st;
        TPW_CUDA_OK(cudaFuncSetAttribute(bool_popcount_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
        bool_popcount_kernel<true><<<(unsigned)tiles, kThreads, SMEM_ALLOC, s>>>(m1, m2, P);
    } else {
        TPW_CUDA_OK(cudaFuncSetAttribute(bool_popcount_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
        bool_popcount_kernel<false><<<(unsigned)tiles, kThreads, SMEM_ALLOC, s>>>(m1, m2, P);
    }
    TPW_LAUNCH_OK("bool_popcount_kernel");
    return TPW_OK;
}
