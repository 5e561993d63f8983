// Dense-contraction metrics (sqeuclidean, euclidean, cosine similarity / distance, correlation,
// linear kernel) on the 5th-generation tensor cores: TMA -> shared memory -> tcgen05.mma with fp32
// accumulators in tensor memory -> tcgen05.ld -> fused epilogue -> global.
//
// Precision.  The inputs are fp32 and the parity contract is rtol 1e-4 / atol 1e-5, which a single
// bf16 or tf32 pass does not meet.  Each operand is therefore split once into a bf16 "high" part
// and a bf16 "low" part (x = xh + xl up to 2^-17 relative) and the cross term is accumulated as
// xh.yh + xh.yl + xl.yh (three MMAs per k-step into the same fp32 accumulator; xl.yl is below the
// fp32 rounding of the sum).  Row norms are summed in fp32 from the unsplit values by the same
// pre-pass.
//
// Kernel.  Persistent, one CTA per SM, 320 threads: warp 0 = TMA producer (one lane), warp 1 =
// tensor-memory owner and MMA issuer (one lane), warps 2..9 = epilogue (each owns the 32 TMEM lanes
// its warp id selects and one half of the columns).  Output tile 128 x 256; k-step 64 bf16 = one 128-byte swizzled row; a stage
// holds xh, xl (2 x 16 KB) and yh, yl (2 x 32 KB); two stages.  The 512 TMEM columns hold two
// 128 x 256 fp32 accumulators so the epilogue of tile t overlaps the MMAs of tile t + 1.
// No cluster launch: every CTA fetches its own tiles, with plain per-CTA TMA loads, from this GPU's memory.
//
// Three more instantiations share the pipeline: (1) kind::tf32 operands (high/low tf32 parts in fp32
// containers, 32 elements per k-step) for the gradient products of the backward and for plain dot
// products, with the reduction cut into chunks of 64 elements whose accumulators the epilogue warps
// add, rounded to nearest, into register-resident sums (the tensor cores add into tensor memory with
// truncation; see dense_backward_tensor below); (2) a row-minimum epilogue that folds each thread's
// accumulator row into one 64-bit key and stores no tile; (3) SELF, which zeroes the diagonal.
//
// Every wait (mbarrier) is bounded; a warp that gives up raises a CTA-wide abort flag that the other
// roles poll, everybody falls through to the final barrier, tensor memory is released, and the
// device status word reports the site.
#include "common.cuh"
#include "tcgen05.cuh"

#include <cuda_bf16.h>
#include <math.h>

namespace tpw {
namespace {

constexpr int BM = 128;           // rows of x1 per tile (TMEM lanes)
constexpr int BN = 256;           // rows of x2 per tile (TMEM columns per accumulator)
constexpr int BK = 64;            // bf16 per k-step: 128 bytes
constexpr int kStages = 2;
constexpr int kMmasPerStep = 4;    // a 128-byte operand row feeds four MMAs of 32 bytes (16 bf16 or 8 tf32) each
constexpr int A_BYTES = BM * BK * 2;          // 16 KB
constexpr int B_BYTES = BN * BK * 2;          // 32 KB
constexpr int STAGE_BYTES = 2 * A_BYTES + 2 * B_BYTES; // xh | xl | yh | yl = 96 KB
constexpr int OFF_BAR = kStages * STAGE_BYTES;
// barriers: full_hi[2], full_lo[2], empty[2], tmem_full[2], tmem_empty[2]; then the TMEM base address and the abort flag
constexpr int OFF_TMEM_PTR = OFF_BAR + 10 * 8;
constexpr int OFF_ABORT = OFF_TMEM_PTR + 4;
// per epilogue warp a 32 x 32 fp32 staging block (4 KB) used to turn "one row per thread" into
// "eight lanes per 128-byte row segment" before the global stores
constexpr int OFF_STAGE = (OFF_ABORT + 4 + 127) / 128 * 128;
constexpr int SMEM_BYTES = OFF_STAGE + 8 * 4096;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
constexpr int kEpilogueWarps = 8;             // two per TMEM lane quarter, each draining half of the columns
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr uint32_t kTmemCols = 512;

struct GemmParams {
    const float *n1sq, *n2sq; // squared row norms [B*N1], [B*N2]
    float *out;
    long long B, N1, N2, D;
    long long tiles_m, tiles_n, tiles;
    int epilogue;
    int self;                 // x2 is x1: the diagonal of the distance epilogues is exactly zero
    int vec_store;            // N2 % 4 == 0 and out 16-byte aligned
    int kchunk;               // k-steps accumulated in tensor memory before the sum moves to registers (0: all)
    unsigned long long *rowmin_keys; // ROWMIN instantiation: [B*N1] keys (float bits << 32 | x2 row), nothing is stored to out
    // TOPK instantiations: per row and per (column tile, half) a sorted list of the k smallest keys,
    // [B*N1][topk_L][topk_k], and [B*N1] published upper bounds of the row's k-th smallest key
    unsigned long long *topk_lists, *topk_thr;
    int topk_k, topk_L;
    long long tn0;            // first column tile of this launch (tiles_n counts from it); top-k runs in column ranges
    int *status;
};

// D[tmem] (+)= A[smem] * B[smem]^T, fp32 accumulate; TF32 = false: bf16 operands (K = 16 per
// instruction), true: tf32 operands in 32-bit containers (K = 8 per instruction)
template <bool TF32>
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    if (TF32)
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
    else
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "setp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
            : "memory");
}
// MN-major 32-bit tile: the only layout tcgen05 takes for it is the 128-byte swizzle with 32-byte
// atoms (layout type 1): rows of 128 bytes are k, four rows form one 512-byte atom (stride between
// 4-row groups in bits [32,46)), and the 32-value blocks along M/N follow each other at the leading
// byte offset in bits [16,30) (here 4096: 32 k-rows of 128 bytes).
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(4096 >> 4) << 16;
    d |= (uint64_t)(512 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)1 << 61;
    return d;
}
// Instruction descriptor: D = fp32 (bits [4,6) = 1); A and B formats in bits [7,10) and [10,13):
// 1 = bf16 under kind::f16, 2 = tf32 under kind::tf32; bit 15 / bit 16 = 1 when A / B is MN-major
// (0: K-major); N >> 3 in bits [17,23), M >> 4 in bits [24,29).
__device__ __forceinline__ uint32_t make_idesc(int M, int N, bool tf32, bool a_mn = false, bool b_mn = false) {
    const uint32_t fmt = tf32 ? 2u : 1u;
    return (1u << 4) | (fmt << 7) | (fmt << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// n1, n2: squared row norms for the two distance epilogues, reciprocal row norms (0 for an all-zero
// row, whose dot products are exactly 0 anyway) for the cosine family.
template <int EPI>
__device__ __forceinline__ float dot_epilogue(float dot, float n1, float n2, bool diag) {
    if (EPI == TPW_DOT_LINEAR) return dot;
    if (EPI == TPW_DOT_SQEUCLIDEAN) return diag ? 0.f : fmaxf(fmaf(-2.f, dot, n1 + n2), 0.f);
    if (EPI == TPW_DOT_EUCLIDEAN) return diag ? 0.f : sqrtf(fmaxf(fmaf(-2.f, dot, n1 + n2), 0.f));
    const float s = dot * (n1 * n2);
    if (EPI == TPW_DOT_COSINE_SIM) return s;
    const float dist = 1.f - s;
    if (EPI == TPW_DOT_COSINE_DIST) return fminf(fmaxf(dist, 0.f), 2.f);
    return dist;
}

// TF32 = false: operands are bf16 high/low parts, 64 per k-step; true: tf32 high/low parts in fp32
// containers, 32 per k-step.  Either way a k-step is one 128-byte swizzled row per operand row and
// four MMAs per operand pair, so the pipeline below is the same.
// Tile index -> (column tile, row tile, batch).  Column tiles vary fastest, so that consecutive tiles
// share the x1 rows and stream the (usually L2-resident) x2 rows -- except for the top-k epilogue, where
// row tiles vary fastest: a row's column tiles are then visited one after another over the run, and the
// bound published by its earlier column tiles prunes the later ones.
template <bool ROW_TILES_FASTEST>
__device__ __forceinline__ void decode_tile(long long tile, const GemmParams &P, long long &tn, long long &tm, long long &b) {
    if (ROW_TILES_FASTEST) {
        tm = tile % P.tiles_m; tile /= P.tiles_m;
        tn = tile % P.tiles_n + P.tn0;
        b = tile / P.tiles_n;
    } else {
        tn = tile % P.tiles_n; tile /= P.tiles_n;
        tm = tile % P.tiles_m;
        b = tile / P.tiles_m;
    }
}

// Sorted insertion into an ascending register-resident list (branch-free: slot t becomes
// min(max(previous slot, key), slot t)); the largest entry falls off the end.
template <int N>
__device__ __forceinline__ void sorted_insert(unsigned long long (&lst)[N], unsigned long long key) {
#pragma unroll
    for (int t = N - 1; t > 0; --t) {
        const unsigned long long hi = lst[t - 1] > key ? lst[t - 1] : key;
        lst[t] = hi < lst[t] ? hi : lst[t];
    }
    lst[0] = key < lst[0] ? key : lst[0];
}

// AMN / BMN (tf32 only): the operand is MN-major, i.e. its global rows run along k and each row holds
// the tile's M (or N) values contiguously, so a matrix can be contracted over its row index without a
// transposed copy.  Such a tile is staged as blocks of {32 values, 32 k-rows} (one TMA box each, 4 KB,
// 128-byte swizzle with 32-byte atoms): block m holds values 32m..32m+31, an MMA consumes 8 k-rows = 1024 bytes.
template <int EPI, bool SELF, bool TF32, bool ROWMIN = false, bool AMN = false, bool BMN = false, int TOPK = 0>
__global__ void __launch_bounds__(kThreads, 1)
gemm_metric_kernel(const __grid_constant__ CUtensorMap map_xh, const __grid_constant__ CUtensorMap map_xl,
                   const __grid_constant__ CUtensorMap map_yh, const __grid_constant__ CUtensorMap map_yl,
                   const GemmParams P) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // a stage lands in two halves so that the xh.yh products can start while xl, yl are still in flight
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + OFF_BAR);   // xh + yh of a stage
    uint64_t *full_lo = full + kStages;                               // xl + yl of a stage
    uint64_t *empty = full_lo + kStages;
    uint64_t *tmem_full = empty + kStages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_ptr = reinterpret_cast<uint32_t *>(smem + OFF_TMEM_PTR);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + OFF_ABORT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int BKE = TF32 ? BK / 2 : BK; // operand elements per k-step
    const int nkb = (int)((P.D + BKE - 1) / BKE);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&full_lo[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], kEpilogueWarps); }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_descriptor(&map_xh);
        tma_prefetch_descriptor(&map_xl);
        tma_prefetch_descriptor(&map_yh);
        tma_prefetch_descriptor(&map_yl);
    }
    if (warp == 1) {
        tmem_alloc(tmem_ptr, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < P.tiles && ok; tile += gridDim.x) {
                long long tn, tm, b;
                decode_tile<TOPK != 0>(tile, P, tn, tm, b);
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t use = it / kStages;
                    if (use > 0 && !wait_or_abort(&empty[s], (use - 1) & 1, abort_flag)) {
                        *abort_flag = 1;
                        if (P.status) atomicCAS(P.status, 0, (4 << 16) | 1);
                        ok = false;
                        break;
                    }
                    unsigned char *st = smem + s * STAGE_BYTES;
                    static_assert(TF32 || !(AMN || BMN), "MN-major staging is laid out for 32-bit operands");
                    mbar_expect_tx(&full[s], A_BYTES + B_BYTES);
                    if constexpr (AMN) {
#pragma unroll
                        for (int m = 0; m < BM / 32; ++m)
                            tma_load_3d(st + m * 4096, &map_xh, &full[s], (int)(tm * BM) + 32 * m, kb * BKE, (int)b);
                    } else {
                        tma_load_3d(st, &map_xh, &full[s], kb * BKE, (int)(tm * BM), (int)b);
                    }
                    if constexpr (BMN) {
#pragma unroll
                        for (int m = 0; m < BN / 32; ++m)
                            tma_load_3d(st + 2 * A_BYTES + m * 4096, &map_yh, &full[s], (int)(tn * BN) + 32 * m, kb * BKE, (int)b);
                    } else {
                        tma_load_3d(st + 2 * A_BYTES, &map_yh, &full[s], kb * BKE, (int)(tn * BN), (int)b);
                    }
                    mbar_expect_tx(&full_lo[s], A_BYTES + B_BYTES);
                    if constexpr (AMN) {
#pragma unroll
                        for (int m = 0; m < BM / 32; ++m)
                            tma_load_3d(st + A_BYTES + m * 4096, &map_xl, &full_lo[s], (int)(tm * BM) + 32 * m, kb * BKE, (int)b);
                    } else {
                        tma_load_3d(st + A_BYTES, &map_xl, &full_lo[s], kb * BKE, (int)(tm * BM), (int)b);
                    }
                    if constexpr (BMN) {
#pragma unroll
                        for (int m = 0; m < BN / 32; ++m)
                            tma_load_3d(st + 2 * A_BYTES + B_BYTES + m * 4096, &map_yl, &full_lo[s], (int)(tn * BN) + 32 * m, kb * BKE, (int)b);
                    } else {
                        tma_load_3d(st + 2 * A_BYTES + B_BYTES, &map_yl, &full_lo[s], kb * BKE, (int)(tn * BN), (int)b);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc(BM, BN, TF32, AMN, BMN);
            uint32_t it = 0, acount = 0;
            bool ok = true;
            const int kchunk = (P.kchunk > 0 && P.kchunk < nkb) ? P.kchunk : nkb;
            for (long long tile = blockIdx.x; tile < P.tiles && ok; tile += gridDim.x) {
                // one accumulator per chunk of k-steps: the tensor cores add into tensor memory with
                // truncation, so long reductions are cut into chunks that the epilogue sums in registers
                for (int kb0 = 0; kb0 < nkb && ok; kb0 += kchunk, ++acount) {
                    const uint32_t a = acount & 1, ause = acount >> 1;
                    if (ause > 0 && !wait_or_abort(&tmem_empty[a], (ause - 1) & 1, abort_flag)) {
                        *abort_flag = 1;
                        if (P.status) atomicCAS(P.status, 0, (4 << 16) | 2);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + a * BN;
                    const int kb1 = kb0 + kchunk < nkb ? kb0 + kchunk : nkb;
                    for (int kb = kb0; kb < kb1; ++kb, ++it) {
                        const int s = it % kStages;
                        if (!wait_or_abort(&full[s], (it / kStages) & 1, abort_flag)) {
                            *abort_flag = 1;
                            if (P.status) atomicCAS(P.status, 0, (4 << 16) | 3);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
                        const uint32_t sb = smem_u32(smem + s * STAGE_BYTES);
                        const uint64_t dxh = AMN ? make_smem_desc_mn(sb) : make_smem_desc(sb);
                        const uint64_t dxl = AMN ? make_smem_desc_mn(sb + A_BYTES) : make_smem_desc(sb + A_BYTES);
                        const uint64_t dyh = BMN ? make_smem_desc_mn(sb + 2 * A_BYTES) : make_smem_desc(sb + 2 * A_BYTES);
                        const uint64_t dyl = BMN ? make_smem_desc_mn(sb + 2 * A_BYTES + B_BYTES) : make_smem_desc(sb + 2 * A_BYTES + B_BYTES);
                        // K-major: one MMA consumes 32 bytes of the swizzled row (16 bf16 or 8 tf32), so the start
                        // address advances by 2 units of 16 bytes; MN-major: 8 k-rows = 1024 bytes = 64 units
                        constexpr uint64_t ka = AMN ? 64 : 2, kbn = BMN ? 64 : 2;
#pragma unroll
                        for (int k = 0; k < kMmasPerStep; ++k)
                            tc_mma<TF32>(d_tmem, dxh + ka * k, dyh + kbn * k, idesc, ((kb - kb0) | k) != 0);
                        if (!wait_or_abort(&full_lo[s], (it / kStages) & 1, abort_flag)) {
                            *abort_flag = 1;
                            if (P.status) atomicCAS(P.status, 0, (4 << 16) | 5);
                            ok = false;
                            break;
                        }
                        tc_fence_after();
#pragma unroll
                        for (int k = 0; k < kMmasPerStep; ++k) {
                            tc_mma<TF32>(d_tmem, dxh + ka * k, dyl + kbn * k, idesc, 1);
                            tc_mma<TF32>(d_tmem, dxl + ka * k, dyh + kbn * k, idesc, 1);
                        }
                        tc_commit(&empty[s]); // the stage may be refilled once these MMAs have read it
                    }
                    if (ok) tc_commit(&tmem_full[a]);
                }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9, TMEM lanes 32*(warp % 4) .. +31, column half (warp-2)/4 ----------------
        const int q = warp & 3;
        const int chalf = (warp - 2) >> 2;
        uint32_t tcount = 0;
        bool ok = true;
        if constexpr (TF32) {
            // Chunked reduction (plain products only): every chunk's accumulator is added, rounded to
            // nearest, into 128 register-resident sums per thread; the tile is stored after its last chunk.
            static_assert(!TF32 || EPI == TPW_DOT_LINEAR, "the tf32 pipeline serves the plain products");
            const int kchunk = (P.kchunk > 0 && P.kchunk < nkb) ? P.kchunk : nkb;
            const int nchunks = (nkb + kchunk - 1) / kchunk;
            uint32_t acount = 0;
            for (long long tile = blockIdx.x; tile < P.tiles && ok; tile += gridDim.x) {
                long long t = tile;
                const long long tn = t % P.tiles_n; t /= P.tiles_n;
                const long long tm = t % P.tiles_m;
                const long long b = t / P.tiles_m;
                float sums[BN / 2];
#pragma unroll
                for (int v = 0; v < BN / 2; ++v) sums[v] = 0.f;
                for (int ch = 0; ch < nchunks && ok; ++ch, ++acount) {
                    const uint32_t a = acount & 1;
                    if (!wait_or_abort(&tmem_full[a], (acount >> 1) & 1, abort_flag)) {
                        *abort_flag = 1;
                        if (lane == 0 && P.status) atomicCAS(P.status, 0, (4 << 16) | 6);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < BN / 64; ++c) {
                        uint32_t r[32];
                        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + a * BN + (chalf * (BN / 64) + c) * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int v = 0; v < 32; ++v) sums[c * 32 + v] += __uint_as_float(r[v]);
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tmem_empty[a]);
                }
                if (!ok) break;
                const long long i = tm * BM + q * 32 + lane;
                const bool row_ok = i < P.N1;
                float *orow = P.out + (b * P.N1 + (row_ok ? i : 0)) * P.N2;
                unsigned char *stg = smem + OFF_STAGE + (warp - 2) * 4096;
                const long long row_base = tm * BM + q * 32;
#pragma unroll
                for (int c = 0; c < BN / 64; ++c) {
                    const long long j0 = tn * BN + (chalf * (BN / 64) + c) * 32;
                    if (j0 >= P.N2) continue;
                    if (P.vec_store && j0 + 32 <= P.N2) {
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            *reinterpret_cast<float4 *>(stg + lane * 128 + ((v ^ (lane & 7)) << 4)) =
                                make_float4(sums[c * 32 + 4 * v], sums[c * 32 + 4 * v + 1], sums[c * 32 + 4 * v + 2], sums[c * 32 + 4 * v + 3]);
                        __syncwarp();
#pragma unroll
                        for (int it = 0; it < 8; ++it) {
                            const int rr = it * 4 + (lane >> 3), cc = lane & 7;
                            const float4 o = *reinterpret_cast<const float4 *>(stg + rr * 128 + ((cc ^ (rr & 7)) << 4));
                            if (row_base + rr < P.N1)
                                reinterpret_cast<float4 *>(P.out + (b * P.N1 + row_base + rr) * P.N2 + j0)[cc] = o;
                        }
                        __syncwarp();
                    } else if (row_ok) {
#pragma unroll
                        for (int v = 0; v < 32; ++v)
                            if (j0 + v < P.N2) orow[j0 + v] = sums[c * 32 + v];
                    }
                }
            }
        } else
        for (long long tile = blockIdx.x; tile < P.tiles && ok; tile += gridDim.x, ++tcount) {
            long long tn, tm, b;
            decode_tile<TOPK != 0>(tile, P, tn, tm, b);
            const uint32_t a = tcount & 1;
            if (!wait_or_abort(&tmem_full[a], (tcount >> 1) & 1, abort_flag)) {
                *abort_flag = 1;
                if (lane == 0 && P.status) atomicCAS(P.status, 0, (4 << 16) | 4);
                ok = false;
                break;
            }
            tc_fence_after();
            const long long i = tm * BM + q * 32 + lane;
            const bool row_ok = i < P.N1;
            const float n1 = (EPI != TPW_DOT_LINEAR && row_ok) ? P.n1sq[b * P.N1 + i] : 0.f;
            float *orow = P.out + (b * P.N1 + (row_ok ? i : 0)) * P.N2;
            const float *n2p = P.n2sq + b * P.N2;
            unsigned long long best = ~0ull;
            // TOPK: a fresh list per tile half; candidates at or above an already published bound of the
            // row's k-th smallest key cannot be among its k smallest and are dropped before the insertion
            unsigned long long lst[TOPK > 0 ? TOPK : 1];
            unsigned long long bound = 0;
            if constexpr (TOPK > 0) {
#pragma unroll
                for (int t = 0; t < TOPK; ++t) lst[t] = ~0ull;
                if (row_ok) bound = *reinterpret_cast<volatile unsigned long long *>(P.topk_thr + b * P.N1 + i);
            }
            if constexpr (TOPK > 0) {
                // eight columns at a time, so that the unrolled body (and its insertion code) stays small;
                // the insertion is entered only when some lane of the warp has a candidate below its bounds
#pragma unroll 1
                for (int g = 0; g < BN / 16; ++g) {
                    const long long j0 = tn * BN + chalf * (BN / 2) + g * 8;
                    if (j0 >= P.N2) break;
                    uint32_t r8[8];
                    tmem_ld8(tmem_base + ((uint32_t)(q * 32) << 16) + a * BN + chalf * (BN / 2) + g * 8, r8);
                    tmem_ld_wait();
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const long long j = j0 + v;
                        const float nn = j < P.N2 ? __ldg(n2p + j) : 0.f;
                        const float o = dot_epilogue<EPI>(__uint_as_float(r8[v]), n1, nn, false);
                        const unsigned long long key = ((unsigned long long)__float_as_uint(o) << 32) | (unsigned long long)(uint32_t)j;
                        const bool cand = j < P.N2 && key < bound && key < lst[TOPK - 1];
                        if (__any_sync(0xffffffffu, cand)) {
                            if (cand) sorted_insert<TOPK>(lst, key);
                        }
                    }
                }
            } else
#pragma unroll 1
            for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); ++c) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + a * BN + c * 32;
                tmem_ld32(taddr, r);
                tmem_ld_wait();
                const long long j0 = tn * BN + c * 32;
                if (j0 >= P.N2) continue;
                if constexpr (ROWMIN) {
                    // streaming row minimum: this thread owns row i and folds its 32 columns into one key
                    // (the epilogue value is non-negative, so its bit pattern orders like an unsigned integer)
#pragma unroll
                    for (int v = 0; v < 32; ++v) {
                        const long long j = j0 + v;
                        const float nn = j < P.N2 ? __ldg(n2p + j) : 0.f;
                        const float o = dot_epilogue<EPI>(__uint_as_float(r[v]), n1, nn, false);
                        const unsigned long long key = ((unsigned long long)__float_as_uint(o) << 32) | (unsigned long long)(uint32_t)j;
                        if (j < P.N2 && key < best) best = key;
                    }
                    continue;
                }
                if (!row_ok && !(P.vec_store && j0 + 32 <= P.N2)) continue;
                if (P.vec_store && j0 + 32 <= P.N2) {
                    // epilogue math on this thread's row, staged with a 16-byte-chunk XOR swizzle ...
                    unsigned char *stg = smem + OFF_STAGE + (warp - 2) * 4096;
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const float4 nn = EPI == TPW_DOT_LINEAR ? make_float4(0.f, 0.f, 0.f, 0.f)
                                                                : __ldg(reinterpret_cast<const float4 *>(n2p + j0) + v);
                        float4 o;
                        o.x = dot_epilogue<EPI>(__uint_as_float(r[4 * v + 0]), n1, nn.x, SELF && i == j0 + 4 * v + 0);
                        o.y = dot_epilogue<EPI>(__uint_as_float(r[4 * v + 1]), n1, nn.y, SELF && i == j0 + 4 * v + 1);
                        o.z = dot_epilogue<EPI>(__uint_as_float(r[4 * v + 2]), n1, nn.z, SELF && i == j0 + 4 * v + 2);
                        o.w = dot_epilogue<EPI>(__uint_as_float(r[4 * v + 3]), n1, nn.w, SELF && i == j0 + 4 * v + 3);
                        *reinterpret_cast<float4 *>(stg + lane * 128 + ((v ^ (lane & 7)) << 4)) = o;
                    }
                    __syncwarp();
                    // ... and written out four full 128-byte row segments per instruction
                    const long long row_base = tm * BM + q * 32;
#pragma unroll
                    for (int it = 0; it < 8; ++it) {
                        const int rr = it * 4 + (lane >> 3), cc = lane & 7;
                        const float4 o = *reinterpret_cast<const float4 *>(stg + rr * 128 + ((cc ^ (rr & 7)) << 4));
                        if (row_base + rr < P.N1)
                            reinterpret_cast<float4 *>(P.out + (b * P.N1 + row_base + rr) * P.N2 + j0)[cc] = o;
                    }
                    __syncwarp();
                } else {
#pragma unroll
                    for (int v = 0; v < 32; ++v) {
                        const long long j = j0 + v;
                        if (j < P.N2)
                            orow[j] = dot_epilogue<EPI>(__uint_as_float(r[v]), n1, EPI == TPW_DOT_LINEAR ? 0.f : __ldg(n2p + j), SELF && i == j);
                    }
                }
            }
            if constexpr (ROWMIN) {
                if (row_ok && best != ~0ull) atomicMin(P.rowmin_keys + b * P.N1 + i, best);
            }
            if constexpr (TOPK > 0) {
                if (row_ok) {
                    unsigned long long *dst = P.topk_lists + ((b * P.N1 + i) * P.topk_L + tn * 2 + chalf) * P.topk_k;
                    unsigned long long kth = ~0ull;
#pragma unroll
                    for (int t = 0; t < TOPK; ++t) {
                        if (t < P.topk_k && lst[t] != ~0ull) dst[t] = lst[t];
                        if (t == P.topk_k - 1) kth = lst[t];
                    }
                    if (kth != ~0ull) atomicMin(P.topk_thr + b * P.N1 + i, kth); // k entries in this list: a valid bound
                }
            }
            // this warp has drained its quarter of accumulator `a`
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[a]);
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// fp32 rows -> bf16 high/low parts (row pitch Dp, zero padded) and a per-row fp32 scalar: the
// squared norm, or (recip != 0) the reciprocal norm with 0 for an all-zero row; one warp per row
__global__ void split_rows_kernel(const float *__restrict__ x, __nv_bfloat16 *__restrict__ hi, __nv_bfloat16 *__restrict__ lo,
                                  float *__restrict__ nsq, long long rows, long long D, long long Dp, int recip) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *row = x + r * D;
        float s = 0.f;
        for (long long k = lane; k < Dp; k += 32) {
            const float v = k < D ? row[k] : 0.f;
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            const __nv_bfloat16 l = __float2bfloat16_rn(v - __bfloat162float(h));
            hi[r * Dp + k] = h;
            lo[r * Dp + k] = l;
            s = fmaf(v, v, s);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) {
            if (recip) {
                const float nrm = sqrtf(s);
                nsq[r] = nrm != 0.f ? __fdiv_rn(1.f, nrm) : 0.f;
            } else {
                nsq[r] = s;
            }
        }
    }
}

inline long long align_up(long long v, long long a) { return (v + a - 1) / a * a; }

// TPW_ENGINE_AUTO: the tensor-core engine pays for its split pre-pass and 128 x 256 tiles only on
// large fp32 problems; everything else stays on the exact fp32/fp64 CUDA-core tile.
inline bool auto_picks_tensor_cores(int dtype, long long B, long long N1, long long N2, long long D) {
    return dtype == TPW_F32 && D >= 64 && N1 >= 128 && N2 >= 256 && (double)B * N1 * N2 * D >= (double)(1ll << 28);
}

struct ScratchLayout {
    long long Dp, off_xh, off_xl, off_yh, off_yl, off_n1, off_n2, total;
};

inline ScratchLayout scratch_layout(long long B, long long N1, long long N2, long long D, bool self) {
    ScratchLayout L;
    L.Dp = align_up(D, 8); // 16-byte row pitch for the tensor maps
    const long long xa = align_up(B * N1 * L.Dp * 2, 1024), ya = self ? 0 : align_up(B * N2 * L.Dp * 2, 1024);
    L.off_xh = 0;
    L.off_xl = xa;
    L.off_yh = self ? L.off_xh : 2 * xa;
    L.off_yl = self ? L.off_xl : 2 * xa + ya;
    L.off_n1 = 2 * xa + 2 * ya;
    L.off_n2 = self ? L.off_n1 : L.off_n1 + align_up(B * N1 * 4, 1024);
    L.total = L.off_n2 + align_up(B * N2 * 4, 1024);
    return L;
}


// ---- gradient products on the tensor cores (tf32 x 3) ---------------------------------------------
//
// grad_x1 = s_mm * (C . X2) + s_row * x1 * rowsum(C),  grad_x2 = s_mm * (C^T . X1) + s_row * x2 * colsum(C)
// with C = g (squared Euclidean, plain products) or g / o (Euclidean).  Each operand is split into
// two tf32 numbers, hi = rn_tf32(v) and lo = rn_tf32(v - hi), and hi.hi + hi.lo + lo.hi is
// accumulated in fp32: 22 bits of every factor take part, so the products carry about 2^-21 of
// relative error, two orders below the float32 parity tolerance even for sums that cancel.

__device__ __forceinline__ float rn_tf32(float v) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(v));
    return __uint_as_float(u);
}

enum { COEF_ID = 0, COEF_DIV_AUX = 1, COEF_COSINE = 2 };
constexpr int PT = 64;        // pre-pass tile edge

struct SplitParams {
    const float *a, *aux;       // [B,R,C]
    const float *n1, *n2;       // COEF_COSINE: row norms [B,R], [B,C]
    float *hi, *lo;             // [B,R,Cp]   (STRAIGHT)
    float *rowpart, *colpart;   // [B,TC,R], [B,TR,C]   (SUMS)
    long long R, C, Cp, TR, TC;
    int vec_in;                 // C % 4 == 0 and 16-byte aligned inputs
    int epilogue;               // COEF_COSINE: what aux holds (tpw_dot_epilogue)
};

// Coefficient of one element and the summands of its row and column sums.
//   COEF_ID:      c = a
//   COEF_DIV_AUX: c = a / aux, 0 where aux == 0                     (Euclidean: g / o)
//   COEF_COSINE:  S = M / (n1 n2) with the "identity" safe divide, aux = S or 1 - S, a = upstream
//                 gradient: c = dM = gs / (n1 n2) (gs where that is 0), and with dd = -c S (0 where
//                 the denominator is 0) the row summand is dd n2[j], the column summand dd n1[i]
//                 (the gradients of the two norm vectors)
template <int MODE>
__device__ __forceinline__ void coefficient(float a, float aux, float na, float nb, int epilogue, float &c, float &rs, float &cs) {
    if (MODE == COEF_ID) {
        c = rs = cs = a;
    } else if (MODE == COEF_DIV_AUX) {
        c = aux != 0.f ? __fdiv_rn(a, aux) : 0.f;
        rs = cs = c;
    } else {
        const float S = epilogue == TPW_DOT_COSINE_SIM ? aux : 1.f - aux;
        const float gs = epilogue == TPW_DOT_COSINE_SIM ? a : -a;
        const float denom = na * nb;
        float dd = 0.f;
        if (denom != 0.f) {
            c = __fdiv_rn(gs, denom);
            dd = -c * S;
        } else {
            c = gs;
        }
        rs = dd * nb;
        cs = dd * na;
    }
}

// One 64 x 64 tile per CTA of 256 threads: coefficient, tf32 high/low copies (row pitch padded to a
// multiple of 4 and zero filled), per-tile row and column sums.
template <int MODE, bool SUMS>
__global__ void __launch_bounds__(256)
split_tile_kernel(const SplitParams P) {
    __shared__ float colacc[SUMS ? 16 * PT : 1];
    const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
    const long long b = blockIdx.z;
    const long long r0 = (long long)blockIdx.y * PT, c0 = (long long)blockIdx.x * PT;
    const float *a = P.a + b * P.R * P.C;
    const float *aux = MODE != COEF_ID ? P.aux + b * P.R * P.C : nullptr;
    const long long col = c0 + 4 * tx;
    float nb[4] = {0.f, 0.f, 0.f, 0.f};
    if (MODE == COEF_COSINE) {
#pragma unroll
        for (int e = 0; e < 4; ++e)
            if (col + e < P.C) nb[e] = P.n2[b * P.C + col + e];
    }
    float colp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r = 0; r < 4; ++r) {
        const long long row = r0 + ty + 16 * r;
        float v[4] = {0.f, 0.f, 0.f, 0.f}, rs[4] = {0.f, 0.f, 0.f, 0.f};
        if (row < P.R) {
            float av[4] = {0.f, 0.f, 0.f, 0.f}, ov[4] = {0.f, 0.f, 0.f, 0.f};
            const bool vec = P.vec_in && col + 3 < P.C;
            if (vec) {
                const float4 t = *reinterpret_cast<const float4 *>(a + row * P.C + col);
                av[0] = t.x; av[1] = t.y; av[2] = t.z; av[3] = t.w;
                if (MODE != COEF_ID) {
                    const float4 o = *reinterpret_cast<const float4 *>(aux + row * P.C + col);
                    ov[0] = o.x; ov[1] = o.y; ov[2] = o.z; ov[3] = o.w;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (col + e < P.C) {
                        av[e] = a[row * P.C + col + e];
                        if (MODE != COEF_ID) ov[e] = aux[row * P.C + col + e];
                    }
            }
            const float na = MODE == COEF_COSINE ? P.n1[b * P.R + row] : 0.f;
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (col + e < P.C) {
                    float cs;
                    coefficient<MODE>(av[e], ov[e], na, nb[e], P.epilogue, v[e], rs[e], cs);
                    colp[e] += cs;
                }
        }
        if (row < P.R && col < P.Cp) {
            float4 h, l;
            h.x = rn_tf32(v[0]); l.x = rn_tf32(v[0] - h.x);
            h.y = rn_tf32(v[1]); l.y = rn_tf32(v[1] - h.y);
            h.z = rn_tf32(v[2]); l.z = rn_tf32(v[2] - h.z);
            h.w = rn_tf32(v[3]); l.w = rn_tf32(v[3] - h.w);
            *reinterpret_cast<float4 *>(P.hi + (b * P.R + row) * P.Cp + col) = h;
            *reinterpret_cast<float4 *>(P.lo + (b * P.R + row) * P.Cp + col) = l;
        }
        if (SUMS) {
            float s = (rs[0] + rs[1]) + (rs[2] + rs[3]);
#pragma unroll
            for (int off = 1; off < 16; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if (tx == 0 && row < P.R) P.rowpart[(b * P.TC + blockIdx.x) * P.R + row] = s;
        }
    }
    if (!SUMS) return;
#pragma unroll
    for (int e = 0; e < 4; ++e) colacc[ty * PT + 4 * tx + e] = colp[e];
    __syncthreads();
    if (tid < PT && c0 + tid < P.C) {
        float s = 0.f;
#pragma unroll
        for (int y = 0; y < 16; ++y) s += colacc[y * PT + tid];
        P.colpart[(b * P.TR + blockIdx.y) * P.C + c0 + tid] = s;
    }
}

// sums[b,n] = part[b,0,n] + part[b,1,n] + ... in that order (deterministic)
__global__ void reduce_partials_kernel(const float *__restrict__ part, float *__restrict__ sums, long long B, long long T, long long N) {
    const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t >= B * N) return;
    const long long b = t / N, n = t % N;
    float s = 0.f;
    for (long long k = 0; k < T; ++k) s += part[(b * T + k) * N + n];
    sums[t] = s;
}

// g[r,k] = s_mm * g[r,k] + s_row * x[r,k] * sums[r]
__global__ void grad_finish_kernel(float *__restrict__ g, const float *__restrict__ x, const float *__restrict__ sums,
                                   long long rows, long long D, float s_mm, float s_row) {
    const long long n = rows * D;
    for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n; t += (long long)gridDim.x * blockDim.x) {
        const float base = s_mm * g[t];
        g[t] = sums ? fmaf(s_row * x[t], sums[t / D], base) : base;
    }
}

struct BwdScratch {
    long long N2p, Dp, TR, TC;
    long long off_chi, off_clo, off_x1hi, off_x1lo, off_x2hi, off_x2lo;
    long long off_rowpart, off_colpart, off_rowsum, off_colsum, total;
};

inline BwdScratch bwd_scratch_layout(long long B, long long N1, long long N2, long long D) {
    BwdScratch L;
    L.N2p = align_up(N2, 4);
    L.Dp = align_up(D, 4);
    L.TR = (N1 + PT - 1) / PT;
    L.TC = (N2 + PT - 1) / PT;
    long long off = 0;
    auto take = [&](long long bytes) { const long long o = off; off += align_up(bytes, 1024); return o; };
    L.off_chi = take(B * N1 * L.N2p * 4);
    L.off_clo = take(B * N1 * L.N2p * 4);
    L.off_x1hi = take(B * N1 * L.Dp * 4);
    L.off_x1lo = take(B * N1 * L.Dp * 4);
    L.off_x2hi = take(B * N2 * L.Dp * 4);
    L.off_x2lo = take(B * N2 * L.Dp * 4);
    L.off_rowpart = take(B * L.TC * N1 * 4);
    L.off_colpart = take(B * L.TR * N2 * 4);
    L.off_rowsum = take(B * N1 * 4);
    L.off_colsum = take(B * N2 * 4);
    L.total = off;
    return L;
}

// The tensor-core gradient products pay for their split pre-pass only on large fp32 problems.
inline bool auto_picks_tensor_backward(int dtype, long long B, long long N1, long long N2, long long D) {
    return dtype == TPW_F32 && D >= 64 && N1 >= 256 && N2 >= 256 && (double)B * N1 * N2 * D >= (double)(1ll << 28);
}

template <int MODE, bool SUMS>
int launch_split(const SplitParams &P, long long B, cudaStream_t s) {
    const long long gx = (P.C + PT - 1) / PT, gy = (P.R + PT - 1) / PT;
    TPW_CHECK_ARG(gy <= 65535 && B <= 65535, "dense backward: more than 65535 row tiles or batches");
    split_tile_kernel<MODE, SUMS><<<dim3((unsigned)gx, (unsigned)gy, (unsigned)B), 256, 0, s>>>(P);
    TPW_LAUNCH_OK("split_tile_kernel");
    return TPW_OK;
}

// One operand of a tf32 product as high/low parts.  K-major (mn = false): rows are the M (or N) index,
// `pitch` elements per row hold k (zero padded).  MN-major (mn = true): rows are k, `pitch` elements
// per row hold the M (or N) index.
struct Tf32Operand {
    const float *hi, *lo;
    long long pitch;
    bool mn;
};

// out[b,m,n] = sum_k A[b](m,k) * Bm[b](n,k); K = length of the reduction.  A K-major operand holds
// `pitch` >= K elements per row (zero beyond K), an MN-major operand has exactly K rows per batch.
int launch_tf32_product(const Tf32Operand &A, const Tf32Operand &Bm, float *out,
                        long long B, long long M, long long N, long long K, cudaStream_t s) {
    CUtensorMap mah, mal, mbh, mbl;
    int st;
    auto encode = [&](CUtensorMap *m, const float *p, const Tf32Operand &o, long long rows, int box_rows) {
        return o.mn ? make_tensor_map_3d_atom32(m, p, 4, o.pitch, K, B, 32, 32)
                    : make_tensor_map_3d(m, p, 4, o.pitch, rows, B, BK / 2, box_rows, true);
    };
    if ((st = encode(&mah, A.hi, A, M, BM)) != TPW_OK) return st;
    if ((st = encode(&mal, A.lo, A, M, BM)) != TPW_OK) return st;
    if ((st = encode(&mbh, Bm.hi, Bm, N, BN)) != TPW_OK) return st;
    if ((st = encode(&mbl, Bm.lo, Bm, N, BN)) != TPW_OK) return st;
    GemmParams P;
    memset(&P, 0, sizeof(P));
    P.out = out;
    P.B = B; P.N1 = M; P.N2 = N; P.D = K; // K-major tails beyond K are zero padding or zero fill
    P.tiles_m = (M + BM - 1) / BM;
    P.tiles_n = (N + BN - 1) / BN;
    P.tiles = B * P.tiles_m * P.tiles_n;
    P.epilogue = TPW_DOT_LINEAR;
    // 64 elements per chunk: measured against float64, the products are then as accurate as the fp32
    // FMA chain of the CUDA-core kernel (the error grows in proportion to the chunk length) at no cost in time
    P.kchunk = 2;
    P.vec_store = (N % 4 == 0 && aligned16(out)) ? 1 : 0;
    P.status = device_status_ptr();
    const long long nsm = sm_count();
    const unsigned grid = (unsigned)(P.tiles < nsm ? P.tiles : nsm);
#define TPW_TF32_LAUNCH(AMN, BMN)                                                                                         \
    do {                                                                                                                  \
        auto kern = gemm_metric_kernel<TPW_DOT_LINEAR, false, true, false, AMN, BMN>;                                     \
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));                 \
        kern<<<grid, kThreads, SMEM_ALLOC, s>>>(mah, mal, mbh, mbl, P);                                                   \
    } while (0)
    if (!A.mn && !Bm.mn) TPW_TF32_LAUNCH(false, false);
    else if (!A.mn && Bm.mn) TPW_TF32_LAUNCH(false, true);
    else if (A.mn && Bm.mn) TPW_TF32_LAUNCH(true, true);
    else return fail(TPW_ERR_UNSUPPORTED, "tf32 product: MN-major A with K-major B is not instantiated");
#undef TPW_TF32_LAUNCH
    TPW_LAUNCH_OK("gemm_metric_kernel (tf32)");
    return TPW_OK;
}

} // namespace
} // namespace tpw

using namespace tpw;

extern "C" int tpw_dot_metric_forward_simt(int dtype, int epilogue, const void *x1, const void *x2, void *out,
                                           int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

// tf32 x 3 forward (plain dot products only): straight hi/lo copies of both operands
static long long tf32_forward_scratch(long long B, long long N1, long long N2, long long D) {
    const long long Dp = align_up(D, 4);
    return 2 * align_up(B * N1 * Dp * 4, 1024) + 2 * align_up(B * N2 * Dp * 4, 1024);
}

namespace tpw {
namespace {
// keys -> (smallest value, optionally its square root; its x2 row)
__global__ void dot_rowmin_finish_kernel(const unsigned long long *__restrict__ keys, float *__restrict__ min_out,
                                         long long *__restrict__ arg_out, long long n, int take_sqrt) {
    const long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    if (t >= n) return;
    const unsigned long long key = keys[t];
    const bool none = key == ~0ull;
    float v = none ? __int_as_float(0x7f800000) : __uint_as_float((uint32_t)(key >> 32));
    if (take_sqrt) v = sqrtf(v);
    if (min_out) min_out[t] = v;
    if (arg_out) arg_out[t] = none ? -1ll : (long long)(uint32_t)key;
}
} // namespace
} // namespace tpw

namespace tpw {
namespace {
// One warp per row: the k smallest of the row's n candidate keys (lists written by the top-k epilogue;
// unused slots hold ~0), ascending.  Every lane keeps the TOPK smallest of its share, then the warp
// extracts the global minimum k times (keys are unique: the x2 row is part of the key).
// bound_out (optional): the k-th smallest key itself, left untouched when fewer than k candidates exist.
template <int TOPK>
__global__ void topk_merge_kernel(const unsigned long long *__restrict__ lists, float *__restrict__ val_out,
                                  long long *__restrict__ idx_out, unsigned long long *__restrict__ bound_out,
                                  long long rows, long long row_stride, long long n, int k, int take_sqrt) {
    const int lane = threadIdx.x & 31;
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    unsigned long long mine[TOPK];
#pragma unroll
    for (int t = 0; t < TOPK; ++t) mine[t] = ~0ull;
    const unsigned long long *src = lists + row * row_stride;
    for (long long e = lane; e < n; e += 32) {
        const unsigned long long key = src[e];
        if (key < mine[TOPK - 1]) sorted_insert<TOPK>(mine, key);
    }
    for (int r = 0; r < k; ++r) {
        unsigned long long m = mine[0];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const unsigned long long other = __shfl_xor_sync(0xffffffffu, m, off);
            m = other < m ? other : m;
        }
        if (m != ~0ull && mine[0] == m) { // the owner pops its head
#pragma unroll
            for (int t = 0; t < TOPK - 1; ++t) mine[t] = mine[t + 1];
            mine[TOPK - 1] = ~0ull;
        }
        if (lane == 0) {
            const bool none = m == ~0ull;
            float v = none ? __int_as_float(0x7f800000) : __uint_as_float((uint32_t)(m >> 32));
            if (take_sqrt) v = sqrtf(v);
            if (val_out) val_out[row * k + r] = v;
            if (idx_out) idx_out[row * k + r] = none ? -1ll : (long long)(uint32_t)m;
            if (bound_out && r == k - 1 && !none) bound_out[row] = m;
        }
    }
}

constexpr int kTopkMax = 16;

struct TopkScratch {
    long long L, off_lists, off_thr, total;
};
inline TopkScratch topk_scratch_layout(long long B, long long N1, long long N2, long long D, long long k) {
    TopkScratch T;
    T.L = 2 * ((N2 + BN - 1) / BN);
    const long long gemm = scratch_layout(B, N1, N2, D, false).total;
    T.off_lists = gemm;
    T.off_thr = gemm + align_up(B * N1 * T.L * k * 8, 1024);
    T.total = T.off_thr + align_up(B * N1 * 8, 1024);
    return T;
}
} // namespace
} // namespace tpw

namespace tpw {
namespace {
// Common front end of the bf16 x 3 launches: splits x1 and x2 into the scratch (bf16 high/low parts, row
// norms: squared, or reciprocal for the cosine family), encodes the four tensor maps and fills the
// problem sizes of `P`.  The caller sets the epilogue-specific fields and launches.
struct Bf16Operands {
    CUtensorMap mxh, mxl, myh, myl;
};
int prepare_bf16_operands(const void *x1, const void *x2, void *scratch, bool reciprocal_norms,
                          long long B, long long N1, long long N2, long long D, cudaStream_t s,
                          Bf16Operands &M, GemmParams &P) {
    const ScratchLayout L = scratch_layout(B, N1, N2, D, false);
    unsigned char *base = static_cast<unsigned char *>(scratch);
    __nv_bfloat16 *xh = reinterpret_cast<__nv_bfloat16 *>(base + L.off_xh), *xl = reinterpret_cast<__nv_bfloat16 *>(base + L.off_xl);
    __nv_bfloat16 *yh = reinterpret_cast<__nv_bfloat16 *>(base + L.off_yh), *yl = reinterpret_cast<__nv_bfloat16 *>(base + L.off_yl);
    float *n1 = reinterpret_cast<float *>(base + L.off_n1), *n2 = reinterpret_cast<float *>(base + L.off_n2);
    const int threads = 256;
    const long long cap = (long long)sm_count() * 16;
    long long blocks = (B * N1 * 32 + threads - 1) / threads;
    split_rows_kernel<<<(unsigned)(blocks < cap ? blocks : cap), threads, 0, s>>>((const float *)x1, xh, xl, n1, B * N1, D, L.Dp, reciprocal_norms ? 1 : 0);
    blocks = (B * N2 * 32 + threads - 1) / threads;
    split_rows_kernel<<<(unsigned)(blocks < cap ? blocks : cap), threads, 0, s>>>((const float *)x2, yh, yl, n2, B * N2, D, L.Dp, reciprocal_norms ? 1 : 0);
    TPW_LAUNCH_OK("split_rows_kernel");
    int st;
    if ((st = make_tensor_map_3d(&M.mxh, xh, 2, L.Dp, N1, B, BK, BM, true)) != TPW_OK) return st;
    if ((st = make_tensor_map_3d(&M.mxl, xl, 2, L.Dp, N1, B, BK, BM, true)) != TPW_OK) return st;
    if ((st = make_tensor_map_3d(&M.myh, yh, 2, L.Dp, N2, B, BK, BN, true)) != TPW_OK) return st;
    if ((st = make_tensor_map_3d(&M.myl, yl, 2, L.Dp, N2, B, BK, BN, true)) != TPW_OK) return st;
    memset(&P, 0, sizeof(P));
    P.n1sq = n1; P.n2sq = n2;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = L.Dp;
    P.tiles_m = (N1 + BM - 1) / BM;
    P.tiles_n = (N2 + BN - 1) / BN;
    P.tiles = B * P.tiles_m * P.tiles_n;
    P.status = device_status_ptr();
    return TPW_OK;
}
} // namespace
} // namespace tpw

extern "C" int tpw_dot_topk_max_k(void) { return kTopkMax; }

extern "C" int64_t tpw_dot_topk_scratch_bytes(int64_t k, int64_t B, int64_t N1, int64_t N2, int64_t D) {
    if (k <= 0 || k > kTopkMax || B <= 0 || N1 <= 0 || N2 <= 0 || D <= 0) return 0;
    return topk_scratch_layout(B, N1, N2, D, k).total;
}

extern "C" int tpw_dot_topk_forward_ws(int epilogue, int k, const void *x1, const void *x2, float *val_out, int64_t *idx_out,
                                       void *scratch, int64_t scratch_bytes,
                                       int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(epilogue == TPW_DOT_SQEUCLIDEAN || epilogue == TPW_DOT_EUCLIDEAN || epilogue == TPW_DOT_COSINE_DIST,
                  "tpw_dot_topk_forward_ws: epilogue must be TPW_DOT_SQEUCLIDEAN, TPW_DOT_EUCLIDEAN or TPW_DOT_COSINE_DIST");
    TPW_CHECK_ARG(k >= 1 && k <= kTopkMax, "tpw_dot_topk_forward_ws: k must be in [1, %d] (got %d)", kTopkMax, k);
    TPW_CHECK_ARG(B > 0 && N1 > 0 && N2 > 0 && D > 0, "tpw_dot_topk_forward_ws: sizes must be positive");
    TPW_CHECK_ARG(x1 && x2 && (val_out || idx_out), "tpw_dot_topk_forward_ws: NULL pointer");
    TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && B < (1ll << 31) && D < (1ll << 31),
                  "tpw_dot_topk_forward_ws: a dimension exceeds 2^31-1");
    const bool cosine = epilogue == TPW_DOT_COSINE_DIST;
    const TopkScratch T = topk_scratch_layout(B, N1, N2, D, k);
    TPW_CHECK_ARG(scratch != nullptr && scratch_bytes >= T.total && aligned16(scratch),
                  "tpw_dot_topk_forward_ws: needs %lld bytes of 16-byte aligned scratch (got %lld)", T.total, (long long)scratch_bytes);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned char *base = static_cast<unsigned char *>(scratch);
    unsigned long long *lists = reinterpret_cast<unsigned long long *>(base + T.off_lists);
    unsigned long long *thr = reinterpret_cast<unsigned long long *>(base + T.off_thr);
    TPW_CUDA_OK(cudaMemsetAsync(lists, 0xFF, (size_t)(T.total - T.off_lists), s)); // lists and bounds: "nothing yet"
    Bf16Operands M;
    GemmParams P;
    int st;
    if ((st = prepare_bf16_operands(x1, x2, scratch, cosine, B, N1, N2, D, s, M, P)) != TPW_OK) return st;
    P.epilogue = cosine ? TPW_DOT_COSINE_DIST : TPW_DOT_SQEUCLIDEAN;
    P.topk_lists = lists; P.topk_thr = thr; P.topk_k = k; P.topk_L = (int)T.L;
    const long long nsm = sm_count();
    const long long tiles_n_all = (N2 + BN - 1) / BN;
    const long long rows = B * N1;
    const unsigned mblocks = (unsigned)((rows * 32 + 255) / 256);
    long long *idx64 = reinterpret_cast<long long *>(idx_out);
    const int take_sqrt = epilogue == TPW_DOT_EUCLIDEAN ? 1 : 0;
#define TPW_TOPK_LAUNCH(EPI, CAP)                                                                                         \
    do {                                                                                                                  \
        auto kern = gemm_metric_kernel<EPI, false, false, false, false, false, CAP>;                                      \
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));                 \
        kern<<<grid, kThreads, SMEM_ALLOC, s>>>(M.mxh, M.mxl, M.myh, M.myl, P);                                           \
    } while (0)
    // Column ranges [0, 1/16), [1/16, 1/4), [1/4, 1) of the column tiles: after each range the lists so far
    // are merged into an exact bound of every row's k-th smallest key, which prunes the next range down to
    // the few candidates that can still matter (an insertion costs the whole warp as soon as one lane has one).
    const long long cut[4] = {0, tiles_n_all >= 16 ? tiles_n_all / 16 : 0, tiles_n_all >= 16 ? tiles_n_all / 4 : 0, tiles_n_all};
    for (int ph = 0; ph < 3; ++ph) {
        if (cut[ph + 1] <= cut[ph]) continue;
        P.tn0 = cut[ph];
        P.tiles_n = cut[ph + 1] - cut[ph];
        P.tiles = B * P.tiles_m * P.tiles_n;
        const unsigned grid = (unsigned)(P.tiles < nsm ? P.tiles : nsm);
        if (cosine) { if (k <= 8) TPW_TOPK_LAUNCH(TPW_DOT_COSINE_DIST, 8); else TPW_TOPK_LAUNCH(TPW_DOT_COSINE_DIST, 16); }
        else { if (k <= 8) TPW_TOPK_LAUNCH(TPW_DOT_SQEUCLIDEAN, 8); else TPW_TOPK_LAUNCH(TPW_DOT_SQEUCLIDEAN, 16); }
        TPW_LAUNCH_OK("gemm_metric_kernel (top-k)");
        const bool last = cut[ph + 1] == tiles_n_all;
        const long long n = 2 * cut[ph + 1] * k; // the lists of all column tiles processed so far
        if (k <= 8) topk_merge_kernel<8><<<mblocks, 256, 0, s>>>(lists, last ? val_out : nullptr, last ? idx64 : nullptr, last ? nullptr : thr,
                                                                  rows, T.L * k, n, k, take_sqrt);
        else topk_merge_kernel<16><<<mblocks, 256, 0, s>>>(lists, last ? val_out : nullptr, last ? idx64 : nullptr, last ? nullptr : thr,
                                                                   rows, T.L * k, n, k, take_sqrt);
    }
#undef TPW_TOPK_LAUNCH
    TPW_LAUNCH_OK("topk_merge_kernel");
    return TPW_OK;
}

extern "C" int64_t tpw_dot_rowmin_scratch_bytes(int64_t B, int64_t N1, int64_t N2, int64_t D) {
    if (B <= 0 || N1 <= 0 || N2 <= 0 || D <= 0) return 0;
    return scratch_layout(B, N1, N2, D, false).total + align_up(B * N1 * 8, 1024);
}

extern "C" int tpw_dot_rowmin_forward_ws(int epilogue, const void *x1, const void *x2, float *min_out, int64_t *arg_out,
                                         void *scratch, int64_t scratch_bytes,
                                         int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(epilogue == TPW_DOT_SQEUCLIDEAN || epilogue == TPW_DOT_EUCLIDEAN || epilogue == TPW_DOT_COSINE_DIST,
                  "tpw_dot_rowmin_forward_ws: epilogue must be TPW_DOT_SQEUCLIDEAN, TPW_DOT_EUCLIDEAN or TPW_DOT_COSINE_DIST");
    const bool cosine = epilogue == TPW_DOT_COSINE_DIST;
    TPW_CHECK_ARG(B > 0 && N1 > 0 && N2 > 0 && D > 0, "tpw_dot_rowmin_forward_ws: sizes must be positive");
    TPW_CHECK_ARG(x1 && x2 && (min_out || arg_out), "tpw_dot_rowmin_forward_ws: NULL pointer");
    TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && B < (1ll << 31) && D < (1ll << 31),
                  "tpw_dot_rowmin_forward_ws: a dimension exceeds 2^31-1");
    const ScratchLayout L = scratch_layout(B, N1, N2, D, false);
    const long long need = L.total + align_up(B * N1 * 8, 1024);
    TPW_CHECK_ARG(scratch != nullptr && scratch_bytes >= need && aligned16(scratch),
                  "tpw_dot_rowmin_forward_ws: needs %lld bytes of 16-byte aligned scratch (got %lld)", need, (long long)scratch_bytes);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned long long *keys = reinterpret_cast<unsigned long long *>(static_cast<unsigned char *>(scratch) + L.total);
    TPW_CUDA_OK(cudaMemsetAsync(keys, 0xFF, (size_t)(B * N1) * 8, s));
    Bf16Operands M;
    GemmParams P;
    int st;
    if ((st = prepare_bf16_operands(x1, x2, scratch, cosine, B, N1, N2, D, s, M, P)) != TPW_OK) return st;
    P.epilogue = cosine ? TPW_DOT_COSINE_DIST : TPW_DOT_SQEUCLIDEAN;
    P.rowmin_keys = keys;
    const long long nsm = sm_count();
    const unsigned grid = (unsigned)(P.tiles < nsm ? P.tiles : nsm);
    if (cosine) {
        auto kern = gemm_metric_kernel<TPW_DOT_COSINE_DIST, false, false, true>;
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
        kern<<<grid, kThreads, SMEM_ALLOC, s>>>(M.mxh, M.mxl, M.myh, M.myl, P);
    } else {
        auto kern = gemm_metric_kernel<TPW_DOT_SQEUCLIDEAN, false, false, true>;
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));
        kern<<<grid, kThreads, SMEM_ALLOC, s>>>(M.mxh, M.mxl, M.myh, M.myl, P);
    }
    TPW_LAUNCH_OK("gemm_metric_kernel (row minimum)");
    dot_rowmin_finish_kernel<<<(unsigned)((B * N1 + 255) / 256), 256, 0, s>>>(keys, min_out, reinterpret_cast<long long *>(arg_out), B * N1,
                                                                             epilogue == TPW_DOT_EUCLIDEAN ? 1 : 0);
    TPW_LAUNCH_OK("dot_rowmin_finish_kernel");
    return TPW_OK;
}

extern "C" int64_t tpw_dot_metric_scratch_bytes(int dtype, int engine, int64_t B, int64_t N1, int64_t N2, int64_t D) {
    if (B <= 0 || N1 <= 0 || N2 <= 0 || D <= 0 || dtype != TPW_F32) return 0;
    if (engine == TPW_ENGINE_TCGEN05_TF32X3) return tf32_forward_scratch(B, N1, N2, D);
    if (engine == TPW_ENGINE_TCGEN05_BF16X3 || (engine == TPW_ENGINE_AUTO && auto_picks_tensor_cores(dtype, B, N1, N2, D)))
        return scratch_layout(B, N1, N2, D, false).total;
    return 0;
}

extern "C" int tpw_dot_metric_forward_ws(int dtype, int epilogue, int engine,
                                         const void *x1, const void *x2, void *out, void *scratch, int64_t scratch_bytes,
                                         int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(engine >= TPW_ENGINE_AUTO && engine <= TPW_ENGINE_TCGEN05_TF32X3, "tpw_dot_metric_forward_ws: bad engine %d", engine);
    if (engine == TPW_ENGINE_TCGEN05_TF32X3) {
        // x1 . x2^T with fp32-chain accuracy: tf32 high/low parts, chunked accumulation (see the gradient products)
        TPW_CHECK_ARG(dtype == TPW_F32 && epilogue == TPW_DOT_LINEAR,
                      "tpw_dot_metric_forward_ws: the tf32 engine computes float32 plain dot products (TPW_DOT_LINEAR) only");
        TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_dot_metric_forward_ws: negative size");
        if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
        TPW_CHECK_ARG(x1 && x2 && out && D > 0, "tpw_dot_metric_forward_ws: NULL pointer or empty feature dimension");
        TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && D < (1ll << 31), "tpw_dot_metric_forward_ws: a dimension exceeds 2^31-1");
        const long long need = tf32_forward_scratch(B, N1, N2, D);
        TPW_CHECK_ARG(scratch != nullptr && scratch_bytes >= need && aligned16(scratch),
                      "tpw_dot_metric_forward_ws: the tf32 engine needs %lld bytes of 16-byte aligned scratch (got %lld)", need, (long long)scratch_bytes);
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const long long Dp = align_up(D, 4), xa = align_up(B * N1 * Dp * 4, 1024), ya = align_up(B * N2 * Dp * 4, 1024);
        unsigned char *base = static_cast<unsigned char *>(scratch);
        float *xhi = reinterpret_cast<float *>(base), *xlo = reinterpret_cast<float *>(base + xa);
        float *yhi = reinterpret_cast<float *>(base + 2 * xa), *ylo = reinterpret_cast<float *>(base + 2 * xa + ya);
        int st;
        for (int side = 0; side < 2; ++side) {
            SplitParams X;
            memset(&X, 0, sizeof(X));
            X.a = static_cast<const float *>(side == 0 ? x1 : x2);
            X.hi = side == 0 ? xhi : yhi;
            X.lo = side == 0 ? xlo : ylo;
            X.R = side == 0 ? N1 : N2; X.C = D; X.Cp = Dp;
            X.vec_in = (D % 4 == 0 && aligned16(X.a)) ? 1 : 0;
            if ((st = launch_split<COEF_ID, false>(X, B, s)) != TPW_OK) return st;
        }
        return launch_tf32_product(Tf32Operand{xhi, xlo, Dp, false}, Tf32Operand{yhi, ylo, Dp, false}, static_cast<float *>(out), B, N1, N2, Dp, s);
    }
    if (engine == TPW_ENGINE_AUTO && auto_picks_tensor_cores(dtype, B, N1, N2, D) && scratch != nullptr &&
        scratch_bytes >= scratch_layout(B, N1, N2, D, false).total)
        engine = TPW_ENGINE_TCGEN05_BF16X3;
    if (engine != TPW_ENGINE_TCGEN05_BF16X3 || dtype != TPW_F32) {
        TPW_CHECK_ARG(engine != TPW_ENGINE_TCGEN05_BF16X3 || dtype == TPW_F64,
                      "tpw_dot_metric_forward_ws: bad dtype %d", dtype);
        return tpw_dot_metric_forward_simt(dtype, epilogue, x1, x2, out, B, N1, N2, D, stream);
    }
    TPW_CHECK_ARG(epilogue >= TPW_DOT_LINEAR && epilogue <= TPW_DOT_EUCLIDEAN, "tpw_dot_metric_forward_ws: bad epilogue %d", epilogue);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_dot_metric_forward_ws: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(x1 && x2 && out, "tpw_dot_metric_forward_ws: NULL pointer");
    TPW_CHECK_ARG(D > 0, "tpw_dot_metric_forward_ws: D must be positive");
    TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && B < (1ll << 31) && D < (1ll << 31),
                  "tpw_dot_metric_forward_ws: a dimension exceeds 2^31-1");
    const bool self = (x1 == x2) && (N1 == N2);
    const ScratchLayout L = scratch_layout(B, N1, N2, D, false);
    TPW_CHECK_ARG(scratch != nullptr && scratch_bytes >= L.total,
                  "tpw_dot_metric_forward_ws: the tensor-core engine needs %lld bytes of scratch (got %lld)",
                  L.total, (long long)scratch_bytes);
    TPW_CHECK_ARG(aligned16(scratch), "tpw_dot_metric_forward_ws: scratch must be 16-byte aligned");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool recip = epilogue == TPW_DOT_COSINE_SIM || epilogue == TPW_DOT_COSINE_DIST || epilogue == TPW_DOT_ONE_MINUS_SIM;
    Bf16Operands M;
    GemmParams P;
    int st;
    if ((st = prepare_bf16_operands(x1, x2, scratch, recip, B, N1, N2, D, s, M, P)) != TPW_OK) return st;
    P.out = static_cast<float *>(out);
    P.epilogue = epilogue;
    P.self = self ? 1 : 0;
    P.vec_store = (N2 % 4 == 0 && aligned16(out)) ? 1 : 0;
    TPW_CHECK_ARG(P.tiles < (1ll << 40), "tpw_dot_metric_forward_ws: too many tiles");
    const long long nsm = sm_count();
    const unsigned grid = (unsigned)(P.tiles < nsm ? P.tiles : nsm);
#define TPW_GEMM_LAUNCH(EPI, SELF)                                                                                        \
    do {                                                                                                                  \
        auto kern = gemm_metric_kernel<EPI, SELF, false>;                                                                        \
        TPW_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC));                 \
        kern<<<grid, kThreads, SMEM_ALLOC, s>>>(M.mxh, M.mxl, M.myh, M.myl, P);                                           \
    } while (0)
    switch (epilogue) {
        case TPW_DOT_LINEAR: TPW_GEMM_LAUNCH(TPW_DOT_LINEAR, false); break;
        case TPW_DOT_COSINE_SIM: TPW_GEMM_LAUNCH(TPW_DOT_COSINE_SIM, false); break;
        case TPW_DOT_COSINE_DIST: TPW_GEMM_LAUNCH(TPW_DOT_COSINE_DIST, false); break;
        case TPW_DOT_ONE_MINUS_SIM: TPW_GEMM_LAUNCH(TPW_DOT_ONE_MINUS_SIM, false); break;
        case TPW_DOT_SQEUCLIDEAN:
            if (self) TPW_GEMM_LAUNCH(TPW_DOT_SQEUCLIDEAN, true); else TPW_GEMM_LAUNCH(TPW_DOT_SQEUCLIDEAN, false);
            break;
        default:
            if (self) TPW_GEMM_LAUNCH(TPW_DOT_EUCLIDEAN, true); else TPW_GEMM_LAUNCH(TPW_DOT_EUCLIDEAN, false);
            break;
    }
#undef TPW_GEMM_LAUNCH
    TPW_LAUNCH_OK("gemm_metric_kernel");
    return TPW_OK;
}

static bool backward_uses_tensor_cores(int dtype, int mode, int engine, int64_t B, int64_t N1, int64_t N2, int64_t D) {
    if (dtype != TPW_F32 || B <= 0 || N1 <= 0 || N2 <= 0 || D <= 0) return false;
    if (mode != TPW_LP_BWD_CDIST && mode != TPW_LP_BWD_PPMINKOWSKI && mode != TPW_LP_BWD_MATMUL) return false;
    if (engine == TPW_ENGINE_TCGEN05_BF16X3 || engine == TPW_ENGINE_TCGEN05_TF32X3) return true;
    return engine == TPW_ENGINE_AUTO && auto_picks_tensor_backward(dtype, B, N1, N2, D);
}

extern "C" int64_t tpw_dot_backward_scratch_bytes(int dtype, int mode, int engine, int64_t B, int64_t N1, int64_t N2, int64_t D) {
    if (!backward_uses_tensor_cores(dtype, mode, engine, B, N1, N2, D)) return 0;
    return bwd_scratch_layout(B, N1, N2, D).total;
}

extern "C" int tpw_cosine_backward_finish(int dtype, void *grad_x, const void *x, const void *norm, const void *term,
                                          int64_t rows, int64_t D, tpw_stream_t stream);

// Shared body of the two entry points below.  coef: COEF_ID / COEF_DIV_AUX / COEF_COSINE.
static int dense_backward_tensor(int coef, int epilogue, bool sums, float s_mm, float s_row,
                                 const void *grad, const void *aux, const void *norm1, const void *norm2,
                                 const void *x1, const void *x2, void *grad_x1, void *grad_x2, void *scratch,
                                 int64_t B, int64_t N1, int64_t N2, int64_t D, cudaStream_t s) {
    const BwdScratch L = bwd_scratch_layout(B, N1, N2, D);
    unsigned char *base = static_cast<unsigned char *>(scratch);
    auto F = [&](long long off) { return reinterpret_cast<float *>(base + off); };
    int st;

    // coefficient matrix C [N1,N2] as tf32 high/low parts, written once: grad_x1 = C . X2 reads it K-major
    // (reduction along its rows), grad_x2 = C^T . X1 reads the same copy MN-major (reduction over its row index)
    SplitParams C;
    memset(&C, 0, sizeof(C));
    C.a = static_cast<const float *>(grad);
    C.aux = static_cast<const float *>(aux);
    C.n1 = static_cast<const float *>(norm1);
    C.n2 = static_cast<const float *>(norm2);
    C.epilogue = epilogue;
    C.hi = F(L.off_chi); C.lo = F(L.off_clo);
    C.rowpart = F(L.off_rowpart); C.colpart = F(L.off_colpart);
    C.R = N1; C.C = N2; C.Cp = L.N2p; C.TR = L.TR; C.TC = L.TC;
    C.vec_in = (N2 % 4 == 0 && aligned16(grad) && (coef == COEF_ID || aligned16(aux))) ? 1 : 0;
    if (coef == COEF_COSINE) st = launch_split<COEF_COSINE, true>(C, B, s);
    else if (coef == COEF_DIV_AUX) st = launch_split<COEF_DIV_AUX, true>(C, B, s);
    else if (sums) st = launch_split<COEF_ID, true>(C, B, s);
    else st = launch_split<COEF_ID, false>(C, B, s);
    if (st != TPW_OK) return st;
    if (sums) {
        reduce_partials_kernel<<<(unsigned)((B * N1 + 255) / 256), 256, 0, s>>>(F(L.off_rowpart), F(L.off_rowsum), B, L.TC, N1);
        reduce_partials_kernel<<<(unsigned)((B * N2 + 255) / 256), 256, 0, s>>>(F(L.off_colpart), F(L.off_colsum), B, L.TR, N2);
        TPW_LAUNCH_OK("reduce_partials_kernel");
    }
    const long long cap = (long long)sm_count() * 8;
    const Tf32Operand Ck{F(L.off_chi), F(L.off_clo), L.N2p, false}, Cmn{F(L.off_chi), F(L.off_clo), L.N2p, true};
    for (int side = 0; side < 2; ++side) {
        void *gout = side == 0 ? grad_x1 : grad_x2;
        if (!gout) continue;
        // side 0: grad_x1[N1,D] = C . X2, X2 [N2,D] contracted over its rows; side 1: grad_x2[N2,D] = C^T . X1
        const void *xk = side == 0 ? x2 : x1;   // operand contracted against (MN-major: its rows are k)
        const void *xo = side == 0 ? x1 : x2;   // rows that receive the gradient
        const long long Nk = side == 0 ? N2 : N1, No = side == 0 ? N1 : N2;
        float *xhi = F(side == 0 ? L.off_x2hi : L.off_x1hi), *xlo = F(side == 0 ? L.off_x2lo : L.off_x1lo);
        SplitParams X;
        memset(&X, 0, sizeof(X));
        X.a = static_cast<const float *>(xk);
        X.hi = xhi; X.lo = xlo;
        X.R = Nk; X.C = D; X.Cp = L.Dp;
        X.vec_in = (D % 4 == 0 && aligned16(xk)) ? 1 : 0;
        if ((st = launch_split<COEF_ID, false>(X, B, s)) != TPW_OK) return st;
        const Tf32Operand Xmn{xhi, xlo, L.Dp, true};
        if (side == 0) st = launch_tf32_product(Ck, Xmn, static_cast<float *>(gout), B, N1, D, N2, s);
        else st = launch_tf32_product(Cmn, Xmn, static_cast<float *>(gout), B, N2, D, N1, s);
        if (st != TPW_OK) return st;
        const float *sumv = F(side == 0 ? L.off_rowsum : L.off_colsum);
        if (coef == COEF_COSINE) {
            // the norm part of the chain: g[r,:] += term[r] * x[r,:] / norm[r]
            if ((st = tpw_cosine_backward_finish(TPW_F32, gout, xo, side == 0 ? norm1 : norm2, sumv, B * No, D, s)) != TPW_OK) return st;
        } else if (sums) {
            const long long n = B * No * D, blocks = (n + 255) / 256;
            grad_finish_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, s>>>(
                static_cast<float *>(gout), static_cast<const float *>(xo), sumv, B * No, D, s_mm, s_row);
            TPW_LAUNCH_OK("grad_finish_kernel");
        }
    }
    return TPW_OK;
}

extern "C" int tpw_dot_backward_ws(int dtype, int mode, int engine, const void *grad, const void *aux,
                                   const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                                   void *scratch, int64_t scratch_bytes,
                                   int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(engine >= TPW_ENGINE_AUTO && engine <= TPW_ENGINE_TCGEN05_TF32X3, "tpw_dot_backward_ws: bad engine %d", engine);
    TPW_CHECK_ARG(mode == TPW_LP_BWD_CDIST || mode == TPW_LP_BWD_PPMINKOWSKI || mode == TPW_LP_BWD_MATMUL,
                  "tpw_dot_backward_ws: mode %d has no contraction form (p = 2 modes and the plain products only)", mode);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_dot_backward_ws: negative size");
    bool tensor = backward_uses_tensor_cores(dtype, mode, engine, B, N1, N2, D);
    if (tensor && engine == TPW_ENGINE_AUTO && (scratch == nullptr || scratch_bytes < bwd_scratch_layout(B, N1, N2, D).total))
        tensor = false;
    if (!tensor) {
        TPW_CHECK_ARG(engine == TPW_ENGINE_AUTO || engine == TPW_ENGINE_SIMT_FP32 || dtype == TPW_F64,
                      "tpw_dot_backward_ws: the tensor-core engine takes float32 only");
        return tpw_lp_backward(dtype, mode, grad, aux, x1, x2, nullptr, grad_x1, grad_x2, B, N1, N2, D, 2.0, stream);
    }
    TPW_CHECK_ARG(grad && x1 && x2 && (grad_x1 || grad_x2), "tpw_dot_backward_ws: NULL pointer");
    TPW_CHECK_ARG(mode != TPW_LP_BWD_CDIST || aux != nullptr, "tpw_dot_backward_ws: the Euclidean mode needs the forward output");
    TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && D < (1ll << 31), "tpw_dot_backward_ws: a dimension exceeds 2^31-1");
    const long long need = bwd_scratch_layout(B, N1, N2, D).total;
    TPW_CHECK_ARG(scratch != nullptr && scratch_bytes >= need,
                  "tpw_dot_backward_ws: the tensor-core engine needs %lld bytes of scratch (got %lld)", need, (long long)scratch_bytes);
    TPW_CHECK_ARG(aligned16(scratch), "tpw_dot_backward_ws: scratch must be 16-byte aligned");
    const float s_mm = mode == TPW_LP_BWD_MATMUL ? 1.f : (mode == TPW_LP_BWD_PPMINKOWSKI ? -2.f : -1.f);
    const float s_row = mode == TPW_LP_BWD_PPMINKOWSKI ? 2.f : 1.f;
    return dense_backward_tensor(mode == TPW_LP_BWD_CDIST ? COEF_DIV_AUX : COEF_ID, 0, mode != TPW_LP_BWD_MATMUL, s_mm, s_row,
                                 grad, aux, nullptr, nullptr, x1, x2, grad_x1, grad_x2, scratch, B, N1, N2, D,
                                 static_cast<cudaStream_t>(stream));
}

extern "C" int tpw_cosine_backward_ws(int epilogue, const void *grad, const void *out, const void *norm1, const void *norm2,
                                      const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                                      void *scratch, int64_t scratch_bytes,
                                      int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(epilogue == TPW_DOT_COSINE_SIM || epilogue == TPW_DOT_COSINE_DIST || epilogue == TPW_DOT_ONE_MINUS_SIM,
                  "tpw_cosine_backward_ws: bad epilogue %d", epilogue);
    TPW_CHECK_ARG(B > 0 && N1 > 0 && N2 > 0 && D > 0, "tpw_cosine_backward_ws: sizes must be positive");
    TPW_CHECK_ARG(grad && out && norm1 && norm2 && x1 && x2 && (grad_x1 || grad_x2), "tpw_cosine_backward_ws: NULL pointer");
    TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && D < (1ll << 31), "tpw_cosine_backward_ws: a dimension exceeds 2^31-1");
    const long long need = bwd_scratch_layout(B, N1, N2, D).total;
    TPW_CHECK_ARG(scratch != nullptr && scratch_bytes >= need,
                  "tpw_cosine_backward_ws: needs %lld bytes of scratch (got %lld)", need, (long long)scratch_bytes);
    TPW_CHECK_ARG(aligned16(scratch), "tpw_cosine_backward_ws: scratch must be 16-byte aligned");
    return dense_backward_tensor(COEF_COSINE, epilogue, true, 1.f, 0.f, grad, out, norm1, norm2, x1, x2, grad_x1, grad_x2, scratch,
                                 B, N1, N2, D, static_cast<cudaStream_t>(stream));
}
