// Boolean pairwise metrics with the pair counts taken on the tensor cores.
//
// n11[i,j] = |x_i & y_j| is the dot product of two 0/1 vectors.  One-byte booleans are exactly the unsigned 8-bit
// operands of tcgen05.mma.kind::i8, whose 32-bit integer accumulators hold the counts exactly (D <= 2^24 < 2^31),
// so the contingency table of every pair is the same set of integers the popcount kernel produces and the shared
// epilogue (bool_epilogue.cuh) turns it into the same float32 bits.  What changes is the bound: the popcount tile
// is pinned at the POPC issue rate (C3, 65536 x 16384 x 1024 bits: 7.9 ms), the integer contraction leaves only
// the operand stream from L2 and the 4-byte output write.
//
// Kernel: persistent, one CTA per SM, 576 threads -- warp 0 issues TMA (one lane), warp 1 owns tensor memory and
// issues the MMAs (one lane), warps 2..17 drain the accumulators (TMEM lane quarter = warp % 4, column quarter =
// (warp - 2) / 4).  Output tile 128 x 256; a k-step is 128 features = one 128-byte swizzled row per operand row,
// consumed by four MMAs of K = 32; three stages of 16 KB (x1) + 32 KB (x2); two 256-column accumulators in tensor
// memory, so the epilogue of tile t overlaps the MMAs of tile t + 1.  The operands are the caller's boolean
// matrices as they lie in memory (row pitch D bytes): no packed or padded copy is made, the TMA unit zero-fills
// rows and features past the edge, and zeros add nothing to a count.  Every CTA loads its own tiles with plain
// per-CTA TMA loads from this GPU's memory.
//
// An epilogue warp stages its 32 x 32 block of results in shared memory (128-byte swizzle) and writes it out either
// with its own 128-bit stores or, for the metrics whose arithmetic is long enough to hide it, by handing the block to
// the copy engine (a TMA store on the output's tensor map, which also clips the rows past N1).
//
// Every mbarrier wait is bounded; a role that gives up raises a CTA-wide abort flag, everybody falls through to the
// final barrier, tensor memory is released and the device status word reports the site.  The one wait without a
// bound of its own is cp.async.bulk.wait_group.read, which returns when the copy engine has read a block this warp
// committed itself.
#include "bool_epilogue.cuh"
#include "common.cuh"

#include <type_traits>
#include "tcgen05.cuh"

#include <stdlib.h>

namespace tpw {
namespace {

constexpr int BM = 128;             // x1 rows per tile (TMEM lanes)
constexpr int BN = 256;             // x2 rows per tile (TMEM columns per accumulator)
constexpr int BKB = 128;            // features (bytes) per k-step
constexpr int kStages = 3;
constexpr int A_BYTES = BM * BKB;   // 16 KB
constexpr int B_BYTES = BN * BKB;   // 32 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int OFF_BAR = kStages * STAGE_BYTES;
// barriers: full[3], empty[3], tmem_full[2], tmem_empty[2]; then the TMEM base address and the abort flag
constexpr int OFF_TMEM_PTR = OFF_BAR + (2 * kStages + 4) * 8;
constexpr int OFF_ABORT = OFF_TMEM_PTR + 4;
constexpr int OFF_STAGE = (OFF_ABORT + 4 + 1023) / 1024 * 1024; // per epilogue warp a 32 x 32 float staging block (1024-byte aligned: it is also the source of a swizzled TMA store)
constexpr int kEpilogueWarps = 16;            // four per TMEM lane quarter, each draining a quarter of the columns
constexpr int OFF_POP = OFF_STAGE + kEpilogueWarps * 4096;      // per epilogue warp the 64 x2 row counts of its column quarter
constexpr int SMEM_BYTES = OFF_POP + kEpilogueWarps * 256;
constexpr int SMEM_ALLOC = SMEM_BYTES + 1024;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr uint32_t kTmemCols = 512;
static_assert(SMEM_ALLOC <= 232448, "exceeds the dynamic shared memory of one CTA");

struct BoolTcParams {
    const int32_t *pop1, *pop2;
    float *out;
    long long B, N1, N2, D;
    long long tiles_m, tiles_n, tiles;
    int metric;
    int vec_store;   // N2 % 4 == 0, out and pop2 16-byte aligned
    int tma_store;   // the staged 32 x 32 blocks leave through the output's tensor map
    float inv_d;     // 1/D when D is a power of two, else 0
    int *status;
};

// D[tmem] (+)= A[smem] * B[smem]^T on unsigned 8-bit operands, 32-bit integer accumulate (K = 32 per instruction)
__device__ __forceinline__ void tc_mma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// Instruction descriptor of kind::i8: D = signed 32-bit (bits [4,6) = 2), A and B unsigned 8-bit (bits [7,10) and
// [10,13) = 0), both K-major (bits 15 and 16 = 0), N >> 3 in bits [17,23), M >> 4 in bits [24,29); dense, no saturation.
__device__ __forceinline__ uint32_t make_idesc_i8(int M, int N) {
    return (2u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// One instantiation per metric: with the metric a compile-time constant the epilogue's switch folds to the one case,
// which keeps the unrolled per-element code small enough for the instruction cache (with a run-time metric the 32
// inlined copies of the whole switch made the epilogue, not the contraction, the bound).
template <int METRIC>
__global__ void __launch_bounds__(kThreads, 1)
bool_count_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y,
                          const __grid_constant__ CUtensorMap map_out, const BoolTcParams P) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + OFF_BAR);
    uint64_t *empty = full + kStages;
    uint64_t *tmem_full = empty + kStages;
    uint64_t *tmem_empty = tmem_full + 2;
    uint32_t *tmem_ptr = reinterpret_cast<uint32_t *>(smem + OFF_TMEM_PTR);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + OFF_ABORT);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (int)((P.D + BKB - 1) / BKB);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(&tmem_full[a], 1); mbar_init(&tmem_empty[a], kEpilogueWarps); }
        *abort_flag = 0;
        mbar_init_fence();
        tma_prefetch_descriptor(&map_x);
        tma_prefetch_descriptor(&map_y);
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
                long long t = tile;
                const long long tn = t % P.tiles_n; t /= P.tiles_n;
                const long long tm = t % P.tiles_m;
                const long long b = t / P.tiles_m;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t use = it / kStages;
                    if (use > 0 && !wait_or_abort(&empty[s], (use - 1) & 1, abort_flag)) {
                        *abort_flag = 1;
                        if (P.status) atomicCAS(P.status, 0, (10 << 16) | 1);
                        ok = false;
                        break;
                    }
                    unsigned char *st = smem + s * STAGE_BYTES;
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_3d(st, &map_x, &full[s], kb * BKB, (int)(tm * BM), (int)b);
                    tma_load_3d(st + A_BYTES, &map_y, &full[s], kb * BKB, (int)(tn * BN), (int)b);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = make_idesc_i8(BM, BN);
            uint32_t it = 0, acount = 0;
            bool ok = true;
            for (long long tile = blockIdx.x; tile < P.tiles && ok; tile += gridDim.x, ++acount) {
                const uint32_t a = acount & 1, ause = acount >> 1;
                if (ause > 0 && !wait_or_abort(&tmem_empty[a], (ause - 1) & 1, abort_flag)) {
                    *abort_flag = 1;
                    if (P.status) atomicCAS(P.status, 0, (10 << 16) | 2);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + a * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % kStages;
                    if (!wait_or_abort(&full[s], (it / kStages) & 1, abort_flag)) {
                        *abort_flag = 1;
                        if (P.status) atomicCAS(P.status, 0, (10 << 16) | 3);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sb = smem_u32(smem + s * STAGE_BYTES);
                    const uint64_t dx = make_smem_desc(sb), dy = make_smem_desc(sb + A_BYTES);
                    // one MMA consumes 32 bytes of the swizzled row: the start address advances by 2 units of 16 bytes
#pragma unroll
                    for (int k = 0; k < BKB / 32; ++k) tc_mma_i8(d_tmem, dx + 2 * k, dy + 2 * k, idesc, (kb | k) != 0);
                    tc_commit(&empty[s]);   // the stage may be refilled once these MMAs have read it
                }
                if (ok) tc_commit(&tmem_full[a]);
            }
        }
    } else {
        // ---------------- epilogue: warps 2..17 ----------------
        const int q = warp & 3;
        const int cpart = (warp - 2) >> 2;           // which quarter of the tile's 256 columns
        constexpr int NCB = BN / 32 / (kEpilogueWarps / 4);   // 32-column blocks per warp and tile
        uint32_t tcount = 0;
        bool ok = true;
        const int D = (int)P.D;
        unsigned char *stg = smem + OFF_STAGE + (warp - 2) * 4096;
        for (long long tile = blockIdx.x; tile < P.tiles && ok; tile += gridDim.x, ++tcount) {
            long long t = tile;
            const long long tn = t % P.tiles_n; t /= P.tiles_n;
            const long long tm = t % P.tiles_m;
            const long long b = t / P.tiles_m;
            const uint32_t a = tcount & 1;
            // What the epilogue needs besides the counts depends on the tile index alone: fetch it before waiting for the
            // accumulator, so that the L2 round trip hides behind the contraction instead of sitting in every column block.
            const long long i = tm * BM + q * 32 + lane;
            const bool row_ok = i < P.N1;
            const int pa = row_ok ? __ldg(P.pop1 + b * P.N1 + i) : 0;
            const int32_t *pb = P.pop2 + b * P.N2;
            int32_t *popw = reinterpret_cast<int32_t *>(smem + OFF_POP + (warp - 2) * 256);
            {
                const long long jc = tn * BN + cpart * (NCB * 32) + lane * 2;   // 64 counts per warp: two per lane
                int2 v = make_int2(0, 0);
                if (P.vec_store && jc + 2 <= P.N2) v = __ldg(reinterpret_cast<const int2 *>(pb + jc));
                else {
                    if (jc + 0 < P.N2) v.x = __ldg(pb + jc + 0);
                    if (jc + 1 < P.N2) v.y = __ldg(pb + jc + 1);
                }
                __syncwarp();   // the previous tile's reads of this area are done
                *reinterpret_cast<int2 *>(popw + lane * 2) = v;
                __syncwarp();
            }
            if (!wait_or_abort(&tmem_full[a], (tcount >> 1) & 1, abort_flag)) {
                *abort_flag = 1;
                if (lane == 0 && P.status) atomicCAS(P.status, 0, (10 << 16) | 4);
                ok = false;
                break;
            }
            tc_fence_after();
            float *orow = P.out + (b * P.N1 + (row_ok ? i : 0)) * P.N2;
            const long long row_base = tm * BM + q * 32;
            // the mean metrics multiply by 1 / D where D is a power of two and divide otherwise: decided here, once per
            // tile, so that the per-element code holds one of the two
            auto drain = [&](auto inv_tag) {
                constexpr int INV = decltype(inv_tag)::value;
#pragma unroll 1
            for (int c = cpart * NCB; c < (cpart + 1) * NCB; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + a * BN + c * 32, r);
                tmem_ld_wait();
                const long long j0 = tn * BN + c * 32;
                if (j0 >= P.N2) continue;
                if (P.vec_store && j0 + 32 <= P.N2) {
                    // this thread's row ...
                    float4 o[8];
#pragma unroll
                    for (int v = 0; v < 8; ++v) {
                        const int4 nb = *reinterpret_cast<const int4 *>(popw + (c - cpart * NCB) * 32 + 4 * v);
                        o[v].x = bool_epilogue<true, INV>(METRIC, (int)r[4 * v + 0], pa, nb.x, D, P.inv_d);
                        o[v].y = bool_epilogue<true, INV>(METRIC, (int)r[4 * v + 1], pa, nb.y, D, P.inv_d);
                        o[v].z = bool_epilogue<true, INV>(METRIC, (int)r[4 * v + 2], pa, nb.z, D, P.inv_d);
                        o[v].w = bool_epilogue<true, INV>(METRIC, (int)r[4 * v + 3], pa, nb.w, D, P.inv_d);
                    }
                    if (P.tma_store) {
                        // by now the copy engine has read the previous block out of the staging area
                        if (lane == 0) tma_store_wait_read();
                        __syncwarp();
                    }
                    // ... staged with a 16-byte-chunk XOR swizzle ...
#pragma unroll
                    for (int v = 0; v < 8; ++v) *reinterpret_cast<float4 *>(stg + lane * 128 + ((v ^ (lane & 7)) << 4)) = o[v];
                    if (P.tma_store) {
                        // ... which is the layout of a 128-byte swizzled 32 x 32 box: one lane hands the block to the copy
                        // engine (rows past N1 are clipped by the tensor map) and the warp goes on to its next block
                        fence_proxy_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            tma_store_3d(&map_out, stg, (int)j0, (int)row_base, (int)b);
                            tma_store_commit();
                        }
                    } else {
                        __syncwarp();
                        // ... and written out four full 128-byte row segments per instruction
#pragma unroll
                        for (int itr = 0; itr < 8; ++itr) {
                            const int rr = itr * 4 + (lane >> 3), cc = lane & 7;
                            const float4 o = *reinterpret_cast<const float4 *>(stg + rr * 128 + ((cc ^ (rr & 7)) << 4));
                            if (row_base + rr < P.N1)
                                __stcs(reinterpret_cast<float4 *>(P.out + (b * P.N1 + row_base + rr) * P.N2 + j0) + cc, o);
                        }
                        __syncwarp();
                    }
                } else if (row_ok) {
#pragma unroll
                    for (int v = 0; v < 32; ++v) {
                        const long long j = j0 + v;
                        if (j < P.N2) orow[j] = bool_epilogue<true, INV>(METRIC, (int)r[v], pa, popw[(c - cpart * NCB) * 32 + v], D, P.inv_d);
                    }
                }
            }
            };
            if (METRIC == TPW_BOOL_EQ_MEAN || METRIC == TPW_BOOL_NE_MEAN) {
                if (P.inv_d != 0.f) drain(std::integral_constant<int, 1>{});
                else drain(std::integral_constant<int, 0>{});
            } else {
                drain(std::integral_constant<int, -1>{});
            }
            // this warp has drained its part of accumulator `a`
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tmem_empty[a]);
        }
    }

    if (warp >= 2 && lane == 0 && P.tma_store) tma_store_wait_read();   // shared memory stays valid until the last block is read
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

} // namespace
} // namespace tpw

using namespace tpw;

// 1 when tpw_bool_metric_forward_tc serves this problem: rows of at least 128 bytes whose pitch keeps every row
// 16-byte aligned (a TMA requirement), counts that stay exact, and enough pairs to fill the persistent grid.
extern "C" int tpw_bool_metric_tc_eligible(int64_t B, int64_t N1, int64_t N2, int64_t D) {
    if (getenv("TPW_DISABLE_BOOL_TC")) return 0;
    // up to 128 features the few-words popcount kernel is faster; the epilogue converts counts below 2^23 exactly with
    // one logic operation and one addition instead of the quarter-rate conversion instruction
    if (B <= 0 || N1 < BM || N2 < BN || D <= 128 || D % 16 != 0 || D >= (1 << 23)) return 0;
    if (N1 >= (1ll << 31) || N2 >= (1ll << 31) || B >= (1ll << 31)) return 0;
    return (double)B * (double)N1 * (double)N2 * (double)D >= 268435456.0 ? 1 : 0;
}

extern "C" int tpw_bool_metric_forward_tc(int metric, const uint8_t *x1, const uint8_t *x2,
                                          const int32_t *x1_popcount, const int32_t *x2_popcount, float *out,
                                          int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream) {
    clear_error();
    TPW_CHECK_ARG(metric >= 0 && metric < TPW_BOOL_METRIC_COUNT, "tpw_bool_metric_forward_tc: unknown metric %d", metric);
    TPW_CHECK_ARG(B >= 0 && N1 >= 0 && N2 >= 0 && D >= 0, "tpw_bool_metric_forward_tc: negative size");
    if (B == 0 || N1 == 0 || N2 == 0) return TPW_OK;
    TPW_CHECK_ARG(D > 0 && D < (1 << 23), "tpw_bool_metric_forward_tc: D must be in [1, 2^23) (exact float32 counts)");
    TPW_CHECK_ARG(D % 16 == 0, "tpw_bool_metric_forward_tc: D must be a multiple of 16 (row pitch in bytes); use tpw_bool_metric_forward");
    TPW_CHECK_ARG(x1 && x2 && x1_popcount && x2_popcount && out, "tpw_bool_metric_forward_tc: NULL pointer");
    TPW_CHECK_ARG(aligned16(x1) && aligned16(x2), "tpw_bool_metric_forward_tc: the boolean matrices must be 16-byte aligned");
    TPW_CHECK_ARG(N1 < (1ll << 31) && N2 < (1ll << 31) && B < (1ll << 31), "tpw_bool_metric_forward_tc: a dimension exceeds 2^31-1");
    BoolTcParams P;
    memset(&P, 0, sizeof(P));
    P.pop1 = x1_popcount; P.pop2 = x2_popcount; P.out = out;
    P.B = B; P.N1 = N1; P.N2 = N2; P.D = D;
    P.metric = metric;
    P.vec_store = (N2 % 4 == 0 && aligned16(out) && aligned16(x2_popcount)) ? 1 : 0;
    P.inv_d = (D & (D - 1)) == 0 ? 1.0f / (float)D : 0.f;
    P.tiles_m = (N1 + BM - 1) / BM;
    P.tiles_n = (N2 + BN - 1) / BN;
    P.tiles = B * P.tiles_m * P.tiles_n;
    P.status = device_status_ptr();
    CUtensorMap mx, my;
    int st = make_tensor_map_3d(&mx, x1, 1, D, N1, B, BKB, BM, true);
    if (st != TPW_OK) return st;
    st = make_tensor_map_3d(&my, x2, 1, D, N2, B, BKB, BN, true);
    if (st != TPW_OK) return st;
    CUtensorMap mo;
    memset(&mo, 0, sizeof(mo));
    // Metrics whose epilogue divides keep a warp busy long enough per block for the copy engine to drain the staging
    // area behind it (jaccard at 65536 x 16384 x 1024: 2.06 -> 1.80 ms); for the sums and the power-of-two means the
    // warp's own 128-bit stores are faster (hamming: 1.32 against 1.49 ms).  TPW_BOOL_TC_STORES=plain|tma overrides.
    const bool cheap = metric == TPW_BOOL_AND_SUM || metric == TPW_BOOL_OR_SUM || metric == TPW_BOOL_XOR_SUM ||
                       metric == TPW_BOOL_EQ_SUM || metric == TPW_BOOL_NE_SUM ||
                       ((metric == TPW_BOOL_EQ_MEAN || metric == TPW_BOOL_NE_MEAN) && P.inv_d != 0.f);
    const char *stores = getenv("TPW_BOOL_TC_STORES");
    P.tma_store = P.vec_store && (stores ? stores[0] == 't' : !cheap) ? 1 : 0;
    if (P.tma_store) {
        st = make_tensor_map_3d(&mo, out, 4, N2, N1, B, 32, 32, true);
        if (st != TPW_OK) return st;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const long long grid = P.tiles < sm_count() ? P.tiles : sm_count();
#define TPW_BOOL_TC_CASE(M)                                                                                                    \
    case M:                                                                                                                    \
        TPW_CUDA_OK(cudaFuncSetAttribute(bool_count_tcgen05_kernel<M>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_ALLOC)); \
        bool_count_tcgen05_kernel<M><<<(unsigned)grid, kThreads, SMEM_ALLOC, s>>>(mx, my, mo, P);                                  \
        break
    switch (metric) {
        TPW_BOOL_TC_CASE(TPW_BOOL_AND_SUM); TPW_BOOL_TC_CASE(TPW_BOOL_OR_SUM); TPW_BOOL_TC_CASE(TPW_BOOL_XOR_SUM);
        TPW_BOOL_TC_CASE(TPW_BOOL_EQ_SUM); TPW_BOOL_TC_CASE(TPW_BOOL_NE_SUM); TPW_BOOL_TC_CASE(TPW_BOOL_EQ_MEAN);
        TPW_BOOL_TC_CASE(TPW_BOOL_NE_MEAN); TPW_BOOL_TC_CASE(TPW_BOOL_JACCARD); TPW_BOOL_TC_CASE(TPW_BOOL_KULSINSKI);
        TPW_BOOL_TC_CASE(TPW_BOOL_KULCZYNSKI1); TPW_BOOL_TC_CASE(TPW_BOOL_YULE); TPW_BOOL_TC_CASE(TPW_BOOL_DICE);
        TPW_BOOL_TC_CASE(TPW_BOOL_ROGERSTANIMOTO); TPW_BOOL_TC_CASE(TPW_BOOL_RUSSELLRAO); TPW_BOOL_TC_CASE(TPW_BOOL_SOKALMICHENER);
        TPW_BOOL_TC_CASE(TPW_BOOL_SOKALSNEATH);
        default: return fail(TPW_ERR_INVALID, "tpw_bool_metric_forward_tc: unknown metric %d", metric);
    }
#undef TPW_BOOL_TC_CASE
    TPW_LAUNCH_OK("bool_count_tcgen05_kernel");
    return TPW_OK;
}
