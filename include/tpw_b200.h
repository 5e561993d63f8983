/*
 * tpw_b200.h -- C ABI of the B200 (sm_100a) pairwise-reduction kernels.
 *
 * Every entry point is torch-free: plain device pointers, sizes and a CUDA stream.
 * Unless a comment says otherwise a call
 *   - is asynchronous on `stream` (a cudaStream_t passed as void*; NULL = legacy default stream),
 *   - runs on the calling thread's current CUDA device,
 *   - allocates no device memory and never synchronises,
 *   - returns TPW_OK (0) or a tpw_status error; tpw_last_error() then holds a message.
 * All matrices are dense row-major:  x1 [B,N1,D], x2 [B,N2,D], out/grad [B,N1,N2]
 * (an unbatched call passes B = 1).  Sizes are int64 so that outputs beyond 2^31
 * elements are addressed correctly.
 *
 * Each declaration cites the interface of inspiros/torchpairwise v0.3.0 that it replaces
 * (paths relative to that project; OPS = torchpairwise/csrc/ops).
 */
#ifndef TPW_B200_H
#define TPW_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TPW_ABI_VERSION 1

#if defined(__GNUC__)
#define TPW_API __attribute__((visibility("default")))
#else
#define TPW_API
#endif

typedef void *tpw_stream_t;

enum tpw_status {
    TPW_OK = 0,
    TPW_ERR_INVALID = 1,     /* bad argument (shape, pointer alignment, enum value) */
    TPW_ERR_UNSUPPORTED = 2, /* valid request that this build has no kernel for */
    TPW_ERR_CUDA = 3,        /* a CUDA runtime/driver call failed */
    TPW_ERR_TIMEOUT = 4      /* a bounded device-side wait gave up (see tpw_device_status) */
};

enum tpw_dtype {
    TPW_F32 = 0,
    TPW_F64 = 1,
    TPW_I32 = 2, /* accepted by tpw_cmp_reduce_forward only */
    TPW_I64 = 3  /* accepted by tpw_cmp_reduce_forward only */
};

/* ---- library ------------------------------------------------------------------------------ */

/* Replaces torchpairwise::_cuda_version / _cuda_arch_flags (csrc/torchpairwise.cpp:28-56). */
TPW_API int tpw_abi_version(void);
TPW_API int tpw_cuda_version(void);          /* CUDART_VERSION the library was built with */
TPW_API const char *tpw_cuda_arch_flags(void); /* "sm_100a" */
/* Thread-local text of the last failure on this thread ("" when none). */
TPW_API const char *tpw_last_error(void);

/*
 * Device-side status word.  Kernels that wait on an mbarrier (TMA, tcgen05) bound the wait;
 * when a wait gives up the kernel records a non-zero code here and returns early, leaving the
 * context usable.  tpw_device_status() synchronises `stream`, copies the word to *code and
 * clears it.  No counterpart in the reference (its kernels never wait).
 */
TPW_API int tpw_device_status(int *code, tpw_stream_t stream);

/*
 * Failure-path self-test: launches one small CTA that waits, with the same bounded-wait code as
 * the TMA / tcgen05 kernels, on an mbarrier that nothing will ever complete.  After `budget_ms`
 * (1..1000) the CTA gives up, records code (15 << 16) | 1 in the device status word and returns;
 * the context stays usable.  Lets a test exercise "a wait ran out" without faulting or hanging
 * the GPU.  No counterpart in the reference.
 */
TPW_API int tpw_selftest_bounded_wait(int budget_ms, tpw_stream_t stream);

/* ---- L_p family on the CUDA cores ---------------------------------------------------------- */

/*
 * out[b,i,j] = ( sum_k w[b,k] * |x1[b,i,k] - x2[b,j,k]|^p ) ^ out_exponent       (finite p > 0)
 * out[b,i,j] =   max_k w[b,k] * |x1[b,i,k] - x2[b,j,k]|                            (p = +inf)
 * out[b,i,j] =   min_k w[b,k] * |x1[b,i,k] - x2[b,j,k]|                            (p = -inf)
 * w may be NULL (all ones).  out_exponent = 1/p gives Minkowski / weighted Minkowski,
 * 1 gives the un-rooted power sum, 1/p - 1 gives the coefficient matrix that the weighted
 * backward consumes.  p = 1, 2, 3 run multiply-only inner loops; other p use exp2/log2.
 *
 * Replaces: at::cdist as called by euclidean/manhattan/minkowski/chebyshev_distances
 * (OPS/pairwise_metrics.cpp:30,48,167,305); _ppminkowski forward
 * (OPS/cuda/ppminkowski_kernel.cu:16-59,62-130); _wminkowski forward incl. its `backward`
 * template flag (OPS/cuda/wminkowski_kernel.cu:16-64,67-143).
 */
TPW_API int tpw_lp_forward(int dtype, const void *x1, const void *x2, const void *w, void *out,
                   int64_t B, int64_t N1, int64_t N2, int64_t D,
                   double p, double out_exponent, tpw_stream_t stream);

/*
 * Streaming row minimum of the same reduction: min_out[b,i] = min_j out[b,i,j] and
 * arg_out[b,i] = the smallest j that attains it, for out as tpw_lp_forward defines it with
 * finite p > 0 or p = +inf.  The [B,N1,N2] matrix is never written: each 128x128 tile is
 * reduced in registers and warp shuffles and folded into one 64-bit key per x1 row.
 * float32 only (TPW_F32), w must be NULL.  A NaN distance ranks above +inf; N2 = 0 gives +inf and -1.
 * scratch: tpw_lp_rowmin_scratch_bytes(B, N1) bytes on the device, 8-byte aligned; the call
 * initialises it.  Either of min_out / arg_out may be NULL.
 *
 * No counterpart in the reference, which materialises the matrix and then sorts every row
 * of it (k_neighbors_mask, OPS/neighbors.cpp:10-35: dists.argsort(1).slice(1, 0, k + 1)).
 */
TPW_API int64_t tpw_lp_rowmin_scratch_bytes(int64_t B, int64_t N1);
TPW_API int tpw_lp_rowmin_forward(int dtype, const void *x1, const void *x2, const void *w,
                          float *min_out, int64_t *arg_out, void *scratch,
                          int64_t B, int64_t N1, int64_t N2, int64_t D,
                          double p, double out_exponent, tpw_stream_t stream);

/*
 * The k nearest x2 rows of every x1 row on few features, ascending: vals[b,i,t] = the t-th smallest out[b,i,j] as
 * tpw_lp_forward defines it (p in {1, 2, 3, +inf}), inds[b,i,t] = its j; exact ties go to the smaller j.
 * float32, D <= tpw_lp_topk_max_features(), k <= min(tpw_lp_topk_max_k(), N2).  One x1 row per thread with its k
 * best keys in registers; every thread walks over all x2 rows of its batch, so nothing but B*N1*k results is
 * written, no scratch is needed, and the result is deterministic.  A NaN distance ranks above +inf.
 * No counterpart in the reference (k_neighbors_mask sorts every row of the materialised matrix,
 * OPS/neighbors.cpp:10-35; its README lists argkmin as future work).
 */
TPW_API int tpw_lp_topk_max_features(void);
TPW_API int tpw_lp_topk_max_k(void);
TPW_API int tpw_lp_topk_forward(int dtype, const void *x1, const void *x2, float *vals, int64_t *inds,
                        int64_t B, int64_t N1, int64_t N2, int64_t D, int k, double p, double out_exponent,
                        tpw_stream_t stream);

/*
 * mask[b,i,j] = (out[b,i,j] <= radius) as one byte (0 / 1) per pair, for out as tpw_lp_forward
 * defines it with finite p > 0 or p = +inf: the comparison of radius_neighbors_mask
 * (OPS/neighbors.cpp:37-58: cdist(x1, x2, metric) <= epsilon) fused into the tile epilogue, so the
 * float matrix is neither written nor read back.  A NaN distance gives 0.  w must be NULL.
 */
TPW_API int tpw_lp_radius_mask_forward(int dtype, const void *x1, const void *x2, const void *w, uint8_t *mask,
                               int64_t B, int64_t N1, int64_t N2, int64_t D,
                               double p, double out_exponent, double radius, tpw_stream_t stream);

/*
 * Condensed self-distances: out[b, i (2N - i - 1) / 2 + (j - i - 1)] = d(x[b,i], x[b,j]) for i < j, i.e.
 * the upper triangle of tpw_lp_forward(x, x) row by row, [B, N (N - 1) / 2].  Tiles on or below the
 * diagonal are skipped, so about half of the pairs are evaluated.  Finite p > 0 or p = +inf.
 * The reference declares pdist and raises "yet to be implemented" (OPS/cpdist.cpp:233-246); its README
 * defines it as cdist(x, x) without the duplicated positions.
 */
TPW_API int tpw_lp_pdist_forward(int dtype, const void *x, void *out, int64_t B, int64_t N, int64_t D,
                         double p, double out_exponent, tpw_stream_t stream);

enum tpw_lp_backward_mode {
    /* ATen cdist backward: aux = forward output o.  p=1: g*sgn(d); p=2: g*d/o;
       other finite p: g*d*|d|^(p-2)/o^(p-1); +inf: g*sgn(d)*[|d|==o]; all 0 where o==0.
       (what autograd runs under OPS/pairwise_metrics.cpp:30,48,167,305) */
    TPW_LP_BWD_CDIST = 0,
    /* _ppminkowski backward: g*p*|d|^(p-1)*sgn(d); aux unused.
       (OPS/cuda/ppminkowski_kernel.cu:133-179) */
    TPW_LP_BWD_PPMINKOWSKI = 1,
    /* _wminkowski backward w.r.t. x1/x2: g*|d|^(p-1)*w_k*aux*sgn(d) with
       aux = S^(1/p-1) from tpw_lp_forward(out_exponent = 1/p-1).
       (OPS/cuda/wminkowski_kernel.cu:146-196) */
    TPW_LP_BWD_WMINKOWSKI = 2,
    /* plain contraction grad_x1 = g @ x2, grad_x2 = g^T @ x1 (aux unused, p ignored); the
       matrix-matrix part of the cosine / correlation / linear-kernel backward
       (autograd of OPS/pairwise_metrics.cpp:64,121,203). */
    TPW_LP_BWD_MATMUL = 3
};

/*
 * grad_x1[b,i,k] = sum_j coef[b,i,j] * phi(x1[b,i,k] - x2[b,j,k])   and the mirrored
 * grad_x2[b,j,k] = sum_i coef[b,i,j] * phi(x2[b,j,k] - x1[b,i,k]); every element is
 * written exactly once (no atomics, fixed summation order, bit-reproducible).
 * Either grad pointer may be NULL to skip that side.  Finite p only, except
 * TPW_LP_BWD_CDIST which also takes p = +inf.
 */
TPW_API int tpw_lp_backward(int dtype, int mode, const void *grad, const void *aux,
                    const void *x1, const void *x2, const void *w,
                    void *grad_x1, void *grad_x2,
                    int64_t B, int64_t N1, int64_t N2, int64_t D,
                    double p, tpw_stream_t stream);

/*
 * tpw_lp_backward with caller scratch: both gradients from ONE walk over the pairs.  A pair's term
 * coef * phi(x1 - x2) is formed once and added to the grad_x1 sum and, negated, to the grad_x2 sum
 * (4 operations per pair and feature where the two launches of tpw_lp_backward execute 6).  The sums of
 * grad_x2 over blocks of 256 rows of x1 go to `scratch` and are added in ascending block order by a
 * second kernel: no atomics, fixed summation order, bit-reproducible; the order differs from
 * tpw_lp_backward's, so the two agree to rounding, not bit for bit.
 * tpw_lp_backward_scratch_bytes() returns 0 where the kernel does not apply (float64, p = +inf, the
 * plain contraction, fewer than 256 rows of x1, N2 or D not a multiple of 4, small problems,
 * TPW_DISABLE_ONEPASS_BWD=1), else the scratch it wants: B * ceil(N1/256) * N2 * D * 4 bytes up to
 * 2 GiB (larger problems run as several launches over batch or row-block ranges).  With scratch ==
 * NULL, less than N2 * D * 4 bytes, a NULL gradient pointer or a pointer that is not 16-byte aligned the
 * call is tpw_lp_backward.  Replaces the same reference kernels as tpw_lp_backward
 * (OPS/cuda/ppminkowski_kernel.cu:133-218, OPS/cuda/wminkowski_kernel.cu:146-196, ATen's cdist backward).
 */
TPW_API int64_t tpw_lp_backward_scratch_bytes(int dtype, int mode, int64_t B, int64_t N1, int64_t N2, int64_t D, double p);
TPW_API int tpw_lp_backward_ws(int dtype, int mode, const void *grad, const void *aux,
                    const void *x1, const void *x2, const void *w,
                    void *grad_x1, void *grad_x2,
                    int64_t B, int64_t N1, int64_t N2, int64_t D,
                    double p, void *scratch, int64_t scratch_bytes, tpw_stream_t stream);

/*
 * grad_w[b,k] = sum_{i,j} grad*aux * |x1-x2|^p / p  (aux as in TPW_LP_BWD_WMINKOWSKI).
 * `scratch` holds B*N1*D elements of `dtype` (per-row partial sums reduced in a second,
 * ordered stage).  Replaces OPS/cuda/wminkowski_kernel.cu:198-221.
 */
TPW_API int tpw_wminkowski_backward_w(int dtype, const void *grad, const void *aux,
                              const void *x1, const void *x2, void *grad_w, void *scratch,
                              int64_t B, int64_t N1, int64_t N2, int64_t D,
                              double p, tpw_stream_t stream);

/*
 * The p = +inf case of TPW_LP_BWD_CDIST (the backward of chebyshev_distances, ATen's cdist backward under
 * OPS/pairwise_metrics.cpp:305) for float32 in three steps: one pass over (i, j, k) finds the coordinate that
 * attains each pair's maximum (compared against the saved forward output `out`) and writes a 4-byte code per
 * pair; two scatter kernels then add +-g into grad_x1 / grad_x2 at that coordinate, one thread per gradient
 * row in a fixed order (deterministic, no atomics).  The dense form does the comparison for every (i, j, k)
 * once per gradient.  Pairs whose maximum is attained by several coordinates (lattice-valued data) make the
 * call fall back, on the device and without a host round trip, to the dense kernel, so the result always
 * equals tpw_lp_backward(TPW_LP_BWD_CDIST, p = +inf).
 * The scratch query returns 0 when the problem is to be given to tpw_lp_backward instead (float64, fewer than
 * 16 or more than 65535 features, an empty dimension); otherwise 256 + 4 * B * N1 * N2 bytes, 16-byte aligned.
 * Either gradient may be NULL.
 */
TPW_API int64_t tpw_chebyshev_backward_scratch_bytes(int dtype, int64_t B, int64_t N1, int64_t N2, int64_t D);
TPW_API int tpw_chebyshev_backward_ws(const void *grad, const void *out, const void *x1, const void *x2,
                              void *grad_x1, void *grad_x2, void *scratch, int64_t scratch_bytes,
                              int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/*
 * Single-coordinate backward of the +-inf variants: for each pair the FIRST k attaining the
 * extreme of w_k*|d_k| receives the gradient (float atomics; grads must be zero-filled by
 * the caller).  w/grad_w may be NULL (un-weighted _ppminkowski form).
 * Replaces OPS/cuda/ppminkowski_kernel.cu:181-218 and OPS/cuda/wminkowski_kernel.cu:223-266.
 */
TPW_API int tpw_lp_inf_backward(int dtype, const void *grad, const void *x1, const void *x2, const void *w,
                        void *grad_x1, void *grad_x2, void *grad_w,
                        int64_t B, int64_t N1, int64_t N2, int64_t D,
                        int negative, tpw_stream_t stream);

/* ---- dense-contraction metrics -------------------------------------------------------------- */

enum tpw_dot_epilogue {
    TPW_DOT_LINEAR = 0,       /* x.y                                  (OPS/pairwise_metrics.cpp:58-65)   */
    TPW_DOT_COSINE_SIM = 1,   /* x.y/(|x||y|), numerator kept when the denominator is 0 (:112-122)        */
    TPW_DOT_COSINE_DIST = 2,  /* clip(1 - cosine_sim, 0, 2)           (:51-56)                           */
    TPW_DOT_ONE_MINUS_SIM = 3,/* 1 - cosine_sim, no clip: correlation on pre-centred rows (:190-204)      */
    TPW_DOT_SQEUCLIDEAN = 4,  /* max(|x|^2 + |y|^2 - 2 x.y, 0)        (:181-188, contraction form)       */
    TPW_DOT_EUCLIDEAN = 5     /* sqrt of the above: ATen's matmul form of cdist(p=2) (:24-31)             */
};

enum tpw_dot_engine {
    TPW_ENGINE_AUTO = 0,
    TPW_ENGINE_SIMT_FP32 = 1,   /* CUDA-core tile, exact fp32/fp64 FMA chain */
    TPW_ENGINE_TCGEN05_BF16X3 = 2, /* TMA-fed tcgen05.mma, bf16 hi/lo split (3 MMAs), fp32 TMEM accumulators */
    TPW_ENGINE_TCGEN05_TF32X3 = 3  /* same pipeline with tf32 hi/lo parts (22 bits per factor) and chunked
                                      accumulation: the gradient products of tpw_dot_backward_ws and, forward,
                                      TPW_DOT_LINEAR only (a plain dot product has no norm to hide bf16 rounding behind) */
};

/*
 * Cross-term metrics.  Row norms are accumulated inside the kernel from the staged tiles.
 * fp64 always uses the SIMT engine.
 */
TPW_API int tpw_dot_metric_forward(int dtype, int epilogue, int engine,
                           const void *x1, const void *x2, void *out,
                           int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/* Bytes of scratch the tcgen05 engine needs for the bf16 hi/lo operand copies (0 for SIMT). */
TPW_API int64_t tpw_dot_metric_scratch_bytes(int dtype, int engine, int64_t B, int64_t N1, int64_t N2, int64_t D);
TPW_API int tpw_dot_metric_forward_ws(int dtype, int epilogue, int engine,
                              const void *x1, const void *x2, void *out, void *scratch, int64_t scratch_bytes,
                              int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/*
 * Streaming row minimum of the squared Euclidean / Euclidean / cosine distance (TPW_DOT_SQEUCLIDEAN,
 * TPW_DOT_EUCLIDEAN, TPW_DOT_COSINE_DIST: clip(1 - S, 0, 2), non-negative) on the tensor cores (float32):
 * min_out[b,i] = min_j d(x1[b,i], x2[b,j]), arg_out[b,i] = the smallest j that attains it.  The bf16 x 3
 * pipeline of tpw_dot_metric_forward_ws with an epilogue in which every thread folds the columns
 * of its row into one 64-bit key; no [B,N1,N2] matrix is written, so the kernel stays bound by the
 * tensor pipe.  Distances carry the rounding of that pipeline (within the float32 parity tolerance);
 * between candidates closer than that the choice may differ from an exact evaluation.
 * scratch: tpw_dot_rowmin_scratch_bytes(...) bytes, 16-byte aligned.  No counterpart in the
 * reference (OPS/neighbors.cpp:10-35 sorts rows of the materialised matrix).
 */
TPW_API int64_t tpw_dot_rowmin_scratch_bytes(int64_t B, int64_t N1, int64_t N2, int64_t D);
TPW_API int tpw_dot_rowmin_forward_ws(int epilogue, const void *x1, const void *x2, float *min_out, int64_t *arg_out,
                              void *scratch, int64_t scratch_bytes,
                              int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/*
 * The k nearest x2 rows of every x1 row (k <= tpw_dot_topk_max_k()), same distances and pipeline as
 * tpw_dot_rowmin_forward_ws: val_out [B,N1,k] ascending, idx_out [B,N1,k] (ties towards the smaller
 * row; -1 / +inf when N2 < k).  Each epilogue thread keeps a sorted register list of the k smallest
 * keys of its accumulator row, candidates at or above an already published bound of the row's k-th
 * smallest are dropped first, the per-tile lists are merged by one warp per row.  Deterministic.
 * No [B,N1,N2] matrix is written (the reference sorts every row of it: OPS/neighbors.cpp:10-35;
 * its README lists argkmin as future work).
 */
TPW_API int tpw_dot_topk_max_k(void);
TPW_API int64_t tpw_dot_topk_scratch_bytes(int64_t k, int64_t B, int64_t N1, int64_t N2, int64_t D);
TPW_API int tpw_dot_topk_forward_ws(int epilogue, int k, const void *x1, const void *x2, float *val_out, int64_t *idx_out,
                            void *scratch, int64_t scratch_bytes,
                            int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/*
 * Backward of the p = 2 metrics and the plain gradient products as two tensor-core contractions:
 *   TPW_LP_BWD_PPMINKOWSKI (sqeuclidean): C = g,      grad_x1 = 2 (x1 * rowsum(C) - C x2),  grad_x2 = 2 (x2 * colsum(C) - C^T x1)
 *   TPW_LP_BWD_CDIST       (euclidean):   C = g / o (0 where o == 0), same without the factor 2; aux = o
 *   TPW_LP_BWD_MATMUL:                    grad_x1 = g x2, grad_x2 = g^T x1
 * (OPS/cpu/ppminkowski_kernel.cpp:131-169 for p = 2; ATen's cdist backward under
 * OPS/pairwise_metrics.cpp:30; the matmul nodes under :64,121,203.)  A pre-pass writes C once as
 * tf32 high/low parts (C x2 reads it K-major, C^T x1 reads the same copy MN-major, no transposed
 * copy), tcgen05.mma accumulates hi.hi + hi.lo + lo.hi in fp32 in chunks of 64 elements that are
 * summed in registers, row and column sums are reduced in a fixed order: deterministic, as
 * accurate as the fp32 FMA chain.
 * engine AUTO picks this for float32 with D >= 64, N1, N2 >= 256 and B*N1*N2*D >= 2^28 when the
 * scratch is large enough, otherwise the call is tpw_lp_backward(p = 2) on the CUDA cores;
 * engine SIMT_FP32 always is; either TCGEN05 value forces the tensor cores (float32 only).
 * scratch: tpw_dot_backward_scratch_bytes(...) bytes (0 = CUDA-core path), 16-byte aligned;
 * about 8 bytes per element of grad.  grad_x1 or grad_x2 may be NULL.
 */
TPW_API int64_t tpw_dot_backward_scratch_bytes(int dtype, int mode, int engine, int64_t B, int64_t N1, int64_t N2, int64_t D);
TPW_API int tpw_dot_backward_ws(int dtype, int mode, int engine, const void *grad, const void *aux,
                        const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                        void *scratch, int64_t scratch_bytes,
                        int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/*
 * Whole backward of cosine_similarity / cosine_distances / correlation's 1 - S on the tensor cores
 * (float32): the element-wise chain of tpw_cosine_backward_prepare is folded into the pre-pass of
 * the two products, so dM is never written as a float32 matrix, and tpw_cosine_backward_finish is
 * applied to both gradients.  Same scratch as tpw_dot_backward_ws with TPW_LP_BWD_MATMUL; callers
 * use it when that size query is positive and the prepare / tpw_lp_backward / finish sequence otherwise.
 * (the autograd chain under OPS/pairwise_metrics.cpp:118-121; OPS/cuda/prf_div_kernel.cu:315-366)
 */
TPW_API int tpw_cosine_backward_ws(int epilogue, const void *grad, const void *out, const void *norm1, const void *norm2,
                           const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                           void *scratch, int64_t scratch_bytes,
                           int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/* Row helpers used by cosine / correlation host code (x.norm(2,-1), x - x.mean(-1):
   OPS/pairwise_metrics.cpp:118-119,197-201). rows = B*N. */
TPW_API int tpw_row_center(int dtype, const void *x, void *out, int64_t rows, int64_t D, tpw_stream_t stream);
TPW_API int tpw_row_norm(int dtype, const void *x, void *norm, int64_t rows, int64_t D, tpw_stream_t stream);

/*
 * Element-wise part of the cosine-similarity backward (the autograd chain of
 * OPS/pairwise_metrics.cpp:118-121: norm, outer product, matmul, prf_div "identity",
 * OPS/cuda/prf_div_kernel.cu:315-366).  `out` is the saved forward result of `epilogue`
 * (COSINE_SIM, COSINE_DIST or ONE_MINUS_SIM), norm1/norm2 the row norms [B,N1]/[B,N2].
 * Writes dM [B,N1,N2] (gradient w.r.t. the raw dot products; may alias nothing),
 * rowterm [B,N1] and colterm [B,N2] (gradients w.r.t. the two norm vectors).  Fixed summation
 * order, no atomics.  The matrix products dM @ x2 and dM^T @ x1 are then TPW_LP_BWD_MATMUL,
 * and tpw_cosine_backward_finish adds term[r] * x[r,:] / norm[r] (rows with a zero norm skipped).
 */
TPW_API int tpw_cosine_backward_prepare(int dtype, int epilogue, const void *grad, const void *out,
                                        const void *norm1, const void *norm2,
                                        void *dM, void *rowterm, void *colterm,
                                        int64_t B, int64_t N1, int64_t N2, tpw_stream_t stream);
TPW_API int tpw_cosine_backward_finish(int dtype, void *grad_x, const void *x, const void *norm, const void *term,
                                       int64_t rows, int64_t D, tpw_stream_t stream);

/* ---- boolean family on packed bits ---------------------------------------------------------- */

/*
 * Packs rows of one-byte booleans (any non-zero byte = 1) into little-endian 32-bit words,
 * `words_per_row` words per row (>= ceil(D/32), tail bits zero), and writes each row's
 * population count.  The reference never packs (one byte per bool, one thread per pair:
 * OPS/cuda/pairwise_binary_kernels.cu:32-53); this is the B200 layout of its inputs.
 */
TPW_API int tpw_bitpack(const uint8_t *src, uint32_t *words, int32_t *row_popcount,
                int64_t rows, int64_t D, int64_t words_per_row, tpw_stream_t stream);

enum tpw_bool_metric {
    TPW_BOOL_AND_SUM = 0, TPW_BOOL_OR_SUM = 1, TPW_BOOL_XOR_SUM = 2,     /* pwand_sum, pwor_sum, pwxor_sum */
    TPW_BOOL_EQ_SUM = 3, TPW_BOOL_NE_SUM = 4,                            /* pweq_sum, pwne_sum */
    TPW_BOOL_EQ_MEAN = 5, TPW_BOOL_NE_MEAN = 6,                          /* pweq_mean, pwne_mean (= hamming) */
    TPW_BOOL_JACCARD = 7, TPW_BOOL_KULSINSKI = 8, TPW_BOOL_KULCZYNSKI1 = 9,
    TPW_BOOL_YULE = 10, TPW_BOOL_DICE = 11, TPW_BOOL_ROGERSTANIMOTO = 12,
    TPW_BOOL_RUSSELLRAO = 13, TPW_BOOL_SOKALMICHENER = 14, TPW_BOOL_SOKALSNEATH = 15,
    TPW_BOOL_METRIC_COUNT = 16
};

/*
 * One AND-popcount tile pass gives n11; with the row popcounts every count of the 2x2
 * contingency table follows exactly, and the epilogue evaluates the metric with the same
 * float32 operation order as the reference's composition (no FMA contraction, IEEE divide),
 * so results are bit-identical.  out is float32 [B,N1,N2].
 * Replaces pw{and,or,xor,eq,ne}_sum / pw{eq,ne}_mean on bool inputs
 * (OPS/cuda/pairwise_binary_kernels.cu:144-220) and the compositions at
 * OPS/pairwise_metrics.cpp:206-243,339-399.
 */
TPW_API int tpw_bool_metric_forward(int metric, const uint32_t *x1_words, const uint32_t *x2_words,
                            const int32_t *x1_popcount, const int32_t *x2_popcount, float *out,
                            int64_t B, int64_t N1, int64_t N2, int64_t D, int64_t words_per_row,
                            tpw_stream_t stream);

/*
 * The same metrics with the pair counts n11 = |x & y| taken on the tensor cores: the one-byte booleans x1
 * [B,N1,D], x2 [B,N2,D] (0 / 1, as they lie in memory; 16-byte aligned, D a multiple of 16) are the unsigned
 * 8-bit operands of tcgen05.mma.kind::i8, whose 32-bit integer accumulators hold the counts exactly, and the
 * epilogue is the one of tpw_bool_metric_forward, so the float32 output is bit-identical to it.  The popcount
 * tile is bound by the POPC issue rate; this kernel by the operand stream from L2 and the output write.
 * x1_popcount / x2_popcount are the row counts tpw_bitpack produces.  tpw_bool_metric_tc_eligible returns 1 for
 * the problems this entry serves (rows of more than 128 and fewer than 2^23 features, at least 128 x 256 pairs per batch, a large
 * enough contraction; TPW_DISABLE_BOOL_TC=1 turns it off), 0 when tpw_bool_metric_forward is to be used.
 * Replaces the same reference code as tpw_bool_metric_forward.
 */
TPW_API int tpw_bool_metric_tc_eligible(int64_t B, int64_t N1, int64_t N2, int64_t D);
TPW_API int tpw_bool_metric_forward_tc(int metric, const uint8_t *x1, const uint8_t *x2,
                               const int32_t *x1_popcount, const int32_t *x2_popcount, float *out,
                               int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

enum tpw_cmp_op { TPW_CMP_EQ = 0, TPW_CMP_NE = 1 };
enum tpw_cmp_reduction { TPW_RED_SUM = 0, TPW_RED_MEAN = 1 };

/*
 * out[b,i,j] = sum_k float(x1[b,i,k] op x2[b,j,k])  (MEAN: divided by float(D)); float32 out.
 * Non-boolean inputs of hamming_distances / pw{eq,ne}_{sum,mean}
 * (OPS/pairwise_metrics.cpp:206-213; OPS/cuda/pairwise_binary_kernels.cu:32-53).
 * dtype: TPW_F32, TPW_F64 (IEEE compare), TPW_I32, TPW_I64.
 */
TPW_API int tpw_cmp_reduce_forward(int dtype, int op, int reduction, const void *x1, const void *x2, float *out,
                           int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/* ---- sums of two-argument terms that are not functions of the difference alone ------------------ */

enum tpw_pair_metric {
    TPW_PAIR_CANBERRA = 0,      /* sum_k |x - y| / (|x| + |y|), zero denominators skipped (OPS/cpu/canberra_kernel.cpp:22-29) */
    TPW_PAIR_ADDITIVE_CHI2 = 1  /* - sum_k (x - y)^2 / (x + y), zero denominators skipped (OPS/cpu/additive_chi2_kernel.cpp:22-31) */
};

/*
 * out[b,i,j] = sum_k term(x1[b,i,k], x2[b,j,k]) on the CUDA-core forward tile, and its backward
 * grad_x1[b,i,k] = sum_j g[b,i,j] d term / d x1 (grad_x2 by symmetry of the terms), deterministic.
 * Replaces _canberra / _additive_chi2_kernel forward and backward
 * (OPS/cpu/canberra_kernel.cpp:85-125, OPS/cpu/additive_chi2_kernel.cpp:88-131 and their CUDA twins).
 */
TPW_API int tpw_pair_sum_forward(int dtype, int metric, const void *x1, const void *x2, void *out,
                         int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);
TPW_API int tpw_pair_sum_backward(int dtype, int metric, const void *grad, const void *x1, const void *x2,
                          void *grad_x1, void *grad_x2,
                          int64_t B, int64_t N1, int64_t N2, int64_t D, tpw_stream_t stream);

/*
 * Jensen-Shannon sums: out[b,i,j] = f(scale * sum_k (x log(x/m) + y log(y/m))), m = (x + y)/2, x = x1[b,i,k],
 * y = x2[b,j,k], f = square root when take_sqrt is 1 (clamped at 0), identity when 0.  A zero entry
 * contributes 0, a negative one +inf (OPS/cpu/rel_entr.h:9-18).  Same forward tile as the sums above.
 * Replaces _sqjensenshannon (OPS/cpu/sqjensenshannon_kernel.cpp:13-81 and its CUDA twin) with
 * scale = 1/(2 log base) or 1/2, and the sqrt_ of jensenshannon_distances (OPS/pairwise_metrics.cpp:326-337).
 * Backward: `out` is the saved forward result when it was computed with take_sqrt = 1 (coefficient
 * grad * scale / (2 out), nothing where out is 0) and NULL otherwise; the derivative of a term with respect
 * to x is log(x/m) where x > 0 and -y/(x + y) at x == 0 (OPS/cpu/sqjensenshannon_kernel.cpp:84-141).
 * Either gradient may be NULL.
 */
TPW_API int tpw_jensenshannon_forward(int dtype, const void *x1, const void *x2, void *out,
                              int64_t B, int64_t N1, int64_t N2, int64_t D, double scale, int take_sqrt,
                              tpw_stream_t stream);
TPW_API int tpw_jensenshannon_backward(int dtype, const void *grad, const void *out, const void *x1, const void *x2,
                               void *grad_x1, void *grad_x2,
                               int64_t B, int64_t N1, int64_t N2, int64_t D, double scale, tpw_stream_t stream);

/* ---- haversine ------------------------------------------------------------------------------- */

/*
 * x1 [B,N1,2], x2 [B,N2,2] = (latitude, longitude) in radians  ->  out [B,N1,N2] = 2 asin(sqrt(a)),
 * a = sin^2(dlat/2) + cos(lat1) cos(lat2) sin^2(dlon/2), evaluated as 2 atan2(sqrt(a), sqrt(1 - a)) with 1 - a
 * formed without cancellation (nearly antipodal pairs keep their accuracy); a point against itself gives exactly 0.  Replaces _haversine (OPS/cpu/haversine_kernel.cpp:12-75 and its CUDA twin).
 * Backward (OPS/cpu/haversine_kernel.cpp:77-217): grad_x1 [B,N1,2], grad_x2 [B,N2,2], either may be NULL;
 * one deterministic pass per gradient, no scratch (the reference materialises a [B,N1,N2] denominator);
 * pairs whose denominator sqrt(a) sqrt(1 - a) is 0 contribute nothing (the reference divides by it).
 */
TPW_API int tpw_haversine_forward(int dtype, const void *x1, const void *x2, void *out,
                          int64_t B, int64_t N1, int64_t N2, tpw_stream_t stream);
TPW_API int tpw_haversine_backward(int dtype, const void *grad, const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                           int64_t B, int64_t N1, int64_t N2, tpw_stream_t stream);

/* ---- directed Hausdorff ---------------------------------------------------------------------- */

/*
 * x1 [B,N1,M1,D], x2 [B,N2,M2,D]  ->  out [B,N1,N2] = sqrt(max_m min_n |x1[m]-x2[n]|^2),
 * idx1/idx2 int64 [B,N1,N2] = the attaining m and n.  The [M1,M2] matrix is never written:
 * each thread keeps one x1 point and streams the x2 cloud through shared memory, row minima
 * are combined with warp shuffles and one 64-bit atomicMax per warp.
 * Tie rule of the reference loop: n = first n reaching the row minimum, m = LAST m whose
 * row minimum equals the maximum.  order1/order2 (int64 [B,M1] / [B,M2], may be NULL) give
 * each point's visiting position when the caller shuffles; ties then follow visiting order.
 * `scratch` holds tpw_hausdorff_scratch_bytes() bytes (8 per set pair plus 8 per x1 point of every set
 * pair), 8-byte aligned, and needs no initialisation.  float64 clouds of up to 16 coordinates keep every
 * row's exact minimum there and scan them once per set pair (TPW_HAUSDORFF_PLAIN_F64=1, or scratch ==
 * NULL, selects the one-CTA-per-pair kernel instead; same bits).  For float32 the hot loop forms the squared distance with fused multiply-adds
 * (7 operations per point pair) and stores every row's approximate minimum there; the finishing kernel
 * re-evaluates the few rows that can hold the maximum with separately rounded multiply and add, the
 * arithmetic of the reference's CPU loop (OPS/cpu/hausdorff_kernel.cpp:30-33), so values and indices are
 * bit-identical to evaluating every point pair that way (TPW_HAUSDORFF_EXACT_LOOP=1 does exactly that).
 * Replaces OPS/cuda/hausdorff_kernel.cu:16-104,107-195.
 */
TPW_API int64_t tpw_hausdorff_scratch_bytes(int64_t B, int64_t N1, int64_t N2, int64_t M1);
TPW_API int tpw_hausdorff_forward(int dtype, const void *x1, const void *x2,
                          const int64_t *order1, const int64_t *order2,
                          void *out, int64_t *idx1, int64_t *idx2, void *scratch,
                          int64_t B, int64_t N1, int64_t N2, int64_t M1, int64_t M2, int64_t D,
                          tpw_stream_t stream);

/*
 * grad_x1[b,i,m*,:] += g*(x1[m*]-x2[n*])/out, grad_x2[b,j,n*,:] -= same; the call zero-fills
 * both gradients first.  Replaces OPS/cuda/hausdorff_kernel.cu:198-246 (the reference re-runs
 * the forward inside its backward, :283-321; here the caller passes the saved forward results).
 */
TPW_API int tpw_hausdorff_backward(int dtype, const void *grad, const void *out,
                           const int64_t *idx1, const int64_t *idx2,
                           const void *x1, const void *x2, void *grad_x1, void *grad_x2,
                           int64_t B, int64_t N1, int64_t N2, int64_t M1, int64_t M2, int64_t D,
                           tpw_stream_t stream);

/*
 * tpw_hausdorff_forward for callers that cannot hand over scratch memory because they are not
 * allowed to allocate when the call is made -- a process that gave the whole GPU to its own pool
 * at start-up, a plug-in host that forbids allocation in its compute callback, a loop that cannot
 * take the device-wide stall an allocation may cause.  Same inputs, outputs and results as
 * tpw_hausdorff_forward, no scratch argument: the 8-byte key per set pair lives in a fixed
 * array inside the library's device image (tpw_hausdorff_static_max_pairs() * 8 bytes = 512 KiB,
 * held by every GPU that loads the library until the process exits).  After a first call on the
 * device, a call performs no allocation of any kind.  Because there is no room for per-row minima
 * the hot loop evaluates every point pair in the reference's separately rounded arithmetic; the
 * results are bit-identical to tpw_hausdorff_forward.
 *   - Limit: B*N1*N2 <= tpw_hausdorff_static_max_pairs() (65536); larger problems are refused
 *     with TPW_ERR_INVALID and a message, nothing is launched.
 *   - The first call on each device looks up the array's device address (a host-side query, not
 *     a stream operation).  Under the runtime's lazy loading that lookup may load this library's
 *     device image on the device -- memory for the image, the array included, and an implicit
 *     synchronisation -- so make one warm-up call per device at start-up, outside any stream capture
 *     and before the region in which nothing may allocate; the guarantee holds from then on.
 *   - The looked-up address is cached per device ordinal; cudaDeviceReset invalidates it, and a
 *     host that resets a device must not call into this library on that device again.
 *   - All calls on a device share the one array; the part a call uses is cleared on `stream`
 *     before its kernels run, but two calls whose kernels may overlap on the GPU (different
 *     streams, or different host threads) would race on it: keep them on one stream or serialise.
 * This entry point has no counterpart in the reference (whose wrappers always allocate).
 */
TPW_API int64_t tpw_hausdorff_static_max_pairs(void);
TPW_API int tpw_hausdorff_forward_static(int dtype, const void *x1, const void *x2,
                                         const int64_t *order1, const int64_t *order2,
                                         void *out, int64_t *idx1, int64_t *idx2,
                                         int64_t B, int64_t N1, int64_t N2, int64_t M1, int64_t M2, int64_t D,
                                         tpw_stream_t stream);

/* ---- element-wise safe divide ---------------------------------------------------------------- */

enum tpw_prf_div_mode { TPW_PRF_ZERO = 0, TPW_PRF_IDENTITY = 1 };

/* out = y != 0 ? x/y : (mode == ZERO ? 0 : x).  Replaces OPS/cuda/prf_div_kernel.cu:24-74. */
TPW_API int tpw_prf_div_forward(int dtype, int mode, const void *x, const void *y, void *out,
                        int64_t n, tpw_stream_t stream);
/* grad_x = y != 0 ? g/y : (IDENTITY ? g : 0); grad_y = y != 0 ? -grad_x*x/y : 0.
   Replaces OPS/cuda/prf_div_kernel.cu:315-366. Either output may be NULL. */
TPW_API int tpw_prf_div_backward(int dtype, int mode, const void *grad, const void *x, const void *y,
                         void *grad_x, void *grad_y, int64_t n, tpw_stream_t stream);

/* ---- measured issue peaks (roofline denominators for the CUDA-core kernels) -------------------- */

/*
 * Runs a register-only microbenchmark on the current device, synchronises, and reports the
 * sustained rate in operations per second: kind 0 = fp32 FMA lane-operations (scalar FFMA),
 * 1 = fp32 FMA lane-operations issued as packed fma.rn.f32x2, 2 = 32-bit POPC lane-operations,
 * 3 = fp32 additions, 4 = fp32 multiplications, 5 = the instruction mix of the p = 3 tiles (subtract,
 * d * |d|, fused multiply-add: three lane-operations per element), 6 = the same three results from
 * fused multiply-adds only, 7 = fp32 compares into a register, 8 = fp32 maxima, 9 = 32-bit integer additions.
 * No counterpart in the reference.
 */
TPW_API int tpw_measure_issue_peak(int kind, double *ops_per_second);

#ifdef __cplusplus
}
#endif
#endif /* TPW_B200_H */
