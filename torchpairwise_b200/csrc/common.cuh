// Shared host/device helpers of the sm_100a pairwise kernels: error plumbing, launch checks,
// and thin wrappers over the PTX used for TMA (cp.async.bulk.tensor) and mbarriers.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/tpw_b200.h"

namespace tpw {

// ---- host-side error text (thread local) ------------------------------------------------------
char *error_buffer();                       // 512 bytes, thread local
int fail(int status, const char *fmt, ...); // formats into error_buffer(), returns status
void clear_error();

#define TPW_CHECK_ARG(cond, ...)                                  \
    do {                                                          \
        if (!(cond)) return ::tpw::fail(TPW_ERR_INVALID, __VA_ARGS__); \
    } while (0)

#define TPW_CUDA_OK(expr)                                                                     \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess)                                                                \
            return ::tpw::fail(TPW_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

#define TPW_LAUNCH_OK(name)                                                                      \
    do {                                                                                         \
        cudaError_t _e = cudaGetLastError();                                                     \
        if (_e != cudaSuccess)                                                                   \
            return ::tpw::fail(TPW_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(_e)); \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Device status word shared by all kernels of the library (one per device that loads it).
// Codes: 0 = fine, otherwise (kernel id << 16) | site.  Kernels receive its device address
// as an argument; NULL is returned when the address cannot be resolved.
int *device_status_ptr();

// True when the environment variable TPW_DISABLE_TMA is set to a non-zero value: every kernel then
// stages its tiles with guarded plain loads (a debugging aid; results are bit-identical).
bool tma_disabled();

// Number of SMs of the current device (cached per device).
int sm_count();

// Builds a tiled tensor map over a dense row-major [dim2, dim1, dim0] tensor (dim0 innermost).
// elem_bytes is 1, 2, 4 or 8; swizzle128 selects CU_TENSOR_MAP_SWIZZLE_128B (inner box must span
// exactly 128 bytes) or no swizzle.  Returns a tpw_status.
int make_tensor_map_3d(CUtensorMap *map, const void *base, int elem_bytes,
                       uint64_t dim0, uint64_t dim1, uint64_t dim2,
                       uint32_t box0, uint32_t box1, bool swizzle128);
// Same with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B: 128-byte rows whose 32-byte groups are permuted by
// the row index modulo 4, the shared-memory layout tcgen05 expects for MN-major 32-bit operands.
int make_tensor_map_3d_atom32(CUtensorMap *map, const void *base, int elem_bytes,
                              uint64_t dim0, uint64_t dim1, uint64_t dim2, uint32_t box0, uint32_t box1);

// lp_small_d.cu: float32 L_p forward for few features (output-bound shapes)
bool lp_small_d_eligible(long long N1, long long N2, long long D, double p);
int lp_small_d_forward(const void *x1, const void *x2, void *out, long long B, long long N1, long long N2, long long D,
                       double p, double out_exponent, cudaStream_t s);
int lp_small_d_mask(const void *x1, const void *x2, unsigned char *mask, long long B, long long N1, long long N2, long long D,
                    double p, double out_exponent, double radius, cudaStream_t s);
bool lp_small_d_rowmin_eligible(long long N1, long long N2, long long D, double p);
int lp_small_d_rowmin(const void *x1, const void *x2, unsigned long long *keys, long long B, long long N1, long long N2, long long D,
                      double p, double out_exponent, cudaStream_t s);

// lp_backward_onepass.cu: both gradients of an L_p reduction from one walk over the pairs (float32).  The query
// returns 0 where that kernel does not apply.
long long lp_backward_onepass_scratch_bytes(int mode, long long B, long long N1, long long N2, long long D, double p);
int lp_backward_onepass(int mode, const void *grad, const void *aux, const void *x1, const void *x2, const void *w,
                        void *grad_x1, void *grad_x2, long long B, long long N1, long long N2, long long D, double p,
                        void *scratch, long long scratch_bytes, cudaStream_t stream);

// lp_backward.cu: the dense cdist backward for p = +inf (float32), run only when *only_if > above on the device
int lp_backward_cdist_inf_if(const unsigned long long *only_if, unsigned long long above, const void *grad, const void *out, const void *x1, const void *x2,
                             void *grad_x1, void *grad_x2, long long B, long long N1, long long N2, long long D,
                             cudaStream_t stream);

// |d|^q in the float kernels.  spec = mode | m << 2 (uniform over a launch): mode 0 is the general
// exp2(q log2 a) (two MUFU operations per element); mode 1 is q = m + 1/2, one approximate square
// root (MUFU.SQRT, 1 ulp) times a^m; mode 2 is the integer q = m as repeated multiplication.
// The special modes cover q <= 4.5 and are both faster and more accurate than the general form.
inline int make_pow_spec(double q) {
    const double fl = floor(q);
    if (q == fl && q >= 1.0 && q <= 4.0) return 2 | ((int)q << 2);
    if (q - fl == 0.5 && fl >= 0.0 && fl <= 4.0) return 1 | ((int)fl << 2);
    return 0;
}

#ifdef __CUDACC__
__device__ __forceinline__ float pow_abs_spec(float a, float q, int spec) {
    const int mode = spec & 3, m = spec >> 2;
    if (mode == 0) return a == 0.f ? 0.f : exp2f(q * __log2f(a));
    float r = 1.f;
    if (mode == 1) asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(a));
    if (m >= 1) r *= a;
    if (m >= 2) r *= a;
    if (m >= 3) r *= a;
    if (m >= 4) r *= a;
    return r;
}
__device__ __forceinline__ double pow_abs_spec(double a, double q, int) { return a == 0.0 ? 0.0 : pow(a, q); }
// 1 / v for one term of a sum, 0 where the term is to be skipped (v == 0).  float: the bare MUFU
// reciprocal (1 ulp, flush-to-zero), so denominators below the smallest normal number count as zero;
// double: the exact divide.
__device__ __forceinline__ float rcp_or_zero(float v) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return fabsf(v) >= 1.17549435e-38f ? r : 0.f;
}
__device__ __forceinline__ double rcp_or_zero(double v) { return v != 0.0 ? 1.0 / v : 0.0; }

// ---- device-side PTX wrappers -----------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Makes freshly initialised mbarriers visible to the async (TMA / tensor-core) proxy.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait: gives up (returns false) once about two seconds of wall time have passed without
// the phase completing, or after `limit` polls, whichever comes first, so a lost completion can
// never hang the GPU.
constexpr uint64_t kWaitBudgetNs = 2000000000ull;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 26)) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = globaltimer_ns();
    for (uint32_t it = 0; it < limit; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 255u && globaltimer_ns() - t0 > kWaitBudgetNs) return false;
    }
    return false;
}

__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// 3-D tiled TMA load global -> shared, completion on an mbarrier.  c0 is the innermost
// coordinate and must keep c0 * element size a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_3d(void *dst, const CUtensorMap *map, uint64_t *bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_u32(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(bar))
        : "memory");
}
// 3-D tiled TMA store shared -> global as a bulk async-group (the tensor map clips what lies outside the tensor; c0
// must keep c0 * element size a multiple of 16 bytes and no coordinate may be negative), its commit, and the wait until
// every committed store has read its shared-memory source.
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *map, const void *src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
                     reinterpret_cast<uint64_t>(map)),
                 "r"(c0), "r"(c1), "r"(c2), "r"(smem_u32(src))
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a tile whose rows are 128
// bytes and which was written with the 128-byte swizzle (tile base 1024-byte aligned).
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
    return row * 128u + ((chunk ^ (row & 7u)) << 4);
}
#endif // __CUDACC__

} // namespace tpw
