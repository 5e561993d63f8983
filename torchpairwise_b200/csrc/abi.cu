// Library plumbing of the C ABI: versioning, thread-local error text, the device status word,
// tensor-map encoding through the driver entry point, and the issue-rate microbenchmarks that
// give the CUDA-core kernels their roofline denominators.
#include "common.cuh"

#include <atomic>

#include <mutex>
#include <stdlib.h>
#include <string.h>

namespace tpw {

static thread_local char t_error[512] = {0};

char *error_buffer() { return t_error; }

void clear_error() { t_error[0] = 0; }

int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    return status;
}

__device__ int g_device_status_word = 0;

static const int kMaxDevices = 64;

// The per-device caches below are read and written from any host thread: atomic slots, and a value that every
// thread computes identically, so a race only repeats the lookup.  A cudaDeviceReset invalidates device addresses;
// a host that resets a device must not keep using this library on it in the same process.
int *device_status_ptr() {
    static std::atomic<int *> cache[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    int *p = cache[dev].load(std::memory_order_acquire);
    if (!p) {
        if (cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_device_status_word) != cudaSuccess) return nullptr;
        cache[dev].store(p, std::memory_order_release);
    }
    return p;
}

bool tma_disabled() {
    static const bool off = [] {
        const char *v = getenv("TPW_DISABLE_TMA");
        return v && v[0] && v[0] != '0';
    }();
    return off;
}

int sm_count() {
    static std::atomic<int> cache[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (!n) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

static encode_tiled_fn resolve_encode_tiled() {
    static encode_tiled_fn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<encode_tiled_fn>(p);
    });
    return fn;
}

static int encode_map_3d(CUtensorMap *map, const void *base, int elem_bytes,
                         uint64_t dim0, uint64_t dim1, uint64_t dim2,
                         uint32_t box0, uint32_t box1, bool swizzle128, CUtensorMapSwizzle swizzle);

int make_tensor_map_3d(CUtensorMap *map, const void *base, int elem_bytes,
                       uint64_t dim0, uint64_t dim1, uint64_t dim2,
                       uint32_t box0, uint32_t box1, bool swizzle128) {
    return encode_map_3d(map, base, elem_bytes, dim0, dim1, dim2, box0, box1, swizzle128,
                         swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE);
}

int make_tensor_map_3d_atom32(CUtensorMap *map, const void *base, int elem_bytes,
                              uint64_t dim0, uint64_t dim1, uint64_t dim2, uint32_t box0, uint32_t box1) {
    return encode_map_3d(map, base, elem_bytes, dim0, dim1, dim2, box0, box1, true, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B);
}

static int encode_map_3d(CUtensorMap *map, const void *base, int elem_bytes,
                         uint64_t dim0, uint64_t dim1, uint64_t dim2,
                         uint32_t box0, uint32_t box1, bool swizzle128, CUtensorMapSwizzle swizzle) {
    encode_tiled_fn encode = resolve_encode_tiled();
    if (!encode) return fail(TPW_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    // The encoder is a driver call and needs a context bound to the calling thread.  A thread that
    // has only ever been handed tensors (an autograd worker, say) may not have one yet: binding the
    // runtime's current device does it.  Once per thread and device.
    {
        static thread_local int bound_device = -1;
        int dev = 0;
        TPW_CUDA_OK(cudaGetDevice(&dev));
        if (bound_device != dev) {
            TPW_CUDA_OK(cudaSetDevice(dev));
            TPW_CUDA_OK(cudaFree(nullptr));
            bound_device = dev;
        }
    }
    CUtensorMapDataType dt;
    switch (elem_bytes) {
        case 1: dt = CU_TENSOR_MAP_DATA_TYPE_UINT8; break;
        case 2: dt = CU_TENSOR_MAP_DATA_TYPE_UINT16; break;
        case 4: dt = CU_TENSOR_MAP_DATA_TYPE_UINT32; break;
        case 8: dt = CU_TENSOR_MAP_DATA_TYPE_UINT64; break;
        default: return fail(TPW_ERR_INVALID, "tensor map: unsupported element size %d", elem_bytes);
    }
    if (!aligned16(base)) return fail(TPW_ERR_INVALID, "tensor map: base address is not 16-byte aligned");
    if ((dim0 * elem_bytes) % 16 != 0) return fail(TPW_ERR_INVALID, "tensor map: row pitch is not a multiple of 16 bytes");
    if (swizzle128 && box0 * (uint32_t)elem_bytes != 128)
        return fail(TPW_ERR_INVALID, "tensor map: a 128-byte swizzled box must span 128 bytes");
    cuuint64_t dims[3] = {dim0, dim1 ? dim1 : 1, dim2 ? dim2 : 1};
    cuuint64_t strides[2] = {dim0 * (uint64_t)elem_bytes, dim0 * dims[1] * (uint64_t)elem_bytes};
    cuuint32_t box[3] = {box0, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(TPW_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return TPW_OK;
}

// ---- issue-rate microbenchmarks ------------------------------------------------------------------
template <int KIND>
__global__ void __launch_bounds__(256) issue_peak_kernel(float *sink, int iters, float seed) {
    float a[16];
    uint32_t u[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        a[i] = seed + (float)(threadIdx.x + i);
        u[i] = __float_as_uint(a[i]) * 2654435761u;
    }
    const float m = 1.0000001f, c = 1e-9f;
    for (int it = 0; it < iters; ++it) {
        if (KIND == 0) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) a[i] = fmaf(a[i], m, c);
        } else if (KIND == 1) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    uint64_t v, mm, cc;
                    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(a[i]), "f"(a[i + 1]));
                    asm("mov.b64 %0, {%1, %1};" : "=l"(mm) : "f"(m));
                    asm("mov.b64 %0, {%1, %1};" : "=l"(cc) : "f"(c));
                    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(v) : "l"(v), "l"(mm), "l"(cc));
                    asm("mov.b64 {%0, %1}, %2;" : "=f"(a[i]), "=f"(a[i + 1]) : "l"(v));
                }
        } else if (KIND == 2) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) u[i] = __popc(u[i]) + u[(i + 1) & 15];
        } else if (KIND == 3) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) asm volatile("add.rn.f32 %0, %0, %1;" : "+f"(a[i]) : "f"(c));
        } else if (KIND == 4) {
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) asm volatile("mul.rn.f32 %0, %0, %1;" : "+f"(a[i]) : "f"(m));
        } else if (KIND == 5) {
            // the instruction mix of the p = 3 tiles: subtract, d * |d|, fused multiply-add (3 operations per element)
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; i += 3) {
                    float d, t;
                    asm volatile("sub.rn.f32 %0, %1, %2;" : "=f"(d) : "f"(a[i]), "f"(m));
                    asm volatile("mul.rn.f32 %0, %1, %2;" : "=f"(t) : "f"(d), "f"(fabsf(d)));
                    asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(a[i]) : "f"(t), "f"(c));
                }
        } else if (KIND == 7) {
            // fp32 compare into a register (1.0 / 0.0)
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) asm volatile("set.eq.f32.f32 %0, %0, %1;" : "+f"(a[i]) : "f"(c));
        } else if (KIND == 8) {
            // fp32 maximum
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) asm volatile("max.f32 %0, %0, %1;" : "+f"(a[i]) : "f"(a[(i + 1) & 15]));
        } else if (KIND == 9) {
            // 32-bit integer addition
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; ++i) asm volatile("add.u32 %0, %0, %1;" : "+r"(u[i]) : "r"(u[(i + 1) & 15]));
        } else {
            // the same three results from fused multiply-adds only
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
                for (int i = 0; i < 16; i += 3) {
                    float d, t;
                    asm volatile("fma.rn.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(m), "f"(-1.0f), "f"(a[i]));
                    asm volatile("fma.rn.f32 %0, %1, %2, %3;" : "=f"(t) : "f"(d), "f"(fabsf(d)), "f"(0.0f));
                    asm volatile("fma.rn.f32 %0, %1, %2, %0;" : "+f"(a[i]) : "f"(t), "f"(c));
                }
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) s += a[i] + (float)u[i];
    if (s == 123.456f) sink[0] = s; // never true in practice; keeps the chains alive
}

// Waits on an mbarrier that nothing ever completes, with a caller-chosen budget, then records
// the give-up in the status word exactly as the production kernels do.
__global__ void wait_selftest_kernel(int *status, unsigned long long budget_ns) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        mbar_init_fence();
    }
    __syncthreads();
    int failed = 0;
    const uint64_t t0 = globaltimer_ns();
    bool done = false;
    for (uint32_t it = 0; it < (1u << 26) && !done; ++it) {
        if (mbar_try_wait(&bar, 0)) done = true;
        else if ((it & 15u) == 15u && globaltimer_ns() - t0 > budget_ns) break;
    }
    if (!done) failed = 1;
    if (__syncthreads_or(failed)) {
        if (threadIdx.x == 0 && status) atomicCAS(status, 0, (15 << 16) | 1);
        return;
    }
}

} // namespace tpw

extern "C" {

int tpw_abi_version(void) { return TPW_ABI_VERSION; }
int tpw_cuda_version(void) { return CUDART_VERSION; }
const char *tpw_cuda_arch_flags(void) { return "sm_100a"; }
const char *tpw_last_error(void) { return tpw::error_buffer(); }

int tpw_device_status(int *code, tpw_stream_t stream) {
    TPW_CHECK_ARG(code != nullptr, "tpw_device_status: code is NULL");
    int *p = tpw::device_status_ptr();
    if (!p) return tpw::fail(TPW_ERR_CUDA, "tpw_device_status: cannot resolve the device status word");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    TPW_CUDA_OK(cudaStreamSynchronize(s));
    TPW_CUDA_OK(cudaMemcpy(code, p, sizeof(int), cudaMemcpyDeviceToHost));
    if (*code != 0) TPW_CUDA_OK(cudaMemset(p, 0, sizeof(int)));
    return TPW_OK;
}

int tpw_selftest_bounded_wait(int budget_ms, tpw_stream_t stream) {
    TPW_CHECK_ARG(budget_ms >= 1 && budget_ms <= 1000, "tpw_selftest_bounded_wait: budget must be 1..1000 ms");
    int *p = tpw::device_status_ptr();
    if (!p) return tpw::fail(TPW_ERR_CUDA, "tpw_selftest_bounded_wait: cannot resolve the device status word");
    tpw::wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(p, (unsigned long long)budget_ms * 1000000ull);
    TPW_LAUNCH_OK("wait_selftest_kernel");
    return TPW_OK;
}

int tpw_measure_issue_peak(int kind, double *ops_per_second) {
    TPW_CHECK_ARG(ops_per_second != nullptr, "tpw_measure_issue_peak: output pointer is NULL");
    TPW_CHECK_ARG(kind >= 0 && kind <= 9, "tpw_measure_issue_peak: kind must be 0 .. 9");
    int *sink_i = tpw::device_status_ptr();
    if (!sink_i) return tpw::fail(TPW_ERR_CUDA, "tpw_measure_issue_peak: no device");
    float *sink = reinterpret_cast<float *>(sink_i); // never written (see kernel)
    const int blocks = tpw::sm_count() * 8, threads = 256, iters = 4096;
    cudaEvent_t e0, e1;
    TPW_CUDA_OK(cudaEventCreate(&e0));
    TPW_CUDA_OK(cudaEventCreate(&e1));
    float best_ms = 1e30f;
    for (int rep = 0; rep < 4; ++rep) {
        cudaEventRecord(e0, 0);
        if (kind == 0) tpw::issue_peak_kernel<0><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 1) tpw::issue_peak_kernel<1><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 2) tpw::issue_peak_kernel<2><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 3) tpw::issue_peak_kernel<3><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 4) tpw::issue_peak_kernel<4><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 5) tpw::issue_peak_kernel<5><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 6) tpw::issue_peak_kernel<6><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 7) tpw::issue_peak_kernel<7><<<blocks, threads>>>(sink, iters, 1.0f);
        else if (kind == 8) tpw::issue_peak_kernel<8><<<blocks, threads>>>(sink, iters, 1.0f);
        else tpw::issue_peak_kernel<9><<<blocks, threads>>>(sink, iters, 1.0f);
        cudaEventRecord(e1, 0);
        cudaError_t e = cudaEventSynchronize(e1);
        if (e != cudaSuccess) {
            cudaEventDestroy(e0);
            cudaEventDestroy(e1);
            return tpw::fail(TPW_ERR_CUDA, "issue peak kernel failed: %s", cudaGetErrorString(e));
        }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        if (rep > 0 && ms < best_ms) best_ms = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    // 4 x 16 operations per iteration; the two mixes run 4 x 6 chains of three operations each
    const double ops = (double)blocks * threads * (double)iters * (kind == 5 || kind == 6 ? 72.0 : 64.0);
    *ops_per_second = ops / (best_ms * 1e-3);
    return TPW_OK;
}

} // extern "C"
