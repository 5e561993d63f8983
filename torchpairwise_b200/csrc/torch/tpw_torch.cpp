// C++ host layer: the reference's operator schemas (namespace `torchpairwise`) bound to the C ABI.
//
// Loading this library makes `torch.ops.torchpairwise.<op>` run the sm_100a kernels for CUDA tensors.
// It works in two modes:
//   * next to the reference extension (loaded first): the schemas already exist, the reference keeps
//     serving CPU tensors, and the AutogradCUDA kernels registered here take over CUDA tensors --
//     including the public ops that the reference implements with at::cdist / matmul
//     (OPS/pairwise_metrics.cpp:30,48,121,167,203,305) and the string dispatcher `cdist`
//     (OPS/cpdist.cpp:149-231), whose body calls the reference functors directly;
//   * stand-alone: the schemas are defined here with the reference's exact strings
//     (OPS/pairwise_metrics.h:73-425, OPS/ppminkowski.cpp:31-38, OPS/wminkowski.cpp:33-40,
//     OPS/hausdorff.cpp:34-39, OPS/pairwise_binary.cpp:151-159, OPS/cpdist.cpp:248-251).
// Each body does what the reference's kernel wrappers do -- checks, contiguous(), leading batch
// dimension, allocation, current stream -- and then calls the C ABI.  Nothing here computes on the
// CPU; a CPU tensor reaching one of these kernels is an error.
#include <ATen/ATen.h>
#include <ATen/core/dispatch/Dispatcher.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <c10/util/Logging.h>
#include <nvtx3/nvToolsExt.h>
#include <torch/autograd.h>
#include <torch/library.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <limits>

#include "../../../include/tpw_b200.h"

namespace {

using at::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;
using OptTensor = c10::optional<Tensor>;

#define TPW_CALL(expr)                                                        \
    do {                                                                      \
        int status_ = (expr);                                                 \
        TORCH_CHECK(status_ == TPW_OK, #expr " failed: ", tpw_last_error());  \
    } while (0)

// Every public operator logs the reference's API-usage string once (OPS/pairwise_metrics.cpp:27,36,45,...;
// OPS/cpdist.cpp:160; OPS/neighbors.cpp:21,48) and brackets its body with an NVTX range, so that a timeline shows the
// operator name around its kernels.  The ranges cost nothing when no profiler is attached.
struct NvtxRange {
    explicit NvtxRange(const char *name) { nvtxRangePushA(name); }
    ~NvtxRange() { nvtxRangePop(); }
    NvtxRange(const NvtxRange &) = delete;
    NvtxRange &operator=(const NvtxRange &) = delete;
};
#define TPW_OP(file, name)                                            \
    C10_LOG_API_USAGE_ONCE("torchpairwise.csrc.ops." file "." name);  \
    NvtxRange nvtx_range_("torchpairwise::" name)

int code_of(const Tensor &t) { return t.scalar_type() == at::kDouble ? TPW_F64 : TPW_F32; }
tpw_stream_t stream_of(const Tensor &t) { return c10::cuda::getCurrentCUDAStream(t.get_device()).stream(); }

at::ScalarType compute_type(at::ScalarType t) {
    if (t == at::kHalf || t == at::kBFloat16) return at::kFloat;
    TORCH_CHECK(t == at::kFloat || t == at::kDouble, "expected a floating point tensor, got ", t);
    return t;
}

void require_cuda(const Tensor &t) {
    TORCH_CHECK(t.is_cuda(), "torchpairwise (B200 build) runs on CUDA tensors only (no CPU path); got a tensor on ", t.device());
}

// OPS/pairwise_metrics.h:10-67
std::pair<Tensor, Tensor> check_pairwise_inputs(const char *name, const Tensor &x1, const OptTensor &x2,
                                                bool boolean = false, bool sets = false) {
    const int64_t lo = sets ? 3 : 2;
    const bool unbatched = x1.dim() == lo;
    TORCH_CHECK(unbatched || x1.dim() == lo + 1, "x1 must be ", lo, "D tensor (unbatched) or ", lo + 1, "D tensor (batched)");
    if (x2.has_value()) {
        const Tensor &b = x2.value();
        TORCH_CHECK(unbatched || b.dim() == lo + 1, "x2 must be ", lo, "D tensor (unbatched) or ", lo + 1, "D tensor (batched)");
        const int64_t f = unbatched ? lo - 1 : lo;
        TORCH_CHECK(b.dim() > f && x1.size(f) == b.size(f), "x1 and x2 must have same number of features. Got: x1.size(", f,
                    ")=", x1.size(f), ", x2.size(", f, ")=", b.dim() > f ? b.size(f) : -1);
    }
    if (boolean) {
        if (x1.scalar_type() != at::kBool || (x2.has_value() && x2->scalar_type() != at::kBool))
            TORCH_WARN("Data was converted to ", at::kBool, " for metric ", name);
        Tensor a = x1.to(at::kBool);
        return {a, x2.has_value() ? x2->to(at::kBool) : a};
    }
    return {x1, x2.has_value() ? x2.value() : x1};
}

struct Prepared {
    Tensor a, b;
    bool unbatched;
    int64_t B, N1, N2, D;
};

// contiguous() + leading batch dimension (e.g. OPS/cuda/ppminkowski_kernel.cu:70-90)
Prepared prepare(const Tensor &x1, const Tensor &x2, at::ScalarType dt) {
    require_cuda(x1);
    require_cuda(x2);
    TORCH_CHECK(x1.get_device() == x2.get_device(), "Expected all tensors to be on the same device");
    const bool unbatched = x1.dim() == 2;
    TORCH_CHECK(unbatched || x1.dim() == 3, "x1 must be 2-D (unbatched) or 3-D (batched) tensor.");
    TORCH_CHECK(x2.dim() == x1.dim(), "x2 must be 2-D (unbatched) or 3-D (batched) tensor.");
    TORCH_CHECK(unbatched || x1.size(0) == x2.size(0), "batch_size of x1 and x2 do not match.");
    TORCH_CHECK(x1.size(-1) == x2.size(-1), "feature dimension of x1 and x2 do not match.");
    Prepared p;
    p.a = x1.to(dt).contiguous();
    p.b = x2.is_same(x1) ? p.a : x2.to(dt).contiguous();
    p.unbatched = unbatched;
    if (unbatched) {
        p.a = p.a.unsqueeze(0);
        p.b = p.b.unsqueeze(0);
    }
    p.B = p.a.size(0); p.N1 = p.a.size(1); p.N2 = p.b.size(1); p.D = p.a.size(2);
    return p;
}

Tensor finish(Tensor out, bool unbatched, at::ScalarType dt) {
    if (unbatched) out = out.squeeze(0);
    return out.scalar_type() == dt ? out : out.to(dt);
}

Tensor lp_forward(const Prepared &p, const Tensor *w, double pw, double exponent) {
    Tensor out = at::empty({p.B, p.N1, p.N2}, p.a.options());
    if (p.D == 0) return out.zero_();
    TPW_CALL(tpw_lp_forward(code_of(p.a), p.a.data_ptr(), p.b.data_ptr(), w ? w->data_ptr() : nullptr, out.data_ptr(),
                            p.B, p.N1, p.N2, p.D, pw, exponent, stream_of(p.a)));
    return out;
}

Tensor dot_forward(const Prepared &p, int epilogue, int engine) {
    Tensor out = at::empty({p.B, p.N1, p.N2}, p.a.options());
    if (p.D == 0) return out.fill_(epilogue == TPW_DOT_COSINE_DIST || epilogue == TPW_DOT_ONE_MINUS_SIM ? 1.0 : 0.0);
    const int64_t bytes = tpw_dot_metric_scratch_bytes(code_of(p.a), engine, p.B, p.N1, p.N2, p.D);
    Tensor scratch;
    if (bytes > 0) scratch = at::empty({bytes}, p.a.options().dtype(at::kByte));
    TPW_CALL(tpw_dot_metric_forward_ws(code_of(p.a), epilogue, engine, p.a.data_ptr(), p.b.data_ptr(), out.data_ptr(),
                                       bytes > 0 ? scratch.data_ptr() : nullptr, bytes, p.B, p.N1, p.N2, p.D, stream_of(p.a)));
    return out;
}

bool tensor_engine_selected(const Prepared &p) {
    return p.a.scalar_type() == at::kFloat && p.D > 0 &&
           tpw_dot_metric_scratch_bytes(TPW_F32, TPW_ENGINE_AUTO, p.B, p.N1, p.N2, p.D) > 0;
}

// Backward of the p = 2 metrics and the plain gradient products: tensor-core contractions when the
// engine rule of tpw_dot_backward_ws picks them (large float32 problems), the CUDA-core kernel
// otherwise.  The split copies take about 8 bytes per element of grad; above TPW_BWD_SCRATCH_GB
// (default 8) the work is cut into groups of batches, or row blocks of one batch whose grad_x2
// contributions are added in block order.
// With `cosine` set (epilogue >= 0, the two norm vectors) the call is the whole cosine-family backward,
// tpw_cosine_backward_ws, with g the upstream gradient and aux the saved forward result; it returns
// false without doing anything when the engine rule keeps the problem on the CUDA cores.
// tpw_lp_backward, through the one-pass kernel (both gradients from one walk over the pairs) where the library offers it
void lp_backward_call(int code, int mode, const Tensor &g, const void *aux, const Tensor &a, const Tensor &b, const void *w,
                      Tensor &g1, Tensor &g2, int64_t B, int64_t N1, int64_t N2, int64_t D, double p) {
    const int64_t bytes = tpw_lp_backward_scratch_bytes(code, mode, B, N1, N2, D, p);
    if (bytes <= 0) {
        TPW_CALL(tpw_lp_backward(code, mode, g.data_ptr(), aux, a.data_ptr(), b.data_ptr(), w, g1.data_ptr(), g2.data_ptr(),
                                 B, N1, N2, D, p, stream_of(a)));
        return;
    }
    Tensor scratch = at::empty({bytes}, a.options().dtype(at::kByte));
    TPW_CALL(tpw_lp_backward_ws(code, mode, g.data_ptr(), aux, a.data_ptr(), b.data_ptr(), w, g1.data_ptr(), g2.data_ptr(),
                                B, N1, N2, D, p, scratch.data_ptr(), bytes, stream_of(a)));
}

struct CosineArgs {
    int epilogue = -1;
    const Tensor *n1 = nullptr, *n2 = nullptr;
};

bool dense_backward(int mode, const Tensor &g, const Tensor *aux, const Tensor &a, const Tensor &b, Tensor &g1, Tensor &g2,
                    const CosineArgs &cosine = CosineArgs()) {
    const int64_t B = a.size(0), N1 = a.size(1), N2 = b.size(1), D = a.size(2);
    const int code = code_of(a);
    auto st = stream_of(a);
    if (tpw_dot_backward_scratch_bytes(code, mode, TPW_ENGINE_AUTO, B, N1, N2, D) <= 0) {
        if (cosine.epilogue >= 0) return false;
        lp_backward_call(code, mode, g, aux ? aux->data_ptr() : nullptr, a, b, nullptr, g1, g2, B, N1, N2, D, 2.0);
        return true;
    }
    const int eng = TPW_ENGINE_TCGEN05_TF32X3;
    const char *env = std::getenv("TPW_BWD_SCRATCH_GB");
    const int64_t cap = static_cast<int64_t>((env ? std::atof(env) : 8.0) * 1073741824.0);
    const int64_t per_batch = tpw_dot_backward_scratch_bytes(code, mode, eng, 1, N1, N2, D);
    int64_t nb = 1, rows = N1;
    if (per_batch <= cap) {
        nb = std::max<int64_t>(1, std::min<int64_t>(B, cap / per_batch));
    } else {
        while (rows > 256 && tpw_dot_backward_scratch_bytes(code, mode, eng, 1, rows, N2, D) > cap)
            rows = std::max<int64_t>(256, (rows / 2 + 255) / 256 * 256);
    }
    const int64_t bytes = tpw_dot_backward_scratch_bytes(code, mode, eng, nb, std::min(rows, N1), N2, D);
    Tensor scratch = at::empty({bytes}, a.options().dtype(at::kByte));
    Tensor part;
    for (int64_t b0 = 0; b0 < B; b0 += nb) {
        const int64_t bn = std::min(nb, B - b0);
        for (int64_t r0 = 0; r0 < N1; r0 += rows) {
            const int64_t rn = std::min(rows, N1 - r0);
            Tensor gv = g.narrow(0, b0, bn).narrow(1, r0, rn), av = a.narrow(0, b0, bn).narrow(1, r0, rn);
            Tensor g1v = g1.narrow(0, b0, bn).narrow(1, r0, rn), g2v = g2.narrow(0, b0, bn);
            if (r0 > 0) {
                if (!part.defined()) part = at::empty_like(g2v);
                g2v = part;
            }
            const void *auxp = aux ? aux->narrow(0, b0, bn).narrow(1, r0, rn).data_ptr() : nullptr;
            if (cosine.epilogue >= 0)
                TPW_CALL(tpw_cosine_backward_ws(cosine.epilogue, gv.data_ptr(), auxp, cosine.n1->narrow(0, b0, bn).narrow(1, r0, rn).data_ptr(),
                                                cosine.n2->narrow(0, b0, bn).data_ptr(), av.data_ptr(), b.narrow(0, b0, bn).data_ptr(),
                                                g1v.data_ptr(), g2v.data_ptr(), scratch.data_ptr(), bytes, bn, rn, N2, D, st));
            else
                TPW_CALL(tpw_dot_backward_ws(code, mode, eng, gv.data_ptr(), auxp, av.data_ptr(), b.narrow(0, b0, bn).data_ptr(),
                                             g1v.data_ptr(), g2v.data_ptr(), scratch.data_ptr(), bytes, bn, rn, N2, D, st));
            if (r0 > 0) g2.narrow(0, b0, bn).add_(part);
        }
    }
    return true;
}

Tensor cmp_reduce(const Tensor &a, const Tensor &b, int op, int red);

// ---- at::cdist as the reference's public ops call it -------------------------------------------------
struct CdistFn : torch::autograd::Function<CdistFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2, double p) {
        at::AutoDispatchBelowADInplaceOrView guard;
        TORCH_CHECK(p >= 0, "cdist only supports non-negative p values");
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype");
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out;
        if (p == 0) out = cmp_reduce(q.a, q.b, TPW_CMP_NE, TPW_RED_SUM).to(q.a.scalar_type());
        else if (std::isinf(p)) out = lp_forward(q, nullptr, p, 1.0);
        else if (p == 2 && tensor_engine_selected(q)) out = dot_forward(q, TPW_DOT_EUCLIDEAN, TPW_ENGINE_AUTO);
        else out = lp_forward(q, nullptr, p, 1.0 / p);
        ctx->save_for_backward({q.a, q.b, out});
        ctx->saved_data["p"] = p;
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const Tensor &a = s[0], &b = s[1], &out = s[2];
        const double p = ctx->saved_data["p"].toDouble();
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = go[0].to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        Tensor g1 = at::empty_like(a), g2 = at::empty_like(b);
        if (p == 0) { g1.zero_(); g2.zero_(); }
        else if (p == 2 && a.numel() > 0 && b.numel() > 0) dense_backward(TPW_LP_BWD_CDIST, g, &out, a, b, g1, g2);
        else if (std::isinf(p) && tpw_chebyshev_backward_scratch_bytes(code_of(a), a.size(0), a.size(1), b.size(1), a.size(2)) > 0) {
            // Chebyshev: find the attaining coordinate of every pair once, then scatter both gradients
            const int64_t bytes = tpw_chebyshev_backward_scratch_bytes(code_of(a), a.size(0), a.size(1), b.size(1), a.size(2));
            Tensor scratch = at::empty({bytes}, a.options().dtype(at::kByte));
            TPW_CALL(tpw_chebyshev_backward_ws(g.data_ptr(), out.data_ptr(), a.data_ptr(), b.data_ptr(), g1.data_ptr(), g2.data_ptr(),
                                               scratch.data_ptr(), bytes, a.size(0), a.size(1), b.size(1), a.size(2), stream_of(a)));
        }
        else lp_backward_call(code_of(a), TPW_LP_BWD_CDIST, g, out.data_ptr(), a, b, nullptr, g1, g2, a.size(0), a.size(1), b.size(1), a.size(2), p);
        return {finish(g1, ub, dt), finish(g2, ub, dt), Tensor()};
    }
};

// ---- _ppminkowski (OPS/autograd/ppminkowski_kernel.cpp:9-46) ------------------------------------------
struct PPMinkowskiFn : torch::autograd::Function<PPMinkowskiFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2, double p) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype (while checking arguments for _ppminkowski_forward)");
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out;
        if (p == 0) out = at::full({q.B, q.N1, q.N2}, static_cast<double>(q.D), q.a.options());
        else if (p == 2 && tensor_engine_selected(q)) out = dot_forward(q, TPW_DOT_SQEUCLIDEAN, TPW_ENGINE_AUTO);
        else out = lp_forward(q, nullptr, p, 1.0);
        ctx->save_for_backward({q.a, q.b});
        ctx->saved_data["p"] = p;
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static std::pair<Tensor, Tensor> raw_backward(const Tensor &grad, const Tensor &a, const Tensor &b, double p, bool ub) {
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = grad.to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        Tensor g1 = at::zeros_like(a), g2 = at::zeros_like(b);
        const int64_t B = a.size(0), N1 = a.size(1), N2 = b.size(1), D = a.size(2);
        if (p != 0 && B * N1 * N2 * D > 0) {
            if (std::isinf(p))
                TPW_CALL(tpw_lp_inf_backward(code_of(a), g.data_ptr(), a.data_ptr(), b.data_ptr(), nullptr, g1.data_ptr(), g2.data_ptr(),
                                             nullptr, B, N1, N2, D, p < 0, stream_of(a)));
            else if (p == 2)
                dense_backward(TPW_LP_BWD_PPMINKOWSKI, g, nullptr, a, b, g1, g2);
            else
                lp_backward_call(code_of(a), TPW_LP_BWD_PPMINKOWSKI, g, nullptr, a, b, nullptr, g1, g2, B, N1, N2, D, p);
        }
        return {g1, g2};
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        auto g = raw_backward(go[0], s[0], s[1], ctx->saved_data["p"].toDouble(), ub);
        return {finish(g.first, ub, dt), finish(g.second, ub, dt), Tensor()};
    }
};

// ---- _sqjensenshannon / jensenshannon_distances (OPS/autograd/sqjensenshannon_kernel.cpp, OPS/pairwise_metrics.cpp:326-337)
double js_scale(const c10::optional<double> &base) { return base.has_value() ? 0.5 / std::log(base.value()) : 0.5; }

struct JensenShannonFn : torch::autograd::Function<JensenShannonFn> {
    // rooted = false: _sqjensenshannon; true: the square root that jensenshannon_distances applies, fused
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2, double scale, bool rooted) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype (while checking arguments for _sqjensenshannon_forward)");
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out = at::empty({q.B, q.N1, q.N2}, q.a.options());
        if (q.D == 0) out.zero_();
        else
            TPW_CALL(tpw_jensenshannon_forward(code_of(q.a), q.a.data_ptr(), q.b.data_ptr(), out.data_ptr(), q.B, q.N1, q.N2, q.D,
                                               scale, rooted ? 1 : 0, stream_of(q.a)));
        ctx->save_for_backward({q.a, q.b, rooted ? out : Tensor()});
        ctx->saved_data["scale"] = scale;
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static std::pair<Tensor, Tensor> raw_backward(const Tensor &grad, const Tensor &a, const Tensor &b, const Tensor &out,
                                                  double scale, bool ub) {
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = grad.to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        Tensor g1 = at::empty_like(a), g2 = at::empty_like(b);
        TPW_CALL(tpw_jensenshannon_backward(code_of(a), g.data_ptr(), out.defined() ? out.data_ptr() : nullptr, a.data_ptr(), b.data_ptr(),
                                            g1.data_ptr(), g2.data_ptr(), a.size(0), a.size(1), b.size(1), a.size(2), scale, stream_of(a)));
        return {g1, g2};
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        auto g = raw_backward(go[0], s[0], s[1], s[2], ctx->saved_data["scale"].toDouble(), ub);
        return {finish(g.first, ub, dt), finish(g.second, ub, dt), Tensor(), Tensor()};
    }
};

// ---- _canberra, _additive_chi2_kernel (OPS/autograd/canberra_kernel.cpp, additive_chi2_kernel.cpp) ----------
struct PairSumFn : torch::autograd::Function<PairSumFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2, int64_t metric) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype");
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out = at::empty({q.B, q.N1, q.N2}, q.a.options());
        if (q.D == 0) out.zero_();
        else
            TPW_CALL(tpw_pair_sum_forward(code_of(q.a), static_cast<int>(metric), q.a.data_ptr(), q.b.data_ptr(), out.data_ptr(),
                                          q.B, q.N1, q.N2, q.D, stream_of(q.a)));
        ctx->save_for_backward({q.a, q.b});
        ctx->saved_data["metric"] = metric;
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static std::pair<Tensor, Tensor> raw_backward(const Tensor &grad, const Tensor &a, const Tensor &b, int metric, bool ub) {
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = grad.to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        Tensor g1 = at::empty_like(a), g2 = at::empty_like(b);
        TPW_CALL(tpw_pair_sum_backward(code_of(a), metric, g.data_ptr(), a.data_ptr(), b.data_ptr(), g1.data_ptr(), g2.data_ptr(),
                                       a.size(0), a.size(1), b.size(1), a.size(2), stream_of(a)));
        return {g1, g2};
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        auto g = raw_backward(go[0], s[0], s[1], static_cast<int>(ctx->saved_data["metric"].toInt()), ub);
        return {finish(g.first, ub, dt), finish(g.second, ub, dt), Tensor()};
    }
};

// ---- _haversine (OPS/autograd/haversine_kernel.cpp, kernels OPS/cpu/haversine_kernel.cpp:12-217) -------------
struct HaversineFn : torch::autograd::Function<HaversineFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype (while checking arguments for _haversine_forward)");
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        TORCH_CHECK(q.D == 2, "feature dimension of x1 and x2 must be 2.");
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out = at::empty({q.B, q.N1, q.N2}, q.a.options());
        TPW_CALL(tpw_haversine_forward(code_of(q.a), q.a.data_ptr(), q.b.data_ptr(), out.data_ptr(), q.B, q.N1, q.N2, stream_of(q.a)));
        ctx->save_for_backward({q.a, q.b});
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static std::pair<Tensor, Tensor> raw_backward(const Tensor &grad, const Tensor &a, const Tensor &b, bool ub) {
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = grad.to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        Tensor g1 = at::empty_like(a), g2 = at::empty_like(b);
        TPW_CALL(tpw_haversine_backward(code_of(a), g.data_ptr(), a.data_ptr(), b.data_ptr(), g1.data_ptr(), g2.data_ptr(),
                                        a.size(0), a.size(1), b.size(1), stream_of(a)));
        return {g1, g2};
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        auto g = raw_backward(go[0], s[0], s[1], ub);
        return {finish(g.first, ub, dt), finish(g.second, ub, dt)};
    }
};

// ---- _wminkowski (OPS/autograd/wminkowski_kernel.cpp:9-50) ---------------------------------------------
struct WMinkowskiFn : torch::autograd::Function<WMinkowskiFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2, const Tensor &w, double p) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type() && in_dt == w.scalar_type(),
                    "x1, x2 and w must have the same dtype (while checking arguments for _wminkowski_forward)");
        require_cuda(w);
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        TORCH_CHECK(q.unbatched ? w.dim() == 1 : w.dim() == 2, "w must be 1-D (unbatched) or 2-D (batched) tensor.");
        Tensor wc = w.to(q.a.scalar_type()).contiguous();
        if (q.unbatched) wc = wc.unsqueeze(0);
        TORCH_CHECK(wc.size(0) == q.B, "batch_size of x1, x2, and w do not match.");
        // the reference compares w.size(1) with N1 here (OPS/cuda/wminkowski_kernel.cu:91); the feature count is meant
        TORCH_CHECK(wc.size(1) == q.D, "feature dimension of x1, x2, and w do not match.");
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out;
        if (p == 0) out = at::full({q.B, q.N1, q.N2}, static_cast<double>(q.D), q.a.options());
        else out = lp_forward(q, &wc, p, std::isinf(p) ? 1.0 : 1.0 / p);
        ctx->save_for_backward({q.a, q.b, wc});
        ctx->saved_data["p"] = p;
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static std::tuple<Tensor, Tensor, Tensor> raw_backward(const Tensor &grad, const Tensor &a, const Tensor &b, const Tensor &w,
                                                           double p, bool ub) {
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = grad.to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        Tensor g1 = at::zeros_like(a), g2 = at::zeros_like(b), gw = at::zeros_like(w);
        const int64_t B = a.size(0), N1 = a.size(1), N2 = b.size(1), D = a.size(2);
        if (p != 0 && B * N1 * N2 * D > 0) {
            if (std::isinf(p)) {
                TPW_CALL(tpw_lp_inf_backward(code_of(a), g.data_ptr(), a.data_ptr(), b.data_ptr(), w.data_ptr(), g1.data_ptr(),
                                             g2.data_ptr(), gw.data_ptr(), B, N1, N2, D, p < 0, stream_of(a)));
            } else {
                Prepared q{a, b, false, B, N1, N2, D};
                Tensor coef = lp_forward(q, &w, p, 1.0 / p - 1.0); // S^(1/p-1), OPS/cuda/wminkowski_kernel.cu:16-37
                lp_backward_call(code_of(a), TPW_LP_BWD_WMINKOWSKI, g, coef.data_ptr(), a, b, w.data_ptr(), g1, g2, B, N1, N2, D, p);
                Tensor scratch = at::empty({B, N1, D}, a.options());
                TPW_CALL(tpw_wminkowski_backward_w(code_of(a), g.data_ptr(), coef.data_ptr(), a.data_ptr(), b.data_ptr(), gw.data_ptr(),
                                                   scratch.data_ptr(), B, N1, N2, D, p, stream_of(a)));
            }
        }
        return {g1, g2, gw};
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        auto g = raw_backward(go[0], s[0], s[1], s[2], ctx->saved_data["p"].toDouble(), ub);
        return {finish(std::get<0>(g), ub, dt), finish(std::get<1>(g), ub, dt), finish(std::get<2>(g), ub, dt), Tensor()};
    }
};

// ---- cosine similarity and its 1 - S variants (OPS/pairwise_metrics.cpp:51-56,112-122,203) ---------------
struct CosineFn : torch::autograd::Function<CosineFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2, int64_t epilogue) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype");
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out = dot_forward(q, static_cast<int>(epilogue), TPW_ENGINE_AUTO);
        ctx->save_for_backward({q.a, q.b, out});
        ctx->saved_data["epilogue"] = epilogue;
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const Tensor &a = s[0], &b = s[1], &out = s[2];
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        const int epilogue = static_cast<int>(ctx->saved_data["epilogue"].toInt());
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = go[0].to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        const int64_t B = a.size(0), N1 = a.size(1), N2 = b.size(1), D = a.size(2);
        const int code = code_of(a);
        auto st = stream_of(a);
        Tensor n1 = at::empty({B, N1}, a.options()), n2 = at::empty({B, N2}, a.options());
        TPW_CALL(tpw_row_norm(code, a.data_ptr(), n1.data_ptr(), B * N1, D, st));
        TPW_CALL(tpw_row_norm(code, b.data_ptr(), n2.data_ptr(), B * N2, D, st));
        Tensor g1 = at::empty_like(a), g2 = at::empty_like(b);
        CosineArgs cos;
        cos.epilogue = epilogue; cos.n1 = &n1; cos.n2 = &n2;
        if (a.numel() > 0 && b.numel() > 0 && dense_backward(TPW_LP_BWD_MATMUL, g, &out, a, b, g1, g2, cos))
            return {finish(g1, ub, dt), finish(g2, ub, dt), Tensor()};
        Tensor dM = at::empty_like(g), rowterm = at::empty({B, N1}, a.options()), colterm = at::empty({B, N2}, a.options());
        TPW_CALL(tpw_cosine_backward_prepare(code, epilogue, g.data_ptr(), out.data_ptr(), n1.data_ptr(), n2.data_ptr(), dM.data_ptr(),
                                             rowterm.data_ptr(), colterm.data_ptr(), B, N1, N2, st));
        dense_backward(TPW_LP_BWD_MATMUL, dM, nullptr, a, b, g1, g2);
        TPW_CALL(tpw_cosine_backward_finish(code, g1.data_ptr(), a.data_ptr(), n1.data_ptr(), rowterm.data_ptr(), B * N1, D, st));
        TPW_CALL(tpw_cosine_backward_finish(code, g2.data_ptr(), b.data_ptr(), n2.data_ptr(), colterm.data_ptr(), B * N2, D, st));
        return {finish(g1, ub, dt), finish(g2, ub, dt), Tensor()};
    }
};

// x - x.mean(-1, keepdim) (OPS/pairwise_metrics.cpp:197-198); its own gradient is the same map
struct RowCenterFn : torch::autograd::Function<RowCenterFn> {
    static Tensor center(const Tensor &x) {
        require_cuda(x);
        const auto in_dt = x.scalar_type();
        Tensor xc = x.to(compute_type(in_dt)).contiguous();
        Tensor out = at::empty_like(xc);
        c10::cuda::CUDAGuard dg(xc.device());
        const int64_t D = xc.size(-1);
        if (xc.numel() > 0)
            TPW_CALL(tpw_row_center(code_of(xc), xc.data_ptr(), out.data_ptr(), xc.numel() / D, D, stream_of(xc)));
        return out.to(in_dt);
    }
    static Tensor forward(AutogradContext *, const Tensor &x) {
        at::AutoDispatchBelowADInplaceOrView guard;
        return center(x);
    }
    static variable_list backward(AutogradContext *, variable_list go) { return {center(go[0])}; }
};

// ---- directed Hausdorff (OPS/autograd/hausdorff_kernel.cpp:9-61) -------------------------------------------
struct HausdorffRun {
    Tensor a, b, out, i1, i2;
    bool unbatched;
    at::ScalarType in_dt;
};

// Checks, contiguous float32/float64 operands with a leading batch dimension, the visiting orders when
// `shuffle` is set, and the forward kernels (OPS/cuda/hausdorff_kernel.cu:107-196).
HausdorffRun hausdorff_run(const Tensor &x1, const Tensor &x2, bool shuffle, c10::optional<at::Generator> generator) {
    require_cuda(x1);
    require_cuda(x2);
    const auto in_dt = x1.scalar_type();
    TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype (while checking arguments for _directed_hausdorff_forward)");
    const bool ub = x1.dim() == 3;
    TORCH_CHECK(ub || x1.dim() == 4, "x1 must be 3-D (unbatched) or 4-D (batched) tensor.");
    TORCH_CHECK(x2.dim() == x1.dim(), "x2 must be 3-D (unbatched) or 4-D (batched) tensor.");
    TORCH_CHECK(ub || x1.size(0) == x2.size(0), "batch_size of x1 and x2 do not match.");
    TORCH_CHECK(x1.size(-1) == x2.size(-1), "feature dimension of x1 and x2 do not match.");
    const auto dt = compute_type(in_dt);
    Tensor a = x1.to(dt).contiguous(), b = x2.is_same(x1) ? a : x2.to(dt).contiguous();
    if (ub) { a = a.unsqueeze(0); b = b.unsqueeze(0); }
    const int64_t B = a.size(0), N1 = a.size(1), M1 = a.size(2), D = a.size(3), N2 = b.size(1), M2 = b.size(2);
    c10::cuda::CUDAGuard dg(a.device());
    Tensor out = at::empty({B, N1, N2}, a.options());
    Tensor i1 = at::empty({B, N1, N2}, a.options().dtype(at::kLong)), i2 = at::empty_like(i1);
    Tensor o1, o2;
    if (shuffle && B > 0) {
        // per batch, x1's permutation then x2's (OPS/cuda/hausdorff_kernel.cu:158-167); order[perm[t]] = t
        o1 = at::empty({B, M1}, i1.options());
        o2 = at::empty({B, M2}, i1.options());
        for (int64_t bb = 0; bb < B; ++bb) {
            Tensor p1 = at::randperm(M1, generator, i1.options()), p2 = at::randperm(M2, generator, i1.options());
            o1[bb].index_put_({p1}, at::arange(M1, i1.options()));
            o2[bb].index_put_({p2}, at::arange(M2, i1.options()));
        }
    }
    const int64_t bytes = std::max<int64_t>(tpw_hausdorff_scratch_bytes(B, N1, N2, M1), 8);
    Tensor scratch = at::empty({bytes}, a.options().dtype(at::kByte));
    TPW_CALL(tpw_hausdorff_forward(code_of(a), a.data_ptr(), b.data_ptr(), o1.defined() ? o1.data_ptr<int64_t>() : nullptr,
                                   o2.defined() ? o2.data_ptr<int64_t>() : nullptr, out.data_ptr(), i1.data_ptr<int64_t>(),
                                   i2.data_ptr<int64_t>(), scratch.data_ptr(), B, N1, N2, M1, M2, D, stream_of(a)));
    return {a, b, out, i1, i2, ub, in_dt};
}

// grad [B,N1,N2] (batched layout) -> one point per set and pair (OPS/cuda/hausdorff_kernel.cu:198-246)
std::pair<Tensor, Tensor> hausdorff_grads(const Tensor &g, const Tensor &a, const Tensor &b, const Tensor &out,
                                          const Tensor &i1, const Tensor &i2) {
    c10::cuda::CUDAGuard dg(a.device());
    Tensor g1 = at::empty_like(a), g2 = at::empty_like(b);
    TPW_CALL(tpw_hausdorff_backward(code_of(a), g.data_ptr(), out.data_ptr(), i1.data_ptr<int64_t>(), i2.data_ptr<int64_t>(),
                                    a.data_ptr(), b.data_ptr(), g1.data_ptr(), g2.data_ptr(), a.size(0), a.size(1), b.size(1),
                                    a.size(2), b.size(2), a.size(3), stream_of(a)));
    return {g1, g2};
}

struct HausdorffFn : torch::autograd::Function<HausdorffFn> {
    static variable_list forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2, bool shuffle,
                                 c10::optional<at::Generator> generator) {
        at::AutoDispatchBelowADInplaceOrView guard;
        HausdorffRun r0 = hausdorff_run(x1, x2, shuffle, generator);
        const Tensor &a = r0.a, &b = r0.b, &out = r0.out, &i1 = r0.i1, &i2 = r0.i2;
        const bool ub = r0.unbatched;
        const auto in_dt = r0.in_dt;
        ctx->save_for_backward({a, b, out, i1, i2});
        ctx->saved_data["unbatched"] = ub;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        Tensor r = finish(out, ub, in_dt), r1 = ub ? i1.squeeze(0) : i1, r2 = ub ? i2.squeeze(0) : i2;
        ctx->mark_non_differentiable({r1, r2});
        return {r, r1, r2};
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const Tensor &a = s[0], &b = s[1], &out = s[2], &i1 = s[3], &i2 = s[4];
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        Tensor g = go[0].to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        auto gg = hausdorff_grads(g, a, b, out, i1, i2);
        const Tensor &g1 = gg.first, &g2 = gg.second;
        return {finish(g1, ub, dt), finish(g2, ub, dt), Tensor(), Tensor()};
    }
};

// ---- boolean / compare-reduce (no autograd: the reference registers none either) ---------------------------
std::tuple<Tensor, Tensor, int64_t> pack_bool(const Tensor &xb) {
    const int64_t B = xb.size(0), N = xb.size(1), D = xb.size(2);
    int64_t W = std::max<int64_t>(4, (D + 31) / 32);
    W = (W + 3) / 4 * 4;
    Tensor words = at::empty({B, N, W}, xb.options().dtype(at::kInt)), pops = at::empty({B, N}, xb.options().dtype(at::kInt));
    Tensor src = xb.contiguous();
    TPW_CALL(tpw_bitpack(static_cast<const uint8_t *>(src.data_ptr()), static_cast<uint32_t *>(words.data_ptr()),
                         static_cast<int32_t *>(pops.data_ptr()), B * N, D, W, stream_of(xb)));
    return {words, pops, W};
}

Tensor bool_metric(const Tensor &x1, const Tensor &x2, int metric) {
    require_cuda(x1);
    require_cuda(x2);
    const bool ub = x1.dim() == 2;
    TORCH_CHECK(ub || x1.dim() == 3, "x1 must be 2-D (unbatched) or 3-D (batched) tensor.");
    TORCH_CHECK(x2.dim() == x1.dim(), "x2 must be 2-D (unbatched) or 3-D (batched) tensor.");
    TORCH_CHECK(ub || x1.size(0) == x2.size(0), "batch_size of x1 and x2 do not match.");
    TORCH_CHECK(x1.size(-1) == x2.size(-1), "feature dimension of x1 and x2 do not match.");
    Tensor a = ub ? x1.unsqueeze(0) : x1, b = ub ? x2.unsqueeze(0) : x2;
    const int64_t B = a.size(0), N1 = a.size(1), N2 = b.size(1), D = a.size(2);
    c10::cuda::CUDAGuard dg(a.device());
    Tensor out = at::empty({B, N1, N2}, a.options().dtype(at::kFloat));
    if (D == 0) {
        out.fill_(metric <= TPW_BOOL_NE_SUM || metric == TPW_BOOL_JACCARD || metric == TPW_BOOL_YULE
                      ? 0.0 : std::numeric_limits<double>::quiet_NaN());
    } else if (out.numel() > 0) {
        auto pa = pack_bool(a);
        auto pb = x2.is_same(x1) ? pa : pack_bool(b);
        Tensor ab = a.contiguous(), bb = x2.is_same(x1) ? ab : b.contiguous();
        if (tpw_bool_metric_tc_eligible(B, N1, N2, D) && reinterpret_cast<uintptr_t>(ab.data_ptr()) % 16 == 0 &&
            reinterpret_cast<uintptr_t>(bb.data_ptr()) % 16 == 0) {
            // large problem: the counts come from the tensor cores (8-bit integer contraction of the 0 / 1 bytes)
            TPW_CALL(tpw_bool_metric_forward_tc(metric, static_cast<const uint8_t *>(ab.data_ptr()), static_cast<const uint8_t *>(bb.data_ptr()),
                                                static_cast<const int32_t *>(std::get<1>(pa).data_ptr()),
                                                static_cast<const int32_t *>(std::get<1>(pb).data_ptr()), out.data_ptr<float>(),
                                                B, N1, N2, D, stream_of(a)));
        } else
        TPW_CALL(tpw_bool_metric_forward(metric, static_cast<const uint32_t *>(std::get<0>(pa).data_ptr()),
                                         static_cast<const uint32_t *>(std::get<0>(pb).data_ptr()),
                                         static_cast<const int32_t *>(std::get<1>(pa).data_ptr()),
                                         static_cast<const int32_t *>(std::get<1>(pb).data_ptr()), out.data_ptr<float>(),
                                         B, N1, N2, D, std::get<2>(pa), stream_of(a)));
    }
    return ub ? out.squeeze(0) : out;
}

// a, b batched, same dtype in {float, double, int, long}
Tensor cmp_reduce(const Tensor &a, const Tensor &b, int op, int red) {
    const int64_t B = a.size(0), N1 = a.size(1), N2 = b.size(1), D = a.size(2);
    Tensor out = at::empty({B, N1, N2}, a.options().dtype(at::kFloat));
    if (D == 0) return out.fill_(red == TPW_RED_MEAN ? std::numeric_limits<double>::quiet_NaN() : 0.0);
    int code;
    switch (a.scalar_type()) {
        case at::kFloat: code = TPW_F32; break;
        case at::kDouble: code = TPW_F64; break;
        case at::kInt: code = TPW_I32; break;
        case at::kLong: code = TPW_I64; break;
        default: TORCH_CHECK(false, "pairwise comparison is not implemented for ", a.scalar_type());
    }
    TPW_CALL(tpw_cmp_reduce_forward(code, op, red, a.data_ptr(), b.data_ptr(), out.data_ptr<float>(), B, N1, N2, D, stream_of(a)));
    return out;
}

// pw{eq,ne}_{sum,mean}: any dtype, result_type promotion, float32 out (OPS/cuda/pairwise_binary_kernels.cu:144-220)
Tensor pairwise_compare(const Tensor &x1, const Tensor &x2, int op, int red) {
    require_cuda(x1);
    require_cuda(x2);
    auto common = at::result_type(x1, x2);
    if (common == at::kBool) {
        const int metric = op == TPW_CMP_EQ ? (red == TPW_RED_MEAN ? TPW_BOOL_EQ_MEAN : TPW_BOOL_EQ_SUM)
                                            : (red == TPW_RED_MEAN ? TPW_BOOL_NE_MEAN : TPW_BOOL_NE_SUM);
        return bool_metric(x1.to(at::kBool), x2.to(at::kBool), metric);
    }
    if (common == at::kHalf || common == at::kBFloat16) common = at::kFloat; // exact widening keeps every comparison
    else if (common == at::kByte || common == at::kChar || common == at::kShort) common = at::kInt;
    Prepared q = prepare(x1.to(common), x2.to(common), common);
    c10::cuda::CUDAGuard dg(q.a.device());
    Tensor out = cmp_reduce(q.a, q.b, op, red);
    return q.unbatched ? out.squeeze(0) : out;
}

Tensor pw_logic(const Tensor &x1, const Tensor &x2, int metric) {
    TORCH_CHECK(at::result_type(x1, x2) == at::kBool, "\"pairwise_binary_reduction_forward\" not implemented for '",
                at::result_type(x1, x2), "'");
    return bool_metric(x1, x2, metric);
}

// ---- prf_div family (OPS/prf_div.cpp:359-400, OPS/cuda/prf_div_kernel.cu, OPS/autograd/prf_div_kernel.cpp) -----
// Every overload is "numerator / denominator where the denominator is non-zero, else 0 (zero) or the
// numerator (identity)": prf_div(self, other) = self / other, prf_ldiv(self, other) = other / self.  A Scalar
// operand is expanded to a tensor of the other operand's shape before the element-wise kernel.
int prf_mode(c10::string_view mode) {
    if (mode == "zero") return TPW_PRF_ZERO;
    if (mode == "identity") return TPW_PRF_IDENTITY;
    TORCH_CHECK(false, "mode must be either zero or identity. Got ", mode);
}

at::ScalarType prf_result_type(at::ScalarType t) {
    return at::isIntegralType(t, /*includeBool=*/true) ? at::kFloat : t;   // OPS/cuda/prf_div_kernel.cu:93-95
}

void prf_same_shape(const Tensor &self, const Tensor &other) {
    TORCH_CHECK(self.sizes() == other.sizes(), "Broadcasting semantic is not implemented for prf_div. "
                "Expect self's shape to be identical to other's shape. Got self.shape=", self.sizes(),
                ", while other.shape=", other.sizes());
}

// num, den: same shape, any dtype; the kernel runs in float32 or float64 and the result has dtype `rt`.
Tensor prf_raw_forward(const Tensor &num, const Tensor &den, int mode, at::ScalarType rt) {
    require_cuda(num);
    require_cuda(den);
    TORCH_CHECK(num.get_device() == den.get_device(), "Expected all tensors to be on the same device");
    const auto ct = compute_type(rt);
    Tensor n = num.to(ct).contiguous(), d = den.to(ct).contiguous();
    c10::cuda::CUDAGuard dg(n.device());
    Tensor out = at::empty_like(n);
    TPW_CALL(tpw_prf_div_forward(code_of(n), mode, n.data_ptr(), d.data_ptr(), out.data_ptr(), n.numel(), stream_of(n)));
    return out.to(rt);
}

// (grad_num, grad_den) in grad's dtype; an unwanted one stays undefined.
std::pair<Tensor, Tensor> prf_raw_backward(const Tensor &grad, const Tensor &num, const Tensor &den, int mode,
                                           bool want_num, bool want_den) {
    require_cuda(grad);
    const auto rt = grad.scalar_type();
    const auto ct = compute_type(rt);
    Tensor g = grad.to(ct).contiguous(), n = num.to(ct).contiguous(), d = den.to(ct).contiguous();
    c10::cuda::CUDAGuard dg(g.device());
    Tensor gn = want_num ? at::empty_like(g) : Tensor(), gd = want_den ? at::empty_like(g) : Tensor();
    TPW_CALL(tpw_prf_div_backward(code_of(g), mode, g.data_ptr(), n.data_ptr(), d.data_ptr(), want_num ? gn.data_ptr() : nullptr,
                                  want_den ? gd.data_ptr() : nullptr, g.numel(), stream_of(g)));
    return {want_num ? gn.to(rt) : gn, want_den ? gd.to(rt) : gd};
}

Tensor scalar_like(const Tensor &t, const at::Scalar &v, at::ScalarType dt) { return at::full_like(t, v, t.options().dtype(dt)); }

struct PRFDivFn : torch::autograd::Function<PRFDivFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &num, const Tensor &den, int64_t mode, int64_t rt) {
        at::AutoDispatchBelowADInplaceOrView guard;
        ctx->save_for_backward({num, den});
        ctx->saved_data["mode"] = mode;
        return prf_raw_forward(num, den, static_cast<int>(mode), static_cast<at::ScalarType>(rt));
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        auto g = prf_raw_backward(go[0], s[0], s[1], static_cast<int>(ctx->saved_data["mode"].toInt()),
                                  ctx->needs_input_grad(0), ctx->needs_input_grad(1));
        if (g.first.defined()) g.first = g.first.to(s[0].scalar_type());
        if (g.second.defined()) g.second = g.second.to(s[1].scalar_type());
        return {g.first, g.second, Tensor(), Tensor()};
    }
};

// In place on `self` (OPS/cuda/prf_div_kernel.cu:189-300; the kernels return at::Tensor by value, as the
// reference's do, so that both libraries can be registered on one schema): `left` selects self = other / self.  The operands are
// saved before `self` is overwritten, so the gradient is that of the out-of-place op.
struct PRFDivInplaceFn : torch::autograd::Function<PRFDivInplaceFn> {
    static Tensor forward(AutogradContext *ctx, Tensor &self, const Tensor &other, int64_t mode, bool left) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto rt = prf_result_type(at::result_type(self, other));
        TORCH_CHECK(at::can_cast(rt, self.scalar_type()), "result type ", rt, " can't be cast to the desired output type ",
                    self.scalar_type());
        ctx->mark_dirty({self});
        const bool track = self.requires_grad() || other.requires_grad();
        Tensor before = track ? self.clone() : self;
        const Tensor &num = left ? other : before, &den = left ? before : other;
        if (track) ctx->save_for_backward({num, den});
        ctx->saved_data["mode"] = mode;
        ctx->saved_data["left"] = left;
        self.copy_(prf_raw_forward(left ? other : self, left ? self : other, static_cast<int>(mode), rt));
        return self;
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const bool left = ctx->saved_data["left"].toBool();
        // inputs are (self, other); saved are (numerator, denominator)
        const bool want_num = ctx->needs_input_grad(left ? 1 : 0), want_den = ctx->needs_input_grad(left ? 0 : 1);
        auto g = prf_raw_backward(go[0], s[0], s[1], static_cast<int>(ctx->saved_data["mode"].toInt()), want_num, want_den);
        if (g.first.defined()) g.first = g.first.to(s[0].scalar_type());
        if (g.second.defined()) g.second = g.second.to(s[1].scalar_type());
        return {left ? g.second : g.first, left ? g.first : g.second, Tensor(), Tensor()};
    }
};

template <bool left>
Tensor prf_div_tensor(const Tensor &self, const Tensor &other, c10::string_view mode) {
    prf_same_shape(self, other);
    const auto rt = static_cast<int64_t>(prf_result_type(at::result_type(self, other)));
    return left ? PRFDivFn::apply(other, self, prf_mode(mode), rt) : PRFDivFn::apply(self, other, prf_mode(mode), rt);
}
template <bool left>
Tensor prf_div_scalar(const Tensor &self, const at::Scalar &other, c10::string_view mode) {
    const auto rt = prf_result_type(at::result_type(self, other));
    Tensor o = scalar_like(self, other, compute_type(rt));
    return left ? PRFDivFn::apply(o, self, prf_mode(mode), static_cast<int64_t>(rt))
                : PRFDivFn::apply(self, o, prf_mode(mode), static_cast<int64_t>(rt));
}
// prf_div.rScalar(s, t) = s / t; prf_ldiv.rScalar(s, t) = t / s (OPS/cuda/prf_div_kernel.cu:181-187)
template <bool left>
Tensor prf_div_rscalar(const at::Scalar &self, const Tensor &other, c10::string_view mode) {
    return prf_div_scalar<!left>(other, self, mode);
}
template <bool left>
Tensor prf_div_inplace(Tensor &self, const Tensor &other, c10::string_view mode) {
    prf_same_shape(self, other);
    PRFDivInplaceFn::apply(self, other, prf_mode(mode), left);
    return self;
}
template <bool left>
Tensor prf_div_inplace_scalar(Tensor &self, const at::Scalar &other, c10::string_view mode) {
    const auto rt = prf_result_type(at::result_type(self, other));
    PRFDivInplaceFn::apply(self, scalar_like(self, other, compute_type(rt)), prf_mode(mode), left);
    return self;
}

// The stand-alone backward ops (OPS/cuda/prf_div_kernel.cu:372-520); gradients in the operands' dtypes.
template <bool left>
std::tuple<Tensor, Tensor> prf_div_backward_op(const Tensor &grad, const Tensor &self, const Tensor &other, c10::string_view mode) {
    auto g = left ? prf_raw_backward(grad, other, self, prf_mode(mode), true, true)
                  : prf_raw_backward(grad, self, other, prf_mode(mode), true, true);
    const Tensor &gs = left ? g.second : g.first, &go = left ? g.first : g.second;
    return std::make_tuple(gs.to(self.scalar_type()), go.to(other.scalar_type()));
}
template <bool left>
Tensor prf_div_backward_scalar_op(const Tensor &grad, const Tensor &self, const at::Scalar &other, c10::string_view mode) {
    Tensor o = scalar_like(self, other, compute_type(grad.scalar_type()));
    auto g = left ? prf_raw_backward(grad, o, self, prf_mode(mode), false, true)
                  : prf_raw_backward(grad, self, o, prf_mode(mode), true, false);
    return (left ? g.second : g.first).to(self.scalar_type());
}
template <bool left>
Tensor prf_div_backward_rscalar_op(const Tensor &grad, const at::Scalar &self, const Tensor &other, c10::string_view mode) {
    Tensor sc = scalar_like(other, self, compute_type(grad.scalar_type()));
    auto g = left ? prf_raw_backward(grad, other, sc, prf_mode(mode), true, false)
                  : prf_raw_backward(grad, sc, other, prf_mode(mode), false, true);
    return (left ? g.first : g.second).to(other.scalar_type());
}

// ---- public ops ------------------------------------------------------------------------------------------------
#define PM "pairwise_metrics"
Tensor cdist_p(const char *name, const Tensor &x1, const OptTensor &x2, double p) {
    auto ab = check_pairwise_inputs(name, x1, x2);
    return CdistFn::apply(ab.first, ab.second, p);
}
Tensor euclidean_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "euclidean_distances");
    return cdist_p("euclidean_distances", x1, x2, 2.0);
}
Tensor manhattan_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "manhattan_distances");
    return cdist_p("manhattan_distances", x1, x2, 1.0);
}
Tensor chebyshev_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "chebyshev_distances");
    return cdist_p("chebyshev_distances", x1, x2, std::numeric_limits<double>::infinity());
}
Tensor minkowski_distances(const Tensor &x1, const OptTensor &x2, double p) {
    TPW_OP(PM, "minkowski_distances");
    return cdist_p("minkowski_distances", x1, x2, p);
}
// the aliases of OPS/pairwise_metrics.cpp:265-270,411-438 log their own names there as well
Tensor cityblock_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "cityblock_distances");
    return cdist_p("manhattan_distances", x1, x2, 1.0);
}
Tensor l1_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "l1_distances");
    return cdist_p("manhattan_distances", x1, x2, 1.0);
}
Tensor l2_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "l2_distances");
    return cdist_p("euclidean_distances", x1, x2, 2.0);
}
Tensor lp_distances(const Tensor &x1, const OptTensor &x2, double p) {
    TPW_OP(PM, "lp_distances");
    return cdist_p("minkowski_distances", x1, x2, p);
}
Tensor linf_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "linf_distances");
    return cdist_p("chebyshev_distances", x1, x2, std::numeric_limits<double>::infinity());
}
Tensor ppminkowski(const Tensor &x1, const Tensor &x2, double p) {
    TPW_OP("ppminkowski", "_ppminkowski");
    return PPMinkowskiFn::apply(x1, x2, p);
}
Tensor wminkowski(const Tensor &x1, const Tensor &x2, const Tensor &w, double p) {
    TPW_OP("wminkowski", "_wminkowski");
    return WMinkowskiFn::apply(x1, x2, w, p);
}
Tensor wminkowski_distances(const Tensor &x1, const OptTensor &x2, double p, const OptTensor &w) {
    TPW_OP(PM, "wminkowski_distances");
    auto ab = check_pairwise_inputs("wminkowski_distances", x1, x2);
    return w.has_value() ? WMinkowskiFn::apply(ab.first, ab.second, w.value(), p) : CdistFn::apply(ab.first, ab.second, p);
}
Tensor sqeuclidean_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "sqeuclidean_distances");
    auto ab = check_pairwise_inputs("sqeuclidean_distances", x1, x2);
    return PPMinkowskiFn::apply(ab.first, ab.second, 2.0);
}
Tensor cosine_similarity(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "cosine_similarity");
    auto ab = check_pairwise_inputs("cosine_similarity", x1, x2);
    return CosineFn::apply(ab.first, ab.second, static_cast<int64_t>(TPW_DOT_COSINE_SIM));
}
Tensor cosine_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "cosine_distances");
    auto ab = check_pairwise_inputs("cosine_similarity", x1, x2);
    return CosineFn::apply(ab.first, ab.second, static_cast<int64_t>(TPW_DOT_COSINE_DIST));
}
Tensor correlation_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "correlation_distances");
    auto ab = check_pairwise_inputs("correlation_distances", x1, x2);
    Tensor c1 = RowCenterFn::apply(ab.first);
    Tensor c2 = x2.has_value() ? RowCenterFn::apply(ab.second) : c1;
    return CosineFn::apply(c1, c2, static_cast<int64_t>(TPW_DOT_ONE_MINUS_SIM));
}
Tensor hamming_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "hamming_distances");
    auto ab = check_pairwise_inputs("hamming_distances", x1, x2);
    return pairwise_compare(ab.first, ab.second, TPW_CMP_NE, TPW_RED_MEAN);
}
template <int METRIC>
Tensor boolean_metric_op(const Tensor &x1, const OptTensor &x2) {
    static const char *names[] = {"", "", "", "", "", "", "", "jaccard_distances", "kulsinski_distances", "kulczynski1_distances",
                                  "yule_distances", "dice_distances", "rogerstanimoto_distances", "russellrao_distances",
                                  "sokalmichener_distances", "sokalsneath_distances"};
    static const std::string usage = std::string("torchpairwise.csrc.ops.pairwise_metrics.") + names[METRIC];
    static const std::string range = std::string("torchpairwise::") + names[METRIC];
    static bool logged = (c10::LogAPIUsage(usage), true);
    (void) logged;
    NvtxRange nvtx_range_(range.c_str());
    if (METRIC == TPW_BOOL_KULSINSKI)
        TORCH_WARN_DEPRECATION("kulsinski_distances is deprecated in SciPy 1.9.0 and might be removed in the future. "
                               "Please use kulczynski1_distances.");
    auto ab = check_pairwise_inputs(names[METRIC], x1, x2, /*boolean=*/true);
    return bool_metric(ab.first, ab.second, METRIC);
}
std::tuple<Tensor, Tensor, Tensor> directed_hausdorff_raw(const Tensor &x1, const Tensor &x2, bool shuffle,
                                                          c10::optional<at::Generator> generator) {
    auto r = HausdorffFn::apply(x1, x2, shuffle, generator);
    return {r[0], r[1], r[2]};
}
std::tuple<Tensor, Tensor, Tensor> directed_hausdorff_distances(const Tensor &x1, const OptTensor &x2, bool shuffle,
                                                                c10::optional<at::Generator> generator) {
    TPW_OP(PM, "directed_hausdorff_distances");
    auto ab = check_pairwise_inputs("directed_hausdorff_distances", x1, x2, false, /*sets=*/true);
    return directed_hausdorff_raw(ab.first, ab.second, shuffle, generator);
}

Tensor sqjensenshannon_raw(const Tensor &x1, const Tensor &x2, c10::optional<double> base) {
    return JensenShannonFn::apply(x1, x2, js_scale(base), false);
}
// OPS/pairwise_metrics.cpp:326-337: rows scaled to sum one (plain tensor operations), then one kernel for the sum and the root
Tensor jensenshannon_distances(const Tensor &x1, const OptTensor &x2, c10::optional<double> base) {
    TPW_OP(PM, "jensenshannon_distances");
    auto ab = check_pairwise_inputs("jensenshannon_distances", x1, x2);
    Tensor n1 = ab.first / ab.first.sum(-1, true);
    Tensor n2 = x2.has_value() ? ab.second / ab.second.sum(-1, true) : n1;
    return JensenShannonFn::apply(n1, n2, js_scale(base), true);
}
Tensor canberra_raw(const Tensor &x1, const Tensor &x2) { return PairSumFn::apply(x1, x2, static_cast<int64_t>(TPW_PAIR_CANBERRA)); }
Tensor additive_chi2_raw(const Tensor &x1, const Tensor &x2) { return PairSumFn::apply(x1, x2, static_cast<int64_t>(TPW_PAIR_ADDITIVE_CHI2)); }
Tensor canberra_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "canberra_distances");
    auto ab = check_pairwise_inputs("canberra_distances", x1, x2);
    return canberra_raw(ab.first, ab.second);
}
// OPS/pairwise_metrics.cpp:124-145 (the sign check synchronises there as well)
Tensor additive_chi2_kernel(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "additive_chi2_kernel");
    auto ab = check_pairwise_inputs("additive_chi2_kernel", x1, x2);
    TORCH_CHECK(ab.first.ge(0).all().item<bool>() && (!x2.has_value() || ab.second.ge(0).all().item<bool>()),
                "All elements of x1 and x2 must be positive");
    return additive_chi2_raw(ab.first, ab.second);
}
Tensor chi2_kernel(const Tensor &x1, const OptTensor &x2, double gamma) {
    TPW_OP(PM, "chi2_kernel");
    return (additive_chi2_kernel(x1, x2) * gamma).exp();
}
// OPS/pairwise_metrics.cpp:308-315 with OPS/cpu/braycurtis_kernel.cpp:22-27: sum |x - y| / sum |x + y| as two L1 passes
Tensor braycurtis_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "braycurtis_distances");
    auto ab = check_pairwise_inputs("braycurtis_distances", x1, x2);
    return CdistFn::apply(ab.first, ab.second, 1.0) / CdistFn::apply(ab.first, ab.second.neg(), 1.0);
}
// OPS/pairwise_metrics.cpp:401-408 with OPS/cpu/snr_kernel.cpp:22-34: var(x2 - x1) / var(x1) per pair.  The deviations of
// x2 - x1 from their mean are the differences of the centred rows, so the first variance is the squared Euclidean
// distance of the centred rows, taken by the direct-difference kernel: a row against itself gives exactly 0.
Tensor snr_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "snr_distances");
    auto ab = check_pairwise_inputs("snr_distances", x1, x2);
    Tensor c1 = RowCenterFn::apply(ab.first);
    Tensor c2 = x2.has_value() ? RowCenterFn::apply(ab.second) : c1;
    Tensor diff_var = PPMinkowskiFn::apply(c1, c2, 2.0);
    Tensor x1_var = c1.pow(2).sum(-1, true);
    return diff_var / x1_var;
}
// OPS/pairwise_metrics.cpp:245-263: weighted Minkowski with w = 1/V (1 where V is 0), p = 2
Tensor seuclidean_distances(const Tensor &x1, const OptTensor &x2, const OptTensor &V) {
    TPW_OP(PM, "seuclidean_distances");
    TORCH_CHECK(!x2.has_value() || V.has_value(), "V is required for seuclidean when x2 is passed.");
    auto ab = check_pairwise_inputs("euclidean_distances", x1, x2);
    Tensor v;
    if (V.has_value()) v = V.value();
    else {
        at::NoGradGuard ng;
        v = ab.first.dim() == 2 ? ab.first.var(at::IntArrayRef{0}) : ab.first.var(at::IntArrayRef{0, 1});
    }
    Tensor w = PRFDivFn::apply(at::ones_like(v), v, static_cast<int64_t>(TPW_PRF_IDENTITY), static_cast<int64_t>(v.scalar_type()));
    return WMinkowskiFn::apply(ab.first, ab.second, w, 2.0);
}
Tensor haversine_raw(const Tensor &x1, const Tensor &x2) { return HaversineFn::apply(x1, x2); }
Tensor haversine_distances(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "haversine_distances");
    auto ab = check_pairwise_inputs("haversine_distances", x1, x2);
    return HaversineFn::apply(ab.first, ab.second);
}

// ---- kernel functions (OPS/pairwise_metrics.cpp:58-110) ---------------------------------------------------------
// x1 x2^T.  The raw dot product has no norm to hide bf16 rounding behind: large float32 problems take the tf32 x 3
// tensor-core pipeline with chunked accumulation (as accurate as the fp32 FMA chain), everything else the exact tile.
struct LinearKernelFn : torch::autograd::Function<LinearKernelFn> {
    static Tensor forward(AutogradContext *ctx, const Tensor &x1, const Tensor &x2) {
        at::AutoDispatchBelowADInplaceOrView guard;
        const auto in_dt = x1.scalar_type();
        TORCH_CHECK(in_dt == x2.scalar_type(), "x1 and x2 must have the same dtype");
        Prepared q = prepare(x1, x2, compute_type(in_dt));
        c10::cuda::CUDAGuard dg(q.a.device());
        Tensor out = dot_forward(q, TPW_DOT_LINEAR, tensor_engine_selected(q) ? TPW_ENGINE_TCGEN05_TF32X3 : TPW_ENGINE_SIMT_FP32);
        ctx->save_for_backward({q.a, q.b});
        ctx->saved_data["unbatched"] = q.unbatched;
        ctx->saved_data["dt"] = static_cast<int64_t>(in_dt);
        return finish(out, q.unbatched, in_dt);
    }
    static variable_list backward(AutogradContext *ctx, variable_list go) {
        auto s = ctx->get_saved_variables();
        const Tensor &a = s[0], &b = s[1];
        const bool ub = ctx->saved_data["unbatched"].toBool();
        const auto dt = static_cast<at::ScalarType>(ctx->saved_data["dt"].toInt());
        c10::cuda::CUDAGuard dg(a.device());
        Tensor g = go[0].to(a.scalar_type()).contiguous();
        if (ub) g = g.unsqueeze(0);
        Tensor g1 = at::zeros_like(a), g2 = at::zeros_like(b);
        if (a.numel() > 0 && b.numel() > 0) dense_backward(TPW_LP_BWD_MATMUL, g, nullptr, a, b, g1, g2);
        return {finish(g1, ub, dt), finish(g2, ub, dt)};
    }
};
Tensor linear_kernel(const Tensor &x1, const OptTensor &x2) {
    TPW_OP(PM, "linear_kernel");
    auto ab = check_pairwise_inputs("linear_kernel", x1, x2);
    return LinearKernelFn::apply(ab.first, ab.second);
}
// the reference divides by x1.size(1) whatever the rank (OPS/pairwise_metrics.cpp:76,88,97,108)
double default_gamma(const Tensor &x1, c10::optional<double> gamma) { return gamma.value_or(1.0 / static_cast<double>(x1.size(1))); }
Tensor polynomial_kernel(const Tensor &x1, const OptTensor &x2, int64_t degree, c10::optional<double> gamma, double coef0) {
    TPW_OP(PM, "polynomial_kernel");
    auto ab = check_pairwise_inputs("polynomial_kernel", x1, x2);
    return (LinearKernelFn::apply(ab.first, ab.second) * default_gamma(x1, gamma) + coef0).pow(degree);
}
Tensor sigmoid_kernel(const Tensor &x1, const OptTensor &x2, c10::optional<double> gamma, double coef0) {
    TPW_OP(PM, "sigmoid_kernel");
    auto ab = check_pairwise_inputs("sigmoid_kernel", x1, x2);
    return (LinearKernelFn::apply(ab.first, ab.second) * default_gamma(x1, gamma) + coef0).tanh();
}
Tensor rbf_kernel(const Tensor &x1, const OptTensor &x2, c10::optional<double> gamma) {
    TPW_OP(PM, "rbf_kernel");
    auto ab = check_pairwise_inputs("sqeuclidean_distances", x1, x2);
    return (PPMinkowskiFn::apply(ab.first, ab.second, 2.0) * -default_gamma(x1, gamma)).exp();
}
// the reference's own backward of this one fails (an in-place exp on the output of cdist); here it is differentiable
Tensor laplacian_kernel(const Tensor &x1, const OptTensor &x2, c10::optional<double> gamma) {
    TPW_OP(PM, "laplacian_kernel");
    auto ab = check_pairwise_inputs("laplacian_kernel", x1, x2);
    return (CdistFn::apply(ab.first, ab.second, 1.0) * -default_gamma(x1, gamma)).exp();
}

// ---- Mahalanobis (OPS/pairwise_metrics.cpp:272-297, OPS/sqmahalanobis.cpp:31-38, OPS/cpu/sqmahalanobis_kernel.cpp:23-31) --
// (x1 - x2) VI (x1 - x2)^T depends on the symmetric part S of VI only.  Where S is positive definite (every inverse
// covariance is) S = L L^T and the form is the squared Euclidean distance of x1 L and x2 L, taken by the
// direct-difference kernel: a sum of squares, exactly 0 for a row against itself and accurate for near-duplicate
// rows.  Otherwise d.e with d = x1 - x2, e = d S is taken as (|d/c + c e|^2 - |d/c - c e|^2) / 4, again two
// direct-difference kernels (c balances the two magnitudes).  Differentiable in x1, x2 and VI through both.
Tensor sqmahalanobis_impl(const Tensor &x1, const Tensor &x2, const Tensor &VI) {
    TORCH_CHECK(x1.scalar_type() == x2.scalar_type() && x1.scalar_type() == VI.scalar_type(),
                "x1, x2 and VI must have the same dtype (while checking arguments for _sqmahalanobis_forward)");
    const bool unbatched = x1.dim() == 2;
    TORCH_CHECK(unbatched || x1.dim() == 3, "x1 must be 2-D (unbatched) or 3-D (batched) tensor.");
    TORCH_CHECK(x2.dim() == x1.dim(), "x2 must be 2-D (unbatched) or 3-D (batched) tensor.");
    TORCH_CHECK(VI.dim() == x1.dim(), "VI must be 2-D (unbatched) or 3-D (batched) tensor.");
    TORCH_CHECK(unbatched || (x1.size(0) == x2.size(0) && x1.size(0) == VI.size(0)), "batch_size of x1, x2, and VI do not match.");
    TORCH_CHECK(x1.size(-1) == x2.size(-1) && x1.size(-1) == VI.size(-2) && VI.size(-1) == VI.size(-2),
                "feature dimension of x1, x2, and VI do not match.");
    const bool same = x2.is_same(x1);
    Tensor S = (VI + VI.transpose(-1, -2)) * 0.5;
    Tensor L, info;
    std::tie(L, info) = at::linalg_cholesky_ex(S, /*upper=*/false, /*check_errors=*/false);
    if (x1.size(-1) > 0 && info.eq(0).all().item<bool>()) {
        Tensor u1 = x1.matmul(L);
        Tensor u2 = same ? u1 : x2.matmul(L);
        return PPMinkowskiFn::apply(u1, u2, 2.0);
    }
    Tensor e1 = x1.matmul(S);
    Tensor e2 = same ? e1 : x2.matmul(S);
    double c = 1.0;
    {
        at::NoGradGuard ng;
        const double nx = x1.norm().item<double>(), ne = e1.norm().item<double>();
        if (nx > 0 && ne > 0 && std::isfinite(nx / ne)) c = std::sqrt(nx / ne);
    }
    Tensor p1 = x1 / c + e1 * c, m1 = x1 / c - e1 * c;
    Tensor p2 = same ? p1 : x2 / c + e2 * c, m2 = same ? m1 : x2 / c - e2 * c;
    return (PPMinkowskiFn::apply(p1, p2, 2.0) - PPMinkowskiFn::apply(m1, m2, 2.0)) * 0.25;
}
Tensor sqmahalanobis_raw(const Tensor &x1, const Tensor &x2, const Tensor &VI) {
    TPW_OP("sqmahalanobis", "_sqmahalanobis");
    require_cuda(x1);
    return sqmahalanobis_impl(x1, x2, VI);
}
std::tuple<Tensor, Tensor, Tensor> sqmahalanobis_backward_op(const Tensor &grad, const Tensor &x1, const Tensor &x2, const Tensor &VI) {
    at::AutoGradMode enable(true);
    Tensor a = x1.detach().requires_grad_(true), b = x2.detach().requires_grad_(true), v = VI.detach().requires_grad_(true);
    Tensor out = sqmahalanobis_impl(a, b, v);
    auto g = torch::autograd::grad({out}, {a, b, v}, {grad.to(out.scalar_type())}, /*retain_graph=*/false, /*create_graph=*/false,
                                   /*allow_unused=*/true);
    auto or_zero = [](const Tensor &t, const Tensor &like) { return t.defined() ? t : at::zeros_like(like); };
    return std::make_tuple(or_zero(g[0], x1), or_zero(g[1], x2), or_zero(g[2], VI));
}
Tensor mahalanobis_distances(const Tensor &x1, const OptTensor &x2, const OptTensor &VI) {
    TPW_OP(PM, "mahalanobis_distances");
    TORCH_CHECK(!x2.has_value() || VI.has_value(), "VI is required for manhalanobis when x2 is passed.");
    auto ab = check_pairwise_inputs("mahalanobis_distances", x1, x2);
    require_cuda(ab.first);
    Tensor vi;
    if (VI.has_value()) vi = VI.value();
    else {
        at::NoGradGuard ng;
        if (ab.first.dim() == 2) vi = at::cov(ab.first.transpose(-1, -2)).inverse().transpose(-1, -2);
        else {
            std::vector<Tensor> covs;
            for (int64_t b = 0; b < ab.first.size(0); ++b) covs.push_back(at::cov(ab.first[b].transpose(-1, -2)));
            vi = at::stack(covs).inverse().transpose(-1, -2);
        }
    }
    return sqmahalanobis_impl(ab.first, ab.second, vi).sqrt();
}

// ---- cdist: string dispatcher with the reference's keyword validation (OPS/cpdist.cpp:35-79,149-231) -----------
const char *const kSupportedMetrics =
    "braycurtis, canberra, chebyshev, cityblock, correlation, cosine, dice, directed_hausdorff, euclidean, hamming, "
    "haversine, jaccard, jensenshannon, kulczynski1, kulsinski, l1, l2, lp, linf, mahalanobis, manhattan, minkowski, "
    "rogerstanimoto, russellrao, seuclidean, snr, sokalmichener, sokalsneath, sqeuclidean, wminkowski, yule";

// Unknown metric: RuntimeError; a keyword the metric does not take: TypeError (OPS/cpdist.cpp:35-79).
void check_metric_and_extra_args(const std::string &m, const OptTensor &w, const OptTensor &V, const OptTensor &VI,
                                 const c10::optional<double> &p, const c10::optional<double> &base, const c10::optional<bool> &shuffle,
                                 const c10::optional<at::Generator> &generator) {
    auto accepts = [&](const char *arg) {
        if (m == "directed_hausdorff") return !strcmp(arg, "shuffle") || !strcmp(arg, "generator");
        if (m == "minkowski" || m == "lp") return !strcmp(arg, "p");
        if (m == "wminkowski") return !strcmp(arg, "w") || !strcmp(arg, "p");
        if (m == "seuclidean") return !strcmp(arg, "V");
        if (m == "mahalanobis") return !strcmp(arg, "VI");
        if (m == "jensenshannon") return !strcmp(arg, "base");
        return false;
    };
    std::string bad;
    auto note = [&](bool given, const char *arg) {
        if (given && !accepts(arg)) bad += (bad.empty() ? "" : ", ") + std::string(arg);
    };
    const bool known = std::string(", ").append(kSupportedMetrics).append(", ").find(", " + m + ", ") != std::string::npos;
    TORCH_CHECK(known, "Got unkown distance metric: ", m, ". Supported metrics are [", kSupportedMetrics, "]");
    note(w.has_value(), "w"); note(V.has_value(), "V"); note(VI.has_value(), "VI"); note(p.has_value(), "p");
    note(base.has_value(), "base"); note(shuffle.has_value(), "shuffle"); note(generator.has_value(), "generator");
    TORCH_CHECK_TYPE(bad.empty(), "torchpairwise::", m, "_distances was called with incompatible arguments ", bad, ".");
}

Tensor cdist_dispatch(const Tensor &x1, const OptTensor &x2, const std::string &m, const OptTensor &w, const OptTensor &V,
                      const OptTensor &VI, c10::optional<double> p, c10::optional<double> base, c10::optional<bool> shuffle,
                      c10::optional<at::Generator> generator) {
    if (m == "euclidean" || m == "l2") return euclidean_distances(x1, x2);
    if (m == "manhattan" || m == "cityblock" || m == "l1") return manhattan_distances(x1, x2);
    if (m == "chebyshev" || m == "linf") return chebyshev_distances(x1, x2);
    if (m == "minkowski" || m == "lp") return minkowski_distances(x1, x2, p.value_or(2));
    if (m == "wminkowski") return wminkowski_distances(x1, x2, p.value_or(2), w);
    if (m == "sqeuclidean") return sqeuclidean_distances(x1, x2);
    if (m == "cosine") return cosine_distances(x1, x2);
    if (m == "correlation") return correlation_distances(x1, x2);
    if (m == "hamming") return hamming_distances(x1, x2);
    if (m == "jensenshannon") return jensenshannon_distances(x1, x2, base);
    if (m == "haversine") return haversine_distances(x1, x2);
    if (m == "canberra") return canberra_distances(x1, x2);
    if (m == "braycurtis") return braycurtis_distances(x1, x2);
    if (m == "snr") return snr_distances(x1, x2);
    if (m == "seuclidean") return seuclidean_distances(x1, x2, V);
    if (m == "mahalanobis") return mahalanobis_distances(x1, x2, VI);
    if (m == "jaccard") return boolean_metric_op<TPW_BOOL_JACCARD>(x1, x2);
    // the reference's cdist routes "kulsinski" through the kulczynski1 functor (OPS/pairwise_metrics.h:557-561)
    if (m == "kulsinski" || m == "kulczynski1") return boolean_metric_op<TPW_BOOL_KULCZYNSKI1>(x1, x2);
    if (m == "yule") return boolean_metric_op<TPW_BOOL_YULE>(x1, x2);
    if (m == "dice") return boolean_metric_op<TPW_BOOL_DICE>(x1, x2);
    if (m == "rogerstanimoto") return boolean_metric_op<TPW_BOOL_ROGERSTANIMOTO>(x1, x2);
    if (m == "russellrao") return boolean_metric_op<TPW_BOOL_RUSSELLRAO>(x1, x2);
    if (m == "sokalmichener") return boolean_metric_op<TPW_BOOL_SOKALMICHENER>(x1, x2);
    if (m == "sokalsneath") return boolean_metric_op<TPW_BOOL_SOKALSNEATH>(x1, x2);
    if (m == "directed_hausdorff") return std::get<0>(directed_hausdorff_distances(x1, x2, shuffle.value_or(false), generator));
    TORCH_CHECK(false, "Got unkown distance metric: ", m, ". Supported metrics are [", kSupportedMetrics, "]");
}

Tensor cdist(const Tensor &x1, const Tensor &x2, c10::string_view metric, const OptTensor &w, const OptTensor &V,
             const OptTensor &VI, c10::optional<double> p, c10::optional<double> base, c10::optional<bool> shuffle,
             c10::optional<at::Generator> generator) {
    TPW_OP("cpdist", "cdist");
    const std::string m(metric.data(), metric.size());
    check_metric_and_extra_args(m, w, V, VI, p, base, shuffle, generator);
    return cdist_dispatch(x1, x2, m, w, V, VI, p, base, shuffle, generator);
}

// The L_p metrics the fused neighbour and condensed kernels serve: exponent p and the exponent applied to the sum.
// Returns false for every other metric, for weights, and for exponents the kernels do not take.
bool lp_metric_of(const std::string &m, const c10::optional<double> &p_arg, double *p, double *out_exponent) {
    const double inf = std::numeric_limits<double>::infinity();
    if (m == "euclidean" || m == "l2") { *p = 2; *out_exponent = 0.5; return true; }
    if (m == "sqeuclidean") { *p = 2; *out_exponent = 1; return true; }
    if (m == "manhattan" || m == "cityblock" || m == "l1") { *p = 1; *out_exponent = 1; return true; }
    if (m == "chebyshev" || m == "linf") { *p = inf; *out_exponent = 1; return true; }
    if (m == "minkowski" || m == "lp") {
        *p = p_arg.value_or(2.0);
        if (!(*p > 0)) return false;
        *out_exponent = std::isinf(*p) ? 1.0 : 1.0 / *p;
        return true;
    }
    return false;
}

// ---- pdist (OPS/cpdist.cpp:233-255: declared with the arguments of cdist, raises "yet to be implemented") ---------
// The condensed upper triangle of cdist(input, input), row by row (the layout of torch.pdist).  The L_p metrics run the
// tile kernel with a condensed epilogue that skips the tiles on or below the diagonal when no gradient is needed;
// everything else, and every differentiable call, evaluates cdist and gathers the triangle.
Tensor pdist(const Tensor &input, c10::string_view metric, const OptTensor &w, const OptTensor &V, const OptTensor &VI,
             c10::optional<double> p, c10::optional<double> base, c10::optional<bool> shuffle,
             c10::optional<at::Generator> generator) {
    TPW_OP("cpdist", "pdist");
    const std::string m(metric.data(), metric.size());
    check_metric_and_extra_args(m, w, V, VI, p, base, shuffle, generator);
    TORCH_CHECK(input.dim() == 2 || input.dim() == 3, "input must be 2D tensor (unbatched) or 3D tensor (batched)");
    require_cuda(input);
    const int64_t n = input.size(-2);
    double pp = 0, ex = 0;
    const auto dt = input.scalar_type();
    if (lp_metric_of(m, p, &pp, &ex) && (dt == at::kFloat || dt == at::kDouble) && input.size(-1) > 0 &&
        !(input.requires_grad() && at::GradMode::is_enabled())) {
        Tensor x = input.contiguous();
        if (x.dim() == 2) x = x.unsqueeze(0);
        c10::cuda::CUDAGuard dg(x.device());
        Tensor out = at::empty({x.size(0), n * (n - 1) / 2}, x.options());
        TPW_CALL(tpw_lp_pdist_forward(code_of(x), x.data_ptr(), out.data_ptr(), x.size(0), n, x.size(2), pp, ex, stream_of(x)));
        return input.dim() == 3 ? out : out.squeeze(0);
    }
    Tensor full = cdist_dispatch(input, input, m, w, V, VI, p, base, shuffle, generator);
    Tensor iu = at::triu_indices(n, n, 1, at::TensorOptions().dtype(at::kLong).device(input.device()));
    return full.index({at::indexing::Ellipsis, iu[0], iu[1]});
}

// ---- neighbour masks (OPS/neighbors.cpp:10-68) -------------------------------------------------------------------
// The reference evaluates cdist and compares / sorts the whole matrix.  Float32 L_p metrics (and, for the k nearest
// rows, the contraction metrics on large problems) go to the fused kernels instead, which never write the
// float matrix; everything else follows the reference's composition with a partial selection in place of the sort.
Tensor radius_neighbors_mask(const Tensor &x1, const OptTensor &x2, double epsilon, c10::string_view metric, const OptTensor &w,
                             const OptTensor &V, const OptTensor &VI, c10::optional<double> p, c10::optional<double> base,
                             c10::optional<bool> shuffle, c10::optional<at::Generator> generator) {
    C10_LOG_API_USAGE_ONCE("torchpairwise.csrc.ops.neighbors.k_neighbors_mask");  // the name the reference logs here too (OPS/neighbors.cpp:48)
    NvtxRange nvtx_range_("torchpairwise::radius_neighbors_mask");
    auto ab = check_pairwise_inputs("radius_neighbors_mask", x1, x2);
    TORCH_CHECK(epsilon >= 0., "epsilon must be non-negative. Got epsilon=", epsilon);
    const std::string m(metric.data(), metric.size());
    check_metric_and_extra_args(m, w, V, VI, p, base, shuffle, generator);
    at::NoGradGuard ng;
    double pp = 0, ex = 0;
    const auto dt = ab.first.scalar_type();
    if (lp_metric_of(m, p, &pp, &ex) && ab.first.is_cuda() && dt == ab.second.scalar_type() && (dt == at::kFloat || dt == at::kDouble) &&
        ab.first.size(-1) > 0 && (ab.first.dim() == 2 || ab.first.dim() == 3)) {
        Prepared q = prepare(ab.first, ab.second, dt);
        // p = 2 on a large float32 problem is faster as a tensor-core contraction plus a compare pass
        if (!(pp == 2.0 && tensor_engine_selected(q))) {
            c10::cuda::CUDAGuard dg(q.a.device());
            Tensor mask = at::empty({q.B, q.N1, q.N2}, q.a.options().dtype(at::kBool));
            TPW_CALL(tpw_lp_radius_mask_forward(code_of(q.a), q.a.data_ptr(), q.b.data_ptr(), nullptr,
                                                static_cast<uint8_t *>(mask.data_ptr()), q.B, q.N1, q.N2, q.D, pp, ex, epsilon,
                                                stream_of(q.a)));
            return q.unbatched ? mask.squeeze(0) : mask;
        }
    }
    return cdist_dispatch(ab.first, ab.second, m, w, V, VI, p, base, shuffle, generator).le(epsilon);
}

Tensor k_neighbors_mask(const Tensor &x1, const OptTensor &x2, int64_t k, c10::string_view metric, const OptTensor &w,
                        const OptTensor &V, const OptTensor &VI, c10::optional<double> p, c10::optional<double> base,
                        c10::optional<bool> shuffle, c10::optional<at::Generator> generator) {
    TPW_OP("neighbors", "k_neighbors_mask");
    auto ab = check_pairwise_inputs("k_neighbors_mask", x1, x2);
    TORCH_CHECK(k >= 0, "k must be non-negative. Got k=", k);
    const std::string m(metric.data(), metric.size());
    check_metric_and_extra_args(m, w, V, VI, p, base, shuffle, generator);
    at::NoGradGuard ng;
    const Tensor &a = ab.first, &b = ab.second;
    auto scatter_mask = [&](const Tensor &inds) {
        Tensor out = at::zeros({a.size(0), b.size(0)}, a.options().dtype(at::kBool));
        return out.scatter_(1, inds, true);
    };
    double pp = 0, ex = 0;
    const bool f32 = a.is_cuda() && a.dim() == 2 && a.scalar_type() == at::kFloat && b.scalar_type() == at::kFloat &&
                     a.size(-1) > 0 && b.size(0) > 0;
    const int64_t kk = k + 1;  // the reference keeps k + 1 columns: the point itself plus k neighbours when x2 is x1
    if (f32 && kk <= b.size(0)) {
        Prepared q = prepare(a, b, at::kFloat);
        c10::cuda::CUDAGuard dg(q.a.device());
        const bool lp = lp_metric_of(m, p, &pp, &ex);
        const bool tensor = tensor_engine_selected(q);
        const int dot_epilogue = (m == "euclidean" || m == "l2") ? TPW_DOT_EUCLIDEAN : m == "sqeuclidean" ? TPW_DOT_SQEUCLIDEAN
                                 : m == "cosine" ? TPW_DOT_COSINE_DIST : -1;
        auto st = stream_of(q.a);
        if (kk == 1 && (lp || (dot_epilogue >= 0 && tensor))) {
            // one column per row: the streaming row minimum, no distance matrix and no sort
            Tensor mins = at::empty({q.B, q.N1}, q.a.options()), args = at::empty({q.B, q.N1}, q.a.options().dtype(at::kLong));
            if (dot_epilogue >= 0 && tensor) {
                const int64_t bytes = tpw_dot_rowmin_scratch_bytes(q.B, q.N1, q.N2, q.D);
                Tensor scratch = at::empty({bytes}, q.a.options().dtype(at::kByte));
                TPW_CALL(tpw_dot_rowmin_forward_ws(dot_epilogue, q.a.data_ptr(), q.b.data_ptr(), mins.data_ptr<float>(),
                                                   args.data_ptr<int64_t>(), scratch.data_ptr(), bytes, q.B, q.N1, q.N2, q.D, st));
            } else {
                const int64_t bytes = std::max<int64_t>(8, tpw_lp_rowmin_scratch_bytes(q.B, q.N1));
                Tensor scratch = at::empty({bytes}, q.a.options().dtype(at::kByte));
                TPW_CALL(tpw_lp_rowmin_forward(TPW_F32, q.a.data_ptr(), q.b.data_ptr(), nullptr, mins.data_ptr<float>(),
                                               args.data_ptr<int64_t>(), scratch.data_ptr(), q.B, q.N1, q.N2, q.D, pp, ex, st));
            }
            return scatter_mask(args.squeeze(0).unsqueeze(1));
        }
        const bool few_p = pp == 1.0 || pp == 2.0 || pp == 3.0 || std::isinf(pp);
        if (lp && few_p && q.D <= tpw_lp_topk_max_features() && q.N1 >= 4096 && kk <= tpw_lp_topk_max_k() &&
            !std::getenv("TPW_DISABLE_SMALL_D")) {
            // few features: one x1 row per thread with its k + 1 best keys in registers
            Tensor vals = at::empty({q.B, q.N1, kk}, q.a.options()), inds = at::empty({q.B, q.N1, kk}, q.a.options().dtype(at::kLong));
            TPW_CALL(tpw_lp_topk_forward(TPW_F32, q.a.data_ptr(), q.b.data_ptr(), vals.data_ptr<float>(), inds.data_ptr<int64_t>(),
                                         q.B, q.N1, q.N2, q.D, static_cast<int>(kk), pp, ex, st));
            return scatter_mask(inds.squeeze(0));
        }
        if (dot_epilogue >= 0 && tensor && kk <= tpw_dot_topk_max_k()) {
            // large problem: the k + 1 nearest rows straight from the tensor-core epilogue
            Tensor vals = at::empty({q.B, q.N1, kk}, q.a.options()), inds = at::empty({q.B, q.N1, kk}, q.a.options().dtype(at::kLong));
            const int64_t bytes = tpw_dot_topk_scratch_bytes(kk, q.B, q.N1, q.N2, q.D);
            Tensor scratch = at::empty({bytes}, q.a.options().dtype(at::kByte));
            TPW_CALL(tpw_dot_topk_forward_ws(dot_epilogue, static_cast<int>(kk), q.a.data_ptr(), q.b.data_ptr(), vals.data_ptr<float>(),
                                             inds.data_ptr<int64_t>(), scratch.data_ptr(), bytes, q.B, q.N1, q.N2, q.D, st));
            return scatter_mask(inds.squeeze(0));
        }
    }
    Tensor dists = cdist_dispatch(a, b, m, w, V, VI, p, base, shuffle, generator);
    // the k + 1 smallest of every row: a partial selection, not the reference's full argsort of each row
    Tensor inds = std::get<1>(dists.topk(std::min<int64_t>(kk, dists.size(1)), 1, /*largest=*/false, /*sorted=*/false));
    return scatter_mask(inds);
}

// torchpairwise::_cuda_version / _cuda_arch_flags (csrc/torchpairwise.cpp:28-56): what the loader of the reference's
// Python package checks (torchpairwise/extension.py:98-136).  Only registered when the reference library is absent.
int64_t cuda_version_op() { return tpw_cuda_version(); }
std::string cuda_arch_flags_op() { return tpw_cuda_arch_flags(); }

// __directed_hausdorff_backward re-runs the forward for the attaining pair, as the reference's backward op does
// (OPS/cuda/hausdorff_kernel.cu:283-321).
std::tuple<Tensor, Tensor> directed_hausdorff_backward_op(const Tensor &grad, const Tensor &x1, const Tensor &x2, bool shuffle,
                                                         c10::optional<at::Generator> generator) {
    HausdorffRun r = hausdorff_run(x1, x2, shuffle, generator);
    Tensor g = grad.to(r.a.scalar_type()).contiguous();
    if (r.unbatched) g = g.unsqueeze(0);
    auto gg = hausdorff_grads(g, r.a, r.b, r.out, r.i1, r.i2);
    return std::make_tuple(finish(gg.first, r.unbatched, r.in_dt), finish(gg.second, r.unbatched, r.in_dt));
}

bool defined(const char *name, const char *overload = "") {
    return c10::Dispatcher::singleton().findSchema({std::string("torchpairwise::") + name, overload}).has_value();
}

#define OPT2 "(Tensor x1, Tensor? x2=None) -> Tensor"

// Schemas, only where the reference extension has not already defined them.
TORCH_LIBRARY_FRAGMENT(torchpairwise, m) {
    auto def = [&](const char *name, const char *sig) {
        if (!defined(name)) m.def((std::string("torchpairwise::") + name + sig).c_str());
    };
    for (const char *n : {"euclidean_distances", "manhattan_distances", "cosine_distances", "cosine_similarity",
                          "sqeuclidean_distances", "correlation_distances", "hamming_distances", "jaccard_distances",
                          "kulsinski_distances", "kulczynski1_distances", "cityblock_distances", "chebyshev_distances",
                          "yule_distances", "dice_distances", "rogerstanimoto_distances", "russellrao_distances",
                          "sokalmichener_distances", "sokalsneath_distances", "l1_distances", "l2_distances", "linf_distances"})
        def(n, OPT2);
    def("minkowski_distances", "(Tensor x1, Tensor? x2=None, float p=2) -> Tensor");
    def("lp_distances", "(Tensor x1, Tensor? x2=None, float p=2) -> Tensor");
    def("wminkowski_distances", "(Tensor x1, Tensor? x2=None, float p=2, Tensor? w=None) -> Tensor");
    def("directed_hausdorff_distances",
        "(Tensor x1, Tensor? x2=None, *, bool shuffle=False, Generator? generator=None) -> (Tensor output, Tensor x1_indices, Tensor x2_indices)");
    def("_ppminkowski", "(Tensor x1, Tensor x2, float p=2) -> Tensor");
    def("__ppminkowski_backward", "(Tensor grad, Tensor x1, Tensor x2, float p) -> (Tensor grad_x1, Tensor grad_x2)");
    def("_wminkowski", "(Tensor x1, Tensor x2, Tensor w, float p=2) -> Tensor");
    def("__wminkowski_backward", "(Tensor grad, Tensor x1, Tensor x2, Tensor w, float p) -> (Tensor grad_x1, Tensor grad_x2, Tensor grad_w)");
    def("_directed_hausdorff",
        "(Tensor x1, Tensor x2, *, bool shuffle=False, Generator? generator=None) -> (Tensor output, Tensor x1_indices, Tensor x2_indices)");
    for (const char *n : {"pwand_sum", "pwor_sum", "pwxor_sum", "pweq_sum", "pwne_sum", "pweq_mean", "pwne_mean"})
        def(n, "(Tensor x1, Tensor x2) -> Tensor");
    for (const char *n : {"haversine_distances", "canberra_distances", "braycurtis_distances", "snr_distances", "additive_chi2_kernel"})
        def(n, OPT2);
    def("chi2_kernel", "(Tensor x1, Tensor? x2=None, float gamma=1.0) -> Tensor");
    def("seuclidean_distances", "(Tensor x1, Tensor? x2=None, Tensor? V=None) -> Tensor");
    def("_canberra", "(Tensor x1, Tensor x2) -> Tensor");
    def("__canberra_backward", "(Tensor grad, Tensor x1, Tensor x2) -> (Tensor grad_x1, Tensor grad_x2)");
    def("_additive_chi2_kernel", "(Tensor x1, Tensor x2) -> Tensor");
    def("__additive_chi2_kernel_backward", "(Tensor grad, Tensor x1, Tensor x2) -> (Tensor grad_x1, Tensor grad_x2)");
    def("jensenshannon_distances", "(Tensor x1, Tensor? x2=None, float? base=None) -> Tensor");
    def("_sqjensenshannon", "(Tensor x1, Tensor x2, float? base=None) -> Tensor");
    def("__sqjensenshannon_backward", "(Tensor grad, Tensor x1, Tensor x2, float? base) -> (Tensor grad_x1, Tensor grad_x2)");
    def("_haversine", "(Tensor x1, Tensor x2) -> Tensor");
    def("__haversine_backward", "(Tensor grad, Tensor x1, Tensor x2) -> (Tensor grad_x1, Tensor grad_x2)");
    def("__directed_hausdorff_backward",
        "(Tensor grad, Tensor x1, Tensor x2, *, bool shuffle=False, Generator? generator=None) -> (Tensor grad_x1, Tensor grad_x2)");
    // OPS/prf_div.cpp:359-400
    auto def_ov = [&](const char *name, const char *overload, const char *sig) {
        if (defined(name, overload))
            return;
        std::string full = std::string("torchpairwise::") + name;
        if (overload[0]) full += std::string(".") + overload;
        m.def((full + sig).c_str());
    };
    for (const char *n : {"prf_div", "prf_ldiv"}) {
        def_ov(n, "", "(Tensor input, Tensor other, str mode=\"zero\") -> Tensor");
        def_ov(n, "Scalar", "(Tensor input, Scalar other, str mode=\"zero\") -> Tensor");
        def_ov(n, "rScalar", "(Scalar input, Tensor other, str mode=\"zero\") -> Tensor");
    }
    for (const char *n : {"prf_div_", "prf_ldiv_"}) {
        def_ov(n, "", "(Tensor(a!) input, Tensor other, str mode=\"zero\") -> Tensor(a!)");
        def_ov(n, "Scalar", "(Tensor(a!) input, Scalar other, str mode=\"zero\") -> Tensor(a!)");
    }
    for (const char *n : {"_prf_div_backward", "_prf_ldiv_backward", "_prf_div__backward", "_prf_ldiv__backward"}) {
        def_ov(n, "", "(Tensor grad, Tensor self, Tensor other, str mode=\"zero\") -> (Tensor grad_self, Tensor grad_other)");
        def_ov(n, "Scalar", "(Tensor grad, Tensor self, Scalar other, str mode=\"zero\") -> Tensor grad_self");
    }
    for (const char *n : {"_prf_div_backward", "_prf_ldiv_backward"})
        def_ov(n, "rScalar", "(Tensor grad, Scalar self, Tensor other, str mode=\"zero\") -> Tensor grad_other");
#define EXTRA_ARGS "Tensor? w=None, Tensor? V=None, Tensor? VI=None, float? p=None, float? base=None, bool? shuffle=None, Generator? generator=None"
    def("cdist", "(Tensor x1, Tensor x2, str metric=\"minkowski\", *, " EXTRA_ARGS ") -> Tensor");
    // OPS/cpdist.cpp:252-255, OPS/neighbors.cpp:60-68
    def("pdist", "(Tensor input, str metric=\"minkowski\", *, " EXTRA_ARGS ") -> Tensor");
    def("k_neighbors_mask", "(Tensor x1, Tensor? x2=None, int k=1, str metric=\"euclidean\", *, " EXTRA_ARGS ") -> Tensor");
    def("radius_neighbors_mask", "(Tensor x1, Tensor? x2=None, float epsilon=0., str metric=\"euclidean\", *, " EXTRA_ARGS ") -> Tensor");
    // OPS/pairwise_metrics.h:114-150,286; OPS/sqmahalanobis.cpp:31-38
    def("linear_kernel", OPT2);
    def("polynomial_kernel", "(Tensor x1, Tensor? x2=None, int degree=3, float? gamma=None, float coef0=1) -> Tensor");
    def("sigmoid_kernel", "(Tensor x1, Tensor? x2=None, float? gamma=None, float coef0=1) -> Tensor");
    def("rbf_kernel", "(Tensor x1, Tensor? x2=None, float? gamma=None) -> Tensor");
    def("laplacian_kernel", "(Tensor x1, Tensor? x2=None, float? gamma=None) -> Tensor");
    def("mahalanobis_distances", "(Tensor x1, Tensor? x2=None, Tensor? VI=None) -> Tensor");
    def("_sqmahalanobis", "(Tensor x1, Tensor x2, Tensor VI) -> Tensor");
    def("__sqmahalanobis_backward", "(Tensor grad, Tensor x1, Tensor x2, Tensor VI) -> (Tensor grad_x1, Tensor grad_x2, Tensor grad_VI)");
    // csrc/torchpairwise.cpp:53-56: defined with their bodies, as there; the reference's own answer stands when it is loaded
    if (!defined("_cuda_version")) m.def("_cuda_version", &cuda_version_op);
    if (!defined("_cuda_arch_flags")) m.def("_cuda_arch_flags", &cuda_arch_flags_op);
}

// CUDA tensors of every op above.  AutogradCUDA sits in front of both the reference's
// CompositeImplicitAutograd bodies and its `Autograd` alias kernels, for CUDA tensors only.
TORCH_LIBRARY_IMPL(torchpairwise, AutogradCUDA, m) {
    m.impl("euclidean_distances", euclidean_distances);
    m.impl("l2_distances", l2_distances);
    m.impl("manhattan_distances", manhattan_distances);
    m.impl("cityblock_distances", cityblock_distances);
    m.impl("l1_distances", l1_distances);
    m.impl("chebyshev_distances", chebyshev_distances);
    m.impl("linf_distances", linf_distances);
    m.impl("minkowski_distances", minkowski_distances);
    m.impl("lp_distances", lp_distances);
    m.impl("linear_kernel", linear_kernel);
    m.impl("polynomial_kernel", polynomial_kernel);
    m.impl("sigmoid_kernel", sigmoid_kernel);
    m.impl("rbf_kernel", rbf_kernel);
    m.impl("laplacian_kernel", laplacian_kernel);
    m.impl("mahalanobis_distances", mahalanobis_distances);
    m.impl("_sqmahalanobis", sqmahalanobis_raw);
    m.impl("__sqmahalanobis_backward", sqmahalanobis_backward_op);  // runs a differentiable composition: needs the autograd key
    m.impl("pdist", pdist);
    m.impl("k_neighbors_mask", k_neighbors_mask);
    m.impl("radius_neighbors_mask", radius_neighbors_mask);
    m.impl("wminkowski_distances", wminkowski_distances);
    m.impl("sqeuclidean_distances", sqeuclidean_distances);
    m.impl("cosine_similarity", cosine_similarity);
    m.impl("cosine_distances", cosine_distances);
    m.impl("correlation_distances", correlation_distances);
    m.impl("hamming_distances", hamming_distances);
    m.impl("jaccard_distances", boolean_metric_op<TPW_BOOL_JACCARD>);
    m.impl("kulsinski_distances", boolean_metric_op<TPW_BOOL_KULSINSKI>);
    m.impl("kulczynski1_distances", boolean_metric_op<TPW_BOOL_KULCZYNSKI1>);
    m.impl("yule_distances", boolean_metric_op<TPW_BOOL_YULE>);
    m.impl("dice_distances", boolean_metric_op<TPW_BOOL_DICE>);
    m.impl("rogerstanimoto_distances", boolean_metric_op<TPW_BOOL_ROGERSTANIMOTO>);
    m.impl("russellrao_distances", boolean_metric_op<TPW_BOOL_RUSSELLRAO>);
    m.impl("sokalmichener_distances", boolean_metric_op<TPW_BOOL_SOKALMICHENER>);
    m.impl("sokalsneath_distances", boolean_metric_op<TPW_BOOL_SOKALSNEATH>);
    m.impl("directed_hausdorff_distances", directed_hausdorff_distances);
    m.impl("_ppminkowski", ppminkowski);
    m.impl("_wminkowski", wminkowski);
    m.impl("_directed_hausdorff", directed_hausdorff_raw);
    m.impl("cdist", cdist);
    m.impl("haversine_distances", haversine_distances);
    m.impl("canberra_distances", canberra_distances);
    m.impl("braycurtis_distances", braycurtis_distances);
    m.impl("snr_distances", snr_distances);
    m.impl("seuclidean_distances", seuclidean_distances);
    m.impl("additive_chi2_kernel", additive_chi2_kernel);
    m.impl("chi2_kernel", chi2_kernel);
    m.impl("_canberra", canberra_raw);
    m.impl("_additive_chi2_kernel", additive_chi2_raw);
    m.impl("jensenshannon_distances", jensenshannon_distances);
    m.impl("_sqjensenshannon", sqjensenshannon_raw);
    m.impl("_haversine", haversine_raw);
    m.impl("prf_div", prf_div_tensor<false>);
    m.impl("prf_ldiv", prf_div_tensor<true>);
    m.impl("prf_div.Scalar", prf_div_scalar<false>);
    m.impl("prf_ldiv.Scalar", prf_div_scalar<true>);
    m.impl("prf_div.rScalar", prf_div_rscalar<false>);
    m.impl("prf_ldiv.rScalar", prf_div_rscalar<true>);
    m.impl("prf_div_", prf_div_inplace<false>);
    m.impl("prf_ldiv_", prf_div_inplace<true>);
    m.impl("prf_div_.Scalar", prf_div_inplace_scalar<false>);
    m.impl("prf_ldiv_.Scalar", prf_div_inplace_scalar<true>);
}

// Ops without a gradient, and the stand-alone backward ops the reference's own Autograd kernels call.
TORCH_LIBRARY_IMPL(torchpairwise, CUDA, m) {
    m.impl("pwand_sum", [](const Tensor &a, const Tensor &b) { return pw_logic(a, b, TPW_BOOL_AND_SUM); });
    m.impl("pwor_sum", [](const Tensor &a, const Tensor &b) { return pw_logic(a, b, TPW_BOOL_OR_SUM); });
    m.impl("pwxor_sum", [](const Tensor &a, const Tensor &b) { return pw_logic(a, b, TPW_BOOL_XOR_SUM); });
    m.impl("pweq_sum", [](const Tensor &a, const Tensor &b) { return pairwise_compare(a, b, TPW_CMP_EQ, TPW_RED_SUM); });
    m.impl("pwne_sum", [](const Tensor &a, const Tensor &b) { return pairwise_compare(a, b, TPW_CMP_NE, TPW_RED_SUM); });
    m.impl("pweq_mean", [](const Tensor &a, const Tensor &b) { return pairwise_compare(a, b, TPW_CMP_EQ, TPW_RED_MEAN); });
    m.impl("pwne_mean", [](const Tensor &a, const Tensor &b) { return pairwise_compare(a, b, TPW_CMP_NE, TPW_RED_MEAN); });
    m.impl("__ppminkowski_backward", [](const Tensor &grad, const Tensor &x1, const Tensor &x2, double p) {
        Prepared q = prepare(x1, x2, compute_type(x1.scalar_type()));
        auto g = PPMinkowskiFn::raw_backward(grad, q.a, q.b, p, q.unbatched);
        return std::make_tuple(finish(g.first, q.unbatched, x1.scalar_type()), finish(g.second, q.unbatched, x1.scalar_type()));
    });
    m.impl("__wminkowski_backward", [](const Tensor &grad, const Tensor &x1, const Tensor &x2, const Tensor &w, double p) {
        Prepared q = prepare(x1, x2, compute_type(x1.scalar_type()));
        Tensor wc = w.to(q.a.scalar_type()).contiguous();
        if (q.unbatched) wc = wc.unsqueeze(0);
        auto g = WMinkowskiFn::raw_backward(grad, q.a, q.b, wc, p, q.unbatched);
        const auto dt = x1.scalar_type();
        return std::make_tuple(finish(std::get<0>(g), q.unbatched, dt), finish(std::get<1>(g), q.unbatched, dt),
                               finish(std::get<2>(g), q.unbatched, dt));
    });
    m.impl("__directed_hausdorff_backward", directed_hausdorff_backward_op);
    m.impl("__sqjensenshannon_backward", [](const Tensor &grad, const Tensor &x1, const Tensor &x2, c10::optional<double> base) {
        Prepared q = prepare(x1, x2, compute_type(x1.scalar_type()));
        auto g = JensenShannonFn::raw_backward(grad, q.a, q.b, Tensor(), js_scale(base), q.unbatched);
        return std::make_tuple(finish(g.first, q.unbatched, x1.scalar_type()), finish(g.second, q.unbatched, x1.scalar_type()));
    });
    m.impl("__canberra_backward", [](const Tensor &grad, const Tensor &x1, const Tensor &x2) {
        Prepared q = prepare(x1, x2, compute_type(x1.scalar_type()));
        auto g = PairSumFn::raw_backward(grad, q.a, q.b, TPW_PAIR_CANBERRA, q.unbatched);
        return std::make_tuple(finish(g.first, q.unbatched, x1.scalar_type()), finish(g.second, q.unbatched, x1.scalar_type()));
    });
    m.impl("__additive_chi2_kernel_backward", [](const Tensor &grad, const Tensor &x1, const Tensor &x2) {
        Prepared q = prepare(x1, x2, compute_type(x1.scalar_type()));
        auto g = PairSumFn::raw_backward(grad, q.a, q.b, TPW_PAIR_ADDITIVE_CHI2, q.unbatched);
        return std::make_tuple(finish(g.first, q.unbatched, x1.scalar_type()), finish(g.second, q.unbatched, x1.scalar_type()));
    });
    m.impl("__haversine_backward", [](const Tensor &grad, const Tensor &x1, const Tensor &x2) {
        Prepared q = prepare(x1, x2, compute_type(x1.scalar_type()));
        auto g = HaversineFn::raw_backward(grad, q.a, q.b, q.unbatched);
        return std::make_tuple(finish(g.first, q.unbatched, x1.scalar_type()), finish(g.second, q.unbatched, x1.scalar_type()));
    });
    m.impl("_prf_div_backward", prf_div_backward_op<false>);
    m.impl("_prf_ldiv_backward", prf_div_backward_op<true>);
    m.impl("_prf_div_backward.Scalar", prf_div_backward_scalar_op<false>);
    m.impl("_prf_ldiv_backward.Scalar", prf_div_backward_scalar_op<true>);
    m.impl("_prf_div_backward.rScalar", prf_div_backward_rscalar_op<false>);
    m.impl("_prf_ldiv_backward.rScalar", prf_div_backward_rscalar_op<true>);
    m.impl("_prf_div__backward", prf_div_backward_op<false>);
    m.impl("_prf_ldiv__backward", prf_div_backward_op<true>);
    m.impl("_prf_div__backward.Scalar", prf_div_backward_scalar_op<false>);
    m.impl("_prf_ldiv__backward.Scalar", prf_div_backward_scalar_op<true>);
}

} // namespace
