// ref_driver.cpp -- C entry points over the UNMODIFIED reference (compiled from its sources where they
// lie; see Makefile).  TEST INFRASTRUCTURE ONLY: it pins the C restatement in te_oracle.c, generates
// the golden fixtures under tests/golden/, and serves as the timed CPU reference in the benchmark.
// Everything here goes through the reference's public API: Tensor, transpose_view/view, matmul,
// Linear, FeedForward, ScaledDot, MultiHeadAttention, GPT, crossEntropyLoss, backward().
//
// The file is compiled twice (see Makefile): without USE_CUDA into _ref/libref_cpu.so, and with USE_CUDA, against
// the reference tree with the TENSOR_GEMM_BACKEND=b200 binding applied, into _ref_cuda/libref_cuda.so.  In the CUDA
// build ref_use_cuda(1) makes every entry point place its tensors and modules on the GPU, so that the same calls
// run the reference's CUDA path with whichever GEMM backend the environment selects (cuBLAS, custom, b200).
#include <chrono>
#include <cstdint>
#include <cstring>
#include <random>
#include <stdexcept>
#include <string>
#include <vector>

#include "tensor/tensor.h"
#include "nn/linear.h"
#include "nn/ffn.h"
#include "nn/scaledot.h"
#include "nn/multi_head_attention.h"
#include "nn/gpt.h"
#include "nn/layernorm.h"
#include "nn/embedding.h"
#include "loss/CrossEntropyLoss.h"

#define REF_API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_err;
bool g_cuda = false;   // place tensors and modules on the GPU (CUDA build only)

Tensor on_device(const Tensor& t) {
#ifdef USE_CUDA
    if (g_cuda) return t.toDevice(Device::CUDA);
#endif
    return t;
}

// Overwrites a module's parameters (on the host, where the constructors create them) and then moves the module.
template <typename M>
std::vector<Tensor> load_params(M& m, const std::vector<const float*>& values) {
    auto p = m.parameters();
    for (size_t i = 0; i < p.size() && i < values.size(); ++i)
        std::memcpy(p[i].data(), values[i], p[i].numel() * sizeof(float));
#ifdef USE_CUDA
    if (g_cuda) {
        m.to_cuda();
        p = m.parameters();
    }
#endif
    return p;
}

// An operand recipe: contiguous base tensor -> optional view(new shape) -> optional transpose_view(t1, t2)
// -> optional second transpose_view(t3, t4).
struct RefView {
    int32_t ndim;
    int64_t shape[8];
    int32_t view_ndim;      // 0 = no view
    int64_t view_shape[8];
    int32_t t1, t2;         // -1 = no transpose
    int32_t t3, t4;         // -1 = no second transpose
};

Tensor from_host(const float* data, const std::vector<int64_t>& shape) {
    Tensor t(shape, DType::Float32, Device::CPU);
    std::memcpy(t.data(), data, t.numel() * sizeof(float));
    return on_device(t);
}

Tensor tokens_from_host(const int64_t* data, const std::vector<int64_t>& shape) {
    Tensor t(shape, DType::Int64, Device::CPU);
    std::memcpy(t.data(), data, t.numel() * sizeof(int64_t));
    return on_device(t);
}

Tensor build(const float* data, const RefView& v) {
    Tensor t = from_host(data, std::vector<int64_t>(v.shape, v.shape + v.ndim));
    if (v.view_ndim > 0) t = t.view(std::vector<int64_t>(v.view_shape, v.view_shape + v.view_ndim));
    if (v.t1 >= 0) t = t.transpose_view((size_t)v.t1, (size_t)v.t2);
    if (v.t3 >= 0) t = t.transpose_view((size_t)v.t3, (size_t)v.t4);
    return t;
}

void copy_out(const Tensor& t, float* dst) {
    Tensor c = t.contiguous().toDevice(Device::CPU);
    std::memcpy(dst, c.data(), c.numel() * sizeof(float));
}

void copy_grad(const Tensor& leaf, float* dst) {
    if (!dst) return;
    auto g = leaf.grad();
    if (!g) throw std::runtime_error("leaf has no gradient");
    copy_out(*g, dst);
}

// Backpropagates an arbitrary upstream gradient: (y * dY).backward() seeds ones, so y receives dY.
void backward_with(const Tensor& y, const float* dy) {
    Tensor w = from_host(dy, y.shape());
    Tensor z = y * w;
    z.backward();
}

template <typename F>
int guarded(F&& f) {
    try {
        f();
        return 0;
    } catch (const std::exception& e) {
        g_err = e.what();
        return 1;
    }
}

}  // namespace

REF_API const char* ref_last_error() { return g_err.c_str(); }

// 1: run on the GPU from now on (fails in the build without USE_CUDA); 0: on the host.
REF_API int ref_use_cuda(int on) {
#ifdef USE_CUDA
    g_cuda = on != 0;
    return 0;
#else
    if (on) { g_err = "this build of the reference has no CUDA path"; return 1; }
    return 0;
#endif
}

// Tensor::matmul on the reference CPU path.  out may be NULL to query the shape / the thrown message only.
REF_API int ref_matmul(const float* a, const RefView* va, const float* b, const RefView* vb, float* out,
                       int64_t* out_shape, int32_t* out_ndim) {
    return guarded([&] {
        Tensor A = build(a, *va), B = build(b, *vb);
        Tensor C = A.matmul(B);
        if (out_ndim) *out_ndim = (int32_t)C.shape().size();
        if (out_shape) for (size_t i = 0; i < C.shape().size(); ++i) out_shape[i] = C.shape()[i];
        if (out) copy_out(C, out);
    });
}

// Strides the reference gives an operand built from the recipe (to feed the same view to the CUDA backend).
REF_API int ref_view_strides(const RefView* v, int64_t* shape, int64_t* strides, int32_t* ndim) {
    return guarded([&] {
        int64_t n = 1;
        for (int i = 0; i < v->ndim; ++i) n *= v->shape[i];
        std::vector<float> zeros((size_t)n, 0.0f);
        Tensor t = build(zeros.data(), *v);
        *ndim = (int32_t)t.shape().size();
        for (size_t i = 0; i < t.shape().size(); ++i) { shape[i] = t.shape()[i]; strides[i] = t.strides()[i]; }
    });
}

// Int32 matmul (tensor_test.cpp:571-595 pins it); 2-D only.
REF_API int ref_matmul_i32(const int32_t* a, const int32_t* b, int32_t* out, int64_t M, int64_t K, int64_t N) {
    return guarded([&] {
        Tensor A({M, K}, DType::Int32, Device::CPU), B({K, N}, DType::Int32, Device::CPU);
        std::memcpy(A.data(), a, sizeof(int32_t) * M * K);
        std::memcpy(B.data(), b, sizeof(int32_t) * K * N);
        Tensor C = A.matmul(B);
        std::memcpy(out, C.data(), sizeof(int32_t) * M * N);
    });
}

// Linear (optionally followed by gelu, as FeedForward's first half does) forward + backward.
// x: [x_shape...] with last dim = in; w: [out,in]; bias: [out].  dy NULL -> forward only.
REF_API int ref_linear(const float* x, const int64_t* x_shape, int32_t x_ndim, const float* w, const float* bias,
                       int64_t in_f, int64_t out_f, int32_t gelu, const float* dy, float* y, float* preact,
                       float* dx, float* dw, float* db) {
    return guarded([&] {
        Linear lin(in_f, out_f, DType::Float32);
        auto params = load_params(lin, {w, bias});
        Tensor X = from_host(x, std::vector<int64_t>(x_shape, x_shape + x_ndim));
        X.setRequiresGrad(true);
        Tensor pre = lin.forward(X);
        if (preact) copy_out(pre, preact);
        Tensor Y = gelu ? pre.gelu() : pre;
        if (y) copy_out(Y, y);
        if (dy) {
            backward_with(Y, dy);
            copy_grad(X, dx);
            copy_grad(params[0], dw);
            copy_grad(params[1], db);
        }
    });
}

// FeedForward::forward (Linear -> GELU -> Linear) + backward.  Parameter order: w1,b1,w2,b2.
REF_API int ref_ffn(const float* x, const int64_t* x_shape, int32_t x_ndim, int64_t embed, int64_t ff,
                    const float* w1, const float* b1, const float* w2, const float* b2, const float* dy, float* y,
                    float* dx, float* dw1, float* db1, float* dw2, float* db2) {
    return guarded([&] {
        FeedForward ffn(embed, ff, DType::Float32);
        auto p = load_params(ffn, {w1, b1, w2, b2});
        Tensor X = from_host(x, std::vector<int64_t>(x_shape, x_shape + x_ndim));
        X.setRequiresGrad(true);
        Tensor Y = ffn.forward(X);
        if (y) copy_out(Y, y);
        if (dy) {
            backward_with(Y, dy);
            copy_grad(X, dx);
            copy_grad(p[0], dw1); copy_grad(p[1], db1); copy_grad(p[2], dw2); copy_grad(p[3], db2);
        }
    });
}

// ScaledDot::forward.  Operands given by recipe so that both contiguous [B,H,T,d] tensors and the
// MultiHeadAttention views ([B,T,E] -> view [B,T,H,hd] -> transpose_view(1,2)) can be exercised.
REF_API int ref_scaled_dot(const float* q, const RefView* vq, const float* k, const RefView* vk, const float* v,
                           const RefView* vv, const float* d_o, float* o, float* dq, float* dk, float* dv) {
    return guarded([&] {
        Tensor Qb = from_host(q, std::vector<int64_t>(vq->shape, vq->shape + vq->ndim));
        Tensor Kb = from_host(k, std::vector<int64_t>(vk->shape, vk->shape + vk->ndim));
        Tensor Vb = from_host(v, std::vector<int64_t>(vv->shape, vv->shape + vv->ndim));
        Qb.setRequiresGrad(true); Kb.setRequiresGrad(true); Vb.setRequiresGrad(true);
        auto apply = [](Tensor t, const RefView& r) {
            if (r.view_ndim > 0) t = t.view(std::vector<int64_t>(r.view_shape, r.view_shape + r.view_ndim));
            if (r.t1 >= 0) t = t.transpose_view((size_t)r.t1, (size_t)r.t2);
            if (r.t3 >= 0) t = t.transpose_view((size_t)r.t3, (size_t)r.t4);
            return t;
        };
        ScaledDot att;
        Tensor O = att.forward(apply(Qb, *vq), apply(Kb, *vk), apply(Vb, *vv));
        if (o) copy_out(O, o);
        if (d_o) {
            backward_with(O, d_o);
            copy_grad(Qb, dq); copy_grad(Kb, dk); copy_grad(Vb, dv);
        }
    });
}

// LayerNorm::forward + LayerNormBackward over x [rows, D].  dy NULL -> forward only.
REF_API int ref_layernorm(const float* x, int64_t rows, int64_t D, const float* gamma, const float* beta, float eps,
                          const float* dy, float* y, float* dx, float* dgamma, float* dbeta) {
    return guarded([&] {
        LayerNorm ln(D, DType::Float32, eps);
        auto p = load_params(ln, {gamma, beta});
        Tensor X = from_host(x, {rows, D});
        X.setRequiresGrad(true);
        Tensor Y = ln.forward(X);
        if (y) copy_out(Y, y);
        if (dy) {
            backward_with(Y, dy);
            copy_grad(X, dx);
            copy_grad(p[0], dgamma);
            copy_grad(p[1], dbeta);
        }
    });
}

// crossEntropyLoss::forward_batched over logits [B, T, V] and int64 targets [B, T], and its backward (seeded with 1).
REF_API int ref_cross_entropy(const float* logits, const int64_t* targets, int64_t B, int64_t T, int64_t V, float* loss,
                              float* dlogits) {
    return guarded([&] {
        Tensor L = from_host(logits, {B, T, V});
        L.setRequiresGrad(true);
        Tensor tg = tokens_from_host(targets, {B, T});
        crossEntropyLoss ce;
        Tensor l = ce.forward_batched(L, tg);
        if (loss) copy_out(l, loss);
        if (dlogits) {
            l.backward();
            copy_grad(L, dlogits);
        }
    });
}

// Embedding::forward over int64 tokens [B, T] (+ backward of an upstream gradient dout [B, T, D] into the table).
REF_API int ref_embedding(const float* table, int64_t vocab, int64_t D, const int64_t* tokens, int64_t B, int64_t T,
                          const float* dout, float* out, float* dtable) {
    return guarded([&] {
        Embedding emb(vocab, D, DType::Float32);
        auto p = load_params(emb, {table});
        Tensor tk = tokens_from_host(tokens, {B, T});
        Tensor Y = emb.forward(tk);
        if (out) copy_out(Y, out);
        if (dout) {
            backward_with(Y, dout);
            copy_grad(p[0], dtable);
        }
    });
}

// MultiHeadAttention::forward + backward.  Parameter order: wq,bq,wk,bk,wv,bv,wo,bo, each w [E,E].
REF_API int ref_mha(const float* x, int64_t B, int64_t T, int64_t E, int64_t H, const float* const* params,
                    const float* dy, float* y, float* dx, float* const* dparams) {
    return guarded([&] {
        MultiHeadAttention mha(E, H, DType::Float32);
        auto p = load_params(mha, std::vector<const float*>(params, params + 8));
        Tensor X = from_host(x, {B, T, E});
        X.setRequiresGrad(true);
        Tensor Y = mha.forward(X);
        if (y) copy_out(Y, y);
        if (dy) {
            backward_with(Y, dy);
            copy_grad(X, dx);
            if (dparams) for (size_t i = 0; i < p.size(); ++i) copy_grad(p[i], dparams[i]);
        }
    });
}

// One GPT training step's forward + backward (src/benchmarks/gpt_benchmark_gpu.cpp:230-236 without the
// optimizer).  Parameters are taken in GPT::parameters() order from one flat buffer; grads come back the same way.
REF_API int ref_gpt_param_count(int64_t vocab, int64_t max_seq, int64_t E, int64_t H, int64_t L, int64_t ff,
                                int64_t* n_tensors, int64_t* sizes /* capacity 256 */, int64_t* ranks) {
    return guarded([&] {
        GPT model(vocab, max_seq, E, H, L, ff, DType::Float32, 0.0f);
        auto p = model.parameters();
        *n_tensors = (int64_t)p.size();
        for (size_t i = 0; i < p.size() && i < 256; ++i) { sizes[i] = (int64_t)p[i].numel(); ranks[i] = (int64_t)p[i].shape().size(); }
    });
}

REF_API int ref_gpt_step(int64_t vocab, int64_t max_seq, int64_t E, int64_t H, int64_t L, int64_t ff, int64_t batch,
                         int64_t seq, const float* flat_params, const int64_t* tokens, const int64_t* targets,
                         float* loss_out, float* logits_out, float* flat_grads) {
    return guarded([&] {
        GPT model(vocab, max_seq, E, H, L, ff, DType::Float32, 0.0f);
        std::vector<const float*> values;
        size_t off = 0;
        for (auto& t : model.parameters()) {
            values.push_back(flat_params + off);
            off += t.numel();
        }
        auto p = load_params(model, values);
        Tensor tok = tokens_from_host(tokens, {batch, seq}), tgt = tokens_from_host(targets, {batch, seq});
        model.zero_grad();
        Tensor logits = model.forward(tok);
        if (logits_out) copy_out(logits, logits_out);
        crossEntropyLoss ce;
        Tensor loss = ce.forward_batched(logits, tgt);
        copy_out(loss, loss_out);
        if (flat_grads) {
            loss.backward();
            off = 0;
            for (auto& t : p) {
                copy_grad(t, flat_grads + off);
                off += t.numel();
            }
        }
    });
}

#ifdef USE_CUDA
// ------------------------------------------------------------------------------------------------------------------
// CUDA build only (_ref_cuda/libref_cuda.so).  Timing of the reference's own Tensor::matmul / GPT step on the GPU under
// the backend the environment selects, and the same module-level calls as above routed through the fused adapter
// (include/torchengine/te_b200_modules.h) so that its GradFn nodes run inside the reference's autograd engine.
#include <cuda_runtime.h>
#include "core/cuda_utils.h"
#include "torchengine/te_b200_modules.h"

// cuBLAS math mode of the reference's process-wide handle: 0 = default FP32 (what the reference runs),
// 1 = TF32 tensor-op math (a comparator the reference never enables).
REF_API int ref_cuda_cublas_tf32(int on) {
    return guarded([&] {
        cublas_check_error(cublasSetMathMode(cuda_cublas_handle(), on ? CUBLAS_TF32_TENSOR_OP_MATH : CUBLAS_DEFAULT_MATH),
                           "cublasSetMathMode");
    });
}

// C = A.B for row-major [M,K].[K,N] through Tensor::matmul on the GPU with the reference benchmark's inputs
// (std::mt19937(42), uniform(-1,1), A filled first; src/benchmarks/matmul_benchmark.cpp:107-110).  Times `iters`
// calls with CUDA events after `warmup` calls; results are kept alive until after the timing because the reference
// frees each result with cudaFree, which synchronises the device.  out (optional, host) receives the last product.
REF_API int ref_cuda_time_matmul(int64_t M, int64_t K, int64_t N, int32_t warmup, int32_t iters, double* ms_per_call, float* out) {
    return guarded([&] {
        std::mt19937 gen(42);
        std::uniform_real_distribution<float> dist(-1.0f, 1.0f);
        std::vector<float> ha((size_t)M * K), hb((size_t)K * N);
        for (auto& v : ha) v = dist(gen);
        for (auto& v : hb) v = dist(gen);
        Tensor A = from_host(ha.data(), {M, K}).toDevice(Device::CUDA);
        Tensor B = from_host(hb.data(), {K, N}).toDevice(Device::CUDA);
        for (int i = 0; i < warmup; ++i) Tensor C = A.matmul(B);
        cuda_check_error(cudaDeviceSynchronize(), "sync");
        cudaEvent_t e0, e1;
        cudaEventCreate(&e0);
        cudaEventCreate(&e1);
        {
            std::vector<Tensor> keep;
            keep.reserve(iters);
            cudaEventRecord(e0, 0);
            for (int i = 0; i < iters; ++i) keep.push_back(A.matmul(B));
            cudaEventRecord(e1, 0);
            cuda_check_error(cudaEventSynchronize(e1), "event sync");
            float ms = 0.0f;
            cudaEventElapsedTime(&ms, e0, e1);
            if (ms_per_call) *ms_per_call = (double)ms / (iters > 0 ? iters : 1);
            if (out && !keep.empty()) copy_out(keep.back(), out);
        }
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    });
}

// The reference's GPT forward + loss + backward on the GPU (src/benchmarks/gpt_benchmark_gpu.cpp:230-236 without the
// optimizer), `steps` times after `warmup`, wall clock around device synchronisation.
REF_API int ref_cuda_gpt_bench(int64_t vocab, int64_t max_seq, int64_t E, int64_t H, int64_t L, int64_t ff, int64_t batch,
                               int64_t seq, const float* flat_params, const int64_t* tokens, const int64_t* targets,
                               int32_t warmup, int32_t steps, double* ms_per_step, float* loss_out) {
    return guarded([&] {
        const bool was = g_cuda;
        g_cuda = true;
        GPT model(vocab, max_seq, E, H, L, ff, DType::Float32, 0.0f);
        std::vector<const float*> values;
        size_t off = 0;
        for (auto& t : model.parameters()) { values.push_back(flat_params + off); off += t.numel(); }
        load_params(model, values);
        Tensor tok = tokens_from_host(tokens, {batch, seq}), tgt = tokens_from_host(targets, {batch, seq});
        g_cuda = was;
        crossEntropyLoss ce;
        auto one = [&] {
            model.zero_grad();
            Tensor logits = model.forward(tok);
            Tensor loss = ce.forward_batched(logits, tgt);
            loss.backward();
            return loss;
        };
        for (int i = 0; i < warmup; ++i) one();
        cuda_check_error(cudaDeviceSynchronize(), "sync");
        const auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < steps; ++i) {
            Tensor loss = one();
            if (i == steps - 1 && loss_out) copy_out(loss, loss_out);
        }
        cuda_check_error(cudaDeviceSynchronize(), "sync");
        const auto t1 = std::chrono::steady_clock::now();
        if (ms_per_step) *ms_per_step = std::chrono::duration<double, std::milli>(t1 - t0).count() / (steps > 0 ? steps : 1);
    });
}

// --- the fused adapter inside the reference's autograd --------------------------------------------------------------

REF_API int ref_fused_linear(const float* x, const int64_t* x_shape, int32_t x_ndim, const float* w, const float* bias,
                             int64_t in_f, int64_t out_f, int32_t gelu, const float* dy, float* y, float* /*preact: not
                             returned by the fused call*/, float* dx, float* dw, float* db) {
    return guarded([&] {
        const bool was = g_cuda;
        g_cuda = true;
        te_b200::FusedLinear lin(in_f, out_f, DType::Float32);
        auto p = load_params(lin, {w, bias});
        Tensor X = from_host(x, std::vector<int64_t>(x_shape, x_shape + x_ndim));
        X.setRequiresGrad(true);
        Tensor Y = gelu ? te_b200::linear_gelu(X, p[0], p[1]) : lin.forward(X);
        if (y) copy_out(Y, y);
        if (dy) {
            backward_with(Y, dy);
            copy_grad(X, dx); copy_grad(p[0], dw); copy_grad(p[1], db);
        }
        g_cuda = was;
    });
}

REF_API int ref_fused_ffn(const float* x, const int64_t* x_shape, int32_t x_ndim, int64_t embed, int64_t ff,
                          const float* w1, const float* b1, const float* w2, const float* b2, const float* dy, float* y,
                          float* dx, float* dw1, float* db1, float* dw2, float* db2) {
    return guarded([&] {
        const bool was = g_cuda;
        g_cuda = true;
        te_b200::FusedFeedForward ffn(embed, ff, DType::Float32);
        auto p = load_params(ffn, {w1, b1, w2, b2});
        Tensor X = from_host(x, std::vector<int64_t>(x_shape, x_shape + x_ndim));
        X.setRequiresGrad(true);
        Tensor Y = ffn.forward(X);
        if (y) copy_out(Y, y);
        if (dy) {
            backward_with(Y, dy);
            copy_grad(X, dx);
            copy_grad(p[0], dw1); copy_grad(p[1], db1); copy_grad(p[2], dw2); copy_grad(p[3], db2);
        }
        g_cuda = was;
    });
}

REF_API int ref_fused_scaled_dot(const float* q, const RefView* vq, const float* k, const RefView* vk, const float* v,
                                 const RefView* vv, const float* d_o, float* o, float* dq, float* dk, float* dv) {
    return guarded([&] {
        const bool was = g_cuda;
        g_cuda = true;
        Tensor Qb = from_host(q, std::vector<int64_t>(vq->shape, vq->shape + vq->ndim));
        Tensor Kb = from_host(k, std::vector<int64_t>(vk->shape, vk->shape + vk->ndim));
        Tensor Vb = from_host(v, std::vector<int64_t>(vv->shape, vv->shape + vv->ndim));
        Qb.setRequiresGrad(true); Kb.setRequiresGrad(true); Vb.setRequiresGrad(true);
        auto apply = [](Tensor t, const RefView& r) {
            if (r.view_ndim > 0) t = t.view(std::vector<int64_t>(r.view_shape, r.view_shape + r.view_ndim));
            if (r.t1 >= 0) t = t.transpose_view((size_t)r.t1, (size_t)r.t2);
            if (r.t3 >= 0) t = t.transpose_view((size_t)r.t3, (size_t)r.t4);
            return t;
        };
        Tensor O = te_b200::scaled_dot(apply(Qb, *vq), apply(Kb, *vk), apply(Vb, *vv));
        if (o) copy_out(O, o);
        if (d_o) {
            backward_with(O, d_o);
            copy_grad(Qb, dq); copy_grad(Kb, dk); copy_grad(Vb, dv);
        }
        g_cuda = was;
    });
}

REF_API int ref_fused_mha(const float* x, int64_t B, int64_t T, int64_t E, int64_t H, const float* const* params,
                          const float* dy, float* y, float* dx, float* const* dparams) {
    return guarded([&] {
        const bool was = g_cuda;
        g_cuda = true;
        te_b200::FusedMultiHeadAttention mha(E, H, DType::Float32);
        auto p = load_params(mha, std::vector<const float*>(params, params + 8));
        Tensor X = from_host(x, {B, T, E});
        X.setRequiresGrad(true);
        Tensor Y = mha.forward(X);
        if (y) copy_out(Y, y);
        if (dy) {
            backward_with(Y, dy);
            copy_grad(X, dx);
            if (dparams) for (size_t i = 0; i < p.size(); ++i) copy_grad(p[i], dparams[i]);
        }
        g_cuda = was;
    });
}
#endif  // USE_CUDA
