// te_b200_modules.h -- reference-side adapter: the fused callers of the B200 backend expressed with
// TorchEngine's own types (Tensor, GradFn, Module), for a build of TorchEngine that has the
// TENSOR_GEMM_BACKEND=b200 binding (b200_backend.patch, same directory) applied.
//
// Include it from TorchEngine code after "tensor/tensor.h" with TorchEngine's src/ directory and the
// directory of te_b200.h on the include path, and link libte_b200.so.  Every function below takes and
// returns TorchEngine tensors on Device::CUDA and records ONE GradFn node where the stock modules record
// several; the node's backward() returns the gradients in the order and shapes the stock nodes produce:
//
//   te_b200::linear(x, W, b)            Linear::forward (src/nn/linear.cpp:14-23): matmul + bias in one kernel;
//                                        backward {dX, dW[out,in], db[out]} replaces MatMulBackward + AddBackward +
//                                        TransposeBackward + reduce_gradient (src/core/grad_fn.cpp:13-58, :93-139, :397-403)
//   te_b200::linear_gelu(x, W, b)       the first half of FeedForward::forward (src/nn/ffn.cpp:12-14) with the GELU
//                                        in the GEMM epilogue; backward adds GeluBackward (grad_fn.cpp:169-204)
//   te_b200::feed_forward(...)          FeedForward::forward (src/nn/ffn.cpp:12-16)
//   te_b200::scaled_dot(Q, K, V)        ScaledDot::forward (src/nn/scaledot.cpp:8-27) on [.., T, d] views; backward
//                                        {dQ, dK, dV} replaces MatMulBackward x2, SoftmaxBackward, DivBackward
//                                        (grad_fn.cpp:126-156, :569-665)
//   te_b200::multi_head_attention(...)  MultiHeadAttention::forward (src/nn/multi_head_attention.cpp:19-42); the head
//                                        split and merge are strides handed to the attention call, not copies
//
// FusedLinear / FusedFeedForward / FusedMultiHeadAttention are Module subclasses that own the stock module (so
// parameters(), zero_grad() and to_cuda() are the stock ones) and override forward() with the calls above.
// There is no CPU path: a tensor that is not on Device::CUDA is refused with std::runtime_error.
#ifndef TE_B200_MODULES_H
#define TE_B200_MODULES_H

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "tensor/tensor.h"
#include "nn/module.h"
#include "nn/linear.h"
#include "nn/ffn.h"
#include "nn/multi_head_attention.h"
#include "te_b200.h"

namespace te_b200 {

inline int precision_from_env() {
    const char* p = std::getenv("TENSOR_GEMM_PRECISION");
    return (p && std::strcmp(p, "3xtf32") == 0) ? TE_PREC_3XTF32 : TE_PREC_TF32;
}

inline void check(int rc) {
    if (rc) throw std::runtime_error(te_b200_last_error());
}

inline void require_cuda(const Tensor& t, const char* who) {
    if (t.device() != Device::CUDA || t.dtype() != DType::Float32)
        throw std::runtime_error(std::string(who) + ": the B200 backend takes Float32 tensors on Device::CUDA only");
}

inline const float* cptr(const Tensor& t) { return static_cast<const float*>(t.data()); }
inline float* mptr(Tensor& t) { return static_cast<float*>(t.data()); }

inline Tensor dense(const Tensor& t) { return t.is_contiguous() ? t : t.contiguous(); }

// ---------------------------------------------------------------------------------------------- Linear

class LinearBackward : public GradFn {   // inputs = {x, W, b}
public:
    std::vector<Tensor> saved;           // linear_gelu stores the value before the GELU here
    bool has_gelu = false;
    std::vector<Tensor> backward(const Tensor& upstream) override {
        const Tensor& x = inputs[0];
        const Tensor& W = inputs[1];
        const int64_t out_f = W.shape()[0], in_f = W.shape()[1];
        const int64_t rows = static_cast<int64_t>(x.numel()) / in_f;
        Tensor dy = dense(upstream);
        if (has_gelu) {                  // GeluBackward: dPre = dY * gelu'(pre), into a fresh buffer (dy may be shared)
            Tensor dpre(dy.shape(), DType::Float32, Device::CUDA);
            check(te_b200_gelu_backward_f32(cuda_b200_ctx(), cptr(saved[0]), cptr(dy), mptr(dpre),
                                            static_cast<int64_t>(dy.numel()), nullptr));
            dy = dpre;
        }
        Tensor xd = dense(x);
        Tensor dx(x.shape(), DType::Float32, Device::CUDA);
        Tensor dw(W.shape(), DType::Float32, Device::CUDA);
        Tensor db(inputs[2].shape(), DType::Float32, Device::CUDA);
        check(te_b200_linear_backward(cuda_b200_ctx(), cptr(xd), cptr(W), cptr(dy), mptr(dx), mptr(dw), mptr(db), rows,
                                      in_f, out_f, precision_from_env(), nullptr));
        return {dx, dw, db};
    }
};

inline Tensor linear_impl(const Tensor& x, const Tensor& W, const Tensor& b, bool gelu) {
    require_cuda(x, "te_b200::linear");
    require_cuda(W, "te_b200::linear");
    require_cuda(b, "te_b200::linear");
    if (W.shape().size() != 2 || !W.is_contiguous()) throw std::runtime_error("te_b200::linear: weight must be a contiguous [out, in] tensor");
    const int64_t out_f = W.shape()[0], in_f = W.shape()[1];
    if (x.shape().empty() || x.shape().back() != in_f) throw std::runtime_error("Inner dimensions must match for matmul");
    Tensor xd = dense(x);
    const int64_t rows = static_cast<int64_t>(x.numel()) / in_f;
    std::vector<int64_t> yshape = x.shape();
    yshape.back() = out_f;
    Tensor y(yshape, DType::Float32, Device::CUDA);
    const bool needs_grad = x.requiredGrad() || W.requiredGrad() || b.requiredGrad();
    auto fn = std::make_shared<LinearBackward>();
    float* pre = nullptr;
    if (gelu && needs_grad) {
        fn->saved.emplace_back(yshape, DType::Float32, Device::CUDA);
        fn->has_gelu = true;
        pre = mptr(fn->saved[0]);
    }
    check(te_b200_linear_forward(cuda_b200_ctx(), cptr(xd), cptr(W), cptr(b), mptr(y), pre, rows, in_f, out_f, gelu ? 1 : 0,
                                 precision_from_env(), nullptr));
    if (needs_grad) {
        fn->inputs = {x, W, b};
        y.setRequiresGrad(true);
        y.setGradFn(fn);
    }
    return y;
}

inline Tensor linear(const Tensor& x, const Tensor& W, const Tensor& b) { return linear_impl(x, W, b, false); }
inline Tensor linear_gelu(const Tensor& x, const Tensor& W, const Tensor& b) { return linear_impl(x, W, b, true); }

inline Tensor feed_forward(const Tensor& x, const Tensor& W1, const Tensor& b1, const Tensor& W2, const Tensor& b2) {
    return linear(linear_gelu(x, W1, b1), W2, b2);
}

// ---------------------------------------------------------------------------------------------- attention

// [.., T, d] operand with unit stride over d, seen as [B, H, T, d]: 4-D as is, 3-D with H = 1, 2-D with B = H = 1.
struct BhtdView {
    int64_t B, H, T, d;
    int64_t strides[3];
};
inline BhtdView bhtd(const Tensor& t, const char* who) {
    const auto& sh = t.shape();
    const auto& st = t.strides();
    const size_t n = sh.size();
    if (n < 2 || n > 4) throw std::runtime_error(std::string(who) + ": operands must have 2 to 4 dimensions");
    if (st[n - 1] != 1 && sh[n - 1] != 1) throw std::runtime_error("CUDA matmul only supports row- or column-major 2D slices");
    BhtdView v;
    v.d = sh[n - 1];
    v.T = sh[n - 2];
    v.H = n >= 3 ? sh[n - 3] : 1;
    v.B = n >= 4 ? sh[n - 4] : 1;
    v.strides[2] = st[n - 2];
    v.strides[1] = n >= 3 ? st[n - 3] : v.T * v.d;
    v.strides[0] = n >= 4 ? st[n - 4] : v.H * v.T * v.d;
    return v;
}

// A gradient buffer for `t`: dense, except that a head view [B, H, T, d] taken from a [B, T, H*d] tensor (heads
// strided inside the sequence step, as MultiHeadAttention::forward builds them) gets the same memory order, so that
// TransposeBackward's transpose_view().contiguous() (src/core/grad_fn.cpp:397-403) finds it contiguous already.
inline Tensor grad_like(const Tensor& t) {
    const auto& sh = t.shape();
    const auto& st = t.strides();
    if (sh.size() == 4 && st[3] == 1 && st[1] == sh[3] && st[2] == sh[1] * sh[3])
        return Tensor({sh[0], sh[2], sh[1], sh[3]}, DType::Float32, Device::CUDA).transpose_view(1, 2);
    return Tensor(sh, DType::Float32, Device::CUDA);
}

class ScaledDotBackward : public GradFn {   // inputs = {Q, K, V}
public:
    std::vector<Tensor> saved;              // {P [B,H,T,T] dense, O the forward output}
    std::vector<Tensor> backward(const Tensor& upstream) override {
        const Tensor& Q = inputs[0];
        const Tensor& K = inputs[1];
        const Tensor& V = inputs[2];
        const BhtdView q = bhtd(Q, "te_b200::scaled_dot"), k = bhtd(K, "te_b200::scaled_dot"), v = bhtd(V, "te_b200::scaled_dot");
        Tensor dO = upstream;
        if (dO.strides().back() != 1) dO = dO.contiguous();
        const Tensor& P = saved[0];
        const Tensor& O = saved[1];
        const BhtdView g = bhtd(dO, "te_b200::scaled_dot"), o = bhtd(O, "te_b200::scaled_dot");
        Tensor dq = grad_like(Q), dk = grad_like(K), dv = grad_like(V);
        const BhtdView gq = bhtd(dq, "te_b200::scaled_dot"), gk = bhtd(dk, "te_b200::scaled_dot"), gv = bhtd(dv, "te_b200::scaled_dot");
        te_attn_bwd_desc t;
        std::memset(&t, 0, sizeof t);
        t.B = q.B; t.H = q.H; t.T = q.T; t.d = q.d;
        t.q = cptr(Q); t.k = cptr(K); t.v = cptr(V);
        t.p = cptr(P); t.o = cptr(O); t.d_o = cptr(dO);
        t.dq = mptr(dq); t.dk = mptr(dk); t.dv = mptr(dv);
        for (int i = 0; i < 3; ++i) {
            t.q_strides[i] = q.strides[i]; t.k_strides[i] = k.strides[i]; t.v_strides[i] = v.strides[i];
            t.o_strides[i] = o.strides[i]; t.d_o_strides[i] = g.strides[i];
            t.dq_strides[i] = gq.strides[i]; t.dk_strides[i] = gk.strides[i]; t.dv_strides[i] = gv.strides[i];
        }
        t.precision = precision_from_env();
        check(te_b200_attention_backward(cuda_b200_ctx(), &t, nullptr));
        return {dq, dk, dv};
    }
};

// out_strides (optional): element strides for B, H, T of the output inside `out`, which the caller allocated; used by
// multi_head_attention to have the heads written straight into the merged [B, T, E] layout.
inline Tensor scaled_dot_into(const Tensor& Q, const Tensor& K, const Tensor& V, Tensor out, const int64_t* out_strides,
                              std::shared_ptr<ScaledDotBackward>* node_out) {
    require_cuda(Q, "te_b200::scaled_dot");
    require_cuda(K, "te_b200::scaled_dot");
    require_cuda(V, "te_b200::scaled_dot");
    const BhtdView q = bhtd(Q, "te_b200::scaled_dot"), k = bhtd(K, "te_b200::scaled_dot"), v = bhtd(V, "te_b200::scaled_dot");
    if (k.B != q.B || k.H != q.H || v.B != q.B || v.H != q.H || k.d != q.d || v.T != k.T)
        throw std::runtime_error("Inner dimensions must match for matmul");
    if (k.T != q.T || v.d != q.d) throw std::runtime_error("te_b200::scaled_dot: Q, K and V must share [B, H, T, d]");
    Tensor P({q.B, q.H, q.T, q.T}, DType::Float32, Device::CUDA);
    te_attn_desc t;
    std::memset(&t, 0, sizeof t);
    t.B = q.B; t.H = q.H; t.T = q.T; t.d = q.d;
    t.q = cptr(Q); t.k = cptr(K); t.v = cptr(V);
    t.p_out = mptr(P);
    t.o = mptr(out);
    for (int i = 0; i < 3; ++i) {
        t.q_strides[i] = q.strides[i]; t.k_strides[i] = k.strides[i]; t.v_strides[i] = v.strides[i];
        t.o_strides[i] = out_strides[i];
    }
    t.precision = precision_from_env();
    check(te_b200_attention_forward(cuda_b200_ctx(), &t, nullptr));
    if (Q.requiredGrad() || K.requiredGrad() || V.requiredGrad()) {
        auto fn = std::make_shared<ScaledDotBackward>();
        fn->inputs = {Q, K, V};
        fn->saved = {P, out};
        if (node_out) *node_out = fn;
        else {
            out.setRequiresGrad(true);
            out.setGradFn(fn);
        }
    }
    return out;
}

inline Tensor scaled_dot(const Tensor& Q, const Tensor& K, const Tensor& V) {
    Tensor out(Q.shape(), DType::Float32, Device::CUDA);
    const BhtdView o = bhtd(out, "te_b200::scaled_dot");
    return scaled_dot_into(Q, K, V, out, o.strides, nullptr);
}

// ---------------------------------------------------------------------------------------------- multi-head attention

// The merge step of MultiHeadAttention::forward (transpose_view(1,2) + reshape, a gather copy and a ReshapeBackward
// node in the stock code) as a stride trick: the attention output for [B, H, T, hd] is written with strides
// [T*E, hd, E] into a [B, T, E] tensor, and the upstream gradient of that tensor is read with the same strides.
class MergedHeadsBackward : public GradFn {   // inputs = {Q, K, V} head views
public:
    std::shared_ptr<ScaledDotBackward> core;
    int64_t B, H, T, hd;
    std::vector<Tensor> backward(const Tensor& upstream) override {
        Tensor g = dense(upstream);               // [B, T, E]
        Tensor as_heads = g.view({B, T, H, hd}).transpose_view(1, 2);
        return core->backward(as_heads);
    }
};

// params in MultiHeadAttention::parameters() order: Wq, bq, Wk, bk, Wv, bv, Wo, bo.
inline Tensor multi_head_attention(const Tensor& x, const std::vector<Tensor>& params, int64_t heads) {
    if (params.size() != 8) throw std::runtime_error("te_b200::multi_head_attention: expected 8 parameter tensors");
    if (x.shape().size() != 3) throw std::runtime_error("te_b200::multi_head_attention: input must be [batch, seq, embed]");
    const int64_t B = x.shape()[0], T = x.shape()[1], E = x.shape()[2];
    if (heads < 1 || E % heads != 0) throw std::runtime_error("embedDim must be divisible by numHeads");
    const int64_t hd = E / heads;
    auto split = [&](const Tensor& t) { return t.view({B, T, heads, hd}).transpose_view(1, 2); };
    Tensor Q = split(linear(x, params[0], params[1]));
    Tensor K = split(linear(x, params[2], params[3]));
    Tensor V = split(linear(x, params[4], params[5]));
    Tensor merged({B, T, E}, DType::Float32, Device::CUDA);
    const int64_t merged_strides[3] = {T * E, hd, E};
    std::shared_ptr<ScaledDotBackward> core;
    scaled_dot_into(Q, K, V, merged, merged_strides, &core);
    if (core) {
        core->saved[1] = merged.view({B, T, heads, hd}).transpose_view(1, 2);
        auto fn = std::make_shared<MergedHeadsBackward>();
        fn->inputs = {Q, K, V};
        fn->core = core;
        fn->B = B; fn->H = heads; fn->T = T; fn->hd = hd;
        merged.setRequiresGrad(true);
        merged.setGradFn(fn);
    }
    return linear(merged, params[6], params[7]);
}

// ---------------------------------------------------------------------------------------------- Module wrappers

class FusedLinear : public Module {
public:
    FusedLinear(int64_t in_features, int64_t out_features, DType dtype) : inner_(in_features, out_features, dtype) {}
    Tensor forward(const Tensor& input) override { return linear(input, inner_.weight(), inner_.bias()); }
    std::vector<Tensor> parameters() override { return inner_.parameters(); }
    void zero_grad() override { inner_.zero_grad(); }
    void to_cuda() override { inner_.to_cuda(); }
    Linear& stock() { return inner_; }
private:
    Linear inner_;
};

class FusedFeedForward : public Module {
public:
    FusedFeedForward(int64_t embed_dim, int64_t ff_dim, DType dtype) : inner_(embed_dim, ff_dim, dtype) {}
    Tensor forward(const Tensor& input) override {
        auto p = inner_.parameters();   // w1, b1, w2, b2
        return feed_forward(input, p[0], p[1], p[2], p[3]);
    }
    std::vector<Tensor> parameters() override { return inner_.parameters(); }
    void zero_grad() override { inner_.zero_grad(); }
    void to_cuda() override { inner_.to_cuda(); }
    FeedForward& stock() { return inner_; }
private:
    FeedForward inner_;
};

class FusedMultiHeadAttention : public Module {
public:
    FusedMultiHeadAttention(int64_t embed_dim, int64_t num_heads, DType dtype) : inner_(embed_dim, num_heads, dtype), heads_(num_heads) {}
    Tensor forward(const Tensor& input) override { return multi_head_attention(input, inner_.parameters(), heads_); }
    std::vector<Tensor> parameters() override { return inner_.parameters(); }
    void zero_grad() override { inner_.zero_grad(); }
    void to_cuda() override { inner_.to_cuda(); }
    MultiHeadAttention& stock() { return inner_; }
private:
    MultiHeadAttention inner_;
    int64_t heads_;
};

}  // namespace te_b200

#endif  // TE_B200_MODULES_H
