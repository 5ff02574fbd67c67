// te_b200.hpp -- header-only C++17 host adapter over the C ABI of te_b200.h.
//
// It carries the names and calling conventions of the reference's host API for the matmul path, so that code
// written against the reference reads the same here:
//   te::Tensor          Tensor(shape, dtype=Float32, Device::CUDA), shape(), strides(), data(), view(),
//                       transpose_view(d1, d2), matmul(other)        (reference src/tensor/tensor.h:92-130, :908)
//   te::Linear          forward(x) = x.matmul(W.transpose_view(1,0)) + b   (reference src/nn/linear.cpp:14-23)
//   te::FeedForward     Linear -> GELU -> Linear                           (reference src/nn/ffn.cpp:12-16)
//   te::ScaledDot       softmax(Q.K^T / sqrt(d)).V and its backward        (reference src/nn/scaledot.cpp:8-27)
//   te::LayerNorm, te::Embedding, te::cross_entropy: the GPT step's kernels around the matmuls
//                       (reference src/nn/layernorm.cpp, src/nn/embedding.cpp, src/loss/CrossEntropyLoss.cpp)
// Errors surface as std::runtime_error with the reference's texts (src/tensor/tensor.h:537, :547, :626, :858).
// Tensors live on the GPU only: this backend has no CPU compute path.  Each Tensor owns (or shares) one device
// buffer from te::CachingAllocator (the reference's CUDAAllocator calls cudaMalloc per tensor, src/core/allocators.h:35-52).
#pragma once
#include <cuda_runtime.h>

#include <cmath>
#include <cstdlib>
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

#include "te_b200.h"

namespace te {

inline void check(int rc) {
    if (rc != TE_OK) {
        const char* msg = te_b200_last_error();
        throw std::runtime_error((msg && *msg) ? msg : te_b200_status_string(rc));
    }
}
inline void cuda_check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// One context per process and device, created on first use (the role of cuda_cublas_handle(),
// reference src/core/cuda_utils.cpp:48-55).  TENSOR_GEMM_PRECISION=3xtf32 selects the FP32-accurate mode.
class Backend {
public:
    static Backend& instance() {
        static Backend b;
        return b;
    }
    te_b200_ctx* ctx() const { return ctx_; }
    int precision() const { return precision_; }
    void set_precision(int p) { precision_ = p; }
    void synchronize() {
        cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
        check(te_b200_check_device_status(ctx_));
    }
private:
    Backend() {
        check(te_b200_init(0, size_t(1) << 30, &ctx_));
        const char* p = std::getenv("TENSOR_GEMM_PRECISION");
        precision_ = (p && std::string(p) == "3xtf32") ? TE_PREC_3XTF32 : TE_PREC_TF32;
    }
    ~Backend() { te_b200_destroy(ctx_); }
    te_b200_ctx* ctx_ = nullptr;
    int precision_ = TE_PREC_TF32;
};

// The CUDA stream this thread's adapter calls are issued on.  Default: the legacy default stream, like the reference's
// launches.  StreamGuard switches it for a scope.  One te_b200 context serves the process, so calls that use its
// workspace must not run concurrently on two streams (te_b200.h); one thread moving from stream to stream is fine.
inline cudaStream_t& current_stream_slot() {
    static thread_local cudaStream_t s = nullptr;
    return s;
}
inline cudaStream_t current_stream() { return current_stream_slot(); }
class StreamGuard {
public:
    explicit StreamGuard(cudaStream_t s) : previous_(current_stream_slot()) { current_stream_slot() = s; }
    ~StreamGuard() { current_stream_slot() = previous_; }
    StreamGuard(const StreamGuard&) = delete;
    StreamGuard& operator=(const StreamGuard&) = delete;
private:
    cudaStream_t previous_;
};

// Device memory for tensors, cached by block size, with stream-ordered reuse.  The reference's CUDAAllocator calls
// cudaMalloc / cudaFree for every tensor (src/core/allocators.h:35-52); both synchronise the device, and a training step
// creates hundreds of temporaries.  Here a freed block goes to a free list of its (rounded) size and the next tensor
// of that size takes it without touching the driver and without waiting for the GPU:
//   * a block belongs to the stream that was current when it was allocated (plus any stream named through
//     record_stream); freeing it costs nothing, because work queued on that stream after the free runs after the
//     block's last use anyway;
//   * a request from the same stream takes the block as it is; a request from another stream takes it after making
//     that stream wait (cudaStreamWaitEvent, no host wait) for an event recorded now on the block's streams.
// set_caching(false) turns it into the reference's behaviour (cudaMalloc / cudaFree per tensor) for comparisons.
class CachingAllocator {
public:
    static CachingAllocator& instance() {
        static CachingAllocator* a = new CachingAllocator();   // never destroyed: tensors with static lifetime may outlive any static
        return *a;
    }
    static size_t rounded(size_t bytes) {
        if (bytes < 512) return 512;
        if (bytes < (size_t(1) << 20)) return (bytes + 511) & ~size_t(511);
        return (bytes + (size_t(2) << 20) - 1) & ~((size_t(2) << 20) - 1);      // large blocks in 2 MiB steps
    }
    void* allocate(size_t bytes, size_t* block_bytes) { return allocate(bytes, block_bytes, current_stream()); }
    void* allocate(size_t bytes, size_t* block_bytes, cudaStream_t stream) {
        const size_t n = rounded(bytes);
        *block_bytes = n;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto range = free_.equal_range(n);
            auto pick = range.second;
            for (auto it = range.first; it != range.second; ++it) {
                if (it->second.used_only_on(stream)) { pick = it; break; }      // same stream: no ordering needed
                if (pick == range.second) pick = it;
            }
            if (pick != range.second) {
                Block blk = std::move(pick->second);
                free_.erase(pick);
                if (!blk.used_only_on(stream)) {
                    order_after(stream, blk.stream);
                    for (cudaStream_t s : blk.also) order_after(stream, s);
                    ++cross_stream_reuses_;
                }
                ++hits_;
                live_[blk.ptr] = Block{blk.ptr, stream, {}};
                return blk.ptr;
            }
        }
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, n);
        if (e != cudaSuccess) {          // out of memory: give the cached blocks back to the driver and retry once
            cudaGetLastError();
            empty_cache();
            e = cudaMalloc(&p, n);
        }
        cuda_check(e, "cudaMalloc");
        std::lock_guard<std::mutex> g(mu_);
        ++device_mallocs_;
        live_[p] = Block{p, stream, {}};
        return p;
    }
    // The block is (also) used by work on `stream`: reuse from any other stream will wait for that work too.
    void record_stream(void* p, cudaStream_t stream) {
        std::lock_guard<std::mutex> g(mu_);
        auto it = live_.find(p);
        if (it == live_.end() || it->second.stream == stream) return;
        for (cudaStream_t s : it->second.also)
            if (s == stream) return;
        it->second.also.push_back(stream);
    }
    void release(void* p, size_t block_bytes) {
        bool give_back = false;
        {
            std::lock_guard<std::mutex> g(mu_);
            auto it = live_.find(p);
            Block blk = it != live_.end() ? std::move(it->second) : Block{p, nullptr, {}};
            if (it != live_.end()) live_.erase(it);
            if (caching_) free_.emplace(block_bytes, std::move(blk));
            else give_back = true;
        }
        if (give_back) cudaFree(p);      // waits for the device, as the reference's allocator does
    }
    void empty_cache() {
        std::multimap<size_t, Block> blocks;
        {
            std::lock_guard<std::mutex> g(mu_);
            blocks.swap(free_);
        }
        for (auto& kv : blocks) cudaFree(kv.second.ptr);
    }
    void set_caching(bool on) {
        {
            std::lock_guard<std::mutex> g(mu_);
            caching_ = on;
        }
        if (!on) empty_cache();
    }
    size_t device_mallocs() const { return device_mallocs_; }            // cudaMalloc calls so far
    size_t cache_hits() const { return hits_; }
    size_t cross_stream_reuses() const { return cross_stream_reuses_; }  // hits that had to order one stream after another
private:
    struct Block {
        void* ptr;
        cudaStream_t stream;                 // the stream the block was allocated for
        std::vector<cudaStream_t> also;      // further streams named through record_stream
        bool used_only_on(cudaStream_t s) const { return stream == s && also.empty(); }
    };
    CachingAllocator() = default;
    // Work queued on `waiter` from now on runs after everything queued on `other` so far.  Called with mu_ held.
    void order_after(cudaStream_t waiter, cudaStream_t other) {
        if (waiter == other) return;
        if (!event_) cuda_check(cudaEventCreateWithFlags(&event_, cudaEventDisableTiming), "cudaEventCreateWithFlags");
        cuda_check(cudaEventRecord(event_, other), "cudaEventRecord");
        cuda_check(cudaStreamWaitEvent(waiter, event_, 0), "cudaStreamWaitEvent");   // captures the record above; the event may be re-recorded at once
    }
    std::mutex mu_;
    std::multimap<size_t, Block> free_;
    std::map<void*, Block> live_;
    cudaEvent_t event_ = nullptr;
    bool caching_ = true;
    size_t device_mallocs_ = 0, hits_ = 0, cross_stream_reuses_ = 0;
};

class Tensor {
public:
    Tensor() = default;
    explicit Tensor(std::vector<int64_t> shape) : shape_(std::move(shape)) {
        strides_.assign(shape_.size(), 1);
        for (int i = (int)shape_.size() - 2; i >= 0; --i) strides_[i] = strides_[i + 1] * shape_[i + 1];
        const size_t n = numel();
        size_t block = 0;
        void* p = CachingAllocator::instance().allocate((n ? n : 1) * sizeof(float), &block);
        storage_ = std::shared_ptr<void>(p, [block](void* q) { CachingAllocator::instance().release(q, block); });
    }
    static Tensor from_host(const std::vector<float>& v, std::vector<int64_t> shape) {
        Tensor t(std::move(shape));
        if (v.size() != t.numel()) throw std::runtime_error("from_host: element count does not match the shape");
        cuda_check(cudaMemcpyAsync(t.data(), v.data(), v.size() * sizeof(float), cudaMemcpyHostToDevice, current_stream()), "cudaMemcpy H2D");
        cuda_check(cudaStreamSynchronize(current_stream()), "cudaStreamSynchronize");      // v may go away after the call
        return t;
    }
    // Row-major copy of the logical contents (views are gathered on the host side).
    std::vector<float> to_host() const {
        int64_t lo = 0, hi = 0;   // span of the view inside the storage, relative to offset_
        for (size_t i = 0; i < shape_.size(); ++i)
            if (shape_[i] > 0) (strides_[i] >= 0 ? hi : lo) += (shape_[i] - 1) * strides_[i];
        std::vector<float> raw((size_t)(hi - lo + 1));
        std::vector<float> out(numel());
        if (out.empty()) return out;
        cuda_check(cudaMemcpyAsync(raw.data(), data() + lo, raw.size() * sizeof(float), cudaMemcpyDeviceToHost, current_stream()), "cudaMemcpy D2H");
        cuda_check(cudaStreamSynchronize(current_stream()), "cudaStreamSynchronize");
        std::vector<int64_t> idx(shape_.size(), 0);
        for (size_t flat = 0; flat < out.size(); ++flat) {
            int64_t off = -lo;
            for (size_t d = 0; d < shape_.size(); ++d) off += idx[d] * strides_[d];
            out[flat] = raw[(size_t)off];
            for (int d = (int)shape_.size() - 1; d >= 0; --d) {
                if (++idx[d] < shape_[d]) break;
                idx[d] = 0;
            }
        }
        return out;
    }

    size_t numel() const {
        size_t n = 1;
        for (int64_t d : shape_) n *= (size_t)d;
        return n;
    }
    const std::vector<int64_t>& shape() const { return shape_; }
    const std::vector<int64_t>& strides() const { return strides_; }   // in elements
    float* data() const { return static_cast<float*>(storage_.get()) + offset_; }   // includes the view offset
    // Tells the allocator that work on `stream` (other than the one the tensor was created on) uses this tensor.
    void record_stream(cudaStream_t stream) const { CachingAllocator::instance().record_stream(storage_.get(), stream); }
    bool is_contiguous() const {
        int64_t run = 1;
        for (int i = (int)shape_.size() - 1; i >= 0; --i) {
            if (shape_[i] != 1 && strides_[i] != run) return false;
            run *= shape_[i];
        }
        return true;
    }

    // Zero-copy stride swap (reference src/tensor/tensor.cpp:590-620).
    Tensor transpose_view(size_t d1, size_t d2) const {
        if (d1 >= shape_.size() || d2 >= shape_.size()) throw std::runtime_error("transpose_view: dimension out of range");
        Tensor t = *this;
        std::swap(t.shape_[d1], t.shape_[d2]);
        std::swap(t.strides_[d1], t.strides_[d2]);
        return t;
    }
    // Zero-copy reshape of a contiguous tensor (reference src/tensor/tensor.cpp:233-255).
    Tensor view(const std::vector<int64_t>& new_shape) const {
        if (!is_contiguous()) throw std::runtime_error("view requires a contiguous tensor");
        size_t n = 1;
        for (int64_t d : new_shape) n *= (size_t)d;
        if (n != numel()) throw std::runtime_error("view: element count mismatch");
        Tensor t = *this;
        t.shape_ = new_shape;
        t.strides_.assign(new_shape.size(), 1);
        for (int i = (int)new_shape.size() - 2; i >= 0; --i) t.strides_[i] = t.strides_[i + 1] * new_shape[i + 1];
        return t;
    }

    // Tensor::matmul (reference src/tensor/tensor.cpp:761-785): >= 2-D operands, NumPy batch broadcasting,
    // fresh contiguous result; asynchronous on the legacy default stream like the reference's launches.
    Tensor matmul(const Tensor& other) const {
        int64_t out_shape[8];
        int out_ndim = 0;
        check(te_b200_matmul_nd(nullptr, nullptr, shape_.data(), strides_.data(), (int)shape_.size(), nullptr,
                                other.shape_.data(), other.strides_.data(), (int)other.shape_.size(), nullptr, out_shape,
                                &out_ndim, TE_PREC_TF32, nullptr));
        Tensor result(std::vector<int64_t>(out_shape, out_shape + out_ndim));
        Backend& be = Backend::instance();
        check(te_b200_matmul_nd(be.ctx(), data(), shape_.data(), strides_.data(), (int)shape_.size(), other.data(),
                                other.shape_.data(), other.strides_.data(), (int)other.shape_.size(), result.data(),
                                nullptr, nullptr, be.precision(), current_stream()));
        return result;
    }

private:
    std::shared_ptr<void> storage_;
    std::vector<int64_t> shape_, strides_;
    int64_t offset_ = 0;
};

// MatMulBackward::backward (reference src/core/grad_fn.cpp:126-139): for C = A.matmul(B) and upstream gradient dC,
//   dA = dC . B^T,  dB = A^T . dC   (both through transpose_view, no copies),
// each summed over the batch dimensions the operand was broadcast along (reduce_gradient, grad_fn.cpp:13-58).
struct MatMulBackward {
    Tensor a, b;   // the inputs of the forward call, held by value like GradFn::inputs
    std::vector<Tensor> backward(const Tensor& dC) const {
        const size_t na = a.shape().size(), nb = b.shape().size();
        Tensor dA = dC.matmul(b.transpose_view(nb - 2, nb - 1));
        Tensor dB = a.transpose_view(na - 2, na - 1).matmul(dC);
        return {reduce_to(dA, a.shape()), reduce_to(dB, b.shape())};
    }
private:
    // Sums the leading (broadcast) batch dimensions of `g` away so that it has `shape`.  Supports the cases the
    // reference's callers produce: the operand had no batch dimensions, or all-ones batch dimensions.
    static Tensor reduce_to(const Tensor& g, const std::vector<int64_t>& shape) {
        if (g.shape() == shape) return g;
        size_t target = 1;
        for (int64_t d : shape) target *= (size_t)d;
        if (target == 0 || g.numel() % target != 0) throw std::runtime_error("reduce_gradient: shapes are not broadcast-compatible");
        const int64_t lead = (int64_t)(g.numel() / target);
        for (size_t i = 0; i + 2 < shape.size(); ++i)
            if (shape[i] != 1) throw std::runtime_error("reduce_gradient: only leading broadcast dimensions are supported");
        Tensor out(shape);
        // g is contiguous [lead, target]: the batch sum is a column sum over `lead` rows
        check(te_b200_colsum_f32(Backend::instance().ctx(), g.data(), lead, (int64_t)target, (int64_t)target, out.data(), current_stream()));
        return out;
    }
};

// Linear::forward with the bias add (and optionally FeedForward's GELU) fused into the GEMM epilogue.
class Linear {
public:
    Linear(int64_t in_features, int64_t out_features)
        : in_(in_features), out_(out_features), weight_({out_features, in_features}), bias_({out_features}) {}
    Tensor& weight() { return weight_; }   // [out, in], as in the reference
    Tensor& bias() { return bias_; }
    Tensor forward(const Tensor& x, bool gelu = false, Tensor* preact = nullptr) const {
        if (x.shape().empty() || x.shape().back() != in_) throw std::runtime_error("Inner dimensions must match for matmul");
        if (!x.is_contiguous()) throw std::runtime_error("Linear::forward expects a contiguous input");
        std::vector<int64_t> ys = x.shape();
        ys.back() = out_;
        Tensor y(ys);
        if (preact) *preact = Tensor(ys);
        Backend& be = Backend::instance();
        check(te_b200_linear_forward(be.ctx(), x.data(), weight_.data(), bias_.data(), y.data(),
                                     preact ? preact->data() : nullptr, (int64_t)(x.numel() / (size_t)in_), in_, out_,
                                     gelu ? 1 : 0, be.precision(), current_stream()));
        return y;
    }
    // {dX, dW[out,in], db[out]} in the order the reference's backward nodes produce them.  With x_preact (x is then
    // GELU(x_preact), the output of a forward(.., gelu = true) call) dX is the gradient of the pre-activation.
    std::vector<Tensor> backward(const Tensor& x, const Tensor& dy, const Tensor* x_preact = nullptr) const {
        Tensor dx(x.shape()), dw({out_, in_}), db({out_});
        Backend& be = Backend::instance();
        check(te_b200_linear_backward_ex(be.ctx(), x.data(), x_preact ? x_preact->data() : nullptr, weight_.data(), dy.data(),
                                         dx.data(), nullptr, nullptr, dw.data(), db.data(), 0, (int64_t)(x.numel() / (size_t)in_),
                                         in_, out_, be.precision(), current_stream()));
        return {dx, dw, db};
    }
private:
    int64_t in_, out_;
    Tensor weight_, bias_;
};

class FeedForward {
public:
    FeedForward(int64_t embed, int64_t ff) : linear1_(embed, ff), linear2_(ff, embed) {}
    Linear& linear1() { return linear1_; }
    Linear& linear2() { return linear2_; }
    Tensor forward(const Tensor& x) const { return linear2_.forward(linear1_.forward(x, /*gelu=*/true)); }
private:
    Linear linear1_, linear2_;
};

class ScaledDot {
public:
    // Q, K, V: [B, H, T, d] tensors or views with unit last-dim stride (the MultiHeadAttention head views).
    Tensor forward(const Tensor& Q, const Tensor& K, const Tensor& V, Tensor* probabilities = nullptr) const {
        if (Q.shape().size() != 4 || Q.shape() != K.shape() || Q.shape() != V.shape())
            throw std::runtime_error("ScaledDot expects Q, K, V of one [B,H,T,d] shape");
        for (const Tensor* t : {&Q, &K, &V})
            if (t->strides()[3] != 1) throw std::runtime_error(te_b200_status_string(TE_ERR_UNSUPPORTED_LAYOUT));
        const int64_t B = Q.shape()[0], H = Q.shape()[1], T = Q.shape()[2], d = Q.shape()[3];
        Tensor p({B, H, T, T}), o({B, H, T, d});
        te_attn_desc a{};
        a.B = B; a.H = H; a.T = T; a.d = d;
        a.q = Q.data(); a.k = K.data(); a.v = V.data();
        for (int i = 0; i < 3; ++i) {
            a.q_strides[i] = Q.strides()[i]; a.k_strides[i] = K.strides()[i]; a.v_strides[i] = V.strides()[i];
            a.o_strides[i] = o.strides()[i];
        }
        a.p_out = p.data(); a.o = o.data();
        Backend& be = Backend::instance();
        a.precision = be.precision();
        check(te_b200_attention_forward(be.ctx(), &a, current_stream()));
        if (probabilities) *probabilities = p;
        return o;
    }

    // Gradients {dQ, dK, dV} given dO, the probabilities and the output of forward(): the backward of its graph in one
    // call (MatMulBackward x2, SoftmaxBackward, DivBackward; reference src/core/grad_fn.cpp:126-156, :569-665).
    std::vector<Tensor> backward(const Tensor& Q, const Tensor& K, const Tensor& V, const Tensor& probabilities,
                                 const Tensor& O, const Tensor& dO) const {
        const int64_t B = Q.shape()[0], H = Q.shape()[1], T = Q.shape()[2], d = Q.shape()[3];
        if (probabilities.shape() != std::vector<int64_t>{B, H, T, T} || !probabilities.is_contiguous())
            throw std::runtime_error("ScaledDot backward expects dense probabilities [B,H,T,T]");
        for (const Tensor* t : {&Q, &K, &V, &O, &dO})
            if (t->shape() != Q.shape() || t->strides()[3] != 1)
                throw std::runtime_error(te_b200_status_string(TE_ERR_UNSUPPORTED_LAYOUT));
        Tensor dq({B, H, T, d}), dk({B, H, T, d}), dv({B, H, T, d});
        te_attn_bwd_desc a{};
        a.B = B; a.H = H; a.T = T; a.d = d;
        a.q = Q.data(); a.k = K.data(); a.v = V.data();
        a.p = probabilities.data(); a.o = O.data(); a.d_o = dO.data();
        a.dq = dq.data(); a.dk = dk.data(); a.dv = dv.data();
        for (int i = 0; i < 3; ++i) {
            a.q_strides[i] = Q.strides()[i]; a.k_strides[i] = K.strides()[i]; a.v_strides[i] = V.strides()[i];
            a.o_strides[i] = O.strides()[i]; a.d_o_strides[i] = dO.strides()[i];
            a.dq_strides[i] = dq.strides()[i]; a.dk_strides[i] = dk.strides()[i]; a.dv_strides[i] = dv.strides()[i];
        }
        Backend& be = Backend::instance();
        a.precision = be.precision();
        check(te_b200_attention_backward(be.ctx(), &a, current_stream()));
        return {dq, dk, dv};
    }
};

// MultiHeadAttention (reference src/nn/multi_head_attention.cpp:19-42) as the two fused calls te_b200_mha_forward /
// te_b200_mha_backward: four Linears, the head split and merge as strides, attention on the head views.
class MultiHeadAttention {
public:
    MultiHeadAttention(int64_t embed_dim, int64_t num_heads)
        : embed_(embed_dim), heads_(num_heads), q_(embed_dim, embed_dim), k_(embed_dim, embed_dim), v_(embed_dim, embed_dim),
          out_(embed_dim, embed_dim) {
        if (num_heads < 1 || embed_dim % num_heads != 0) throw std::runtime_error("embedDim must be divisible by numHeads");
    }
    // in MultiHeadAttention::parameters() order: q, k, v, out projections
    Linear& q_proj() { return q_; }
    Linear& k_proj() { return k_; }
    Linear& v_proj() { return v_; }
    Linear& out_proj() { return out_; }

    // What forward() keeps for backward(): the projections (q | k | v as the column blocks of one [B,T,3E] tensor,
    // computed as one product against the gathered [3E,E] weight wqkv), the probabilities, the merged head outputs.
    struct Saved { Tensor x, qkv, wqkv, p, attn; };

    // x: [B, T, E] contiguous.  residual (optional, [B, T, E]) is added to the result: x + MHA(...) of a transformer block.
    Tensor forward(const Tensor& x, Saved* saved = nullptr, const Tensor* residual = nullptr) {
        if (x.shape().size() != 3 || x.shape()[2] != embed_) throw std::runtime_error("Inner dimensions must match for matmul");
        if (!x.is_contiguous()) throw std::runtime_error("MultiHeadAttention::forward expects a contiguous input");
        const int64_t B = x.shape()[0], T = x.shape()[1];
        Saved s{x, Tensor({B, T, 3 * embed_}), Tensor({3 * embed_ * embed_ + 3 * embed_}), Tensor({B, heads_, T, T}),
                Tensor(x.shape())};
        Tensor y(x.shape());
        te_mha_desc m{};
        m.B = B; m.T = T; m.E = embed_; m.H = heads_;
        m.x = x.data();
        m.wq = q_.weight().data(); m.bq = q_.bias().data(); m.wk = k_.weight().data(); m.bk = k_.bias().data();
        m.wv = v_.weight().data(); m.bv = v_.bias().data(); m.wo = out_.weight().data(); m.bo = out_.bias().data();
        m.q = s.qkv.data(); m.k = m.q + embed_; m.v = m.q + 2 * embed_; m.ld_qkv = 3 * embed_; m.wqkv = s.wqkv.data();
        m.p = s.p.data(); m.attn = s.attn.data();
        m.y = y.data();
        m.residual = residual ? residual->data() : nullptr;
        Backend& be = Backend::instance();
        m.precision = be.precision();
        check(te_b200_mha_forward(be.ctx(), &m, current_stream()));
        if (saved) *saved = s;
        return y;
    }

    // {dX, dWq, dbq, dWk, dbk, dWv, dbv, dWo, dbo}: the input gradient followed by the parameter gradients in
    // parameters() order, as the reference's backward nodes deliver them.
    std::vector<Tensor> backward(const Saved& s, const Tensor& dy) {
        const int64_t B = s.x.shape()[0], T = s.x.shape()[1];
        if (dy.shape() != s.x.shape() || !dy.is_contiguous()) throw std::runtime_error("MultiHeadAttention backward expects a contiguous [B,T,E] gradient");
        std::vector<Tensor> g = {Tensor(s.x.shape())};
        for (int i = 0; i < 4; ++i) {
            g.emplace_back(std::vector<int64_t>{embed_, embed_});
            g.emplace_back(std::vector<int64_t>{embed_});
        }
        Tensor dqkv(s.qkv.shape()), dwqkv(s.wqkv.shape()), dattn(s.x.shape());
        te_mha_bwd_desc m{};
        m.B = B; m.T = T; m.E = embed_; m.H = heads_;
        m.x = s.x.data();
        m.wq = q_.weight().data(); m.wk = k_.weight().data(); m.wv = v_.weight().data(); m.wo = out_.weight().data();
        m.q = s.qkv.data(); m.k = m.q + embed_; m.v = m.q + 2 * embed_; m.ld_qkv = 3 * embed_;
        m.wqkv = s.wqkv.data(); m.dwqkv = dwqkv.data();
        m.p = s.p.data(); m.attn = s.attn.data();
        m.dy = dy.data(); m.dx = g[0].data();
        m.dwq = g[1].data(); m.dbq = g[2].data(); m.dwk = g[3].data(); m.dbk = g[4].data();
        m.dwv = g[5].data(); m.dbv = g[6].data(); m.dwo = g[7].data(); m.dbo = g[8].data();
        m.dq = dqkv.data(); m.dk = m.dq + embed_; m.dv = m.dq + 2 * embed_; m.dattn = dattn.data();
        Backend& be = Backend::instance();
        m.precision = be.precision();
        check(te_b200_mha_backward(be.ctx(), &m, current_stream()));
        return g;
    }
private:
    int64_t embed_, heads_;
    Linear q_, k_, v_, out_;
};

// Int64 device array for token ids and class targets (the reference keeps them in Int64 tensors).
class IndexArray {
public:
    explicit IndexArray(const std::vector<int64_t>& host) : n_(host.size()) {
        size_t block = 0;
        void* p = CachingAllocator::instance().allocate((n_ ? n_ : 1) * sizeof(int64_t), &block);
        storage_ = std::shared_ptr<void>(p, [block](void* q) { CachingAllocator::instance().release(q, block); });
        cuda_check(cudaMemcpyAsync(p, host.data(), n_ * sizeof(int64_t), cudaMemcpyHostToDevice, current_stream()), "cudaMemcpy H2D");
        cuda_check(cudaStreamSynchronize(current_stream()), "cudaStreamSynchronize");
    }
    const int64_t* data() const { return static_cast<const int64_t*>(storage_.get()); }
    size_t size() const { return n_; }
private:
    std::shared_ptr<void> storage_;
    size_t n_;
};

// LayerNorm over the last dimension (reference src/nn/layernorm.cpp:19-82); backward returns {dx, dgamma, dbeta} in the
// order LayerNormBackward does (src/core/grad_fn.cpp:405-538).
class LayerNorm {
public:
    explicit LayerNorm(int64_t normalized_shape, float eps = 1e-5f)
        : dim_(normalized_shape), eps_(eps),
          weight_(Tensor::from_host(std::vector<float>((size_t)normalized_shape, 1.0f), {normalized_shape})),
          bias_(Tensor::from_host(std::vector<float>((size_t)normalized_shape, 0.0f), {normalized_shape})) {}
    Tensor& weight() { return weight_; }
    Tensor& bias() { return bias_; }
    Tensor forward(const Tensor& x) const {
        if (x.shape().empty() || x.shape().back() != dim_)
            throw std::runtime_error("Last dimension of input must match normalized_shape");
        if (!x.is_contiguous()) throw std::runtime_error("LayerNorm requires a contiguous input");
        Tensor y(x.shape());
        Backend& be = Backend::instance();
        check(te_b200_layernorm_forward(be.ctx(), x.data(), weight_.data(), bias_.data(), y.data(),
                                        (int64_t)(x.numel() / (size_t)dim_), dim_, eps_, current_stream()));
        return y;
    }
    std::vector<Tensor> backward(const Tensor& x, const Tensor& dy) const {
        if (!x.is_contiguous() || !dy.is_contiguous() || x.shape() != dy.shape())
            throw std::runtime_error("CUDA LayerNormBackward requires contiguous x and pathDownGrad");
        Tensor dx(x.shape()), dg({dim_}), db({dim_});
        Backend& be = Backend::instance();
        check(te_b200_layernorm_backward(be.ctx(), x.data(), weight_.data(), dy.data(), dx.data(), dg.data(), db.data(),
                                         (int64_t)(x.numel() / (size_t)dim_), dim_, eps_, current_stream()));
        return {dx, dg, db};
    }
private:
    int64_t dim_;
    float eps_;
    Tensor weight_, bias_;
};

// Embedding lookup (reference src/nn/embedding.cpp:18-60) with the optional positional table that GPT::forward adds
// (src/nn/gpt.cpp:30-69), and the table gradient of EmbeddingBackward (src/core/grad_fn.cpp:688-760).
class Embedding {
public:
    Embedding(int64_t num_embeddings, int64_t dim) : vocab_(num_embeddings), dim_(dim), weight_({num_embeddings, dim}) {}
    Tensor& weight() { return weight_; }
    // tokens: batch * seq_len ids; result [batch, seq_len, dim]
    Tensor forward(const IndexArray& tokens, int64_t batch, int64_t seq_len, const Tensor* positional = nullptr) const {
        if ((int64_t)tokens.size() != batch * seq_len) throw std::runtime_error("Embedding: token count does not match the shape");
        Tensor out({batch, seq_len, dim_});
        Backend& be = Backend::instance();
        check(te_b200_embedding_forward(be.ctx(), weight_.data(), tokens.data(), positional ? positional->data() : nullptr,
                                        out.data(), batch * seq_len, seq_len, dim_, vocab_, current_stream()));
        return out;
    }
    Tensor backward(const IndexArray& tokens, const Tensor& dout) const {
        Tensor dw({vocab_, dim_});
        Backend& be = Backend::instance();
        check(te_b200_embedding_backward(be.ctx(), tokens.data(), dout.data(), dw.data(), (int64_t)tokens.size(), dim_, vocab_, current_stream()));
        return dw;
    }
private:
    int64_t vocab_, dim_;
    Tensor weight_;
};

// crossEntropyLoss::forward_batched over logits [B, T, V] (reference src/loss/CrossEntropyLoss.cpp:47-127): returns the
// mean loss as a 1-element tensor and, when asked, the gradient CrossEntropyBatchedBackward would produce for an upstream
// gradient of 1 (src/core/grad_fn.cpp:271-346).
inline Tensor cross_entropy(const Tensor& logits, const IndexArray& targets, Tensor* dlogits = nullptr) {
    if (logits.shape().size() != 3) throw std::runtime_error("forward_batched expects 3D logits [B, T, V]");
    if (!logits.is_contiguous()) throw std::runtime_error("cross_entropy requires contiguous logits");
    const int64_t V = logits.shape()[2], rows = logits.shape()[0] * logits.shape()[1];
    if ((int64_t)targets.size() != rows) throw std::runtime_error("forward_batched expects 2D targets [B, T]");
    Tensor loss({1});
    Tensor grad = dlogits ? Tensor(logits.shape()) : Tensor();
    Backend& be = Backend::instance();
    check(te_b200_cross_entropy(be.ctx(), logits.data(), targets.data(), loss.data(), dlogits ? grad.data() : nullptr, 1.0f, rows, V, current_stream()));
    if (dlogits) *dlogits = grad;
    return loss;
}

}  // namespace te
