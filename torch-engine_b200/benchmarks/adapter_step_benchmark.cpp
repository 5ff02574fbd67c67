// Forward + backward of a stack of transformer blocks through the C++ host adapter (include/te_b200.hpp), issued the
// way an eager framework issues it: every intermediate and every gradient is a fresh te::Tensor.  The same step is
// timed twice, with the adapter's caching allocator and with the allocation behaviour of the reference's CUDAAllocator
// (cudaMalloc for every tensor, cudaFree when it dies: reference src/core/allocators.h:35-52), so the figure shows
// what the allocator is worth on this path.  Sizes default to the GPT benchmark configuration (6 blocks, d_model 384,
// 6 heads, feed-forward 1536, batch 64 x context 256; reference src/benchmarks/gpt_benchmark_gpu.cpp:12-33).
//
//   adapter_step_benchmark [steps] [layers] [batch] [context] [d_model] [heads]
//
// Prints one JSON line per allocator mode.  The block is LayerNorm -> MultiHeadAttention (+ residual) -> LayerNorm ->
// Linear+GELU -> Linear, as reference src/nn/transformer_block.cpp:15-35 without the second residual add (the adapter
// has no stand-alone elementwise add; the step schedule of the Python harness folds that add into the GEMM).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "te_b200.hpp"

using te::Tensor;

namespace {

struct Block {
    te::LayerNorm ln1, ln2;
    te::MultiHeadAttention mha;
    te::Linear lin1, lin2;
    Block(int64_t E, int64_t H, int64_t ff) : ln1(E), ln2(E), mha(E, H), lin1(E, ff), lin2(ff, E) {}
};

struct Saved {
    Tensor x, h1, y1, h2, pre, f;
    te::MultiHeadAttention::Saved mha;
};

void fill(Tensor& t, std::mt19937& rng, float scale) {
    std::vector<float> v(t.numel(), 0.0f);
    if (scale > 0.0f) {
        std::normal_distribution<float> d(0.0f, scale);
        for (float& x : v) x = d(rng);
    }
    t = Tensor::from_host(v, t.shape());
}

// One forward + backward over all blocks; returns a value that depends on the whole step.
float step(std::vector<Block>& blocks, const Tensor& input, const Tensor& upstream) {
    std::vector<Saved> saved(blocks.size());
    Tensor x = input;
    for (size_t l = 0; l < blocks.size(); ++l) {
        Block& b = blocks[l];
        Saved& s = saved[l];
        s.x = x;
        s.h1 = b.ln1.forward(x);
        s.y1 = b.mha.forward(s.h1, &s.mha, &x);
        s.h2 = b.ln2.forward(s.y1);
        s.f = b.lin1.forward(s.h2, /*gelu=*/true, &s.pre);
        x = b.lin2.forward(s.f);
    }
    Tensor g = upstream;
    std::vector<Tensor> keep;       // parameter gradients of the step, alive until its end like an optimizer's inputs
    for (size_t l = blocks.size(); l-- > 0;) {
        Block& b = blocks[l];
        Saved& s = saved[l];
        std::vector<Tensor> g2 = b.lin2.backward(s.f, g);
        std::vector<Tensor> g1 = b.lin1.backward(s.h2, g2[0], &s.pre);
        std::vector<Tensor> n2 = b.ln2.backward(s.y1, g1[0]);
        std::vector<Tensor> m = b.mha.backward(s.mha, n2[0]);
        std::vector<Tensor> n1 = b.ln1.backward(s.x, m[0]);
        g = n1[0];
        for (std::vector<Tensor>* v : {&g2, &g1, &n2, &m, &n1})
            for (size_t i = 1; i < v->size(); ++i) keep.push_back((*v)[i]);
    }
    // what leaves the device at the end of a step is small (a loss, a norm): here the column sums of the input gradient
    Tensor sums({g.shape().back()});
    te::check(te_b200_colsum_f32(te::Backend::instance().ctx(), g.data(), (int64_t)(g.numel() / (size_t)g.shape().back()), g.shape().back(),
                                 g.shape().back(), sums.data(), te::current_stream()));
    return sums.to_host()[0];
}

}  // namespace

int main(int argc, char** argv) {
    const int steps = argc > 1 ? std::atoi(argv[1]) : 10;
    const int layers = argc > 2 ? std::atoi(argv[2]) : 6;
    const int64_t B = argc > 3 ? std::atoll(argv[3]) : 64, T = argc > 4 ? std::atoll(argv[4]) : 256;
    const int64_t E = argc > 5 ? std::atoll(argv[5]) : 384, H = argc > 6 ? std::atoll(argv[6]) : 6;
    try {
        std::mt19937 rng(42);
        std::vector<Block> blocks;
        blocks.reserve(layers);
        for (int l = 0; l < layers; ++l) {
            blocks.emplace_back(E, H, 4 * E);
            Block& b = blocks.back();
            for (te::Linear* lin : {&b.mha.q_proj(), &b.mha.k_proj(), &b.mha.v_proj(), &b.mha.out_proj(), &b.lin1, &b.lin2}) {
                fill(lin->weight(), rng, 0.02f);
                fill(lin->bias(), rng, 0.0f);
            }
        }
        Tensor input({B, T, E}), upstream({B, T, E});
        fill(input, rng, 1.0f);
        fill(upstream, rng, 1.0f / (float)(B * T));
        te::CachingAllocator& al = te::CachingAllocator::instance();
        float check[2] = {0.0f, 0.0f};
        for (int mode = 0; mode < 2; ++mode) {
            const bool caching = mode == 0;
            al.set_caching(caching);
            for (int w = 0; w < 3; ++w) check[mode] = step(blocks, input, upstream);
            te::Backend::instance().synchronize();
            const size_t mallocs0 = al.device_mallocs(), hits0 = al.cache_hits();
            const auto t0 = std::chrono::steady_clock::now();
            for (int s = 0; s < steps; ++s) check[mode] = step(blocks, input, upstream);
            te::Backend::instance().synchronize();
            const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / steps;
            std::printf("{\"benchmark\": \"adapter_transformer_blocks_fwd_bwd\", \"allocator\": \"%s\", \"layers\": %d, \"tokens\": %lld, "
                        "\"d_model\": %lld, \"heads\": %lld, \"steps\": %d, \"ms_per_step\": %.3f, \"tokens_per_s\": %.0f, "
                        "\"cuda_mallocs_per_step\": %.1f, \"cache_hits_per_step\": %.1f, \"checksum\": %.9g}\n",
                        caching ? "caching" : "cudaMalloc_per_tensor", layers, (long long)(B * T), (long long)E, (long long)H, steps, ms,
                        1e3 * (double)(B * T) / ms, (double)(al.device_mallocs() - mallocs0) / steps,
                        (double)(al.cache_hits() - hits0) / steps, (double)check[mode]);
            std::fflush(stdout);
        }
        al.set_caching(true);
        if (check[0] != check[1]) {
            std::printf("FAIL: the two allocator modes disagree (%.9g vs %.9g)\n", (double)check[0], (double)check[1]);
            return 1;
        }
    } catch (const std::exception& e) {
        std::printf("FAIL: %s\n", e.what());
        return 1;
    }
    return 0;
}
