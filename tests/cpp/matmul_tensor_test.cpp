// GPU check of the C++ host adapter (include/te_b200.hpp), laid out like the reference's own plain-main CUDA
// check of Tensor::matmul (reference src/tests/cuda_matmul_tensor_test.cpp) and its throw / shape tests
// (reference src/tests/tensor_test.cpp:597-725): same inputs, same expected values, exit code 0 on success.
#include <cmath>
#include <cstdio>
#include <iostream>
#include <numeric>
#include <vector>

#include "te_b200.hpp"

using te::Tensor;

static int failures = 0;

static void expect_values(const char* what, const Tensor& t, const std::vector<float>& want, float tol) {
    std::vector<float> got = t.to_host();
    bool ok = got.size() == want.size();
    for (size_t i = 0; ok && i < want.size(); ++i) ok = std::fabs(got[i] - want[i]) <= tol;
    std::cout << (ok ? "ok   " : "FAIL ") << what << "\n";
    if (!ok) ++failures;
}

template <typename F>
static void expect_throw(const char* what, F&& f, const std::string& message) {
    bool ok = false;
    try {
        f();
    } catch (const std::runtime_error& e) {
        ok = (message == e.what());
        if (!ok) std::cout << "     got message: " << e.what() << "\n";
    }
    std::cout << (ok ? "ok   " : "FAIL ") << what << "\n";
    if (!ok) ++failures;
}

static std::vector<float> iota(int n) {
    std::vector<float> v(n);
    std::iota(v.begin(), v.end(), 1.0f);
    return v;
}

int main() {
    try {
        // 2-D: A 2x3 . B 3x4
        Tensor a = Tensor::from_host(iota(6), {2, 3});
        Tensor b = Tensor::from_host(iota(12), {3, 4});
        expect_values("2x3 . 3x4", a.matmul(b), {38, 44, 50, 56, 83, 98, 113, 128}, 1e-5f);
        // transposed-A view
        Tensor a2 = Tensor::from_host(iota(6), {3, 2});
        expect_values("transpose_view(0,1) . 3x4", a2.transpose_view(0, 1).matmul(b), {61, 70, 79, 88, 76, 88, 100, 112}, 1e-5f);
        // batched 3-D
        Tensor a3 = Tensor::from_host(iota(12), {2, 2, 3});
        Tensor b3 = Tensor::from_host(iota(24), {2, 3, 4});
        expect_values("batched 2x(2x3 . 3x4)", a3.matmul(b3),
                      {38, 44, 50, 56, 83, 98, 113, 128, 416, 440, 464, 488, 569, 602, 635, 668}, 1e-4f);
        // f32 2x3 . 3x2
        expect_values("2x3 . 3x2", a.matmul(Tensor::from_host(iota(6), {3, 2})), {22, 28, 49, 64}, 0.0f);
        // broadcast (1,2,3) @ (3,3,4) -> (3,2,4)
        Tensor c = Tensor::from_host(iota(6), {1, 2, 3}).matmul(Tensor::from_host(iota(36), {3, 3, 4}));
        const bool shape_ok = c.shape() == std::vector<int64_t>({3, 2, 4});
        std::cout << (shape_ok ? "ok   " : "FAIL ") << "broadcast result shape\n";
        if (!shape_ok) ++failures;
        // the reference's throw cases, with its texts
        expect_throw("inner dimension mismatch", [&] { Tensor({2, 3}).matmul(Tensor({2, 2})); },
                     "Inner dimensions must match for matmul");
        expect_throw("batch 3 vs 2", [&] { Tensor({3, 2, 3}).matmul(Tensor({2, 3, 4})); },
                     "Batch dimensions are not broadcastable");
        expect_throw("batch 2 vs 3", [&] { Tensor({2, 2, 3}).matmul(Tensor({3, 3, 4})); },
                     "Batch dimensions are not broadcastable");
        expect_throw("1-D operand", [&] { Tensor({3}).matmul(Tensor({3, 2})); },
                     "Matmul requires tensors with at least 2 dimensions");
        // MatMulBackward with a broadcast weight: A [2,2,3] . B [3,2], dC = ones -> dA rows = row sums of B,
        // dB = sum over both batches of A^T . ones (the reference reduces the [2,3,2] product over its batch dim)
        {
            Tensor A3 = Tensor::from_host(iota(12), {2, 2, 3});
            Tensor B2 = Tensor::from_host({1, 2, 3, 4, 5, 6}, {3, 2});
            Tensor dC = Tensor::from_host(std::vector<float>(8, 1.0f), {2, 2, 2});
            te::MatMulBackward node{A3, B2};
            std::vector<Tensor> g = node.backward(dC);
            expect_values("MatMulBackward dA", g[0], {3, 7, 11, 3, 7, 11, 3, 7, 11, 3, 7, 11}, 1e-5f);
            // column sums of A over all 4 rows: (1+4+7+10, 2+5+8+11, 3+6+9+12) = (22, 26, 30), repeated for both columns
            expect_values("MatMulBackward dB (reduced over the broadcast batch)", g[1], {22, 22, 26, 26, 30, 30}, 1e-4f);
            const bool shapes_ok = g[0].shape() == A3.shape() && g[1].shape() == B2.shape();
            std::cout << (shapes_ok ? "ok   " : "FAIL ") << "MatMulBackward gradient shapes\n";
            if (!shapes_ok) ++failures;
        }
        // Linear: y = x.W^T + b with W [out,in]
        te::Linear lin(3, 2);
        lin.weight() = Tensor::from_host({1, 0, -1, 2, 1, 0}, {2, 3});
        lin.bias() = Tensor::from_host({0.5f, -1.0f}, {2});
        expect_values("Linear forward", lin.forward(a), {1 - 3 + 0.5f, 2 + 2 - 1.0f, 4 - 6 + 0.5f, 8 + 5 - 1.0f}, 1e-5f);
        // ScaledDot on MultiHeadAttention-style head views: uniform keys give the mean of V
        for (const int64_t hd : {int64_t(8), int64_t(32)}) {     // 32: the fused kernels in TF32 mode; 8: the GEMM sequence
        const int64_t B = 2, T = 4, H = 2;
        std::vector<float> q(B * T * H * hd, 0.0f), v(B * T * H * hd);
        for (size_t i = 0; i < v.size(); ++i) v[i] = float(i % 7);
        auto heads = [&](const std::vector<float>& x) { return Tensor::from_host(x, {B, T, H * hd}).view({B, T, H, hd}).transpose_view(1, 2); };
        Tensor o = te::ScaledDot().forward(heads(q), heads(q), heads(v));
        std::vector<float> want(B * H * T * hd);
        for (int64_t bb = 0; bb < B; ++bb) for (int64_t h = 0; h < H; ++h) for (int64_t t = 0; t < T; ++t) for (int64_t e = 0; e < hd; ++e) {
            float s = 0;
            for (int64_t tt = 0; tt < T; ++tt) s += v[((bb * T + tt) * H + h) * hd + e];
            want[((bb * H + h) * T + t) * hd + e] = s / T;
        }
        expect_values("ScaledDot on head views", o, want, 1e-2f);
        // Backward with zero queries and keys: P = 1/T everywhere, so dV is the mean of dO over the queries for every
        // key, and dQ = dS.K and dK = dS^T.Q vanish with K and Q.
        Tensor p_saved;
        Tensor qh = heads(q), vh = heads(v);
        Tensor o2 = te::ScaledDot().forward(qh, qh, vh, &p_saved);
        std::vector<float> go(B * H * T * hd);
        for (size_t i = 0; i < go.size(); ++i) go[i] = float(int(i % 5) - 2);
        std::vector<Tensor> grads = te::ScaledDot().backward(qh, qh, vh, p_saved, o2, Tensor::from_host(go, {B, H, T, hd}));
        std::vector<float> want_dv(B * H * T * hd), zeros(B * H * T * hd, 0.0f);
        for (int64_t bh = 0; bh < B * H; ++bh) for (int64_t t = 0; t < T; ++t) for (int64_t e = 0; e < hd; ++e) {
            float s = 0;
            for (int64_t tt = 0; tt < T; ++tt) s += go[(bh * T + tt) * hd + e];
            want_dv[(bh * T + t) * hd + e] = s / T;
        }
        expect_values("ScaledDot backward dV", grads[2], want_dv, 1e-2f);
        expect_values("ScaledDot backward dQ", grads[0], zeros, 1e-6f);
        expect_values("ScaledDot backward dK", grads[1], zeros, 1e-6f);
        }
        // MultiHeadAttention with zero query/key projections (uniform attention) and identity value/output projections:
        // every position receives the mean of x over its sequence; with a residual input, x is added on top.
        for (const int64_t E : {int64_t(16), int64_t(64)}) {      // head size 8: GEMM sequence; 32: the fused kernels (TF32 mode)
            const int64_t B = 2, T = 4, H = 2;
            te::MultiHeadAttention mha(E, H);
            std::vector<float> zero_w(E * E, 0.0f), eye(E * E, 0.0f), zero_b(E, 0.0f);
            for (int64_t i = 0; i < E; ++i) eye[i * E + i] = 1.0f;
            mha.q_proj().weight() = Tensor::from_host(zero_w, {E, E});  mha.q_proj().bias() = Tensor::from_host(zero_b, {E});
            mha.k_proj().weight() = Tensor::from_host(zero_w, {E, E});  mha.k_proj().bias() = Tensor::from_host(zero_b, {E});
            mha.v_proj().weight() = Tensor::from_host(eye, {E, E});     mha.v_proj().bias() = Tensor::from_host(zero_b, {E});
            mha.out_proj().weight() = Tensor::from_host(eye, {E, E});   mha.out_proj().bias() = Tensor::from_host(zero_b, {E});
            std::vector<float> xs(B * T * E);
            for (size_t i = 0; i < xs.size(); ++i) xs[i] = float(int(i % 11) - 5);
            Tensor x = Tensor::from_host(xs, {B, T, E});
            std::vector<float> want(xs.size());
            for (int64_t b = 0; b < B; ++b) for (int64_t e = 0; e < E; ++e) {
                float m = 0;
                for (int64_t t = 0; t < T; ++t) m += xs[(b * T + t) * E + e];
                for (int64_t t = 0; t < T; ++t) want[(b * T + t) * E + e] = m / T + xs[(b * T + t) * E + e];
            }
            te::MultiHeadAttention::Saved saved;
            expect_values("MultiHeadAttention forward + residual", mha.forward(x, &saved, &x), want, 2e-2f);
            // dy = 1: the out projection (identity) passes it on, every key gets T * (1/T) of it, the value projection
            // (identity) passes that on: dx = 1; query and key paths vanish with Q = K = 0.  dbo = B*T.
            std::vector<Tensor> g = mha.backward(saved, Tensor::from_host(std::vector<float>(xs.size(), 1.0f), {B, T, E}));
            expect_values("MultiHeadAttention backward dx", g[0], std::vector<float>(xs.size(), 1.0f), 1e-2f);
            expect_values("MultiHeadAttention backward dbo", g[8], std::vector<float>(E, float(B * T)), 1e-4f);
            expect_values("MultiHeadAttention backward dbq", g[2], std::vector<float>(E, 0.0f), 1e-5f);
        }
        // LayerNorm: a row of 1..8 normalises to (j - 4.5) / sqrt(5.25 + eps); with gain 2 and shift 1 on top
        {
            te::LayerNorm ln(8);
            ln.weight() = Tensor::from_host(std::vector<float>(8, 2.0f), {8});
            ln.bias() = Tensor::from_host(std::vector<float>(8, 1.0f), {8});
            std::vector<float> xs(16), want(16);
            for (int r = 0; r < 2; ++r) for (int j = 0; j < 8; ++j) {
                xs[r * 8 + j] = float(j + 1) * float(r + 1);
                want[r * 8 + j] = 2.0f * (float(j) - 3.5f) / std::sqrt(5.25f + 1e-5f / float((r + 1) * (r + 1))) + 1.0f;
            }
            Tensor x = Tensor::from_host(xs, {2, 8});
            expect_values("LayerNorm forward", ln.forward(x), want, 1e-4f);
            // dy = 1 everywhere: dbeta = number of rows, dgamma = column sums of x_hat, dx = 0 (a constant shift of y)
            std::vector<Tensor> g = ln.backward(x, Tensor::from_host(std::vector<float>(16, 1.0f), {2, 8}));
            expect_values("LayerNorm backward dx", g[0], std::vector<float>(16, 0.0f), 1e-5f);
            expect_values("LayerNorm backward dbeta", g[2], std::vector<float>(8, 2.0f), 1e-6f);
            std::vector<float> want_dg(8);
            for (int j = 0; j < 8; ++j) want_dg[j] = (want[j] - 1.0f) / 2.0f + (want[8 + j] - 1.0f) / 2.0f;
            expect_values("LayerNorm backward dgamma", g[1], want_dg, 1e-4f);
        }
        // Embedding lookup + positional sum, its table gradient, and the mean cross-entropy of uniform logits (= log V)
        {
            te::Embedding emb(5, 4);
            std::vector<float> table(20);
            for (int i = 0; i < 20; ++i) table[i] = float(i);
            emb.weight() = Tensor::from_host(table, {5, 4});
            te::IndexArray tok({4, 0, 4, 2, 1, 1});                    // batch 2, seq_len 3
            Tensor pos = Tensor::from_host({100, 100, 100, 100, 200, 200, 200, 200, 300, 300, 300, 300}, {3, 4});
            std::vector<float> want;
            const int ids[6] = {4, 0, 4, 2, 1, 1};
            for (int i = 0; i < 6; ++i) for (int j = 0; j < 4; ++j) want.push_back(table[ids[i] * 4 + j] + 100.0f * float(i % 3 + 1));
            expect_values("Embedding + positions", emb.forward(tok, 2, 3, &pos), want, 0.0f);
            Tensor dw = emb.backward(tok, Tensor::from_host(std::vector<float>(24, 1.0f), {2, 3, 4}));
            expect_values("Embedding backward", dw, {1, 1, 1, 1, 2, 2, 2, 2, 1, 1, 1, 1, 0, 0, 0, 0, 2, 2, 2, 2}, 0.0f);
            Tensor dlogits;
            Tensor loss = te::cross_entropy(Tensor::from_host(std::vector<float>(2 * 3 * 5, 0.25f), {2, 3, 5}), tok, &dlogits);
            expect_values("cross-entropy of uniform logits", loss, {std::log(5.0f)}, 1e-6f);
            std::vector<float> want_g(30, 0.2f / 6.0f);
            for (int i = 0; i < 6; ++i) want_g[i * 5 + ids[i]] = (0.2f - 1.0f) / 6.0f;
            expect_values("cross-entropy gradient", dlogits, want_g, 1e-7f);
        }
        // Temporaries of a repeated step come out of the allocator's cache: no further cudaMalloc after the first pass.
        {
            Tensor x = Tensor::from_host(std::vector<float>(64 * 48, 0.5f), {64, 48});
            Tensor w = Tensor::from_host(std::vector<float>(48 * 32, 0.25f), {48, 32});
            auto step = [&]() { Tensor y = x.matmul(w); Tensor z = y.matmul(w.transpose_view(0, 1)); return z.to_host()[0]; };
            const float first = step();
            const size_t mallocs = te::CachingAllocator::instance().device_mallocs();
            const size_t hits = te::CachingAllocator::instance().cache_hits();
            float last = first;
            for (int it = 0; it < 10; ++it) last = step();
            if (te::CachingAllocator::instance().device_mallocs() != mallocs || te::CachingAllocator::instance().cache_hits() < hits + 20 ||
                last != first) {
                std::cout << "FAIL caching allocator: " << te::CachingAllocator::instance().device_mallocs() - mallocs
                          << " new cudaMalloc calls in 10 repeated steps\n";
                ++failures;
            } else {
                std::cout << "ok   caching allocator reuses blocks\n";
            }
        }
        {   // stream-ordered reuse: a block freed by work on one stream and taken by another stream is ordered behind it
            te::Backend::instance().synchronize();
            cudaStream_t s1 = nullptr, s2 = nullptr;
            te::cuda_check(cudaStreamCreateWithFlags(&s1, cudaStreamNonBlocking), "cudaStreamCreate");
            te::cuda_check(cudaStreamCreateWithFlags(&s2, cudaStreamNonBlocking), "cudaStreamCreate");
            te::CachingAllocator& al = te::CachingAllocator::instance();
            const int64_t n = 1536;          // a size no other check uses, so the free list holds exactly the blocks below
            std::vector<float> ones((size_t)(n * n), 1.0f), eye((size_t)(n * n), 0.0f);
            for (int64_t i = 0; i < n; ++i) eye[(size_t)(i * n + i)] = 2.0f;
            bool ok = true;
            float* first_block = nullptr;
            Tensor a, w, y2;
            {
                te::StreamGuard on1(s1);
                a = Tensor::from_host(ones, {n, n});
                w = Tensor::from_host(eye, {n, n});
                Tensor chain = a;
                for (int it = 0; it < 20; ++it) chain = chain.matmul(w);      // 20 products queued on s1; temporaries reused in stream order
                first_block = chain.data();
                y2 = chain;                                                   // keep the last one
            }
            const size_t cross0 = al.cross_stream_reuses(), hits0 = al.cache_hits();
            Tensor z;
            {
                te::StreamGuard on2(s2);
                // the temporaries of the chain above are free blocks of s1 whose kernels may still be running: s2 may
                // take one, but only behind s1's queue
                Tensor t = Tensor::from_host(ones, {n, n});
                z = t.matmul(w);
            }
            te::cuda_check(cudaStreamSynchronize(s1), "sync s1");
            te::cuda_check(cudaStreamSynchronize(s2), "sync s2");
            ok = ok && al.cache_hits() > hits0 && al.cross_stream_reuses() > cross0;
            {
                te::StreamGuard on1(s1);
                const std::vector<float> got = y2.to_host();       // 2^20 everywhere if no block was overwritten early
                ok = ok && got[0] == 1048576.0f && got[(size_t)(n * n - 1)] == 1048576.0f && got[(size_t)(n * (n / 2) + 7)] == 1048576.0f;
            }
            {
                te::StreamGuard on2(s2);
                const std::vector<float> got = z.to_host();
                ok = ok && got[0] == 2.0f && got[(size_t)(n * n - 1)] == 2.0f;
            }
            // record_stream: a tensor of s1 used by work on s2 is only handed to s1 again behind s2
            {
                const size_t cross1 = al.cross_stream_reuses();
                {
                    Tensor shared_t;
                    {
                        te::StreamGuard on1(s1);
                        shared_t = Tensor::from_host(ones, {n, n});
                    }
                    te::StreamGuard on2(s2);
                    shared_t.record_stream(s2);
                    Tensor r = shared_t.matmul(w);
                }   // shared_t and r are free now; shared_t's block lists s1 and s2
                te::StreamGuard on1(s1);
                std::vector<Tensor> grab;
                for (int i = 0; i < 8; ++i) grab.emplace_back(std::vector<int64_t>{n, n});     // drains the free list of this size
                ok = ok && al.cross_stream_reuses() > cross1;
            }
            // the reference's behaviour for comparison runs: every tensor is a cudaMalloc, every release a cudaFree
            al.set_caching(false);
            const size_t mallocs0 = al.device_mallocs();
            { Tensor t1({n, n}); Tensor t2({n, n}); }
            { Tensor t3({n, n}); }
            ok = ok && al.device_mallocs() == mallocs0 + 3;
            al.set_caching(true);
            (void)first_block;
            te::cuda_check(cudaStreamDestroy(s1), "cudaStreamDestroy");
            te::cuda_check(cudaStreamDestroy(s2), "cudaStreamDestroy");
            if (!ok) {
                std::cout << "FAIL caching allocator: stream-ordered reuse\n";
                ++failures;
            } else {
                std::cout << "ok   caching allocator orders reuse across streams\n";
            }
        }
        te::Backend::instance().synchronize();
    } catch (const std::exception& e) {
        std::cout << "FAIL unexpected exception: " << e.what() << "\n";
        return 1;
    }
    if (failures == 0) std::cout << "All C++ adapter checks passed.\n";
    return failures == 0 ? 0 : 1;
}
