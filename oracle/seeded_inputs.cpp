// seeded_inputs.cpp -- the reference benchmarks' input generators.  TEST INFRASTRUCTURE ONLY.
// The reference fills A then B from one std::mt19937(42) through std::uniform_real_distribution<float>(-1, 1)
// (src/benchmarks/matmul_benchmark.cpp:107-110, src/tests/cuda_test.cpp:355-358).  The distributions are
// library-defined, so the same library is used here instead of re-deriving them.
#include <cstdint>
#include <random>

#define ORACLE_API extern "C" __attribute__((visibility("default")))

struct OracleRng {
    std::mt19937 gen32;
    std::mt19937_64 gen64;
};

ORACLE_API OracleRng* oracle_rng_create(uint64_t seed) {
    OracleRng* r = new OracleRng();
    r->gen32.seed(static_cast<uint32_t>(seed));
    r->gen64.seed(seed);
    return r;
}
ORACLE_API void oracle_rng_destroy(OracleRng* r) { delete r; }

ORACLE_API void oracle_rng_uniform_f32(OracleRng* r, float* out, int64_t n, float lo, float hi) {
    std::uniform_real_distribution<float> dist(lo, hi);
    for (int64_t i = 0; i < n; ++i) out[i] = dist(r->gen32);
}
ORACLE_API void oracle_rng_normal_f32(OracleRng* r, float* out, int64_t n, float mean, float stddev) {
    std::normal_distribution<float> dist(mean, stddev);
    for (int64_t i = 0; i < n; ++i) out[i] = dist(r->gen32);
}
// Token ids uniform in [0, bound) from the 64-bit engine.
ORACLE_API void oracle_rng_tokens_i64(OracleRng* r, int64_t* out, int64_t n, int64_t bound) {
    std::uniform_int_distribution<int64_t> dist(0, bound - 1);
    for (int64_t i = 0; i < n; ++i) out[i] = dist(r->gen64);
}
