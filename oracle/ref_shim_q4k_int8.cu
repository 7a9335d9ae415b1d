// ref_shim_q4k_int8.cu — compiles the reference's Q4_K int8-MMQ test
// (tests/test_mmq_q4k_int8.cu) unmodified, with its main() renamed, and exports its
// seeded generators (:434-451) and host references (:340-371 float model, :373-432
// int8 model) so golden vectors come from the reference's own code.
// TEST INFRASTRUCTURE ONLY; nothing is copied, the include path comes from the Makefile.
#define main ref_q4k_int8_test_main
#include "tests/test_mmq_q4k_int8.cu"
#undef main

extern "C" void ref_q4k_fill(void* W, int n_blocks, uint32_t seed) {
    std::vector<block_q4_K> v((size_t)n_blocks);
    fill_random_q4k(v, seed);
    memcpy(W, v.data(), v.size() * sizeof(block_q4_K));
}
extern "C" void ref_half_fill(uint16_t* X, int n, uint32_t seed, float lo, float hi) {
    std::vector<half> v((size_t)n);
    fill_random_half(v, seed, lo, hi);
    memcpy(X, v.data(), v.size() * sizeof(half));
}
extern "C" void ref_q4k_models(const void* W, const uint16_t* X, uint16_t* Y_float, uint16_t* Y_int8,
                               int M, int N, int K) {
    std::vector<block_q4_K> w((size_t)M * (K / 256));
    memcpy(w.data(), W, w.size() * sizeof(block_q4_K));
    std::vector<half> x((size_t)N * K), y((size_t)N * M);
    memcpy(x.data(), X, x.size() * sizeof(half));
    host_reference(w, x, y, M, N, K);
    memcpy(Y_float, y.data(), y.size() * sizeof(half));
    host_int8_reference(w, x, y, M, N, K);
    memcpy(Y_int8, y.data(), y.size() * sizeof(half));
}
