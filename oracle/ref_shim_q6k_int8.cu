// ref_shim_q6k_int8.cu — compiles the reference's Q6_K int8-MMQ test
// (tests/test_mmq_q6k_int8.cu) unmodified, with its main() renamed, and exports its
// seeded generators (:257-271) and host references (:202-222 float model, :224-255
// int8 model).  TEST INFRASTRUCTURE ONLY; nothing is copied.
#define main ref_q6k_int8_test_main
#include "tests/test_mmq_q6k_int8.cu"
#undef main

extern "C" void ref_q6k_fill(void* W, int n_blocks, uint32_t seed) {
    std::vector<block_q6_K> v((size_t)n_blocks);
    fill_q6k(v, seed);
    memcpy(W, v.data(), v.size() * sizeof(block_q6_K));
}
extern "C" void ref_q6k_half_fill(uint16_t* X, int n, uint32_t seed) {
    std::vector<half> v((size_t)n);
    fill_half(v, seed);
    memcpy(X, v.data(), v.size() * sizeof(half));
}
extern "C" void ref_q6k_models(const void* W, const uint16_t* X, uint16_t* Y_float, uint16_t* Y_int8,
                               int M, int N, int K) {
    std::vector<block_q6_K> w((size_t)M * (K / 256));
    memcpy(w.data(), W, w.size() * sizeof(block_q6_K));
    std::vector<half> x((size_t)N * K), y((size_t)N * M);
    memcpy(x.data(), X, x.size() * sizeof(half));
    host_ref(w, x, y, M, N, K);
    memcpy(Y_float, y.data(), y.size() * sizeof(half));
    host_int8_ref(w, x, y, M, N, K);
    memcpy(Y_int8, y.data(), y.size() * sizeof(half));
}
