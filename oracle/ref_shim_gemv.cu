// ref_shim_gemv.cu — builds the reference's own GEMV translation unit, unmodified,
// from where it lies (include path given by oracle/Makefile) and exports its
// file-local CPU golden `gemv_quant_cpu` (src/kernels/gemv_q4.cu:2519-2631) through
// a C symbol.  TEST INFRASTRUCTURE ONLY: no reference source text is copied here;
// the product library never links this object.
#include "src/kernels/gemv_q4.cu"

extern "C" int ref_gemv_quant_cpu(float* y, const void* W, int ggml_type,
                                  const uint16_t* x_bits, int M, int K) {
    std::vector<half> hx((size_t)K);
    memcpy(hx.data(), x_bits, (size_t)K * sizeof(half));
    std::vector<float> hy;
    if (!jllm::gemv_quant_cpu(hy, W, ggml_type, hx, M, K)) return 0;
    memcpy(y, hy.data(), (size_t)M * sizeof(float));
    return 1;
}
