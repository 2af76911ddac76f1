// Checker built from the reference's own device code. TEST INFRASTRUCTURE ONLY.
//
// The reference's src/cuda_kernels.cu guards its NVFP4 quantiser kernels and its dp4a ternary GEMMs only by
// BITNET_EGGROLL_HAS_CUTLASS; the block-scaled GEMM itself sits behind the CUTLASS SM120 guard and compiles to
// a stub on any other architecture. With a CUTLASS header tree on the include path (see the Makefile: the
// location is passed in, nothing of CUTLASS or of the reference is copied into this repository) the file
// therefore compiles for sm_100a from where it lies, and the extern "C" wrappers below let the GPU tests run the
// reference's own quantisers, dp4a ternary GEMM and rank-r helpers next to this library's on the same inputs.
#include "cuda_kernels.h"

#define REF_API extern "C" __attribute__((visibility("default")))
#define ST(s) static_cast<cudaStream_t>(s)

// 0 = Warp16 (the reference's default), 1 = Warp4. In the Warp16 kernels (and the Warp4 embedding kernel) lane 0 alone
// executes sixteen __shfl_sync calls whose mask names sixteen lanes (src/cuda_kernels.cu:1612-1622 and the same
// pattern at :1869, :2003, :2100, :2340, :2580, :2845); what the other lanes' codes read as is then undefined. The
// scale bytes, the int8 copies and each block's first code do not depend on that gather; the Warp4 kernels are
// well-formed and produce every code.
REF_API void refq_nvfp4_set_quant_mode(int mode) {
    bitnet_cuda::nvfp4_set_quant_mode(mode ? bitnet_cuda::Nvfp4QuantMode::Warp4 : bitnet_cuda::Nvfp4QuantMode::Warp16);
}

REF_API size_t refq_nvfp4_sfa_bytes(int m, int n, int k) { return bitnet_cuda::nvfp4_sfa_bytes(m, n, k); }
REF_API size_t refq_nvfp4_sfb_bytes(int m, int n, int k) { return bitnet_cuda::nvfp4_sfb_bytes(m, n, k); }

REF_API void refq_nvfp4_quantize_a(const int8_t* in, int m, int n, int k_in, int k_out, void* out, void* sfa, void* stream) {
    bitnet_cuda::nvfp4_quantize_a(in, m, n, k_in, k_out, out, sfa, ST(stream));
}
REF_API void refq_nvfp4_quantize_b(const int8_t* in, int m, int n, int k_in, int k_out, void* out, void* sfb, void* stream) {
    bitnet_cuda::nvfp4_quantize_b(in, m, n, k_in, k_out, out, sfb, ST(stream));
}
REF_API void refq_nvfp4_quantize_wqkv_fused(const int8_t* wq, const int8_t* wk, const int8_t* wv, const int8_t* wb, int batch, int hidden,
                                            int k_out, int rows_total, float qs, float ks, float vs, float bs, void* out, void* sfb,
                                            void* stream) {
    bitnet_cuda::nvfp4_quantize_wqkv_fused(wq, wk, wv, wb, batch, hidden, k_out, rows_total, qs, ks, vs, bs, out, sfb, ST(stream));
}
REF_API void refq_embedding_lookup_noise_quantize_nvfp4(const uint8_t* tokens_t, int token_stride, const int8_t* emb_w,
                                                        const int8_t* emb_noise, int hidden, int batch, float noise_scale, int anti_sign,
                                                        int8_t* out_q, void* out_nvfp4, void* sfa, void* stream) {
    bitnet_cuda::embedding_lookup_noise_quantize_nvfp4(tokens_t, token_stride, emb_w, emb_noise, hidden, batch, noise_scale, anti_sign,
                                                       out_q, out_nvfp4, sfa, ST(stream));
}
REF_API void refq_add_pos_gelu_quantize_nvfp4(const float* in, const float* pos_t, int hidden, int batch, float act_scale, int8_t* out_q,
                                              void* out_nvfp4, void* sfa, void* stream) {
    bitnet_cuda::add_pos_gelu_quantize_nvfp4(in, pos_t, hidden, batch, act_scale, out_q, out_nvfp4, sfa, ST(stream));
}
REF_API void refq_gelu_quantize_nvfp4(const float* in, int rows, int cols_in, int cols_out, float act_scale, int8_t* out_q,
                                      void* out_nvfp4, void* sfa, void* stream) {
    bitnet_cuda::gelu_quantize_nvfp4(in, rows, cols_in, cols_out, act_scale, out_q, out_nvfp4, sfa, ST(stream));
}
REF_API void refq_activation_quantize_nvfp4(const float* in, int rows, int cols_in, int cols_out, int activation, int8_t* out_q,
                                            void* out_nvfp4, void* sfa, void* stream) {
    bitnet_cuda::activation_quantize_nvfp4(in, rows, cols_in, cols_out, activation, out_q, out_nvfp4, sfa, ST(stream));
}
REF_API void refq_absmean_norm_q_nvfp4(const int8_t* in, int hidden, int batch, int cols_out, float scale, int8_t* out_q, void* out_nvfp4,
                                       void* sfa, void* stream) {
    bitnet_cuda::absmean_norm_q_nvfp4(in, hidden, batch, cols_out, scale, out_q, out_nvfp4, sfa, ST(stream));
}
REF_API void refq_add_scaled_to_int8_absmean_norm_q_nvfp4(int8_t* inout, const float* in, int hidden, int batch, int cols_out,
                                                          float add_scale, float norm_scale, int8_t* out_q, void* out_nvfp4, void* sfa,
                                                          void* stream) {
    bitnet_cuda::add_scaled_to_int8_absmean_norm_q_nvfp4(inout, in, hidden, batch, cols_out, add_scale, norm_scale, out_q, out_nvfp4, sfa,
                                                         ST(stream));
}
REF_API void refq_gemm_ternary_f(const int8_t* x, const int8_t* w, const float* scale_x, int rows, int cols, int batch, float out_scale,
                                 float* out, void* stream) {
    bitnet_cuda::gemm_ternary_f(x, w, scale_x, rows, cols, batch, out_scale, out, ST(stream));
}
REF_API void refq_gemm_ternary_f_noise(const int8_t* x, const int8_t* w, const int8_t* w_noise, const float* scale_x, int rows, int cols,
                                       int batch, float out_scale, float noise_scale, float* out, void* stream) {
    bitnet_cuda::gemm_ternary_f_noise(x, w, w_noise, scale_x, rows, cols, batch, out_scale, noise_scale, out, ST(stream));
}
REF_API void refq_lora_compute_t(const int8_t* x, const int8_t* B, int cols, int batch, int rank, int32_t* t, void* stream) {
    bitnet_cuda::lora_compute_t(x, B, cols, batch, rank, t, ST(stream));
}
REF_API void refq_lora_add(const int32_t* t, const int8_t* A, int rows, int batch, int rank, float scale, float* out, void* stream) {
    bitnet_cuda::lora_add(t, A, rows, batch, rank, scale, out, ST(stream));
}
REF_API void refq_gemm_ternary_lora_f(const int8_t* x, const int8_t* w, const float* scale_x, int rows, int cols, int batch,
                                      float out_scale, const int8_t* A, const int32_t* t, int rank, float lora_scale, float* out,
                                      void* stream) {
    bitnet_cuda::gemm_ternary_lora_f(x, w, scale_x, rows, cols, batch, out_scale, A, t, rank, lora_scale, out, ST(stream));
}
REF_API void refq_split_qkvb_fused(const float* in, int batch, int hidden, int fused_cols, float* q, float* k, float* v, float* beta,
                                   float beta_bias, int use_vec4, void* stream) {
    bitnet_cuda::split_qkvb_fused(in, batch, hidden, fused_cols, q, k, v, beta, beta_bias, use_vec4 != 0, ST(stream));
}
