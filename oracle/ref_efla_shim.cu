// Checker built from the reference's own device code. TEST INFRASTRUCTURE ONLY.
//
// The reference's src/efla_lm_kernels.cu needs no CUTLASS, so it is compiled for sm_100a straight from where it
// lies (see the Makefile; nothing of it is copied into this repository) and exposed through the extern "C"
// wrappers below. GPU tests run the reference's own EFLA step, cross-entropy, noise and ES-update kernels next to
// this library's kernels on the same inputs.
#include "efla_lm_kernels.h"

#define REF_API extern "C" __attribute__((visibility("default")))

REF_API void ref_efla_step_half_qkv_fused(void* S, const float* qkv, int fused_cols, float beta_bias, int hidden, int batch, int method,
                                          float eps, float* out, float* q_norm, float* k_usage, float* kS, float* diff, float* alpha,
                                          void* stream) {
    efla_lm_cuda::efla_step_half_qkv_fused(static_cast<__half*>(S), qkv, fused_cols, beta_bias, hidden, batch, method, eps, out, q_norm,
                                           k_usage, kS, diff, alpha, static_cast<cudaStream_t>(stream));
}
REF_API void ref_efla_step_fused_half(void* S, const float* q, const float* k, const float* v, const float* beta_raw, float beta_bias,
                                      int hidden, int batch, int method, float eps, float* out, void* stream) {
    efla_lm_cuda::efla_step_fused_half(static_cast<__half*>(S), q, k, v, beta_raw, beta_bias, hidden, batch, method, eps, out,
                                       static_cast<cudaStream_t>(stream));
}
REF_API void ref_cross_entropy_loss(const float* logits, const float* bias, const float* bias_noise, float bns, const uint8_t* targets_t,
                                    int token_stride, int vocab, int batch, float* loss_accum, void* stream) {
    efla_lm_cuda::cross_entropy_loss(logits, bias, bias_noise, bns, targets_t, token_stride, vocab, batch, loss_accum,
                                     static_cast<cudaStream_t>(stream));
}
REF_API void ref_fill_ternary_noise(int8_t* out, size_t n, uint64_t seed, int use_clt, int clt_k, void* stream) {
    efla_lm_cuda::fill_ternary_noise(out, n, seed, use_clt != 0, clt_k, static_cast<cudaStream_t>(stream));
}
REF_API void ref_fill_pair_seeds(uint64_t base_seed, uint64_t epoch, int pairs, uint64_t* out, void* stream) {
    efla_lm_cuda::fill_pair_seeds(base_seed, epoch, pairs, out, static_cast<cudaStream_t>(stream));
}
REF_API void ref_init_shadow_from_weights(const int8_t* w, float* shadow, int n, void* stream) {
    efla_lm_cuda::init_shadow_from_weights(w, shadow, n, static_cast<cudaStream_t>(stream));
}
REF_API void ref_compute_z_sumsq(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs, int n, int use_clt,
                                 int clt_k, float* Z, float* sumsq, void* stream) {
    efla_lm_cuda::compute_z_sumsq(pair_weights, pair_seeds, salt, pairs, n, use_clt != 0, clt_k, Z, sumsq, static_cast<cudaStream_t>(stream));
}
REF_API void ref_update_inv_rms(const float* sumsq, float* rms_ema, int use_adaptive, float beta, float eps, int n, float* inv_rms,
                                void* stream) {
    efla_lm_cuda::update_inv_rms(sumsq, rms_ema, use_adaptive != 0, beta, eps, n, inv_rms, static_cast<cudaStream_t>(stream));
}
REF_API void ref_update_shadow_ternary_device(int8_t* w, float* shadow, const float* Z, int n, const float* inv_rms, float lr, float thresh,
                                              void* stream) {
    efla_lm_cuda::update_shadow_ternary_device(w, shadow, Z, n, inv_rms, lr, thresh, static_cast<cudaStream_t>(stream));
}
