// C++ entry points with the reference's own names and signatures (namespaces bitnet_cuda and efla_lm_cuda,
// reference: src/cuda_kernels.h:8-454 and src/efla_lm_kernels.h:8-342), exported by libbnf4.so so that the
// reference driver (src/train_efla_lm.cpp) links against this library unchanged. Each is a thin wrapper over the
// extern "C" function named bnf4_<same name>; like the reference they return void. A non-zero status is kept in
// bnf4_last_error() and thrown as std::runtime_error. Entry points of non-default experiment flags exist for link
// compatibility and report "unsupported" that way.

#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

#include <stdexcept>

// The reference's entry points return void and its driver checks its own CUDA calls with an exception (cuda_check,
// src/train_efla_lm.cpp:46-50). A failure inside one of these wrappers is reported the same way: the message is kept in
// bnf4_last_error() and thrown as std::runtime_error, so a driver that reaches an entry point outside this path, or passes
// arguments a kernel rejects, stops with a diagnostic instead of continuing on unwritten buffers.
static void chk(int rc) {
    if (rc != 0) throw std::runtime_error(bnf4_last_error());
}
#define UNSUPPORTED(name) chk(bnf4::set_error(BNF4_ERR_UNSUPPORTED, #name ": not part of the NVFP4 population-evaluation path"))

namespace bitnet_cuda {

enum class Nvfp4Schedule { Auto = 0, Cooperative = 1, Pingpong = 2 };
enum class Nvfp4QuantMode { Warp16 = 0, Warp4 = 1 };
enum class Nvfp4StageCount { Auto = 0, Stages2 = 2, Stages3 = 3, Stages4 = 4 };
enum class Nvfp4Decomposition { Heuristic = 0, DataParallel = 1, SplitK = 2, StreamK = 3 };

// ---- default path ---------------------------------------------------------------------------------------------
size_t nvfp4_sfa_bytes(int m, int n, int k) { return bnf4_nvfp4_sfa_bytes(m, n, k); }
size_t nvfp4_sfb_bytes(int m, int n, int k) { return bnf4_nvfp4_sfb_bytes(m, n, k); }
// The tuning knobs of the reference select among CUTLASS instantiations; one hand-written kernel serves all shapes here.
void nvfp4_init() {}
void nvfp4_set_schedule(Nvfp4Schedule) {}
void nvfp4_set_quant_mode(Nvfp4QuantMode) {}
void nvfp4_set_stage_count(Nvfp4StageCount) {}
void nvfp4_set_decomposition(Nvfp4Decomposition) {}
void nvfp4_set_verbose(bool) {}
void nvfp4_set_splits(int) {}

bool nvfp4_prepare_gemm(const void* d_a, const void* d_b, const void* d_sfa, const void* d_sfb, int m, int n, int k, float alpha,
                        float beta, const float* d_c, float* d_d, cudaStream_t stream) {
    return bnf4_nvfp4_prepare_gemm(d_a, d_b, d_sfa, d_sfb, m, n, k, alpha, beta, d_c, d_d, stream) == 0;
}
void nvfp4_quantize_a(const int8_t* d_in, int m, int n, int k_in, int k_out, void* d_out, void* d_sfa, cudaStream_t stream) {
    chk(bnf4_nvfp4_quantize_a(d_in, m, n, k_in, k_out, d_out, d_sfa, stream));
}
void nvfp4_quantize_b(const int8_t* d_in, int m, int n, int k_in, int k_out, void* d_out, void* d_sfb, cudaStream_t stream) {
    chk(bnf4_nvfp4_quantize_b(d_in, m, n, k_in, k_out, d_out, d_sfb, stream));
}
void nvfp4_quantize_wqkv_fused(const int8_t* d_wq, const int8_t* d_wk, const int8_t* d_wv, const int8_t* d_wb, int batch, int hidden,
                               int k_out, int rows_total, float q_scale, float k_scale, float v_scale, float b_scale, void* d_out,
                               void* d_sfb, cudaStream_t stream) {
    chk(bnf4_nvfp4_quantize_wqkv_fused(d_wq, d_wk, d_wv, d_wb, batch, hidden, k_out, rows_total, q_scale, k_scale, v_scale, b_scale, d_out, d_sfb,
                                   stream));
}
void embedding_lookup_noise_quantize_nvfp4(const uint8_t* d_tokens_t, int token_stride, const int8_t* d_emb_w, const int8_t* d_emb_noise,
                                           int hidden, int batch, float noise_scale, int anti_sign, int8_t* d_out_q, void* d_out_nvfp4,
                                           void* d_sfa, cudaStream_t stream) {
    chk(bnf4_embedding_lookup_noise_quantize_nvfp4(d_tokens_t, token_stride, d_emb_w, d_emb_noise, hidden, batch, noise_scale, anti_sign, d_out_q,
                                               d_out_nvfp4, d_sfa, stream));
}
void add_pos_gelu_quantize_nvfp4(const float* d_in, const float* d_pos_t, int hidden, int batch, float act_scale, int8_t* d_out_q,
                                 void* d_out_nvfp4, void* d_sfa, cudaStream_t stream) {
    chk(bnf4_add_pos_gelu_quantize_nvfp4(d_in, d_pos_t, hidden, batch, act_scale, d_out_q, d_out_nvfp4, d_sfa, stream));
}
void activation_quantize_nvfp4(const float* d_in, int rows, int cols_in, int cols_out, int activation, int8_t* d_out_q, void* d_out_nvfp4,
                               void* d_sfa, cudaStream_t stream) {
    chk(bnf4_activation_quantize_nvfp4(d_in, rows, cols_in, cols_out, activation, d_out_q, d_out_nvfp4, d_sfa, stream));
}
void gelu_quantize_nvfp4(const float* d_in, int rows, int cols_in, int cols_out, float act_scale, int8_t* d_out_q, void* d_out_nvfp4,
                         void* d_sfa, cudaStream_t stream) {
    chk(bnf4_gelu_quantize_nvfp4(d_in, rows, cols_in, cols_out, act_scale, d_out_q, d_out_nvfp4, d_sfa, stream));
}
void absmean_norm_q_nvfp4(const int8_t* d_in, int hidden, int batch, int cols_out, float scale, int8_t* d_out_q, void* d_out_nvfp4,
                          void* d_sfa, cudaStream_t stream) {
    chk(bnf4_absmean_norm_q_nvfp4(d_in, hidden, batch, cols_out, scale, d_out_q, d_out_nvfp4, d_sfa, stream));
}
void add_scaled_to_int8_absmean_norm_q_nvfp4(int8_t* d_inout, const float* d_in, int hidden, int batch, int cols_out, float add_scale,
                                             float norm_scale, int8_t* d_out_q, void* d_out_nvfp4, void* d_sfa, cudaStream_t stream) {
    chk(bnf4_add_scaled_to_int8_absmean_norm_q_nvfp4(d_inout, d_in, hidden, batch, cols_out, add_scale, norm_scale, d_out_q, d_out_nvfp4, d_sfa,
                                                 stream));
}
void split_qkvb_fused(const float* d_in, int batch, int hidden, int fused_cols, float* d_q, float* d_k, float* d_v, float* d_beta,
                      float beta_bias, bool /*use_vec4*/, cudaStream_t stream) {
    chk(bnf4_split_qkvb_fused(d_in, batch, hidden, fused_cols, d_q, d_k, d_v, d_beta, beta_bias, stream));
}
void gemm_ternary_f_nvfp4(const void* d_a, const void* d_b, const void* d_sfa, const void* d_sfb, int m, int n, int k, float alpha, float beta,
                          const float* d_c, float* d_d, cudaStream_t stream) {
    chk(bnf4_gemm_ternary_f_nvfp4(d_a, d_b, d_sfa, d_sfb, m, n, k, alpha, beta, d_c, d_d, stream));
}
void gemm_ternary_f_nvfp4_gelu_i8(const void* d_a, const void* d_b, const void* d_sfa, const void* d_sfb, int m, int n, int k, float alpha,
                                  float beta, const float* d_c, float act_scale, int8_t* d_d, cudaStream_t stream) {
    chk(bnf4_gemm_ternary_f_nvfp4_gelu_i8(d_a, d_b, d_sfa, d_sfb, m, n, k, alpha, beta, d_c, act_scale, d_d, stream));
}
void gemm_ternary_f(const int8_t* d_x, const int8_t* d_w, const float* d_scale_x, int rows, int cols, int batch, float out_scale,
                    float* d_out, cudaStream_t stream) {
    chk(bnf4_gemm_ternary_f(d_x, d_w, d_scale_x, rows, cols, batch, out_scale, d_out, stream));
}
void lora_compute_t(const int8_t* d_x, const int8_t* d_B, int cols, int batch, int rank, int32_t* d_t, cudaStream_t stream) {
    chk(bnf4_lora_compute_t(d_x, d_B, cols, batch, rank, d_t, stream));
}
void lora_add(const int32_t* d_t, const int8_t* d_A, int rows, int batch, int rank, float scale, float* d_out, cudaStream_t stream) {
    chk(bnf4_lora_add(d_t, d_A, rows, batch, rank, scale, d_out, stream));
}
void gemm_ternary_lora_f(const int8_t* d_x, const int8_t* d_w, const float* d_scale_x, int rows, int cols, int batch, float out_scale,
                         const int8_t* d_A, const int32_t* d_t, int rank, float lora_scale, float* d_out, cudaStream_t stream) {
    chk(bnf4_gemm_ternary_f(d_x, d_w, d_scale_x, rows, cols, batch, out_scale, d_out, stream));
    chk(bnf4_lora_add(d_t, d_A, rows, batch, rank, lora_scale, d_out, stream));
}

// ---- experiment flags of the reference that are outside this path ---------------------------------------------------
void gemm_ternary(const int8_t*, const int8_t*, int, int, int, float, float*, cudaStream_t) { UNSUPPORTED(gemm_ternary); }
void gemm_ternary_act_quant(const int8_t*, const int8_t*, const float*, int, int, int, float, int, int8_t*, cudaStream_t) {
    UNSUPPORTED(gemm_ternary_act_quant);
}
void gemm_ternary_gelu_quant(const int8_t*, const int8_t*, const int8_t*, const float*, int, int, int, float, float, float, int8_t*,
                             cudaStream_t) {
    UNSUPPORTED(gemm_ternary_gelu_quant);
}
void gemm_ternary_lora_act_quant(const int8_t*, const int8_t*, const float*, int, int, int, float, const int8_t*, const int32_t*, int, float,
                                 int, int8_t*, cudaStream_t) {
    UNSUPPORTED(gemm_ternary_lora_act_quant);
}
void gemm_ternary_sparse_act_quant(const int8_t*, const int8_t*, const float*, int, int, int, float, const int32_t*, const int32_t*,
                                   const int8_t*, float, int, int8_t*, cudaStream_t) {
    UNSUPPORTED(gemm_ternary_sparse_act_quant);
}
void head_gemm_cross_entropy(const int8_t*, const int8_t*, const int8_t*, const float*, int, int, int, float, float, const float*,
                             const float*, float, const uint8_t*, int, float*, cudaStream_t) {
    UNSUPPORTED(head_gemm_cross_entropy);
}
void gemm_ternary_f_noise(const int8_t*, const int8_t*, const int8_t*, const float*, int, int, int, float, float, float*, cudaStream_t) {
    UNSUPPORTED(gemm_ternary_f_noise);
}
void gemm_ternary_f_noise_tiled(const int8_t*, const int8_t*, const int8_t*, const float*, int, int, int, float, float, float*,
                                cudaStream_t) {
    UNSUPPORTED(gemm_ternary_f_noise_tiled);
}
void gemm_qkvb_fused(const int8_t*, const int8_t*, const int8_t*, const int8_t*, const int8_t*, const int8_t*, const int8_t*, const int8_t*,
                     const int8_t*, const float*, int, int, int, float, float, float, float, float, float*, float*, float*, float*,
                     cudaStream_t) {
    UNSUPPORTED(gemm_qkvb_fused);
}
void pack_ternary_i2(const int8_t*, int, int, uint32_t*, cudaStream_t) { UNSUPPORTED(pack_ternary_i2); }
void pack_ternary_i2_bitnet(const int8_t*, int, int, uint32_t*, cudaStream_t) { UNSUPPORTED(pack_ternary_i2_bitnet); }
void init_i2_lut() {}
void gemm_ternary_f_i2(const int8_t*, const uint32_t*, const float*, int, int, int, float, float*, cudaStream_t) { UNSUPPORTED(gemm_ternary_f_i2); }
void gemm_ternary_f_i2_noise(const int8_t*, const uint32_t*, const uint32_t*, const float*, int, int, int, float, float, float*,
                             cudaStream_t) {
    UNSUPPORTED(gemm_ternary_f_i2_noise);
}
void gemm_ternary_f_i2_bitnet(const int8_t*, const uint32_t*, const float*, int, int, int, float, float*, cudaStream_t) {
    UNSUPPORTED(gemm_ternary_f_i2_bitnet);
}
void gemm_ternary_f_i2_bitnet_noise(const int8_t*, const uint32_t*, const uint32_t*, const float*, int, int, int, float, float, float*,
                                    cudaStream_t) {
    UNSUPPORTED(gemm_ternary_f_i2_bitnet_noise);
}
void gemm_ternary_f_cutlass(const int8_t*, const int8_t*, int, int, int, float, float*, cudaStream_t) { UNSUPPORTED(gemm_ternary_f_cutlass); }
void gemm_ternary_sparse_f(const int8_t*, const int8_t*, const float*, int, int, int, float, const int32_t*, const int32_t*, const int8_t*,
                           float, float*, cudaStream_t) {
    UNSUPPORTED(gemm_ternary_sparse_f);
}
void sparse_add(const int32_t*, const int32_t*, const int8_t*, int, int, int, const int8_t*, float, float*, cudaStream_t) {
    UNSUPPORTED(sparse_add);
}
void activation_quantize(const float*, int8_t*, int, int, cudaStream_t) { UNSUPPORTED(activation_quantize); }
void embed_update_plain(const uint8_t*, int, const int8_t*, int, int, int8_t*, cudaStream_t) { UNSUPPORTED(embed_update_plain); }
void embed_update_lora(const uint8_t*, int, const int8_t*, const int8_t*, const int8_t*, int, int, int, float, int8_t*, cudaStream_t) {
    UNSUPPORTED(embed_update_lora);
}
void embed_update_sparse(const uint8_t*, int, const int8_t*, const int16_t*, int, int, float, int8_t*, cudaStream_t) {
    UNSUPPORTED(embed_update_sparse);
}

}  // namespace bitnet_cuda

namespace efla_lm_cuda {

struct NoiseDesc {
    int8_t* out = nullptr;
    size_t n = 0;
    uint64_t seed = 0;
};
static_assert(sizeof(NoiseDesc) == sizeof(bnf4_noise_desc), "NoiseDesc layout");

// ---- default path ---------------------------------------------------------------------------------------------
void add_scaled(float* d_out, const float* d_noise, int n, float scale, cudaStream_t stream) { chk(bnf4_add_scaled(d_out, d_noise, n, scale, stream)); }
void init_shadow_from_weights(const int8_t* d_w, float* d_shadow, int n, cudaStream_t stream) { chk(bnf4_init_shadow_from_weights(d_w, d_shadow, n, stream)); }
void fill_pair_seeds(uint64_t base_seed, uint64_t epoch, int pairs, uint64_t* d_out, cudaStream_t stream) {
    chk(bnf4_fill_pair_seeds(base_seed, epoch, pairs, d_out, stream));
}
void compute_z_sumsq(const float* d_pair_weights, const uint64_t* d_pair_seeds, uint64_t salt, int pairs, int n, bool use_clt, int clt_k,
                     float* d_Z, float* d_sumsq, cudaStream_t stream) {
    chk(bnf4_compute_z_sumsq(d_pair_weights, d_pair_seeds, salt, pairs, n, use_clt ? 1 : 0, clt_k, d_Z, d_sumsq, stream));
}
void update_inv_rms(const float* d_sumsq, float* d_rms_ema, bool use_adaptive, float adaptive_beta, float adaptive_eps, int n,
                    float* d_inv_rms, cudaStream_t stream) {
    chk(bnf4_update_inv_rms(d_sumsq, d_rms_ema, use_adaptive ? 1 : 0, adaptive_beta, adaptive_eps, n, d_inv_rms, stream));
}
void update_shadow_ternary(int8_t* d_w, float* d_shadow, const float* d_Z, int n, float inv_rms, float lr, float thresh, cudaStream_t stream) {
    chk(bnf4_update_shadow_ternary(d_w, d_shadow, d_Z, n, inv_rms, lr, thresh, stream));
}
void update_shadow_ternary_device(int8_t* d_w, float* d_shadow, const float* d_Z, int n, const float* d_inv_rms, float lr, float thresh,
                                  cudaStream_t stream) {
    chk(bnf4_update_shadow_ternary_device(d_w, d_shadow, d_Z, n, d_inv_rms, lr, thresh, stream));
}
void efla_step(float* d_S, const float* d_q, const float* d_k, const float* d_v, const float* d_beta_raw, float beta_bias, int hidden,
               int batch, int method, float eps, bool /*use_fuse_diff*/, float* d_out, float*, float*, float*, float*, float*,
               cudaStream_t stream) {
    chk(bnf4_efla_step(d_S, 0, d_q, d_k, d_v, d_beta_raw, beta_bias, hidden, batch, method, eps, d_out, stream));
}
void efla_step_half(__half* d_S, const float* d_q, const float* d_k, const float* d_v, const float* d_beta_raw, float beta_bias, int hidden,
                    int batch, int method, float eps, bool, bool, bool, float* d_out, float*, float*, __half*, float*, float*, __half*, float*,
                    cudaStream_t stream) {
    chk(bnf4_efla_step(d_S, 1, d_q, d_k, d_v, d_beta_raw, beta_bias, hidden, batch, method, eps, d_out, stream));
}
void efla_step_qkv_fused(float* d_S, const float* d_qkv, int fused_cols, float beta_bias, int hidden, int batch, int method, float eps,
                         float* d_out, float*, float*, float*, float*, float*, cudaStream_t stream) {
    chk(bnf4_efla_step_qkv_fused(d_S, d_qkv, fused_cols, beta_bias, hidden, batch, method, eps, d_out, stream));
}
void efla_step_half_qkv_fused(__half* d_S, const float* d_qkv, int fused_cols, float beta_bias, int hidden, int batch, int method, float eps,
                              float* d_out, float*, float*, float*, float*, float*, cudaStream_t stream) {
    chk(bnf4_efla_step_half_qkv_fused(d_S, d_qkv, fused_cols, beta_bias, hidden, batch, method, eps, d_out, stream));
}
void efla_step_fused(float* d_S, const float* d_q, const float* d_k, const float* d_v, const float* d_beta_raw, float beta_bias, int hidden,
                     int batch, int method, float eps, float* d_out, cudaStream_t stream) {
    chk(bnf4_efla_step(d_S, 0, d_q, d_k, d_v, d_beta_raw, beta_bias, hidden, batch, method, eps, d_out, stream));
}
void efla_step_fused_half(__half* d_S, const float* d_q, const float* d_k, const float* d_v, const float* d_beta_raw, float beta_bias,
                          int hidden, int batch, int method, float eps, float* d_out, cudaStream_t stream) {
    chk(bnf4_efla_step(d_S, 1, d_q, d_k, d_v, d_beta_raw, beta_bias, hidden, batch, method, eps, d_out, stream));
}
void cross_entropy_loss(const float* d_logits, const float* d_bias, const float* d_bias_noise, float bias_noise_scale,
                        const uint8_t* d_targets_t, int token_stride, int vocab, int batch, float* d_loss_accum, cudaStream_t stream) {
    chk(bnf4_cross_entropy_loss(d_logits, d_bias, d_bias_noise, bias_noise_scale, d_targets_t, token_stride, vocab, batch, d_loss_accum, stream));
}
void fill_ternary_noise(int8_t* d_out, size_t n, uint64_t seed, bool use_clt, int clt_k, cudaStream_t stream) {
    chk(bnf4_fill_ternary_noise(d_out, n, seed, use_clt ? 1 : 0, clt_k, stream));
}
void fill_ternary_noise_batched(NoiseDesc* d_descs, int num_desc, int max_blocks, bool use_clt, int clt_k, cudaStream_t stream) {
    chk(bnf4_fill_ternary_noise_batched(reinterpret_cast<const bnf4_noise_desc*>(d_descs), num_desc, max_blocks, use_clt ? 1 : 0, clt_k, stream));
}
void fill_float_noise(float* d_out, int n, uint64_t seed, bool use_clt, int clt_k, cudaStream_t stream) {
    chk(bnf4_fill_float_noise(d_out, n, seed, use_clt ? 1 : 0, clt_k, stream));
}

// ---- non-default model variants ---------------------------------------------------------------------------------------
void embedding_lookup_noise(const uint8_t*, int, const int8_t*, const int8_t*, int, int, float, int, float*, cudaStream_t) {
    UNSUPPORTED(embedding_lookup_noise);
}
void add_pos_gelu_quantize(const float*, const float*, int, int, float, int8_t*, cudaStream_t) { UNSUPPORTED(add_pos_gelu_quantize); }
void add_pos_gelu(const float*, const float*, int, int, float, float*, cudaStream_t) { UNSUPPORTED(add_pos_gelu); }
void gelu_quantize(const float*, int, float, int8_t*, cudaStream_t) { UNSUPPORTED(gelu_quantize); }
void add_scaled_i8(float*, const int8_t*, int, float, cudaStream_t) { UNSUPPORTED(add_scaled_i8); }
void add_scaled_to_int8(int8_t*, const float*, int, float, cudaStream_t) { UNSUPPORTED(add_scaled_to_int8); }
void add_scaled_to_int8_absmean_norm_q(int8_t*, const float*, int, int, float, float, int8_t*, cudaStream_t) {
    UNSUPPORTED(add_scaled_to_int8_absmean_norm_q);
}
void layernorm_quantize(const float*, int, int, float, float, int8_t*, cudaStream_t) { UNSUPPORTED(layernorm_quantize); }
void absmean_norm_q(const int8_t*, int, int, float, int8_t*, cudaStream_t) { UNSUPPORTED(absmean_norm_q); }
void update_shadow_ternary_device_packed(int8_t*, uint32_t*, float*, const float*, int, const float*, float, float, cudaStream_t) {
    UNSUPPORTED(update_shadow_ternary_device_packed);
}
void update_shadow_ternary_device_packed_bitnet(int8_t*, uint32_t*, float*, const float*, int, const float*, float, float, cudaStream_t) {
    UNSUPPORTED(update_shadow_ternary_device_packed_bitnet);
}
void efla_step_lowrank(float*, float*, const float*, const float*, const float*, const float*, float, float, float, int, int, int, float,
                       float*, cudaStream_t) {
    UNSUPPORTED(efla_step_lowrank);
}

}  // namespace efla_lm_cuda
