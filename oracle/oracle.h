// Declarations shared by the oracle translation units. TEST INFRASTRUCTURE ONLY (see oracle.cpp).
#pragma once
#include <cstddef>
#include <cstdint>

extern "C" {

// Model description used by orc_model_forward*. Field meaning follows TrainConfig
// (src/train_efla_lm.cpp:186-300) and EflaLmWeights (:419-431) of the reference.
struct orc_model_cfg {
    int vocab;        // 256
    int hidden;       // H
    int layers;       // L
    int mlp_mult;     // F = mlp_mult * H
    int seq;          // T
    int batch;        // B
    int heads;        // 1 reproduces the reference; head_dim = H / heads
    int rank;         // 0: dense full-matrix noise (the reference's live path); r > 0: rank-r
    int sigma_shift;  // sigma = 2^-sigma_shift
    int use_clt;
    int clt_k;
    int method;       // 0 DeltaNet, 1 EFLA
    float act_scale;
    float mlp_act_scale;
    float ln_scale;
    float residual_scale;
    float mlp_residual_scale;
    float eps;
};

struct orc_model_weights {
    const int8_t* emb;    // [V][H]
    const int8_t* win;    // [H][H]
    const int8_t* wq;     // [L][H][H]
    const int8_t* wk;     // [L][H][H]
    const int8_t* wv;     // [L][H][H]
    const int8_t* wbeta;  // [L][H]
    const int8_t* ff1;    // [L][F][H]
    const int8_t* ff2;    // [L][H][F]
    const int8_t* head;   // [V][H]
    const float* head_bias;  // [V]
    const float* beta_bias;  // [L]
    const float* pos;        // [T][H]
};

// Optional taps: any non-null pointer receives that intermediate for the evaluated member
// (row index = b*T + t). Used to localise a device/oracle mismatch.
struct orc_model_taps {
    int8_t* emb_q;     // [R][H]
    float* inproj;     // [R][H]
    int8_t* x_q0;      // [R][H]  after pos+gelu
    float* qkv;        // [L][R][fused_cols]
    float* attn_y;     // [L][R][H]
    int8_t* ff1_q;     // [L][R][F]
    float* ff2_y;      // [L][R][H]
    int8_t* x_q;       // [L][R][H]  residual stream after each layer
    int8_t* y_q;       // [L][R][H]  normed stream after each layer
    float* logits;     // [R][V]
};

// Handle = base weights quantised once (DeviceWeights / quantize_nvfp4_base_weights,
// src/train_efla_lm.cpp:439-651, 1207-1310). The weight arrays must outlive the handle.
void* orc_model_create(const orc_model_cfg* cfg, const orc_model_weights* w);
void orc_model_destroy(void* handle);
// Mean next-token cross-entropy of one member (pair_seed, anti_sign in {+1,-1,0}); tokens/targets are
// uint8 [B][T]. Layer-major evaluation order (all T tokens of a layer at once).
double orc_model_forward(void* handle, const uint8_t* tokens, const uint8_t* targets, uint64_t pair_seed,
                         int anti_sign, orc_model_taps* taps);
// Same arithmetic in the reference's token-major order (src/train_efla_lm.cpp:2762-3371), kept to
// demonstrate that re-ordering the loops does not change any value.
double orc_model_forward_token_major(void* handle, const uint8_t* tokens, const uint8_t* targets,
                                     uint64_t pair_seed, int anti_sign);

// from oracle.cpp
uint64_t orc_mix(uint64_t a, uint64_t b);
int orc_noise_hash(uint64_t seed, uint64_t idx, int use_clt, int clt_k);
void orc_fill_noise(int8_t* out, size_t n, uint64_t seed, int use_clt, int clt_k);
size_t orc_sf_bytes(int rows, int K);
void orc_quantize_rowmajor(const int8_t* in, int rows, int k_in, int k_out, uint8_t* out, uint8_t* sf);
void orc_quantize_wqkv_fused(const int8_t* wq, const int8_t* wk, const int8_t* wv, const int8_t* wb, int hidden,
                             int k_out, float q_scale, float k_scale, float v_scale, float b_scale, uint8_t* out,
                             uint8_t* sf);
void orc_embedding_quant(const uint8_t* tokens, int token_stride, const int8_t* emb_w, const int8_t* emb_noise,
                         int hidden, int rows, float noise_scale, int anti_sign, int8_t* out_q, uint8_t* out,
                         uint8_t* sf);
void orc_embedding_lowrank_quant(const uint8_t* tokens, int token_stride, const int8_t* emb_w, const int8_t* A,
                                 const int8_t* B, int rank, int hidden, int rows, float scale, int8_t* out_q,
                                 uint8_t* out, uint8_t* sf);
void orc_add_pos_gelu_quant(const float* in, const float* pos, const int* pos_row, int hidden, int rows,
                            float act_scale, int8_t* out_q, uint8_t* out, uint8_t* sf);
void orc_activation_quant(const float* in, int rows, int cols_in, int cols_out, int mode, float act_scale,
                          int8_t* out_q, uint8_t* out, uint8_t* sf);
void orc_absmean_norm_q(int8_t* inout, const float* add_in, int hidden, int rows, float add_scale, float norm_scale,
                        int8_t* out_q, uint8_t* out, uint8_t* sf);
void orc_gemm_nvfp4(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, int m, int n, int k,
                    float alpha, float beta, const float* c, int ldc, float* d, int ldd, int gelu_i8,
                    float act_scale, int8_t* d8);
void orc_lora_compute_t(const int8_t* x, const int8_t* B, int cols, int batch, int rank, int32_t* t);
void orc_lora_add(const int32_t* t, const int8_t* A, int rows, int batch, int rank, float scale, float* out, int ldo);
void orc_efla_step_half_qkv_fused(uint16_t* S, const float* qkv, int fused_cols, float beta_bias, int hidden,
                                  int heads, int batch, int method, float eps, float* out);
void orc_efla_scan(const float* qkv, int fused_cols, const float* beta_bias_seq, int hidden, int heads, int seqs,
                   int T, int method, float eps, float* out);
void orc_set_num_threads(int n);
void orc_gaussian_f32(uint64_t seed, uint64_t tag, size_t n, float scale, float* out);
void orc_quantize_direct_f32(const float* in, int rows, int k_in, int k_out, uint8_t* codes, uint8_t* sf);
// What-if variants of the scan (state rounding cadence, operand precision); (1, 0) = the reference.
void orc_set_efla_variant(int state_round_every, int operand_bits);
double orc_cross_entropy_sum(const float* logits, int ld, const float* bias, const float* bias_noise, float bns,
                             const uint8_t* targets, int target_stride, int vocab, int rows, float* row_loss);
}

// Salts of the per-matrix noise streams (src/train_efla_lm.cpp:3822-3833).
namespace orc_salt {
constexpr uint64_t kEmb = 0x111111ULL, kWin = 0x222222ULL, kWq = 0x333333ULL, kWk = 0x444444ULL,
                   kWv = 0x555555ULL, kWbeta = 0x666666ULL, kFf1 = 0x999999ULL, kFf2 = 0xAAAAAAULL,
                   kHead = 0x777777ULL, kHeadBias = 0x888888ULL, kBetaBias = 0x9999999ULL, kPos = 0xBEEFF00DULL;
// Sub-streams of a matrix seed for the two rank-r factors (this build's definition; the reference
// has no live rank-r driver): A = noise(mix(seed, kFactorA), row*rank + r), B likewise per column.
constexpr uint64_t kFactorA = 0xA11CEULL, kFactorB = 0xB0BULL;
}  // namespace orc_salt
