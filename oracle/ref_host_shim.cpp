// Checker built from the reference's own host code. TEST INFRASTRUCTURE ONLY.
//
// The reference's driver translation unit (src/train_efla_lm.cpp) is #included here unmodified, from where it
// lies, with its main() renamed; nothing of it is copied into this repository. Its file-static host functions
// become callable through the small extern "C" surface below, which the tests use to pin the CPU oracle
// (rng, noise hash, ternary init, fitness shaping, token cross-entropy, batch sampling) against the real reference code.
// The device entry points the driver references are resolved by libbnf4.so -- linking this file is at the
// same time the proof that the reference driver links against the library unchanged.
#define main ref_train_main
#include "train_efla_lm.cpp"
#undef main

#include <cstring>

extern "C" {

#define REF_API __attribute__((visibility("default")))

REF_API uint64_t ref_mix(uint64_t a, uint64_t b) { return rng::mix(a, b); }
REF_API uint64_t ref_splitmix64(uint64_t* st) { return rng::splitmix64(*st); }
REF_API int ref_ternary_from_u64(uint64_t x) { return rng::ternary_from_u64(x); }
REF_API int ref_noise_hash(uint64_t seed, uint64_t idx, int anti, int use_clt, int clt_k) {
    return noise_hash(seed, idx, anti, use_clt != 0, clt_k);
}
REF_API float ref_init_rand(int8_t* out, int rows, int cols, uint64_t seed) {
    TernaryMatrix m;
    m.init_rand(rows, cols, seed);
    std::memcpy(out, m.w.data(), m.w.size());
    return m.out_scale;
}
REF_API void ref_shape_pair_weights(float* w, int n, int mode, float clip) {
    TrainConfig cfg;
    cfg.fitness_mode = mode == 0 ? TrainConfig::FitnessMode::CenteredRank
                                 : (mode == 1 ? TrainConfig::FitnessMode::ZScore : TrainConfig::FitnessMode::Sign);
    cfg.fitness_clip = clip;
    std::vector<float> v(w, w + n);
    shape_pair_weights(v, cfg);
    std::memcpy(w, v.data(), sizeof(float) * n);
}
REF_API float ref_cross_entropy_token(const float* logits, const float* bias, const float* bias_noise, float bns, int vocab, int y) {
    return cross_entropy_loss_token(logits, bias, bias_noise, bns, vocab, y);
}
REF_API int ref_qkv_fused_cols_aligned(int hidden) { return qkv_fused_cols_aligned(hidden, true); }
REF_API uint64_t ref_count_parameters(int vocab, int hidden, int layers, int mlp_mult, int seq, int train_pos) {
    TrainConfig cfg;
    cfg.vocab = vocab; cfg.hidden = hidden; cfg.layers = layers; cfg.mlp_mult = mlp_mult; cfg.seq_len = seq; cfg.train_pos = train_pos != 0;
    return count_parameters(cfg);
}
// The reference's batch sampler on a corpus file (src/dataset.cpp:39-54). Returns 0 on success.
REF_API int ref_sample_batch_packed(const char* path, int batch, int seq_len, uint64_t seed, uint8_t* inputs, uint8_t* targets) {
    ByteDataset ds;
    if (!ds.load_file(path)) return 1;
    ds.sample_batch_packed(batch, seq_len, seed, inputs, targets);
    return 0;
}
// The reference driver itself (argv as for its executable), running on this library's kernels.
REF_API int ref_train(int argc, char** argv) { return ref_train_main(argc, argv); }
}
