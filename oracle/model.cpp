// CPU oracle, part 2: one member's fitness forward. TEST INFRASTRUCTURE ONLY (see oracle.cpp).
//
// Restates CudaEflaLm::evaluate_loss (src/train_efla_lm.cpp:2117-3431) with the default flags
// (NVFP4 GEMMs, fused QKV stack, int8 residual, abs-mean norm, fp16 EFLA state), plus the per-pair
// seed derivation of eval_worker (:5344-5468).
//
// Two perturbation forms:
//   rank == 0  dense: each matrix gets a full int8 noise matrix, quantised to NVFP4 and applied as a
//              second GEMM with beta = 1 (the reference's live path, :2349-2379, :2507-2523).
//   rank  > 0  rank-r: y += s * sum_r t[b,r]*A[i,r], t = x_int8 . B (exact int32) -- the math of the
//              reference's lora_compute_t / gemm_lora_f kernels (src/cuda_kernels.cu:370-390,
//              1271-1305), which its driver never calls. Scale s = ((anti*sigma)*out_scale)*c_r with
//              c_r = sqrt(3/8)/sqrt(r), so that every entry of the effective perturbation keeps the
//              variance 8/3 of the dense CLT noise.
// One documented simplification: the reference's perturbed ff1 uses CUTLASS' GELU_taylor epilogue
// while its unperturbed evaluation uses the tanhf GELU (:2724-2757); the tanhf form is used for both.

#include <cmath>
#include <cstring>
#include <vector>

#include "oracle.h"

namespace {

using namespace orc_salt;

struct QMat {  // a weight matrix quantised to NVFP4
    int rows = 0, cols = 0;
    std::vector<uint8_t> codes, sf;
};

static QMat quantize_w(const int8_t* w, int rows, int cols) {
    QMat q;
    q.rows = rows;
    q.cols = cols;
    q.codes.assign((size_t)rows * cols / 2, 0);
    q.sf.assign(orc_sf_bytes(rows, cols), 0);
    orc_quantize_rowmajor(w, rows, cols, cols, q.codes.data(), q.sf.data());
    return q;
}

static QMat quantize_qkv(const int8_t* wq, const int8_t* wk, const int8_t* wv, const int8_t* wb, int H, float s) {
    QMat q;
    q.rows = 3 * H + 1;
    q.cols = H;
    q.codes.assign((size_t)q.rows * H / 2 + 8, 0);
    q.sf.assign(orc_sf_bytes(q.rows, H), 0);
    orc_quantize_wqkv_fused(wq, wk, wv, wb, H, H, s, s, s, s, q.codes.data(), q.sf.data());
    return q;
}

struct Model {
    orc_model_cfg cfg;
    orc_model_weights w;
    int H, F, L, V, T, B, fused_cols;
    float s_h, s_f;  // 1/sqrt(H), 1/sqrt(F)
    QMat win, head;
    std::vector<QMat> qkv, ff1, ff2;
};

struct Activ {  // an activation in its three forms
    std::vector<int8_t> q;
    std::vector<uint8_t> codes, sf;
    void resize(int rows, int cols) {
        q.assign((size_t)rows * cols, 0);
        codes.assign((size_t)rows * cols / 2, 0);
        sf.assign(orc_sf_bytes(rows, cols), 0);
    }
};

struct Pert {  // per-pair perturbation context
    const Model* m;
    uint64_t pair_seed;
    float ns;  // anti * sigma
    float c_r;
};

static float c_rank(int rank) { return rank > 0 ? 0.6123724356957945f / std::sqrt((float)rank) : 0.0f; }

// out[rows x N] (ld) = alpha * (x . W^T) + perturbation(seed)
static void pert_gemm(const Pert& p, const Activ& x, int rows, const QMat& W, float alpha, uint64_t seed, float* out,
                      int ld) {
    const Model& m = *p.m;
    const int N = W.rows, K = W.cols;
    orc_gemm_nvfp4(x.codes.data(), W.codes.data(), x.sf.data(), W.sf.data(), rows, N, K, alpha, 0.0f, nullptr, 0, out,
                   ld, 0, 0.0f, nullptr);
    if (p.ns == 0.0f) return;
    if (m.cfg.rank == 0) {
        std::vector<int8_t> E((size_t)N * K);
        orc_fill_noise(E.data(), E.size(), seed, m.cfg.use_clt, m.cfg.clt_k);
        QMat qe = quantize_w(E.data(), N, K);
        orc_gemm_nvfp4(x.codes.data(), qe.codes.data(), x.sf.data(), qe.sf.data(), rows, N, K, alpha * p.ns, 1.0f, out,
                       ld, out, ld, 0, 0.0f, nullptr);
    } else {
        const int r = m.cfg.rank;
        std::vector<int8_t> A((size_t)N * r), Bm((size_t)K * r);
        orc_fill_noise(A.data(), A.size(), orc_mix(seed, kFactorA), m.cfg.use_clt, m.cfg.clt_k);
        orc_fill_noise(Bm.data(), Bm.size(), orc_mix(seed, kFactorB), m.cfg.use_clt, m.cfg.clt_k);
        std::vector<int32_t> t((size_t)rows * r);
        orc_lora_compute_t(x.q.data(), Bm.data(), K, rows, r, t.data());
        orc_lora_add(t.data(), A.data(), N, rows, r, (p.ns * alpha) * p.c_r, out, ld);
    }
}

// Fused QKV(+beta) projection of layer l: out[rows x fused_cols]; columns [0,H) q, [H,2H) k, [2H,3H) v, 3H beta_raw.
static void pert_qkv(const Pert& p, const Activ& x, int rows, int l, float* out) {
    const Model& m = *p.m;
    const int H = m.H, N = 3 * H + 1, ld = m.fused_cols;
    const QMat& W = m.qkv[l];
    orc_gemm_nvfp4(x.codes.data(), W.codes.data(), x.sf.data(), W.sf.data(), rows, N, H, 1.0f, 0.0f, nullptr, 0, out,
                   ld, 0, 0.0f, nullptr);
    if (p.ns == 0.0f) return;
    const uint64_t lu = (uint64_t)l;
    const uint64_t seeds[4] = {orc_mix(p.pair_seed, orc_mix(lu, kWq)), orc_mix(p.pair_seed, orc_mix(lu, kWk)),
                               orc_mix(p.pair_seed, orc_mix(lu, kWv)), orc_mix(p.pair_seed, orc_mix(lu, kWbeta))};
    const int grows[4] = {H, H, H, 1};
    if (m.cfg.rank == 0) {
        std::vector<int8_t> E[4];
        for (int g = 0; g < 4; ++g) {
            E[g].resize((size_t)grows[g] * H);
            orc_fill_noise(E[g].data(), E[g].size(), seeds[g], m.cfg.use_clt, m.cfg.clt_k);
        }
        QMat qe = quantize_qkv(E[0].data(), E[1].data(), E[2].data(), E[3].data(), H, m.s_h);
        orc_gemm_nvfp4(x.codes.data(), qe.codes.data(), x.sf.data(), qe.sf.data(), rows, N, H, p.ns, 1.0f, out, ld, out,
                       ld, 0, 0.0f, nullptr);
    } else {
        const int r = m.cfg.rank;
        for (int g = 0; g < 4; ++g) {
            std::vector<int8_t> A((size_t)grows[g] * r), Bm((size_t)H * r);
            orc_fill_noise(A.data(), A.size(), orc_mix(seeds[g], kFactorA), m.cfg.use_clt, m.cfg.clt_k);
            orc_fill_noise(Bm.data(), Bm.size(), orc_mix(seeds[g], kFactorB), m.cfg.use_clt, m.cfg.clt_k);
            std::vector<int32_t> t((size_t)rows * r);
            orc_lora_compute_t(x.q.data(), Bm.data(), H, rows, r, t.data());
            orc_lora_add(t.data(), A.data(), grows[g], rows, r, (p.ns * m.s_h) * p.c_r, out + (size_t)g * H, ld);
        }
    }
}

static void embed(const Pert& p, const uint8_t* tokens, int token_stride, int rows, Activ& out) {
    const Model& m = *p.m;
    const uint64_t seed = orc_mix(p.pair_seed, kEmb);
    if (m.cfg.rank == 0 || p.ns == 0.0f) {
        std::vector<int8_t> E;
        if (p.ns != 0.0f) {
            E.resize((size_t)m.V * m.H);
            orc_fill_noise(E.data(), E.size(), seed, m.cfg.use_clt, m.cfg.clt_k);
        }
        const float sigma = std::fabs(p.ns);
        orc_embedding_quant(tokens, token_stride, m.w.emb, E.empty() ? nullptr : E.data(), m.H, rows, sigma,
                            p.ns > 0 ? 1 : (p.ns < 0 ? -1 : 0), out.q.data(), out.codes.data(), out.sf.data());
    } else {
        const int r = m.cfg.rank;
        std::vector<int8_t> A((size_t)m.V * r), Bm((size_t)m.H * r);
        orc_fill_noise(A.data(), A.size(), orc_mix(seed, kFactorA), m.cfg.use_clt, m.cfg.clt_k);
        orc_fill_noise(Bm.data(), Bm.size(), orc_mix(seed, kFactorB), m.cfg.use_clt, m.cfg.clt_k);
        orc_embedding_lowrank_quant(tokens, token_stride, m.w.emb, A.data(), Bm.data(), r, m.H, rows, p.ns * p.c_r,
                                    out.q.data(), out.codes.data(), out.sf.data());
    }
}

struct PairVectors {  // the small per-pair vectors (src/train_efla_lm.cpp:5372-5388, 5452-5455)
    std::vector<float> pos_noisy, head_bias_noise, beta_bias_eff;
};

static PairVectors pair_vectors(const Pert& p) {
    const Model& m = *p.m;
    PairVectors v;
    v.pos_noisy.resize((size_t)m.T * m.H);
    const uint64_t pos_seed = orc_mix(p.pair_seed, kPos);
    for (size_t i = 0; i < v.pos_noisy.size(); ++i) {
        const float nz = p.ns != 0.0f ? (float)orc_noise_hash(pos_seed, i, m.cfg.use_clt, m.cfg.clt_k) : 0.0f;
        v.pos_noisy[i] = std::fmaf(p.ns, nz, m.w.pos[i]);
    }
    v.head_bias_noise.resize(m.V);
    const uint64_t hb_seed = orc_mix(p.pair_seed, kHeadBias);
    for (int i = 0; i < m.V; ++i) v.head_bias_noise[i] = (float)orc_noise_hash(hb_seed, i, m.cfg.use_clt, m.cfg.clt_k);
    v.beta_bias_eff.resize(m.L);
    const uint64_t bb_seed = orc_mix(p.pair_seed, kBetaBias);
    for (int l = 0; l < m.L; ++l) {
        const float nz = p.ns != 0.0f ? (float)orc_noise_hash(bb_seed, l, m.cfg.use_clt, m.cfg.clt_k) : 0.0f;
        v.beta_bias_eff[l] = std::fmaf(p.ns, nz, m.w.beta_bias[l]);
    }
    return v;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) void* orc_model_create(const orc_model_cfg* cfg,
                                                                          const orc_model_weights* w) {
    Model* m = new Model;
    m->cfg = *cfg;
    m->w = *w;
    m->H = cfg->hidden;
    m->F = cfg->hidden * cfg->mlp_mult;
    m->L = cfg->layers;
    m->V = cfg->vocab;
    m->T = cfg->seq;
    m->B = cfg->batch;
    m->fused_cols = (3 * m->H + 1 + 31) & ~31;  // qkv_fused_cols_aligned, src/train_efla_lm.cpp:433-437
    m->s_h = 1.0f / std::sqrt((float)m->H);
    m->s_f = 1.0f / std::sqrt((float)m->F);
    const size_t hh = (size_t)m->H * m->H, hf = (size_t)m->H * m->F;
    m->win = quantize_w(w->win, m->H, m->H);
    m->head = quantize_w(w->head, m->V, m->H);
    for (int l = 0; l < m->L; ++l) {
        m->qkv.push_back(quantize_qkv(w->wq + l * hh, w->wk + l * hh, w->wv + l * hh, w->wbeta + (size_t)l * m->H, m->H,
                                      m->s_h));
        m->ff1.push_back(quantize_w(w->ff1 + l * hf, m->F, m->H));
        m->ff2.push_back(quantize_w(w->ff2 + l * hf, m->H, m->F));
    }
    return m;
}

extern "C" __attribute__((visibility("default"))) void orc_model_destroy(void* handle) {
    delete static_cast<Model*>(handle);
}

extern "C" __attribute__((visibility("default"))) double orc_model_forward(void* handle, const uint8_t* tokens,
                                                                            const uint8_t* targets,
                                                                            uint64_t pair_seed, int anti_sign,
                                                                            orc_model_taps* taps) {
    const Model& m = *static_cast<Model*>(handle);
    const int H = m.H, F = m.F, L = m.L, V = m.V, T = m.T, R = m.B * m.T, FC = m.fused_cols;
    Pert p{&m, pair_seed, anti_sign == 0 ? 0.0f : (float)anti_sign / (float)(1 << m.cfg.sigma_shift),
           c_rank(m.cfg.rank)};
    const PairVectors pv = pair_vectors(p);

    Activ a_h, a_f;
    a_h.resize(R, H);
    a_f.resize(R, F);
    std::vector<int8_t> x_q((size_t)R * H);
    std::vector<float> f_h((size_t)R * H), f_f((size_t)R * F), qkv((size_t)R * FC, 0.0f), y((size_t)R * H);
    std::vector<int> pos_row(R);
    for (int r = 0; r < R; ++r) pos_row[r] = r % T;

    embed(p, tokens, 1, R, a_h);  // tokens [B][T] flat == row order b*T+t
    if (taps && taps->emb_q) std::memcpy(taps->emb_q, a_h.q.data(), a_h.q.size());
    pert_gemm(p, a_h, R, m.win, m.s_h, orc_mix(pair_seed, kWin), f_h.data(), H);
    if (taps && taps->inproj) std::memcpy(taps->inproj, f_h.data(), f_h.size() * 4);
    orc_add_pos_gelu_quant(f_h.data(), pv.pos_noisy.data(), pos_row.data(), H, R, m.cfg.act_scale, x_q.data(),
                           a_h.codes.data(), a_h.sf.data());
    if (taps && taps->x_q0) std::memcpy(taps->x_q0, x_q.data(), x_q.size());
    orc_absmean_norm_q(x_q.data(), nullptr, H, R, 0.0f, m.cfg.ln_scale, a_h.q.data(), a_h.codes.data(), a_h.sf.data());

    std::vector<float> bb_seq(m.B);
    for (int l = 0; l < L; ++l) {
        const uint64_t lu = (uint64_t)l;
        pert_qkv(p, a_h, R, l, qkv.data());
        if (taps && taps->qkv) std::memcpy(taps->qkv + (size_t)l * R * FC, qkv.data(), qkv.size() * 4);
        for (int b = 0; b < m.B; ++b) bb_seq[b] = pv.beta_bias_eff[l];
        orc_efla_scan(qkv.data(), FC, bb_seq.data(), H, m.cfg.heads, m.B, T, m.cfg.method, m.cfg.eps, y.data());
        if (taps && taps->attn_y) std::memcpy(taps->attn_y + (size_t)l * R * H, y.data(), y.size() * 4);
        orc_absmean_norm_q(x_q.data(), y.data(), H, R, m.cfg.residual_scale, m.cfg.ln_scale, a_h.q.data(),
                           a_h.codes.data(), a_h.sf.data());
        pert_gemm(p, a_h, R, m.ff1[l], m.s_h, orc_mix(pair_seed, orc_mix(lu, kFf1)), f_f.data(), F);
        orc_activation_quant(f_f.data(), R, F, F, 3, m.cfg.mlp_act_scale, a_f.q.data(), a_f.codes.data(),
                             a_f.sf.data());
        if (taps && taps->ff1_q) std::memcpy(taps->ff1_q + (size_t)l * R * F, a_f.q.data(), a_f.q.size());
        pert_gemm(p, a_f, R, m.ff2[l], m.s_f, orc_mix(pair_seed, orc_mix(lu, kFf2)), y.data(), H);
        if (taps && taps->ff2_y) std::memcpy(taps->ff2_y + (size_t)l * R * H, y.data(), y.size() * 4);
        orc_absmean_norm_q(x_q.data(), y.data(), H, R, m.cfg.mlp_residual_scale, m.cfg.ln_scale, a_h.q.data(),
                           a_h.codes.data(), a_h.sf.data());
        if (taps && taps->x_q) std::memcpy(taps->x_q + (size_t)l * R * H, x_q.data(), x_q.size());
        if (taps && taps->y_q) std::memcpy(taps->y_q + (size_t)l * R * H, a_h.q.data(), a_h.q.size());
    }
    std::vector<float> logits((size_t)R * V);
    pert_gemm(p, a_h, R, m.head, m.s_h, orc_mix(pair_seed, kHead), logits.data(), V);
    if (taps && taps->logits) std::memcpy(taps->logits, logits.data(), logits.size() * 4);
    const double total = orc_cross_entropy_sum(logits.data(), V, m.w.head_bias, pv.head_bias_noise.data(), p.ns,
                                               targets, 1, V, R, nullptr);
    return total / (double)R;
}

extern "C" __attribute__((visibility("default"))) double orc_model_forward_token_major(void* handle,
                                                                                         const uint8_t* tokens,
                                                                                         const uint8_t* targets,
                                                                                         uint64_t pair_seed,
                                                                                         int anti_sign) {
    const Model& m = *static_cast<Model*>(handle);
    const int H = m.H, F = m.F, L = m.L, V = m.V, T = m.T, B = m.B, FC = m.fused_cols;
    const int hd = H / m.cfg.heads;
    Pert p{&m, pair_seed, anti_sign == 0 ? 0.0f : (float)anti_sign / (float)(1 << m.cfg.sigma_shift),
           c_rank(m.cfg.rank)};
    const PairVectors pv = pair_vectors(p);
    Activ a_h, a_f;
    a_h.resize(B, H);
    a_f.resize(B, F);
    std::vector<int8_t> x_q((size_t)B * H);
    std::vector<float> f_h((size_t)B * H), f_f((size_t)B * F), qkv((size_t)B * FC, 0.0f), y((size_t)B * H),
        logits((size_t)B * V);
    std::vector<uint16_t> S((size_t)L * B * H * hd, 0);
    std::vector<int> pos_row(B);
    double total = 0.0;
    for (int t = 0; t < T; ++t) {
        for (int b = 0; b < B; ++b) pos_row[b] = t;
        embed(p, tokens + t, T, B, a_h);
        pert_gemm(p, a_h, B, m.win, m.s_h, orc_mix(pair_seed, kWin), f_h.data(), H);
        orc_add_pos_gelu_quant(f_h.data(), pv.pos_noisy.data(), pos_row.data(), H, B, m.cfg.act_scale, x_q.data(),
                               a_h.codes.data(), a_h.sf.data());
        orc_absmean_norm_q(x_q.data(), nullptr, H, B, 0.0f, m.cfg.ln_scale, a_h.q.data(), a_h.codes.data(),
                           a_h.sf.data());
        for (int l = 0; l < L; ++l) {
            const uint64_t lu = (uint64_t)l;
            pert_qkv(p, a_h, B, l, qkv.data());
            orc_efla_step_half_qkv_fused(S.data() + (size_t)l * B * H * hd, qkv.data(), FC, pv.beta_bias_eff[l], H,
                                         m.cfg.heads, B, m.cfg.method, m.cfg.eps, y.data());
            orc_absmean_norm_q(x_q.data(), y.data(), H, B, m.cfg.residual_scale, m.cfg.ln_scale, a_h.q.data(),
                               a_h.codes.data(), a_h.sf.data());
            pert_gemm(p, a_h, B, m.ff1[l], m.s_h, orc_mix(pair_seed, orc_mix(lu, kFf1)), f_f.data(), F);
            orc_activation_quant(f_f.data(), B, F, F, 3, m.cfg.mlp_act_scale, a_f.q.data(), a_f.codes.data(),
                                 a_f.sf.data());
            pert_gemm(p, a_f, B, m.ff2[l], m.s_f, orc_mix(pair_seed, orc_mix(lu, kFf2)), y.data(), H);
            orc_absmean_norm_q(x_q.data(), y.data(), H, B, m.cfg.mlp_residual_scale, m.cfg.ln_scale, a_h.q.data(),
                               a_h.codes.data(), a_h.sf.data());
        }
        pert_gemm(p, a_h, B, m.head, m.s_h, orc_mix(pair_seed, kHead), logits.data(), V);
        total += orc_cross_entropy_sum(logits.data(), V, m.w.head_bias, pv.head_bias_noise.data(), p.ns, targets + t, T,
                                       V, B, nullptr);
    }
    return total / (double)(T * B);
}
