// Population driver: layer-major, wave-batched evaluation of perturbed members and the ES update.
//
// Host-side re-design of the reference's CudaEflaLm::evaluate_loss (src/train_efla_lm.cpp:2117-3431), the
// per-pair seed derivation of eval_worker (:5344-5468), DeviceWeights / quantize_nvfp4_base_weights (:439-651,
// 1207-1310) and gpu_update_matrix (:4304-4358). The op order inside a layer is the reference's; the loop
// order is inverted (layers outside, tokens inside) which changes no value because only the recurrent state
// couples time steps.

#include <algorithm>
#include <cmath>
#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {

namespace {

constexpr float kCRankBase = 0.6123724356957945f;  // sqrt(3/8)

// Kernel classes for the optional timing breakdown (bnf4_model_get_timing).
enum KernelClass : int {
    KC_GEN_NOISE = 0, KC_BETA_BIAS, KC_EMBED, KC_GEMM_WIN, KC_POS_GELU_NORM, KC_GEMM_QKV, KC_EFLA, KC_ADD_NORM, KC_GEMM_FF1,
    KC_GEMM_FF2, KC_GEMM_HEAD, KC_CROSS_ENTROPY, KC_UPDATE_Z, KC_UPDATE_APPLY, KC_REQUANTIZE, KC_NORM_QUANT, kNumClasses
};
const char* const kClassNames[kNumClasses] = {"gen_noise", "beta_bias", "embed_quant", "gemm_win", "pos_gelu_norm_quant", "gemm_qkv",
                                              "efla_scan", "add_norm_quant", "gemm_ff1_gelu_fp4", "gemm_ff2", "gemm_head",
                                              "cross_entropy", "update_z_sumsq", "update_apply", "requantize_weights", "norm_quant"};

// One entry of the per-step noise table: dst[pair][...] filled from the counter hash.
struct GenDesc {
    int8_t* dst;
    long long pair_stride;
    uint64_t salt;    // mixed with the pair seed
    uint64_t factor;  // 0: plain vector, else sub-stream (kFactorA / kFactorB) of the matrix seed
    int n_major;      // rows (A), columns (B) or vector length
    int rank;         // 1 for plain vectors
    int transposed;   // store element (major, r) at r*n_major + major instead of major*rank + r
};

// block_map[b] = (descriptor << 20) | block within that descriptor: every launched block has work.
__global__ void gen_noise_kernel(const GenDesc* __restrict__ descs, const uint32_t* __restrict__ block_map, int block0, int pair0,
                                 const uint64_t* __restrict__ pair_seeds, int use_clt, int clt_k) {
    const uint32_t bm = block_map[block0 + blockIdx.x];
    const GenDesc d = descs[bm >> 20];
    const int pair = pair0 + blockIdx.y;
    const long long n = static_cast<long long>(d.n_major) * d.rank;
    const long long idx = static_cast<long long>(bm & 0xfffffu) * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    uint64_t seed = mix_u64(pair_seeds[pair], d.salt);
    if (d.factor != 0) seed = mix_u64(seed, d.factor);
    const int v = noise_hash(seed, static_cast<uint64_t>(idx), use_clt != 0, clt_k);
    long long o = idx;
    if (d.transposed) {
        const long long major = idx / d.rank, r = idx - major * d.rank;
        o = r * d.n_major + major;
    }
    d.dst[static_cast<size_t>(pair) * d.pair_stride + o] = static_cast<int8_t>(v);
}

// beta_bias_eff[l][member] = beta_bias[l] + ns(member) * noise[pair][l]   (reference: src/train_efla_lm.cpp:2912-2917)
__global__ void beta_bias_kernel(const float* __restrict__ beta_bias, const int8_t* __restrict__ noise, int layers, int members,
                                 float sigma, float* __restrict__ out) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= layers * members) return;
    const int l = i / members, m = i - l * members;
    const float ns = (m & 1) ? -sigma : sigma;
    const float nz = sigma != 0.0f ? static_cast<float>(noise[static_cast<size_t>(m >> 1) * layers + l]) : 0.0f;
    out[i] = fmaf(ns, nz, beta_bias[l]);
}

struct Model {
    bnf4_model_cfg cfg;
    int V, H, F, L, T, B, R, FC, r, hd;
    float s_h, s_f, sigma, c_r;
    int W;          // members per wave
    long long M;    // rows per wave
    size_t device_bytes = 0;
    std::vector<void*> allocs;

    // weights
    int8_t *emb, *win, *wq, *wk, *wv, *wbeta, *ff1, *ff2, *head;
    float *head_bias, *beta_bias, *pos;
    float *sh_emb, *sh_win, *sh_wq, *sh_wk, *sh_wv, *sh_wbeta, *sh_ff1, *sh_ff2, *sh_head;  // fp32 shadows
    float* rms_ema;  // [27 matrices + 3 vectors]
    // NVFP4 copies of the base weights
    uint8_t *q_win, *sfq_win, *q_head, *sfq_head;
    std::vector<uint8_t*> q_qkv, sfq_qkv, q_ff1, sfq_ff1, q_ff2, sfq_ff2;
    // tokens
    uint8_t *tokens, *targets;
    // per-step noise (all pairs)
    uint64_t* pair_seeds;
    int pairs_step = 0;
    int8_t *embA, *embB, *A_win, *tB_win, *A_head, *tB_head, *pos_noise, *hb_noise, *bb_noise;
    std::vector<int8_t*> A_qkv, tB_qkv, A_ff1, tB_ff1, A_ff2, tB_ff2;
    GenDesc* gen_descs;
    uint32_t* gen_block_map;
    int num_gen = 0;
    int gen_blocks = 0, gen_blocks_factors = 0;
    int eval_begin = 0, eval_end = 0;  // pairs whose evaluation-only noise the last prepare_step generated
    // wave buffers
    int8_t* x_q;
    uint8_t *a_h, *sf_h, *a_f, *sf_f;
    float *qkv, *y, *bb_eff, *ce_partial, *losses;
    // input stage computed once per (member, distinct token) when the vocabulary is smaller than a member's rows
    bool dedup_input = false;
    uint8_t *tok_ident, *emb_a, *emb_sf;
    int32_t* emb_t;
    float* y_emb;
    int32_t *t_a, *t_f;
    // update scratch
    float *Z, *Z_all, *sumsq, *inv_rms;
    UpdApplyDesc* upd_descs;  // table, block partials and inv_rms of the batched apply phase
    float *upd_partial, *upd_inv;
    ZLowrankDesc *zdesc, *zdesc_ext;  // device tables of the update's matrices: Z inside Z_all / inside a caller's buffer
    int launches_per_wave = 0;
    float* h_step = nullptr;    // bnf4_model_es_step: pinned losses [2 * max_pairs] + pair weights [max_pairs]
    float* d_step_w = nullptr;  // ... and the shaped pair weights on the device
    // dense (rank 0) mode: the reference driver's own perturbation, one materialised noise matrix per weight matrix and pair,
    // applied as a second GEMM with beta = 1 (src/train_efla_lm.cpp:2359-2367). One pair per wave.
    bool dense = false;
    uint64_t step_seed = 0, step_epoch = 0;
    int8_t* E_all = nullptr;                 // noise of one pair, all matrices back to back (order of update_matrices)
    uint8_t *qe_win, *sfe_win, *qe_head, *sfe_head;
    std::vector<uint8_t*> qe_qkv, sfe_qkv, qe_ff1, sfe_ff1, qe_ff2, sfe_ff2;
    bnf4_noise_desc* noise_descs = nullptr;  // device table for the batched fill
    float* ff1_f = nullptr;                  // [2R][F] fp32 base product of ff1
    int8_t* ff1_q = nullptr;                 // [2R][F] int8 GELU output

    // optional replay of a wave's launch sequence as a CUDA graph (the reference's --cuda_graph, src/train_efla_lm.cpp:3779-3819):
    // a wave is identified by everything its launches take from the host; the first run of a wave is eager (it fills lazily
    // built tables and sets function attributes), the second is captured on a private stream, later ones are graph launches.
    // A captured wave leaves its losses in the model's own buffer; a small copy behind the graph takes them to the caller's.
    struct WaveGraph {
        int p0, nm, opt_tma, opt_chunked;
        uint32_t sigma_bits;
        int seen = 0;         // eager runs so far
        bool failed = false;  // the capture was refused: this wave stays eager
        cudaGraphExec_t exec = nullptr;
        int launches = 0;
    };
    bool use_graph = false;
    std::vector<WaveGraph> graphs;
    cudaStream_t cap_stream = nullptr;
    long long graph_launches = 0;
    void drop_graphs() {
        for (WaveGraph& g : graphs)
            if (g.exec) cudaGraphExecDestroy(g.exec);
        graphs.clear();
    }

    // optional per-kernel-class timing with CUDA events on the launching stream
    bool timing = false;
    struct Span { int cls; cudaEvent_t a, b; };
    std::vector<Span> spans;
    std::vector<cudaEvent_t> free_events;
    double class_ms[kNumClasses] = {};
    long long class_launches[kNumClasses] = {};

    cudaEvent_t get_event() {
        if (!free_events.empty()) { cudaEvent_t e = free_events.back(); free_events.pop_back(); return e; }
        cudaEvent_t e = nullptr;
        cudaEventCreate(&e);
        return e;
    }

    template <typename Tp>
    int alloc(Tp** p, size_t count, bool zero = true) {
        void* ptr = nullptr;
        const size_t bytes = ((count * sizeof(Tp) + 255) / 256) * 256;
        int rc = check_cuda(cudaMalloc(&ptr, bytes), "cudaMalloc(model)");
        if (rc) return rc;
        allocs.push_back(ptr);
        device_bytes += bytes;
        if (zero) {
            rc = check_cuda(cudaMemset(ptr, 0, bytes), "cudaMemset(model)");
            if (rc) return rc;
        }
        *p = static_cast<Tp*>(ptr);
        return BNF4_OK;
    }
};

// Records an event pair around the launches issued while it is alive (only when timing is on).
struct TimedScope {
    Model& m;
    cudaStream_t st;
    int cls, n;
    cudaEvent_t a = nullptr;
    TimedScope(Model& m_, int cls_, cudaStream_t st_, int n_ = 1) : m(m_), st(st_), cls(cls_), n(n_) {
        if (m.timing) { a = m.get_event(); cudaEventRecord(a, st); }
    }
    ~TimedScope() {
        if (m.timing) {
            cudaEvent_t b = m.get_event();
            cudaEventRecord(b, st);
            m.spans.push_back({cls, a, b});
            m.class_launches[cls] += n;
        }
    }
};

#define TRY(expr)              \
    do {                       \
        const int rc_ = (expr); \
        if (rc_) return rc_;   \
    } while (0)

int quantize_base(Model& m, cudaStream_t st) {
    auto plain = [&](const int8_t* w, int rows, int cols, uint8_t* codes, uint8_t* sf) {
        bnf4_rowquant_desc p = {};
        p.rows = rows; p.cols_in = cols; p.cols_out = cols; p.in_i8 = w; p.ld_in = cols; p.out_codes = codes; p.out_sf = sf;
        return rowquant_dispatch(FE_INT8, p, st);
    };
    TRY(plain(m.win, m.H, m.H, m.q_win, m.sfq_win));
    TRY(plain(m.head, m.V, m.H, m.q_head, m.sfq_head));
    const size_t hh = static_cast<size_t>(m.H) * m.H, hf = static_cast<size_t>(m.H) * m.F;
    for (int l = 0; l < m.L; ++l) {
        bnf4_rowquant_desc p = {};
        p.rows = 3 * m.H + 1; p.cols_in = m.H; p.cols_out = m.H;
        p.wq = m.wq + l * hh; p.wk = m.wk + l * hh; p.wv = m.wv + l * hh; p.wb = m.wbeta + static_cast<size_t>(l) * m.H;
        p.q_scale = p.k_scale = p.v_scale = p.b_scale = m.s_h;
        p.out_codes = m.q_qkv[l]; p.out_sf = m.sfq_qkv[l];
        TRY(rowquant_dispatch(FE_WQKV, p, st));
        TRY(plain(m.ff1 + l * hf, m.F, m.H, m.q_ff1[l], m.sfq_ff1[l]));
        TRY(plain(m.ff2 + l * hf, m.H, m.F, m.q_ff2[l], m.sfq_ff2[l]));
    }
    return BNF4_OK;
}

// One wave: members [0, nm) of the wave correspond to pairs [p0, p0 + nm/2). sigma == 0 evaluates the base model.
int run_wave(Model& m, int p0, int nm, float sigma, float* losses_out, cudaStream_t st) {
    const int H = m.H, F = m.F, L = m.L, V = m.V, R = m.R, FC = m.FC, r = m.r;
    const int rows = nm * R;
    const bool pert = sigma != 0.0f;
    const int rank = pert ? r : 0;
    const size_t P0 = static_cast<size_t>(p0);
    int launches = 0;

    {   // per-member beta bias for every layer
        const int n = L * nm;
        TimedScope ts(m, KC_BETA_BIAS, st);
        beta_bias_kernel<<<(n + 127) / 128, 128, 0, st>>>(m.beta_bias, m.bb_noise + P0 * L, L, nm, sigma, m.bb_eff);
        TRY(check_launch("beta_bias_kernel"));
        ++launches;
    }
    // The embedding row and its input projection depend on (member, token) only. With a byte vocabulary there are V = 256
    // distinct tokens against R = B*T rows per member, so both are computed once per (member, token) (nm*V rows) and the
    // pos+GELU+norm stage gathers its input row by token. Same values as the row-by-row form, 1/16 of the work at R = 4096.
    const bool dedup = m.dedup_input;
    const int erows = dedup ? nm * V : rows;
    const int e_rpm = dedup ? V : R;
    {   // embedding -> codes, scales, t for win
        TimedScope ts(m, KC_EMBED, st);
        bnf4_rowquant_desc p = {};
        p.rows = erows; p.cols_in = H; p.cols_out = H; p.rows_per_member = e_rpm; p.sigma = sigma; p.c_rank = m.c_r;
        p.tokens = dedup ? m.tok_ident : m.tokens; p.token_stride = 1; p.row_mod = e_rpm; p.emb_w = m.emb;
        p.embA = m.embA + P0 * V * r; p.embB = m.embB + P0 * H * r; p.embA_pair_stride = static_cast<long long>(V) * r;
        p.embB_pair_stride = static_cast<long long>(H) * r; p.rank = r;
        p.out_codes = dedup ? m.emb_a : m.a_h; p.out_sf = dedup ? m.emb_sf : m.sf_h;
        if (pert) { p.tvec = m.tB_win + P0 * H * r; p.tvec_pair_stride = static_cast<long long>(H) * r; p.nvec = r; p.t_out = dedup ? m.emb_t : m.t_a; }
        TRY(rowquant_dispatch(FE_EMBED_LOWRANK, p, st));
        ++launches;
    }
    auto gemm_rows = [&](int cls, int grows, int g_rpm, const uint8_t* a, const uint8_t* sfa, const uint8_t* b, const uint8_t* sfb, int n, int k,
                         float alpha, float* d, int ldd, const int8_t* A, long long A_stride, const int32_t* t, int t_stride, float out_scale,
                         int group_cols) {
        TimedScope ts(m, cls, st);
        bnf4_gemm_desc g = {};
        g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.m = grows; g.n = n; g.k = k; g.alpha = alpha; g.d = d; g.ldd = ldd;
        g.epilogue = EPI_F32; g.rank = rank; g.rows_per_member = g_rpm; g.lora_t = t; g.t_stride = t_stride; g.lora_A = A;
        g.lora_A_pair_stride = A_stride; g.lora_scale = (sigma * out_scale) * m.c_r; g.group_cols = group_cols;
        return gemm_nvfp4_launch(g, st);
    };
    auto gemm = [&](int cls, const uint8_t* a, const uint8_t* sfa, const uint8_t* b, const uint8_t* sfb, int n, int k, float alpha, float* d,
                    int ldd, const int8_t* A, long long A_stride, const int32_t* t, int t_stride, float out_scale, int group_cols) {
        return gemm_rows(cls, rows, R, a, sfa, b, sfb, n, k, alpha, d, ldd, A, A_stride, t, t_stride, out_scale, group_cols);
    };
    // input projection -> y (per row) or y_emb (per member and token)
    TRY(gemm_rows(KC_GEMM_WIN, erows, e_rpm, dedup ? m.emb_a : m.a_h, dedup ? m.emb_sf : m.sf_h, m.q_win, m.sfq_win, H, H, m.s_h,
                  dedup ? m.y_emb : m.y, H, m.A_win + P0 * H * r, static_cast<long long>(H) * r, dedup ? m.emb_t : m.t_a, r, m.s_h, 0));
    ++launches;
    {   // + pos, GELU -> residual stream x_q; abs-mean norm -> a_h; t for qkv[0]
        TimedScope ts(m, KC_POS_GELU_NORM, st);
        bnf4_rowquant_desc p = {};
        p.rows = rows; p.cols_in = H; p.cols_out = H; p.rows_per_member = R; p.sigma = sigma;
        p.in_f32 = dedup ? m.y_emb : m.y; p.ld_in = H; p.inout_i8 = m.x_q; p.pos = m.pos; p.pos_mod = m.T;
        if (dedup) { p.gather_rows = V; p.tokens = m.tokens; p.token_stride = 1; p.row_mod = R; }
        p.pos_noise = pert ? m.pos_noise + P0 * m.T * H : nullptr; p.noise_pair_stride = static_cast<long long>(m.T) * H;
        p.act_scale = m.cfg.act_scale; p.norm_scale = m.cfg.ln_scale; p.out_codes = m.a_h; p.out_sf = m.sf_h;
        if (pert) { p.tvec = m.tB_qkv[0] + P0 * 4 * r * H; p.tvec_pair_stride = static_cast<long long>(4) * r * H; p.nvec = 4 * r; p.t_out = m.t_a; }
        TRY(rowquant_dispatch(FE_POS_GELU_ABSMEAN, p, st));
        ++launches;
    }
    // With heads of 64 and the chunked scan, q | k | v travel as IEEE halves (the scan rounds its operands to fp16 anyway) and
    // so does the scan's output: the projection writes [rows][3H] halves + [rows] fp32 beta_raw into the qkv buffer, the
    // scan writes [rows][H] halves into the y buffer. Otherwise everything stays fp32 (the reference's interface).
    const bool half_io = m.hd == 64 && g_efla_chunked != 0;
    __half* qkv16 = reinterpret_cast<__half*>(m.qkv);
    float* beta16 = m.qkv + (static_cast<size_t>(rows) * 3 * H + 1) / 2;  // behind the halves
    for (int l = 0; l < L; ++l) {
        // fused QKV(+beta) projection; out_scale is folded into the weight scales (alpha = 1)
        if (half_io) {
            TimedScope ts(m, KC_GEMM_QKV, st);
            bnf4_gemm_desc g = {};
            g.a = m.a_h; g.b = m.q_qkv[l]; g.sfa = m.sf_h; g.sfb = m.sfq_qkv[l]; g.m = rows; g.n = 3 * H + 1; g.k = H; g.alpha = 1.0f;
            g.epilogue = EPI_F16; g.d_f16 = qkv16; g.ld_f16 = 3 * H; g.n_f16 = 3 * H; g.d = beta16; g.ldd = 1;
            g.rank = rank; g.rows_per_member = R; g.lora_t = m.t_a; g.t_stride = 4 * r; g.lora_A = m.A_qkv[l] + P0 * (3 * H + 1) * r;
            g.lora_A_pair_stride = static_cast<long long>(3 * H + 1) * r; g.lora_scale = (sigma * m.s_h) * m.c_r; g.group_cols = H;
            TRY(gemm_nvfp4_launch(g, st));
        } else {
            TRY(gemm(KC_GEMM_QKV, m.a_h, m.sf_h, m.q_qkv[l], m.sfq_qkv[l], 3 * H + 1, H, 1.0f, m.qkv, FC, m.A_qkv[l] + P0 * (3 * H + 1) * r,
                     static_cast<long long>(3 * H + 1) * r, m.t_a, 4 * r, m.s_h, H));
        }
        ++launches;
        {   // recurrence over the whole sequence -> y
            TimedScope ts(m, KC_EFLA, st);
            bnf4_efla_desc e = {};
            e.state = nullptr; e.state_fp16 = 1;
            if (half_io) {
                e.q = qkv16; e.k = qkv16 + H; e.v = qkv16 + 2 * H; e.beta_raw = beta16; e.ld_qkv = 3 * H; e.ld_beta = 1;
                e.qkv_f16 = 1; e.out_f16 = 1; e.out = m.y; e.ld_out = H;
            } else {
                e.q = m.qkv; e.k = m.qkv + H; e.v = m.qkv + 2 * H; e.beta_raw = m.qkv + 3 * H; e.ld_qkv = FC; e.ld_beta = FC;
                e.out = m.y; e.ld_out = H;
            }
            e.beta_bias_seq = m.bb_eff + static_cast<size_t>(l) * nm; e.seqs_per_bias = m.B;
            e.hidden = H; e.heads = m.cfg.heads; e.seqs = static_cast<long long>(nm) * m.B; e.T = m.T; e.method = m.cfg.method;
            e.eps = m.cfg.eps;
            // the generic kernel addresses sequences with blockIdx.z: split large waves
            if (m.hd == 64) {
                TRY(efla_launch(e, st));
                ++launches;
            } else {
                for (long long s0 = 0; s0 < e.seqs; s0 += 32768) {
                    bnf4_efla_desc ee = e;
                    const long long cnt = std::min<long long>(32768, e.seqs - s0);
                    const size_t ro = static_cast<size_t>(s0) * m.T;
                    ee.q = m.qkv + ro * FC; ee.k = m.qkv + H + ro * FC; ee.v = m.qkv + 2 * H + ro * FC; ee.beta_raw = e.beta_raw + ro * FC;
                    ee.out = m.y + ro * H; ee.seqs = cnt;
                    if ((s0 % m.B) != 0) return set_error(BNF4_ERR_INVALID, "efla split not aligned to batch");
                    ee.beta_bias_seq = e.beta_bias_seq + s0 / m.B;
                    TRY(efla_launch(ee, st));
                    ++launches;
                }
            }
        }
        {   // residual add + abs-mean norm -> a_h; t for ff1
            TimedScope ts(m, KC_ADD_NORM, st);
            bnf4_rowquant_desc p = {};
            p.rows = rows; p.cols_in = H; p.cols_out = H; p.rows_per_member = R; p.sigma = sigma;
            p.inout_i8 = m.x_q; p.in_f32 = m.y; p.ld_in = H; p.in_f16 = half_io ? 1 : 0;
            p.add_scale = m.cfg.residual_scale; p.norm_scale = m.cfg.ln_scale;
            p.out_codes = m.a_h; p.out_sf = m.sf_h;
            if (pert) { p.tvec = m.tB_ff1[l] + P0 * r * H; p.tvec_pair_stride = static_cast<long long>(r) * H; p.nvec = r; p.t_out = m.t_a; }
            TRY(rowquant_dispatch(FE_ADD_ABSMEAN, p, st));
            ++launches;
        }
        {   // ff1 with GELU -> int8 -> FP4 epilogue, projections for ff2
            TimedScope ts(m, KC_GEMM_FF1, st);
            if (pert) TRY(check_cuda(cudaMemsetAsync(m.t_f, 0, static_cast<size_t>(rows) * r * sizeof(int32_t), st), "cudaMemsetAsync(t_f)"));
            bnf4_gemm_desc g = {};
            g.a = m.a_h; g.b = m.q_ff1[l]; g.sfa = m.sf_h; g.sfb = m.sfq_ff1[l]; g.m = rows; g.n = F; g.k = H; g.alpha = m.s_h;
            g.epilogue = EPI_GELU_FP4; g.act_scale = m.cfg.mlp_act_scale; g.d_codes = m.a_f; g.d_sf = m.sf_f;
            g.rank = rank; g.rows_per_member = R; g.lora_t = m.t_a; g.t_stride = r; g.lora_A = m.A_ff1[l] + P0 * F * r;
            g.lora_A_pair_stride = static_cast<long long>(F) * r; g.lora_scale = (sigma * m.s_h) * m.c_r;
            if (pert) { g.next_tvec = m.tB_ff2[l] + P0 * r * F; g.next_tvec_pair_stride = static_cast<long long>(r) * F; g.next_nvec = r; g.next_t = m.t_f; }
            TRY(gemm_nvfp4_launch(g, st));
            ++launches;
        }
        {   // ff2, added into the residual stream by the epilogue: the fp32 product never leaves the SM
            TimedScope ts(m, KC_GEMM_FF2, st);
            bnf4_gemm_desc g = {};
            g.a = m.a_f; g.b = m.q_ff2[l]; g.sfa = m.sf_f; g.sfb = m.sfq_ff2[l]; g.m = rows; g.n = H; g.k = F; g.alpha = m.s_f;
            g.epilogue = EPI_ADD_I8; g.resid = m.x_q; g.ld_resid = H; g.add_scale = m.cfg.mlp_residual_scale;
            g.rank = rank; g.rows_per_member = R; g.lora_t = m.t_f; g.t_stride = r; g.lora_A = m.A_ff2[l] + P0 * H * r;
            g.lora_A_pair_stride = static_cast<long long>(H) * r; g.lora_scale = (sigma * m.s_f) * m.c_r;
            TRY(gemm_nvfp4_launch(g, st));
            ++launches;
        }
        {   // abs-mean norm of the residual stream -> a_h; t for the next layer's qkv or the head
            const bool last = (l == L - 1);
            TimedScope ts(m, KC_NORM_QUANT, st);
            bnf4_rowquant_desc p = {};
            p.rows = rows; p.cols_in = H; p.cols_out = H; p.rows_per_member = R; p.sigma = sigma;
            p.in_i8 = m.x_q; p.ld_in = H; p.norm_scale = m.cfg.ln_scale;
            p.out_codes = m.a_h; p.out_sf = m.sf_h;
            if (pert) {
                if (last) { p.tvec = m.tB_head + P0 * r * H; p.tvec_pair_stride = static_cast<long long>(r) * H; p.nvec = r; }
                else { p.tvec = m.tB_qkv[l + 1] + P0 * 4 * r * H; p.tvec_pair_stride = static_cast<long long>(4) * r * H; p.nvec = 4 * r; }
                p.t_out = m.t_a;
            }
            TRY(rowquant_dispatch(FE_ABSMEAN, p, st));
            ++launches;
        }
    }
    // head -> logits (in the qkv buffer, leading dimension V), cross-entropy per member
    TRY(gemm(KC_GEMM_HEAD, m.a_h, m.sf_h, m.q_head, m.sfq_head, V, H, m.s_h, m.qkv, V, m.A_head + P0 * V * r, static_cast<long long>(V) * r, m.t_a, r, m.s_h, 0));
    ++launches;
    TimedScope ts_ce(m, KC_CROSS_ENTROPY, st, 2);
    TRY(bnf4_cross_entropy_population(m.qkv, V, m.head_bias, pert ? m.hb_noise + P0 * V : nullptr, sigma, m.targets, V, nm, R, m.ce_partial,
                                      losses_out, st));
    launches += 2;
    m.launches_per_wave = launches;
    return BNF4_OK;
}

// run_wave, replayed from a captured graph when the model's graph mode is on (never while the timing breakdown records events:
// events recorded during a capture cannot be read back). Results are those of the eager launches: same kernels, same arguments.
int run_wave_cached(Model& m, int p0, int nm, float sigma, float* losses_out, cudaStream_t st) {
    if (!m.use_graph || m.timing) return run_wave(m, p0, nm, sigma, losses_out, st);
    const uint32_t sb = __builtin_bit_cast(uint32_t, sigma);
    Model::WaveGraph* e = nullptr;
    for (Model::WaveGraph& g : m.graphs)
        if (g.p0 == p0 && g.nm == nm && g.sigma_bits == sb && g.opt_tma == g_gemm_allow_tma_store && g.opt_chunked == g_efla_chunked) e = &g;
    if (e == nullptr) {
        if (m.graphs.size() >= 1024) m.drop_graphs();  // more distinct waves than any population makes: start over
        Model::WaveGraph g = {};
        g.p0 = p0; g.nm = nm; g.sigma_bits = sb; g.opt_tma = g_gemm_allow_tma_store; g.opt_chunked = g_efla_chunked;
        m.graphs.push_back(g);
        e = &m.graphs.back();
    }
    if (e->failed || e->seen == 0) {
        ++e->seen;
        return run_wave(m, p0, nm, sigma, losses_out, st);
    }
    if (e->exec == nullptr) {
        if (m.cap_stream == nullptr && cudaStreamCreateWithFlags(&m.cap_stream, cudaStreamNonBlocking) != cudaSuccess) m.cap_stream = nullptr;
        cudaGraph_t graph = nullptr;
        bool ok = m.cap_stream != nullptr && cudaStreamBeginCapture(m.cap_stream, cudaStreamCaptureModeThreadLocal) == cudaSuccess;
        if (ok) {
            const int rc = run_wave(m, p0, nm, sigma, m.losses, m.cap_stream);  // nothing executes: the launches become nodes
            ok = cudaStreamEndCapture(m.cap_stream, &graph) == cudaSuccess && graph != nullptr && rc == BNF4_OK;
        }
        if (ok) ok = cudaGraphInstantiate(&e->exec, graph, 0) == cudaSuccess;
        if (graph) cudaGraphDestroy(graph);
        if (!ok) {
            cudaGetLastError();
            e->exec = nullptr;
            e->failed = true;
            return run_wave(m, p0, nm, sigma, losses_out, st);
        }
        e->launches = m.launches_per_wave;
    }
    m.launches_per_wave = e->launches;
    ++m.graph_launches;
    TRY(check_cuda(cudaGraphLaunch(e->exec, st), "cudaGraphLaunch(wave)"));
    if (losses_out == m.losses) return BNF4_OK;
    return check_cuda(cudaMemcpyAsync(losses_out, m.losses, static_cast<size_t>(nm) * sizeof(float), cudaMemcpyDeviceToDevice, st), "cudaMemcpyAsync(wave losses)");
}

// Offsets of the matrices inside E_all, in the order emb, win, per layer (wq, wk, wv, wbeta, ff1, ff2), head.
struct DenseLayout {
    size_t emb, win, head;
    std::vector<size_t> wq, wk, wv, wbeta, ff1, ff2;
    size_t total;
};
DenseLayout dense_layout(const Model& m) {
    DenseLayout d;
    const size_t vh = static_cast<size_t>(m.V) * m.H, hh = static_cast<size_t>(m.H) * m.H, hf = static_cast<size_t>(m.H) * m.F;
    size_t o = 0;
    d.emb = o; o += vh;
    d.win = o; o += hh;
    for (int l = 0; l < m.L; ++l) {
        d.wq.push_back(o); o += hh;
        d.wk.push_back(o); o += hh;
        d.wv.push_back(o); o += hh;
        d.wbeta.push_back(o); o += (static_cast<size_t>(m.H) + 15) / 16 * 16;
        d.ff1.push_back(o); o += hf;
        d.ff2.push_back(o); o += hf;
    }
    d.head = o; o += vh;
    d.total = o;
    return d;
}

// One antithetic pair in the reference driver's own form: dense CLT noise matrices from the pair's seeds
// (set_noise_seeds, src/train_efla_lm.cpp:1946-2012), quantised to NVFP4 like the base weights, every projection as
// D = alpha A W^T followed by D += (+-sigma alpha) A E^T (gemm_noisy :2349-2379, gemm_qkvb :2507-2523, gemm_ff1_gelu :2724-2747),
// rows [0, R) = the + member, [R, 2R) = the - member. Layer-major over the tokens like the rank-r path.
int run_pair_dense(Model& m, int pair, float* losses_out, cudaStream_t st) {
    const int H = m.H, F = m.F, L = m.L, V = m.V, R = m.R, FC = m.FC;
    const int rows = 2 * R;
    const float sigma = m.sigma;
    const DenseLayout lay = dense_layout(m);
    const uint64_t pair_seed = mix_u64(m.step_seed, mix_u64(m.step_epoch, static_cast<uint64_t>(pair)));
    {   // noise of all matrices in one launch, then their NVFP4 copies
        std::vector<bnf4_noise_desc> nd;
        const size_t vh = static_cast<size_t>(V) * H, hh = static_cast<size_t>(H) * H, hf = static_cast<size_t>(H) * F;
        nd.push_back({m.E_all + lay.emb, vh, mix_u64(pair_seed, kSaltEmb)});
        nd.push_back({m.E_all + lay.win, hh, mix_u64(pair_seed, kSaltWin)});
        for (int l = 0; l < L; ++l) {
            const uint64_t lu = static_cast<uint64_t>(l);
            nd.push_back({m.E_all + lay.wq[l], hh, mix_u64(pair_seed, mix_u64(lu, kSaltWq))});
            nd.push_back({m.E_all + lay.wk[l], hh, mix_u64(pair_seed, mix_u64(lu, kSaltWk))});
            nd.push_back({m.E_all + lay.wv[l], hh, mix_u64(pair_seed, mix_u64(lu, kSaltWv))});
            nd.push_back({m.E_all + lay.wbeta[l], static_cast<size_t>(H), mix_u64(pair_seed, mix_u64(lu, kSaltWbeta))});
            nd.push_back({m.E_all + lay.ff1[l], hf, mix_u64(pair_seed, mix_u64(lu, kSaltFf1))});
            nd.push_back({m.E_all + lay.ff2[l], hf, mix_u64(pair_seed, mix_u64(lu, kSaltFf2))});
        }
        nd.push_back({m.E_all + lay.head, vh, mix_u64(pair_seed, kSaltHead)});
        TRY(check_cuda(cudaMemcpyAsync(m.noise_descs, nd.data(), nd.size() * sizeof(bnf4_noise_desc), cudaMemcpyHostToDevice, st), "cudaMemcpyAsync(noise_descs)"));
        TRY(check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize"));  // nd is a stack object: the copy must have read it
        size_t maxn = 0;
        for (const bnf4_noise_desc& x : nd) maxn = std::max(maxn, x.n);
        TimedScope ts(m, KC_GEN_NOISE, st, 1);
        TRY(bnf4_fill_ternary_noise_batched(m.noise_descs, static_cast<int>(nd.size()), static_cast<int>((maxn + 255) / 256), m.cfg.use_clt, m.cfg.clt_k, st));
        auto plain = [&](const int8_t* w, int r_, int c_, uint8_t* codes, uint8_t* sf) {
            bnf4_rowquant_desc q = {};
            q.rows = r_; q.cols_in = c_; q.cols_out = c_; q.in_i8 = w; q.ld_in = c_; q.out_codes = codes; q.out_sf = sf;
            return rowquant_dispatch(FE_INT8, q, st);
        };
        TRY(plain(m.E_all + lay.win, H, H, m.qe_win, m.sfe_win));
        TRY(plain(m.E_all + lay.head, V, H, m.qe_head, m.sfe_head));
        for (int l = 0; l < L; ++l) {
            bnf4_rowquant_desc q = {};
            q.rows = 3 * H + 1; q.cols_in = H; q.cols_out = H;
            q.wq = m.E_all + lay.wq[l]; q.wk = m.E_all + lay.wk[l]; q.wv = m.E_all + lay.wv[l]; q.wb = m.E_all + lay.wbeta[l];
            q.q_scale = q.k_scale = q.v_scale = q.b_scale = m.s_h;
            q.out_codes = m.qe_qkv[l]; q.out_sf = m.sfe_qkv[l];
            TRY(rowquant_dispatch(FE_WQKV, q, st));
            TRY(plain(m.E_all + lay.ff1[l], F, H, m.qe_ff1[l], m.sfe_ff1[l]));
            TRY(plain(m.E_all + lay.ff2[l], H, F, m.qe_ff2[l], m.sfe_ff2[l]));
        }
    }
    {
        TimedScope ts(m, KC_BETA_BIAS, st);
        beta_bias_kernel<<<(2 * L + 127) / 128, 128, 0, st>>>(m.beta_bias, m.bb_noise + static_cast<size_t>(pair) * L, L, 2, sigma, m.bb_eff);
        TRY(check_launch("beta_bias_kernel"));
    }
    // base product into d, then the two members' noise products added in place (alpha = +-sigma * alpha_base, beta = 1)
    auto noisy = [&](int cls, const uint8_t* a, const uint8_t* sfa, int a_k, const uint8_t* b, const uint8_t* sfb, const uint8_t* be, const uint8_t* sfbe,
                     int n, float alpha, float* d, int ldd) -> int {
        TimedScope ts(m, cls, st, 3);
        bnf4_gemm_desc g = {};
        g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.m = rows; g.n = n; g.k = a_k; g.alpha = alpha; g.d = d; g.ldd = ldd; g.epilogue = EPI_F32;
        TRY(gemm_nvfp4_launch(g, st));
        for (int mem = 0; mem < 2; ++mem) {
            bnf4_gemm_desc e = g;
            e.a = a + static_cast<size_t>(mem) * R * a_k / 2;
            e.sfa = sfa + sf_offset(mem * R, 0, sf_k_atoms(a_k));
            e.b = be; e.sfb = sfbe; e.m = R;
            e.alpha = (mem == 0 ? sigma : -sigma) * alpha; e.beta = 1.0f;
            e.c = d + static_cast<size_t>(mem) * R * ldd; e.ldc = ldd; e.d = d + static_cast<size_t>(mem) * R * ldd;
            TRY(gemm_nvfp4_launch(e, st));
        }
        return BNF4_OK;
    };
    {   // embedding with the pair's dense noise: both members in one launch, the sign follows the member
        TimedScope ts(m, KC_EMBED, st);
        bnf4_rowquant_desc q = {};
        q.rows = rows; q.cols_in = H; q.cols_out = H; q.rows_per_member = R; q.sigma = sigma;
        q.tokens = m.tokens; q.token_stride = 1; q.row_mod = R; q.emb_w = m.emb; q.emb_noise = m.E_all + lay.emb; q.noise_pair_stride = 0;
        q.out_codes = m.a_h; q.out_sf = m.sf_h;
        TRY(rowquant_dispatch(FE_EMBED_DENSE, q, st));
    }
    TRY(noisy(KC_GEMM_WIN, m.a_h, m.sf_h, H, m.q_win, m.sfq_win, m.qe_win, m.sfe_win, H, m.s_h, m.y, H));
    {
        TimedScope ts(m, KC_POS_GELU_NORM, st);
        bnf4_rowquant_desc q = {};
        q.rows = rows; q.cols_in = H; q.cols_out = H; q.rows_per_member = R; q.sigma = sigma;
        q.in_f32 = m.y; q.ld_in = H; q.inout_i8 = m.x_q; q.pos = m.pos; q.pos_mod = m.T;
        q.pos_noise = m.pos_noise + static_cast<size_t>(pair) * m.T * H; q.noise_pair_stride = 0;
        q.act_scale = m.cfg.act_scale; q.norm_scale = m.cfg.ln_scale; q.out_codes = m.a_h; q.out_sf = m.sf_h;
        TRY(rowquant_dispatch(FE_POS_GELU_ABSMEAN, q, st));
    }
    for (int l = 0; l < L; ++l) {
        // fused q | k | v | beta projection: out_scale folded into the scale bytes of W and of E alike (alpha = 1, noise alpha = +-sigma)
        TRY(noisy(KC_GEMM_QKV, m.a_h, m.sf_h, H, m.q_qkv[l], m.sfq_qkv[l], m.qe_qkv[l], m.sfe_qkv[l], 3 * H + 1, 1.0f, m.qkv, FC));
        {
            TimedScope ts(m, KC_EFLA, st);
            bnf4_efla_desc e = {};
            e.state = nullptr; e.state_fp16 = 1; e.q = m.qkv; e.k = m.qkv + H; e.v = m.qkv + 2 * H; e.beta_raw = m.qkv + 3 * H;
            e.ld_qkv = FC; e.ld_beta = FC; e.beta_bias_seq = m.bb_eff + static_cast<size_t>(l) * 2; e.seqs_per_bias = m.B;
            e.hidden = H; e.heads = m.cfg.heads; e.seqs = 2LL * m.B; e.T = m.T; e.method = m.cfg.method; e.eps = m.cfg.eps;
            e.out = m.y; e.ld_out = H;
            TRY(efla_launch(e, st));
        }
        {
            TimedScope ts(m, KC_ADD_NORM, st);
            bnf4_rowquant_desc q = {};
            q.rows = rows; q.cols_in = H; q.cols_out = H; q.rows_per_member = R; q.sigma = sigma;
            q.inout_i8 = m.x_q; q.in_f32 = m.y; q.ld_in = H; q.add_scale = m.cfg.residual_scale; q.norm_scale = m.cfg.ln_scale;
            q.out_codes = m.a_h; q.out_sf = m.sf_h;
            TRY(rowquant_dispatch(FE_ADD_ABSMEAN, q, st));
        }
        {   // ff1: base product in fp32, the noise product through the GELU -> int8 epilogue with C = base, then NVFP4
            TimedScope ts(m, KC_GEMM_FF1, st, 4);
            bnf4_gemm_desc g = {};
            g.a = m.a_h; g.b = m.q_ff1[l]; g.sfa = m.sf_h; g.sfb = m.sfq_ff1[l]; g.m = rows; g.n = F; g.k = H; g.alpha = m.s_h;
            g.d = m.ff1_f; g.ldd = F; g.epilogue = EPI_F32;
            TRY(gemm_nvfp4_launch(g, st));
            for (int mem = 0; mem < 2; ++mem) {
                bnf4_gemm_desc e = {};
                e.a = m.a_h + static_cast<size_t>(mem) * R * H / 2; e.sfa = m.sf_h + sf_offset(mem * R, 0, sf_k_atoms(H));
                e.b = m.qe_ff1[l]; e.sfb = m.sfe_ff1[l]; e.m = R; e.n = F; e.k = H;
                e.alpha = (mem == 0 ? sigma : -sigma) * m.s_h; e.beta = 1.0f; e.c = m.ff1_f + static_cast<size_t>(mem) * R * F; e.ldc = F;
                e.epilogue = EPI_GELU_I8; e.act_scale = m.cfg.mlp_act_scale; e.d_i8 = m.ff1_q + static_cast<size_t>(mem) * R * F; e.ld_i8 = F;
                TRY(gemm_nvfp4_launch(e, st));
            }
            bnf4_rowquant_desc q = {};
            q.rows = rows; q.cols_in = F; q.cols_out = F; q.in_i8 = m.ff1_q; q.ld_in = F; q.out_codes = m.a_f; q.out_sf = m.sf_f;
            TRY(rowquant_dispatch(FE_INT8, q, st));
        }
        TRY(noisy(KC_GEMM_FF2, m.a_f, m.sf_f, F, m.q_ff2[l], m.sfq_ff2[l], m.qe_ff2[l], m.sfe_ff2[l], H, m.s_f, m.y, H));
        {
            TimedScope ts(m, KC_NORM_QUANT, st);
            bnf4_rowquant_desc q = {};
            q.rows = rows; q.cols_in = H; q.cols_out = H; q.rows_per_member = R; q.sigma = sigma;
            q.inout_i8 = m.x_q; q.in_f32 = m.y; q.ld_in = H; q.add_scale = m.cfg.mlp_residual_scale; q.norm_scale = m.cfg.ln_scale;
            q.out_codes = m.a_h; q.out_sf = m.sf_h;
            TRY(rowquant_dispatch(FE_ADD_ABSMEAN, q, st));
        }
    }
    TRY(noisy(KC_GEMM_HEAD, m.a_h, m.sf_h, H, m.q_head, m.sfq_head, m.qe_head, m.sfe_head, V, m.s_h, m.qkv, V));
    TimedScope ts_ce(m, KC_CROSS_ENTROPY, st, 2);
    return bnf4_cross_entropy_population(m.qkv, V, m.head_bias, m.hb_noise + static_cast<size_t>(pair) * V, sigma, m.targets, V, 2, R, m.ce_partial,
                                         losses_out, st);
}

}  // namespace
}  // namespace bnf4

using namespace bnf4;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
static inline Model* M(void* h) { return static_cast<Model*>(h); }

namespace {

// One ternary matrix of the model as the update sees it: weights, shadow, the two noise factors and its shape.
struct UpdMatrix {
    int8_t* w;
    float* shadow;
    const int8_t* A;
    long long A_stride;
    const int8_t* Bt;
    long long B_stride;
    int rows, cols;
};

// Fixed order = order of the RMS-EMA slots.
std::vector<UpdMatrix> update_matrices(Model& m) {
    const int V = m.V, H = m.H, F = m.F, L = m.L, r = m.r;
    const size_t hh = static_cast<size_t>(H) * H, hf = static_cast<size_t>(H) * F;
    std::vector<UpdMatrix> v;
    v.push_back({m.emb, m.sh_emb, m.embA, static_cast<long long>(V) * r, m.embB, static_cast<long long>(H) * r, V, H});
    v.push_back({m.win, m.sh_win, m.A_win, static_cast<long long>(H) * r, m.tB_win, static_cast<long long>(H) * r, H, H});
    for (int l = 0; l < L; ++l) {
        const long long As = static_cast<long long>(3 * H + 1) * r, Bs = static_cast<long long>(4) * r * H;
        int8_t* ws[4] = {m.wq + l * hh, m.wk + l * hh, m.wv + l * hh, m.wbeta + static_cast<size_t>(l) * H};
        float* ss[4] = {m.sh_wq + l * hh, m.sh_wk + l * hh, m.sh_wv + l * hh, m.sh_wbeta + static_cast<size_t>(l) * H};
        const int grows[4] = {H, H, H, 1};
        for (int g = 0; g < 4; ++g)
            v.push_back({ws[g], ss[g], m.A_qkv[l] + static_cast<size_t>(g) * H * r, As, m.tB_qkv[l] + static_cast<size_t>(g) * r * H, Bs, grows[g], H});
        v.push_back({m.ff1 + l * hf, m.sh_ff1 + l * hf, m.A_ff1[l], static_cast<long long>(F) * r, m.tB_ff1[l], static_cast<long long>(r) * H, F, H});
        v.push_back({m.ff2 + l * hf, m.sh_ff2 + l * hf, m.A_ff2[l], static_cast<long long>(H) * r, m.tB_ff2[l], static_cast<long long>(r) * F, H, F});
    }
    v.push_back({m.head, m.sh_head, m.A_head, static_cast<long long>(V) * r, m.tB_head, static_cast<long long>(H) * r, V, H});
    return v;
}

// The fp32 vectors of the update, after the matrices in the Z buffer (reference: update_vector, src/train_efla_lm.cpp:5648-5657).
struct UpdVector {
    float* v;
    int n;
    uint64_t salt;
};
std::vector<UpdVector> update_vectors(Model& m) {
    return {{m.head_bias, m.V, kSaltHeadBias}, {m.beta_bias, m.L, kSaltBetaBias}, {m.pos, m.T * m.H, kSaltPos}};
}
// A vector is computed in element ranges by the ranks only when that saves real work.
inline bool vector_sharded(int n, int nshards) { return nshards > 1 && n >= 4096 && (n % nshards) == 0; }
long long z_matrix_elems(Model& m) {
    long long n = 0;
    for (const UpdMatrix& x : update_matrices(m)) n += static_cast<long long>(x.rows) * x.cols;
    return n;
}

// Device table of the matrices with Z laid out back to back from z_base (the order of update_matrices).
std::vector<ZLowrankDesc> z_descs(Model& m, float* z_base) {
    std::vector<ZLowrankDesc> d;
    long long off = 0;
    for (const UpdMatrix& x : update_matrices(m)) {
        d.push_back({x.A, x.A_stride, x.Bt, x.B_stride, z_base + off, x.rows, x.cols});
        off += static_cast<long long>(x.rows) * x.cols;
    }
    return d;
}

// Z of all matrices (the rows of this shard) in one launch. z_ext == nullptr: into the model's own buffer.
int update_z(Model& m, const float* pair_weights, int shard, int nshards, float* z_ext, cudaStream_t st) {
    const std::vector<ZLowrankDesc> h = z_descs(m, z_ext != nullptr ? z_ext : m.Z_all);
    const ZLowrankDesc* dtab = m.zdesc;
    if (z_ext != nullptr) {
        // pageable source: the copy is staged before the call returns, so the host vector may go out of scope
        TRY(check_cuda(cudaMemcpyAsync(m.zdesc_ext, h.data(), h.size() * sizeof(ZLowrankDesc), cudaMemcpyHostToDevice, st), "cudaMemcpyAsync(zdesc)"));
        dtab = m.zdesc_ext;
    }
    float* zb = z_ext != nullptr ? z_ext : m.Z_all;
    TimedScope ts(m, KC_UPDATE_Z, st, 4);
    if (m.dense) {
        // Z[i] = sum_p w_p noise(mix(seed_p, salt), i) per matrix: the reference's compute_z_sumsq (src/efla_lm_kernels.cu:1854-1890),
        // rows of a sharded matrix by element range
        const int L = m.L;
        std::vector<uint64_t> salts = {kSaltEmb, kSaltWin};
        for (int l = 0; l < L; ++l)
            for (uint64_t sl : {kSaltWq, kSaltWk, kSaltWv, kSaltWbeta, kSaltFf1, kSaltFf2}) salts.push_back(mix_u64(static_cast<uint64_t>(l), sl));
        salts.push_back(kSaltHead);
        long long zo = 0;
        for (size_t i = 0; i < h.size(); ++i) {
            const long long n = static_cast<long long>(h[i].rows) * h[i].cols;
            long long i0 = 0, cnt = n;
            if (nshards > 1 && h[i].rows >= nshards && (h[i].rows % nshards) == 0) { cnt = n / nshards; i0 = shard * cnt; }
            TRY(z_dense_launch(pair_weights, m.pair_seeds, salts[i], m.pairs_step, static_cast<int>(i0), static_cast<int>(cnt), m.cfg.use_clt, m.cfg.clt_k,
                               zb + zo + i0, st));
            zo += n;
        }
    } else {
        TRY(z_lowrank_launch(pair_weights, dtab, h.data(), static_cast<int>(h.size()), m.pairs_step, m.r, m.c_r, shard, nshards, st));
    }
    long long off = z_matrix_elems(m);
    for (const UpdVector& x : update_vectors(m)) {
        int i0 = 0, cnt = x.n;
        if (vector_sharded(x.n, nshards)) { cnt = x.n / nshards; i0 = shard * cnt; }
        TRY(z_dense_launch(pair_weights, m.pair_seeds, x.salt, m.pairs_step, i0, cnt, m.cfg.use_clt, m.cfg.clt_k, zb + off + i0, st));
        off += x.n;
    }
    return BNF4_OK;
}

// Applies the precomputed Z of every tensor (sum of squares, RMS-EMA, gated update: four launches for all of them) and
// re-quantises the base weights.
int update_apply(Model& m, const float* pair_weights, const float* z_all, const bnf4_update_cfg* u, cudaStream_t st) {
    (void)pair_weights;
    const int P = m.pairs_step;
    const int L = m.L;
    const float thresh = u->thresh * std::sqrt(static_cast<float>(P));
    std::vector<UpdApplyDesc> h;
    int slot = 0, block0 = 0;
    long long off = 0;
    for (const UpdMatrix& x : update_matrices(m)) {
        const int n = x.rows * x.cols;
        h.push_back({x.w, x.shadow, z_all + off, m.rms_ema + (slot++), n, block0});
        block0 += (n + 255) / 256;
        off += n;
    }
    for (const UpdVector& x : update_vectors(m)) {
        const float* Z = z_all + off;
        off += x.n;
        if (x.v == m.pos && !u->train_pos) continue;
        h.push_back({nullptr, x.v, Z, m.rms_ema + (slot++), x.n, block0});
        block0 += (x.n + 255) / 256;
    }
    {
        TimedScope ts(m, KC_UPDATE_APPLY, st, 3);
        // pageable source: the copy is staged before the call returns
        TRY(check_cuda(cudaMemcpyAsync(m.upd_descs, h.data(), h.size() * sizeof(UpdApplyDesc), cudaMemcpyHostToDevice, st), "cudaMemcpyAsync(upd_descs)"));
        TRY(update_apply_batched(m.upd_descs, static_cast<int>(h.size()), block0, m.upd_partial, m.upd_inv, u->use_adaptive, u->adaptive_beta,
                                 u->adaptive_eps, u->lr, thresh, st));
    }
    TimedScope ts(m, KC_REQUANTIZE, st, 2 + 3 * L);
    return quantize_base(m, st);
}

}  // namespace

extern "C" {

int bnf4_model_destroy(void* handle) {
    if (!handle) return BNF4_OK;
    Model* m = M(handle);
    cudaDeviceSynchronize();
    m->drop_graphs();
    if (m->cap_stream) cudaStreamDestroy(m->cap_stream);
    for (void* p : m->allocs) cudaFree(p);
    if (m->h_step) cudaFreeHost(m->h_step);
    if (m->d_step_w) cudaFree(m->d_step_w);
    for (cudaEvent_t e : m->free_events) cudaEventDestroy(e);
    for (const Model::Span& sp : m->spans) { cudaEventDestroy(sp.a); cudaEventDestroy(sp.b); }
    delete m;
    return BNF4_OK;
}

int bnf4_model_create(const bnf4_model_cfg* cfg, void** handle) {
    if (!cfg || !handle) return set_error(BNF4_ERR_INVALID, "model_create: null argument");
    *handle = nullptr;
    if (cfg->vocab <= 0 || cfg->vocab > 1024) return set_error(BNF4_ERR_INVALID, "model_create: vocab=%d outside [1,1024]", cfg->vocab);
    if (cfg->hidden <= 0 || (cfg->hidden % 64) != 0) return set_error(BNF4_ERR_INVALID, "model_create: hidden=%d must be a multiple of 64", cfg->hidden);
    if (cfg->layers <= 0 || cfg->mlp_mult <= 0 || cfg->seq <= 0 || cfg->batch <= 0) return set_error(BNF4_ERR_INVALID, "model_create: bad shape");
    if (cfg->heads <= 0 || (cfg->hidden % cfg->heads) != 0 || ((cfg->hidden / cfg->heads) % 32) != 0)
        return set_error(BNF4_ERR_INVALID, "model_create: heads=%d needs head_dim %% 32 == 0", cfg->heads);
    if (cfg->rank < 0 || cfg->rank > 4) return set_error(BNF4_ERR_INVALID, "model_create: rank=%d outside [0,4]", cfg->rank);
    if (cfg->rank == 0 && ((cfg->batch * cfg->seq) % 128) != 0)
        return set_error(BNF4_ERR_INVALID, "model_create: the dense (rank 0) mode needs batch * seq to be a multiple of 128");
    if (cfg->sigma_shift < 0 || cfg->sigma_shift > 30) return set_error(BNF4_ERR_INVALID, "model_create: sigma_shift");
    if (cfg->max_pairs <= 0) return set_error(BNF4_ERR_INVALID, "model_create: max_pairs");
    if (cfg->hidden > 4096) return set_error(BNF4_ERR_INVALID, "model_create: hidden above 4096");
    if (static_cast<long long>(cfg->hidden) * cfg->mlp_mult > 8192) return set_error(BNF4_ERR_INVALID, "model_create: mlp width above 8192");

    Model* m = new Model;
    m->cfg = *cfg;
    m->V = cfg->vocab; m->H = cfg->hidden; m->F = cfg->hidden * cfg->mlp_mult; m->L = cfg->layers; m->T = cfg->seq; m->B = cfg->batch;
    m->R = m->B * m->T; m->FC = (3 * m->H + 1 + 31) & ~31; m->hd = m->H / cfg->heads;
    m->dense = cfg->rank == 0;
    m->r = m->dense ? 1 : cfg->rank;  // the rank-r tables are sized for rank 1 (and left unused) in the dense mode
    m->s_h = 1.0f / std::sqrt(static_cast<float>(m->H));
    m->s_f = 1.0f / std::sqrt(static_cast<float>(m->F));
    m->sigma = 1.0f / static_cast<float>(1 << cfg->sigma_shift);
    m->c_r = kCRankBase / std::sqrt(static_cast<float>(m->r));
    // default wave: as many members as fit about 12 GB of wave buffers, at most 256 (larger waves amortise launches
    // and tile tails; beyond 256 the gain is below 1 %)
    const double row_bytes = m->H * (1.0 + 0.5625 + 4.0) + m->F * 0.5625 + m->FC * 4.0 + 20.0 * m->r;
    const int w_auto = static_cast<int>(std::min(256.0, std::max(2.0, 12e9 / (row_bytes * static_cast<double>(m->R)))));
    int W = cfg->wave_members > 0 ? cfg->wave_members : w_auto;
    if (m->dense) W = 2;  // one pair per wave: its noise matrices exist once
    W = std::min(W, 2 * cfg->max_pairs);
    W = std::max(2, W & ~1);
    m->W = W;
    m->M = static_cast<long long>(W) * m->R;
    if (m->M > 0x7fffffffLL / 8) { delete m; return set_error(BNF4_ERR_INVALID, "model_create: wave of %d members is too large", W); }

    const int V = m->V, H = m->H, F = m->F, L = m->L, T = m->T, r = m->r, P = cfg->max_pairs;
    const size_t hh = static_cast<size_t>(H) * H, hf = static_cast<size_t>(H) * F;
    int rc = 0;
#define A_(ptr, count) if (!rc) rc = m->alloc(&m->ptr, (count))
    A_(emb, static_cast<size_t>(V) * H); A_(win, hh); A_(wq, L * hh); A_(wk, L * hh); A_(wv, L * hh); A_(wbeta, static_cast<size_t>(L) * H);
    A_(ff1, L * hf); A_(ff2, L * hf); A_(head, static_cast<size_t>(V) * H);
    A_(head_bias, V); A_(beta_bias, L); A_(pos, static_cast<size_t>(T) * H);
    A_(sh_emb, static_cast<size_t>(V) * H); A_(sh_win, hh); A_(sh_wq, L * hh); A_(sh_wk, L * hh); A_(sh_wv, L * hh);
    A_(sh_wbeta, static_cast<size_t>(L) * H); A_(sh_ff1, L * hf); A_(sh_ff2, L * hf); A_(sh_head, static_cast<size_t>(V) * H);
    A_(rms_ema, 3 + 6 * static_cast<size_t>(L) + 3);
    A_(q_win, hh / 2); A_(sfq_win, sf_bytes(H, H)); A_(q_head, static_cast<size_t>(V) * H / 2); A_(sfq_head, sf_bytes(V, H));
    m->q_qkv.resize(L); m->sfq_qkv.resize(L); m->q_ff1.resize(L); m->sfq_ff1.resize(L); m->q_ff2.resize(L); m->sfq_ff2.resize(L);
    m->A_qkv.resize(L); m->tB_qkv.resize(L); m->A_ff1.resize(L); m->tB_ff1.resize(L); m->A_ff2.resize(L); m->tB_ff2.resize(L);
    for (int l = 0; l < L && !rc; ++l) {
        A_(q_qkv[l], static_cast<size_t>(m->FC) * H / 2); A_(sfq_qkv[l], sf_bytes(m->FC, H));
        A_(q_ff1[l], hf / 2); A_(sfq_ff1[l], sf_bytes(F, H)); A_(q_ff2[l], hf / 2); A_(sfq_ff2[l], sf_bytes(H, F));
        A_(A_qkv[l], static_cast<size_t>(P) * (3 * H + 1) * r); A_(tB_qkv[l], static_cast<size_t>(P) * 4 * r * H);
        A_(A_ff1[l], static_cast<size_t>(P) * F * r); A_(tB_ff1[l], static_cast<size_t>(P) * r * H);
        A_(A_ff2[l], static_cast<size_t>(P) * H * r); A_(tB_ff2[l], static_cast<size_t>(P) * r * F);
    }
    A_(tokens, m->R); A_(targets, m->R);
    A_(pair_seeds, P);
    A_(embA, static_cast<size_t>(P) * V * r); A_(embB, static_cast<size_t>(P) * H * r);
    A_(A_win, static_cast<size_t>(P) * H * r); A_(tB_win, static_cast<size_t>(P) * H * r);
    A_(A_head, static_cast<size_t>(P) * V * r); A_(tB_head, static_cast<size_t>(P) * H * r);
    A_(pos_noise, static_cast<size_t>(P) * T * H); A_(hb_noise, static_cast<size_t>(P) * V); A_(bb_noise, static_cast<size_t>(P) * L);
    const size_t Mr = static_cast<size_t>(m->M);
    A_(x_q, Mr * H); A_(a_h, Mr * H / 2); A_(sf_h, sf_bytes(static_cast<int>(Mr), H)); A_(a_f, Mr * F / 2); A_(sf_f, sf_bytes(static_cast<int>(Mr), F));
    m->dedup_input = V <= 256 && V < m->R;
    if (m->dedup_input) {
        const size_t Er = static_cast<size_t>(W) * V;
        A_(tok_ident, V); A_(emb_a, Er * H / 2); A_(emb_sf, sf_bytes(static_cast<int>(Er), H)); A_(emb_t, Er * r); A_(y_emb, Er * H);
    }
    A_(qkv, Mr * m->FC); A_(y, Mr * H); A_(bb_eff, static_cast<size_t>(L) * W); A_(ce_partial, static_cast<size_t>(W) * 16); A_(losses, W);
    A_(t_a, Mr * 4 * r); A_(t_f, Mr * r);
    if (m->dense) {
        const DenseLayout lay = dense_layout(*m);
        A_(E_all, lay.total);
        A_(qe_win, hh / 2); A_(sfe_win, sf_bytes(H, H)); A_(qe_head, static_cast<size_t>(V) * H / 2); A_(sfe_head, sf_bytes(V, H));
        m->qe_qkv.resize(L); m->sfe_qkv.resize(L); m->qe_ff1.resize(L); m->sfe_ff1.resize(L); m->qe_ff2.resize(L); m->sfe_ff2.resize(L);
        for (int l = 0; l < L && !rc; ++l) {
            A_(qe_qkv[l], static_cast<size_t>(m->FC) * H / 2); A_(sfe_qkv[l], sf_bytes(m->FC, H));
            A_(qe_ff1[l], hf / 2); A_(sfe_ff1[l], sf_bytes(F, H)); A_(qe_ff2[l], hf / 2); A_(sfe_ff2[l], sf_bytes(H, F));
        }
        A_(noise_descs, 3 + 6 * static_cast<size_t>(L));
        A_(ff1_f, Mr * F); A_(ff1_q, Mr * F);
    }
    A_(Z, static_cast<size_t>(T) * H + V + L); A_(sumsq, 1); A_(inv_rms, 1);
    {
        size_t zn = static_cast<size_t>(V) + L + static_cast<size_t>(T) * H;
        for (const UpdMatrix& x : update_matrices(*m)) zn += static_cast<size_t>(x.rows) * x.cols;
        const size_t nd = update_matrices(*m).size();
        A_(Z_all, zn); A_(zdesc, nd); A_(zdesc_ext, nd);
        size_t nblk = (static_cast<size_t>(V) + 255) / 256 + (static_cast<size_t>(L) + 255) / 256 + (static_cast<size_t>(T) * H + 255) / 256;
        for (const UpdMatrix& x : update_matrices(*m)) nblk += (static_cast<size_t>(x.rows) * x.cols + 255) / 256;
        A_(upd_descs, nd + 3); A_(upd_partial, nblk); A_(upd_inv, nd + 3);
    }
#undef A_
    if (rc) { bnf4_model_destroy(m); return rc; }
    {
        const std::vector<ZLowrankDesc> zd = z_descs(*m, m->Z_all);
        rc = check_cuda(cudaMemcpy(m->zdesc, zd.data(), zd.size() * sizeof(ZLowrankDesc), cudaMemcpyHostToDevice), "cudaMemcpy(zdesc)");
        if (rc) { bnf4_model_destroy(m); return rc; }
    }

    if (m->dedup_input) {
        std::vector<uint8_t> ident(V);
        for (int v = 0; v < V; ++v) ident[v] = static_cast<uint8_t>(v);
        rc = check_cuda(cudaMemcpy(m->tok_ident, ident.data(), V, cudaMemcpyHostToDevice), "cudaMemcpy(tok_ident)");
        if (rc) { bnf4_model_destroy(m); return rc; }
    }
    // noise table
    std::vector<GenDesc> gd;
    auto factor_pair = [&](int8_t* A, long long A_stride, long long A_off, int rows, int8_t* Bt, long long B_stride, long long B_off, int cols,
                           uint64_t salt) {
        gd.push_back({A + A_off, A_stride, salt, kFactorA, rows, r, 0});
        gd.push_back({Bt + B_off, B_stride, salt, kFactorB, cols, r, 1});
    };
    factor_pair(m->embA, static_cast<long long>(V) * r, 0, V, m->embB, static_cast<long long>(H) * r, 0, H, kSaltEmb);
    factor_pair(m->A_win, static_cast<long long>(H) * r, 0, H, m->tB_win, static_cast<long long>(H) * r, 0, H, kSaltWin);
    factor_pair(m->A_head, static_cast<long long>(V) * r, 0, V, m->tB_head, static_cast<long long>(H) * r, 0, H, kSaltHead);
    for (int l = 0; l < L; ++l) {
        const uint64_t lu = static_cast<uint64_t>(l);
        const uint64_t gs[4] = {mix_u64(lu, kSaltWq), mix_u64(lu, kSaltWk), mix_u64(lu, kSaltWv), mix_u64(lu, kSaltWbeta)};
        const int grows[4] = {H, H, H, 1};
        for (int g = 0; g < 4; ++g)
            factor_pair(m->A_qkv[l], static_cast<long long>(3 * H + 1) * r, static_cast<long long>(g) * H * r, grows[g], m->tB_qkv[l],
                        static_cast<long long>(4) * r * H, static_cast<long long>(g) * r * H, H, gs[g]);
        factor_pair(m->A_ff1[l], static_cast<long long>(F) * r, 0, F, m->tB_ff1[l], static_cast<long long>(r) * H, 0, H, mix_u64(lu, kSaltFf1));
        factor_pair(m->A_ff2[l], static_cast<long long>(H) * r, 0, H, m->tB_ff2[l], static_cast<long long>(r) * F, 0, F, mix_u64(lu, kSaltFf2));
    }
    gd.push_back({m->pos_noise, static_cast<long long>(T) * H, kSaltPos, 0, T * H, 1, 0});
    gd.push_back({m->hb_noise, V, kSaltHeadBias, 0, V, 1, 0});
    gd.push_back({m->bb_noise, L, kSaltBetaBias, 0, L, 1, 0});
    m->num_gen = static_cast<int>(gd.size());
    std::vector<uint32_t> bmap;
    for (size_t i = 0; i < gd.size(); ++i) {
        // the last three tables (positional, head-bias and beta-bias noise) are read by the evaluation of a pair only;
        // the factor tables before them are also read by the update, for all pairs
        if (i + 3 == gd.size()) m->gen_blocks_factors = static_cast<int>(bmap.size());
        const long long nb = (static_cast<long long>(gd[i].n_major) * gd[i].rank + 255) / 256;
        if (nb > 0xfffff || i > 0xfff) { bnf4_model_destroy(m); return set_error(BNF4_ERR_INVALID, "model_create: noise table too large"); }
        for (long long b = 0; b < nb; ++b) bmap.push_back(static_cast<uint32_t>(i << 20) | static_cast<uint32_t>(b));
    }
    m->gen_blocks = static_cast<int>(bmap.size());
    rc = m->alloc(&m->gen_descs, gd.size());
    if (!rc) rc = check_cuda(cudaMemcpy(m->gen_descs, gd.data(), gd.size() * sizeof(GenDesc), cudaMemcpyHostToDevice), "cudaMemcpy(gen_descs)");
    if (!rc) rc = m->alloc(&m->gen_block_map, bmap.size());
    if (!rc) rc = check_cuda(cudaMemcpy(m->gen_block_map, bmap.data(), bmap.size() * sizeof(uint32_t), cudaMemcpyHostToDevice), "cudaMemcpy(gen_block_map)");
    if (rc) { bnf4_model_destroy(m); return rc; }
    *handle = m;
    return BNF4_OK;
}

size_t bnf4_model_device_bytes(void* handle) { return handle ? M(handle)->device_bytes : 0; }
int bnf4_model_launches_per_wave(void* handle) { return handle ? M(handle)->launches_per_wave : 0; }
int bnf4_model_wave_members(void* handle) { return handle ? M(handle)->W : 0; }

int bnf4_model_set_weights(void* handle, const bnf4_model_weights* w) {
    if (!handle || !w) return set_error(BNF4_ERR_INVALID, "model_set_weights: null argument");
    Model& m = *M(handle);
    const size_t vh = static_cast<size_t>(m.V) * m.H, hh = static_cast<size_t>(m.H) * m.H, hf = static_cast<size_t>(m.H) * m.F;
    struct Item { void* d; const void* h; size_t bytes; float* shadow; size_t n; };
    const Item items[] = {
        {m.emb, w->emb, vh, m.sh_emb, vh}, {m.win, w->win, hh, m.sh_win, hh}, {m.wq, w->wq, m.L * hh, m.sh_wq, m.L * hh},
        {m.wk, w->wk, m.L * hh, m.sh_wk, m.L * hh}, {m.wv, w->wv, m.L * hh, m.sh_wv, m.L * hh},
        {m.wbeta, w->wbeta, static_cast<size_t>(m.L) * m.H, m.sh_wbeta, static_cast<size_t>(m.L) * m.H},
        {m.ff1, w->ff1, m.L * hf, m.sh_ff1, m.L * hf}, {m.ff2, w->ff2, m.L * hf, m.sh_ff2, m.L * hf}, {m.head, w->head, vh, m.sh_head, vh},
        {m.head_bias, w->head_bias, m.V * sizeof(float), nullptr, 0}, {m.beta_bias, w->beta_bias, m.L * sizeof(float), nullptr, 0},
        {m.pos, w->pos, static_cast<size_t>(m.T) * m.H * sizeof(float), nullptr, 0}};
    for (const Item& it : items) {
        if (!it.h) return set_error(BNF4_ERR_INVALID, "model_set_weights: null weight array");
        TRY(check_cuda(cudaMemcpy(it.d, it.h, it.bytes, cudaMemcpyHostToDevice), "cudaMemcpy(weights)"));
        if (it.shadow) TRY(bnf4_init_shadow_from_weights(static_cast<const int8_t*>(it.d), it.shadow, static_cast<int>(it.n), nullptr));
    }
    TRY(check_cuda(cudaMemset(m.rms_ema, 0, (6 + 6 * static_cast<size_t>(m.L)) * sizeof(float)), "cudaMemset(rms_ema)"));
    TRY(quantize_base(m, nullptr));
    return check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
}

// Optimiser state = the fp32 shadows of the nine weight tensors (same order and sizes as bnf4_model_weights' int8 members,
// concatenated) and the RMS-EMA scalars (6 + 6 * layers). Together with the weights it is everything a resumed run needs.
namespace {
struct ShadowItem { float* d; size_t n; };
void shadow_items(Model& m, ShadowItem (&out)[9]) {
    const size_t vh = static_cast<size_t>(m.V) * m.H, hh = static_cast<size_t>(m.H) * m.H, hf = static_cast<size_t>(m.H) * m.F;
    const ShadowItem items[9] = {{m.sh_emb, vh}, {m.sh_win, hh}, {m.sh_wq, m.L * hh}, {m.sh_wk, m.L * hh}, {m.sh_wv, m.L * hh},
                                 {m.sh_wbeta, static_cast<size_t>(m.L) * m.H}, {m.sh_ff1, m.L * hf}, {m.sh_ff2, m.L * hf}, {m.sh_head, vh}};
    for (int i = 0; i < 9; ++i) out[i] = items[i];
}
}  // namespace

int bnf4_model_optimizer_state_sizes(void* handle, size_t* shadow_floats, size_t* ema_floats) {
    if (!handle) return set_error(BNF4_ERR_INVALID, "model_optimizer_state_sizes: null handle");
    Model& m = *M(handle);
    ShadowItem it[9];
    shadow_items(m, it);
    size_t n = 0;
    for (const ShadowItem& x : it) n += x.n;
    if (shadow_floats) *shadow_floats = n;
    if (ema_floats) *ema_floats = 6 + 6 * static_cast<size_t>(m.L);
    return BNF4_OK;
}

int bnf4_model_get_optimizer_state(void* handle, float* h_shadow, float* h_ema) {
    if (!handle || !h_shadow || !h_ema) return set_error(BNF4_ERR_INVALID, "model_get_optimizer_state: null argument");
    Model& m = *M(handle);
    TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    ShadowItem it[9];
    shadow_items(m, it);
    size_t off = 0;
    for (const ShadowItem& x : it) {
        TRY(check_cuda(cudaMemcpy(h_shadow + off, x.d, x.n * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy(shadow)"));
        off += x.n;
    }
    return check_cuda(cudaMemcpy(h_ema, m.rms_ema, (6 + 6 * static_cast<size_t>(m.L)) * sizeof(float), cudaMemcpyDeviceToHost), "cudaMemcpy(rms_ema)");
}

int bnf4_model_set_optimizer_state(void* handle, const float* h_shadow, const float* h_ema) {
    if (!handle || !h_shadow || !h_ema) return set_error(BNF4_ERR_INVALID, "model_set_optimizer_state: null argument");
    Model& m = *M(handle);
    TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    ShadowItem it[9];
    shadow_items(m, it);
    size_t off = 0;
    for (const ShadowItem& x : it) {
        TRY(check_cuda(cudaMemcpy(x.d, h_shadow + off, x.n * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(shadow)"));
        off += x.n;
    }
    return check_cuda(cudaMemcpy(m.rms_ema, h_ema, (6 + 6 * static_cast<size_t>(m.L)) * sizeof(float), cudaMemcpyHostToDevice), "cudaMemcpy(rms_ema)");
}

int bnf4_model_get_weights(void* handle, bnf4_model_weights* w) {
    if (!handle || !w) return set_error(BNF4_ERR_INVALID, "model_get_weights: null argument");
    Model& m = *M(handle);
    TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    const size_t vh = static_cast<size_t>(m.V) * m.H, hh = static_cast<size_t>(m.H) * m.H, hf = static_cast<size_t>(m.H) * m.F;
    struct Item { const void* d; void* h; size_t bytes; };
    const Item items[] = {{m.emb, w->emb, vh}, {m.win, w->win, hh}, {m.wq, w->wq, m.L * hh}, {m.wk, w->wk, m.L * hh}, {m.wv, w->wv, m.L * hh},
                          {m.wbeta, w->wbeta, static_cast<size_t>(m.L) * m.H}, {m.ff1, w->ff1, m.L * hf}, {m.ff2, w->ff2, m.L * hf},
                          {m.head, w->head, vh}, {m.head_bias, w->head_bias, m.V * sizeof(float)}, {m.beta_bias, w->beta_bias, m.L * sizeof(float)},
                          {m.pos, w->pos, static_cast<size_t>(m.T) * m.H * sizeof(float)}};
    for (const Item& it : items)
        if (it.h) TRY(check_cuda(cudaMemcpy(it.h, it.d, it.bytes, cudaMemcpyDeviceToHost), "cudaMemcpy(weights)"));
    return BNF4_OK;
}

int bnf4_model_set_tokens(void* handle, const uint8_t* tokens, const uint8_t* targets, int on_device, void* stream) {
    if (!handle || !tokens || !targets) return set_error(BNF4_ERR_INVALID, "model_set_tokens: null argument");
    Model& m = *M(handle);
    const cudaMemcpyKind kind = on_device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice;
    TRY(check_cuda(cudaMemcpyAsync(m.tokens, tokens, m.R, kind, S(stream)), "cudaMemcpyAsync(tokens)"));
    return check_cuda(cudaMemcpyAsync(m.targets, targets, m.R, kind, S(stream)), "cudaMemcpyAsync(targets)");
}

int bnf4_model_prepare_step_range(void* handle, uint64_t seed, uint64_t epoch, int pairs, int eval_begin, int eval_count, void* stream) {
    if (!handle) return set_error(BNF4_ERR_INVALID, "model_prepare_step: null handle");
    Model& m = *M(handle);
    if (pairs <= 0 || pairs > m.cfg.max_pairs) return set_error(BNF4_ERR_INVALID, "model_prepare_step: pairs=%d outside [1,%d]", pairs, m.cfg.max_pairs);
    if (pairs > 65535) return set_error(BNF4_ERR_INVALID, "model_prepare_step: at most 65535 pairs");
    if (eval_begin < 0 || eval_count < 0 || eval_begin + eval_count > pairs)
        return set_error(BNF4_ERR_INVALID, "model_prepare_step: evaluation range [%d,%d) outside the %d pairs of the step", eval_begin, eval_begin + eval_count, pairs);
    m.pairs_step = pairs;
    m.eval_begin = eval_begin;
    m.eval_end = eval_begin + eval_count;
    m.step_seed = seed;
    m.step_epoch = epoch;
    TRY(bnf4_fill_pair_seeds(seed, epoch, pairs, m.pair_seeds, stream));
    TimedScope ts(m, KC_GEN_NOISE, S(stream), 3);
    // rank-r factors of all pairs (the update reads them all; the dense mode has none) ...
    if (!m.dense) {
        gen_noise_kernel<<<dim3(m.gen_blocks_factors, pairs), 256, 0, S(stream)>>>(m.gen_descs, m.gen_block_map, 0, 0, m.pair_seeds, m.cfg.use_clt, m.cfg.clt_k);
        TRY(check_launch("gen_noise_kernel"));
    }
    // ... and the per-pair vectors only for the pairs this process evaluates
    if (eval_count > 0) {
        gen_noise_kernel<<<dim3(m.gen_blocks - m.gen_blocks_factors, eval_count), 256, 0, S(stream)>>>(m.gen_descs, m.gen_block_map, m.gen_blocks_factors,
                                                                                                        eval_begin, m.pair_seeds, m.cfg.use_clt, m.cfg.clt_k);
        TRY(check_launch("gen_noise_kernel"));
    }
    return BNF4_OK;
}

int bnf4_model_prepare_step(void* handle, uint64_t seed, uint64_t epoch, int pairs, void* stream) {
    return bnf4_model_prepare_step_range(handle, seed, epoch, pairs, 0, pairs, stream);
}

int bnf4_model_eval_pairs(void* handle, int pair_begin, int pair_count, float* losses, void* stream) {
    if (!handle || !losses) return set_error(BNF4_ERR_INVALID, "model_eval_pairs: null argument");
    Model& m = *M(handle);
    if (pair_begin < 0 || pair_count < 0 || pair_begin + pair_count > m.pairs_step)
        return set_error(BNF4_ERR_INVALID, "model_eval_pairs: pairs [%d,%d) outside the prepared step of %d pairs", pair_begin, pair_begin + pair_count, m.pairs_step);
    if (pair_count > 0 && (pair_begin < m.eval_begin || pair_begin + pair_count > m.eval_end))
        return set_error(BNF4_ERR_INVALID, "model_eval_pairs: pairs [%d,%d) outside the range [%d,%d) the step was prepared for", pair_begin,
                         pair_begin + pair_count, m.eval_begin, m.eval_end);
    if (m.dense) {
        for (int p = 0; p < pair_count; ++p) TRY(run_pair_dense(m, pair_begin + p, losses + 2 * static_cast<size_t>(p), S(stream)));
        return BNF4_OK;
    }
    const int wave_pairs = m.W / 2;
    for (int p = 0; p < pair_count; p += wave_pairs) {
        const int np = std::min(wave_pairs, pair_count - p);
        TRY(run_wave_cached(m, pair_begin + p, 2 * np, m.sigma, losses + 2 * static_cast<size_t>(p), S(stream)));
    }
    return BNF4_OK;
}

int bnf4_model_eval_base(void* handle, float* loss, void* stream) {
    if (!handle || !loss) return set_error(BNF4_ERR_INVALID, "model_eval_base: null argument");
    Model& m = *M(handle);
    TRY(run_wave_cached(m, 0, 2, 0.0f, m.losses, S(stream)));
    return check_cuda(cudaMemcpyAsync(loss, m.losses, sizeof(float), cudaMemcpyDeviceToDevice, S(stream)), "cudaMemcpyAsync(loss)");
}

int bnf4_model_update(void* handle, const float* pair_weights, const bnf4_update_cfg* u, void* stream) {
    if (!handle || !pair_weights || !u) return set_error(BNF4_ERR_INVALID, "model_update: null argument");
    Model& m = *M(handle);
    if (m.pairs_step <= 0) return set_error(BNF4_ERR_INVALID, "model_update: no prepared step");
    TRY(update_z(m, pair_weights, 0, 1, nullptr, S(stream)));
    return update_apply(m, pair_weights, m.Z_all, u, S(stream));
}

int bnf4_model_update_z_layout(void* handle, int nshards, int max_entries, long long* offsets, long long* elems, int* sharded,
                               long long* total_elems) {
    if (!handle || nshards < 1) { set_error(BNF4_ERR_INVALID, "model_update_z_layout: bad argument"); return -1; }
    Model& m = *M(handle);
    const std::vector<UpdMatrix> mats = update_matrices(m);
    const std::vector<UpdVector> vecs = update_vectors(m);
    const int total = static_cast<int>(mats.size() + vecs.size());
    if (total > max_entries && (offsets || elems || sharded)) {
        set_error(BNF4_ERR_INVALID, "model_update_z_layout: %d entries needed, room for %d", total, max_entries);
        return -1;
    }
    long long off = 0;
    for (size_t i = 0; i < mats.size(); ++i) {
        const long long n = static_cast<long long>(mats[i].rows) * mats[i].cols;
        if (offsets) offsets[i] = off;
        if (elems) elems[i] = n;
        if (sharded) sharded[i] = (nshards > 1 && mats[i].rows >= nshards && (mats[i].rows % nshards) == 0) ? 1 : 0;
        off += n;
    }
    for (size_t i = 0; i < vecs.size(); ++i) {
        const size_t j = mats.size() + i;
        if (offsets) offsets[j] = off;
        if (elems) elems[j] = vecs[i].n;
        if (sharded) sharded[j] = vector_sharded(vecs[i].n, nshards) ? 1 : 0;
        off += vecs[i].n;
    }
    if (total_elems) *total_elems = off;
    return total;
}

int bnf4_model_update_z(void* handle, const float* pair_weights, int shard, int nshards, float* z_all, void* stream) {
    if (!handle || !pair_weights || !z_all) return set_error(BNF4_ERR_INVALID, "model_update_z: null argument");
    if (nshards < 1 || shard < 0 || shard >= nshards) return set_error(BNF4_ERR_INVALID, "model_update_z: shard %d of %d", shard, nshards);
    Model& m = *M(handle);
    if (m.pairs_step <= 0) return set_error(BNF4_ERR_INVALID, "model_update_z: no prepared step");
    return update_z(m, pair_weights, shard, nshards, z_all, S(stream));
}

int bnf4_model_update_apply(void* handle, const float* pair_weights, const float* z_all, const bnf4_update_cfg* u, void* stream) {
    if (!handle || !pair_weights || !z_all || !u) return set_error(BNF4_ERR_INVALID, "model_update_apply: null argument");
    Model& m = *M(handle);
    if (m.pairs_step <= 0) return set_error(BNF4_ERR_INVALID, "model_update_apply: no prepared step");
    return update_apply(m, pair_weights, z_all, u, S(stream));
}

int bnf4_model_es_step(void* handle, const bnf4_es_step_cfg* cfg, const bnf4_collectives* coll, float* d_losses_all, void* stream) {
    if (!handle || !cfg || !d_losses_all) return set_error(BNF4_ERR_INVALID, "model_es_step: null argument");
    Model& m = *M(handle);
    const int world = cfg->world, rank = cfg->rank, pairs = cfg->pairs;
    if (world < 1 || rank < 0 || rank >= world) return set_error(BNF4_ERR_INVALID, "model_es_step: rank %d of %d", rank, world);
    if (pairs <= 0 || (pairs % world) != 0) return set_error(BNF4_ERR_INVALID, "model_es_step: pairs=%d must be a positive multiple of world=%d", pairs, world);
    if (world > 1 && (!coll || !coll->allgather_inplace)) return set_error(BNF4_ERR_INVALID, "model_es_step: more than one rank needs the all-gather callback");
    cudaStream_t st = S(stream);
    const int count = pairs / world, begin = rank * count;
    TRY(bnf4_model_prepare_step_range(handle, cfg->seed, cfg->epoch, pairs, begin, count, stream));
    TRY(bnf4_model_eval_pairs(handle, begin, count, d_losses_all + 2 * static_cast<size_t>(begin), stream));
    if (world > 1 && coll->allgather_inplace(coll->ctx, d_losses_all, 2 * static_cast<size_t>(count) * sizeof(float), stream) != 0)
        return set_error(BNF4_ERR_CUDA, "model_es_step: the all-gather of the losses failed");
    // fitness shaping on the host, like the reference (src/train_efla_lm.cpp:5466, 5476): f_p = -(loss+ - loss-)
    if (m.h_step == nullptr) {
        TRY(check_cuda(cudaMallocHost(&m.h_step, 3 * static_cast<size_t>(m.cfg.max_pairs) * sizeof(float)), "cudaMallocHost(es_step)"));
        TRY(check_cuda(cudaMalloc(&m.d_step_w, static_cast<size_t>(m.cfg.max_pairs) * sizeof(float)), "cudaMalloc(es_step)"));
    }
    float* h_losses = m.h_step;
    float* h_w = m.h_step + 2 * static_cast<size_t>(m.cfg.max_pairs);
    TRY(check_cuda(cudaMemcpyAsync(h_losses, d_losses_all, 2 * static_cast<size_t>(pairs) * sizeof(float), cudaMemcpyDeviceToHost, st), "cudaMemcpyAsync(losses)"));
    TRY(check_cuda(cudaStreamSynchronize(st), "cudaStreamSynchronize"));
    for (int p = 0; p < pairs; ++p) h_w[p] = -(h_losses[2 * p] - h_losses[2 * p + 1]);
    TRY(bnf4_shape_pair_weights(h_w, pairs, cfg->fitness_mode, cfg->fitness_clip));
    TRY(check_cuda(cudaMemcpyAsync(m.d_step_w, h_w, static_cast<size_t>(pairs) * sizeof(float), cudaMemcpyHostToDevice, st), "cudaMemcpyAsync(pair weights)"));
    if (world == 1) {
        TRY(update_z(m, m.d_step_w, 0, 1, nullptr, st));
        return update_apply(m, m.d_step_w, m.Z_all, &cfg->update, st);
    }
    // Z by rows over the ranks into the model's own buffer (the layout does not depend on the number of shards), gathered in place
    TRY(update_z(m, m.d_step_w, rank, world, m.Z_all, st));
    const std::vector<UpdMatrix> mats = update_matrices(m);
    const std::vector<UpdVector> vecs = update_vectors(m);
    if (coll->group_begin && coll->group_begin(coll->ctx) != 0) return set_error(BNF4_ERR_CUDA, "model_es_step: group_begin failed");
    long long off = 0;
    int failed = 0;
    for (size_t i = 0; i < mats.size() + vecs.size() && !failed; ++i) {
        const bool is_mat = i < mats.size();
        const long long n = is_mat ? static_cast<long long>(mats[i].rows) * mats[i].cols : vecs[i - mats.size()].n;
        const bool sharded = is_mat ? (mats[i].rows >= world && (mats[i].rows % world) == 0) : vector_sharded(vecs[i - mats.size()].n, world);
        if (sharded) failed = coll->allgather_inplace(coll->ctx, m.Z_all + off, static_cast<size_t>(n / world) * sizeof(float), stream);
        off += n;
    }
    if (coll->group_end && coll->group_end(coll->ctx) != 0) failed = 1;
    if (failed) return set_error(BNF4_ERR_CUDA, "model_es_step: the all-gather of the noise sums failed");
    return update_apply(m, m.d_step_w, m.Z_all, &cfg->update, st);
}

int bnf4_model_set_timing(void* handle, int enable) {
    if (!handle) return set_error(BNF4_ERR_INVALID, "model_set_timing: null handle");
    Model& m = *M(handle);
    m.timing = enable != 0;
    for (int c = 0; c < kNumClasses; ++c) { m.class_ms[c] = 0.0; m.class_launches[c] = 0; }
    for (auto& sp : m.spans) { m.free_events.push_back(sp.a); m.free_events.push_back(sp.b); }
    m.spans.clear();
    return BNF4_OK;
}

int bnf4_model_set_graph(void* handle, int enable) {
    if (!handle) return set_error(BNF4_ERR_INVALID, "model_set_graph: null handle");
    Model& m = *M(handle);
    if (enable == 0 && m.use_graph) {
        TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));  // a cached graph may still be running
        m.drop_graphs();
    }
    m.use_graph = enable != 0;
    return BNF4_OK;
}

long long bnf4_model_graph_launches(void* handle) { return handle ? M(handle)->graph_launches : 0; }

int bnf4_model_num_kernel_classes(void) { return kNumClasses; }
const char* bnf4_model_kernel_class_name(int cls) { return (cls >= 0 && cls < kNumClasses) ? kClassNames[cls] : ""; }

int bnf4_model_get_timing(void* handle, double* ms, long long* launches, int n) {
    if (!handle || !ms || !launches) return set_error(BNF4_ERR_INVALID, "model_get_timing: null argument");
    Model& m = *M(handle);
    TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    for (auto& sp : m.spans) {
        float t = 0.0f;
        if (cudaEventElapsedTime(&t, sp.a, sp.b) == cudaSuccess) m.class_ms[sp.cls] += t;
        m.free_events.push_back(sp.a);
        m.free_events.push_back(sp.b);
    }
    m.spans.clear();
    for (int c = 0; c < n && c < kNumClasses; ++c) { ms[c] = m.class_ms[c]; launches[c] = m.class_launches[c]; }
    return BNF4_OK;
}

int bnf4_model_read_buffer(void* handle, const char* name, void* h_dst, size_t bytes) {
    if (!handle || !name || !h_dst) return set_error(BNF4_ERR_INVALID, "model_read_buffer: null argument");
    Model& m = *M(handle);
    const size_t Mr = static_cast<size_t>(m.M);
    const std::string n(name);
    const void* src = nullptr;
    size_t size = 0;
    if (n == "x_q") { src = m.x_q; size = Mr * m.H; }
    else if (n == "a_h") { src = m.a_h; size = Mr * m.H / 2; }
    else if (n == "sf_h") { src = m.sf_h; size = sf_bytes(static_cast<int>(Mr), m.H); }
    else if (n == "a_f") { src = m.a_f; size = Mr * m.F / 2; }
    else if (n == "sf_f") { src = m.sf_f; size = sf_bytes(static_cast<int>(Mr), m.F); }
    else if (n == "qkv") { src = m.qkv; size = Mr * m.FC * sizeof(float); }
    else if (n == "y") { src = m.y; size = Mr * m.H * sizeof(float); }
    else if (n == "t_a") { src = m.t_a; size = Mr * 4 * m.r * sizeof(int32_t); }
    else if (n == "t_f") { src = m.t_f; size = Mr * m.r * sizeof(int32_t); }
    else if (n == "losses") { src = m.losses; size = m.W * sizeof(float); }
    else return set_error(BNF4_ERR_INVALID, "model_read_buffer: unknown buffer '%s'", name);
    TRY(check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize"));
    return check_cuda(cudaMemcpy(h_dst, src, std::min(bytes, size), cudaMemcpyDeviceToHost), "cudaMemcpy(read_buffer)");
}

}  // extern "C"
