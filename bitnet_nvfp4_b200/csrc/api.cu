// extern "C" surface of libbnf4: library state, size helpers, quantisers and GEMM entry points.
// Each function mirrors the argument meaning of the reference function named in include/bnf4.h.

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {

namespace {
thread_local char g_err[512] = "";
std::atomic<unsigned long long> g_launches{0};
}  // namespace

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return BNF4_OK;
    const int code = (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? BNF4_ERR_NO_DEVICE : BNF4_ERR_CUDA;
    return set_error(code, "%s: %s", what, cudaGetErrorString(e));
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

int check_launch(const char* what) {
    count_launch();
    return check_cuda(cudaGetLastError(), what);
}

}  // namespace bnf4

using namespace bnf4;

static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

const char* bnf4_last_error(void) { return g_err; }
const char* bnf4_version(void) { return "bnf4 0.1 (sm_100a)"; }
unsigned long long bnf4_launch_count(void) { return g_launches.load(); }

int bnf4_set_option(const char* name, int value) {
    if (name && std::strcmp(name, "gemm_tma_store") == 0) {
        if (value != 0 && value != 1) return set_error(BNF4_ERR_INVALID, "gemm_tma_store must be 0 or 1");
        g_gemm_allow_tma_store = value;
        return BNF4_OK;
    }
    if (name && std::strcmp(name, "efla_chunked") == 0) {
        if (value != 0 && value != 1) return set_error(BNF4_ERR_INVALID, "efla_chunked must be 0 or 1");
        g_efla_chunked = value;
        return BNF4_OK;
    }
    return set_error(BNF4_ERR_INVALID, "unknown option '%s'", name ? name : "(null)");
}

int bnf4_device_error(void* stream, int* code) { return gemm_nvfp4_device_error(S(stream), code); }

int bnf4_struct_sizes(int* rowquant_desc_bytes, int* gemm_desc_bytes) {
    if (rowquant_desc_bytes) *rowquant_desc_bytes = static_cast<int>(sizeof(bnf4_rowquant_desc));
    if (gemm_desc_bytes) *gemm_desc_bytes = static_cast<int>(sizeof(bnf4_gemm_desc));
    return BNF4_OK;
}

size_t bnf4_nvfp4_matrix_bytes(int rows, int cols) { return (static_cast<size_t>(rows) * static_cast<size_t>(cols) * 4 + 7) / 8; }
size_t bnf4_nvfp4_sfa_bytes(int m, int /*n*/, int k) { return sf_bytes(m, k); }
size_t bnf4_nvfp4_sfb_bytes(int /*m*/, int n, int k) { return sf_bytes(n, k); }

// --------------------------------------------------------------------------------------------- quantisers
int bnf4_rowquant(int front_end, const bnf4_rowquant_desc* desc, void* stream) {
    if (!desc) return set_error(BNF4_ERR_INVALID, "bnf4_rowquant: null descriptor");
    return rowquant_dispatch(front_end, *desc, S(stream));
}

int bnf4_nvfp4_quantize_a(const int8_t* in, int m, int /*n*/, int k_in, int k_out, void* out, void* sfa, void* stream) {
    if (m <= 0 || k_out <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = m; p.cols_in = k_in; p.cols_out = k_out; p.in_i8 = in; p.ld_in = k_in;
    p.out_codes = static_cast<uint8_t*>(out); p.out_sf = static_cast<uint8_t*>(sfa);
    return rowquant_dispatch(FE_INT8, p, S(stream));
}

int bnf4_nvfp4_quantize_b(const int8_t* in, int /*m*/, int n, int k_in, int k_out, void* out, void* sfb, void* stream) {
    if (n <= 0 || k_out <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = n; p.cols_in = k_in; p.cols_out = k_out; p.in_i8 = in; p.ld_in = k_in;
    p.out_codes = static_cast<uint8_t*>(out); p.out_sf = static_cast<uint8_t*>(sfb);
    return rowquant_dispatch(FE_INT8, p, S(stream));
}

int bnf4_nvfp4_quantize_wqkv_fused(const int8_t* wq, const int8_t* wk, const int8_t* wv, const int8_t* wb, int /*batch*/,
                                   int hidden, int k_out, int rows_total, float q_scale, float k_scale, float v_scale,
                                   float b_scale, void* out, void* sfb, void* stream) {
    if (hidden <= 0 || k_out <= 0 || rows_total <= 0) return BNF4_OK;
    const int rows_valid = 3 * hidden + 1;
    if (rows_total < rows_valid) return set_error(BNF4_ERR_INVALID, "quantize_wqkv_fused: rows_total=%d < 3*hidden+1", rows_total);
    if (k_out != hidden) return set_error(BNF4_ERR_INVALID, "quantize_wqkv_fused: k_out must equal hidden");
    bnf4_rowquant_desc p = {};
    p.rows = rows_valid; p.cols_in = hidden; p.cols_out = k_out;
    p.wq = wq; p.wk = wk; p.wv = wv; p.wb = wb;
    p.q_scale = q_scale; p.k_scale = k_scale; p.v_scale = v_scale; p.b_scale = b_scale;
    p.out_codes = static_cast<uint8_t*>(out); p.out_sf = static_cast<uint8_t*>(sfb);
    return rowquant_dispatch(FE_WQKV, p, S(stream));
}

int bnf4_embedding_lookup_noise_quantize_nvfp4(const uint8_t* tokens_t, int token_stride, const int8_t* emb_w,
                                               const int8_t* emb_noise, int hidden, int batch, float noise_scale,
                                               int anti_sign, int8_t* out_q, void* out_nvfp4, void* sfa, void* stream) {
    if (batch <= 0 || hidden <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = batch; p.cols_in = hidden; p.cols_out = hidden;
    p.tokens = tokens_t; p.token_stride = token_stride; p.emb_w = emb_w; p.emb_noise = emb_noise;
    p.sigma = noise_scale; p.anti_fixed = anti_sign;
    p.out_q = out_q; p.ld_q = hidden; p.out_codes = static_cast<uint8_t*>(out_nvfp4); p.out_sf = static_cast<uint8_t*>(sfa);
    return rowquant_dispatch(FE_EMBED_DENSE, p, S(stream));
}

int bnf4_add_pos_gelu_quantize_nvfp4(const float* in, const float* pos_t, int hidden, int batch, float act_scale,
                                     int8_t* out_q, void* out_nvfp4, void* sfa, void* stream) {
    if (batch <= 0 || hidden <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = batch; p.cols_in = hidden; p.cols_out = hidden; p.in_f32 = in; p.ld_in = hidden;
    p.pos = pos_t; p.pos_mod = 0; p.act_scale = act_scale;
    p.out_q = out_q; p.ld_q = hidden; p.out_codes = static_cast<uint8_t*>(out_nvfp4); p.out_sf = static_cast<uint8_t*>(sfa);
    return rowquant_dispatch(FE_POS_GELU, p, S(stream));
}

int bnf4_activation_quantize_nvfp4(const float* in, int rows, int cols_in, int cols_out, int activation, int8_t* out_q,
                                   void* out_nvfp4, void* sfa, void* stream) {
    if (rows <= 0 || cols_out <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = rows; p.cols_in = cols_in; p.cols_out = cols_out; p.in_f32 = in; p.ld_in = cols_in;
    p.act_mode = activation; p.act_scale = 1.0f;
    p.out_q = out_q; p.ld_q = cols_out; p.out_codes = static_cast<uint8_t*>(out_nvfp4); p.out_sf = static_cast<uint8_t*>(sfa);
    return rowquant_dispatch(FE_ACT, p, S(stream));
}

int bnf4_gelu_quantize_nvfp4(const float* in, int rows, int cols_in, int cols_out, float act_scale, int8_t* out_q,
                             void* out_nvfp4, void* sfa, void* stream) {
    if (rows <= 0 || cols_out <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = rows; p.cols_in = cols_in; p.cols_out = cols_out; p.in_f32 = in; p.ld_in = cols_in;
    p.act_mode = 3; p.act_scale = act_scale;
    p.out_q = out_q; p.ld_q = cols_out; p.out_codes = static_cast<uint8_t*>(out_nvfp4); p.out_sf = static_cast<uint8_t*>(sfa);
    return rowquant_dispatch(FE_ACT, p, S(stream));
}

int bnf4_absmean_norm_q_nvfp4(const int8_t* in, int hidden, int batch, int cols_out, float scale, int8_t* out_q,
                              void* out_nvfp4, void* sfa, void* stream) {
    if (batch <= 0 || hidden <= 0 || cols_out <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = batch; p.cols_in = hidden; p.cols_out = cols_out; p.in_i8 = in; p.ld_in = hidden; p.norm_scale = scale;
    p.out_q = out_q; p.ld_q = hidden; p.out_codes = static_cast<uint8_t*>(out_nvfp4); p.out_sf = static_cast<uint8_t*>(sfa);
    return rowquant_dispatch(FE_ABSMEAN, p, S(stream));
}

int bnf4_add_scaled_to_int8_absmean_norm_q_nvfp4(int8_t* inout, const float* in, int hidden, int batch, int cols_out,
                                                 float add_scale, float norm_scale, int8_t* out_q, void* out_nvfp4,
                                                 void* sfa, void* stream) {
    if (batch <= 0 || hidden <= 0 || cols_out <= 0) return BNF4_OK;
    bnf4_rowquant_desc p = {};
    p.rows = batch; p.cols_in = hidden; p.cols_out = cols_out; p.inout_i8 = inout; p.in_f32 = in; p.ld_in = hidden;
    p.add_scale = add_scale; p.norm_scale = norm_scale;
    p.out_q = out_q; p.ld_q = hidden; p.out_codes = static_cast<uint8_t*>(out_nvfp4); p.out_sf = static_cast<uint8_t*>(sfa);
    return rowquant_dispatch(FE_ADD_ABSMEAN, p, S(stream));
}

// --------------------------------------------------------------------------------------------- GEMM
int bnf4_gemm_nvfp4_ex(const bnf4_gemm_desc* desc, void* stream) {
    if (!desc) return set_error(BNF4_ERR_INVALID, "bnf4_gemm_nvfp4_ex: null descriptor");
    return gemm_nvfp4_launch(*desc, S(stream));
}

int bnf4_gemm_ternary_f_nvfp4(const void* a, const void* b, const void* sfa, const void* sfb, int m, int n, int k,
                              float alpha, float beta, const float* c, float* d, void* stream) {
    bnf4_gemm_desc g = {};
    g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.m = m; g.n = n; g.k = k; g.alpha = alpha; g.beta = beta;
    g.c = c; g.ldc = n; g.d = d; g.ldd = n; g.epilogue = EPI_F32;
    return gemm_nvfp4_launch(g, S(stream));
}

int bnf4_gemm_ternary_f_nvfp4_gelu_i8(const void* a, const void* b, const void* sfa, const void* sfb, int m, int n,
                                      int k, float alpha, float beta, const float* c, float act_scale, int8_t* d,
                                      void* stream) {
    bnf4_gemm_desc g = {};
    g.a = a; g.b = b; g.sfa = sfa; g.sfb = sfb; g.m = m; g.n = n; g.k = k; g.alpha = alpha; g.beta = beta;
    g.c = c; g.ldc = n; g.d_i8 = d; g.ld_i8 = n; g.epilogue = EPI_GELU_I8; g.act_scale = act_scale;
    return gemm_nvfp4_launch(g, S(stream));
}

int bnf4_nvfp4_prepare_gemm(const void* a, const void* b, const void* sfa, const void* sfb, int m, int n, int k,
                            float /*alpha*/, float /*beta*/, const float* /*c*/, float* d, void* /*stream*/) {
    if (!a || !b || !sfa || !sfb || !d) return set_error(BNF4_ERR_INVALID, "nvfp4_prepare_gemm: null operand");
    if (m <= 0 || n <= 0 || k <= 0 || (k % 64) != 0) return set_error(BNF4_ERR_INVALID, "nvfp4_prepare_gemm: unsupported shape %dx%dx%d", m, n, k);
    return BNF4_OK;
}

// Host function (reference: shape_pair_weights src/train_efla_lm.cpp:3898-3952). Ties in the rank sort are
// broken by index so that every rank of a data-parallel job shapes identically. `mode` takes the values of the
// reference's TrainConfig::FitnessMode (src/train_efla_lm.cpp:260): 0 sign, 1 z-score, 2 centered rank.
int bnf4_shape_pair_weights(float* w, int n, int mode, float clip) {
    if (n <= 0) return BNF4_OK;
    if (!w) return set_error(BNF4_ERR_INVALID, "shape_pair_weights: null pointer");
    if (mode == BNF4_FITNESS_SIGN) {
        for (int i = 0; i < n; ++i) w[i] = w[i] > 0.0f ? 1.0f : (w[i] < 0.0f ? -1.0f : 0.0f);
        return BNF4_OK;
    }
    if (mode == BNF4_FITNESS_CENTERED_RANK) {
        std::vector<int> order(n);
        for (int i = 0; i < n; ++i) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return w[a] < w[b]; });
        std::vector<float> ranked(n);
        if (n == 1) ranked[0] = 0.0f;
        else
            for (int r = 0; r < n; ++r) ranked[order[r]] = static_cast<float>(r) / static_cast<float>(n - 1) - 0.5f;
        for (int i = 0; i < n; ++i) w[i] = ranked[i];
    } else if (mode != BNF4_FITNESS_ZSCORE) {
        return set_error(BNF4_ERR_INVALID, "shape_pair_weights: unknown mode %d", mode);
    }
    float mean = 0.0f;
    for (int i = 0; i < n; ++i) mean += w[i];
    mean /= static_cast<float>(n);
    float var = 0.0f;
    for (int i = 0; i < n; ++i) var += (w[i] - mean) * (w[i] - mean);
    var /= static_cast<float>(n);
    const float stdv = std::sqrt(var) + 1e-6f;
    for (int i = 0; i < n; ++i) {
        float d = (w[i] - mean) / stdv;
        if (d > clip) d = clip;
        if (d < -clip) d = -clip;
        w[i] = d;
    }
    return BNF4_OK;
}

}  // extern "C"
