// EFLA / DeltaNet recurrent linear-attention kernels.
//
// Per row (one sequence position) and per head (reference math: src/efla_lm_kernels.cu:590-726, split form
// :821-913 prepare, :1108-1141 kS, :1186-1197 diff, :1328-1356 update, :1563-1590 readout):
//   q^ = q * rsqrt(sum q^2 + eps);  lambda = max(sum k^2, eps);  beta = sigmoid(beta_raw + beta_bias)
//   alpha = -expm1(-beta*lambda) / (lambda + eps)            (EFLA; DeltaNet: alpha = beta, k <- k*rsqrt(lambda+eps))
//   kS[n] = sum_d k[d] S[d,n];  diff = v - kS;  S[d,n] <- fp16_rn(S[d,n] + alpha k[d] diff[n]);  y[n] = sum_d S[d,n] q^[d]
// The reference keeps S (hidden x hidden, fp16) in HBM and streams it four times per token through six
// kernels. Columns of S are independent, so here the state never leaves the SM:
//   * scan kernel, head_dim 64: one warp owns one (sequence, head); the 64x64 state lives in registers
//     (each lane owns two columns) for all T tokens; q/k/v of the next token are prefetched while the
//     current one is processed. HBM traffic is the algorithmic minimum: read q,k,v,beta, write y.
//   * generic kernel, any head_dim: one CTA owns a column slice of one (sequence, head) in shared
//     memory; also serves the reference's single-step entry points (state loaded from / stored to HBM).
// heads == 1 reproduces the reference; beta is one scalar per row, q-norm / lambda / alpha are per head.

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {

namespace {

__device__ __forceinline__ float sigmoidf_dev(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename ST> struct StateCvt;
template <> struct StateCvt<__half> {
    static __device__ __forceinline__ float load(__half h) { return __half2float(h); }
    static __device__ __forceinline__ __half store(float f) { return __float2half_rn(f); }
};
template <> struct StateCvt<float> {
    static __device__ __forceinline__ float load(float h) { return h; }
    static __device__ __forceinline__ float store(float f) { return f; }
};

// ------------------------------------------------------------------------------------------------
// Generic kernel: grid (column slices, heads, sequences), blockDim.x = columns per slice (multiple of 32).
// ------------------------------------------------------------------------------------------------
template <typename ST>
__global__ void efla_generic_kernel(const EflaParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int hd = p.hidden / p.heads;
    const int nc = blockDim.x;
    const int j = threadIdx.x;
    const int n = blockIdx.x * nc + j;  // column within the head
    const int h = blockIdx.y;
    const long long seq = blockIdx.z;
    const bool col_ok = n < hd;

    ST* S = reinterpret_cast<ST*>(smem);                                  // [hd][nc]
    float* q_sh = reinterpret_cast<float*>(smem + sizeof(ST) * hd * nc);  // [hd]
    float* k_sh = q_sh + hd;                                              // [hd]
    float* red = k_sh + hd;                                               // [2 * 32 + 4]

    ST* Sg = nullptr;
    if (p.state != nullptr) Sg = reinterpret_cast<ST*>(p.state) + (static_cast<size_t>(seq) * p.heads + h) * hd * hd;
    for (int d = 0; d < hd; ++d) S[d * nc + j] = (Sg != nullptr && col_ok) ? Sg[static_cast<size_t>(d) * hd + n] : StateCvt<ST>::store(0.0f);

    const float beta_bias = p.beta_bias_seq != nullptr ? p.beta_bias_seq[seq / p.seqs_per_bias] : p.beta_bias;
    const int lane = j & 31, warp = j >> 5, nwarps = nc >> 5;

    for (int t = 0; t < p.T; ++t) {
        const size_t row = static_cast<size_t>(seq) * p.T + t;
        const float* qr = p.q + row * p.ld_qkv + h * hd;
        const float* kr = p.k + row * p.ld_qkv + h * hd;
        const float* vr = p.v + row * p.ld_qkv + h * hd;
        __syncthreads();  // previous step finished with q_sh / k_sh
        float qss = 0.0f, kss = 0.0f;
        for (int d = j; d < hd; d += nc) {
            const float qv = qr[d], kv = kr[d];
            q_sh[d] = qv;
            k_sh[d] = kv;
            qss = fmaf(qv, qv, qss);
            kss = fmaf(kv, kv, kss);
        }
        qss = warp_sum_f(qss);
        kss = warp_sum_f(kss);
        if (lane == 0) { red[warp] = qss; red[32 + warp] = kss; }
        __syncthreads();
        if (j == 0) {
            float qt = 0.0f, kt = 0.0f;
            for (int w = 0; w < nwarps; ++w) { qt += red[w]; kt += red[32 + w]; }
            const float beta = sigmoidf_dev(p.beta_raw[row * p.ld_beta] + beta_bias);
            const float lambda = kt < p.eps ? p.eps : kt;
            float alpha, kscale = 1.0f;
            if (p.method == 0) { alpha = beta; kscale = rsqrtf(lambda + p.eps); }
            else alpha = -expm1f(-(beta * lambda)) / (lambda + p.eps);
            red[64] = rsqrtf(qt + p.eps);
            red[65] = alpha;
            red[66] = kscale;
        }
        __syncthreads();
        const float q_inv = red[64], alpha = red[65], kscale = red[66];
        if (col_ok) {
            float acc = 0.0f;
            for (int d = 0; d < hd; ++d) acc = fmaf(k_sh[d] * kscale, StateCvt<ST>::load(S[d * nc + j]), acc);
            const float diff = vr[n] - acc;
            float y = 0.0f;
            for (int d = 0; d < hd; ++d) {
                const float sc = alpha * (k_sh[d] * kscale);
                const ST sn = StateCvt<ST>::store(fmaf(sc, diff, StateCvt<ST>::load(S[d * nc + j])));
                S[d * nc + j] = sn;
                y = fmaf(StateCvt<ST>::load(sn), q_sh[d] * q_inv, y);
            }
            p.out[row * p.ld_out + h * hd + n] = y;
        }
    }
    if (Sg != nullptr && col_ok)
        for (int d = 0; d < hd; ++d) Sg[static_cast<size_t>(d) * hd + n] = S[d * nc + j];
}

// ------------------------------------------------------------------------------------------------
// Scan kernel for head_dim 64, fp16-rounded state held in registers (fp32 containers), zero initial state.
// One warp = one (sequence, head); lane owns columns lane and lane+32.
// ------------------------------------------------------------------------------------------------
constexpr int kScanWarps = 4;

// NCOL = 2: one warp per (sequence, head), lane owns columns lane and lane+32 (128 state registers).
// NCOL = 1: two warps per (sequence, head), lane owns one column (64 state registers, twice the warps per SM).
// The state is held as float2 pairs over adjacent rows (d, d+1) so that the three multiply-adds per state element
// (k.S, the rank-1 update, S.q^) issue as packed fma.rn.f32x2 instructions.
template <int NCOL>
__global__ void __launch_bounds__(kScanWarps * 32, NCOL == 1 ? 4 : 2) efla_scan64_kernel(const EflaParams p) {
    constexpr int HD = 64, HP = HD / 2;
    __shared__ __align__(16) float sh[kScanWarps][3][HD];  // k, q^, alpha*k per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long wunit = static_cast<long long>(blockIdx.x) * kScanWarps + warp;
    const long long unit = NCOL == 1 ? (wunit >> 1) : wunit;  // (sequence, head)
    const int colbase = NCOL == 1 ? static_cast<int>(wunit & 1) * 32 : 0;
    if (unit >= p.seqs * static_cast<long long>(p.heads)) return;
    const long long seq = unit / p.heads;
    const int h = static_cast<int>(unit - seq * p.heads);
    const float beta_bias = p.beta_bias_seq != nullptr ? p.beta_bias_seq[seq / p.seqs_per_bias] : p.beta_bias;

    float2 S[NCOL][HP];  // S[c][j] = (S[2j][col c], S[2j+1][col c])
#pragma unroll
    for (int c = 0; c < NCOL; ++c)
#pragma unroll
        for (int j = 0; j < HP; ++j) S[c][j] = make_float2(0.0f, 0.0f);

    const size_t row0 = static_cast<size_t>(seq) * p.T;
    const float* qb = p.q + row0 * p.ld_qkv + h * HD;
    const float* kb = p.k + row0 * p.ld_qkv + h * HD;
    const float* vb = p.v + row0 * p.ld_qkv + h * HD;
    const float* bb = p.beta_raw + row0 * p.ld_beta;
    float* ob = p.out + row0 * p.ld_out + h * HD;

    // prefetch token 0 (q and k: all 64 elements across the warp; v: this lane's columns)
    float q0 = qb[lane], q1 = qb[lane + 32], k0 = kb[lane], k1 = kb[lane + 32], br = bb[0];
    float vv[NCOL];
#pragma unroll
    for (int c = 0; c < NCOL; ++c) vv[c] = vb[colbase + lane + 32 * c];

    float* k_s = sh[warp][0];
    float* q_s = sh[warp][1];
    float* a_s = sh[warp][2];

    for (int t = 0; t < p.T; ++t) {
        const float cq0 = q0, cq1 = q1, ck0 = k0, ck1 = k1, cbr = br;
        float cv[NCOL];
#pragma unroll
        for (int c = 0; c < NCOL; ++c) cv[c] = vv[c];
        if (t + 1 < p.T) {
            const size_t o = static_cast<size_t>(t + 1) * p.ld_qkv;
            q0 = qb[o + lane]; q1 = qb[o + lane + 32];
            k0 = kb[o + lane]; k1 = kb[o + lane + 32];
#pragma unroll
            for (int c = 0; c < NCOL; ++c) vv[c] = vb[o + colbase + lane + 32 * c];
            br = bb[static_cast<size_t>(t + 1) * p.ld_beta];
        }
        const float qss = warp_sum_f(fmaf(cq0, cq0, cq1 * cq1));
        const float kss = warp_sum_f(fmaf(ck0, ck0, ck1 * ck1));
        const float q_inv = rsqrtf(qss + p.eps);
        const float lambda = kss < p.eps ? p.eps : kss;
        const float beta = sigmoidf_dev(cbr + beta_bias);
        float alpha, kscale = 1.0f;
        if (p.method == 0) { alpha = beta; kscale = rsqrtf(lambda + p.eps); }
        else alpha = -expm1f(-(beta * lambda)) / (lambda + p.eps);

        __syncwarp();
        k_s[lane] = ck0 * kscale; k_s[lane + 32] = ck1 * kscale;
        q_s[lane] = cq0 * q_inv;  q_s[lane + 32] = cq1 * q_inv;
        a_s[lane] = alpha * (ck0 * kscale); a_s[lane + 32] = alpha * (ck1 * kscale);
        __syncwarp();

        // kS for this lane's columns: two packed partial sums per column (even / odd rows twice over)
        float2 acc[NCOL][2];
#pragma unroll
        for (int c = 0; c < NCOL; ++c) acc[c][0] = acc[c][1] = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < HP; j += 2) {
            const float4 kk = *reinterpret_cast<const float4*>(k_s + 2 * j);
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
                acc[c][0] = __ffma2_rn(make_float2(kk.x, kk.y), S[c][j], acc[c][0]);
                acc[c][1] = __ffma2_rn(make_float2(kk.z, kk.w), S[c][j + 1], acc[c][1]);
            }
        }
        float2 diff2[NCOL];
#pragma unroll
        for (int c = 0; c < NCOL; ++c) {
            const float d = cv[c] - ((acc[c][0].x + acc[c][0].y) + (acc[c][1].x + acc[c][1].y));
            diff2[c] = make_float2(d, d);
        }

        // state update (rounded to fp16 every step) fused with the readout of the updated state
        float2 y[NCOL][2];
#pragma unroll
        for (int c = 0; c < NCOL; ++c) y[c][0] = y[c][1] = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int j = 0; j < HP; j += 2) {
            const float4 ak = *reinterpret_cast<const float4*>(a_s + 2 * j);
            const float4 qq = *reinterpret_cast<const float4*>(q_s + 2 * j);
#pragma unroll
            for (int c = 0; c < NCOL; ++c) {
                const float2 s0 = __ffma2_rn(make_float2(ak.x, ak.y), diff2[c], S[c][j]);
                const float2 s1 = __ffma2_rn(make_float2(ak.z, ak.w), diff2[c], S[c][j + 1]);
                const float2 r0 = __half22float2(__floats2half2_rn(s0.x, s0.y));
                const float2 r1 = __half22float2(__floats2half2_rn(s1.x, s1.y));
                S[c][j] = r0;
                S[c][j + 1] = r1;
                y[c][0] = __ffma2_rn(r0, make_float2(qq.x, qq.y), y[c][0]);
                y[c][1] = __ffma2_rn(r1, make_float2(qq.z, qq.w), y[c][1]);
            }
        }
#pragma unroll
        for (int c = 0; c < NCOL; ++c)
            ob[static_cast<size_t>(t) * p.ld_out + colbase + lane + 32 * c] = (y[c][0].x + y[c][0].y) + (y[c][1].x + y[c][1].y);
    }
}

}  // namespace

int g_efla_cols_per_lane = 2;  // host toggle (option "efla_cols_per_lane")

int efla_launch(const EflaParams& p, cudaStream_t stream) {
    if (p.seqs <= 0 || p.T <= 0) return BNF4_OK;
    if (p.heads <= 0 || p.hidden <= 0 || (p.hidden % p.heads) != 0) return set_error(BNF4_ERR_INVALID, "efla: hidden=%d heads=%d", p.hidden, p.heads);
    if (!p.q || !p.k || !p.v || !p.beta_raw || !p.out) return set_error(BNF4_ERR_INVALID, "efla: null pointer");
    const int hd = p.hidden / p.heads;
    if (p.state == nullptr && p.state_fp16 && hd == 64 && !p.force_generic) {
        const long long units = p.seqs * static_cast<long long>(p.heads);
        if (g_efla_cols_per_lane == 2) {
            const long long ctas = (units + kScanWarps - 1) / kScanWarps;
            efla_scan64_kernel<2><<<static_cast<unsigned>(ctas), kScanWarps * 32, 0, stream>>>(p);
        } else {
            const long long ctas = (2 * units + kScanWarps - 1) / kScanWarps;
            efla_scan64_kernel<1><<<static_cast<unsigned>(ctas), kScanWarps * 32, 0, stream>>>(p);
        }
        return check_launch("efla_scan64_kernel");
    }
    if ((hd % 32) != 0) return set_error(BNF4_ERR_INVALID, "efla: head_dim=%d must be a multiple of 32", hd);
    if (p.seqs > 65535) return set_error(BNF4_ERR_INVALID, "efla (generic kernel): at most 65535 sequences per call");
    const int nc = hd >= 64 ? 64 : 32;
    const size_t ssz = p.state_fp16 ? sizeof(__half) : sizeof(float);
    const size_t smem = ssz * hd * nc + sizeof(float) * (2 * hd + 72);
    const dim3 grid(static_cast<unsigned>((hd + nc - 1) / nc), static_cast<unsigned>(p.heads), static_cast<unsigned>(p.seqs));
    if (p.state_fp16) {
        if (smem > 48 * 1024) {
            const int rc = check_cuda(cudaFuncSetAttribute(efla_generic_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)), "cudaFuncSetAttribute(efla)");
            if (rc) return rc;
        }
        efla_generic_kernel<__half><<<grid, nc, smem, stream>>>(p);
    } else {
        if (smem > 48 * 1024) {
            const int rc = check_cuda(cudaFuncSetAttribute(efla_generic_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)), "cudaFuncSetAttribute(efla)");
            if (rc) return rc;
        }
        efla_generic_kernel<float><<<grid, nc, smem, stream>>>(p);
    }
    return check_launch("efla_generic_kernel");
}

}  // namespace bnf4

using namespace bnf4;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

int bnf4_efla_scan(const bnf4_efla_desc* desc, void* stream) {
    if (!desc) return set_error(BNF4_ERR_INVALID, "bnf4_efla_scan: null descriptor");
    return efla_launch(*desc, S(stream));
}

static int efla_step_common(void* state, int state_fp16, const float* q, const float* k, const float* v, const float* beta_raw,
                            int ld_qkv, int ld_beta, float beta_bias, int hidden, int batch, int method, float eps, float* out,
                            void* stream) {
    if (batch <= 0 || hidden <= 0) return BNF4_OK;
    if (!state) return set_error(BNF4_ERR_INVALID, "efla_step: null state");
    bnf4_efla_desc d = {};
    d.state = state; d.state_fp16 = state_fp16;
    d.q = q; d.k = k; d.v = v; d.beta_raw = beta_raw; d.ld_qkv = ld_qkv; d.ld_beta = ld_beta;
    d.beta_bias = beta_bias; d.beta_bias_seq = nullptr; d.seqs_per_bias = 1;
    d.hidden = hidden; d.heads = 1; d.seqs = batch; d.T = 1; d.method = method; d.eps = eps;
    d.out = out; d.ld_out = hidden;
    return efla_launch(d, S(stream));
}

int bnf4_efla_step_half_qkv_fused(void* S_half, const float* qkv, int fused_cols, float beta_bias, int hidden, int batch,
                                  int method, float eps, float* out, void* stream) {
    if (!qkv) return set_error(BNF4_ERR_INVALID, "efla_step_half_qkv_fused: null qkv");
    return efla_step_common(S_half, 1, qkv, qkv + hidden, qkv + 2 * hidden, qkv + 3 * hidden, fused_cols, fused_cols, beta_bias,
                            hidden, batch, method, eps, out, stream);
}

int bnf4_efla_step_qkv_fused(float* S_f32, const float* qkv, int fused_cols, float beta_bias, int hidden, int batch, int method,
                             float eps, float* out, void* stream) {
    if (!qkv) return set_error(BNF4_ERR_INVALID, "efla_step_qkv_fused: null qkv");
    return efla_step_common(S_f32, 0, qkv, qkv + hidden, qkv + 2 * hidden, qkv + 3 * hidden, fused_cols, fused_cols, beta_bias,
                            hidden, batch, method, eps, out, stream);
}

int bnf4_efla_step(void* state, int state_fp16, const float* q, const float* k, const float* v, const float* beta_raw,
                   float beta_bias, int hidden, int batch, int method, float eps, float* out, void* stream) {
    return efla_step_common(state, state_fp16, q, k, v, beta_raw, hidden, 1, beta_bias, hidden, batch, method, eps, out, stream);
}

}  // extern "C"
