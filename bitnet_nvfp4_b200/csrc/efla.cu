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

__global__ void __launch_bounds__(kScanWarps * 32, 2) efla_scan64_kernel(const EflaParams p) {
    constexpr int HD = 64;
    __shared__ __align__(16) float sh[kScanWarps][3][HD];  // k, q^, alpha*k per warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long unit = static_cast<long long>(blockIdx.x) * kScanWarps + warp;  // (sequence, head)
    if (unit >= p.seqs * static_cast<long long>(p.heads)) return;
    const long long seq = unit / p.heads;
    const int h = static_cast<int>(unit - seq * p.heads);
    const float beta_bias = p.beta_bias_seq != nullptr ? p.beta_bias_seq[seq / p.seqs_per_bias] : p.beta_bias;

    float S0[HD], S1[HD];
#pragma unroll
    for (int d = 0; d < HD; ++d) { S0[d] = 0.0f; S1[d] = 0.0f; }

    const size_t row0 = static_cast<size_t>(seq) * p.T;
    const float* qb = p.q + row0 * p.ld_qkv + h * HD;
    const float* kb = p.k + row0 * p.ld_qkv + h * HD;
    const float* vb = p.v + row0 * p.ld_qkv + h * HD;
    const float* bb = p.beta_raw + row0 * p.ld_beta;
    float* ob = p.out + row0 * p.ld_out + h * HD;

    // prefetch token 0
    float q0 = qb[lane], q1 = qb[lane + 32], k0 = kb[lane], k1 = kb[lane + 32], v0 = vb[lane], v1 = vb[lane + 32], br = bb[0];

    float* k_s = sh[warp][0];
    float* q_s = sh[warp][1];
    float* a_s = sh[warp][2];

    for (int t = 0; t < p.T; ++t) {
        const float cq0 = q0, cq1 = q1, ck0 = k0, ck1 = k1, cv0 = v0, cv1 = v1, cbr = br;
        if (t + 1 < p.T) {
            const size_t o = static_cast<size_t>(t + 1) * p.ld_qkv;
            q0 = qb[o + lane]; q1 = qb[o + lane + 32];
            k0 = kb[o + lane]; k1 = kb[o + lane + 32];
            v0 = vb[o + lane]; v1 = vb[o + lane + 32];
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

        // kS for this lane's two columns, four partial sums per column
        float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            const float4 kk = *reinterpret_cast<const float4*>(k_s + d);
            a0[0] = fmaf(kk.x, S0[d], a0[0]); a1[0] = fmaf(kk.x, S1[d], a1[0]);
            a0[1] = fmaf(kk.y, S0[d + 1], a0[1]); a1[1] = fmaf(kk.y, S1[d + 1], a1[1]);
            a0[2] = fmaf(kk.z, S0[d + 2], a0[2]); a1[2] = fmaf(kk.z, S1[d + 2], a1[2]);
            a0[3] = fmaf(kk.w, S0[d + 3], a0[3]); a1[3] = fmaf(kk.w, S1[d + 3], a1[3]);
        }
        const float diff0 = cv0 - ((a0[0] + a0[1]) + (a0[2] + a0[3]));
        const float diff1 = cv1 - ((a1[0] + a1[1]) + (a1[2] + a1[3]));

        // state update (rounded to fp16 every step) fused with the readout of the updated state
        float y0[4] = {0.f, 0.f, 0.f, 0.f}, y1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int d = 0; d < HD; d += 4) {
            const float4 ak = *reinterpret_cast<const float4*>(a_s + d);
            const float4 qq = *reinterpret_cast<const float4*>(q_s + d);
            const float akv[4] = {ak.x, ak.y, ak.z, ak.w};
            const float qv[4] = {qq.x, qq.y, qq.z, qq.w};
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const __half2 hh = __floats2half2_rn(fmaf(akv[u], diff0, S0[d + u]), fmaf(akv[u], diff1, S1[d + u]));
                const float2 ff = __half22float2(hh);
                S0[d + u] = ff.x;
                S1[d + u] = ff.y;
                y0[u] = fmaf(ff.x, qv[u], y0[u]);
                y1[u] = fmaf(ff.y, qv[u], y1[u]);
            }
        }
        ob[static_cast<size_t>(t) * p.ld_out + lane] = (y0[0] + y0[1]) + (y0[2] + y0[3]);
        ob[static_cast<size_t>(t) * p.ld_out + lane + 32] = (y1[0] + y1[1]) + (y1[2] + y1[3]);
    }
}

}  // namespace

int efla_launch(const EflaParams& p, cudaStream_t stream) {
    if (p.seqs <= 0 || p.T <= 0) return BNF4_OK;
    if (p.heads <= 0 || p.hidden <= 0 || (p.hidden % p.heads) != 0) return set_error(BNF4_ERR_INVALID, "efla: hidden=%d heads=%d", p.hidden, p.heads);
    if (!p.q || !p.k || !p.v || !p.beta_raw || !p.out) return set_error(BNF4_ERR_INVALID, "efla: null pointer");
    const int hd = p.hidden / p.heads;
    if (p.state == nullptr && p.state_fp16 && hd == 64 && !p.force_generic) {
        const long long units = p.seqs * static_cast<long long>(p.heads);
        const long long ctas = (units + kScanWarps - 1) / kScanWarps;
        efla_scan64_kernel<<<static_cast<unsigned>(ctas), kScanWarps * 32, 0, stream>>>(p);
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
