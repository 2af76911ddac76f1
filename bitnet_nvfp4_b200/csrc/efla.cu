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


// ------------------------------------------------------------------------------------------------
// Tensor-core form of the scan kernel (head_dim 64, fp16-rounded state, zero initial state).
//
// The state is exactly representable in fp16 (it is rounded to fp16 every token), so it lives in registers ONLY as
// packed halves, laid out as the A fragments of mma.sync.m16n8k16 with A[n][d] = S[d,n]. Per token and per 16 x 16
// tile of the state:
//   1. update:   S32 = S16 * I + (alpha k) diff^T      two m16n8k8 MMAs against an 8 x 8 identity; the rank-1 term,
//                computed with packed fp32 multiplies, enters as the fp32 accumulator C, so the tensor core performs the
//                fp16 -> fp32 widening and the addition in one step;
//   2. rounding: S16' = fp16_rn(S32)                   packed conversions, which directly produce the next A fragment;
//   3. readout:  D += S16' * B                          one m16n8k16 MMA with B[d][j] = { q^ hi, q^ mid 2^11, k' hi,
//                k' mid 2^11, 0, 0, 0, 0 }: columns 0-1 give y_t = S'^T q^_t, columns 2-3 give k'.S' of the NEXT token.
// x = hi + mid is the two-term fp16 split of an fp32 value (hi = fp16(x), mid = fp16((x - hi) 2^11) / 2^11, error
// <= 2^-24 |x|), so every product is exact in fp32. Compared with the multiply-add kernels the deviations are the
// order/rounding of fp32 accumulation inside the tensor core and one extra fp32 rounding of (alpha k)*diff before
// the addition; both are far below the fp16 rounding of the state that follows.
//
// Fragment coordinates (g = lane / 4, tq = lane % 4): for n-tile mt and d-tile ks the lane holds S[d][n] for
// n = 16 mt + g + {0, 8} and d = 16 ks + 2 tq + {0, 1, 8, 9}.
// ------------------------------------------------------------------------------------------------
// Shared-memory order of a 64-vector ("permuted"): element d sits at ((d % 8) / 2) * 16 + (d / 16) * 4 + (d % 2) + 2 * ((d / 8) % 2),
// so that the 16 values a lane needs (d = 16 ks + 2 tq + {0, 1, 8, 9}, ks = 0..3) are contiguous at tq * 16.

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// d = a (16 x 16) * b (16 x 8): no accumulator input
__device__ __forceinline__ void mma_f16_16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%10, %10, %10, %10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// d (in place) += a (16 x 8) * b (8 x 8)
__device__ __forceinline__ void mma_f16_1688(float& d0, float& d1, float& d2, float& d3, uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5}, {%6}, {%0, %1, %2, %3};"
        : "+f"(d0), "+f"(d1), "+f"(d2), "+f"(d3)
        : "r"(a0), "r"(a1), "r"(b0));
}
// c (16 x 8, fp16, in place) += a (16 x 8) * b (8 x 8): fp16 accumulators, one rounding to nearest of the exact sum
__device__ __forceinline__ void mma_f16acc_1688(uint32_t& c0, uint32_t& c1, uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k8.row.col.f16.f16.f16.f16 {%0, %1}, {%2, %3}, {%4}, {%0, %1};" : "+r"(c0), "+r"(c1) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 hv = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&hv);
}

constexpr int kScanRing = 12;                // ring of raw q/k/v/beta per warp: three groups of four tokens
constexpr int kScanSlotFloats = 3 * 64 + 4;  // q[64], k[64], v[64], beta (+ padding to 16 bytes)
constexpr int kScanVecBufs = 8;              // prepared vectors per warp: two groups of four tokens
constexpr int kScanMmaCtasPerSm = 3;
// dynamic shared memory per warp: ring, alpha*k (fp32), and the four fp16 columns q^ hi, q^ mid, k hi, k mid
constexpr int kScanWarpSmemBytes = kScanRing * kScanSlotFloats * 4 + kScanVecBufs * 64 * 4 + kScanVecBufs * 4 * 64 * 2;
constexpr int kScanMmaSmemBytes = kScanWarps * kScanWarpSmemBytes;
constexpr int kScan2CtasPerSm = 4;
constexpr int kScan2QkRing = 8;                // q, k, beta of two groups of four tokens
constexpr int kScan2QkSlotFloats = 2 * 64 + 4;  // q[64], k[64], beta (+ padding to 16 bytes)
// per warp: q/k ring, v ring, (hi, mid) words of alpha * k, the four fp16 columns q^ hi, q^ mid, k hi, k mid, eight zero words
constexpr int kScan2WarpSmemBytes = kScan2QkRing * kScan2QkSlotFloats * 4 + kScanRing * 64 * 4 + kScanVecBufs * 64 * 4 + kScanVecBufs * 4 * 64 * 2 + 32;
constexpr int kScan2SmemBytes = kScanWarps * kScan2WarpSmemBytes;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(kScanWarps * 32, kScanMmaCtasPerSm) efla_scan64_mma_kernel(const EflaParams p) {
    constexpr int HD = 64;
    extern __shared__ __align__(16) uint8_t scan_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float* in_sh = reinterpret_cast<float*>(scan_smem + warp * kScanWarpSmemBytes);  // [kScanRing][kScanSlotFloats]
    float* a_sh = in_sh + kScanRing * kScanSlotFloats;                               // [kScanVecBufs][64]   alpha * k, permuted
    __half* b_sh = reinterpret_cast<__half*>(a_sh + kScanVecBufs * HD);              // [kScanVecBufs][4][64] q^ hi, q^ mid, k hi, k mid, permuted
    const long long unit = static_cast<long long>(blockIdx.x) * kScanWarps + warp;  // (sequence, head)
    if (unit >= p.seqs * static_cast<long long>(p.heads)) return;
    const long long seq = unit / p.heads;
    const int h = static_cast<int>(unit - seq * p.heads);
    const float beta_bias = p.beta_bias_seq != nullptr ? p.beta_bias_seq[seq / p.seqs_per_bias] : p.beta_bias;
    const int g = lane >> 2, tq = lane & 3;

    uint32_t Sh[4][4][4];  // [mt][ks][i]: the A fragment (i = 0: n = g, d pair 2tq; 1: n = g + 8; 2: n = g, d pair 2tq + 8; 3: n = g + 8)
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) Sh[mt][ks][i] = 0u;
    // 8 x 8 identity as a B fragment: this lane holds rows 2tq, 2tq + 1 of column g
    const uint32_t ident = pack_half2(2 * tq == g ? 1.0f : 0.0f, 2 * tq + 1 == g ? 1.0f : 0.0f);

    const size_t row0 = static_cast<size_t>(seq) * p.T;
    const float* qb = p.q + row0 * p.ld_qkv + h * HD;
    const float* kb = p.k + row0 * p.ld_qkv + h * HD;
    const float* vb = p.v + row0 * p.ld_qkv + h * HD;
    const float* bb = p.beta_raw + row0 * p.ld_beta;
    float* ob = p.out + row0 * p.ld_out + h * HD;

    // asynchronous copy of four tokens' inputs (one group) into their ring slots; every lane commits one group, empty or not
    auto issue_group = [&](int tok0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int tok = tok0 + j;
            if (tok < p.T) {
                float* slot = in_sh + (tok % kScanRing) * kScanSlotFloats;
                const size_t o = static_cast<size_t>(tok) * p.ld_qkv;
                const int l16 = lane & 15;
                cp_async16(slot + (lane < 16 ? 0 : HD) + 4 * l16, (lane < 16 ? qb : kb) + o + 4 * l16);
                if (lane < 16) cp_async16(slot + 2 * HD + 4 * l16, vb + o + 4 * l16);
                else if (lane == 16) cp_async4(slot + 3 * HD, bb + static_cast<size_t>(tok) * p.ld_beta);
            }
        }
        cp_async_commit();
    };

    // Per-token vectors, four tokens at a time: lanes 8 j .. 8 j + 7 prepare token tok0 + j, eight elements each
    // (d = 8 l + e), so the reductions are three shuffle levels deep and the scalar chain (sigmoid, expm1, divisions)
    // runs once per four tokens. The permuted layout puts the element pairs (d, d + 1) next to each other, so the
    // packed fp16 conversions are stored as they are.
    const int pj = lane >> 3, pl = lane & 7;
    auto prepare4 = [&](int tok0) {
        const int tok = min(tok0 + pj, p.T - 1);  // past the end: the last token again (never used)
        const float* slot = in_sh + (tok % kScanRing) * kScanSlotFloats;
        const int buf = (tok0 + pj) % kScanVecBufs;
        const float4 qa = *reinterpret_cast<const float4*>(slot + 8 * pl), qc = *reinterpret_cast<const float4*>(slot + 8 * pl + 4);
        const float4 ka = *reinterpret_cast<const float4*>(slot + HD + 8 * pl), kc = *reinterpret_cast<const float4*>(slot + HD + 8 * pl + 4);
        const float rbr = slot[3 * HD];
        const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qc.x, qc.y, qc.z, qc.w};
        const float kv[8] = {ka.x, ka.y, ka.z, ka.w, kc.x, kc.y, kc.z, kc.w};
        float qss = 0.0f, kss = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) { qss = fmaf(qv[e], qv[e], qss); kss = fmaf(kv[e], kv[e], kss); }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            qss += __shfl_xor_sync(0xffffffffu, qss, o);
            kss += __shfl_xor_sync(0xffffffffu, kss, o);
        }
        const float q_inv = rsqrtf(qss + p.eps);
        const float lambda = kss < p.eps ? p.eps : kss;
        const float beta = sigmoidf_dev(rbr + beta_bias);
        float alpha, kscale = 1.0f;
        if (p.method == 0) { alpha = beta; kscale = rsqrtf(lambda + p.eps); }
        else alpha = -expm1f(-(beta * lambda)) / (lambda + p.eps);
        // element d = 8 pl + e sits at (e / 2) * 16 + (pl / 2) * 4 + (e % 2) + 2 * (pl % 2) of the permuted order
        const int pbase = (pl >> 1) * 4 + 2 * (pl & 1);
        float* a_dst = a_sh + buf * HD + pbase;
        __half* b_dst = b_sh + buf * 4 * HD + pbase;
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
            const float kn0 = kv[2 * e2] * kscale, kn1 = kv[2 * e2 + 1] * kscale, qn0 = qv[2 * e2] * q_inv, qn1 = qv[2 * e2 + 1] * q_inv;
            *reinterpret_cast<float2*>(a_dst + 16 * e2) = make_float2(alpha * kn0, alpha * kn1);
            // two-term fp16 splits with packed conversions
            const __half2 qh = __floats2half2_rn(qn0, qn1), kh = __floats2half2_rn(kn0, kn1);
            const float2 qhf = __half22float2(qh), khf = __half22float2(kh);
            const __half2 qm = __floats2half2_rn((qn0 - qhf.x) * 2048.0f, (qn1 - qhf.y) * 2048.0f);
            const __half2 km = __floats2half2_rn((kn0 - khf.x) * 2048.0f, (kn1 - khf.y) * 2048.0f);
            *reinterpret_cast<__half2*>(b_dst + 0 * HD + 16 * e2) = qh;
            *reinterpret_cast<__half2*>(b_dst + 1 * HD + 16 * e2) = qm;
            *reinterpret_cast<__half2*>(b_dst + 2 * HD + 16 * e2) = kh;
            *reinterpret_cast<__half2*>(b_dst + 3 * HD + 16 * e2) = km;
        }
    };

    float kS[4][2];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) kS[mt][0] = kS[mt][1] = 0.0f;  // zero initial state
    issue_group(0);
    issue_group(4);
    cp_async_wait<0>();
    __syncwarp();
    prepare4(0);

    int rg = 0;  // ring group (four slots) that holds tokens t0 .. t0 + 3
    for (int t0 = 0; t0 < p.T; t0 += 4) {
        const int gb = (t0 >> 2) & 1;  // vector buffers gb * 4 .. gb * 4 + 3 hold tokens t0 .. t0 + 3
        {
            // start of a group of four tokens: fetch the group after next, prepare the next one
            __syncwarp();  // everyone is done with the ring slots and vector buffers of the previous group
            issue_group(t0 + 8);
            cp_async_wait<1>();  // everything but the newest group has landed: tokens <= t0 + 7
            __syncwarp();
            prepare4(t0 + 4);
            __syncwarp();
        }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = t0 + j;
        if (t >= p.T) break;
        const int cur = gb * 4 + j, nxt = j < 3 ? cur + 1 : (gb ^ 1) * 4;
        const float* vslot = in_sh + (rg * 4 + j) * kScanSlotFloats + 2 * HD;
        float2 diff2[4][2];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt)
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const float d = vslot[16 * mt + 8 * hh + g] - kS[mt][hh];
                diff2[mt][hh] = make_float2(d, d);
            }

        // per d-tile operands: alpha*k pairs (update) and the B fragment: columns 0,1 = q^ of token t, 2,3 = k of token t+1
        const float* a_src = a_sh + cur * HD + tq * 16;
        const __half* b_src = b_sh + ((g < 2 ? cur : nxt) * 4 + (g & 3)) * HD + tq * 16;
        float D[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) D[mt][0] = D[mt][1] = D[mt][2] = D[mt][3] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const float4 av = *reinterpret_cast<const float4*>(a_src + ks * 4);
            uint2 bf = *reinterpret_cast<const uint2*>(b_src + ks * 4);
            if (g >= 4) bf = make_uint2(0u, 0u);
            const float2 alo = make_float2(av.x, av.y), ahi = make_float2(av.z, av.w);
            // the four n-tiles are independent: issue each stage for all of them so that MMA latency overlaps
            float cs[4][8];
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                // rank-1 term for the lane's elements: (d pair) x (n = g, g + 8)
                const float2 c0 = __fmul2_rn(alo, diff2[mt][0]), c1 = __fmul2_rn(alo, diff2[mt][1]);
                const float2 c2 = __fmul2_rn(ahi, diff2[mt][0]), c3 = __fmul2_rn(ahi, diff2[mt][1]);
                cs[mt][0] = c0.x; cs[mt][1] = c0.y; cs[mt][2] = c1.x; cs[mt][3] = c1.y;
                cs[mt][4] = c2.x; cs[mt][5] = c2.y; cs[mt][6] = c3.x; cs[mt][7] = c3.y;
            }
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                mma_f16_1688(cs[mt][0], cs[mt][1], cs[mt][2], cs[mt][3], Sh[mt][ks][0], Sh[mt][ks][1], ident);  // d pair 2tq
                mma_f16_1688(cs[mt][4], cs[mt][5], cs[mt][6], cs[mt][7], Sh[mt][ks][2], Sh[mt][ks][3], ident);  // d pair 2tq + 8
            }
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                Sh[mt][ks][0] = pack_half2(cs[mt][0], cs[mt][1]);  // the state is rounded to fp16 every token
                Sh[mt][ks][1] = pack_half2(cs[mt][2], cs[mt][3]);
                Sh[mt][ks][2] = pack_half2(cs[mt][4], cs[mt][5]);
                Sh[mt][ks][3] = pack_half2(cs[mt][6], cs[mt][7]);
            }
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
                mma_f16_16816(D[mt], Sh[mt][ks][0], Sh[mt][ks][1], Sh[mt][ks][2], Sh[mt][ks][3], bf.x, bf.y);
        }

        // column pair of this lane: tq = 0 -> (q^ hi, q^ mid): y of token t;  tq = 1 -> (k hi, k mid): k.S of token t + 1
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            const float r0 = fmaf(D[mt][1], 1.0f / 2048.0f, D[mt][0]);  // n = 16 mt + g
            const float r1 = fmaf(D[mt][3], 1.0f / 2048.0f, D[mt][2]);  // n = 16 mt + g + 8
            if (tq == 0) {
                ob[static_cast<size_t>(t) * p.ld_out + 16 * mt + g] = r0;
                ob[static_cast<size_t>(t) * p.ld_out + 16 * mt + 8 + g] = r1;
            }
            kS[mt][0] = __shfl_sync(0xffffffffu, r0, (lane & ~3) | 1);
            kS[mt][1] = __shfl_sync(0xffffffffu, r1, (lane & ~3) | 1);
        }
      }
        rg = rg == 2 ? 0 : rg + 1;
    }
    cp_async_wait<0>();
}

__global__ void __launch_bounds__(kScanWarps * 32, kScan2CtasPerSm) efla_scan64_mma2_kernel(const EflaParams p) {
    constexpr int HD = 64;
    extern __shared__ __align__(16) uint8_t scan_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // raw inputs: q, k, beta are dead once their group of four tokens has been prepared (two groups in the ring: one being
    // prepared, one in flight); v is read token by token one group later (three groups)
    float* qk_sh = reinterpret_cast<float*>(scan_smem + warp * kScan2WarpSmemBytes);   // [kScan2QkRing][kScan2QkSlotFloats]
    float* v_sh = qk_sh + kScan2QkRing * kScan2QkSlotFloats;                            // [kScanRing][64]
    uint32_t* kw_sh = reinterpret_cast<uint32_t*>(v_sh + kScanRing * HD);               // [kScanVecBufs][64] (hi, mid) halves of alpha * k; d at (d % 8) * 8 + d / 8
    __half* b_sh = reinterpret_cast<__half*>(kw_sh + kScanVecBufs * HD);                  // [kScanVecBufs][4][64] q^ hi, q^ mid, k hi, k mid, permuted
    uint32_t* zero_sh = reinterpret_cast<uint32_t*>(b_sh + kScanVecBufs * 4 * HD);        // [8] zeros: the alpha * k words of lanes whose rows of B are zero
    if (lane < 8) zero_sh[lane] = 0u;
    const long long unit = static_cast<long long>(blockIdx.x) * kScanWarps + warp;  // (sequence, head)
    if (unit >= p.seqs * static_cast<long long>(p.heads)) return;
    const long long seq = unit / p.heads;
    const int h = static_cast<int>(unit - seq * p.heads);
    const float beta_bias = p.beta_bias_seq != nullptr ? p.beta_bias_seq[seq / p.seqs_per_bias] : p.beta_bias;
    const int g = lane >> 2, tq = lane & 3;

    uint32_t Sh[4][4][4];  // [mt][ks][i]: the A fragment (i = 0: n = g, d pair 2tq; 1: n = g + 8; 2: n = g, d pair 2tq + 8; 3: n = g + 8)
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) Sh[mt][ks][i] = 0u;

    const size_t row0 = static_cast<size_t>(seq) * p.T;
    const float* qb = p.q + row0 * p.ld_qkv + h * HD;
    const float* kb = p.k + row0 * p.ld_qkv + h * HD;
    const float* vb = p.v + row0 * p.ld_qkv + h * HD;
    const float* bb = p.beta_raw + row0 * p.ld_beta;
    float* ob = p.out + row0 * p.ld_out + h * HD;

    // asynchronous copy of four tokens' inputs (one group) into their ring slots; every lane commits one group, empty or not
    auto issue_group = [&](int tok0) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int tok = tok0 + j;
            if (tok < p.T) {
                float* slot = qk_sh + (tok % kScan2QkRing) * kScan2QkSlotFloats;
                const size_t o = static_cast<size_t>(tok) * p.ld_qkv;
                const int l16 = lane & 15;
                cp_async16(slot + (lane < 16 ? 0 : HD) + 4 * l16, (lane < 16 ? qb : kb) + o + 4 * l16);
                if (lane < 16) cp_async16(v_sh + (tok % kScanRing) * HD + 4 * l16, vb + o + 4 * l16);
                else if (lane == 16) cp_async4(slot + 2 * HD, bb + static_cast<size_t>(tok) * p.ld_beta);
            }
        }
        cp_async_commit();
    };

    // Per-token vectors, four tokens at a time: lanes 8 j .. 8 j + 7 prepare token tok0 + j, eight elements each
    // (d = 8 l + e), so the reductions are three shuffle levels deep and the scalar chain (sigmoid, expm1, divisions)
    // runs once per four tokens. The permuted layout puts the element pairs (d, d + 1) next to each other, so the
    // packed fp16 conversions are stored as they are.
    const int pj = lane >> 3, pl = lane & 7;
    auto prepare4 = [&](int tok0) {
        const int tok = min(tok0 + pj, p.T - 1);  // past the end: the last token again (never used)
        const float* slot = qk_sh + (tok % kScan2QkRing) * kScan2QkSlotFloats;
        const int buf = (tok0 + pj) % kScanVecBufs;
        const float4 qa = *reinterpret_cast<const float4*>(slot + 8 * pl), qc = *reinterpret_cast<const float4*>(slot + 8 * pl + 4);
        const float4 ka = *reinterpret_cast<const float4*>(slot + HD + 8 * pl), kc = *reinterpret_cast<const float4*>(slot + HD + 8 * pl + 4);
        const float rbr = slot[2 * HD];
        const float qv[8] = {qa.x, qa.y, qa.z, qa.w, qc.x, qc.y, qc.z, qc.w};
        const float kv[8] = {ka.x, ka.y, ka.z, ka.w, kc.x, kc.y, kc.z, kc.w};
        float qss = 0.0f, kss = 0.0f;
#pragma unroll
        for (int e = 0; e < 8; ++e) { qss = fmaf(qv[e], qv[e], qss); kss = fmaf(kv[e], kv[e], kss); }
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) {
            qss += __shfl_xor_sync(0xffffffffu, qss, o);
            kss += __shfl_xor_sync(0xffffffffu, kss, o);
        }
        const float q_inv = rsqrtf(qss + p.eps);
        const float lambda = kss < p.eps ? p.eps : kss;
        const float beta = sigmoidf_dev(rbr + beta_bias);
        float alpha, kscale = 1.0f;
        if (p.method == 0) { alpha = beta; kscale = rsqrtf(lambda + p.eps); }
        else alpha = -expm1f(-(beta * lambda)) / (lambda + p.eps);
        // element d = 8 pl + e sits at (e / 2) * 16 + (pl / 2) * 4 + (e % 2) + 2 * (pl % 2) of the permuted order
        const int pbase = (pl >> 1) * 4 + 2 * (pl & 1);
        uint32_t* kw_dst = kw_sh + buf * HD + pl;
        __half* b_dst = b_sh + buf * 4 * HD + pbase;
#pragma unroll
        for (int e2 = 0; e2 < 4; ++e2) {
            const float kn0 = kv[2 * e2] * kscale, kn1 = kv[2 * e2 + 1] * kscale, qn0 = qv[2 * e2] * q_inv, qn1 = qv[2 * e2 + 1] * q_inv;
            {   // alpha * k as unscaled (hi, mid) halves, one word per element
                const float ak0 = alpha * kn0, ak1 = alpha * kn1;
                const __half2 ah = __floats2half2_rn(ak0, ak1);
                const float2 ahf = __half22float2(ah);
                const __half2 am = __floats2half2_rn(ak0 - ahf.x, ak1 - ahf.y);
                kw_dst[(2 * e2) * 8] = __byte_perm(*reinterpret_cast<const uint32_t*>(&ah), *reinterpret_cast<const uint32_t*>(&am), 0x5410);
                kw_dst[(2 * e2 + 1) * 8] = __byte_perm(*reinterpret_cast<const uint32_t*>(&ah), *reinterpret_cast<const uint32_t*>(&am), 0x7632);
            }
            // two-term fp16 splits with packed conversions
            const __half2 qh = __floats2half2_rn(qn0, qn1), kh = __floats2half2_rn(kn0, kn1);
            const float2 qhf = __half22float2(qh), khf = __half22float2(kh);
            const __half2 qm = __floats2half2_rn((qn0 - qhf.x) * 2048.0f, (qn1 - qhf.y) * 2048.0f);
            const __half2 km = __floats2half2_rn((kn0 - khf.x) * 2048.0f, (kn1 - khf.y) * 2048.0f);
            *reinterpret_cast<__half2*>(b_dst + 0 * HD + 16 * e2) = qh;
            *reinterpret_cast<__half2*>(b_dst + 1 * HD + 16 * e2) = qm;
            *reinterpret_cast<__half2*>(b_dst + 2 * HD + 16 * e2) = kh;
            *reinterpret_cast<__half2*>(b_dst + 3 * HD + 16 * e2) = km;
        }
    };

    float kS[4][2];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt) kS[mt][0] = kS[mt][1] = 0.0f;  // zero initial state
    issue_group(0);
    issue_group(4);
    cp_async_wait<0>();
    __syncwarp();
    prepare4(0);

    float* orow = ob + g;  // this lane's output columns of the current token
    int rg = 0;  // ring group (four slots) that holds tokens t0 .. t0 + 3
    for (int t0 = 0; t0 < p.T; t0 += 4) {
        const int gb = (t0 >> 2) & 1;  // vector buffers gb * 4 .. gb * 4 + 3 hold tokens t0 .. t0 + 3
        {
            // start of a group of four tokens: fetch the group after next, prepare the next one
            __syncwarp();  // everyone is done with the ring slots and vector buffers of the previous group
            issue_group(t0 + 8);
            cp_async_wait<1>();  // everything but the newest group has landed: tokens <= t0 + 7
            __syncwarp();
            prepare4(t0 + 4);
            __syncwarp();
        }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int t = t0 + j;
        if (t >= p.T) break;
        const int cur = gb * 4 + j, nxt = j < 3 ? cur + 1 : (gb ^ 1) * 4;
        const float* vslot = v_sh + (rg * 4 + j) * HD;
        // A operand of the update for rows n = g, g + 8 of every n-tile: lanes tq = 1 hold diff hi (columns 2, 3), lanes tq = 2
        // diff mid (columns 4, 5), where hi = diff with the mantissa cut to 11 bits and mid = diff - hi (exact in fp32, then
        // rounded to fp16: diff = hi + mid to 2^-21). Lanes tq = 0 and 3 hold finite values that meet zero rows of B. The
        // k.S of this token sits in the lane's own readout columns (2 tq, 2 tq + 1 hold k hi, k mid for tq >= 1).
        uint32_t da[4][2];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            const float d0 = vslot[16 * mt + g] - kS[mt][0], d1 = vslot[16 * mt + 8 + g] - kS[mt][1];
            const float h0 = __uint_as_float(__float_as_uint(d0) & 0xffffe000u), h1 = __uint_as_float(__float_as_uint(d1) & 0xffffe000u);
            const float x0 = tq == 1 ? h0 : d0 - h0, x1 = tq == 1 ? h1 : d1 - h1;
            da[mt][0] = pack_half2(x0, x0);
            da[mt][1] = pack_half2(x1, x1);
        }
        // B operand of the update for d = 8 j + g (j = 2 ks + half): rows (2, 3) and (4, 5) = (hi, mid) of alpha * k[d]
        const uint32_t* kw_src = (tq == 1 || tq == 2) ? kw_sh + cur * HD + g * 8 : zero_sh;
        const uint4 kwa = *reinterpret_cast<const uint4*>(kw_src), kwb = *reinterpret_cast<const uint4*>(kw_src + 4);
        const uint32_t kw[8] = {kwa.x, kwa.y, kwa.z, kwa.w, kwb.x, kwb.y, kwb.z, kwb.w};
        // B fragment of the readout: columns 0,1 = q^ (hi, mid) of token t; 2,3 = 4,5 = 6,7 = k (hi, mid) of token t + 1, so that
        // lanes tq >= 1 find k.S of the next token in their own accumulator columns
        const __half* b_src = b_sh + (g < 2 ? cur * 4 + g : nxt * 4 + 2 + (g & 1)) * HD + tq * 16;
        // update with fp16 accumulators: S16' = fp16_rn(S16 + diff (alpha k)^T), the state registers are both C and D. n-tile by
        // n-tile, so that the first MMAs of a token need only the first n-tile's diff
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                mma_f16acc_1688(Sh[mt][ks][0], Sh[mt][ks][1], da[mt][0], da[mt][1], kw[2 * ks]);
                mma_f16acc_1688(Sh[mt][ks][2], Sh[mt][ks][3], da[mt][0], da[mt][1], kw[2 * ks + 1]);
            }
        }
        // readout, d-tile by d-tile: the four n-tiles' accumulation chains interleave and finish in n-tile order
        float D[4][4];
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            const uint2 bf = *reinterpret_cast<const uint2*>(b_src + ks * 4);
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                if (ks == 0) mma_f16_16816_zero(D[mt], Sh[mt][ks][0], Sh[mt][ks][1], Sh[mt][ks][2], Sh[mt][ks][3], bf.x, bf.y);
                else mma_f16_16816(D[mt], Sh[mt][ks][0], Sh[mt][ks][1], Sh[mt][ks][2], Sh[mt][ks][3], bf.x, bf.y);
            }
        }

        // column pair of this lane: tq = 0 -> (q^ hi, q^ mid): y of token t;  tq >= 1 -> (k hi, k mid): k.S of token t + 1
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            kS[mt][0] = fmaf(D[mt][1], 1.0f / 2048.0f, D[mt][0]);  // n = 16 mt + g
            kS[mt][1] = fmaf(D[mt][3], 1.0f / 2048.0f, D[mt][2]);  // n = 16 mt + g + 8
            if (tq == 0) {
                orow[16 * mt] = kS[mt][0];
                orow[16 * mt + 8] = kS[mt][1];
            }
        }
        orow += p.ld_out;
      }
        rg = rg == 2 ? 0 : rg + 1;
    }
    cp_async_wait<0>();
}

}  // namespace

int g_efla_cols_per_lane = 2;  // host toggle (option "efla_cols_per_lane")
int g_efla_mma = 2;            // host toggle (option "efla_mma"): 2 = tensor-core scan kernel with fp16 accumulators (default),
                               // 1 = tensor-core scan kernel with the fp32 rank-1 term, 0 = multiply-add scan kernel

int efla_launch(const EflaParams& p, cudaStream_t stream) {
    if (p.seqs <= 0 || p.T <= 0) return BNF4_OK;
    if (p.heads <= 0 || p.hidden <= 0 || (p.hidden % p.heads) != 0) return set_error(BNF4_ERR_INVALID, "efla: hidden=%d heads=%d", p.hidden, p.heads);
    if (!p.q || !p.k || !p.v || !p.beta_raw || !p.out) return set_error(BNF4_ERR_INVALID, "efla: null pointer");
    const int hd = p.hidden / p.heads;
    if (p.state == nullptr && p.state_fp16 && hd == 64 && !p.force_generic) {
        const long long units = p.seqs * static_cast<long long>(p.heads);
        const bool aligned = ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15) == 0 &&
                             (p.ld_qkv % 4) == 0;  // 16-byte asynchronous copies of q, k, v
        if (g_efla_mma >= 2 && aligned) {
            const long long ctas = (units + kScanWarps - 1) / kScanWarps;
            static bool configured2[64] = {};
            int dev = 0;
            int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
            if (rc) return rc;
            if (dev < 0 || dev >= 64 || !configured2[dev]) {
                rc = check_cuda(cudaFuncSetAttribute(efla_scan64_mma2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScan2SmemBytes), "cudaFuncSetAttribute(efla_scan64_mma2_kernel)");
                if (rc) return rc;
                if (dev >= 0 && dev < 64) configured2[dev] = true;
            }
            efla_scan64_mma2_kernel<<<static_cast<unsigned>(ctas), kScanWarps * 32, kScan2SmemBytes, stream>>>(p);
            return check_launch("efla_scan64_mma2_kernel");
        }
        if (g_efla_mma && aligned) {
            const long long ctas = (units + kScanWarps - 1) / kScanWarps;
            // function attributes are per device: set once for each device this process uses
            static bool configured[64] = {};
            int dev = 0;
            int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
            if (rc) return rc;
            if (dev < 0 || dev >= 64 || !configured[dev]) {
                rc = check_cuda(cudaFuncSetAttribute(efla_scan64_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScanMmaSmemBytes), "cudaFuncSetAttribute(efla_scan64_mma_kernel)");
                if (rc) return rc;
                if (dev >= 0 && dev < 64) configured[dev] = true;
            }
            efla_scan64_mma_kernel<<<static_cast<unsigned>(ctas), kScanWarps * 32, kScanMmaSmemBytes, stream>>>(p);
            return check_launch("efla_scan64_mma_kernel");
        }
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
