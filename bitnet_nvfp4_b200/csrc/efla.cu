// EFLA / DeltaNet recurrent linear-attention kernels.
//
// Per row (one sequence position) and per head (reference math: src/efla_lm_kernels.cu:590-726, split form
// :821-913 prepare, :1108-1141 kS, :1186-1197 diff, :1328-1356 update, :1563-1590 readout):
//   q^ = q * rsqrt(sum q^2 + eps);  lambda = max(sum k^2, eps);  beta = sigmoid(beta_raw + beta_bias)
//   alpha = -expm1(-beta*lambda) / (lambda + eps)            (EFLA; DeltaNet: alpha = beta, k <- k*rsqrt(lambda+eps))
//   kS[n] = sum_d k[d] S[d,n];  diff = v - kS;  S[d,n] <- fp16_rn(S[d,n] + alpha k[d] diff[n]);  y[n] = sum_d S[d,n] q^[d]
// The reference keeps S (hidden x hidden, fp16) in HBM and streams it four times per token through six
// kernels. Columns of S are independent, so here the state never leaves the SM:
//   * scan kernel, head_dim 64: one warp owns one (sequence, head); the 64x64 state lives in registers as
//     tensor-core fragments for all T tokens; q/k/v of later tokens arrive through asynchronous copies while
//     the current one is processed. HBM traffic is the algorithmic minimum: read q,k,v,beta, write y.
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
        const float* qr = static_cast<const float*>(p.q) + row * p.ld_qkv + h * hd;
        const float* kr = static_cast<const float*>(p.k) + row * p.ld_qkv + h * hd;
        const float* vr = static_cast<const float*>(p.v) + row * p.ld_qkv + h * hd;
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
            static_cast<float*>(p.out)[row * p.ld_out + h * hd + n] = y;
        }
    }
    if (Sg != nullptr && col_ok)
        for (int d = 0; d < hd; ++d) Sg[static_cast<size_t>(d) * hd + n] = S[d * nc + j];
}

constexpr int kScanWarps = 4;

// ------------------------------------------------------------------------------------------------
// Scan kernel for head_dim 64 (fp16-rounded state, zero initial state): one warp owns one (sequence, head) for all T
// tokens.
//
// The state is exactly representable in fp16 (it is rounded to fp16 every token), so it lives in registers ONLY as
// packed halves, laid out as the A fragments of mma.sync.m16n8k16 with A[n][d] = S[d,n] -- which are at the same time
// the C/D fragments of two m16n8k8 MMAs with fp16 accumulators. Per token and per 16 x 16 tile of the state:
//   1. update:   S16' = fp16_rn(S16 + diff (alpha k)^T)   two m16n8k8.f16.f16.f16.f16 MMAs whose accumulator registers
//                are the state: A holds diff split into fp16 (hi, mid) over four K columns, B the (hi, mid) halves of
//                alpha k, so the tensor core forms the exact partial products, adds the state and rounds once;
//   2. readout:  D += S16' * B                             one m16n8k16 MMA (fp32 accumulators) with B[d][j] = { q^ hi,
//                q^ mid 2^11, 3 x (k' hi, k' mid 2^11) }: columns 0-1 give y_t = S'^T q^_t, the others k'.S' of the NEXT
//                token in every other lane's own columns.
// x = hi + mid is the two-term fp16 split of an fp32 value (hi = fp16(x), mid = fp16((x - hi) 2^11) / 2^11, error
// <= 2^-24 |x|), so every product is exact in fp32.
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
// c (16 x 8, fp16, in place) += a (16 x 8) * b (8 x 8): fp16 accumulators, one rounding to nearest of the exact sum
__device__ __forceinline__ void mma_f16acc_1688(uint32_t& c0, uint32_t& c1, uint32_t a0, uint32_t a1, uint32_t b0) {
    asm("mma.sync.aligned.m16n8k8.row.col.f16.f16.f16.f16 {%0, %1}, {%2, %3}, {%4}, {%0, %1};" : "+r"(c0), "+r"(c1) : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 hv = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&hv);
}

constexpr int kScanRing = 12;                // ring of raw v per warp: three groups of four tokens
constexpr int kScanVecBufs = 8;              // prepared vectors per warp: two groups of four tokens
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
    const float* qb = static_cast<const float*>(p.q) + row0 * p.ld_qkv + h * HD;
    const float* kb = static_cast<const float*>(p.k) + row0 * p.ld_qkv + h * HD;
    const float* vb = static_cast<const float*>(p.v) + row0 * p.ld_qkv + h * HD;
    const float* bb = p.beta_raw + row0 * p.ld_beta;
    float* ob = static_cast<float*>(p.out) + row0 * p.ld_out + h * HD;

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


// ------------------------------------------------------------------------------------------------
// Chunked scan kernel for head_dim 64 (zero initial state): the delta rule of 16 tokens at a time as dense tensor-core
// contractions (the WY / UT-transform form). With S0 the state at the start of a chunk, K, Q^, V the chunk's rows
// (16 x 64), a_s = alpha_s:
//     W  = V - K S0                        (16 x 64)   the tokens' v - k.S against the chunk's initial state
//     L[t,s] = a_s (k_t . k_s), s < t      (16 x 16)   how token s's update changes token t's k.S
//     U  = (I + L)^-1 W                                 the tokens' true "diff" rows u_t = v_t - k_t.S_{t-1}
//     Y  = Q^ S0 + P U,  P[t,s] = a_s (q^_t . k_s), s <= t      the readouts y_t = S_t^T q^_t
//     S' = S0 + (a K)^T U                               the state after the chunk
// This is the same recurrence as the per-token form (src/efla_lm_kernels.cu:590-726) in exact arithmetic. What differs
// is rounding: the state is rounded to fp16 at the end of every chunk instead of after every token, and the operands of
// the contractions are fp16 with fp32 accumulation. Against the per-token form the outputs move by about 1.5e-3 of
// max |y| -- the size of the fp16 rounding noise that the per-token form itself carries relative to exact arithmetic.
//
// One warp owns one (sequence, head). Everything is held transposed so that accumulator fragments turn into the next
// contraction's A fragments without shuffles: the state lives in registers as the A fragments of S^T (n x d, the layout
// of the per-token kernel), W^T, U^T, Y^T are (n x token) accumulators, and K, Q^, a K, T = (I + L)^-1 and P are read from
// shared memory as B fragments with ldmatrix. (I + L)^-1 is formed by forward substitution in fp32, one column per lane.
// Per chunk: 128 m16n8k16 MMAs (the per-token kernel: 768 MMAs for 16 tokens) and about 700 other warp instructions.
// ------------------------------------------------------------------------------------------------
constexpr int kChunk = 16;
constexpr int kChunkWarps = 4;
constexpr int kCkQKStride = 72;  // floats per row of the raw q / k tiles: 16-byte pieces of two lanes per row never share a bank group
constexpr int kCkVStride = 68;   // floats per row of the raw v tile: the accumulator-shaped reads are conflict-free
constexpr int kCkHStride = 72;   // halves per row of the prepared operands (-K, Q^, a K): conflict-free ldmatrix rows
constexpr int kCkTStride = 24;   // halves per row of T and P
// the same tiles when q, k, v arrive as halves: strides in halves (160-byte q / k rows, 144-byte v rows)
constexpr int kCkQKStrideH = 80;
constexpr int kCkVStrideH = 72;
constexpr int kCkYStrideH = 72;  // halves per row of the output staging tile (in the -K / Q^ region, dead once their fragments are loaded)
constexpr int kCkRawQ = 0;
constexpr int kCkRawK = kCkRawQ + kChunk * kCkQKStride * 4;
constexpr int kCkRawV = kCkRawK + kChunk * kCkQKStride * 4;
constexpr int kCkBeta = kCkRawV + kChunk * kCkVStride * 4;
constexpr int kCkAlpha = kCkBeta + kChunk * 4;
constexpr int kCkL = kCkAlpha + kChunk * 4;
constexpr int kCkNK = kCkL + kChunk * kChunk * 4;
constexpr int kCkQh = kCkNK + kChunk * kCkHStride * 2;
constexpr int kCkAK = kCkQh + kChunk * kCkHStride * 2;
constexpr int kCkT = kCkAK + kChunk * kCkHStride * 2;
constexpr int kCkP = kCkT + kChunk * kCkTStride * 2;
constexpr int kCkWarpBytes = kCkP + kChunk * kCkTStride * 2;
constexpr int kCkSmemBytes = kChunkWarps * kCkWarpBytes;
static_assert(kCkWarpBytes % 16 == 0 && kCkL % 16 == 0 && kCkNK % 16 == 0 && kCkT % 16 == 0, "16-byte aligned shared-memory regions");

__device__ __forceinline__ void mma_f16acc_16816(uint32_t& c0, uint32_t& c1, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f16.f16.f16.f16 {%0, %1}, {%2, %3, %4, %5}, {%6, %7}, {%0, %1};"
        : "+r"(c0), "+r"(c1)
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t saddr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr) : "memory");
}

__device__ __forceinline__ void stmatrix_x4_trans(uint32_t saddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.trans.shared.b16 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}

template <bool IN16, bool OUT16>
__global__ void __launch_bounds__(kChunkWarps * 32, 2) efla_chunk16_kernel(const EflaParams p) {
    constexpr int HD = 64;
    extern __shared__ __align__(16) uint8_t scan_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* wsm = scan_smem + warp * kCkWarpBytes;
    float* rawq = reinterpret_cast<float*>(wsm + kCkRawQ);
    float* rawk = reinterpret_cast<float*>(wsm + kCkRawK);
    float* rawv = reinterpret_cast<float*>(wsm + kCkRawV);
    float* beta_sh = reinterpret_cast<float*>(wsm + kCkBeta);
    float* alpha_sh = reinterpret_cast<float*>(wsm + kCkAlpha);
    float* L_sh = reinterpret_cast<float*>(wsm + kCkL);
    __half* nk_sh = reinterpret_cast<__half*>(wsm + kCkNK);
    __half* qh_sh = reinterpret_cast<__half*>(wsm + kCkQh);
    __half* ak_sh = reinterpret_cast<__half*>(wsm + kCkAK);
    __half* t_sh = reinterpret_cast<__half*>(wsm + kCkT);
    __half* p_sh = reinterpret_cast<__half*>(wsm + kCkP);
    __half* y_sh = nk_sh;  // output staging (OUT16): the -K / Q^ tiles are dead once their fragments sit in registers
    static_assert(kChunk * kCkYStrideH * 2 <= 2 * kChunk * kCkHStride * 2, "output staging fits the -K / Q^ region");
    const long long unit = static_cast<long long>(blockIdx.x) * kChunkWarps + warp;  // (sequence, head)
    if (unit >= p.seqs * static_cast<long long>(p.heads)) return;
    // the grid has fewer than 2^32 / 4 CTAs: 32-bit divisions (a 64-bit one costs more than a chunk's scalar work)
    const unsigned useq = static_cast<unsigned>(unit) / static_cast<unsigned>(p.heads);
    const long long seq = useq;
    const int h = static_cast<int>(static_cast<unsigned>(unit) - useq * static_cast<unsigned>(p.heads));
    const float beta_bias = p.beta_bias_seq != nullptr ? p.beta_bias_seq[useq / static_cast<unsigned>(p.seqs_per_bias)] : p.beta_bias;
    const int g = lane >> 2, tq = lane & 3;

    // state S^T as A fragments: Sh[mt][ks][i] holds S[d][n] for n = 16 mt + g (+ 8 for odd i), d = 16 ks + 2 tq + {0, 1} (+ 8 for i >= 2)
    uint32_t Sh[4][4][4];
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) Sh[mt][ks][i] = 0u;

    const size_t row0 = static_cast<size_t>(seq) * p.T;
    // element type of q, k, v: fp32 or (IN16) halves; ld_qkv counts elements of that type
    const float* qb = static_cast<const float*>(p.q) + row0 * p.ld_qkv + h * HD;
    const float* kb = static_cast<const float*>(p.k) + row0 * p.ld_qkv + h * HD;
    const float* vb = static_cast<const float*>(p.v) + row0 * p.ld_qkv + h * HD;
    const __half* qbh = static_cast<const __half*>(p.q) + row0 * p.ld_qkv + h * HD;
    const __half* kbh = static_cast<const __half*>(p.k) + row0 * p.ld_qkv + h * HD;
    const __half* vbh = static_cast<const __half*>(p.v) + row0 * p.ld_qkv + h * HD;
    const float* bb = p.beta_raw + row0 * p.ld_beta;
    float* ob = static_cast<float*>(p.out) + row0 * p.ld_out + h * HD;
    __half* obh = static_cast<__half*>(p.out) + row0 * p.ld_out + h * HD;
    __half* rawqh = reinterpret_cast<__half*>(rawq);
    __half* rawkh = reinterpret_cast<__half*>(rawk);
    __half* rawvh = reinterpret_cast<__half*>(rawv);

    // asynchronous copy of one chunk's q, k, v, beta rows into the raw tiles (16-byte pieces)
    auto issue_chunk = [&](int t0) {
        if constexpr (IN16) {  // 8 pieces per 128-byte row: lane = piece within a group of four rows
            const int piece = lane & 7, rsel = lane >> 3;
#pragma unroll
            for (int j = 0; j < kChunk / 4; ++j) {
                const int r = 4 * j + rsel;
                if (t0 + r < p.T) {
                    const size_t o = static_cast<size_t>(t0 + r) * p.ld_qkv + 8 * piece;
                    cp_async16(rawqh + r * kCkQKStrideH + 8 * piece, qbh + o);
                    cp_async16(rawkh + r * kCkQKStrideH + 8 * piece, kbh + o);
                    cp_async16(rawvh + r * kCkVStrideH + 8 * piece, vbh + o);
                }
            }
        } else {  // 16 pieces per 256-byte row: lane = piece within a pair of rows
            const int piece = lane & 15, rsel = lane >> 4;
#pragma unroll
            for (int j = 0; j < kChunk / 2; ++j) {
                const int r = 2 * j + rsel;
                if (t0 + r < p.T) {
                    const size_t o = static_cast<size_t>(t0 + r) * p.ld_qkv + 4 * piece;
                    cp_async16(rawq + r * kCkQKStride + 4 * piece, qb + o);
                    cp_async16(rawk + r * kCkQKStride + 4 * piece, kb + o);
                    cp_async16(rawv + r * kCkVStride + 4 * piece, vb + o);
                }
            }
        }
        if (lane < kChunk && t0 + lane < p.T) cp_async4(beta_sh + lane, bb + static_cast<size_t>(t0 + lane) * p.ld_beta);
        cp_async_commit();
    };

    // ldmatrix row addresses of this lane: matrix j = lane / 8, row lane % 8
    const int lm_j = lane >> 3, lm_r = lane & 7;
    // operands stored [token][d]: matrices (tokens 0-7 | d 0-7), (0-7 | 8-15), (8-15 | 0-7), (8-15 | 8-15) of a 16-wide d block
    const uint32_t lm_tok_off = static_cast<uint32_t>(((lm_j >> 1) * 8 + lm_r) * kCkHStride + (lm_j & 1) * 8) * 2u;
    const uint32_t nk_addr = static_cast<uint32_t>(__cvta_generic_to_shared(nk_sh)) + lm_tok_off;
    const uint32_t qh_addr = static_cast<uint32_t>(__cvta_generic_to_shared(qh_sh)) + lm_tok_off;
    const uint32_t lm_ts_off = static_cast<uint32_t>(((lm_j >> 1) * 8 + lm_r) * kCkTStride + (lm_j & 1) * 8) * 2u;
    const uint32_t t_addr = static_cast<uint32_t>(__cvta_generic_to_shared(t_sh)) + lm_ts_off;
    const uint32_t p_addr = static_cast<uint32_t>(__cvta_generic_to_shared(p_sh)) + lm_ts_off;
    // a K read transposed: matrices (tokens 0-7 | d-tile), (8-15 | d-tile), (0-7 | d-tile + 1), (8-15 | d-tile + 1)
    const uint32_t ak_addr = static_cast<uint32_t>(__cvta_generic_to_shared(ak_sh)) +
                             static_cast<uint32_t>(((lm_j & 1) * 8 + lm_r) * kCkHStride + (lm_j >> 1) * 8) * 2u;

    // V read and Y written through transposing matrix loads / stores: matrix j = lane / 8 covers tokens 8 (j >> 1) .. + 7 and
    // columns 16 mt + 8 (j & 1) .. + 7; a thread's register pair is (column g, tokens 2 tq and 2 tq + 1): the accumulator layout
    const uint32_t v_addr = static_cast<uint32_t>(__cvta_generic_to_shared(rawvh)) +
                            static_cast<uint32_t>(((lm_j >> 1) * 8 + lm_r) * kCkVStrideH + (lm_j & 1) * 8) * 2u;
    const uint32_t y_addr = static_cast<uint32_t>(__cvta_generic_to_shared(y_sh)) +
                            static_cast<uint32_t>(((lm_j >> 1) * 8 + lm_r) * kCkYStrideH + (lm_j & 1) * 8) * 2u;
    issue_chunk(0);
    for (int t0 = 0; t0 < p.T; t0 += kChunk) {
        cp_async_wait<0>();
        __syncwarp();
        // ---------------- per-token scalars and fp16 operands: two lanes per token, alternate 16-byte pieces ----------------
        {
            const int tt = lane >> 1, hh = lane & 1;
            const bool valid = t0 + tt < p.T;
            // the lane's 32 elements of q and of k: 16-byte pieces 2 j + hh (four fp32, or eight halves: elements
            // 8 (2 j + hh) .. + 7); element e of the register array is column kcol(e)
            float qv[32], kv[32];
            if constexpr (IN16) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint4 a = *reinterpret_cast<const uint4*>(rawqh + tt * kCkQKStrideH + (2 * j + hh) * 8);
                    const uint4 b = *reinterpret_cast<const uint4*>(rawkh + tt * kCkQKStrideH + (2 * j + hh) * 8);
                    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[e])), fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[e]));
                        qv[8 * j + 2 * e] = valid ? fa.x : 0.0f; qv[8 * j + 2 * e + 1] = valid ? fa.y : 0.0f;
                        kv[8 * j + 2 * e] = valid ? fb.x : 0.0f; kv[8 * j + 2 * e + 1] = valid ? fb.y : 0.0f;
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float4 a = *reinterpret_cast<const float4*>(rawq + tt * kCkQKStride + (2 * j + hh) * 4);
                    const float4 b = *reinterpret_cast<const float4*>(rawk + tt * kCkQKStride + (2 * j + hh) * 4);
                    qv[4 * j] = valid ? a.x : 0.0f; qv[4 * j + 1] = valid ? a.y : 0.0f; qv[4 * j + 2] = valid ? a.z : 0.0f; qv[4 * j + 3] = valid ? a.w : 0.0f;
                    kv[4 * j] = valid ? b.x : 0.0f; kv[4 * j + 1] = valid ? b.y : 0.0f; kv[4 * j + 2] = valid ? b.z : 0.0f; kv[4 * j + 3] = valid ? b.w : 0.0f;
                }
            }
            float qss = 0.0f, kss = 0.0f;
#pragma unroll
            for (int e = 0; e < 32; ++e) { qss = fmaf(qv[e], qv[e], qss); kss = fmaf(kv[e], kv[e], kss); }
            qss += __shfl_xor_sync(0xffffffffu, qss, 1);
            kss += __shfl_xor_sync(0xffffffffu, kss, 1);
            const float q_inv = rsqrtf(qss + p.eps);
            const float lambda = kss < p.eps ? p.eps : kss;
            const float beta = sigmoidf_dev((valid ? beta_sh[tt] : 0.0f) + beta_bias);
            float alpha, kscale = 1.0f;
            if (p.method == 0) { alpha = beta; kscale = rsqrtf(lambda + p.eps); }
            else alpha = -expm1f(-(beta * lambda)) / (lambda + p.eps);
            if (!valid) alpha = 0.0f;
            if (hh == 0) alpha_sh[tt] = alpha;
            const float nks = -kscale, aks = alpha * kscale;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                // register elements 4 j .. 4 j + 3 are four consecutive columns starting at c0
                const int c0 = IN16 ? (2 * (j >> 1) + hh) * 8 + 4 * (j & 1) : (2 * j + hh) * 4;
                const int o = tt * kCkHStride + c0;
                uint2 wq, wk, wa;
                wq.x = pack_half2(qv[4 * j] * q_inv, qv[4 * j + 1] * q_inv); wq.y = pack_half2(qv[4 * j + 2] * q_inv, qv[4 * j + 3] * q_inv);
                wk.x = pack_half2(kv[4 * j] * nks, kv[4 * j + 1] * nks);     wk.y = pack_half2(kv[4 * j + 2] * nks, kv[4 * j + 3] * nks);
                wa.x = pack_half2(kv[4 * j] * aks, kv[4 * j + 1] * aks);     wa.y = pack_half2(kv[4 * j + 2] * aks, kv[4 * j + 3] * aks);
                *reinterpret_cast<uint2*>(qh_sh + o) = wq;
                *reinterpret_cast<uint2*>(nk_sh + o) = wk;
                *reinterpret_cast<uint2*>(ak_sh + o) = wa;
            }
        }
        // ---------------- W^T starts as V^T: element (n, token) of this lane's accumulator positions ----------------
        float Wc[4][2][4];
        if constexpr (IN16) {
            // rows past the end of the sequence may hold stale halves: their columns of W are never used (alpha = 0 masks
            // them out of L and P, and their outputs are not written), but they must be finite
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, v_addr + mt * 32);
#pragma unroll
                for (int nt = 0; nt < 2; ++nt) {
                    const bool valid0 = t0 + 8 * nt + 2 * tq < p.T, valid1 = t0 + 8 * nt + 2 * tq + 1 < p.T;
                    const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&vf[2 * nt])), hi = __half22float2(*reinterpret_cast<const __half2*>(&vf[2 * nt + 1]));
                    Wc[mt][nt][0] = valid0 ? lo.x : 0.0f; Wc[mt][nt][1] = valid1 ? lo.y : 0.0f;
                    Wc[mt][nt][2] = valid0 ? hi.x : 0.0f; Wc[mt][nt][3] = valid1 ? hi.y : 0.0f;
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int tok = 8 * nt + 2 * tq + e;
                    const bool valid = t0 + tok < p.T;
#pragma unroll
                    for (int mt = 0; mt < 4; ++mt) {
                        Wc[mt][nt][e] = valid ? rawv[tok * kCkVStride + 16 * mt + g] : 0.0f;
                        Wc[mt][nt][2 + e] = valid ? rawv[tok * kCkVStride + 16 * mt + 8 + g] : 0.0f;
                    }
                }
        }
        __syncwarp();  // the raw tiles are free, the prepared operands are visible
        issue_chunk(t0 + kChunk);

        // ---------------- W^T = V^T + S0^T (-K^T); G = K K^T; -Q^ K^T ----------------
        uint32_t kf[4][4], qf[4][4];  // per 16-wide d block: B fragments {b0, b1} for tokens 0-7 (regs 0, 1) and 8-15 (regs 2, 3)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            ldmatrix_x4(kf[ks], nk_addr + ks * 32);
            ldmatrix_x4(qf[ks], qh_addr + ks * 32);
        }
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
                    mma_f16_16816(Wc[mt][nt], Sh[mt][ks][0], Sh[mt][ks][1], Sh[mt][ks][2], Sh[mt][ks][3], kf[ks][2 * nt], kf[ks][2 * nt + 1]);
        float Gc[2][4], Xc[2][4];  // rows t = g (+ 8 for i >= 2), columns s = 8 nt + 2 tq + (i & 1);  Xc = -(q^_t . k_s)
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) Gc[nt][i] = Xc[nt][i] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                mma_f16_16816(Gc[nt], kf[ks][0], kf[ks][2], kf[ks][1], kf[ks][3], kf[ks][2 * nt], kf[ks][2 * nt + 1]);
                mma_f16_16816(Xc[nt], qf[ks][0], qf[ks][2], qf[ks][1], qf[ks][3], kf[ks][2 * nt], kf[ks][2 * nt + 1]);
            }
        // L[t][s] = a_s G[t][s] (s < t) in fp32 for the substitution; P[t][s] = a_s (q^_t . k_s) (s <= t) in fp16
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const int s0 = 8 * nt + 2 * tq;
            const float2 al = *reinterpret_cast<const float2*>(alpha_sh + s0);
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int t = g + 8 * hr;
                const float l0 = s0 < t ? al.x * Gc[nt][2 * hr] : 0.0f, l1 = s0 + 1 < t ? al.y * Gc[nt][2 * hr + 1] : 0.0f;
                const float p0 = s0 <= t ? -al.x * Xc[nt][2 * hr] : 0.0f, p1 = s0 + 1 <= t ? -al.y * Xc[nt][2 * hr + 1] : 0.0f;
                *reinterpret_cast<float2*>(L_sh + t * kChunk + s0) = make_float2(l0, l1);
                *reinterpret_cast<uint32_t*>(p_sh + t * kCkTStride + s0) = pack_half2(p0, p1);
            }
        }
        __syncwarp();
        // ---------------- T = (I + L)^-1 by forward substitution, lane c owns column c ----------------
        {
            const int c = lane & 15;
            float col[kChunk];
#pragma unroll
            for (int t = 0; t < kChunk; ++t) {
                float acc = t == c ? 1.0f : 0.0f;
#pragma unroll
                for (int s4 = 0; s4 < t; s4 += 4) {
                    const float4 lv = *reinterpret_cast<const float4*>(L_sh + t * kChunk + s4);
                    acc = fmaf(-lv.x, col[s4], acc);
                    if (s4 + 1 < t) acc = fmaf(-lv.y, col[s4 + 1], acc);
                    if (s4 + 2 < t) acc = fmaf(-lv.z, col[s4 + 2], acc);
                    if (s4 + 3 < t) acc = fmaf(-lv.w, col[s4 + 3], acc);
                }
                col[t] = acc;
            }
            if (lane < kChunk) {
#pragma unroll
                for (int t = 0; t < kChunk; ++t) t_sh[t * kCkTStride + c] = __float2half_rn(col[t]);
            }
        }
        __syncwarp();
        uint32_t tf[4], pf[4];
        ldmatrix_x4(tf, t_addr);
        ldmatrix_x4(pf, p_addr);
        // ---------------- U^T = W^T T^T ----------------
        uint32_t Up[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            const uint32_t w0 = pack_half2(Wc[mt][0][0], Wc[mt][0][1]), w1 = pack_half2(Wc[mt][0][2], Wc[mt][0][3]);
            const uint32_t w2 = pack_half2(Wc[mt][1][0], Wc[mt][1][1]), w3 = pack_half2(Wc[mt][1][2], Wc[mt][1][3]);
            float Uc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) mma_f16_16816_zero(Uc[nt], w0, w1, w2, w3, tf[2 * nt], tf[2 * nt + 1]);
            Up[mt][0] = pack_half2(Uc[0][0], Uc[0][1]); Up[mt][1] = pack_half2(Uc[0][2], Uc[0][3]);
            Up[mt][2] = pack_half2(Uc[1][0], Uc[1][1]); Up[mt][3] = pack_half2(Uc[1][2], Uc[1][3]);
        }
        // ---------------- Y^T = S0^T Q^^T + U^T P^T ----------------
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            float Yc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) mma_f16_16816_zero(Yc[nt], Up[mt][0], Up[mt][1], Up[mt][2], Up[mt][3], pf[2 * nt], pf[2 * nt + 1]);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
                    mma_f16_16816(Yc[nt], Sh[mt][ks][0], Sh[mt][ks][1], Sh[mt][ks][2], Sh[mt][ks][3], qf[ks][2 * nt], qf[ks][2 * nt + 1]);
            if constexpr (OUT16) {  // staged as halves (one transposing matrix store per 16 columns), written out row by row below
                stmatrix_x4_trans(y_addr + mt * 32, pack_half2(Yc[0][0], Yc[0][1]), pack_half2(Yc[0][2], Yc[0][3]), pack_half2(Yc[1][0], Yc[1][1]),
                                  pack_half2(Yc[1][2], Yc[1][3]));
            } else {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tl = 8 * nt + 2 * tq + e;
                        if (t0 + tl < p.T) {
                            float* orow = ob + static_cast<size_t>(t0 + tl) * p.ld_out + 16 * mt + g;
                            orow[0] = Yc[nt][e];
                            orow[8] = Yc[nt][2 + e];
                        }
                    }
            }
        }
        if constexpr (OUT16) {
            __syncwarp();
            // 16 rows x 128 bytes: 16-byte pieces, eight per row
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int tl = 4 * j + (lane >> 3), piece = lane & 7;
                if (t0 + tl < p.T)
                    *reinterpret_cast<uint4*>(obh + static_cast<size_t>(t0 + tl) * p.ld_out + 8 * piece) =
                        *reinterpret_cast<const uint4*>(y_sh + tl * kCkYStrideH + 8 * piece);
            }
        }
        // ---------------- S^T += U^T (a K): fp16 accumulators = the state registers, rounded once per chunk ----------------
#pragma unroll
        for (int dp = 0; dp < 4; ++dp) {
            uint32_t af[4];
            ldmatrix_x4_trans(af, ak_addr + dp * 32);
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                mma_f16acc_16816(Sh[mt][dp][0], Sh[mt][dp][1], Up[mt][0], Up[mt][1], Up[mt][2], Up[mt][3], af[0], af[1]);
                mma_f16acc_16816(Sh[mt][dp][2], Sh[mt][dp][3], Up[mt][0], Up[mt][1], Up[mt][2], Up[mt][3], af[2], af[3]);
            }
        }
    }
    cp_async_wait<0>();
}


// ------------------------------------------------------------------------------------------------
// The chunked scan for the case the batched driver runs: method 1 (k is used unscaled), q | k | v as halves. The chunk's
// recurrence is rewritten so that every tensor-core operand is a tile as it arrived from global memory:
//   with  U~_t = a_t U_t  (U the per-token updates, a_t = alpha_t):
//       (I + diag(a) G_strict) U~ = diag(a) W,     W = V - K S0,  G = K K^T
//       Y = diag(q_inv) (Q S0 + (Q K^T, lower triangle incl. diagonal) U~),        S += K^T U~
// so K and Q enter the MMAs unscaled (ldmatrix straight from the raw tiles), alpha scales rows of G and columns of W^T, and the
// query normalisation scales the finished output. No prepared operand tiles are written: the preparation phase only
// computes the per-token scalars. The raw k tile is double-buffered because the state update at the end of a chunk still
// reads it while the next chunk is being fetched.
// ------------------------------------------------------------------------------------------------
constexpr int kM1Stride = 72;  // halves per row of the raw tiles: conflict-free for ldmatrix rows and for the 16-byte reads of eight rows
constexpr int kM1RawQ = 0;
constexpr int kM1RawK = kM1RawQ + kChunk * kM1Stride * 2;       // two buffers
constexpr int kM1RawV = kM1RawK + 2 * kChunk * kM1Stride * 2;
constexpr int kM1Y = kM1RawV + kChunk * kM1Stride * 2;          // output staging
constexpr int kM1Beta = kM1Y + kChunk * kM1Stride * 2;
constexpr int kM1Alpha = kM1Beta + kChunk * 4;
constexpr int kM1Qinv = kM1Alpha + kChunk * 4;
constexpr int kM1L = kM1Qinv + kChunk * 4;
constexpr int kM1T = kM1L + kChunk * kChunk * 4;
constexpr int kM1P = kM1T + kChunk * kCkTStride * 2;
constexpr int kM1WarpBytes = kM1P + kChunk * kCkTStride * 2;
constexpr int kM1SmemBytes = kChunkWarps * kM1WarpBytes;
static_assert(kM1WarpBytes % 16 == 0 && kM1L % 16 == 0 && kM1T % 16 == 0 && kM1Beta % 16 == 0, "16-byte aligned shared-memory regions");

template <bool OUT16>
__global__ void __launch_bounds__(kChunkWarps * 32, 2) efla_chunk16_m1_kernel(const EflaParams p) {
    constexpr int HD = 64;
    extern __shared__ __align__(16) uint8_t scan_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t* wsm = scan_smem + warp * kM1WarpBytes;
    __half* rawq = reinterpret_cast<__half*>(wsm + kM1RawQ);
    __half* rawk = reinterpret_cast<__half*>(wsm + kM1RawK);   // + buffer * kChunk * kM1Stride
    __half* rawv = reinterpret_cast<__half*>(wsm + kM1RawV);
    __half* y_sh = reinterpret_cast<__half*>(wsm + kM1Y);
    float* beta_sh = reinterpret_cast<float*>(wsm + kM1Beta);
    float* alpha_sh = reinterpret_cast<float*>(wsm + kM1Alpha);
    float* qinv_sh = reinterpret_cast<float*>(wsm + kM1Qinv);
    float* L_sh = reinterpret_cast<float*>(wsm + kM1L);
    __half* t_sh = reinterpret_cast<__half*>(wsm + kM1T);
    __half* p_sh = reinterpret_cast<__half*>(wsm + kM1P);
    // Persistent warps: each walks (sequence, head) units with a grid stride and fetches the first chunk of its next unit while the
    // last chunk of the present one is computed, so that no unit starts with an exposed trip to DRAM.
    const unsigned total_units = static_cast<unsigned>(p.seqs * static_cast<long long>(p.heads));  // below 2^31 (checked by the host)
    const unsigned unit_stride = gridDim.x * kChunkWarps;
    unsigned unit = blockIdx.x * kChunkWarps + warp;
    if (unit >= total_units) return;
    const int g = lane >> 2, tq = lane & 3;
    // first row of a unit's sequence and its head (32-bit division: a 64-bit one costs more than a chunk's scalar work)
    struct UnitAt { size_t row0; int h; unsigned useq; };
    auto unit_at = [&](unsigned u) {
        UnitAt a;
        a.useq = u / static_cast<unsigned>(p.heads);
        a.h = static_cast<int>(u - a.useq * static_cast<unsigned>(p.heads));
        a.row0 = static_cast<size_t>(a.useq) * p.T;
        return a;
    };

    // asynchronous copy of one chunk's q, k, v, beta rows (16-byte pieces, eight per 128-byte row); rows past the end of the
    // sequence are zero-filled so that everything derived from them stays finite
    auto issue_chunk = [&](const UnitAt& ua, int t0, int kbuf) {
        const int piece = lane & 7, rsel = lane >> 3;
        __half* rk = rawk + kbuf * kChunk * kM1Stride;
        const __half* qbh = static_cast<const __half*>(p.q) + ua.row0 * p.ld_qkv + ua.h * HD;
        const __half* kbh = static_cast<const __half*>(p.k) + ua.row0 * p.ld_qkv + ua.h * HD;
        const __half* vbh = static_cast<const __half*>(p.v) + ua.row0 * p.ld_qkv + ua.h * HD;
        const float* bb = p.beta_raw + ua.row0 * p.ld_beta;
#pragma unroll
        for (int j = 0; j < kChunk / 4; ++j) {
            const int r = 4 * j + rsel;
            if (t0 + r < p.T) {
                const size_t o = static_cast<size_t>(t0 + r) * p.ld_qkv + 8 * piece;
                cp_async16(rawq + r * kM1Stride + 8 * piece, qbh + o);
                cp_async16(rk + r * kM1Stride + 8 * piece, kbh + o);
                cp_async16(rawv + r * kM1Stride + 8 * piece, vbh + o);
            } else {
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4*>(rawq + r * kM1Stride + 8 * piece) = z;
                *reinterpret_cast<uint4*>(rk + r * kM1Stride + 8 * piece) = z;
                *reinterpret_cast<uint4*>(rawv + r * kM1Stride + 8 * piece) = z;
            }
        }
        if (lane < kChunk && t0 + lane < p.T) cp_async4(beta_sh + lane, bb + static_cast<size_t>(t0 + lane) * p.ld_beta);
        cp_async_commit();
    };

    // ldmatrix row addresses of this lane: matrix j = lane / 8, row lane % 8
    const int lm_j = lane >> 3, lm_r = lane & 7;
    // tiles stored [token][d]: matrices (tokens 0-7 | d 0-7), (0-7 | 8-15), (8-15 | 0-7), (8-15 | 8-15) of a 16-wide d block
    const uint32_t lm_tok_off = static_cast<uint32_t>(((lm_j >> 1) * 8 + lm_r) * kM1Stride + (lm_j & 1) * 8) * 2u;
    const uint32_t q_addr = static_cast<uint32_t>(__cvta_generic_to_shared(rawq)) + lm_tok_off;
    const uint32_t k_addr0 = static_cast<uint32_t>(__cvta_generic_to_shared(rawk)) + lm_tok_off;
    const uint32_t lm_ts_off = static_cast<uint32_t>(((lm_j >> 1) * 8 + lm_r) * kCkTStride + (lm_j & 1) * 8) * 2u;
    // T^T read transposed: matrices (s 0-7 | t 0-7), (s 8-15 | t 0-7), (s 0-7 | t 8-15), (s 8-15 | t 8-15)
    const uint32_t tt_addr = static_cast<uint32_t>(__cvta_generic_to_shared(t_sh)) +
                             static_cast<uint32_t>(((lm_j & 1) * 8 + lm_r) * kCkTStride + (lm_j >> 1) * 8) * 2u;
    const uint32_t p_addr = static_cast<uint32_t>(__cvta_generic_to_shared(p_sh)) + lm_ts_off;
    // K read transposed: matrices (tokens 0-7 | d-tile), (8-15 | d-tile), (0-7 | d-tile + 1), (8-15 | d-tile + 1)
    const uint32_t kt_addr0 = static_cast<uint32_t>(__cvta_generic_to_shared(rawk)) +
                              static_cast<uint32_t>(((lm_j & 1) * 8 + lm_r) * kM1Stride + (lm_j >> 1) * 8) * 2u;
    // V read and Y written through transposing matrix loads / stores (tokens 8 (j >> 1) .., columns 16 mt + 8 (j & 1) ..)
    const uint32_t v_addr = static_cast<uint32_t>(__cvta_generic_to_shared(rawv)) + lm_tok_off;
    const uint32_t y_addr = static_cast<uint32_t>(__cvta_generic_to_shared(y_sh)) + lm_tok_off;
    constexpr uint32_t kKBufBytes = kChunk * kM1Stride * 2;

    int kbuf = 0;
    issue_chunk(unit_at(unit), 0, 0);
    for (; unit < total_units; unit += unit_stride) {
    const UnitAt ua = unit_at(unit);
    const float beta_bias = p.beta_bias_seq != nullptr ? p.beta_bias_seq[ua.useq / static_cast<unsigned>(p.seqs_per_bias)] : p.beta_bias;
    float* ob = static_cast<float*>(p.out) + ua.row0 * p.ld_out + ua.h * HD;
    __half* obh = static_cast<__half*>(p.out) + ua.row0 * p.ld_out + ua.h * HD;
    uint32_t Sh[4][4][4];  // state S^T as A fragments, as in efla_chunk16_kernel
#pragma unroll
    for (int mt = 0; mt < 4; ++mt)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int i = 0; i < 4; ++i) Sh[mt][ks][i] = 0u;
    for (int t0 = 0; t0 < p.T; t0 += kChunk, kbuf ^= 1) {
        cp_async_wait<0>();
        __syncwarp();
        // ---------------- operand fragments straight from the raw tiles; W^T starts as -V^T ----------------
        uint32_t kf[4][4], qf[4][4];  // per 16-wide d block: B fragments {b0, b1} for tokens 0-7 (regs 0, 1) and 8-15 (regs 2, 3)
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            ldmatrix_x4(kf[ks], k_addr0 + kbuf * kKBufBytes + ks * 32);
            ldmatrix_x4(qf[ks], q_addr + ks * 32);
        }
        float Wc[4][2][4];  // -(V - K S0)^T = S0^T K^T - V^T
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            uint32_t vf[4];
            ldmatrix_x4_trans(vf, v_addr + mt * 32);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float2 lo = __half22float2(*reinterpret_cast<const __half2*>(&vf[2 * nt])), hi = __half22float2(*reinterpret_cast<const __half2*>(&vf[2 * nt + 1]));
                Wc[mt][nt][0] = -lo.x; Wc[mt][nt][1] = -lo.y;
                Wc[mt][nt][2] = -hi.x; Wc[mt][nt][3] = -hi.y;
            }
        }
        // The squared norms of k and q are the diagonals of K K^T and Q Q^T, which the tensor cores produce below. They land in
        // the eight lanes with tq == g / 2 (tokens g and g + 8); each hands token g + 8 to its neighbour lane ^ 1, so sixteen
        // lanes run the scalar chain for one token each. Those lanes take their beta now: the next chunk's copy overwrites it.
        const bool diag_lane = tq == (g >> 1);
        const bool helper_lane = (tq ^ 1) == (g >> 1);
        const int my_tok = g + (helper_lane ? 8 : 0);
        float braw = 0.0f;
        if ((diag_lane || helper_lane) && t0 + my_tok < p.T) braw = beta_sh[my_tok];
        __syncwarp();  // q, v and beta are consumed
        if (t0 + kChunk < p.T) issue_chunk(ua, t0 + kChunk, kbuf ^ 1);
        else if (unit + unit_stride < total_units) issue_chunk(unit_at(unit + unit_stride), 0, kbuf ^ 1);

#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int mt = 0; mt < 4; ++mt)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
                    mma_f16_16816(Wc[mt][nt], Sh[mt][ks][0], Sh[mt][ks][1], Sh[mt][ks][2], Sh[mt][ks][3], kf[ks][2 * nt], kf[ks][2 * nt + 1]);
        float Gc[2][4], Xc[2][4], Qc[2][4];  // rows t = g (+ 8 for i >= 2), columns s = 8 nt + 2 tq + (i & 1);  Xc = q_t . k_s, Qc = q_t . q_s
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) Gc[nt][i] = Xc[nt][i] = Qc[nt][i] = 0.0f;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                mma_f16_16816(Gc[nt], kf[ks][0], kf[ks][2], kf[ks][1], kf[ks][3], kf[ks][2 * nt], kf[ks][2 * nt + 1]);
                mma_f16_16816(Xc[nt], qf[ks][0], qf[ks][2], qf[ks][1], qf[ks][3], kf[ks][2 * nt], kf[ks][2 * nt + 1]);
                mma_f16_16816(Qc[nt], qf[ks][0], qf[ks][2], qf[ks][1], qf[ks][3], qf[ks][2 * nt], qf[ks][2 * nt + 1]);
            }
        // ---------------- per-token scalars from the diagonals (exact fp16 products accumulated in fp32) ----------------
        {
            const int e = g & 1;
            float kss = e ? Gc[0][1] : Gc[0][0], qss = e ? Qc[0][1] : Qc[0][0];              // token g (valid in the diagonal lanes)
            const float kss_hi = e ? Gc[1][3] : Gc[1][2], qss_hi = e ? Qc[1][3] : Qc[1][2];  // token g + 8
            const float k_from = __shfl_xor_sync(0xffffffffu, kss_hi, 1), q_from = __shfl_xor_sync(0xffffffffu, qss_hi, 1);
            if (helper_lane) { kss = k_from; qss = q_from; }
            if (diag_lane || helper_lane) {
                const float lambda = kss < p.eps ? p.eps : kss;
                // sigmoid and the final quotient with the fast exponential / division (about 2 ulp each: far below the fp16
                // rounding of every operand alpha touches); expm1f keeps its accuracy for small beta * lambda
                const float beta = __fdividef(1.0f, 1.0f + __expf(-(braw + beta_bias)));
                alpha_sh[my_tok] = t0 + my_tok < p.T ? __fdividef(-expm1f(-(beta * lambda)), lambda + p.eps) : 0.0f;
                qinv_sh[my_tok] = rsqrtf(qss + p.eps);
            }
        }
        __syncwarp();
        // L[t][s] = a_t G[t][s] (s < t) in fp32 for the substitution; P[t][s] = q_t . k_s (s <= t) in fp16
        {
            const float a_lo = alpha_sh[g], a_hi = alpha_sh[g + 8];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const int s0 = 8 * nt + 2 * tq;
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {
                    const int t = g + 8 * hr;
                    const float at = hr ? a_hi : a_lo;
                    // the substitution reads L below the diagonal only: no mask needed there; P feeds an MMA and is masked
                    const float l0 = at * Gc[nt][2 * hr], l1 = at * Gc[nt][2 * hr + 1];
                    const float p0 = s0 <= t ? Xc[nt][2 * hr] : 0.0f, p1 = s0 + 1 <= t ? Xc[nt][2 * hr + 1] : 0.0f;
                    *reinterpret_cast<float2*>(L_sh + t * kChunk + s0) = make_float2(l0, l1);
                    *reinterpret_cast<uint32_t*>(p_sh + t * kCkTStride + s0) = pack_half2(p0, p1);
                }
            }
        }
        __syncwarp();
        // ---------------- T = (I + L)^-1 by forward substitution, lane c owns column c ----------------
        {
            const int c = lane & 15;
            float col[kChunk];
#pragma unroll
            for (int t = 0; t < kChunk; ++t) {
                float acc = t == c ? 1.0f : 0.0f;
#pragma unroll
                for (int s4 = 0; s4 < t; s4 += 4) {
                    const float4 lv = *reinterpret_cast<const float4*>(L_sh + t * kChunk + s4);
                    acc = fmaf(-lv.x, col[s4], acc);
                    if (s4 + 1 < t) acc = fmaf(-lv.y, col[s4 + 1], acc);
                    if (s4 + 2 < t) acc = fmaf(-lv.z, col[s4 + 2], acc);
                    if (s4 + 3 < t) acc = fmaf(-lv.w, col[s4 + 3], acc);
                }
                col[t] = acc;
            }
            if (lane < kChunk) {  // the column as one row of T^T: sixteen halves, two 16-byte stores
                uint32_t w[8];
#pragma unroll
                for (int t = 0; t < kChunk; t += 2) w[t >> 1] = pack_half2(col[t], col[t + 1]);
                uint4* dst = reinterpret_cast<uint4*>(t_sh + c * kCkTStride);
                dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
                dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
        }
        __syncwarp();
        uint32_t tf[4], pf[4];
        ldmatrix_x4_trans(tf, tt_addr);  // T^T stored [s][t]: transposed on the way in, the fragments are those of T stored [t][s]
        ldmatrix_x4(pf, p_addr);
        // ---------------- U~^T = (diag(a) W)^T T^T: the columns (tokens) of -W^T are scaled by -a ----------------
        float na[2][2], qi[2][2];  // [nt][e]: token 8 nt + 2 tq + e
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            const float2 al = *reinterpret_cast<const float2*>(alpha_sh + 8 * nt + 2 * tq);
            const float2 q2 = *reinterpret_cast<const float2*>(qinv_sh + 8 * nt + 2 * tq);
            na[nt][0] = -al.x; na[nt][1] = -al.y;
            qi[nt][0] = q2.x; qi[nt][1] = q2.y;
        }
        uint32_t Up[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            // packed fp32 pairs (tokens 2 tq and 2 tq + 1): each half rounds like the scalar multiply
            const float2 na0 = make_float2(na[0][0], na[0][1]), na1 = make_float2(na[1][0], na[1][1]);
            const float2 x0 = __fmul2_rn(na0, make_float2(Wc[mt][0][0], Wc[mt][0][1])), x1 = __fmul2_rn(na0, make_float2(Wc[mt][0][2], Wc[mt][0][3]));
            const float2 x2 = __fmul2_rn(na1, make_float2(Wc[mt][1][0], Wc[mt][1][1])), x3 = __fmul2_rn(na1, make_float2(Wc[mt][1][2], Wc[mt][1][3]));
            const uint32_t w0 = pack_half2(x0.x, x0.y), w1 = pack_half2(x1.x, x1.y), w2 = pack_half2(x2.x, x2.y), w3 = pack_half2(x3.x, x3.y);
            float Uc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) mma_f16_16816_zero(Uc[nt], w0, w1, w2, w3, tf[2 * nt], tf[2 * nt + 1]);
            Up[mt][0] = pack_half2(Uc[0][0], Uc[0][1]); Up[mt][1] = pack_half2(Uc[0][2], Uc[0][3]);
            Up[mt][2] = pack_half2(Uc[1][0], Uc[1][1]); Up[mt][3] = pack_half2(Uc[1][2], Uc[1][3]);
        }
        // ---------------- Y^T = (S0^T Q^T + U~^T P^T) diag(q_inv) ----------------
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            float Yc[2][4];
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) mma_f16_16816_zero(Yc[nt], Up[mt][0], Up[mt][1], Up[mt][2], Up[mt][3], pf[2 * nt], pf[2 * nt + 1]);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
                    mma_f16_16816(Yc[nt], Sh[mt][ks][0], Sh[mt][ks][1], Sh[mt][ks][2], Sh[mt][ks][3], qf[ks][2 * nt], qf[ks][2 * nt + 1]);
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
                const float2 q2 = make_float2(qi[nt][0], qi[nt][1]);
                const float2 lo = __fmul2_rn(q2, make_float2(Yc[nt][0], Yc[nt][1])), hi = __fmul2_rn(q2, make_float2(Yc[nt][2], Yc[nt][3]));
                Yc[nt][0] = lo.x; Yc[nt][1] = lo.y; Yc[nt][2] = hi.x; Yc[nt][3] = hi.y;
            }
            if constexpr (OUT16) {
                stmatrix_x4_trans(y_addr + mt * 32, pack_half2(Yc[0][0], Yc[0][1]), pack_half2(Yc[0][2], Yc[0][3]), pack_half2(Yc[1][0], Yc[1][1]),
                                  pack_half2(Yc[1][2], Yc[1][3]));
            } else {
#pragma unroll
                for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int tl = 8 * nt + 2 * tq + e;
                        if (t0 + tl < p.T) {
                            float* orow = ob + static_cast<size_t>(t0 + tl) * p.ld_out + 16 * mt + g;
                            orow[0] = Yc[nt][e];
                            orow[8] = Yc[nt][2 + e];
                        }
                    }
            }
        }
        if constexpr (OUT16) {
            __syncwarp();
#pragma unroll
            for (int j = 0; j < 4; ++j) {  // 16 rows x 128 bytes: 16-byte pieces, eight per row
                const int tl = 4 * j + (lane >> 3), piece = lane & 7;
                if (t0 + tl < p.T)
                    *reinterpret_cast<uint4*>(obh + static_cast<size_t>(t0 + tl) * p.ld_out + 8 * piece) =
                        *reinterpret_cast<const uint4*>(y_sh + tl * kM1Stride + 8 * piece);
            }
        }
        // ---------------- S^T += U~^T K: fp16 accumulators = the state registers, rounded once per chunk ----------------
#pragma unroll
        for (int dp = 0; dp < 4; ++dp) {
            uint32_t af[4];
            ldmatrix_x4_trans(af, kt_addr0 + kbuf * kKBufBytes + dp * 32);
#pragma unroll
            for (int mt = 0; mt < 4; ++mt) {
                mma_f16acc_16816(Sh[mt][dp][0], Sh[mt][dp][1], Up[mt][0], Up[mt][1], Up[mt][2], Up[mt][3], af[0], af[1]);
                mma_f16acc_16816(Sh[mt][dp][2], Sh[mt][dp][3], Up[mt][0], Up[mt][1], Up[mt][2], Up[mt][3], af[2], af[3]);
            }
        }
        __syncwarp();  // the staging tile and this chunk's k buffer are free for the chunk after the next
    }
    }
    cp_async_wait<0>();
}

}  // namespace

int g_efla_chunked = 1;  // host toggle (option "efla_chunked"): what BNF4_EFLA_AUTO picks for heads of 64 with on-chip state

int efla_launch(const EflaParams& p, cudaStream_t stream) {
    if (p.seqs <= 0 || p.T <= 0) return BNF4_OK;
    if (p.heads <= 0 || p.hidden <= 0 || (p.hidden % p.heads) != 0) return set_error(BNF4_ERR_INVALID, "efla: hidden=%d heads=%d", p.hidden, p.heads);
    if (!p.q || !p.k || !p.v || !p.beta_raw || !p.out) return set_error(BNF4_ERR_INVALID, "efla: null pointer");
    const int hd = p.hidden / p.heads;
    if (p.variant < 0 || p.variant > 3) return set_error(BNF4_ERR_INVALID, "efla: variant=%d outside [0,3]", p.variant);
    const bool regs_ok = p.state == nullptr && p.state_fp16 && hd == 64 &&
                         ((reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v)) & 15) == 0 &&
                         (p.ld_qkv % 4) == 0;  // 16-byte asynchronous copies of q, k, v
    if ((p.qkv_f16 || p.out_f16) && (!regs_ok || p.variant == BNF4_EFLA_GENERIC || p.variant == BNF4_EFLA_PER_TOKEN))
        return set_error(BNF4_ERR_INVALID, "efla: fp16 q, k, v or output are supported by the chunked kernel only");
    if ((p.variant == BNF4_EFLA_PER_TOKEN || p.variant == BNF4_EFLA_CHUNKED) && !regs_ok)
        return set_error(BNF4_ERR_INVALID, "efla: the register-state kernels need head_dim 64, no HBM state, an fp16 state and 16-byte aligned q, k, v");
    if (regs_ok && p.variant != BNF4_EFLA_GENERIC) {
        const bool chunked = p.variant == BNF4_EFLA_CHUNKED || (p.variant == BNF4_EFLA_AUTO && g_efla_chunked != 0);
        const long long units = p.seqs * static_cast<long long>(p.heads);
        if (units > 0x7fffffffLL) return set_error(BNF4_ERR_INVALID, "efla: more than 2^31 (sequence, head) units in one call");
        const long long ctas = (units + kScanWarps - 1) / kScanWarps;
        static_assert(kScanWarps == kChunkWarps, "one grid computation for both register-state kernels");
        // function attributes are per device: set once for each device this process uses
        static bool configured[64] = {};
        int dev = 0;
        int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
        if (rc) return rc;
        if (dev < 0 || dev >= 64 || !configured[dev]) {
            rc = check_cuda(cudaFuncSetAttribute(efla_scan64_mma2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kScan2SmemBytes), "cudaFuncSetAttribute(efla_scan64_mma2_kernel)");
            if (rc) return rc;
            rc = check_cuda(cudaFuncSetAttribute(efla_chunk16_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCkSmemBytes), "cudaFuncSetAttribute(efla_chunk16_kernel)");
            if (!rc) rc = check_cuda(cudaFuncSetAttribute(efla_chunk16_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCkSmemBytes), "cudaFuncSetAttribute(efla_chunk16_kernel)");
            if (!rc) rc = check_cuda(cudaFuncSetAttribute(efla_chunk16_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCkSmemBytes), "cudaFuncSetAttribute(efla_chunk16_kernel)");
            if (!rc) rc = check_cuda(cudaFuncSetAttribute(efla_chunk16_kernel<true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCkSmemBytes), "cudaFuncSetAttribute(efla_chunk16_kernel)");
            if (!rc) rc = check_cuda(cudaFuncSetAttribute(efla_chunk16_m1_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kM1SmemBytes), "cudaFuncSetAttribute(efla_chunk16_m1_kernel)");
            if (!rc) rc = check_cuda(cudaFuncSetAttribute(efla_chunk16_m1_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kM1SmemBytes), "cudaFuncSetAttribute(efla_chunk16_m1_kernel)");
            if (rc) return rc;
            if (dev >= 0 && dev < 64) configured[dev] = true;
        }
        if (chunked) {
            if (p.qkv_f16 && ((p.ld_qkv % 8) != 0)) return set_error(BNF4_ERR_INVALID, "efla: fp16 q, k, v need ld_qkv %% 8 == 0");
            if (p.out_f16 && (((p.ld_out % 8) != 0) || (reinterpret_cast<uintptr_t>(p.out) & 15))) return set_error(BNF4_ERR_INVALID, "efla: fp16 output needs 16-byte aligned rows");
            const unsigned grid = static_cast<unsigned>(ctas);
            if (p.qkv_f16 && p.method == 1) {  // the batched driver's case: raw-operand kernel, persistent warps (two CTAs per SM)
                int sms = 0;
                rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute");
                if (rc) return rc;
                const unsigned pgrid = std::min(grid, static_cast<unsigned>(2 * sms));
                if (p.out_f16) efla_chunk16_m1_kernel<true><<<pgrid, kChunkWarps * 32, kM1SmemBytes, stream>>>(p);
                else efla_chunk16_m1_kernel<false><<<pgrid, kChunkWarps * 32, kM1SmemBytes, stream>>>(p);
            } else if (p.qkv_f16 && p.out_f16) efla_chunk16_kernel<true, true><<<grid, kChunkWarps * 32, kCkSmemBytes, stream>>>(p);
            else if (p.qkv_f16) efla_chunk16_kernel<true, false><<<grid, kChunkWarps * 32, kCkSmemBytes, stream>>>(p);
            else if (p.out_f16) efla_chunk16_kernel<false, true><<<grid, kChunkWarps * 32, kCkSmemBytes, stream>>>(p);
            else efla_chunk16_kernel<false, false><<<grid, kChunkWarps * 32, kCkSmemBytes, stream>>>(p);
            return check_launch("efla_chunk16_kernel");
        }
        if (p.qkv_f16 || p.out_f16) return set_error(BNF4_ERR_INVALID, "efla: fp16 q, k, v or output are supported by the chunked kernel only");
        efla_scan64_mma2_kernel<<<static_cast<unsigned>(ctas), kScanWarps * 32, kScan2SmemBytes, stream>>>(p);
        return check_launch("efla_scan64_mma2_kernel");
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
