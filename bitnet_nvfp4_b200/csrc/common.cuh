// Shared device/host helpers for the B200 (sm_100a) kernels of this library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstddef>
#include <cstdint>

// ---------------------------------------------------------------------------------------------
// Error reporting. Every extern "C" entry point returns 0 on success or one of these codes and
// records a message readable through bnf4_last_error().
// ---------------------------------------------------------------------------------------------
enum Bnf4Status : int {
    BNF4_OK = 0,
    BNF4_ERR_INVALID = 1,      // bad argument (null pointer, unsupported shape, misalignment)
    BNF4_ERR_CUDA = 2,         // a CUDA runtime/driver call failed
    BNF4_ERR_UNSUPPORTED = 3,  // entry point exists for link compatibility only
    BNF4_ERR_DEVICE = 4,       // a kernel reported a device-side error (e.g. a bounded wait gave up)
    BNF4_ERR_NO_DEVICE = 5,    // no sm_100 GPU present
};

namespace bnf4 {

int set_error(int code, const char* fmt, ...);
int check_cuda(cudaError_t e, const char* what);
int check_launch(const char* what);

// ---------------------------------------------------------------------------------------------
// Counter-based rng (bit-compatible with the reference's src/rng.h:7-29 and
// src/efla_lm_kernels.cu:49-86).
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint64_t splitmix64_next(uint64_t& state) {
    uint64_t z = (state += 0x9e3779b97f4a7c15ULL);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

__host__ __device__ __forceinline__ uint64_t mix_u64(uint64_t a, uint64_t b) {
    uint64_t x = a ^ (b + 0x9e3779b97f4a7c15ULL + (a << 6) + (a >> 2));
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
}

__host__ __device__ __forceinline__ int ternary_from_u64(uint64_t x) {
    const uint32_t r = static_cast<uint32_t>(x & 0xFFu);
    return (r < 85u) ? -1 : ((r < 170u) ? 0 : 1);
}

__host__ __device__ __forceinline__ int noise_hash(uint64_t seed, uint64_t idx, bool use_clt, int clt_k) {
    if (!use_clt) return ternary_from_u64(mix_u64(seed, idx));
    const int k = clt_k > 0 ? clt_k : 1;
    uint64_t st = mix_u64(seed, idx);
    int sum = 0;
    for (int i = 0; i < k; ++i) sum += ternary_from_u64(splitmix64_next(st));
    return sum;
}

// Salts of the per-matrix noise streams (reference: src/train_efla_lm.cpp:3822-3833).
constexpr uint64_t kSaltEmb = 0x111111ULL, kSaltWin = 0x222222ULL, kSaltWq = 0x333333ULL, kSaltWk = 0x444444ULL,
                   kSaltWv = 0x555555ULL, kSaltWbeta = 0x666666ULL, kSaltFf1 = 0x999999ULL, kSaltFf2 = 0xAAAAAAULL,
                   kSaltHead = 0x777777ULL, kSaltHeadBias = 0x888888ULL, kSaltBetaBias = 0x9999999ULL,
                   kSaltPos = 0xBEEFF00DULL;
// Sub-streams of a matrix seed for the two rank-r factors.
constexpr uint64_t kFactorA = 0xA11CEULL, kFactorB = 0xB0BULL;

// ---------------------------------------------------------------------------------------------
// Integer rounding / clipping (reference: src/cuda_kernels.cu:46-55, src/efla_lm_kernels.cu:12-26).
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int clip_int8(int v) { return max(-127, min(127, v)); }
__device__ __forceinline__ int clip_ternary(int v) { return max(-1, min(1, v)); }
__device__ __forceinline__ int rint_to_int(float x) { return __float2int_rn(x); }

// tanh-form GELU (reference: src/cuda_kernels.cu:57-62).
__device__ __forceinline__ float gelu_tanh(float x) {
    const float c = 0.7978845608028654f;
    const float x3 = x * x * x;
    return 0.5f * x * (1.0f + tanhf(c * fmaf(0.044715f, x3, x)));
}

// gelu_tanh(x) * act_scale for values that are about to be rounded to an integer: a fast evaluation
// (x * sigmoid(2u) with the hardware exponential, absolute error far below 1e-3) decides every case except
// those within 1e-3 of a rounding boundary, which are re-evaluated with the tanhf form. The integer obtained
// after rounding is therefore the one the tanhf form gives.
__device__ __forceinline__ float gelu_scaled(float x, float act_scale) {
    const float c = 0.7978845608028654f;
    const float u = c * fmaf(0.044715f, x * x * x, x);
    float f = __fdividef(x, 1.0f + __expf(-2.0f * u)) * act_scale;
    const float d = fabsf(f - rintf(f));
    if (fabsf(d - 0.5f) < 1e-3f * fmaxf(1.0f, fabsf(f)) || !(fabsf(f) < 1e6f)) f = gelu_tanh(x) * act_scale;
    return f;
}

// clip8(rint(gelu_tanh(x) * act_scale)) without tanhf on the common path.
//   gelu_tanh(x) = 0.5 x (1 + tanh u) = x - x / (1 + e^(2u)),   u = c (x + 0.044715 x^3)
// evaluated with ex2.approx and rcp.approx (absolute error below 1e-6 |x act_scale|). The value is clamped to
// +-127, rounded with the 1.5*2^23 trick and returned still biased: q = float_as_int(t) - kRoundBiasBits, and the low
// byte of float_as_int(t) is q as an int8. `ok` is cleared when the value lies within twice the error bound of a
// rounding boundary; the caller then takes gelu_q8_exact, so the integer is always the one the tanhf form gives.
constexpr float kRoundBias = 12582912.0f;      // 1.5 * 2^23
constexpr int kRoundBiasBits = 0x4B400000;     // its bit pattern
// four signed bytes -> four floats (exact small integers)
__device__ __forceinline__ void bytes4_to_float(uint32_t w, float* out) {
    const uint32_t u = w ^ 0x80808080u;  // byte + 128 as an unsigned byte
    const float off = kRoundBias + 128.0f;
    // packed fp32 pairs: each half is the scalar subtraction
    const float2 noff = make_float2(-off, -off);
    const float2 lo = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(u, static_cast<uint32_t>(kRoundBiasBits), 0x7650)),
                                             __uint_as_float(__byte_perm(u, static_cast<uint32_t>(kRoundBiasBits), 0x7651))), noff);
    const float2 hi = __fadd2_rn(make_float2(__uint_as_float(__byte_perm(u, static_cast<uint32_t>(kRoundBiasBits), 0x7652)),
                                             __uint_as_float(__byte_perm(u, static_cast<uint32_t>(kRoundBiasBits), 0x7653))), noff);
    out[0] = lo.x; out[1] = lo.y; out[2] = hi.x; out[3] = hi.y;
}
// low bytes of four floats biased by kRoundBias -> one word of four int8
__device__ __forceinline__ uint32_t biased4_to_bytes(float a, float b, float c, float d) {
    return __byte_perm(__byte_perm(__float_as_uint(a), __float_as_uint(b), 0x0040), __byte_perm(__float_as_uint(c), __float_as_uint(d), 0x0040), 0x5410);
}
// Residual-stream update of the reference's add_scaled_to_int8 step (src/cuda_kernels.cu:3033-3143):
// clip8(old + rint(y * add_scale)), computed on biased floats; returns the new value still biased by kRoundBias.
__device__ __forceinline__ float resid_add_biased(float oldf, float y, float add_scale) {
    const float t_r = __fmul_rn(y, add_scale) + kRoundBias;
    return fminf(fmaxf(t_r + oldf, kRoundBias - 127.0f), kRoundBias + 127.0f);
}
__device__ __forceinline__ float gelu_q8_fast(float x, float act_scale, bool& ok, float& clamped) {
    const float kB = 2.0f * 0.7978845608028654f * 1.4426950408889634f;  // 2 c log2(e)
    const float kA = kB * 0.044715f;
    const float u2 = x * fmaf(x * x, kA, kB);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(u2));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(e + 1.0f));
    const float xs = x * act_scale;
    const float f = fmaf(-xs, r, xs);
    const float fc = fminf(fmaxf(f, -127.0f), 127.0f);
    const float t = fc + kRoundBias;
    const float d = fabsf(fc - (t - kRoundBias)) - 0.5f;
    ok = ok && (fabsf(d) > fmaf(fabsf(xs), 2e-6f, 2e-6f));
    clamped = fc;
    return t;
}
// max(a, b, c) in one instruction (sm_100)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// Two values at a time with packed fp32 instructions (each half rounds like the scalar instruction, so the biased results
// equal gelu_q8_fast's). `back` receives the rounded integers as floats. The boundary test is done on squares and as a
// running maximum: a value is safe iff d^2 + tol < 1/4 (stricter than |d| < 1/2 - tol for the same tol = 2e-6 (1 + |x act_scale|));
// `worst` accumulates max(d^2 + 2e-6 |x act_scale|) over the caller's group, to be compared once with kGeluSafe.
constexpr float kGeluSafe = 0.25f - 2e-6f;
__device__ __forceinline__ void gelu_q8_fast2(float x0, float x1, float act_scale, bool lower_clamp, float& worst, float& t0, float& t1,
                                              float& back0, float& back1) {
    const float kB = 2.0f * 0.7978845608028654f * 1.4426950408889634f;  // 2 c log2(e)
    const float kA = kB * 0.044715f;
    const float2 x = make_float2(x0, x1);
    const float2 u2 = __fmul2_rn(x, __ffma2_rn(__fmul2_rn(x, x), make_float2(kA, kA), make_float2(kB, kB)));
    float e0, e1, r0, r1;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e0) : "f"(u2.x));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e1) : "f"(u2.y));
    const float2 ep = __fadd2_rn(make_float2(e0, e1), make_float2(1.0f, 1.0f));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r0) : "f"(ep.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r1) : "f"(ep.y));
    const float2 xs = __fmul2_rn(x, make_float2(act_scale, act_scale));
    const float2 nxs = __fmul2_rn(x, make_float2(-act_scale, -act_scale));
    float2 f = __ffma2_rn(nxs, make_float2(r0, r1), xs);
    f.x = fminf(f.x, 127.0f);
    f.y = fminf(f.y, 127.0f);
    if (lower_clamp) {  // gelu(x) >= -0.17 |x|: only a huge act_scale can reach -127
        f.x = fmaxf(f.x, -127.0f);
        f.y = fmaxf(f.y, -127.0f);
    }
    const float2 t = __fadd2_rn(f, make_float2(kRoundBias, kRoundBias));
    const float2 back = __fadd2_rn(t, make_float2(-kRoundBias, -kRoundBias));
    const float2 d = __fadd2_rn(f, make_float2(-back.x, -back.y));
    const float2 d2 = __fmul2_rn(d, d);
    worst = fmax3(worst, fmaf(fabsf(xs.x), 2e-6f, d2.x), fmaf(fabsf(xs.y), 2e-6f, d2.y));
    t0 = t.x; t1 = t.y;
    back0 = back.x; back1 = back.y;
}
__device__ __forceinline__ int gelu_q8_exact(float x, float act_scale) {
    return clip_int8(__float2int_rn(gelu_tanh(x) * act_scale));
}
// Out-of-line form of the exact path for four values (the rare fallback of the unrolled epilogues: keeping the tanhf
// code out of line keeps their instruction footprint small). Returns the biased rounded values and the integers as floats.
static __device__ __noinline__ void gelu_q8_exact4(float x0, float x1, float x2, float x3, float act_scale, float* tb, float* fc) {
    const float xs[4] = {x0, x1, x2, x3};
#pragma unroll 1
    for (int e = 0; e < 4; ++e) {
        const int q = gelu_q8_exact(xs[e], act_scale);
        tb[e] = __int_as_float(q + kRoundBiasBits);
        fc[e] = static_cast<float>(q);
    }
}
__device__ __forceinline__ int gelu_q8(float x, float act_scale) {
    bool ok = true;
    float fc;
    const float t = gelu_q8_fast(x, act_scale, ok, fc);
    if (ok) return __float_as_int(t) - kRoundBiasBits;
    return gelu_q8_exact(x, act_scale);
}

// ---------------------------------------------------------------------------------------------
// NVFP4 number formats.
//   e2m1: magnitudes {0,.5,1,1.5,2,3,4,6}, bit 3 = sign, round-to-nearest-even, saturating.
//   ue4m3: unsigned e4m3, bias 7, subnormal step 2^-9, max 448 (0x7e), RNE, saturating.
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint32_t e2m1_encode(float x) {
    const uint32_t sign = (x < 0.0f || (x == 0.0f && (1.0f / x) < 0.0f)) ? 8u : 0u;
    const float a = x < 0.0f ? -x : x;
    uint32_t c;
    if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return sign | c;
}

__device__ __forceinline__ uint32_t ue4m3_encode(float x) {
    if (!(x > 0.0f)) return 0u;
    if (x >= 448.0f) return 0x7eu;
    if (x < 0.015625f) return static_cast<uint32_t>(__float2int_rn(x * 512.0f));
    const uint32_t bits = __float_as_uint(x);
    int e = static_cast<int>(bits >> 23) - 127;
    const uint32_t man = bits & 0x7fffffu;
    // round the 23-bit mantissa to 3 bits, ties to even
    uint32_t q = man >> 20;
    const uint32_t rem = man & 0xfffffu;
    if (rem > 0x80000u || (rem == 0x80000u && (q & 1u))) q += 1;
    if (q == 8u) { q = 0; e += 1; }
    uint32_t code = (static_cast<uint32_t>(e + 7) << 3) | q;
    return code > 0x7eu ? 0x7eu : code;
}

__host__ __device__ __forceinline__ float ue4m3_decode(uint32_t b) {
    const uint32_t e = (b >> 3) & 0xfu;
    const uint32_t m = b & 7u;
    if (e == 0u) return static_cast<float>(m) * 0.001953125f;
#if defined(__CUDA_ARCH__)
    return __uint_as_float(((e + 120u) << 23) | (m << 20));
#else
    union { uint32_t u; float f; } cv;
    cv.u = ((e + 120u) << 23) | (m << 20);
    return cv.f;
#endif
}

// Byte offset of the scale factor of (row r, 16-element K-block kb) of a [rows x K] operand:
// 512-byte atoms of 128 rows x 4 K-blocks, (r%32)*16 + ((r%128)/32)*4 + kb%4 inside an atom,
// atoms ordered K-fastest. One atom is exactly what one tcgen05.cp 32x128b.warpx4 moves to TMEM.
__host__ __device__ __forceinline__ size_t sf_offset(int r, int kb, int k_atoms) {
    return (static_cast<size_t>(r >> 7) * k_atoms + static_cast<size_t>(kb >> 2)) * 512 +
           static_cast<size_t>(r & 31) * 16 + static_cast<size_t>((r & 127) >> 5) * 4 + static_cast<size_t>(kb & 3);
}
__host__ __device__ __forceinline__ int sf_k_atoms(int K) { return ((K + 15) / 16 + 3) / 4; }
__host__ __device__ __forceinline__ size_t sf_bytes(int rows, int K) {
    return static_cast<size_t>((rows + 127) / 128) * 128 * static_cast<size_t>(sf_k_atoms(K)) * 4;
}

// Quantise one block of 16 int8 values (already in registers as 4 packed words, little-endian) to
// a ue4m3 scale byte and 16 e2m1 codes (two 32-bit words, element i in nibble i).
// row_scale multiplies the scale before rounding when use_row_scale (stacked-QKV weights).
__device__ __forceinline__ void quant_block16(const int (&w)[4], float row_scale, bool use_row_scale, uint32_t& sf_byte,
                                              uint32_t& code_lo, uint32_t& code_hi) {
    int amax = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int v = static_cast<int>(static_cast<int8_t>((w[i] >> (8 * j)) & 0xff));
            amax = max(amax, abs(v));
        }
    }
    float scale = (amax > 0) ? (static_cast<float>(amax) / 6.0f) : 1.0f;
    if (use_row_scale) scale *= row_scale;
    uint32_t sq = ue4m3_encode(scale);
    float scale_f = ue4m3_decode(sq);
    if (scale_f == 0.0f) { sq = 0x38u; scale_f = 1.0f; }
    sf_byte = sq;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int v = static_cast<int>(static_cast<int8_t>((w[i] >> (8 * j)) & 0xff));
            const uint32_t c = e2m1_encode(__fdiv_rn(static_cast<float>(v), scale_f));
            const int e = i * 4 + j;
            if (e < 8) lo |= c << (4 * e);
            else hi |= c << (4 * (e - 8));
        }
    }
    code_lo = lo;
    code_hi = hi;
}

// ---------------------------------------------------------------------------------------------
// Table-driven block quantiser. For int8 inputs both outputs depend only on (amax, |v|):
//   scale byte = sf_lut[amax],  code(v) = code_lut[amax][|v|] | sign(v) << 3
// with exactly the arithmetic of quant_block16 (amax/6 -> ue4m3, v/scale -> e2m1, IEEE division).
// The table (16 KiB + 128 B, built on the host by get_quant_lut()) lives in global memory and is read
// through the L1: the 16 values of a block share one amax, i.e. one 128-byte row.
// ---------------------------------------------------------------------------------------------
constexpr int kQuantLutCodeBytes = 128 * 128;
// A compact per-block table follows the first one, meant to be copied to shared memory: for every amax one 8-byte
// entry {fl(1 / decoded scale) as fp32 bits, scale byte}. With it the codes need no per-element look-up (e2m1x8_int below).
constexpr int kQuantBlockTabOffset = kQuantLutCodeBytes + 128;
constexpr int kQuantBlockTabBytes = 128 * 8;
constexpr int kQuantLutBytes = kQuantBlockTabOffset + kQuantBlockTabBytes;
// Device pointer to the table of the current device (allocated and filled on first use); nullptr + error on failure.
const uint8_t* get_quant_lut();

__device__ __forceinline__ void quant_block16_lut(const int (&a)[16], const uint8_t* __restrict__ lut, uint32_t& sf_byte,
                                                  uint32_t& code_lo, uint32_t& code_hi) {
    int mag[16];
    int amax = 0;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        mag[e] = min(abs(a[e]), 127);  // -128 is treated as -127 (the reference never produces it: values are clipped to +-127)
        amax = max(amax, mag[e]);
    }
    sf_byte = __ldg(lut + kQuantLutCodeBytes + amax);
    const uint8_t* row = lut + amax * 128;
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const uint32_t c = static_cast<uint32_t>(__ldg(row + mag[e])) | ((static_cast<uint32_t>(a[e]) >> 28) & 8u);
        if (e < 8) lo |= c << (4 * e);
        else hi |= c << (4 * (e - 8));
    }
    code_lo = lo;
    code_hi = hi;
}

// e2m1 codes of eight integers held as floats (|n| <= 127) under the block's reciprocal scale r = fl(1 / scale), low nibble
// first: the result of e2m1(n / scale) with IEEE division. n * r is formed with one rounding onto a grid of 2^-12 (fused
// multiply-add with 1.5 * 2^11, then subtracted again): a quotient that lies exactly on a rounding boundary of e2m1 (a
// multiple of 1/4) lands on it exactly, and any other quotient is at least 2^-6 away from every boundary (n is an integer,
// the scale has four significant bits), so the conversion instruction rounds as the division would have.
constexpr float kCodeSnap = 3072.0f;
__device__ __forceinline__ uint32_t e2m1x8_int(const float* n, float r) {
    float2 q[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        q[i] = __fadd2_rn(__ffma2_rn(make_float2(n[2 * i], n[2 * i + 1]), make_float2(r, r), make_float2(kCodeSnap, kCodeSnap)),
                          make_float2(-kCodeSnap, -kCodeSnap));
    uint32_t out;
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t}"
        : "=r"(out)
        : "f"(q[0].x), "f"(q[0].y), "f"(q[1].x), "f"(q[1].y), "f"(q[2].x), "f"(q[2].y), "f"(q[3].x), "f"(q[3].y));
    return out;
}
// The same for values still biased by kRoundBias (bit pattern = kRoundBiasBits + n).
__device__ __forceinline__ uint32_t e2m1x8_biased(const float* tb, float r) {
    float n[8];
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const float2 u = __fadd2_rn(make_float2(tb[i], tb[i + 1]), make_float2(-kRoundBias, -kRoundBias));
        n[i] = u.x;
        n[i + 1] = u.y;
    }
    return e2m1x8_int(n, r);
}

// Host twin of ue4m3_encode (used to build the table).
inline uint32_t ue4m3_encode_host(float x) {
    if (!(x > 0.0f)) return 0u;
    if (x >= 448.0f) return 0x7eu;
    if (x < 0.015625f) return static_cast<uint32_t>(nearbyintf(x * 512.0f));
    int e;
    const float m = frexpf(x, &e) * 2.0f;  // [1,2)
    e -= 1;
    int q = static_cast<int>(nearbyintf((m - 1.0f) * 8.0f));
    if (q == 8) { q = 0; e += 1; }
    const uint32_t code = (static_cast<uint32_t>(e + 7) << 3) | static_cast<uint32_t>(q);
    return code > 0x7eu ? 0x7eu : code;
}

__device__ __forceinline__ int pack4_i8(int a, int b, int c, int d) {
    return (a & 0xff) | ((b & 0xff) << 8) | ((c & 0xff) << 16) | ((d & 0xff) << 24);
}

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace bnf4
