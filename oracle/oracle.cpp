// CPU oracle for the population-evaluation hot path of catid/bitnet_nvfp4.
//
// TEST INFRASTRUCTURE ONLY. This file is the checker the CUDA library is compared against; it is
// never linked into, imported by, or called from the product library. Only the test-suite, the
// smoke check and the benchmark's cpu_baseline / reference arm may load it.
//
// It restates, in plain host C++, the arithmetic of the reference's device kernels. Each function
// cites the reference file:line it follows (paths are relative to the reference project root).
//
// Parity pins:
//   * rng / noise / ternary init / fitness shaping: pinned against the reference's own host code
//     (src/rng.h, src/train_efla_lm.cpp) compiled where it lies (see ref_host_shim.cpp).
//   * e2m1 / ue4m3 codecs and the scale-factor layout: the reference takes these from NVIDIA
//     CUTLASS (an un-vendored, unpinned submodule); pinned against golden tables produced from the
//     CUTLASS 4.5.0 headers that ship in this image (tests/golden/).
//   * forward kernels (quantisers, GEMM, EFLA, CE, update): the reference has no tests or golden
//     vectors for them and its NVFP4 path cannot run on this hardware -> "parity unpinned" for
//     those beyond the pins above; efla/CE/update are additionally cross-checked against the
//     reference's own efla_lm_kernels.cu compiled for sm_100a when a GPU is present.
//
// Floating-point contract: compiled with -ffp-contract=off; every fused multiply-add that the
// device code performs is written as an explicit fmaf() here.

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API extern "C" __attribute__((visibility("default")))

namespace orc {

// ---------------------------------------------------------------------------------------------
// rng  (src/rng.h:7-29)
// ---------------------------------------------------------------------------------------------
static inline uint64_t splitmix64(uint64_t& state) {
    uint64_t z = (state += 0x9e3779b97f4a7c15ULL);
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ULL;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebULL;
    return z ^ (z >> 31);
}

static inline uint64_t mix(uint64_t a, uint64_t b) {
    uint64_t x = a ^ (b + 0x9e3779b97f4a7c15ULL + (a << 6) + (a >> 2));
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return x;
}

static inline int8_t ternary_from_u64(uint64_t x) {
    const uint8_t r = static_cast<uint8_t>(x & 0xFF);
    if (r < 85) return -1;
    if (r < 170) return 0;
    return 1;
}

// src/efla_lm_kernels.cu:73-86 (device) and src/train_efla_lm.cpp:137-145 (host twin).
static inline int8_t noise_hash(uint64_t seed, uint64_t idx, bool use_clt, int clt_k) {
    if (!use_clt) return ternary_from_u64(mix(seed, idx));
    const int k = clt_k > 0 ? clt_k : 1;
    uint64_t st = mix(seed, idx);
    int sum = 0;
    for (int i = 0; i < k; ++i) sum += ternary_from_u64(splitmix64(st));
    return static_cast<int8_t>(sum);
}

// ---------------------------------------------------------------------------------------------
// small helpers  (src/cuda_kernels.cu:46-62, src/efla_lm_kernels.cu:12-37)
// ---------------------------------------------------------------------------------------------
static inline int8_t clip_int8(int v) { return v > 127 ? 127 : (v < -127 ? -127 : (int8_t)v); }
static inline int8_t clip_ternary(int v) { return v > 1 ? 1 : (v < -1 ? -1 : (int8_t)v); }
// __float2int_rn: round-to-nearest-even, saturating.
static inline int rint_to_int(float x) {
    if (!(x == x)) return 0;
    if (x >= 2147483648.0f) return 2147483647;
    if (x <= -2147483648.0f) return (-2147483647 - 1);
    return static_cast<int>(std::nearbyintf(x));
}
static inline float gelu(float x) {
    const float c = 0.7978845608028654f;
    const float x3 = x * x * x;
    return 0.5f * x * (1.0f + std::tanh(c * std::fmaf(0.044715f, x3, x)));
}
static inline float sigmoidf(float x) { return 1.0f / (1.0f + std::exp(-x)); }

// IEEE binary16 <-> binary32, round-to-nearest-even (matches __float2half_rn / __half2float).
static inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) return (uint16_t)(sign | (absx > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (absx >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to >= 65520 -> inf
    if (absx < 0x33000001u) return (uint16_t)sign;               // < 2^-25 (or == 2^-25 tie->0)
    int e = (int)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) {  // subnormal half
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        m &= 0x7fffffu;
    }
    const uint32_t q = m >> shift;
    const uint32_t rem = m & ((1u << shift) - 1u);
    const uint32_t half = 1u << (shift - 1);
    uint32_t h = base + q;
    if (rem > half || (rem == half && (q & 1u))) h += 1;
    return (uint16_t)(sign | h);
}
static inline float f16_to_f32(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    const uint32_t e = (h >> 10) & 0x1fu;
    const uint32_t m = h & 0x3ffu;
    uint32_t x;
    if (e == 0) {
        if (m == 0) {
            x = sign;
        } else {
            const float v = (float)m * 5.9604644775390625e-08f;  // m * 2^-24
            std::memcpy(&x, &v, 4);
            x |= sign;
        }
    } else if (e == 31) {
        x = sign | 0x7f800000u | (m << 13);
    } else {
        x = sign | ((e + 112u) << 23) | (m << 13);
    }
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

// ---------------------------------------------------------------------------------------------
// number formats. The reference uses cutlass::float_e2m1_t / float_ue4m3_t
// (src/cuda_kernels.cu:1420-1421,1581,1611). CUTLASS is absent from the reference tree; these are
// restatements of the published formats: e2m1 = {0,.5,1,1.5,2,3,4,6} with sign bit 3, RNE,
// saturating; ue4m3 = unsigned e4m3 (bias 7, subnormal step 2^-9, max 448 = 0x7e), RNE, saturating.
// ---------------------------------------------------------------------------------------------
static inline uint8_t e2m1_encode(float x) {
    const uint8_t sign = std::signbit(x) ? 0x8 : 0x0;
    const float a = std::fabs(x);
    uint8_t c;
    if (!(a == a)) c = 7;
    else if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return sign | c;
}
static const float kE2M1[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
static inline float e2m1_decode(uint8_t c) {
    const float v = kE2M1[c & 7];
    return (c & 8) ? -v : v;
}
static inline uint8_t ue4m3_encode(float x) {
    if (!(x > 0.0f)) return 0;
    if (x >= 448.0f) return 0x7e;
    if (x < 0.015625f) {  // below min normal 2^-6: subnormal grid of 2^-9
        const int q = (int)std::nearbyintf(x * 512.0f);
        return (uint8_t)q;  // q == 8 lands on 0x08 = min normal
    }
    int e;
    const float fr = std::frexp(x, &e);  // x = fr * 2^e, fr in [0.5,1)
    const float m = fr * 2.0f;            // [1,2)
    e -= 1;
    int q = (int)std::nearbyintf((m - 1.0f) * 8.0f);
    if (q == 8) { q = 0; e += 1; }
    int code = ((e + 7) << 3) | q;
    if (code > 0x7e) code = 0x7e;
    return (uint8_t)code;
}
static inline float ue4m3_decode(uint8_t b) {
    const int e = (b >> 3) & 0xf;
    const int m = b & 7;
    if (e == 0) return (float)m * 0.001953125f;  // m * 2^-9
    if (e == 15 && m == 7) return NAN;
    return std::ldexp(1.0f + (float)m * 0.125f, e - 7);
}

// Scale-factor byte offset of (row r, K-block kb) for a [rows x K] operand: the
// Sm1xxBlockScaledConfig<16> K-major atom ((32,4),(16,4)):((16,4),(0,1)) tiled K-fastest
// (src/cuda_kernels.cu:3837-3847, 4019-4020 use cutlass/detail/sm100_blockscaled_layout.hpp).
static inline size_t sf_offset(int r, int kb, int K) {
    const int kt = ((K + 15) / 16 + 3) / 4;
    return ((size_t)(r / 128) * kt + (size_t)(kb / 4)) * 512 + (size_t)(r % 32) * 16 +
           (size_t)((r % 128) / 32) * 4 + (size_t)(kb % 4);
}
static inline size_t sf_bytes(int rows, int K) {
    const int kt = ((K + 15) / 16 + 3) / 4;
    return (size_t)((rows + 127) / 128) * 128 * (size_t)kt * 4;
}

// One 16-element block: int8 values -> scale byte + 16 e2m1 codes
// (src/cuda_kernels.cu:1574-1611). row_scale multiplies the scale before ue4m3 rounding
// (fused-QKV stack, src/cuda_kernels.cu:2805-2810); pass 1 otherwise.
static inline void quant_block16(const int8_t* v, int count_in, float row_scale, bool use_row_scale,
                                 uint8_t* sf_byte, uint8_t* codes /*16*/) {
    float max_abs = 0.0f;
    for (int i = 0; i < count_in; ++i) max_abs = std::max(max_abs, std::fabs((float)v[i]));
    float scale = (max_abs > 0.0f) ? (max_abs / 6.0f) : 1.0f;
    if (use_row_scale) scale *= row_scale;
    uint8_t sq = ue4m3_encode(scale);
    float scale_f = ue4m3_decode(sq);
    if (scale_f == 0.0f) { sq = 0x38; scale_f = 1.0f; }
    *sf_byte = sq;
    for (int i = 0; i < 16; ++i) {
        const float vf = (i < count_in ? (float)v[i] : 0.0f) / scale_f;
        codes[i] = e2m1_encode(vf);
    }
}

static inline void store_nibble(uint8_t* out, size_t elem, uint8_t code) {
    uint8_t& b = out[elem >> 1];
    if (elem & 1) b = (uint8_t)((b & 0x0f) | (code << 4));
    else b = (uint8_t)((b & 0xf0) | (code & 0x0f));
}

// Quantise one int8 row of `cols_in` values into codes (row stride cols_out) + scale bytes.
static void quant_row(const int8_t* row_vals, int row, int cols_in, int cols_out, float row_scale,
                      bool use_row_scale, uint8_t* out, uint8_t* sf) {
    for (int k0 = 0; k0 < cols_out; k0 += 16) {
        const int cin = std::max(0, std::min(16, cols_in - k0));
        const int cout = std::min(16, cols_out - k0);
        uint8_t sq, codes[16];
        quant_block16(row_vals + k0, cin, row_scale, use_row_scale, &sq, codes);
        sf[sf_offset(row, k0 / 16, cols_out)] = sq;
        for (int i = 0; i < cout; ++i) store_nibble(out, (size_t)row * cols_out + k0 + i, codes[i]);
    }
}

}  // namespace orc

using namespace orc;

// =============================================================================================
// C entry points (loaded with ctypes by the tests / bench)
// =============================================================================================

// Thread count of the OpenMP loops: launchers such as torchrun export OMP_NUM_THREADS=1 to their workers.
ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads() {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

ORC_API uint64_t orc_splitmix64(uint64_t* state) { return splitmix64(*state); }
ORC_API uint64_t orc_mix(uint64_t a, uint64_t b) { return mix(a, b); }
ORC_API int orc_ternary_from_u64(uint64_t x) { return ternary_from_u64(x); }
ORC_API int orc_noise_hash(uint64_t seed, uint64_t idx, int use_clt, int clt_k) {
    return noise_hash(seed, idx, use_clt != 0, clt_k);
}
// fill_ternary_noise (src/efla_lm_kernels.cu:352-360)
ORC_API void orc_fill_noise(int8_t* out, size_t n, uint64_t seed, int use_clt, int clt_k) {
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i) out[i] = noise_hash(seed, (uint64_t)i, use_clt != 0, clt_k);
}
// TernaryMatrix::init_rand (src/train_efla_lm.cpp:174-183)
ORC_API void orc_init_rand_ternary(int8_t* out, size_t n, uint64_t seed) {
    uint64_t st = seed;
    for (size_t i = 0; i < n; ++i) out[i] = ternary_from_u64(splitmix64(st));
}
// fill_pair_seeds (src/efla_lm_kernels.cu:1844-1852)
ORC_API void orc_fill_pair_seeds(uint64_t base_seed, uint64_t epoch, int pairs, uint64_t* out) {
    for (int p = 0; p < pairs; ++p) out[p] = mix(base_seed, mix(epoch, (uint64_t)p));
}

ORC_API int orc_e2m1_encode(float x) { return e2m1_encode(x); }
ORC_API float orc_e2m1_decode(int c) { return e2m1_decode((uint8_t)c); }
ORC_API int orc_ue4m3_encode(float x) { return ue4m3_encode(x); }
ORC_API float orc_ue4m3_decode(int b) { return ue4m3_decode((uint8_t)b); }
ORC_API size_t orc_sf_offset(int r, int kb, int K) { return sf_offset(r, kb, K); }
ORC_API size_t orc_sf_bytes(int rows, int K) { return sf_bytes(rows, K); }
ORC_API int orc_f32_to_f16(float f) { return f32_to_f16(f); }
ORC_API float orc_f16_to_f32(int h) { return f16_to_f32((uint16_t)h); }

// ---------------------------------------------------------------------------------------------
// a1: nvfp4_quantize_a / nvfp4_quantize_b (src/cuda_kernels.cu:1545-1625, 4013-4037, 4240-4264)
// in: int8 [rows x k_in]; out: packed e2m1 [rows x k_out], sf in the layout above.
// ---------------------------------------------------------------------------------------------
ORC_API void orc_quantize_rowmajor(const int8_t* in, int rows, int k_in, int k_out, uint8_t* out, uint8_t* sf) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        std::vector<int8_t> tmp((size_t)k_out + 16, 0);
        for (int j = 0; j < std::min(k_in, k_out); ++j) tmp[j] = in[(size_t)r * k_in + j];
        quant_row(tmp.data(), r, std::min(k_in, k_out), k_out, 1.0f, false, out, sf);
    }
}

// nvfp4_quantize_wqkv_fused (src/cuda_kernels.cu:2748-2854): rows [Wq;Wk;Wv;wbeta], 3H+1 valid rows,
// per-group output scale folded into the block scale before ue4m3 rounding.
ORC_API void orc_quantize_wqkv_fused(const int8_t* wq, const int8_t* wk, const int8_t* wv, const int8_t* wb,
                                     int hidden, int k_out, float q_scale, float k_scale, float v_scale,
                                     float b_scale, uint8_t* out, uint8_t* sf) {
    const int rows = 3 * hidden + 1;
#pragma omp parallel for schedule(static)
    for (int row = 0; row < rows; ++row) {
        const int group = row / hidden;
        const int rig = row - group * hidden;
        const int8_t* src;
        float rs;
        if (group == 0) { src = wq + (size_t)rig * hidden; rs = q_scale; }
        else if (group == 1) { src = wk + (size_t)rig * hidden; rs = k_scale; }
        else if (group == 2) { src = wv + (size_t)rig * hidden; rs = v_scale; }
        else { src = wb; rs = b_scale; }
        std::vector<int8_t> tmp((size_t)k_out + 16, 0);
        for (int j = 0; j < std::min(hidden, k_out); ++j) tmp[j] = src[j];
        quant_row(tmp.data(), row, std::min(hidden, k_out), k_out, rs, true, out, sf);
    }
}

// ---------------------------------------------------------------------------------------------
// a2: fused quantise front-ends. Each produces the int8 copy, the e2m1 codes and the scale bytes.
// ---------------------------------------------------------------------------------------------
// embedding_lookup_noise_quantize_nvfp4 (src/cuda_kernels.cu:2014-2109).
// tokens: one token per row at stride token_stride. Dense-noise form.
ORC_API void orc_embedding_quant(const uint8_t* tokens, int token_stride, const int8_t* emb_w,
                                 const int8_t* emb_noise, int hidden, int rows, float noise_scale,
                                 int anti_sign, int8_t* out_q, uint8_t* out, uint8_t* sf) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const int tok = tokens[(size_t)r * token_stride];
        std::vector<int8_t> v((size_t)hidden + 16, 0);
        for (int j = 0; j < hidden; ++j) {
            float f = (float)emb_w[(size_t)tok * hidden + j];
            if (emb_noise && noise_scale != 0.0f && anti_sign != 0) {
                f = std::fmaf((float)anti_sign * noise_scale, (float)emb_noise[(size_t)tok * hidden + j], f);
            }
            v[j] = clip_int8(rint_to_int(f));
            out_q[(size_t)r * hidden + j] = v[j];
        }
        quant_row(v.data(), r, hidden, hidden, 1.0f, false, out, sf);
    }
}

// Rank-r embedding perturbation: embed_update_lora_kernel's element formula
// (src/cuda_kernels.cu:1360-1389): ev = emb[tok][j] + s * sum_r A[tok][r]*B[j][r], rounded + clipped.
ORC_API void orc_embedding_lowrank_quant(const uint8_t* tokens, int token_stride, const int8_t* emb_w,
                                         const int8_t* A, const int8_t* B, int rank, int hidden, int rows,
                                         float scale, int8_t* out_q, uint8_t* out, uint8_t* sf) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const int tok = tokens[(size_t)r * token_stride];
        std::vector<int8_t> v((size_t)hidden + 16, 0);
        for (int j = 0; j < hidden; ++j) {
            int pert = 0;
            for (int q = 0; q < rank; ++q) pert += (int)A[(size_t)tok * rank + q] * (int)B[(size_t)j * rank + q];
            const float ev = std::fmaf(scale, (float)pert, (float)emb_w[(size_t)tok * hidden + j]);
            v[j] = clip_int8(rint_to_int(ev));
            out_q[(size_t)r * hidden + j] = v[j];
        }
        quant_row(v.data(), r, hidden, hidden, 1.0f, false, out, sf);
    }
}

// add_pos_gelu_quantize_nvfp4 (src/cuda_kernels.cu:2260-2349). pos: per-row pointer offset given by
// pos_row[r] (index of the positional row to add), so one call can cover all time steps.
ORC_API void orc_add_pos_gelu_quant(const float* in, const float* pos, const int* pos_row, int hidden, int rows,
                                    float act_scale, int8_t* out_q, uint8_t* out, uint8_t* sf) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        const float* p = pos + (size_t)(pos_row ? pos_row[r] : 0) * hidden;
        std::vector<int8_t> v((size_t)hidden + 16, 0);
        for (int j = 0; j < hidden; ++j) {
            float f = in[(size_t)r * hidden + j] + p[j];
            f = gelu(f) * act_scale;
            v[j] = clip_int8(rint_to_int(f));
            out_q[(size_t)r * hidden + j] = v[j];
        }
        quant_row(v.data(), r, hidden, hidden, 1.0f, false, out, sf);
    }
}

// gelu_quantize_nvfp4 (src/cuda_kernels.cu:2500-2589) and activation_quantize_nvfp4 (:1783-1878).
// mode 0: none, 1: relu, 2: tanh(f/127)*127, 3: gelu(f)*act_scale.
ORC_API void orc_activation_quant(const float* in, int rows, int cols_in, int cols_out, int mode, float act_scale,
                                  int8_t* out_q, uint8_t* out, uint8_t* sf) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        std::vector<int8_t> v((size_t)cols_out + 16, 0);
        const int n = std::min(cols_in, cols_out);
        for (int j = 0; j < n; ++j) {
            float f = in[(size_t)r * cols_in + j];
            if (mode == 1) { if (f < 0.0f) f = 0.0f; }
            else if (mode == 2) f = std::tanh(f / 127.0f) * 127.0f;
            else if (mode == 3) f = gelu(f) * act_scale;
            v[j] = clip_int8(rint_to_int(f));
            out_q[(size_t)r * cols_out + j] = v[j];
        }
        quant_row(v.data(), r, n, cols_out, 1.0f, false, out, sf);
    }
}

// absmean_norm_q_nvfp4 (src/cuda_kernels.cu:2928-3031) and, when add_in != nullptr,
// add_scaled_to_int8_absmean_norm_q_nvfp4 (:3033-3143): x8 = clip8(x8 + rint(y*add_scale)) first.
// Sum of |int8| is exact in fp32 for hidden <= 2^17, so summation order is immaterial.
ORC_API void orc_absmean_norm_q(int8_t* inout, const float* add_in, int hidden, int rows, float add_scale,
                                float norm_scale, int8_t* out_q, uint8_t* out, uint8_t* sf) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        int8_t* x = inout + (size_t)r * hidden;
        float sum_abs = 0.0f;
        for (int j = 0; j < hidden; ++j) {
            if (add_in) {
                const int q = rint_to_int(add_in[(size_t)r * hidden + j] * add_scale);
                x[j] = clip_int8((int)x[j] + q);
            }
            sum_abs += std::fabs((float)x[j]);
        }
        float abs_mean = sum_abs / (float)hidden;
        if (abs_mean < 1.0f) abs_mean = 1.0f;
        const float inv = norm_scale / abs_mean;
        std::vector<int8_t> v((size_t)hidden + 16, 0);
        for (int j = 0; j < hidden; ++j) {
            v[j] = clip_int8(rint_to_int((float)x[j] * inv));
            out_q[(size_t)r * hidden + j] = v[j];
        }
        quant_row(v.data(), r, hidden, hidden, 1.0f, false, out, sf);
    }
}

// ---------------------------------------------------------------------------------------------
// a4: gemm_ternary_f_nvfp4 (src/cuda_kernels.cu:4342-4473; CUTLASS block-scaled semantics):
// D[m,n] = alpha * sum_kb( sfa[m,kb]*sfb[n,kb] * sum_{k in kb} a[m,k]*b[n,k] ) + beta*C[m,n]
// a5 (gelu_i8 != 0): D8 = clip8(rint(gelu(D) * act_scale))  (src/cuda_kernels.cu:4475-4607,
// 3178-3194; GELU here is the in-tree tanhf form, src/cuda_kernels.cu:57-62).
// The 16-element inner sums are exact (operands are multiples of 0.5 with |v| <= 6).
// ---------------------------------------------------------------------------------------------
static void decode_operand(const uint8_t* codes, const uint8_t* sf, int rows, int K, std::vector<int8_t>& v2,
                           std::vector<float>& s) {
    const int nkb = K / 16;
    v2.assign((size_t)rows * K, 0);
    s.assign((size_t)rows * nkb, 0.0f);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        for (int k = 0; k < K; ++k) {
            const size_t e = (size_t)r * K + k;
            const uint8_t c = (codes[e >> 1] >> ((e & 1) * 4)) & 0xf;
            v2[e] = (int8_t)(int)(e2m1_decode(c) * 2.0f);
        }
        for (int kb = 0; kb < nkb; ++kb) s[(size_t)r * nkb + kb] = ue4m3_decode(sf[sf_offset(r, kb, K)]);
    }
}

ORC_API void orc_gemm_nvfp4(const uint8_t* a, const uint8_t* b, const uint8_t* sfa, const uint8_t* sfb, int m,
                            int n, int k, float alpha, float beta, const float* c, int ldc, float* d, int ldd,
                            int gelu_i8, float act_scale, int8_t* d8) {
    std::vector<int8_t> a2, b2;
    std::vector<float> sa, sb;
    decode_operand(a, sfa, m, k, a2, sa);
    decode_operand(b, sfb, n, k, b2, sb);
    const int nkb = k / 16;
#pragma omp parallel for schedule(static)
    for (int i = 0; i < m; ++i) {
        const int8_t* ar = &a2[(size_t)i * k];
        for (int j = 0; j < n; ++j) {
            const int8_t* br = &b2[(size_t)j * k];
            float acc = 0.0f;
            for (int kb = 0; kb < nkb; ++kb) {
                int dot = 0;
                for (int t = 0; t < 16; ++t) dot += (int)ar[kb * 16 + t] * (int)br[kb * 16 + t];
                acc = std::fmaf(sa[(size_t)i * nkb + kb] * sb[(size_t)j * nkb + kb], (float)dot * 0.25f, acc);
            }
            float v = alpha * acc;
            if (beta != 0.0f) v = std::fmaf(beta, c[(size_t)i * ldc + j], v);
            if (gelu_i8) d8[(size_t)i * ldd + j] = clip_int8(rint_to_int(gelu(v) * act_scale));
            else d[(size_t)i * ldd + j] = v;
        }
    }
}

// a3: gemm_ternary_f (src/cuda_kernels.cu:740-762, 163-192): exact int32 sum per 256-column group,
// fp32 across groups with scale_x[g], then * out_scale. x [batch x cols], w [rows x cols].
ORC_API void orc_gemm_ternary_f(const int8_t* x, const int8_t* w, const float* scale_x, int rows, int cols,
                                int batch, float out_scale, float* out) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < batch; ++b) {
        for (int i = 0; i < rows; ++i) {
            const int8_t* xr = x + (size_t)b * cols;
            const int8_t* wr = w + (size_t)i * cols;
            float acc = 0.0f;
            int j = 0;
            for (; j + 256 <= cols; j += 256) {
                int s = 0;
                for (int t = 0; t < 256; ++t) s += (int)xr[j + t] * (int)wr[j + t];
                acc = std::fmaf(scale_x ? scale_x[j / 256] : 1.0f, (float)s, acc);
            }
            for (; j < cols; j += 32) {
                int s = 0;
                for (int t = 0; t < 32 && j + t < cols; ++t) s += (int)xr[j + t] * (int)wr[j + t];
                acc = std::fmaf(scale_x ? scale_x[j / 256] : 1.0f, (float)s, acc);
            }
            out[(size_t)b * rows + i] = acc * out_scale;
        }
    }
}

// a6 rank-r: lora_compute_t (src/cuda_kernels.cu:370-390): t[b,r] = sum_j x[b,j]*B[j,r] (exact int32).
ORC_API void orc_lora_compute_t(const int8_t* x, const int8_t* B, int cols, int batch, int rank, int32_t* t) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < batch; ++b)
        for (int r = 0; r < rank; ++r) {
            int acc = 0;
            for (int j = 0; j < cols; ++j) acc += (int)x[(size_t)b * cols + j] * (int)B[(size_t)j * rank + r];
            t[(size_t)b * rank + r] = acc;
        }
}
// lora_add (src/cuda_kernels.cu:392-410) / epilogue of gemm_lora_f_kernel (:1293-1303):
// out[b,i] += scale * float(sum_r t[b,r]*A[i,r]).
ORC_API void orc_lora_add(const int32_t* t, const int8_t* A, int rows, int batch, int rank, float scale, float* out,
                          int ldo) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < rows; ++i) {
            int pert = 0;
            for (int r = 0; r < rank; ++r) pert += t[(size_t)b * rank + r] * (int)A[(size_t)i * rank + r];
            float& o = out[(size_t)b * ldo + i];
            o = std::fmaf(scale, (float)pert, o);
        }
}

// ---------------------------------------------------------------------------------------------
// a7: EFLA step on the fused-QKV row layout, fp16 state (src/efla_lm_kernels.cu:821-913 prepare,
// :1108-1141 kS, :1186-1197 diff, :1328-1356 update with __floats2half2_rn, :1563-1590 readout;
// compact single-kernel statement :590-726). heads*head_dim == hidden; heads==1 is the reference.
// qkv row: [q(H) | k(H) | v(H) | beta_raw]; S: [batch][heads][hd][hd] fp16 bits (d-major, n fastest).
// beta is one scalar per row; q-norm, lambda and alpha are per head.
// ---------------------------------------------------------------------------------------------
static void efla_step_row(uint16_t* S, const float* qkv_row, float beta_bias, int hidden, int heads, int method,
                          float eps, float* out_row) {
    const int hd = hidden / heads;
    const float beta = sigmoidf(qkv_row[3 * hidden] + beta_bias);
    std::vector<float> qn(hd), ku(hd), kS(hd), diff(hd);
    for (int h = 0; h < heads; ++h) {
        const float* q = qkv_row + h * hd;
        const float* k = qkv_row + hidden + h * hd;
        const float* v = qkv_row + 2 * hidden + h * hd;
        uint16_t* Sh = S + (size_t)h * hd * hd;
        float qss = 0.0f, kss = 0.0f;
        for (int j = 0; j < hd; ++j) { qss = std::fmaf(q[j], q[j], qss); kss = std::fmaf(k[j], k[j], kss); }
        const float q_inv = 1.0f / std::sqrt(qss + eps);
        const float lambda = kss < eps ? eps : kss;
        float alpha;
        if (method == 0) alpha = beta;
        else alpha = -std::expm1(-(beta * lambda)) / (lambda + eps);
        const float kinv = (method == 0) ? 1.0f / std::sqrt(lambda + eps) : 1.0f;
        for (int j = 0; j < hd; ++j) { qn[j] = q[j] * q_inv; ku[j] = (method == 0) ? k[j] * kinv : k[j]; }
        for (int n = 0; n < hd; ++n) {
            float acc = 0.0f;
            for (int d = 0; d < hd; ++d) acc = std::fmaf(ku[d], f16_to_f32(Sh[(size_t)d * hd + n]), acc);
            kS[n] = acc;
            diff[n] = v[n] - acc;
        }
        for (int d = 0; d < hd; ++d) {
            const float sc = alpha * ku[d];
            for (int n = 0; n < hd; ++n) {
                const float s = std::fmaf(sc, diff[n], f16_to_f32(Sh[(size_t)d * hd + n]));
                Sh[(size_t)d * hd + n] = f32_to_f16(s);
            }
        }
        for (int n = 0; n < hd; ++n) {
            float acc = 0.0f;
            for (int d = 0; d < hd; ++d) acc = std::fmaf(f16_to_f32(Sh[(size_t)d * hd + n]), qn[d], acc);
            out_row[h * hd + n] = acc;
        }
    }
}

ORC_API void orc_efla_step_half_qkv_fused(uint16_t* S, const float* qkv, int fused_cols, float beta_bias, int hidden,
                                          int heads, int batch, int method, float eps, float* out) {
#pragma omp parallel for schedule(static)
    for (int b = 0; b < batch; ++b)
        efla_step_row(S + (size_t)b * hidden * (hidden / heads), qkv + (size_t)b * fused_cols, beta_bias, hidden,
                      heads, method, eps, out + (size_t)b * hidden);
}

// ---------------------------------------------------------------------------------------------
// Inputs of the single-GEMM benchmark configuration. The reference has no Gaussian generator (its noise is the CLT sum of
// ternary draws above), so the N(0,1) map for fp32 test inputs is DEFINED here: Box-Muller on two 53-bit uniforms drawn
// with the reference's counter functions, element idx of stream (seed, tag) -> st = mix(mix(seed, tag), idx),
// u1 = ((splitmix64(st) >> 11) + 1) 2^-53 in (0, 1], u2 = (splitmix64(st) >> 11) 2^-53, z = sqrt(-2 ln u1) cos(2 pi u2),
// evaluated in double and rounded once to fp32 after the scale.
// ---------------------------------------------------------------------------------------------
ORC_API void orc_gaussian_f32(uint64_t seed, uint64_t tag, size_t n, float scale, float* out) {
    const uint64_t base = orc_mix(seed, tag);
#pragma omp parallel for schedule(static)
    for (long long i = 0; i < (long long)n; ++i) {
        uint64_t st = orc_mix(base, (uint64_t)i);
        const double u1 = (double)((orc_splitmix64(&st) >> 11) + 1) * (1.0 / 9007199254740992.0);
        const double u2 = (double)(orc_splitmix64(&st) >> 11) * (1.0 / 9007199254740992.0);
        out[i] = (float)((double)scale * std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925286766559 * u2));
    }
}

// fp32 rows straight to NVFP4 (no int8 stage): the block rule of nvfp4_quantize_rowmajor (src/cuda_kernels.cu:1545-1625)
// applied to fp32 values: amax = max |x|, s = amax > 0 ? amax / 6 : 1, sq = ue4m3(s) (1.0 if that decodes to 0),
// codes = e2m1(x / float(sq)). Columns past k_in are zero.
ORC_API void orc_quantize_direct_f32(const float* in, int rows, int k_in, int k_out, uint8_t* codes, uint8_t* sf) {
    std::memset(codes, 0, (size_t)rows * k_out / 2);
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r)
        for (int kb = 0; kb < k_out / 16; ++kb) {
            float x[16], amax = 0.0f;
            for (int e = 0; e < 16; ++e) {
                const int c = kb * 16 + e;
                x[e] = c < k_in ? in[(size_t)r * k_in + c] : 0.0f;
                amax = std::fmax(amax, std::fabs(x[e]));
            }
            const float s = amax > 0.0f ? amax / 6.0f : 1.0f;
            int sq = orc_ue4m3_encode(s);
            float sfv = orc_ue4m3_decode(sq);
            if (sfv == 0.0f) { sq = 0x38; sfv = 1.0f; }
            sf[orc_sf_offset(r, kb, k_out)] = (uint8_t)sq;
            for (int e = 0; e < 16; ++e) {
                const size_t idx = (size_t)r * k_out + kb * 16 + e;
                const int c = orc_e2m1_encode(x[e] / sfv);
                codes[idx / 2] |= (uint8_t)(c << (4 * (idx & 1)));
            }
        }
}

// ---------------------------------------------------------------------------------------------
// What-if variants of the scan, used only to measure how far a faster formulation may depart from the
// reference's rounding before the per-member loss leaves its 1e-4 bar. state_round_every: 1 = the reference
// (state rounded to fp16 after every token, src/efla_lm_kernels.cu:1349); C > 1 = state carried in fp32 and
// rounded to fp16 after every C-th token (a chunked delta rule that keeps an fp16 state between chunks);
// 0 = never rounded. operand_bits: 0 = fp32 operands (the reference); otherwise q_hat, k, alpha*k and v-k.S are
// rounded to that many explicit mantissa bits (10 = tf32/fp16 precision, 7 = bf16) before every product, which is
// what a tensor-core contraction with fp32 accumulation would see. Process-global; default = the reference.
// ---------------------------------------------------------------------------------------------
static int g_state_round_every = 1;
static int g_operand_bits = 0;
ORC_API void orc_set_efla_variant(int state_round_every, int operand_bits) {
    g_state_round_every = state_round_every;
    g_operand_bits = operand_bits;
}

static inline float round_mantissa(float x, int bits) {
    if (bits <= 0 || bits >= 23) return x;
    uint32_t u;
    std::memcpy(&u, &x, 4);
    const int drop = 23 - bits;
    const uint32_t half = (1u << (drop - 1)) - 1u + ((u >> drop) & 1u);  // round to nearest even
    u = (u + half) & ~((1u << drop) - 1u);
    std::memcpy(&x, &u, 4);
    return x;
}

static void efla_scan_variant_seq(const float* qkv, int fused_cols, float beta_bias, int hidden, int heads, int T,
                                  int method, float eps, float* out, int round_every, int bits) {
    const int hd = hidden / heads;
    std::vector<float> S((size_t)hidden * hd, 0.0f), qn(hd), ku(hd), ak(hd), diff(hd);
    for (int t = 0; t < T; ++t) {
        const float* row = qkv + (size_t)t * fused_cols;
        const float beta = sigmoidf(row[3 * hidden] + beta_bias);
        for (int h = 0; h < heads; ++h) {
            const float* q = row + h * hd;
            const float* k = row + hidden + h * hd;
            const float* v = row + 2 * hidden + h * hd;
            float* Sh = S.data() + (size_t)h * hd * hd;
            float qss = 0.0f, kss = 0.0f;
            for (int j = 0; j < hd; ++j) { qss = std::fmaf(q[j], q[j], qss); kss = std::fmaf(k[j], k[j], kss); }
            const float q_inv = 1.0f / std::sqrt(qss + eps);
            const float lambda = kss < eps ? eps : kss;
            const float alpha = method == 0 ? beta : -std::expm1(-(beta * lambda)) / (lambda + eps);
            const float kinv = (method == 0) ? 1.0f / std::sqrt(lambda + eps) : 1.0f;
            for (int j = 0; j < hd; ++j) {
                const float kj = (method == 0) ? k[j] * kinv : k[j];
                qn[j] = round_mantissa(q[j] * q_inv, bits);
                ku[j] = round_mantissa(kj, bits);
                ak[j] = round_mantissa(alpha * kj, bits);
            }
            for (int n = 0; n < hd; ++n) {
                float acc = 0.0f;
                for (int d = 0; d < hd; ++d) acc = std::fmaf(ku[d], Sh[(size_t)d * hd + n], acc);
                diff[n] = round_mantissa(v[n] - acc, bits);
            }
            const bool round_now = round_every > 0 && ((t + 1) % round_every == 0);
            for (int d = 0; d < hd; ++d)
                for (int n = 0; n < hd; ++n) {
                    const float s = std::fmaf(ak[d], diff[n], Sh[(size_t)d * hd + n]);
                    Sh[(size_t)d * hd + n] = round_now ? f16_to_f32(f32_to_f16(s)) : s;
                }
            for (int n = 0; n < hd; ++n) {
                float acc = 0.0f;
                for (int d = 0; d < hd; ++d) acc = std::fmaf(Sh[(size_t)d * hd + n], qn[d], acc);
                out[(size_t)t * hidden + h * hd + n] = acc;
            }
        }
    }
}

// Sequence form: qkv [seqs][T][fused_cols], state zero-initialised per sequence, out [seqs][T][hidden].
// beta_bias_seq: one value per sequence (per-member perturbed bias).
ORC_API void orc_efla_scan(const float* qkv, int fused_cols, const float* beta_bias_seq, int hidden, int heads,
                           int seqs, int T, int method, float eps, float* out) {
    const int hd = hidden / heads;
    if (g_state_round_every != 1 || g_operand_bits != 0) {
#pragma omp parallel for schedule(dynamic, 1)
        for (int s = 0; s < seqs; ++s)
            efla_scan_variant_seq(qkv + (size_t)s * T * fused_cols, fused_cols, beta_bias_seq[s], hidden, heads, T, method,
                                  eps, out + (size_t)s * T * hidden, g_state_round_every, g_operand_bits);
        return;
    }
#pragma omp parallel for schedule(dynamic, 1)
    for (int s = 0; s < seqs; ++s) {
        std::vector<uint16_t> S((size_t)hidden * hd, 0);
        for (int t = 0; t < T; ++t)
            efla_step_row(S.data(), qkv + ((size_t)s * T + t) * fused_cols, beta_bias_seq[s], hidden, heads, method,
                          eps, out + ((size_t)s * T + t) * hidden);
    }
}

// ---------------------------------------------------------------------------------------------
// a10: cross_entropy_loss (src/efla_lm_kernels.cu:252-311). Returns the SUM over rows of
// -(v_y - max - log(sum exp(v - max) + 1e-9)), v = logit + bias + bns*bias_noise.
// Row losses are fp32; the sum over rows is taken in double (the reference uses unordered float
// atomics, src/efla_lm_kernels.cu:309).
// ---------------------------------------------------------------------------------------------
ORC_API double orc_cross_entropy_sum(const float* logits, int ld, const float* bias, const float* bias_noise,
                                     float bns, const uint8_t* targets, int target_stride, int vocab, int rows,
                                     float* row_loss) {
    double total = 0.0;
#pragma omp parallel for schedule(static) reduction(+ : total)
    for (int r = 0; r < rows; ++r) {
        const float* lg = logits + (size_t)r * ld;
        auto at = [&](int i) {
            float v = lg[i];
            if (bias) v += bias[i];
            if (bias_noise) v = std::fmaf(bns, bias_noise[i], v);
            return v;
        };
        float maxv = -INFINITY;
        for (int i = 0; i < vocab; ++i) maxv = std::max(maxv, at(i));
        float sum = 0.0f;
        for (int i = 0; i < vocab; ++i) sum += std::exp(at(i) - maxv);
        const int y = targets[(size_t)r * target_stride];
        const float lp = at(y) - maxv - std::log(sum + 1e-9f);
        if (row_loss) row_loss[r] = -lp;
        total += (double)(-lp);
    }
    return total;
}

// ---------------------------------------------------------------------------------------------
// a11: shape_pair_weights (src/train_efla_lm.cpp:3898-3952). mode = the reference's
// TrainConfig::FitnessMode value (src/train_efla_lm.cpp:260): 0 sign, 1 z-score, 2 centered rank.
// Ties in the rank sort are broken by index (the reference's std::sort leaves them unspecified).
// ---------------------------------------------------------------------------------------------
ORC_API void orc_shape_pair_weights(float* w, int n, int mode, float clip) {
    if (n <= 0) return;
    if (mode == 0) {
        for (int i = 0; i < n; ++i) w[i] = w[i] > 0.0f ? 1.0f : (w[i] < 0.0f ? -1.0f : 0.0f);
        return;
    }
    if (mode == 2) {
        std::vector<int> order(n);
        for (int i = 0; i < n; ++i) order[i] = i;
        std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return w[a] < w[b]; });
        std::vector<float> ranked(n);
        if (n == 1) ranked[0] = 0.0f;
        else
            for (int r = 0; r < n; ++r) ranked[order[r]] = (float)r / (float)(n - 1) - 0.5f;
        for (int i = 0; i < n; ++i) w[i] = ranked[i];
    }
    float mean = 0.0f;
    for (int i = 0; i < n; ++i) mean += w[i];
    mean /= (float)n;
    float var = 0.0f;
    for (int i = 0; i < n; ++i) var += (w[i] - mean) * (w[i] - mean);
    var /= (float)n;
    const float stdv = std::sqrt(var) + 1e-6f;
    for (int i = 0; i < n; ++i) {
        float d = (w[i] - mean) / stdv;
        if (d > clip) d = clip;
        if (d < -clip) d = -clip;
        w[i] = d;
    }
}

// ---------------------------------------------------------------------------------------------
// a8: ES update (src/efla_lm_kernels.cu:1854-1922, 2003-2021; call order src/train_efla_lm.cpp:4304-4358).
// dense mode: Z[i] = sum_p w_p * eps(mix(seed_p, salt), i), p ascending, fused multiply-add.
// sumsq: per-256 block pairwise tree in fp32 (the reference's shared-memory tree), block partials
// added in double. inv_rms: the reference's rsqrtf(ema+eps) is evaluated as 1/sqrt (IEEE ops).
// ---------------------------------------------------------------------------------------------
static double sumsq_blocks(const float* Z, int n) {
    double total = 0.0;
    for (int b0 = 0; b0 < n; b0 += 256) {
        float sh[256];
        for (int i = 0; i < 256; ++i) sh[i] = (b0 + i < n) ? Z[b0 + i] * Z[b0 + i] : 0.0f;
        for (int stride = 128; stride > 0; stride >>= 1)
            for (int i = 0; i < stride; ++i) sh[i] += sh[i + stride];
        total += (double)sh[0];
    }
    return total;
}

// The sum of squares alone (for callers that assemble Z from row ranges before reducing it).
ORC_API float orc_sumsq(const float* Z, int n) { return (float)sumsq_blocks(Z, n); }

ORC_API float orc_compute_z_sumsq(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs,
                                  int n, int use_clt, int clt_k, float* Z) {
    std::vector<uint64_t> seeds(pairs);
    for (int p = 0; p < pairs; ++p) seeds[p] = mix(pair_seeds[p], salt);
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n; ++i) {
        float z = 0.0f;
        for (int p = 0; p < pairs; ++p) {
            const float w = pair_weights[p];
            if (w == 0.0f) continue;
            z = std::fmaf(w, (float)noise_hash(seeds[p], (uint64_t)i, use_clt != 0, clt_k), z);
        }
        Z[i] = z;
    }
    return (float)sumsq_blocks(Z, n);
}

// rank-r mode: eps_p[i,j] = sum_r A_p[i,r]*B_p[j,r] (exact int), Z = c * sum_p w_p*eps_p (p ascending, fma).
// A_p[i,r] = noise(mix(seed_p', 0xA11CE), i*rank+r), B_p[j,r] = noise(mix(seed_p', 0xB0B), j*rank+r),
// seed_p' = mix(pair_seed[p], salt).
ORC_API float orc_compute_z_sumsq_lowrank(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt,
                                          int pairs, int rows, int cols, int rank, int use_clt, int clt_k,
                                          float cscale, float* Z) {
    std::vector<int8_t> A((size_t)pairs * rows * rank), B((size_t)pairs * cols * rank);
#pragma omp parallel for schedule(static)
    for (int p = 0; p < pairs; ++p) {
        const uint64_t sm = mix(pair_seeds[p], salt);
        const uint64_t sa = mix(sm, 0xA11CEULL), sb = mix(sm, 0xB0BULL);
        for (int i = 0; i < rows * rank; ++i) A[(size_t)p * rows * rank + i] = noise_hash(sa, (uint64_t)i, use_clt != 0, clt_k);
        for (int i = 0; i < cols * rank; ++i) B[(size_t)p * cols * rank + i] = noise_hash(sb, (uint64_t)i, use_clt != 0, clt_k);
    }
#pragma omp parallel for schedule(static)
    for (int i = 0; i < rows; ++i)
        for (int j = 0; j < cols; ++j) {
            float z = 0.0f;
            for (int p = 0; p < pairs; ++p) {
                const float w = pair_weights[p];
                if (w == 0.0f) continue;
                int e = 0;
                for (int r = 0; r < rank; ++r)
                    e += (int)A[((size_t)p * rows + i) * rank + r] * (int)B[((size_t)p * cols + j) * rank + r];
                z = std::fmaf(w, (float)e, z);
            }
            Z[(size_t)i * cols + j] = cscale * z;
        }
    return (float)sumsq_blocks(Z, rows * cols);
}

ORC_API float orc_update_inv_rms(float sumsq, float* rms_ema, int use_adaptive, float beta, float eps, int n) {
    float inv = 1.0f;
    if (use_adaptive) {
        const float ms = sumsq / (float)n;
        float ema = *rms_ema;
        if (ema == 0.0f) ema = ms;
        ema = std::fmaf(beta, ema, (1.0f - beta) * ms);
        *rms_ema = ema;
        inv = 1.0f / std::sqrt(ema + eps);
    }
    return inv;
}

ORC_API void orc_update_shadow_ternary(int8_t* w, float* shadow, const float* Z, int n, float inv_rms, float lr,
                                       float thresh) {
#pragma omp parallel for schedule(static)
    for (int i = 0; i < n; ++i) {
        const float g = inv_rms * Z[i];
        if (std::fabs(g) < thresh) continue;
        const float s = std::fmaf(lr, g, shadow[i]);
        shadow[i] = s;
        w[i] = clip_ternary(rint_to_int(s));
    }
}

// update_vector, plain (no adam/momentum) branch (src/train_efla_lm.cpp:4085-4189), with the GPU
// form of inv_rms (see header note). Used for head_bias, beta_bias and pos.
ORC_API void orc_update_vector(float* v, int n, const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt,
                               int pairs, int use_clt, int clt_k, float* rms_ema, int use_adaptive, float beta,
                               float eps, float lr, float thresh) {
    std::vector<float> Z(n);
    const float sumsq = orc_compute_z_sumsq(pair_weights, pair_seeds, salt, pairs, n, use_clt, clt_k, Z.data());
    const float inv = orc_update_inv_rms(sumsq, rms_ema, use_adaptive, beta, eps, n);
    for (int i = 0; i < n; ++i) {
        const float g = inv * Z[i];
        if (std::fabs(g) < thresh) continue;
        v[i] = std::fmaf(lr, g, v[i]);
    }
}
