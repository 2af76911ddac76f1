/*
 * bnf4.h -- C ABI of libbnf4: the population-evaluation hot path of catid/bitnet_nvfp4 for
 * NVIDIA B200 (sm_100a).
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name starts with h_.
 *   - `stream` is a cudaStream_t passed as void*; all work is stream-ordered, nothing synchronises
 *     unless the comment says so. The caller makes the target device current (cudaSetDevice) first.
 *   - The caller owns every buffer. Size helpers below give the byte counts.
 *   - Every function returns 0 on success, or a BNF4_ERR_* code; bnf4_last_error() then returns a
 *     message (thread-local). The reference's functions return void and swallow errors.
 *   - There is no CPU fallback: without an sm_100 device every compute entry point fails with
 *     BNF4_ERR_NO_DEVICE / BNF4_ERR_CUDA.
 *
 * Each entry point names the reference interface it replaces (file:line in the reference project).
 * The reference's own C++ names (namespaces bitnet_cuda / efla_lm_cuda) are exported by the same
 * library as thin wrappers over these functions, so the reference driver links unchanged.
 */
#ifndef BNF4_H_
#define BNF4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define BNF4_OK 0
#define BNF4_ERR_INVALID 1
#define BNF4_ERR_CUDA 2
#define BNF4_ERR_UNSUPPORTED 3
#define BNF4_ERR_DEVICE 4
#define BNF4_ERR_NO_DEVICE 5

/* ---------------------------------------------------------------------------------------------
 * Library state
 * ------------------------------------------------------------------------------------------- */
const char* bnf4_last_error(void);
const char* bnf4_version(void);
/* Number of kernels this library has launched from this process (all threads). */
unsigned long long bnf4_launch_count(void);
/* Options: "gemm_tma_store" (1 default = fp32 tiles leave through swizzled staging and TMA stores; 0 = direct stores);
 * "efla_chunked" (what BNF4_EFLA_AUTO means for heads of 64 with on-chip state: 1 = the chunked kernel, 0 = the
 * per-token kernel that reproduces the reference's fp16 rounding of the state after every token).
 * Returns BNF4_ERR_INVALID for an unknown name or a value outside the listed ones. */
int bnf4_set_option(const char* name, int value);
/* Reads and clears the device-side error word set by a kernel whose bounded wait expired.
 * Synchronises `stream`. *code = 0 when clean. */
int bnf4_device_error(void* stream, int* code);
/* sizeof() of the two descriptor structs below, for bindings that mirror them (ctypes, cgo, JNI). */
int bnf4_struct_sizes(int* rowquant_desc_bytes, int* gemm_desc_bytes);

/* ---------------------------------------------------------------------------------------------
 * Size helpers.  reference: nvfp4_matrix_bytes src/cuda_kernels.h:351-354,
 * nvfp4_sfa_bytes / nvfp4_sfb_bytes src/cuda_kernels.cu:3836-3848.
 * Scale factors: one ue4m3 byte per 16 K-elements, stored in 512-byte atoms of 128 rows x 4 blocks.
 * ------------------------------------------------------------------------------------------- */
size_t bnf4_nvfp4_matrix_bytes(int rows, int cols);
size_t bnf4_nvfp4_sfa_bytes(int m, int n, int k);
size_t bnf4_nvfp4_sfb_bytes(int m, int n, int k);

/* ---------------------------------------------------------------------------------------------
 * Quantisers: int8 / fp32 rows -> int8 copy + packed e2m1 codes + ue4m3 scale bytes.
 * Column counts must be multiples of 16 (the reference also handles ragged tails; unused by its driver).
 * ------------------------------------------------------------------------------------------- */
/* reference: nvfp4_quantize_a src/cuda_kernels.cu:4013-4037 (kernel :1545-1625) */
int bnf4_nvfp4_quantize_a(const int8_t* in, int m, int n, int k_in, int k_out, void* out, void* sfa, void* stream);
/* reference: nvfp4_quantize_b src/cuda_kernels.cu:4240-4264 */
int bnf4_nvfp4_quantize_b(const int8_t* in, int m, int n, int k_in, int k_out, void* out, void* sfb, void* stream);
/* fp32 rows straight to NVFP4 (no int8 stage): scale byte = ue4m3(max|x| / 6) per 16 elements (1.0 where that rounds to
 * zero), codes = e2m1(x / scale), the rules of nvfp4_quantize_a applied to fp32 values. The reference's driver always
 * quantises through int8 (src/cuda_kernels.cu:1783-1878); this is the "quantised on the fly from fp32" form, whose fp32
 * tensor scale is the GEMM's alpha. k_in <= k_out, k_out a multiple of 16 (columns past k_in read as zero). */
int bnf4_nvfp4_quantize_f32(const float* in, int rows, int k_in, int k_out, void* out, void* sf, void* stream);
/* reference: nvfp4_quantize_wqkv_fused src/cuda_kernels.cu:4266-4306 (kernel :2748-2854) */
int bnf4_nvfp4_quantize_wqkv_fused(const int8_t* wq, const int8_t* wk, const int8_t* wv, const int8_t* wb, int batch,
                                   int hidden, int k_out, int rows_total, float q_scale, float k_scale, float v_scale,
                                   float b_scale, void* out, void* sfb, void* stream);
/* reference: embedding_lookup_noise_quantize_nvfp4 src/cuda_kernels.cu:4039-4086 (kernel :2014-2109) */
int bnf4_embedding_lookup_noise_quantize_nvfp4(const uint8_t* tokens_t, int token_stride, const int8_t* emb_w,
                                               const int8_t* emb_noise, int hidden, int batch, float noise_scale,
                                               int anti_sign, int8_t* out_q, void* out_nvfp4, void* sfa, void* stream);
/* reference: add_pos_gelu_quantize_nvfp4 src/cuda_kernels.cu:4088-4126 (kernel :2260-2349) */
int bnf4_add_pos_gelu_quantize_nvfp4(const float* in, const float* pos_t, int hidden, int batch, float act_scale,
                                     int8_t* out_q, void* out_nvfp4, void* sfa, void* stream);
/* reference: activation_quantize_nvfp4 src/cuda_kernels.cu:4128-4160 (kernel :1783-1878) */
int bnf4_activation_quantize_nvfp4(const float* in, int rows, int cols_in, int cols_out, int activation, int8_t* out_q,
                                   void* out_nvfp4, void* sfa, void* stream);
/* reference: gelu_quantize_nvfp4 src/cuda_kernels.cu:4162-4194 (kernel :2500-2589) */
int bnf4_gelu_quantize_nvfp4(const float* in, int rows, int cols_in, int cols_out, float act_scale, int8_t* out_q,
                             void* out_nvfp4, void* sfa, void* stream);
/* reference: absmean_norm_q_nvfp4 src/cuda_kernels.cu:4196-4215 (kernel :2928-3031) */
int bnf4_absmean_norm_q_nvfp4(const int8_t* in, int hidden, int batch, int cols_out, float scale, int8_t* out_q,
                              void* out_nvfp4, void* sfa, void* stream);
/* reference: add_scaled_to_int8_absmean_norm_q_nvfp4 src/cuda_kernels.cu:4217-4238 (kernel :3033-3143) */
int bnf4_add_scaled_to_int8_absmean_norm_q_nvfp4(int8_t* inout, const float* in, int hidden, int batch, int cols_out,
                                                 float add_scale, float norm_scale, int8_t* out_q, void* out_nvfp4,
                                                 void* sfa, void* stream);

/* Generic row quantiser with population addressing and rank-r projections (no reference counterpart;
 * it is what the batched population driver uses). front_end: see BNF4_FE_*. */
#define BNF4_FE_INT8 0
#define BNF4_FE_WQKV 1
#define BNF4_FE_EMBED_DENSE 2
#define BNF4_FE_EMBED_LOWRANK 3
#define BNF4_FE_POS_GELU 4
#define BNF4_FE_POS_GELU_ABSMEAN 5
#define BNF4_FE_ACT 6
#define BNF4_FE_ABSMEAN 7
#define BNF4_FE_ADD_ABSMEAN 8

typedef struct bnf4_rowquant_desc {
    int rows, cols_in, cols_out;
    /* row -> member = row / rows_per_member -> pair = member / 2, sign + for even members, - for odd.
     * rows_per_member == 0: a single member whose sign is anti_fixed. */
    int rows_per_member;
    int anti_fixed;
    float sigma;  /* perturbation magnitude (0 disables noise) */
    float c_rank; /* rank-r normalisation constant sqrt(3/8)/sqrt(rank) */
    const int8_t* in_i8;
    const float* in_f32;
    int ld_in;
    int8_t* inout_i8; /* int8 residual stream [rows][cols_in] */
    const int8_t *wq, *wk, *wv, *wb;
    float q_scale, k_scale, v_scale, b_scale;
    const uint8_t* tokens;
    int token_stride;
    int row_mod; /* token row = row % row_mod (0: row) */
    const int8_t* emb_w;
    const int8_t* emb_noise; /* [pair][V][H] */
    const int8_t* embA;      /* [pair][V][rank] */
    const int8_t* embB;      /* [pair][rank][H] */
    long long embA_pair_stride, embB_pair_stride;
    int rank;
    const float* pos;         /* [pos rows][H] */
    const int8_t* pos_noise;  /* [pair][pos rows][H] or NULL */
    int pos_mod;              /* positional row = row_in_member % pos_mod (0: row 0) */
    long long noise_pair_stride;
    int act_mode; /* 0 none, 1 relu, 2 tanh(x/127)*127, 3 gelu(x)*act_scale */
    float act_scale, add_scale, norm_scale;
    int8_t* out_q; /* optional int8 copy */
    int ld_q;
    uint8_t* out_codes;
    uint8_t* out_sf;
    /* t_out[row][v] = sum_k q[row][k] * tvec[pair][v][k], exact int32 */
    const int8_t* tvec;
    long long tvec_pair_stride;
    int nvec;
    int32_t* t_out;
    int vec_ok, vec_ok_q; /* set by the library */
    /* BNF4_FE_POS_GELU(_ABSMEAN) only: when > 0 the fp32 input is a table of gather_rows rows per member and the input
     * row of output row (member, i) is member * gather_rows + tokens[(i % row_mod) * token_stride] (row_mod 0: i). */
    int gather_rows;
    int in_f16; /* BNF4_FE_ADD_ABSMEAN: in_f32 points at IEEE halves and ld_in counts halves (16-byte aligned rows) */
} bnf4_rowquant_desc;

int bnf4_rowquant(int front_end, const bnf4_rowquant_desc* desc, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Block-scaled FP4 GEMM (tcgen05).  A [M][K] and B [N][K] are K-major packed e2m1, k % 64 == 0.
 * ------------------------------------------------------------------------------------------- */
/* reference: gemm_ternary_f_nvfp4 src/cuda_kernels.cu:4342-4473.  D = alpha*A*B^T + beta*C, fp32 row-major [m][n]. */
int bnf4_gemm_ternary_f_nvfp4(const void* a, const void* b, const void* sfa, const void* sfb, int m, int n, int k,
                              float alpha, float beta, const float* c, float* d, void* stream);
/* reference: gemm_ternary_f_nvfp4_gelu_i8 src/cuda_kernels.cu:4475-4607.  D8 = clip8(rint(gelu(alpha*A*B^T + beta*C) * act_scale)). */
int bnf4_gemm_ternary_f_nvfp4_gelu_i8(const void* a, const void* b, const void* sfa, const void* sfb, int m, int n,
                                      int k, float alpha, float beta, const float* c, float act_scale, int8_t* d,
                                      void* stream);
/* reference: nvfp4_prepare_gemm src/cuda_kernels.cu:3902-4011 (plan warm-up; here: argument validation only). */
int bnf4_nvfp4_prepare_gemm(const void* a, const void* b, const void* sfa, const void* sfb, int m, int n, int k,
                            float alpha, float beta, const float* c, float* d, void* stream);

#define BNF4_EPI_F32 0
#define BNF4_EPI_GELU_I8 1
#define BNF4_EPI_GELU_FP4 2
#define BNF4_EPI_ADD_I8 3 /* resid = clip8(resid + rint(v * add_scale)), in place: the add of the reference's
                           * add_scaled_to_int8_absmean_norm_q_nvfp4 (src/cuda_kernels.cu:3033-3143) applied by the GEMM
                           * that produces v, so that the fp32 product never travels through HBM; follow it with the
                           * BNF4_FE_ABSMEAN quantiser over resid; |v * add_scale| must stay below 2^15 */
#define BNF4_EPI_F16 4 /* D rounded to IEEE half (round to nearest even) for the leading n_f16 columns, fp32 for the rest: the
                          fused q | k | v | beta projection feeding the chunked EFLA scan, which rounds its operands to fp16 anyway */

/* Full form: strides, fused epilogues and the rank-r perturbation
 *   D += s_member * sum_r t[m][g*rank + r] * A_pair[n][r]
 * (math of the reference's lora kernels, src/cuda_kernels.cu:370-410, 1271-1305, which its driver never calls). */
typedef struct bnf4_gemm_desc {
    const void* a;
    const void* b;
    const void* sfa;
    const void* sfb;
    int m, n, k;
    float alpha, beta;
    const float* c;
    int ldc;
    float* d;
    int ldd;
    int epilogue;
    float act_scale;
    int8_t* d_i8;
    int ld_i8;
    uint8_t* d_codes; /* BNF4_EPI_GELU_FP4: codes [M][N/2] and scale atoms for (M,N) */
    uint8_t* d_sf;
    int rank;            /* 0 disables the perturbation; at most 4 */
    int rows_per_member; /* member = row / rows_per_member (0: one member, positive sign) */
    const int32_t* lora_t; /* [M][t_stride] */
    int t_stride;
    const int8_t* lora_A; /* [pair][N][rank] */
    long long lora_A_pair_stride;
    float lora_scale; /* magnitude; the member's sign is applied by the kernel */
    int group_cols;   /* columns per stacked group (0: one group); group g reads t[g*rank ..] */
    const int8_t* next_tvec; /* BNF4_EPI_GELU_FP4: [pair][next_nvec][N] */
    long long next_tvec_pair_stride;
    int next_nvec;
    int32_t* next_t; /* [M][next_nvec], zeroed by the caller; accumulated with integer atomics */
    int8_t* resid;   /* BNF4_EPI_ADD_I8: [M][ld_resid] int8, read and written */
    int ld_resid;
    float add_scale;
    void* d_f16;     /* BNF4_EPI_F16: columns [0, n_f16) as IEEE halves [M][ld_f16]; columns [n_f16, n) as fp32 in d, where
                        column j lands at d[row * ldd + (j - n_f16)] */
    int ld_f16;      /* in halves, a multiple of 8 */
    int n_f16;       /* a multiple of 32 */
} bnf4_gemm_desc;

int bnf4_gemm_nvfp4_ex(const bnf4_gemm_desc* desc, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Exact-integer ternary GEMM (the reference's non-NVFP4 fallback).
 * reference: gemm_ternary_f src/cuda_kernels.cu:3725-3739 (kernels :740-762, :163-192).
 * out[b,i] = out_scale * sum_g scale_x[g] * (int32 sum over the g-th group of 256 columns of x[b,:]*w[i,:]);
 * scale_x == NULL means all ones. x [batch][cols] int8, w [rows][cols] int8, out [batch][rows] fp32.
 * ------------------------------------------------------------------------------------------- */
int bnf4_gemm_ternary_f(const int8_t* x, const int8_t* w, const float* scale_x, int rows, int cols, int batch,
                        float out_scale, float* out, void* stream);
/* reference: lora_compute_t src/cuda_kernels.cu:5003-5012 (kernel :370-390). t[b,r] = sum_j x[b,j]*B[j,r], B [cols][rank]. */
int bnf4_lora_compute_t(const int8_t* x, const int8_t* B, int cols, int batch, int rank, int32_t* t, void* stream);
/* reference: lora_add src/cuda_kernels.cu:5014-5024 (kernel :392-410). out[b,i] += scale * sum_r t[b,r]*A[i,r]. */
int bnf4_lora_add(const int32_t* t, const int8_t* A, int rows, int batch, int rank, float scale, float* out, void* stream);
/* reference: split_qkvb_fused src/cuda_kernels.cu:4308-4340 (kernels :2856-2926). */
int bnf4_split_qkvb_fused(const float* in, int batch, int hidden, int fused_cols, float* q, float* k, float* v,
                          float* beta, float beta_bias, void* stream);

/* ---------------------------------------------------------------------------------------------
 * EFLA / DeltaNet linear-attention recurrence. State stays on chip for all T steps of a call.
 * ------------------------------------------------------------------------------------------- */
typedef struct bnf4_efla_desc {
    void* state;    /* optional HBM state [seqs][heads][hd][hd]; loaded before and stored after the T steps.
                       NULL: zero initial state, final state discarded (whole-sequence scan). */
    int state_fp16; /* 1: state is rounded to fp16 after every step (the reference default); 0: fp32 state */
    const void* q; /* fp32 (or halves, see qkv_f16): row r = seq*T + t at q + r*ld_qkv; head h at column h*hd (likewise k, v) */
    const void* k;
    const void* v;
    const float* beta_raw; /* row r at beta_raw + r*ld_beta */
    int ld_qkv, ld_beta;
    float beta_bias;            /* used when beta_bias_seq == NULL */
    const float* beta_bias_seq; /* bias of sequence s = beta_bias_seq[s / seqs_per_bias] */
    int seqs_per_bias;
    int hidden, heads;
    long long seqs;
    int T;
    int method; /* 0 DeltaNet, 1 EFLA */
    float eps;
    void* out; /* fp32 (or halves, see out_f16): row r at out + r*ld_out */
    int ld_out;
    int variant; /* BNF4_EFLA_*: which kernel runs. AUTO: for heads of 64 with no HBM state, the chunked or the per-token
                    register-state kernel as option "efla_chunked" says; the generic kernel otherwise. */
    int qkv_f16; /* 1: q, k, v are IEEE halves and ld_qkv counts halves (chunked kernel only; 16-byte aligned rows) */
    int out_f16; /* 1: out is IEEE halves and ld_out counts halves (chunked kernel only; 16-byte aligned rows) */
} bnf4_efla_desc;
#define BNF4_EFLA_AUTO 0
#define BNF4_EFLA_GENERIC 1   /* any head_dim, state in shared memory (and in HBM between calls), per-token fp16 rounding */
#define BNF4_EFLA_PER_TOKEN 2 /* heads of 64: state in registers, rounded to fp16 after every token like the reference */
#define BNF4_EFLA_CHUNKED 3   /* heads of 64: 16 tokens per step as tensor-core contractions, state rounded to fp16 per chunk */

int bnf4_efla_scan(const bnf4_efla_desc* desc, void* stream);
/* reference: efla_step_half_qkv_fused src/efla_lm_kernels.cu:2367-2447 (6 kernels; one here). The scratch
 * pointers of the reference signature are accepted and ignored. heads = 1. */
int bnf4_efla_step_half_qkv_fused(void* S_half, const float* qkv, int fused_cols, float beta_bias, int hidden,
                                  int batch, int method, float eps, float* out, void* stream);
/* reference: efla_step_qkv_fused src/efla_lm_kernels.cu:2181-2221 (fp32 state). */
int bnf4_efla_step_qkv_fused(float* S, const float* qkv, int fused_cols, float beta_bias, int hidden, int batch,
                             int method, float eps, float* out, void* stream);
/* reference: efla_step / efla_step_half / efla_step_fused / efla_step_fused_half
 * src/efla_lm_kernels.cu:2134-2179, 2223-2365, 2449-2483 (separate q, k, v [batch][hidden], beta_raw [batch]). */
int bnf4_efla_step(void* S, int state_fp16, const float* q, const float* k, const float* v, const float* beta_raw,
                   float beta_bias, int hidden, int batch, int method, float eps, float* out, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Cross-entropy fitness.
 * ------------------------------------------------------------------------------------------- */
/* reference: cross_entropy_loss src/efla_lm_kernels.cu:2509-2523 (kernel :252-311). Adds the summed loss of
 * `batch` rows to *loss_accum. The sum is formed in a fixed order (the reference uses float atomics). */
int bnf4_cross_entropy_loss(const float* logits, const float* bias, const float* bias_noise, float bias_noise_scale,
                            const uint8_t* targets_t, int token_stride, int vocab, int batch, float* loss_accum,
                            void* stream);
/* Population form: logits [members*rows_per_member][ld]; targets [rows_per_member] shared by all members;
 * bias_noise int8 [pair][vocab] (pair = member/2, sign by parity, magnitude sigma).
 * loss_mean[member] = mean over the member's rows. partial: scratch of members*16 floats. */
int bnf4_cross_entropy_population(const float* logits, int ld, const float* bias, const int8_t* bias_noise,
                                  float sigma, const uint8_t* targets, int vocab, int members, int rows_per_member,
                                  float* partial, float* loss_mean, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Noise generation (counter hash; bit-exact with the reference's host and device generators).
 * ------------------------------------------------------------------------------------------- */
/* reference: fill_ternary_noise src/efla_lm_kernels.cu:2525-2535 (kernel :352-360) */
int bnf4_fill_ternary_noise(int8_t* out, size_t n, uint64_t seed, int use_clt, int clt_k, void* stream);
/* reference: struct NoiseDesc src/efla_lm_kernels.h:306-310 */
typedef struct bnf4_noise_desc {
    int8_t* out;
    size_t n;
    uint64_t seed;
} bnf4_noise_desc;
/* reference: fill_ternary_noise_batched src/efla_lm_kernels.cu:2537-2550 (kernel :362-374); descs is a device array */
int bnf4_fill_ternary_noise_batched(const bnf4_noise_desc* descs, int num_desc, int max_blocks, int use_clt, int clt_k,
                                    void* stream);
/* reference: fill_float_noise src/efla_lm_kernels.cu:2552-2562 (kernel :376-385) */
int bnf4_fill_float_noise(float* out, int n, uint64_t seed, int use_clt, int clt_k, void* stream);

/* ---------------------------------------------------------------------------------------------
 * ES update.
 * ------------------------------------------------------------------------------------------- */
/* reference: init_shadow_from_weights src/efla_lm_kernels.cu:2023-2030 (kernel :1836-1842) */
int bnf4_init_shadow_from_weights(const int8_t* w, float* shadow, int n, void* stream);
/* reference: fill_pair_seeds src/efla_lm_kernels.cu:2032-2040 (kernel :1844-1852) */
int bnf4_fill_pair_seeds(uint64_t base_seed, uint64_t epoch, int pairs, uint64_t* out, void* stream);
/* reference: compute_z_sumsq src/efla_lm_kernels.cu:2042-2059 (kernel :1854-1890).
 * Z[i] = sum_p w_p * noise(mix(seed_p, salt), i) (p ascending, fused multiply-add); sum(Z^2) is ADDED to *sumsq.
 * The sum of squares is reduced in a fixed order (per-256 tree, then block partials in double).
 * Scratch: the block partials go to ONE library-owned buffer per device, shared by this function,
 * bnf4_compute_z_sumsq_lowrank and bnf4_sumsq on every stream and host thread (256 KiB allocated with cudaMalloc on the
 * first call, enough for n <= 16,777,216). Consequences for the caller:
 *   - two of these calls that may overlap in time (different streams, or threads without ordering) race on the
 *     partials: order them, as for bnf4_compute_z_sumsq_static;
 *   - a call with a larger n than any before grows the buffer: cudaDeviceSynchronize, cudaFree, cudaMalloc in the
 *     middle of the stream. That is not allowed during stream capture and waits for every stream of the device; make
 *     one call with the largest n during set-up (bnf4_sumsq on any buffer of that size will do), or use the _static
 *     entry point, which never allocates. The batched driver (bnf4_model_*) keeps its own buffers and never comes here. */
int bnf4_compute_z_sumsq(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs, int n,
                         int use_clt, int clt_k, float* Z, float* sumsq, void* stream);
/* No counterpart in the reference. Same arguments, arithmetic and result as bnf4_compute_z_sumsq, for callers that
 * cannot let a library allocate device memory: a host whose own allocator has reserved all of HBM (a library
 * cudaMalloc would fail), a loop that cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply, or a
 * process held to a fixed device footprint. This entry point calls no allocator at all (no cudaMalloc, no cudaFree,
 * no pool or library routine that allocates); the caller still supplies every input and output buffer, and the block
 * partials of sum(Z^2) go to a 1 MiB array built into the library's device image.
 *   - Limit: n <= 67,108,864 elements (262,144 partials of 256 elements). Larger n returns BNF4_ERR_INVALID and
 *     launches nothing.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress, with that device
 *     current) and caches it; make that first call during set-up, before any stream capture begins.
 *   - The array is one per device and shared by every call, on every stream and host thread; it keeps whatever the
 *     last call left. Each call overwrites every partial it later reads, so nothing has to be cleared, but two calls
 *     that may overlap in time (different streams, or different threads without ordering) race on it: order them. */
int bnf4_compute_z_sumsq_static(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs, int n,
                                int use_clt, int clt_k, float* Z, float* sumsq, void* stream);
/* Rank-r form: Z[i*cols+j] = cscale * sum_p w_p * sum_r A[p][i][r]*B[p][r][j] with A [pairs][rows][rank] and
 * B [pairs][rank][cols] int8 (the same factor buffers the forward pass uses). */
int bnf4_compute_z_sumsq_lowrank(const float* pair_weights, const int8_t* A, long long A_pair_stride, const int8_t* B,
                                 long long B_pair_stride, int pairs, int rows, int cols, int rank, float cscale,
                                 float* Z, float* sumsq, void* stream);
/* The two halves of the call above, for callers that compute row ranges of Z on different ranks and exchange them
 * before the (order-sensitive) sum of squares: rows [r0, r0+n) of Z come from passing A + r0*rank, Z + r0*cols, rows = n. */
int bnf4_compute_z_lowrank(const float* pair_weights, const int8_t* A, long long A_pair_stride, const int8_t* B,
                           long long B_pair_stride, int pairs, int rows, int cols, int rank, float cscale, float* Z,
                           void* stream);
/* *sumsq += sum Z[i]^2, with the block structure and summation order of bnf4_compute_z_sumsq. */
int bnf4_sumsq(const float* Z, int n, float* sumsq, void* stream);
/* reference: update_inv_rms src/efla_lm_kernels.cu:2061-2073 (kernel :2003-2021). inv_rms = 1/sqrt(ema+eps)
 * evaluated with IEEE sqrt and divide (the reference's rsqrtf is within 2 ulp of it). */
int bnf4_update_inv_rms(const float* sumsq, float* rms_ema, int use_adaptive, float adaptive_beta, float adaptive_eps,
                        int n, float* inv_rms, void* stream);
/* reference: update_shadow_ternary_device src/efla_lm_kernels.cu:2088-2099 (kernel :1908-1922) */
int bnf4_update_shadow_ternary_device(int8_t* w, float* shadow, const float* Z, int n, const float* inv_rms, float lr,
                                      float thresh, void* stream);
/* reference: update_shadow_ternary src/efla_lm_kernels.cu:2075-2086 (kernel :1892-1906) */
int bnf4_update_shadow_ternary(int8_t* w, float* shadow, const float* Z, int n, float inv_rms, float lr, float thresh,
                               void* stream);
/* Device twin of the reference's host update_vector (plain branch), src/train_efla_lm.cpp:4085-4189:
 * v[i] += lr * g where g = inv_rms * Z[i], skipped when |g| < thresh. */
int bnf4_update_vector_device(float* v, const float* Z, int n, const float* inv_rms, float lr, float thresh,
                              void* stream);
/* reference: add_scaled src/efla_lm_kernels.cu:1769-1779 (out[i] += scale * noise[i]) */
int bnf4_add_scaled(float* out, const float* noise, int n, float scale, void* stream);
/* Sign / z-score / centered-rank shaping of the pair fitness vector on the host (pure function, no GPU):
 * reference shape_pair_weights src/train_efla_lm.cpp:3898-3952; ties broken by index. `mode` takes the integer
 * values of the reference's TrainConfig::FitnessMode (src/train_efla_lm.cpp:260), so a driver can pass
 * (int)cfg.fitness_mode unchanged; the reference's default is centered rank. */
#define BNF4_FITNESS_SIGN 0
#define BNF4_FITNESS_ZSCORE 1
#define BNF4_FITNESS_CENTERED_RANK 2
int bnf4_shape_pair_weights(float* h_w, int n, int mode, float clip);

/* ---------------------------------------------------------------------------------------------
 * Population driver: the B200-native re-design of CudaEflaLm::evaluate_loss + eval_worker + gpu_update_matrix
 * (reference: src/train_efla_lm.cpp:2117-3431, 5344-5468, 4304-4358).
 *
 * The reference evaluates one member at a time, token by token (M = batch rows per GEMM, ~8.7k launches and
 * one blocking sync per member). Here a wave of members is evaluated layer by layer: every GEMM of a layer
 * covers all tokens of all members of the wave (M = members * batch * seq rows), the recurrent state stays on
 * chip for the whole sequence, and the per-member perturbation is the rank-r form fused into the GEMM
 * epilogue. Row r of a wave buffer is (member, b, t) = (r / (B*T), (r / T) % B, r % T).
 * Members 2p and 2p+1 are the + and - evaluations of antithetic pair p.
 * ------------------------------------------------------------------------------------------- */
typedef struct bnf4_model_cfg {
    int vocab;        /* 256 */
    int hidden;       /* H, multiple of 64 */
    int layers;       /* L */
    int mlp_mult;     /* F = mlp_mult * H */
    int seq;          /* T */
    int batch;        /* B */
    int heads;        /* head_dim = H / heads; 1 reproduces the reference */
    int rank;         /* rank of the per-member perturbation, 1..4; 0 = the reference driver's dense form: one materialised CLT
                         noise matrix per weight matrix and pair, applied as a second GEMM with beta = 1 (one pair per wave,
                         batch * seq a multiple of 128; a reference-exact mode, not a fast one) */
    int sigma_shift;  /* sigma = 2^-sigma_shift */
    int use_clt;
    int clt_k;
    int method;       /* 0 DeltaNet, 1 EFLA */
    float act_scale, mlp_act_scale, ln_scale, residual_scale, mlp_residual_scale, eps;
    int max_pairs;    /* pairs per ES step (population / 2) */
    int wave_members; /* members evaluated per wave (even); 0 = library default: what fits ~12 GB of wave buffers, at most 256 */
} bnf4_model_cfg;

/* Host-side weight set (reference: EflaLmWeights src/train_efla_lm.cpp:419-431 plus the positional table). */
typedef struct bnf4_model_weights {
    int8_t* emb;      /* [V][H] */
    int8_t* win;      /* [H][H] */
    int8_t* wq;       /* [L][H][H] */
    int8_t* wk;       /* [L][H][H] */
    int8_t* wv;       /* [L][H][H] */
    int8_t* wbeta;    /* [L][H] */
    int8_t* ff1;      /* [L][F][H] */
    int8_t* ff2;      /* [L][H][F] */
    int8_t* head;     /* [V][H] */
    float* head_bias; /* [V] */
    float* beta_bias; /* [L] */
    float* pos;       /* [T][H] */
} bnf4_model_weights;

typedef struct bnf4_update_cfg {
    float lr;
    float thresh;        /* the update is skipped where |inv_rms * Z| < thresh * sqrt(pairs) */
    int use_adaptive;    /* RMS-EMA normalisation */
    float adaptive_beta; /* 0.95 */
    float adaptive_eps;  /* 1e-3 */
    int train_pos;       /* also update the positional table */
} bnf4_update_cfg;

/* Allocates every device buffer of the model on the current device (cudaMalloc). */
int bnf4_model_create(const bnf4_model_cfg* cfg, void** handle);
int bnf4_model_destroy(void* handle);
/* Bytes of device memory held by the model. */
size_t bnf4_model_device_bytes(void* handle);
/* h_w: host arrays. Uploads, resets the fp32 shadow weights to the int8 values (reference: init_shadow_from_weights),
 * clears the RMS-EMA state and quantises the base weights to NVFP4. Synchronises. */
int bnf4_model_set_weights(void* handle, const bnf4_model_weights* h_w);
/* Copies the current int8 weights / fp32 vectors (and optionally the shadow weights) back to host arrays. Synchronises. */
int bnf4_model_get_weights(void* handle, bnf4_model_weights* h_w);
/* tokens / targets: uint8 [B][T] (device pointers when on_device != 0, else host). */
int bnf4_model_set_tokens(void* handle, const uint8_t* tokens, const uint8_t* targets, int on_device, void* stream);
/* Derives pair seeds (mix(seed, mix(epoch, p))) and generates every per-pair noise vector of the step:
 * rank-r factors of all 27 matrices, positional / head-bias / beta-bias noise. pairs <= cfg.max_pairs. */
int bnf4_model_prepare_step(void* handle, uint64_t seed, uint64_t epoch, int pairs, void* stream);
/* Evaluates pairs [pair_begin, pair_begin + pair_count): losses[2*i], losses[2*i+1] = mean cross-entropy of the
 * + and - member of pair pair_begin + i. Device output. */
int bnf4_model_eval_pairs(void* handle, int pair_begin, int pair_count, float* losses, void* stream);
/* bnf4_model_prepare_step for a process that evaluates only pairs [eval_begin, eval_begin + eval_count) of the step: the
 * rank-r factors are generated for all pairs (the update reads them all), the noise that only an evaluation reads
 * (positional table, head bias, beta bias: two thirds of the bytes) for that range only. bnf4_model_eval_pairs rejects
 * pairs outside the range. */
int bnf4_model_prepare_step_range(void* handle, uint64_t seed, uint64_t epoch, int pairs, int eval_begin, int eval_count,
                                  void* stream);
/* Mean cross-entropy of the unperturbed model on the current tokens (device output, 1 float). */
int bnf4_model_eval_base(void* handle, float* loss, void* stream);
/* pair_weights: shaped fitness of ALL pairs of the step (device, `pairs` floats as passed to prepare_step).
 * Applies the ES update to all ternary matrices and fp32 vectors and re-quantises the base weights.
 * Deterministic: every rank that calls it with the same inputs ends with identical bits. */
int bnf4_model_update(void* handle, const float* pair_weights, const bnf4_update_cfg* ucfg, void* stream);
/* The same update with the dominant part -- Z = sum_p w_p * noise_p for every ternary matrix -- split by rows over
 * `nshards` ranks (the reference replicates it on every worker, src/train_efla_lm.cpp:5560-5660):
 *   1. bnf4_model_update_z_layout: for tensor i of the model (the ternary matrices in a fixed order, then head bias,
 *      beta bias and the positional table), offsets[i] / elems[i] locate its Z inside one caller-owned fp32 buffer
 *      `z_all`, and sharded[i] tells whether it is computed in nshards equal contiguous parts (matrices whose rows
 *      divide by nshards, vectors of at least 4096 elements; otherwise every rank computes the whole tensor). Returns
 *      the number of tensors (<= max_entries, at most 6 + 6 per layer) or -1; *total_elems receives the size of
 *      z_all in floats.
 *   2. bnf4_model_update_z: rank `shard` fills its part of every sharded tensor (all of the others) in z_all.
 *   3. the caller all-gathers each sharded tensor in place (contiguous blocks in rank order);
 *   4. bnf4_model_update_apply: sum of squares, RMS normalisation, shadow/ternary update of all matrices and the update of
 *      the fp32 vectors from z_all, and re-quantisation: the same kernels in the same order as bnf4_model_update, hence the same bits. */
int bnf4_model_update_z_layout(void* handle, int nshards, int max_entries, long long* offsets, long long* elems, int* sharded,
                               long long* total_elems);
int bnf4_model_update_z(void* handle, const float* pair_weights, int shard, int nshards, float* z_all, void* stream);
int bnf4_model_update_apply(void* handle, const float* pair_weights, const float* z_all, const bnf4_update_cfg* ucfg, void* stream);

/* The whole ES step of one rank in ONE call, for hosts that run one process per GPU (what population.es_step does over
 * torch.distributed, and what replaces the body of the reference's epoch loop between eval_worker and the vector updates,
 * src/train_efla_lm.cpp:5344-5657): noise for the step -> this rank's pairs [rank * pairs / world, (rank + 1) * pairs / world)
 * -> all-gather of the per-member losses -> f_p = -(loss+ - loss-) shaped on the host (bnf4_shape_pair_weights; one stream
 * synchronisation and a round trip of 8 * pairs bytes, as the reference) -> noise sums Z by rows over the ranks -> in-place
 * all-gather of every sharded Z -> apply. The library links no communication library: the caller supplies the two
 * collectives as callbacks over its own communicator (NCCL: ncclAllGather with sendbuff = recv + rank * bytes_per_rank).
 * Every rank must make the call with the same cfg except `rank`; all ranks end with identical weights, bit-identical to
 * the single-process step. world == 1 needs no callbacks (coll may be NULL). pairs must be a multiple of world (ragged
 * shards: compose the calls above by hand). d_losses_all receives all 2 * pairs losses on every rank. */
typedef struct bnf4_collectives {
    void* ctx;
    /* In place, on `stream`: rank r's block is the bytes_per_rank bytes at d_recv + r * bytes_per_rank. 0 = success. */
    int (*allgather_inplace)(void* ctx, void* d_recv, size_t bytes_per_rank, void* stream);
    /* Optional brackets around the batch of Z all-gathers (ncclGroupStart / ncclGroupEnd); either may be NULL. */
    int (*group_begin)(void* ctx);
    int (*group_end)(void* ctx);
} bnf4_collectives;
typedef struct bnf4_es_step_cfg {
    uint64_t seed;
    uint64_t epoch;
    int pairs;          /* of the whole population */
    int rank, world;
    int fitness_mode;   /* BNF4_FITNESS_* */
    float fitness_clip;
    bnf4_update_cfg update;
} bnf4_es_step_cfg;
int bnf4_model_es_step(void* handle, const bnf4_es_step_cfg* cfg, const bnf4_collectives* coll, float* d_losses_all, void* stream);
/* Debug/verification access to an internal wave buffer by name ("x_q", "a_h", "sf_h", "a_f", "sf_f", "qkv", "y",
 * "t_a", "t_f", "losses"): copies min(bytes, size) bytes to host. Synchronises. */
int bnf4_model_read_buffer(void* handle, const char* name, void* h_dst, size_t bytes);
/* Kernels launched by the last bnf4_model_eval_pairs wave (for accounting). */
int bnf4_model_launches_per_wave(void* handle);
/* Checkpoint / resume (the reference has none). The optimiser state is the fp32 shadows of the nine int8 weight tensors
 * (concatenated in the member order of bnf4_model_weights) and the RMS-EMA scalars; call bnf4_model_set_weights first
 * (it resets the state), then bnf4_model_set_optimizer_state. Host pointers; these calls synchronise the device. */
int bnf4_model_optimizer_state_sizes(void* handle, size_t* shadow_floats, size_t* ema_floats);
int bnf4_model_get_optimizer_state(void* handle, float* h_shadow, float* h_ema);
int bnf4_model_set_optimizer_state(void* handle, const float* h_shadow, const float* h_ema);
/* Members evaluated per wave (the configured value, or the library's choice when the configuration says 0). */
int bnf4_model_wave_members(void* handle);
/* CUDA-graph replay of the evaluation (replaces the reference's --cuda_graph mode, get_or_create_graph in
 * src/train_efla_lm.cpp:3779-3819). When enabled, bnf4_model_eval_pairs / _eval_base / _es_step launch each wave of members
 * as one graph: a wave (its first pair, member count, sigma) runs eagerly the first time it is seen, is captured
 * on a stream of the library's own the second time, and is a single cudaGraphLaunch into the caller's stream from then on (the
 * per-step noise and the re-quantised weights live at fixed addresses, so a captured wave stays valid across steps). Same
 * kernels, same arguments, same results. The rank-0 (dense) mode and runs with the timing breakdown enabled stay eager; a wave
 * whose capture the runtime refuses stays eager too. Disabling synchronises the device and drops the cached graphs.
 * bnf4_model_graph_launches counts the graph launches since the model was created. */
int bnf4_model_set_graph(void* handle, int enable);
long long bnf4_model_graph_launches(void* handle);
/* Optional timing breakdown: when enabled, the driver brackets every kernel class with CUDA events on the launching
 * stream. bnf4_model_get_timing synchronises and returns accumulated milliseconds and launches per class since the
 * last bnf4_model_set_timing call. */
int bnf4_model_set_timing(void* handle, int enable);
int bnf4_model_num_kernel_classes(void);
const char* bnf4_model_kernel_class_name(int cls);
int bnf4_model_get_timing(void* handle, double* ms, long long* launches, int n);

#ifdef __cplusplus
}
#endif
#endif /* BNF4_H_ */
