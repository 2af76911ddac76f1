// Internal launcher interface between the translation units of the library (not installed).
#pragma once

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

#include "bnf4.h"

namespace bnf4 {

// ---------------------------------------------------------------------------------------------
// Row quantisers (rowquant.cu). Parameter block = the public bnf4_rowquant_desc.
// ---------------------------------------------------------------------------------------------
enum RowFrontEnd : int {
    FE_INT8 = BNF4_FE_INT8,                          // int8 rows in
    FE_WQKV = BNF4_FE_WQKV,                          // stacked [Wq;Wk;Wv;wbeta] rows, per-group scale folded into the block scale
    FE_EMBED_DENSE = BNF4_FE_EMBED_DENSE,            // emb[tok] + ns * noise[tok]
    FE_EMBED_LOWRANK = BNF4_FE_EMBED_LOWRANK,        // emb[tok] + ns*c_r * sum_r A[tok,r] B[j,r]
    FE_POS_GELU = BNF4_FE_POS_GELU,                  // gelu(in + pos) * act_scale
    FE_POS_GELU_ABSMEAN = BNF4_FE_POS_GELU_ABSMEAN,  // the above, kept as the residual stream, then abs-mean normalised
    FE_ACT = BNF4_FE_ACT,                            // none / relu / tanh / gelu*act_scale
    FE_ABSMEAN = BNF4_FE_ABSMEAN,                    // abs-mean norm of int8 rows
    FE_ADD_ABSMEAN = BNF4_FE_ADD_ABSMEAN,            // x8 = clip8(x8 + rint(y*add_scale)); abs-mean norm
};

constexpr int kMaxTVec = 16;  // rank-r projections per row (4 stacked groups x rank 4)

using RowQuantParams = bnf4_rowquant_desc;
int rowquant_dispatch(int front_end, RowQuantParams p, cudaStream_t stream);

// ---------------------------------------------------------------------------------------------
// Block-scaled FP4 GEMM on tcgen05 (gemm_tcgen05.cu). Parameter block = the public bnf4_gemm_desc.
// ---------------------------------------------------------------------------------------------
enum GemmEpilogue : int {
    EPI_F32 = BNF4_EPI_F32,            // fp32 D
    EPI_GELU_I8 = BNF4_EPI_GELU_I8,    // int8 D = clip8(rint(gelu(v) * act_scale))
    EPI_GELU_FP4 = BNF4_EPI_GELU_FP4,  // the above re-quantised to e2m1 codes + ue4m3 scales (+ int8 copy, + t of the next GEMM)
    EPI_ADD_I8 = BNF4_EPI_ADD_I8,      // int8 residual stream updated in place: clip8(resid + rint(v * add_scale))
    EPI_F16 = BNF4_EPI_F16,            // leading columns as IEEE halves, the rest fp32
};

using GemmParams = bnf4_gemm_desc;
int gemm_nvfp4_launch(const GemmParams& p, cudaStream_t stream);
// Reads and clears the device-side error word of the GEMM kernels (0 = none). Synchronises the stream.
int gemm_nvfp4_device_error(cudaStream_t stream, int* out_code);
extern int g_gemm_allow_tma_store;

// EFLA recurrence (efla.cu). Parameter block = the public bnf4_efla_desc.
using EflaParams = bnf4_efla_desc;
int efla_launch(const EflaParams& p, cudaStream_t stream);
extern int g_efla_chunked;

// Rank-r noise sums Z of a table of matrices in one launch (es_kernels.cu).
struct ZLowrankDesc {
    const int8_t* A;  // [pairs][rows][rank]
    long long A_ps;
    const int8_t* B;  // [pairs][rank][cols]
    long long B_ps;
    float* Z;         // [rows][cols]
    int rows, cols;
};
int z_lowrank_launch(const float* pair_weights, const ZLowrankDesc* d_descs, const ZLowrankDesc* h_descs, int ndesc, int pairs, int rank,
                     float cscale, int shard, int nshards, cudaStream_t stream);

// Apply phase of the ES update over a table of tensors (es_kernels.cu).
struct UpdApplyDesc {
    int8_t* w;       // ternary weights (nullptr for an fp32 vector)
    float* target;   // fp32 shadow of a matrix, or the vector itself
    const float* Z;  // noise sum
    float* ema;      // the tensor's RMS-EMA slot
    int n;
    int block0;      // first 256-element block of this tensor in the launch
};
int update_apply_batched(const UpdApplyDesc* d_descs, int ndesc, int total_blocks, float* partial, float* inv_rms, int use_adaptive, float beta,
                         float eps, float lr, float thresh, cudaStream_t stream);
int z_dense_launch(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs, int idx0, int n, int use_clt, int clt_k,
                   float* Z, cudaStream_t stream);

void count_launch();

}  // namespace bnf4
