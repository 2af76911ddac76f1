// Exact-integer ternary GEMM and the small rank-r helper kernels of the reference's non-NVFP4 path.
//
// Reference semantics (file:line in the reference project):
//   gemm_ternary_f     src/cuda_kernels.cu:740-762 with gemm_row_accum :163-192 -- int32 dp4a sum per group
//                      of 256 columns, fp32 accumulation across groups with scale_x[g], then * out_scale
//   lora_compute_t     src/cuda_kernels.cu:370-390
//   lora_add           src/cuda_kernels.cu:392-410
//   split_qkvb_fused   src/cuda_kernels.cu:2856-2926
// Under NVFP4 this GEMM is only a fallback (the beta row when its shape is not tensor-core friendly), so the
// kernel favours exactness and simplicity: a 32x32 output tile per CTA, operands staged in shared memory as
// packed int8 words, __dp4a inner product.

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {

namespace {

constexpr int TB = 32;   // batch rows per tile
constexpr int TR = 32;   // weight rows per tile
constexpr int TKW = 64;  // 32-bit words (=256 int8 columns, one scale group) per K step

__global__ void __launch_bounds__(256) gemm_ternary_f_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ w,
                                                             const float* __restrict__ scale_x, float out_scale, int cols,
                                                             int rows, int batch, float* __restrict__ out) {
    __shared__ int xs[TB][TKW + 1];
    __shared__ int ws[TR][TKW + 1];
    const int b0 = blockIdx.y * TB, i0 = blockIdx.x * TR;
    const int tb = threadIdx.x >> 3;         // 0..31 batch row in tile
    const int ti = (threadIdx.x & 7) * 4;    // 4 weight rows per thread
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < cols; k0 += 256) {
        __syncthreads();
        for (int e = threadIdx.x; e < TB * TKW; e += 256) {
            const int r = e / TKW, c = e % TKW;
            int wx = 0, ww = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int col = k0 + c * 4 + j;
                if (col < cols) {
                    if (b0 + r < batch) wx |= (static_cast<int>(x[static_cast<size_t>(b0 + r) * cols + col]) & 0xff) << (8 * j);
                    if (i0 + r < rows) ww |= (static_cast<int>(w[static_cast<size_t>(i0 + r) * cols + col]) & 0xff) << (8 * j);
                }
            }
            xs[r][c] = wx;
            ws[r][c] = ww;
        }
        __syncthreads();
        // a full group of 256 columns is one exact int32 sum; a tail is split into 32-column pieces like the
        // reference does (all pieces of one step share scale_x[k0/256])
        const float sx = scale_x != nullptr ? scale_x[k0 / 256] : 1.0f;
        const int words = min(TKW, (cols - k0 + 3) / 4);
        const bool full = (cols - k0) >= 256;
        const int piece = full ? TKW : 8;
        for (int c0 = 0; c0 < words; c0 += piece) {
            int s[4] = {0, 0, 0, 0};
            const int c1 = min(words, c0 + piece);
            for (int c = c0; c < c1; ++c) {
                const int xv = xs[tb][c];
#pragma unroll
                for (int u = 0; u < 4; ++u) s[u] = __dp4a(xv, ws[ti + u][c], s[u]);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) acc[u] = fmaf(sx, static_cast<float>(s[u]), acc[u]);
        }
    }
    if (b0 + tb < batch) {
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + ti + u < rows) out[static_cast<size_t>(b0 + tb) * rows + i0 + ti + u] = __fmul_rn(acc[u], out_scale);
    }
}

__global__ void lora_t_kernel(const int8_t* __restrict__ x, const int8_t* __restrict__ B, int cols, int batch, int rank,
                              int32_t* __restrict__ t) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= batch * rank) return;
    const int b = warp / rank, r = warp - b * rank;
    int acc = 0;
    for (int j = lane; j < cols; j += 32) acc += static_cast<int>(x[static_cast<size_t>(b) * cols + j]) * static_cast<int>(B[static_cast<size_t>(j) * rank + r]);
    acc = __reduce_add_sync(0xffffffffu, acc);
    if (lane == 0) t[static_cast<size_t>(b) * rank + r] = acc;
}

__global__ void lora_add_kernel(const int32_t* __restrict__ t, const int8_t* __restrict__ A, int rows, int batch, int rank,
                                float scale, float* __restrict__ out) {
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (row >= rows || b >= batch) return;
    int pert = 0;
    for (int r = 0; r < rank; ++r) pert += t[static_cast<size_t>(b) * rank + r] * static_cast<int>(A[static_cast<size_t>(row) * rank + r]);
    float& o = out[static_cast<size_t>(b) * rows + row];
    o = fmaf(scale, static_cast<float>(pert), o);
}

__global__ void split_qkvb_kernel(const float* __restrict__ in, int batch, int hidden, int fused_cols, float* __restrict__ q,
                                  float* __restrict__ k, float* __restrict__ v, float* __restrict__ beta, float beta_bias) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (b >= batch || c >= hidden) return;
    const size_t base = static_cast<size_t>(b) * fused_cols;
    const size_t ob = static_cast<size_t>(b) * hidden + c;
    q[ob] = in[base + c];
    k[ob] = in[base + hidden + c];
    v[ob] = in[base + 2 * hidden + c];
    if (c == 0) beta[b] = in[base + 3 * hidden] + beta_bias;
}

}  // namespace
}  // namespace bnf4

using namespace bnf4;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

int bnf4_gemm_ternary_f(const int8_t* x, const int8_t* w, const float* scale_x, int rows, int cols, int batch, float out_scale,
                        float* out, void* stream) {
    if (rows <= 0 || batch <= 0) return BNF4_OK;
    if (!x || !w || !out || cols <= 0) return set_error(BNF4_ERR_INVALID, "gemm_ternary_f: bad argument");
    if ((batch + TB - 1) / TB > 65535) return set_error(BNF4_ERR_INVALID, "gemm_ternary_f: batch too large");
    const dim3 grid((rows + TR - 1) / TR, (batch + TB - 1) / TB);
    gemm_ternary_f_kernel<<<grid, 256, 0, S(stream)>>>(x, w, scale_x, out_scale, cols, rows, batch, out);
    return check_launch("gemm_ternary_f_kernel");
}

int bnf4_lora_compute_t(const int8_t* x, const int8_t* B, int cols, int batch, int rank, int32_t* t, void* stream) {
    if (batch <= 0 || rank <= 0) return BNF4_OK;
    const int warps = batch * rank;
    lora_t_kernel<<<(warps + 3) / 4, 128, 0, S(stream)>>>(x, B, cols, batch, rank, t);
    return check_launch("lora_t_kernel");
}

int bnf4_lora_add(const int32_t* t, const int8_t* A, int rows, int batch, int rank, float scale, float* out, void* stream) {
    if (batch <= 0 || rows <= 0) return BNF4_OK;
    if (batch > 65535) return set_error(BNF4_ERR_INVALID, "lora_add: batch too large");
    lora_add_kernel<<<dim3((rows + 127) / 128, batch), 128, 0, S(stream)>>>(t, A, rows, batch, rank, scale, out);
    return check_launch("lora_add_kernel");
}

int bnf4_split_qkvb_fused(const float* in, int batch, int hidden, int fused_cols, float* q, float* k, float* v, float* beta,
                          float beta_bias, void* stream) {
    if (batch <= 0 || hidden <= 0) return BNF4_OK;
    if (batch > 65535) return set_error(BNF4_ERR_INVALID, "split_qkvb_fused: batch too large");
    split_qkvb_kernel<<<dim3((hidden + 127) / 128, batch), 128, 0, S(stream)>>>(in, batch, hidden, fused_cols, q, k, v, beta, beta_bias);
    return check_launch("split_qkvb_kernel");
}

}  // extern "C"
