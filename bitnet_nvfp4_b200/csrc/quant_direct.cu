// fp32 rows -> NVFP4 without the int8 stage: one ue4m3 scale per 16 elements from the block's max |x|, codes
// e2m1(x / scale). The reference's live path always goes through int8 first (src/cuda_kernels.cu:1783-1878); this is the
// "quantised on the fly from fp32" form of the benchmark description, with the same scale rule (max / 6, rounded to ue4m3,
// a scale that rounds to zero replaced by 1) and the same code rounding as nvfp4_quantize_rowmajor (:1545-1625).
// One thread per 16-element block; bandwidth-bound (64 bytes in, 9 out per block).

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {
namespace {

__global__ void quant_direct_f32_kernel(const float* __restrict__ in, int rows, int k_in, int k_out, long long ld_in,
                                        uint8_t* __restrict__ codes, uint8_t* __restrict__ sf, int k_atoms) {
    const int blocks_per_row = k_out >> 4;
    const long long gid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (gid >= static_cast<long long>(rows) * blocks_per_row) return;
    const int row = static_cast<int>(gid / blocks_per_row), kb = static_cast<int>(gid - static_cast<long long>(row) * blocks_per_row);
    const float* src = in + static_cast<size_t>(row) * ld_in + kb * 16;
    float x[16];
    if (kb * 16 + 16 <= k_in && ((reinterpret_cast<uintptr_t>(src) & 15) == 0)) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(src) + j);
            x[4 * j] = v.x; x[4 * j + 1] = v.y; x[4 * j + 2] = v.z; x[4 * j + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) x[e] = (kb * 16 + e < k_in) ? src[e] : 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int e = 0; e < 16; ++e) amax = fmaxf(amax, fabsf(x[e]));
    const float scale = amax > 0.0f ? __fdiv_rn(amax, 6.0f) : 1.0f;
    uint32_t sq = ue4m3_encode(scale);
    float scale_f = ue4m3_decode(sq);
    if (scale_f == 0.0f) { sq = 0x38u; scale_f = 1.0f; }
    uint32_t lo = 0, hi = 0;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const uint32_t c = e2m1_encode(__fdiv_rn(x[e], scale_f));
        if (e < 8) lo |= c << (4 * e);
        else hi |= c << (4 * (e - 8));
    }
    *reinterpret_cast<uint2*>(codes + (static_cast<size_t>(row) * k_out + kb * 16) / 2) = make_uint2(lo, hi);
    sf[sf_offset(row, kb, k_atoms)] = static_cast<uint8_t>(sq);
}

}  // namespace
}  // namespace bnf4

using namespace bnf4;

extern "C" int bnf4_nvfp4_quantize_f32(const float* in, int rows, int k_in, int k_out, void* out, void* sf, void* stream) {
    if (rows <= 0 || k_out <= 0) return BNF4_OK;
    if (!in || !out || !sf) return set_error(BNF4_ERR_INVALID, "nvfp4_quantize_f32: null pointer");
    if ((k_out % 16) != 0 || k_in <= 0 || k_in > k_out) return set_error(BNF4_ERR_INVALID, "nvfp4_quantize_f32: k_out=%d must be a multiple of 16 and >= k_in=%d", k_out, k_in);
    if (reinterpret_cast<uintptr_t>(out) & 7) return set_error(BNF4_ERR_INVALID, "nvfp4_quantize_f32: codes must be 8-byte aligned");
    const long long blocks = static_cast<long long>(rows) * (k_out / 16);
    const int threads = 128;
    quant_direct_f32_kernel<<<static_cast<unsigned>((blocks + threads - 1) / threads), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        in, rows, k_in, k_out, k_in, static_cast<uint8_t*>(out), static_cast<uint8_t*>(sf), sf_k_atoms(k_out));
    return check_launch("quant_direct_f32_kernel");
}
