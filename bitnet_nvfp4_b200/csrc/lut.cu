// Host-built lookup table of the NVFP4 block quantiser for int8 inputs (see quant_block16_lut in common.cuh).

#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {

namespace {
std::mutex g_lut_mu;
uint8_t* g_lut[64] = {};
}  // namespace

const uint8_t* get_quant_lut() {
    int dev = 0;
    if (check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return nullptr;
    if (dev < 0 || dev >= 64) { set_error(BNF4_ERR_INVALID, "device index %d out of range", dev); return nullptr; }
    std::lock_guard<std::mutex> lock(g_lut_mu);
    if (g_lut[dev] != nullptr) return g_lut[dev];
    std::vector<uint8_t> h(kQuantLutBytes, 0);
    for (int amax = 0; amax < 128; ++amax) {
        const float scale = amax > 0 ? static_cast<float>(amax) / 6.0f : 1.0f;
        uint32_t sq = ue4m3_encode_host(scale);
        float sf = ue4m3_decode(sq);
        if (sf == 0.0f) { sq = 0x38u; sf = 1.0f; }
        h[kQuantLutCodeBytes + amax] = static_cast<uint8_t>(sq);
        for (int a = 0; a < 128; ++a) h[amax * 128 + a] = static_cast<uint8_t>(e2m1_encode(static_cast<float>(a) / sf) & 7u);
        const float rcp = 1.0f / sf;
        uint32_t rcp_bits;
        memcpy(&rcp_bits, &rcp, 4);
        uint8_t* entry = h.data() + kQuantBlockTabOffset + amax * 8;
        memcpy(entry, &rcp_bits, 4);
        memcpy(entry + 4, &sq, 4);
    }
    uint8_t* d = nullptr;
    if (check_cuda(cudaMalloc(&d, kQuantLutBytes), "cudaMalloc(quant lut)")) return nullptr;
    if (check_cuda(cudaMemcpy(d, h.data(), kQuantLutBytes, cudaMemcpyHostToDevice), "cudaMemcpy(quant lut)")) {
        cudaFree(d);
        return nullptr;
    }
    g_lut[dev] = d;
    return d;
}

}  // namespace bnf4
