// Generates golden vectors for the NVFP4 number formats and the scale-factor layout from NVIDIA CUTLASS headers
// (the third-party dependency the reference takes them from: cutlass::float_e2m1_t, cutlass::float_ue4m3_t and
// cutlass::detail::Sm1xxBlockScaledConfig<16>, reference src/cuda_kernels.cu:1420-1421, 3837-3847).
// Build + run: see gen_golden.py. Output: a flat binary consumed by gen_golden.py.
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

#include <cutlass/detail/sm100_blockscaled_layout.hpp>
#include <cutlass/float_subbyte.h>
#include <cutlass/float8.h>
#include <cute/tensor.hpp>

int main(int argc, char** argv) {
    FILE* f = fopen(argv[1], "wb");
    // 1. e2m1: every int8 value divided by every ue4m3 scale that a block scale can take (amax/6 for amax 1..127), plus a float sweep
    std::vector<float> xs;
    for (int i = -2000; i <= 2000; ++i) xs.push_back(i * 0.005f);  // [-10, 10], hits all ties
    xs.push_back(128.0f); xs.push_back(1e9f); xs.push_back(-1e9f); xs.push_back(-0.0f);
    uint32_t n = xs.size();
    fwrite(&n, 4, 1, f);
    fwrite(xs.data(), 4, n, f);
    for (float x : xs) { uint8_t c = cutlass::float_e2m1_t(x).storage & 0xf; fwrite(&c, 1, 1, f); }
    // 2. ue4m3: sweep over magnitudes incl. subnormals, underflow and saturation
    std::vector<float> ys;
    for (int amax = 0; amax <= 127; ++amax) ys.push_back(amax > 0 ? amax / 6.0f : 1.0f);
    for (int i = 0; i < 4000; ++i) ys.push_back(0.0001f * i * i * 0.0003f + 1e-4f * i);
    for (float v : {0.0009f, 0.0015f, 0.00737f, 447.9f, 448.0f, 460.0f, 480.0f, 1e6f, 0.0073656956f}) ys.push_back(v);
    n = ys.size();
    fwrite(&n, 4, 1, f);
    fwrite(ys.data(), 4, n, f);
    for (float y : ys) {
        cutlass::float_ue4m3_t q(y);
        uint8_t b = q.storage;
        float back = static_cast<float>(q);
        fwrite(&b, 1, 1, f);
        fwrite(&back, 4, 1, f);
    }
    // 3. scale-factor layout: offsets of (row, k) for several shapes, and the allocation sizes
    using Cfg = cutlass::detail::Sm1xxBlockScaledConfig<16>;
    const int shapes[][2] = {{32, 512}, {32, 1024}, {4096, 512}, {1, 512}, {1568, 512}, {129, 64}, {300, 2048}, {256, 128}};
    n = sizeof(shapes) / sizeof(shapes[0]);
    fwrite(&n, 4, 1, f);
    for (auto& s : shapes) {
        const int rows = s[0], K = s[1];
        auto layout = Cfg::tile_atom_to_shape_SFA(cute::make_shape(rows, 1, K, 1));
        const uint64_t bytes = cute::size(cute::filter_zeros(layout));
        fwrite(&rows, 4, 1, f); fwrite(&K, 4, 1, f); fwrite(&bytes, 8, 1, f);
        for (int r = 0; r < rows; ++r)
            for (int k = 0; k < K; k += 16) {
                const uint32_t off = layout(cute::make_coord(r, k, 0));
                fwrite(&off, 4, 1, f);
            }
        // SFB uses the same atom on (N, K)
        auto layout_b = Cfg::tile_atom_to_shape_SFB(cute::make_shape(1, rows, K, 1));
        const uint32_t probe = layout_b(cute::make_coord(rows - 1, K - 16, 0));
        fwrite(&probe, 4, 1, f);
    }
    fclose(f);
    return 0;
}
