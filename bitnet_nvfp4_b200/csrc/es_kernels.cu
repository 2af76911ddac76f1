// Cross-entropy fitness, counter-hash noise and the ES weight update (bandwidth / integer-pipe kernels).
//
// Reference semantics restated here (file:line in the reference project):
//   cross entropy          src/efla_lm_kernels.cu:252-311
//   noise fill             src/efla_lm_kernels.cu:73-86, 352-385
//   pair seeds             src/efla_lm_kernels.cu:1844-1852
//   Z and sum of squares   src/efla_lm_kernels.cu:1854-1890
//   inv_rms                src/efla_lm_kernels.cu:2003-2021
//   shadow update          src/efla_lm_kernels.cu:1892-1922
// All reductions run in a fixed order so that every rank of a data-parallel job computes identical bits
// (the reference uses unordered float atomics).

#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {

namespace {

// ------------------------------------------------------------------------------------------------
// Cross entropy. One warp per row; lane l holds logits l, l+32, ...
// ------------------------------------------------------------------------------------------------
constexpr int kCeMaxPerLane = 32;  // vocab <= 1024

__device__ __forceinline__ float ce_row_loss(const float* lg, const float* bias, const float* noise_f, const int8_t* noise_i,
                                             float bns, int vocab, int y, int lane) {
    float v[kCeMaxPerLane];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < kCeMaxPerLane; ++j) {
        const int i = lane + 32 * j;
        if (i < vocab) {
            float x = lg[i];
            if (bias != nullptr) x += bias[i];
            if (noise_f != nullptr) x = fmaf(bns, noise_f[i], x);
            if (noise_i != nullptr) x = fmaf(bns, static_cast<float>(noise_i[i]), x);
            v[j] = x;
            mx = fmaxf(mx, x);
        } else {
            v[j] = -INFINITY;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < kCeMaxPerLane; ++j) {
        const int i = lane + 32 * j;
        if (i < vocab) sum += expf(v[j] - mx);
    }
    sum = warp_sum_f(sum);
    // the target's value lives in lane y%32, slot y/32
    float vy = 0.0f;
#pragma unroll
    for (int j = 0; j < kCeMaxPerLane; ++j)
        if (j == (y >> 5)) vy = v[j];
    vy = __shfl_sync(0xffffffffu, vy, y & 31);
    return -(vy - mx - logf(sum + 1e-9f));
}

// API form: a single CTA sums the rows of one token step in a fixed order and adds the total to *loss_accum.
__global__ void __launch_bounds__(256) ce_step_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                      const float* __restrict__ bias_noise, float bns,
                                                      const uint8_t* __restrict__ targets_t, int token_stride, int vocab, int batch,
                                                      float* loss_accum) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float acc = 0.0f;
    for (int b = warp; b < batch; b += 8) {
        const int y = static_cast<int>(targets_t[static_cast<size_t>(b) * token_stride]);
        acc += ce_row_loss(logits + static_cast<size_t>(b) * vocab, bias, bias_noise, nullptr, bns, vocab, y, lane);
    }
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t += part[w];
        loss_accum[0] += t;
    }
}

// Population form: grid (16 chunks, members). partial[member*16 + chunk] = sum of the chunk's row losses.
constexpr int kCeChunks = 16;
__global__ void __launch_bounds__(256) ce_population_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias,
                                                            const int8_t* __restrict__ bias_noise, float sigma,
                                                            const uint8_t* __restrict__ targets, int vocab, int rows_per_member,
                                                            float* __restrict__ partial) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = blockIdx.y, chunk = blockIdx.x;
    const int per = (rows_per_member + kCeChunks - 1) / kCeChunks;
    const int r0 = chunk * per, r1 = min(rows_per_member, r0 + per);
    const float bns = (member & 1) ? -sigma : sigma;
    const int8_t* nz = bias_noise != nullptr ? bias_noise + static_cast<size_t>(member >> 1) * vocab : nullptr;
    float acc = 0.0f;
    for (int r = r0 + warp; r < r1; r += 8) {
        const size_t row = static_cast<size_t>(member) * rows_per_member + r;
        acc += ce_row_loss(logits + row * ld, bias, nullptr, nz, bns, vocab, static_cast<int>(targets[r]), lane);
    }
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t += part[w];
        partial[member * kCeChunks + chunk] = t;
    }
}

// Streaming form of the same reduction for 16-byte aligned rows and vocab % 4 == 0: lane l owns the float4 groups
// l, l + 32, ... of a row (NV4 groups), the member's bias and noise stay in registers for all rows, and RPI rows are in
// flight per warp so that the load latency of one row hides behind the reductions of the others. The warps walk the
// rows in the same order and add the row losses in the same order as ce_population_kernel.
template <int NV4, int RPI>
__global__ void __launch_bounds__(256) ce_population_vec_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ bias,
                                                                const int8_t* __restrict__ bias_noise, float sigma,
                                                                const uint8_t* __restrict__ targets, int vocab, int rows_per_member,
                                                                float* __restrict__ partial) {
    __shared__ float part[8];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int member = blockIdx.y, chunk = blockIdx.x;
    const int per = (rows_per_member + kCeChunks - 1) / kCeChunks;
    const int r0 = chunk * per, r1 = min(rows_per_member, r0 + per);
    const float bns = (member & 1) ? -sigma : sigma;
    const int groups = vocab >> 2;
    float4 bv[NV4], nv[NV4];
#pragma unroll
    for (int j = 0; j < NV4; ++j) {
        const int gi = lane + 32 * j;
        bv[j] = nv[j] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (gi < groups) {
            if (bias != nullptr) bv[j] = *reinterpret_cast<const float4*>(bias + 4 * gi);
            if (bias_noise != nullptr) {
                const char4 c = *reinterpret_cast<const char4*>(bias_noise + static_cast<size_t>(member >> 1) * vocab + 4 * gi);
                nv[j] = make_float4(static_cast<float>(c.x), static_cast<float>(c.y), static_cast<float>(c.z), static_cast<float>(c.w));
            }
        }
    }
    float acc = 0.0f;
    for (int rb = r0 + warp; rb < r1; rb += 8 * RPI) {
        float4 x[RPI][NV4];
        int y[RPI];
#pragma unroll
        for (int i = 0; i < RPI; ++i) {
            const int r = rb + 8 * i;
            y[i] = r < r1 ? static_cast<int>(targets[r]) : 0;
            const float* lg = logits + (static_cast<size_t>(member) * rows_per_member + min(r, r1 - 1)) * ld;
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                const int gi = lane + 32 * j;
                x[i][j] = gi < groups ? __ldcs(reinterpret_cast<const float4*>(lg) + gi) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
        }
#pragma unroll
        for (int i = 0; i < RPI; ++i) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < NV4; ++j) {
                if (lane + 32 * j < groups) {  // (x + bias) + bns * noise, like the scalar kernel (zero bias / noise when absent)
                    x[i][j].x = fmaf(bns, nv[j].x, x[i][j].x + bv[j].x);
                    x[i][j].y = fmaf(bns, nv[j].y, x[i][j].y + bv[j].y);
                    x[i][j].z = fmaf(bns, nv[j].z, x[i][j].z + bv[j].z);
                    x[i][j].w = fmaf(bns, nv[j].w, x[i][j].w + bv[j].w);
                }
                mx = fmaxf(fmaxf(mx, fmaxf(x[i][j].x, x[i][j].y)), fmaxf(x[i][j].z, x[i][j].w));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            float sum = 0.0f;
#pragma unroll
            for (int j = 0; j < NV4; ++j) sum += (expf(x[i][j].x - mx) + expf(x[i][j].y - mx)) + (expf(x[i][j].z - mx) + expf(x[i][j].w - mx));
            sum = warp_sum_f(sum);
            // the target's logit is re-read (one broadcast load per row) and perturbed with the same two operations
            const int r = min(rb + 8 * i, r1 - 1);
            float vy = logits[(static_cast<size_t>(member) * rows_per_member + r) * ld + y[i]];
            if (bias != nullptr) vy += bias[y[i]];
            if (bias_noise != nullptr) vy = fmaf(bns, static_cast<float>(bias_noise[static_cast<size_t>(member >> 1) * vocab + y[i]]), vy);
            if (rb + 8 * i < r1) acc += -(vy - mx - logf(sum + 1e-9f));
        }
    }
    if (lane == 0) part[warp] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float t = 0.0f;
        for (int w = 0; w < 8; ++w) t += part[w];
        partial[member * kCeChunks + chunk] = t;
    }
}

__global__ void ce_finalize_kernel(const float* __restrict__ partial, int members, int rows_per_member, float* __restrict__ loss_mean) {
    const int m = blockIdx.x * blockDim.x + threadIdx.x;
    if (m >= members) return;
    double t = 0.0;
    for (int c = 0; c < kCeChunks; ++c) t += static_cast<double>(partial[m * kCeChunks + c]);
    loss_mean[m] = static_cast<float>(t / static_cast<double>(rows_per_member));
}

// ------------------------------------------------------------------------------------------------
// Noise
// ------------------------------------------------------------------------------------------------
__global__ void fill_noise_kernel(int8_t* __restrict__ out, size_t n, uint64_t seed, int use_clt, int clt_k) {
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx < n) out[idx] = static_cast<int8_t>(noise_hash(seed, idx, use_clt != 0, clt_k));
}
__global__ void fill_noise_batched_kernel(const bnf4_noise_desc* __restrict__ descs, int num_desc, int use_clt, int clt_k) {
    const int di = blockIdx.y;
    if (di >= num_desc) return;
    const bnf4_noise_desc d = descs[di];
    const size_t idx = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (idx < d.n) d.out[idx] = static_cast<int8_t>(noise_hash(d.seed, idx, use_clt != 0, clt_k));
}
__global__ void fill_float_noise_kernel(float* __restrict__ out, int n, uint64_t seed, int use_clt, int clt_k) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) out[idx] = static_cast<float>(noise_hash(seed, static_cast<uint64_t>(idx), use_clt != 0, clt_k));
}
__global__ void pair_seeds_kernel(uint64_t base_seed, uint64_t epoch, int pairs, uint64_t* __restrict__ out) {
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p < pairs) out[p] = mix_u64(base_seed, mix_u64(epoch, static_cast<uint64_t>(p)));
}

// ------------------------------------------------------------------------------------------------
// ES update
// ------------------------------------------------------------------------------------------------
__global__ void init_shadow_kernel(const int8_t* __restrict__ w, float* __restrict__ shadow, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) shadow[i] = static_cast<float>(w[i]);
}

// Z for the dense (full-matrix noise) form; 256 threads per block, one element each.
// Elements idx0 .. idx0 + n - 1 of the vector (the hash is keyed by the element's index in the whole vector) go to Z[0 .. n).
__global__ void __launch_bounds__(256) z_dense_kernel(const float* __restrict__ pair_weights, const uint64_t* __restrict__ pair_seeds,
                                                      uint64_t salt, int pairs, int idx0, int n, int use_clt, int clt_k, float* __restrict__ Z) {
    extern __shared__ uint8_t zsm[];
    uint64_t* seeds = reinterpret_cast<uint64_t*>(zsm);
    float* wts = reinterpret_cast<float*>(zsm + sizeof(uint64_t) * 256);
    const int idx = blockIdx.x * 256 + threadIdx.x;
    float z = 0.0f;
    for (int p0 = 0; p0 < pairs; p0 += 256) {
        __syncthreads();
        if (p0 + threadIdx.x < pairs) {
            seeds[threadIdx.x] = mix_u64(pair_seeds[p0 + threadIdx.x], salt);
            wts[threadIdx.x] = pair_weights[p0 + threadIdx.x];
        }
        __syncthreads();
        const int cnt = min(256, pairs - p0);
        if (idx < n) {
            // four independent hash chains in flight; the multiply-adds stay in pair order (pairs of weight zero are skipped,
            // like in the reference)
            int p = 0;
            for (; p + 4 <= cnt; p += 4) {
                float e[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) e[q] = static_cast<float>(noise_hash(seeds[p + q], static_cast<uint64_t>(idx0 + idx), use_clt != 0, clt_k));
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float w = wts[p + q];
                    if (w != 0.0f) z = fmaf(w, e[q], z);
                }
            }
            for (; p < cnt; ++p) {
                const float w = wts[p];
                if (w == 0.0f) continue;
                z = fmaf(w, static_cast<float>(noise_hash(seeds[p], static_cast<uint64_t>(idx0 + idx), use_clt != 0, clt_k)), z);
            }
        }
    }
    if (idx < n) Z[idx] = z;
}

// Rank-r form of Z: Z[i][j] = cscale * sum_p w_p * (sum_r A[p][i][r] * B[p][r][j]), pairs in ascending order with one fused
// multiply-add per pair (reference: src/efla_lm_kernels.cu:1854-1890 applied to the factored noise). The inner sum is a
// small integer, so it is formed exactly in fp32 from factors converted once while they are staged in shared memory.
//
// One launch covers a table of matrices (all ternary matrices of a model): block b locates its matrix and its
// 32-row x 64-column tile by walking the table. Thread (ty, tx) of the 8 x 16 thread tile keeps a 4 x 4 block of Z in
// registers, so one pair costs three shared-memory loads (weight, 4 values of A, 4 of B) for 32 arithmetic
// instructions; factors arrive in chunks of PC pairs, the next chunk's global loads in flight while the current one is
// consumed (registers -> the other shared-memory buffer, one barrier per chunk). With nshards > 1 a matrix whose rows
// divide by nshards is computed only for the rows of this shard.
constexpr int kZTileRows = 32, kZTileCols = 64, kZThreads = 128;

__device__ __forceinline__ void z_shard_rows(int rows, int shard, int nshards, int& r0, int& nr) {
    r0 = 0;
    nr = rows;
    if (nshards > 1 && rows >= nshards && (rows % nshards) == 0) { nr = rows / nshards; r0 = shard * nr; }
}

template <int RANK>
__global__ void __launch_bounds__(kZThreads) z_lowrank_tiles_kernel(const float* __restrict__ pair_weights, const ZLowrankDesc* __restrict__ descs,
                                                                    int ndesc, const ZLowrankDesc single, int pairs, float cscale, int shard,
                                                                    int nshards) {
    constexpr int PC = RANK <= 2 ? 16 : 8;  // pairs per chunk
    constexpr int TR = kZTileRows, TC = kZTileCols;
    constexpr int A_PER_THREAD = PC * TR * RANK / kZThreads;        // bytes of A per thread and chunk
    constexpr int B_PER_THREAD = PC * RANK * (TC / 4) / kZThreads;  // 4-byte words of B per thread and chunk
    __shared__ __align__(16) float a_sh[2][PC][RANK][TR];
    __shared__ __align__(16) float b_sh[2][PC][RANK][TC];
    __shared__ float w_sh[2][PC];

    // which matrix, which tile
    ZLowrankDesc d = single;
    int tile = static_cast<int>(blockIdx.x);
    int r0 = 0, nr = d.rows;
    if (ndesc > 0) {
        int i = 0;
        for (;;) {
            d = descs[i];
            z_shard_rows(d.rows, shard, nshards, r0, nr);
            const int tiles = ((nr + TR - 1) / TR) * ((d.cols + TC - 1) / TC);
            if (tile < tiles) break;
            tile -= tiles;
            if (++i >= ndesc) return;
        }
    }
    const int tiles_x = (d.cols + TC - 1) / TC;
    const int by = tile / tiles_x, bx = tile - by * tiles_x;
    const int row_base = r0 + by * TR, row_end = r0 + nr, col_base = bx * TC;
    const int tid = static_cast<int>(threadIdx.x), ty = tid >> 4, tx = tid & 15;
    const bool b_words = ((reinterpret_cast<uintptr_t>(d.B) & 3) == 0) && ((d.B_ps & 3) == 0) && ((d.cols & 3) == 0);

    int a_raw[A_PER_THREAD];
    uint32_t b_raw[B_PER_THREAD];
    float w_raw = 0.0f;
    auto fetch = [&](int p0) {
#pragma unroll
        for (int k = 0; k < A_PER_THREAD; ++k) {
            const int e = tid + k * kZThreads;
            const int pp = e / (TR * RANK), rem = e - pp * (TR * RANK);  // rem = row * RANK + r: contiguous in A
            const int row = row_base + rem / RANK;
            a_raw[k] = (p0 + pp < pairs && row < row_end) ? static_cast<int>(d.A[static_cast<size_t>(p0 + pp) * d.A_ps + static_cast<size_t>(row_base) * RANK + rem]) : 0;
        }
#pragma unroll
        for (int k = 0; k < B_PER_THREAD; ++k) {
            const int e = tid + k * kZThreads;
            const int pp = e / (RANK * (TC / 4)), rem = e - pp * (RANK * (TC / 4)), r = rem / (TC / 4), c = (rem - r * (TC / 4)) * 4;
            const int col = col_base + c;
            uint32_t v = 0;
            if (p0 + pp < pairs && col < d.cols) {
                const int8_t* src = d.B + static_cast<size_t>(p0 + pp) * d.B_ps + static_cast<size_t>(r) * d.cols + col;
                if (b_words) {
                    v = *reinterpret_cast<const uint32_t*>(src);
                } else {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        if (col + q < d.cols) v |= (static_cast<uint32_t>(static_cast<uint8_t>(src[q]))) << (8 * q);
                }
            }
            b_raw[k] = v;
        }
        if (tid < PC) w_raw = (p0 + tid < pairs) ? pair_weights[p0 + tid] : 0.0f;
    };
    auto stage = [&](int buf) {
#pragma unroll
        for (int k = 0; k < A_PER_THREAD; ++k) {
            const int e = tid + k * kZThreads;
            const int pp = e / (TR * RANK), rem = e - pp * (TR * RANK);
            a_sh[buf][pp][rem % RANK][rem / RANK] = static_cast<float>(a_raw[k]);
        }
#pragma unroll
        for (int k = 0; k < B_PER_THREAD; ++k) {
            const int e = tid + k * kZThreads;
            const int pp = e / (RANK * (TC / 4)), rem = e - pp * (RANK * (TC / 4)), r = rem / (TC / 4), c = (rem - r * (TC / 4)) * 4;
            float f[4];
            bytes4_to_float(b_raw[k], f);
            *reinterpret_cast<float4*>(&b_sh[buf][pp][r][c]) = make_float4(f[0], f[1], f[2], f[3]);
        }
        if (tid < PC) w_sh[buf][tid] = w_raw;
    };

    float z[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) z[i][j] = 0.0f;

    fetch(0);
    stage(0);
    __syncthreads();
    int buf = 0;
    for (int p0 = 0; p0 < pairs; p0 += PC, buf ^= 1) {
        const bool more = p0 + PC < pairs;
        if (more) fetch(p0 + PC);
        const int cnt = min(PC, pairs - p0);
#pragma unroll 4
        for (int pp = 0; pp < cnt; ++pp) {
            const float w = w_sh[buf][pp];
            float e[4][4];
#pragma unroll
            for (int r = 0; r < RANK; ++r) {
                const float4 a4 = *reinterpret_cast<const float4*>(&a_sh[buf][pp][r][ty * 4]);
                const float4 b4 = *reinterpret_cast<const float4*>(&b_sh[buf][pp][r][tx * 4]);
                const float av[4] = {a4.x, a4.y, a4.z, a4.w}, bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) e[i][j] = r == 0 ? __fmul_rn(av[i], bv[j]) : fmaf(av[i], bv[j], e[i][j]);  // exact: small integers
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) z[i][j] = fmaf(w, e[i][j], z[i][j]);
        }
        if (more) stage(buf ^ 1);
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int row = row_base + ty * 4 + i;
        if (row >= row_end) continue;
        float* dst = d.Z + static_cast<size_t>(row) * d.cols + col_base + tx * 4;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (col_base + tx * 4 + j < d.cols) dst[j] = __fmul_rn(cscale, z[i][j]);
    }
}

// Sum of squares, stage 1: block b reduces Z[256b .. 256b+255] with the reference's shared-memory tree.
__global__ void __launch_bounds__(256) sumsq_blocks_kernel(const float* __restrict__ Z, int n, float* __restrict__ partial) {
    __shared__ float sh[256];
    const int idx = blockIdx.x * 256 + threadIdx.x;
    const float z = idx < n ? Z[idx] : 0.0f;
    sh[threadIdx.x] = __fmul_rn(z, z);
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
// stage 2: one warp adds the block partials in double (lane-contiguous ranges, then lanes in order) and
// accumulates into *sumsq.
__global__ void sumsq_final_kernel(const float* __restrict__ partial, int nblocks, float* sumsq) {
    __shared__ double lane_sum[32];
    const int lane = threadIdx.x;
    const int per = (nblocks + 31) / 32;
    double t = 0.0;
    for (int b = lane * per; b < min(nblocks, (lane + 1) * per); ++b) t += static_cast<double>(partial[b]);
    lane_sum[lane] = t;
    __syncwarp();
    if (lane == 0) {
        double tot = 0.0;
        for (int l = 0; l < 32; ++l) tot += lane_sum[l];
        sumsq[0] += static_cast<float>(tot);
    }
}

__global__ void inv_rms_kernel(const float* __restrict__ sumsq, float* __restrict__ rms_ema, int use_adaptive, float beta, float eps,
                               int n, float* __restrict__ inv_rms_out) {
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    float inv = 1.0f;
    if (use_adaptive) {
        const float ms = __fdiv_rn(sumsq[0], static_cast<float>(n));
        float ema = rms_ema[0];
        if (ema == 0.0f) ema = ms;
        ema = fmaf(beta, ema, __fmul_rn(1.0f - beta, ms));
        rms_ema[0] = ema;
        inv = __fdiv_rn(1.0f, __fsqrt_rn(ema + eps));
    }
    inv_rms_out[0] = inv;
}

__global__ void update_shadow_kernel(int8_t* __restrict__ w, float* __restrict__ shadow, const float* __restrict__ Z, int n,
                                     const float* __restrict__ inv_rms_dev, float inv_rms_host, float lr, float thresh) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float inv = inv_rms_dev != nullptr ? inv_rms_dev[0] : inv_rms_host;
    const float g = __fmul_rn(inv, Z[i]);
    if (fabsf(g) < thresh) return;
    const float s = fmaf(lr, g, shadow[i]);
    shadow[i] = s;
    w[i] = static_cast<int8_t>(clip_ternary(__float2int_rn(s)));
}

__global__ void update_vector_kernel(float* __restrict__ v, const float* __restrict__ Z, int n, const float* __restrict__ inv_rms,
                                     float lr, float thresh) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float g = __fmul_rn(inv_rms[0], Z[i]);
    if (fabsf(g) < thresh) return;
    v[i] = fmaf(lr, g, v[i]);
}

__global__ void add_scaled_kernel(float* __restrict__ out, const float* __restrict__ noise, int n, float scale) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = fmaf(scale, noise[i], out[i]);
}

// ---- the apply phase of the ES update for a table of tensors: four launches instead of five per tensor -------------------
// Same arithmetic, block structure and summation order as sumsq_blocks / sumsq_final / inv_rms / update_shadow /
// update_vector above, so the bits are those of the per-tensor calls. Block b of the grid belongs to the tensor whose
// [block0, block0 + ceil(n / 256)) contains it.
__device__ __forceinline__ int find_tensor(const UpdApplyDesc* __restrict__ d, int ndesc, int block) {
    int lo = 0, hi = ndesc - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (d[mid].block0 <= block) lo = mid; else hi = mid - 1;
    }
    return lo;
}
__global__ void __launch_bounds__(256) sumsq_blocks_batched_kernel(const UpdApplyDesc* __restrict__ d, int ndesc, float* __restrict__ partial) {
    __shared__ float sh[256];
    __shared__ int ti;
    if (threadIdx.x == 0) ti = find_tensor(d, ndesc, static_cast<int>(blockIdx.x));
    __syncthreads();
    const UpdApplyDesc& x = d[ti];
    const int idx = (static_cast<int>(blockIdx.x) - x.block0) * 256 + threadIdx.x;
    const float z = idx < x.n ? x.Z[idx] : 0.0f;
    sh[threadIdx.x] = __fmul_rn(z, z);
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = sh[0];
}
// one warp per tensor; then its lane 0 turns the sum into inv_rms (and advances the tensor's RMS-EMA)
__global__ void sumsq_final_inv_rms_batched_kernel(const UpdApplyDesc* __restrict__ d, const float* __restrict__ partial, int use_adaptive,
                                                   float beta, float eps, float* __restrict__ inv_rms_out) {
    __shared__ double lane_sum[32];
    const UpdApplyDesc& x = d[blockIdx.x];
    const int lane = threadIdx.x;
    const int nblocks = (x.n + 255) / 256;
    const float* part = partial + x.block0;
    const int per = (nblocks + 31) / 32;
    double t = 0.0;
    for (int b = lane * per; b < min(nblocks, (lane + 1) * per); ++b) t += static_cast<double>(part[b]);
    lane_sum[lane] = t;
    __syncwarp();
    if (lane == 0) {
        double tot = 0.0;
        for (int l = 0; l < 32; ++l) tot += lane_sum[l];
        const float sumsq = static_cast<float>(tot);
        float inv = 1.0f;
        if (use_adaptive) {
            const float ms = __fdiv_rn(sumsq, static_cast<float>(x.n));
            float ema = x.ema[0];
            if (ema == 0.0f) ema = ms;
            ema = fmaf(beta, ema, __fmul_rn(1.0f - beta, ms));
            x.ema[0] = ema;
            inv = __fdiv_rn(1.0f, __fsqrt_rn(ema + eps));
        }
        inv_rms_out[blockIdx.x] = inv;
    }
}
__global__ void __launch_bounds__(256) update_batched_kernel(const UpdApplyDesc* __restrict__ d, int ndesc, const float* __restrict__ inv_rms,
                                                             float lr, float thresh) {
    __shared__ int ti;
    if (threadIdx.x == 0) ti = find_tensor(d, ndesc, static_cast<int>(blockIdx.x));
    __syncthreads();
    const UpdApplyDesc& x = d[ti];
    const int i = (static_cast<int>(blockIdx.x) - x.block0) * 256 + threadIdx.x;
    if (i >= x.n) return;
    const float g = __fmul_rn(inv_rms[ti], x.Z[i]);
    if (fabsf(g) < thresh) return;
    const float s = fmaf(lr, g, x.target[i]);
    x.target[i] = s;
    if (x.w != nullptr) x.w[i] = static_cast<int8_t>(clip_ternary(__float2int_rn(s)));
}

// library-owned scratch for the block partials of sum(Z^2), one per device
struct Scratch {
    float* ptr = nullptr;
    size_t floats = 0;
};
std::mutex g_scratch_mu;
Scratch g_scratch[64];

int get_scratch(size_t floats, float** out) {
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return set_error(BNF4_ERR_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    Scratch& s = g_scratch[dev];
    if (s.floats < floats) {
        // stream-ordered users of the old buffer may still be running: synchronise before freeing it
        if (s.ptr != nullptr) {
            rc = check_cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
            if (rc) return rc;
            cudaFree(s.ptr);
            s.ptr = nullptr;
            s.floats = 0;
        }
        const size_t want = floats < 65536 ? 65536 : floats;
        rc = check_cuda(cudaMalloc(&s.ptr, want * sizeof(float)), "cudaMalloc(sumsq scratch)");
        if (rc) return rc;
        s.floats = want;
    }
    *out = s.ptr;
    return BNF4_OK;
}

}  // namespace

// Dense-noise Z of elements idx0 .. idx0 + n - 1 of a vector into Z[0 .. n).
int z_dense_launch(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs, int idx0, int n, int use_clt, int clt_k,
                   float* Z, cudaStream_t st) {
    if (n <= 0) return BNF4_OK;
    z_dense_kernel<<<(n + 255) / 256, 256, 256 * (sizeof(uint64_t) + sizeof(float)), st>>>(pair_weights, pair_seeds, salt, pairs, idx0, n, use_clt, clt_k, Z);
    return check_launch("z_dense_kernel");
}

// Apply phase for a table of tensors (block0 filled by the caller: running sum of ceil(n / 256)); partial holds one float
// per block, inv_rms one per tensor.
int update_apply_batched(const UpdApplyDesc* d_descs, int ndesc, int total_blocks, float* partial, float* inv_rms, int use_adaptive, float beta,
                         float eps, float lr, float thresh, cudaStream_t st) {
    if (ndesc <= 0 || total_blocks <= 0) return BNF4_OK;
    sumsq_blocks_batched_kernel<<<total_blocks, 256, 0, st>>>(d_descs, ndesc, partial);
    int rc = check_launch("sumsq_blocks_batched_kernel");
    if (rc) return rc;
    sumsq_final_inv_rms_batched_kernel<<<ndesc, 32, 0, st>>>(d_descs, partial, use_adaptive, beta, eps, inv_rms);
    rc = check_launch("sumsq_final_inv_rms_batched_kernel");
    if (rc) return rc;
    update_batched_kernel<<<total_blocks, 256, 0, st>>>(d_descs, ndesc, inv_rms, lr, thresh);
    return check_launch("update_batched_kernel");
}

// d_descs: the table in device memory (nullptr with ndesc == 0: the single matrix h_descs[0], passed by value).
// h_descs: the same table in host memory, for the grid size.
int z_lowrank_launch(const float* pair_weights, const ZLowrankDesc* d_descs, const ZLowrankDesc* h_descs, int ndesc, int pairs, int rank,
                     float cscale, int shard, int nshards, cudaStream_t st) {
    if (rank < 1 || rank > 4) return set_error(BNF4_ERR_INVALID, "compute_z_lowrank: rank=%d outside [1,4]", rank);
    if (nshards < 1 || shard < 0 || shard >= nshards) return set_error(BNF4_ERR_INVALID, "compute_z_lowrank: shard %d of %d", shard, nshards);
    if (pairs <= 0) return set_error(BNF4_ERR_INVALID, "compute_z_lowrank: pairs=%d", pairs);
    long long tiles = 0;
    for (int i = 0; i < std::max(ndesc, 1); ++i) {
        int nr = h_descs[i].rows;
        if (ndesc > 0 && nshards > 1 && nr >= nshards && (nr % nshards) == 0) nr /= nshards;
        tiles += static_cast<long long>((nr + kZTileRows - 1) / kZTileRows) * ((h_descs[i].cols + kZTileCols - 1) / kZTileCols);
    }
    if (tiles <= 0) return BNF4_OK;
    if (tiles > 0x7fffffffLL) return set_error(BNF4_ERR_INVALID, "compute_z_lowrank: too many tiles");
    const unsigned grid = static_cast<unsigned>(tiles);
    const ZLowrankDesc single = h_descs[0];
    switch (rank) {
        case 1: z_lowrank_tiles_kernel<1><<<grid, kZThreads, 0, st>>>(pair_weights, d_descs, ndesc, single, pairs, cscale, shard, nshards); break;
        case 2: z_lowrank_tiles_kernel<2><<<grid, kZThreads, 0, st>>>(pair_weights, d_descs, ndesc, single, pairs, cscale, shard, nshards); break;
        case 3: z_lowrank_tiles_kernel<3><<<grid, kZThreads, 0, st>>>(pair_weights, d_descs, ndesc, single, pairs, cscale, shard, nshards); break;
        default: z_lowrank_tiles_kernel<4><<<grid, kZThreads, 0, st>>>(pair_weights, d_descs, ndesc, single, pairs, cscale, shard, nshards); break;
    }
    return check_launch("z_lowrank_tiles_kernel");
}

namespace {

int sumsq_into(const float* Z, int n, float* sumsq, cudaStream_t st) {
    const int nblocks = (n + 255) / 256;
    float* partial = nullptr;
    int rc = get_scratch(static_cast<size_t>(nblocks), &partial);
    if (rc) return rc;
    sumsq_blocks_kernel<<<nblocks, 256, 0, st>>>(Z, n, partial);
    rc = check_launch("sumsq_blocks_kernel");
    if (rc) return rc;
    sumsq_final_kernel<<<1, 32, 0, st>>>(partial, nblocks, sumsq);
    return check_launch("sumsq_final_kernel");
}

}  // namespace

int sumsq_with_scratch(const float* Z, int n, float* partial, float* sumsq, cudaStream_t st) {
    const int nblocks = (n + 255) / 256;
    sumsq_blocks_kernel<<<nblocks, 256, 0, st>>>(Z, n, partial);
    int rc = check_launch("sumsq_blocks_kernel");
    if (rc) return rc;
    sumsq_final_kernel<<<1, 32, 0, st>>>(partial, nblocks, sumsq);
    return check_launch("sumsq_final_kernel");
}

}  // namespace bnf4

using namespace bnf4;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

int bnf4_cross_entropy_loss(const float* logits, const float* bias, const float* bias_noise, float bias_noise_scale,
                            const uint8_t* targets_t, int token_stride, int vocab, int batch, float* loss_accum, void* stream) {
    if (batch <= 0) return BNF4_OK;
    if (!logits || !targets_t || !loss_accum) return set_error(BNF4_ERR_INVALID, "cross_entropy_loss: null pointer");
    if (vocab <= 0 || vocab > 32 * kCeMaxPerLane) return set_error(BNF4_ERR_INVALID, "cross_entropy_loss: vocab=%d outside [1,%d]", vocab, 32 * kCeMaxPerLane);
    ce_step_kernel<<<1, 256, 0, S(stream)>>>(logits, bias, bias_noise, bias_noise_scale, targets_t, token_stride, vocab, batch, loss_accum);
    return check_launch("ce_step_kernel");
}

int bnf4_cross_entropy_population(const float* logits, int ld, const float* bias, const int8_t* bias_noise, float sigma,
                                  const uint8_t* targets, int vocab, int members, int rows_per_member, float* partial,
                                  float* loss_mean, void* stream) {
    if (members <= 0 || rows_per_member <= 0) return BNF4_OK;
    if (!logits || !targets || !partial || !loss_mean) return set_error(BNF4_ERR_INVALID, "cross_entropy_population: null pointer");
    if (vocab <= 0 || vocab > 32 * kCeMaxPerLane) return set_error(BNF4_ERR_INVALID, "cross_entropy_population: vocab=%d", vocab);
    if (members > 65535) return set_error(BNF4_ERR_INVALID, "cross_entropy_population: at most 65535 members per call");
    const dim3 grid(kCeChunks, members);
    const bool vec = (vocab % 4) == 0 && (ld % 4) == 0 && ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(bias)) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(bias_noise) & 3) == 0;
    if (vec && vocab <= 128)
        ce_population_vec_kernel<1, 4><<<grid, 256, 0, S(stream)>>>(logits, ld, bias, bias_noise, sigma, targets, vocab, rows_per_member, partial);
    else if (vec && vocab <= 256)
        ce_population_vec_kernel<2, 4><<<grid, 256, 0, S(stream)>>>(logits, ld, bias, bias_noise, sigma, targets, vocab, rows_per_member, partial);
    else if (vec && vocab <= 512)
        ce_population_vec_kernel<4, 2><<<grid, 256, 0, S(stream)>>>(logits, ld, bias, bias_noise, sigma, targets, vocab, rows_per_member, partial);
    else if (vec)
        ce_population_vec_kernel<8, 1><<<grid, 256, 0, S(stream)>>>(logits, ld, bias, bias_noise, sigma, targets, vocab, rows_per_member, partial);
    else
        ce_population_kernel<<<grid, 256, 0, S(stream)>>>(logits, ld, bias, bias_noise, sigma, targets, vocab, rows_per_member, partial);
    int rc = check_launch("ce_population_kernel");
    if (rc) return rc;
    ce_finalize_kernel<<<(members + 127) / 128, 128, 0, S(stream)>>>(partial, members, rows_per_member, loss_mean);
    return check_launch("ce_finalize_kernel");
}

int bnf4_fill_ternary_noise(int8_t* out, size_t n, uint64_t seed, int use_clt, int clt_k, void* stream) {
    if (n == 0) return BNF4_OK;
    if (!out) return set_error(BNF4_ERR_INVALID, "fill_ternary_noise: null pointer");
    fill_noise_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, S(stream)>>>(out, n, seed, use_clt, clt_k);
    return check_launch("fill_noise_kernel");
}

int bnf4_fill_ternary_noise_batched(const bnf4_noise_desc* descs, int num_desc, int max_blocks, int use_clt, int clt_k, void* stream) {
    if (num_desc <= 0 || max_blocks <= 0) return BNF4_OK;
    if (!descs) return set_error(BNF4_ERR_INVALID, "fill_ternary_noise_batched: null pointer");
    fill_noise_batched_kernel<<<dim3(max_blocks, num_desc), 256, 0, S(stream)>>>(descs, num_desc, use_clt, clt_k);
    return check_launch("fill_noise_batched_kernel");
}

int bnf4_fill_float_noise(float* out, int n, uint64_t seed, int use_clt, int clt_k, void* stream) {
    if (n <= 0) return BNF4_OK;
    fill_float_noise_kernel<<<(n + 255) / 256, 256, 0, S(stream)>>>(out, n, seed, use_clt, clt_k);
    return check_launch("fill_float_noise_kernel");
}

int bnf4_init_shadow_from_weights(const int8_t* w, float* shadow, int n, void* stream) {
    if (n <= 0) return BNF4_OK;
    init_shadow_kernel<<<(n + 255) / 256, 256, 0, S(stream)>>>(w, shadow, n);
    return check_launch("init_shadow_kernel");
}

int bnf4_fill_pair_seeds(uint64_t base_seed, uint64_t epoch, int pairs, uint64_t* out, void* stream) {
    if (pairs <= 0) return BNF4_OK;
    pair_seeds_kernel<<<(pairs + 255) / 256, 256, 0, S(stream)>>>(base_seed, epoch, pairs, out);
    return check_launch("pair_seeds_kernel");
}

int bnf4_compute_z_sumsq(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs, int n, int use_clt,
                         int clt_k, float* Z, float* sumsq, void* stream) {
    if (n <= 0) return BNF4_OK;
    if (!pair_weights || !pair_seeds || !Z || !sumsq) return set_error(BNF4_ERR_INVALID, "compute_z_sumsq: null pointer");
    z_dense_kernel<<<(n + 255) / 256, 256, 256 * (sizeof(uint64_t) + sizeof(float)), S(stream)>>>(pair_weights, pair_seeds, salt, pairs, 0, n, use_clt, clt_k, Z);
    const int rc = check_launch("z_dense_kernel");
    if (rc) return rc;
    return sumsq_into(Z, n, sumsq, S(stream));
}

int bnf4_compute_z_lowrank(const float* pair_weights, const int8_t* A, long long A_pair_stride, const int8_t* B,
                           long long B_pair_stride, int pairs, int rows, int cols, int rank, float cscale, float* Z, void* stream) {
    if (rows <= 0 || cols <= 0) return BNF4_OK;
    if (!pair_weights || !A || !B || !Z) return set_error(BNF4_ERR_INVALID, "compute_z_lowrank: null pointer");
    const ZLowrankDesc d = {A, A_pair_stride, B, B_pair_stride, Z, rows, cols};
    return z_lowrank_launch(pair_weights, nullptr, &d, 0, pairs, rank, cscale, 0, 1, S(stream));
}

int bnf4_sumsq(const float* Z, int n, float* sumsq, void* stream) {
    if (n <= 0) return BNF4_OK;
    if (!Z || !sumsq) return set_error(BNF4_ERR_INVALID, "sumsq: null pointer");
    return sumsq_into(Z, n, sumsq, S(stream));
}

int bnf4_compute_z_sumsq_lowrank(const float* pair_weights, const int8_t* A, long long A_pair_stride, const int8_t* B,
                                 long long B_pair_stride, int pairs, int rows, int cols, int rank, float cscale, float* Z,
                                 float* sumsq, void* stream) {
    if (rows <= 0 || cols <= 0) return BNF4_OK;
    if (!sumsq) return set_error(BNF4_ERR_INVALID, "compute_z_sumsq_lowrank: null pointer");
    const int rc = bnf4_compute_z_lowrank(pair_weights, A, A_pair_stride, B, B_pair_stride, pairs, rows, cols, rank, cscale, Z, stream);
    if (rc) return rc;
    return sumsq_into(Z, rows * cols, sumsq, S(stream));
}

int bnf4_update_inv_rms(const float* sumsq, float* rms_ema, int use_adaptive, float adaptive_beta, float adaptive_eps, int n,
                        float* inv_rms, void* stream) {
    if (!sumsq || !rms_ema || !inv_rms) return set_error(BNF4_ERR_INVALID, "update_inv_rms: null pointer");
    inv_rms_kernel<<<1, 1, 0, S(stream)>>>(sumsq, rms_ema, use_adaptive, adaptive_beta, adaptive_eps, n, inv_rms);
    return check_launch("inv_rms_kernel");
}

int bnf4_update_shadow_ternary_device(int8_t* w, float* shadow, const float* Z, int n, const float* inv_rms, float lr,
                                      float thresh, void* stream) {
    if (n <= 0) return BNF4_OK;
    if (!inv_rms) return set_error(BNF4_ERR_INVALID, "update_shadow_ternary_device: null inv_rms");
    update_shadow_kernel<<<(n + 255) / 256, 256, 0, S(stream)>>>(w, shadow, Z, n, inv_rms, 0.0f, lr, thresh);
    return check_launch("update_shadow_kernel");
}

int bnf4_update_shadow_ternary(int8_t* w, float* shadow, const float* Z, int n, float inv_rms, float lr, float thresh, void* stream) {
    if (n <= 0) return BNF4_OK;
    update_shadow_kernel<<<(n + 255) / 256, 256, 0, S(stream)>>>(w, shadow, Z, n, nullptr, inv_rms, lr, thresh);
    return check_launch("update_shadow_kernel");
}

int bnf4_update_vector_device(float* v, const float* Z, int n, const float* inv_rms, float lr, float thresh, void* stream) {
    if (n <= 0) return BNF4_OK;
    update_vector_kernel<<<(n + 255) / 256, 256, 0, S(stream)>>>(v, Z, n, inv_rms, lr, thresh);
    return check_launch("update_vector_kernel");
}

int bnf4_add_scaled(float* out, const float* noise, int n, float scale, void* stream) {
    if (n <= 0) return BNF4_OK;
    add_scaled_kernel<<<(n + 255) / 256, 256, 0, S(stream)>>>(out, noise, n, scale);
    return check_launch("add_scaled_kernel");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------
// bnf4_compute_z_sumsq_static: the dense Z / sum-of-squares step with no allocation of any kind.
//
// bnf4_compute_z_sumsq keeps its block partials in a buffer the library obtains from cudaMalloc the first time
// it is needed on a device and replaces by a larger one when a longer vector arrives. Some hosts cannot accept
// that: a trainer whose own allocator has already reserved the whole of HBM (a library cudaMalloc then fails
// although the job has memory to spare), a serving loop in which the implicit device-wide synchronisation of
// cudaMalloc / cudaFree stalls every other stream, or a process that must keep a fixed, auditable device
// footprint. For them the partials live in the array below, which is part of the loaded module image: it exists
// as soon as the library is loaded on a device and is never resized or released.
//
// Capacity: kStaticPartials block partials of 256 elements each, i.e. n <= 67,108,864 (an 8192 x 8192 matrix);
// longer vectors are refused with BNF4_ERR_INVALID and nothing is launched.
// ---------------------------------------------------------------------------------------------------
static constexpr int kStaticPartials = 262144;  // 1 MiB of device memory per device
static constexpr long long kStaticMaxN = 256LL * kStaticPartials;
static __device__ __align__(256) float g_static_partials[kStaticPartials];

namespace {
std::mutex g_static_mu;
float* g_static_ptr[64] = {};  // device address of g_static_partials, per device ordinal; filled on first use

// Resolves the device address of the array for the CURRENT device (each device holds its own copy of a
// __device__ variable). Host code never uses the array's name as an address: only the pointer obtained here
// is handed to kernels.
int static_partials(float** out) {
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= 64) return set_error(BNF4_ERR_INVALID, "device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (g_static_ptr[dev] == nullptr) {
        float* ptr = nullptr;
        rc = check_cuda(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_partials), "cudaGetSymbolAddress(static partials)");
        if (rc) return rc;
        if (ptr == nullptr) return set_error(BNF4_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return BNF4_OK;
}
}  // namespace

extern "C" int bnf4_compute_z_sumsq_static(const float* pair_weights, const uint64_t* pair_seeds, uint64_t salt, int pairs, int n,
                                           int use_clt, int clt_k, float* Z, float* sumsq, void* stream) {
    if (n <= 0) return BNF4_OK;
    if (!pair_weights || !pair_seeds || !Z || !sumsq) return set_error(BNF4_ERR_INVALID, "compute_z_sumsq_static: null pointer");
    if (static_cast<long long>(n) > kStaticMaxN)
        return set_error(BNF4_ERR_INVALID, "compute_z_sumsq_static: n=%d exceeds the built-in scratch capacity of %lld elements; "
                         "use bnf4_compute_z_sumsq or split the vector", n, kStaticMaxN);
    float* partial = nullptr;
    int rc = static_partials(&partial);
    if (rc) return rc;
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    z_dense_kernel<<<(n + 255) / 256, 256, 256 * (sizeof(uint64_t) + sizeof(float)), st>>>(pair_weights, pair_seeds, salt, pairs, 0, n, use_clt, clt_k, Z);
    rc = check_launch("z_dense_kernel");
    if (rc) return rc;
    // Every partial the final kernel reads (indices 0 .. ceil(n/256)-1) is written by the block kernel of this same
    // call first, so stale contents left by an earlier call are never observed and nothing needs clearing.
    return sumsq_with_scratch(Z, n, partial, sumsq, st);
}
