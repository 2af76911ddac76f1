// Block-scaled FP4 (NVFP4: e2m1 data, one ue4m3 scale per 16 K-elements) GEMM for sm_100a.
//
//   D[m,n] = alpha * sum_kb sfa[m,kb] * sfb[n,kb] * sum_{k in kb} a[m,k] * b[n,k]  (+ beta * C[m,n])
//            (+ s_member * sum_r t[m][g*rank+r] * A_pair[n][r])                      rank-r perturbation
//
// replaces the reference's CUTLASS Sm120 kernel behind gemm_ternary_f_nvfp4 /
// gemm_ternary_f_nvfp4_gelu_i8 (reference: src/cuda_kernels.cu:3145-3310, 4342-4607) and fuses the
// rank-r term of gemm_lora_f_kernel (reference: src/cuda_kernels.cu:1271-1305) into the tile epilogue.
//
// Structure of one CTA (128 x 128 output tiles, 576 threads):
//   warp 0      producer: TMA tiles of A and B (128 rows x 128 bytes = 256 K-elements, 128B swizzle) and
//               bulk copies of the matching scale-factor atoms into a ring of shared-memory stages
//   warp 1      owns TMEM; per stage copies the scale atoms to TMEM (tcgen05.cp 32x128b.warpx4) and issues
//               tcgen05.mma.kind::mxf4nvf4.block_scale (M128 x N128 x K64) accumulating fp32 in TMEM
//   warps 2..17 epilogue: tcgen05.ld the accumulator (four warps per TMEM lane quadrant, 32 columns each), apply
//               alpha/beta/rank-r/GELU, and store (TMA store through swizzled staging, or direct)
// The kernel is persistent (one CTA per SM, tiles assigned round-robin): the producer runs up to four k-blocks
// ahead, and two TMEM accumulators let the MMAs of tile i+1 overlap the epilogue of tile i. Every mbarrier wait is bounded: on expiry the kernel records an error
// word, leaves its role loop, frees TMEM and returns.

#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"

namespace bnf4 {

namespace {

constexpr int BM = 128;             // tile rows
constexpr int BN = 128;             // tile columns
constexpr int BK = 256;             // K elements per stage (128 bytes of packed e2m1 per row)
constexpr int UMMA_K = 64;          // K elements per tcgen05.mma
constexpr int kStages = 4;
constexpr int kStageABytes = BM * 128;
constexpr int kStageBBytes = BN * 128;
constexpr int kStageSfBytes = 4 * 512;  // four 128-row x 64-K atoms
constexpr int kEpiWarps = 16;
constexpr int kEpiBufBytes = 32 * 32 * 4;  // one 32 x 32 fp32 box
constexpr int kThreads = 64 + kEpiWarps * 32;
constexpr int kTmemCols = 512;      // two 128-column accumulators + kStages * 32 scale columns, rounded to a power of two
constexpr int kAccCol = 0;
constexpr int kSfCol = 256;

constexpr int kSmemA = 0;
constexpr int kSmemB = kSmemA + kStages * kStageABytes;
constexpr int kSmemSfa = kSmemB + kStages * kStageBBytes;
constexpr int kSmemSfb = kSmemSfa + kStages * kStageSfBytes;
constexpr int kSmemEpi = kSmemSfb + kStages * kStageSfBytes;
constexpr int kSmemLora = kSmemEpi + kEpiWarps * kEpiBufBytes;
constexpr int kSmemBar = kSmemLora + kEpiWarps * 4 * 32 * 4;  // per epilogue warp: [4][32] floats of the pair's A factor
constexpr int kSmemTotal = kSmemBar + 128;
constexpr int kSmemAlloc = kSmemTotal + 1024;  // slack for manual 1024-byte alignment

constexpr long long kWaitCycles = 2000000000LL;  // ~1 s bound on every mbarrier wait

__device__ int g_gemm_error = 0;
}  // namespace
int g_gemm_allow_tma_store = 1;  // host toggle: 0 forces the direct-store epilogue
namespace {

// ------------------------------------------------------------------------------------------------
// PTX wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One attempt: the thread may be suspended by the hardware for up to ~20 us and is woken as soon as the phase completes,
// so a waiting role issues a handful of instructions per attempt instead of spinning through the issue slots the
// epilogue warps need.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(20000u)
        : "memory");
    return ok != 0;
}
// Bounded wait. Returns false (and records `code`) if the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > kWaitCycles) {
            atomicCAS(&g_gemm_error, 0, code);
            return false;
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_cp_sf(uint32_t taddr, uint64_t sdesc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void tc_mma_nvf4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t tsfa,
                                            uint32_t tsfb, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(tsfa), "r"(tsfb)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
// prmt.b32 in its default mode: a selector nibble with bit 3 set replicates the sign of the selected byte
__device__ __forceinline__ uint32_t prmt_b32(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
    return d;
}
// Four bytes of the int8 residual stream updated with four accumulators: clip8(old + rint(v * add_scale)). rint is the low 16
// bits of the biased float (the product is clamped first so that the field cannot wrap), added to the sign-extended old
// bytes and clipped with packed 16-bit integer operations, two elements per instruction.
__device__ __forceinline__ uint32_t resid_add_word(uint32_t old4, float v0, float v1, float v2, float v3, float add_scale) {
    const uint32_t t0 = __float_as_uint(fminf(fmaxf(__fmul_rn(v0, add_scale), -512.0f), 512.0f) + kRoundBias);
    const uint32_t t1 = __float_as_uint(fminf(fmaxf(__fmul_rn(v1, add_scale), -512.0f), 512.0f) + kRoundBias);
    const uint32_t t2 = __float_as_uint(fminf(fmaxf(__fmul_rn(v2, add_scale), -512.0f), 512.0f) + kRoundBias);
    const uint32_t t3 = __float_as_uint(fminf(fmaxf(__fmul_rn(v3, add_scale), -512.0f), 512.0f) + kRoundBias);
    const uint32_t r01 = __byte_perm(t0, t1, 0x5410), r23 = __byte_perm(t2, t3, 0x5410);
    const uint32_t o01 = prmt_b32(old4, 0u, 0x9180u), o23 = prmt_b32(old4, 0u, 0xB3A2u);
    const uint32_t s01 = __vmins2(__viaddmax_s16x2(r01, o01, 0xff81ff81u), 0x007f007fu);
    const uint32_t s23 = __vmins2(__viaddmax_s16x2(r23, o23, 0xff81ff81u), 0x007f007fu);
    return __byte_perm(s01, s23, 0x6420);
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (sm_100 format): start address >> 4 in bits [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), version 1 in [46,48), layout type in [61,64).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fffu) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fffu) << 32;
    d |= 1ull << 46;
    d |= static_cast<uint64_t>(layout) << 61;
    return d;
}
constexpr uint32_t kLayoutNone = 0, kLayoutSw128 = 2;

// Instruction descriptor of kind::mxf4nvf4 (block-scaled): a/b format e2m1 (=1) at bits 7 and 10,
// K-major A and B, N>>3 at bit 17, ue4m3 scales (bit 23 = 0), M>>4 at bit 24, scale ids 0, dense K = 64.
constexpr uint32_t kIdesc = (1u << 7) | (1u << 10) | (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);

struct KernelArgs {
    GemmParams p;
    int use_tma_store;
    int k_atoms;  // scale atoms along K
    uint32_t group_magic;  // ceil(2^32 / group_cols) (0 when group_cols == 0)
    const uint8_t* lut;  // table of the block quantiser (EPI_GELU_FP4)
    int total_tiles;
    int n_tiles;  // tiles along N; blockIdx.x = m_tile * n_tiles + n_tile (N fastest: CTAs that share A rows run together)
};

// One lane of a converged warp (the same one every time in practice). The role loops below run in all 32 lanes with
// warp-uniform control flow and values, and only the issuing instructions sit under this predicate: addresses, descriptors and
// counters then qualify for the uniform datapath instead of being moved there instruction by instruction from a divergent lane.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Persistent kernel: one CTA per SM walks the tile list (tile = m_tile * n_tiles + n_tile, N fastest so that
// CTAs working at the same time share rows of A through L2). Three roles run concurrently on different tiles:
// the producer prefetches operands up to kStages k-blocks ahead, the MMA warp fills one of two TMEM
// accumulators while the sixteen epilogue warps drain the other one.
// RK: 4 = the instance for rank-4 perturbation terms (its epilogue applies the four factors with packed multiply-adds);
// 1 = the instance for the batched driver's common case (rank 1, no C operand, every 128-row tile inside one member), which carries
// none of the general paths; 0 = everything else.
template <int EPI, int RK>
__global__ void __launch_bounds__(kThreads, 1) gemm_nvfp4_kernel(const __grid_constant__ CUtensorMap map_a,
                                                                 const __grid_constant__ CUtensorMap map_b,
                                                                 const __grid_constant__ CUtensorMap map_d,
                                                                 const KernelArgs args) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const GemmParams& p = args.p;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int num_ks = (p.k + BK - 1) / BK;
    const int total_tiles = args.total_tiles;

    const uint32_t bar_full = smem_base + kSmemBar;               // kStages x 8 bytes
    const uint32_t bar_empty = bar_full + 8 * kStages;            // kStages x 8 bytes
    const uint32_t bar_acc_full = bar_empty + 8 * kStages;        // 2 x 8 bytes
    const uint32_t bar_acc_empty = bar_acc_full + 16;             // 2 x 8 bytes
    const uint32_t tmem_slot = bar_acc_empty + 16;                // 4 bytes
    volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + kSmemBar + 16 * kStages + 32);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, 1);
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, kEpiWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot_gen;

    if (warp == 0) {
        // ------------------------------ producer ------------------------------
        {
            // running indices instead of divisions, addresses advanced by constants
            int kc = 0;  // k-block counter across tiles
            int s = 0;
            uint32_t empty_parity = 1;  // parity of the phase that precedes the first completion: the first pass does not wait
            bool ok = true;
            const int step_n = static_cast<int>(gridDim.x % static_cast<unsigned>(args.n_tiles)), step_m = static_cast<int>(gridDim.x / static_cast<unsigned>(args.n_tiles));
            int m_tile = static_cast<int>(blockIdx.x / static_cast<unsigned>(args.n_tiles)) - step_m;
            int n_tile = static_cast<int>(blockIdx.x % static_cast<unsigned>(args.n_tiles)) - step_n;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                n_tile += step_n;
                m_tile += step_m;
                if (n_tile >= args.n_tiles) { n_tile -= args.n_tiles; ++m_tile; }
                const uint8_t* sfa_src = static_cast<const uint8_t*>(p.sfa) + static_cast<size_t>(m_tile) * args.k_atoms * 512;
                const uint8_t* sfb_src = static_cast<const uint8_t*>(p.sfb) + static_cast<size_t>(n_tile) * args.k_atoms * 512;
                const int my = m_tile * BM, ny = n_tile * BN;
                int atoms_left = args.k_atoms;
                for (int ks = 0; ks < num_ks; ++ks, ++kc) {
                    if (kc >= kStages) {
                        ok = __all_sync(0xffffffffu, mbar_wait(bar_empty + 8 * s, empty_parity, 1));
                        if (!ok) break;
                    }
                    const uint32_t sf_bytes_stage = static_cast<uint32_t>(min(4, atoms_left)) * 512u;
                    atoms_left -= 4;
                    const uint32_t bar = bar_full + 8 * s;
                    if (elect_one()) {
                        mbar_expect_tx(bar, kStageABytes + kStageBBytes + 2 * sf_bytes_stage);
                        tma_load_2d(smem_base + kSmemA + s * kStageABytes, &map_a, ks * 128, my, bar);
                        tma_load_2d(smem_base + kSmemB + s * kStageBBytes, &map_b, ks * 128, ny, bar);
                        bulk_load_1d(smem_base + kSmemSfa + s * kStageSfBytes, sfa_src, sf_bytes_stage, bar);
                        bulk_load_1d(smem_base + kSmemSfb + s * kStageSfBytes, sfb_src, sf_bytes_stage, bar);
                    }
                    __syncwarp();
                    sfa_src += 2048;
                    sfb_src += 2048;
                    if (++s == kStages) { s = 0; empty_parity ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        {
            // The issue rate of this role bounds the mainloop (it shares an issue port with four busy epilogue warps), so the loop
            // is kept lean: descriptors are a stage-0 constant plus a stage / K-step increment of the 14-bit start-address field
            // (bytes >> 4), and the four K-steps of a full stage are unrolled.
            const uint64_t adesc0 = smem_desc(smem_base + kSmemA, 16, 1024, kLayoutSw128);
            const uint64_t bdesc0 = smem_desc(smem_base + kSmemB, 16, 1024, kLayoutSw128);
            const uint64_t sfadesc0 = smem_desc(smem_base + kSmemSfa, 0, 128, kLayoutNone);
            const uint64_t sfbdesc0 = smem_desc(smem_base + kSmemSfb, 0, 128, kLayoutNone);
            int kc = 0, it = 0;
            int s = 0;
            uint32_t full_parity = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
                const int buf = it & 1;
                if (it >= 2) {  // the epilogue must have drained this accumulator (tile it-2)
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_acc_empty + 8 * buf, ((it >> 1) - 1) & 1, 4));
                    if (!ok) break;
                    tc_fence_after();
                }
                const uint32_t acc_col = tmem_base + kAccCol + buf * BN;
                for (int ks = 0; ks < num_ks; ++ks, ++kc) {
                    ok = __all_sync(0xffffffffu, mbar_wait(bar_full + 8 * s, full_parity, 2));
                    if (!ok) break;
                    tc_fence_after();
                    const int nk = min(4, (p.k - ks * BK) / UMMA_K);
                    const uint32_t t_sfa = tmem_base + kSfCol + s * 32;
                    const uint32_t t_sfb = t_sfa + 16;
                    const uint64_t sfa_d = sfadesc0 + static_cast<uint64_t>(s * (kStageSfBytes >> 4));
                    const uint64_t sfb_d = sfbdesc0 + static_cast<uint64_t>(s * (kStageSfBytes >> 4));
                    const uint64_t a_d = adesc0 + static_cast<uint64_t>(s * (kStageABytes >> 4));
                    const uint64_t b_d = bdesc0 + static_cast<uint64_t>(s * (kStageBBytes >> 4));
                    if (elect_one()) {
                        if (nk == 4) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                tc_cp_sf(t_sfa + 4 * j, sfa_d + static_cast<uint64_t>(j * (512 >> 4)));
                                tc_cp_sf(t_sfb + 4 * j, sfb_d + static_cast<uint64_t>(j * (512 >> 4)));
                            }
                            tc_mma_nvf4(acc_col, a_d, b_d, kIdesc, t_sfa, t_sfb, ks > 0 ? 1u : 0u);
#pragma unroll
                            for (int j = 1; j < 4; ++j)
                                tc_mma_nvf4(acc_col, a_d + static_cast<uint64_t>(j * (32 >> 4)), b_d + static_cast<uint64_t>(j * (32 >> 4)), kIdesc,
                                            t_sfa + 4 * j, t_sfb + 4 * j, 1u);
                        } else {
                            for (int j = 0; j < nk; ++j) {
                                tc_cp_sf(t_sfa + 4 * j, sfa_d + static_cast<uint64_t>(j * (512 >> 4)));
                                tc_cp_sf(t_sfb + 4 * j, sfb_d + static_cast<uint64_t>(j * (512 >> 4)));
                            }
                            for (int j = 0; j < nk; ++j)
                                tc_mma_nvf4(acc_col, a_d + static_cast<uint64_t>(j * (32 >> 4)), b_d + static_cast<uint64_t>(j * (32 >> 4)), kIdesc,
                                            t_sfa + 4 * j, t_sfb + 4 * j, (ks > 0 || j > 0) ? 1u : 0u);
                        }
                        tc_commit(bar_empty + 8 * s);  // frees this smem stage once the MMAs above have read it
                        if (ks == num_ks - 1) tc_commit(bar_acc_full + 8 * buf);  // accumulator of this tile complete
                    }
                    __syncwarp();
                    if (++s == kStages) { s = 0; full_parity ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------ epilogue: 16 warps, four per TMEM lane quadrant, 32 columns each ------------------------------
        const int ew = warp - 2;   // 0..15
        const int q = warp & 3;    // TMEM lane quadrant this warp may access
        const int c = ew >> 2;     // 32-column chunk of the tile handled by this warp
        const uint32_t epi_buf = smem_base + kSmemEpi + ew * kEpiBufBytes;
        uint8_t* epi_gen = smem_gen + kSmemEpi + ew * kEpiBufBytes;
        bool ok = true;
        int it = 0;
        int stage_half = 0;  // EPI_F16: which half of the staging buffer the next store uses
        if constexpr (EPI == EPI_GELU_FP4) {
            // The block quantiser's table ({1 / scale, scale byte} per amax, 1 KB) lives in the staging area the fp32 epilogue would use.
            if (ew * 32 + lane < 128)
                reinterpret_cast<uint2*>(smem_gen + kSmemEpi)[ew * 32 + lane] =
                    __ldg(reinterpret_cast<const uint2*>(args.lut + kQuantBlockTabOffset) + ew * 32 + lane);
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiWarps * 32) : "memory");
        }
        // Perturbation context of one tile: this thread's row (projections t, sign, pair) and, when all rows of the tile
        // belong to one pair (always true when rows_per_member is a multiple of 128), this thread's element of the
        // pair's A factor for the tile's columns. It is fetched one tile ahead so that the global-load latency hides
        // behind the previous tile's epilogue.
        struct LoraCtx {
            int pair;
            float lsign;
            int tr[4];    // raw integers: converted to float only when the tile is processed, so that nothing waits
            int aval[4];  // on these loads earlier;  aval[r] = A[pair][col0 + lane][r]
            bool a_staged;
        };
        const int row_in_tile = q * 32 + lane;
        // Tile coordinates advance by additions (tiles are walked in steps of gridDim.x): no division per tile.
        const int step_n = static_cast<int>(gridDim.x % static_cast<unsigned>(args.n_tiles)), step_m = static_cast<int>(gridDim.x / static_cast<unsigned>(args.n_tiles));
        struct TileIdx { int m_tile, n_tile; };
        auto advance = [&](TileIdx& t) {
            t.n_tile += step_n;
            t.m_tile += step_m;
            if (t.n_tile >= args.n_tiles) { t.n_tile -= args.n_tiles; ++t.m_tile; }
        };
        // Members are visited in ascending order, so when tiles never straddle members (rows_per_member a multiple of the
        // tile height) the member of the next tile is tracked with comparisons instead of a division per row.
        const bool tile_uniform_member = p.rows_per_member > 0 && (p.rows_per_member % BM) == 0;
        int trk_member = 0;
        long long trk_end = p.rows_per_member;  // first row of member trk_member + 1
        const uint32_t group_magic = args.group_magic;  // ceil(2^32 / group_cols): exact quotients for columns below 65536
        auto fetch_ctx = [&](const TileIdx& t, bool valid, LoraCtx& cx) {
            cx.pair = 0;
            cx.lsign = 0.0f;
            cx.tr[0] = cx.tr[1] = cx.tr[2] = cx.tr[3] = 0;
            cx.aval[0] = cx.aval[1] = cx.aval[2] = cx.aval[3] = 0;
            cx.a_staged = false;
            if (p.rank <= 0 || !valid) return;
            const int m0_ = t.m_tile * BM, n0_ = t.n_tile * BN;
            const long long row_ = static_cast<long long>(m0_) + row_in_tile;
            const int col0_ = n0_ + c * 32;
            int pair_first, pair_last;
            if (tile_uniform_member) {
                while (m0_ >= trk_end) { ++trk_member; trk_end += p.rows_per_member; }
                pair_first = pair_last = trk_member >> 1;
                if (row_ < p.m) {
                    cx.pair = pair_first;
                    cx.lsign = (trk_member & 1) ? -p.lora_scale : p.lora_scale;
                }
            } else {
                // rows fit 31 bits (p.m is an int): 32-bit divisions
                const unsigned rpm = static_cast<unsigned>(p.rows_per_member);
                if (row_ < p.m) {
                    const int member = p.rows_per_member > 0 ? static_cast<int>(static_cast<unsigned>(row_) / rpm) : 0;
                    cx.pair = member >> 1;
                    cx.lsign = (member & 1) ? -p.lora_scale : p.lora_scale;
                }
                const unsigned last_row = static_cast<unsigned>(min(static_cast<long long>(p.m), static_cast<long long>(m0_) + BM) - 1);
                pair_first = p.rows_per_member > 0 ? static_cast<int>(static_cast<unsigned>(m0_) / rpm) >> 1 : 0;
                pair_last = p.rows_per_member > 0 ? static_cast<int>(last_row / rpm) >> 1 : 0;
            }
            if (row_ < p.m && col0_ < p.n) {
                const int g = p.group_cols > 0 ? static_cast<int>(__umulhi(static_cast<uint32_t>(col0_), group_magic)) : 0;
                const int* tp = p.lora_t + static_cast<size_t>(row_) * p.t_stride + g * p.rank;
                cx.tr[0] = __ldg(tp);
                if (p.rank > 1) {
                    cx.tr[1] = __ldg(tp + 1);
                    if (p.rank > 2) cx.tr[2] = __ldg(tp + 2);
                    if (p.rank > 3) cx.tr[3] = __ldg(tp + 3);
                }
            }
            cx.a_staged = (pair_first == pair_last);
            const int n = col0_ + lane;
            if (cx.a_staged && n < p.n) {
                const int8_t* Ag = p.lora_A + static_cast<size_t>(pair_first) * p.lora_A_pair_stride + static_cast<size_t>(n) * p.rank;
                cx.aval[0] = __ldg(Ag);
                if (p.rank > 1) {
                    cx.aval[1] = __ldg(Ag + 1);
                    if (p.rank > 2) cx.aval[2] = __ldg(Ag + 2);
                    if (p.rank > 3) cx.aval[3] = __ldg(Ag + 3);
                }
            }
        };
        // The common case (rank 1, tiles inside one member) with as few instructions as possible: this phase sits on the serial
        // path of every tile.
        constexpr bool R4 = RK == 4, R1 = RK == 1;
        const bool fast_ctx = R1 || (p.rank == 1 && tile_uniform_member);
        const int* t_row = p.rank > 0 ? p.lora_t + static_cast<size_t>(row_in_tile) * p.t_stride : nullptr;
        auto fetch_fast = [&](const TileIdx& t, bool valid, LoraCtx& cx) {
            cx.pair = 0;
            cx.lsign = 0.0f;
            cx.tr[0] = 0;
            cx.aval[0] = 0;
            cx.a_staged = true;
            if (!valid) return;
            const int m0_ = t.m_tile * BM, col0_ = t.n_tile * BN + c * 32;
            while (m0_ >= trk_end) { ++trk_member; trk_end += p.rows_per_member; }
            cx.pair = trk_member >> 1;
            if ((R1 || m0_ + row_in_tile < p.m) && col0_ < p.n) {
                const int g = p.group_cols > 0 ? static_cast<int>(__umulhi(static_cast<uint32_t>(col0_), group_magic)) : 0;
                cx.tr[0] = __ldg(t_row + static_cast<size_t>(m0_) * p.t_stride + g);
                cx.lsign = (trk_member & 1) ? -p.lora_scale : p.lora_scale;
            }
            if (col0_ + lane < p.n) cx.aval[0] = __ldg(p.lora_A + static_cast<size_t>(cx.pair) * p.lora_A_pair_stride + col0_ + lane);
        };
        TileIdx cur_t{static_cast<int>(blockIdx.x / static_cast<unsigned>(args.n_tiles)), static_cast<int>(blockIdx.x % static_cast<unsigned>(args.n_tiles))};
        TileIdx nxt_t = cur_t;
        // EPI_ADD_I8 through TMA: this warp's 32 x 32-byte box of the residual stream is loaded one tile ahead into one of
        // three 1 KB buffers (each with its own mbarrier), updated in place and stored from there. A lane-per-row access to
        // global memory touches 32 lines per instruction and kept the load/store unit busy for a third of the tile period.
        const bool res_tma = EPI == EPI_ADD_I8 && args.use_tma_store != 0;
        const uint32_t rbar = epi_buf + 3072;
        int rb_cur = 0, rb_last = 2;
        uint32_t r_par = 0;  // bit b: parity of the phase to wait for on buffer b
        bool have_cur = false, have_nxt = false;
        auto issue_res_load = [&](const TileIdx& t, bool valid) {
            const int col0_ = t.n_tile * BN + c * 32;
            have_nxt = valid && col0_ < p.n;
            if (!have_nxt) return;
            rb_last = rb_last == 2 ? 0 : rb_last + 1;
            if (lane == 0) {
                bulk_wait_read<1>();  // the store that last read this buffer (three tiles back) has left shared memory
                mbar_expect_tx(rbar + 8 * rb_last, 1024);
                tma_load_2d(epi_buf + rb_last * 1024, &map_d, col0_, t.m_tile * BM + q * 32, rbar + 8 * rb_last);
            }
        };
        if constexpr (EPI == EPI_ADD_I8) {
            if (res_tma) {
                if (lane == 0) {
                    mbar_init(rbar, 1);
                    mbar_init(rbar + 8, 1);
                    mbar_init(rbar + 16, 1);
                    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
                    fence_async_smem();
                }
                __syncwarp();
                issue_res_load(cur_t, static_cast<int>(blockIdx.x) < total_tiles);
            }
        }
        LoraCtx nxt;
        nxt.tr[1] = nxt.tr[2] = nxt.tr[3] = 0;
        nxt.aval[1] = nxt.aval[2] = nxt.aval[3] = 0;
        if (R1 || fast_ctx) fetch_fast(cur_t, static_cast<int>(blockIdx.x) < total_tiles, nxt);
        else fetch_ctx(cur_t, static_cast<int>(blockIdx.x) < total_tiles, nxt);
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++it) {
            const int buf = it & 1;
            cur_t = nxt_t;
            advance(nxt_t);
            const int m0 = cur_t.m_tile * BM, n0 = cur_t.n_tile * BN;
            const long long row = static_cast<long long>(m0) + row_in_tile;
            const bool row_ok = R1 || row < p.m;  // (the rank-1 instance runs with m a multiple of the tile height)
            const int col0 = n0 + c * 32;
            const bool chunk_ok = col0 < p.n;  // warp-uniform

            const int pair = nxt.pair;
            const float lsign = nxt.lsign;
            float tr[4] = {static_cast<float>(nxt.tr[0]), 0.0f, 0.0f, 0.0f};
            const bool a_staged = nxt.a_staged;
            float* loraA_sh = reinterpret_cast<float*>(smem_gen + kSmemLora) + ew * 4 * 32;  // this warp's [4][32]
            if (R1 || fast_ctx) {
                __syncwarp();  // the previous tile's reads are done
                loraA_sh[lane] = static_cast<float>(nxt.aval[0]);
                __syncwarp();
                fetch_fast(nxt_t, tile + static_cast<int>(gridDim.x) < total_tiles, nxt);
            } else if (p.rank > 0) {
                tr[1] = static_cast<float>(nxt.tr[1]);
                tr[2] = static_cast<float>(nxt.tr[2]);
                tr[3] = static_cast<float>(nxt.tr[3]);
                __syncwarp();  // the previous tile's reads are done
                if (a_staged) {
#pragma unroll
                    for (int r = 0; r < 4; ++r)
                        if (r < p.rank) loraA_sh[r * 32 + lane] = static_cast<float>(nxt.aval[r]);
                }
                __syncwarp();
                fetch_ctx(nxt_t, tile + static_cast<int>(gridDim.x) < total_tiles, nxt);
            }

            // EPI_ADD_I8: this thread's 32 bytes of the residual stream, requested before the wait for the accumulator
            int4 res0 = make_int4(0, 0, 0, 0), res1 = make_int4(0, 0, 0, 0);
            bool res_vec = false;
            if constexpr (EPI == EPI_ADD_I8) {
                if (res_tma) {
                    have_cur = have_nxt;
                    rb_cur = rb_last;
                    issue_res_load(nxt_t, tile + static_cast<int>(gridDim.x) < total_tiles);
                } else if (row_ok && chunk_ok) {
                    const int8_t* xr = p.resid + static_cast<size_t>(row) * p.ld_resid + col0;
                    res_vec = ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) && (col0 + 32 <= p.n);
                    if (res_vec) {
                        res0 = *reinterpret_cast<const int4*>(xr);
                        res1 = *reinterpret_cast<const int4*>(xr + 16);
                    }
                }
            }

            ok = mbar_wait(bar_acc_full + 8 * buf, (it >> 1) & 1, 3);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();

            uint32_t acc[32];
            tmem_ld32(tmem_base + kAccCol + buf * BN + (static_cast<uint32_t>(q * 32) << 16) + c * 32, acc);
            tmem_ld_wait();
            // this warp no longer needs the accumulator: hand it back to the MMA warp
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
            if (!chunk_ok) continue;

            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j += 2) {  // packed fp32 pairs: each half rounds like the scalar instruction
                const float2 t2 = __fmul2_rn(make_float2(p.alpha, p.alpha), make_float2(__uint_as_float(acc[j]), __uint_as_float(acc[j + 1])));
                v[j] = t2.x;
                v[j + 1] = t2.y;
            }
            if (!R1 && p.beta != 0.0f && row_ok) {
                const float* crow = p.c + static_cast<size_t>(row) * p.ldc + col0;
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.n) v[j] = fmaf(p.beta, crow[j], v[j]);
            }
            if ((R1 || p.rank > 0) && row_ok) {
                // sum_r t[r]*A[n][r] is an integer below 2^24: float products and sums are exact
                if constexpr (R4) {
                    if (a_staged) {
                        const float2 ls2 = make_float2(lsign, lsign);
                        const float2 t0 = make_float2(tr[0], tr[0]), t1 = make_float2(tr[1], tr[1]), t2 = make_float2(tr[2], tr[2]), t3 = make_float2(tr[3], tr[3]);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 a0 = *reinterpret_cast<const float4*>(loraA_sh + 4 * j), a1 = *reinterpret_cast<const float4*>(loraA_sh + 32 + 4 * j);
                            const float4 a2 = *reinterpret_cast<const float4*>(loraA_sh + 64 + 4 * j), a3 = *reinterpret_cast<const float4*>(loraA_sh + 96 + 4 * j);
                            float2 lo = __fmul2_rn(t0, make_float2(a0.x, a0.y)), hi = __fmul2_rn(t0, make_float2(a0.z, a0.w));
                            lo = __ffma2_rn(t1, make_float2(a1.x, a1.y), lo); hi = __ffma2_rn(t1, make_float2(a1.z, a1.w), hi);
                            lo = __ffma2_rn(t2, make_float2(a2.x, a2.y), lo); hi = __ffma2_rn(t2, make_float2(a2.z, a2.w), hi);
                            lo = __ffma2_rn(t3, make_float2(a3.x, a3.y), lo); hi = __ffma2_rn(t3, make_float2(a3.z, a3.w), hi);
                            lo = __ffma2_rn(ls2, lo, make_float2(v[4 * j + 0], v[4 * j + 1]));
                            hi = __ffma2_rn(ls2, hi, make_float2(v[4 * j + 2], v[4 * j + 3]));
                            v[4 * j + 0] = lo.x; v[4 * j + 1] = lo.y; v[4 * j + 2] = hi.x; v[4 * j + 3] = hi.y;
                        }
                    } else {
                        const int8_t* Ap = p.lora_A + static_cast<size_t>(pair) * p.lora_A_pair_stride + static_cast<size_t>(col0) * 4;
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < p.n) {
                                float pert = 0.0f;
#pragma unroll
                                for (int r = 0; r < 4; ++r) pert = fmaf(tr[r], static_cast<float>(Ap[j * 4 + r]), pert);
                                v[j] = fmaf(lsign, pert, v[j]);
                            }
                        }
                    }
                } else if (R1 || (a_staged && p.rank == 1)) {
                    const float2 tr2 = make_float2(tr[0], tr[0]), ls2 = make_float2(lsign, lsign);
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 a4 = *reinterpret_cast<const float4*>(loraA_sh + 4 * j);
                        const float2 lo = __ffma2_rn(ls2, __fmul2_rn(tr2, make_float2(a4.x, a4.y)), make_float2(v[4 * j + 0], v[4 * j + 1]));
                        const float2 hi = __ffma2_rn(ls2, __fmul2_rn(tr2, make_float2(a4.z, a4.w)), make_float2(v[4 * j + 2], v[4 * j + 3]));
                        v[4 * j + 0] = lo.x; v[4 * j + 1] = lo.y; v[4 * j + 2] = hi.x; v[4 * j + 3] = hi.y;
                    }
                } else if (a_staged) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float4 pert = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                        for (int r = 0; r < p.rank; ++r) {
                            const float trr = r == 0 ? tr[0] : (r == 1 ? tr[1] : (r == 2 ? tr[2] : tr[3]));
                            const float4 a4 = *reinterpret_cast<const float4*>(loraA_sh + r * 32 + 4 * j);
                            pert.x = fmaf(trr, a4.x, pert.x);
                            pert.y = fmaf(trr, a4.y, pert.y);
                            pert.z = fmaf(trr, a4.z, pert.z);
                            pert.w = fmaf(trr, a4.w, pert.w);
                        }
                        v[4 * j + 0] = fmaf(lsign, pert.x, v[4 * j + 0]);
                        v[4 * j + 1] = fmaf(lsign, pert.y, v[4 * j + 1]);
                        v[4 * j + 2] = fmaf(lsign, pert.z, v[4 * j + 2]);
                        v[4 * j + 3] = fmaf(lsign, pert.w, v[4 * j + 3]);
                    }
                } else {
                    const int8_t* Ap = p.lora_A + static_cast<size_t>(pair) * p.lora_A_pair_stride + static_cast<size_t>(col0) * p.rank;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (col0 + j < p.n) {
                            float pert = 0.0f;
#pragma unroll
                            for (int r = 0; r < 4; ++r)
                                if (r < p.rank) pert = fmaf(tr[r], static_cast<float>(Ap[static_cast<size_t>(j) * p.rank + r]), pert);
                            v[j] = fmaf(lsign, pert, v[j]);
                        }
                    }
                }
            }

            if constexpr (EPI == EPI_F32) {
                if (args.use_tma_store) {
                    // stage the 32x32 box in 128B-swizzled shared memory, then one TMA store (clips at M and N)
                    if (it > 0) {
                        if (lane == 0) bulk_wait_read<0>();
                        __syncwarp();
                    }
                    float4* dst = reinterpret_cast<float4*>(epi_gen + lane * 128);
#pragma unroll
                    for (int j = 0; j < 8; ++j) dst[j ^ (lane & 7)] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&map_d, epi_buf, col0, m0 + q * 32);
                        bulk_commit();
                    }
                } else if (row_ok) {
                    float* drow = p.d + static_cast<size_t>(row) * p.ldd + col0;
                    const bool vec = ((reinterpret_cast<uintptr_t>(drow) & 15) == 0) && (col0 + 32 <= p.n);
                    if (vec) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(drow)[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.n) drow[j] = v[j];
                    }
                }
            } else if constexpr (EPI == EPI_F16) {
                if (col0 < p.n_f16) {
                    // 32 rows x 32 halves staged as 64-byte rows, then one TMA store (clips at M; n_f16 is a multiple of 32).
                    // Two staging halves alternate, so only the store before the previous one has to have left shared memory.
                    if (lane == 0) bulk_wait_read<1>();
                    __syncwarp();
                    uint4* dst = reinterpret_cast<uint4*>(epi_gen + stage_half * 2048 + lane * 64);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int jj = j;
                        const __half2 h0 = __floats2half2_rn(v[8 * jj], v[8 * jj + 1]), h1 = __floats2half2_rn(v[8 * jj + 2], v[8 * jj + 3]);
                        const __half2 h2 = __floats2half2_rn(v[8 * jj + 4], v[8 * jj + 5]), h3 = __floats2half2_rn(v[8 * jj + 6], v[8 * jj + 7]);
                        dst[jj] = make_uint4(*reinterpret_cast<const uint32_t*>(&h0), *reinterpret_cast<const uint32_t*>(&h1),
                                             *reinterpret_cast<const uint32_t*>(&h2), *reinterpret_cast<const uint32_t*>(&h3));
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&map_d, epi_buf + stage_half * 2048, col0, m0 + q * 32);
                        bulk_commit();
                    }
                    stage_half ^= 1;
                } else if (R1) {  // (the rank-1 instance runs with at most one fp32 column behind the halves)
                    if (col0 == p.n_f16) p.d[static_cast<size_t>(row) * p.ldd] = v[0];
                } else if (row_ok) {
                    float* drow = p.d + static_cast<size_t>(row) * p.ldd + (col0 - p.n_f16);
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < p.n) drow[j] = v[j];
                }
            } else if constexpr (EPI == EPI_ADD_I8) {
                if (res_tma) {
                    if (have_cur) {
                        ok = __all_sync(0xffffffffu, mbar_wait(rbar + 8 * rb_cur, (r_par >> rb_cur) & 1u, 5));
                        if (!ok) break;
                        r_par ^= 1u << rb_cur;
                        int4* rrow = reinterpret_cast<int4*>(epi_gen + rb_cur * 1024 + lane * 32);
                        res0 = rrow[0];
                        res1 = rrow[1];
                        const uint32_t rw[8] = {static_cast<uint32_t>(res0.x), static_cast<uint32_t>(res0.y), static_cast<uint32_t>(res0.z), static_cast<uint32_t>(res0.w),
                                                static_cast<uint32_t>(res1.x), static_cast<uint32_t>(res1.y), static_cast<uint32_t>(res1.z), static_cast<uint32_t>(res1.w)};
                        uint32_t upd[8];
#pragma unroll
                        for (int g = 0; g < 8; ++g) upd[g] = resid_add_word(rw[g], v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3], p.add_scale);
                        rrow[0] = make_int4(static_cast<int>(upd[0]), static_cast<int>(upd[1]), static_cast<int>(upd[2]), static_cast<int>(upd[3]));
                        rrow[1] = make_int4(static_cast<int>(upd[4]), static_cast<int>(upd[5]), static_cast<int>(upd[6]), static_cast<int>(upd[7]));
                        fence_async_smem();
                        __syncwarp();
                        if (lane == 0) {  // clips at M and N
                            tma_store_2d(&map_d, epi_buf + rb_cur * 1024, col0, m0 + q * 32);
                            bulk_commit();
                        }
                    }
                } else if (row_ok) {
                    int8_t* xr = p.resid + static_cast<size_t>(row) * p.ld_resid + col0;
                    if (res_vec) {
                        const uint32_t rw[8] = {static_cast<uint32_t>(res0.x), static_cast<uint32_t>(res0.y), static_cast<uint32_t>(res0.z), static_cast<uint32_t>(res0.w),
                                                static_cast<uint32_t>(res1.x), static_cast<uint32_t>(res1.y), static_cast<uint32_t>(res1.z), static_cast<uint32_t>(res1.w)};
                        uint32_t upd[8];
#pragma unroll
                        for (int g = 0; g < 8; ++g) upd[g] = resid_add_word(rw[g], v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3], p.add_scale);
                        reinterpret_cast<int4*>(xr)[0] = make_int4(static_cast<int>(upd[0]), static_cast<int>(upd[1]), static_cast<int>(upd[2]), static_cast<int>(upd[3]));
                        reinterpret_cast<int4*>(xr)[1] = make_int4(static_cast<int>(upd[4]), static_cast<int>(upd[5]), static_cast<int>(upd[6]), static_cast<int>(upd[7]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            if (col0 + j < p.n) {
                                const float t = resid_add_biased(static_cast<float>(xr[j]), v[j], p.add_scale);
                                xr[j] = static_cast<int8_t>(__float_as_int(t) - kRoundBiasBits);
                            }
                        }
                    }
                }
            } else {
                // GELU -> int8 (reference: src/cuda_kernels.cu:3178-3194; tanh-form GELU, clip to +-127)
                if (!R1 && col0 + 32 > p.n) {  // (the rank-1 instance runs with n a multiple of 32)
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j >= p.n) v[j] = 0.0f;  // gelu(0) = 0
                }
                // One 16-element scale block at a time: its 16 values take the fast evaluation in one straight-line stretch (no
                // branch between groups, so the scheduler interleaves them); a group with a value too close to a rounding
                // boundary is flagged and redone with the tanhf form (about one group in a thousand). tb holds the rounded
                // values still biased by 1.5 * 2^23: the low byte of the bit pattern is the int8.
                const bool lower_clamp = !R1 && p.act_scale > 700.0f;  // gelu(x) >= -0.17 |x|: only a huge act_scale reaches -127 (those calls run the general instance)
                // entry address from the bit pattern of (amax + kRoundBias): (bits - kRoundBiasBits) * 8, folded into one constant
                const uint32_t tab_c = smem_base + kSmemEpi - (static_cast<uint32_t>(kRoundBiasBits) << 3);
                int w[8];
                uint32_t sfv[2] = {0u, 0u}, codes[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    float tb[16];
                    float am = 0.0f;  // max |value| of the block
                    uint32_t bad = 0;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int j = 16 * blk + 4 * g;
                        float worst = 0.0f;
                        float fc[4];  // the rounded integers as floats
                        gelu_q8_fast2(v[j], v[j + 1], p.act_scale, lower_clamp, worst, tb[4 * g], tb[4 * g + 1], fc[0], fc[1]);
                        gelu_q8_fast2(v[j + 2], v[j + 3], p.act_scale, lower_clamp, worst, tb[4 * g + 2], tb[4 * g + 3], fc[2], fc[3]);
                        bad |= worst < kGeluSafe ? 0u : (1u << g);
                        am = fmax3(fmax3(am, fabsf(fc[0]), fabsf(fc[1])), fabsf(fc[2]), fabsf(fc[3]));
                    }
                    if (bad != 0) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            if ((bad >> g) & 1u) {
                                const int j = 16 * blk + 4 * g;
                                float tbx[4], fcx[4];
                                gelu_q8_exact4(v[j], v[j + 1], v[j + 2], v[j + 3], p.act_scale, tbx, fcx);
#pragma unroll
                                for (int e = 0; e < 4; ++e) tb[4 * g + e] = tbx[e];
                            }
                        }
                        am = 0.0f;
#pragma unroll
                        for (int e = 0; e < 16; ++e) am = fmaxf(am, fabsf(tb[e] - kRoundBias));
                    }
#pragma unroll
                    for (int g = 0; g < 4; ++g)
                        w[4 * blk + g] = static_cast<int>(__byte_perm(__byte_perm(__float_as_uint(tb[4 * g]), __float_as_uint(tb[4 * g + 1]), 0x0040),
                                                                      __byte_perm(__float_as_uint(tb[4 * g + 2]), __float_as_uint(tb[4 * g + 3]), 0x0040), 0x5410));
                    if constexpr (EPI == EPI_GELU_FP4) {
                        // {1 / scale, scale byte} of the block from the table; the codes from the conversion instruction
                        // applied to n / scale (e2m1x8_int)
                        uint32_t rbits, sbyte;
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(rbits), "=r"(sbyte) : "r"((__float_as_uint(am + kRoundBias) << 3) + tab_c));
                        sfv[blk] = sbyte;
                        codes[2 * blk] = e2m1x8_biased(tb, __uint_as_float(rbits));
                        codes[2 * blk + 1] = e2m1x8_biased(tb + 8, __uint_as_float(rbits));
                    }
                }
                if (!(R1 && EPI == EPI_GELU_FP4) && row_ok && p.d_i8 != nullptr) {  // (the rank-1 FP4 instance writes no int8 copy)
                    int8_t* drow = p.d_i8 + static_cast<size_t>(row) * p.ld_i8 + col0;
                    if (((reinterpret_cast<uintptr_t>(drow) & 15) == 0) && col0 + 32 <= p.n) {
                        reinterpret_cast<int4*>(drow)[0] = make_int4(w[0], w[1], w[2], w[3]);
                        reinterpret_cast<int4*>(drow)[1] = make_int4(w[4], w[5], w[6], w[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < p.n) drow[j] = static_cast<int8_t>((w[j >> 2] >> (8 * (j & 3))) & 0xff);
                    }
                }
                if constexpr (EPI == EPI_GELU_FP4) {
                    if (row_ok) {
                        const uint32_t s0 = sfv[0], s1 = sfv[1], lo0 = codes[0], hi0 = codes[1], lo1 = codes[2], hi1 = codes[3];
                        *reinterpret_cast<uint4*>(p.d_codes + (static_cast<size_t>(row) * p.n + col0) / 2) = make_uint4(lo0, hi0, lo1, hi1);
                        const int kb = col0 >> 4;
                        *reinterpret_cast<uint16_t*>(p.d_sf + sf_offset(static_cast<int>(row), kb, sf_k_atoms(p.n))) =
                            static_cast<uint16_t>(s0 | (s1 << 8));
                        if (R1 || p.next_nvec > 0) {  // (the rank-1 FP4 instance always feeds one projection)
                            const int8_t* tv = p.next_tvec + static_cast<size_t>(pair) * p.next_tvec_pair_stride + col0;
                            const int nv_ = R1 ? 1 : p.next_nvec;  // (the rank-1 instance runs with at most one projection)
                            for (int vv = 0; vv < nv_; ++vv) {
                                const int4* bv = reinterpret_cast<const int4*>(tv + static_cast<size_t>(vv) * p.n);
                                const int4 b0 = __ldg(bv), b1 = __ldg(bv + 1);
                                int a = 0;
                                a = __dp4a(w[0], b0.x, a); a = __dp4a(w[1], b0.y, a); a = __dp4a(w[2], b0.z, a); a = __dp4a(w[3], b0.w, a);
                                a = __dp4a(w[4], b1.x, a); a = __dp4a(w[5], b1.y, a); a = __dp4a(w[6], b1.z, a); a = __dp4a(w[7], b1.w, a);
                                atomicAdd(p.next_t + static_cast<size_t>(row) * p.next_nvec + vv, a);
                            }
                        }
                    }
                }
            }
        }
        if constexpr (EPI == EPI_F32 || EPI == EPI_F16 || EPI == EPI_ADD_I8) {
            if (args.use_tma_store) {
                if (lane == 0) bulk_wait_read<0>();
                __syncwarp();
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

int make_map_2d(CUtensorMap* map, CUtensorMapDataType dt, const void* base, uint64_t dim0, uint64_t dim1, uint64_t stride1_bytes,
                uint32_t box0, uint32_t box1, const char* what, CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
    EncodeTiledFn fn = get_encode_fn();
    if (fn == nullptr) return set_error(BNF4_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {dim0, dim1};
    const cuuint64_t strides[1] = {stride1_bytes};
    const cuuint32_t box[2] = {box0, box1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(BNF4_ERR_CUDA, "cuTensorMapEncodeTiled(%s) failed with %d", what, static_cast<int>(r));
    return BNF4_OK;
}

template <int EPI, int RK>
int launch_t(const CUtensorMap& ma, const CUtensorMap& mb, const CUtensorMap& md, const KernelArgs& args, dim3 grid,
             cudaStream_t stream) {
    // function attributes are per device: set once for each device this process uses
    static bool configured[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return check_cuda(cudaGetLastError(), "cudaGetDevice");
    if (dev < 0 || dev >= 64 || !configured[dev]) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_nvfp4_kernel<EPI, RK>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemAlloc);
        if (e != cudaSuccess) return check_cuda(e, "cudaFuncSetAttribute(gemm_nvfp4_kernel)");
        if (dev >= 0 && dev < 64) configured[dev] = true;
    }
    gemm_nvfp4_kernel<EPI, RK><<<grid, kThreads, kSmemAlloc, stream>>>(ma, mb, md, args);
    return check_launch("gemm_nvfp4_kernel");
}

}  // namespace

int gemm_nvfp4_launch(const GemmParams& p, cudaStream_t stream) {
    if (p.m <= 0 || p.n <= 0) return BNF4_OK;
    if (p.k <= 0 || (p.k % 64) != 0) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: k=%d must be a positive multiple of 64", p.k);
    if (!p.a || !p.b || !p.sfa || !p.sfb) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: null operand");
    if ((reinterpret_cast<uintptr_t>(p.a) & 15) || (reinterpret_cast<uintptr_t>(p.b) & 15) || (reinterpret_cast<uintptr_t>(p.sfa) & 15) ||
        (reinterpret_cast<uintptr_t>(p.sfb) & 15))
        return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: operands and scale factors must be 16-byte aligned");
    if (p.beta != 0.0f && p.c == nullptr) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: beta != 0 needs C");
    if (p.rank < 0 || p.rank > 4) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: rank=%d outside [0,4]", p.rank);
    if (p.rank > 0 && (!p.lora_t || !p.lora_A)) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: rank > 0 needs t and A");
    if (p.group_cols > 0 && (p.group_cols % 32) != 0) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: group_cols must be a multiple of 32");
    if (p.epilogue == EPI_F32 && !p.d) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: null D");
    if (p.epilogue == EPI_GELU_I8 && !p.d_i8) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: null int8 D");
    if (p.epilogue == EPI_ADD_I8 && (!p.resid || p.ld_resid < p.n)) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: the residual epilogue needs resid and ld_resid >= n");
    if (p.epilogue == EPI_F16) {
        if (!p.d_f16 || p.n_f16 <= 0 || (p.n_f16 % 32) != 0 || p.n_f16 > p.n) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: the fp16 epilogue needs d_f16 and n_f16 a multiple of 32 within n");
        if ((reinterpret_cast<uintptr_t>(p.d_f16) & 15) || (p.ld_f16 % 8) != 0 || p.ld_f16 < p.n_f16) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: fp16 D misaligned");
        if (p.n > p.n_f16 && (!p.d || p.ldd < p.n - p.n_f16)) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: the fp32 tail of the fp16 epilogue needs d and ldd >= n - n_f16");
    }
    if (p.epilogue == EPI_GELU_FP4) {
        if (!p.d_codes || !p.d_sf) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: null FP4 D");
        if ((p.n % 32) != 0) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: FP4 output needs n %% 32 == 0");
        if ((reinterpret_cast<uintptr_t>(p.d_codes) & 15) || (reinterpret_cast<uintptr_t>(p.d_sf) & 3))
            return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: FP4 output misaligned");
        if (p.next_nvec < 0 || p.next_nvec > 4) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: next_nvec outside [0,4]");
        if (p.next_nvec > 0 && ((reinterpret_cast<uintptr_t>(p.next_tvec) & 15) || (p.next_tvec_pair_stride & 15)))
            return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: next_tvec misaligned");
    }

    CUtensorMap ma, mb, md;
    int rc = make_map_2d(&ma, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.a, static_cast<uint64_t>(p.k) / 2, static_cast<uint64_t>(p.m),
                         static_cast<uint64_t>(p.k) / 2, 128, BM, "A");
    if (rc) return rc;
    rc = make_map_2d(&mb, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.b, static_cast<uint64_t>(p.k) / 2, static_cast<uint64_t>(p.n),
                     static_cast<uint64_t>(p.k) / 2, 128, BN, "B");
    if (rc) return rc;
    KernelArgs args;
    args.p = p;
    args.k_atoms = sf_k_atoms(p.k);
    args.group_magic = p.group_cols > 0 ? static_cast<uint32_t>(((1ull << 32) + static_cast<unsigned long long>(p.group_cols) - 1) / static_cast<unsigned long long>(p.group_cols)) : 0u;
    if (p.group_cols > 0 && p.n >= 65536) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: column groups need n < 65536");
    args.lut = nullptr;
    if (p.epilogue == EPI_GELU_FP4) {
        args.lut = get_quant_lut();
        if (args.lut == nullptr) return BNF4_ERR_CUDA;
    }
    args.use_tma_store = 0;
    if (p.epilogue == EPI_F32 && (reinterpret_cast<uintptr_t>(p.d) & 15) == 0 && (p.ldd % 4) == 0 && p.ldd >= p.n) {
        rc = make_map_2d(&md, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.d, static_cast<uint64_t>(p.n), static_cast<uint64_t>(p.m),
                         static_cast<uint64_t>(p.ldd) * 4, 32, 32, "D");
        if (rc) return rc;
        args.use_tma_store = g_gemm_allow_tma_store != 0;  // 0 direct stores, 1 TMA stores
    } else if (p.epilogue == EPI_F16) {
        // the half columns leave through a 32 x 32 box of halves (64-byte rows, unswizzled staging)
        rc = make_map_2d(&md, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, p.d_f16, static_cast<uint64_t>(p.n_f16), static_cast<uint64_t>(p.m),
                         static_cast<uint64_t>(p.ld_f16) * 2, 32, 32, "D (fp16)", CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        args.use_tma_store = 1;
    } else if (p.epilogue == EPI_ADD_I8 && (reinterpret_cast<uintptr_t>(p.resid) & 15) == 0 && (p.ld_resid % 16) == 0) {
        // the residual stream enters and leaves through 32-row x 32-byte boxes
        rc = make_map_2d(&md, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.resid, static_cast<uint64_t>(p.n), static_cast<uint64_t>(p.m),
                         static_cast<uint64_t>(p.ld_resid), 32, 32, "residual stream", CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc) return rc;
        args.use_tma_store = g_gemm_allow_tma_store != 0;
    } else {
        md = ma;  // unused
    }
    args.n_tiles = (p.n + BN - 1) / BN;
    const long long tiles = static_cast<long long>(args.n_tiles) * ((p.m + BM - 1) / BM);
    if (tiles > 0x7fffffffLL) return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: too many tiles");
    args.total_tiles = static_cast<int>(tiles);
    int dev = 0, sms = 0;
    rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    rc = check_cuda(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev), "cudaDeviceGetAttribute");
    if (rc) return rc;
    const dim3 grid(static_cast<unsigned>(std::min<long long>(tiles, sms)), 1, 1);
    const bool gelu = p.epilogue == EPI_GELU_FP4 || p.epilogue == EPI_GELU_I8;
    const bool gelu_plain = !gelu || (p.act_scale <= 700.0f && (p.n % 32) == 0 && (p.epilogue == EPI_GELU_FP4 ? (p.next_nvec == 1 && p.d_i8 == nullptr) : p.next_nvec <= 1));
    const int rk = p.rank == 4 ? 4 : ((p.rank == 1 && p.beta == 0.0f && p.rows_per_member > 0 && (p.rows_per_member % BM) == 0 && (p.m % BM) == 0 && gelu_plain && (p.epilogue != EPI_F16 || p.n - p.n_f16 <= 1)) ? 1 : 0);
    switch (p.epilogue) {
        case EPI_F32: return rk == 4 ? launch_t<EPI_F32, 4>(ma, mb, md, args, grid, stream) : (rk == 1 ? launch_t<EPI_F32, 1>(ma, mb, md, args, grid, stream) : launch_t<EPI_F32, 0>(ma, mb, md, args, grid, stream));
        case EPI_GELU_I8: return rk == 4 ? launch_t<EPI_GELU_I8, 4>(ma, mb, md, args, grid, stream) : (rk == 1 ? launch_t<EPI_GELU_I8, 1>(ma, mb, md, args, grid, stream) : launch_t<EPI_GELU_I8, 0>(ma, mb, md, args, grid, stream));
        case EPI_GELU_FP4: return rk == 4 ? launch_t<EPI_GELU_FP4, 4>(ma, mb, md, args, grid, stream) : (rk == 1 ? launch_t<EPI_GELU_FP4, 1>(ma, mb, md, args, grid, stream) : launch_t<EPI_GELU_FP4, 0>(ma, mb, md, args, grid, stream));
        case EPI_ADD_I8: return rk == 4 ? launch_t<EPI_ADD_I8, 4>(ma, mb, md, args, grid, stream) : (rk == 1 ? launch_t<EPI_ADD_I8, 1>(ma, mb, md, args, grid, stream) : launch_t<EPI_ADD_I8, 0>(ma, mb, md, args, grid, stream));
        case EPI_F16: return rk == 4 ? launch_t<EPI_F16, 4>(ma, mb, md, args, grid, stream) : (rk == 1 ? launch_t<EPI_F16, 1>(ma, mb, md, args, grid, stream) : launch_t<EPI_F16, 0>(ma, mb, md, args, grid, stream));
    }
    return set_error(BNF4_ERR_INVALID, "gemm_nvfp4: unknown epilogue %d", p.epilogue);
}

int gemm_nvfp4_device_error(cudaStream_t stream, int* out_code) {
    int rc = check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    if (rc) return rc;
    int code = 0;
    rc = check_cuda(cudaMemcpyFromSymbol(&code, g_gemm_error, sizeof(int)), "cudaMemcpyFromSymbol(g_gemm_error)");
    if (rc) return rc;
    if (code != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    }
    if (out_code) *out_code = code;
    if (code != 0) return set_error(BNF4_ERR_DEVICE, "gemm_nvfp4: a bounded wait expired in the kernel (role code %d)", code);
    return BNF4_OK;
}

}  // namespace bnf4
