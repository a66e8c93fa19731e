// Device helpers shared by the tcgen05 kernels: mbarrier, TMA, UMMA descriptors.
#pragma once
#include <cuda.h>

#include "conv_args.cuh"

namespace ogle {

namespace tc {

constexpr int kTileM = 128;
constexpr int kChunk = 32;              // reduction elements per pipeline stage (128 bytes)
constexpr int kABytes = kTileM * 128;   // one A tile
constexpr uint32_t kSpinLimit = 1u << 22;

constexpr int kMaxGatherK = 224;     // reduction indices of the gather form (k * k * C rounded up to 32); offsets fit 16 bits

struct TcArgs {
    int flat;                 // 1: rows are a flat range of pixels (pointwise / gemm)
    int tn, th, tw;           // output pixels per tile along n, h, w (tn*th*tw <= 128)
    int tiles_w, tiles_h;     // tile grid along w and h (n follows)
    int N, Ho, Wo;            // output extent (flat: rows = Wo)
    int stride, pad, dil, kernel;
    int chunks_per_tap, Cp32;
    int K, Kp, Ks, koff;      // output channels, padded to 4, row stride, first channel
    int BN, n_tiles;          // N tile and how many cover Kp
    int act;
    float lo, hi;
    float alpha, beta;
    int bias_mode;            // 0 none, 1 full matrix C[m][ldc], 2 per-column vector
    int ldc;
    int passes;               // 1 (TF32) or 3 (split mode: a TF32 pass + a BF16 pass of the cross terms)
    int stages;
    int tmem_cols;
    int n_acc;                // accumulator buffers in tensor memory (2 or 4)
    int total_tiles;          // m_tiles * n_tiles (persistent kernel)
    int epi_groups, xf_groups; // persistent kernel: warp groups per role (1 or 2)
    int epi_slabs;            // staging slabs (128 rows x 32 columns) per epilogue group (1 or 2)
    // Two outputs from one pass (sibling convolutions over the same input, filters stacked):
    // columns [0, K1) go to the first tensor, columns [split_col, K) to the second.
    // split_col is a multiple of 32 (0 = single output).
    int split_col, K1;
    // Split reduction: each tile is computed by split_k work items over consecutive ranges of
    // chunks_per_split reduction chunks; their partial tiles are combined by TMA reduce-add
    // stores into an output the host zeroed. Used (activation none only) when the tiles alone
    // would leave most SMs idle or a last round mostly empty. total_work = total_tiles * split_k.
    int split_k, chunks_per_split, total_work;
    // Split reduction through a workspace (ws_mode = 1; any number of ranges, any activation): work item
    // (tile, ks) stores its raw partial tile - no bias, no activation - into slice ks of a scratch tensor
    // of ws_cols columns through the first output map (which then describes the scratch tensor: slices
    // follow one another along its outermost extent, ws_slice rows (flat form) or images apart), and
    // a second, small kernel adds the slices in a fixed order, then bias and activation. Results do not
    // depend on which block finishes first.
    int ws_mode, ws_cols, ws_slice;
    // Gather form (k x k convolution over at most four input channels, e.g. an RGB stem): the
    // activation "tile" that TMA delivers is the tile's input window of 16-byte pixels
    // (g_iw x g_ih of them, halo included), once per reduction chunk; the operand-split warps
    // build the 128 x 32 operand of the chunk from it, row r = window values of output pixel r
    // at reduction indices k = (ky * g_k + kx) * g_C + c, zero padded to a multiple of 32
    // (chunks_per_tap chunks; kernel = 1 in this form). g_C = input channels, g_k = filter
    // size, g_bytes = window bytes rounded up to 1 KB (its slot at the end of every stage).
    int gather, g_iw, g_ih, g_C, g_bytes, g_k;
    // Residual operand (one-SM form, unsplit reduction): res[pixel * res_ld + channel] is added to the
    // convolution's value (after the bias, before the activation) - a residual block's Add and activation in
    // the convolution's own pass. Null = none.
    const float* res;
    int res_ld;
    uint32_t spin_limit;      // polls a role waits for its turn before it gives up (kSpinLimit by default)
};

// Polls of the role waits for the launches that follow (see ogle_cuda_set_wait_limit).
uint32_t role_wait_limit();

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with the given parity. false = gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}

// K-major operand tile, 128-byte rows, 128-byte swizzle, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr & 0x3FFFFu) >> 4);   // start address, bits [0,14)
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused with swizzle), bits [16,30)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset, bits [32,46)
    d |= (uint64_t)1 << 46;                              // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// One reduction chunk (32 elements = four K=8 steps) issued from a single asm block.
// A lone thread issues every MMA of the block, and a warp can only issue an instruction
// every few cycles, so descriptor arithmetic per MMA is kept to one 64-bit add.
// Descriptors advance by 32 bytes (2 in encoded units) per K step inside the swizzle atom.
__device__ __forceinline__ void umma_tf32_chunk(uint32_t tmem_d, uint64_t ad, uint64_t bd, uint32_t idesc,
                                                uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "add.s64 a1, %1, 2;\n\tadd.s64 b1, %2, 2;\n\t"
        "add.s64 a2, %1, 4;\n\tadd.s64 b2, %2, 4;\n\t"
        "add.s64 a3, %1, 6;\n\tadd.s64 b3, %2, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], a1, b1, %3, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], a2, b2, %3, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], a3, b3, %3, q;\n\t}"
        ::"r"(tmem_d), "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate_first) : "memory");
}

// A chunk of the BF16 pass of the split mode: operands are 128-byte rows of 64 bf16
// ([a_hi | a_lo] against [b_lo | b_hi]), K = 16 per instruction, so the same four
// 32-byte steps cover the chunk.
__device__ __forceinline__ void umma_bf16_chunk(uint32_t tmem_d, uint64_t ad, uint64_t bd, uint32_t idesc,
                                                uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "add.s64 a1, %1, 2;\n\tadd.s64 b1, %2, 2;\n\t"
        "add.s64 a2, %1, 4;\n\tadd.s64 b2, %2, 4;\n\t"
        "add.s64 a3, %1, 6;\n\tadd.s64 b3, %2, 6;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a1, b1, %3, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a2, b2, %3, q;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], a3, b3, %3, q;\n\t}"
        ::"r"(tmem_d), "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate_first) : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Operand split: piece index (row * 8 + 16-byte piece) -> the piece a thread takes instead, with the rows of
// every group of eight permuted to 0,4,1,5,2,6,3,7 (a bijection on the pieces of a tile).
__device__ __forceinline__ int split_row_order(int i) {
    const int x = i >> 3;
    const int r = (x & ~7) | ((x & 1) << 2) | ((x >> 1) & 3);
    return (r << 3) | (i & 7);
}

// Records the first error seen by any block in the library's device status word.
__device__ __forceinline__ void record_error(int* flag, int code) { atomicCAS(flag, 0, code); }


}  // namespace tc
}  // namespace ogle
