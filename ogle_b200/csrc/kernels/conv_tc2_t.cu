// Channels-on-M form of the persistent tcgen05 kernel, for convolutions with at most 128 output
// channels (stacked channels of a two-output launch included): the accumulator is kept
// transposed,
//
//   D[128 channels (TMEM lanes)][256 pixels (TMEM columns)] += F[128 x 32] * X[256 x 32]^T
//
// i.e. the filter tile is the M-side operand and TWO 128-pixel activation tiles, side by side in
// shared memory, are the N-side operand. A tcgen05.mma costs about the same 140-150 cycles for
// any N up to ~180 columns, so a layer with 64-128 output channels pays that floor once per 256
// pixels here instead of once per 128 pixels in the pixels-on-M form (conv_tc2.cu). Measured
// on the 3x3 heads and 64/128-channel 3x3 layers, which sit on that floor: 1.5x in one-pass
// TF32, 1.2-1.3x in the fp32-grade mode (where the shared-memory traffic of the operand split,
// 256 rows per chunk here, then sets the pace).
//
// Roles and pipeline as in conv_tc2.cu (two TMA producer threads, one MMA thread, operand-split
// warp groups for the fp32-grade mode); what differs:
//   - a work item is a pair of consecutive 128-pixel tiles; the activation producer issues two
//     copies per chunk, into adjacent slots, and the split warps convert 256 rows per chunk;
//   - the filter tile has FR = round_up(K, 32) rows; the instruction reads 128, the rows beyond FR
//     are whatever follows in shared memory and only reach accumulator lanes nobody reads;
//   - one epilogue group; warp q owns channels [32q, 32q + 32): for each pixel tile it reads its
//     lanes 32 pixels at a time (tcgen05.ld), adds its channel's bias, applies the activation and
//     writes staging[pixel][channel] - a warp-wide 32-bit store is one 128-byte row, swizzled like a
//     TMA box - then stores the 128-pixel x 32-channel slab with one TMA tensor store of its own. No
//     barrier between the warps of a round; when fewer slabs than active warps fit in shared memory
//     the warps take turns in rounds.
// A split reduction through scratch (ws_mode, as in conv_tc2.cu) is supported: work item (pair, ks) multiplies
// the chunks of range ks and stores its raw partial tiles into slice ks of the scratch tensor.
// Every output value is the same sum of the same products in the same order as in the other forms.
// All waits are bounded and the abort path is the one of conv_tc2.cu.
#include <cuda_bf16.h>

#include <cstdlib>

#include "tc_common.cuh"

namespace ogle {
namespace {

using namespace tc;

constexpr int kThreadsT = 608;
constexpr int kMaxStagesT = 8;
constexpr int kSlabBytes = kTileM * 128;       // 128 pixels x 32 channels

__device__ __forceinline__ bool wait_t(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < limit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done) : "r"(addr), "r"(parity) : "memory");
        if (done) return true;
        if ((spin & 255u) == 255u && *abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ void tma_store_4d_t(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tmem_ld32_t(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

struct TCoord { int m_tile, n0, h0, w0; };

__device__ __forceinline__ TCoord t_coord(const TcArgs& a, int m_tile) {
    TCoord c;
    c.m_tile = m_tile;
    c.n0 = 0; c.h0 = 0;
    if (a.flat) {
        c.w0 = m_tile * kTileM;
    } else {
        const int tw_i = m_tile % a.tiles_w;
        const int t = m_tile / a.tiles_w;
        c.w0 = tw_i * a.tw;
        c.h0 = (t % a.tiles_h) * a.th;
        c.n0 = (t / a.tiles_h) * a.tn;
    }
    return c;
}

struct TItem { int pair, ks, c_begin, c_end; };
__device__ __forceinline__ TItem t_item(const TcArgs& a, int w, int chunks) {
    TItem it;
    if (!a.ws_mode) { it.pair = w; it.ks = 0; it.c_begin = 0; it.c_end = chunks; return it; }
    it.pair = w / a.split_k;
    it.ks = w - it.pair * a.split_k;
    it.c_begin = it.ks * a.chunks_per_split;
    it.c_end = it.c_begin + a.chunks_per_split < chunks ? it.c_begin + a.chunks_per_split : chunks;
    return it;
}

// a.BN holds FR (filter rows loaded per chunk, a multiple of 32, at most 128); a.total_tiles the number of
// 128-pixel tiles; a.total_work the number of tile pairs; a.epi_slabs the staging slabs (1..4).
template <bool kRes>
__global__ void __launch_bounds__(kThreadsT, 1)
conv_tc2_t_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBhi,
                  const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmY,
                  const __grid_constant__ CUtensorMap tmY2, const float* __restrict__ bias, const TcArgs a, int* err_flag) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStagesT], bar_xf[kMaxStagesT], bar_empty[kMaxStagesT];
    __shared__ __align__(8) uint64_t bar_acc_full[2], bar_acc_empty[2];
    __shared__ __align__(8) uint64_t bar_drain;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;
    __shared__ int s_issued[2];

    grid_dependency_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool split = a.passes == 3;
    const int FR = a.BN;
    const uint32_t x_bytes = 2u * kABytes;                 // two pixel tiles, fp32
    const uint32_t f_bytes = (uint32_t)FR * 128u;
    const uint32_t stage_bytes = (split ? 2u : 1u) * (x_bytes + f_bytes);
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // stage: X fp32 (2 tiles) | X cross bf16 (2 tiles) | F hi | F cross      (one-pass mode: X | F)
    auto sX = [&](int s) { return base + (uint32_t)s * stage_bytes; };
    auto sF = [&](int s) { return sX(s) + (split ? 2u : 1u) * x_bytes; };
    const uint32_t staging_off = (uint32_t)a.stages * stage_bytes;
    {
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        // the filter operand is read as 128 rows: what lies behind the last stage's last filter section must be ours
        const uint32_t need = (base - smem_u32(smem_raw)) + staging_off + (uint32_t)a.epi_slabs * (uint32_t)kSlabBytes;
        if (need > dyn || (uint32_t)a.epi_slabs * (uint32_t)kSlabBytes < (uint32_t)(kTileM - FR) * 128u) {
            if (threadIdx.x == 0) record_error(err_flag, 9);
            return;
        }
    }
    const int chunks = a.kernel * a.kernel * a.chunks_per_tap;
    const int rows_in_tile = a.flat ? kTileM : a.tn * a.th * a.tw;
    const int m_tiles = a.total_tiles;
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 32 * 18) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmBhi)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmBlo)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmY)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmY2)) : "memory");
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&bar_full[s], 2);
            mbar_init(&bar_xf[s], (uint32_t)(a.xf_groups * 128));
            mbar_init(&bar_empty[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_acc_full[i], 1);
            mbar_init(&bar_acc_empty[i], 128);
        }
        mbar_init(&bar_drain, 1);
        s_abort = 0;
        s_issued[0] = 0; s_issued[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(512u));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;
    grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------ TMA producer: the two pixel tiles of each chunk
        if (lane == 0) {
            const uint32_t tx = 2u * (uint32_t)rows_in_tile * 128u;
            int s = 0;
            uint32_t wrap = 0;
            int issued = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x) {
                const TItem wi = t_item(a, w, chunks);
                const TCoord t0 = t_coord(a, 2 * wi.pair), t1 = t_coord(a, 2 * wi.pair + 1);
                const int ax0 = a.flat ? t0.w0 : t0.w0 * a.stride - a.pad, ay0 = a.flat ? 0 : t0.h0 * a.stride - a.pad;
                const int ax1 = a.flat ? t1.w0 : t1.w0 * a.stride - a.pad, ay1 = a.flat ? 0 : t1.h0 * a.stride - a.pad;
                int ky = 0, kx = 0, c0 = 0;
                if (wi.c_begin != 0) {
                    const int tap0 = wi.c_begin / a.chunks_per_tap;
                    ky = tap0 / a.kernel;
                    kx = tap0 - ky * a.kernel;
                    c0 = (wi.c_begin - tap0 * a.chunks_per_tap) * kChunk;
                }
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    if (wrap > 0) ok = wait_t(&bar_empty[s], (wrap - 1) & 1u, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 21); break; }
                    mbar_expect_tx(&bar_full[s], tx);
                    // (a pair whose second tile lies past the end reads the zero fill there)
                    tma_load_4d(sX(s), &tmA, &bar_full[s], c0, ax0 + kx * a.dil, ay0 + ky * a.dil, t0.n0);
                    tma_load_4d(sX(s) + kABytes, &tmA, &bar_full[s], c0, ax1 + kx * a.dil, ay1 + ky * a.dil, t1.n0);
                    ++issued;
                    if (++s == a.stages) { s = 0; ++wrap; }
                    c0 += kChunk;
                    if (c0 == a.Cp32) { c0 = 0; if (++kx == a.kernel) { kx = 0; ++ky; } }
                }
            }
            if (!ok) s_abort = 1;
            s_issued[0] = issued;
        }
    } else if (warp == 18) {
        // ------------------------------------------------ TMA producer: filter tiles
        if (lane == 0) {
            const uint32_t tx = (split ? 2u : 1u) * f_bytes;
            int s = 0;
            uint32_t wrap = 0;
            int issued = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x) {
                const TItem wi = t_item(a, w, chunks);
                int brow = wi.c_begin * kChunk;
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    if (wrap > 0) ok = wait_t(&bar_empty[s], (wrap - 1) & 1u, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 27); break; }
                    mbar_expect_tx(&bar_full[s], tx);
                    tma_load_2d(sF(s), &tmBhi, &bar_full[s], brow, 0);
                    if (split) tma_load_2d(sF(s) + f_bytes, &tmBlo, &bar_full[s], brow, 0);
                    ++issued;
                    if (++s == a.stages) { s = 0; ++wrap; }
                    brow += kChunk;
                }
            }
            if (!ok) s_abort = 1;
            s_issued[1] = issued;
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // M = 128 (filter rows), N = 256 (pixels)
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            const uint32_t idesc_bf16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int ti = 0;
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x, ++ti) {
                const int as = ti & 1, use = ti >> 1;
                if (use > 0) ok = wait_t(&bar_acc_empty[as], (uint32_t)((use - 1) & 1), abort_flag, a.spin_limit);
                if (!ok) { record_error(err_flag, 25); s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_d + (uint32_t)(as * 256);
                const TItem wi = t_item(a, w, chunks);
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    ok = wait_t(&bar_full[s], ph, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 22); s_abort = 1; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t fd = umma_desc(sF(s)), xd = umma_desc(sX(s));
                    umma_tf32_chunk(d, fd, xd, idesc, it > wi.c_begin ? 1u : 0u);         // f_hi x x (x read as its high part)
                    if (split) {
                        ok = wait_t(&bar_xf[s], ph, abort_flag, a.spin_limit);
                        if (!ok) { record_error(err_flag, 22); s_abort = 1; break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        // [f_lo | f_hi] x [x_hi | x_lo] in BF16
                        umma_bf16_chunk(d, fd + (f_bytes >> 4), xd + (x_bytes >> 4), idesc_bf16, 1u);
                    }
                    umma_commit(&bar_empty[s]);
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(&bar_acc_full[as]);
            }
            if (!ok) {
                umma_commit(&bar_drain);
                mbar_wait(&bar_drain, 0u);
            }
        }
    } else if (warp >= 10) {
        // --------------------------------------------------- operand split (fp32-grade mode): 256 rows per chunk
        const int xg = (warp - 10) >> 2;
        if (split && xg < a.xf_groups) {
            const int nthr = a.xf_groups * 128;
            const int t = threadIdx.x - 320;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x) {
                const TItem wi = t_item(a, w, chunks);
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    ok = wait_t(&bar_full[s], ph, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 23); s_abort = 1; break; }
                    float4* pa = reinterpret_cast<float4*>(base_ptr + (size_t)s * stage_bytes);
                    uint2* p2 = reinterpret_cast<uint2*>(pa + x_bytes / 16);
                    // 2048 16-byte pieces over 256 threads: eight per thread, all loads issued before the first
                    // conversion so that their latencies overlap
                    constexpr int kPieces = (2 * kABytes / 16) / 256;
                    float4 v8[kPieces];
                    if (nthr == 256) {
#pragma unroll
                        for (int u = 0; u < kPieces; ++u) v8[u] = pa[split_row_order(t + u * 256)];
                    }
#pragma unroll
                    for (int u = 0; u < kPieces; ++u) {
                        if (nthr != 256 && u > 0) break;
                        for (int i0 = t + u * 256; i0 < (int)(x_bytes / 16); i0 += (nthr == 256 ? (int)(x_bytes / 16) : nthr)) {
                            const int i = split_row_order(i0);      // see conv_tc2.cu: halves the stores' bank conflicts
                            const float4 v = nthr == 256 ? v8[u] : pa[i];
                            const int r = i >> 3, j = (i & 7) ^ (r & 7);
                            float4 h;
                            h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
                            h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
                            h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
                            h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
                            const __nv_bfloat162 h01 = __floats2bfloat162_rn(h.x, h.y), h23 = __floats2bfloat162_rn(h.z, h.w);
                            const __nv_bfloat162 l01 = __floats2bfloat162_rn(v.x - h.x, v.y - h.y), l23 = __floats2bfloat162_rn(v.z - h.z, v.w - h.w);
                            uint2 hv, lv;
                            hv.x = *reinterpret_cast<const uint32_t*>(&h01); hv.y = *reinterpret_cast<const uint32_t*>(&h23);
                            lv.x = *reinterpret_cast<const uint32_t*>(&l01); lv.y = *reinterpret_cast<const uint32_t*>(&l23);
                            const int ch = (j >> 1) ^ (r & 7), cl = (4 + (j >> 1)) ^ (r & 7);
                            p2[r * 16 + ch * 2 + (j & 1)] = hv;
                            p2[r * 16 + cl * 2 + (j & 1)] = lv;
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(&bar_xf[s]);
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp >= 2 && warp < 6) {
        // ------------------------------------------------------------------ epilogue (one group)
        const int q = warp & 3;                      // TMEM lane quarter = channels [32q, 32q + 32)
        const int active_warps = FR >> 5;
        const int ch = q * 32 + lane;                // stacked channel (accumulator lane) of this thread
        // which output this warp's slab belongs to, and its first column there
        // (partial tiles bound for the scratch tensor keep the stacked channel order and are stored raw:
        // no bias, no activation - the second kernel applies them after adding the slices)
        const bool raw = a.ws_mode != 0;
        const bool second = !raw && a.split_col > 0 && q * 32 >= a.split_col;
        const int lcol = second ? q * 32 - a.split_col : q * 32;
        const int kout = raw ? FR : (second ? a.K - a.split_col : (a.split_col > 0 ? a.K1 : a.K));
        const bool real = lcol + lane < kout;        // padded lanes are written as zeros
        const float my_b = (!raw && a.bias_mode == 2 && real && ch < a.K) ? a.beta * bias[ch] : 0.f;
        const int act = raw ? OGLE_ACT_NONE : a.act;
        const CUtensorMap* my_map = second ? &tmY2 : &tmY;
        bool ok = true;
        int ti = 0;
        for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x, ++ti) {
            const int as = ti & 1, use = ti >> 1;
            const TItem wi = t_item(a, w, chunks);
            ok = wait_t(&bar_acc_full[as], (uint32_t)(use & 1), abort_flag, a.spin_limit);
            if (!ok) { record_error(err_flag, 24); s_abort = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the warps take the staging slabs in rounds of epi_slabs warps
            const bool turns = a.epi_slabs < active_warps;
            for (int r0 = 0; r0 < active_warps; r0 += a.epi_slabs) {
                const bool mine = q >= r0 && q < r0 + a.epi_slabs && q < active_warps;
                if (mine) {
                    unsigned char* slab = base_ptr + staging_off + (size_t)(q - r0) * kSlabBytes;
                    const uint32_t slab_addr = base + staging_off + (uint32_t)(q - r0) * (uint32_t)kSlabBytes;
                    for (int pt = 0; pt < 2; ++pt) {
                        const TCoord tc_ = t_coord(a, 2 * wi.pair + pt);
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        __syncwarp();
                        // residual operand. Usually a tile's pixels are one contiguous run of the tensor's pixels
                        // (the flat form; whole-width rows of one image; whole images): pixel = run0 + column for
                        // the first run_n columns. Otherwise the tile's pixels are walked in accumulator-column order
                        // (column fastest, then row, then image); (rw, rh, rn) is the pixel of the next column.
                        long run0 = 0;
                        int run_n = -1;                      // -1: no contiguous run, walk
                        if (kRes) {
                            if (a.flat) {
                                run0 = tc_.w0;
                                const long left = (long)a.Wo - tc_.w0;
                                run_n = left < 0 ? 0 : (left > kTileM ? kTileM : (int)left);
                            } else if (a.tw == a.Wo && (a.tn == 1 || a.th == a.Ho)) {
                                run0 = ((long)tc_.n0 * a.Ho + tc_.h0) * a.Wo;
                                long left;
                                if (a.tn == 1) left = tc_.n0 < a.N ? (long)(a.Ho - tc_.h0 < a.th ? a.Ho - tc_.h0 : a.th) * a.Wo : 0;
                                else left = (long)(a.N - tc_.n0 < a.tn ? a.N - tc_.n0 : a.tn) * a.Ho * a.Wo;
                                run_n = left < 0 ? 0 : (int)left;
                            }
                        }
                        const float* res_run = kRes ? a.res + run0 * a.res_ld + lcol + lane : nullptr;
                        int rw = 0, rh = 0, rn = 0;
#pragma unroll 1
                        for (int g = 0; g < 4; ++g) {
                            uint32_t r[32];
                            const uint32_t taddr = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * 256 + pt * 128 + g * 32);
                            tmem_ld32_t(r, taddr);
                            float rr[32];
                            if (kRes) {
                                // this channel's residual values of the 32 pixels, all loads issued before any is used
                                if (run_n >= 0) {
                                    const float* rp = res_run + (long)(g * 32) * a.res_ld;
#pragma unroll
                                    for (int j = 0; j < 32; ++j)
                                        rr[j] = (real && g * 32 + j < run_n) ? __ldg(rp + (long)j * a.res_ld) : 0.f;
                                } else {
#pragma unroll
                                    for (int j = 0; j < 32; ++j) {
                                        long pixel = -1;
                                        const int n = tc_.n0 + rn, h = tc_.h0 + rh, w_ = tc_.w0 + rw;
                                        if (rn < a.tn && n < a.N && h < a.Ho && w_ < a.Wo) pixel = ((long)n * a.Ho + h) * a.Wo + w_;
                                        if (++rw == a.tw) { rw = 0; if (++rh == a.th) { rh = 0; ++rn; } }
                                        rr[j] = (real && pixel >= 0) ? __ldg(a.res + pixel * a.res_ld + lcol + lane) : 0.f;
                                    }
                                }
                            }
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                float v = 0.f;
                                if (real) {
                                    v = fmaf(a.alpha, __uint_as_float(r[j]), my_b);
                                    if (kRes) v += rr[j];
                                    v = apply_act(v, act, a.lo, a.hi);
                                }
                                const int px = g * 32 + j;
                                // row px of the slab, 16-byte piece (lane / 4) swizzled by the row, word lane % 4
                                *reinterpret_cast<float*>(slab + px * 128 + ((((lane >> 2) ^ (px & 7))) << 4) + ((lane & 3) << 2)) = v;
                            }
                        }
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0) {
                            if (tc_.m_tile < m_tiles) {
                                // (scratch: slice ks lies ws_slice rows resp. images further on)
                                if (a.flat) tma_store_4d_t(my_map, slab_addr, lcol, tc_.w0 + (raw ? wi.ks * a.ws_slice : 0), 0, 0);
                                else tma_store_4d_t(my_map, slab_addr, lcol, tc_.w0, tc_.h0, tc_.n0 + (raw ? wi.ks * a.ws_slice : 0));
                            }
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    }
                }
                // when the warps take turns, the next round (of this tile or the first of the next) reuses these
                // slabs: their stores must have been read, and every warp of the round must be through
                if (turns) {
                    if (mine && lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
            }
            // every value of this buffer has been read by now (each warp read its own lanes)
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&bar_acc_empty[as]);
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    }

    // ------------------------------------------------------------------ teardown (as in conv_tc2.cu)
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        if (threadIdx.x == 0) {
            const int na = s_issued[0], nb = s_issued[1];
            const int lo = na < nb ? na : nb, hi = na < nb ? nb : na;
            for (int i = lo; i < hi; ++i) mbar_arrive(&bar_full[i % a.stages]);
            for (int i = (hi > a.stages ? hi - a.stages : 0); i < hi; ++i)
                mbar_wait(&bar_full[i % a.stages], (uint32_t)((i / a.stages) & 1));
        }
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(512u));
    }
}

}  // namespace

// Launch of the channels-on-M form. The filter maps must have boxes of t.BN (= FR) rows. m_tiles counts the
// 128-pixel tiles; a work item is a pair of consecutive ones.
int launch_tc_t(TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo,
                const CUtensorMap& mY, const CUtensorMap& mY2, long m_tiles, const float* bias, int* err_flag,
                cudaStream_t s) {
    const int FR = t.BN;
    if (FR % 32 || FR < 32 || FR > 128 || t.n_tiles != 1 || t.gather || t.bias_mode == 1 || (t.res && t.split_col > 0))
        return OGLE_ERR_UNSUPPORTED;
    if (t.split_k < 1) t.split_k = 1;
    if ((t.split_k > 1) != (t.ws_mode != 0) || (t.ws_mode && t.res)) return OGLE_ERR_UNSUPPORTED;   // splits go through scratch only
    const size_t stage = (size_t)(t.passes == 3 ? 2 : 1) * (2 * kABytes + (size_t)FR * 128);
    const size_t kBudget = 224 * 1024;
    t.xf_groups = t.passes == 3 ? 2 : 1;
    t.epi_groups = 1;
    // staging slabs: one per active warp if two stages still fit beside them, else fewer (the warps take turns);
    // never less than what the 128-row read of the last filter section reaches into
    const int active = FR / 32;
    int slabs = active;
    while (slabs > 1 && (kBudget - (size_t)slabs * kSlabBytes) / stage < 2) --slabs;
    if (slabs == 3 && active == 4) slabs = 2;           // rounds of equal size
    if ((size_t)slabs * kSlabBytes < (size_t)(kTileM - FR) * 128) slabs = (int)(((size_t)(kTileM - FR) * 128 + kSlabBytes - 1) / kSlabBytes);
    t.epi_slabs = slabs;
    int stages = (int)((kBudget - (size_t)slabs * kSlabBytes) / stage);
    if (stages > kMaxStagesT) stages = kMaxStagesT;
    if (stages < 2) return OGLE_ERR_UNSUPPORTED;
    t.stages = stages;
    t.n_acc = 2;
    t.tmem_cols = 512;
    if (m_tiles <= 0 || m_tiles > 0x3fffffffL) return OGLE_ERR_UNSUPPORTED;
    t.total_tiles = (int)m_tiles;
    t.spin_limit = role_wait_limit();
    const int all_chunks = t.kernel * t.kernel * t.chunks_per_tap;
    t.chunks_per_split = (all_chunks + t.split_k - 1) / t.split_k;
    if ((long)(t.split_k - 1) * t.chunks_per_split >= all_chunks && t.split_k > 1) return OGLE_ERR_UNSUPPORTED;   // an empty range
    t.total_work = (int)((m_tiles + 1) / 2) * t.split_k;
    static thread_local int attr_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(conv_tc2_t_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(conv_tc2_t_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_device = dev;
    }
    static thread_local int sms = 0;
    if (!sms) {
        cudaDeviceProp prop;
        sms = cudaGetDeviceProperties(&prop, dev) == cudaSuccess ? prop.multiProcessorCount : kNumSMs;
    }
    const unsigned grid = (unsigned)(t.total_work < sms ? t.total_work : sms);
    if (t.res)
        launch_overlapped(conv_tc2_t_kernel<true>, dim3(grid), dim3(kThreadsT), kBudget, s, mA, mBhi, mBlo, mY, mY2, bias, t, err_flag);
    else
        launch_overlapped(conv_tc2_t_kernel<false>, dim3(grid), dim3(kThreadsT), kBudget, s, mA, mBhi, mBlo, mY, mY2, bias, t, err_flag);
    return finish_launch();
}

}  // namespace ogle
