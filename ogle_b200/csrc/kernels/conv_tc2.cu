// Persistent tcgen05 kernel for the dense contractions (conv2d general/pointwise
// as implicit GEMM, gemm; tile shapes and tensor maps come from conv_tc.cu):
// one block per SM walks a list of output tiles and every stage of the pipeline
// overlaps with the others ACROSS tiles:
//
//   warp 0, 18  TMA producers (activation tiles / filter tiles): keep a ring of operand
//               stages full, running ahead into the next tile while the current one is
//               still being multiplied; two issuing threads because one tensor copy
//               costs its issuer over a hundred cycles;
//   warp 1      MMA issuer: accumulates tile i into one of 2-4 tensor-memory buffers while
//               the epilogues drain earlier tiles from the others;
//   warps 2-9   two epilogue groups of four warps, taking alternate tiles:
//               tcgen05.ld -> bias / activation -> shared-memory staging in the
//               128-byte swizzle -> TMA tensor store (fully coalesced, clipped at the
//               tensor edge by the hardware);
//   warps 10-17 two operand-split groups for the split (fp32-grade) mode: they write the
//               BF16 operand [a_hi | a_lo] of the cross-term pass next to each activation
//               tile (idle in one-pass mode).
// Each group's work item has a latency of about a microsecond (shared-memory round
// trip plus a proxy fence); two groups per role keep that off the critical path.
//
// HBM traffic per tile is the algorithmic minimum: the activation tile is read
// once, the output tile written once; filters come from L2.
// All mbarrier waits are bounded and abort the block cleanly: the role records a code in
// the status word and raises the block's abort flag, the other roles leave at their next
// wait, the MMA issuer waits for the multiplies it has issued, the teardown waits for the
// operand copies still in flight, and only then is tensor memory freed and the block retired.
// The number of polls of the role waits can be shortened at run time (ogle_cuda_set_wait_limit,
// for tests of this path); the waits of the abort path itself always use the full bound.
#include <cuda_bf16.h>

#include <cstdlib>

#include "tc_common.cuh"

namespace ogle {
namespace {

using namespace tc;

constexpr int kThreads2 = 608;
constexpr int kMaxStages = 8;
constexpr int kStagingBytes = kTileM * 128;   // one 128-row x 32-column fp32 slab

// Bounded wait of a role for its turn; also gives up early when another role of the block has
// aborted. `limit` is the number of polls (kSpinLimit unless the host shortened it).
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
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

__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t (&r)[32], uint32_t taddr) {
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

struct TileCoord { int n_tile, n0, h0, w0; };

__device__ __forceinline__ TileCoord tile_coord(const TcArgs& a, int tile) {
    TileCoord c;
    c.n_tile = tile % a.n_tiles;
    const int m_tile = tile / a.n_tiles;
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

struct WorkItem { int tile, ks, c_begin, c_end; };

// kSplit is a compile-time switch so that the common, unsplit kernel carries none of this
template <bool kSplit>
__device__ __forceinline__ WorkItem work_item(const TcArgs& a, int w, int chunks) {
    WorkItem it;
    if (!kSplit) {
        it.tile = w; it.ks = 0; it.c_begin = 0; it.c_end = chunks;
    } else {
        it.tile = w / a.split_k;
        it.ks = w - it.tile * a.split_k;
        it.c_begin = it.ks * a.chunks_per_split;
        it.c_end = it.c_begin + a.chunks_per_split < chunks ? it.c_begin + a.chunks_per_split : chunks;
    }
    return it;
}

__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

template <bool kSplit>
__global__ void __launch_bounds__(kThreads2, 1)
conv_tc2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBhi,
                const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmY,
                const __grid_constant__ CUtensorMap tmY2, const float* __restrict__ bias, const TcArgs a, int* err_flag) {
    // 1024-byte alignment (the 128-byte swizzle atom) comes from the declaration, so that
    // every byte of the 224 KB request is usable
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kMaxStages], bar_xf[kMaxStages], bar_empty[kMaxStages];
    __shared__ __align__(8) uint64_t bar_acc_full[4], bar_acc_empty[4];
    __shared__ __align__(8) uint64_t bar_drain;     // abort path: the MMAs issued so far have finished
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;
    __shared__ int s_issued[2];                     // operand copies issued by the two producers (abort path)
    __shared__ __align__(16) float s_bias[2][256];
    __shared__ __align__(8) short s_goff[kMaxGatherK];   // gather form: window offset of each reduction index

    grid_dependency_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool split = a.passes == 3;
    const uint32_t b_bytes = (uint32_t)a.BN * 128u;
    const uint32_t stage_bytes = (split ? 2u : 1u) * (kABytes + b_bytes) + (a.gather ? (uint32_t)a.g_bytes : 0u);
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // ring of operand stages (A | A cross (bf16 hi|lo) | B_hi | B cross (bf16 lo|hi)), then the output staging slabs
    auto sA = [&](int s) { return base + (uint32_t)s * stage_bytes; };
    auto sBhi = [&](int s) { return sA(s) + (split ? 2u : 1u) * kABytes; };
    auto sWin = [&](int s) { return sA(s) + (split ? 2u : 1u) * (kABytes + b_bytes); };   // gather form: input window
    const uint32_t staging_off = (uint32_t)a.stages * stage_bytes;
    {
        // the layout must fit what the launch reserved (it does when the base is 1024-aligned as
        // declared); checked, not assumed, because an overrun would write past the block's window
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        const uint32_t need = (base - smem_u32(smem_raw)) + staging_off +
                              (uint32_t)(a.epi_groups * a.epi_slabs) * (uint32_t)kStagingBytes;
        if (need > dyn) {
            if (threadIdx.x == 0) record_error(err_flag, 9);
            return;
        }
    }

    const int chunks = a.kernel * a.kernel * a.chunks_per_tap;
    const int acc_cols = a.BN;     // tensor-memory columns of one accumulator
    const int rows_in_tile = a.flat ? kTileM : a.tn * a.th * a.tw;
    volatile int* abort_flag = &s_abort;

    if (threadIdx.x == 32 * 18) {
        // the copy descriptors are fetched while the barriers and tensor memory are being set up
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmA)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmBhi)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmBlo)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmY)) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(&tmY2)) : "memory");
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&bar_full[s], 2);     // one arrive.expect_tx from each producer
            mbar_init(&bar_xf[s], (uint32_t)(a.xf_groups * 128));
            mbar_init(&bar_empty[s], 1);
        }
        for (int i = 0; i < 4; ++i) {
            mbar_init(&bar_acc_full[i], 1);
            mbar_init(&bar_acc_empty[i], 128);
        }
        mbar_init(&bar_drain, 1);
        s_abort = 0;
        s_issued[0] = 0; s_issued[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (a.gather) {
        // reduction index k = (ky * kernel + kx) * C + c -> float offset of that value in the
        // [g_ih][g_iw][4] input window relative to the output pixel's first tap; -1 = padding column
        const int kred = a.g_k * a.g_k * a.g_C;
        for (int k = threadIdx.x; k < a.chunks_per_tap * kChunk && k < kMaxGatherK; k += blockDim.x) {
            int off = -1;
            if (k < kred) {
                const int tap = k / a.g_C, c = k - tap * a.g_C;
                const int ky = tap / a.g_k, kx = tap - ky * a.g_k;
                off = (ky * a.g_iw + kx) * 4 + c;
            }
            s_goff[k] = (short)off;
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)a.tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;
    // barriers, tensor memory and tables are set up; what follows reads and writes global memory
    grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint32_t tx = (uint32_t)rows_in_tile * 128u;
            // ring position kept incrementally (no divisions in this loop: one thread feeds
            // the whole pipeline and every cycle here is on the critical path)
            int s = 0;                 // stage of the next chunk
            uint32_t wrap = 0;         // how many times the ring has wrapped
            int issued = 0;            // chunks in flight bookkeeping for the abort path
            bool ok = true;
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x) {
                const WorkItem wi = work_item<kSplit>(a, w, chunks);
                const TileCoord tc_ = tile_coord(a, wi.tile);
                const int ax = a.flat ? tc_.w0 : tc_.w0 * a.stride - a.pad;
                const int ay = a.flat ? 0 : tc_.h0 * a.stride - a.pad;
                // position of the first chunk: filter row, filter column, channel offset
                int ky = 0, kx = 0, c0 = 0;
                if (kSplit && wi.c_begin != 0) {      // only the later ranges of a split reduction pay the divisions
                    const int tap0 = wi.c_begin / a.chunks_per_tap;
                    ky = tap0 / a.kernel;
                    kx = tap0 - ky * a.kernel;
                    c0 = (wi.c_begin - tap0 * a.chunks_per_tap) * kChunk;
                }
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    if (wrap > 0) ok = wait_or_abort(&bar_empty[s], (wrap - 1) & 1u, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 1); break; }
                    if (a.gather) {
                        mbar_expect_tx(&bar_full[s], (uint32_t)(a.g_iw * a.g_ih * 16));
                        tma_load_4d(sWin(s), &tmA, &bar_full[s], 0, ax, ay, tc_.n0);
                    } else {
                        mbar_expect_tx(&bar_full[s], tx);
                        tma_load_4d(sA(s), &tmA, &bar_full[s], c0, ax + kx * a.dil, ay + ky * a.dil, tc_.n0);
                    }
                    ++issued;
                    if (++s == a.stages) { s = 0; ++wrap; }
                    // next chunk: channels fastest, then filter column, then filter row
                    c0 += kChunk;
                    if (c0 == a.Cp32) { c0 = 0; if (++kx == a.kernel) { kx = 0; ++ky; } }
                }
            }
            if (!ok) s_abort = 1;
            s_issued[0] = issued;      // the teardown waits for these copies if the block aborts
        }
    } else if (warp == 18) {
        // ------------------------------------------------ TMA producer, filter tiles
        if (lane == 0) {
            const uint32_t tx = (split ? 2u : 1u) * b_bytes;
            int s = 0;
            uint32_t wrap = 0;
            int issued = 0;
            bool ok = true;
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x) {
                const WorkItem wi = work_item<kSplit>(a, w, chunks);
                const int bcol = (wi.tile % a.n_tiles) * a.BN;
                int brow = wi.c_begin * kChunk;
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    if (wrap > 0) ok = wait_or_abort(&bar_empty[s], (wrap - 1) & 1u, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 7); break; }
                    mbar_expect_tx(&bar_full[s], tx);
                    tma_load_2d(sBhi(s), &tmBhi, &bar_full[s], brow, bcol);
                    if (split) tma_load_2d(sBhi(s) + b_bytes, &tmBlo, &bar_full[s], brow, bcol);   // the BF16 cross operand
                    ++issued;
                    if (++s == a.stages) { s = 0; ++wrap; }
                    brow += kChunk;       // packed filter rows follow the chunk order
                }
            }
            if (!ok) s_abort = 1;
            s_issued[1] = issued;
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a.BN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            // kind::f16 with BF16 operands (format code 1), fp32 accumulation
            const uint32_t idesc_bf16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.BN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            int s = 0;
            uint32_t ph = 0;           // parity of the ring pass
            bool ok = true;
            int ti = 0;
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x, ++ti) {
                const WorkItem wi = work_item<kSplit>(a, w, chunks);
                const int as = a.n_acc == 4 ? (ti & 3) : (ti & 1), use = a.n_acc == 4 ? (ti >> 2) : (ti >> 1);
                if (use > 0) ok = wait_or_abort(&bar_acc_empty[as], (uint32_t)((use - 1) & 1), abort_flag, a.spin_limit);
                if (!ok) { record_error(err_flag, 5); s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_d + (uint32_t)(as * acc_cols);
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    // gather form: the operand exists only once the split warps have built it
                    ok = wait_or_abort(a.gather ? &bar_xf[s] : &bar_full[s], ph, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 2); s_abort = 1; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ad = umma_desc(sA(s)), bd = umma_desc(sBhi(s));
                    const uint32_t acc_flag = it > (kSplit ? wi.c_begin : 0) ? 1u : 0u;     // the first chunk overwrites
                    umma_tf32_chunk(d, ad, bd, idesc, acc_flag);            // a x b_hi (a is read as its high part)
                    if (split) {
                        // cross terms [a_hi | a_lo] x [b_lo | b_hi] in BF16, once the split role has
                        // written the activation parts
                        if (!a.gather) {
                            ok = wait_or_abort(&bar_xf[s], ph, abort_flag, a.spin_limit);
                            if (!ok) { record_error(err_flag, 2); s_abort = 1; break; }
                            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        }
                        umma_bf16_chunk(d, ad + (kABytes >> 4), bd + (b_bytes >> 4), idesc_bf16, 1u);
                    }
                    umma_commit(&bar_empty[s]);
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(&bar_acc_full[as]);
            }
            if (!ok) {
                // abort: the multiplies already issued still read shared memory and write tensor
                // memory; the block may free neither before they are done
                umma_commit(&bar_drain);
                mbar_wait(&bar_drain, 0u);
            }
        }
    } else if (warp >= 10) {
        // --------------------------------------------------- operand split (split mode)
        // Builds the BF16 operand of the cross-term pass next to the activation tile:
        // row r = [bf16(a_hi) x 32 | bf16(a_lo) x 32] (128 bytes, same 128-byte swizzle), with
        // a_hi = the value with its low 13 mantissa bits cleared (what the TF32 pass reads)
        // and a_lo = a - a_hi. The fp32 tile itself is left as TMA delivered it. One or two
        // warp groups work on EVERY chunk together.
        const int xg = (warp - 10) >> 2;           // group 0 or 1
        if ((split || a.gather) && xg < a.xf_groups) {
            const int nthr = a.xf_groups * 128;
            const int t = threadIdx.x - 320;       // 0 .. nthr-1
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            // gather form: a thread always builds the same 16-byte piece (t & 7) of the same rows, so the
            // rows' offsets into the input window are computed once: g_row[q] for row (t >> 3) + q * nthr / 8.
            // The four reduction indices of the piece change with the chunk and come from s_goff.
            int g_row[4] = {0, 0, 0, 0};
            if (a.gather) {
                for (int q = 0; q < 4; ++q) {
                    const int r = (t >> 3) + q * (nthr >> 3);
                    const int ry = r / a.tw, rx = r - ry * a.tw;          // tn == 1, tw * th == 128 in this form
                    g_row[q] = ((ry * a.stride) * a.g_iw + rx * a.stride) * 4;
                }
            }
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x) {
                const WorkItem wi = work_item<kSplit>(a, w, chunks);
                for (int it = wi.c_begin; it < wi.c_end; ++it) {
                    ok = wait_or_abort(&bar_full[s], ph, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 3); s_abort = 1; break; }
                    float4* pa = reinterpret_cast<float4*>(base_ptr + (size_t)s * stage_bytes);
                    float4* pl = pa + kABytes / 16;
                    uint2* p2 = reinterpret_cast<uint2*>(pl);                 // 8-byte pieces of the BF16 tile
                    if (a.gather) {
                        // build the operand from the input window: one 16-byte piece (4 values) per step;
                        // which values and which rows this thread handles never changes (see g_off / g_row)
                        const float* win = reinterpret_cast<const float*>(base_ptr + (size_t)s * stage_bytes +
                                                                          (split ? 2u : 1u) * (kABytes + b_bytes));
                        const int j = t & 7;
                        const short4 go = *reinterpret_cast<const short4*>(&s_goff[it * kChunk + j * 4]);
                        const int g_off[4] = {go.x, go.y, go.z, go.w};
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            if (q * nthr >= kABytes / 16) break;
                            const int r = (t >> 3) + q * (nthr >> 3);
                            const float* w0 = win + g_row[q];
                            float v[4];
#pragma unroll
                            for (int l = 0; l < 4; ++l) v[l] = g_off[l] >= 0 ? w0[g_off[l]] : 0.f;
                            pa[(r << 3) + (j ^ (r & 7))] = make_float4(v[0], v[1], v[2], v[3]);
                            if (split) {
                                float h[4];
#pragma unroll
                                for (int l = 0; l < 4; ++l) h[l] = __uint_as_float(__float_as_uint(v[l]) & 0xffffe000u);
                                const __nv_bfloat162 h01 = __floats2bfloat162_rn(h[0], h[1]), h23 = __floats2bfloat162_rn(h[2], h[3]);
                                const __nv_bfloat162 l01 = __floats2bfloat162_rn(v[0] - h[0], v[1] - h[1]),
                                                     l23 = __floats2bfloat162_rn(v[2] - h[2], v[3] - h[3]);
                                uint2 hv, lv;
                                hv.x = *reinterpret_cast<const uint32_t*>(&h01); hv.y = *reinterpret_cast<const uint32_t*>(&h23);
                                lv.x = *reinterpret_cast<const uint32_t*>(&l01); lv.y = *reinterpret_cast<const uint32_t*>(&l23);
                                const int ch = (j >> 1) ^ (r & 7), cl = (4 + (j >> 1)) ^ (r & 7);
                                p2[r * 16 + ch * 2 + (j & 1)] = hv;
                                p2[r * 16 + cl * 2 + (j & 1)] = lv;
                            }
                        }
                    } else
                    for (int i0 = t; i0 < kABytes / 16; i0 += nthr) {
                        // rows of a group of eight are taken in the order 0,4,1,5,2,6,3,7: the four rows a warp
                        // handles at once then put their BF16 halves into both halves of the banks (rows r and
                        // r + 4 swizzle to different 64-byte halves), two wavefronts per store instead of four
                        const int i = split_row_order(i0);
                        const float4 v = pa[i];
                        const int r = i >> 3, j = (i & 7) ^ (r & 7);          // row; logical 16-byte chunk = channels 4j..4j+3
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
                        // bf16 column 4j (hi) / 32 + 4j (lo): 16-byte chunk j/2 resp. 4 + j/2, half j & 1
                        const int ch = (j >> 1) ^ (r & 7), cl = (4 + (j >> 1)) ^ (r & 7);
                        p2[r * 16 + ch * 2 + (j & 1)] = hv;
                        p2[r * 16 + cl * 2 + (j & 1)] = lv;
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(&bar_xf[s]);
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int eg = (warp - 2) >> 2;               // group 0 or 1
        if (eg < a.epi_groups) {
            const int t = (threadIdx.x - 64) & 127;
            const int q = warp & 3;                   // TMEM lane quarter this warp may read
            const int row = q * 32 + lane;
            const int bar_id = 1 + eg;
            float* my_bias = s_bias[eg];
            // each group owns one or two staging slabs and fills them in rounds
            const uint32_t my_staging = staging_off + (uint32_t)(eg * a.epi_slabs) * (uint32_t)kStagingBytes;
            unsigned char* staging = base_ptr + my_staging;
            bool ok = true;
            int ti = 0;
            int staged_nbase = -1;
            int round_no = 0;          // rounds of this group so far (selects the staging slab)
            for (int w = blockIdx.x; w < a.total_work && ok; w += gridDim.x, ++ti) {
                if (ti % a.epi_groups != eg) continue;
                const WorkItem wi = work_item<kSplit>(a, w, chunks);
                const TileCoord tc_ = tile_coord(a, wi.tile);
                const int as = a.n_acc == 4 ? (ti & 3) : (ti & 1), use = a.n_acc == 4 ? (ti >> 2) : (ti >> 1);
                const int nbase = tc_.n_tile * a.BN;
                int groups = (a.Kp - nbase + 31) / 32;
                if (groups > a.BN / 32) groups = a.BN / 32;
                long pix = 0;
                if (a.bias_mode == 1) {
                    pix = (long)tc_.w0 + row;
                    if (pix >= a.Wo) pix = a.Wo - 1;  // clipped rows are dropped by the store; keep reads in range
                }
                // bias of this tile's columns (pre-multiplied by beta), staged while the accumulator
                // is still being produced; skipped when the previous tile had the same columns.
                // Safe to overwrite here: every thread of the group passed the sync that follows the
                // last read of the previous tile's values.
                // (with a split reduction only the first work item of a tile adds the bias)
                const int bias_key = kSplit ? nbase * 2 + (wi.ks == 0 ? 1 : 0) : nbase;
                if (bias_key != staged_nbase) {
                    for (int i = t; i < a.BN; i += 128)
                        my_bias[i] = (a.bias_mode == 2 && (!kSplit || (wi.ks == 0 && !a.ws_mode)) && nbase + i < a.K) ? a.beta * bias[nbase + i] : 0.f;
                    staged_nbase = bias_key;
                }
                // residual operand: this thread's pixel (its accumulator row) in the residual tensor
                const float* res_row = nullptr;
                if (!kSplit && a.res) {
                    if (a.flat) {
                        const long pixel = (long)tc_.w0 + row;
                        if (pixel < a.Wo) res_row = a.res + pixel * a.res_ld;
                    } else if (row < rows_in_tile) {
                        const int rw = row % a.tw, t2 = row / a.tw;
                        const int rh = t2 % a.th, rn = t2 / a.th;
                        const int n = tc_.n0 + rn, h = tc_.h0 + rh, w_ = tc_.w0 + rw;
                        if (n < a.N && h < a.Ho && w_ < a.Wo) res_row = a.res + (((long)n * a.Ho + h) * a.Wo + w_) * a.res_ld;
                    }
                }
                ok = wait_or_abort(&bar_acc_full[as], (uint32_t)(use & 1), abort_flag, a.spin_limit);
                if (!ok) { record_error(err_flag, 4); s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // one 32-column slab per round through a ring of one or two staging slabs: a slab
                // is reused once the store issued from it (one or two rounds ago) has read it, so
                // with two slabs a round never waits for the store of the round just before
                for (int g0 = 0; g0 < groups; ++g0) {
                    const int sb = round_no % a.epi_slabs;
                    ++round_no;
                    if (t == 0) {
                        if (a.epi_slabs == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                    group_sync(bar_id);
                    {
                        const int b = 0;
                        const int col = g0 * 32;
                        uint32_t r[32];
                        const uint32_t taddr = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * acc_cols + col);
                        tmem_ld32(r, taddr);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        if (g0 + b == groups - 1) {
                            // this thread's part of the accumulator is in registers: hand the buffer back
                            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                            mbar_arrive(&bar_acc_empty[as]);
                        }
                        float4* dst = reinterpret_cast<float4*>(staging + (size_t)sb * kStagingBytes + (size_t)row * 128);
                        // which output this slab belongs to, and its first column there
                        // (a partial tile bound for the workspace keeps the stacked column order of the accumulator)
                        const bool to_ws = kSplit && a.ws_mode;
                        const bool second = !to_ws && a.split_col > 0 && nbase + col >= a.split_col;
                        const int lcol = second ? nbase + col - a.split_col : nbase + col;
                        const int kout = to_ws ? a.ws_cols : (second ? a.K - a.split_col : (a.split_col > 0 ? a.K1 : a.K));
                        const bool fast = a.bias_mode != 1 && lcol + 32 <= kout;
                        if (fast) {
                            // every column is a real channel and the bias is per column:
                            // two instructions per value, bias read as 128-bit vectors;
                            // all values first, then the eight 128-bit stores back to back
                            // (measured faster than storing as they come)
                            const float4* bv = reinterpret_cast<const float4*>(my_bias + col);
                            float4 o[8];
#pragma unroll
                            for (int c4 = 0; c4 < 8; ++c4) {
                                const float4 bb = bv[c4];
                                float4 v;
                                v.x = fmaf(a.alpha, __uint_as_float(r[c4 * 4 + 0]), bb.x);
                                v.y = fmaf(a.alpha, __uint_as_float(r[c4 * 4 + 1]), bb.y);
                                v.z = fmaf(a.alpha, __uint_as_float(r[c4 * 4 + 2]), bb.z);
                                v.w = fmaf(a.alpha, __uint_as_float(r[c4 * 4 + 3]), bb.w);
                                if (!kSplit && res_row) {
                                    const float4 rr = __ldg(reinterpret_cast<const float4*>(res_row + lcol) + c4);
                                    v.x += rr.x; v.y += rr.y; v.z += rr.z; v.w += rr.w;
                                }
                                if (a.act == OGLE_ACT_RELU) {
                                    v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
                                } else if (a.act == OGLE_ACT_CLIP) {
                                    v.x = fminf(fmaxf(v.x, a.lo), a.hi); v.y = fminf(fmaxf(v.y, a.lo), a.hi);
                                    v.z = fminf(fmaxf(v.z, a.lo), a.hi); v.w = fminf(fmaxf(v.w, a.lo), a.hi);
                                }
                                o[c4] = v;
                            }
                            // 128-byte swizzle: 16-byte chunk index XOR (row mod 8)
#pragma unroll
                            for (int c4 = 0; c4 < 8; ++c4) dst[c4 ^ (row & 7)] = o[c4];
                        } else {
#pragma unroll
                            for (int c4 = 0; c4 < 8; ++c4) {
                                float v[4];
#pragma unroll
                                for (int l = 0; l < 4; ++l) {
                                    const int n = lcol + c4 * 4 + l;
                                    float acc = a.alpha * __uint_as_float(r[c4 * 4 + l]);
                                    if (n < kout) {
                                        if (a.bias_mode == 2) acc += my_bias[col + c4 * 4 + l];
                                        else if (a.bias_mode == 1) acc = fmaf(a.beta, bias[pix * a.ldc + n], acc);
                                        if (!kSplit && res_row) acc += __ldg(res_row + n);
                                        acc = apply_act(acc, a.act, a.lo, a.hi);
                                    } else {
                                        acc = 0.f;         // padded lanes stay zero
                                    }
                                    v[l] = acc;
                                }
                                dst[c4 ^ (row & 7)] = make_float4(v[0], v[1], v[2], v[3]);
                            }
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    group_sync(bar_id);
                    if (t == 0) {
                        {
                            const uint32_t src = base + my_staging + (uint32_t)sb * (uint32_t)kStagingBytes;
                            int col = nbase + g0 * 32;
                            const CUtensorMap* my = &tmY;
                            const bool to_ws = kSplit && a.ws_mode;
                            if (!to_ws && a.split_col > 0 && col >= a.split_col) { col -= a.split_col; my = &tmY2; }
                            if (to_ws) {
                                // slice ks of the scratch tensor; the reduce kernel adds the slices
                                if (a.flat) tma_store_4d(&tmY, src, col, tc_.w0 + wi.ks * a.ws_slice, 0, 0);
                                else tma_store_4d(&tmY, src, col, tc_.w0, tc_.h0, tc_.n0 + wi.ks * a.ws_slice);
                            } else if (kSplit) {
                                if (a.flat) tma_reduce_add_4d(my, src, col, tc_.w0, 0, 0);
                                else tma_reduce_add_4d(my, src, col, tc_.w0, tc_.h0, tc_.n0);
                            } else if (a.flat) {
                                tma_store_4d(my, src, col, tc_.w0, 0, 0);
                            } else {
                                tma_store_4d(my, src, col, tc_.w0, tc_.h0, tc_.n0);
                            }
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
            // the staging slabs must outlive the stores that read them (their writes to global memory are
            // complete, like every write of the grid, when the grid is)
            if (t == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
    }

    // ------------------------------------------------------------------ teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (s_abort) {
        // Some role gave up. Every role has left its loop (a role that was not waiting finished
        // what it had issued), but operand copies may still be in flight towards this block's
        // shared memory, and the block must not retire before they have landed. A ring stage's
        // barrier completes when BOTH producers have announced their copy and the bytes are in;
        // the producers may have stopped up to a ring apart, so first supply the announcement
        // the other one never made, then wait (full bound) for the last ring of stages.
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)a.tmem_cols));
    }
}

int num_sms() {
    static thread_local int sms = 0, sms_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (sms_device != dev) {
        cudaDeviceProp prop;
        if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return kNumSMs;
        sms = prop.multiProcessorCount;
        sms_device = dev;
    }
    return sms;
}

}  // namespace

int launch_tc_v2(TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo,
                 const CUtensorMap& mY, const CUtensorMap& mY2, long m_tiles, const float* bias, int* err_flag,
                 cudaStream_t s) {
    if (t.BN % 32 || t.BN > 256) return OGLE_ERR_UNSUPPORTED;
    const size_t stage = (size_t)(t.passes == 3 ? 2 : 1) * (kABytes + (size_t)t.BN * 128) + (t.gather ? (size_t)t.g_bytes : 0);
    // Shared memory is split between the operand ring and the epilogue's staging slabs
    // (128 rows x 32 columns each). Preference: two epilogue groups with two slabs each;
    // give slabs back to the ring while that buys another stage and the ring is shallow.
    const size_t kBudget = 224 * 1024;
    const int chunks = t.kernel * t.kernel * t.chunks_per_tap;
    t.xf_groups = (t.passes == 3 || t.gather) ? 2 : 1;   // both operand-split groups work on each chunk
    t.epi_groups = 2;
    t.epi_slabs = 2;
    if (t.passes == 3 && chunks >= 8) {
        // long reductions: the epilogue is rare, the ring needs the room
        t.epi_groups = 1;
        t.epi_slabs = 1;
    } else {
        auto stages_with = [&](int groups, int slabs) { return (int)((kBudget - (size_t)groups * slabs * kStagingBytes) / stage); };
        // (measured: the bandwidth-bound pointwise layers want the second slab more than a
        // fourth stage; reductions of 16+ chunks want the stage)
        const int shallow = chunks >= 16 ? 4 : 3;
        if (stages_with(2, 2) < shallow && stages_with(2, 1) > stages_with(2, 2)) t.epi_slabs = 1;
        if (stages_with(t.epi_groups, t.epi_slabs) < 2) { t.epi_groups = 1; t.epi_slabs = 1; }
    }
    if (const char* e = getenv("OGLE_TC_XF_GROUPS")) t.xf_groups = ((t.passes == 3 || t.gather) && e[0] == '2') ? 2 : 1;
    if (t.gather) t.xf_groups = 2;        // the gather code is laid out for 256 threads
    if (const char* e = getenv("OGLE_TC_EPI_GROUPS")) t.epi_groups = e[0] == '1' ? 1 : 2;
    if (const char* e = getenv("OGLE_TC_EPI_SLABS")) t.epi_slabs = e[0] == '1' ? 1 : 2;
    const size_t staging = (size_t)t.epi_groups * t.epi_slabs * kStagingBytes;
    const size_t budget = kBudget - staging;
    int stages = (int)(budget / stage);
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) return OGLE_ERR_UNSUPPORTED;
    t.stages = stages;
    // accumulators: two, or four when they fit the 512 columns of tensor memory - the multiplies
    // of a tile can then start while the epilogues of the two tiles before it still drain theirs
    const int acc_cols = t.BN;
    t.n_acc = 4 * acc_cols <= 512 ? 4 : 2;
    int cols = 32;
    while (cols < t.n_acc * acc_cols) cols <<= 1;
    t.tmem_cols = cols;
    const long total = m_tiles * t.n_tiles;
    if (total <= 0 || total > 0x7fffffffL) return OGLE_ERR_UNSUPPORTED;
    t.total_tiles = (int)total;
    t.spin_limit = role_wait_limit();
    if (t.split_k < 1) t.split_k = 1;
    if (total * t.split_k > 0x7fffffffL) return OGLE_ERR_UNSUPPORTED;
    t.total_work = (int)(total * t.split_k);
    t.chunks_per_split = (chunks + t.split_k - 1) / t.split_k;
    // Always the whole budget, also when the layout needs less: a block then has its SM to
    // itself whatever else is running, so its tensor-memory allocation can never wait for
    // another resident block's columns.
    const size_t smem = kBudget;
    if (stage * stages + staging > smem) return OGLE_ERR_UNSUPPORTED;
    static thread_local int attr_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(conv_tc2_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(conv_tc2_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_device = dev;
    }
    const int sms = num_sms();
    const unsigned grid = (unsigned)(t.total_work < sms ? t.total_work : sms);
    if (t.split_k > 1)
        launch_overlapped(conv_tc2_kernel<true>, dim3(grid), dim3(kThreads2), smem, s, mA, mBhi, mBlo, mY, mY2, bias, t, err_flag);
    else
        launch_overlapped(conv_tc2_kernel<false>, dim3(grid), dim3(kThreads2), smem, s, mA, mBhi, mBlo, mY, mY2, bias, t, err_flag);
    return finish_launch();
}

}  // namespace ogle
