// Two-SM form of the persistent tcgen05 kernel (see conv_tc2.cu for the one-SM form and the
// roles): a cluster of two blocks computes a tile of 256 output pixels x BN output channels
// with tcgen05.mma.cta_group::2. Each block of the pair
//   - loads the activation tile of ITS 128 pixels and builds its BF16 cross operand,
//   - loads only ITS half of the filter tile (BN / 2 output channels); the tensor cores of
//     both SMs read both halves,
//   - holds the accumulator rows of its 128 pixels (all BN columns) in its tensor memory and
//     runs its own epilogue over them.
// This halves the filter bytes each SM's TMA writes and the size of its ring stage (three
// stages instead of two at 256 columns in the fp32-grade mode); the tensor cores of both SMs
// still read both halves, so the time per chunk stays what it was and the gain (1-10 % per
// layer, measured) comes from the deeper ring.
//
// The even block of the pair (the leader) issues every multiply. The odd block's warp 1 is a
// relay: it watches the odd block's operand barriers and arrives on the leader's. Completion
// of the multiplies is signalled to both blocks' barriers by one multicast commit.
// No operand copy is multicast: each block's TMA loads write its own shared memory and
// complete on its own barrier.
//
// Every wait is bounded, as in the one-SM form; a role that gives up raises the abort flag of
// both blocks, the leader waits for the multiplies it has issued, the pair meets at a cluster
// barrier, each block waits for its own copies in flight, and tensor memory is freed last.
#include <cuda_bf16.h>

#include <cstdlib>

#include "tc_common.cuh"

namespace ogle {
namespace {

using namespace tc;

constexpr int kThreadsP = 608;
constexpr int kMaxStagesP = 8;
constexpr int kStagingBytesP = kTileM * 128;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory object in block `cta` of the cluster
__device__ __forceinline__ uint32_t peer_addr(uint32_t local, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(cta));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void store_flag_cluster(uint32_t cluster_addr, int v) {
    asm volatile("st.relaxed.cluster.shared::cluster.u32 [%0], %1;" ::"r"(cluster_addr), "r"(v) : "memory");
}

// Bounded wait with cluster-scope acquire (the barrier may be arrived on by the other block);
// gives up early when a role of either block has aborted.
__device__ __forceinline__ bool wait_pair(uint64_t* bar, uint32_t parity, volatile int* abort_flag, uint32_t limit) {
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

__device__ __forceinline__ void group_sync_p(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

__device__ __forceinline__ void tma_store_4d_p(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

__device__ __forceinline__ void tmem_ld32_p(uint32_t (&r)[32], uint32_t taddr) {
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

// One reduction chunk of the pair's tile: four K steps issued by the leader for both SMs.
__device__ __forceinline__ void umma2_tf32_chunk(uint32_t tmem_d, uint64_t ad, uint64_t bd, uint32_t idesc,
                                                 uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "add.s64 a1, %1, 2;\n\tadd.s64 b1, %2, 2;\n\t"
        "add.s64 a2, %1, 4;\n\tadd.s64 b2, %2, 4;\n\t"
        "add.s64 a3, %1, 6;\n\tadd.s64 b3, %2, 6;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], a1, b1, %3, q;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], a2, b2, %3, q;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], a3, b3, %3, q;\n\t}"
        ::"r"(tmem_d), "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate_first) : "memory");
}
__device__ __forceinline__ void umma2_bf16_chunk(uint32_t tmem_d, uint64_t ad, uint64_t bd, uint32_t idesc,
                                                 uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 a1, a2, a3, b1, b2, b3;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "setp.eq.b32 q, 0, 0;\n\t"
        "add.s64 a1, %1, 2;\n\tadd.s64 b1, %2, 2;\n\t"
        "add.s64 a2, %1, 4;\n\tadd.s64 b2, %2, 4;\n\t"
        "add.s64 a3, %1, 6;\n\tadd.s64 b3, %2, 6;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a1, b1, %3, q;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a2, b2, %3, q;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], a3, b3, %3, q;\n\t}"
        ::"r"(tmem_d), "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate_first) : "memory");
}
// The multiplies issued so far by this thread, in both SMs: arrive on the barrier at this
// shared-memory offset in both blocks of the pair.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void umma2_commit_local(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

struct PairCoord { int n_tile, m_tile, n0, h0, w0; };

// work item w of the pair -> this block's 128-pixel tile (m_tile may be one past the last when
// the tile count is odd: loads then read the zero fill, stores are skipped)
__device__ __forceinline__ PairCoord pair_coord(const TcArgs& a, int w, uint32_t rank) {
    PairCoord c;
    c.n_tile = w % a.n_tiles;
    c.m_tile = (w / a.n_tiles) * 2 + (int)rank;
    c.n0 = 0; c.h0 = 0;
    if (a.flat) {
        c.w0 = c.m_tile * kTileM;
    } else {
        const int tw_i = c.m_tile % a.tiles_w;
        const int t = c.m_tile / a.tiles_w;
        c.w0 = tw_i * a.tw;
        c.h0 = (t % a.tiles_h) * a.th;
        c.n0 = (t / a.tiles_h) * a.tn;
    }
    return c;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsP, 1)
conv_tc2_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBhi,
                     const __grid_constant__ CUtensorMap tmBlo, const __grid_constant__ CUtensorMap tmY,
                     const __grid_constant__ CUtensorMap tmY2, const float* __restrict__ bias, const TcArgs a, int* err_flag) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // same layout in both blocks: an address taken in one names the same object in the other
    __shared__ __align__(8) uint64_t bar_full[kMaxStagesP], bar_xf[kMaxStagesP], bar_empty[kMaxStagesP];
    __shared__ __align__(8) uint64_t bar_pfull[kMaxStagesP], bar_pxf[kMaxStagesP];   // leader: the other block's operands are in
    __shared__ __align__(8) uint64_t bar_acc_full[2], bar_acc_empty[2];
    __shared__ __align__(8) uint64_t bar_drain;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;
    __shared__ int s_issued[2];
    __shared__ __align__(16) float s_bias[2][256];

    grid_dependency_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();
    const bool leader = rank == 0;
    const bool split = a.passes == 3;
    const int half = a.BN >> 1;                       // filter rows (output channels) this block loads
    const uint32_t b_bytes = (uint32_t)half * 128u;
    const uint32_t stage_bytes = (split ? 2u : 1u) * (kABytes + b_bytes);
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    auto sA = [&](int s) { return base + (uint32_t)s * stage_bytes; };
    auto sBhi = [&](int s) { return sA(s) + (split ? 2u : 1u) * kABytes; };
    const uint32_t staging_off = (uint32_t)a.stages * stage_bytes;
    {
        uint32_t dyn;
        asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(dyn));
        const uint32_t need = (base - smem_u32(smem_raw)) + staging_off +
                              (uint32_t)(a.epi_groups * a.epi_slabs) * (uint32_t)kStagingBytesP;
        if (need > dyn) {                             // the same in both blocks: both leave
            if (threadIdx.x == 0) record_error(err_flag, 9);
            return;
        }
    }
    const int chunks = a.kernel * a.kernel * a.chunks_per_tap;
    const int acc_cols = a.BN;
    const int rows_in_tile = a.flat ? kTileM : a.tn * a.th * a.tw;
    const int m_tiles = a.total_tiles / a.n_tiles;
    const int n_pairs = (int)(gridDim.x >> 1), my_pair = (int)(blockIdx.x >> 1);
    volatile int* abort_flag = &s_abort;
    const uint32_t peer_abort = peer_addr(smem_u32(&s_abort), rank ^ 1u);
    auto raise_abort = [&]() { s_abort = 1; store_flag_cluster(peer_abort, 1); };

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
            mbar_init(&bar_pfull[s], 1);
            mbar_init(&bar_pxf[s], 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bar_acc_full[i], 1);
            mbar_init(&bar_acc_empty[i], 256);        // the epilogue groups of both blocks
        }
        mbar_init(&bar_drain, 1);
        s_abort = 0;
        s_issued[0] = 0; s_issued[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        // one warp of each block, together
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)a.tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();          // both blocks' barriers and tensor memory exist before either touches the other's
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;
    grid_dependency_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer, this block's pixels
        if (lane == 0) {
            const uint32_t tx = (uint32_t)rows_in_tile * 128u;
            int s = 0;
            uint32_t wrap = 0;
            int issued = 0;
            bool ok = true;
            for (int w = my_pair; w < a.total_work && ok; w += n_pairs) {
                const PairCoord pc = pair_coord(a, w, rank);
                const int ax = a.flat ? pc.w0 : pc.w0 * a.stride - a.pad;
                const int ay = a.flat ? 0 : pc.h0 * a.stride - a.pad;
                int ky = 0, kx = 0, c0 = 0;
                for (int it = 0; it < chunks; ++it) {
                    if (wrap > 0) ok = wait_pair(&bar_empty[s], (wrap - 1) & 1u, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 11); break; }
                    mbar_expect_tx(&bar_full[s], tx);
                    tma_load_4d(sA(s), &tmA, &bar_full[s], c0, ax + kx * a.dil, ay + ky * a.dil, pc.n0);
                    ++issued;
                    if (++s == a.stages) { s = 0; ++wrap; }
                    c0 += kChunk;
                    if (c0 == a.Cp32) { c0 = 0; if (++kx == a.kernel) { kx = 0; ++ky; } }
                }
            }
            if (!ok) raise_abort();
            s_issued[0] = issued;
        }
    } else if (warp == 18) {
        // ------------------------------------------------ TMA producer, this block's half of the filter tile
        if (lane == 0) {
            const uint32_t tx = (split ? 2u : 1u) * b_bytes;
            int s = 0;
            uint32_t wrap = 0;
            int issued = 0;
            bool ok = true;
            for (int w = my_pair; w < a.total_work && ok; w += n_pairs) {
                const int bcol = (w % a.n_tiles) * a.BN + (int)rank * half;
                int brow = 0;
                for (int it = 0; it < chunks; ++it) {
                    if (wrap > 0) ok = wait_pair(&bar_empty[s], (wrap - 1) & 1u, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 17); break; }
                    mbar_expect_tx(&bar_full[s], tx);
                    tma_load_2d(sBhi(s), &tmBhi, &bar_full[s], brow, bcol);
                    if (split) tma_load_2d(sBhi(s) + b_bytes, &tmBlo, &bar_full[s], brow, bcol);
                    ++issued;
                    if (++s == a.stages) { s = 0; ++wrap; }
                    brow += kChunk;
                }
            }
            if (!ok) raise_abort();
            s_issued[1] = issued;
        }
    } else if (warp == 1 && leader) {
        // -------------------------------------------------------------- MMA issuer (leader block)
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a.BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            const uint32_t idesc_bf16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.BN >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            int ti = 0;
            for (int w = my_pair; w < a.total_work && ok; w += n_pairs, ++ti) {
                const int as = ti & 1, use = ti >> 1;
                if (use > 0) ok = wait_pair(&bar_acc_empty[as], (uint32_t)((use - 1) & 1), abort_flag, a.spin_limit);
                if (!ok) { record_error(err_flag, 15); raise_abort(); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d = tmem_d + (uint32_t)(as * acc_cols);
                for (int it = 0; it < chunks; ++it) {
                    ok = wait_pair(&bar_full[s], ph, abort_flag, a.spin_limit) &&
                         wait_pair(&bar_pfull[s], ph, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 12); raise_abort(); break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ad = umma_desc(sA(s)), bd = umma_desc(sBhi(s));
                    umma2_tf32_chunk(d, ad, bd, idesc, it > 0 ? 1u : 0u);
                    if (split) {
                        ok = wait_pair(&bar_xf[s], ph, abort_flag, a.spin_limit) &&
                             wait_pair(&bar_pxf[s], ph, abort_flag, a.spin_limit);
                        if (!ok) { record_error(err_flag, 12); raise_abort(); break; }
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        umma2_bf16_chunk(d, ad + (kABytes >> 4), bd + (b_bytes >> 4), idesc_bf16, 1u);
                    }
                    umma2_commit_both(&bar_empty[s]);
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma2_commit_both(&bar_acc_full[as]);
            }
            if (!ok) {
                umma2_commit_local(&bar_drain);
                mbar_wait(&bar_drain, 0u);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------- relay (the other block): tell the leader
        // when this block's operands of a stage are in, and at the end wait until the last
        // completions the leader multicasts have landed here
        if (lane == 0) {
            const uint32_t l_pfull = peer_addr(smem_u32(&bar_pfull[0]), 0u), l_pxf = peer_addr(smem_u32(&bar_pxf[0]), 0u);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            long done = 0;
            for (int w = my_pair; w < a.total_work && ok; w += n_pairs) {
                for (int it = 0; it < chunks; ++it) {
                    ok = wait_pair(&bar_full[s], ph, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 13); raise_abort(); break; }
                    mbar_arrive_cluster(l_pfull + (uint32_t)s * 8u);
                    if (split) {
                        ok = wait_pair(&bar_xf[s], ph, abort_flag, a.spin_limit);
                        if (!ok) { record_error(err_flag, 13); raise_abort(); break; }
                        mbar_arrive_cluster(l_pxf + (uint32_t)s * 8u);
                    }
                    ++done;
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                }
            }
            if (ok) {
                // chunk i completes phase (i / stages) of bar_empty[i % stages]
                for (long i = done > a.stages ? done - a.stages : 0; i < done && ok; ++i)
                    ok = wait_pair(&bar_empty[i % a.stages], (uint32_t)((i / a.stages) & 1), abort_flag, a.spin_limit);
                if (!ok) { record_error(err_flag, 16); raise_abort(); }
            }
        }
    } else if (warp >= 10) {
        // --------------------------------------------------- operand split (split mode), this block's pixels
        const int xg = (warp - 10) >> 2;
        if (split && xg < a.xf_groups) {
            const int nthr = a.xf_groups * 128;
            const int t = threadIdx.x - 320;
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int w = my_pair; w < a.total_work && ok; w += n_pairs) {
                for (int it = 0; it < chunks; ++it) {
                    ok = wait_pair(&bar_full[s], ph, abort_flag, a.spin_limit);
                    if (!ok) { record_error(err_flag, 14); raise_abort(); break; }
                    float4* pa = reinterpret_cast<float4*>(base_ptr + (size_t)s * stage_bytes);
                    uint2* p2 = reinterpret_cast<uint2*>(pa + kABytes / 16);
                    for (int i0 = t; i0 < kABytes / 16; i0 += nthr) {
                        const int i = split_row_order(i0);      // see conv_tc2.cu: halves the stores' bank conflicts
                        const float4 v = pa[i];
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
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    mbar_arrive(&bar_xf[s]);
                    if (++s == a.stages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue, this block's pixels
        const int eg = (warp - 2) >> 2;
        if (eg < a.epi_groups) {
            const int t = (threadIdx.x - 64) & 127;
            const int q = warp & 3;
            const int row = q * 32 + lane;
            const int bar_id = 1 + eg;
            float* my_bias = s_bias[eg];
            const uint32_t my_staging = staging_off + (uint32_t)(eg * a.epi_slabs) * (uint32_t)kStagingBytesP;
            unsigned char* staging = base_ptr + my_staging;
            // the leader's barrier counts the arrivals of both blocks' groups
            const uint32_t l_acc_empty = peer_addr(smem_u32(&bar_acc_empty[0]), 0u);
            bool ok = true;
            int ti = 0;
            int staged_nbase = -1;
            int round_no = 0;
            for (int w = my_pair; w < a.total_work && ok; w += n_pairs, ++ti) {
                if (ti % a.epi_groups != eg) continue;
                const PairCoord pc = pair_coord(a, w, rank);
                const bool live = pc.m_tile < m_tiles;
                const int as = ti & 1, use = ti >> 1;
                const int nbase = pc.n_tile * a.BN;
                int groups = (a.Kp - nbase + 31) / 32;
                if (groups > a.BN / 32) groups = a.BN / 32;
                long pix = 0;
                if (a.bias_mode == 1) {
                    pix = (long)pc.w0 + row;
                    if (pix >= a.Wo) pix = a.Wo - 1;
                }
                if (nbase != staged_nbase) {
                    for (int i = t; i < a.BN; i += 128)
                        my_bias[i] = (a.bias_mode == 2 && nbase + i < a.K) ? a.beta * bias[nbase + i] : 0.f;
                    staged_nbase = nbase;
                }
                ok = wait_pair(&bar_acc_full[as], (uint32_t)(use & 1), abort_flag, a.spin_limit);
                if (!ok) { record_error(err_flag, 18); raise_abort(); break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int g0 = 0; g0 < groups; ++g0) {
                    const int sb = round_no % a.epi_slabs;
                    ++round_no;
                    if (t == 0) {
                        if (a.epi_slabs == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                    group_sync_p(bar_id);
                    const int col = g0 * 32;
                    uint32_t r[32];
                    const uint32_t taddr = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * acc_cols + col);
                    tmem_ld32_p(r, taddr);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (g0 == groups - 1) {
                        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                        mbar_arrive_cluster(l_acc_empty + (uint32_t)as * 8u);
                    }
                    float4* dst = reinterpret_cast<float4*>(staging + (size_t)sb * kStagingBytesP + (size_t)row * 128);
                    const bool second = a.split_col > 0 && nbase + col >= a.split_col;
                    const int lcol = second ? nbase + col - a.split_col : nbase + col;
                    const int kout = second ? a.K - a.split_col : (a.split_col > 0 ? a.K1 : a.K);
                    const bool fast = a.bias_mode != 1 && lcol + 32 <= kout;
                    if (fast) {
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
                            if (a.act == OGLE_ACT_RELU) {
                                v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
                            } else if (a.act == OGLE_ACT_CLIP) {
                                v.x = fminf(fmaxf(v.x, a.lo), a.hi); v.y = fminf(fmaxf(v.y, a.lo), a.hi);
                                v.z = fminf(fmaxf(v.z, a.lo), a.hi); v.w = fminf(fmaxf(v.w, a.lo), a.hi);
                            }
                            o[c4] = v;
                        }
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
                                    acc = apply_act(acc, a.act, a.lo, a.hi);
                                } else {
                                    acc = 0.f;
                                }
                                v[l] = acc;
                            }
                            dst[c4 ^ (row & 7)] = make_float4(v[0], v[1], v[2], v[3]);
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    group_sync_p(bar_id);
                    if (t == 0) {
                        if (live) {
                            const uint32_t src = base + my_staging + (uint32_t)sb * (uint32_t)kStagingBytesP;
                            int ocol = nbase + g0 * 32;
                            const CUtensorMap* my = &tmY;
                            if (a.split_col > 0 && ocol >= a.split_col) { ocol -= a.split_col; my = &tmY2; }
                            if (a.flat) tma_store_4d_p(my, src, ocol, pc.w0, 0, 0);
                            else tma_store_4d_p(my, src, ocol, pc.w0, pc.h0, pc.n0);
                        }
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
            }
            if (t == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        }
    }

    // ------------------------------------------------------------------ teardown
    // Every role of both blocks has left its loop; the multiplies have finished (their results
    // were read, or the leader drained them). After the cluster barrier neither block touches
    // the other's shared memory again.
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();
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
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)a.tmem_cols));
    }
}

}  // namespace

int num_sms_for_pairs() {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return kNumSMs;
    return prop.multiProcessorCount;
}

// Launch of the two-SM form. The filter maps must have boxes of BN / 2 rows. m_tiles counts the
// 128-pixel tiles; a work item is a pair of consecutive ones times one N tile.
int launch_tc_pair(TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo,
                   const CUtensorMap& mY, const CUtensorMap& mY2, long m_tiles, const float* bias, int* err_flag,
                   cudaStream_t s) {
    if (t.BN % 64 || t.BN > 256 || t.BN < 64 || t.gather || t.split_k > 1 || t.ws_mode) return OGLE_ERR_UNSUPPORTED;
    const size_t stage = (size_t)(t.passes == 3 ? 2 : 1) * (kABytes + (size_t)(t.BN / 2) * 128);
    const size_t kBudget = 224 * 1024;
    t.xf_groups = t.passes == 3 ? 2 : 1;
    t.epi_groups = 2;
    t.epi_slabs = 1;
    if ((kBudget - 4 * kStagingBytesP) / stage >= 4) t.epi_slabs = 2;
    if (const char* e = getenv("OGLE_TC_EPI_GROUPS")) t.epi_groups = e[0] == '1' ? 1 : 2;
    if (const char* e = getenv("OGLE_TC_EPI_SLABS")) t.epi_slabs = e[0] == '1' ? 1 : 2;
    const size_t staging = (size_t)t.epi_groups * t.epi_slabs * kStagingBytesP;
    int stages = (int)((kBudget - staging) / stage);
    if (stages > kMaxStagesP) stages = kMaxStagesP;
    if (stages < 2) return OGLE_ERR_UNSUPPORTED;
    t.stages = stages;
    t.n_acc = 2;
    int cols = 32;
    while (cols < 2 * t.BN) cols <<= 1;
    t.tmem_cols = cols;
    const long total = m_tiles * t.n_tiles;
    if (total <= 0 || total > 0x7fffffffL) return OGLE_ERR_UNSUPPORTED;
    t.total_tiles = (int)total;
    t.spin_limit = role_wait_limit();
    t.split_k = 1;
    t.total_work = (int)(((m_tiles + 1) / 2) * t.n_tiles);
    t.chunks_per_split = t.kernel * t.kernel * t.chunks_per_tap;
    static thread_local int attr_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(conv_tc2_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_device = dev;
    }
    static thread_local int sms = 0;
    if (!sms) sms = num_sms_for_pairs();
    int pairs = sms / 2;
    if (t.total_work < pairs) pairs = t.total_work;
    launch_overlapped(conv_tc2_pair_kernel, dim3((unsigned)(2 * pairs)), dim3(kThreadsP), kBudget, s, mA, mBhi, mBlo, mY, mY2, bias, t,
                      err_flag);
    return finish_launch();
}

}  // namespace ogle
