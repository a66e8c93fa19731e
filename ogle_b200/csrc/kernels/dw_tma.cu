// Depthwise 3x3 convolution (stride 1 or 2, channel count a multiple of 32) as a
// persistent, TMA-fed, HBM-bound kernel.
//
// One block per SM slot walks a list of tiles. A tile is th x tw output pixels of
// one image for a slab of 32 channels; tw is the map's width when that is at most 32
// (so 19- and 10-wide maps are covered without ragged column tiles), else 32 or 16. Its input window, halo included, is ONE TMA
// box [IH rows][IW cols][32 channels]; pixels outside the image arrive as zeros,
// which is the convolution's padding. A ring of two to four shared-memory stages: while
// the block computes tile i from one stage, the TMA engine fills the others with the next tiles, so
// the only HBM traffic is the input read once (halo rows come from L2) and the
// output written once, both as 128-byte runs.
// A thread owns 4 channels (one float4) of one output column and slides a 3-row
// window down RPG output rows of it; 8 lanes cover one pixel's 128 bytes, so
// shared-memory reads are conflict-free. The 32 pixel slots of a block are split into
// 32 / tw row groups.
#include <cstdlib>

#include "tc_common.cuh"
#include "tma_host.h"

namespace ogle {
namespace {

using namespace tc;

constexpr int kDwSmemMax = 110 * 1024;   // two blocks per SM
constexpr int kDwMaxStages = 4;

struct DwTiles {
    int tiles_x, tiles_y, cblocks;   // tile grid per image, 32-channel slabs
    int tw, th, row_groups;          // tile shape: th = RPG * row_groups
    int iw, ih;                      // input window of a tile, halo included
    int stages;                      // tiles in flight per block (2..4)
    long total;
};

template <int S, int RPG>
__global__ void __launch_bounds__(256)
dw3x3_tma_kernel(const __grid_constant__ CUtensorMap tmX, const float4* __restrict__ w, const float* __restrict__ bias,
                 float4* __restrict__ y, const ConvArgs a, const DwTiles tl, int* err_flag) {
    constexpr int CB = 8;                          // float4s (32 channels) per tile
    constexpr int ROWS_IN = (RPG - 1) * S + 3;
    const int TW = tl.tw, TH = tl.th, IW = tl.iw;
    const uint32_t kTileBytes = (uint32_t)(tl.ih * tl.iw * CB * 16);
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kDwMaxStages];

    const uint32_t base = (smem_u32(smem_raw) + 127u) & ~127u;
    const float4* stage0 = reinterpret_cast<const float4*>(smem_raw + (base - smem_u32(smem_raw)));

    const int out_q = a.Ks >> 2, off_q = a.koff >> 2;
    const int c = threadIdx.x % CB;
    const int slot = threadIdx.x / CB;
    const int col = slot % TW, rg = slot / TW;
    const bool active = rg < tl.row_groups;        // slots past tw * row_groups idle

    grid_dependency_trigger();
    if (threadIdx.x == 0) {
        for (int i = 0; i < kDwMaxStages; ++i) mbar_init(&bar_full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    grid_dependency_wait();         // nothing from global memory before this point
    __syncthreads();

    // tile id -> (channel slab fastest, then x, y, image): neighbouring blocks share halo rows in L2
    // (tile counts fit 32 bits: the launch refuses more)
    auto issue = [&](long tile, int stage) {
        unsigned t = (unsigned)tile;
        const int cb = (int)(t % (unsigned)tl.cblocks); t /= (unsigned)tl.cblocks;
        const int tx = (int)(t % (unsigned)tl.tiles_x); t /= (unsigned)tl.tiles_x;
        const int ty = (int)(t % (unsigned)tl.tiles_y); t /= (unsigned)tl.tiles_y;
        const int n = (int)t;
        mbar_expect_tx(&bar_full[stage], kTileBytes);
        tma_load_4d(base + (uint32_t)stage * kTileBytes, &tmX, &bar_full[stage], cb * 32, tx * TW * S - a.pad,
                    ty * TH * S - a.pad, n);
    };

    // prologue: fill all but one stage; each iteration then tops the ring up before computing
    const int nst = tl.stages;
    long issued = 0;                               // tiles whose copy was started (thread 0 only)
    if (threadIdx.x == 0)
        for (int k = 0; k < nst - 1; ++k)
            if ((long)blockIdx.x + (long)k * gridDim.x < tl.total) { issue((long)blockIdx.x + (long)k * gridDim.x, k); ++issued; }
    long it = 0;
    int stage = 0;
    uint32_t phase = 0;
    float4 wk[9];
    float4 bv = make_float4(0.f, 0.f, 0.f, 0.f);
    int loaded_cb = -1;
    for (long tile = blockIdx.x; tile < tl.total; tile += gridDim.x, ++it) {
        // the stage refilled here was last read by tile it-1, which every thread finished
        // before the __syncthreads at the bottom of the previous iteration
        if (threadIdx.x == 0) {
            const long ahead = tile + (long)(nst - 1) * gridDim.x;
            if (ahead < tl.total) { issue(ahead, stage == 0 ? nst - 1 : stage - 1); ++issued; }
        }
        unsigned t = (unsigned)tile;
        const int cb = (int)(t % (unsigned)tl.cblocks); t /= (unsigned)tl.cblocks;
        const int tx = (int)(t % (unsigned)tl.tiles_x); t /= (unsigned)tl.tiles_x;
        const int ty = (int)(t % (unsigned)tl.tiles_y); t /= (unsigned)tl.tiles_y;
        const int n = (int)t;
        const int cq = cb * CB + c;
        // filter taps and bias of this channel slab: when the grid is a multiple of the slab
        // count every tile of a block has the same slab, and they are loaded once
        if (cb != loaded_cb) {
#pragma unroll
            for (int k = 0; k < 9; ++k) wk[k] = w[k * (a.Kp >> 2) + cq];
            bv = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a.has_bias) bv = make_float4(bias[cq * 4], bias[cq * 4 + 1], bias[cq * 4 + 2], bias[cq * 4 + 3]);
            loaded_cb = cb;
        }

        if (!mbar_wait(&bar_full[stage], phase)) {
            if (threadIdx.x == 0) {
                record_error(err_flag, 6);
                // let the later copies already in flight land (bounded) before the block retires
                for (long j = it + 1; j < issued; ++j) mbar_wait(&bar_full[j % nst], (uint32_t)((j / nst) & 1));
            }
            break;   // uniform: every thread waits on the same barrier with the same bound
        }
        const float4* tile_s = stage0 + (size_t)stage * (kTileBytes / 16);
        if (active) {
        float4 acc[RPG];
#pragma unroll
        for (int r = 0; r < RPG; ++r) acc[r] = bv;
        const int row0 = rg * RPG * S;
#pragma unroll
        for (int r = 0; r < ROWS_IN; ++r) {
            float4 v[3];
#pragma unroll
            for (int kx = 0; kx < 3; ++kx) v[kx] = tile_s[((row0 + r) * IW + col * S + kx) * CB + c];
#pragma unroll
            for (int o = 0; o < RPG; ++o) {
                const int ky = r - o * S;
                if (ky < 0 || ky > 2) continue;
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    const float4 f = wk[ky * 3 + kx];
                    acc[o].x = fmaf(f.x, v[kx].x, acc[o].x);
                    acc[o].y = fmaf(f.y, v[kx].y, acc[o].y);
                    acc[o].z = fmaf(f.z, v[kx].z, acc[o].z);
                    acc[o].w = fmaf(f.w, v[kx].w, acc[o].w);
                }
            }
        }
        const int ox = tx * TW + col;
        if (ox < a.Wo) {
#pragma unroll
            for (int o = 0; o < RPG; ++o) {
                const int oy = ty * TH + rg * RPG + o;
                if (oy >= a.Ho) continue;
                y[(((long)n * a.Ho + oy) * a.Wo + ox) * out_q + off_q + cq] = apply_act4(acc[o], a.act, a.lo, a.hi);
            }
        }
        }
        __syncthreads();
        if (++stage == nst) { stage = 0; phase ^= 1u; }
    }
}

template <int S, int RPG>
int launch(const ConvArgs& a, const DwTiles& shape, const float* x, const float* w, const float* bias, float* y, cudaStream_t s) {
    CUtensorMap mX;
    const cuuint64_t dims[4] = {(cuuint64_t)a.C, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.N};
    const cuuint64_t str[3] = {(cuuint64_t)a.Cs * 4, (cuuint64_t)a.Cs * 4 * a.W, (cuuint64_t)a.Cs * 4 * a.W * a.H};
    const cuuint32_t box[4] = {32, (cuuint32_t)shape.iw, (cuuint32_t)shape.ih, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    if (!make_map_sw(CU_TENSOR_MAP_SWIZZLE_NONE, &mX, x, 4, dims, str, box, es)) return OGLE_ERR_CUDA;
    DwTiles tl = shape;
    tl.tiles_x = (a.Wo + tl.tw - 1) / tl.tw;
    tl.tiles_y = (a.Ho + tl.th - 1) / tl.th;
    tl.cblocks = a.K / 32;
    tl.total = (long)tl.tiles_x * tl.tiles_y * tl.cblocks * a.N;
    const size_t smem = (size_t)tl.stages * tl.ih * tl.iw * 8 * 16 + 128;
    static thread_local int attr_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(dw3x3_tma_kernel<S, RPG>, cudaFuncAttributeMaxDynamicSharedMemorySize, kDwSmemMax);
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_device = dev;
    }
    if (tl.total > 0x7fffffffL) return OGLE_ERR_UNSUPPORTED;
    long blocks = (long)kNumSMs * 2;
    // a multiple of the channel-slab count: block b then always works on slab b % cblocks
    if (tl.cblocks <= blocks) blocks -= blocks % tl.cblocks;
    if (blocks > tl.total) blocks = tl.total;
    launch_overlapped(dw3x3_tma_kernel<S, RPG>, dim3((unsigned)blocks), dim3(256), smem, s, mX, reinterpret_cast<const float4*>(w),
                      bias, reinterpret_cast<float4*>(y), a, tl, error_flag_ptr());
    return finish_launch();
}

// Tile shape for a map: full-width tiles when the map is at most 16 wide, equal parts up to 48; the rows per
// thread (one of the compiled RPG values) that leaves the fewest idle output rows.
// Returns the chosen RPG, or 0 when no shape fits two stages in kDwSmemMax.
int choose_shape(const ConvArgs& a, DwTiles* t) {
    const int S = a.stride;
    int tw = a.Wo <= 32 ? a.Wo : (S == 1 ? 32 : 16);
    // Widths that would leave many of the 32 pixel slots of a block idle are cut into equal parts
    // (measured at batch 256: 19 -> 2 x 10 is 6 % faster, 38 -> 3 x 13 is 18 % faster than 32 + 6)
    if (a.Wo >= 17 && a.Wo <= 32) tw = (a.Wo + 1) / 2;
    else if (a.Wo > 32 && a.Wo <= 48) tw = (a.Wo + 2) / 3;
    if (const char* e = getenv("OGLE_DW_TW")) { const int v = atoi(e); if (v >= 1 && v <= 32) tw = v < a.Wo ? v : a.Wo; }
    const int force_rpg = getenv("OGLE_DW_RPG") ? atoi(getenv("OGLE_DW_RPG")) : 0;
    const int groups = 32 / tw;
    static const int kRpg1[] = {10, 8, 7, 5, 4, 2}, kRpg2[] = {7, 5, 4, 2};
    const int* cand = S == 1 ? kRpg1 : kRpg2;
    const int ncand = S == 1 ? 6 : 4;
    int best = 0;
    long best_cost = -1;
    for (int i = 0; i < ncand; ++i) {
        const int rpg = cand[i], th = rpg * groups;
        if (force_rpg && rpg != force_rpg) continue;
        const int iw = (tw - 1) * S + 3, ih = (th - 1) * S + 3;
        if (iw > 256 || ih > 256) continue;
        if (2 * (size_t)ih * iw * 128 + 128 > (size_t)kDwSmemMax) continue;
        const long tiles_y = (a.Ho + th - 1) / th;
        // rows computed (idle ones included) plus a charge per tile for its halo rows
        long cost = tiles_y * (th * S + 2);
        // a single channel slab (32 channels): neighbouring blocks then work on neighbouring
        // tiles of the same rows, and a ring of three shallower tiles measured 20 % faster
        // than two deep ones on the 150x150 map
        if (a.K == 32 && 3 * (size_t)ih * iw * 128 + 128 > (size_t)kDwSmemMax) cost *= 2;
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost; best = rpg;
            t->tw = tw; t->th = th; t->row_groups = groups; t->iw = iw; t->ih = ih;
            // as many tiles in flight as fit: HBM latency x bandwidth needs ~90 KB per SM
            int st = (int)((size_t)(kDwSmemMax - 128) / ((size_t)ih * iw * 128));
            t->stages = st > kDwMaxStages ? kDwMaxStages : st;
        }
    }
    return best;
}

}  // namespace

bool dw_tma_supported(const ConvArgs& a) {
    if (!(a.kernel == 3 && a.dil == 1 && a.pad <= 1 && (a.stride == 1 || a.stride == 2) && a.K % 32 == 0 && a.C == a.K &&
          a.Wo >= 8 && a.Ho >= 4 && encode_fn() != nullptr))
        return false;
    DwTiles t;
    return choose_shape(a, &t) != 0;
}

int launch_dw_tma(const ConvArgs& a, const float* x, const float* w, const float* bias, float* y, cudaStream_t s) {
    DwTiles t = {};
    const int rpg = choose_shape(a, &t);
    if (a.stride == 1) {
        switch (rpg) {
            case 10: return launch<1, 10>(a, t, x, w, bias, y, s);
            case 8: return launch<1, 8>(a, t, x, w, bias, y, s);
            case 7: return launch<1, 7>(a, t, x, w, bias, y, s);
            case 5: return launch<1, 5>(a, t, x, w, bias, y, s);
            case 4: return launch<1, 4>(a, t, x, w, bias, y, s);
            case 2: return launch<1, 2>(a, t, x, w, bias, y, s);
        }
    } else {
        switch (rpg) {
            case 7: return launch<2, 7>(a, t, x, w, bias, y, s);
            case 5: return launch<2, 5>(a, t, x, w, bias, y, s);
            case 4: return launch<2, 4>(a, t, x, w, bias, y, s);
            case 2: return launch<2, 2>(a, t, x, w, bias, y, s);
        }
    }
    return OGLE_ERR_UNSUPPORTED;
}

}  // namespace ogle
