// Direct 3x3 convolution for inputs of at most four channels (the RGB stem of an image
// network: 3 -> 32 channels, stride 2). With so few input channels the implicit-GEMM
// kernels waste their tiles on padding. This layer moves 16 bytes in and (at stride 2)
// 32 bytes out per input pixel while doing 27 multiply-adds per output value, so HBM and
// the FP32 pipes bound it about equally; the kernel is built to keep both busy:
//
//  * persistent blocks walk a list of tiles (rows x columns of one image); the input
//    window of a tile, halo included, is ONE TMA box of 16-byte pixels whose out-of-image
//    part arrives as zeros (the padding); two stages, so the next tile loads while this
//    one is computed;
//  * a warp owns a run of PL*PXT output pixels of one row, PL = 32 / (K/8) pixel lanes x
//    K/8 channel groups: a thread accumulates PXT pixels (interleaved across the lanes,
//    which makes the shared-memory reads conflict-free) x 8 channels in registers;
//  * per filter tap the thread reads its 8x3 weights once (128-bit shared loads) and one
//    float4 per pixel: about one load per eleven multiply-adds, no bounds checks and no
//    address arithmetic in the inner loop.
#include "tc_common.cuh"
#include "tma_host.h"

namespace ogle {
namespace {

using namespace tc;

constexpr int kStemSmemMax = 100 * 1024;
constexpr int kStemStages = 3;          // input tiles in flight or in use per block

struct StemTiles {
    int kgroups, pl;                 // channel groups of 8; pixel lanes per warp
    int segs, rows;                  // warps of a tile: segs across, rows down
    int seg_px;                      // output pixels per warp = pl * PXT
    int tiles_x, tiles_y;
    int iw, ih;                      // input window of a tile
    int total;                       // tiles; 32-bit so that the per-tile index arithmetic is
};

// Two fp32 values in one 64-bit register, and the packed multiply-add of sm_100.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// KP: the padded output channel count when it is known at compile time (32, the usual stem), so that
// every shared-memory offset inside the tap loops is an immediate; 0 = read it from the arguments.
template <int S, int PXT, int CIN, int KP>
__global__ void __launch_bounds__(256, 2)
conv3x3_smallc_kernel(const __grid_constant__ CUtensorMap tmX, const float* __restrict__ w, const float* __restrict__ bias,
                      float* __restrict__ y, const ConvArgs a, const StemTiles tl, int* err_flag) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[kStemStages];
    // weights [9][CIN][Kp] + bias [Kp], then the two input stages (128-byte aligned)
    float* s_w = reinterpret_cast<float*>(smem_raw);
    const int Kp = KP ? KP : a.Kp;
    const int kgroups = KP ? KP / 8 : tl.kgroups;
    const int pls = KP ? 32 / (KP / 8) : tl.pl;           // pixel lanes per warp
    const int wn = 9 * CIN * Kp;
    const uint32_t w_bytes = (uint32_t)((wn + Kp) * 4 + 127) & ~127u;
    const uint32_t stage_bytes = (uint32_t)(tl.ih * tl.iw * 16);      // what one TMA box delivers
    const uint32_t stage_pitch = (stage_bytes + 127u) & ~127u;        // TMA destinations are 128-byte aligned
    const uint32_t base = smem_u32(smem_raw) + w_bytes;
    const float4* stage0 = reinterpret_cast<const float4*>(smem_raw + w_bytes);

    grid_dependency_trigger();
    if (threadIdx.x == 0) {
        for (int i = 0; i < kStemStages; ++i) mbar_init(&bar_full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    grid_dependency_wait();         // nothing from global memory before this point
    for (int i = threadIdx.x; i < wn; i += blockDim.x) {
        const int k = i % Kp, c = (i / Kp) % CIN, tap = i / (Kp * CIN);
        s_w[i] = c < a.C ? w[(tap * a.Cp + c) * Kp + k] : 0.f;     // tap-major packed filter
    }
    for (int i = threadIdx.x; i < Kp; i += blockDim.x) s_w[wn + i] = (a.has_bias && i < a.K) ? bias[i] : 0.f;
    __syncthreads();

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kg = lane % kgroups, pl = lane / kgroups;
    const int seg = warp % tl.segs, row = warp / tl.segs;
    const bool active = row < tl.rows;
    const float* wk = s_w + kg * 8;
    const int tile_px = tl.segs * tl.seg_px;        // output columns per tile

    // tile index -> (column tile, row tile, image), 32-bit (a 64-bit division costs as much as
    // a tenth of a tile's multiply-adds)
    const uint32_t tiles_x = (uint32_t)tl.tiles_x, tiles_y = (uint32_t)tl.tiles_y;
    auto issue = [&](uint32_t tile, int stage) {
        const uint32_t q = tile / tiles_x, tx = tile - q * tiles_x;
        const uint32_t n = q / tiles_y, ty = q - n * tiles_y;
        mbar_expect_tx(&bar_full[stage], stage_bytes);
        tma_load_4d(base + (uint32_t)stage * stage_pitch, &tmX, &bar_full[stage], 0, (int)tx * tile_px * S - a.pad,
                    (int)ty * tl.rows * S - a.pad, (int)n);
    };

    const uint32_t total = (uint32_t)tl.total;
    const bool full_k = kg * 8 + 8 <= a.K;           // every lane of this thread's eight is a real channel
    // ring of kStemStages input tiles: the tiles of the next kStemStages - 1 rounds are in flight
    // while one is being used
    if (threadIdx.x == 0)
        for (int i = 0; i < kStemStages - 1; ++i)
            if (blockIdx.x + (uint32_t)i * gridDim.x < total) issue(blockIdx.x + (uint32_t)i * gridDim.x, i);
    uint32_t it = 0;
    int stage = 0;
    uint32_t phase = 0;
    for (uint32_t tile = blockIdx.x; tile < total; tile += gridDim.x, ++it) {
        // the stage refilled here was last read by tile it-1, finished before the barrier at the loop's end
        {
            const uint32_t ahead = tile + (uint32_t)(kStemStages - 1) * gridDim.x;
            int refill = stage + kStemStages - 1;
            if (refill >= kStemStages) refill -= kStemStages;
            if (threadIdx.x == 0 && ahead < total) issue(ahead, refill);
        }
        const uint32_t tq = tile / tiles_x;
        const int tx = (int)(tile - tq * tiles_x);
        const int n = (int)(tq / tiles_y);
        const int ty = (int)(tq - (uint32_t)n * tiles_y);
        if (!mbar_wait(&bar_full[stage], phase)) {
            if (threadIdx.x == 0) record_error(err_flag, 8);
            break;   // uniform: every thread waits on the same barrier with the same bound
        }
        if (active) {
            const float4* tile_s = stage0 + (size_t)stage * (stage_pitch / 16);
            // accumulators and filter taps as pairs of adjacent channels: one fma.rn.f32x2 does two of the
            // multiply-adds (same IEEE fma per lane, same order of accumulation as the scalar form)
            unsigned long long acc2[PXT][4];
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                const unsigned long long b = pack2(s_w[wn + kg * 8 + 2 * m], s_w[wn + kg * 8 + 2 * m + 1]);
#pragma unroll
                for (int i = 0; i < PXT; ++i) acc2[i][m] = b;
            }
            const int lc = seg * tl.seg_px + pl;                      // first local output column of this thread
            const float4* prow = tile_s + (size_t)(row * S) * tl.iw + lc * S;
            const int step = pls * S;                                 // input columns between this thread's pixels
#pragma unroll
            for (int ky = 0; ky < 3; ++ky) {
#pragma unroll
                for (int kx = 0; kx < 3; ++kx) {
                    unsigned long long f2[CIN][4];
#pragma unroll
                    for (int c = 0; c < CIN; ++c) {
                        const ulonglong2 f0 = *reinterpret_cast<const ulonglong2*>(wk + ((ky * 3 + kx) * CIN + c) * Kp);
                        const ulonglong2 f1 = *reinterpret_cast<const ulonglong2*>(wk + ((ky * 3 + kx) * CIN + c) * Kp + 4);
                        f2[c][0] = f0.x; f2[c][1] = f0.y; f2[c][2] = f1.x; f2[c][3] = f1.y;
                    }
                    const float4* p = prow + ky * tl.iw + kx;
#pragma unroll
                    for (int i = 0; i < PXT; ++i) {
                        const float4 q = p[i * step];
                        const float u[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
                        for (int c = 0; c < CIN; ++c) {
                            const unsigned long long uu = pack2(u[c], u[c]);
#pragma unroll
                            for (int m = 0; m < 4; ++m) acc2[i][m] = fma2(f2[c][m], uu, acc2[i][m]);
                        }
                    }
                }
            }
            float acc[PXT][8];
#pragma unroll
            for (int i = 0; i < PXT; ++i)
#pragma unroll
                for (int m = 0; m < 4; ++m) unpack2(acc2[i][m], acc[i][2 * m], acc[i][2 * m + 1]);
            const int oy = ty * tl.rows + row;
            if (oy < a.Ho) {
                float* yrow = y + (((long)n * a.Ho + oy) * a.Wo) * a.Ks + a.koff + kg * 8;
#pragma unroll
                for (int i = 0; i < PXT; ++i) {
                    const int ox = tx * tile_px + lc + i * pls;
                    if (ox >= a.Wo) continue;
                    float v[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = apply_act(acc[i][j], a.act, a.lo, a.hi);
                    if (!full_k) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (kg * 8 + j >= a.K) v[j] = 0.f;       // padded lanes stay zero
                    }
                    float* dst = yrow + (long)ox * a.Ks;
                    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
            }
        }
        __syncthreads();
        if (++stage == kStemStages) { stage = 0; phase ^= 1u; }
    }
}

// Tile shape: eight warps as segs x rows; a TMA box is at most 256 columns wide.
bool choose_shape(const ConvArgs& a, int pxt, StemTiles* t) {
    const int S = a.stride;
    t->kgroups = a.Kp / 8;
    t->pl = 32 / t->kgroups;
    t->seg_px = t->pl * pxt;
    const int segs_needed = (a.Wo + t->seg_px - 1) / t->seg_px;
    int max_segs = ((256 - 3) / S + 1) / t->seg_px;       // box width (cols - 1) * S + 3 <= 256
    if (max_segs > 8) max_segs = 8;
    if (max_segs < 1) return false;
    const int parts = (segs_needed + max_segs - 1) / max_segs;
    t->segs = (segs_needed + parts - 1) / parts;
    t->rows = 8 / t->segs;
    if (t->rows > a.Ho) t->rows = a.Ho;
    t->tiles_x = (segs_needed + t->segs - 1) / t->segs;
    t->tiles_y = (a.Ho + t->rows - 1) / t->rows;
    t->iw = (t->segs * t->seg_px - 1) * S + 3;
    t->ih = (t->rows - 1) * S + 3;
    const long total = (long)t->tiles_x * t->tiles_y * a.N;
    if (total > 0x7fffffffL - 2 * kNumSMs) return false;     // tile + grid stays below 2^31
    t->total = (int)total;
    const size_t smem = kStemStages * (((size_t)t->ih * t->iw * 16 + 127) / 128 * 128) + (size_t)(9 * 4 * a.Kp + a.Kp) * 4 + 256;
    return t->iw <= 256 && t->ih <= 256 && smem <= (size_t)kStemSmemMax;
}

// Pixels per thread: the candidate that leaves the fewest idle pixel slots across a row.
int choose_pxt(const ConvArgs& a, StemTiles* t) {
    static const int cand[] = {5, 4};
    int best = 0;
    long best_slots = -1;
    for (int pxt : cand) {
        StemTiles s;
        if (!choose_shape(a, pxt, &s)) continue;
        const long slots = (long)s.tiles_x * s.segs * s.seg_px * s.tiles_y * s.rows;
        if (best_slots < 0 || slots < best_slots) { best_slots = slots; best = pxt; *t = s; }
    }
    return best;
}

template <int S, int PXT, int CIN, int KP>
int launch(const ConvArgs& a, const StemTiles& tl, const float* x, const float* w, const float* bias, float* y, cudaStream_t s) {
    CUtensorMap mX;
    const cuuint64_t dims[4] = {4, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.N};
    const cuuint64_t str[3] = {(cuuint64_t)a.Cs * 4, (cuuint64_t)a.Cs * 4 * a.W, (cuuint64_t)a.Cs * 4 * a.W * a.H};
    const cuuint32_t box[4] = {4, (cuuint32_t)tl.iw, (cuuint32_t)tl.ih, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    if (!make_map_sw(CU_TENSOR_MAP_SWIZZLE_NONE, &mX, x, 4, dims, str, box, es)) return OGLE_ERR_CUDA;
    const size_t w_bytes = ((size_t)(9 * CIN * a.Kp + a.Kp) * 4 + 127) / 128 * 128;
    const size_t smem = w_bytes + kStemStages * (((size_t)tl.ih * tl.iw * 16 + 127) / 128 * 128) + 128;
    static thread_local int attr_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(conv3x3_smallc_kernel<S, PXT, CIN, KP>, cudaFuncAttributeMaxDynamicSharedMemorySize, kStemSmemMax);
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_device = dev;
    }
    int blocks = kNumSMs * 2;
    if (blocks > tl.total) blocks = tl.total;
    launch_overlapped(conv3x3_smallc_kernel<S, PXT, CIN, KP>, dim3((unsigned)blocks), dim3(256), smem, s, mX, w, bias, y, a, tl,
                      error_flag_ptr());
    return finish_launch();
}

template <int S, int PXT>
int launch_c(const ConvArgs& a, const StemTiles& tl, const float* x, const float* w, const float* bias, float* y, cudaStream_t s) {
    if (a.Kp == 32) {
        if (a.C == 3) return launch<S, PXT, 3, 32>(a, tl, x, w, bias, y, s);
        return launch<S, PXT, 4, 32>(a, tl, x, w, bias, y, s);
    }
    if (a.C == 3) return launch<S, PXT, 3, 0>(a, tl, x, w, bias, y, s);
    return launch<S, PXT, 4, 0>(a, tl, x, w, bias, y, s);
}

}  // namespace

bool conv_smallc_supported(const ConvArgs& a) {
    if (!(a.group == 1 && a.kernel == 3 && a.dil == 1 && (a.stride == 1 || a.stride == 2) && a.C <= 4 && a.Cp == 4 &&
          (a.Cs & 3) == 0 && (a.Kp == 8 || a.Kp == 16 || a.Kp == 32 || a.Kp == 64) && encode_fn() != nullptr))
        return false;
    StemTiles t;
    return choose_pxt(a, &t) != 0;
}

int launch_conv_smallc(const ConvArgs& a, const float* x, const float* w_tap_major, const float* bias, float* y,
                       cudaStream_t s) {
    StemTiles t = {};
    const int pxt = choose_pxt(a, &t);
    if (a.stride == 1) {
        if (pxt == 5) return launch_c<1, 5>(a, t, x, w_tap_major, bias, y, s);
        if (pxt == 4) return launch_c<1, 4>(a, t, x, w_tap_major, bias, y, s);
    } else {
        if (pxt == 5) return launch_c<2, 5>(a, t, x, w_tap_major, bias, y, s);
        if (pxt == 4) return launch_c<2, 4>(a, t, x, w_tap_major, bias, y, s);
    }
    return OGLE_ERR_UNSUPPORTED;
}

}  // namespace ogle
