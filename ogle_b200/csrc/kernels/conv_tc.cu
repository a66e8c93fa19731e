// Host side of the tcgen05 tensor-core path for the dense contractions: conv2d (general
// and pointwise, as implicit GEMM) and gemm. Builds the TMA tensor maps, chooses tile
// shapes and launches the persistent kernel of conv_tc2.cu.
//
//   D[128 x BN] (fp32, in TMEM)  +=  A[128 x 32] * B[BN x 32]^T   per 32-wide reduction chunk
//
// A = activations, fetched by TMA straight from the NHWC4 tensor: one 4-D box per
//     filter tap, [tn images][th rows][tw cols][32 channels], zero-filled outside
//     the image (that is the convolution's padding), traversal stride = conv stride.
// B = filter, pre-packed K-major [out channel][tap][channel] (see FilterLayout).
// Both land in shared memory in the 128-byte swizzle that the UMMA shared-memory
// descriptors name.
//
// Math modes: OGLE_MATH_TF32 issues one tensor-core pass (operands carry 10 mantissa
// bits). OGLE_MATH_TF32X3 recovers fp32-grade accuracy from three products,
// hi*hi + hi*lo + lo*hi (the dropped lo*lo term is 2^-22 relative): hi*hi as a TF32
// pass, the two cross terms as one BF16 pass over K-concatenated operands
// [a_hi | a_lo] x [b_lo | b_hi] (eight mantissa bits are ample for terms that are
// themselves 2^-11 of the result). The filter parts are made when it is packed; the
// activation parts in shared memory while the pipeline runs.
#include <atomic>
#include <cmath>
#include <cstdlib>

#include "tc_common.cuh"
#include "tma_host.h"

namespace ogle {

int launch_tc_v2(tc::TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo,
                 const CUtensorMap& mY, const CUtensorMap& mY2, long m_tiles, const float* bias, int* err_flag,
                 cudaStream_t s);
int launch_tc_t(tc::TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo,
                const CUtensorMap& mY, const CUtensorMap& mY2, long m_tiles, const float* bias, int* err_flag,
                cudaStream_t s);
int launch_tc_pair(tc::TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo,
                   const CUtensorMap& mY, const CUtensorMap& mY2, long m_tiles, const float* bias, int* err_flag,
                   cudaStream_t s);

__device__ int g_tc_error = 0;   // first error seen by any block (0 = none)

int* error_flag_ptr() {
    // per-device address of the status word
    static thread_local int* ptr = nullptr;
    static thread_local int ptr_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (ptr_device != dev) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_tc_error) != cudaSuccess) return nullptr;
        ptr = static_cast<int*>(p);
        ptr_device = dev;
    }
    return ptr;
}

namespace {

using namespace tc;

// N tiling of the persistent kernel: multiples of 32 columns (one staging slab each).
// Picks the width that minimises (rounds of one tile per SM) x (time of a tile), with a
// tile's time modelled by its tensor-core instructions: one instruction costs about 100
// cycles up to ~180 columns (bound by the shared-memory fetch of its 128-row A operand)
// and 0.55 cycles per column beyond.
// wide_ties: among widths of equal cost take the wider one even when everything fits in one round - for
// layers whose reduction can be split through scratch, which fills the SMs better than narrow tiles do (a
// narrow tile pays the same instruction floor as a wide one).
void choose_n_tiling_v2(int Kp, long m_tiles, TcArgs* t, int requested = 0, bool wide_ties = false) {
    const int kmax = (Kp + 31) / 32 * 32;
    auto mma = [](int n) { const double c = 0.55 * n; return c < 100.0 ? 100.0 : c; };
    int best_bn = 32;
    double best_cost = -1.0;
    for (int bn = 32; bn <= 256 && bn <= kmax; bn += 32) {
        const int n_tiles = (Kp + bn - 1) / bn;
        // the last tile of an uneven split is narrower; even splits are what the candidates give
        const long tiles = m_tiles * n_tiles;
        const long rounds = (tiles + kNumSMs - 1) / kNumSMs;
        double per_tile;
        per_tile = (t->passes == 3 ? 2.0 : 1.0) * mma(bn);     // split mode: a TF32 and a BF16 instruction per step
        const double cost = (double)rounds * per_tile;
        // equal cost: the wider tile when there are several rounds (fewer passes over A), the
        // narrower one when everything fits in one round (more SMs busy, shorter epilogues)
        if (best_cost < 0 || cost < best_cost || (cost == best_cost && (rounds > 1 || wide_ties))) { best_cost = cost; best_bn = bn; }
    }
    if (const char* e = getenv("OGLE_TC_BN")) {      // experiments: force the tile width
        const int v = atoi(e);
        if (v >= 32 && v <= 256 && v % 32 == 0 && v <= kmax) best_bn = v;
    }
    if (requested >= 32 && requested <= 256 && requested % 32 == 0 && requested <= kmax) best_bn = requested;
    t->BN = best_bn;
    t->n_tiles = (Kp + best_bn - 1) / best_bn;
}

// Two-SM form (conv_tc2_pair.cu): 0 = the built-in rule, 1 = never, 2 = wherever it can run.
int pair_mode_override() {
    static const int v = [] { const char* e = getenv("OGLE_TC_PAIR"); return e ? (e[0] == '0' ? 1 : (e[0] == '1' ? 2 : 0)) : 0; }();
    return v;
}

bool split_k_enabled() {
    static const bool v = [] { const char* e = getenv("OGLE_TC_SPLIT_K"); return !(e && e[0] == '0'); }();
    return v;
}

// Whether a launch takes the channels-on-M form (conv_tc2_t.cu): at most 128 (stacked) output channels, an
// unsplit reduction, no gather, at least two 128-pixel tiles, and the caller asked for it (2) or the
// environment forces it for experiments.
bool want_channels_on_m(const TcArgs& t, int Kp_total, long m_tiles, int requested, bool through_scratch = false) {
    static const int mode = [] { const char* e = getenv("OGLE_TC_T"); return e ? (e[0] == '0' ? 1 : (e[0] == '1' ? 2 : 0)) : 0; }();
    if (t.gather || t.bias_mode == 1 || Kp_total > 128 || m_tiles < 2) return false;
    // a split reduction only in the form that goes through scratch
    if (through_scratch ? !(t.ws_mode && t.split_k > 1) : (t.split_k > 1 || t.ws_mode)) return false;
    if (mode == 1 || requested == 1) return false;
    return mode == 2 || requested == 2;
}

// Whether a launch takes the two-SM form: it can (no gather, no split reduction, a tile width that
// halves into multiples of 32 columns, at least one pair of tiles) and either the caller asked for it
// or the rule holds: wide tiles, a reduction long enough that operand traffic dominates, and enough
// pairs of tiles for two rounds of the GPU's SM pairs.
bool want_pair(const TcArgs& t, long m_tiles, int requested) {
    if (t.gather || t.split_k > 1 || t.ws_mode || t.BN % 64 || m_tiles < 2) return false;
    const int mode = pair_mode_override();
    if (mode == 1 || requested == 1) return false;
    if (mode == 2 || requested == 2) return true;
    return false;
}

}  // namespace

bool conv_tc_supported(const ConvArgs& a, int variant) {
    if (variant != CONV_GENERAL && variant != CONV_POINTWISE) return false;
    if (a.group != 1) return false;
    if (a.Cp < 16 || a.kernel * a.kernel * a.Cp < 32) return false;   // too few channels per tap: the RGB stem stays on CUDA cores
    if (a.kernel > 7) return false;
    if (!encode_fn()) return false;
    if (variant == CONV_GENERAL) {
        const int tw = a.Wo < 128 ? a.Wo : 128;
        if ((tw - 1) * a.stride + 1 > 256) return false;     // TMA box limit
    }
    return true;
}

// y2 != null: two-output form. a.K counts the stacked filters (first conv's K1 channels,
// zero rows up to split_col, then the second conv's); y receives [0, K1), y2 the rest.
// The gather form of the kernel: 3x3, at most three input channels stored as 16-byte pixels
// (the RGB stem), whole reduction (9 x C <= 27 values) in one chunk.
// Tile of the gather form: tw x th output pixels of one image, tw * th = 128; the shape that
// wastes the fewest rows among those whose input window (halo included) is at most 1024
// pixels = 16 KB of shared memory per stage and at most 256 pixels wide (a TMA box limit).
static bool gather_tile(const ConvArgs& a, int* tw_out, int* th_out) {
    long best = -1;
    for (int tw = 128; tw >= 16; tw >>= 1) {
        const int th = kTileM / tw;
        const int iw = (tw - 1) * a.stride + a.kernel, ih = (th - 1) * a.stride + a.kernel;
        if (iw > 256 || iw * ih > 1024) continue;
        const long covered = (long)((a.Wo + tw - 1) / tw) * tw * ((a.Ho + th - 1) / th) * th;
        if (best < 0 || covered < best) { best = covered; *tw_out = tw; *th_out = th; }
    }
    return best >= 0;
}

bool conv_tc_gather_supported(const ConvArgs& a, int variant) {
    // 3x3 layers have the direct small-channel kernel, which is as fast on the networks measured: the
    // gather form is opt-in for them and the default for the larger filters, which have no such kernel
    static const bool enabled3 = [] { const char* e = getenv("OGLE_TC_GATHER"); return e && e[0] == '1'; }();
    static const bool disabled = [] { const char* e = getenv("OGLE_TC_GATHER"); return e && e[0] == '0'; }();
    if (disabled || (a.kernel == 3 && !enabled3)) return false;
    int tw, th;
    return variant == CONV_GENERAL && filter_compact(a.C / a.group, a.kernel, a.group) && a.dil == 1 &&
           filter_compact_cols(a.C, a.kernel) <= kMaxGatherK &&
           (a.stride == 1 || a.stride == 2) && a.Cp == 4 && a.Cs == 4 && a.Wo >= 16 && a.K <= 256 && gather_tile(a, &tw, &th) &&
           encode_fn() != nullptr;
}

// Adds the slices of a split reduction in slice order, then bias and activation, and writes the
// output tensor(s). One thread per four channels of a pixel. ws: [slices][rows_stride rows][ws_cols];
// y: stride Ks, first channel koff, K real channels (lanes K..up4(K)-1 written as zero); with y2 the
// columns from split_col on go to the second tensor (dense, K2 channels).
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float4* __restrict__ ws, int slices, long slice_q, int ws_cols_q, long rows,
                     const float* __restrict__ bias, int act, float lo, float hi,
                     float4* __restrict__ y, int Ks_q, int koff_q, int K, int out_q,
                     float4* __restrict__ y2, int split_col, int K2, int out2_q) {
    grid_dependency_trigger();
    grid_dependency_wait();
    const int per_row = out_q + out2_q;
    const long total = rows * per_row;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
        const long m = i / per_row;
        int c = int(i - m * per_row);
        const bool second = c >= out_q;
        if (second) c -= out_q;
        const int col = (second ? split_col : 0) + c * 4;          // column in the stacked accumulator order
        const int real = second ? K2 : K;
        const float4* src = ws + m * ws_cols_q + (col >> 2);
        float4 acc = src[0];
        for (int s = 1; s < slices; ++s) {
            const float4 v = src[(long)s * slice_q];
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float r[4] = {acc.x, acc.y, acc.z, acc.w};
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            const int n = c * 4 + l;
            if (n < real) {
                if (bias) r[l] += bias[col + l];
                r[l] = apply_act(r[l], act, lo, hi);
            } else {
                r[l] = 0.f;                                         // padded lanes stay zero
            }
        }
        const float4 o = make_float4(r[0], r[1], r[2], r[3]);
        if (second) y2[m * out2_q + c] = o;
        else y[m * Ks_q + koff_q + c] = o;
    }
}

// ws / ws_bytes: scratch for a split reduction of more than two ranges (or of a layer with an
// activation), may be null. ws_needed != null: plan only - no tensor maps, no launch - and report the
// scratch size this layer would like.
int launch_conv_tc(const ConvArgs& a, int variant, int math_mode, const float* x, const float* w_hi,
                   const float* w_lo, const float* bias, float* y, cudaStream_t s, float* y2, int K1,
                   int split_col, void* ws, size_t ws_bytes, size_t* ws_needed, const float* residual, int res_ld) {
    const bool plan_only = ws_needed != nullptr;
    if (residual && (y2 || res_ld < a.Kp || (res_ld & 3))) return OGLE_ERR_UNSUPPORTED;
    if (plan_only) *ws_needed = 0;
    TcArgs t = {};
    if (y2) {
        if (split_col <= 0 || (split_col & 31) || K1 <= 0 || K1 > split_col || split_col >= a.K ||
            a.koff != 0)
            return OGLE_ERR_UNSUPPORTED;
        t.split_col = split_col;
        t.K1 = K1;
    }
    // channel extents and row strides of the output tensor(s)
    const int kp_a = y2 ? up4(K1) : a.Kp, ks_a = y2 ? up4(K1) : a.Ks;
    const int kp_b = y2 ? up4(a.K - split_col) : a.Kp;
    const int taps = a.kernel * a.kernel;
    t.Cp32 = (a.C + 31) / 32 * 32;
    t.chunks_per_tap = t.Cp32 / kChunk;
    t.kernel = a.kernel; t.stride = a.stride; t.pad = a.pad; t.dil = a.dil;
    t.K = a.K; t.Kp = a.Kp; t.Ks = a.Ks; t.koff = a.koff;
    t.act = a.act; t.lo = a.lo; t.hi = a.hi;
    t.alpha = 1.f; t.beta = 1.f; t.bias_mode = a.has_bias ? 2 : 0; t.ldc = 0;
    t.passes = math_mode == OGLE_MATH_TF32X3 ? 3 : 1;
    const bool v2 = true;

    CUtensorMap mA, mBhi, mBlo, mY, mY2;
    long m_tiles;
    // planning needs the tile geometry only
    auto make_map = [&](CUtensorMap* m, const void* p, int rank, const cuuint64_t* d, const cuuint64_t* st, const cuuint32_t* b,
                        const cuuint32_t* e) { return plan_only ? true : ogle::make_map(m, p, rank, d, st, b, e); };
    auto make_map_sw = [&](CUtensorMapSwizzle sw, CUtensorMap* m, const void* p, int rank, const cuuint64_t* d,
                           const cuuint64_t* st, const cuuint32_t* b, const cuuint32_t* e) {
        return plan_only ? true : ogle::make_map_sw(sw, m, p, rank, d, st, b, e);
    };
    if (variant == CONV_POINTWISE) {
        t.flat = 1;
        t.N = 1; t.Ho = 1; t.Wo = (int)a.M;
        t.tn = 1; t.th = 1; t.tw = kTileM;
        m_tiles = (a.M + kTileM - 1) / kTileM;
        const cuuint64_t dims[4] = {(cuuint64_t)a.Cp, (cuuint64_t)a.M, 1, 1};
        const cuuint64_t str[3] = {(cuuint64_t)a.Cs * 4, (cuuint64_t)a.Cs * 4 * (cuuint64_t)a.M, (cuuint64_t)a.Cs * 4 * (cuuint64_t)a.M};
        const cuuint32_t box[4] = {kChunk, kTileM, 1, 1};
        const cuuint32_t es[4] = {1, 1, 1, 1};
        if (!make_map(&mA, x, 4, dims, str, box, es)) return OGLE_ERR_CUDA;
        if (v2) {
            const cuuint64_t yd[4] = {(cuuint64_t)kp_a, (cuuint64_t)a.M, 1, 1};
            const cuuint64_t ys[3] = {(cuuint64_t)ks_a * 4, (cuuint64_t)ks_a * 4 * (cuuint64_t)a.M, (cuuint64_t)ks_a * 4 * (cuuint64_t)a.M};
            if (!make_map(&mY, y + a.koff, 4, yd, ys, box, es)) return OGLE_ERR_CUDA;
            if (y2) {
                const cuuint64_t yd2[4] = {(cuuint64_t)kp_b, (cuuint64_t)a.M, 1, 1};
                const cuuint64_t ys2[3] = {(cuuint64_t)kp_b * 4, (cuuint64_t)kp_b * 4 * (cuuint64_t)a.M, (cuuint64_t)kp_b * 4 * (cuuint64_t)a.M};
                if (!make_map(&mY2, y2, 4, yd2, ys2, box, es)) return OGLE_ERR_CUDA;
            }
        }
    } else if (conv_tc_gather_supported(a, variant) && !y2) {
        t.flat = 0;
        t.N = a.N; t.Ho = a.Ho; t.Wo = a.Wo;
        t.gather = 1; t.g_C = a.C; t.g_k = a.kernel;
        t.kernel = 1;                                            // the reduction is a run of gathered chunks
        t.Cp32 = filter_compact_cols(a.C, a.kernel); t.chunks_per_tap = t.Cp32 / kChunk;
        if (!gather_tile(a, &t.tw, &t.th)) return OGLE_ERR_UNSUPPORTED;
        t.tn = 1;
        t.tiles_w = (a.Wo + t.tw - 1) / t.tw;
        t.tiles_h = (a.Ho + t.th - 1) / t.th;
        m_tiles = (long)t.tiles_w * t.tiles_h * a.N;
        t.g_iw = (t.tw - 1) * a.stride + a.kernel;
        t.g_ih = (t.th - 1) * a.stride + a.kernel;
        t.g_bytes = (t.g_iw * t.g_ih * 16 + 1023) / 1024 * 1024;
        const cuuint64_t dims[4] = {4, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.N};
        const cuuint64_t str[3] = {(cuuint64_t)a.Cs * 4, (cuuint64_t)a.Cs * 4 * a.W, (cuuint64_t)a.Cs * 4 * a.W * a.H};
        const cuuint32_t box[4] = {4, (cuuint32_t)t.g_iw, (cuuint32_t)t.g_ih, 1};
        const cuuint32_t es[4] = {1, 1, 1, 1};
        if (!make_map_sw(CU_TENSOR_MAP_SWIZZLE_NONE, &mA, x, 4, dims, str, box, es)) return OGLE_ERR_CUDA;
        const cuuint64_t yd[4] = {(cuuint64_t)kp_a, (cuuint64_t)a.Wo, (cuuint64_t)a.Ho, (cuuint64_t)a.N};
        const cuuint64_t ys[3] = {(cuuint64_t)ks_a * 4, (cuuint64_t)ks_a * 4 * a.Wo, (cuuint64_t)ks_a * 4 * a.Wo * a.Ho};
        const cuuint32_t yb[4] = {kChunk, (cuuint32_t)t.tw, (cuuint32_t)t.th, 1};
        if (!make_map(&mY, y + a.koff, 4, yd, ys, yb, es)) return OGLE_ERR_CUDA;
    } else {
        t.flat = 0;
        t.N = a.N; t.Ho = a.Ho; t.Wo = a.Wo;
        const bool may_split = v2 && a.act == OGLE_ACT_NONE && split_k_enabled() && taps * t.chunks_per_tap >= 16;
        if (a.Wo >= kTileM) {
            const int parts = (a.Wo + kTileM - 1) / kTileM;
            t.tw = (a.Wo + parts - 1) / parts; t.th = 1; t.tn = 1;
        } else {
            // full-width tiles of th rows from tn consecutive images (th * tn * Wo <= 128):
            // take the shape that needs the fewest rounds of one tile per SM; among equals the
            // tallest, whose filter taps overlap most in L2
            t.tw = a.Wo;
            long best = -1;
            for (int th = 1; th <= a.Ho && th * a.Wo <= kTileM; ++th) {
                int tn = kTileM / (th * a.Wo);
                if (tn > a.N) tn = a.N;
                if ((th - 1) * a.stride + 1 > 256) continue;          // TMA box limit
                const long tiles = (long)((a.Ho + th - 1) / th) * ((a.N + tn - 1) / tn);
                // in half-rounds; a reduction split in two (see below) can fill a ragged last round
                long rounds = 2 * ((tiles + kNumSMs - 1) / kNumSMs);
                if (may_split && (2 * tiles + kNumSMs - 1) / kNumSMs < rounds) rounds = (2 * tiles + kNumSMs - 1) / kNumSMs;
                if (best < 0 || rounds <= best) { best = rounds; t.th = th; t.tn = tn; }
            }
        }
        t.tiles_w = (a.Wo + t.tw - 1) / t.tw;
        t.tiles_h = (a.Ho + t.th - 1) / t.th;
        m_tiles = (long)t.tiles_w * t.tiles_h * ((a.N + t.tn - 1) / t.tn);
        const cuuint64_t dims[4] = {(cuuint64_t)a.Cp, (cuuint64_t)a.W, (cuuint64_t)a.H, (cuuint64_t)a.N};
        const cuuint64_t str[3] = {(cuuint64_t)a.Cs * 4, (cuuint64_t)a.Cs * 4 * a.W, (cuuint64_t)a.Cs * 4 * a.W * a.H};
        // the box spans the traversed input extent; one element in `stride` is taken
        const cuuint32_t box[4] = {kChunk, (cuuint32_t)((t.tw - 1) * a.stride + 1), (cuuint32_t)((t.th - 1) * a.stride + 1),
                                   (cuuint32_t)t.tn};
        const cuuint32_t es[4] = {1, (cuuint32_t)a.stride, (cuuint32_t)a.stride, 1};
        if (!make_map(&mA, x, 4, dims, str, box, es)) return OGLE_ERR_CUDA;
        if (v2) {
            const cuuint64_t yd[4] = {(cuuint64_t)kp_a, (cuuint64_t)a.Wo, (cuuint64_t)a.Ho, (cuuint64_t)a.N};
            const cuuint64_t ys[3] = {(cuuint64_t)ks_a * 4, (cuuint64_t)ks_a * 4 * a.Wo, (cuuint64_t)ks_a * 4 * a.Wo * a.Ho};
            const cuuint32_t yb[4] = {kChunk, (cuuint32_t)t.tw, (cuuint32_t)t.th, (cuuint32_t)t.tn};
            const cuuint32_t ye[4] = {1, 1, 1, 1};
            if (!make_map(&mY, y + a.koff, 4, yd, ys, yb, ye)) return OGLE_ERR_CUDA;
            if (y2) {
                const cuuint64_t yd2[4] = {(cuuint64_t)kp_b, (cuuint64_t)a.Wo, (cuuint64_t)a.Ho, (cuuint64_t)a.N};
                const cuuint64_t ys2[3] = {(cuuint64_t)kp_b * 4, (cuuint64_t)kp_b * 4 * a.Wo, (cuuint64_t)kp_b * 4 * a.Wo * a.Ho};
                if (!make_map(&mY2, y2, 4, yd2, ys2, yb, ye)) return OGLE_ERR_CUDA;
            }
        }
    }
    choose_n_tiling_v2(a.Kp, m_tiles, &t, a.n_tile,
                       (plan_only || (ws != nullptr && aligned16(ws))) && !t.gather && split_k_enabled() &&
                           taps * t.chunks_per_tap >= 16);
    const int Kp128 = (a.K + 127) / 128 * 128;
    const cuuint64_t bcols = t.gather ? (cuuint64_t)t.Cp32 : (cuuint64_t)taps * t.Cp32;
    const cuuint64_t bdims[2] = {bcols, (cuuint64_t)Kp128};
    const cuuint64_t bstr[1] = {bcols * 4};
    const cuuint32_t bbox[2] = {kChunk, (cuuint32_t)t.BN};
    const cuuint32_t bes[2] = {1, 1};
    if (!make_map(&mBhi, w_hi, 2, bdims, bstr, bbox, bes)) return OGLE_ERR_CUDA;
    if (!make_map(&mBlo, w_lo, 2, bdims, bstr, bbox, bes)) return OGLE_ERR_CUDA;
    if (v2) {
        // Split the reduction when whole tiles would leave SMs idle (few tiles) or a last round
        // mostly empty. Two forms:
        //  - through scratch memory (the caller lent some): any number of ranges and any activation;
        //    each range stores its partial tile into its own slice and a small second kernel adds the
        //    slices in slice order, then bias and activation - bit-reproducible whatever the order in
        //    which blocks finish;
        //  - in place, two ranges, no activation: the output (a dense tensor, or this convolution's
        //    channel slice of a wider one) is zeroed first and the two partial tiles are added to it by
        //    TMA reduce stores; a sum of two addends onto zero does not depend on their order either.
        t.split_k = 1;
        const int chunks = t.kernel * t.kernel * t.chunks_per_tap;
        const double tiles = (double)m_tiles * t.n_tiles;
        const int ws_cols = t.n_tiles * t.BN;
        // rows (flat form) or images between consecutive slices: whole tiles, so that a tile that
        // hangs over the end of its slice writes padding, not the next slice
        const long slice_units = t.flat ? m_tiles * kTileM : (long)((a.N + t.tn - 1) / t.tn) * t.tn;
        const size_t slice_bytes = (size_t)(t.flat ? slice_units : slice_units * a.Ho * a.Wo) * ws_cols * sizeof(float);
        if (split_k_enabled() && chunks >= 8 && !residual) {      // (a residual operand is added by whole tiles only)
            // cost of the layer in units of one reduction chunk of one tile: rounds of one work item per SM,
            // each item paying its chunks plus a fixed fill / drain of about four chunks
            auto cost_of = [&](int k) {
                const int cps = (chunks + k - 1) / k;
                return ceil(tiles * k / kNumSMs) * (cps + 4.0);
            };
            double best = cost_of(1);
            int best_k = 1;
            bool best_ws = false;
            if (a.act == OGLE_ACT_NONE && chunks / 2 >= 8 && cost_of(2) + 2.0 < 0.9 * best) { best = cost_of(2) + 2.0; best_k = 2; }
            const bool ws_usable = plan_only || (ws != nullptr && aligned16(ws));
            if (ws_usable && !t.gather) {
                static const int cand[] = {2, 3, 4, 6, 8, 12, 16};
                for (int k : cand) {
                    if (chunks / k < 4) break;
                    if (!plan_only && slice_bytes * k > ws_bytes) break;
                    if (slice_bytes * k > ((size_t)192 << 20)) break;
                    // + the second kernel: a launch and a pass over k slices
                    const double c = cost_of(k) + 10.0 + 0.5 * k;
                    if (c < 0.85 * best) { best = c; best_k = k; best_ws = true; }
                }
            }
            if (a.split >= 1) {
                // the caller's choice, as far as it can be served: the in-place form for two ranges without an
                // activation, else the scratch form when scratch of the right size was lent
                int k = a.split;
                while (k > 1 && chunks / k < 1) --k;
                const bool fits = ws_usable && !t.gather && (plan_only || slice_bytes * k <= ws_bytes) &&
                                  slice_bytes * k <= ((size_t)192 << 20);
                if (k == 1) { best_k = 1; best_ws = false; }
                else if (k == 2 && a.act == OGLE_ACT_NONE && !fits) { best_k = 2; best_ws = false; }
                else if (fits) { best_k = k; best_ws = true; }
            }
            t.split_k = best_k;
            t.ws_mode = best_ws ? 1 : 0;
            const int cps = (chunks + t.split_k - 1) / t.split_k;
            while (t.split_k > 1 && (t.split_k - 1) * cps >= chunks) --t.split_k;     // no empty ranges
            if (t.split_k == 1) t.ws_mode = 0;
        }
        if (plan_only) {
            *ws_needed = t.ws_mode ? slice_bytes * t.split_k : 0;
            return OGLE_OK;
        }
        if (t.ws_mode) {
            // channels-on-M form: the scratch tensor is as wide as the filter tile (never wider than planned)
            const bool on_m = want_channels_on_m(t, a.Kp, m_tiles, a.on_m, true);
            const int wcols = on_m ? (a.Kp + 31) / 32 * 32 : ws_cols;
            const size_t wslice_bytes = (size_t)(t.flat ? slice_units : slice_units * a.Ho * a.Wo) * wcols * sizeof(float);
            t.ws_cols = wcols;
            t.ws_slice = (int)slice_units;
            const int act = t.act;
            const float lo = t.lo, hi = t.hi;
            t.act = OGLE_ACT_NONE;                 // the raw sums go to the scratch tensor
            const cuuint32_t es[4] = {1, 1, 1, 1};
            if (t.flat) {
                const cuuint64_t wd[4] = {(cuuint64_t)wcols, (cuuint64_t)slice_units * t.split_k, 1, 1};
                const cuuint64_t wst[3] = {(cuuint64_t)wcols * 4, (cuuint64_t)wcols * 4 * wd[1], (cuuint64_t)wcols * 4 * wd[1]};
                const cuuint32_t wb[4] = {kChunk, kTileM, 1, 1};
                if (!ogle::make_map(&mY, ws, 4, wd, wst, wb, es)) return OGLE_ERR_CUDA;
            } else {
                const cuuint64_t wd[4] = {(cuuint64_t)wcols, (cuuint64_t)a.Wo, (cuuint64_t)a.Ho, (cuuint64_t)slice_units * t.split_k};
                const cuuint64_t wst[3] = {(cuuint64_t)wcols * 4, (cuuint64_t)wcols * 4 * a.Wo, (cuuint64_t)wcols * 4 * a.Wo * a.Ho};
                const cuuint32_t wb[4] = {kChunk, (cuuint32_t)t.tw, (cuuint32_t)t.th, (cuuint32_t)t.tn};
                if (!ogle::make_map(&mY, ws, 4, wd, wst, wb, es)) return OGLE_ERR_CUDA;
            }
            int rc;
            if (on_m) {
                t.BN = wcols;
                t.n_tiles = 1;
                const cuuint32_t fbox[2] = {kChunk, (cuuint32_t)t.BN};
                if (!ogle::make_map(&mBhi, w_hi, 2, bdims, bstr, fbox, bes)) return OGLE_ERR_CUDA;
                if (!ogle::make_map(&mBlo, w_lo, 2, bdims, bstr, fbox, bes)) return OGLE_ERR_CUDA;
                rc = launch_tc_t(t, mA, mBhi, mBlo, mY, mY, m_tiles, nullptr, error_flag_ptr(), s);
            } else {
                rc = launch_tc_v2(t, mA, mBhi, mBlo, mY, mY, m_tiles, nullptr, error_flag_ptr(), s);
            }
            if (rc != OGLE_OK) return rc;
            const long rows = a.M;
            const long slice_q = (long)(wslice_bytes / 16);
            const int out_q = kp_a / 4, out2_q = y2 ? kp_b / 4 : 0;
            const long items = rows * (out_q + out2_q);
            launch_overlapped(splitk_reduce_kernel, dim3(grid_for(items, 256)), dim3(256), 0, s,
                              reinterpret_cast<const float4*>(ws), t.split_k, slice_q, wcols / 4, rows,
                              a.has_bias ? bias : (const float*)nullptr, act, lo, hi, reinterpret_cast<float4*>(y), ks_a / 4,
                              a.koff / 4, y2 ? K1 : a.K, out_q, reinterpret_cast<float4*>(y2), split_col,
                              y2 ? a.K - split_col : 0, out2_q);
            return finish_launch();
        }
        if (t.split_k > 1) {
            const size_t rows = (size_t)a.M;
            if (ks_a == kp_a) {
                if (cudaMemsetAsync(y + a.koff, 0, rows * (size_t)ks_a * sizeof(float), s) != cudaSuccess) return OGLE_ERR_CUDA;
            } else if (cudaMemset2DAsync(y + a.koff, (size_t)ks_a * sizeof(float), 0, (size_t)kp_a * sizeof(float), rows, s) !=
                       cudaSuccess) {
                return OGLE_ERR_CUDA;
            }
            if (y2 && cudaMemsetAsync(y2, 0, rows * (size_t)kp_b * sizeof(float), s) != cudaSuccess) return OGLE_ERR_CUDA;
        }
        t.res = residual;
        t.res_ld = res_ld;
        if (want_channels_on_m(t, a.Kp, m_tiles, a.on_m)) {
            // the filter tile is the M-side operand: all (stacked) channels in one tile of FR rows
            t.BN = (a.Kp + 31) / 32 * 32;
            t.n_tiles = 1;
            const cuuint32_t fbox[2] = {kChunk, (cuuint32_t)t.BN};
            if (!ogle::make_map(&mBhi, w_hi, 2, bdims, bstr, fbox, bes)) return OGLE_ERR_CUDA;
            if (!ogle::make_map(&mBlo, w_lo, 2, bdims, bstr, fbox, bes)) return OGLE_ERR_CUDA;
            return launch_tc_t(t, mA, mBhi, mBlo, mY, y2 ? mY2 : mY, m_tiles, bias, error_flag_ptr(), s);
        }
        if (!residual && want_pair(t, m_tiles, a.pair)) {
            // each block of a pair loads half of the filter tile's rows
            const cuuint32_t hbox[2] = {kChunk, (cuuint32_t)(t.BN / 2)};
            if (!ogle::make_map(&mBhi, w_hi, 2, bdims, bstr, hbox, bes)) return OGLE_ERR_CUDA;
            if (!ogle::make_map(&mBlo, w_lo, 2, bdims, bstr, hbox, bes)) return OGLE_ERR_CUDA;
            return launch_tc_pair(t, mA, mBhi, mBlo, mY, y2 ? mY2 : mY, m_tiles, bias, error_flag_ptr(), s);
        }
        return launch_tc_v2(t, mA, mBhi, mBlo, mY, y2 ? mY2 : mY, m_tiles, bias, error_flag_ptr(), s);
    }
    return OGLE_ERR_UNSUPPORTED;
}

// gemm through the same kernel. B must be K-major: either the caller's B when
// transB == 1 (one-pass mode only) or a packed hi/lo copy made by gemm_pack_b.
bool gemm_tc_supported(const OgleGemmParams& p, const float* A, const float* B) {
    if (p.K < 64 || !encode_fn()) return false;
    if (p.math_mode == OGLE_MATH_TF32 && p.transB == 1 && aligned16(B)) return true;
    return false;
}

static int launch_gemm_common(const OgleGemmParams& p, const float* A, const float* Bhi, const float* Blo,
                              long b_row_stride, long b_rows, const float* C, float* Y, cudaStream_t s, int passes) {
    TcArgs t = {};
    t.flat = 1; t.N = 1; t.Ho = 1; t.Wo = p.M; t.tn = 1; t.th = 1; t.tw = kTileM;
    t.kernel = 1; t.stride = 1; t.pad = 0; t.dil = 1;
    t.Cp32 = (p.K + 31) / 32 * 32;
    t.chunks_per_tap = t.Cp32 / kChunk;
    t.K = p.N; t.Kp = up4(p.N); t.Ks = p.ldy; t.koff = 0;
    t.act = OGLE_ACT_NONE;
    t.alpha = p.alpha; t.beta = p.beta; t.bias_mode = p.bias_mode; t.ldc = p.ldc;
    t.passes = passes;
    const bool v2 = true;
    const long m_tiles = (p.M + kTileM - 1) / kTileM;
    choose_n_tiling_v2(t.Kp, m_tiles, &t);
    CUtensorMap mA, mBhi, mBlo, mY;
    const cuuint64_t dims[4] = {(cuuint64_t)p.K, (cuuint64_t)p.M, 1, 1};
    const cuuint64_t str[3] = {(cuuint64_t)p.lda * 4, (cuuint64_t)p.lda * 4 * (cuuint64_t)p.M, (cuuint64_t)p.lda * 4 * (cuuint64_t)p.M};
    const cuuint32_t box[4] = {kChunk, kTileM, 1, 1};
    const cuuint32_t es[4] = {1, 1, 1, 1};
    if (!make_map(&mA, A, 4, dims, str, box, es)) return OGLE_ERR_CUDA;
    const cuuint64_t bdims[2] = {(cuuint64_t)(Blo ? t.Cp32 : p.K), (cuuint64_t)b_rows};
    const cuuint64_t bstr[1] = {(cuuint64_t)b_row_stride * 4};
    const cuuint32_t bbox[2] = {kChunk, (cuuint32_t)t.BN};
    const cuuint32_t bes[2] = {1, 1};
    if (!make_map(&mBhi, Bhi, 2, bdims, bstr, bbox, bes)) return OGLE_ERR_CUDA;
    if (!make_map(&mBlo, Blo ? Blo : Bhi, 2, bdims, bstr, bbox, bes)) return OGLE_ERR_CUDA;
    if (v2) {
        const cuuint64_t yd[4] = {(cuuint64_t)t.Kp, (cuuint64_t)p.M, 1, 1};
        const cuuint64_t ys[3] = {(cuuint64_t)p.ldy * 4, (cuuint64_t)p.ldy * 4 * (cuuint64_t)p.M, (cuuint64_t)p.ldy * 4 * (cuuint64_t)p.M};
        if (!make_map(&mY, Y, 4, yd, ys, box, es)) return OGLE_ERR_CUDA;
        return launch_tc_v2(t, mA, mBhi, mBlo, mY, mY, m_tiles, C, error_flag_ptr(), s);
    }
    return OGLE_ERR_UNSUPPORTED;
}

int launch_gemm_tc(const OgleGemmParams& p, const float* A, const float* B, const float* C, float* Y, cudaStream_t s) {
    return launch_gemm_common(p, A, B, nullptr, p.ldb, p.N, C, Y, s, 1);
}

int launch_gemm_tc_packed(const OgleGemmParams& p, const float* A, const float* Bhi, const float* Blo,
                          const float* C, float* Y, cudaStream_t s) {
    const long Cp32 = (p.K + 31) / 32 * 32;
    const long rows = (p.N + 127) / 128 * 128;
    return launch_gemm_common(p, A, Bhi, Blo, Cp32, rows, C, Y, s, p.math_mode == OGLE_MATH_TF32X3 ? 3 : 1);
}

namespace {
std::atomic<uint32_t> g_role_wait_limit{tc::kSpinLimit};
}
uint32_t tc::role_wait_limit() { return g_role_wait_limit.load(std::memory_order_relaxed); }
void set_role_wait_limit(long polls) {
    g_role_wait_limit.store(polls < 0 ? tc::kSpinLimit : (polls > long(tc::kSpinLimit) ? tc::kSpinLimit : uint32_t(polls)),
                            std::memory_order_relaxed);
}

int read_tc_error() {
    int v = 0;
    if (cudaMemcpyFromSymbol(&v, g_tc_error, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
int clear_tc_error() {
    const int z = 0;
    return cudaMemcpyToSymbol(g_tc_error, &z, sizeof(int)) == cudaSuccess ? 0 : -1;
}

}  // namespace ogle
