// tcgen05 tensor-core path for the dense contractions: conv2d (general and
// pointwise, as implicit GEMM) and gemm.
//
//   D[128 x BN] (fp32, in TMEM)  +=  A[128 x 32] * B[BN x 32]^T   per 32-wide reduction chunk
//
// A = activations, fetched by TMA straight from the NHWC4 tensor: one 4-D box per
//     filter tap, [tn images][th rows][tw cols][32 channels], zero-filled outside
//     the image (that is the convolution's padding), traversal stride = conv stride.
// B = filter, pre-packed K-major [out channel][tap][channel] (see FilterLayout).
// Both land in shared memory in the 128-byte swizzle that the UMMA shared-memory
// descriptors name; one elected thread issues tcgen05.mma.kind::tf32 with the
// accumulator in tensor memory; four warps read it back with tcgen05.ld, apply
// bias / activation and store 128-bit vectors.
//
// Math modes: OGLE_MATH_TF32 issues one MMA per step (operands carry 10 mantissa
// bits). OGLE_MATH_TF32X3 splits both operands into hi (top 10 mantissa bits) and
// lo (exact remainder) and accumulates hi*hi + lo*hi + hi*lo, which recovers fp32
// accuracy (the dropped lo*lo term is 2^-22 relative). The filter is split when it
// is packed; activations are split in shared memory by the four epilogue warps
// while the pipeline runs.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocation + MMA
// issue, warps 2-5 = operand split (3-pass mode) then epilogue. All waits on
// mbarriers are bounded: a wait that gives up records an error code, and every
// role falls through to the common teardown that frees tensor memory.
#include <cmath>
#include <cstdlib>

#include "tc_common.cuh"
#include "tma_host.h"

namespace ogle {

int launch_tc_v2(tc::TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo,
                 const CUtensorMap& mY, const CUtensorMap& mY2, long m_tiles, const float* bias, int* err_flag,
                 cudaStream_t s);

__device__ int g_tc_error = 0;   // first error seen by any block (0 = none)

namespace {

using namespace tc;
constexpr int kThreads = 192;

__global__ void __launch_bounds__(kThreads)
conv_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmBhi,
               const __grid_constant__ CUtensorMap tmBlo, const float* __restrict__ bias, float* __restrict__ y,
               const TcArgs a, int* err_flag) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t bar_full[4], bar_xf[4], bar_empty[4], bar_accum;
    __shared__ uint32_t tmem_slot;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool split = a.passes == 3;
    const uint32_t b_bytes = (uint32_t)a.BN * 128u;
    const uint32_t stage_bytes = (split ? 2u : 1u) * (kABytes + b_bytes);
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    unsigned char* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    // stage layout: A | (A_lo) | B_hi | (B_lo)
    auto sA = [&](int s) { return base + (uint32_t)s * stage_bytes; };
    auto sAlo = [&](int s) { return sA(s) + kABytes; };
    auto sBhi = [&](int s) { return sA(s) + (split ? 2u : 1u) * kABytes; };
    auto sBlo = [&](int s) { return sBhi(s) + b_bytes; };

    const int n_tile = blockIdx.x % a.n_tiles;
    const int m_tile = blockIdx.x / a.n_tiles;
    int n0 = 0, h0 = 0, w0 = 0;
    if (a.flat) {
        w0 = m_tile * kTileM;
    } else {
        const int tw_i = m_tile % a.tiles_w;
        const int t = m_tile / a.tiles_w;
        w0 = tw_i * a.tw;
        h0 = (t % a.tiles_h) * a.th;
        n0 = (t / a.tiles_h) * a.tn;
    }
    const int total = a.kernel * a.kernel * a.chunks_per_tap;
    const int rows_in_tile = a.flat ? kTileM : a.tn * a.th * a.tw;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_xf[s], 128);
            mbar_init(&bar_empty[s], 1);
        }
        mbar_init(&bar_accum, 1);
        s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"((uint32_t)a.tmem_cols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_d = tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            const uint32_t tx = (uint32_t)rows_in_tile * 128u + (split ? 2u : 1u) * b_bytes;
            int issued = 0;
            bool ok = true;
            for (int it = 0; it < total && ok; ++it) {
                const int s = it % a.stages, j = it / a.stages;
                if (j > 0) ok = mbar_wait(&bar_empty[s], (uint32_t)((j - 1) & 1));
                if (!ok) { record_error(err_flag, 1); break; }
                const int tap = it / a.chunks_per_tap;
                const int c0 = (it - tap * a.chunks_per_tap) * kChunk;
                const int ky = tap / a.kernel, kx = tap - ky * a.kernel;
                mbar_expect_tx(&bar_full[s], tx);
                if (a.flat) tma_load_4d(sA(s), &tmA, &bar_full[s], c0, w0, 0, 0);
                else tma_load_4d(sA(s), &tmA, &bar_full[s], c0, w0 * a.stride - a.pad + kx * a.dil,
                                 h0 * a.stride - a.pad + ky * a.dil, n0);
                tma_load_2d(sBhi(s), &tmBhi, &bar_full[s], tap * a.Cp32 + c0, n_tile * a.BN);
                if (split) tma_load_2d(sBlo(s), &tmBlo, &bar_full[s], tap * a.Cp32 + c0, n_tile * a.BN);
                issued = it + 1;
            }
            if (!ok) {
                // let the copies already in flight land before the block retires
                s_abort = 1;
                for (int it = (issued > a.stages ? issued - a.stages : 0); it < issued; ++it)
                    mbar_wait(&bar_full[it % a.stages], (uint32_t)((it / a.stages) & 1));
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            // instruction descriptor: D fp32, A/B tf32, both K-major, N, M = 128
            const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(a.BN >> 3) << 17) | ((uint32_t)(kTileM >> 4) << 24);
            bool ok = true;
            for (int it = 0; it < total; ++it) {
                const int s = it % a.stages;
                const uint32_t ph = (uint32_t)((it / a.stages) & 1);
                ok = mbar_wait(split ? &bar_xf[s] : &bar_full[s], ph);
                if (!ok) { record_error(err_flag, 2); s_abort = 1; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int k = 0; k < kChunk / 8; ++k) {
                    const uint64_t ad = umma_desc(sA(s) + k * 32), bd = umma_desc(sBhi(s) + k * 32);
                    umma_tf32(tmem_d, ad, bd, idesc, (it > 0 || k > 0) ? 1u : 0u);
                    if (split) {
                        umma_tf32(tmem_d, umma_desc(sAlo(s) + k * 32), bd, idesc, 1u);
                        umma_tf32(tmem_d, ad, umma_desc(sBlo(s) + k * 32), idesc, 1u);
                    }
                }
                umma_commit(&bar_empty[s]);   // frees the stage once these MMAs have read it
            }
            umma_commit(&bar_accum);          // accumulator complete (arrives even after an abort)
        }
    } else {
        // --------------------------------------- operand split, then the epilogue
        const int t = threadIdx.x - 64;       // 0..127
        bool ok = true;
        if (split) {
            for (int it = 0; it < total && ok; ++it) {
                const int s = it % a.stages;
                const uint32_t ph = (uint32_t)((it / a.stages) & 1);
                ok = mbar_wait(&bar_full[s], ph);
                if (!ok) { record_error(err_flag, 3); break; }
                float4* pa = reinterpret_cast<float4*>(base_ptr + (size_t)s * stage_bytes);
                float4* pl = pa + kABytes / 16;
#pragma unroll
                for (int i = 0; i < kABytes / 16 / 128; ++i) {
                    const float4 v = pa[t + i * 128];
                    float4 h;
                    h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
                    h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
                    h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
                    h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
                    pa[t + i * 128] = h;
                    pl[t + i * 128] = make_float4(v.x - h.x, v.y - h.y, v.z - h.z, v.w - h.w);
                }
                // make the generic-proxy writes visible to the tensor core's async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&bar_xf[s]);
            }
        }
        if (ok) ok = mbar_wait(&bar_accum, 0);
        if (!ok) record_error(err_flag, 4);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok && !s_abort) {
            const int q = warp & 3;                       // TMEM lane quarter this warp may read
            const int row = q * 32 + lane;
            bool valid = row < rows_in_tile;
            long pix = 0;
            if (a.flat) {
                pix = (long)w0 + row;
                valid = valid && pix < a.Wo;
            } else {
                const int wi = row % a.tw, r2 = row / a.tw;
                const int hi_ = r2 % a.th, ni = r2 / a.th;
                const int ow = w0 + wi, oh = h0 + hi_, on = n0 + ni;
                valid = valid && ow < a.Wo && oh < a.Ho && on < a.N;
                pix = ((long)on * a.Ho + oh) * a.Wo + ow;
            }
            float* out = y + pix * a.Ks + a.koff;
            const float* crow = (a.bias_mode == 1) ? bias + pix * a.ldc : bias;
            const int nbase = n_tile * a.BN;
            for (int c = 0; c < a.BN; c += 16) {
                if (nbase + c >= a.Kp) break;             // uniform across the warp
                uint32_t r[16];
                const uint32_t taddr = tmem_d + ((uint32_t)(q * 32) << 16) + (uint32_t)c;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                    : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                      "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                    : "r"(taddr));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (valid) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const int n = nbase + c + g * 4;
                        if (n >= a.Kp) break;
                        float v[4];
#pragma unroll
                        for (int l = 0; l < 4; ++l) {
                            float acc = a.alpha * __uint_as_float(r[g * 4 + l]);
                            if (n + l < a.K) {
                                if (a.bias_mode) acc = fmaf(a.beta, crow[n + l], acc);
                                acc = apply_act(acc, a.act, a.lo, a.hi);
                            } else {
                                acc = 0.f;                 // padded lanes stay zero
                            }
                            v[l] = acc;
                        }
                        *reinterpret_cast<float4*>(out + n) = make_float4(v[0], v[1], v[2], v[3]);
                    }
                }
            }
        }
    }

    // ------------------------------------------------------------------ teardown
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((uint32_t)a.tmem_cols));
    }
}

// ------------------------------------------------------------------ host side
}  // namespace

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

int next_pow2(int v) { int p = 32; while (p < v) p <<= 1; return p; }

// Picks N tiling, stage count and shared memory; launches.
int launch_tc(TcArgs& t, const CUtensorMap& mA, const CUtensorMap& mBhi, const CUtensorMap& mBlo, long m_tiles,
              const float* bias, float* y, cudaStream_t s) {
    const int total = t.kernel * t.kernel * t.chunks_per_tap;
    const size_t stage = (size_t)(t.passes == 3 ? 2 : 1) * (kABytes + (size_t)t.BN * 128);
    int stages = total < 4 ? total : 4;
    // keep several blocks resident per SM where the tile is small: overlap between
    // blocks stands in for a deeper pipeline inside one
    while (stages > 2 && stage * stages > 96 * 1024) --stages;
    if (stage * stages + 1024 > 220 * 1024) return OGLE_ERR_UNSUPPORTED;
    t.stages = stages;
    t.tmem_cols = next_pow2(t.BN);
    const size_t smem = stage * stages + 1024;
    static thread_local int attr_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_device = dev;
    }
    const long blocks = m_tiles * t.n_tiles;
    if (blocks <= 0 || blocks > 0x7fffffffL) return OGLE_ERR_UNSUPPORTED;
    conv_tc_kernel<<<(unsigned)blocks, kThreads, smem, s>>>(mA, mBhi, mBlo, bias, y, t, error_flag_ptr());
    return finish_launch();
}

// 2 = persistent kernel (default), 1 = one tile per block. OGLE_TC_VARIANT overrides.
int tc_variant() {
    static int v = [] {
        const char* e = getenv("OGLE_TC_VARIANT");
        return (e && e[0] == '1') ? 1 : 2;
    }();
    return v;
}

// N tiling of the persistent kernel: multiples of 32 columns (one staging slab each).
// Picks the width that minimises (rounds of one tile per SM) x (time of a tile), with a
// tile's time modelled by its tensor-core instructions: one instruction costs about 100
// cycles up to ~180 columns (bound by the shared-memory fetch of its 128-row A operand)
// and 0.55 cycles per column beyond.
void choose_n_tiling_v2(int Kp, long m_tiles, TcArgs* t) {
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
        if (t->passes == 3) per_tile = bn <= 128 ? mma(2 * bn) + mma(bn) : 3.0 * mma(bn);
        else per_tile = mma(bn);
        const double cost = (double)rounds * per_tile;
        // equal cost: the wider tile when there are several rounds (fewer passes over A), the
        // narrower one when everything fits in one round (more SMs busy, shorter epilogues)
        if (best_cost < 0 || cost < best_cost || (cost == best_cost && rounds > 1)) { best_cost = cost; best_bn = bn; }
    }
    if (const char* e = getenv("OGLE_TC_BN")) {      // experiments: force the tile width
        const int v = atoi(e);
        if (v >= 32 && v <= 256 && v % 32 == 0 && v <= kmax) best_bn = v;
    }
    t->BN = best_bn;
    t->n_tiles = (Kp + best_bn - 1) / best_bn;
}

bool split_k_enabled() {
    static const bool v = [] { const char* e = getenv("OGLE_TC_SPLIT_K"); return !(e && e[0] == '0'); }();
    return v;
}

void choose_n_tiling(int Kp, TcArgs* t) {
    int bn = (Kp + 15) / 16 * 16;
    if (bn > 256) {
        // split evenly into tiles of at most 256 columns
        const int parts = (Kp + 255) / 256;
        bn = ((Kp + parts - 1) / parts + 15) / 16 * 16;
    }
    t->BN = bn;
    t->n_tiles = (Kp + bn - 1) / bn;
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
int launch_conv_tc(const ConvArgs& a, int variant, int math_mode, const float* x, const float* w_hi,
                   const float* w_lo, const float* bias, float* y, cudaStream_t s, float* y2, int K1,
                   int split_col) {
    TcArgs t = {};
    if (y2) {
        if (tc_variant() != 2 || split_col <= 0 || (split_col & 31) || K1 <= 0 || K1 > split_col || split_col >= a.K ||
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
    const bool v2 = tc_variant() == 2;

    CUtensorMap mA, mBhi, mBlo, mY, mY2;
    long m_tiles;
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
    } else {
        t.flat = 0;
        t.N = a.N; t.Ho = a.Ho; t.Wo = a.Wo;
        const bool may_split = v2 && a.act == OGLE_ACT_NONE && a.koff == 0 && (y2 != nullptr || a.Ks == a.Kp) &&
                               split_k_enabled() && taps * t.chunks_per_tap >= 16;
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
    if (v2) choose_n_tiling_v2(a.Kp, m_tiles, &t);
    else choose_n_tiling(a.Kp, &t);
    const int Kp128 = (a.K + 127) / 128 * 128;
    const cuuint64_t bdims[2] = {(cuuint64_t)taps * t.Cp32, (cuuint64_t)Kp128};
    const cuuint64_t bstr[1] = {(cuuint64_t)taps * t.Cp32 * 4};
    const cuuint32_t bbox[2] = {kChunk, (cuuint32_t)t.BN};
    const cuuint32_t bes[2] = {1, 1};
    if (!make_map(&mBhi, w_hi, 2, bdims, bstr, bbox, bes)) return OGLE_ERR_CUDA;
    if (!make_map(&mBlo, w_lo, 2, bdims, bstr, bbox, bes)) return OGLE_ERR_CUDA;
    if (v2) {
        // Split the reduction when whole tiles would leave SMs idle (few tiles) or a last round
        // mostly empty. Needs a linear epilogue (no activation) and outputs that may be zeroed
        // (dense tensors, not slices of a wider one): the partial tiles are added in place.
        t.split_k = 1;
        const int chunks = taps * t.chunks_per_tap;
        if (a.act == OGLE_ACT_NONE && a.koff == 0 && (y2 != nullptr || a.Ks == a.Kp) && split_k_enabled()) {
            const double tiles = (double)m_tiles * t.n_tiles;
            double best = ceil(tiles / kNumSMs);
            // two ranges at most: the sum of two partial tiles onto zero does not depend on the
            // order in which they arrive, so results stay bit-reproducible; three or more would not
            for (int k = 2; k <= 2 && chunks / k >= 8; ++k) {
                const double cost = ceil(tiles * k / kNumSMs) / k + 0.03 * (k - 1);   // + per-item fill/drain
                if (cost < 0.9 * best) { best = cost; t.split_k = k; }
            }
            const int cps = (chunks + t.split_k - 1) / t.split_k;
            while (t.split_k > 1 && (t.split_k - 1) * cps >= chunks) --t.split_k;     // no empty ranges
        }
        if (t.split_k > 1) {
            const size_t rows = (size_t)a.M;
            if (cudaMemsetAsync(y, 0, rows * (size_t)ks_a * sizeof(float), s) != cudaSuccess) return OGLE_ERR_CUDA;
            if (y2 && cudaMemsetAsync(y2, 0, rows * (size_t)kp_b * sizeof(float), s) != cudaSuccess) return OGLE_ERR_CUDA;
        }
        return launch_tc_v2(t, mA, mBhi, mBlo, mY, y2 ? mY2 : mY, m_tiles, bias, error_flag_ptr(), s);
    }
    return launch_tc(t, mA, mBhi, mBlo, m_tiles, bias, y, s);
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
    const bool v2 = tc_variant() == 2;
    const long m_tiles = (p.M + kTileM - 1) / kTileM;
    if (v2) choose_n_tiling_v2(t.Kp, m_tiles, &t);
    else choose_n_tiling(t.Kp, &t);
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
    return launch_tc(t, mA, mBhi, mBlo, m_tiles, C, Y, s);
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
