// CUDA-core (fp32 FMA) conv2d kernels:
//   - depthwise 3x3 (stride 1 or 2) and a generic depthwise loop: HBM-bound, one
//     thread owns a float4 of channels for a 2x2 patch of output pixels so the
//     overlapping input rows are reused from registers;
//   - grouped (non-depthwise) direct convolution: scalar, rarely used;
//   - dense implicit GEMM for group == 1 in OGLE_MATH_FP32 mode and for layers
//     whose reduction is too short for the tensor-core pipeline (the RGB stem).
#include "conv_args.cuh"

namespace ogle {

bool dw_tma_supported(const ConvArgs& a);
int launch_dw_tma(const ConvArgs& a, const float* x, const float* w, const float* bias, float* y, cudaStream_t s);

// Bias holds exactly K floats; lanes past K read as zero.
__device__ __forceinline__ float4 load_bias4(const float* bias, int c, int K, int has_bias) {
    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has_bias) {
        if (c + 0 < K) b.x = bias[c + 0];
        if (c + 1 < K) b.y = bias[c + 1];
        if (c + 2 < K) b.z = bias[c + 2];
        if (c + 3 < K) b.w = bias[c + 3];
    }
    return b;
}

// ---------------------------------------------------------------- depthwise
template <int S>
__global__ void __launch_bounds__(128)
dw3x3_kernel(const float4* __restrict__ x, const float4* __restrict__ w, const float* __restrict__ bias,
             float4* __restrict__ y, ConvArgs a) {
    constexpr int K = 3, TY = 2, TX = 2;
    constexpr int PH = (TY - 1) * S + K, PW = (TX - 1) * S + K;
    const int C4 = a.Kp >> 2, in_q = a.Cs >> 2, out_q = a.Ks >> 2, off_q = a.koff >> 2;
    const int gy = (a.Ho + TY - 1) / TY, gx = (a.Wo + TX - 1) / TX;
    const long total = (long)a.N * gy * gx * C4;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        const int c4 = int(t % C4); t /= C4;
        const int px = int(t % gx); t /= gx;
        const int py = int(t % gy); t /= gy;
        const int n = int(t);
        const int oy0 = py * TY, ox0 = px * TX;
        const int iy0 = oy0 * S - a.pad, ix0 = ox0 * S - a.pad;
        float4 wk[9];
#pragma unroll
        for (int k = 0; k < 9; ++k) wk[k] = w[k * C4 + c4];
        const float4 b = load_bias4(bias, c4 * 4, a.K, a.has_bias);
        float4 acc[TY][TX];
#pragma unroll
        for (int ty = 0; ty < TY; ++ty)
#pragma unroll
            for (int tx = 0; tx < TX; ++tx) acc[ty][tx] = b;
#pragma unroll
        for (int r = 0; r < PH; ++r) {
            const int iy = iy0 + r;
            if (iy < 0 || iy >= a.H) continue;  // zero padding: skipped taps add nothing
            const float4* row = x + ((long)n * a.H + iy) * a.W * in_q + c4;
            float4 v[PW];
#pragma unroll
            for (int c = 0; c < PW; ++c) {
                const int ix = ix0 + c;
                v[c] = (ix >= 0 && ix < a.W) ? row[(long)ix * in_q] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int ty = 0; ty < TY; ++ty) {
                if (r < ty * S || r >= ty * S + K) continue;
                const int ky = r - ty * S;
#pragma unroll
                for (int tx = 0; tx < TX; ++tx)
#pragma unroll
                    for (int kx = 0; kx < K; ++kx) {
                        const float4 f = wk[ky * 3 + kx];
                        const float4 u = v[tx * S + kx];
                        acc[ty][tx].x = fmaf(f.x, u.x, acc[ty][tx].x);
                        acc[ty][tx].y = fmaf(f.y, u.y, acc[ty][tx].y);
                        acc[ty][tx].z = fmaf(f.z, u.z, acc[ty][tx].z);
                        acc[ty][tx].w = fmaf(f.w, u.w, acc[ty][tx].w);
                    }
            }
        }
#pragma unroll
        for (int ty = 0; ty < TY; ++ty)
#pragma unroll
            for (int tx = 0; tx < TX; ++tx) {
                const int oy = oy0 + ty, ox = ox0 + tx;
                if (oy >= a.Ho || ox >= a.Wo) continue;
                float4 r = apply_act4(acc[ty][tx], a.act, a.lo, a.hi);
                // lanes past K stay zero (their weights and bias are zero; a clip
                // with lo > 0 must not lift them)
                const int c = c4 * 4;
                if (c >= a.K) r.x = 0.f;
                if (c + 1 >= a.K) r.y = 0.f;
                if (c + 2 >= a.K) r.z = 0.f;
                if (c + 3 >= a.K) r.w = 0.f;
                y[(((long)n * a.Ho + oy) * a.Wo + ox) * out_q + off_q + c4] = r;
            }
    }
}


// Any kernel size / dilation / stride, depthwise.
__global__ void dw_generic_kernel(const float4* __restrict__ x, const float4* __restrict__ w,
                                  const float* __restrict__ bias, float4* __restrict__ y, ConvArgs a) {
    const int C4 = a.Kp >> 2, in_q = a.Cs >> 2, out_q = a.Ks >> 2, off_q = a.koff >> 2;
    const long total = a.M * C4;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        const int c4 = int(t % C4); t /= C4;
        const int ox = int(t % a.Wo); t /= a.Wo;
        const int oy = int(t % a.Ho); t /= a.Ho;
        const int n = int(t);
        float4 acc = load_bias4(bias, c4 * 4, a.K, a.has_bias);
        for (int ky = 0; ky < a.kernel; ++ky)
            for (int kx = 0; kx < a.kernel; ++kx) {
                const int iy = oy * a.stride + ky * a.dil - a.pad, ix = ox * a.stride + kx * a.dil - a.pad;
                if (iy < 0 || iy >= a.H || ix < 0 || ix >= a.W) continue;
                const float4 u = x[(((long)n * a.H + iy) * a.W + ix) * in_q + c4];
                const float4 f = w[(ky * a.kernel + kx) * C4 + c4];
                acc.x = fmaf(f.x, u.x, acc.x); acc.y = fmaf(f.y, u.y, acc.y);
                acc.z = fmaf(f.z, u.z, acc.z); acc.w = fmaf(f.w, u.w, acc.w);
            }
        float4 r = apply_act4(acc, a.act, a.lo, a.hi);
        const int c = c4 * 4;
        if (c >= a.K) r.x = 0.f;
        if (c + 1 >= a.K) r.y = 0.f;
        if (c + 2 >= a.K) r.z = 0.f;
        if (c + 3 >= a.K) r.w = 0.f;
        y[(((long)n * a.Ho + oy) * a.Wo + ox) * out_q + off_q + c4] = r;
    }
}

// ------------------------------------------------------------------ grouped
// One thread per output scalar; packed filter [tap][Cp][Kp] with Cp = round_up(C/group,4).
__global__ void grouped_kernel(const float* __restrict__ x, const float* __restrict__ w,
                               const float* __restrict__ bias, float* __restrict__ y, ConvArgs a) {
    const long total = a.M * a.Kp;
    const int Cg = a.C / a.group, Kg = a.K / a.group;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        const int k = int(t % a.Kp); t /= a.Kp;
        const int ox = int(t % a.Wo); t /= a.Wo;
        const int oy = int(t % a.Ho); t /= a.Ho;
        const int n = int(t);
        float r = 0.f;
        if (k < a.K) {
            const int g = k / Kg;
            float acc = 0.f;
            for (int ky = 0; ky < a.kernel; ++ky)
                for (int kx = 0; kx < a.kernel; ++kx) {
                    const int iy = oy * a.stride + ky * a.dil - a.pad, ix = ox * a.stride + kx * a.dil - a.pad;
                    if (iy < 0 || iy >= a.H || ix < 0 || ix >= a.W) continue;
                    const float* px = x + (((long)n * a.H + iy) * a.W + ix) * a.Cs + g * Cg;
                    const float* pw = w + (long)(ky * a.kernel + kx) * a.Cp * a.Kp + k;
                    for (int c = 0; c < Cg; ++c) acc = fmaf(px[c], pw[(long)c * a.Kp], acc);
                }
            acc += a.has_bias ? bias[k] : 0.f;
            r = apply_act(acc, a.act, a.lo, a.hi);
        }
        y[(((long)n * a.Ho + oy) * a.Wo + ox) * a.Ks + a.koff + k] = r;
    }
}

// ------------------------------------------------------- dense implicit GEMM
// D[m][k] = sum_r A[m][r] * B[r][k]; m = output pixel, r = (tap, channel),
// A gathered from the NHWC4 input with zero fill outside the image,
// B = tap-major packed filter [taps*Cp][Kp].
template <int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
conv_igemm_kernel(const float* __restrict__ x, const float* __restrict__ wp,
                  const float* __restrict__ bias, float* __restrict__ y, ConvArgs a) {
    constexpr int BK = 16;
    constexpr int NT = (BM / TM) * (BN / TN);
    constexpr int A_LD = BM * (BK / 4) / NT;       // float4 loads of A per thread per tile
    constexpr int B_F4 = BK * BN / 4;              // float4s in a B tile
    constexpr int B_LD = (B_F4 + NT - 1) / NT;
    static_assert(BM * (BK / 4) % NT == 0, "A tile must divide over the threads");
    static_assert(TM % 4 == 0 && TN == 4, "register tile shape");

    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN];

    const int tid = threadIdx.x;
    const long m0 = (long)blockIdx.x * BM;
    const int n0 = blockIdx.y * BN;
    const int R = a.kernel * a.kernel * a.Cp;   // reduction length, multiple of 4
    const int ntiles = (R + BK - 1) / BK;

    // per-thread A rows (fixed for the whole reduction)
    int a_row[A_LD], a_kq[A_LD], a_iy0[A_LD], a_ix0[A_LD];
    long a_img[A_LD];
    bool a_ok[A_LD];
#pragma unroll
    for (int j = 0; j < A_LD; ++j) {
        const int idx = tid + j * NT;
        a_row[j] = idx >> 2;
        a_kq[j] = idx & 3;
        const long m = m0 + a_row[j];
        a_ok[j] = m < a.M;
        const long mm = a_ok[j] ? m : 0;
        const int ox = int(mm % a.Wo);
        const long t = mm / a.Wo;
        const int oy = int(t % a.Ho);
        const long n = t / a.Ho;
        a_iy0[j] = oy * a.stride - a.pad;
        a_ix0[j] = ox * a.stride - a.pad;
        a_img[j] = n * a.H;
    }

    float4 ra[A_LD], rb[B_LD];
    auto load_tile = [&](int kt) {
#pragma unroll
        for (int j = 0; j < A_LD; ++j) {
            const int r = kt * BK + a_kq[j] * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (a_ok[j] && r < R) {
                const int tap = r / a.Cp, c = r - tap * a.Cp;
                const int ky = tap / a.kernel, kx = tap - ky * a.kernel;
                const int iy = a_iy0[j] + ky * a.dil, ix = a_ix0[j] + kx * a.dil;
                if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W && c < a.Cs)
                    v = *reinterpret_cast<const float4*>(x + ((a_img[j] + iy) * a.W + ix) * a.Cs + c);
            }
            ra[j] = v;
        }
#pragma unroll
        for (int j = 0; j < B_LD; ++j) {
            const int idx = tid + j * NT;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (idx < B_F4) {
                const int kr = idx / (BN / 4), nc = (idx % (BN / 4)) * 4;
                const int r = kt * BK + kr;
                if (r < R && n0 + nc < a.Kp)
                    v = *reinterpret_cast<const float4*>(wp + (long)r * a.Kp + n0 + nc);
            }
            rb[j] = v;
        }
    };
    auto store_tile = [&](int buf) {
#pragma unroll
        for (int j = 0; j < A_LD; ++j) {
            const int k = a_kq[j] * 4;
            As[buf][k + 0][a_row[j]] = ra[j].x;
            As[buf][k + 1][a_row[j]] = ra[j].y;
            As[buf][k + 2][a_row[j]] = ra[j].z;
            As[buf][k + 3][a_row[j]] = ra[j].w;
        }
#pragma unroll
        for (int j = 0; j < B_LD; ++j) {
            const int idx = tid + j * NT;
            if (idx < B_F4) {
                const int kr = idx / (BN / 4), nc = (idx % (BN / 4)) * 4;
                *reinterpret_cast<float4*>(&Bs[buf][kr][nc]) = rb[j];
            }
        }
    };

    const int ty = tid / (BN / TN), tx = tid % (BN / TN);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    load_tile(0);
    store_tile(0);
    __syncthreads();
    for (int kt = 0; kt < ntiles; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < ntiles) load_tile(kt + 1);
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float av[TM];
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                const float4 t4 = *reinterpret_cast<const float4*>(&As[buf][k][ty * TM + i]);
                av[i] = t4.x; av[i + 1] = t4.y; av[i + 2] = t4.z; av[i + 3] = t4.w;
            }
            const float4 b4 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * TN]);
            const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        if (kt + 1 < ntiles) {
            store_tile(buf ^ 1);
            __syncthreads();
        }
    }

    const int nc = n0 + tx * TN;
    if (nc >= a.Kp) return;
    const float4 b = load_bias4(bias, nc, a.K, a.has_bias);
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long m = m0 + ty * TM + i;
        if (m >= a.M) continue;
        float4 r = make_float4(acc[i][0] + b.x, acc[i][1] + b.y, acc[i][2] + b.z, acc[i][3] + b.w);
        r = apply_act4(r, a.act, a.lo, a.hi);
        if (nc + 0 >= a.K) r.x = 0.f;
        if (nc + 1 >= a.K) r.y = 0.f;
        if (nc + 2 >= a.K) r.z = 0.f;
        if (nc + 3 >= a.K) r.w = 0.f;
        *reinterpret_cast<float4*>(y + m * a.Ks + a.koff + nc) = r;
    }
}

bool conv_smallc_supported(const ConvArgs& a);
int launch_conv_smallc(const ConvArgs& a, const float* x, const float* w_tap_major, const float* bias, float* y,
                       cudaStream_t s);

int launch_conv_simt(const ConvArgs& a, int variant, const float* x, const float* w,
                     const float* bias, float* y, cudaStream_t s) {
    if (variant == CONV_DEPTHWISE) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        const float4* w4 = reinterpret_cast<const float4*>(w);
        const float* b4 = bias;
        float4* y4 = reinterpret_cast<float4*>(y);
        const int C4 = a.Kp / 4;
        if (dw_tma_supported(a)) {
            return launch_dw_tma(a, x, w, bias, y, s);
        } else if (a.kernel == 3 && a.dil == 1 && (a.stride == 1 || a.stride == 2)) {
            const long items = (long)a.N * ((a.Ho + 1) / 2) * ((a.Wo + 1) / 2) * C4;
            if (a.stride == 1) dw3x3_kernel<1><<<grid_for(items, 128, 16), 128, 0, s>>>(x4, w4, b4, y4, a);
            else dw3x3_kernel<2><<<grid_for(items, 128, 16), 128, 0, s>>>(x4, w4, b4, y4, a);
        } else {
            dw_generic_kernel<<<grid_for(a.M * C4, 256), 256, 0, s>>>(x4, w4, b4, y4, a);
        }
        return finish_launch();
    }
    if (variant == CONV_GROUPED) {
        grouped_kernel<<<grid_for(a.M * a.Kp, 256), 256, 0, s>>>(x, w, bias, y, a);
        return finish_launch();
    }
    if (variant == CONV_GENERAL && conv_smallc_supported(a)) return launch_conv_smallc(a, x, w, bias, y, s);
    if (a.Kp <= 32) {
        dim3 grid(div_up(a.M, 128), div_up(a.Kp, 32));
        conv_igemm_kernel<128, 32, 4, 4><<<grid, 256, 0, s>>>(x, w, bias, y, a);
    } else {
        dim3 grid(div_up(a.M, 128), div_up(a.Kp, 64));
        conv_igemm_kernel<128, 64, 8, 4><<<grid, 256, 0, s>>>(x, w, bias, y, a);
    }
    return finish_launch();
}

}  // namespace ogle
