// Direct 3x3 convolution for inputs of at most four channels (the RGB stem of an image
// network: 3 -> 32 channels, stride 2). With so few input channels the implicit-GEMM
// kernels waste their tiles on padding; here the work is laid out for the memory system
// instead: the layer moves 16 bytes in and (at stride 2) 32 bytes out per input pixel and
// is bound by HBM once the arithmetic (27 multiply-adds per output value) is kept on
// registers.
//
// One thread computes two horizontally adjacent output pixels x eight output channels:
// the input patch (3 rows x 3 + stride columns, one float4 per pixel) sits in registers,
// the filter [tap][c][K] in shared memory is read as 128-bit vectors that serve both
// pixels, and the threads that share a pixel pair read the same input addresses (one
// transaction). A warp writes 128-byte output rows of 32 channels in full sectors.
#include "conv_args.cuh"

namespace ogle {

namespace {

template <int S>
__global__ void __launch_bounds__(256)
conv3x3_smallc_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                      float* __restrict__ y, const ConvArgs a, const int kgroups, const long items) {
    extern __shared__ float4 s_w4[];                 // [9][C][Kp] floats, then [Kp] bias
    float* s_w = reinterpret_cast<float*>(s_w4);
    const int wn = 9 * a.C * a.Kp;
    for (int i = threadIdx.x; i < wn; i += blockDim.x) {
        const int k = i % a.Kp, c = (i / a.Kp) % a.C, tap = i / (a.Kp * a.C);
        s_w[i] = w[(tap * a.Cp + c) * a.Kp + k];     // tap-major packed filter, channels past C dropped
    }
    for (int i = threadIdx.x; i < a.Kp; i += blockDim.x) s_w[wn + i] = (a.has_bias && i < a.K) ? bias[i] : 0.f;
    __syncthreads();

    constexpr int PW = 3 + S;                         // patch columns for two outputs
    const int wpairs = (a.Wo + 1) / 2;
    const long item = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= items) return;
    long t = item;
    const int kg = int(t % kgroups); t /= kgroups;
    const int wp = int(t % wpairs); t /= wpairs;
    const int ho = int(t % a.Ho);
    const int n = int(t / a.Ho);
    const int wo = wp * 2;
    const int iy0 = ho * S - a.pad, ix0 = wo * S - a.pad;

    float acc[2][8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { acc[0][j] = s_w[wn + kg * 8 + j]; acc[1][j] = acc[0][j]; }

#pragma unroll
    for (int r = 0; r < 3; ++r) {
        const int iy = iy0 + r;
        float4 p[PW];
#pragma unroll
        for (int cidx = 0; cidx < PW; ++cidx) {
            const int ix = ix0 + cidx;
            p[cidx] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (iy >= 0 && iy < a.H && ix >= 0 && ix < a.W)
                p[cidx] = __ldg(reinterpret_cast<const float4*>(x + (((long)n * a.H + iy) * a.W + ix) * a.Cs));
        }
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
            const float* wt = s_w + ((r * 3 + kx) * a.C) * a.Kp + kg * 8;
            const float u0[4] = {p[kx].x, p[kx].y, p[kx].z, p[kx].w};
            const float u1[4] = {p[kx + S].x, p[kx + S].y, p[kx + S].z, p[kx + S].w};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                if (c < a.C) {
                    const float4 f0 = *reinterpret_cast<const float4*>(wt + c * a.Kp);
                    const float4 f1 = *reinterpret_cast<const float4*>(wt + c * a.Kp + 4);
                    const float f[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        acc[0][j] = fmaf(f[j], u0[c], acc[0][j]);
                        acc[1][j] = fmaf(f[j], u1[c], acc[1][j]);
                    }
                }
            }
        }
    }

#pragma unroll
    for (int px = 0; px < 2; ++px) {
        if (wo + px >= a.Wo) continue;
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            v[j] = apply_act(acc[px][j], a.act, a.lo, a.hi);
            if (kg * 8 + j >= a.K) v[j] = 0.f;       // padded lanes stay zero
        }
        float* dst = y + (((long)n * a.Ho + ho) * a.Wo + wo + px) * a.Ks + a.koff + kg * 8;
        *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
}

}  // namespace

bool conv_smallc_supported(const ConvArgs& a) {
    return a.group == 1 && a.kernel == 3 && a.dil == 1 && (a.stride == 1 || a.stride == 2) && a.C <= 4 && a.Cp == 4 &&
           (a.Cs & 3) == 0 && (a.Kp == 8 || a.Kp == 16 || a.Kp == 32 || a.Kp == 64);
}

int launch_conv_smallc(const ConvArgs& a, const float* x, const float* w_tap_major, const float* bias, float* y,
                       cudaStream_t s) {
    const int kgroups = a.Kp / 8;
    const long items = (long)a.N * a.Ho * ((a.Wo + 1) / 2) * kgroups;
    const long blocks = (items + 255) / 256;
    if (blocks > 0x7fffffffL) return OGLE_ERR_UNSUPPORTED;
    const size_t smem = (size_t)(9 * a.C * a.Kp + a.Kp) * sizeof(float);
    if (a.stride == 1) conv3x3_smallc_kernel<1><<<(unsigned)blocks, 256, smem, s>>>(x, w_tap_major, bias, y, a, kgroups, items);
    else conv3x3_smallc_kernel<2><<<(unsigned)blocks, 256, smem, s>>>(x, w_tap_major, bias, y, a, kgroups, items);
    return finish_launch();
}

}  // namespace ogle
