// Argument block and packed-filter layout shared by the conv2d kernels.
#pragma once
#include "common.cuh"

namespace ogle {

enum ConvVariant { CONV_GENERAL = 0, CONV_POINTWISE = 1, CONV_DEPTHWISE = 2, CONV_GROUPED = 3 };

struct ConvArgs {
    int N, H, W, C, Cs;        // input: channels and channel stride (floats per pixel)
    int Ho, Wo, K, Ks, koff;   // output: channels, channel stride, first channel offset
    int kernel, stride, pad, dil, group;
    int Cp, Kp;                // packed filter extents: round_up(C/group,4), round_up(K,4)
    int act;                   // effective activation after the per-variant quirks
    float lo, hi;
    int has_bias;
    long M;                    // N*Ho*Wo output pixels
    int n_tile;                // requested output channels per tile of the tensor-core path (0 = choose)
    int split;                 // requested number of reduction ranges (0 = choose)
    int on_m;                  // channels-on-M form of the tensor-core path: 0 = choose (off), 1 = no, 2 = where it can run
    int pair;                  // two-SM form of the tensor-core path: 0 = choose, 1 = no, 2 = where it can run
};

// Packed filter blob, in this order (all sections 256-byte aligned):
//   section 0  "tap-major"  [kernel*kernel][Cp][Kp] fp32, zero padded: read by the
//              CUDA-core kernels with the output channel fastest, so that a warp's
//              weight loads are contiguous. For depthwise Cp == 1: [taps][Kp].
//   section 1  "k-major hi" [Kp128][kernel*kernel][Cp32] fp32 with the low 13
//              mantissa bits cleared: B operand of the tcgen05 path (TMA tiles of
//              128 output channels x 32 reduction elements).
//   section 2  "k-major cross" same size: per 32-channel chunk of a row, 64 bf16 values
//              [w - hi(w) x 32 | w x 32]: B operand of the BF16 cross-term pass of the
//              split mode (against [a_hi | a_lo]); moved by TMA as 128-byte rows like section 1.
// Sections 1 and 2 exist only for group == 1.
struct FilterLayout {
    size_t tap_major_bytes, kmajor_bytes;   // one k-major section
    size_t off_hi, off_lo, total;
    int Kp128, Cp32;
};

inline size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// k x k filters (k = 3, 5, 7) over at most four input channels (an RGB stem) keep their k-major
// sections in the compact form [Kp128][cols]: column (ky * k + kx) * Cg + c, zero padded to
// cols = a multiple of 32 - matching the operand the tensor-core kernel gathers for such layers.
inline bool filter_compact(int Cg, int kernel, int group) {
    return group == 1 && Cg <= 4 && (kernel == 3 || kernel == 5 || kernel == 7) && kernel * kernel * Cg <= 224;
}
inline int filter_compact_cols(int Cg, int kernel) { return (kernel * kernel * Cg + 31) / 32 * 32; }

inline FilterLayout filter_layout(int K, int Cg, int kernel, int group, int Cp) {
    FilterLayout L;
    const int taps = kernel * kernel;
    L.tap_major_bytes = align256(size_t(taps) * Cp * up4(K) * sizeof(float));
    L.Kp128 = (K + 127) / 128 * 128;
    L.Cp32 = (Cg + 31) / 32 * 32;
    L.kmajor_bytes = group == 1 ? align256(size_t(L.Kp128) * taps * L.Cp32 * sizeof(float)) : 0;
    if (filter_compact(Cg, kernel, group))
        L.kmajor_bytes = align256(size_t(L.Kp128) * filter_compact_cols(Cg, kernel) * sizeof(float));
    L.off_hi = L.tap_major_bytes;
    L.off_lo = L.off_hi + L.kmajor_bytes;
    L.total = L.off_lo + L.kmajor_bytes;
    return L;
}

// Entry points of the individual translation units.
int launch_conv_simt(const ConvArgs& a, int variant, const float* x, const float* w_tap_major,
                     const float* bias, float* y, cudaStream_t s);

}  // namespace ogle
