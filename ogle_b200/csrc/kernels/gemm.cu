// Gemm: Y[M,N] = alpha * A[M,K] * (transB ? B[N,K]^T : B[K,N]) + beta * C.
// OGLE_MATH_FP32 runs the register-tiled CUDA-core kernel below; the TF32 modes
// go to the tcgen05 path when the shape allows it.
#include <cuda_bf16.h>

#include "common.cuh"

namespace ogle {

int launch_gemm_tc(const OgleGemmParams& p, const float* A, const float* B, const float* C,
                   float* Y, cudaStream_t s);
bool gemm_tc_supported(const OgleGemmParams& p, const float* A, const float* B);
int launch_gemm_tc_packed(const OgleGemmParams& p, const float* A, const float* Bhi, const float* Blo,
                          const float* C, float* Y, cudaStream_t s);

// B [K][ldb] (or [N][ldb] when transB) -> two K-major sections of [round_up(N,128)][round_up(K,32)]
// 4-byte slots each: the fp32 values with the low 13 mantissa bits cleared (operand of the TF32
// pass), and per 32-element chunk of a row the 64 bf16 values [b_lo x 32 | b x 32] (operand of
// the BF16 cross-term pass, against [a_hi | a_lo]).
__global__ void gemm_pack_b_kernel(const float* __restrict__ B, float* __restrict__ hi, __nv_bfloat16* __restrict__ cross,
                                   int K, int N, int ldb, int transB, int Kp32, int Np128) {
    const long total = (long)Np128 * Kp32;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const int k = int(i % Kp32), n = int(i / Kp32);
        float v = 0.f;
        if (k < K && n < N) v = transB ? B[(long)n * ldb + k] : B[(long)k * ldb + n];
        const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        hi[i] = h;
        const long chunk = (long)n * Kp32 + (k & ~31);        // first slot of this 32-element chunk
        cross[chunk * 2 + (k & 31)] = __float2bfloat16_rn(v - h);
        cross[chunk * 2 + 32 + (k & 31)] = __float2bfloat16_rn(v);
    }
}

template <bool TRANSB>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ C,
                 float* __restrict__ Y, OgleGemmParams p) {
    constexpr int BM = 128, BN = 64, BK = 16, TM = 8, TN = 4, NT = 256;
    __shared__ __align__(16) float As[2][BK][BM + 4];
    __shared__ __align__(16) float Bs[2][BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
    const int ntiles = (p.K + BK - 1) / BK;

    float4 ra[2], rb;
    // A: 128 rows x 4 float4 per tile; B (no trans): 16 rows x 16 float4; B (trans): 64 rows x 4 float4
    auto load_tile = [&](int kt) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int idx = tid + j * NT;
            const int row = idx >> 2, kq = idx & 3;
            const int m = m0 + row, k = kt * BK + kq * 4;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < p.M && k < p.K) {
                const float* src = A + (long)m * p.lda + k;
                if (k + 3 < p.K) v = *reinterpret_cast<const float4*>(src);
                else { v.x = src[0]; if (k + 1 < p.K) v.y = src[1]; if (k + 2 < p.K) v.z = src[2]; }
            }
            ra[j] = v;
        }
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (!TRANSB) {
            const int kr = tid >> 4, nc = (tid & 15) * 4;
            const int k = kt * BK + kr, n = n0 + nc;
            if (k < p.K && n < p.N) {
                const float* src = B + (long)k * p.ldb + n;
                if (n + 3 < p.N) v = *reinterpret_cast<const float4*>(src);
                else { v.x = src[0]; if (n + 1 < p.N) v.y = src[1]; if (n + 2 < p.N) v.z = src[2]; }
            }
        } else {
            const int row = tid >> 2, kq = tid & 3;
            const int n = n0 + row, k = kt * BK + kq * 4;
            if (n < p.N && k < p.K) {
                const float* src = B + (long)n * p.ldb + k;
                if (k + 3 < p.K) v = *reinterpret_cast<const float4*>(src);
                else { v.x = src[0]; if (k + 1 < p.K) v.y = src[1]; if (k + 2 < p.K) v.z = src[2]; }
            }
        }
        rb = v;
    };
    auto store_tile = [&](int buf) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int idx = tid + j * NT;
            const int row = idx >> 2, k = (idx & 3) * 4;
            As[buf][k + 0][row] = ra[j].x; As[buf][k + 1][row] = ra[j].y;
            As[buf][k + 2][row] = ra[j].z; As[buf][k + 3][row] = ra[j].w;
        }
        if (!TRANSB) {
            const int kr = tid >> 4, nc = (tid & 15) * 4;
            *reinterpret_cast<float4*>(&Bs[buf][kr][nc]) = rb;
        } else {
            const int row = tid >> 2, k = (tid & 3) * 4;
            Bs[buf][k + 0][row] = rb.x; Bs[buf][k + 1][row] = rb.y;
            Bs[buf][k + 2][row] = rb.z; Bs[buf][k + 3][row] = rb.w;
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
            const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][ty * TM]);
            const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][ty * TM + 4]);
            const float4 b4 = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * TN]);
            const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
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
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = nc + j;
            if (n >= p.ldy) continue;
            float v = 0.f;   // pad lanes n in [N, ldy) are written as zero
            if (n < p.N) {
                v = p.alpha * acc[i][j];
                if (p.bias_mode == 1) v = fmaf(p.beta, C[(long)m * p.ldc + n], v);
                else if (p.bias_mode == 2) v = fmaf(p.beta, C[n], v);
            }
            Y[(long)m * p.ldy + n] = v;
        }
    }
}

}  // namespace ogle

using namespace ogle;

static int normalize_gemm(OgleGemmParams* p) {
    if (p->M <= 0 || p->K <= 0 || p->N <= 0) return OGLE_ERR_INVALID;
    if (p->lda == 0) p->lda = up4(p->K);
    if (p->ldb == 0) p->ldb = p->transB ? up4(p->K) : up4(p->N);
    if (p->ldy == 0) p->ldy = up4(p->N);
    if (p->ldc == 0) p->ldc = up4(p->N);
    if (p->lda < p->K || p->ldy < p->N || p->ldb < (p->transB ? p->K : p->N)) return OGLE_ERR_INVALID;
    if ((p->lda & 3) || (p->ldb & 3) || (p->ldy & 3)) return OGLE_ERR_ALIGNMENT;
    if (p->bias_mode < 0 || p->bias_mode > 2) return OGLE_ERR_INVALID;
    if (p->bias_mode == 1 && p->ldc < p->N) return OGLE_ERR_INVALID;
    if (p->math_mode < OGLE_MATH_FP32 || p->math_mode > OGLE_MATH_TF32X3) return OGLE_ERR_INVALID;
    return OGLE_OK;
}

extern "C" size_t ogle_cuda_gemm_packed_b_bytes(const OgleGemmParams* pp) {
    if (!pp) return 0;
    OgleGemmParams p = *pp;
    if (normalize_gemm(&p) != OGLE_OK) return 0;
    const size_t half = size_t((p.N + 127) / 128 * 128) * size_t((p.K + 31) / 32 * 32) * sizeof(float);
    return 2 * ((half + 255) / 256 * 256);
}

extern "C" int ogle_cuda_gemm_pack_b(const OgleGemmParams* pp, const float* B, void* packed, ogle_stream_t stream) {
    if (!pp || !B || !packed) return OGLE_ERR_INVALID;
    OgleGemmParams p = *pp;
    int rc = normalize_gemm(&p);
    if (rc != OGLE_OK) return rc;
    if (!aligned16(packed)) return OGLE_ERR_ALIGNMENT;
    const int Kp32 = (p.K + 31) / 32 * 32, Np128 = (p.N + 127) / 128 * 128;
    const size_t half = (size_t(Np128) * Kp32 * sizeof(float) + 255) / 256 * 256;
    float* hi = static_cast<float*>(packed);
    float* lo = reinterpret_cast<float*>(static_cast<char*>(packed) + half);
    gemm_pack_b_kernel<<<grid_for((long)Np128 * Kp32, 256), 256, 0, (cudaStream_t)stream>>>(B, hi, reinterpret_cast<__nv_bfloat16*>(lo), p.K, p.N, p.ldb,
                                                                                            p.transB, Kp32, Np128);
    return finish_launch();
}

extern "C" int ogle_cuda_gemm_packed(const OgleGemmParams* pp, const float* A, const void* packed_b, const float* C,
                                     float* Y, ogle_stream_t stream) {
    if (!pp || !A || !packed_b || !Y) return OGLE_ERR_INVALID;
    OgleGemmParams p = *pp;
    int rc = normalize_gemm(&p);
    if (rc != OGLE_OK) return rc;
    if (p.bias_mode && !C) return OGLE_ERR_INVALID;
    if (p.math_mode == OGLE_MATH_FP32) return OGLE_ERR_INVALID;
    if (!aligned16(A) || !aligned16(Y) || !aligned16(packed_b)) return OGLE_ERR_ALIGNMENT;
    const int Kp32 = (p.K + 31) / 32 * 32, Np128 = (p.N + 127) / 128 * 128;
    const size_t half = (size_t(Np128) * Kp32 * sizeof(float) + 255) / 256 * 256;
    const float* hi = static_cast<const float*>(packed_b);
    const float* lo = reinterpret_cast<const float*>(static_cast<const char*>(packed_b) + half);
    return launch_gemm_tc_packed(p, A, hi, lo, C, Y, (cudaStream_t)stream);
}

extern "C" int ogle_cuda_gemm_ws(const OgleGemmParams* pp, const float* A, const float* B, const float* C, float* Y,
                                 void* workspace, size_t workspace_bytes, ogle_stream_t stream) {
    if (!pp) return OGLE_ERR_INVALID;
    if (pp->math_mode == OGLE_MATH_FP32) return ogle_cuda_gemm(pp, A, B, C, Y, stream);
    const size_t need = ogle_cuda_gemm_packed_b_bytes(pp);
    if (need == 0) return OGLE_ERR_INVALID;
    if (!workspace || workspace_bytes < need) return OGLE_ERR_INVALID;
    int rc = ogle_cuda_gemm_pack_b(pp, B, workspace, stream);
    if (rc != OGLE_OK) return rc;
    return ogle_cuda_gemm_packed(pp, A, workspace, C, Y, stream);
}

extern "C" int ogle_cuda_gemm(const OgleGemmParams* pp, const float* A, const float* B, const float* C,
                              float* Y, ogle_stream_t stream) {
    if (!pp || !A || !B || !Y) return OGLE_ERR_INVALID;
    OgleGemmParams p = *pp;
    int rc0 = normalize_gemm(&p);
    if (rc0 != OGLE_OK) return rc0;
    if (p.bias_mode && !C) return OGLE_ERR_INVALID;
    if (!aligned16(A) || !aligned16(B) || !aligned16(Y)) return OGLE_ERR_ALIGNMENT;
    cudaStream_t s = (cudaStream_t)stream;
    if (p.math_mode != OGLE_MATH_FP32 && gemm_tc_supported(p, A, B)) return launch_gemm_tc(p, A, B, C, Y, s);
    dim3 grid(div_up(p.M, 128), div_up(p.ldy, 64));
    if (p.transB) gemm_simt_kernel<true><<<grid, 256, 0, s>>>(A, B, C, Y, p);
    else gemm_simt_kernel<false><<<grid, 256, 0, s>>>(A, B, C, Y, p);
    return finish_launch();
}
