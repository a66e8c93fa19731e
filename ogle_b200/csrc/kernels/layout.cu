// Layout conversion and glue kernels: pad/unpad of the last dimension to 4,
// NCHW -> NHWC4, 4-D transpose, reshape and concat. All are pure data movement
// (HBM-bound); none needs shared memory.
#include "common.cuh"

namespace ogle {

// [rows][last] dense -> [rows][stride], zero fill. One thread per output float4.
__global__ void pad4_kernel(const float* __restrict__ src, float* __restrict__ dst,
                            long rows, int last, int stride) {
    grid_dependency_trigger();
    grid_dependency_wait();
    const int q = stride >> 2;
    const long total = rows * q;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const long r = q == 1 ? i : i / q;      // RGB -> RGB0: one vector per row, no division
        const int c = int(i - r * q) * 4;
        const float* s = src + r * last + c;
        float4 v;
        v.x = c + 0 < last ? s[0] : 0.f;
        v.y = c + 1 < last ? s[1] : 0.f;
        v.z = c + 2 < last ? s[2] : 0.f;
        v.w = c + 3 < last ? s[3] : 0.f;
        reinterpret_cast<float4*>(dst)[i] = v;
    }
}

// [rows][stride] -> [rows][last] dense. One thread per output element.
__global__ void unpad4_kernel(const float* __restrict__ src, float* __restrict__ dst,
                              long rows, int last, int stride) {
    const long total = rows * last;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const long r = i / last;
        const int c = int(i - r * last);
        dst[i] = src[r * stride + c];
    }
}

__global__ void nchw_to_nhwc4_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                     int N, int C, int H, int W) {
    const int c4n = (C + 3) >> 2;
    const long total = (long)N * H * W * c4n;
    const long hw = (long)H * W;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const int c4 = int(i % c4n);
        const long p = i / c4n;       // n*H*W + h*W + w
        const long n = p / hw;
        const long s = p - n * hw;
        const float* b = src + (n * C + c4 * 4) * hw + s;
        float4 v;
        v.x = c4 * 4 + 0 < C ? b[0] : 0.f;
        v.y = c4 * 4 + 1 < C ? b[hw] : 0.f;
        v.z = c4 * 4 + 2 < C ? b[2 * hw] : 0.f;
        v.w = c4 * 4 + 3 < C ? b[3 * hw] : 0.f;
        reinterpret_cast<float4*>(dst)[i] = v;
    }
}

struct Shape4 { int d[4]; };

// One thread per padded output float. out dim i = in dim perm[i].
__global__ void transpose_kernel(const float* __restrict__ x, float* __restrict__ y,
                                 Shape4 is, Shape4 os, Shape4 perm) {
    const int os3p = (os.d[3] + 3) & ~3, is3p = (is.d[3] + 3) & ~3;
    const long total = (long)os.d[0] * os.d[1] * os.d[2] * os3p;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        int o[4];
        o[3] = int(t % os3p); t /= os3p;
        o[2] = int(t % os.d[2]); t /= os.d[2];
        o[1] = int(t % os.d[1]); t /= os.d[1];
        o[0] = int(t);
        float v = 0.f;
        if (o[3] < os.d[3]) {
            int in[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) in[perm.d[k]] = o[k];
            v = x[(((long)in[0] * is.d[1] + in[1]) * is.d[2] + in[2]) * is3p + in[3]];
        }
        y[i] = v;
    }
}

// Same logical order, different padded last dimension. One thread per output float4
// (four consecutive elements of an output row; lanes past out_last are written as zero).
// rows_per_block > 0: output row r goes to block r / rows_per_block at block_stride_q float4s
// per block (a slice of a wider tensor); 0: dense.
template <typename Index>
__global__ void reshape_kernel(const float* __restrict__ x, float4* __restrict__ y,
                               Index n, int in_last, int out_last, Index rows_per_block, long block_stride_q) {
    grid_dependency_trigger();
    grid_dependency_wait();
    const int ip = (in_last + 3) & ~3, oq = ((out_last + 3) & ~3) >> 2;
    const Index total = n / out_last * oq;
    for (Index i = blockIdx.x * (Index)blockDim.x + threadIdx.x; i < total; i += (Index)gridDim.x * blockDim.x) {
        const Index r = i / oq;
        const int c = int(i - r * oq) * 4;
        const Index e = r * out_last + c;           // logical index of the first lane
        Index q = e / in_last;
        int rem = int(e - q * in_last);
        float v[4];
#pragma unroll
        for (int l = 0; l < 4; ++l) {
            v[l] = c + l < out_last ? x[q * ip + rem] : 0.f;
            if (++rem == in_last) { rem = 0; ++q; }
        }
        long dst = (long)i;
        if (rows_per_block) {
            const Index b = r / rows_per_block;
            dst = (long)b * block_stride_q + (long)(r - b * rows_per_block) * oq + (c >> 2);
        }
        y[dst] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

struct ConcatArgs {
    const float* in[OGLE_MAX_CONCAT_INPUTS];
    int in_axis[OGLE_MAX_CONCAT_INPUTS];   // extent of each input on the axis
    int axis_start[OGLE_MAX_CONCAT_INPUTS + 1];
    int n_inputs;
    int axis;
    int os[4];
};

// Fast path: axis != 3, or axis == 3 with every slice a multiple of 4 channels.
// One thread per output float4; each input is read once and the output written once.
// Four independent 16-byte loads are issued before the first store, and the index
// arithmetic is 32-bit when the tensor allows it (64-bit divisions cost more than the copy).
// False when the element belongs to a slice that is already in place (null input): not stored.
template <typename Index>
__device__ __forceinline__ bool concat_fetch(const ConcatArgs& a, Index i, int q, float4* out) {
    Index t = i;
    int o[4];
    o[3] = int(t % q) * 4; t /= q;
    o[2] = int(t % a.os[2]); t /= a.os[2];
    o[1] = int(t % a.os[1]); t /= a.os[1];
    o[0] = int(t);
    const int pos = o[a.axis];
    int k = 0;
    while (k + 1 < a.n_inputs && pos >= a.axis_start[k + 1]) ++k;
    int s[4] = {a.os[0], a.os[1], a.os[2], a.os[3]};
    s[a.axis] = a.in_axis[k];
    o[a.axis] = pos - a.axis_start[k];
    if (a.in[k] == nullptr) return false;
    const int s3p = (s[3] + 3) & ~3;
    const long off = (((long)o[0] * s[1] + o[1]) * s[2] + o[2]) * s3p + o[3];
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (o[3] < s3p) v = __ldg(reinterpret_cast<const float4*>(a.in[k] + off));
    *out = v;
    return true;
}

template <typename Index>
__global__ void __launch_bounds__(256) concat_vec_kernel(ConcatArgs a, float4* __restrict__ y) {
    grid_dependency_trigger();
    grid_dependency_wait();
    const int q = ((a.os[3] + 3) & ~3) >> 2;
    const Index total = (Index)a.os[0] * a.os[1] * a.os[2] * q;
    const Index step = (Index)gridDim.x * blockDim.x;
    Index i = blockIdx.x * (Index)blockDim.x + threadIdx.x;
    for (; i + 3 * step < total; i += 4 * step) {
        float4 v[4];
        bool ok[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) ok[u] = concat_fetch<Index>(a, i + u * step, q, &v[u]);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (ok[u]) y[i + u * step] = v[u];
    }
    for (; i < total; i += step) {
        float4 v;
        if (concat_fetch<Index>(a, i, q, &v)) y[i] = v;
    }
}

// General path (channel-axis slices not multiples of 4): one thread per output float.
__global__ void concat_scalar_kernel(ConcatArgs a, float* __restrict__ y) {
    const int op = (a.os[3] + 3) & ~3;
    const long total = (long)a.os[0] * a.os[1] * a.os[2] * op;
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        long t = i;
        int o[4];
        o[3] = int(t % op); t /= op;
        o[2] = int(t % a.os[2]); t /= a.os[2];
        o[1] = int(t % a.os[1]); t /= a.os[1];
        o[0] = int(t);
        float v = 0.f;
        if (o[3] < a.os[3]) {
            const int pos = o[a.axis];
            int k = 0;
            while (k + 1 < a.n_inputs && pos >= a.axis_start[k + 1]) ++k;
            int s[4] = {a.os[0], a.os[1], a.os[2], a.os[3]};
            s[a.axis] = a.in_axis[k];
            o[a.axis] = pos - a.axis_start[k];
            const int s3p = (s[3] + 3) & ~3;
            v = a.in[k][(((long)o[0] * s[1] + o[1]) * s[2] + o[2]) * s3p + o[3]];
        }
        y[i] = v;
    }
}

}  // namespace ogle

using namespace ogle;

extern "C" {

int ogle_cuda_pad4(const float* dense, float* padded, long rows, int last, int stride,
                   ogle_stream_t stream) {
    if (rows < 0 || last <= 0) return OGLE_ERR_INVALID;
    if (stride == 0) stride = up4(last);
    if (stride < last || (stride & 3)) return OGLE_ERR_INVALID;
    if (rows == 0) return OGLE_OK;
    if (!dense || !padded) return OGLE_ERR_INVALID;
    if (!aligned16(padded)) return OGLE_ERR_ALIGNMENT;
    const long items = rows * (stride / 4);
    launch_overlapped(pad4_kernel, dim3(grid_for(items, 256)), dim3(256), 0, (cudaStream_t)stream, dense, padded, rows, last, stride);
    return finish_launch();
}

int ogle_cuda_unpad4(const float* padded, float* dense, long rows, int last, int stride,
                     ogle_stream_t stream) {
    if (rows < 0 || last <= 0) return OGLE_ERR_INVALID;
    if (stride == 0) stride = up4(last);
    if (stride < last) return OGLE_ERR_INVALID;
    if (rows == 0) return OGLE_OK;
    if (!dense || !padded) return OGLE_ERR_INVALID;
    unpad4_kernel<<<grid_for(rows * last, 256), 256, 0, (cudaStream_t)stream>>>(padded, dense, rows, last, stride);
    return finish_launch();
}

int ogle_cuda_nchw_to_nhwc4(const float* nchw, float* nhwc4, int N, int C, int H, int W,
                            ogle_stream_t stream) {
    if (N <= 0 || C <= 0 || H <= 0 || W <= 0 || !nchw || !nhwc4) return OGLE_ERR_INVALID;
    if (!aligned16(nhwc4)) return OGLE_ERR_ALIGNMENT;
    const long items = (long)N * H * W * ((C + 3) / 4);
    nchw_to_nhwc4_kernel<<<grid_for(items, 256), 256, 0, (cudaStream_t)stream>>>(nchw, nhwc4, N, C, H, W);
    return finish_launch();
}

int ogle_cuda_transpose(const float* x, float* y, const int in_shape[4], const int perm[4],
                        ogle_stream_t stream) {
    if (!x || !y || !in_shape || !perm) return OGLE_ERR_INVALID;
    Shape4 is, os, pm;
    int seen = 0;
    for (int i = 0; i < 4; ++i) {
        if (perm[i] < 0 || perm[i] > 3 || in_shape[i] <= 0) return OGLE_ERR_INVALID;
        seen |= 1 << perm[i];
        is.d[i] = in_shape[i];
        pm.d[i] = perm[i];
    }
    if (seen != 15) return OGLE_ERR_INVALID;
    for (int i = 0; i < 4; ++i) os.d[i] = is.d[pm.d[i]];
    const long items = (long)os.d[0] * os.d[1] * os.d[2] * up4(os.d[3]);
    transpose_kernel<<<grid_for(items, 256), 256, 0, (cudaStream_t)stream>>>(x, y, is, os, pm);
    return finish_launch();
}

static int launch_reshape(const float* x, float* y, long n_elements, int in_last, int out_last, long rows_per_block,
                          long block_stride, ogle_stream_t stream) {
    if (!x || !y || n_elements <= 0 || in_last <= 0 || out_last <= 0) return OGLE_ERR_INVALID;
    if (n_elements % in_last || n_elements % out_last) return OGLE_ERR_INVALID;
    const long rows = n_elements / out_last;
    const long items = rows * up4(out_last);
    if (!aligned16(y)) return OGLE_ERR_ALIGNMENT;
    long extent = items;              // floats of the destination that may be addressed
    if (rows_per_block) {
        if (rows_per_block < 0 || rows % rows_per_block || (block_stride & 3) || block_stride < rows_per_block * up4(out_last))
            return OGLE_ERR_INVALID;
        extent = rows / rows_per_block * block_stride;
    }
    const long vecs = items / 4;
    if (n_elements < 0x7fffffffL && items < 0x7fffffffL && extent < 0x7fffffffL)     // 32-bit index arithmetic when it fits (the usual case)
        launch_overlapped(reshape_kernel<unsigned>, dim3(grid_for(vecs, 256)), dim3(256), 0, (cudaStream_t)stream,
                          x, reinterpret_cast<float4*>(y), (unsigned)n_elements, in_last, out_last, (unsigned)rows_per_block,
                          block_stride / 4);
    else
        launch_overlapped(reshape_kernel<long>, dim3(grid_for(vecs, 256)), dim3(256), 0, (cudaStream_t)stream,
                          x, reinterpret_cast<float4*>(y), n_elements, in_last, out_last, rows_per_block, block_stride / 4);
    return finish_launch();
}

int ogle_cuda_reshape(const float* x, float* y, long n_elements, int in_last, int out_last,
                      ogle_stream_t stream) {
    return launch_reshape(x, y, n_elements, in_last, out_last, 0, 0, stream);
}

int ogle_cuda_reshape_placed(const float* x, float* y, long n_elements, int in_last, int out_last,
                             long rows_per_block, long block_stride, ogle_stream_t stream) {
    if (rows_per_block <= 0) return OGLE_ERR_INVALID;
    return launch_reshape(x, y, n_elements, in_last, out_last, rows_per_block, block_stride, stream);
}

int ogle_cuda_concat(const OgleConcatParams* p, const float* const* inputs, float* y,
                     ogle_stream_t stream) {
    if (!p || !inputs || !y) return OGLE_ERR_INVALID;
    if (p->n_inputs < 1 || p->n_inputs > OGLE_MAX_CONCAT_INPUTS || p->axis < 0 || p->axis > 3)
        return OGLE_ERR_INVALID;
    ConcatArgs a;
    a.n_inputs = p->n_inputs;
    a.axis = p->axis;
    for (int d = 0; d < 4; ++d) a.os[d] = p->in_shapes[0][d];
    a.os[p->axis] = 0;
    bool vec_ok = aligned16(y), any_input = false, any_placed = false;
    for (int i = 0; i < p->n_inputs; ++i) {
        for (int d = 0; d < 4; ++d) {
            if (p->in_shapes[i][d] <= 0) return OGLE_ERR_INVALID;
            if (d != p->axis && p->in_shapes[i][d] != p->in_shapes[0][d]) return OGLE_ERR_INVALID;
        }
        a.in[i] = inputs[i];              // null: the slice is already in place
        a.in_axis[i] = p->in_shapes[i][p->axis];
        a.axis_start[i] = a.os[p->axis];
        a.os[p->axis] += a.in_axis[i];
        if (inputs[i]) any_input = true;
        else any_placed = true;
        if (inputs[i] && !aligned16(inputs[i])) vec_ok = false;
        if (p->axis == 3 && (a.in_axis[i] & 3) && i + 1 < p->n_inputs) vec_ok = false;
    }
    a.axis_start[p->n_inputs] = a.os[p->axis];
    if (!any_input) return OGLE_OK;                       // every slice in place: nothing to copy
    if (any_placed && !vec_ok) return OGLE_ERR_UNSUPPORTED;   // in-place slices need the 16-byte path
    const int op = up4(a.os[3]);
    const long rows = (long)a.os[0] * a.os[1] * a.os[2];
    if (vec_ok) {
        const long vecs = rows * (op / 4);
        if (vecs + 4L * kNumSMs * 8 * 256 < (1L << 31))
            launch_overlapped(concat_vec_kernel<int>, dim3(grid_for(vecs, 256)), dim3(256), 0, (cudaStream_t)stream, a,
                              reinterpret_cast<float4*>(y));
        else
            launch_overlapped(concat_vec_kernel<long>, dim3(grid_for(vecs, 256)), dim3(256), 0, (cudaStream_t)stream, a,
                              reinterpret_cast<float4*>(y));
    } else {
        concat_scalar_kernel<<<grid_for(rows * op, 256), 256, 0, (cudaStream_t)stream>>>(a, y);
    }
    return finish_launch();
}

}  // extern "C"
