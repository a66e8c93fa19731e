// SSD box decoder and detection post-process.
//
// decode: one thread per anchor, 128-bit loads/stores (HBM-bound).
// detect: one thread block per image. The block reads the image's logits once,
// turns them into softmax scores kept in shared memory, and then warps select
// the top-k per class (or per image): each lane holds its share of the class's
// scores in registers and the k-th largest is found bit by bit (radix select over
// shared memory for more than 2048 anchors), followed by a bitonic sort of the
// <= 256 survivors, so logits and boxes cross HBM exactly once and nothing is
// staged in global memory.
#include "common.cuh"

namespace ogle {

__global__ void ssd_decode_kernel(const float4* __restrict__ pred, const float4* __restrict__ anchors,
                                  float4* __restrict__ out, long total, int A, float4 var) {
    for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total;
         i += (long)gridDim.x * blockDim.x) {
        const float4 p = pred[i];
        const float4 a = anchors[i % A];
        // decoder.glsl:21-27, products taken left to right as written there
        const float w = expf(p.z * var.z) * a.z;
        const float h = expf(p.w * var.w) * a.w;
        const float cx = p.x * var.x * a.z + a.x;
        const float cy = p.y * var.y * a.w + a.y;
        out[i] = make_float4(cx - 0.5f * w, cy - 0.5f * h, cx + 0.5f * w, cy + 0.5f * h);
    }
}

constexpr int kMaxTopK = 256;

// Warp-collective: sorts list[0..n) (n <= kMaxTopK packed keys) descending in place
// (padded to a power of two with zeros, bitonic network). Returns min(n, kMaxTopK).
__device__ __noinline__ int warp_sort_list(unsigned long long* list, int n) {
    const int lane = threadIdx.x & 31;
    if (n > kMaxTopK) n = kMaxTopK;
    int P = 32;
    while (P < n) P <<= 1;
    for (int i = n + lane; i < P; i += 32) list[i] = 0ull;
    __syncwarp();
    for (int size = 2; size <= P; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int t = lane; t < P / 2; t += 32) {
                const int lo = 2 * t - (t & (stride - 1));
                const int hi = lo + stride;
                const bool desc = ((lo & size) == 0);
                const unsigned long long a = list[lo], b = list[hi];
                if ((a < b) == desc) { list[lo] = b; list[hi] = a; }
            }
            __syncwarp();
        }
    }
    return n;
}

// Warp-collective: selects the `k` largest scores among vals[0..A) that exceed
// `thr` (ties: lower index first) and leaves them in list[0..n) sorted by
// (score descending, index ascending) as packed keys
// (score_bits << 32 | ~index). hist: 256 warp-private counters. Returns n.
__device__ __noinline__ int warp_select_topk(const float* vals, int A, float thr, int k,
                                unsigned long long* list, unsigned* hist) {
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xffffffffu;
    // count candidates
    int n_valid = 0;
    for (int base = 0; base < A; base += 32) {
        const int i = base + lane;
        const bool ok = i < A && vals[i] > thr;
        n_valid += __popc(__ballot_sync(full, ok));
    }
    unsigned T = 0;          // bits of the k-th largest score
    int need_eq = 0;         // how many entries equal to T are taken
    bool take_all = n_valid <= k;
    if (!take_all) {
        unsigned prefix = 0, mask = 0;
        int remaining = k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int b = lane; b < 256; b += 32) hist[b] = 0;
            __syncwarp();
            for (int base = 0; base < A; base += 32) {
                const int i = base + lane;
                const float v = i < A ? vals[i] : 0.f;
                const unsigned bits = __float_as_uint(v);
                const bool ok = i < A && v > thr && (bits & mask) == prefix;
                const unsigned active = __ballot_sync(full, ok);
                if (ok) {
                    const unsigned d = (bits >> shift) & 255u;
                    const unsigned peers = __match_any_sync(active, d);
                    if (lane == __ffs(peers) - 1) atomicAdd(&hist[d], (unsigned)__popc(peers));
                }
            }
            __syncwarp();
            // lane owns bins [lane*8, lane*8+8); suffix sums from the top bin down
            unsigned mine[8];
            unsigned lane_sum = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) { mine[j] = hist[lane * 8 + j]; lane_sum += mine[j]; }
            unsigned above = 0;  // elements in bins owned by higher lanes
            for (int l = 31; l > 0; --l) {
                const unsigned s_l = __shfl_sync(full, lane_sum, l);
                if (l > lane) above += s_l;
            }
            // find the digit inside this lane's bins, if the k-th element falls here
            int found_digit = -1;
            unsigned cnt_above_digit = 0;
            unsigned run = above;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                if (found_digit < 0 && run < (unsigned)remaining && run + mine[j] >= (unsigned)remaining) {
                    found_digit = lane * 8 + j;
                    cnt_above_digit = run;
                }
                run += mine[j];
            }
            const unsigned who = __ballot_sync(full, found_digit >= 0);
            const int src = __ffs(who) - 1;   // exactly one lane finds it
            const int digit = __shfl_sync(full, found_digit, src);
            const unsigned cab = __shfl_sync(full, cnt_above_digit, src);
            prefix |= (unsigned)digit << shift;
            mask |= 255u << shift;
            remaining -= (int)cab;
            __syncwarp();
        }
        T = prefix;
        need_eq = remaining;
    }
    // ordered compaction: everything above T, and the first need_eq equal to T
    int n = 0, eq_taken = 0;
    for (int base = 0; base < A; base += 32) {
        const int i = base + lane;
        const float v = i < A ? vals[i] : 0.f;
        const unsigned bits = __float_as_uint(v);
        const bool ok = i < A && v > thr;
        const bool gt = ok && (take_all || bits > T);
        const bool eq = ok && !take_all && bits == T;
        const unsigned m_eq = __ballot_sync(full, eq);
        const int eq_rank = eq_taken + __popc(m_eq & ((1u << lane) - 1u));
        const bool sel = gt || (eq && eq_rank < need_eq);
        const unsigned m_sel = __ballot_sync(full, sel);
        if (sel) {
            const int pos = n + __popc(m_sel & ((1u << lane) - 1u));
            if (pos < kMaxTopK)
                list[pos] = ((unsigned long long)bits << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
        }
        n += __popc(m_sel);
        eq_taken += __popc(m_eq);
    }
    return warp_sort_list(list, n);
}

// Register-resident variant for A <= 32 * kRegPer and thr >= 0: each lane keeps its
// A/32 scores in registers (0 = not a candidate; candidates are positive floats, which
// order like their bit patterns), finds the bits of the k-th largest one bit at a time
// from the top (a count per bit: lane-local compares and one warp reduction, no shared
// memory, no atomics), then compacts in index order and sorts as above.
constexpr int kRegPer = 64;

__device__ int warp_select_topk_reg(const float* vals, int A, float thr, int k, unsigned long long* list) {
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xffffffffu;
    unsigned bits[kRegPer];
    int local = 0;
#pragma unroll
    for (int j = 0; j < kRegPer; ++j) {
        const int i = j * 32 + lane;
        const float v = i < A ? vals[i] : 0.f;
        bits[j] = (i < A && v > thr) ? __float_as_uint(v) : 0u;
        local += bits[j] != 0u;
    }
    const int n_valid = __reduce_add_sync(full, local);
    const bool take_all = n_valid <= k;
    unsigned T = 0;
    int need_eq = 0;
    if (!take_all) {
        unsigned prefix = 0;
        int remaining = k;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned cand = prefix | (1u << bit);
            const unsigned hi = ~((1u << bit) - 1u);
            int c = 0;
#pragma unroll
            for (int j = 0; j < kRegPer; ++j) c += (bits[j] & hi) == cand;
            const int total = __reduce_add_sync(full, c);
            if (total >= remaining) prefix = cand;      // the k-th largest has this bit set
            else remaining -= total;                    // all of those rank above it
        }
        T = prefix;
        need_eq = remaining;
    }
    int n = 0, eq_taken = 0;
#pragma unroll
    for (int j = 0; j < kRegPer; ++j) {
        if (j * 32 >= A) break;
        const int i = j * 32 + lane;
        const unsigned b = bits[j];
        const bool ok = b != 0u;
        const bool gt = ok && (take_all || b > T);
        const bool eq = ok && !take_all && b == T;
        const unsigned m_eq = __ballot_sync(full, eq);
        const int eq_rank = eq_taken + __popc(m_eq & ((1u << lane) - 1u));
        const bool sel = gt || (eq && eq_rank < need_eq);
        const unsigned m_sel = __ballot_sync(full, sel);
        if (sel) {
            const int pos = n + __popc(m_sel & ((1u << lane) - 1u));
            if (pos < kMaxTopK) list[pos] = ((unsigned long long)b << 32) | (unsigned long long)(0xffffffffu - (unsigned)i);
        }
        n += __popc(m_sel);
        eq_taken += __popc(m_eq);
    }
    return warp_sort_list(list, n);
}

struct DetectArgs {
    int N, A, C, logit_stride, mode, top_k, image_w, image_h;
    float score_thr, nms_thr;
    int classes_per_pass;   // mode 1: foreground classes whose scores fit in shared memory at once
    int parts;              // mode 1: blocks per image, each taking a contiguous range of the foreground classes
    const OgleImageDesc* frames;   // mode 0: per-image frame sizes, or null
};

// Dynamic shared memory layout:
//   float scores[classes_per_pass][A]         (mode 0: scores[A] then int cls[A])
//   per warp: 2 KB scratch (histogram, then the sorted list)
__global__ void __launch_bounds__(640)
ssd_detect_kernel(const float* __restrict__ logits, const float4* __restrict__ boxes,
                  float* __restrict__ out_score, int* __restrict__ out_anchor, int* __restrict__ out_class,
                  float4* __restrict__ out_box, int* __restrict__ out_count, DetectArgs a) {
    extern __shared__ __align__(16) unsigned char smem[];
    const int parts = a.mode == 1 ? a.parts : 1;
    const int n = blockIdx.x / parts, part = blockIdx.x - n * parts;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const float* lg = logits + (long)n * a.A * a.logit_stride;
    const float4* bx = boxes + (long)n * a.A;

    if (a.mode == 1) {
        float* scores = reinterpret_cast<float*>(smem);
        unsigned char* wbase = smem + (size_t)a.classes_per_pass * a.A * sizeof(float);
        wbase += (16 - (reinterpret_cast<uintptr_t>(wbase) & 15)) & 15;
        unsigned long long* list = reinterpret_cast<unsigned long long*>(wbase + (size_t)warp * 2048);
        unsigned* hist = reinterpret_cast<unsigned*>(list);
        const int rows = (a.C - 1) * a.top_k;
        const int per_part = (a.C - 1 + parts - 1) / parts;
        const int c_lo = 1 + part * per_part, c_hi = min(a.C, c_lo + per_part);     // this block's classes
        for (int c0 = c_lo; c0 < c_hi; c0 += a.classes_per_pass) {
            const int nc = min(a.classes_per_pass, c_hi - c0);
            // softmax exactly as the reference post-process does: exp of the raw
            // logits, summed in class order, then one divide per class
            if (nc == c_hi - c_lo && a.C <= 32 && (a.logit_stride & 3) == 0 && a.logit_stride <= 32) {
                // the whole row in registers: 128-bit loads, every exponential taken once
                for (int i = tid; i < a.A; i += blockDim.x) {
                    const float4* row4 = reinterpret_cast<const float4*>(lg + (long)i * a.logit_stride);
                    float e[32];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (q * 4 < a.logit_stride) v = row4[q];
                        e[q * 4 + 0] = v.x; e[q * 4 + 1] = v.y; e[q * 4 + 2] = v.z; e[q * 4 + 3] = v.w;
                    }
                    float total = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (j < a.C) { e[j] = expf(e[j]); total += e[j]; }
#pragma unroll
                    for (int j = 1; j < 32; ++j)
                        if (j >= c0 && j < c0 + nc) scores[(j - c0) * a.A + i] = e[j] / total;
                }
            } else {
                for (int i = tid; i < a.A; i += blockDim.x) {
                    const float* row = lg + (long)i * a.logit_stride;
                    float total = 0.f;
                    for (int j = 0; j < a.C; ++j) total += expf(row[j]);
                    for (int j = 0; j < nc; ++j) scores[j * a.A + i] = expf(row[c0 + j]) / total;
                }
            }
            __syncthreads();
            for (int j = warp; j < nc; j += nwarps) {
                const int cls = c0 + j;
                const int cnt = (a.A <= 32 * kRegPer && a.score_thr >= 0.f)
                                    ? warp_select_topk_reg(scores + j * a.A, a.A, a.score_thr, a.top_k, list)
                                    : warp_select_topk(scores + j * a.A, a.A, a.score_thr, a.top_k, list, hist);
                const long base = (long)n * rows + (long)(cls - 1) * a.top_k;
                for (int r = lane; r < a.top_k; r += 32) {
                    float sc = 0.f; int an = -1;
                    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (r < cnt) {
                        const unsigned long long key = list[r];
                        sc = __uint_as_float((unsigned)(key >> 32));
                        an = (int)(0xffffffffu - (unsigned)(key & 0xffffffffull));
                        b = bx[an];
                    }
                    out_score[base + r] = sc;
                    out_anchor[base + r] = an;
                    out_class[base + r] = r < cnt ? cls : 0;
                    out_box[base + r] = b;
                }
                if (lane == 0) out_count[(long)n * (a.C - 1) + cls - 1] = cnt;
                __syncwarp();
            }
            __syncthreads();
        }
        return;
    }

    // mode 0: the reference Detector's rule (detector.cc:150-228)
    float* scores = reinterpret_cast<float*>(smem);
    int* best = reinterpret_cast<int*>(scores + a.A);
    unsigned char* wbase = reinterpret_cast<unsigned char*>(best + a.A);
    wbase += (16 - (reinterpret_cast<uintptr_t>(wbase) & 15)) & 15;
    unsigned long long* list = reinterpret_cast<unsigned long long*>(wbase);          // 2 KB
    int* rect = reinterpret_cast<int*>(wbase + 2048);                                  // [256][4]
    int* keep = rect + kMaxTopK * 4;                                                   // [256]
    __shared__ int s_cnt;
    for (int i = tid; i < a.A; i += blockDim.x) {
        const float* row = lg + (long)i * a.logit_stride;
        float total = expf(row[0]);
        int max_id = 0;
        float max_e = 0.f;
        for (int j = 1; j < a.C; ++j) {
            const float e = expf(row[j]);
            total += e;
            if (max_e < e) { max_e = e; max_id = j; }
        }
        scores[i] = max_e / total;
        best[i] = max_id;
    }
    __syncthreads();
    if (warp == 0) {
        const int cnt = warp_select_topk(scores, a.A, a.score_thr, a.top_k, list, reinterpret_cast<unsigned*>(rect));
        if (lane == 0) s_cnt = cnt;
    }
    __syncthreads();
    const int cnt = s_cnt;
    // integer pixel rectangles of the frame the image came from (detector.cc:179-180,199-214):
    // cv::Rect members are int, so float -> int truncates
    const int image_w = a.frames ? a.frames[n].width : a.image_w;
    const int image_h = a.frames ? a.frames[n].height : a.image_h;
    for (int r = tid; r < cnt; r += blockDim.x) {
        const int an = (int)(0xffffffffu - (unsigned)(list[r] & 0xffffffffull));
        const float4 b = bx[an];
        const float xmin = b.x * image_w, ymin = b.y * image_h;
        const float xmax = b.z * image_w, ymax = b.w * image_h;
        rect[r * 4 + 0] = (int)xmin; rect[r * 4 + 1] = (int)ymin;
        rect[r * 4 + 2] = (int)(xmax - xmin); rect[r * 4 + 3] = (int)(ymax - ymin);
    }
    __syncthreads();
    // detector.cc:127-148: box j is dropped if ANY earlier box i (dropped or not)
    // overlaps it by more than the threshold
    for (int j = tid; j < cnt; j += blockDim.x) {
        int k = 1;
        if (a.nms_thr > 0.f) {
            const float xmin1 = rect[j * 4], ymin1 = rect[j * 4 + 1];
            const float xmax1 = rect[j * 4] + rect[j * 4 + 2], ymax1 = rect[j * 4 + 1] + rect[j * 4 + 3];
            for (int i = 0; i < j; ++i) {
                const float xmin0 = rect[i * 4], ymin0 = rect[i * 4 + 1];
                const float xmax0 = rect[i * 4] + rect[i * 4 + 2], ymax0 = rect[i * 4 + 1] + rect[i * 4 + 3];
                const float w = fmaxf(0.0f, fminf(xmax0, xmax1) - fmaxf(xmin0, xmin1));
                const float h = fmaxf(0.0f, fminf(ymax0, ymax1) - fmaxf(ymin0, ymin1));
                const float inter = w * h;
                const float uni = (xmax0 - xmin0) * (ymax0 - ymin0) + (xmax1 - xmin1) * (ymax1 - ymin1) - inter;
                const float iou = uni <= 0.0f ? 0.0f : inter / uni;
                if (iou > a.nms_thr) { k = 0; break; }
            }
        }
        keep[j] = k;
    }
    __syncthreads();
    // ordered compaction of the survivors by warp 0
    if (warp == 0) {
        int nout = 0;
        const long base = (long)n * a.top_k;
        for (int b0 = 0; b0 < cnt; b0 += 32) {
            const int j = b0 + lane;
            const bool k = j < cnt && keep[j];
            const unsigned m = __ballot_sync(0xffffffffu, k);
            if (k) {
                const int pos = nout + __popc(m & ((1u << lane) - 1u));
                const unsigned long long key = list[j];
                const int an = (int)(0xffffffffu - (unsigned)(key & 0xffffffffull));
                out_score[base + pos] = __uint_as_float((unsigned)(key >> 32));
                out_anchor[base + pos] = an;
                out_class[base + pos] = best[an];
                out_box[base + pos] = make_float4((float)rect[j * 4], (float)rect[j * 4 + 1],
                                                  (float)rect[j * 4 + 2], (float)rect[j * 4 + 3]);
            }
            nout += __popc(m);
        }
        for (int r = nout + lane; r < a.top_k; r += 32) {
            out_score[base + r] = 0.f; out_anchor[base + r] = -1; out_class[base + r] = 0;
            out_box[base + r] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (lane == 0) out_count[n] = nout;
    }
}

}  // namespace ogle

using namespace ogle;

extern "C" {

int ogle_cuda_ssd_decode(const float* pred, const float* anchors, float* out, int N, int A,
                         const float variances[4], ogle_stream_t stream) {
    if (!pred || !anchors || !out || !variances || N <= 0 || A <= 0) return OGLE_ERR_INVALID;
    if (!aligned16(pred) || !aligned16(anchors) || !aligned16(out)) return OGLE_ERR_ALIGNMENT;
    const long total = (long)N * A;
    const float4 var = make_float4(variances[0], variances[1], variances[2], variances[3]);
    ssd_decode_kernel<<<grid_for(total, 256), 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const float4*>(pred), reinterpret_cast<const float4*>(anchors),
        reinterpret_cast<float4*>(out), total, A, var);
    return finish_launch();
}

int ogle_cuda_ssd_detect(const OgleDetectParams* p, const float* logits, const float* boxes,
                         float* out_score, int* out_anchor, int* out_class, float* out_box,
                         int* out_count, ogle_stream_t stream) {
    if (!p || !logits || !boxes || !out_score || !out_anchor || !out_class || !out_box || !out_count)
        return OGLE_ERR_INVALID;
    if (p->N <= 0 || p->A <= 0 || p->C < 2 || p->top_k <= 0 || p->top_k > kMaxTopK) return OGLE_ERR_INVALID;
    if (p->mode < 0 || p->mode > 1) return OGLE_ERR_INVALID;
    const int ls = p->logit_stride ? p->logit_stride : p->C;
    if (ls < p->C) return OGLE_ERR_INVALID;
    if (!aligned16(boxes) || !aligned16(out_box)) return OGLE_ERR_ALIGNMENT;
    DetectArgs a;
    a.N = p->N; a.A = p->A; a.C = p->C; a.logit_stride = ls; a.mode = p->mode; a.top_k = p->top_k;
    a.image_w = p->image_w; a.image_h = p->image_h; a.score_thr = p->score_thr; a.nms_thr = p->nms_thr;
    a.frames = p->mode == 0 ? p->frame_sizes : nullptr;
    if (a.frames && (reinterpret_cast<uintptr_t>(a.frames) & 7)) return OGLE_ERR_ALIGNMENT;
    static const size_t kSmemBudget = 200 * 1024;
    int threads;
    size_t smem;
    if (p->mode == 1) {
        // Two blocks per image, each with half of the foreground classes, when that lets two
        // blocks share an SM and the batch is a few rounds of SMs at most (more, smaller blocks
        // fill the last round better; for large batches the softmax done twice costs more than
        // that gains); one warp per class, ~100 registers each.
        const size_t per_warp = 2048;
        const size_t per_class = (size_t)p->A * sizeof(float);
        const int fg = p->C - 1;
        a.parts = 1;
        if (fg >= 8 && p->N <= 4 * kNumSMs) {
            const int half = (fg + 1) / 2;
            const size_t need = (size_t)half * per_class + per_warp * (size_t)half + 16;
            if (need <= 108 * 1024) a.parts = 2;
        }
        const int classes = (fg + a.parts - 1) / a.parts;
        int warps = classes < 20 ? classes : 20;
        if (warps < 1) warps = 1;
        threads = warps * 32;
        const size_t warp_bytes = per_warp * (size_t)warps + 16;
        const size_t budget = a.parts == 2 ? 108 * 1024 : kSmemBudget;
        if (per_class + warp_bytes > budget) return OGLE_ERR_UNSUPPORTED;
        size_t cpp = (budget - warp_bytes) / per_class;
        if (cpp > (size_t)classes) cpp = classes;
        a.classes_per_pass = (int)cpp;
        smem = cpp * per_class + warp_bytes;
    } else {
        threads = 256;
        a.classes_per_pass = 0;
        a.parts = 1;
        smem = (size_t)p->A * 8 + 16 + 2048 + kMaxTopK * 5 * sizeof(int);
        if (smem > kSmemBudget) return OGLE_ERR_UNSUPPORTED;
    }
    static thread_local int attr_set_for_device = -1;
    int dev = 0;
    cudaGetDevice(&dev);
    if (attr_set_for_device != dev) {
        cudaError_t e = cudaFuncSetAttribute(ssd_detect_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)(kSmemBudget + 4096));
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_set_for_device = dev;
    }
    ssd_detect_kernel<<<p->N * (p->mode == 1 ? a.parts : 1), threads, smem, (cudaStream_t)stream>>>(
        logits, reinterpret_cast<const float4*>(boxes), out_score, out_anchor, out_class,
        reinterpret_cast<float4*>(out_box), out_count, a);
    return finish_launch();
}

}  // extern "C"
