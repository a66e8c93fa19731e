// SSD box decoder and detection post-process.
//
// decode: one thread per anchor, 128-bit loads/stores (HBM-bound).
// detect: one thread block per image. The block reads the image's logits once,
// turns them into softmax scores kept in shared memory, and then warps select
// the top-k per class (or per image): each lane holds its share of the class's
// scores in registers, the k-th largest is found by a radix select and the
// <= 256 survivors are ordered by a stable radix sort (for more than 1952 anchors:
// radix select over shared memory and a bitonic sort), so logits and boxes cross HBM
// exactly once and nothing is staged in global memory.
#include "common.cuh"

namespace ogle {

__global__ void ssd_decode_kernel(const float4* __restrict__ pred, const float4* __restrict__ anchors,
                                  float4* __restrict__ out, long total, int A, float4 var) {
    grid_dependency_trigger();
    grid_dependency_wait();
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

// Selection for up to 32 * kPer scores and thr >= 0, used by the per-class mode: radix select, then a
// stable radix sort of the survivors, all inside one warp.
//  - Lane l owns the contiguous index range [l * per, l * per + per) (per odd, so that the 32 lanes read
//    different shared-memory banks) and keeps its scores in registers as keys = bits(score) - bits(thr):
//    positive floats order like their bit patterns, a key of 0 marks "not a candidate", and the keys of
//    (thr, 1] span only range_bits bits (26 for thr = 0.01).
//  - The k-th largest key is found digit by digit from the top (9 bits at a time: three passes for 26 bits)
//    with a 512-bin histogram in the warp's scratch.
//  - Survivors (keys above the k-th, and the first few equal to it in index order) are written out in index
//    order - each lane's range is contiguous, so two prefix sums over the lanes place them - and sorted by
//    key, descending, with a stable LSD radix sort (8 bits at a time, elements held in registers, ranks
//    within a group of 32 from match.any). Stability keeps equal scores in index order.
// Scratch (kWarpScratch bytes): select: hist[512] u32 at 0; sort: keys[256] u32 at 0, idx[256] u16 at 1024,
// digit counts[512] u32 at 1536. On return keys/idx hold the n survivors in output order.
constexpr int kPer = 61;
constexpr int kWarpScratch = 3584;

__device__ __forceinline__ unsigned warp_excl_scan(unsigned v, unsigned* total) {
    const int lane = threadIdx.x & 31;
    unsigned incl = v;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const unsigned t = __shfl_up_sync(0xffffffffu, incl, off);
        if (lane >= off) incl += t;
    }
    *total = __shfl_sync(0xffffffffu, incl, 31);
    return incl - v;
}

__device__ int warp_topk_radix(const float* vals, int A, float thr, int k, unsigned char* scratch) {
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xffffffffu;
    const unsigned thr_bits = __float_as_uint(thr);
    const unsigned max_key = thr_bits < 0x3f800000u ? 0x3f800000u - thr_bits : 1u;     // scores never exceed 1
    const int range_bits = 32 - __clz(max_key);
    const int per = ((A + 31) >> 5) | 1;
    const int i0 = lane * per;
    unsigned key[kPer];
    int local = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const int i = i0 + j;
        unsigned kk = 0;
        if (j < per && i < A) {
            const float v = vals[i];
            if (v > thr) kk = __float_as_uint(v) - thr_bits;
        }
        key[j] = kk;
        local += kk != 0u;
    }
    const int n_valid = __reduce_add_sync(full, local);
    const bool take_all = n_valid <= k;
    unsigned T = 0;
    int need_eq = 0;
    if (!take_all) {
        unsigned* hist = reinterpret_cast<unsigned*>(scratch);
        unsigned prefix = 0, mask = 0;
        int remaining = k;
        for (int hi_bit = range_bits; hi_bit > 0;) {
            const int w = hi_bit >= 9 ? 9 : hi_bit;
            const int shift = hi_bit - w;
            const unsigned dmask = (1u << w) - 1u;
            for (int b = lane; b < 512; b += 32) hist[b] = 0;
            __syncwarp();
#pragma unroll
            for (int j = 0; j < kPer; ++j) {
                const unsigned kk = key[j];
                if (kk != 0u && (kk & mask) == prefix) atomicAdd(&hist[(kk >> shift) & dmask], 1u);
            }
            __syncwarp();
            // lane owns bins [16 * lane, 16 * lane + 16); walk down from the top bin
            unsigned mine[16];
            unsigned lane_sum = 0;
            const uint4* h4 = reinterpret_cast<const uint4*>(hist + lane * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 v = h4[q];
                mine[q * 4 + 0] = v.x; mine[q * 4 + 1] = v.y; mine[q * 4 + 2] = v.z; mine[q * 4 + 3] = v.w;
                lane_sum += v.x + v.y + v.z + v.w;
            }
            unsigned incl = lane_sum;              // sum over this lane and all higher lanes
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const unsigned t = __shfl_down_sync(full, incl, off);
                if (lane + off < 32) incl += t;
            }
            unsigned run = incl - lane_sum;        // candidates in bins above this lane's
            int found = -1;
            unsigned cab = 0;
#pragma unroll
            for (int q = 15; q >= 0; --q) {
                if (found < 0 && run < (unsigned)remaining && run + mine[q] >= (unsigned)remaining) {
                    found = lane * 16 + q;
                    cab = run;
                }
                run += mine[q];
            }
            const unsigned who = __ballot_sync(full, found >= 0);
            const int src = __ffs(who) - 1;        // exactly one lane finds it
            const int digit = __shfl_sync(full, found, src);
            cab = __shfl_sync(full, cab, src);
            prefix |= (unsigned)digit << shift;
            mask |= dmask << shift;
            remaining -= (int)cab;
            hi_bit = shift;
            __syncwarp();
        }
        T = prefix;
        need_eq = remaining;
    }
    // survivors in index order
    unsigned cnt_gt = 0, cnt_eq = 0;
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const unsigned kk = key[j];
        cnt_gt += (kk != 0u) && (take_all || kk > T);
        cnt_eq += (kk != 0u) && !take_all && kk == T;
    }
    unsigned tot_eq, tot_sel;
    const unsigned eq_before = warp_excl_scan(cnt_eq, &tot_eq);
    unsigned take_eq = 0;
    if ((unsigned)need_eq > eq_before) take_eq = min(cnt_eq, (unsigned)need_eq - eq_before);
    unsigned pos = warp_excl_scan(cnt_gt + take_eq, &tot_sel);
    const int n = (int)(tot_sel < (unsigned)kMaxTopK ? tot_sel : (unsigned)kMaxTopK);
    unsigned* keys = reinterpret_cast<unsigned*>(scratch);
    unsigned short* idx = reinterpret_cast<unsigned short*>(scratch + 1024);
    unsigned* counts = reinterpret_cast<unsigned*>(scratch + 1536);
    __syncwarp();
#pragma unroll
    for (int j = 0; j < kPer; ++j) {
        const unsigned kk = key[j];
        const bool gt = (kk != 0u) && (take_all || kk > T);
        const bool eq = (kk != 0u) && !take_all && kk == T;
        bool sel = gt;
        if (eq && take_eq > 0) { sel = true; --take_eq; }
        if (sel) {
            if (pos < (unsigned)kMaxTopK) { keys[pos] = kk; idx[pos] = (unsigned short)(i0 + j); }
            ++pos;
        }
    }
    __syncwarp();
    // stable LSD radix sort, descending: eight elements per lane in registers, position p = c * 32 + lane
    unsigned e_key[8], e_idx[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        const int p = c * 32 + lane;
        e_key[c] = p < n ? keys[p] : 0u;
        e_idx[c] = p < n ? idx[p] : 0u;
    }
    const int n_chunks = (n + 31) >> 5;
    for (int shift = 0; shift < range_bits; shift += 9) {
        for (int b = lane; b < 512; b += 32) counts[b] = 0;
        __syncwarp();
        for (int c = 0; c < n_chunks; ++c) {
            const bool ok = c * 32 + lane < n;
            const unsigned d = 511u - ((e_key[c] >> shift) & 511u);
            const unsigned act = __ballot_sync(full, ok);
            if (ok) {
                const unsigned peers = __match_any_sync(act, d);
                if (lane == __ffs(peers) - 1) counts[d] += (unsigned)__popc(peers);
            }
            __syncwarp();
        }
        // exclusive prefix over the 512 digits (digit 0 = largest key digit comes first)
        {
            unsigned v[16], sum = 0;
            uint4* c4 = reinterpret_cast<uint4*>(counts + lane * 16);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint4 t = c4[q];
                v[q * 4 + 0] = t.x; v[q * 4 + 1] = t.y; v[q * 4 + 2] = t.z; v[q * 4 + 3] = t.w;
                sum += t.x + t.y + t.z + t.w;
            }
            unsigned tot;
            unsigned run = warp_excl_scan(sum, &tot);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 t;
                t.x = run; run += v[q * 4 + 0];
                t.y = run; run += v[q * 4 + 1];
                t.z = run; run += v[q * 4 + 2];
                t.w = run; run += v[q * 4 + 3];
                c4[q] = t;
            }
        }
        __syncwarp();
        for (int c = 0; c < n_chunks; ++c) {
            const bool ok = c * 32 + lane < n;
            const unsigned d = 511u - ((e_key[c] >> shift) & 511u);
            const unsigned act = __ballot_sync(full, ok);
            unsigned peers = 0, base = 0;
            if (ok) {
                peers = __match_any_sync(act, d);
                base = counts[d];
                const unsigned dst = base + (unsigned)__popc(peers & ((1u << lane) - 1u));
                keys[dst] = e_key[c];
                idx[dst] = (unsigned short)e_idx[c];
            }
            __syncwarp();
            if (ok && lane == __ffs(peers) - 1) counts[d] = base + (unsigned)__popc(peers);
            __syncwarp();
        }
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const int p = c * 32 + lane;
            if (p < n) { e_key[c] = keys[p]; e_idx[c] = idx[p]; }
        }
        __syncwarp();
    }
    return n;
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
    grid_dependency_trigger();
    grid_dependency_wait();
    const int parts = a.mode == 1 ? a.parts : 1;
    const int n = blockIdx.x / parts, part = blockIdx.x - n * parts;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;
    const float* lg = logits + (long)n * a.A * a.logit_stride;
    const float4* bx = boxes + (long)n * a.A;

    if (a.mode == 1) {
        float* scores = reinterpret_cast<float*>(smem);
        unsigned char* wbase = smem + (size_t)a.classes_per_pass * a.A * sizeof(float);
        wbase += (16 - (reinterpret_cast<uintptr_t>(wbase) & 15)) & 15;
        unsigned char* my_scratch = wbase + (size_t)warp * kWarpScratch;
        unsigned long long* list = reinterpret_cast<unsigned long long*>(my_scratch);
        unsigned* hist = reinterpret_cast<unsigned*>(list);
        // the radix path: one lane range of at most kPer scores each, 16-bit anchor indices, thr >= 0
        const bool radix = (((a.A + 31) >> 5) | 1) <= kPer && a.A <= 65535 && a.score_thr >= 0.f;
        const unsigned thr_bits = __float_as_uint(a.score_thr);
        const int rows = (a.C - 1) * a.top_k;
        const int per_part = (a.C - 1 + parts - 1) / parts;
        const int c_lo = 1 + part * per_part, c_hi = min(a.C, c_lo + per_part);     // this block's classes
        for (int c0 = c_lo; c0 < c_hi; c0 += a.classes_per_pass) {
            const int nc = min(a.classes_per_pass, c_hi - c0);
            // softmax as the reference post-process does it - exp of the raw logits, summed in class
            // order - with the per-class divide replaced by one IEEE reciprocal of the sum and a
            // multiply per class (scores within one ulp of the reference's quotient)
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
                    const float inv = 1.0f / total;
#pragma unroll
                    for (int j = 1; j < 32; ++j)
                        if (j >= c0 && j < c0 + nc) scores[(j - c0) * a.A + i] = fminf(e[j] * inv, 1.0f);
                }
            } else {
                for (int i = tid; i < a.A; i += blockDim.x) {
                    const float* row = lg + (long)i * a.logit_stride;
                    float total = 0.f;
                    for (int j = 0; j < a.C; ++j) total += expf(row[j]);
                    const float inv = 1.0f / total;
                    for (int j = 0; j < nc; ++j) scores[j * a.A + i] = fminf(expf(row[c0 + j]) * inv, 1.0f);
                }
            }
            __syncthreads();
            for (int j = warp; j < nc; j += nwarps) {
                const int cls = c0 + j;
                const int cnt = radix ? warp_topk_radix(scores + j * a.A, a.A, a.score_thr, a.top_k, my_scratch)
                                      : warp_select_topk(scores + j * a.A, a.A, a.score_thr, a.top_k, list, hist);
                const unsigned* r_keys = reinterpret_cast<const unsigned*>(my_scratch);
                const unsigned short* r_idx = reinterpret_cast<const unsigned short*>(my_scratch + 1024);
                const long base = (long)n * rows + (long)(cls - 1) * a.top_k;
                for (int r = lane; r < a.top_k; r += 32) {
                    float sc = 0.f; int an = -1;
                    float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (r < cnt) {
                        if (radix) {
                            sc = __uint_as_float(r_keys[r] + thr_bits);
                            an = (int)r_idx[r];
                        } else {
                            const unsigned long long key = list[r];
                            sc = __uint_as_float((unsigned)(key >> 32));
                            an = (int)(0xffffffffu - (unsigned)(key & 0xffffffffull));
                        }
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
    launch_overlapped(ssd_decode_kernel, dim3(grid_for(total, 256)), dim3(256), 0, (cudaStream_t)stream,
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
    static const size_t kSmemBudget = 224 * 1024;
    int threads;
    size_t smem;
    if (p->mode == 1) {
        // Two blocks per image, each with half of the foreground classes, when that lets two
        // blocks share an SM and the batch is a few rounds of SMs at most (more, smaller blocks
        // fill the last round better; for large batches the softmax done twice costs more than
        // that gains); one warp per class, ~100 registers each.
        const size_t per_warp = kWarpScratch;
        const size_t per_class = (size_t)p->A * sizeof(float);
        const int fg = p->C - 1;
        a.parts = 1;
        if (fg >= 8 && p->N <= 4 * kNumSMs) {
            const int half = (fg + 1) / 2;
            const size_t need = (size_t)half * per_class + per_warp * (size_t)half + 16;
            if (need <= 112 * 1024) a.parts = 2;
        }
        const int classes = (fg + a.parts - 1) / a.parts;
        int warps = classes < 20 ? classes : 20;
        if (warps < 1) warps = 1;
        threads = warps * 32;
        const size_t warp_bytes = per_warp * (size_t)warps + 16;
        const size_t budget = a.parts == 2 ? 112 * 1024 : kSmemBudget;
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
                                             (int)(kSmemBudget + 2048));
        if (e != cudaSuccess) { set_last_error(e); return OGLE_ERR_CUDA; }
        attr_set_for_device = dev;
    }
    launch_overlapped(ssd_detect_kernel, dim3(p->N * (p->mode == 1 ? a.parts : 1)), dim3(threads), smem, (cudaStream_t)stream,
                      logits, reinterpret_cast<const float4*>(boxes), out_score, out_anchor, out_class,
                      reinterpret_cast<float4*>(out_box), out_count, a);
    return finish_launch();
}

}  // extern "C"
