// Token sampling on the device: greedy, temperature, and nucleus (top-p), one CTA per row of logits.
//
// Meanings follow the reference project's samplers (paths under inference/sampler/):
//   greedy       first maximum wins                                   Sampler.java:144-157
//   temperature  logits / T, softmax over the vocabulary, then the first index i with
//                u < cdf_i in index order, else the last index        Sampler.java:81-101, CategoricalSampler.java:31-42
//   top-p        candidates p >= (1 - top_p) / (n - 1); take them in descending order until their
//                sum exceeds top_p; draw r = u * sum; first candidate (descending) with r < cdf
//                                                                     ToppSampler.java:61-80,110-156
// The uniform number u of each row is an input (the host derives it from seed, request and step
// counters), so a request's draws do not depend on which batch it sits in.  Sums that decide a
// token are either accumulated in a fixed order or in integers, so a row always gives the same
// token.  Equal probabilities are ordered by index in the nucleus.  When few tokens pass the cutoff (a peaked
// distribution, the usual case at the reference's default temperature 0.1) they are gathered into shared
// memory; up to 1,024 of them are ordered by counting and walked like the reference does, in float32.
// Otherwise (a longer list, or the whole row when more than 4,093 pass) the nucleus is found without sorting:
// the bits of the probability at which the descending running mass crosses a target are decided
// two at a time, each pair by one pass of masked sums over the row (two such descents: for top_p, then for the draw).
#include <limits.h>
#include "common.cuh"

namespace b200 {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;
constexpr int kCandidateCap = 4096;  // nucleus candidates that are gathered into shared memory (32 KB)

__global__ void __launch_bounds__(kSampleThreads)
argmax_rows_kernel(const float* __restrict__ logits, int ld, int* __restrict__ out, int V) {
    __shared__ float best_s[kSampleWarps];
    __shared__ int idx_s[kSampleWarps];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int idx = INT_MAX;
    auto take = [&](float v, int i) { if (v > best) { best = v; idx = i; } };   // a thread meets its indices in rising order
    int done = 0;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // 16 bytes per load and four loads in flight per thread: the row (half a megabyte of a vocabulary of 128k, just
        // written, so in L2) is a dozen trips to L2 otherwise
        const float4* row4 = reinterpret_cast<const float4*>(row);
        const int n4 = V / 4;
        for (int i = threadIdx.x; i < n4; i += 4 * kSampleThreads) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
                v[u] = i + u * kSampleThreads < n4 ? row4[i + u * kSampleThreads] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int at = 4 * (i + u * kSampleThreads);
                take(v[u].x, at); take(v[u].y, at + 1); take(v[u].z, at + 2); take(v[u].w, at + 3);
            }
        }
        done = 4 * n4;
    }
    for (int i = done + threadIdx.x; i < V; i += kSampleThreads) take(row[i], i);
    auto merge = [](float& b, int& i, float ob, int oi) {
        if (ob > b || (ob == b && oi < i)) { b = ob; i = oi; }
    };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        merge(best, idx, ob, oi);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_s[warp] = best; idx_s[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = best_s[lane];
        idx = idx_s[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            merge(best, idx, ob, oi);
        }
        if (lane == 0) out[blockIdx.x] = idx == INT_MAX ? 0 : idx;
    }
}

struct SampleShared {
    unsigned long long sum_u64[3][kSampleWarps + 1];
    unsigned int sum_u32[kSampleWarps + 1];
    float seg_sum[kSampleWarps];
    unsigned int seg_cnt[kSampleWarps];
    float red[33];
    int answer;
};

constexpr double kMassScale = 1099511627776.0;  // 2^40: probabilities become integers, sums exact

// Sums of three 64-bit values and one 32-bit value per thread over the CTA; every thread gets all of them.
__device__ __forceinline__ void block_sum_mass(unsigned long long (&m)[3], unsigned int& c, SampleShared& sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int k = 0; k < 3; ++k) m[k] += __shfl_xor_sync(0xffffffffu, m[k], o);
        c += __shfl_xor_sync(0xffffffffu, c, o);
    }
    __syncthreads();
    if (lane == 0) {
#pragma unroll
        for (int k = 0; k < 3; ++k) sh.sum_u64[k][warp] = m[k];
        sh.sum_u32[warp] = c;
    }
    __syncthreads();
    if (warp == 0) {
        unsigned long long mm[3] = {sh.sum_u64[0][lane], sh.sum_u64[1][lane], sh.sum_u64[2][lane]};
        unsigned int cc = sh.sum_u32[lane];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int k = 0; k < 3; ++k) mm[k] += __shfl_xor_sync(0xffffffffu, mm[k], o);
            cc += __shfl_xor_sync(0xffffffffu, cc, o);
        }
        if (lane == 0) {
#pragma unroll
            for (int k = 0; k < 3; ++k) sh.sum_u64[k][kSampleWarps] = mm[k];
            sh.sum_u32[kSampleWarps] = cc;
        }
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < 3; ++k) m[k] = sh.sum_u64[k][kSampleWarps];
    c = sh.sum_u32[kSampleWarps];
}

struct Crossing {
    unsigned int key;                 // bits of the probability at which the running mass first exceeds the target
    unsigned long long above;         // mass of the candidates with a larger probability
    unsigned long long mass_eq;       // mass and number of the candidates with exactly that probability
    unsigned int cnt_eq;
    bool found;                       // false: the whole candidate mass does not exceed the target (`above` is all of it)
};

// p * 2^40 is exact in float32 (a power-of-two scale), so the integer part is the same as in double
__device__ __forceinline__ unsigned long long mass_of(float p) { return (unsigned long long)(p * 1099511627776.0f); }

// Walks the candidates (p >= cutoff) in descending order of p, without sorting: the bits of the crossing
// probability are decided two at a time from the top, each pair with one pass of masked sums over the row
// (probabilities are non-negative floats, so their bit patterns order like integers).  Masses are integers
// (p * 2^40): the sums do not depend on the order of addition.  `probs` is 16-byte aligned when V % 4 == 0.
__device__ Crossing mass_descent(const float* __restrict__ probs, int V, float cutoff, unsigned long long target,
                                 SampleShared& sh) {
    unsigned int prefix = 0;
    unsigned long long above = 0;
    const bool vec = (V & 3) == 0;
    // bits 30 .. 0 of a non-negative float: bit 30 alone first, then pairs (29,28) .. (1,0)
    for (int lo = 30; lo >= 0; lo -= 2) {
        const int width = lo == 30 ? 1 : 2;               // bits [lo, lo + width)
        const unsigned int high = ~((1u << (lo + width)) - 1u);
        const unsigned int field = (1u << width) - 1u;
        unsigned long long m[3] = {0, 0, 0};              // mass with field value >= 3, >= 2, >= 1
        unsigned int c = 0;
        auto take = [&](float p) {
            const unsigned int key = __float_as_uint(p);
            if (p >= cutoff && (key & high) == prefix) {
                const unsigned int f = (key >> lo) & field;
                const unsigned long long q = mass_of(p);
                if (f >= 3) m[0] += q;
                if (f >= 2) m[1] += q;
                if (f >= 1) m[2] += q;
            }
        };
        if (vec) {
            // four 16-byte loads are requested before the first is used: a pass is bound by the latency of L2
            const float4* p4 = reinterpret_cast<const float4*>(probs);
            const int n4 = V / 4;
            for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * kSampleThreads) {
                float4 v[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int i = i0 + k * kSampleThreads;
                    v[k] = i < n4 ? p4[i] : make_float4(-1.f, -1.f, -1.f, -1.f);  // negative: below any cutoff
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) { take(v[k].x); take(v[k].y); take(v[k].z); take(v[k].w); }
            }
        } else {
            for (int i = threadIdx.x; i < V; i += kSampleThreads) take(probs[i]);
        }
        block_sum_mass(m, c, sh);
        // field values from the top: the crossing lies in the first one whose cumulative mass exceeds the target
        unsigned int chosen = 0;
        unsigned long long taken = m[2];                  // everything with field >= 1 lies above field 0
        for (unsigned int f = field; f >= 1; --f) {
            if (above + m[3 - f] > target) { chosen = f; taken = f == field ? 0 : m[3 - f - 1]; break; }
        }
        above += taken;
        prefix |= chosen << lo;
    }
    unsigned long long m[3] = {0, 0, 0};
    unsigned int c = 0;
    for (int i = threadIdx.x; i < V; i += kSampleThreads) {
        const float p = probs[i];
        if (p >= cutoff && __float_as_uint(p) == prefix) { m[0] += mass_of(p); ++c; }
    }
    block_sum_mass(m, c, sh);
    Crossing r;
    r.key = prefix;
    r.above = above;
    r.mass_eq = m[0];
    r.cnt_eq = c;
    r.found = c > 0 && above + m[0] > target;
    return r;
}

// A warp's segment [lo, hi) of a row is cut into one contiguous chunk per lane (a multiple of four elements),
// so that prefix sums over (lane, element) run in index order.  `chunk_exp_sum` adds this lane's exponentials in
// index order, four independent 16-byte loads at a time when the row allows it.
__device__ __forceinline__ int lane_chunk(int lo, int hi) { return (((hi - lo + 31) / 32) + 3) & ~3; }

__device__ __forceinline__ float chunk_exp_sum(const float* __restrict__ row, int begin, int end, float inv_t, float zmax, bool vec) {
    float sum = 0.f;
    int i = begin;
    if (vec) {
        for (; i + 16 <= end; i += 16) {
            float4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = *reinterpret_cast<const float4*>(row + i + 4 * k);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                sum += expf(v[k].x * inv_t - zmax);
                sum += expf(v[k].y * inv_t - zmax);
                sum += expf(v[k].z * inv_t - zmax);
                sum += expf(v[k].w * inv_t - zmax);
            }
        }
    }
    for (; i < end; ++i) sum += expf(row[i] * inv_t - zmax);
    return sum;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ uniforms,
                   int* __restrict__ out, int V, float temperature, float top_p, float* __restrict__ probs_scratch) {
    __shared__ SampleShared sh;
    const float* row = logits + (size_t)blockIdx.x * ld;
    const float u = uniforms[blockIdx.x];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // each warp owns a contiguous segment of the vocabulary so that prefix sums run in index order
    const int seg = (((V + kSampleWarps - 1) / kSampleWarps + 31) / 32) * 32;
    const int seg_lo = min(V, warp * seg), seg_hi = min(V, (warp + 1) * seg);

    // logits are multiplied by 1 / temperature (Sampler.java:85 divides; the difference is one rounding)
    const float inv_t = 1.0f / temperature;
    const bool vec = (V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0;
    float zmax = -INFINITY;
    if (vec) {
        const float4* r4 = reinterpret_cast<const float4*>(row);
        const int n4 = V / 4;
        for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * kSampleThreads) {
            float4 v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int i = i0 + k * kSampleThreads;
                v[k] = i < n4 ? r4[i] : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) zmax = fmaxf(zmax, fmaxf(fmaxf(v[k].x, v[k].y), fmaxf(v[k].z, v[k].w)) * inv_t);
        }
    } else {
        for (int i = threadIdx.x; i < V; i += kSampleThreads) zmax = fmaxf(zmax, row[i] * inv_t);
    }
    zmax = block_max(zmax, sh.red);

    const int chunk = lane_chunk(seg_lo, seg_hi);
    const int my_lo = min(seg_hi, seg_lo + lane * chunk), my_hi = min(seg_hi, my_lo + chunk);
    float part = chunk_exp_sum(row, my_lo, my_hi, inv_t, zmax, vec);
    const float my_sum = part;
    part = warp_sum(part);
    if (lane == 0) sh.seg_sum[warp] = part;
    if (threadIdx.x == 0) sh.answer = V - 1;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < kSampleWarps; ++w) total += sh.seg_sum[w];

    const bool nucleus = top_p > 0.f && top_p < 1.f;
    if (!nucleus) {
        // inverse CDF in index order, on the scale of the unnormalised exponentials
        const float target = u * total;
        float excl = 0.f;
        int w_star = -1;
        for (int w = 0; w < kSampleWarps; ++w) {
            if (target < excl + sh.seg_sum[w]) { w_star = w; break; }
            excl += sh.seg_sum[w];
        }
        if (warp == w_star) {
            // the lane whose chunk holds the target, then the element inside that chunk
            float incl = my_sum;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const float n = __shfl_up_sync(0xffffffffu, incl, o);
                if (lane >= o) incl += n;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, my_lo < my_hi && target < excl + incl);
            if (hit == 0) {
                if (lane == 0) sh.answer = seg_hi - 1;  // the target lies within rounding of the segment's end
            } else if (lane == __ffs(hit) - 1) {
                float running = excl + incl - my_sum;
                int answer = my_hi - 1;
                for (int i = my_lo; i < my_hi; ++i) {
                    running += expf(row[i] * inv_t - zmax);
                    if (target < running) { answer = i; break; }
                }
                sh.answer = answer;
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) out[blockIdx.x] = sh.answer;
        return;
    }

    // nucleus: the kept set is the shortest descending prefix of the candidates whose mass exceeds top_p.
    // The probabilities are written once to scratch (this row's V floats) and read back by every pass.
    float* probs = probs_scratch + (size_t)blockIdx.x * V;
    float cutoff = (1.0f - top_p) / (float)(V - 1);
    unsigned int n_cand = 0;
    const float inv_total = 1.0f / total;
    for (int i0 = seg_lo + lane; i0 < seg_hi; i0 += 128) {  // four loads in flight per lane
        float x[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) x[k] = i0 + 32 * k < seg_hi ? row[i0 + 32 * k] : -INFINITY;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            if (i0 + 32 * k < seg_hi) {
                const float p = expf(x[k] * inv_t - zmax) * inv_total;
                probs[i0 + 32 * k] = p;
                n_cand += p >= cutoff ? 1u : 0u;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) n_cand += __shfl_xor_sync(0xffffffffu, n_cand, o);
    if (lane == 0) sh.seg_cnt[warp] = n_cand;
    __syncthreads();
    // With a peaked distribution few tokens pass the cutoff.  Then they are gathered, in index order, into
    // shared memory and everything below works on that short list instead of the row.
    __shared__ __align__(16) float cand_p[kCandidateCap];
    __shared__ int cand_i[kCandidateCap];
    unsigned int total_cand = 0, my_first = 0;
    for (int w = 0; w < kSampleWarps; ++w) {
        if (w == warp) my_first = total_cand;
        total_cand += sh.seg_cnt[w];
    }
    const bool gathered = total_cand > 0 && total_cand <= (unsigned)kCandidateCap - 3;
    if (gathered) {
        unsigned int at = my_first;
        for (int base = seg_lo; base < seg_hi; base += 32) {
            const int i = base + lane;
            const float p = i < seg_hi ? probs[i] : -1.f;  // the element this lane wrote above
            const bool in = p >= cutoff;
            const unsigned mask = __ballot_sync(0xffffffffu, in);
            if (in) {
                const unsigned int k = at + __popc(mask & ((1u << lane) - 1u));
                cand_p[k] = p;
                cand_i[k] = i;
            }
            at += __popc(mask);
        }
        if (threadIdx.x < 3) cand_p[total_cand + threadIdx.x] = -1.f;  // padding to a multiple of four: below any cutoff
    }
    __syncthreads();
    if (gathered && total_cand <= (unsigned)kSampleThreads) {
        // A short list (the usual case at low temperature): every thread finds the place of one candidate in
        // descending order (ties by index) by counting, and one thread walks the ordered list the way the
        // reference does, adding in float32 (ToppSampler.java:110-156).
        __shared__ float ord_p[kSampleThreads];
        __shared__ int ord_i[kSampleThreads];
        const int n = (int)total_cand;
        if ((int)threadIdx.x < n) {
            const float p = cand_p[threadIdx.x];
            int place = 0;
            for (int j = 0; j < n; ++j) {
                const float q = cand_p[j];
                place += (q > p || (q == p && j < (int)threadIdx.x)) ? 1 : 0;  // the list is in index order
            }
            ord_p[place] = p;
            ord_i[place] = cand_i[threadIdx.x];
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float cum = 0.f;
            int last = n - 1;
            for (int j = 0; j < n; ++j) {
                cum += ord_p[j];
                if (cum > top_p) { last = j; break; }
            }
            const float r = u * cum;
            float cdf = 0.f;
            int answer = ord_i[last];
            for (int j = 0; j <= last; ++j) {
                cdf += ord_p[j];
                if (r < cdf) { answer = ord_i[j]; break; }
            }
            out[blockIdx.x] = answer;
        }
        return;
    }
    const float* src = gathered ? cand_p : probs;
    const int n_src = gathered ? (int)((total_cand + 3u) & ~3u) : V;
    const unsigned long long target1 = (unsigned long long)((double)top_p * kMassScale);
    Crossing first = mass_descent(src, n_src, cutoff, target1, sh);
    unsigned long long kept_mass;
    if (first.found) {
        const unsigned long long q1 = first.mass_eq / first.cnt_eq;
        unsigned long long m = q1 ? (target1 - first.above) / q1 + 1 : first.cnt_eq;
        if (m > first.cnt_eq) m = first.cnt_eq;
        kept_mass = first.above + m * q1;
    } else {
        kept_mass = first.above + first.mass_eq;
    }
    unsigned long long target2;
    if (kept_mass == 0) {  // no candidate passes the cutoff: take the most probable token
        cutoff = 0.f;
        target2 = 0;
    } else {
        target2 = (unsigned long long)((double)u * (double)kept_mass);
        if (target2 >= kept_mass) target2 = kept_mass - 1;
    }
    Crossing second = mass_descent(src, n_src, cutoff, target2, sh);
    if (!second.found) {  // cannot happen while target2 < kept mass; keep the last index as the reference's fallback
        if (threadIdx.x == 0) out[blockIdx.x] = V - 1;
        return;
    }
    const unsigned int key2 = second.key;
    const unsigned long long q2 = second.mass_eq / second.cnt_eq;
    unsigned long long m2 = q2 ? (target2 - second.above) / q2 + 1 : 1;
    if (m2 > second.cnt_eq) m2 = second.cnt_eq;
    if (m2 < 1) m2 = 1;

    // the m2-th token, in index order, whose probability has exactly the bits key2
    const int seg2 = (((n_src + kSampleWarps - 1) / kSampleWarps + 31) / 32) * 32;
    const int lo2 = min(n_src, warp * seg2), hi2 = min(n_src, (warp + 1) * seg2);
    __syncthreads();  // seg_cnt is used again
    unsigned int cnt = 0;
    for (int i = lo2 + lane; i < hi2; i += 32) {
        const float p = src[i];
        cnt += (p >= cutoff && __float_as_uint(p) == key2) ? 1u : 0u;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    if (lane == 0) sh.seg_cnt[warp] = cnt;
    __syncthreads();
    unsigned long long before = 0;
    int w_star = -1;
    for (int w = 0; w < kSampleWarps; ++w) {
        if (m2 <= before + sh.seg_cnt[w]) { w_star = w; break; }
        before += sh.seg_cnt[w];
    }
    if (warp == w_star) {
        unsigned long long seen = before;
        int answer = hi2 - 1;
        for (int base = lo2; base < hi2; base += 32) {
            const int i = base + lane;
            bool match = false;
            if (i < hi2) {
                const float p = src[i];
                match = p >= cutoff && __float_as_uint(p) == key2;
            }
            const unsigned mask = __ballot_sync(0xffffffffu, match);
            const unsigned long long n = __popc(mask);
            if (seen + n >= m2) {
                unsigned mm = mask;
                for (unsigned long long k = seen + 1; k < m2; ++k) mm &= mm - 1;  // drop the lowest set bits
                answer = base + __ffs(mm) - 1;
                break;
            }
            seen += n;
        }
        if (lane == 0) sh.answer = gathered ? cand_i[min(answer, (int)total_cand - 1)] : answer;
    }
    __syncthreads();
    if (threadIdx.x == 0) out[blockIdx.x] = sh.answer;
}

}  // namespace b200

extern "C" int b200_argmax_rows(const float* logits, int ld, int* out, int n_rows, int vocab, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0) return b200::kErrBadArgument;
    return b200::launch_pdl(b200::argmax_rows_kernel, dim3(n_rows), dim3(b200::kSampleThreads), 0, stream, logits, ld, out,
                            vocab);
}

// `probs_scratch`: n_rows * vocab floats of workspace, needed only for nucleus sampling (0 < top_p < 1).
extern "C" int b200_sample_rows(const float* logits, int ld, const float* uniforms, int* out, int n_rows, int vocab,
                                float temperature, float top_p, float* probs_scratch, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || !(temperature > 0.f) || top_p < 0.f || top_p > 1.f) return b200::kErrBadArgument;
    if (vocab < 2 && top_p > 0.f && top_p < 1.f) top_p = 1.f;  // the cutoff divides by (n - 1)
    if (top_p > 0.f && top_p < 1.f && probs_scratch == nullptr) return 10003;
    b200::sample_rows_kernel<<<n_rows, b200::kSampleThreads, 0, stream>>>(logits, ld, uniforms, out, vocab,
                                                                          temperature, top_p, probs_scratch);
    return b200::launch_status();
}
