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
// token.  Equal probabilities are ordered by index in the nucleus.
#include <limits.h>
#include "common.cuh"

namespace b200 {

constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;

__global__ void __launch_bounds__(kSampleThreads)
argmax_rows_kernel(const float* __restrict__ logits, int ld, int* __restrict__ out, int V) {
    __shared__ float best_s[kSampleWarps];
    __shared__ int idx_s[kSampleWarps];
    pdl_launch_dependents();
    pdl_wait();
    const float* row = logits + (size_t)blockIdx.x * ld;
    float best = -INFINITY;
    int idx = INT_MAX;
    for (int i = threadIdx.x; i < V; i += kSampleThreads) {
        const float v = row[i];
        if (v > best) { best = v; idx = i; }
    }
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
    unsigned long long hist_mass[256];
    unsigned int hist_cnt[256];
    float seg_sum[kSampleWarps];
    unsigned int seg_cnt[kSampleWarps];
    float red[33];
    // results of one radix descent
    unsigned int key;
    unsigned long long above, mass_eq;
    unsigned int cnt_eq;
    int found;
    int answer;
};

constexpr double kMassScale = 1099511627776.0;  // 2^40: probabilities become integers, sums exact

// Walks the candidates (p >= cutoff) in descending order of p and stops at the value where the
// running mass first exceeds `target`.  Leaves in sh: the bits of that value, the mass strictly
// above it, and the count and mass of the candidates equal to it.  found = 0 when the whole
// candidate mass does not exceed target (then `above` is that whole mass).
__device__ void radix_descent(const float* row, int V, float temperature, float zmax, float total, float cutoff,
                              unsigned long long target, SampleShared& sh) {
    unsigned int prefix = 0;
    unsigned long long above = 0;
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int b = threadIdx.x; b < 256; b += kSampleThreads) { sh.hist_mass[b] = 0; sh.hist_cnt[b] = 0; }
        __syncthreads();
        for (int base = 0; base < V; base += kSampleThreads) {
            const int i = base + threadIdx.x;
            int bin = -1;
            unsigned long long q = 0;
            if (i < V) {
                const float p = expf(row[i] / temperature - zmax) / total;
                if (p >= cutoff) {
                    const unsigned int key = __float_as_uint(p);
                    if (pass == 0 || (key >> (shift + 8)) == (prefix >> (shift + 8))) {
                        bin = (key >> shift) & 255;
                        q = (unsigned long long)((double)p * kMassScale);
                    }
                }
            }
            int all_same;
            __match_all_sync(0xffffffffu, bin, &all_same);
            if (all_same) {  // the common case in a flat distribution: one atomic for the warp
                if (bin >= 0) {
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
                    if ((threadIdx.x & 31) == 0) {
                        atomicAdd(&sh.hist_mass[bin], q);
                        atomicAdd(&sh.hist_cnt[bin], 32u);
                    }
                }
            } else if (bin >= 0) {
                atomicAdd(&sh.hist_mass[bin], q);
                atomicAdd(&sh.hist_cnt[bin], 1u);
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            unsigned long long cum = above;
            int chosen = -1;
            for (int b = 255; b >= 0; --b) {
                if (sh.hist_cnt[b] == 0) continue;
                if (cum + sh.hist_mass[b] > target) { chosen = b; break; }
                cum += sh.hist_mass[b];
            }
            sh.above = cum;
            sh.found = chosen >= 0;
            if (chosen >= 0) {
                sh.key = prefix | ((unsigned int)chosen << shift);
                sh.mass_eq = sh.hist_mass[chosen];
                sh.cnt_eq = sh.hist_cnt[chosen];
            }
        }
        __syncthreads();
        if (!sh.found) return;
        prefix = sh.key;
        above = sh.above;
        __syncthreads();
    }
}

__global__ void __launch_bounds__(kSampleThreads)
sample_rows_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ uniforms,
                   int* __restrict__ out, int V, float temperature, float top_p) {
    __shared__ SampleShared sh;
    const float* row = logits + (size_t)blockIdx.x * ld;
    const float u = uniforms[blockIdx.x];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

    // each warp owns a contiguous segment of the vocabulary so that prefix sums run in index order
    const int seg = (((V + kSampleWarps - 1) / kSampleWarps + 31) / 32) * 32;
    const int seg_lo = min(V, warp * seg), seg_hi = min(V, (warp + 1) * seg);

    float zmax = -INFINITY;
    for (int i = threadIdx.x; i < V; i += kSampleThreads) zmax = fmaxf(zmax, row[i] / temperature);
    zmax = block_max(zmax, sh.red);

    float part = 0.f;
    for (int i = seg_lo + lane; i < seg_hi; i += 32) part += expf(row[i] / temperature - zmax);
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
            float running = excl;
            int answer = seg_hi - 1;
            for (int base = seg_lo; base < seg_hi; base += 32) {
                const int i = base + lane;
                float e = i < seg_hi ? expf(row[i] / temperature - zmax) : 0.f;
#pragma unroll
                for (int o = 1; o < 32; o <<= 1) {
                    const float n = __shfl_up_sync(0xffffffffu, e, o);
                    if (lane >= o) e += n;
                }
                const unsigned hit = __ballot_sync(0xffffffffu, i < seg_hi && target < running + e);
                if (hit) { answer = base + __ffs(hit) - 1; break; }
                running += __shfl_sync(0xffffffffu, e, 31);
            }
            if (lane == 0) sh.answer = answer;
        }
        __syncthreads();
        if (threadIdx.x == 0) out[blockIdx.x] = sh.answer;
        return;
    }

    // nucleus: the kept set is the shortest descending prefix of the candidates whose mass exceeds top_p
    float cutoff = (1.0f - top_p) / (float)(V - 1);
    const unsigned long long target1 = (unsigned long long)((double)top_p * kMassScale);
    radix_descent(row, V, temperature, zmax, total, cutoff, target1, sh);
    unsigned long long kept_mass;
    if (sh.found) {
        const unsigned long long q1 = sh.cnt_eq ? sh.mass_eq / sh.cnt_eq : 0;
        unsigned long long m = q1 ? (target1 - sh.above) / q1 + 1 : sh.cnt_eq;
        if (m > sh.cnt_eq) m = sh.cnt_eq;
        kept_mass = sh.above + m * q1;
    } else {
        kept_mass = sh.above;
    }
    __syncthreads();
    unsigned long long target2;
    if (kept_mass == 0) {  // no candidate passes the cutoff: take the most probable token
        cutoff = 0.f;
        target2 = 0;
    } else {
        target2 = (unsigned long long)((double)u * (double)kept_mass);
        if (target2 >= kept_mass) target2 = kept_mass - 1;
    }
    radix_descent(row, V, temperature, zmax, total, cutoff, target2, sh);
    if (!sh.found) {  // cannot happen while target2 < kept mass; keep the last index as the reference's fallback
        if (threadIdx.x == 0) out[blockIdx.x] = V - 1;
        return;
    }
    const unsigned int key2 = sh.key;
    const unsigned long long q2 = sh.cnt_eq ? sh.mass_eq / sh.cnt_eq : 0;
    unsigned long long m2 = q2 ? (target2 - sh.above) / q2 + 1 : 1;
    if (m2 > sh.cnt_eq) m2 = sh.cnt_eq;
    if (m2 < 1) m2 = 1;
    __syncthreads();

    // the m2-th token, in index order, whose probability has exactly the bits key2
    unsigned int cnt = 0;
    for (int i = seg_lo + lane; i < seg_hi; i += 32) {
        const float p = expf(row[i] / temperature - zmax) / total;
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
        int answer = seg_hi - 1;
        for (int base = seg_lo; base < seg_hi; base += 32) {
            const int i = base + lane;
            bool match = false;
            if (i < seg_hi) {
                const float p = expf(row[i] / temperature - zmax) / total;
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
        if (lane == 0) sh.answer = answer;
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

extern "C" int b200_sample_rows(const float* logits, int ld, const float* uniforms, int* out, int n_rows, int vocab,
                                float temperature, float top_p, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    if (vocab <= 0 || !(temperature > 0.f) || top_p < 0.f || top_p > 1.f) return b200::kErrBadArgument;
    if (vocab < 2 && top_p > 0.f && top_p < 1.f) top_p = 1.f;  // the cutoff divides by (n - 1)
    b200::sample_rows_kernel<<<n_rows, b200::kSampleThreads, 0, stream>>>(logits, ld, uniforms, out, vocab,
                                                                          temperature, top_p);
    return b200::launch_status();
}
