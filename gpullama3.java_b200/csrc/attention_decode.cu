// Decode attention in bfloat16: one new token per sequence attends over its cached keys and values.
//
// The cache of the live sequences is, next to the weights, what a decode step has to read, so the
// kernel is a stream of K and V pages from HBM.  One CTA takes (a span of keys, one kv head, one
// sequence); the query heads that share the kv head (n_heads / n_kv_heads, up to 16) are the rows
// of the tensor-core tiles, so each key and value is read once for all of them.  Long sequences
// are cut into spans so that a small batch still fills the GPU (`n_splits` per sequence on average;
// a longer sequence of the batch gets more of them, see span_plan); every span leaves an
// unnormalised partial (running max m, sum l, output o) in scratch memory and a second kernel
// merges the spans in a fixed order (no atomics).  The mathematics is the reference's
// (inference/InferenceCore.java:106-145 of the reference project): scores q.k / sqrt(d) over the
// cached positions, softmax, weighted sum of values; the online form with running max is the one
// its GPU kernel uses (tornadovm/TransformerComputeKernelsLayered.java:431-502).
//
// Layouts: keys [page][kv_head][64][d]; values transposed [page][kv_head][d][64].  Both are
// loaded 16 bytes per lane straight into mma.m16n8k16 fragments:
//   S[heads x keys] = Q K^T : K rows are the "col" operand; lane (g, t) takes dims 8t..8t+7 of a
//       key row.  Within a block of 32 keys, tile i column c holds key (c/2)*8 + 2i + (c%2), so
//       that over the four tiles lane t ends up with the probabilities of keys 8t..8t+7 ...
//   O[heads x d] += P V : ... which is exactly one 16-byte load of a V^T row (dim, keys 8t..8t+7).
//
// Fused variant (b200_attention_decode_rope): the step's own rotation and cache write are done
// here instead of in a kernel of their own.  Each CTA rotates the queries of its heads in registers
// (inference/InferenceCore.java:83-95); the CTA of the last span also rotates the new key, stores it
// and the new value at the sequence's last position (:100-101) and feeds that one key to the softmax
// directly as a partial of its own (m = score, l = 1, o = v), so the cache is only ever read for
// positions written by earlier steps.
//
// Sizes: head_dim 32, 64, 96 or 128; group size (heads per kv head) <= 16.  Others are refused.
#include "attention_decode_static.h"
#include <cstdint>
#include "common.cuh"

namespace b200 {

constexpr int kAttnDecodeWarps = 4;
constexpr int kAttnDecodeThreads = kAttnDecodeWarps * 32;

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the same with rows 8..15 of the first operand absent (zero): only the two sums of row g are kept
__device__ __forceinline__ void mma16816_lo(float& d0, float& d1, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    float junk2, junk3;
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%10,%10};"
                 : "+f"(d0), "+f"(d1), "=f"(junk2), "=f"(junk3)
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// keep the first n (0..8) bfloat16 of a 16-byte register group, zero the rest
__device__ __forceinline__ uint4 keep_first(uint4 v, int n) {
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int left = n - 2 * i;
        w[i] = left >= 2 ? w[i] : (left == 1 ? (w[i] & 0xffffu) : 0u);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Partials in scratch: o [span][head][d] floats, then ml [span][head][2] floats, `span` counted over all sequences
// (n_seqs x n_splits of them at most; sequence i's are prefix_i .. prefix_i + count_i - 1 of span_plan).
struct RopeArgs {            // what the fused variant needs beyond the plain one
    const float* inv_freq;   // [head_dim / 2]
    int pairing;             // 0: (2j, 2j+1); 1: (j, j + head_dim/2)
    int write_cache;         // 0: the layer reads a cache another layer wrote in this step (queries are still rotated)
};

// rotated element d of a head's vector x (raw, bfloat16); cs, sn: cosine and sine of the position's angle per pair
__device__ __forceinline__ float rotate_elem(const __nv_bfloat16* x, int d, int D, const float* cs_tab, const float* sn_tab, int pairing) {
    const int half = D / 2;
    int j, d0, d1;
    bool first;
    if (pairing == 0) { j = d >> 1; d0 = d & ~1; d1 = d0 + 1; first = (d & 1) == 0; }
    else { j = d < half ? d : d - half; d0 = j; d1 = j + half; first = d < half; }
    const float sn = sn_tab[j], cs = cs_tab[j];
    const float v0 = __bfloat162float(x[d0]), v1 = __bfloat162float(x[d1]);
    return first ? v0 * cs - v1 * sn : v0 * sn + v1 * cs;
}

// How the n_seqs x n_splits CTAs of a kv head are shared out among the sequences.  Every sequence gets one span and a
// share of the others in proportion to the blocks of 32 keys it reads, so that in a batch of unequal lengths the CTAs of
// the longest sequence do not outlast all others (equal lengths: n_splits each, as if there were no plan).  The spans of
// sequence i are numbered prefix_i .. prefix_i + count_i - 1 among all spans; partial results are stored under that
// number, and the merge kernel evaluates the same plan.  Lengths are read before the dependency wait, like kv_lens[seq].
constexpr int kSpanPlanMaxSeqs = 64;   // larger batches (whose grids fill the GPU with one or two spans) keep equal counts

__device__ __forceinline__ int cached_blocks(const int* __restrict__ kv_lens, int i, int window, bool own_key_apart) {
    const int kv_len = kv_lens[i];
    const int lo = window > 0 ? max(0, kv_len - window) : 0;
    const int n_cached = own_key_apart ? kv_len - 1 : kv_len;
    return n_cached > lo ? (n_cached - 1) / 32 - lo / 32 + 1 : 0;
}

// prefix and count of sequence `seq` (find_cta < 0), or of the sequence that owns CTA number `find_cta`; false if that
// CTA is left over (the counts are rounded down, so up to n_seqs CTAs of a kv head may be)
__device__ __forceinline__ bool span_plan(const int* __restrict__ kv_lens, int n_seqs, int n_splits, int window,
                                          bool own_key_apart, int seq, int find_cta, int& owner, int& prefix, int& count) {
    bool planned = n_splits > 1 && n_seqs <= kSpanPlanMaxSeqs;
    unsigned int total = 0;
    if (planned) {
        for (int i = 0; i < n_seqs; ++i) total += (unsigned int)cached_blocks(kv_lens, i, window, own_key_apart);
        planned = total > 0 && total < (1u << 20);   // (the products below stay inside 32 bits)
    }
    if (!planned) {
        owner = find_cta < 0 ? seq : find_cta / n_splits;
        prefix = owner * n_splits;
        count = n_splits;
        return true;
    }
    const unsigned int spare = (unsigned int)n_seqs * (unsigned int)(n_splits - 1);
    int at = 0;
    bool found = false;
    for (int i = 0; i < n_seqs; ++i) {
        const int c = 1 + (int)((unsigned int)cached_blocks(kv_lens, i, window, own_key_apart) * spare / total);
        if (find_cta < 0 ? i == seq : (find_cta >= at && find_cta < at + c)) {
            owner = i; prefix = at; count = c; found = true;
        }
        at += c;
    }
    return found;
}

// KB: head_dim / 32.  FUSED: rotation and cache write of the step done here.  HI: the group has more than 8 heads,
// so rows 8..15 of the tiles exist (without them a lane keeps half the sums, and more CTAs fit an SM).
template <int KB, bool FUSED, bool HI>
__global__ void __launch_bounds__(kAttnDecodeThreads)
attention_decode_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
                        const int* __restrict__ kv_lens, const int* __restrict__ page_table, int table_stride,
                        __nv_bfloat16* __restrict__ k_pool, __nv_bfloat16* __restrict__ v_pool,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int n_heads, int n_kv_heads,
                        int window, int n_splits, RopeArgs rope) {
    constexpr int D = KB * 32;
    constexpr int NJ = D / 8;  // output tiles of 8 dims
    constexpr int SLOTS = kAttnDecodeWarps + (FUSED ? 1 : 0);  // partials merged per CTA: the warps, and the new key
    // Rows of the tiles that exist: 8 without the upper half.  (Shared memory is taken from the SM's L1, through which the
    // kernel's loads travel: the less of it a CTA holds, the more bytes the SM keeps in flight.)
    constexpr int RS = HI ? 16 : 8;
    extern __shared__ float smem[];  // [SLOTS][RS][D] outputs, [SLOTS][RS][2] (m, l); fused: q [RS][D], k [D], v [D], cos [D/2], sin [D/2]
    float* o_s = smem;
    float* ml_s = smem + SLOTS * RS * D;
    float* q_s = ml_s + SLOTS * RS * 2;
    float* k_s = q_s + RS * D;
    float* v_s = k_s + D;
    float* cs_s = v_s + D;       // fused: cosine and sine of the step's position for each of the D/2 pairs
    float* sn_s = cs_s + D / 2;

    const int kvh = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int group = n_heads / n_kv_heads;
    pdl_launch_dependents();
    // Lengths and page tables were copied to the device before the step's first kernel started, so they are read
    // before the wait for the predecessor; the queries, the step's key and value and the cache are read after it.
    // Which sequence this CTA works for, as which of its spans, and how many spans that sequence has:
    int seq, span_first, span_count;
    if (!span_plan(kv_lens, (int)gridDim.z, n_splits, window, FUSED && rope.write_cache, -1,
                   (int)(blockIdx.z * gridDim.x + blockIdx.x), seq, span_first, span_count)) {
        pdl_wait();   // (a CTA that is left over; it still waits, so that this kernel's end implies its predecessor's)
        return;
    }
    const int split = (int)(blockIdx.z * gridDim.x + blockIdx.x) - span_first;
    const int kv_len = kv_lens[seq];
    const int lo = window > 0 ? max(0, kv_len - window) : 0;
    // keys read from the cache: all of them, or all but the step's own when this kernel writes that one
    const int n_cached = (FUSED && rope.write_cache) ? kv_len - 1 : kv_len;
    const int first_block = lo / 32, last_block = n_cached > lo ? (n_cached - 1) / 32 : first_block - 1;
    const int per_split = max(1, (last_block - first_block + 1 + span_count - 1) / span_count);
    const int blk_begin = first_block + split * per_split;
    const int blk_end = min(blk_begin + per_split, last_block + 1);
    const int* pages = page_table + (size_t)seq * table_stride;
    const size_t page_stride = (size_t)n_kv_heads * kPageTokens * D;
    const size_t head_off = (size_t)kvh * kPageTokens * D;

    const int first_page = blk_begin + warp < blk_end ? pages[(blk_begin + warp) * 32 / kPageTokens] : 0;
    if (FUSED) {
        // The angles of the step's position, once per CTA and before the wait (they need only the length and the
        // frequencies): a lane that evaluated the sines and cosines of its own sixteen dimensions spent more
        // instructions there than on its keys.
        for (int j = threadIdx.x; j < D / 2; j += kAttnDecodeThreads) sincosf((float)(kv_len - 1) * rope.inv_freq[j], &sn_s[j], &cs_s[j]);
        __syncthreads();
    }
    pdl_wait();
    // query fragments: rows = the heads of this group (rows >= group are zero)
    uint4 ql[KB], qh[HI ? KB : 1];
    {
        const __nv_bfloat16* qrow = q + (size_t)seq * q_row_stride + (size_t)kvh * group * D;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            ql[kb] = g < group ? *reinterpret_cast<const uint4*>(qrow + (size_t)g * D + kb * 32 + t * 8) : make_uint4(0, 0, 0, 0);
            if (HI) qh[kb] = g + 8 < group ? *reinterpret_cast<const uint4*>(qrow + (size_t)(g + 8) * D + kb * 32 + t * 8) : make_uint4(0, 0, 0, 0);
        }
        if (FUSED) {
            // rotate in registers.  A lane holds dims 32 kb + 8 t .. + 7 of its rows: interleaved partners sit
            // side by side; half partners (d, d + D/2) sit in blocks kb and kb + KB/2 of the same lane.
            const int pos = kv_len - 1;
            uint32_t* lo32 = reinterpret_cast<uint32_t*>(ql);
            uint32_t* hi32 = reinterpret_cast<uint32_t*>(qh);
            auto unpack = [](uint32_t w, float& a, float& b) { a = __uint_as_float(w << 16); b = __uint_as_float(w & 0xffff0000u); };
            if (rope.pairing == 0) {
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float sn = sn_s[(kb * 32 + t * 8) / 2 + e], cs = cs_s[(kb * 32 + t * 8) / 2 + e];
#pragma unroll
                        for (int h = 0; h < (HI ? 2 : 1); ++h) {
                            uint32_t* w = (h ? hi32 : lo32) + kb * 4 + e;
                            float v0, v1;
                            unpack(*w, v0, v1);
                            *w = pack_bf16(v0 * cs - v1 * sn, v0 * sn + v1 * cs);
                        }
                    }
            } else {
#pragma unroll
                for (int kb = 0; kb < KB / 2; ++kb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float sn[2] = {sn_s[kb * 32 + t * 8 + 2 * e], sn_s[kb * 32 + t * 8 + 2 * e + 1]};
                        const float cs[2] = {cs_s[kb * 32 + t * 8 + 2 * e], cs_s[kb * 32 + t * 8 + 2 * e + 1]};
#pragma unroll
                        for (int h = 0; h < (HI ? 2 : 1); ++h) {
                            uint32_t* wa = (h ? hi32 : lo32) + kb * 4 + e;               // dims d, d + 1
                            uint32_t* wb = (h ? hi32 : lo32) + (kb + KB / 2) * 4 + e;    // dims d + D/2, d + D/2 + 1
                            float a0, a1, b0, b1;
                            unpack(*wa, a0, a1);
                            unpack(*wb, b0, b1);
                            *wa = pack_bf16(a0 * cs[0] - b0 * sn[0], a1 * cs[1] - b1 * sn[1]);
                            *wb = pack_bf16(a0 * sn[0] + b0 * cs[0], a1 * sn[1] + b1 * cs[1]);
                        }
                    }
            }
        }
    }
    float o[NJ][4];
#pragma unroll
    for (int j = 0; j < NJ; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) o[j][i] = 0.f;
    float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;  // rows g and g + 8; l is this lane's share
    // scores are scaled by a multiplication: a division by sqrt(d) that is no power of two (head sizes 32, 96, 128) is a
    // subroutine that, with this kernel's registers all taken, cost more than the block's tensor-core work
    const float inv_sqrt_d = 1.f / sqrtf((float)D);

    for (int blk = blk_begin + warp; blk < blk_end; blk += kAttnDecodeWarps) {
        const int base = blk * 32;
        const size_t page_base = (size_t)(blk == blk_begin + warp ? first_page : pages[base / kPageTokens]) * page_stride + head_off;
        const int in_page = base % kPageTokens;
        const __nv_bfloat16* kp = k_pool + page_base;
        const __nv_bfloat16* vp = v_pool + page_base;

        // all loads of the block are issued before the arithmetic that needs them
        uint4 kf[4][KB];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = (g >> 1) * 8 + 2 * i + (g & 1);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                kf[i][kb] = ldg_stream(kp + (size_t)(in_page + key) * D + kb * 32 + t * 8);
        }
        uint4 vf[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j) vf[j] = ldg_stream(vp + (size_t)(8 * j + g) * kPageTokens + in_page + t * 8);

        float s[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                if (HI) {
                    mma16816(s[i], ql[kb].x, qh[kb].x, ql[kb].y, qh[kb].y, kf[i][kb].x, kf[i][kb].y);
                    mma16816(s[i], ql[kb].z, qh[kb].z, ql[kb].w, qh[kb].w, kf[i][kb].z, kf[i][kb].w);
                } else {
                    mma16816_lo(s[i][0], s[i][1], ql[kb].x, ql[kb].y, kf[i][kb].x, kf[i][kb].y);
                    mma16816_lo(s[i][0], s[i][1], ql[kb].z, ql[kb].w, kf[i][kb].z, kf[i][kb].w);
                }
            }
        }
        // lane t's columns of tile i are keys base + 8t + 2i and + 2i + 1
        float bm_lo = -INFINITY, bm_hi = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = base + 8 * t + 2 * i + e;
                const bool ok = key >= lo && key < n_cached;
                s[i][e] = ok ? s[i][e] * inv_sqrt_d : -INFINITY;
                bm_lo = fmaxf(bm_lo, s[i][e]);
                if (HI) {
                    s[i][2 + e] = ok ? s[i][2 + e] * inv_sqrt_d : -INFINITY;
                    bm_hi = fmaxf(bm_hi, s[i][2 + e]);
                }
            }
        bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 1));
        bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 2));
        if (HI) {
            bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 1));
            bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 2));
        }
        const float mn_lo = fmaxf(m_lo, bm_lo), mn_hi = HI ? fmaxf(m_hi, bm_hi) : 0.f;
        // a block always holds at least one valid key (blocks run from lo/32 to (n_cached-1)/32), so mn is finite
        const float c_lo = expf(m_lo - mn_lo), c_hi = HI ? expf(m_hi - mn_hi) : 0.f;
        m_lo = mn_lo;
        m_hi = mn_hi;
        l_lo *= c_lo;
        l_hi *= c_hi;
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            o[j][0] *= c_lo;
            o[j][1] *= c_lo;
            if (HI) { o[j][2] *= c_hi; o[j][3] *= c_hi; }
        }
        uint32_t pa[4][2];  // per tile: packed probabilities of rows g and g + 8
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float p0 = expf(s[i][0] - mn_lo), p1 = expf(s[i][1] - mn_lo);
            l_lo += p0 + p1;
            pa[i][0] = pack_bf16(p0, p1);
            if (HI) {
                const float p2 = expf(s[i][2] - mn_hi), p3 = expf(s[i][3] - mn_hi);
                l_hi += p2 + p3;
                pa[i][1] = pack_bf16(p2, p3);
            }
        }
        const int n_valid = n_cached - (base + 8 * t);  // keys of this lane's V slice that exist
#pragma unroll
        for (int j = 0; j < NJ; ++j) {
            const uint4 v = n_valid >= 8 ? vf[j] : keep_first(vf[j], max(n_valid, 0));
            if (HI) {
                mma16816(o[j], pa[0][0], pa[0][1], pa[1][0], pa[1][1], v.x, v.y);
                mma16816(o[j], pa[2][0], pa[2][1], pa[3][0], pa[3][1], v.z, v.w);
            } else {
                mma16816_lo(o[j][0], o[j][1], pa[0][0], pa[1][0], v.x, v.y);
                mma16816_lo(o[j][0], o[j][1], pa[2][0], pa[3][0], v.z, v.w);
            }
        }
    }

    // the lanes of a row share l; then the warps of the CTA are merged through shared memory
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    if (HI) {
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
        l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    }
    float* ow = o_s + (size_t)warp * RS * D;
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
        ow[g * D + 8 * j + 2 * t] = o[j][0];
        ow[g * D + 8 * j + 2 * t + 1] = o[j][1];
        if (HI) {   // (without these rows the merge below never reads them: it stops at the group's last head)
            ow[(g + 8) * D + 8 * j + 2 * t] = o[j][2];
            ow[(g + 8) * D + 8 * j + 2 * t + 1] = o[j][3];
        }
    }
    if (t == 0) {
        ml_s[(warp * RS + g) * 2] = m_lo;
        ml_s[(warp * RS + g) * 2 + 1] = l_lo;
        if (HI) {
            ml_s[(warp * RS + g + 8) * 2] = m_hi;
            ml_s[(warp * RS + g + 8) * 2 + 1] = l_hi;
        }
    }
    if (FUSED) {
        // The step's own key and value.  The CTA of the last span stores them at the sequence's last position
        // and adds them to the softmax as one more partial: m = q.k / sqrt(d), l = 1, o = v.
        const bool mine = rope.write_cache && split == span_count - 1;
        if (mine) {
            const int pos = kv_len - 1;
            const __nv_bfloat16* row = q + (size_t)seq * q_row_stride;
            const __nv_bfloat16* k_raw = row + (size_t)n_heads * D + (size_t)kvh * D;
            const __nv_bfloat16* v_raw = k_raw + (size_t)n_kv_heads * D;
            const size_t page_base = (size_t)pages[pos / kPageTokens] * page_stride + head_off;
            for (int d = threadIdx.x; d < D; d += kAttnDecodeThreads) {
                const __nv_bfloat16 kr = __float2bfloat16_rn(rotate_elem(k_raw, d, D, cs_s, sn_s, rope.pairing));
                k_pool[page_base + (size_t)(pos % kPageTokens) * D + d] = kr;
                v_pool[page_base + (size_t)d * kPageTokens + (pos % kPageTokens)] = v_raw[d];
                k_s[d] = __bfloat162float(kr);
                v_s[d] = __bfloat162float(v_raw[d]);
            }
            if (warp == 0) {  // the rotated queries, as the tensor cores see them
                const uint32_t* lo32 = reinterpret_cast<const uint32_t*>(ql);
                const uint32_t* hi32 = reinterpret_cast<const uint32_t*>(qh);
#pragma unroll
                for (int kb = 0; kb < KB; ++kb)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int d = kb * 32 + t * 8 + 2 * e;
                        q_s[g * D + d] = __uint_as_float(lo32[kb * 4 + e] << 16);
                        q_s[g * D + d + 1] = __uint_as_float(lo32[kb * 4 + e] & 0xffff0000u);
                        if (HI) {
                            q_s[(g + 8) * D + d] = __uint_as_float(hi32[kb * 4 + e] << 16);
                            q_s[(g + 8) * D + d + 1] = __uint_as_float(hi32[kb * 4 + e] & 0xffff0000u);
                        }
                    }
            }
        }
        __syncthreads();
        for (int idx = warp; idx < RS; idx += kAttnDecodeWarps) {   // a warp per head: its lanes share the dimensions
            float sc = -INFINITY;
            if (mine && idx < group) {
                float dot = 0.f;
                for (int d = lane; d < D; d += 32) dot += q_s[idx * D + d] * k_s[d];
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
                sc = dot * inv_sqrt_d;
            }
            if (lane == 0) {
                ml_s[(kAttnDecodeWarps * RS + idx) * 2] = sc;
                ml_s[(kAttnDecodeWarps * RS + idx) * 2 + 1] = mine && idx < group ? 1.f : 0.f;
            }
        }
        for (int idx = threadIdx.x; idx < group * D; idx += kAttnDecodeThreads)
            o_s[(size_t)kAttnDecodeWarps * RS * D + idx] = mine ? v_s[idx % D] : 0.f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < group * D; idx += kAttnDecodeThreads) {
        const int row = idx / D, d = idx % D;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < SLOTS; ++w) m = fmaxf(m, ml_s[(w * RS + row) * 2]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < SLOTS; ++w) {
            const float mw = ml_s[(w * RS + row) * 2];
            const float f = mw == -INFINITY ? 0.f : expf(mw - m);
            l += ml_s[(w * RS + row) * 2 + 1] * f;
            acc += o_s[((size_t)w * RS + row) * D + d] * f;
        }
        const int head = kvh * group + row;
        if (n_splits == 1) {
            out[((size_t)seq * n_heads + head) * D + d] = __float2bfloat16_rn(acc / l);
        } else {
            const size_t p = (size_t)(span_first + split) * n_heads + head;
            part_o[p * D + d] = acc;
            if (d == 0) { part_ml[p * 2] = m; part_ml[p * 2 + 1] = l; }
        }
    }
}

// `first`: index of the row's first partial result; the next span's lies `stride` partials further.
template <int N>
__device__ __forceinline__ void merge_spans_at_once(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                    __nv_bfloat16* __restrict__ out, size_t row, size_t first, size_t stride,
                                                    int count, int D) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float ms[N], ls[N], po[N];
#pragma unroll
        for (int j = 0; j < N; ++j) {
            const bool ok = j < count;
            const size_t q = first + (size_t)j * stride;
            ms[j] = ok ? part_ml[2 * q] : -INFINITY;
            ls[j] = ok ? part_ml[2 * q + 1] : 0.f;
            po[j] = ok ? part_o[q * D + d] : 0.f;
        }
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < N; ++j) m = fmaxf(m, ms[j]);
        float l = 0.f, acc = 0.f;
#pragma unroll
        for (int j = 0; j < N; ++j) {
            if (j < count) {
                const float f = ms[j] == -INFINITY ? 0.f : expf(ms[j] - m);
                l += ls[j] * f;
                acc += po[j] * f;
            }
        }
        out[row * D + d] = __float2bfloat16_rn(acc / l);
    }
}

// One CTA per (sequence, head), one thread per dimension.  The sequence's spans are found by the plan the attention
// kernel followed (evaluated before the dependency wait).  The partial results of up to 8 spans are requested
// together before any is used (a loop over a run-time count of spans that loads, scales and adds one span at a time
// pays one round trip to L2 per span); they are added in span order, so the sum is the same.
__global__ void attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                              __nv_bfloat16* __restrict__ out, const int* __restrict__ kv_lens, int n_heads,
                                              int n_splits, int D, int window, int own_key_apart) {
    pdl_launch_dependents();
    const size_t row = blockIdx.x;  // seq * n_heads + head
    const int seq = (int)(blockIdx.x / n_heads), head = (int)(blockIdx.x % n_heads);
    int owner, span_first, count;
    span_plan(kv_lens, (int)(gridDim.x / n_heads), n_splits, window, own_key_apart != 0, seq, -1, owner, span_first, count);
    pdl_wait();
    const size_t first = (size_t)span_first * n_heads + head, stride = (size_t)n_heads;
    // up to 16 spans: everything a thread needs is asked for at once (one trip to L2 instead of one for the maxima and one
    // for the rest, per group of 8 spans); the arithmetic and its order are those of the general path below
    if (count <= 8) { merge_spans_at_once<8>(part_o, part_ml, out, row, first, stride, count, D); return; }
    if (count <= 16) { merge_spans_at_once<16>(part_o, part_ml, out, row, first, stride, count, D); return; }
    float m = -INFINITY;
    for (int s0 = 0; s0 < count; s0 += 8) {
        float ms[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) ms[j] = s0 + j < count ? part_ml[2 * (first + (size_t)(s0 + j) * stride)] : -INFINITY;
#pragma unroll
        for (int j = 0; j < 8; ++j) m = fmaxf(m, ms[j]);
    }
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
        float l = 0.f, acc = 0.f;
        for (int s0 = 0; s0 < count; s0 += 8) {
            float ms[8], ls[8], po[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int sp = s0 + j;
                const bool ok = sp < count;
                const size_t q = first + (size_t)sp * stride;
                ms[j] = ok ? part_ml[2 * q] : -INFINITY;
                ls[j] = ok ? part_ml[2 * q + 1] : 0.f;
                po[j] = ok ? part_o[q * D + d] : 0.f;
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (s0 + j < count) {
                    const float f = ms[j] == -INFINITY ? 0.f : expf(ms[j] - m);
                    l += ls[j] * f;
                    acc += po[j] * f;
                }
            }
        }
        out[row * D + d] = __float2bfloat16_rn(acc / l);
    }
}

}  // namespace b200

// Floats of scratch the call needs for (n_seqs, n_heads, head_dim, n_splits); 0 when n_splits == 1.
extern "C" long long b200_attention_decode_scratch_floats(int n_seqs, int n_heads, int head_dim, int n_splits) {
    if (n_splits <= 1) return 0;
    return (long long)n_seqs * n_heads * n_splits * (head_dim + 2);
}

namespace b200 {

static int launch_attention_decode(const void* q, int q_row_stride, void* out, const int* kv_lens, const int* page_table,
                                   int table_stride, void* k_pool, void* v_pool, float* scratch, long long scratch_floats,
                                   int n_seqs, int n_heads, int n_kv_heads, int head_dim, int window, int n_splits,
                                   bool fused, RopeArgs rope, bool early_start, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0 || n_splits < 1) return kErrBadArgument;
    const int group = n_heads / n_kv_heads;
    if (group > 16 || head_dim % 32 != 0 || head_dim < 32 || head_dim > 128 || q_row_stride % 8 != 0) return kErrUnsupportedSize;
    if (n_seqs > 65535 || n_kv_heads > 65535) return kErrUnsupportedSize;
    // queries, keys and values are read 16 bytes at a time
    if ((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) != 0) return kErrUnsupportedSize;
    if (fused && rope.pairing == 1 && head_dim != 64 && head_dim != 128) return kErrUnsupportedSize;
    if (fused && (rope.pairing < 0 || rope.pairing > 1 || rope.inv_freq == nullptr)) return kErrBadArgument;
    if (scratch_floats < b200_attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits)) return 10003;
    float* part_o = scratch;
    float* part_ml = scratch + (size_t)n_seqs * n_heads * n_splits * head_dim;
    dim3 grid(n_splits, n_kv_heads, n_seqs);
    const int slots = kAttnDecodeWarps + (fused ? 1 : 0);
    const int tile_rows = group > 8 ? 16 : 8;   // rows of the tiles that exist (see the kernel)
    const size_t smem = sizeof(float) * ((size_t)slots * tile_rows * (head_dim + 2) + (fused ? (tile_rows + 3) * head_dim : 0));
    auto qq = (const __nv_bfloat16*)q;
    auto kk = (__nv_bfloat16*)k_pool;
    auto vv = (__nv_bfloat16*)v_pool;
    auto oo = (__nv_bfloat16*)out;
    int st = 0;
#define B200_LAUNCH(KB, F) do { if (group > 8) B200_LAUNCH_H(KB, F, true); else B200_LAUNCH_H(KB, F, false); } while (0)
#define B200_LAUNCH_H(KB, F, HI)                                                                                    \
    do {                                                                                                            \
        auto kernel = attention_decode_kernel<KB, F, HI>;                                                             \
        if (smem > 48 * 1024) {                                                                                     \
            static bool configured = false;                                                                         \
            if (!configured) {                                                                                      \
                if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) \
                    return (int)cudaGetLastError();                                                                 \
                configured = true;                                                                                  \
            }                                                                                                       \
        }                                                                                                           \
        st = launch_pdl_cluster(kernel, grid, dim3(kAttnDecodeThreads), smem, stream, dim3(1, 1, 1), early_start, qq,   \
                                q_row_stride, oo, kv_lens, page_table, table_stride, kk, vv, part_o, part_ml, n_heads,  \
                                n_kv_heads, window, n_splits, rope);                                                 \
    } while (0)
#define B200_PICK(KB) do { if (fused) B200_LAUNCH(KB, true); else B200_LAUNCH(KB, false); } while (0)
    switch (head_dim / 32) {
        case 1: B200_PICK(1); break;
        case 2: B200_PICK(2); break;
        case 3: B200_PICK(3); break;
        default: B200_PICK(4); break;
    }
#undef B200_PICK
#undef B200_LAUNCH
#undef B200_LAUNCH_H
    if (st != 0 || n_splits == 1) return st;
    return launch_pdl(attention_decode_merge_kernel, dim3(n_seqs * n_heads), dim3(head_dim <= 64 ? 64 : 128), 0, stream,
                      (const float*)part_o, (const float*)part_ml, oo, kv_lens, n_heads, n_splits, head_dim, window,
                      (fused && rope.write_cache) ? 1 : 0);
}

}  // namespace b200

// How many CTAs of the kernel for (head_dim, heads per kv head, fused or not) one SM holds at once: what the choice of
// spans should plan for (heads of 64 hold four, heads of 128 two).  0 for sizes the kernel does not take.
extern "C" int b200_attention_decode_ctas_per_sm(int head_dim, int group, int fused) {
    using namespace b200;
    if (group < 1 || group > 16 || head_dim % 32 != 0 || head_dim < 32 || head_dim > 128) return 0;
    const int slots = kAttnDecodeWarps + (fused ? 1 : 0);
    const int tile_rows = group > 8 ? 16 : 8;   // rows of the tiles that exist (see the kernel)
    const size_t smem = sizeof(float) * ((size_t)slots * tile_rows * (head_dim + 2) + (fused ? (tile_rows + 3) * head_dim : 0));
    int n = 0;
    cudaError_t e = cudaSuccess;
#define B200_OCC_H(KB, F, HI)                                                                                          \
    do {                                                                                                              \
        auto kernel = attention_decode_kernel<KB, F, HI>;                                                             \
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e == cudaSuccess) e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kAttnDecodeThreads, smem); \
    } while (0)
#define B200_OCC(KB)                                                                                                   \
    do {                                                                                                              \
        if (fused) { if (group > 8) B200_OCC_H(KB, true, true); else B200_OCC_H(KB, true, false); }                   \
        else { if (group > 8) B200_OCC_H(KB, false, true); else B200_OCC_H(KB, false, false); }                       \
    } while (0)
    switch (head_dim / 32) {
        case 1: B200_OCC(1); break;
        case 2: B200_OCC(2); break;
        case 3: B200_OCC(3); break;
        default: B200_OCC(4); break;
    }
#undef B200_OCC
#undef B200_OCC_H
    if (e != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

// Queries already rotated, keys and values of the step already in the cache.  early_start: whether the kernel
// may be scheduled while its predecessor on the stream still runs (0 for a long kernel that fills the GPU).
extern "C" int b200_attention_decode(const void* q, int q_row_stride, void* out, const int* kv_lens,
                                     const int* page_table, int table_stride, const void* k_pool, const void* v_pool,
                                     float* scratch, long long scratch_floats, int n_seqs, int n_heads, int n_kv_heads,
                                     int head_dim, int window, int n_splits, int early_start, cudaStream_t stream) {
    return b200::launch_attention_decode(q, q_row_stride, out, kv_lens, page_table, table_stride, const_cast<void*>(k_pool),
                                         const_cast<void*>(v_pool), scratch, scratch_floats, n_seqs, n_heads, n_kv_heads,
                                         head_dim, window, n_splits, false, b200::RopeArgs{nullptr, 0, 0}, early_start != 0, stream);
}

// The fused variant: `qkv` holds the step's raw projections [n_seqs, (n_heads + 2 n_kv_heads) head_dim]; queries
// are rotated here, and with write_cache the new key (rotated) and value are stored at position kv_len - 1.
// Rotary dimension = head_dim.  Half pairing needs head_dim 64 or 128.
extern "C" int b200_attention_decode_rope(const void* qkv, int q_row_stride, void* out, const int* kv_lens,
                                          const int* page_table, int table_stride, void* k_pool, void* v_pool,
                                          float* scratch, long long scratch_floats, int n_seqs, int n_heads,
                                          int n_kv_heads, int head_dim, int window, int n_splits, const float* inv_freq,
                                          int pairing, int write_cache, int early_start, cudaStream_t stream) {
    return b200::launch_attention_decode(qkv, q_row_stride, out, kv_lens, page_table, table_stride, k_pool, v_pool, scratch,
                                         scratch_floats, n_seqs, n_heads, n_kv_heads, head_dim, window, n_splits, true,
                                         b200::RopeArgs{inv_freq, pairing, write_cache}, early_start != 0, stream);
}

// ---------------------------------------------------------------------------------------------
// The variant with built-in scratch (see attention_decode_static.h for who needs it and why).
namespace b200 {

constexpr long long kStaticScratchFloats = 2ll << 20;  // 2 Mi floats = 8 MiB per GPU that loads this library
constexpr int kErrStaticScratchExceeded = 10004;
constexpr int kMaxDevices = 64;

// In host code this name is only a handle of the symbol, not a device address: the address each
// device gave the array is looked up below and it is that pointer the kernels receive.
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static float* g_static_scratch_address[kMaxDevices];  // per device; filled by the first call on it

}  // namespace b200

extern "C" long long b200_attention_decode_static_capacity(void) { return b200::kStaticScratchFloats; }

extern "C" int b200_attention_decode_static(const void* q, int q_row_stride, void* out, const int* kv_lens,
                                            const int* page_table, int table_stride, const void* k_pool,
                                            const void* v_pool, int n_seqs, int n_heads, int n_kv_heads, int head_dim,
                                            int window, int n_splits, cudaStream_t stream) {
    using namespace b200;
    if (n_seqs <= 0) return 0;
    if (n_splits < 1) return kErrBadArgument;
    const long long need = b200_attention_decode_scratch_floats(n_seqs, n_heads, head_dim, n_splits);
    if (need > kStaticScratchFloats) return kErrStaticScratchExceeded;
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= kMaxDevices) return kErrBadArgument;
    float* scratch = g_static_scratch_address[device];
    if (scratch == nullptr) {  // set-up, once per device, with that device current
        e = cudaGetSymbolAddress((void**)&scratch, g_static_scratch);
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_address[device] = scratch;
    }
    // Not started early: the kernel reads kv_lens and page_table as soon as it is scheduled, and a caller of
    // this entry point may well have written them with the kernel just before it on the stream.
    return b200_attention_decode(q, q_row_stride, out, kv_lens, page_table, table_stride, k_pool, v_pool, scratch,
                                 kStaticScratchFloats, n_seqs, n_heads, n_kv_heads, head_dim, window, n_splits, 0, stream);
}
