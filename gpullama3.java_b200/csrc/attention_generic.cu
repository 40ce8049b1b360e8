// Causal grouped-query attention over the paged cache, one CTA per (token, query head).
//
// The plain kernel of both precisions: it serves every way of cutting the work (whole prompts,
// chunks that continue a cached prefix, single decoded tokens) because each query token only
// knows its own position and reads keys 0..position of its sequence from the cache, as
// inference/InferenceCore.java:106-145 of the reference project does for one token:
//     score_t = (q . k_t) / sqrt(head_dim),  t <= position      (:116-125)
//     p = softmax(score) (max, exp, sum, divide)                 (:128)
//     out = sum_t p_t v_t                                        (:136-144)
// Query head h reads kv head h / (n_heads / n_kv_heads).  The softmax is computed online over
// tiles of 128 keys in 32-bit.  `window` > 0 keeps only the last `window` keys.
#include "common.cuh"

namespace b200 {

constexpr int kAttnThreads = 128;

template <typename T> struct Vec16;  // 16-byte vector of storage type T
template <> struct Vec16<float> {
    static constexpr int kElems = 4;
    __device__ static void load(const float* p, float* f) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int kElems = 8;
    __device__ static void load(const __nv_bfloat16* p, float* f) {
        const uint4 v = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
};

// Loads are laid out for the cache, not for the arithmetic.  Keys of a page lie row after row ([64 tokens][head_dim]):
// four lanes share a key and read 64 contiguous bytes of its row per step, so a warp instruction covers eight rows
// instead of 32 lines that are head_dim apart; two exchanges give each key its dot product.  Values lie transposed
// ([head_dim][64 tokens]): a lane is a key, a warp instruction reads 32 neighbouring tokens of one dimension, and the
// 32 products of 32 dimensions are summed over the lanes by halving (16 + 8 + 4 + 2 + 1 exchanges), after which
// lane l holds dimension l of the block.  A warp takes 32 keys of each tile of 128; all four share the running maximum.
template <typename T>
__global__ void __launch_bounds__(kAttnThreads)
attention_paged_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out,
                       const int* __restrict__ positions, const int* __restrict__ seq_ids,
                       const int* __restrict__ page_table, int table_stride, const T* __restrict__ k_pool,
                       const T* __restrict__ v_pool, int n_heads, int n_kv_heads, int head_dim, int window,
                       float* __restrict__ part_o, float* __restrict__ part_ml) {
    constexpr int E = Vec16<T>::kElems;     // elements per 16-byte load
    extern __shared__ float smem[];
    float* q_s = smem;                      // [head_dim]
    float* s_s = q_s + head_dim;            // [kAttnThreads] scores of the tile
    float* red = s_s + kAttnThreads;        // [33]
    float* part = red + 33;                 // [4 warps][dim blocks * 32] partial outputs

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int* pages = page_table + (size_t)seq_ids[t] * table_stride;
    const int first = window > 0 ? max(0, pos - window + 1) : 0;
    // With gridDim.z > 1 the keys first .. pos are cut into that many spans of whole tiles, one CTA each, which leave
    // unnormalised partial results (maximum, sum, output) for attention_paged_merge_kernel: a decode step has few
    // (token, head) pairs and long rows of keys.
    const int n_splits = gridDim.z, split = blockIdx.z;
    const int tiles = (pos - first) / kAttnThreads + 1, per_split = (tiles + n_splits - 1) / n_splits;
    const int lo = first + split * per_split * kAttnThreads;
    const int last = min(pos, lo + per_split * kAttnThreads - 1);   // (lo > last: an empty span)
    const size_t page_stride = (size_t)n_kv_heads * kPageTokens * head_dim;
    const size_t head_off = (size_t)g * kPageTokens * head_dim;
    const int dim_blocks = (head_dim + 31) / 32;     // at most 8

    const T* qr = q + (size_t)t * q_row_stride + (size_t)h * head_dim;
    for (int d = tid; d < head_dim; d += kAttnThreads) q_s[d] = to_f32<T>(qr[d]);
    __syncthreads();

    float acc[8];                            // lane l: dimensions 32 b + l of this warp's keys
#pragma unroll
    for (int b = 0; b < 8; ++b) acc[b] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    const float sqrt_d = sqrtf((float)head_dim);
    const int sub = lane & 3;                // which quarter of a key's 16-byte pieces this lane reads
    const int vecs = head_dim / E;           // 16-byte pieces per key row

    for (int base = lo; base <= last; base += kAttnThreads) {
        // ---- scores of this warp's 32 keys, eight keys per step
        const int wbase = base + warp * 32;
#pragma unroll 1
        for (int k8 = 0; k8 < 32; k8 += 8) {
            const int key = wbase + k8 + (lane >> 2);
            float dot = 0.f;
            if (key <= last) {
                const T* kr = k_pool + (size_t)pages[key / kPageTokens] * page_stride + head_off +
                              (size_t)(key % kPageTokens) * head_dim;
                for (int v = sub; v < vecs; v += 4) {
                    float f[E];
                    Vec16<T>::load(kr + v * E, f);
#pragma unroll
                    for (int e = 0; e < E; ++e) dot += q_s[v * E + e] * f[e];
                }
            }
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            if (sub == 0) s_s[warp * 32 + k8 + (lane >> 2)] = dot;
        }
        __syncwarp();
        const int key = base + tid;          // from here on a thread is a key
        const float s = key <= last ? s_s[tid] / sqrt_d : -INFINITY;
        const float m_tile = block_max(s, red);
        const float m_new = fmaxf(m_run, m_tile);
        const float p = key <= last ? expf(s - m_new) : 0.f;
        const float l_tile = block_sum(p, red);
        const float corr = expf(m_run - m_new);  // 0 on the first tile (m_run = -inf)
        l_run = l_run * corr + l_tile;
        m_run = m_new;
        // ---- this warp's 32 keys times their values, 32 dimensions at a time
        const bool any = wbase <= last;       // (uniform in the warp)
        const T* vr = nullptr;
        if (key <= last) vr = v_pool + (size_t)pages[key / kPageTokens] * page_stride + head_off + (key % kPageTokens);
#pragma unroll
        for (int b = 0; b < 8; ++b) {
            if (b >= dim_blocks) break;
            acc[b] *= corr;
            if (!any) continue;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int d = b * 32 + i;
                v[i] = (vr != nullptr && d < head_dim) ? p * to_f32<T>(vr[(size_t)d * kPageTokens]) : 0.f;
            }
            // sum over the lanes by halving: afterwards v[0] of lane l is the sum of everybody's v[l]
#pragma unroll
            for (int half = 16; half >= 1; half >>= 1) {
                const bool upper = (lane & half) != 0;
#pragma unroll
                for (int i = 0; i < half; ++i) {
                    const float send = upper ? v[i] : v[i + half];
                    const float keep = upper ? v[i + half] : v[i];
                    v[i] = keep + __shfl_xor_sync(0xffffffffu, send, half);
                }
            }
            acc[b] += v[0];
        }
    }

    // the four warps' partial outputs meet in shared memory and are added in warp order
#pragma unroll
    for (int b = 0; b < 8; ++b)
        if (b < dim_blocks) part[(warp * dim_blocks + b) * 32 + lane] = acc[b];
    __syncthreads();
    T* o = out + ((size_t)t * n_heads + h) * head_dim;
    const size_t row = ((size_t)t * n_heads + h) * n_splits + split;
    for (int d = tid; d < head_dim; d += kAttnThreads) {
        float a = 0.f;
        for (int w = 0; w < kAttnThreads / 32; ++w) a += part[w * dim_blocks * 32 + d];
        if (n_splits == 1) o[d] = from_f32<T>(a / l_run);
        else part_o[row * head_dim + d] = a;
    }
    if (n_splits > 1 && tid == 0) {
        part_ml[row * 2] = m_run;
        part_ml[row * 2 + 1] = l_run;
    }
}

// out[row] = sum_s o_s exp(m_s - m) / sum_s l_s exp(m_s - m) over the spans of a (token, head) row, in span order
template <typename T>
__global__ void attention_paged_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                             T* __restrict__ out, int n_splits, int head_dim) {
    const size_t row = blockIdx.x;
    const float* ml = part_ml + row * n_splits * 2;
    float m = -INFINITY;
    for (int s = 0; s < n_splits; ++s) m = fmaxf(m, ml[2 * s]);
    for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
        float l = 0.f, acc = 0.f;
        for (int s = 0; s < n_splits; ++s) {
            const float f = ml[2 * s] == -INFINITY ? 0.f : expf(ml[2 * s] - m);
            l += ml[2 * s + 1] * f;
            acc += part_o[(row * n_splits + s) * head_dim + d] * f;
        }
        out[row * head_dim + d] = from_f32<T>(acc / l);
    }
}

}  // namespace b200

// n_splits > 1 cuts every row of keys into that many spans (scratch: n_tokens * n_heads * n_splits * (head_dim + 2)
// floats) and merges them with a second kernel; 1 needs no scratch.
extern "C" int b200_attention_paged(const void* q, int q_row_stride, void* out, int dtype, const int* positions,
                                    const int* seq_ids, const int* page_table, int table_stride, const void* k_pool,
                                    const void* v_pool, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                    int window, int n_splits, float* scratch, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (n_splits < 1 || n_splits > 64 || (n_splits > 1 && scratch == nullptr)) return b200::kErrBadArgument;
    if (head_dim % 16 != 0 || head_dim < 16 || head_dim > 256) return b200::kErrUnsupportedSize;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return b200::kErrBadArgument;
    const size_t smem = sizeof(float) * (head_dim + b200::kAttnThreads + 33 + (size_t)(b200::kAttnThreads / 32) * ((head_dim + 31) / 32) * 32);
    dim3 grid(n_tokens, n_heads, n_splits);
    float* part_o = scratch;
    float* part_ml = scratch != nullptr ? scratch + (size_t)n_tokens * n_heads * n_splits * head_dim : nullptr;
    B200_DISPATCH_DTYPE(dtype, T,
        b200::attention_paged_kernel<T><<<grid, b200::kAttnThreads, smem, stream>>>(
            (const T*)q, q_row_stride, (T*)out, positions, seq_ids, page_table, table_stride, (const T*)k_pool,
            (const T*)v_pool, n_heads, n_kv_heads, head_dim, window, part_o, part_ml);
        if (n_splits > 1)
            b200::attention_paged_merge_kernel<T><<<n_tokens * n_heads, 64, 0, stream>>>(part_o, part_ml, (T*)out, n_splits, head_dim));
    return b200::launch_status();
}
