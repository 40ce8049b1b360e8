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

template <typename T>
__global__ void __launch_bounds__(kAttnThreads)
attention_paged_kernel(const T* __restrict__ q, int q_row_stride, T* __restrict__ out,
                       const int* __restrict__ positions, const int* __restrict__ seq_ids,
                       const int* __restrict__ page_table, int table_stride, const T* __restrict__ k_pool,
                       const T* __restrict__ v_pool, int n_heads, int n_kv_heads, int head_dim, int window) {
    extern __shared__ float smem[];
    float* q_s = smem;                      // [head_dim]
    float* s_s = q_s + head_dim;            // [kAttnThreads] scores / probabilities of the tile
    float* red = s_s + kAttnThreads;        // [33]
    float* part = red + 33;                 // [groups * head_dim] partial outputs

    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int g = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int* pages = page_table + (size_t)seq_ids[t] * table_stride;
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const size_t page_stride = (size_t)n_kv_heads * kPageTokens * head_dim;
    const size_t head_off = (size_t)g * kPageTokens * head_dim;

    const T* qr = q + (size_t)t * q_row_stride + (size_t)h * head_dim;
    for (int d = tid; d < head_dim; d += kAttnThreads) q_s[d] = to_f32<T>(qr[d]);
    __syncthreads();

    // output mapping: `groups` groups of threads share the keys of a tile; a thread owns up to two dims
    const int groups = head_dim <= kAttnThreads ? kAttnThreads / head_dim : 1;
    const bool active = head_dim <= kAttnThreads ? tid < groups * head_dim : true;
    const int grp = head_dim <= kAttnThreads ? tid / head_dim : 0;
    const int d0 = head_dim <= kAttnThreads ? tid % head_dim : tid;
    const int d1 = d0 + kAttnThreads;  // used only when head_dim > kAttnThreads
    float acc0 = 0.f, acc1 = 0.f, m_run = -INFINITY, l_run = 0.f;
    const float sqrt_d = sqrtf((float)head_dim);

    for (int base = lo; base <= pos; base += kAttnThreads) {
        const int key = base + tid;
        float s = -INFINITY;
        if (key <= pos) {
            const T* kr = k_pool + (size_t)pages[key / kPageTokens] * page_stride + head_off +
                          (size_t)(key % kPageTokens) * head_dim;
            float dot = 0.f;
            for (int d = 0; d < head_dim; d += Vec16<T>::kElems) {
                float f[Vec16<T>::kElems];
                Vec16<T>::load(kr + d, f);
#pragma unroll
                for (int e = 0; e < Vec16<T>::kElems; ++e) dot += q_s[d + e] * f[e];
            }
            s = dot / sqrt_d;
        }
        const float m_tile = block_max(s, red);
        const float m_new = fmaxf(m_run, m_tile);
        const float p = key <= pos ? expf(s - m_new) : 0.f;
        s_s[tid] = p;
        const float l_tile = block_sum(p, red);  // contains the barrier that publishes s_s
        const float corr = expf(m_run - m_new);  // 0 on the first tile (m_run = -inf)
        l_run = l_run * corr + l_tile;
        m_run = m_new;
        acc0 *= corr;
        acc1 *= corr;
        if (active) {
            const int n_keys = min(kAttnThreads, pos - base + 1);
            for (int i = grp; i < n_keys; i += groups) {
                const int kk = base + i;
                // values are stored transposed: [head_dim][kPageTokens] per page and kv head
                const T* vr = v_pool + (size_t)pages[kk / kPageTokens] * page_stride + head_off + (kk % kPageTokens);
                const float pi = s_s[i];
                if (d0 < head_dim) acc0 += pi * to_f32<T>(vr[(size_t)d0 * kPageTokens]);
                if (d1 < head_dim) acc1 += pi * to_f32<T>(vr[(size_t)d1 * kPageTokens]);
            }
        }
        __syncthreads();
    }

    T* o = out + ((size_t)t * n_heads + h) * head_dim;
    if (head_dim <= kAttnThreads) {
        if (active) part[grp * head_dim + d0] = acc0;
        __syncthreads();
        if (tid < head_dim) {
            float a = 0.f;
            for (int gi = 0; gi < groups; ++gi) a += part[gi * head_dim + tid];
            o[tid] = from_f32<T>(a / l_run);
        }
    } else {
        if (d0 < head_dim) o[d0] = from_f32<T>(acc0 / l_run);
        if (d1 < head_dim) o[d1] = from_f32<T>(acc1 / l_run);
    }
}

}  // namespace b200

extern "C" int b200_attention_paged(const void* q, int q_row_stride, void* out, int dtype, const int* positions,
                                    const int* seq_ids, const int* page_table, int table_stride, const void* k_pool,
                                    const void* v_pool, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                    int window, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (head_dim % 16 != 0 || head_dim < 16 || head_dim > 256) return b200::kErrUnsupportedSize;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return b200::kErrBadArgument;
    const int groups = head_dim <= b200::kAttnThreads ? b200::kAttnThreads / head_dim : 1;
    const size_t smem = sizeof(float) * (head_dim + b200::kAttnThreads + 33 + (size_t)groups * head_dim);
    dim3 grid(n_tokens, n_heads);
    B200_DISPATCH_DTYPE(dtype, T,
        b200::attention_paged_kernel<T><<<grid, b200::kAttnThreads, smem, stream>>>(
            (const T*)q, q_row_stride, (T*)out, positions, seq_ids, page_table, table_stride, (const T*)k_pool,
            (const T*)v_pool, n_heads, n_kv_heads, head_dim, window));
    return b200::launch_status();
}
