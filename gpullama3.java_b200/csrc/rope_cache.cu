// Rotary position encoding of queries and keys, fused with the write of keys and values into
// the paged cache.
//
// For the pair (v0, v1) of one head with inverse frequency f_j at position p:
//     a = p * f_j (32-bit) ;  v0' = v0 cos a - v1 sin a ;  v1' = v0 sin a + v1 cos a
// which is inference/InferenceCore.java:83-95 with the table of inference/operation/RoPE.java:30-32
// (reference project paths) evaluated in place of looked up.  Keys are cached rotated, values
// untouched (InferenceCore.java:100-101).  `pairing` 0 pairs (2j, 2j+1) as the reference does;
// 1 pairs (j, j + rotary_dim/2), the layout of checkpoints whose q/k rows were not permuted.
// Dimensions at and beyond rotary_dim pass through unrotated.
//
// Cache layout of one cache entry.  Keys: [page][kv_head][kPageTokens][head_dim] (a row per
// position).  Values: [page][kv_head][head_dim][kPageTokens] (transposed: a row per dimension,
// positions contiguous), which is the operand layout the attention kernels multiply
// probabilities with.  The page of position p of sequence s is
// page_table[s * table_stride + p / kPageTokens].
#include "common.cuh"

namespace b200 {

constexpr int kMaxRotaryPairs = 256;  // rotary_dim <= 512

template <typename T>
__global__ void rope_cache_write_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                        const int* __restrict__ seq_ids, const int* __restrict__ page_table,
                                        int table_stride, const float* __restrict__ inv_freq, T* __restrict__ k_pool,
                                        T* __restrict__ v_pool, int n_heads, int n_kv_heads, int head_dim,
                                        int rotary_dim, int pairing, int write_cache) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int q_dim = n_heads * head_dim, kv_dim = n_kv_heads * head_dim;
    T* row = qkv + (size_t)t * (q_dim + 2 * kv_dim);
    const int half = rotary_dim / 2;

    size_t cache_base = 0, v_base = 0;
    if (write_cache) {
        const int page = page_table[(size_t)seq_ids[t] * table_stride + pos / kPageTokens];
        cache_base = ((size_t)page * n_kv_heads * kPageTokens + (pos % kPageTokens)) * head_dim;
        v_base = (size_t)page * n_kv_heads * kPageTokens * head_dim + (pos % kPageTokens);
    }
    const size_t head_stride = (size_t)kPageTokens * head_dim;

    // the angles of this position are the same for every head: one sine and cosine per frequency
    __shared__ float sin_s[kMaxRotaryPairs], cos_s[kMaxRotaryPairs];
    for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf((float)pos * inv_freq[j], &sin_s[j], &cos_s[j]);
    __syncthreads();

    // rotated pairs of queries (in place) and keys (into the cache)
    const int n_units = (n_heads + n_kv_heads) * half;
    for (int u = threadIdx.x; u < n_units; u += blockDim.x) {
        const int h = u / half, j = u % half;
        const int i0 = pairing == 0 ? 2 * j : j;
        const int i1 = pairing == 0 ? 2 * j + 1 : j + half;
        const float s = sin_s[j], c = cos_s[j];
        if (h < n_heads) {
            T* v = row + h * head_dim;
            const float v0 = to_f32<T>(v[i0]), v1 = to_f32<T>(v[i1]);
            v[i0] = from_f32<T>(v0 * c - v1 * s);
            v[i1] = from_f32<T>(v0 * s + v1 * c);
        } else if (write_cache) {
            const int g = h - n_heads;
            const T* v = row + q_dim + g * head_dim;
            const float v0 = to_f32<T>(v[i0]), v1 = to_f32<T>(v[i1]);
            T* dst = k_pool + cache_base + g * head_stride;
            dst[i0] = from_f32<T>(v0 * c - v1 * s);
            dst[i1] = from_f32<T>(v0 * s + v1 * c);
        }
    }
    if (!write_cache) return;
    // unrotated tail of the keys, and the values
    const int tail = head_dim - rotary_dim;
    for (int u = threadIdx.x; u < n_kv_heads * tail; u += blockDim.x) {
        const int g = u / tail, d = rotary_dim + u % tail;
        k_pool[cache_base + g * head_stride + d] = row[q_dim + g * head_dim + d];
    }
    for (int u = threadIdx.x; u < kv_dim; u += blockDim.x) {
        const int g = u / head_dim, d = u % head_dim;
        v_pool[v_base + g * head_stride + (size_t)d * kPageTokens] = row[q_dim + kv_dim + u];
    }
}

}  // namespace b200

extern "C" int b200_rope_cache_write(void* qkv, int dtype, const int* positions, const int* seq_ids,
                                     const int* page_table, int table_stride, const float* inv_freq, void* k_pool,
                                     void* v_pool, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     int rotary_dim, int pairing, int write_cache, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) || (pairing != 0 && pairing != 1))
        return b200::kErrBadArgument;
    if (rotary_dim / 2 > b200::kMaxRotaryPairs) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(dtype, T,
        return b200::launch_pdl(b200::rope_cache_write_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)qkv,
                                positions, seq_ids, page_table, table_stride, inv_freq, (T*)k_pool, (T*)v_pool, n_heads,
                                n_kv_heads, head_dim, rotary_dim, pairing, write_cache));
    return b200::launch_status();
}
