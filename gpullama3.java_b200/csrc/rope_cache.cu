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

// The same for many tokens (prompts): one CTA takes kRopeTile consecutive tokens, moves 16 bytes per access,
// and writes the values of a run of tokens that lies aligned in one page as whole 32-byte pieces of the
// transposed rows instead of one element at a time.  Needs rotary_dim == head_dim and vectors that do not
// straddle a pair's halves; the launcher falls back to the kernel above otherwise.
constexpr int kRopeTile = 16;
constexpr int kRopeThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kRopeThreads)
rope_cache_write_tiled_kernel(T* __restrict__ qkv, const int* __restrict__ positions, const int* __restrict__ seq_ids,
                              const int* __restrict__ page_table, int table_stride, const float* __restrict__ inv_freq,
                              T* __restrict__ k_pool, T* __restrict__ v_pool, int n_tokens, int n_heads, int n_kv_heads,
                              int head_dim, int pairing, int write_cache) {
    constexpr int VEC = 16 / (int)sizeof(T);
    extern __shared__ __align__(16) unsigned char rope_smem[];
    const int half = head_dim / 2;
    float* sin_s = reinterpret_cast<float*>(rope_smem);              // [tile][half]
    float* cos_s = sin_s + kRopeTile * half;                         // [tile][half]
    T* v_s = reinterpret_cast<T*>(cos_s + kRopeTile * half);         // [tile][kv_dim]
    __shared__ int pos_s[kRopeTile], page_s[kRopeTile];
    __shared__ int aligned_s;
    pdl_launch_dependents();
    pdl_wait();
    const int t0 = blockIdx.x * kRopeTile, n_here = min(kRopeTile, n_tokens - t0);
    const int q_dim = n_heads * head_dim, kv_dim = n_kv_heads * head_dim, row_len = q_dim + 2 * kv_dim;
    if (threadIdx.x < kRopeTile) {
        const int i = threadIdx.x;
        const int pos = i < n_here ? positions[t0 + i] : 0;
        pos_s[i] = pos;
        page_s[i] = (i < n_here && write_cache) ? page_table[(size_t)seq_ids[t0 + i] * table_stride + pos / kPageTokens] : 0;
    }
    __syncthreads();
    if (threadIdx.x == 0) {  // a full tile of one page, positions pos0 .. pos0 + 15 with pos0 a multiple of 16?
        bool aligned = n_here == kRopeTile && (pos_s[0] % kRopeTile) == 0;
        for (int i = 1; i < kRopeTile && aligned; ++i) aligned = pos_s[i] == pos_s[0] + i && page_s[i] == page_s[0];
        aligned_s = aligned ? 1 : 0;
    }
    for (int u = threadIdx.x; u < n_here * half; u += kRopeThreads)
        sincosf((float)pos_s[u / half] * inv_freq[u % half], &sin_s[u], &cos_s[u]);
    // The columns of a tile are cut among the CTAs of grid.y, so that a prompt of a few thousand tokens still gives
    // every SM several CTAs: this one takes units [w_lo, w_hi) of every token and value columns [c_lo, c_hi).
    const int slice = blockIdx.y, n_slices = gridDim.y;
    const int c_lo = (int)((long long)(kv_dim / VEC) * slice / n_slices) * VEC;
    const int c_hi = (int)((long long)(kv_dim / VEC) * (slice + 1) / n_slices) * VEC;
    const int c_n = c_hi - c_lo;
    // values of the tile into shared memory, 16 bytes at a time
    if (write_cache) {
        const int vecs = c_n / VEC;
        for (int u = threadIdx.x; u < n_here * vecs; u += kRopeThreads) {
            const int i = u / vecs, v = u % vecs;
            *reinterpret_cast<uint4*>(v_s + (size_t)i * c_n + v * VEC) =
                *reinterpret_cast<const uint4*>(qkv + (size_t)(t0 + i) * row_len + q_dim + kv_dim + c_lo + v * VEC);
        }
    }
    __syncthreads();

    // queries (in place) and keys (into the cache): a unit is one vector of a head and, for the half pairing, its partner
    const int vec_per_head = pairing == 0 ? head_dim / VEC : half / VEC;
    const int units_per_token = (n_heads + (write_cache ? n_kv_heads : 0)) * vec_per_head;
    const size_t head_stride = (size_t)kPageTokens * head_dim;
    // Four units per thread are read before the first is rotated and written: a unit is a dependent read, rotate,
    // write, and one at a time the kernel waits for memory four times as often.
    constexpr int kBatch = 4;
    const int w_lo = (int)((long long)units_per_token * slice / n_slices);
    const int w_n = (int)((long long)units_per_token * (slice + 1) / n_slices) - w_lo;
    const int n_units = n_here * w_n;
    for (int u0 = threadIdx.x; u0 < n_units; u0 += kRopeThreads * kBatch) {
        uint4 lo[kBatch], hi[kBatch];
        T* dst[kBatch];
        int tok[kBatch], vec[kBatch];
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            const int u = u0 + b * kRopeThreads;
            if (u >= n_units) { dst[b] = nullptr; continue; }
            const int i = u / w_n, w = w_lo + u % w_n;
            const int h = w / vec_per_head, v = w % vec_per_head;
            T* src = qkv + (size_t)(t0 + i) * row_len + (size_t)h * head_dim;  // query heads, then key heads: contiguous
            dst[b] = src;
            if (h >= n_heads)
                dst[b] = k_pool + ((size_t)page_s[i] * n_kv_heads * kPageTokens + (pos_s[i] % kPageTokens)) * head_dim +
                         (size_t)(h - n_heads) * head_stride;
            tok[b] = i;
            vec[b] = v;
            lo[b] = *reinterpret_cast<const uint4*>(src + v * VEC);
            if (pairing != 0) hi[b] = *reinterpret_cast<const uint4*>(src + half + v * VEC);
        }
#pragma unroll
        for (int b = 0; b < kBatch; ++b) {
            if (dst[b] == nullptr) continue;
            const float* sn = sin_s + tok[b] * half;
            const float* cs = cos_s + tok[b] * half;
            const int v = vec[b];
            if (pairing == 0) {
                T* e = reinterpret_cast<T*>(&lo[b]);
#pragma unroll
                for (int k = 0; k < VEC; k += 2) {
                    const int j = (v * VEC + k) / 2;
                    const float v0 = to_f32<T>(e[k]), v1 = to_f32<T>(e[k + 1]);
                    e[k] = from_f32<T>(v0 * cs[j] - v1 * sn[j]);
                    e[k + 1] = from_f32<T>(v0 * sn[j] + v1 * cs[j]);
                }
                *reinterpret_cast<uint4*>(dst[b] + v * VEC) = lo[b];
            } else {
                T* a = reinterpret_cast<T*>(&lo[b]);
                T* c = reinterpret_cast<T*>(&hi[b]);
#pragma unroll
                for (int k = 0; k < VEC; ++k) {
                    const int j = v * VEC + k;
                    const float v0 = to_f32<T>(a[k]), v1 = to_f32<T>(c[k]);
                    a[k] = from_f32<T>(v0 * cs[j] - v1 * sn[j]);
                    c[k] = from_f32<T>(v0 * sn[j] + v1 * cs[j]);
                }
                *reinterpret_cast<uint4*>(dst[b] + v * VEC) = lo[b];
                *reinterpret_cast<uint4*>(dst[b] + half + v * VEC) = hi[b];
            }
        }
    }
    if (!write_cache) return;
    // values, transposed: row (kv head, dim) of the page gets the tile's positions
    if (aligned_s) {
        const size_t base = (size_t)page_s[0] * n_kv_heads * head_stride + (pos_s[0] % kPageTokens);
        for (int u = threadIdx.x; u < c_n; u += kRopeThreads) {
            const int g = (c_lo + u) / head_dim, d = (c_lo + u) % head_dim;
            alignas(16) T run[kRopeTile];
#pragma unroll
            for (int i = 0; i < kRopeTile; ++i) run[i] = v_s[(size_t)i * c_n + u];
            uint4* dst = reinterpret_cast<uint4*>(v_pool + base + g * head_stride + (size_t)d * kPageTokens);
#pragma unroll
            for (int q = 0; q < (int)(kRopeTile * sizeof(T) / 16); ++q) dst[q] = reinterpret_cast<const uint4*>(run)[q];
        }
    } else {
        for (int u = threadIdx.x; u < n_here * c_n; u += kRopeThreads) {
            const int i = u / c_n, w = c_lo + u % c_n, g = w / head_dim, d = w % head_dim;
            v_pool[(size_t)page_s[i] * n_kv_heads * head_stride + g * head_stride + (size_t)d * kPageTokens +
                   (pos_s[i] % kPageTokens)] = v_s[u];
        }
    }
}

// Cosine and sine of position * frequency for every token of a pass and every pair of a head: what a product that
// rotates in its own epilogue reads instead of evaluating them once per head.  The same expression as in the kernels above.
__global__ void rope_angles_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                   float2* __restrict__ out, int n_tokens, int half) {
    pdl_launch_dependents();
    pdl_wait();
    const int u = blockIdx.x * blockDim.x + threadIdx.x;   // pair-major: out[pair][token]
    if (u >= n_tokens * half) return;
    float sn, cs;
    sincosf((float)positions[u % n_tokens] * inv_freq[u / n_tokens], &sn, &cs);
    out[u] = make_float2(cs, sn);
}

}  // namespace b200

// out [half][n_tokens] pairs (cos, sin), float32
extern "C" int b200_rope_angles(const int* positions, const float* inv_freq, float* out, int n_tokens, int half,
                                cudaStream_t stream) {
    if (n_tokens <= 0 || half <= 0) return 0;
    const long long n = (long long)n_tokens * half;
    return b200::launch_pdl(b200::rope_angles_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, positions, inv_freq,
                            reinterpret_cast<float2*>(out), n_tokens, half);
}

extern "C" int b200_rope_cache_write(void* qkv, int dtype, const int* positions, const int* seq_ids,
                                     const int* page_table, int table_stride, const float* inv_freq, void* k_pool,
                                     void* v_pool, int n_tokens, int n_heads, int n_kv_heads, int head_dim,
                                     int rotary_dim, int pairing, int write_cache, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1) || (pairing != 0 && pairing != 1))
        return b200::kErrBadArgument;
    if (rotary_dim / 2 > b200::kMaxRotaryPairs) return b200::kErrUnsupportedSize;
    // prompts: tiles of tokens with 16-byte accesses, when the sizes fit its vectors and its shared memory
    {
        const int vec = dtype == b200::kF32 ? 4 : 8, esize = dtype == b200::kF32 ? 4 : 2;
        const long long kv_dim = (long long)n_kv_heads * head_dim, row = (long long)(n_heads + 2 * n_kv_heads) * head_dim;
        const long long smem = (long long)b200::kRopeTile * head_dim * 4 + (long long)b200::kRopeTile * kv_dim * esize;
        const bool fits = rotary_dim == head_dim && (pairing == 0 ? head_dim % vec == 0 : (head_dim / 2) % vec == 0) &&
                          row % vec == 0 && kv_dim % vec == 0 && smem <= 48 * 1024 &&
                          (((uintptr_t)qkv | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) == 0;
        if (n_tokens >= 4 * b200::kRopeTile && fits) {
            const int grid = (n_tokens + b200::kRopeTile - 1) / b200::kRopeTile;
            // two CTAs of this kernel fit an SM (registers): cut the columns so that one wave of CTAs covers the prompt
            static int n_sms = 0;
            if (n_sms == 0) {
                int dev = 0;
                if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0)
                    n_sms = 148;
            }
            const int slices = grid >= 2 * n_sms ? 1 : (2 * n_sms / grid > 8 ? 8 : 2 * n_sms / grid);
            B200_DISPATCH_DTYPE(dtype, T,
                return b200::launch_pdl(b200::rope_cache_write_tiled_kernel<T>, dim3(grid, slices), dim3(b200::kRopeThreads),
                                        (size_t)smem, stream, (T*)qkv, positions, seq_ids, page_table, table_stride, inv_freq,
                                        (T*)k_pool, (T*)v_pool, n_tokens, n_heads, n_kv_heads, head_dim, pairing, write_cache));
        }
    }
    B200_DISPATCH_DTYPE(dtype, T,
        return b200::launch_pdl(b200::rope_cache_write_kernel<T>, dim3(n_tokens), dim3(256), 0, stream, (T*)qkv,
                                positions, seq_ids, page_table, table_stride, inv_freq, (T*)k_pool, (T*)v_pool, n_heads,
                                n_kv_heads, head_dim, rotary_dim, pairing, write_cache));
    return b200::launch_status();
}
