// Prefill attention in bfloat16: causal grouped-query attention of whole prompts (or chunks that
// continue a cached prefix) over the paged cache, flash style.
//
// A CTA takes a tile of consecutive query tokens of one sequence and one query head and walks over
// the keys 0..position in blocks of 32, keeping the running max, the running sum and the
// unnormalised output in registers (the online softmax the reference's GPU kernel uses,
// tornadovm/TransformerComputeKernelsLayered.java:431-502 of the reference project; formulas of
// inference/InferenceCore.java:106-145).  Keys and values are read from the cache after this
// step's tokens were written there, so a chunk sees its own keys and the cached prefix alike.
// K rows and V^T rows go 16 bytes per lane straight into mma.m16n8k16 fragments, with the key
// order inside a block chosen so that the probabilities a lane holds after Q K^T are those of the
// 8 consecutive keys its V^T load covers (same scheme as the decode kernel).
//
// Sizes: head_dim 32, 64, 96, 128.  Each warp owns 32 query rows (head_dim <= 64) or 16.
#include "common.cuh"

namespace b200 {

constexpr int kPrefillWarps = 4;
constexpr int kPrefillThreads = kPrefillWarps * 32;

__device__ __forceinline__ void mma_pf(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                       uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float fast_exp2(float x) {  // 2^x, relative error about 2^-22; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ uint4 keep_first8(uint4 v, int n) {
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int left = n - 2 * i;
        w[i] = left >= 2 ? w[i] : (left == 1 ? (w[i] & 0xffffu) : 0u);
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

template <int KB, int MT>  // head_dim / 32; 16-row tiles per warp
__global__ void __launch_bounds__(kPrefillThreads)
attention_prefill_kernel(const __nv_bfloat16* __restrict__ q, int q_row_stride, __nv_bfloat16* __restrict__ out,
                         const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                         const int* __restrict__ page_table, int table_stride,
                         const __nv_bfloat16* __restrict__ k_pool, const __nv_bfloat16* __restrict__ v_pool,
                         int n_heads, int n_kv_heads, int window) {
    constexpr int D = KB * 32, NJ = D / 8, TILE = kPrefillWarps * MT * 16;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int tok0 = cu_seqlens[seq], q_len = cu_seqlens[seq + 1] - tok0;
    const int n_tiles = (q_len + TILE - 1) / TILE;
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // long tiles first
    if (tile >= n_tiles) return;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int kvh = head / (n_heads / n_kv_heads);
    const int kv_len = kv_lens[seq], start = kv_len - q_len;  // position of the sequence's first query token
    const int* pages = page_table + (size_t)seq * table_stride;
    const size_t page_stride = (size_t)n_kv_heads * kPageTokens * D;
    const size_t head_off = (size_t)kvh * kPageTokens * D;

    // this warp's rows: query index (in the sequence's tokens of this step) and position
    const int row0 = tile * TILE + warp * MT * 16;
    if (row0 >= q_len) return;  // whole warp beyond the sequence
    int qi[MT][2], pos[MT][2];
    uint4 ql[MT][KB], qh[MT][KB];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            qi[mt][r] = row0 + mt * 16 + g + 8 * r;
            pos[mt][r] = start + min(qi[mt][r], q_len - 1);  // rows past the end mirror the last one (never stored)
        }
        const __nv_bfloat16* r_lo = q + (size_t)(tok0 + min(qi[mt][0], q_len - 1)) * q_row_stride + (size_t)head * D;
        const __nv_bfloat16* r_hi = q + (size_t)(tok0 + min(qi[mt][1], q_len - 1)) * q_row_stride + (size_t)head * D;
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            ql[mt][kb] = *reinterpret_cast<const uint4*>(r_lo + kb * 32 + t * 8);
            qh[mt][kb] = *reinterpret_cast<const uint4*>(r_hi + kb * 32 + t * 8);
        }
    }
    float o[MT][NJ][4], m_run[MT][2], l_run[MT][2];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        m_run[mt][0] = m_run[mt][1] = -INFINITY;
        l_run[mt][0] = l_run[mt][1] = 0.f;
#pragma unroll
        for (int j = 0; j < NJ; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[mt][j][i] = 0.f;
    }
    const float scale_log2 = 1.4426950408889634f / sqrtf((float)D);  // log2(e) / sqrt(d)

    // keys this warp needs: from the window's start of its first row to its last row's position
    const int p_first = start + row0, p_last = start + min(row0 + MT * 16, q_len) - 1;
    const int k_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    for (int blk = k_lo / 32; blk <= p_last / 32; ++blk) {
        const int base = blk * 32;
        const size_t page_base = (size_t)pages[base / kPageTokens] * page_stride + head_off;
        const int in_page = base % kPageTokens;
        const __nv_bfloat16* kp = k_pool + page_base;
        const __nv_bfloat16* vp = v_pool + page_base;
        uint4 kf[4][KB];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = (g >> 1) * 8 + 2 * i + (g & 1);
#pragma unroll
            for (int kb = 0; kb < KB; ++kb)
                kf[i][kb] = __ldg(reinterpret_cast<const uint4*>(kp + (size_t)(in_page + key) * D + kb * 32 + t * 8));
        }
        uint4 vf[NJ];
#pragma unroll
        for (int j = 0; j < NJ; ++j)
            vf[j] = __ldg(reinterpret_cast<const uint4*>(vp + (size_t)(8 * j + g) * kPageTokens + in_page + t * 8));
        // no masking is needed when every key of the block is visible to every row of the warp
        const bool full = base + 31 <= p_first && (window <= 0 || base >= p_last - window + 1);
        const int n_valid = kv_len - (base + 8 * t);
        if (n_valid < 8) {
#pragma unroll
            for (int j = 0; j < NJ; ++j) vf[j] = keep_first8(vf[j], max(n_valid, 0));
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            float s[4][4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
#pragma unroll
                for (int c = 0; c < 4; ++c) s[i][c] = 0.f;
#pragma unroll
                for (int kb = 0; kb < KB; ++kb) {
                    mma_pf(s[i], ql[mt][kb].x, qh[mt][kb].x, ql[mt][kb].y, qh[mt][kb].y, kf[i][kb].x, kf[i][kb].y);
                    mma_pf(s[i], ql[mt][kb].z, qh[mt][kb].z, ql[mt][kb].w, qh[mt][kb].w, kf[i][kb].z, kf[i][kb].w);
                }
            }
            // scores stay in units of q.k; exp((s - m) / sqrt(d)) is evaluated as exp2((s - m) * scale_log2)
            float bm[2] = {-INFINITY, -INFINITY};
            if (!full) {
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int key = base + 8 * t + 2 * i + e;
#pragma unroll
                        for (int r = 0; r < 2; ++r) {
                            const bool ok = key <= pos[mt][r] && (window <= 0 || key > pos[mt][r] - window);
                            if (!ok) s[i][2 * r + e] = -INFINITY;
                        }
                    }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                bm[0] = fmaxf(bm[0], fmaxf(s[i][0], s[i][1]));
                bm[1] = fmaxf(bm[1], fmaxf(s[i][2], s[i][3]));
            }
            float corr[2], mn[2], mn_scaled[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 1));
                bm[r] = fmaxf(bm[r], __shfl_xor_sync(0xffffffffu, bm[r], 2));
                mn[r] = fmaxf(m_run[mt][r], bm[r]);
                // a row may see no key of this block (its position lies before it): nothing changes for it
                corr[r] = mn[r] == m_run[mt][r] ? 1.f : fast_exp2((m_run[mt][r] - mn[r]) * scale_log2);
                m_run[mt][r] = mn[r];
                mn_scaled[r] = mn[r] == -INFINITY ? 0.f : mn[r] * scale_log2;  // exp2(-inf - 0) = 0 for masked keys
            }
            // the running maximum rarely moves after the first blocks: rescale only when some row's did
            if (!__all_sync(0xffffffffu, corr[0] == 1.f && corr[1] == 1.f)) {
                l_run[mt][0] *= corr[0];
                l_run[mt][1] *= corr[1];
#pragma unroll
                for (int j = 0; j < NJ; ++j) {
                    o[mt][j][0] *= corr[0]; o[mt][j][1] *= corr[0];
                    o[mt][j][2] *= corr[1]; o[mt][j][3] *= corr[1];
                }
            }
            uint32_t pa[4][2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float p0 = fast_exp2(fmaf(s[i][0], scale_log2, -mn_scaled[0]));
                const float p1 = fast_exp2(fmaf(s[i][1], scale_log2, -mn_scaled[0]));
                const float p2 = fast_exp2(fmaf(s[i][2], scale_log2, -mn_scaled[1]));
                const float p3 = fast_exp2(fmaf(s[i][3], scale_log2, -mn_scaled[1]));
                l_run[mt][0] += p0 + p1;
                l_run[mt][1] += p2 + p3;
                pa[i][0] = pack2(p0, p1);
                pa[i][1] = pack2(p2, p3);
            }
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                mma_pf(o[mt][j], pa[0][0], pa[0][1], pa[1][0], pa[1][1], vf[j].x, vf[j].y);
                mma_pf(o[mt][j], pa[2][0], pa[2][1], pa[3][0], pa[3][1], vf[j].z, vf[j].w);
            }
        }
    }

#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            float l = l_run[mt][r];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            if (qi[mt][r] < q_len) {
                __nv_bfloat16* orow = out + ((size_t)(tok0 + qi[mt][r]) * n_heads + head) * D;
#pragma unroll
                for (int j = 0; j < NJ; ++j)
                    *reinterpret_cast<uint32_t*>(orow + 8 * j + 2 * t) = pack2(o[mt][j][2 * r] / l, o[mt][j][2 * r + 1] / l);
            }
        }
}

}  // namespace b200

extern "C" int b200_attention_prefill(const void* q, int q_row_stride, void* out, const int* cu_seqlens,
                                      const int* kv_lens, const int* page_table, int table_stride, const void* k_pool,
                                      const void* v_pool, int n_seqs, int max_q_len, int n_heads, int n_kv_heads,
                                      int head_dim, int window, cudaStream_t stream) {
    using namespace b200;
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return kErrBadArgument;
    if (head_dim % 32 != 0 || head_dim < 32 || head_dim > 128 || q_row_stride % 8 != 0) return kErrUnsupportedSize;
    if (n_seqs > 65535 || n_heads > 65535) return kErrUnsupportedSize;
    const int mt = head_dim <= 64 ? 2 : 1;
    const int tile = kPrefillWarps * mt * 16;
    dim3 grid((max_q_len + tile - 1) / tile, n_heads, n_seqs);
    auto qq = (const __nv_bfloat16*)q;
    auto kk = (const __nv_bfloat16*)k_pool;
    auto vv = (const __nv_bfloat16*)v_pool;
    auto oo = (__nv_bfloat16*)out;
#define B200_LAUNCH(KB, MT)                                                                                       \
    attention_prefill_kernel<KB, MT><<<grid, kPrefillThreads, 0, stream>>>(qq, q_row_stride, oo, cu_seqlens, kv_lens, \
        page_table, table_stride, kk, vv, n_heads, n_kv_heads, window)
    switch (head_dim / 32) {
        case 1: B200_LAUNCH(1, 2); break;
        case 2: B200_LAUNCH(2, 2); break;
        case 3: B200_LAUNCH(3, 1); break;
        default: B200_LAUNCH(4, 1); break;
    }
#undef B200_LAUNCH
    return launch_status();
}
