// Prefill attention on tcgen05 tensor cores (bfloat16, head_dim 64 or 128): causal grouped-query attention of
// packed prompt tokens over the paged cache, flash style.
//
// One CTA owns 128 consecutive query tokens of one sequence and one query head and walks over the keys
// 0 .. position in blocks of 128 (two cache pages).  Per block:
//     S = Q K^T          tcgen05.mma 128 x 128 x 64, both operands from shared memory, S in tensor memory
//     P = exp2((S - m) * log2(e) / sqrt(d))   128 threads, one query row each, read S with tcgen05.ld,
//                        write P as bfloat16 into shared memory in the layout the next MMA wants
//     O += P V           tcgen05.mma 128 x 64 x 128, P from shared memory, V^T pages as they lie in the cache
// with the running maximum and sum of the online softmax in registers and O in tensor memory (formulas of
// inference/InferenceCore.java:106-145 of the reference project, online form of
// tornadovm/TransformerComputeKernelsLayered.java:431-502).  The reference maximum of a row only moves
// when a block's maximum exceeds it by more than 2^8 (then O and l are rescaled), which is exact and
// saves most rescaling passes.  Q, K pages and V^T pages arrive by TMA (128-byte swizzle) through a
// two-stage ring.  With head_dim 64 two CTAs fit on an SM, so one CTA's softmax overlaps the other's MMAs.
//
// Roles (320 threads): warp 0 lane 0 issues TMA; warp 1 lane 0 issues MMAs (warp 1 owns the 256 TMEM
// columns: S 128, O head_dim); warps 2-9 are the softmax (two threads per query row) and the epilogue.  Every mbarrier wait is bounded;
// a wait that gives up sets a status word and all roles fall through to the common exit.
#include <type_traits>

#include "tcgen05.cuh"

namespace b200 {

constexpr int kFaThreads = 320;  // TMA warp, MMA warp, eight softmax warps
constexpr int kFaRows = 128, kFaKeys = 128;

__device__ int g_fa_status = 0;

// Operand tiles are stored as "atoms" of 64 elements (128 bytes, one swizzle span) along the contraction:
// Q and K as D/64 atoms of 128 rows, V^T as one atom of D rows per page, P as two atoms of 128 rows.
template <int D>
struct FaSmem {
    alignas(1024) __nv_bfloat16 q[kFaRows * D];            // D/64 atoms [128 rows x 64 dims]
    alignas(1024) __nv_bfloat16 k[2][kFaKeys * D];         // per stage: D/64 atoms [128 keys x 64 dims] (two pages each)
    alignas(1024) __nv_bfloat16 v[2][2][D * 64];           // per stage and page: [D dims x 64 keys] (V^T as cached)
    alignas(1024) __nv_bfloat16 p[2][kFaRows * 64];        // probabilities: keys 0-63 and 64-127 of the block
    alignas(8) uint64_t q_full;
    uint64_t kv_full[2], kv_empty[2];
    uint64_t s_full, p_full, o_full;
    uint32_t tmem_base;
    int abort_flag;
    // exchange between the two threads of a row (512 bytes: the struct must stay within 113 KB): block maxima
    // rounded to bfloat16 (any common reference close to the maximum will do), and at the end the sum
    union { __nv_bfloat16 row_max[2][kFaRows]; float row_sum[kFaRows]; };
};

__device__ __forceinline__ void mbar_arrive_fa(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
          "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
          "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
          "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
          "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
          "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
          "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
          "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}


// The values of a block arrive as whole pages, and the page that holds a sequence's last key also holds whatever an
// earlier owner left behind it.  Those keys get probability 0, but 0 times a value that is not finite is not 0: the
// values of keys at or beyond the sequence's end are therefore set to zero in shared memory before O += P V reads
// them.  v0, v1: the block's two halves of 64 keys, each [D][64] bfloat16 in 128-byte rows with the 128-byte swizzle
// (the 16-byte chunk index XORed with row % 8); first_stale: the first such key, counted from the block's first.
template <int D>
__device__ __forceinline__ void zero_values_beyond_end(__nv_bfloat16* v0, __nv_bfloat16* v1, int first_stale, int tid, int n_threads) {
    for (int item = tid; item < 2 * D * 8; item += n_threads) {
        const int h = item / (D * 8), d = (item / 8) % D, ch = item % 8;
        const int first = first_stale - 64 * h - 8 * ch;  // within this chunk of 8 keys
        if (first >= 8) continue;
        uint8_t* chunk = reinterpret_cast<uint8_t*>(h ? v1 : v0) + d * 128 + ((ch ^ (d & 7)) * 16);
        if (first <= 0) {
            *reinterpret_cast<uint4*>(chunk) = make_uint4(0u, 0u, 0u, 0u);
        } else {
            for (int k = first; k < 8; ++k) reinterpret_cast<uint16_t*>(chunk)[k] = 0;
        }
    }
}

template <int D>
__global__ void __launch_bounds__(kFaThreads, D == 64 ? 2 : 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                            const int* __restrict__ page_table, int table_stride, int n_heads, int n_kv_heads,
                            int window, int k_rows_total, int v_rows_total) {
    // Two CTAs share an SM only if each stays within 113 KB, which leaves no room for an alignment pad: the
    // dynamic shared memory of a kernel without static shared memory starts at the CTA's window, 1024-aligned;
    // if it ever does not, the kernel records that and leaves.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    if ((smem_u32(smem_raw) & 1023u) != 0) {
        if (threadIdx.x == 0) atomicCAS(&g_fa_status, 0, 7 << 8);
        return;
    }
    FaSmem<D>& sm = *reinterpret_cast<FaSmem<D>*>(smem_raw);
    constexpr int kAtoms = D / 64;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seq = blockIdx.z, head = blockIdx.y;
    const int tok0 = cu_seqlens[seq], q_len = cu_seqlens[seq + 1] - tok0;
    const int n_tiles = (q_len + kFaRows - 1) / kFaRows;
    const int tile = (int)gridDim.x - 1 - (int)blockIdx.x;  // long tiles first
    if (tile >= n_tiles) return;
    const int kvh = head / (n_heads / n_kv_heads);
    const int kv_len = kv_lens[seq], start = kv_len - q_len;
    const int q0 = tile * kFaRows;
    const int rows_here = min(kFaRows, q_len - q0);
    const int p_first = start + q0, p_last = start + q0 + rows_here - 1;  // positions of the first and last row
    const int key_lo = window > 0 ? max(0, p_first - window + 1) : 0;
    const int blk_begin = key_lo / kFaKeys, blk_end = p_last / kFaKeys + 1;  // key blocks [begin, end)
    const int* pages = page_table + (size_t)seq * table_stride;
    const int n_pages_seq = (kv_len + kPageTokens - 1) / kPageTokens;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&sm.kv_full[s], 1); mbar_init(&sm.kv_empty[s], 1); }
        mbar_init(&sm.s_full, 1);
        mbar_init(&sm.p_full, 8);
        mbar_init(&sm.o_full, 1);
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_s = sm.tmem_base, tmem_o = sm.tmem_base + 128;  // S: 128 columns, O: D columns
    volatile int* abort_flag = &sm.abort_flag;
    pdl_launch_dependents();
    pdl_wait();  // the set-up above overlapped the kernel before; its results are read from here on

    if (warp == 0 && lane == 0) {
        // ---- producer: Q once, then per block two K pages and two V^T pages
        mbar_expect_tx(&sm.q_full, kFaRows * D * 2);
#pragma unroll
        for (int a = 0; a < kAtoms; ++a) tma_load_2d(sm.q + a * kFaRows * 64, &map_q, head * D + a * 64, tok0 + q0, &sm.q_full);
        int it = 0;
        for (int blk = blk_begin; blk < blk_end; ++blk, ++it) {
            const int s = it & 1;
            if (it >= 2 && !mbar_wait(&sm.kv_empty[s], ((it >> 1) - 1) & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_fa_status, 0, (1 << 8) | s); break;
            }
            mbar_expect_tx(&sm.kv_full[s], 2 * (64 * D * 2) + 2 * (D * 64 * 2));
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int lp = blk * 2 + h;  // logical page; pages the sequence does not have are read as zeros
                const bool have = lp < n_pages_seq;
                const int page = have ? pages[lp] : 0;
#pragma unroll
                for (int a = 0; a < kAtoms; ++a)  // keys 64 h .. of atom a (dims 64 a ..)
                    tma_load_2d(sm.k[s] + a * kFaKeys * 64 + h * 64 * 64, &map_k, a * 64,
                                have ? (page * n_kv_heads + kvh) * 64 : k_rows_total, &sm.kv_full[s]);
                tma_load_2d(sm.v[s][h], &map_v, 0, have ? (page * n_kv_heads + kvh) * D : v_rows_total, &sm.kv_full[s]);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        constexpr uint32_t idesc_s = umma_idesc_bf16(kFaRows, kFaKeys);
        constexpr uint32_t idesc_o = umma_idesc_bf16(kFaRows, D);
        bool ok = mbar_wait(&sm.q_full, 0, abort_flag);
        if (!ok) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, 2 << 8); }
        int it = 0;
        for (int blk = blk_begin; blk < blk_end && ok; ++blk, ++it) {
            const int s = it & 1;
            if (!mbar_wait(&sm.kv_full[s], (it >> 1) & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_fa_status, 0, (3 << 8) | s); ok = false; break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const uint64_t qd = umma_desc(sm.q + (kk / 4) * kFaRows * 64) + 2 * (kk % 4);
                const uint64_t kd = umma_desc(sm.k[s] + (kk / 4) * kFaKeys * 64) + 2 * (kk % 4);
                umma_bf16(tmem_s, qd, kd, idesc_s, kk != 0);
            }
            umma_commit(&sm.s_full);  // also means: the previous block's P V has finished
            if (!mbar_wait(&sm.p_full, it & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_fa_status, 0, 4 << 8); ok = false; break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kFaKeys / 16; ++kk) {
                const uint64_t pd = umma_desc(sm.p[kk / 4]) + 2 * (kk % 4);
                const uint64_t vd = umma_desc(sm.v[s][kk / 4]) + 2 * (kk % 4);
                umma_bf16(tmem_o, pd, vd, idesc_o, (it | kk) != 0);
            }
            umma_commit(&sm.kv_empty[s]);
        }
        if (ok) umma_commit(&sm.o_full);
    } else if (warp >= 2) {
        // ---- softmax and epilogue.  Eight warps: warp w reads TMEM lanes 32 (w % 4) .. + 31 (query rows); the two
        // warps of a lane quarter split a block's 128 keys (and O's 64 dims) in halves.  The two threads of a row
        // agree on the row's maximum through shared memory, so both take the same decisions.
        const int quarter = warp & 3, half = (warp - 2) >> 2;
        const int r = quarter * 32 + lane;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        const int pos = start + q0 + min(r, rows_here - 1);  // rows past the end mirror the last one (never stored)
        const float scale_log2 = 1.4426950408889634f / sqrtf((float)D);
        float m_ref = -INFINITY, l = 0.f;  // reference maximum (units of q.k); this thread's share of the running sum
        bool ok = true;
        int it = 0;
        for (int blk = blk_begin; blk < blk_end; ++blk, ++it) {
            ok = mbar_wait(&sm.s_full, it & 1, abort_flag);
            if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, (5 << 8) | quarter); }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int base = blk * kFaKeys + half * 64;  // first key of this thread's half
            const bool masked = blk * kFaKeys + kFaKeys - 1 > p_first || (window > 0 && blk * kFaKeys < p_last - window + 1);
            const int lo_key = window > 0 ? pos - window + 1 : 0;
            // pass 1: the block's maximum of this row (this thread's 64 keys, then both halves together)
            float m_blk = -INFINITY;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float v[32];
                tmem_ld32(tmem_s + lane_base + half * 64 + c * 32, v);
                if (masked) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int key = base + c * 32 + j;
                        if (key <= pos && key >= lo_key) m_blk = fmaxf(m_blk, v[j]);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j += 2) m_blk = fmaxf(m_blk, fmaxf(v[j], v[j + 1]));
                }
            }
            sm.row_max[half][r] = __float2bfloat16_rn(m_blk);
            asm volatile("bar.sync 1, 256;" ::: "memory");
            m_blk = fmaxf(__bfloat162float(sm.row_max[0][r]), __bfloat162float(sm.row_max[1][r]));
            // the reference maximum moves only when the block exceeds it by more than 2^8 after scaling
            const bool move = m_blk > m_ref && (m_ref == -INFINITY || (m_blk - m_ref) * scale_log2 > 8.f);
            if (__any_sync(0xffffffffu, move)) {
                const float m_new = move ? m_blk : m_ref;
                const float corr = (m_ref == -INFINITY) ? 0.f : ex2((m_ref - m_new) * scale_log2);
                l *= corr;
                if (it > 0) {  // O holds earlier blocks: rescale this row's half of the dims (whole warps take part)
#pragma unroll 1
                    for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
                        float o[32];
                        tmem_ld32(tmem_o + lane_base + c0, o);
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] *= corr;
                        tmem_st32(tmem_o + lane_base + c0, o);
                    }
                }
                m_ref = m_new;
            }
            const float m_scaled = m_ref == -INFINITY ? 0.f : m_ref * scale_log2;
            // pass 2: probabilities, written as bfloat16 in the K-major 128-byte-swizzled layout of an MMA operand
            uint8_t* row_base = reinterpret_cast<uint8_t*>(sm.p[half]) + r * 128;
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float v[32];
                tmem_ld32(tmem_s + lane_base + half * 64 + c * 32, v);
                uint32_t pk[16];
                float l0 = 0.f, l1 = 0.f;
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    float p0 = ex2(fmaf(v[j], scale_log2, -m_scaled));
                    float p1 = ex2(fmaf(v[j + 1], scale_log2, -m_scaled));
                    if (masked) {
                        const int key = base + c * 32 + j;
                        if (!(key <= pos && key >= lo_key)) p0 = 0.f;
                        if (!(key + 1 <= pos && key + 1 >= lo_key)) p1 = 0.f;
                    }
                    __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                    l0 += p0;
                    l1 += p1;
                    pk[j / 2] = *reinterpret_cast<uint32_t*>(&h);
                }
                l += l0 + l1;
                // 32 keys = 4 chunks of 16 bytes; the chunk index is XORed with row % 8 inside its 128-byte row
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    const int chunk = (c * 4 + ch) ^ (r & 7);
                    *reinterpret_cast<uint4*>(row_base + chunk * 16) = make_uint4(pk[4 * ch], pk[4 * ch + 1], pk[4 * ch + 2], pk[4 * ch + 3]);
                }
            }
            if ((blk + 1) * kFaKeys > kv_len) {  // the block holds the sequence's end: see zero_values_beyond_end
                const int s = it & 1;
                if (mbar_wait(&sm.kv_full[s], (it >> 1) & 1, abort_flag))  // has completed; taken for the values' visibility
                    zero_values_beyond_end<D>(sm.v[s][0], sm.v[s][1], kv_len - blk * kFaKeys, (int)threadIdx.x - 64, kFaThreads - 64);
            }
            // P is in shared memory (visible to the tensor cores' proxy) and S has been read: the MMA thread may go on
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_fa(&sm.p_full);
        }
        if (ok) {
            ok = mbar_wait(&sm.o_full, 0, abort_flag);
            if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, (6 << 8) | quarter); }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        // the row's sum is the two halves' shares together (the barriers are reached by all 256 threads, ok or not)
        asm volatile("bar.sync 1, 256;" ::: "memory");   // every thread is done with the maxima that share this memory
        if (half == 1) sm.row_sum[r] = l;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (half == 0) { l += sm.row_sum[r]; sm.row_sum[r] = l; }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv_l = 1.0f / sm.row_sum[r];
            __nv_bfloat16* orow = out + ((size_t)(tok0 + q0 + r) * n_heads + head) * D;
#pragma unroll 1
            for (int c0 = half * (D / 2); c0 < (half + 1) * (D / 2); c0 += 32) {
                float o[32];
                tmem_ld32(tmem_o + lane_base + c0, o);
                if (r < rows_here) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        __nv_bfloat162 a = __floats2bfloat162_rn(o[8 * j] * inv_l, o[8 * j + 1] * inv_l);
                        __nv_bfloat162 b = __floats2bfloat162_rn(o[8 * j + 2] * inv_l, o[8 * j + 3] * inv_l);
                        __nv_bfloat162 c = __floats2bfloat162_rn(o[8 * j + 4] * inv_l, o[8 * j + 5] * inv_l);
                        __nv_bfloat162 d = __floats2bfloat162_rn(o[8 * j + 6] * inv_l, o[8 * j + 7] * inv_l);
                        *reinterpret_cast<uint4*>(orow + c0 + 8 * j) =
                            make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b),
                                       *reinterpret_cast<uint32_t*>(&c), *reinterpret_cast<uint32_t*>(&d));
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(256) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// The pair kernel (head_dim 64 or 128, no window): one CTA owns 256 consecutive query tokens as two tiles of 128
// and keeps both in flight.  Each tile has its own S and O in tensor memory and its own warpgroup of
// softmax threads, ONE thread per query row: the thread reads its row of S (128 scores) into registers in
// one go, so the maximum, the exponentials and the sum need no exchange between threads and no second
// read.  While the softmax of one tile runs, the tensor cores form the other tile's scores and outputs
// (a tile's next scores are issued as soon as its threads hold the current ones), and every K and V block serves both
// tiles.  The grid is one CTA per SM; each takes (pair, head, sequence) units from a counter, longest first.  The probabilities never touch shared memory: the thread writes its row of P as bfloat16 pairs into
// tensor memory and O += P V takes its A operand from there.  One CTA per SM (tensor memory, 512 columns:
// 2 x 128 of S, 2 x 64 of O, 2 x 64 of P; shared memory: Q 32 KB, four stages of K and V 128 KB).
// stages of K and V: what fits beside the two Q tiles (head_dim 64: 32 KB + 4 x 32 KB; 128: 64 KB + 2 x 64 KB)
template <int D> struct PairStages { static constexpr int value = D == 64 ? 4 : 2; };
// Three warpgroups: the softmax warps of tile 0, those of tile 1, and the warps that only issue (TMA, one MMA warp per
// tile, one idle).  The issuing warpgroup hands most of its registers back and the two softmax warpgroups take them
// (setmaxnreg): a softmax thread holds its row's 128 scores and wants more than the 168 registers an even split gives.
constexpr int kPairThreads = 384;
constexpr int kPairTmaWarp = 8, kPairMmaWarp0 = 9, kPairMmaWarp1 = 10;
constexpr int kPairRegsIssuers = 56, kPairRegsSoftmax = 224;   // 128 x 56 + 256 x 224 = 64,512 of the SM's 65,536

template <int D>
struct PairSmem {
    alignas(1024) __nv_bfloat16 q[2][kFaRows * D];
    alignas(1024) __nv_bfloat16 k[PairStages<D>::value][kFaKeys * D];
    alignas(1024) __nv_bfloat16 v[PairStages<D>::value][2][D * 64];
    alignas(8) uint64_t q_full;
    uint64_t kv_full[PairStages<D>::value], kv_empty[PairStages<D>::value];
    uint64_t s_full[2], s_free[2], p_full[2], pv_done[2];
    uint64_t exp_turn[2];  // the two tiles' softmax threads take turns at the exponentials
    uint32_t tmem_base;
    int abort_flag;
    int unit;  // the unit of work the CTA is on
};

__device__ __forceinline__ void tmem_ld32_issue(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
// Completes the loads issued before it; the registers are operands so that no use of them can move above it.
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tie32(uint32_t (&r)[32]) {
    asm volatile("" : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                      "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                      "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                      "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
                 :: "memory");
}

// arithmetic on pairs of floats in one instruction, and the maximum of three
__device__ __forceinline__ unsigned long long pack2(float a, float b) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(a), "f"(b));
    return v;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 16 registers (32 bfloat16) of this thread's row into 16 consecutive columns of tensor memory
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
          "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}
// D[tmem] (+)= A[tmem] B[smem]: A's row i lies in lane i, its K elements as bfloat16 pairs along the columns
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, int accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// Work counters, kept on the device so that a launch needs nothing from the host (it may be replayed from a
// graph): words 0 and 1 count units, word 2 is the number of launches that have ended, word 3 counts the CTAs of
// the running launch that have ended.  A launch takes its units from word (launches ended) % 2 and zeroes the
// other word for the launch after it; its last CTA advances word 2.  Launches on a device must follow one
// another in one stream.
__device__ unsigned int g_pair_ctl[4];

template <int D>
__global__ void __launch_bounds__(kPairThreads, 1)
attention_prefill_pair_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                              const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                              const int* __restrict__ cu_seqlens, const int* __restrict__ kv_lens,
                              const int* __restrict__ page_table, int table_stride, int n_heads, int n_kv_heads,
                              int k_rows_total, int v_rows_total, int n_seqs, int n_pairs) {
    static_assert(D == 64 || D == 128, "the pair kernel is laid out for head_dim 64 and 128");
    // Tensor memory, 512 columns.  Tile t: S in columns 128 t, O in 256 + D t.  P (bfloat16 pairs, 64 columns): with
    // head_dim 64 in columns 384 + 64 t; with head_dim 128 nothing is left, so P overwrites the first half of S, which
    // its thread has read into registers by then, and the next scores are only issued after O += P V.
    constexpr bool kEarlyScores = D == 64;
    constexpr int kAtoms = D / 64;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    PairSmem<D>& sm = *reinterpret_cast<PairSmem<D>*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < PairStages<D>::value; ++s) { mbar_init(&sm.kv_full[s], 1); mbar_init(&sm.kv_empty[s], 2); }
        for (int t = 0; t < 2; ++t) {
            mbar_init(&sm.s_full[t], 1); mbar_init(&sm.s_free[t], 4); mbar_init(&sm.p_full[t], 4); mbar_init(&sm.pv_done[t], 1);
            mbar_init(&sm.exp_turn[t], 4);
        }
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    }
    if (warp == kPairMmaWarp0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;  // tile t: S in columns 128 t, O in 256 + 64 t, P (bfloat16 pairs) in 384 + 64 t
    volatile int* abort_flag = &sm.abort_flag;
    pdl_launch_dependents();
    pdl_wait();  // the set-up above overlapped the kernel before; its results are read from here on
    const unsigned int launches_ended = *reinterpret_cast<volatile unsigned int*>(&g_pair_ctl[2]);
    const int counter = (int)(launches_ended & 1u);
    if (blockIdx.x == 0 && threadIdx.x == 0) g_pair_ctl[counter ^ 1] = 0;
    // The exponentials of a block keep the special-function units busy; reading S, the maximum and the hand-over
    // do not.  So the two tiles' softmax threads alternate: a tile computes its exponentials only while it holds
    // the turn, and the other tile's remaining work runs meanwhile.  Tile 0 has the first turn.
    if (warp >= 4 && warp < 8 && lane == 0) mbar_arrive_fa(&sm.exp_turn[0]);

    // The CTA stays and takes one unit of work after another from a counter: a unit is (pair of tiles, head,
    // sequence), the pairs with the most keys first, so that the SMs finish together.  The barriers are never
    // set up again: every role counts the phases each barrier has been through (the same numbers everywhere,
    // they follow from the units alone).
    const int total_units = n_pairs * n_heads * n_seqs;
    int units_done = 0;            // phases of q_full
    int kv_base = 0;               // K/V blocks of earlier units: block g uses stage g % stages, phase g / stages
    int tile_blocks[2] = {0, 0};   // phases of s_full[t], s_free[t], p_full[t] and pv_done[t]
    int kv_ready = 0;  // MMA threads: blocks (counted over all units) whose K and V this thread knows to have landed

    // The unit loop exists twice, once for the softmax warpgroups and once for the issuing warpgroup, each behind its own
    // register reallocation: the compiler then gives each copy the registers its warps really have.
    auto run_units = [&](auto role) {
        constexpr int ROLE = decltype(role)::value;   // 1: softmax warps, 0: TMA and MMA warps (and the idle one)
        for (;;) {
            __syncthreads();  // the unit before is finished everywhere: tensor memory, Q and the unit number are free
            if (threadIdx.x == 0) sm.unit = (int)atomicAdd(&g_pair_ctl[counter], 1u);
            __syncthreads();
            const int unit = sm.unit;
            if (unit >= total_units || *abort_flag) break;
            const int pair = n_pairs - 1 - unit / (n_heads * n_seqs);
            const int seq = (unit % (n_heads * n_seqs)) / n_heads, head = unit % n_heads;
            const int tok0 = cu_seqlens[seq], q_len = cu_seqlens[seq + 1] - tok0;
            const int q0 = pair * 2 * kFaRows;
            if (q0 >= q_len) continue;  // this sequence has no such rows
            const int kvh = head / (n_heads / n_kv_heads);
            const int kv_len = kv_lens[seq], start = kv_len - q_len;
            // tile t: rows q0 + 128 t .. ; its key blocks are 0 .. nb[t] - 1 (causal), nb[1] = 0 when the tile has no rows
            const int rows0 = min(kFaRows, q_len - q0), rows1 = max(0, min(kFaRows, q_len - q0 - kFaRows));
            const int nb0 = (start + q0 + rows0 - 1) / kFaKeys + 1;
            const int nb1 = rows1 > 0 ? (start + q0 + kFaRows + rows1 - 1) / kFaKeys + 1 : 0;
            const int nb = max(nb0, nb1);

            if (ROLE == 0 && warp == kPairTmaWarp && lane == 0) {
                // ---- producer: both Q tiles, then per block two K pages and two V^T pages
                const int* pages = page_table + (size_t)seq * table_stride;
                const int n_pages_seq = (kv_len + kPageTokens - 1) / kPageTokens;
                mbar_expect_tx(&sm.q_full, (rows1 > 0 ? 2 : 1) * kFaRows * D * 2);
#pragma unroll
                for (int a = 0; a < kAtoms; ++a) {  // an operand tile is stored as atoms of 64 dims (one swizzle span)
                    tma_load_2d(sm.q[0] + a * kFaRows * 64, &map_q, head * D + a * 64, tok0 + q0, &sm.q_full);
                    if (rows1 > 0) tma_load_2d(sm.q[1] + a * kFaRows * 64, &map_q, head * D + a * 64, tok0 + q0 + kFaRows, &sm.q_full);
                }
                for (int j = 0; j < nb; ++j) {
                    const int g = kv_base + j, s = g % PairStages<D>::value;
                    if (g >= PairStages<D>::value && !mbar_wait(&sm.kv_empty[s], ((g / PairStages<D>::value) - 1) & 1, abort_flag)) {
                        *abort_flag = 1; atomicCAS(&g_fa_status, 0, (11 << 8) | s); break;
                    }
                    mbar_expect_tx(&sm.kv_full[s], 2 * (64 * D * 2) + 2 * (D * 64 * 2));
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const int lp = j * 2 + h;  // logical page; pages the sequence does not have are read as zeros
                        const bool have = lp < n_pages_seq;
                        const int page = have ? pages[lp] : 0;
#pragma unroll
                        for (int a = 0; a < kAtoms; ++a)
                            tma_load_2d(sm.k[s] + a * kFaKeys * 64 + h * 64 * 64, &map_k, a * 64,
                                        have ? (page * n_kv_heads + kvh) * 64 : k_rows_total, &sm.kv_full[s]);
                        tma_load_2d(sm.v[s][h], &map_v, 0, have ? (page * n_kv_heads + kvh) * D : v_rows_total, &sm.kv_full[s]);
                    }
                }
            } else if (ROLE == 0 && (warp == kPairMmaWarp0 || warp == kPairMmaWarp1) && lane == 0) {
                // ---- MMA issuers, one thread per tile.  A tile's next scores
                // S(i+1) only need its S columns free, which its softmax threads report as soon as they hold block
                // i's scores in registers (s_free); its outputs O += P(i) V(i) need the probabilities (p_full).  So
                // per block the thread issues S(i+1), then PV(i): the tensor cores form the next scores while the
                // softmax of the current ones runs, and the two tiles' threads keep the pipe fed between them.
                const int t = warp == kPairMmaWarp0 ? 0 : 1;
                const int nbt = t == 0 ? nb0 : nb1, nb_other = t == 0 ? nb1 : nb0;
                constexpr uint32_t idesc_s = umma_idesc_bf16(kFaRows, kFaKeys);
                constexpr uint32_t idesc_o = umma_idesc_bf16(kFaRows, D);
                bool ok = nbt > 0;
                kv_ready = max(kv_ready, kv_base);  // blocks of earlier units this tile never read are not waited for now
                if (ok && !mbar_wait(&sm.q_full, units_done & 1, abort_flag)) {
                    *abort_flag = 1; atomicCAS(&g_fa_status, 0, 12 << 8); ok = false;
                }
                auto need_block = [&](int j) {
                    while (ok && kv_ready <= kv_base + j) {
                        const int s = kv_ready % PairStages<D>::value;
                        if (!mbar_wait(&sm.kv_full[s], (kv_ready / PairStages<D>::value) & 1, abort_flag)) {
                            *abort_flag = 1; atomicCAS(&g_fa_status, 0, (13 << 8) | s); ok = false;
                        } else {
                            ++kv_ready;
                        }
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                };
                // operand descriptors; a 16-element step along K adds 2 (32 bytes) to the start address field
                auto scores = [&](int j) {  // S = Q K_j^T
                    const __nv_bfloat16* kt = sm.k[(kv_base + j) % PairStages<D>::value];
#pragma unroll
                    for (int kk = 0; kk < D / 16; ++kk)
                        umma_bf16(tmem + 128 * t, umma_desc(sm.q[t] + (kk / 4) * kFaRows * 64) + 2 * (kk % 4),
                                  umma_desc(kt + (kk / 4) * kFaKeys * 64) + 2 * (kk % 4), idesc_s, kk != 0);
                    umma_commit(&sm.s_full[t]);
                };
                if (ok) {
                    need_block(0);
                    if (ok) scores(0);
                }
                for (int i = 0; i < nbt && ok; ++i) {
                    if (kEarlyScores && i + 1 < nbt) {
                        if (!mbar_wait(&sm.s_free[t], (tile_blocks[t] + i) & 1, abort_flag)) {
                            *abort_flag = 1; atomicCAS(&g_fa_status, 0, (17 << 8) | t); ok = false; break;
                        }
                        need_block(i + 1);
                        if (!ok) break;
                        scores(i + 1);
                    }
                    if (!mbar_wait(&sm.p_full[t], (tile_blocks[t] + i) & 1, abort_flag)) {
                        *abort_flag = 1; atomicCAS(&g_fa_status, 0, (14 << 8) | t); ok = false; break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const int s = (kv_base + i) % PairStages<D>::value;
                    const uint64_t vd0 = umma_desc(sm.v[s][0]), vd1 = umma_desc(sm.v[s][1]);
#pragma unroll
                    for (int kk = 0; kk < kFaKeys / 16; ++kk)  // O += P V_i; 16 keys = 8 columns of P
                        umma_bf16_a_tmem(tmem + 256 + D * t, tmem + (D == 64 ? 384 + 64 * t : 128 * t) + 8 * kk,
                                         (kk < 4 ? vd0 : vd1) + 2 * (kk % 4), idesc_o, (i | kk) != 0);
                    umma_commit(&sm.pv_done[t]);
                    if (!kEarlyScores && i + 1 < nbt) {  // P lies where the next scores go: they follow the product that reads it
                        need_block(i + 1);
                        if (!ok) break;
                        scores(i + 1);
                    }
                    // a stage is free after two arrivals: one from each tile that reads the block, two from a lone reader
                    umma_commit(&sm.kv_empty[s]);
                    if (i >= nb_other) umma_commit(&sm.kv_empty[s]);
                }
            } else if (ROLE == 1) {
                // ---- softmax and epilogue: warpgroup t = warp / 4 serves tile t, thread = query row = TMEM lane
                const int t = warp >> 2, quarter = warp & 3;
                const int r = quarter * 32 + lane;
                const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
                const int rows_t = t == 0 ? rows0 : rows1, nbt = t == 0 ? nb0 : nb1;
                const int p_first = start + q0 + kFaRows * t;
                const int pos = p_first + min(r, max(rows_t, 1) - 1);  // rows past the end mirror the last one (never stored)
                const float scale_log2 = 1.4426950408889634f / sqrtf((float)D);
                const uint32_t tmem_s = tmem + 128 * t, tmem_o = tmem + 256 + D * t, tmem_p = D == 64 ? tmem + 384 + 64 * t : tmem_s;
                float m_ref = -INFINITY, l = 0.f;
                bool ok = true;
                for (int j = 0; j < nbt; ++j) {
                    ok = mbar_wait(&sm.s_full[t], (tile_blocks[t] + j) & 1, abort_flag);
                    if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, (15 << 8) | (t * 4 + quarter)); }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t sr[4][32];  // this row's 128 scores
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld32_issue(tmem_s + lane_base + c * 32, sr[c]);
                    tmem_ld_wait();
#pragma unroll
                    for (int c = 0; c < 4; ++c) tie32(sr[c]);
                    // the scores are in registers: the next block's scores may be formed
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive_fa(&sm.s_free[t]);
                    const int base = j * kFaKeys;
                    const bool masked = base + kFaKeys - 1 > p_first;  // the block reaches beyond the tile's first row
                    float m_blk = -INFINITY;
                    if (masked) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (base + c * 32 + i <= pos) m_blk = fmaxf(m_blk, __uint_as_float(sr[c][i]));
                    } else {
                        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                        for (int c = 0; c < 4; ++c)
#pragma unroll
                            for (int i = 0; i < 32; i += 2)
                                m4[c] = max3(m4[c], __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
                        m_blk = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
                    }
                    // the block before must have left P and O alone before either is touched (it has, long ago, as a rule)
                    if (j > 0) {
                        ok = mbar_wait(&sm.pv_done[t], (tile_blocks[t] + j - 1) & 1, abort_flag);
                        if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, (18 << 8) | (t * 4 + quarter)); }
                        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                        if (!ok) break;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    }
                    // the reference maximum moves only when the block exceeds it by more than 2^8 after scaling
                    const bool move = m_blk > m_ref && (m_ref == -INFINITY || (m_blk - m_ref) * scale_log2 > 8.f);
                    if (__any_sync(0xffffffffu, move)) {
                        const float m_new = move ? m_blk : m_ref;
                        const float corr = (m_ref == -INFINITY) ? 0.f : ex2((m_ref - m_new) * scale_log2);
                        l *= corr;
                        if (j > 0) {  // O holds earlier blocks: rescale this row (whole warps take part in the TMEM access)
#pragma unroll 1
                            for (int c0 = 0; c0 < D; c0 += 32) {
                                float o[32];
                                tmem_ld32(tmem_o + lane_base + c0, o);
#pragma unroll
                                for (int i = 0; i < 32; ++i) o[i] *= corr;
                                tmem_st32(tmem_o + lane_base + c0, o);
                            }
                        }
                        m_ref = m_new;
                    }
                    const float m_scaled = m_ref == -INFINITY ? 0.f : m_ref * scale_log2;
                    ok = mbar_wait(&sm.exp_turn[t], (kv_base + j) & 1, abort_flag);
                    if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, (19 << 8) | (t * 4 + quarter)); }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) break;
                    // probabilities as bfloat16 pairs into this row's lane of P: key k of the block in column k / 2
                    float l4[4] = {0.f, 0.f, 0.f, 0.f};
                    if (masked) {  // the few blocks on the diagonal: every key is compared with the row's position
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t pk[16];
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                const int key = base + c * 32 + i;
                                const float p0 = key <= pos ? ex2(fmaf(__uint_as_float(sr[c][i]), scale_log2, -m_scaled)) : 0.f;
                                const float p1 = key + 1 <= pos ? ex2(fmaf(__uint_as_float(sr[c][i + 1]), scale_log2, -m_scaled)) : 0.f;
                                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                                l4[c] += p0 + p1;
                                pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
                            }
                            tmem_st16(tmem_p + lane_base + 16 * c, pk);
                        }
                    } else {       // two keys per multiply-add and per addition
                        const unsigned long long scale2 = pack2(scale_log2, scale_log2), shift2 = pack2(-m_scaled, -m_scaled);
                        // Every other pair of keys gets its powers of two from a cubic on the multiply-add pipe instead
                        // of the special-function unit, which would otherwise bound the block: 2^x = 2^n * 2^f with
                        // n = round(x) (taken from the bits of x + 1.5 * 2^23) and f = x - n in [-0.5, 0.5]; the cubic is
                        // within 1.5e-4 of 2^f, a thirtieth of what rounding the probability to bfloat16 loses.
                        const unsigned long long magic2 = pack2(12582912.f, 12582912.f), unmagic2 = pack2(-12582912.f, -12582912.f);
                        const unsigned long long minus1 = pack2(-1.f, -1.f);
                        const unsigned long long k0 = pack2(0.9999280571937561f, 0.9999280571937561f), k1 = pack2(0.6932609677314758f, 0.6932609677314758f);
                        const unsigned long long k2 = pack2(0.2426111251115799f, 0.2426111251115799f), k3 = pack2(0.05517162010073662f, 0.05517162010073662f);
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            uint32_t pk[16];
                            unsigned long long sum2 = pack2(0.f, 0.f);
#pragma unroll
                            for (int i = 0; i < 32; i += 2) {
                                float x0, x1, p0, p1;
                                unpack2(fma2(pack2(__uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1])), scale2, shift2), x0, x1);
                                if (D != 64 || (i & 6) != 2) {
                                    p0 = ex2(x0);
                                    p1 = ex2(x1);
                                } else {
                                    const unsigned long long xc = pack2(fmaxf(x0, -126.f), fmaxf(x1, -126.f));
                                    const unsigned long long tt = add2(xc, magic2);
                                    const unsigned long long f = fma2(add2(tt, unmagic2), minus1, xc);
                                    float q0, q1, t0, t1;
                                    unpack2(fma2(fma2(fma2(k3, f, k2), f, k1), f, k0), q0, q1);
                                    unpack2(tt, t0, t1);
                                    p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(t0) << 23));
                                    p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(t1) << 23));
                                }
                                __nv_bfloat162 h = __floats2bfloat162_rn(p0, p1);
                                sum2 = add2(sum2, pack2(p0, p1));
                                pk[i / 2] = *reinterpret_cast<uint32_t*>(&h);
                            }
                            float s0, s1;
                            unpack2(sum2, s0, s1);
                            l4[c] = s0 + s1;
                            tmem_st16(tmem_p + lane_base + 16 * c, pk);
                        }
                    }
                    l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
                    __syncwarp();
                    if (lane == 0) mbar_arrive_fa(&sm.exp_turn[1 - t]);  // the other tile's turn
                    if ((j + 1) * kFaKeys > kv_len) {  // the block holds the sequence's end: see zero_values_beyond_end
                        const int g = kv_base + j, s = g % PairStages<D>::value;  // (both tiles may do this: they write the same zeros)
                        if (mbar_wait(&sm.kv_full[s], (g / PairStages<D>::value) & 1, abort_flag))
                            zero_values_beyond_end<D>(sm.v[s][0], sm.v[s][1], kv_len - j * kFaKeys, quarter * 32 + lane, 128);
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    }
                    // P is in tensor memory and S has been read: the MMA thread may go on
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive_fa(&sm.p_full[t]);
                }
                for (int j = nbt; j < nb && ok; ++j) {  // rounds in which only the other tile has a block: pass the turn on
                    ok = mbar_wait(&sm.exp_turn[t], (kv_base + j) & 1, abort_flag);
                    if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, (20 << 8) | (t * 4 + quarter)); }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    __syncwarp();
                    if (ok && lane == 0) mbar_arrive_fa(&sm.exp_turn[1 - t]);
                }
                if (ok && nbt > 0) {
                    ok = mbar_wait(&sm.pv_done[t], (tile_blocks[t] + nbt - 1) & 1, abort_flag);
                    if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_fa_status, 0, (16 << 8) | (t * 4 + quarter)); }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (ok) {
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                        const float inv_l = 1.0f / l;
                        __nv_bfloat16* orow = out + ((size_t)(tok0 + q0 + kFaRows * t + r) * n_heads + head) * D;
#pragma unroll 1
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            float o[32];
                            tmem_ld32(tmem_o + lane_base + c0, o);
                            if (r < rows_t) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    __nv_bfloat162 a = __floats2bfloat162_rn(o[8 * i] * inv_l, o[8 * i + 1] * inv_l);
                                    __nv_bfloat162 b = __floats2bfloat162_rn(o[8 * i + 2] * inv_l, o[8 * i + 3] * inv_l);
                                    __nv_bfloat162 c = __floats2bfloat162_rn(o[8 * i + 4] * inv_l, o[8 * i + 5] * inv_l);
                                    __nv_bfloat162 d = __floats2bfloat162_rn(o[8 * i + 6] * inv_l, o[8 * i + 7] * inv_l);
                                    *reinterpret_cast<uint4*>(orow + c0 + 8 * i) =
                                        make_uint4(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b),
                                                   *reinterpret_cast<uint32_t*>(&c), *reinterpret_cast<uint32_t*>(&d));
                                }
                            }
                        }
                    }
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            }
            // the same bookkeeping in every thread
            ++units_done;
            kv_base += nb;
            tile_blocks[0] += nb0;
            tile_blocks[1] += nb1;
        }
    };
    if (warp < 8) {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kPairRegsSoftmax));
        run_units(std::integral_constant<int, 1>{});
    } else {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kPairRegsIssuers));
        run_units(std::integral_constant<int, 0>{});
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kPairMmaWarp0) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(sm.tmem_base), "r"(512) : "memory");
    }
    if (threadIdx.x == 0) {  // the last CTA to end hands the counters over to the next launch
        __threadfence();
        if (atomicAdd(&g_pair_ctl[3], 1u) == gridDim.x - 1) {
            g_pair_ctl[3] = 0;
            __threadfence();
            g_pair_ctl[2] = launches_ended + 1;
        }
    }
}

// 2-D bfloat16 view [rows, cols] with row stride ld elements and boxes of box_cols x box_rows, 128-byte swizzle.
static bool make_map_2d(CUtensorMap* map, const void* base, long long rows, int cols, long long ld, int box_cols, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace b200

extern "C" int b200_attention_prefill_tc_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, b200::g_fa_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(b200::g_fa_status, &zero, sizeof(int));
    return v;
}

namespace b200 {
template <int D>
static int launch_fa(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, const int* cu_seqlens,
                     const int* kv_lens, const int* page_table, int table_stride, int n_seqs, int max_q_len, int n_heads,
                     int n_kv_heads, int window, int k_rows, int v_rows, cudaStream_t stream) {
    static_assert(D != 64 || sizeof(FaSmem<64>) <= 113 * 1024, "two CTAs per SM need at most 113 KB each");
    const size_t smem = sizeof(FaSmem<D>);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    dim3 grid((max_q_len + kFaRows - 1) / kFaRows, n_heads, n_seqs);
    return launch_pdl(attention_prefill_tc_kernel<D>, grid, dim3(kFaThreads), smem, stream, mq, mk, mv, (__nv_bfloat16*)out,
                      cu_seqlens, kv_lens, page_table, table_stride, n_heads, n_kv_heads, window, k_rows, v_rows);
}
}  // namespace b200

namespace b200 {
template <int D>
static int launch_pair(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out, const int* cu_seqlens,
                       const int* kv_lens, const int* page_table, int table_stride, int n_seqs, int max_q_len, int n_heads,
                       int n_kv_heads, int k_rows, int v_rows, cudaStream_t stream) {
    const size_t smem = sizeof(PairSmem<D>) + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attention_prefill_pair_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int n_pairs = (max_q_len + 2 * kFaRows - 1) / (2 * kFaRows);
    const long long units = (long long)n_pairs * n_heads * n_seqs;
    if (units >= (1ll << 31)) return kErrUnsupportedSize;
    int dev = 0, n_sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return kErrBadArgument;
    const int grid = (int)(units < n_sms ? units : n_sms);  // one CTA per SM; each takes units until none are left
    return launch_pdl(attention_prefill_pair_kernel<D>, dim3(grid), dim3(kPairThreads), smem, stream, mq, mk, mv,
                      (__nv_bfloat16*)out, cu_seqlens, kv_lens, page_table, table_stride, n_heads, n_kv_heads, k_rows, v_rows,
                      n_seqs, n_pairs);
}
}  // namespace b200

// q: packed rows of q_row_stride elements whose first n_heads * head_dim are the rotated queries (n_rows of them);
// k_pool [n_pages][n_kv_heads][64][head_dim], v_pool [n_pages][n_kv_heads][head_dim][64] (values transposed).
// head_dim 64 or 128.
extern "C" int b200_attention_prefill_tc(const void* q, int q_row_stride, int n_rows, void* out, const int* cu_seqlens,
                                         const int* kv_lens, const int* page_table, int table_stride,
                                         const void* k_pool, const void* v_pool, int n_pages, int n_seqs, int max_q_len,
                                         int n_heads, int n_kv_heads, int head_dim, int window, cudaStream_t stream) {
    using namespace b200;
    if (n_seqs <= 0 || max_q_len <= 0) return 0;
    if (n_kv_heads <= 0 || n_heads % n_kv_heads != 0) return kErrBadArgument;
    if ((head_dim != 64 && head_dim != 128) || q_row_stride % 8 != 0 ||
        (((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool | (uintptr_t)out) & 15))
        return kErrUnsupportedSize;
    if (n_seqs > 65535 || n_heads > 65535) return kErrUnsupportedSize;
    const long long k_rows = (long long)n_pages * n_kv_heads * 64, v_rows = (long long)n_pages * n_kv_heads * head_dim;
    if (k_rows >= (1ll << 31) || v_rows >= (1ll << 31)) return kErrUnsupportedSize;
    CUtensorMap mq, mk, mv;
    if (!make_map_2d(&mq, q, n_rows, n_heads * head_dim, q_row_stride, 64, kFaRows) ||
        !make_map_2d(&mk, k_pool, k_rows, head_dim, head_dim, 64, 64) || !make_map_2d(&mv, v_pool, v_rows, 64, 64, 64, head_dim))
        return kErrUnsupportedSize;
    // tiles in pairs when there are enough pairs to give every SM one (fewer: the single-tile kernel fills more SMs)
    if (window <= 0 && (long long)((max_q_len + 2 * kFaRows - 1) / (2 * kFaRows)) * n_heads * n_seqs >= device_sm_count()) {
        if (head_dim == 64)
            return launch_pair<64>(mq, mk, mv, out, cu_seqlens, kv_lens, page_table, table_stride, n_seqs, max_q_len, n_heads,
                                   n_kv_heads, (int)k_rows, (int)v_rows, stream);
        return launch_pair<128>(mq, mk, mv, out, cu_seqlens, kv_lens, page_table, table_stride, n_seqs, max_q_len, n_heads,
                                n_kv_heads, (int)k_rows, (int)v_rows, stream);
    }
    if (head_dim == 64)
        return launch_fa<64>(mq, mk, mv, out, cu_seqlens, kv_lens, page_table, table_stride, n_seqs, max_q_len, n_heads,
                             n_kv_heads, window, (int)k_rows, (int)v_rows, stream);
    return launch_fa<128>(mq, mk, mv, out, cu_seqlens, kv_lens, page_table, table_stride, n_seqs, max_q_len, n_heads,
                          n_kv_heads, window, (int)k_rows, (int)v_rows, stream);
}
