// Matrix product for decode steps in bfloat16: C[M, N] = A[M, K] W[N, K]^T for M <= 16 tokens.
//
// A decode step reads every weight once and does little arithmetic with it, so this kernel is
// built around the stream of W from HBM: each lane loads 16 contiguous bytes of a weight row
// straight into tensor-core fragments (no shared-memory staging), warps of a CTA split K between
// them, and the partial sums meet in shared memory in a fixed order (no atomics: the result does
// not depend on scheduling).  The reference does the same product with one work-group per output
// row and a tree reduction (tornadovm/TransformerComputeKernelsLayered.java:901-930 of the
// reference project); its fused residual (:766-784) and SiLU-gate (:808-826) variants are the
// epilogues here.
//
// Fragment trick: mma.m16n8k16 wants, per lane, weight elements (row g, k = 2t, 2t+1, 2t+8, 2t+9).
// A dot product does not care in which order k is summed as long as both operands agree, so
// lane (g, t) takes the 8 consecutive elements k0 + 8t .. 8t+7 of row g (one 16-byte load) and
// feeds them to two MMAs; the activation fragment is the same 16-byte slice of the token's row.
//
// Sizes: K a multiple of 32, rows 16-byte aligned; any N; M <= 16.  Other shapes are refused
// (kErrUnsupportedSize) and the caller takes the plain kernel.
#include "common.cuh"

namespace b200 {

constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kUnroll = 4;  // k-blocks of 32 in flight per warp

__device__ __forceinline__ uint4 load_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint4 load_cached(const void* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ROWS: weight rows per CTA (16, or 8 for narrow outputs so that more CTAs pull on HBM).
// NT: token tiles of 8.  EPI: 0 store, 1 residual add (C float), 2 gated SiLU.
template <int ROWS, int NT, int EPI, typename TC>
__global__ void __launch_bounds__(kDecodeThreads)
gemm_decode_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, int ldw,
                   TC* __restrict__ C, int ldc, int M, int N, int K) {
    __shared__ float red[kDecodeWarps][NT * 8][ROWS];
    __shared__ float fin[NT * 8][ROWS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * ROWS;
    const int r_lo = min(row0 + g, N - 1);            // clamped: rows past N are read but never stored
    const int r_hi = min(row0 + g + 8, N - 1);
    const __nv_bfloat16* w_lo = W + (size_t)r_lo * ldw + t * 8;
    const __nv_bfloat16* w_hi = W + (size_t)r_hi * ldw + t * 8;
    const __nv_bfloat16* a_row[NT];
    bool a_ok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        a_ok[n] = n * 8 + g < M;
        a_row[n] = A + (size_t)min(n * 8 + g, M - 1) * lda + t * 8;
    }
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.f;

    const int n_blocks = K / 32;
    uint4 wl[kUnroll], wh[kUnroll];
    auto load_weights = [&](int kb0) {
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) {
            const int kb = kb0 + u;
            wl[u] = kb < n_blocks ? load_stream(w_lo + kb * 32) : make_uint4(0, 0, 0, 0);
            wh[u] = (ROWS == 16 && kb < n_blocks) ? load_stream(w_hi + kb * 32) : make_uint4(0, 0, 0, 0);
        }
    };
    // the first weights are on their way before the kernel that produces the activations has finished
    load_weights(warp * kUnroll);
    pdl_launch_dependents();
    pdl_wait();
    for (int kb0 = warp * kUnroll; kb0 < n_blocks; kb0 += kDecodeWarps * kUnroll) {
        uint4 av[kUnroll][NT];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int n = 0; n < NT; ++n)
                av[u][n] = (a_ok[n] && kb0 + u < n_blocks) ? load_cached(a_row[n] + (kb0 + u) * 32) : make_uint4(0, 0, 0, 0);
        uint4 cl[kUnroll], ch[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) { cl[u] = wl[u]; ch[u] = wh[u]; }
        load_weights(kb0 + kDecodeWarps * kUnroll);  // next round's weights, in flight during this round's MMAs
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                mma_bf16(acc[n], cl[u].x, ch[u].x, cl[u].y, ch[u].y, av[u][n].x, av[u][n].y);
                mma_bf16(acc[n], cl[u].z, ch[u].z, cl[u].w, ch[u].w, av[u][n].z, av[u][n].w);
            }
    }

    // partial sums of the warps meet in shared memory; thread (row, token) adds them in warp order
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        red[warp][n * 8 + 2 * t][g] = acc[n][0];
        red[warp][n * 8 + 2 * t + 1][g] = acc[n][1];
        if (ROWS == 16) {
            red[warp][n * 8 + 2 * t][g + 8] = acc[n][2];
            red[warp][n * 8 + 2 * t + 1][g + 8] = acc[n][3];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < NT * 8 * ROWS; idx += kDecodeThreads) {
        const int token = idx / ROWS, row = idx % ROWS;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kDecodeWarps; ++w) s += red[w][token][row];
        if (EPI == 2) {
            fin[token][row] = s;
        } else if (token < M && row0 + row < N) {
            TC* c = C + (size_t)token * ldc + row0 + row;
            if (EPI == 1) *c = from_f32<TC>(to_f32<TC>(*c) + s);
            else *c = from_f32<TC>(s);
        }
    }
    if (EPI == 2) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < NT * 8 * (ROWS / 2); idx += kDecodeThreads) {
            const int token = idx / (ROWS / 2), pair = idx % (ROWS / 2);
            if (token < M && row0 + 2 * pair + 1 < N) {
                const float gate = fin[token][2 * pair], up = fin[token][2 * pair + 1];
                C[(size_t)token * ldc + (row0 >> 1) + pair] = from_f32<TC>((gate / (1.0f + expf(-gate))) * up);
            }
        }
    }
}

template <int ROWS, int NT, typename TC>
static int launch_epi(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi,
                      cudaStream_t stream) {
    const int grid = (N + ROWS - 1) / ROWS;
    auto a = (const __nv_bfloat16*)A;
    auto w = (const __nv_bfloat16*)W;
    const dim3 g(grid), b(kDecodeThreads);
    if (epi == 0) return launch_pdl(gemm_decode_kernel<ROWS, NT, 0, TC>, g, b, 0, stream, a, lda, w, ldw, (TC*)C, ldc, M, N, K);
    if (epi == 1) return launch_pdl(gemm_decode_kernel<ROWS, NT, 1, TC>, g, b, 0, stream, a, lda, w, ldw, (TC*)C, ldc, M, N, K);
    return launch_pdl(gemm_decode_kernel<ROWS, NT, 2, TC>, g, b, 0, stream, a, lda, w, ldw, (TC*)C, ldc, M, N, K);
}

}  // namespace b200

// A, W bfloat16; C bfloat16 or float32 (c_dtype); epilogue 0 store, 1 residual add (C float32), 2 gated SiLU.
extern "C" int b200_gemm_decode(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M,
                                int N, int K, int epilogue, cudaStream_t stream) {
    using namespace b200;
    if (M <= 0 || N <= 0) return 0;
    if (M > 16 || K < 32 || K % 32 != 0 || lda % 8 != 0 || ldw % 8 != 0) return kErrUnsupportedSize;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return kErrUnsupportedSize;
    if (epilogue < 0 || epilogue > 2 || (epilogue == 1 && c_dtype != kF32) || (epilogue == 2 && (N & 1)))
        return kErrBadArgument;
    const bool narrow = N <= 4096;  // few rows: 8 per CTA so that at least ~2 CTAs per SM stream weights
    const bool two = M > 8;
#define B200_GO(ROWS, NT)                                                                                     \
    return c_dtype == kF32 ? launch_epi<ROWS, NT, float>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, stream)   \
                           : launch_epi<ROWS, NT, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, stream)
    if (c_dtype != kF32 && c_dtype != kBF16) return kErrBadArgument;
    if (narrow) { if (two) { B200_GO(8, 2); } else { B200_GO(8, 1); } }
    if (two) { B200_GO(16, 2); } else { B200_GO(16, 1); }
#undef B200_GO
}
