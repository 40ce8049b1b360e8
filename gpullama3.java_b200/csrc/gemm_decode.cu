// Matrix product for decode steps in bfloat16: C[M, N] = A[M, K] W[N, K]^T for M <= 64 tokens.
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
// Sizes: K a multiple of 32, rows 16-byte aligned; any N; M <= 64.  Other shapes are refused
// (kErrUnsupportedSize) and the caller takes the plain kernel.
#include "common.cuh"

namespace b200 {

constexpr int kDecodeWarps = 8;
constexpr int kDecodeThreads = kDecodeWarps * 32;

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

// MT: 16-row tiles of weight rows per CTA (ROWS = 16 * MT), or MT = 0 for 8 rows (narrow outputs, so that
// more CTAs pull on HBM).  NT: token tiles of 8.  EPI: 0 store, 1 residual add (C float), 2 gated SiLU.
template <int MT, int NT, int EPI, typename TC, int U>  // U: k-blocks of 32 in flight per warp
__global__ void __launch_bounds__(kDecodeThreads)
gemm_decode_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, int ldw,
                   TC* __restrict__ C, int ldc, int M, int N, int K) {
    constexpr int ROWS = MT == 0 ? 8 : 16 * MT;
    constexpr int MTT = MT == 0 ? 1 : MT;            // tiles actually multiplied
    constexpr bool HI = MT != 0;                     // rows g + 8 of a tile exist
    extern __shared__ float red_raw[];               // [warps][NT * 8][ROWS] partial sums, then [NT * 8][ROWS]
    float (*red)[NT * 8][ROWS] = reinterpret_cast<float (*)[NT * 8][ROWS]>(red_raw);
    float (*fin)[ROWS] = reinterpret_cast<float (*)[ROWS]>(red_raw + kDecodeWarps * NT * 8 * ROWS);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = blockIdx.x * ROWS;
    const __nv_bfloat16* w_lo[MTT];
    const __nv_bfloat16* w_hi[MTT];
#pragma unroll
    for (int m = 0; m < MTT; ++m) {  // clamped: rows past N are read but never stored
        w_lo[m] = W + (size_t)min(row0 + 16 * m + g, N - 1) * ldw + t * 8;
        w_hi[m] = W + (size_t)min(row0 + 16 * m + g + 8, N - 1) * ldw + t * 8;
    }
    const __nv_bfloat16* a_row[NT];
    bool a_ok[NT];
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        a_ok[n] = n * 8 + g < M;
        a_row[n] = A + (size_t)min(n * 8 + g, M - 1) * lda + t * 8;
    }
    float acc[MTT][NT][4];
#pragma unroll
    for (int m = 0; m < MTT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][n][i] = 0.f;

    const int n_blocks = K / 32;
    uint4 wl[U][MTT], wh[U][MTT];
    auto load_weights = [&](int kb0) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int kb = kb0 + u;
#pragma unroll
            for (int m = 0; m < MTT; ++m) {
                wl[u][m] = kb < n_blocks ? load_stream(w_lo[m] + kb * 32) : make_uint4(0, 0, 0, 0);
                wh[u][m] = (HI && kb < n_blocks) ? load_stream(w_hi[m] + kb * 32) : make_uint4(0, 0, 0, 0);
            }
        }
    };
    // the first weights are on their way before the kernel that produces the activations has finished
    load_weights(warp * U);
    pdl_launch_dependents();
    pdl_wait();
    for (int kb0 = warp * U; kb0 < n_blocks; kb0 += kDecodeWarps * U) {
        uint4 cl[U][MTT], ch[U][MTT];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int m = 0; m < MTT; ++m) { cl[u][m] = wl[u][m]; ch[u][m] = wh[u][m]; }
        load_weights(kb0 + kDecodeWarps * U);  // next round's weights, in flight during this round's MMAs
        // activation fragments of the round are all requested before the first MMA needs one
        uint4 av[U][NT];
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int n = 0; n < NT; ++n)
                av[u][n] = (a_ok[n] && kb0 + u < n_blocks) ? load_cached(a_row[n] + (kb0 + u) * 32) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < U; ++u)
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int m = 0; m < MTT; ++m) {
                    mma_bf16(acc[m][n], cl[u][m].x, ch[u][m].x, cl[u][m].y, ch[u][m].y, av[u][n].x, av[u][n].y);
                    mma_bf16(acc[m][n], cl[u][m].z, ch[u][m].z, cl[u][m].w, ch[u][m].w, av[u][n].z, av[u][n].w);
                }
    }

    // partial sums of the warps meet in shared memory; thread (row, token) adds them in warp order
#pragma unroll
    for (int m = 0; m < MTT; ++m)
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            red[warp][n * 8 + 2 * t][16 * m + g] = acc[m][n][0];
            red[warp][n * 8 + 2 * t + 1][16 * m + g] = acc[m][n][1];
            if (HI) {
                red[warp][n * 8 + 2 * t][16 * m + g + 8] = acc[m][n][2];
                red[warp][n * 8 + 2 * t + 1][16 * m + g + 8] = acc[m][n][3];
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

template <int MT, int NT, int EPI, typename TC, int U>
static int launch_u(const __nv_bfloat16* a, int lda, const __nv_bfloat16* w, int ldw, void* C, int ldc, int M, int N,
                    int K, cudaStream_t stream) {
    constexpr int ROWS = MT == 0 ? 8 : 16 * MT;
    const size_t smem = sizeof(float) * (kDecodeWarps + 1) * NT * 8 * ROWS;
    auto kernel = gemm_decode_kernel<MT, NT, EPI, TC, U>;
    if (smem > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                return (int)cudaGetLastError();
            configured = true;
        }
    }
    return launch_pdl(kernel, dim3((N + ROWS - 1) / ROWS), dim3(kDecodeThreads), smem, stream, a, lda, w, ldw, (TC*)C, ldc,
                      M, N, K);
}

template <int MT, int NT, int EPI, typename TC>
static int launch_one(const __nv_bfloat16* a, int lda, const __nv_bfloat16* w, int ldw, void* C, int ldc, int M, int N,
                      int K, cudaStream_t stream) {
    constexpr int MTT = MT == 0 ? 1 : MT;
    if (MTT * NT >= 8) return launch_u<MT, NT, EPI, TC, 2>(a, lda, w, ldw, C, ldc, M, N, K, stream);
    // 8-row CTAs of a short grid (at most two per SM) can afford twice the loads in flight; a longer grid
    // needs the registers for a third and fourth resident CTA instead
    if (MT == 0 && NT == 1 && N <= 2 * 148 * 8) return launch_u<MT, NT, EPI, TC, (MT == 0 && NT == 1) ? 8 : 4>(a, lda, w, ldw, C, ldc, M, N, K, stream);
    return launch_u<MT, NT, EPI, TC, 4>(a, lda, w, ldw, C, ldc, M, N, K, stream);
}

template <int MT, int NT, typename TC>
static int launch_epi(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi,
                      cudaStream_t stream) {
    auto a = (const __nv_bfloat16*)A;
    auto w = (const __nv_bfloat16*)W;
    if (epi == 0) return launch_one<MT, NT, 0, TC>(a, lda, w, ldw, C, ldc, M, N, K, stream);
    if (epi == 1) return launch_one<MT, NT, 1, TC>(a, lda, w, ldw, C, ldc, M, N, K, stream);
    return launch_one<MT, NT, 2, TC>(a, lda, w, ldw, C, ldc, M, N, K, stream);
}

}  // namespace b200

// A, W bfloat16; C bfloat16 or float32 (c_dtype); epilogue 0 store, 1 residual add (C float32), 2 gated SiLU.
extern "C" int b200_gemm_decode(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M,
                                int N, int K, int epilogue, cudaStream_t stream) {
    using namespace b200;
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K < 32 || K % 32 != 0 || lda % 8 != 0 || ldw % 8 != 0) return kErrUnsupportedSize;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return kErrUnsupportedSize;
    if (epilogue < 0 || epilogue > 2 || (epilogue == 1 && c_dtype != kF32) || (epilogue == 2 && (N & 1)))
        return kErrBadArgument;
    if (c_dtype != kF32 && c_dtype != kBF16) return kErrBadArgument;
    const bool narrow = N <= 4096;  // few rows: fewer per CTA so that enough CTAs stream weights
#define B200_GO(MT, NT)                                                                                       \
    return c_dtype == kF32 ? launch_epi<MT, NT, float>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, stream)     \
                           : launch_epi<MT, NT, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, stream)
    if (M <= 8) { if (narrow) { B200_GO(0, 1); } else { B200_GO(1, 1); } }
    if (M <= 16) { if (narrow) { B200_GO(0, 2); } else { B200_GO(1, 2); } }
    // more tokens: every weight fragment meets 4 or 8 token tiles; wide outputs take 32 rows per CTA so
    // that the activations, which each CTA reads in full, are re-read half as often
    if (M <= 32) { if (narrow) { B200_GO(1, 4); } else { B200_GO(2, 4); } }
    if (narrow) { B200_GO(1, 8); } else { B200_GO(2, 8); }
#undef B200_GO
}
