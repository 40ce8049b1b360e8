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
//
// A norm between two products can be split between them (b200_gemm_decode_linked, M <= 16): RMSNorm of a row
// x is w * x * r with r = rsqrt(mean(x^2) + eps) (inference/InferenceCore.java:47-56), and r, one number per
// row, commutes with the next product.  The product that completes x (residual epilogue) also writes
// bfloat16(x * w) and, per CTA, the sum of squares of the x it holds; the next product multiplies its
// sums by r, which it gets by adding the partial sums in CTA order.  No kernel in between, no atomics.
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
struct NormLink {
    // this product's rows of A are x * w of a norm: multiply the sums of row t by rsqrt(sum_i in_partials[t][i] / dim + eps)
    const float* in_partials;   // [M][n_in] or null
    int n_in;
    float eps;
    int dim;
    // this product completes a residual row x (epilogue 1): also write bfloat16(x * w) and this CTA's sum of x^2
    const void* out_weight;     // [N] norm weights, or null
    int out_weight_f32;         // their type: 1 float32, 0 bfloat16
    __nv_bfloat16* out_act;     // [M][ld_out_act]
    int ld_out_act;
    float* out_partials;        // [M][gridDim.x]
};

// LINK: the product is a half of a split norm (the plain product is compiled without any of that)
template <int MT, int NT, int EPI, typename TC, int U, bool LINK>  // U: k-blocks of 32 in flight per warp
__global__ void __launch_bounds__(kDecodeThreads)
gemm_decode_kernel(const __nv_bfloat16* __restrict__ A, int lda, const __nv_bfloat16* __restrict__ W, int ldw,
                   TC* __restrict__ C, int ldc, int M, int N, int K, NormLink link) {
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
    // What the epilogue will add to is asked for now, not at the CTA's tail (one element per thread when the
    // tile has no more elements than threads; a larger tile reads late).
    constexpr bool kEarlyC = EPI == 1 && NT * 8 * ROWS <= kDecodeThreads;
    float c_early = 0.f, w_early = 0.f;
    if (kEarlyC && (int)threadIdx.x < NT * 8 * ROWS) {
        const int token = threadIdx.x / ROWS, row = threadIdx.x % ROWS;
        if (token < M && row0 + row < N) {
            c_early = to_f32<TC>(C[(size_t)token * ldc + row0 + row]);
            if (LINK && NT <= 2 && link.out_weight != nullptr)
                w_early = link.out_weight_f32 ? reinterpret_cast<const float*>(link.out_weight)[row0 + row]
                                              : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(link.out_weight)[row0 + row]);
        }
    }
    // The norm's factor of each row, made while the first weights are in flight: warp w adds the partial sums of
    // squares of rows w and w + 8 in a fixed order.  (Measured: here it costs nothing; after the main loop, at
    // the tail of every CTA, it cost 1 to 3 us per product.)
    __shared__ float row_factor[16];
    if (LINK && NT <= 2 && link.in_partials != nullptr) {
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            const int token = warp + 8 * n;
            float sum = 0.f;
            if (token < M)
                for (int col = lane; col < link.n_in; col += 32) sum += link.in_partials[(size_t)token * link.n_in + col];
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
            if (lane == 0) row_factor[token] = rsqrtf(sum / (float)link.dim + link.eps);
        }
    }
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
        if (LINK && NT <= 2 && link.in_partials != nullptr) s *= row_factor[token];
        float square = 0.f;
        if (EPI == 2) {
            fin[token][row] = s;
        } else if (token < M && row0 + row < N) {
            TC* c = C + (size_t)token * ldc + row0 + row;
            if (EPI == 1) {
                const float x = (kEarlyC ? c_early : to_f32<TC>(*c)) + s;
                *c = from_f32<TC>(x);
                if (LINK && NT <= 2 && link.out_weight != nullptr) {
                    const float w = kEarlyC ? w_early
                                  : link.out_weight_f32 ? reinterpret_cast<const float*>(link.out_weight)[row0 + row]
                                                        : __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(link.out_weight)[row0 + row]);
                    link.out_act[(size_t)token * link.ld_out_act + row0 + row] = __float2bfloat16_rn(x * w);
                    square = x * x;
                }
            } else {
                *c = from_f32<TC>(s);
            }
        }
        if (LINK && EPI == 1 && NT <= 2 && link.out_weight != nullptr) {
            // the ROWS threads of a token are neighbours in a warp: their squares are added in a fixed tree
#pragma unroll
            for (int off = ROWS / 2; off > 0; off >>= 1) square += __shfl_xor_sync(0xffffffffu, square, off);
            if (row == 0 && token < M) link.out_partials[(size_t)token * gridDim.x + blockIdx.x] = square;
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

template <int MT, int NT, int EPI, typename TC, int U, bool LINK>
static int launch_u(const __nv_bfloat16* a, int lda, const __nv_bfloat16* w, int ldw, void* C, int ldc, int M, int N,
                    int K, const NormLink& link, cudaStream_t stream) {
    constexpr int ROWS = MT == 0 ? 8 : 16 * MT;
    const size_t smem = sizeof(float) * (kDecodeWarps + 1) * NT * 8 * ROWS;
    auto kernel = gemm_decode_kernel<MT, NT, EPI, TC, U, LINK>;
    if (smem > 48 * 1024) {
        static bool configured = false;
        if (!configured) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
                return (int)cudaGetLastError();
            configured = true;
        }
    }
    return launch_pdl(kernel, dim3((N + ROWS - 1) / ROWS), dim3(kDecodeThreads), smem, stream, a, lda, w, ldw, (TC*)C, ldc,
                      M, N, K, link);
}

template <int MT, int NT, int EPI, typename TC>
static int launch_one(const __nv_bfloat16* a, int lda, const __nv_bfloat16* w, int ldw, void* C, int ldc, int M, int N,
                      int K, const NormLink& link, cudaStream_t stream) {
    constexpr int MTT = MT == 0 ? 1 : MT;
    constexpr bool kCanLink = NT <= 2;
    const bool linked = kCanLink && (link.in_partials != nullptr || link.out_weight != nullptr);
#define B200_U(UU)                                                                                                  \
    do {                                                                                                            \
        if (linked) return launch_u<MT, NT, EPI, TC, UU, kCanLink>(a, lda, w, ldw, C, ldc, M, N, K, link, stream);   \
        return launch_u<MT, NT, EPI, TC, UU, false>(a, lda, w, ldw, C, ldc, M, N, K, link, stream);                  \
    } while (0)
    if (MTT * NT >= 8) B200_U(2);
    // 8-row CTAs of a short grid (at most two per SM) can afford twice the loads in flight; a longer grid
    // needs the registers for a third and fourth resident CTA instead
    if (MT == 0 && NT == 1 && N <= 2 * device_sm_count() * 8) B200_U(((MT == 0 && NT == 1) ? 8 : 4));
    // up to three CTAs per SM: six k-blocks in flight, where that saves rounds (hidden 3072: o in 2 rounds instead of 3,
    // down in 6 instead of 8; the 3B shape's step 2.21 -> 2.13 ms)
    if (MT == 0 && NT == 1 && N <= 3 * device_sm_count() * 8 && (K / 32 + 47) / 48 < (K / 32 + 31) / 32)
        B200_U(((MT == 0 && NT == 1) ? 6 : 4));
    B200_U(4);
#undef B200_U
}

template <int MT, int NT, typename TC>
static int launch_epi(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epi,
                      const NormLink& link, cudaStream_t stream) {
    auto a = (const __nv_bfloat16*)A;
    auto w = (const __nv_bfloat16*)W;
    if (epi == 0) return launch_one<MT, NT, 0, TC>(a, lda, w, ldw, C, ldc, M, N, K, link, stream);
    if (epi == 1) return launch_one<MT, NT, 1, TC>(a, lda, w, ldw, C, ldc, M, N, K, link, stream);
    return launch_one<MT, NT, 2, TC>(a, lda, w, ldw, C, ldc, M, N, K, link, stream);
}

}  // namespace b200

namespace b200 {

static bool decode_narrow(int N) { return N <= 4096; }  // few rows: fewer per CTA so that enough CTAs stream weights
static int decode_rows_per_cta(int M, int N) {
    const bool narrow = decode_narrow(N);
    if (M <= 16) return narrow ? 8 : 16;
    return narrow ? 16 : 32;
}

static int gemm_decode_launch(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M, int N,
                              int K, int epilogue, const NormLink& link, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K < 32 || K % 32 != 0 || lda % 8 != 0 || ldw % 8 != 0) return kErrUnsupportedSize;
    if (((uintptr_t)A | (uintptr_t)W) & 15) return kErrUnsupportedSize;
    if (epilogue < 0 || epilogue > 2 || (epilogue == 1 && c_dtype != kF32) || (epilogue == 2 && (N & 1)))
        return kErrBadArgument;
    if (c_dtype != kF32 && c_dtype != kBF16) return kErrBadArgument;
    const bool narrow = decode_narrow(N);
#define B200_GO(MT, NT)                                                                                             \
    return c_dtype == kF32 ? launch_epi<MT, NT, float>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, link, stream)     \
                           : launch_epi<MT, NT, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, link, stream)
    if (M <= 8) { if (narrow) { B200_GO(0, 1); } else { B200_GO(1, 1); } }
    if (M <= 16) { if (narrow) { B200_GO(0, 2); } else { B200_GO(1, 2); } }
    // more tokens: every weight fragment meets 4 or 8 token tiles; wide outputs take 32 rows per CTA so
    // that the activations, which each CTA reads in full, are re-read half as often
    if (M <= 32) { if (narrow) { B200_GO(1, 4); } else { B200_GO(2, 4); } }
    if (narrow) { B200_GO(1, 8); } else { B200_GO(2, 8); }
#undef B200_GO
}

}  // namespace b200

// A, W bfloat16; C bfloat16 or float32 (c_dtype); epilogue 0 store, 1 residual add (C float32), 2 gated SiLU.
extern "C" int b200_gemm_decode(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M,
                                int N, int K, int epilogue, cudaStream_t stream) {
    return b200::gemm_decode_launch(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, b200::NormLink{}, stream);
}

// How many CTAs, hence partial sums per row, the product (M, N) runs with.
extern "C" int b200_gemm_decode_ctas(int M, int N) {
    if (M <= 0 || N <= 0) return 0;
    const int rows = b200::decode_rows_per_cta(M, N);
    return (N + rows - 1) / rows;
}

// The same product as one half, or both halves, of a split norm (M <= 16).
//   in_partials [M][n_in] (or null): A holds x * w of the norm; every sum of row t is multiplied by
//       rsqrt(sum(in_partials[t]) / norm_dim + eps) before the epilogue.
//   out_weight [N] (or null; epilogue 1 only): after the residual add, bfloat16(x * out_weight) goes to
//       out_act [M][ld_out_act] and this CTA's sum of x^2 per row to out_partials [M][b200_gemm_decode_ctas(M, N)].
extern "C" int b200_gemm_decode_linked(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M,
                                       int N, int K, int epilogue, const float* in_partials, int n_in, float eps,
                                       int norm_dim, const void* out_weight, int out_weight_dtype, void* out_act,
                                       int ld_out_act, float* out_partials, cudaStream_t stream) {
    using namespace b200;
    if (M > 16) return kErrUnsupportedSize;
    if (in_partials != nullptr && (n_in <= 0 || norm_dim <= 0)) return kErrBadArgument;
    if (out_weight != nullptr && (epilogue != 1 || out_act == nullptr || out_partials == nullptr || ld_out_act < N ||
                                  (out_weight_dtype != kF32 && out_weight_dtype != kBF16)))
        return kErrBadArgument;
    NormLink link{};
    link.in_partials = in_partials;
    link.n_in = n_in;
    link.eps = eps;
    link.dim = norm_dim;
    link.out_weight = out_weight;
    link.out_weight_f32 = out_weight_dtype == kF32 ? 1 : 0;
    link.out_act = (__nv_bfloat16*)out_act;
    link.ld_out_act = ld_out_act;
    link.out_partials = out_partials;
    return gemm_decode_launch(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, link, stream);
}
