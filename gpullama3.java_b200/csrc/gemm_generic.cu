// Plain matrix product C = A W^T with 32-bit FMA accumulation, any storage types, any sizes.
//
// A is [M, K] (activations, row-major, row stride lda), W is [N, K] (a weight as the reference
// stores it: one row per output, core/model/tensor/FloatTensor.java:98-100 of the reference
// project).  Three kernels: tiles of 128 x 128 for prompts, of 64 x 64 for fewer than 128 rows, and a weight-streaming one for a decode step's few rows
// (further down).  This is the kernel of the true 32-bit path (no tensor cores, no reduced-precision
// matrix mode) and the fallback of the bfloat16 path for sizes or storage types the tensor-core
// kernels refuse.  Epilogues:
//   0  store         C[M, N] = acc                       (C of type TC)
//   1  residual add  C[M, N] += acc                      (C is the 32-bit residual stream)
//   2  gated SiLU    C[M, N/2] = silu(acc[2j]) * acc[2j+1]   (W holds gate and up rows interleaved;
//                    silu(g) = g / (1 + exp(-g)), inference/InferenceCore.java:163-166)
#include "common.cuh"

namespace b200 {

constexpr int kTileM = 64, kTileN = 64, kTileK = 16, kGemmThreads = 256;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(kGemmThreads)
gemm_generic_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw, TC* __restrict__ C, int ldc,
                    int M, int N, int K, int epilogue) {
    __shared__ float As[kTileK][kTileM + 4];
    __shared__ float Ws[kTileK][kTileN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * kTileM, n0 = blockIdx.x * kTileN;
    const int tx = tid % 16, ty = tid / 16;  // thread owns rows ty*4..+3, columns tx*4..+3
    float acc[4][4] = {};

    for (int k0 = 0; k0 < K; k0 += kTileK) {
        // 64 x 16 elements of each operand, 4 per thread; consecutive threads read along K
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * kGemmThreads;
            const int r = e / kTileK, c = e % kTileK;
            const int k = k0 + c;
            As[c][r] = (m0 + r < M && k < K) ? to_f32<TA>(A[(size_t)(m0 + r) * lda + k]) : 0.f;
            Ws[c][r] = (n0 + r < N && k < K) ? to_f32<TW>(W[(size_t)(n0 + r) * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < kTileK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; w[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
        if (epilogue == 2) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < N) {
                    const float gate = acc[i][j], up = acc[i][j + 1];
                    C[(size_t)m * ldc + n / 2] = from_f32<TC>((gate / (1.0f + expf(-gate))) * up);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + tx * 4 + j;
                if (n >= N) continue;
                TC* c = C + (size_t)m * ldc + n;
                if (epilogue == 1) *c = from_f32<TC>(to_f32<TC>(*c) + acc[i][j]);
                else *c = from_f32<TC>(acc[i][j]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same product for prompts (M >= 128): tiles of 128 x 128, a thread owns 8 x 8 sums, so that a k-step costs four
// 16-byte shared-memory loads per 64 multiply-adds instead of eight 4-byte loads per 16; the next tile's operands are
// fetched into registers while the current one is multiplied.  Still plain 32-bit FMA in a fixed order of k.
constexpr int kBigM = 128, kBigN = 128, kBigK = 16, kBigThreads = 256;

template <typename TA, typename TW, typename TC>
__global__ void __launch_bounds__(kBigThreads)
gemm_generic_big_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw, TC* __restrict__ C, int ldc,
                        int M, int N, int K, int epilogue) {
    __shared__ __align__(16) float As[kBigK][kBigM + 4];
    __shared__ __align__(16) float Ws[kBigK][kBigN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * kBigM, n0 = blockIdx.x * kBigN;
    const int tx = tid % 16, ty = tid / 16;   // rows ty * 8 .. + 7, columns tx * 8 .. + 7
    float acc[8][8] = {};
    float ra[8], rw[8];                        // this thread's share of the next tile: 8 elements of each operand
    auto fetch = [&](int k0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = tid + i * kBigThreads, r = e / kBigK, k = k0 + e % kBigK;   // 16 lanes read along k
            ra[i] = (m0 + r < M && k < K) ? to_f32<TA>(A[(size_t)(m0 + r) * lda + k]) : 0.f;
            rw[i] = (n0 + r < N && k < K) ? to_f32<TW>(W[(size_t)(n0 + r) * ldw + k]) : 0.f;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += kBigK) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = tid + i * kBigThreads, r = e / kBigK, c = e % kBigK;
            As[c][r] = ra[i];
            Ws[c][r] = rw[i];
        }
        __syncthreads();
        if (k0 + kBigK < K) fetch(k0 + kBigK);
#pragma unroll
        for (int k = 0; k < kBigK; ++k) {
            const float4 a0 = *reinterpret_cast<const float4*>(&As[k][ty * 8]), a1 = *reinterpret_cast<const float4*>(&As[k][ty * 8 + 4]);
            const float4 w0 = *reinterpret_cast<const float4*>(&Ws[k][tx * 8]), w1 = *reinterpret_cast<const float4*>(&Ws[k][tx * 8 + 4]);
            const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
            const float w[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int m = m0 + ty * 8 + i;
        if (m >= M) continue;
        if (epilogue == 2) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const int n = n0 + tx * 8 + j;
                if (n + 1 < N) {
                    const float gate = acc[i][j], up = acc[i][j + 1];
                    C[(size_t)m * ldc + n / 2] = from_f32<TC>((gate / (1.0f + expf(-gate))) * up);
                }
            }
        } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int n = n0 + tx * 8 + j;
                if (n >= N) continue;
                TC* c = C + (size_t)m * ldc + n;
                if (epilogue == 1) *c = from_f32<TC>(to_f32<TC>(*c) + acc[i][j]);
                else *c = from_f32<TC>(acc[i][j]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// The same product for a decode step's few rows (M <= 16): tiles of 64 tokens would leave the FMA units idle and
// read every weight through shared memory for nothing.  Here the weight rows are streamed 16 bytes per lane, every
// element meeting all M tokens' activations (which stay in L1); see gemm_fewrows_kernel.
template <typename T> __device__ __forceinline__ float4 load4(const T* p);
template <> __device__ __forceinline__ float4 load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 load4<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
}

constexpr int kFewWarps = 8, kFewThreads = kFewWarps * 32, kFewRows = 4;

// sum over the lanes of a warp by halving: afterwards v[0] of lane l is the sum of every lane's v[l] (31 exchanges
// for 32 numbers, where a butterfly per number would need 160)
__device__ __forceinline__ float reduce_by_halving(float (&v)[32], int lane) {
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
    return v[0];
}

// A CTA owns four consecutive weight rows (two gate/up pairs of the gated epilogue); its eight warps split K between
// them (a warp takes 128 elements of every 1024), so that a narrow output still gives every SM several CTAs and each
// activation element loaded from L1 meets four weight rows.  MT tokens (8 or 16): 4 x MT sums per lane, summed over
// the lanes by halving and over the warps in shared memory in warp order.  Still plain 32-bit FMA.
template <typename TA, typename TW, typename TC, int MT>
__global__ void __launch_bounds__(kFewThreads)
gemm_fewrows_kernel(const TA* __restrict__ A, int lda, const TW* __restrict__ W, int ldw, TC* __restrict__ C, int ldc,
                    int M, int N, int K, int epilogue) {
    __shared__ float part[kFewWarps][kFewRows * MT];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kFewRows;
    const TW* w[kFewRows];
#pragma unroll
    for (int r = 0; r < kFewRows; ++r) w[r] = W + (size_t)min(n0 + r, N - 1) * ldw;   // clamped: read, never stored
    float acc[kFewRows * MT];
#pragma unroll
    for (int i = 0; i < kFewRows * MT; ++i) acc[i] = 0.f;
#pragma unroll 2
    for (int k = (warp * 32 + lane) * 4; k < K; k += kFewWarps * 128) {
        float4 wv[kFewRows];
#pragma unroll
        for (int r = 0; r < kFewRows; ++r) wv[r] = load4<TW>(w[r] + k);
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            if (m < M) {
                const float4 x = load4<TA>(A + (size_t)m * lda + k);
#pragma unroll
                for (int r = 0; r < kFewRows; ++r)
                    acc[r * MT + m] = fmaf(wv[r].w, x.w, fmaf(wv[r].z, x.z, fmaf(wv[r].y, x.y, fmaf(wv[r].x, x.x, acc[r * MT + m]))));
            }
        }
    }
    // lane l ends up with sum number l (and l + 32 for 16 tokens) of this warp
#pragma unroll
    for (int b = 0; b < kFewRows * MT / 32; ++b) {
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = acc[b * 32 + i];
        part[warp][b * 32 + lane] = reduce_by_halving(v, lane);
    }
    __syncthreads();
    // thread i < 4 * MT: row i / MT, token i % MT; the warps' sums are added in warp order
    const int i = threadIdx.x;
    if (i >= kFewRows * MT) return;
    const int r = i / MT, m = i % MT, n = n0 + r;
    float sum = 0.f;
#pragma unroll
    for (int wp = 0; wp < kFewWarps; ++wp) sum += part[wp][i];
    if (epilogue == 2) {
        float up = 0.f;   // the gate row's thread also adds up the up row (the next row of the CTA)
        if ((r & 1) == 0) {
#pragma unroll
            for (int wp = 0; wp < kFewWarps; ++wp) up += part[wp][i + MT];
            if (m < M && n + 1 < N) C[(size_t)m * ldc + n / 2] = from_f32<TC>((sum / (1.0f + expf(-sum))) * up);
        }
    } else if (m < M && n < N) {
        TC* c = C + (size_t)m * ldc + n;
        if (epilogue == 1) *c = from_f32<TC>(to_f32<TC>(*c) + sum);
        else *c = from_f32<TC>(sum);
    }
}

template <typename TA, typename TW, typename TC>
static int launch_fewrows(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int epilogue,
                          cudaStream_t stream) {
    const dim3 grid((N + kFewRows - 1) / kFewRows);
    if (M <= 8)
        gemm_fewrows_kernel<TA, TW, TC, 8><<<grid, kFewThreads, 0, stream>>>((const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K, epilogue);
    else
        gemm_fewrows_kernel<TA, TW, TC, 16><<<grid, kFewThreads, 0, stream>>>((const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K, epilogue);
    return launch_status();
}

}  // namespace b200

extern "C" int b200_gemm_generic(const void* A, int a_dtype, int lda, const void* W, int w_dtype, int ldw, void* C,
                                 int c_dtype, int ldc, int M, int N, int K, int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || epilogue < 0 || epilogue > 2) return b200::kErrBadArgument;
    if (epilogue == 1 && c_dtype != b200::kF32) return b200::kErrBadArgument;
    if (epilogue == 2 && (N & 1)) return b200::kErrBadArgument;
    // a decode step's few rows: rows of 4 elements at a time, when the rows start on such a boundary
    const size_t a_el = a_dtype == b200::kF32 ? 4 : 2, w_el = w_dtype == b200::kF32 ? 4 : 2;
    if (M <= 16 && K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && ((uintptr_t)A % (4 * a_el)) == 0 && ((uintptr_t)W % (4 * w_el)) == 0) {
        B200_DISPATCH_DTYPE(a_dtype, TA, B200_DISPATCH_DTYPE2(w_dtype, TW, B200_DISPATCH_DTYPE3(c_dtype, TC,
            return b200::launch_fewrows<TA, TW, TC>(A, lda, W, ldw, C, ldc, M, N, K, epilogue, stream))));
    }
    if (M >= b200::kBigM && (M + b200::kBigM - 1) / b200::kBigM <= 65535) {
        dim3 big((N + b200::kBigN - 1) / b200::kBigN, (M + b200::kBigM - 1) / b200::kBigM);
        B200_DISPATCH_DTYPE(a_dtype, TA, B200_DISPATCH_DTYPE2(w_dtype, TW, B200_DISPATCH_DTYPE3(c_dtype, TC,
            b200::gemm_generic_big_kernel<TA, TW, TC><<<big, b200::kBigThreads, 0, stream>>>(
                (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K, epilogue))));
        return b200::launch_status();
    }
    dim3 grid((N + b200::kTileN - 1) / b200::kTileN, (M + b200::kTileM - 1) / b200::kTileM);
    if (grid.y > 65535) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(a_dtype, TA, B200_DISPATCH_DTYPE2(w_dtype, TW, B200_DISPATCH_DTYPE3(c_dtype, TC,
        b200::gemm_generic_kernel<TA, TW, TC><<<grid, b200::kGemmThreads, 0, stream>>>(
            (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K, epilogue))));
    return b200::launch_status();
}
