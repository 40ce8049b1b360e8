// Plain matrix product C = A W^T with 32-bit FMA accumulation, any storage types, any sizes.
//
// A is [M, K] (activations, row-major, row stride lda), W is [N, K] (a weight as the reference
// stores it: one row per output, core/model/tensor/FloatTensor.java:98-100 of the reference
// project).  This is the kernel of the true 32-bit path (no tensor cores, no reduced-precision
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

}  // namespace b200

extern "C" int b200_gemm_generic(const void* A, int a_dtype, int lda, const void* W, int w_dtype, int ldw, void* C,
                                 int c_dtype, int ldc, int M, int N, int K, int epilogue, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || epilogue < 0 || epilogue > 2) return b200::kErrBadArgument;
    if (epilogue == 1 && c_dtype != b200::kF32) return b200::kErrBadArgument;
    if (epilogue == 2 && (N & 1)) return b200::kErrBadArgument;
    dim3 grid((N + b200::kTileN - 1) / b200::kTileN, (M + b200::kTileM - 1) / b200::kTileM);
    if (grid.y > 65535) return b200::kErrUnsupportedSize;
    B200_DISPATCH_DTYPE(a_dtype, TA, B200_DISPATCH_DTYPE2(w_dtype, TW, B200_DISPATCH_DTYPE3(c_dtype, TC,
        b200::gemm_generic_kernel<TA, TW, TC><<<grid, b200::kGemmThreads, 0, stream>>>(
            (const TA*)A, lda, (const TW*)W, ldw, (TC*)C, ldc, M, N, K, epilogue))));
    return b200::launch_status();
}
