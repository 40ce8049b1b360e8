// RMSNorm over rows of the 32-bit residual stream.
//   ss = sum(x^2) / dim + eps ;  out = w * ((1 / sqrt(ss)) * x)
// as inference/InferenceCore.java:47-56 of the reference project computes it (eps inside the root,
// added after the mean; the weight multiplies plainly).  The sum of squares and the scale are
// 32-bit whatever the storage types.  `rows` (optional) selects which rows of x are normalised,
// so that only the positions whose logits are wanted reach the output head.
#include "common.cuh"

namespace b200 {

template <typename TW, typename TO>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                               const int* __restrict__ rows, int dim, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
    float ss = 0.f;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float v = xr[i]; ss += v * v; }
    ss = block_sum(ss, scratch);
    const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
    TO* o = out + (size_t)r * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TO>(to_f32<TW>(w[i]) * (scale * xr[i]));
}

}  // namespace b200

extern "C" int b200_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype,
                            const int* rows, int n_rows, int dim, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const int threads = dim >= 1024 ? 256 : 128;
    B200_DISPATCH_DTYPE(w_dtype, TW, B200_DISPATCH_DTYPE2(out_dtype, TO,
        return b200::launch_pdl(b200::rmsnorm_kernel<TW, TO>, dim3(n_rows), dim3(threads), 0, stream, x, (const TW*)w,
                                (TO*)out, rows, dim, eps)));
    return b200::launch_status();
}
