// RMSNorm over rows of the 32-bit residual stream.
//   ss = sum(x^2) / dim + eps ;  out = w * ((1 / sqrt(ss)) * x)
// as inference/InferenceCore.java:47-56 of the reference project computes it (eps inside the root,
// added after the mean; the weight multiplies plainly).  The sum of squares and the scale are
// 32-bit whatever the storage types.  `rows` (optional) selects which rows of x are normalised,
// so that only the positions whose logits are wanted reach the output head.
#include "common.cuh"

namespace b200 {

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&f)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&f)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xffff0000u);
    f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xffff0000u);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&f)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&f)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

constexpr int kNormThreads = 256;
constexpr int kNormKeep = 4;  // groups of 4 elements a thread keeps in registers between the two passes

// VEC: rows are read and written four elements at a time (dim a multiple of 4, pointers aligned); the first
// kNormKeep * 4 * 256 elements of a row stay in registers, so x is read once for the usual widths.
template <typename TW, typename TO, bool VEC>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
               const int* __restrict__ rows, int dim, float eps) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
    TO* o = out + (size_t)r * dim;
    float ss = 0.f;
    if (VEC) {
        float keep[kNormKeep][4];
#pragma unroll
        for (int k = 0; k < kNormKeep; ++k) {
            const int i = (k * kNormThreads + threadIdx.x) * 4;
            if (i < dim) {
                load4<float>(xr + i, keep[k]);
#pragma unroll
                for (int e = 0; e < 4; ++e) ss += keep[k][e] * keep[k][e];
            }
        }
        for (int i = (kNormKeep * kNormThreads + threadIdx.x) * 4; i < dim; i += kNormThreads * 4) {
            float v[4];
            load4<float>(xr + i, v);
#pragma unroll
            for (int e = 0; e < 4; ++e) ss += v[e] * v[e];
        }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
#pragma unroll
        for (int k = 0; k < kNormKeep; ++k) {
            const int i = (k * kNormThreads + threadIdx.x) * 4;
            if (i < dim) {
                float wv[4], y[4];
                load4<TW>(w + i, wv);
#pragma unroll
                for (int e = 0; e < 4; ++e) y[e] = wv[e] * (scale * keep[k][e]);
                store4<TO>(o + i, y);
            }
        }
        for (int i = (kNormKeep * kNormThreads + threadIdx.x) * 4; i < dim; i += kNormThreads * 4) {
            float v[4], wv[4], y[4];
            load4<float>(xr + i, v);
            load4<TW>(w + i, wv);
#pragma unroll
            for (int e = 0; e < 4; ++e) y[e] = wv[e] * (scale * v[e]);
            store4<TO>(o + i, y);
        }
    } else {
        for (int i = threadIdx.x; i < dim; i += blockDim.x) { const float v = xr[i]; ss += v * v; }
        ss = block_sum(ss, scratch);
        const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
        for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = from_f32<TO>(to_f32<TW>(w[i]) * (scale * xr[i]));
    }
}

// One warp per row for the usual widths (dim = 128 * KEEP): the whole row sits in the warp's registers after one
// round of 16-byte loads that are all in flight together, the sum of squares is a shuffle tree, and no barrier is
// needed; a CTA of eight warps takes eight rows.
constexpr int kNormWarps = 8;

template <typename TW, typename TO, int KEEP>
__global__ void __launch_bounds__(kNormWarps * 32)
rmsnorm_warp_kernel(const float* __restrict__ x, const TW* __restrict__ w, TO* __restrict__ out,
                    const int* __restrict__ rows, int n_rows, float eps) {
    constexpr int dim = KEEP * 128;
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * kNormWarps + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * dim;
    float keep[KEEP][4];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < KEEP; ++k) load4<float>(xr + (k * 32 + lane) * 4, keep[k]);
#pragma unroll
    for (int k = 0; k < KEEP; ++k)
#pragma unroll
        for (int e = 0; e < 4; ++e) ss += keep[k][e] * keep[k][e];
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float scale = 1.0f / sqrtf(ss / (float)dim + eps);
    TO* o = out + (size_t)r * dim;
#pragma unroll
    for (int k = 0; k < KEEP; ++k) {
        float wv[4], y[4];
        load4<TW>(w + (k * 32 + lane) * 4, wv);
#pragma unroll
        for (int e = 0; e < 4; ++e) y[e] = wv[e] * (scale * keep[k][e]);
        store4<TO>(o + (k * 32 + lane) * 4, y);
    }
}

template <typename TW, typename TO, int KEEP>
static int launch_norm_warp(const float* x, const void* w, void* out, const int* rows, int n_rows, float eps, cudaStream_t stream) {
    return launch_pdl(rmsnorm_warp_kernel<TW, TO, KEEP>, dim3((n_rows + kNormWarps - 1) / kNormWarps), dim3(kNormWarps * 32), 0,
                      stream, x, (const TW*)w, (TO*)out, rows, n_rows, eps);
}

}  // namespace b200

extern "C" int b200_rmsnorm(const float* x, const void* w, int w_dtype, void* out, int out_dtype,
                            const int* rows, int n_rows, int dim, float eps, cudaStream_t stream) {
    if (n_rows <= 0) return 0;
    const bool vec = dim % 4 == 0 && ((((uintptr_t)x) | ((uintptr_t)w) | ((uintptr_t)out)) & 15) == 0;
    if (vec && n_rows >= 1024 && dim % 1024 == 0 && dim <= 4096) {   // rows for every SM several times over, of a usual width: a warp per row
        B200_DISPATCH_DTYPE(w_dtype, TW, B200_DISPATCH_DTYPE2(out_dtype, TO,
            switch (dim / 1024) {
                case 1: return b200::launch_norm_warp<TW, TO, 8>(x, w, out, rows, n_rows, eps, stream);
                case 2: return b200::launch_norm_warp<TW, TO, 16>(x, w, out, rows, n_rows, eps, stream);
                case 3: return b200::launch_norm_warp<TW, TO, 24>(x, w, out, rows, n_rows, eps, stream);
                default: return b200::launch_norm_warp<TW, TO, 32>(x, w, out, rows, n_rows, eps, stream);
            }));
    }
    B200_DISPATCH_DTYPE(w_dtype, TW, B200_DISPATCH_DTYPE2(out_dtype, TO,
        return vec ? b200::launch_pdl(b200::rmsnorm_kernel<TW, TO, true>, dim3(n_rows), dim3(b200::kNormThreads), 0, stream, x,
                                      (const TW*)w, (TO*)out, rows, dim, eps)
                   : b200::launch_pdl(b200::rmsnorm_kernel<TW, TO, false>, dim3(n_rows), dim3(b200::kNormThreads), 0, stream, x,
                                      (const TW*)w, (TO*)out, rows, dim, eps)));
    return b200::launch_status();
}
