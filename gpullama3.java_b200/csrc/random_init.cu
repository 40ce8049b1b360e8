// Random weights on the device: element i of a tensor is a fixed function of (key, i), the same
// function weights/random_init.py evaluates with numpy, so that a model filled here and a model
// folder written on the CPU from the same seed hold the same bits.  The reference project has no
// random-weights mode (its loader, model/loader/ModelLoader.java:233-303, only reads files).
//
// value(i) = offset + scale * (s(i) - 524280), where s(i) is the sum of the sixteen 16-bit fields
// of outputs 4i .. 4i+3 of the splitmix64 sequence started at `key`: an integer below 2^20, so its
// conversion to float is exact, and the one multiplication and the one addition that follow round
// the same way everywhere (they are kept apart: no fused multiply-add).  The sum of sixteen uniform
// numbers is normal to a good approximation (bounded at 6.9 standard deviations).
#include "common.cuh"

namespace b200 {

__device__ __forceinline__ unsigned long long splitmix64_at(unsigned long long key, unsigned long long n) {
    unsigned long long z = key + (n + 1ull) * 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

template <typename T>
__global__ void random_fill_kernel(T* __restrict__ out, long long n, unsigned long long key, float scale, float offset) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        unsigned int sum = 0;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const unsigned long long z = splitmix64_at(key, 4ull * (unsigned long long)i + r);
            sum += (unsigned int)(z & 0xFFFFull) + (unsigned int)((z >> 16) & 0xFFFFull) +
                   (unsigned int)((z >> 32) & 0xFFFFull) + (unsigned int)(z >> 48);
        }
        const float centred = (float)((int)sum - 524280);
        out[i] = from_f32<T>(__fadd_rn(offset, __fmul_rn(centred, scale)));
    }
}

}  // namespace b200

extern "C" int b200_random_fill(void* out, int dtype, long long n, unsigned long long key, float scale, float offset,
                                cudaStream_t stream) {
    if (n <= 0) return 0;
    const long long want = (n + 255) / 256;
    const unsigned int blocks = (unsigned int)(want < b200::device_sm_count() * 32 ? want : b200::device_sm_count() * 32);
    B200_DISPATCH_DTYPE(dtype, T,
        b200::random_fill_kernel<T><<<blocks, 256, 0, stream>>>((T*)out, n, key, scale, offset));
    return b200::launch_status();
}
