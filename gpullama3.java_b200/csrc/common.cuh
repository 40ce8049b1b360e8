// Shared helpers of the sm_100a kernel libraries.
//
// Every library exports plain C functions ("extern \"C\" int b200_*") that take raw device
// pointers, sizes and a cudaStream_t, launch on that stream and return the cudaError_t of the
// launch as an int (0 = success).  Nothing here allocates device memory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

namespace b200 {

// Storage types a tensor may have.  The codes are part of the C ABI (python passes them).
enum DType : int { kF32 = 0, kBF16 = 1 };

// Tokens of one cache page.  A sequence's keys and values live in pages of this many positions.
constexpr int kPageTokens = 64;

// Error codes returned for arguments a kernel refuses (distinct from cudaError_t values).
constexpr int kErrBadArgument = 10001;
constexpr int kErrUnsupportedSize = 10002;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a CTA of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

inline int launch_status() { return (int)cudaPeekAtLastError(); }

// SMs of the current device (asked once per device; 148, a B200's, only if the driver does not answer).
inline int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    return cached[dev];
}

// Programmatic dependent launch.  A kernel launched with launch_pdl may start while its
// predecessor on the stream is still running; it must call pdl_wait() before it touches anything a
// predecessor wrote (or writes anything a predecessor reads).  What it does before that call
// (index arithmetic, loading weights, which no kernel writes) overlaps the predecessor's tail and
// the launch latency.  pdl_launch_dependents() lets the successor be scheduled as soon as every
// CTA of this kernel has started.  Every thread of such a kernel calls pdl_wait(), so that the
// completion of a kernel implies the completion of everything before it.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

inline bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("GPULLAMA3_B200_NO_PDL");
        on = (e && e[0] && e[0] != '0') ? 0 : 1;
    }
    return on == 1;
}

// The general form: CTAs grouped into thread-block clusters of `cluster` (1, 1, 1: no clusters), and
// `early_start` false for a kernel that should find the GPU empty.  A long kernel whose grid just fills the
// SMs is such a kernel: started early, its CTAs settle wherever the predecessor's CTAs leave room, unevenly, and
// the SMs that got more of them finish late.
template <typename... KArgs, typename... Args>
inline int launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              dim3 cluster, bool early_start, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    if (cluster.x * cluster.y * cluster.z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = cluster.x;
        attr[n].val.clusterDim.y = cluster.y;
        attr[n].val.clusterDim.z = cluster.z;
        ++n;
    }
    if (pdl_enabled() && early_start) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

template <typename... KArgs, typename... Args>
inline int launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    return launch_pdl_cluster(kernel, grid, block, smem, stream, dim3(1, 1, 1), true, args...);
}

// Thread-block clusters: barrier over all threads of the cluster, and reads of a peer CTA's shared memory.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address, in the cluster's shared window, of `local` as it sits in the CTA of rank `rank`.
__device__ __forceinline__ uint32_t cluster_peer_address(const void* local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;"
                 : "=r"(remote) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    return remote;
}
__device__ __forceinline__ float cluster_load_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr));
    return v;
}

}  // namespace b200

// Calls `body` with `T` bound to the storage type of `code`; unknown codes return kErrBadArgument.
#define B200_DISPATCH_DTYPE(code, T, ...)                                   \
    do {                                                                    \
        if ((code) == b200::kF32) { using T = float; __VA_ARGS__; }         \
        else if ((code) == b200::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return b200::kErrBadArgument;                                  \
    } while (0)

// Same as B200_DISPATCH_DTYPE; a second and third name because a macro cannot expand inside itself.
#define B200_DISPATCH_DTYPE2(code, T, ...)                                  \
    do {                                                                    \
        if ((code) == b200::kF32) { using T = float; __VA_ARGS__; }         \
        else if ((code) == b200::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return b200::kErrBadArgument;                                  \
    } while (0)
#define B200_DISPATCH_DTYPE3(code, T, ...)                                  \
    do {                                                                    \
        if ((code) == b200::kF32) { using T = float; __VA_ARGS__; }         \
        else if ((code) == b200::kBF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
        else return b200::kErrBadArgument;                                  \
    } while (0)
