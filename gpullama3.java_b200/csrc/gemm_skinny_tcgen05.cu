// Matrix product for steps with few tokens (17 .. 128) in bfloat16 on tcgen05 tensor cores:
//     C[M, N] = A[M, K] W[N, K]^T,  M small, N and K large.
// With so few tokens the product is a stream of W from HBM, so the roles of the operands are
// swapped against the prefill kernel: 128 weight rows are the M side of the tensor-core tile and
// the tokens are its N side (BT = 32, 64 or 128 columns of tensor memory).  TMA brings a
// 128 x 64 slice of W and a BT x 64 slice of A per stage through a ring (24 KB per stage at 64 tokens;
// 8 stages and one CTA per SM, or 4 stages and two), one thread issues tcgen05.mma, four warps read
// the accumulator back.
// (The reference does these products one output row per work-group,
// tornadovm/TransformerComputeKernelsLayered.java:901-930 of the reference project.)
//
// Narrow outputs (few tiles of 128 rows) would leave most SMs idle, so K is also cut into
// `k_splits` spans (up to 8), one CTA each, and the CTAs of a tile form a thread-block cluster.
// Each CTA leaves its partial tile in its own shared memory; after a cluster barrier every CTA
// adds up, for its share of the tokens, the partials of all spans in span order through
// distributed shared memory and applies the epilogue.  No scratch in global memory, no atomics:
// the sum does not depend on timing.
//
// Epilogues: 0 store, 1 residual add into float32 C, 2 silu(gate) * up on interleaved rows.
#include "tcgen05.cuh"

namespace b200 {

constexpr int kSkinnyThreads = 192;
constexpr int kRowsPerTile = 128;

__device__ int g_skinny_status = 0;

template <int BT, int STAGES>
struct SkinnySmem {
    alignas(1024) __nv_bfloat16 w[STAGES][kRowsPerTile * BK];
    alignas(1024) __nv_bfloat16 a[STAGES][BT * BK];
    alignas(8) uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
};

template <int EPI, typename TC>
__device__ __forceinline__ void skinny_emit(TC* __restrict__ C, int ldc, int token, int n, int N, float v, int lane) {
    if (EPI == 2) {
        const float other = __shfl_xor_sync(0xffffffffu, v, 1);  // lanes 2i, 2i+1 hold a gate row and its up row
        if ((lane & 1) == 0 && n + 1 < N) C[(size_t)token * ldc + (n >> 1)] = from_f32<TC>((v / (1.0f + expf(-v))) * other);
    } else if (n < N) {
        TC* c = C + (size_t)token * ldc + n;
        if (EPI == 1) *c = from_f32<TC>(to_f32<TC>(*c) + v);
        else *c = from_f32<TC>(v);
    }
}

template <int BT, int STAGES, int EPI, typename TC>
__global__ void __launch_bounds__(kSkinnyThreads, STAGES <= 4 ? 2 : 1)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_a,
                   TC* __restrict__ C, int ldc, int M, int N, int K, int blocks_per_split) {
    extern __shared__ uint8_t smem_raw[];
    auto& sm = *reinterpret_cast<SkinnySmem<BT, STAGES>*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y, k_splits = gridDim.y;  // the cluster is (1, k_splits, 1)
    const int n0 = tile * kRowsPerTile;
    const int kb_total = (K + BK - 1) / BK;
    const int kb_begin = split * blocks_per_split;
    const int k_iters = max(0, min(kb_total, kb_begin + blocks_per_split) - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        mbar_init(&sm.acc_full, 1);
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(BT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    volatile int* abort_flag = &sm.abort_flag;
    pdl_launch_dependents();

    if (warp == 0 && lane == 0) {
        // ---- producer.  Weights do not depend on earlier kernels: the first stages of W are on their way
        // before the wait for the kernel that produces the activations.
        const int early = min(k_iters, STAGES);
        for (int it = 0; it < early; ++it) {
            mbar_expect_tx(&sm.full[it], (kRowsPerTile + BT) * BK * 2);
            tma_load_2d(sm.w[it], &map_w, (kb_begin + it) * BK, n0, &sm.full[it]);
        }
        pdl_wait();
        for (int it = 0; it < early; ++it) tma_load_2d(sm.a[it], &map_a, (kb_begin + it) * BK, 0, &sm.full[it]);
        for (int it = STAGES; it < k_iters; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&sm.empty[s], ((it / STAGES) - 1) & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_skinny_status, 0, (1 << 8) | s); break;
            }
            mbar_expect_tx(&sm.full[s], (kRowsPerTile + BT) * BK * 2);
            tma_load_2d(sm.w[s], &map_w, (kb_begin + it) * BK, n0, &sm.full[s]);
            tma_load_2d(sm.a[s], &map_a, (kb_begin + it) * BK, 0, &sm.full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: 128 weight rows x BT tokens
        constexpr uint32_t idesc = umma_idesc_bf16(kRowsPerTile, BT);
        bool ok = true;
        pdl_wait();  // no stage can fill before the predecessor has ended (A comes from it): sleep, do not poll

        for (int it = 0; it < k_iters; ++it) {
            const int s = it % STAGES;
            if (!mbar_wait(&sm.full[s], (it / STAGES) & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_skinny_status, 0, (2 << 8) | s); ok = false; break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t wd = umma_desc(sm.w[s]), ad = umma_desc(sm.a[s]);
#pragma unroll
            for (int k = 0; k < BK / 16; ++k) umma_bf16(tmem, wd + 2 * k, ad + 2 * k, idesc, (it | k) != 0);
            umma_commit(&sm.empty[s]);
        }
        if (ok && k_iters > 0) umma_commit(&sm.acc_full);
    }
    // every thread waits for the predecessor before global memory written by earlier kernels is touched below
    pdl_wait();

    if (warp >= 2) {
        // ---- epilogue.  Thread (quarter, lane) owns weight row n0 + 32 * quarter + lane; a TMEM load gives it
        // 32 tokens of that row; for one token the lanes of a warp are 32 consecutive outputs.
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane, n = n0 + r;
        bool ok = true;
        if (k_iters > 0) {
            ok = mbar_wait(&sm.acc_full, 0, abort_flag);
            if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_skinny_status, 0, (3 << 8) | quarter); }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BT; c0 += 32) {
                if (c0 >= M) break;
                float v[32];
                if (k_iters > 0) {
                    tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + c0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.f;
                }
                if (k_splits == 1 && EPI == 2) {
                    // lanes 2i, 2i+1 hold a gate row and its up row: one exchange per token pair gives the even
                    // lane the up value of the even token and the odd lane the gate value of the odd token
                    const bool odd = lane & 1;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? v[j] : v[j + 1], 1);
                        const float gate = odd ? got : v[j], up = odd ? v[j + 1] : got;
                        const int token = c0 + j + (odd ? 1 : 0);
                        if (token < M && (n | 1) < N)
                            C[(size_t)token * ldc + (n >> 1)] = from_f32<TC>(gate * __frcp_rn(1.0f + __expf(-gate)) * up);
                    }
                } else if (k_splits == 1) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < M) skinny_emit<EPI, TC>(C, ldc, c0 + j, n, N, v[j], lane);
                } else {
                    // the stage buffers are free once the accumulator is complete: the partial tile
                    // [token][row] goes where the first stages of W were (and, with a shallow ring and
                    // 128 tokens, on into the stages of A, which follow W without a gap)
                    using Smem = SkinnySmem<BT, STAGES>;
                    static_assert(offsetof(Smem, a) == sizeof(sm.w), "A follows W");
                    static_assert((size_t)BT * kRowsPerTile * 4 <= sizeof(sm.w) + sizeof(sm.a), "partial tile fits");
                    float* p = reinterpret_cast<float*>(sm.w) + (size_t)c0 * kRowsPerTile + r;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (c0 + j < M) p[(size_t)j * kRowsPerTile] = v[j];
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (k_splits > 1) {
        __syncthreads();    // the role branches have joined again: whole warps reach the cluster barrier
        cluster_sync_all();  // every span's partial tile is in its CTA's shared memory
        if (warp >= 2) {
            const int quarter = warp & 3;
            const int r = quarter * 32 + lane, n = n0 + r;
            uint32_t peer[8];  // this thread's row of the partial tile in every span's CTA
#pragma unroll
            for (int sp = 0; sp < 8; ++sp)
                peer[sp] = cluster_peer_address(reinterpret_cast<const float*>(sm.w) + r, sp < k_splits ? sp : 0);
            // this CTA's share of the tokens, two at a time so that up to 16 remote loads are in flight
            for (int token = split; token < M; token += 2 * k_splits) {
                const int token2 = token + k_splits;
                float v0[8], v1[8];
#pragma unroll
                for (int sp = 0; sp < 8; ++sp) {
                    v0[sp] = sp < k_splits ? cluster_load_f32(peer[sp] + (uint32_t)token * kRowsPerTile * 4) : 0.f;
                    v1[sp] = (sp < k_splits && token2 < M) ? cluster_load_f32(peer[sp] + (uint32_t)token2 * kRowsPerTile * 4) : 0.f;
                }
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int sp = 0; sp < 8; ++sp) { s0 += v0[sp]; s1 += v1[sp]; }  // span order, zeros beyond k_splits
                skinny_emit<EPI, TC>(C, ldc, token, n, N, s0, lane);
                if (token2 < M) skinny_emit<EPI, TC>(C, ldc, token2, n, N, s1, lane);
            }
        }
        cluster_sync_all();  // no CTA leaves while a peer may still read its shared memory
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BT) : "memory");
    }
}

template <int BT, int STAGES, int EPI, typename TC>
static int launch_skinny(const CUtensorMap& mw, const CUtensorMap& ma, void* C, int ldc, int M, int N, int K,
                         int k_splits, int blocks_per_split, cudaStream_t stream) {
    const size_t smem = sizeof(SkinnySmem<BT, STAGES>) + 1024;
    static bool configured = false;
    auto kernel = gemm_skinny_kernel<BT, STAGES, EPI, TC>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + kRowsPerTile - 1) / kRowsPerTile, k_splits);
    cfg.blockDim = dim3(kSkinnyThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n_attr = 0;
    if (pdl_enabled()) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        ++n_attr;
    }
    if (k_splits > 1) {  // the spans of one tile are one cluster
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 1;
        attr[n_attr].val.clusterDim.y = k_splits;
        attr[n_attr].val.clusterDim.z = 1;
        ++n_attr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n_attr;
    return (int)cudaLaunchKernelEx(&cfg, kernel, mw, ma, (TC*)C, ldc, M, N, K, blocks_per_split);
}

template <int BT, int STAGES>
static int dispatch_skinny(const CUtensorMap& mw, const CUtensorMap& ma, void* C, int c_dtype, int ldc, int M, int N,
                           int K, int epilogue, int k_splits, int bps, cudaStream_t st) {
    if (epilogue == 2) return launch_skinny<BT, STAGES, 2, __nv_bfloat16>(mw, ma, C, ldc, M, N, K, k_splits, bps, st);
    if (epilogue == 1) return launch_skinny<BT, STAGES, 1, float>(mw, ma, C, ldc, M, N, K, k_splits, bps, st);
    if (c_dtype == kF32) return launch_skinny<BT, STAGES, 0, float>(mw, ma, C, ldc, M, N, K, k_splits, bps, st);
    return launch_skinny<BT, STAGES, 0, __nv_bfloat16>(mw, ma, C, ldc, M, N, K, k_splits, bps, st);
}

static int token_tile(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }

static int sm_count() {  // of the current device
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        cached[dev] = (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && n > 0) ? n : 148;
    }
    return cached[dev];
}

}  // namespace b200

extern "C" int b200_gemm_skinny_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, b200::g_skinny_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(b200::g_skinny_status, &zero, sizeof(int));
    return v;
}

// How many spans K is cut into for (M, N, K) on a GPU with n_sms SMs (1 .. 8).
extern "C" int b200_gemm_skinny_splits(int M, int N, int K, int n_sms) {
    using namespace b200;
    if (M <= 0 || N <= 0 || K < 8) return 1;
    const int tiles = (N + kRowsPerTile - 1) / kRowsPerTile;
    const int kb = (K + BK - 1) / BK;
    // Measured on B200 (two CTAs of the shallow ring per SM): narrow outputs want as many spans as keep the
    // grid within two CTAs per SM, up to 8, each span with at least 4 stages of work; an output that fills
    // half the SMs with its tiles alone is not cut.
    int splits = 1;
    if (tiles * 2 <= n_sms)
        for (int s = 8; s >= 2; s /= 2)
            if (tiles * s <= 2 * n_sms && kb >= 4 * s) { splits = s; break; }
    const int bps = (kb + splits - 1) / splits;
    return (kb + bps - 1) / bps;                 // no empty span
}

extern "C" int b200_gemm_skinny(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M,
                                int N, int K, int epilogue, int k_splits, cudaStream_t stream) {
    using namespace b200;
    if (M <= 0 || N <= 0) return 0;
    if (M > 128 || K < 8 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || (((uintptr_t)A | (uintptr_t)W) & 15)) return kErrUnsupportedSize;
    if (epilogue < 0 || epilogue > 2 || (epilogue == 1 && c_dtype != kF32) || (epilogue == 2 && ((N & 1) || c_dtype != kBF16)))
        return kErrBadArgument;
    if (c_dtype != kF32 && c_dtype != kBF16) return kErrBadArgument;
    const int kb = (K + BK - 1) / BK;
    if (k_splits < 1 || k_splits > 8 || k_splits > kb) return kErrBadArgument;
    const int bps = (kb + k_splits - 1) / k_splits;
    const int bt = token_tile(M);
    CUtensorMap mw, ma;
    if (!make_map(&mw, W, N, K, ldw, kRowsPerTile) || !make_map(&ma, A, M, K, lda, bt)) return kErrUnsupportedSize;
    // Two ring depths.  Deep (one CTA per SM, 8 stages): a grid of one wave without K spans, where a second
    // resident CTA would have nothing to do.  Shallow (half the stages, two CTAs per SM): every other grid;
    // clusters of spans fill the SMs twice over, and in a grid of many waves one CTA's start-up and epilogue
    // hide behind its neighbour's stream.
    const int tiles = (N + kRowsPerTile - 1) / kRowsPerTile;
    const bool shallow = k_splits > 1 || tiles > sm_count();
    if (bt == 32) {
        if (shallow) return dispatch_skinny<32, 4>(mw, ma, C, c_dtype, ldc, M, N, K, epilogue, k_splits, bps, stream);
        return dispatch_skinny<32, 8>(mw, ma, C, c_dtype, ldc, M, N, K, epilogue, k_splits, bps, stream);
    }
    if (bt == 64) {
        if (shallow) return dispatch_skinny<64, 4>(mw, ma, C, c_dtype, ldc, M, N, K, epilogue, k_splits, bps, stream);
        return dispatch_skinny<64, 8>(mw, ma, C, c_dtype, ldc, M, N, K, epilogue, k_splits, bps, stream);
    }
    if (shallow) return dispatch_skinny<128, 3>(mw, ma, C, c_dtype, ldc, M, N, K, epilogue, k_splits, bps, stream);
    return dispatch_skinny<128, 6>(mw, ma, C, c_dtype, ldc, M, N, K, epilogue, k_splits, bps, stream);
}
