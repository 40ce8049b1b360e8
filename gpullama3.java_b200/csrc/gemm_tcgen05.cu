// Prefill matrix product in bfloat16 on the 5th-generation tensor cores:
//     C[M, N] = A[M, K] W[N, K]^T      (A activations, W a weight as stored: one row per output)
// The reference computes the same products row by row on CUDA cores
// (tornadovm/TransformerComputeKernelsLayered.java:901-930 of the reference project, fused
// residual :766-784, fused SiLU gate :808-826); here a 128 x BN tile of C is accumulated in
// tensor memory by tcgen05.mma, fed by TMA through a ring of shared-memory stages.
//
// Persistent CTAs (one per SM) each compute a sequence of tiles.  Roles (192 threads):
//   warp 0, one lane   producer: waits for a free stage, arms its mbarrier with the byte count and
//                      issues two TMA loads (A box 64x128, W box 64xBN; 128-byte swizzle)
//   warp 1, one lane   issues four tcgen05.mma (K = 16 each) per stage into the TMEM accumulator,
//                      then tcgen05.commit onto the stage's "empty" mbarrier; after a tile's last stage
//                      a commit onto that accumulator's "full" mbarrier.  Two accumulators (2 x BN columns
//                      of TMEM, owned by warp 1) alternate, so the next tile's main loop runs while the
//                      epilogue warps still read the previous tile out.
//   warps 2..5         epilogue: tcgen05.ld 32 lanes x 32 columns at a time, then one of
//                      0 store (bfloat16 or float32), 1 residual add into float32 C,
//                      2 silu(gate) * up on interleaved gate/up columns (bfloat16 out, N/2 wide).
//                      The residual add leaves the SM as a bulk tensor reduction: a warp puts its 32 x 32
//                      sums into shared memory and one cp.reduce.async.bulk.tensor (.add, float32) lets the
//                      L2 add them to C; the SM never reads the residual stream, and nothing is strided (a
//                      thread per row would touch 32 rows with every access).  Each element is added once.
//                      (Stores of bfloat16 results through such boxes were measured and gained nothing.)
//                      3 the query/key/value product of a prompt pass: rotation and cache write (RopeEpilogue).
// Three kernels share these roles and epilogues: the one just described; pairs of CTAs on 256-row tiles
// (gemm_tcgen05_pair_kernel, tcgen05 cta_group::2), which large products take; and K cut into spans over a cluster
// (gemm_tcgen05_spans_kernel) for few tiles with a long K.  Tiles are walked in bands of rows (tile_coords).
// Edges: TMA zero-fills rows and K beyond the tensors, stores are bounds-checked, so any M, N and
// any K that keeps rows 16-byte aligned (K % 8 == 0) are accepted.
// Every mbarrier wait is bounded: when a wait gives up, the kernel records a code in a status
// word, all roles fall through to the common exit, TMEM is freed and the kernel returns.
#include "tcgen05.cuh"

namespace b200 {

constexpr int BM = 128;
constexpr int kGemmTcThreads = 192;

__device__ int g_gemm_status = 0;  // 0 ok; else (role << 8 | stage) of the wait that gave up

template <int BN, int STAGES>
struct GemmSmem {
    alignas(1024) __nv_bfloat16 a[STAGES][BM * BK];
    alignas(1024) __nv_bfloat16 b[STAGES][BN * BK];
    alignas(8) uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];   // MMA -> epilogue: accumulator b holds a finished tile
    uint64_t acc_empty[2];  // epilogue -> MMA: accumulator b has been read out
    uint32_t tmem_base;
    int abort_flag;
};

// What the residual epilogue adds beside the ring: one 32 x 32 float32 box per epilogue warp (128-byte swizzle).
struct ResidualStage {
    alignas(1024) float box[4][32 * 32];
};

// C[box at (col, row)] += the 32 x 32 float32 box in shared memory, done by the L2 (rows and columns beyond C are clipped)
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, int col, int row, const void* src) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(map), "r"(col), "r"(row), "r"(smem_u32(src)) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// What the fused-projection epilogue (EPI 3) needs: the product is the query, key and value projection of T tokens
// ([T, (heads + 2 kv_heads) head_dim], heads of head_dim 64 or 128 lying whole inside a 256-column tile), and its
// epilogue does what a kernel of its own does otherwise (inference/InferenceCore.java:83-101 of the reference project):
// queries are rotated and stored to C, keys are rotated and stored at their position in the cache pages, values are
// stored there transposed.  Every sum is first rounded to bfloat16, as the stored projection would be, then rotated in
// float32 with the angles of the token's position (cosine and sine per pair, made once per pass) and rounded again:
// the same bits as the two kernels one after the other.
struct RopeEpilogue {
    const int* positions;      // [T]
    const int* seq_ids;        // [T]
    const int* page_table;     // [n_seqs][table_stride]
    int table_stride;
    const float2* angles;      // [head_dim / 2][T]: (cos, sin) of position * frequency (a warp's 32 tokens read neighbours)
    int n_tokens;              // T
    __nv_bfloat16* k_pool;     // [page][kv_head][64][head_dim]
    __nv_bfloat16* v_pool;     // [page][kv_head][head_dim][64]
    int n_heads, n_kv_heads, head_dim;
    int pairing;               // 0: (2j, 2j+1); 1: (j, j + head_dim/2)
    int write_cache;           // 0: keys and values are dropped (the layer reads a cache another layer writes)
};

__device__ __forceinline__ float round_bf16(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&v)[32]) {   // dst 16-byte aligned
    uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]), p1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
        __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]), p3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
        d[j] = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                          *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
    }
}

// One warp's 32 rows of a tile that holds whole heads.  Row = token; a head's columns are taken 32 at a time (with the
// half pairing together with the 32 columns head_dim / 2 further on, where the partners are).
template <int BN>
__device__ __forceinline__ void epilogue_qkv_rope(uint32_t acc, int quarter, int lane, int m0, int n0, int M, int N,
                                                  __nv_bfloat16* __restrict__ C, int ldc, const RopeEpilogue& rp) {
    const int row = m0 + quarter * 32 + lane;
    const bool live = row < M;
    const int D = rp.head_dim, half = D / 2;
    const int q_dim = rp.n_heads * D, kv_dim = rp.n_kv_heads * D;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int pos = live ? rp.positions[row] : 0;
    const float2* ang = rp.angles + (live ? row : 0);   // pair i of this token: ang[i * T]
    const size_t T = (size_t)rp.n_tokens;
    size_t page = 0;
    if (live && rp.write_cache && n0 + BN > q_dim) page = (size_t)rp.page_table[(size_t)rp.seq_ids[row] * rp.table_stride + pos / 64];
    const int in_page = pos % 64;
#pragma unroll 1
    for (int h0 = 0; h0 < BN; h0 += D) {
        const int n = n0 + h0;            // first column of the head: a whole head of queries, keys or values
        if (n >= N) break;
        if (n >= q_dim + kv_dim) {        // values: transposed into the page, one element per dimension
            if (!rp.write_cache) continue;
            const int kvh = (n - q_dim - kv_dim) / D;
            __nv_bfloat16* dst = rp.v_pool + ((page * rp.n_kv_heads + kvh) * D) * 64 + in_page;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float v[32];
                tmem_ld32(acc + lane_base + h0 + c0, v);
                if (live) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) dst[(size_t)(c0 + j) * 64] = __float2bfloat16_rn(v[j]);
                }
            }
            continue;
        }
        __nv_bfloat16* dst;               // where the rotated head goes
        if (n < q_dim) {
            dst = C + (size_t)(live ? row : 0) * ldc + n;
        } else {
            if (!rp.write_cache) continue;
            const int kvh = (n - q_dim) / D;
            dst = rp.k_pool + ((page * rp.n_kv_heads + kvh) * 64 + in_page) * D;
        }
        if (rp.pairing == 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                float v[32];
                tmem_ld32(acc + lane_base + h0 + c0, v);
                if (!live) continue;
#pragma unroll
                for (int j = 0; j < 32; j += 2) {
                    const float2 a = ang[(size_t)((c0 + j) / 2) * T];
                    const float v0 = round_bf16(v[j]), v1 = round_bf16(v[j + 1]);
                    v[j] = v0 * a.x - v1 * a.y;
                    v[j + 1] = v0 * a.y + v1 * a.x;
                }
                store_bf16x32(dst + c0, v);
            }
        } else {
#pragma unroll 1
            for (int c0 = 0; c0 < half; c0 += 32) {
                float lo[32], hi[32];
                tmem_ld32(acc + lane_base + h0 + c0, lo);
                tmem_ld32(acc + lane_base + h0 + half + c0, hi);
                if (!live) continue;
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const float2 a = ang[(size_t)(c0 + j) * T];
                    const float v0 = round_bf16(lo[j]), v1 = round_bf16(hi[j]);
                    lo[j] = v0 * a.x - v1 * a.y;
                    hi[j] = v0 * a.y + v1 * a.x;
                }
                store_bf16x32(dst + c0, lo);
                store_bf16x32(dst + half + c0, hi);
            }
        }
    }
}

// The epilogue of one 128 x BN accumulator (TMEM columns acc .. acc + BN) by one of the four epilogue warps: warp
// `quarter` reads TMEM lanes 32 * quarter .. + 31, which are rows m0 + 32 * quarter .. of C; a thread holds one row, 32
// columns at a time.  `box` is the warp's 32 x 32 float32 staging box for the bulk reduction (EPI 1 with reduce_c).
template <int BN, int EPI, typename TC>
__device__ __forceinline__ void epilogue_tile(uint32_t acc, int quarter, int lane, int m0, int n0, int M, int N,
                                              TC* __restrict__ C, int ldc, int reduce_c, const CUtensorMap* map_c, float* box,
                                              const RopeEpilogue& rope) {
    if constexpr (EPI == 3) {
        epilogue_qkv_rope<BN>(acc, quarter, lane, m0, n0, M, N, reinterpret_cast<__nv_bfloat16*>(C), ldc, rope);
        return;
    }
    const int row = m0 + quarter * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        if (n0 + c0 >= N) break;  // uniform: whole chunk beyond the matrix
        float v[32];
        tmem_ld32(acc + ((uint32_t)(quarter * 32) << 16) + c0, v);
        if (EPI == 1 && reduce_c) {
            // the box is free once the reduction before has read it; row `lane` of the box, its eight
            // 16-byte pieces at piece ^ (row % 8): the layout the tensor map's 128-byte swizzle expects
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
            float* box_row = box + lane * 32;
#pragma unroll
            for (int j = 0; j < 8; ++j)
                *reinterpret_cast<float4*>(box_row + ((j ^ (lane & 7)) << 2)) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) {   // (columns of the box beyond C are clipped by the reduction, and so are rows beyond M)
                tma_reduce_add_2d(map_c, n0 + c0, m0 + quarter * 32, box);
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
            continue;
        }
        if (row >= M) continue;
        const int col = n0 + c0;
        if (EPI == 2) {
            TC* dst = C + (size_t)row * ldc + (col >> 1);
            if (col + 32 <= N && ((uintptr_t)dst & 15) == 0 && sizeof(TC) == 2) {
                uint32_t pk[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const float g0 = v[4 * j], u0 = v[4 * j + 1], g1 = v[4 * j + 2], u1 = v[4 * j + 3];
                    __nv_bfloat162 h = __floats2bfloat162_rn((g0 / (1.0f + expf(-g0))) * u0, (g1 / (1.0f + expf(-g1))) * u1);
                    pk[j] = *reinterpret_cast<uint32_t*>(&h);
                }
                uint4* d = reinterpret_cast<uint4*>(dst);
                d[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                d[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (col + 2 * j + 1 < N) dst[j] = from_f32<TC>((v[2 * j] / (1.0f + expf(-v[2 * j]))) * v[2 * j + 1]);
            }
        } else {
            TC* dst = C + (size_t)row * ldc + col;
            const bool whole = col + 32 <= N && ((uintptr_t)dst & 15) == 0;
            if (EPI == 1) {  // C is the float32 residual stream
                float* d = reinterpret_cast<float*>(dst);
                if (whole) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float4 r = *reinterpret_cast<float4*>(d + j);
                        r.x += v[j]; r.y += v[j + 1]; r.z += v[j + 2]; r.w += v[j + 3];
                        *reinterpret_cast<float4*>(d + j) = r;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) if (col + j < N) d[j] += v[j];
                }
            } else if (sizeof(TC) == 2 && whole) {
                uint4* d = reinterpret_cast<uint4*>(dst);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[8 * j], v[8 * j + 1]);
                    __nv_bfloat162 p1 = __floats2bfloat162_rn(v[8 * j + 2], v[8 * j + 3]);
                    __nv_bfloat162 p2 = __floats2bfloat162_rn(v[8 * j + 4], v[8 * j + 5]);
                    __nv_bfloat162 p3 = __floats2bfloat162_rn(v[8 * j + 6], v[8 * j + 7]);
                    d[j] = make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                                      *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (col + j < N) dst[j] = from_f32<TC>(v[j]);
            }
        }
    }
}

// The order of tiles: bands of kBandTiles rows of tiles, and inside a band down the rows first.  The CTAs that run at
// the same time then share a few blocks of W and the band's blocks of A, and W comes from memory once per band instead
// of once per row of tiles (a W larger than the L2 would otherwise stream from memory again and again).
constexpr int kBandTiles = 8;
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int band = tile / (kBandTiles * tiles_n), within = tile - band * kBandTiles * tiles_n;
    const int rows = min(kBandTiles, tiles_m - band * kBandTiles);
    tn = within / rows;
    tm = band * kBandTiles + (within - tn * rows);
}

// Persistent: CTA c computes tiles c, c + gridDim.x, ... in that order.  Two accumulators of BN columns live in tensor
// memory: while the epilogue warps read tile i out of one, the MMA thread already fills the other with tile i + 1.
template <int BN, int STAGES, int EPI, typename TC>
__global__ void __launch_bounds__(kGemmTcThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_c, int reduce_c, TC* __restrict__ C, int ldc, int M, int N, int K,
                    const RopeEpilogue rope) {
    extern __shared__ uint8_t smem_raw[];
    auto& sm = *reinterpret_cast<GemmSmem<BN, STAGES>*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    // (the residual epilogue's boxes follow the ring; the launch asks for them only when reduce_c is set)
    ResidualStage& cs = *reinterpret_cast<ResidualStage*>(reinterpret_cast<uint8_t*>(&sm) + ((sizeof(GemmSmem<BN, STAGES>) + 1023) & ~(size_t)1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + BM - 1) / BM, n_tiles = tiles_n * tiles_m;
    const int k_iters = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.acc_full[b], 1); mbar_init(&sm.acc_empty[b], 4); }
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        if (EPI == 1 && reduce_c) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
    }
    if (warp == 1) {  // tensor memory for two accumulators of BN columns x 128 lanes
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    volatile int* abort_flag = &sm.abort_flag;
    // barriers and tensor memory were set up while the kernel before may still have been running; its results
    // (A, and C for the residual epilogue) are touched only from here on
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---- producer
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * BM, n0 = tn * BN;
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(&sm.empty[s], ((it / STAGES) - 1) & 1, abort_flag)) {
                    *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (1 << 8) | s); ok = false; break;
                }
                mbar_expect_tx(&sm.full[s], (BM + BN) * BK * 2);
                tma_load_2d(sm.a[s], &map_a, k * BK, m0, &sm.full[s]);
                tma_load_2d(sm.b[s], &map_w, k * BK, n0, &sm.full[s]);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer
        constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
        int it = 0, local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            // the first use of each accumulator finds it free (a fresh barrier passes a wait for parity 1)
            if (!mbar_wait(&sm.acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (4 << 8) | buf); break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + buf * BN;
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(&sm.full[s], (it / STAGES) & 1, abort_flag)) {
                    *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (2 << 8) | s); ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = umma_desc(sm.a[s]), bd = umma_desc(sm.b[s]);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)  // 16 elements = 32 bytes further along K: +2 in the address field
                    umma_bf16(acc, ad + 2 * kk, bd + 2 * kk, idesc, (k | kk) != 0);
                umma_commit(&sm.empty[s]);  // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(&sm.acc_full[buf]);
        }
    } else if (warp >= 2) {
        // ---- epilogue: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
            const int buf = local & 1;
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * BM, n0 = tn * BN;
            bool ok = mbar_wait(&sm.acc_full[buf], (local >> 1) & 1, abort_flag);
            if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (3 << 8) | quarter); }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            epilogue_tile<BN, EPI, TC>(tmem + buf * BN, quarter, lane, m0, n0, M, N, C, ldc, reduce_c, &map_c, cs.box[quarter], rope);
            // this warp has read its lanes of the accumulator out: once all four have, the MMA thread may reuse it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
        }
        // the reductions this thread issued are complete (their sums are in C) before the kernel ends
        if (EPI == 1 && reduce_c && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same product by pairs of CTAs (tcgen05 cta_group::2).  The single-CTA kernel above is bound by the rate at which
// an SM can ask for operand rows (a 128 x 256 tile wants 384 rows of 128 bytes per k-step), not by its tensor core.
// Here the two CTAs of a cluster share one 256 x BN tile: each loads its own 128 rows of A and only half of the W
// stage (BN / 2 rows), the leader's MMA thread issues M = 256 instructions that read both CTAs' shared memory, and
// each CTA's tensor memory receives the 128 rows of the tile that belong to its rows of A.  Per flop an SM asks for a
// third fewer rows.  No operand is multicast: every load is an ordinary TMA load of the CTA's own box.
//   full[s]       on the leader, 2 arrivals: each CTA's producer announces its bytes there (the peer remotely) and
//                 both CTAs' loads complete on it, so one wait tells the MMA thread that the stage is whole
//   empty[s]      in each CTA, signalled by the leader's tcgen05.commit (to both CTAs at once)
//   acc_full[b]   in each CTA, likewise; acc_empty[b] on the leader, 8 arrivals (four epilogue warps of each CTA)
template <int BN, int STAGES>
struct PairSmem {
    alignas(1024) __nv_bfloat16 a[STAGES][BM * BK];
    alignas(1024) __nv_bfloat16 b[STAGES][(BN / 2) * BK];
    alignas(8) uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// an arrival (with bytes to expect) on an mbarrier given by its address in the cluster's shared window.  Relaxed: it
// publishes nothing the thread wrote (a release at cluster scope costs most of a microsecond, every k-step).
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar_addr, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.relaxed.cluster.shared::cluster.b64 _, [%0], %1;" ::"r"(bar_addr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
// TMA load into this CTA's shared memory whose completion is counted on an mbarrier of either CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t bar_addr) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(bar_addr) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, int accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the MMAs issued so far are complete, on the mbarrier at this address in both CTAs of the pair
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(both) : "memory");
}

template <int BN, int STAGES, int EPI, typename TC>
__global__ void __launch_bounds__(kGemmTcThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                         const __grid_constant__ CUtensorMap map_c, int reduce_c, TC* __restrict__ C, int ldc, int M, int N, int K,
                         const RopeEpilogue rope) {
    using Smem = PairSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    auto& sm = *reinterpret_cast<Smem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    ResidualStage& cs = *reinterpret_cast<ResidualStage*>(reinterpret_cast<uint8_t*>(&sm) + ((sizeof(Smem) + 1023) & ~(size_t)1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();          // 0: the leader, which issues the MMAs
    const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    const int tiles_n = (N + BN - 1) / BN, tiles_m = (M + 2 * BM - 1) / (2 * BM), n_tiles = tiles_n * tiles_m;
    const int k_iters = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 2); mbar_init(&sm.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sm.acc_full[b], 1); mbar_init(&sm.acc_empty[b], 8); }
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
        if (EPI == 1 && reduce_c) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
    }
    if (warp == 1) {  // two accumulators of BN columns in both CTAs' tensor memory: one warp of each CTA asks
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before either signals the other
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    volatile int* abort_flag = &sm.abort_flag;
    // one MMA writes both CTAs' tensor memory at the same address: the two allocations must agree
    if (threadIdx.x == 0) {
        uint32_t other;
        asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(other) : "r"(cluster_peer_address(&sm.tmem_base, rank ^ 1)));
        if (other != tmem) { *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (8 << 8) | rank); }
    }
    __syncthreads();
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        // ---- producer of this CTA's half of every stage
        int it = 0;
        bool ok = !*abort_flag;
        for (int tile = pair; tile < n_tiles && ok; tile += n_pairs) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * 2 * BM + rank * BM, n0 = tn * BN + rank * (BN / 2);
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(&sm.empty[s], ((it / STAGES) - 1) & 1, abort_flag)) {
                    *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (9 << 8) | s); ok = false; break;
                }
                const uint32_t full = cluster_peer_address(&sm.full[s], 0);
                if (rank == 0) mbar_expect_tx(&sm.full[s], (BM + BN / 2) * BK * 2);
                else mbar_expect_tx_cluster(full, (BM + BN / 2) * BK * 2);
                tma_load_2d_pair(sm.a[s], &map_a, k * BK, m0, full);
                tma_load_2d_pair(sm.b[s], &map_w, k * BK, n0, full);
            }
        }
    } else if (warp == 1 && lane == 0 && rank == 0) {
        // ---- MMA issuer of the pair
        constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN);
        int it = 0, local = 0;
        bool ok = !*abort_flag;
        for (int tile = pair; tile < n_tiles && ok; tile += n_pairs, ++local) {
            const int buf = local & 1;
            if (!mbar_wait(&sm.acc_empty[buf], ((local >> 1) & 1) ^ 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (12 << 8) | buf); break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem + buf * BN;
            for (int k = 0; k < k_iters; ++k, ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(&sm.full[s], (it / STAGES) & 1, abort_flag)) {
                    *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (10 << 8) | s); ok = false; break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t ad = umma_desc(sm.a[s]), bd = umma_desc(sm.b[s]);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)
                    umma_bf16_pair(acc, ad + 2 * kk, bd + 2 * kk, idesc, (k | kk) != 0);
                umma_commit_pair(&sm.empty[s]);
            }
            if (ok) umma_commit_pair(&sm.acc_full[buf]);
        }
    } else if (warp >= 2) {
        // ---- epilogue of this CTA's 128 rows of every tile
        const int quarter = warp & 3;
        int local = 0;
        for (int tile = pair; tile < n_tiles; tile += n_pairs, ++local) {
            const int buf = local & 1;
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * 2 * BM + rank * BM, n0 = tn * BN;
            bool ok = mbar_wait(&sm.acc_full[buf], (local >> 1) & 1, abort_flag);
            if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (11 << 8) | quarter); }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (m0 < M) epilogue_tile<BN, EPI, TC>(tmem + buf * BN, quarter, lane, m0, n0, M, N, C, ldc, reduce_c, &map_c, cs.box[quarter], rope);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_peer_address(&sm.acc_empty[buf], 0));
        }
        if (EPI == 1 && reduce_c && lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    cluster_sync_all();  // neither CTA leaves, or gives its tensor memory back, while the other may still signal it or compute into it
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The same product for a few hundred tokens and a long K (the down product of a short prompt): its few tiles
// leave most SMs idle and each CTA walks the whole of K alone.  Here the K range of a tile is cut into 2 or 4
// spans, one CTA each, which form a thread-block cluster.  Every CTA accumulates its span in tensor memory, copies
// the 128 x 128 partial tile to its shared memory (where the ring was), and after a cluster barrier each CTA adds,
// for its share of the tile's rows, the partial tiles in span order through distributed shared memory and runs
// the epilogue on whole rows (512 contiguous bytes per warp).  No atomics: the result does not depend on timing.
constexpr int kSplitBN = 128;
constexpr int kSplitStages = 6;
constexpr int kSplitPitch = kSplitBN + 4;  // floats per row of the partial tile: float4 stores of 8 rows hit 32 banks

__device__ __forceinline__ float4 cluster_load_f32x4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr));
    return v;
}

template <int EPI, typename TC>
__global__ void __launch_bounds__(kGemmTcThreads, 1)
gemm_tcgen05_spans_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
                          TC* __restrict__ C, int ldc, int M, int N, int K, int blocks_per_span) {
    constexpr int BN = kSplitBN, STAGES = kSplitStages;
    using Smem = GemmSmem<BN, STAGES>;
    static_assert(sizeof(float) * BM * kSplitPitch <= sizeof(Smem::a), "the partial tile fits in the stages of A");
    extern __shared__ uint8_t smem_raw[];
    auto& sm = *reinterpret_cast<Smem*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (N + BN - 1) / BN;
    const int tile = blockIdx.x, span = blockIdx.y, n_spans = gridDim.y;  // the cluster is (1, n_spans, 1)
    const int m0 = (tile / tiles_n) * BM, n0 = (tile % tiles_n) * BN;
    const int kb_total = (K + BK - 1) / BK;
    const int kb_begin = span * blocks_per_span;
    const int k_iters = max(0, min(kb_total, kb_begin + blocks_per_span) - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        mbar_init(&sm.acc_full[0], 1);
        sm.abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    volatile int* abort_flag = &sm.abort_flag;
    float* partial = reinterpret_cast<float*>(sm.a);  // [BM][kSplitPitch] once the accumulator is complete
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0 && lane == 0) {
        for (int k = 0; k < k_iters; ++k) {
            const int s = k % STAGES;
            if (k >= STAGES && !mbar_wait(&sm.empty[s], ((k / STAGES) - 1) & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (5 << 8) | s); break;
            }
            mbar_expect_tx(&sm.full[s], (BM + BN) * BK * 2);
            tma_load_2d(sm.a[s], &map_a, (kb_begin + k) * BK, m0, &sm.full[s]);
            tma_load_2d(sm.b[s], &map_w, (kb_begin + k) * BK, n0, &sm.full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
        bool ok = true;
        for (int k = 0; k < k_iters; ++k) {
            const int s = k % STAGES;
            if (!mbar_wait(&sm.full[s], (k / STAGES) & 1, abort_flag)) {
                *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (6 << 8) | s); ok = false; break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t ad = umma_desc(sm.a[s]), bd = umma_desc(sm.b[s]);
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) umma_bf16(tmem, ad + 2 * kk, bd + 2 * kk, idesc, (k | kk) != 0);
            umma_commit(&sm.empty[s]);
        }
        if (ok && k_iters > 0) umma_commit(&sm.acc_full[0]);
    } else if (warp >= 2) {
        // the accumulator's rows to shared memory: warp w reads TMEM lanes 32 * (w % 4) .. + 31, a row per thread
        const int quarter = warp & 3, r = quarter * 32 + lane;
        bool ok = true;
        if (k_iters > 0) {
            ok = mbar_wait(&sm.acc_full[0], 0, abort_flag);
            if (!ok && lane == 0) { *abort_flag = 1; atomicCAS(&g_gemm_status, 0, (7 << 8) | quarter); }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                float v[32];
                if (k_iters > 0) {
                    tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + c0, v);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0.f;
                }
                float4* dst = reinterpret_cast<float4*>(partial + (size_t)r * kSplitPitch + c0);
#pragma unroll
                for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();     // the roles have joined again: whole warps reach the cluster barrier
    cluster_sync_all();  // every span's partial tile is in its CTA's shared memory
    if (warp >= 2) {
        const int rows_here = BM / n_spans;  // n_spans is 2 or 4
        const int col = n0 + 4 * lane;
        uint32_t peer[4];
#pragma unroll
        for (int sp = 0; sp < 4; ++sp) peer[sp] = cluster_peer_address(partial + 4 * lane, sp < n_spans ? sp : 0);
#pragma unroll 2
        for (int i = warp - 2; i < rows_here; i += 4) {
            const int r = span * rows_here + i, row = m0 + r;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int sp = 0; sp < 4; ++sp) {
                if (sp < n_spans) {
                    const float4 p = cluster_load_f32x4(peer[sp] + (uint32_t)r * kSplitPitch * 4);
                    acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
                }
            }
            if (row >= M || col >= N) continue;
            const float v[4] = {acc.x, acc.y, acc.z, acc.w};
            if (EPI == 2) {  // columns are gate, up, gate, up
                TC* dst = C + (size_t)row * ldc + (col >> 1);
                const float h0 = (v[0] / (1.0f + expf(-v[0]))) * v[1], h1 = (v[2] / (1.0f + expf(-v[2]))) * v[3];
                if (col + 4 <= N && ((uintptr_t)dst & 3) == 0 && sizeof(TC) == 2) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(h0, h1);
                    *reinterpret_cast<__nv_bfloat162*>(dst) = h;
                } else {
                    if (col + 1 < N) dst[0] = from_f32<TC>(h0);
                    if (col + 3 < N) dst[1] = from_f32<TC>(h1);
                }
            } else {
                TC* dst = C + (size_t)row * ldc + col;
                const bool whole = col + 4 <= N && ((uintptr_t)dst & (sizeof(TC) * 4 - 1)) == 0;
                if (EPI == 1) {  // C is the float32 residual stream
                    float* d = reinterpret_cast<float*>(dst);
                    if (whole) {
                        float4 x = *reinterpret_cast<float4*>(d);
                        x.x += v[0]; x.y += v[1]; x.z += v[2]; x.w += v[3];
                        *reinterpret_cast<float4*>(d) = x;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j) if (col + j < N) d[j] += v[j];
                    }
                } else if (whole && sizeof(TC) == 4) {
                    *reinterpret_cast<float4*>(dst) = acc;
                } else if (whole) {
                    __nv_bfloat162 p0 = __floats2bfloat162_rn(v[0], v[1]), p1 = __floats2bfloat162_rn(v[2], v[3]);
                    *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1));
                } else {
#pragma unroll
                    for (int j = 0; j < 4; ++j) if (col + j < N) dst[j] = from_f32<TC>(v[j]);
                }
            }
        }
    }
    cluster_sync_all();  // no CTA leaves while a peer may still read its shared memory
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(BN) : "memory");
    }
}

static int sm_count() {
    static int n_sms = 0;
    if (n_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n_sms <= 0)
            n_sms = 148;
    }
    return n_sms;
}

// Width of the tiles for an M x N product.  The widest tile moves the fewest operand bytes per flop and wins whenever
// its tiles fill the SMs; a product of few tiles (a few hundred tokens, a narrow output) leaves SMs idle, and narrower
// tiles, each finished sooner, end it earlier.  A CTA's tiles run one after another, so the estimate is the number of
// rounds times the time of one tile, which follows the bytes a tile's k-step brings in (48, 32, 24 KB) rather than
// its tensor-core cycles; the relative times below are measured (M 192..4096 at widths 2048..16384).  Ties go to
// the wider tile.
static int tile_width_for(int M, int N) {
    const long long tiles_m = (M + BM - 1) / BM;
    const int widths[3] = {256, 128, 64}, tile_time[3] = {128, 85, 66};
    int best = 256;
    long long best_time = 0;
    for (int i = 0; i < 3; ++i) {
        const long long tiles = tiles_m * ((N + widths[i] - 1) / widths[i]);
        const long long time = ((tiles + sm_count() - 1) / sm_count()) * tile_time[i];
        if (i == 0 || time < best_time) { best = widths[i]; best_time = time; }
    }
    return best;
}

// float32 C [rows, cols] with row stride ld (elements) as boxes of 32 x 32, 128-byte swizzle: what the residual
// epilogue's bulk reductions address.  False when C does not lie on the 16-byte grid a tensor map needs.
static bool make_map_c(CUtensorMap* map, const void* base, int rows, int cols, int ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn || ((uintptr_t)base & 15) != 0 || ld % 4 != 0) return false;
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t elem[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int STAGES, int EPI, typename TC>
static int launch_tc(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, cudaStream_t stream,
                     const RopeEpilogue& rope = RopeEpilogue{}) {
    CUtensorMap ma, mw, mc = {};
    if (!make_map(&ma, A, M, K, lda, BM) || !make_map(&mw, W, N, K, ldw, BN)) return kErrUnsupportedSize;
    // the residual sum as bulk reductions where C allows a tensor map (else thread by thread, as the other epilogues)
    const int reduce_c = (EPI == 1 && make_map_c(&mc, C, M, N, ldc)) ? 1 : 0;
    const size_t smem = ((sizeof(GemmSmem<BN, STAGES>) + 1023) & ~(size_t)1023) + (EPI == 1 ? sizeof(ResidualStage) : 0) + 1024;
    static bool configured = false;
    auto kernel = gemm_tcgen05_kernel<BN, STAGES, EPI, TC>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int n_sms = sm_count();
    const long long n_tiles = (long long)((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    dim3 grid((unsigned)(n_tiles < n_sms ? n_tiles : n_sms));
    return launch_pdl(kernel, dim3(grid), dim3(kGemmTcThreads), smem, stream, ma, mw, mc, reduce_c, (TC*)C, ldc, M, N, K, rope);
}

template <int BN, int STAGES>
static int launch_width(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M, int N, int K,
                        int epilogue, cudaStream_t stream) {
    if (epilogue == 2) return launch_tc<BN, STAGES, 2, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    if (epilogue == 1) return launch_tc<BN, STAGES, 1, float>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    if (c_dtype == kF32) return launch_tc<BN, STAGES, 0, float>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    return launch_tc<BN, STAGES, 0, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, stream);
}

// How many CTA pairs can run at once (a pair needs two SMs that can form a cluster; each CTA fills its SM).
template <typename Kernel>
static int resident_pairs(Kernel kernel, size_t smem) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * sm_count());
    cfg.blockDim = dim3(kGemmTcThreads);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}

template <int BN, int STAGES, int EPI, typename TC>
static int launch_pair(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, cudaStream_t stream,
                       const RopeEpilogue& rope = RopeEpilogue{}) {
    CUtensorMap ma, mw, mc = {};
    if (!make_map(&ma, A, M, K, lda, BM) || !make_map(&mw, W, N, K, ldw, BN / 2)) return kErrUnsupportedSize;
    const int reduce_c = (EPI == 1 && make_map_c(&mc, C, M, N, ldc)) ? 1 : 0;
    const size_t smem = ((sizeof(PairSmem<BN, STAGES>) + 1023) & ~(size_t)1023) + (EPI == 1 ? sizeof(ResidualStage) : 0) + 1024;
    static int pairs = -1;
    auto kernel = gemm_tcgen05_pair_kernel<BN, STAGES, EPI, TC>;
    if (pairs < 0) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        pairs = resident_pairs(kernel, smem);
    }
    if (pairs <= 0) return kErrUnsupportedSize;
    const long long n_tiles = (long long)((N + BN - 1) / BN) * ((M + 2 * BM - 1) / (2 * BM));
    const unsigned n_pairs = (unsigned)(n_tiles < pairs ? n_tiles : pairs);
    return launch_pdl_cluster(kernel, dim3(2 * n_pairs), dim3(kGemmTcThreads), smem, stream, dim3(2, 1, 1), true,
                              ma, mw, mc, reduce_c, (TC*)C, ldc, M, N, K, rope);
}

template <int BN, int STAGES>
static int launch_pair_width(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M, int N, int K,
                             int epilogue, cudaStream_t stream) {
    if (epilogue == 2) return launch_pair<BN, STAGES, 2, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    if (epilogue == 1) return launch_pair<BN, STAGES, 1, float>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    if (c_dtype == kF32) return launch_pair<BN, STAGES, 0, float>(A, lda, W, ldw, C, ldc, M, N, K, stream);
    return launch_pair<BN, STAGES, 0, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, stream);
}

// Spans of K per tile for the cluster kernel (1: the plain kernel).  Worth it when the 128 x 128 tiles times the spans
// still fit the SMs, a span keeps 8 k-steps or more, and the estimate (k-steps of a span plus 12 for the cluster's
// barriers and the second pass over the tile, in the units of tile_width_for) beats the plain kernel's.
static int k_spans_for(int M, int N, int K) {
    const long long tiles = (long long)((M + BM - 1) / BM) * ((N + kSplitBN - 1) / kSplitBN);
    const int kb = (K + BK - 1) / BK;
    const int widths[3] = {256, 128, 64}, tile_time[3] = {128, 85, 66};
    long long plain = 0;
    for (int i = 0; i < 3; ++i) {
        const long long t = (long long)((M + BM - 1) / BM) * ((N + widths[i] - 1) / widths[i]);
        const long long time = ((t + sm_count() - 1) / sm_count()) * tile_time[i] * kb;
        if (i == 0 || time < plain) plain = time;
    }
    for (int spans = 4; spans >= 2; spans -= 2) {
        if (tiles * spans > sm_count() || kb / spans < 8) continue;
        if ((long long)((kb + spans - 1) / spans + 12) * 85 < plain) return spans;
    }
    return 1;
}

template <int EPI, typename TC>
static int launch_spans(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int N, int K, int spans,
                        cudaStream_t stream) {
    CUtensorMap ma, mw;
    if (!make_map(&ma, A, M, K, lda, BM) || !make_map(&mw, W, N, K, ldw, kSplitBN)) return kErrUnsupportedSize;
    const size_t smem = sizeof(GemmSmem<kSplitBN, kSplitStages>) + 1024;
    static bool configured = false;
    auto kernel = gemm_tcgen05_spans_kernel<EPI, TC>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = true;
    }
    const int kb = (K + BK - 1) / BK;
    const int tiles = ((N + kSplitBN - 1) / kSplitBN) * ((M + BM - 1) / BM);
    return launch_pdl_cluster(kernel, dim3(tiles, spans), dim3(kGemmTcThreads), smem, stream, dim3(1, spans, 1), true,
                              ma, mw, (TC*)C, ldc, M, N, K, (kb + spans - 1) / spans);
}

}  // namespace b200

// Reads and clears the status word of the tensor-core GEMM (0 = every wait completed).  Synchronises.
extern "C" int b200_gemm_tcgen05_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, b200::g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    cudaMemcpyToSymbol(b200::g_gemm_status, &zero, sizeof(int));
    return v;
}

// A, W bfloat16; C bfloat16 or float32; epilogue 0 store, 1 residual add (C float32), 2 gated SiLU (C bfloat16).
// Spans of K that the product's shape asks for (1: none).
extern "C" int b200_gemm_tcgen05_k_spans(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    return b200::k_spans_for(M, N, K);
}

// tile_width: 256, 128 or 64 output columns per tile; 0 lets the product's shape decide.
// k_spans: 2 or 4 cuts K among the CTAs of a cluster (128-column tiles; tile_width is then ignored), 1 never does,
// 0 lets the shape decide.
// cta_pair: 1 computes 256-row tiles by pairs of CTAs (tile_width 256 or 128), -1 never does, 0 lets the shape decide.
extern "C" int b200_gemm_tcgen05(const void* A, int lda, const void* W, int ldw, void* C, int c_dtype, int ldc, int M,
                                 int N, int K, int epilogue, int tile_width, int k_spans, int cta_pair, cudaStream_t stream) {
    using namespace b200;
    if (M <= 0 || N <= 0) return 0;
    if (K < 8 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || (((uintptr_t)A | (uintptr_t)W) & 15)) return kErrUnsupportedSize;
    if (epilogue < 0 || epilogue > 2 || (epilogue == 1 && c_dtype != kF32) || (epilogue == 2 && ((N & 1) || c_dtype != kBF16)))
        return kErrBadArgument;
    if (c_dtype != kF32 && c_dtype != kBF16) return kErrBadArgument;
    if (k_spans != 0 && k_spans != 1 && k_spans != 2 && k_spans != 4) return kErrBadArgument;
    if (cta_pair > 0) {
        if (tile_width == 128) return launch_pair_width<128, 8>(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream);
        if (tile_width == 256 || tile_width == 0) return launch_pair_width<256, 6>(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream);
        return kErrBadArgument;
    }
    // left the choice: pairs of CTAs as soon as their 256 x 256 tiles occupy two thirds of the SMs (measured: from there on
    // the pair kernel is the faster one at every shape tried, by 5 to 25 %)
    if (cta_pair == 0 && tile_width == 0 && k_spans == 0) {
        const long long pair_tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
        if (pair_tiles * 3 >= (long long)(sm_count() / 2) * 2) {
            const int st = launch_pair_width<256, 6>(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream);
            if (st != kErrUnsupportedSize) return st;   // (no two SMs that can form a pair: the single-CTA kernels below)
        }
    }
    const int spans = k_spans > 0 ? k_spans : (tile_width > 0 ? 1 : k_spans_for(M, N, K));
    if (spans > 1) {
        if ((K + BK - 1) / BK < spans) return kErrBadArgument;
        if (epilogue == 2) return launch_spans<2, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, spans, stream);
        if (epilogue == 1) return launch_spans<1, float>(A, lda, W, ldw, C, ldc, M, N, K, spans, stream);
        if (c_dtype == kF32) return launch_spans<0, float>(A, lda, W, ldw, C, ldc, M, N, K, spans, stream);
        return launch_spans<0, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, spans, stream);
    }
    // a stage holds 16 KB of A and BN / 8 KB of W: the narrower the tile, the deeper the ring
    const int width = tile_width > 0 ? tile_width : tile_width_for(M, N);
    if (width == 256) return launch_width<256, 4>(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream);
    if (width == 128) return launch_width<128, 6>(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream);
    if (width == 64) return launch_width<64, 8>(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, epilogue, stream);
    return kErrBadArgument;
}

// The query, key and value projection of a prompt pass with rotation and cache write in its epilogue (see RopeEpilogue).
// A [M, K] activations, W [(n_heads + 2 n_kv_heads) head_dim, K], C [M, ldc] receives the rotated queries (its key and
// value columns are left untouched).  Taken when the heads are 64 or 128 wide and the shape is one for 256-column tiles
// (pairs of CTAs, or single CTAs whose wide tiles fill the SMs); kErrUnsupportedSize otherwise, and the caller runs the
// product and the rotation kernel one after the other.
extern "C" int b200_gemm_tcgen05_qkv_rope(const void* A, int lda, const void* W, int ldw, void* C, int ldc, int M, int K,
                                          const int* positions, const int* seq_ids, const int* page_table, int table_stride,
                                          const float* angles, void* k_pool, void* v_pool, int n_heads, int n_kv_heads,
                                          int head_dim, int pairing, int write_cache, cudaStream_t stream) {
    using namespace b200;
    if (M <= 0) return 0;
    if (K < 8 || K % 8 != 0 || lda % 8 != 0 || ldw % 8 != 0 || ldc % 8 != 0 ||
        (((uintptr_t)A | (uintptr_t)W | (uintptr_t)C | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) || ((uintptr_t)angles & 7))
        return kErrUnsupportedSize;
    if ((head_dim != 64 && head_dim != 128) || n_heads <= 0 || n_kv_heads <= 0 || (pairing != 0 && pairing != 1))
        return kErrUnsupportedSize;
    if (write_cache && (k_pool == nullptr || v_pool == nullptr)) return kErrBadArgument;
    const int N = (n_heads + 2 * n_kv_heads) * head_dim;
    RopeEpilogue rope;
    rope.positions = positions; rope.seq_ids = seq_ids; rope.page_table = page_table; rope.table_stride = table_stride;
    rope.angles = reinterpret_cast<const float2*>(angles);
    rope.n_tokens = M;
    rope.k_pool = (__nv_bfloat16*)k_pool; rope.v_pool = (__nv_bfloat16*)v_pool;
    rope.n_heads = n_heads; rope.n_kv_heads = n_kv_heads; rope.head_dim = head_dim; rope.pairing = pairing;
    rope.write_cache = write_cache ? 1 : 0;
    const long long pair_tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
    if (pair_tiles * 3 >= (long long)(sm_count() / 2) * 2) {
        const int st = launch_pair<256, 6, 3, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, stream, rope);
        if (st != kErrUnsupportedSize) return st;
    }
    if (k_spans_for(M, N, K) == 1 && tile_width_for(M, N) == 256)
        return launch_tc<256, 4, 3, __nv_bfloat16>(A, lda, W, ldw, C, ldc, M, N, K, stream, rope);
    return kErrUnsupportedSize;
}
