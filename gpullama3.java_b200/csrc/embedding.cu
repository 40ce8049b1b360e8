// Token embedding: x[t, :] = table[tokens[t], :], written to the 32-bit residual stream.
// Restates the row copy of inference/InferenceCore.java:69 (reference project path) for a packed
// batch of tokens on the device.
#include "common.cuh"

namespace b200 {

template <typename TW>
__global__ void embed_gather_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                    float* __restrict__ out, int dim, int vocab) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int tok = tokens[t];
    float* o = out + (size_t)t * dim;
    if (tok < 0 || tok >= vocab) {  // refused on the host already; never read out of the table
        for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = 0.f;
        return;
    }
    const TW* row = table + (size_t)tok * dim;
    for (int i = threadIdx.x; i < dim; i += blockDim.x) o[i] = to_f32<TW>(row[i]);
}

}  // namespace b200

extern "C" int b200_embed_gather(const void* table, int table_dtype, const int* tokens, float* out,
                                 int n_tokens, int dim, int vocab, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    B200_DISPATCH_DTYPE(table_dtype, TW,
        return b200::launch_pdl(b200::embed_gather_kernel<TW>, dim3(n_tokens), dim3(256), 0, stream, (const TW*)table,
                                tokens, out, dim, vocab));
    return b200::launch_status();
}
