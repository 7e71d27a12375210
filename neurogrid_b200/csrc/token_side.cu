// Per-layer token input: x += rmsnorm(W_proj (gelu_tanh(W_gate x) * e[token])) * w, one block per row.
//
//   x: the float32 residual stream [n_rows, H], complete (every pending sum added);
//   e: [vocab, dim] float32, the layer's columns of the token table;  W_gate [dim, H], W_proj [H, dim], w [H] float32.
// Everything is float32: the row's dim gate values, then y = W_proj g (kept in shared memory), its mean
// square, and the sum into the stream.  A row's result does not depend on the batch.
#include "ng_common.cuh"

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

__global__ void __launch_bounds__(256)
token_side_kernel(float* __restrict__ h, const int* __restrict__ tokens, const float* __restrict__ table,
                  const float* __restrict__ w_gate, const float* __restrict__ w_proj, const float* __restrict__ w_norm,
                  int H, int dim, int vocab, float eps, const int* __restrict__ row_entry, int* __restrict__ status) {
    extern __shared__ float sm[];
    float* g = sm;              // [dim]
    float* y = sm + dim;        // [H]
    __shared__ float red[32];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    if (row_entry[row] < 0) return;
    int tok = tokens[row];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, NG_STATUS_BAD_TOKEN);
        tok = 0;
    }
    float* hr = h + (size_t)row * H;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    for (int i = warp; i < dim; i += nwarp) {
        const float* w = w_gate + (size_t)i * H;
        float acc = 0.f;
        for (int j = lane; j < H; j += 32) acc = fmaf(hr[j], w[j], acc);
        acc = ng_warp_sum(acc);
        if (lane == 0) g[i] = gelu_tanh(acc) * table[(size_t)tok * dim + i];
    }
    __syncthreads();
    float ss = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        const float* w = w_proj + (size_t)j * dim;
        float acc = 0.f;
        for (int i = 0; i < dim; ++i) acc = fmaf(w[i], g[i], acc);
        y[j] = acc;
        ss += acc * acc;
    }
    ss = ng_block_sum(ss, red);
    const float r = rsqrtf(ss / (float)H + eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) hr[j] += y[j] * r * w_norm[j];
}

NG_EXPORT int ng_token_side(float* h, const int* tokens, const float* table, const float* w_gate, const float* w_proj,
                            const float* w_norm, const int* row_entry, int n_rows, int H, int dim, int vocab, float eps,
                            int* status, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    const size_t smem = ((size_t)dim + H) * sizeof(float);
    if (H <= 0 || dim <= 0 || vocab <= 0 || smem > 48 * 1024) return NG_BAD_SIZE;
    NG_LAUNCH((token_side_kernel), n_rows, 256, smem, stream, h, tokens, table, w_gate, w_proj, w_norm, H, dim, vocab, eps,
              row_entry, status);
    return ng_launch_status();
}
