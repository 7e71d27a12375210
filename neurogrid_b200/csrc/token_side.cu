// Per-layer token input: x += rmsnorm(W_proj (gelu_tanh(W_gate x) * e[token])) * w.
//
//   x: the float32 residual stream [n_rows, H], complete (every pending sum added);
//   e: [vocab, dim] float32, the layer's columns of the token table;
//   W_gate [dim, H], W_proj^T [dim, H] (transposed when bound, so that both are read along H), w [H] float32.
// Everything is float32.  A block takes R rows (8 for long steps, so that the two matrices are read once per
// eight rows; 1 for short ones): the rows are staged in shared memory, a warp per gate value forms the
// R dot products, then a thread per column forms y for the R rows, which replaces the staged rows; the
// mean squares are reduced per row and the sum goes into the stream.  A row's arithmetic does not depend
// on R or on the other rows: every dot product is walked in the same order.
#include "ng_common.cuh"

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

template <int R, int TS_THREADS>
__global__ void __launch_bounds__(TS_THREADS)
token_side_kernel(float* __restrict__ h, const int* __restrict__ tokens, const float* __restrict__ table,
                  const float* __restrict__ w_gate, const float* __restrict__ w_proj_t, const float* __restrict__ w_norm,
                  int n_rows, int H, int dim, int vocab, float eps, const int* __restrict__ row_entry,
                  int* __restrict__ status) {
    extern __shared__ float sm[];
    float* buf = sm;                 // [R][H]: the rows, then y
    float* g = sm + (size_t)R * H;   // [R][dim]
    __shared__ float red[R][TS_THREADS / 32];
    __shared__ float scale[R];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int r0 = blockIdx.x * R;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    constexpr int NW = TS_THREADS / 32;
    bool live[R];
    int tok[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        live[r] = r0 + r < n_rows && row_entry[r0 + r] >= 0;
        tok[r] = live[r] ? tokens[r0 + r] : 0;
        if (tok[r] < 0 || tok[r] >= vocab) {
            if (tid == 0) atomicOr(status, NG_STATUS_BAD_TOKEN);
            tok[r] = 0;
        }
    }
#pragma unroll
    for (int r = 0; r < R; ++r)
        for (int j = tid; j < H; j += TS_THREADS) buf[(size_t)r * H + j] = live[r] ? h[(size_t)(r0 + r) * H + j] : 0.f;
    __syncthreads();
    const bool vec = (H % 4) == 0;                       // rows of the matrices start on 16-byte boundaries
    for (int i = warp; i < dim; i += NW) {
        const float* w = w_gate + (size_t)i * H;
        float acc[R];
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] = 0.f;
        if (vec) {
#pragma unroll 4
            for (int j = lane * 4; j < H; j += 128) {
                const float4 wv = *reinterpret_cast<const float4*>(w + j);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float4 xv = *reinterpret_cast<const float4*>(buf + (size_t)r * H + j);
                    acc[r] = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, acc[r]))));
                }
            }
        } else {
            for (int j = lane; j < H; j += 32) {
                const float wv = w[j];
#pragma unroll
                for (int r = 0; r < R; ++r) acc[r] = fmaf(buf[(size_t)r * H + j], wv, acc[r]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const float a = ng_warp_sum(acc[r]);
            if (lane == 0) g[r * dim + i] = gelu_tanh(a) * table[(size_t)tok[r] * dim + i];
        }
    }
    __syncthreads();
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; ++r) ss[r] = 0.f;
    if (vec) {
        for (int j = tid * 4; j < H; j += 4 * TS_THREADS) {          // four columns a thread
            float4 acc[R];
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
            for (int i = 0; i < dim; ++i) {
                const float4 wv = *reinterpret_cast<const float4*>(w_proj_t + (size_t)i * H + j);
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    const float gv = g[r * dim + i];
                    acc[r].x = fmaf(wv.x, gv, acc[r].x);
                    acc[r].y = fmaf(wv.y, gv, acc[r].y);
                    acc[r].z = fmaf(wv.z, gv, acc[r].z);
                    acc[r].w = fmaf(wv.w, gv, acc[r].w);
                }
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                *reinterpret_cast<float4*>(buf + (size_t)r * H + j) = acc[r];
                ss[r] += acc[r].x * acc[r].x + acc[r].y * acc[r].y + acc[r].z * acc[r].z + acc[r].w * acc[r].w;
            }
        }
    } else {
        for (int j = tid; j < H; j += TS_THREADS) {
            float acc[R];
#pragma unroll
            for (int r = 0; r < R; ++r) acc[r] = 0.f;
            for (int i = 0; i < dim; ++i) {
                const float wv = w_proj_t[(size_t)i * H + j];
#pragma unroll
                for (int r = 0; r < R; ++r) acc[r] = fmaf(wv, g[r * dim + i], acc[r]);
            }
#pragma unroll
            for (int r = 0; r < R; ++r) {
                buf[(size_t)r * H + j] = acc[r];
                ss[r] += acc[r] * acc[r];
            }
        }
    }
    __syncthreads();                                     // the sum below reads columns other threads wrote
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const float s = ng_warp_sum(ss[r]);
        if (lane == 0) red[r][warp] = s;
    }
    __syncthreads();
    if (tid < R) {
        float s = 0.f;
        for (int k = 0; k < NW; ++k) s += red[tid][k];
        scale[tid] = rsqrtf(s / (float)H + eps);
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; ++r) {
        if (!live[r]) continue;
        float* hr = h + (size_t)(r0 + r) * H;
        for (int j = tid; j < H; j += TS_THREADS) hr[j] += buf[(size_t)r * H + j] * scale[r] * w_norm[j];
    }
}

template <int R, int TS_THREADS>
static int token_side_launch(float* h, const int* tokens, const float* table, const float* w_gate, const float* w_proj_t,
                             const float* w_norm, const int* row_entry, int n_rows, int H, int dim, int vocab, float eps,
                             int* status, cudaStream_t stream) {
    const size_t smem = (size_t)R * ((size_t)H + dim) * sizeof(float);
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(token_side_kernel<R, TS_THREADS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
            return NG_LAUNCH_FAILED;
        configured = true;
    }
    NG_LAUNCH((token_side_kernel<R, TS_THREADS>), (n_rows + R - 1) / R, TS_THREADS, smem, stream, h, tokens, table, w_gate, w_proj_t,
              w_norm, n_rows, H, dim, vocab, eps, row_entry, status);
    return ng_launch_status();
}

// ---------------------------------------------------------------------------------------------- steps of few rows
// A block per row would leave most of the GPU idle and stream both matrices through one SM, so the same sums
// are dealt to many blocks: `gate` forms eight gate values a block (a warp each, the same walk as above),
// `proj` forms y for 128 columns a block and the partial sum of their squares, `apply` adds up the partial
// sums in ascending order and adds the normed y into the stream.  `scratch`: g [n_rows, dim], y [n_rows, H],
// partial sums [n_rows, ceil(H / 128)], float32.
__global__ void __launch_bounds__(256)
token_side_gate_kernel(const float* __restrict__ h, const int* __restrict__ tokens, const float* __restrict__ table,
                       const float* __restrict__ w_gate, float* __restrict__ g, int H, int dim, int vocab,
                       const int* __restrict__ row_entry, int* __restrict__ status) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.y, lane = threadIdx.x & 31;
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= dim || row_entry[row] < 0) return;
    int tok = tokens[row];
    if (tok < 0 || tok >= vocab) {
        if (lane == 0) atomicOr(status, NG_STATUS_BAD_TOKEN);
        tok = 0;
    }
    const float* x = h + (size_t)row * H;
    const float* w = w_gate + (size_t)i * H;
    float acc = 0.f;
    if (H % 4 == 0) {
#pragma unroll 4
        for (int j = lane * 4; j < H; j += 128) {
            const float4 wv = *reinterpret_cast<const float4*>(w + j), xv = *reinterpret_cast<const float4*>(x + j);
            acc = fmaf(xv.x, wv.x, fmaf(xv.y, wv.y, fmaf(xv.z, wv.z, fmaf(xv.w, wv.w, acc))));
        }
    } else {
        for (int j = lane; j < H; j += 32) acc = fmaf(x[j], w[j], acc);
    }
    acc = ng_warp_sum(acc);
    if (lane == 0) g[(size_t)row * dim + i] = gelu_tanh(acc) * table[(size_t)tok * dim + i];
}

__global__ void __launch_bounds__(128)
token_side_proj_kernel(const float* __restrict__ g, const float* __restrict__ w_proj_t, float* __restrict__ y,
                       float* __restrict__ ss_part, int H, int dim, int n_slices, const int* __restrict__ row_entry) {
    __shared__ float red[32];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.y;
    if (row_entry[row] < 0) return;
    const int j = blockIdx.x * 128 + threadIdx.x;
    const float* gr = g + (size_t)row * dim;
    float acc = 0.f;
    if (j < H) {
#pragma unroll 8
        for (int i = 0; i < dim; ++i) acc = fmaf(w_proj_t[(size_t)i * H + j], gr[i], acc);
        y[(size_t)row * H + j] = acc;
    }
    const float ss = ng_block_sum(acc * acc, red);
    if (threadIdx.x == 0) ss_part[(size_t)row * n_slices + blockIdx.x] = ss;
}

__global__ void __launch_bounds__(256)
token_side_apply_kernel(float* __restrict__ h, const float* __restrict__ y, const float* __restrict__ ss_part,
                        const float* __restrict__ w_norm, int H, int n_slices, float eps, const int* __restrict__ row_entry) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    if (row_entry[row] < 0) return;
    float ss = 0.f;
    for (int k = 0; k < n_slices; ++k) ss += ss_part[(size_t)row * n_slices + k];
    const float r = rsqrtf(ss / (float)H + eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) h[(size_t)row * H + j] += y[(size_t)row * H + j] * r * w_norm[j];
}

// float32 values of scratch the few-rows path needs (0: the step is long enough for the fused kernel)
NG_EXPORT long long ng_token_side_scratch(int n_rows, int H, int dim) {
    return n_rows < 128 ? (long long)n_rows * ((long long)dim + H + (H + 127) / 128) : 0;
}

NG_EXPORT int ng_token_side(float* h, const int* tokens, const float* table, const float* w_gate, const float* w_proj_t,
                            const float* w_norm, const int* row_entry, int n_rows, int H, int dim, int vocab, float eps,
                            int* status, float* scratch, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (H <= 0 || dim <= 0 || vocab <= 0) return NG_BAD_SIZE;
    if (scratch && n_rows < 128) {
        const int n_slices = (H + 127) / 128;
        float* g = scratch;
        float* y = g + (size_t)n_rows * dim;
        float* part = y + (size_t)n_rows * H;
        NG_LAUNCH((token_side_gate_kernel), dim3((dim + 7) / 8, n_rows), 256, 0, stream, (const float*)h, tokens, table, w_gate,
                  g, H, dim, vocab, row_entry, status);
        NG_LAUNCH((token_side_proj_kernel), dim3(n_slices, n_rows), 128, 0, stream, (const float*)g, w_proj_t, y, part, H, dim,
                  n_slices, row_entry);
        NG_LAUNCH((token_side_apply_kernel), n_rows, 256, 0, stream, h, (const float*)y, (const float*)part, w_norm, H,
                  n_slices, eps, row_entry);
        return ng_launch_status();
    }
    const size_t per_row = ((size_t)H + dim) * sizeof(float), cap = 160 * 1024;
    if (per_row > cap) return NG_BAD_SIZE;
#define TS_GO(RR, TT) return token_side_launch<RR, TT>(h, tokens, table, w_gate, w_proj_t, w_norm, row_entry, n_rows, H, dim, vocab, eps, status, stream)
    if (n_rows >= 512 && 8 * per_row <= cap) TS_GO(8, 512);
    if (n_rows >= 128 && 4 * per_row <= cap) TS_GO(4, 512);
    TS_GO(1, 1024);            // few rows: a block's speed is its loads in flight
}
