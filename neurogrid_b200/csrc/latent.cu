// Latent attention, the row kernels around its attention core.
//
// latent_prep: a row of the stacked down projection is [c_q raw (rq) | c raw (rkv) | gate logits (nH)].
//   c_q = c_q raw / sqrt(mean(c_q raw^2) + eps) * wq        -> cq_out [n_rows, rq]      (activation type)
//   c   = c raw   / sqrt(mean(c raw^2) + eps) * wkv         -> the row's place in the layer's pages
//                                                             [pages, 1, page_size, rp], columns rkv..rp zero
//   gate = sigmoid(gate logits)                             -> gate_out [n_rows, nH]    (float32)
// Both norms and the gate are float32; only what a matrix product or the cache reads is rounded.
//
// head_gate: y[row, h, :] *= gate[row, h] for rows of [n_rows, nH * width].
#include "ng_common.cuh"

template <typename T>
__global__ void __launch_bounds__(128)
latent_prep_kernel(const T* __restrict__ x, const float* __restrict__ wq, const float* __restrict__ wkv,
                   T* __restrict__ cq_out, T* __restrict__ pages, float* __restrict__ gate_out,
                   const int* __restrict__ table, int table_stride, const int* __restrict__ positions,
                   const int* __restrict__ row_entry, int rq, int rkv, int rp, int nH, int page_size, int num_pages,
                   float eps, int* __restrict__ status) {
    __shared__ float red[32];
    ng_pdl_trigger();
    ng_pdl_wait();
    const int row = blockIdx.x;
    const int entry = row_entry[row];
    if (entry < 0) return;
    const T* xr = x + (size_t)row * (rq + rkv + nH);
    float ss = 0.f;
    for (int i = threadIdx.x; i < rq; i += blockDim.x) {
        const float v = ng_ld(xr + i);
        ss += v * v;
    }
    ss = ng_block_sum(ss, red);
    const float r1 = rsqrtf(ss / (float)rq + eps);
    for (int i = threadIdx.x; i < rq; i += blockDim.x) ng_st(cq_out + (size_t)row * rq + i, ng_ld(xr + i) * r1 * wq[i]);
    ss = 0.f;
    for (int i = threadIdx.x; i < rkv; i += blockDim.x) {
        const float v = ng_ld(xr + rq + i);
        ss += v * v;
    }
    ss = ng_block_sum(ss, red);
    const float r2 = rsqrtf(ss / (float)rkv + eps);
    const int pos = positions[row];
    const int page = pos >= 0 ? table[(size_t)entry * table_stride + pos / page_size] : -1;
    if (page < 0 || page >= num_pages) {
        if (threadIdx.x == 0) atomicOr(status, NG_STATUS_BAD_PAGE);
    } else {
        T* dst = pages + ((size_t)page * page_size + (pos % page_size)) * rp;
        for (int i = threadIdx.x; i < rp; i += blockDim.x)
            ng_st(dst + i, i < rkv ? ng_ld(xr + rq + i) * r2 * wkv[i] : 0.f);
    }
    for (int h = threadIdx.x; h < nH; h += blockDim.x)
        gate_out[(size_t)row * nH + h] = 1.f / (1.f + expf(-ng_ld(xr + rq + rkv + h)));
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ y, const float* __restrict__ gate, size_t total, int nH, int width) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t rh = i / width;              // row * nH + head
    ng_st(y + i, ng_ld(y + i) * gate[rh]);
}

NG_EXPORT int ng_latent_prep(const void* x, const float* wq, const float* wkv, void* cq_out, void* pages,
                             float* gate_out, const int* table, int table_stride, const int* positions,
                             const int* row_entry, int n_rows, int rq, int rkv, int rp, int nH, int page_size,
                             int num_pages, float eps, int* status, int act_bf16, cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (rq <= 0 || rkv <= 0 || rp < rkv || nH <= 0 || page_size <= 0) return NG_BAD_SIZE;
    if (act_bf16)
        NG_LAUNCH((latent_prep_kernel<__nv_bfloat16>), n_rows, 128, 0, stream, (const __nv_bfloat16*)x, wq, wkv,
                  (__nv_bfloat16*)cq_out, (__nv_bfloat16*)pages, gate_out, table, table_stride, positions, row_entry,
                  rq, rkv, rp, nH, page_size, num_pages, eps, status);
    else
        NG_LAUNCH((latent_prep_kernel<float>), n_rows, 128, 0, stream, (const float*)x, wq, wkv, (float*)cq_out,
                  (float*)pages, gate_out, table, table_stride, positions, row_entry, rq, rkv, rp, nH, page_size,
                  num_pages, eps, status);
    return ng_launch_status();
}

NG_EXPORT int ng_head_gate(void* y, const float* gate, int n_rows, int nH, int width, int act_bf16,
                           cudaStream_t stream) {
    if (n_rows <= 0) return NG_OK;
    if (nH <= 0 || width <= 0) return NG_BAD_SIZE;
    const size_t total = (size_t)n_rows * nH * width;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (act_bf16)
        NG_LAUNCH((head_gate_kernel<__nv_bfloat16>), blocks, 256, 0, stream, (__nv_bfloat16*)y, gate, total, nH, width);
    else
        NG_LAUNCH((head_gate_kernel<float>), blocks, 256, 0, stream, (float*)y, gate, total, nH, width);
    return ng_launch_status();
}
