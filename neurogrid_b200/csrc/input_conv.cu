// Input convolution of a sublayer: out[t] = u[t] + sum_{k<L} w[d,k] * u[t-(L-1)+k] per channel d,
// over a ragged batch of prompt portions and single tokens (tap L-1 multiplies the current token).
// u before the first row of a portion comes from the request's state slot (its last L-1 inputs,
// float32), u before position 0 is zero whatever the slot holds; after the portion the slot holds
// the last L-1 inputs again.
//
// Grid: (channel blocks, token tiles, entries).  A thread owns one channel of one tile and walks
// its tokens in order with the last L-1 inputs in registers.  Only tile 0 of an entry reads the
// slot and only tile 0 writes it, after all its reads: no other block touches a slot in use.
// The sum is float32, taps ascending, so a token's result does not depend on the cut.
#include "ng_common.cuh"

#define IC_MAX_L 8
#define IC_TILE 32
#define IC_THREADS 128

template <typename T, int L>
__global__ void __launch_bounds__(IC_THREADS)
input_conv_kernel(const T* __restrict__ u, const float* __restrict__ w, float* __restrict__ state,
                  T* __restrict__ out, const int* __restrict__ cu_q, const int* __restrict__ ctx_before,
                  const int* __restrict__ slots, int H) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.z;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    const int t0 = blockIdx.y * IC_TILE;
    const int d = blockIdx.x * IC_THREADS + threadIdx.x;
    if (t0 >= qlen || d >= H) return;
    const int ctx = ctx_before[e];
    float* st = state + (size_t)slots[e] * (L - 1) * H + d;        // st[j*H]: u at position ctx-(L-1)+j
    const T* ur = u + (size_t)q0 * H + d;
    T* orow = out + (size_t)q0 * H + d;
    float wk[L], hist[L - 1], old[L - 1];
#pragma unroll
    for (int k = 0; k < L; ++k) wk[k] = w[(size_t)d * L + k];
    const bool first = t0 == 0;
#pragma unroll
    for (int j = 0; j < L - 1; ++j)
        old[j] = (first && ctx - (L - 1) + j >= 0) ? st[(size_t)j * H] : 0.f;
    // hist[j] = u at chunk index t0-(L-1)+j
#pragma unroll
    for (int j = 0; j < L - 1; ++j) {
        const int ti = t0 - (L - 1) + j;
        hist[j] = ti >= 0 ? ng_ld(ur + (size_t)ti * H) : old[j];
    }
    const int t1 = min(t0 + IC_TILE, qlen);
    for (int t = t0; t < t1; ++t) {
        const float x = ng_ld(ur + (size_t)t * H);
        float acc = 0.f;
#pragma unroll
        for (int k = 0; k < L - 1; ++k)
            acc = fmaf(wk[k], hist[k], acc);
        acc = fmaf(wk[L - 1], x, acc);
        ng_st(orow + (size_t)t * H, x + acc);
#pragma unroll
        for (int k = 0; k < L - 2; ++k)
            hist[k] = hist[k + 1];
        hist[L - 2] = x;
    }
    if (first) {
        // the slot after the portion: u at positions ctx+qlen-(L-1)+j, from the portion or from what the slot held
#pragma unroll
        for (int j = 0; j < L - 1; ++j) {
            const int ti = qlen - (L - 1) + j;
            float v = 0.f;
            if (ti >= 0) v = ng_ld(ur + (size_t)ti * H);
            else {
#pragma unroll
                for (int k = 0; k < L - 1; ++k)
                    if (k == ti + (L - 1)) v = old[k];
            }
            st[(size_t)j * H] = v;
        }
    }
}

// u, out: [n_rows, H] of the activation type; w: [H, L] float32; state: [slots, L-1, H] float32.
NG_EXPORT int ng_input_conv(const void* u, const float* w, float* state, void* out, const int* cu_q,
                            const int* ctx_before, const int* slots, int n_entries, int max_q, int H, int L,
                            int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0 || max_q <= 0) return NG_OK;
    if (H <= 0 || L < 2 || L > IC_MAX_L) return NG_BAD_SIZE;
    dim3 grid((H + IC_THREADS - 1) / IC_THREADS, (max_q + IC_TILE - 1) / IC_TILE, n_entries);
    if (grid.y > 65535 || grid.z > 65535) return NG_BAD_SIZE;
#define IC_CASE(LL)                                                                                                   \
    case LL:                                                                                                          \
        if (act_bf16)                                                                                                 \
            NG_LAUNCH((input_conv_kernel<__nv_bfloat16, LL>), grid, IC_THREADS, 0, stream, (const __nv_bfloat16*)u, w, \
                      state, (__nv_bfloat16*)out, cu_q, ctx_before, slots, H);                                        \
        else                                                                                                          \
            NG_LAUNCH((input_conv_kernel<float, LL>), grid, IC_THREADS, 0, stream, (const float*)u, w, state,         \
                      (float*)out, cu_q, ctx_before, slots, H);                                                       \
        break;
    switch (L) {
        IC_CASE(2) IC_CASE(3) IC_CASE(4) IC_CASE(5) IC_CASE(6) IC_CASE(7) IC_CASE(8)
    }
    return ng_launch_status();
}
