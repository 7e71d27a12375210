// Retention: linear attention with a fixed decay per head, as a recurrence over a ragged batch.
//
//   per head:  S_t = decay * S_(t-1) + k_t v_t^T   (S: [dk, dv], float32, one per request and head)
//              o_t = S_t^T q_t ;  out_t = o_t / sqrt(mean(o_t^2) + eps) * silu(g_t)
//   q and k are rotated first (the first rot_dims coordinates of a head, coordinate i with
//   i + rot_dims/2, angle = position * inv_freq[i]); k is scaled by dk^(-1/2) after the rotation.
//
// Input rows are [q (nH*dk) | k (nH*dk) | v (nH*dv) | g (nH*dv)] of the activation type; everything
// that enters the recurrence (angles, rotation, scaling, decay, state, the head's norm, the gate) is
// float32.  One block per (entry, head) walks the entry's tokens in order, so a token's result does
// not depend on how its request was cut or on what else is in the step.  The state lies in registers:
// thread (g, j) keeps rows g*R .. g*R+R-1 of column j of S; the partial dot products of the groups
// are added in ascending g.  The slot is read at the start (zero when the request has no tokens yet)
// and written at the end.
#include "ng_common.cuh"

template <typename T, int R, int MAXT>
__global__ void __launch_bounds__(MAXT)
retention_kernel(const T* __restrict__ x, const float* __restrict__ inv_freq, int rot_dims,
                 const float* __restrict__ decay, float* __restrict__ state, T* __restrict__ out,
                 const int* __restrict__ cu_q, const int* __restrict__ ctx_before, const int* __restrict__ slots,
                 int nH, int dk, int dv, int G, float eps) {
    extern __shared__ float sm[];
    float* qs = sm;                 // [dk]
    float* ks = qs + dk;            // [dk]
    float* part = ks + dk;          // [G * dv]
    float* red = part + G * dv;     // [32]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.x, head = blockIdx.y;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    if (qlen <= 0) return;
    const int ctx = ctx_before[e];
    const int tid = threadIdx.x;
    const int j = tid % dv, g = tid / dv;          // blockDim.x is a multiple of 32 >= G * dv
    const bool live = g < G;
    const int i0 = g * R;
    const size_t ld = 2 * (size_t)nH * (dk + dv);
    const size_t off_q = (size_t)head * dk, off_k = (size_t)nH * dk + off_q;
    const size_t off_v = 2 * (size_t)nH * dk + (size_t)head * dv, off_g = off_v + (size_t)nH * dv;
    float* S = state + ((size_t)slots[e] * nH + head) * dk * dv;
    const float lam = decay[head];
    const float kscale = rsqrtf((float)dk);
    const int half = rot_dims / 2;
    float s[R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
        const int i = i0 + r;
        s[r] = (live && ctx > 0 && i < dk) ? S[(size_t)i * dv + j] : 0.f;
    }
    for (int t = 0; t < qlen; ++t) {
        const T* row = x + (size_t)(q0 + t) * ld;
        const float pos = (float)(ctx + t);
        for (int i = tid; i < dk; i += blockDim.x) {
            float qv = ng_ld(row + off_q + i), kv = ng_ld(row + off_k + i);
            if (i < rot_dims) {
                const int p = i < half ? i : i - half;
                float sn, cs;
                sincosf(pos * inv_freq[p], &sn, &cs);
                const int mate = i < half ? i + half : i - half;
                const float qm = ng_ld(row + off_q + mate), km = ng_ld(row + off_k + mate);
                // the pair (a, b) = (x[p], x[p + half]) becomes (a cos - b sin, b cos + a sin)
                qv = i < half ? qv * cs - qm * sn : qv * cs + qm * sn;
                kv = i < half ? kv * cs - km * sn : kv * cs + km * sn;
            }
            qs[i] = qv;
            ks[i] = kv * kscale;
        }
        __syncthreads();
        if (live) {
            const float vj = ng_ld(row + off_v + j);
            float acc = 0.f;
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const int i = i0 + r;
                if (i < dk) {
                    s[r] = fmaf(lam, s[r], ks[i] * vj);
                    acc = fmaf(s[r], qs[i], acc);
                }
            }
            part[g * dv + j] = acc;
        }
        __syncthreads();
        float o = 0.f;
        if (tid < dv)
            for (int gg = 0; gg < G; ++gg) o += part[gg * dv + tid];
        const float ss = ng_block_sum(tid < dv ? o * o : 0.f, red);
        if (tid < dv) {
            const float gate = ng_ld(row + off_g + tid);
            const float y = o * rsqrtf(ss / (float)dv + eps) * (gate / (1.f + expf(-gate)));
            ng_st(out + (size_t)(q0 + t) * nH * dv + (size_t)head * dv + tid, y);
        }
        __syncthreads();
    }
    if (live) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int i = i0 + r;
            if (i < dk) S[(size_t)i * dv + j] = s[r];
        }
    }
}

// x: [n_rows, 2*nH*(dk+dv)], out: [n_rows, nH*dv], activation type; inv_freq: float32 [rot_dims/2];
// decay: float32 [nH]; state: float32 [slots, nH, dk, dv].
NG_EXPORT int ng_retention(const void* x, const float* inv_freq, int rot_dims, const float* decay, float* state,
                           void* out, const int* cu_q, const int* ctx_before, const int* slots, int n_entries,
                           int nH, int dk, int dv, float eps, int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0) return NG_OK;
    if (nH <= 0 || dk <= 0 || dv <= 0 || rot_dims < 0 || rot_dims > dk || rot_dims % 2 || (rot_dims && !inv_freq))
        return NG_BAD_SIZE;
    // rows of S per thread and the block size that goes with them: 16 rows up to 512 threads, else 64 rows
    // up to 256 threads, else 64 rows in a block of up to 1024 threads (large heads; that build keeps part of
    // its state in local memory)
    int R = 16, maxt = 512;
    int G = (dk + R - 1) / R;
    if ((size_t)G * dv > 512) {
        R = 64;
        G = (dk + R - 1) / R;
        maxt = (size_t)G * dv > 256 ? 1024 : 256;
    }
    if ((size_t)G * dv > 1024) return NG_BAD_SIZE;
    const int threads = ((G * dv + 31) / 32) * 32;
    const size_t smem = (2 * (size_t)dk + (size_t)G * dv + 32) * sizeof(float);
    if (smem > 48 * 1024) return NG_BAD_SIZE;
    dim3 grid(n_entries, nH);
    if (grid.y > 65535) return NG_BAD_SIZE;
#define RET_LAUNCH(TT, RR, MT)                                                                                     \
    NG_LAUNCH((retention_kernel<TT, RR, MT>), grid, threads, smem, stream, (const TT*)x, inv_freq, rot_dims, decay, \
              state, (TT*)out, cu_q, ctx_before, slots, nH, dk, dv, G, eps)
    if (act_bf16) {
        if (R == 16) RET_LAUNCH(__nv_bfloat16, 16, 512);
        else if (maxt == 256) RET_LAUNCH(__nv_bfloat16, 64, 256);
        else RET_LAUNCH(__nv_bfloat16, 64, 1024);
    } else {
        if (R == 16) RET_LAUNCH(float, 16, 512);
        else if (maxt == 256) RET_LAUNCH(float, 64, 256);
        else RET_LAUNCH(float, 64, 1024);
    }
    return ng_launch_status();
}
