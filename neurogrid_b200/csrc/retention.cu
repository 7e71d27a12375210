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

// ---------------------------------------------------------------------------------------------- portions, chunk by chunk
// The same recurrence for long portions: a block per (entry, head) walks its tokens in chunks of RC and
// works inside a chunk with matrix products in shared memory (float32 FFMA throughout):
//     A[i][j] = (q_i . k_j) * decay^(i-j)  for j <= i                       (scores inside the chunk)
//     o_i     = sum_j A[i][j] v_j + decay^(i+1) * S^T q_i                   (S: the state before the chunk)
//     S      <- decay^RC * S + sum_j decay^(RC-1-j) k_j v_j^T
// which is the token-by-token recurrence with its sums regrouped: the results differ from it by rounding
// only.  Powers of the decay come from repeated multiplication in float32.
#define RC 32
#define RC_THREADS 256

template <typename T>
__global__ void __launch_bounds__(RC_THREADS)
retention_chunk_kernel(const T* __restrict__ x, const float* __restrict__ inv_freq, int rot_dims,
                       const float* __restrict__ decay, float* __restrict__ state, T* __restrict__ out,
                       const int* __restrict__ cu_q, const int* __restrict__ ctx_before, const int* __restrict__ slots,
                       int nH, int dk, int dv, float eps) {
    extern __shared__ float sm[];
    const int ldq = dk + 1;
    float* Qs = sm;                          // [RC][dk+1]
    float* Ks = Qs + RC * ldq;               // [RC][dk+1]
    float* Vs = Ks + RC * ldq;               // [RC][dv]
    float* As = Vs + RC * dv;                // [RC][RC+1]
    float* Ss = As + RC * (RC + 1);          // [dk][dv]
    float* Os = Ss + dk * dv;                // [RC][dv]
    float* pw = Os + RC * dv;                // [RC+1]  decay^n
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.x, head = blockIdx.y;
    const int q0 = cu_q[e];
    const int qlen = cu_q[e + 1] - q0;
    if (qlen <= 0) return;
    const int ctx = ctx_before[e];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const size_t ld = 2 * (size_t)nH * (dk + dv);
    const size_t off_q = (size_t)head * dk, off_k = (size_t)nH * dk + off_q;
    const size_t off_v = 2 * (size_t)nH * dk + (size_t)head * dv, off_g = off_v + (size_t)nH * dv;
    float* S = state + ((size_t)slots[e] * nH + head) * dk * dv;
    const float lam = decay[head];
    const float kscale = rsqrtf((float)dk);
    const int half = rot_dims / 2;
    for (int i = tid; i < dk * dv; i += RC_THREADS) Ss[i] = ctx > 0 ? S[i] : 0.f;
    if (tid == 0) {
        float p = 1.f;
        for (int n = 0; n <= RC; ++n) {
            pw[n] = p;
            p *= lam;
        }
    }
    for (int c0 = 0; c0 < qlen; c0 += RC) {
        const int n = min(RC, qlen - c0);
        __syncthreads();
        // q and k of the chunk, rotated (pairs p, p + half) and scaled; v as it is
        for (int idx = tid; idx < n * dk; idx += RC_THREADS) {
            const int t = idx / dk, i = idx % dk;
            const T* row = x + (size_t)(q0 + c0 + t) * ld;
            float qv = ng_ld(row + off_q + i), kv = ng_ld(row + off_k + i);
            if (i < rot_dims) {
                const int p = i < half ? i : i - half;
                float sn, cs;
                sincosf((float)(ctx + c0 + t) * inv_freq[p], &sn, &cs);
                const int mate = i < half ? i + half : i - half;
                const float qm = ng_ld(row + off_q + mate), km = ng_ld(row + off_k + mate);
                qv = i < half ? qv * cs - qm * sn : qv * cs + qm * sn;
                kv = i < half ? kv * cs - km * sn : kv * cs + km * sn;
            }
            Qs[t * ldq + i] = qv;
            Ks[t * ldq + i] = kv * kscale;
        }
        for (int idx = tid; idx < n * dv; idx += RC_THREADS) {
            const int t = idx / dv, v = idx % dv;
            Vs[t * dv + v] = ng_ld(x + (size_t)(q0 + c0 + t) * ld + off_v + v);
        }
        __syncthreads();
        for (int idx = tid; idx < n * RC; idx += RC_THREADS) {
            const int i = idx / RC, j = idx % RC;
            float a = 0.f;
            if (j <= i) {
                const float* qi = Qs + i * ldq;
                const float* kj = Ks + j * ldq;
                for (int d = 0; d < dk; ++d) a = fmaf(qi[d], kj[d], a);
                a *= pw[i - j];
            }
            As[i * (RC + 1) + j] = a;
        }
        __syncthreads();
        for (int idx = tid; idx < n * dv; idx += RC_THREADS) {
            const int i = idx / dv, v = idx % dv;
            float inter = 0.f;
            const float* qi = Qs + i * ldq;
            for (int d = 0; d < dk; ++d) inter = fmaf(qi[d], Ss[d * dv + v], inter);
            float acc = inter * pw[i + 1];
            const float* ai = As + i * (RC + 1);
            for (int j = 0; j <= i; ++j) acc = fmaf(ai[j], Vs[j * dv + v], acc);
            Os[i * dv + v] = acc;
        }
        __syncthreads();
        // the state after the chunk's n tokens
        for (int idx = tid; idx < dk * dv; idx += RC_THREADS) {
            const int d = idx / dv, v = idx % dv;
            float acc = Ss[idx] * pw[n];
            for (int j = 0; j < n; ++j) acc = fmaf(Ks[j * ldq + d] * pw[n - 1 - j], Vs[j * dv + v], acc);
            Ss[idx] = acc;
        }
        // each head's o over its root mean square, times silu(gate): a warp per row
        for (int i = warp; i < n; i += RC_THREADS / 32) {
            float ss = 0.f;
            for (int v = lane; v < dv; v += 32) ss += Os[i * dv + v] * Os[i * dv + v];
            ss = ng_warp_sum(ss);
            const float r = rsqrtf(ss / (float)dv + eps);
            const T* row = x + (size_t)(q0 + c0 + i) * ld;
            T* orow = out + (size_t)(q0 + c0 + i) * nH * dv + (size_t)head * dv;
            for (int v = lane; v < dv; v += 32) {
                const float gate = ng_ld(row + off_g + v);
                ng_st(orow + v, Os[i * dv + v] * r * (gate / (1.f + expf(-gate))));
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < dk * dv; i += RC_THREADS) S[i] = Ss[i];
}

static size_t retention_chunk_smem(int dk, int dv) {
    return ((size_t)2 * RC * (dk + 1) + 2 * (size_t)RC * dv + (size_t)RC * (RC + 1) + (size_t)dk * dv + RC + 1) * sizeof(float);
}

// Whether the chunked kernel takes these head sizes (its state and tiles must fit in shared memory).
NG_EXPORT int ng_retention_chunked_takes(int dk, int dv) {
    return dk > 0 && dv > 0 && retention_chunk_smem(dk, dv) <= 200 * 1024;
}

NG_EXPORT int ng_retention_chunked(const void* x, const float* inv_freq, int rot_dims, const float* decay, float* state,
                                   void* out, const int* cu_q, const int* ctx_before, const int* slots, int n_entries,
                                   int nH, int dk, int dv, float eps, int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0) return NG_OK;
    if (nH <= 0 || !ng_retention_chunked_takes(dk, dv) || rot_dims < 0 || rot_dims > dk || rot_dims % 2 ||
        (rot_dims && !inv_freq))
        return NG_BAD_SIZE;
    const size_t smem = retention_chunk_smem(dk, dv);
    static bool configured[2] = {false, false};
    if (!configured[act_bf16 ? 1 : 0]) {
        cudaError_t err = act_bf16 ? cudaFuncSetAttribute(retention_chunk_kernel<__nv_bfloat16>,
                                                          cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
                                   : cudaFuncSetAttribute(retention_chunk_kernel<float>,
                                                          cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (err != cudaSuccess) return NG_LAUNCH_FAILED;
        configured[act_bf16 ? 1 : 0] = true;
    }
    dim3 grid(n_entries, nH);
    if (grid.y > 65535) return NG_BAD_SIZE;
    if (act_bf16)
        NG_LAUNCH((retention_chunk_kernel<__nv_bfloat16>), grid, RC_THREADS, smem, stream, (const __nv_bfloat16*)x, inv_freq,
                  rot_dims, decay, state, (__nv_bfloat16*)out, cu_q, ctx_before, slots, nH, dk, dv, eps);
    else
        NG_LAUNCH((retention_chunk_kernel<float>), grid, RC_THREADS, smem, stream, (const float*)x, inv_freq, rot_dims,
                  decay, state, (float*)out, cu_q, ctx_before, slots, nH, dk, dv, eps);
    return ng_launch_status();
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
