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
// The same recurrence for long portions, with its sums regrouped so that the chunks of a portion run side by
// side.  With chunks of RC tokens, n the tokens of a chunk, S the state before it:
//     U      = sum_j decay^(n-1-j) k_j v_j^T                                (what the chunk adds to the state)
//     S'     = decay^n * S + U                                              (the state after it)
//     A[i][j] = (q_i . k_j) * decay^(i-j)  for j <= i                       (scores inside the chunk)
//     o_i    = sum_j A[i][j] v_j + decay^(i+1) * S^T q_i
// Three kernels: `local` forms U of every chunk (a block per chunk, head and slice of value columns);
// `scan` walks a request's chunks in order, one thread per state element, leaves each chunk's S where its U
// was and the last S' in the request's slot; `out` forms o of every chunk from its own q, k, v and its S.
// A fourth divides each head's o (float32 scratch) by its root mean square and applies the gate.  Small
// matrix products in shared memory, a register tile per thread, float32 FFMA throughout; powers of the decay
// come from repeated multiplication.  The results differ from the token-by-token kernel's by rounding only.
// Chunk c of entry e keeps its U / S in slot  cu_q[e] / RC + e + c  of the scratch: slots of different
// entries do not meet, and rows / RC + entries + 1 slots are enough.
#define RC 32
#define RC_THREADS 128

struct RetGeom {
    int nH, dk, dv, dvs, rot_dims;
};

// q and/or k of a chunk into shared memory, rotated (pairs p, p + half) and k scaled; rows past n are zero
template <typename T, bool WANT_Q>
__device__ __forceinline__ void ret_load_qk(const T* __restrict__ x, size_t ld, size_t off_q, size_t off_k, int row0,
                                            int n, int pos0, const float* __restrict__ inv_freq, int rot_dims, int dk,
                                            float kscale, float* Qs, float* Ks) {
    const int ldq = dk + 1, half = rot_dims / 2;
    for (int idx = threadIdx.x; idx < RC * dk; idx += RC_THREADS) {
        const int t = idx / dk, i = idx % dk;
        float qv = 0.f, kv = 0.f;
        if (t < n) {
            const T* row = x + (size_t)(row0 + t) * ld;
            if (WANT_Q) qv = ng_ld(row + off_q + i);
            kv = ng_ld(row + off_k + i);
            if (i < rot_dims) {
                const int p = i < half ? i : i - half;
                float sn, cs;
                sincosf((float)(pos0 + t) * inv_freq[p], &sn, &cs);
                const int mate = i < half ? i + half : i - half;
                const float km = ng_ld(row + off_k + mate);
                kv = i < half ? kv * cs - km * sn : kv * cs + km * sn;
                if (WANT_Q) {
                    const float qm = ng_ld(row + off_q + mate);
                    qv = i < half ? qv * cs - qm * sn : qv * cs + qm * sn;
                }
            }
        }
        if (WANT_Q) Qs[t * ldq + i] = qv;
        Ks[t * ldq + i] = kv * kscale;
    }
}

__device__ __forceinline__ void ret_powers(float* pw, float lam) {
    if (threadIdx.x == 0) {
        float p = 1.f;
        for (int n = 0; n <= RC; ++n) {
            pw[n] = p;
            p *= lam;
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(RC_THREADS)
retention_local_kernel(const T* __restrict__ x, const float* __restrict__ inv_freq, const float* __restrict__ decay,
                       float* __restrict__ u_scratch, const int* __restrict__ cu_q, const int* __restrict__ ctx_before,
                       RetGeom g) {
    extern __shared__ float sm[];
    const int dk = g.dk, dv = g.dv, dvs = g.dvs, nH = g.nH, ldq = dk + 1;
    float* Ks = sm;                          // [RC][dk+1]
    float* Vs = Ks + RC * ldq;               // [RC][dvs]
    float* pw = Vs + RC * dvs;               // [RC+1]
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.x, c = blockIdx.y, slices = dv / dvs;
    const int head = blockIdx.z / slices, v0 = (blockIdx.z % slices) * dvs;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    if (c * RC >= qlen) return;
    const int n = min(RC, qlen - c * RC);
    const size_t ld = 2 * (size_t)nH * (dk + dv);
    const size_t off_k = (size_t)nH * dk + (size_t)head * dk;
    const size_t off_v = 2 * (size_t)nH * dk + (size_t)head * dv + v0;
    ret_powers(pw, decay[head]);
    ret_load_qk<T, false>(x, ld, 0, off_k, q0 + c * RC, n, ctx_before[e] + c * RC, inv_freq, g.rot_dims, dk,
                          rsqrtf((float)dk), nullptr, Ks);
    for (int idx = threadIdx.x; idx < RC * dvs; idx += RC_THREADS) {
        const int t = idx / dvs, v = idx % dvs;
        Vs[idx] = t < n ? ng_ld(x + (size_t)(q0 + c * RC + t) * ld + off_v + v) : 0.f;
    }
    __syncthreads();
    float* U = u_scratch + (((size_t)(q0 / RC + e + c)) * nH + head) * dk * dv + v0;      // row d at U + d * dv
    for (int tile = threadIdx.x; tile < ((dk + 7) / 8) * (dvs / 4); tile += RC_THREADS) {
        const int d0 = (tile / (dvs / 4)) * 8, c0v = (tile % (dvs / 4)) * 4;
        float acc[8][4] = {};
        for (int j = 0; j < n; ++j) {
            const float4 vv = *reinterpret_cast<const float4*>(Vs + j * dvs + c0v);
            const float w = pw[n - 1 - j];
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                const float kv = (d0 + r < dk ? Ks[j * ldq + d0 + r] : 0.f) * w;
                acc[r][0] = fmaf(kv, vv.x, acc[r][0]);
                acc[r][1] = fmaf(kv, vv.y, acc[r][1]);
                acc[r][2] = fmaf(kv, vv.z, acc[r][2]);
                acc[r][3] = fmaf(kv, vv.w, acc[r][3]);
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (d0 + r >= dk) break;
            *reinterpret_cast<float4*>(U + (size_t)(d0 + r) * dv + c0v) = make_float4(acc[r][0], acc[r][1], acc[r][2], acc[r][3]);
        }
    }
}

// One thread per state element of a (request, head): S before each chunk replaces the chunk's U; the last S' is the slot's.
__global__ void retention_scan_kernel(float* __restrict__ u_scratch, float* __restrict__ state,
                                      const float* __restrict__ decay, const int* __restrict__ cu_q,
                                      const int* __restrict__ ctx_before, const int* __restrict__ slots, int nH, int dk, int dv) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.y, head = blockIdx.z;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    if (qlen <= 0 || i >= dk * dv) return;
    const float lam = decay[head];
    float full = 1.f;
    for (int k = 0; k < RC; ++k) full *= lam;                        // decay^RC, by the same multiplications as the tables
    float* S = state + ((size_t)slots[e] * nH + head) * dk * dv + i;
    float s = ctx_before[e] > 0 ? *S : 0.f;
    const int nc = (qlen + RC - 1) / RC;
    float* U0 = u_scratch + (((size_t)(q0 / RC + e)) * nH + head) * dk * dv + i;
    const size_t stride = (size_t)nH * dk * dv;
    // eight chunks' additions are fetched at once: the walk itself is a chain, the loads need not be
    for (int c0 = 0; c0 < nc; c0 += 8) {
        float u[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) u[k] = c0 + k < nc ? U0[(size_t)(c0 + k) * stride] : 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k;
            if (c >= nc) break;
            U0[(size_t)c * stride] = s;
            float f = full;
            if (c == nc - 1 && qlen % RC) {
                f = 1.f;
                for (int m = 0; m < qlen % RC; ++m) f *= lam;
            }
            s = fmaf(s, f, u[k]);
        }
    }
    *S = s;
}

template <typename T>
__global__ void __launch_bounds__(RC_THREADS)
retention_out_kernel(const T* __restrict__ x, const float* __restrict__ inv_freq, const float* __restrict__ decay,
                     const float* __restrict__ u_scratch, float* __restrict__ o_scratch, const int* __restrict__ cu_q,
                     const int* __restrict__ ctx_before, RetGeom g) {
    extern __shared__ float sm[];
    const int dk = g.dk, dv = g.dv, dvs = g.dvs, nH = g.nH, ldq = dk + 1, lda = RC + 1;
    float* Qs = sm;                          // [RC][dk+1]
    float* Ks = Qs + RC * ldq;               // [RC][dk+1]
    float* Vs = Ks + RC * ldq;               // [RC][dvs]
    float* As = Vs + RC * dvs;               // [RC][RC+1]
    float* pw = As + RC * lda;               // [RC+1]
    // the state before the chunk, [dk][dvs]: in k's place once the scores are formed when it fits there (more blocks
    // a SM), behind the rest otherwise
    const bool s_over_k = dk * dvs <= RC * ldq;
    float* Ss = s_over_k ? Ks : sm + ((2 * RC * ldq + RC * dvs + RC * lda + RC + 1 + 3) & ~3);      // 16-byte aligned
    ng_pdl_trigger();
    ng_pdl_wait();
    const int e = blockIdx.x, c = blockIdx.y, slices = dv / dvs;
    const int head = blockIdx.z / slices, v0 = (blockIdx.z % slices) * dvs;
    const int q0 = cu_q[e], qlen = cu_q[e + 1] - q0;
    if (c * RC >= qlen) return;
    const int n = min(RC, qlen - c * RC);
    const int tid = threadIdx.x;
    const size_t ld = 2 * (size_t)nH * (dk + dv);
    const size_t off_q = (size_t)head * dk, off_k = (size_t)nH * dk + off_q;
    const size_t off_v = 2 * (size_t)nH * dk + (size_t)head * dv + v0;
    ret_powers(pw, decay[head]);
    ret_load_qk<T, true>(x, ld, off_q, off_k, q0 + c * RC, n, ctx_before[e] + c * RC, inv_freq, g.rot_dims, dk,
                         rsqrtf((float)dk), Qs, Ks);
    for (int idx = tid; idx < RC * dvs; idx += RC_THREADS) {
        const int t = idx / dvs, v = idx % dvs;
        Vs[idx] = t < n ? ng_ld(x + (size_t)(q0 + c * RC + t) * ld + off_v + v) : 0.f;
    }
    const float* Sb = u_scratch + (((size_t)(q0 / RC + e + c)) * nH + head) * dk * dv + v0;
    if (!s_over_k)
        for (int idx = tid; idx < dk * (dvs / 4); idx += RC_THREADS) {
            const int d = idx / (dvs / 4), v4 = (idx % (dvs / 4)) * 4;
            *reinterpret_cast<float4*>(Ss + d * dvs + v4) = *reinterpret_cast<const float4*>(Sb + (size_t)d * dv + v4);
        }
    __syncthreads();
    {   // A: a 2 x 4 tile per thread (16 x 8 tiles cover RC x RC)
        const int i0 = (tid / 8) * 2, j0 = (tid % 8) * 4;
        float a[2][4] = {};
        if (j0 <= i0 + 1) {
            for (int d = 0; d < dk; ++d) {
                const float qa = Qs[i0 * ldq + d], qb = Qs[(i0 + 1) * ldq + d];
#pragma unroll
                for (int cc = 0; cc < 4; ++cc) {
                    const float kv = Ks[(j0 + cc) * ldq + d];
                    a[0][cc] = fmaf(qa, kv, a[0][cc]);
                    a[1][cc] = fmaf(qb, kv, a[1][cc]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) {
                const int i = i0 + r, j = j0 + cc;
                As[i * lda + j] = j <= i ? a[r][cc] * pw[i - j] : 0.f;
            }
    }
    __syncthreads();
    if (s_over_k) {                          // k is done with: the state takes its place
        for (int idx = tid; idx < dk * (dvs / 4); idx += RC_THREADS) {
            const int d = idx / (dvs / 4), v4 = (idx % (dvs / 4)) * 4;
            *reinterpret_cast<float4*>(Ss + d * dvs + v4) = *reinterpret_cast<const float4*>(Sb + (size_t)d * dv + v4);
        }
        __syncthreads();
    }
    // o: 4 x 2 tiles over RC x dvs;  inside the chunk (A V) and from the state (Q S), kept apart until the end
    for (int tile = tid; tile < (RC / 4) * (dvs / 2); tile += RC_THREADS) {
        const int i0 = (tile / (dvs / 2)) * 4, c0v = (tile % (dvs / 2)) * 2;
        float in[4][2] = {}, st[4][2] = {};
        for (int j = 0; j < RC; ++j) {
            const float2 vv = *reinterpret_cast<const float2*>(Vs + j * dvs + c0v);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float av = As[(i0 + r) * lda + j];
                in[r][0] = fmaf(av, vv.x, in[r][0]);
                in[r][1] = fmaf(av, vv.y, in[r][1]);
            }
        }
        for (int d = 0; d < dk; ++d) {
            const float2 sv = *reinterpret_cast<const float2*>(Ss + d * dvs + c0v);
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const float qv = Qs[(i0 + r) * ldq + d];
                st[r][0] = fmaf(qv, sv.x, st[r][0]);
                st[r][1] = fmaf(qv, sv.y, st[r][1]);
            }
        }
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int i = i0 + r;
            if (i < n) {
                float* dst = o_scratch + (size_t)(q0 + c * RC + i) * nH * dv + (size_t)head * dv + v0 + c0v;
                dst[0] = in[r][0] + pw[i + 1] * st[r][0];
                dst[1] = in[r][1] + pw[i + 1] * st[r][1];
            }
        }
    }
}

// out[row, head, :] = o[row, head, :] / sqrt(mean(o^2) + eps) * silu(gate): a warp per (row, head)
template <typename T>
__global__ void retention_norm_gate_kernel(const float* __restrict__ o, const T* __restrict__ x, T* __restrict__ out,
                                           int n_rows, int nH, int dk, int dv, float eps) {
    ng_pdl_trigger();
    ng_pdl_wait();
    const int w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= n_rows * nH) return;
    const int row = w / nH, head = w % nH;
    const float* orow = o + (size_t)row * nH * dv + (size_t)head * dv;
    const T* g = x + (size_t)row * 2 * nH * (dk + dv) + 2 * (size_t)nH * dk + (size_t)nH * dv + (size_t)head * dv;
    float ss = 0.f;
    for (int v = lane; v < dv; v += 32) ss += orow[v] * orow[v];
    ss = ng_warp_sum(ss);
    const float r = rsqrtf(ss / (float)dv + eps);
    for (int v = lane; v < dv; v += 32) {
        const float gate = ng_ld(g + v);
        ng_st(out + (size_t)row * nH * dv + (size_t)head * dv + v, orow[v] * r * (gate / (1.f + expf(-gate))));
    }
}

static int retention_chunk_slice(int dv) { return dv % 32 == 0 ? 32 : dv; }
static size_t retention_out_smem(int dk, int dv) {
    const int dvs = retention_chunk_slice(dv);
    const size_t base = (size_t)2 * RC * (dk + 1) + (size_t)RC * dvs + (size_t)RC * (RC + 1) + RC + 1;
    const size_t state = (size_t)dk * dvs <= (size_t)RC * (dk + 1) ? 0 : (size_t)dk * dvs + 4;   // else it lies in k's place
    return (base + state) * sizeof(float);
}
static size_t retention_local_smem(int dk, int dv) {
    return ((size_t)RC * (dk + 1) + (size_t)RC * retention_chunk_slice(dv) + RC + 1) * sizeof(float);
}

// Whether the chunked kernels take these head sizes (tiles must fit in shared memory; value columns in fours).
NG_EXPORT int ng_retention_chunked_takes(int dk, int dv) {
    return dk > 0 && dv > 0 && dv % 4 == 0 && retention_out_smem(dk, dv) <= 200 * 1024;
}

// float32 values of `u_scratch` for a step of n_rows rows in n_entries entries
NG_EXPORT long long ng_retention_chunked_scratch(int n_rows, int n_entries, int nH, int dk, int dv) {
    return ((long long)n_rows / RC + n_entries + 1) * nH * dk * dv;
}

// As ng_retention; `o_scratch`: float32 [n_rows, nH*dv] (the heads' outputs before their norm); `u_scratch`:
// ng_retention_chunked_scratch float32 values (every chunk's addition to the state, then the state before it).
NG_EXPORT int ng_retention_chunked(const void* x, const float* inv_freq, int rot_dims, const float* decay, float* state,
                                   void* out, float* o_scratch, float* u_scratch, const int* cu_q, const int* ctx_before,
                                   const int* slots, int n_entries, int n_rows, int max_q, int nH, int dk, int dv, float eps,
                                   int act_bf16, cudaStream_t stream) {
    if (n_entries <= 0 || n_rows <= 0 || max_q <= 0) return NG_OK;
    if (nH <= 0 || !ng_retention_chunked_takes(dk, dv) || rot_dims < 0 || rot_dims > dk || rot_dims % 2 ||
        (rot_dims && !inv_freq) || !o_scratch || !u_scratch)
        return NG_BAD_SIZE;
    const int dvs = retention_chunk_slice(dv);
    const RetGeom g{nH, dk, dv, dvs, rot_dims};
    static bool configured[2] = {false, false};
    const int which = act_bf16 ? 1 : 0;
    if (!configured[which]) {
        cudaError_t e1, e2;
        if (act_bf16) {
            e1 = cudaFuncSetAttribute(retention_out_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            e2 = cudaFuncSetAttribute(retention_local_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        } else {
            e1 = cudaFuncSetAttribute(retention_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            e2 = cudaFuncSetAttribute(retention_local_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        }
        if (e1 != cudaSuccess || e2 != cudaSuccess) return NG_LAUNCH_FAILED;
        configured[which] = true;
    }
    dim3 grid(n_entries, (max_q + RC - 1) / RC, nH * (dv / dvs));
    dim3 sgrid((dk * dv + 255) / 256, n_entries, nH);
    if (grid.y > 65535 || grid.z > 65535 || sgrid.y > 65535 || sgrid.z > 65535) return NG_BAD_SIZE;
    const unsigned nblocks = (unsigned)(((size_t)n_rows * nH + 7) / 8);
    const size_t sl = retention_local_smem(dk, dv), so = retention_out_smem(dk, dv);
    if (act_bf16) {
        typedef __nv_bfloat16 B;
        NG_LAUNCH((retention_local_kernel<B>), grid, RC_THREADS, sl, stream, (const B*)x, inv_freq, decay, u_scratch, cu_q, ctx_before, g);
        NG_LAUNCH((retention_scan_kernel), sgrid, 256, 0, stream, u_scratch, state, decay, cu_q, ctx_before, slots, nH, dk, dv);
        NG_LAUNCH((retention_out_kernel<B>), grid, RC_THREADS, so, stream, (const B*)x, inv_freq, decay, (const float*)u_scratch, o_scratch, cu_q, ctx_before, g);
        NG_LAUNCH((retention_norm_gate_kernel<B>), nblocks, 256, 0, stream, (const float*)o_scratch, (const B*)x, (B*)out, n_rows, nH, dk, dv, eps);
    } else {
        NG_LAUNCH((retention_local_kernel<float>), grid, RC_THREADS, sl, stream, (const float*)x, inv_freq, decay, u_scratch, cu_q, ctx_before, g);
        NG_LAUNCH((retention_scan_kernel), sgrid, 256, 0, stream, u_scratch, state, decay, cu_q, ctx_before, slots, nH, dk, dv);
        NG_LAUNCH((retention_out_kernel<float>), grid, RC_THREADS, so, stream, (const float*)x, inv_freq, decay, (const float*)u_scratch, o_scratch, cu_q, ctx_before, g);
        NG_LAUNCH((retention_norm_gate_kernel<float>), nblocks, 256, 0, stream, (const float*)o_scratch, (const float*)x, (float*)out, n_rows, nH, dk, dv, eps);
    }
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
