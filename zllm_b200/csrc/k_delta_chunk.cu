// Gated delta rule in its chunked form: 64 tokens of a head advance the state in one step of dense algebra
// instead of 64 dependent updates. The reference has no such kernel (src/kernels/delta_rule.wgsl runs every
// token serially); this is the same recurrence (src/ref/qwen35.zig:493-546), reassociated, all in f32:
//
//   per token t of a chunk that starts at state S0, with G_t = g_1 + ... + g_t:
//     delta_t = beta_t (v_t - e^{G_t} S0^T k_t - sum_{s<t} e^{G_t - G_s} (k_s.k_t) delta_s)
//     o_t     = (e^{G_t} S0^T q_t + sum_{s<=t} e^{G_t - G_s} (k_s.q_t) delta_s) / sqrt(d)
//     S_C     = e^{G_C} S0 + sum_s e^{G_C - G_s} k_s delta_s^T
//   With A[t][s] = beta_t e^{G_t-G_s} (k_t.k_s) (s < t) the deltas solve (I + A) Delta = diag(beta)(V - Gamma K S0),
//   so Delta = T' (V - Gamma K S0) with T' = (I + A)^-1 diag(beta). Every decay factor is e^{difference <= 0}.
//
// Two kernels:
//   delta_chunk_prep  one CTA per (chunk, value head), all chunks in parallel: A, its inverse T' and
//                     P[t][s] = e^{G_t-G_s} (q_t.k_s) / sqrt(d) (s <= t) do not depend on the state
//   delta_chunk_scan  one CTA per (value head, 16 state columns), serial over chunks: U = K S0, Y = Q S0,
//                     Delta = T'(V - Gamma U), O = Gamma Y / sqrt(d) + P Delta, S <- e^{G_C} S + (decayed K)^T Delta.
//                     Column b of S depends only on column b, so the column slices are independent.
// The remainder of a step (tokens past the last whole chunk), the conv history and a kept state go through the
// recurrent kernel.

#include "zcu_internal.h"

namespace {

constexpr int CH = 64;     // tokens per chunk
constexpr int CD = 128;    // head dimension this form is built for
constexpr int KP = CD + 4; // padded row of a K/Q tile in shared memory (keeps 16-byte alignment, spreads banks)
constexpr int TP = CH + 4; // padded row of a T'/P tile
constexpr int SC = 16;     // state columns per scan CTA
constexpr int PREP_T = 256, SCAN_T = 512;

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }

// ---------------------------------------------------------------------------------------------- prep
// grid (chunks, v_heads). Writes tp[(c * v_heads + j)][64][64], pm[...][64][64], gc[...][64] (cumulative g).
__global__ void __launch_bounds__(PREP_T) delta_chunk_prep(PDeltaRule p, const float* __restrict__ conv, const float* __restrict__ g,
                                                          const float* __restrict__ beta, float* __restrict__ tp,
                                                          float* __restrict__ pm, float* __restrict__ gc) {
    extern __shared__ __align__(16) float sm[];
    float* Ks = sm;                 // [64][KP]
    float* Qs = Ks + CH * KP;       // [64][KP]
    float* As = Qs + CH * KP;       // [64][TP]
    float* Gs = As + CH * TP;       // [64]
    float* Bs = Gs + CH;            // [64]
    const int tid = threadIdx.x, c = blockIdx.x, j = blockIdx.y;
    const int kh = j % (int)p.k_heads, key_dim = (int)p.k_heads * CD;
    const size_t tok0 = (size_t)c * CH;
    const size_t unit = (size_t)c * p.v_heads + j;
    if (tid < CH) {
        Gs[tid] = g[(tok0 + tid) * p.v_heads + j];
        Bs[tid] = beta[(tok0 + tid) * p.v_heads + j];
    }
    for (int i = tid; i < CH * (CD / 4); i += PREP_T) {
        const int t = i / (CD / 4), a4 = i % (CD / 4);
        const float* row = conv + (tok0 + t) * p.conv_stride + (size_t)kh * CD + 4 * a4;
        *reinterpret_cast<float4*>(Qs + t * KP + 4 * a4) = ld4(row);
        *reinterpret_cast<float4*>(Ks + t * KP + 4 * a4) = ld4(row + key_dim);
    }
    __syncthreads();
    if (tid == 0) {  // cumulative log-decay, summed in token order
        float run = 0.f;
        for (int t = 0; t < CH; t++) {
            run = __fadd_rn(run, Gs[t]);
            Gs[t] = run;
        }
    }
    // K K^T and Q K^T: thread (ty, tx) owns tokens t = ty + 16 i and s = tx + 16 i'
    const int tx = tid % 16, ty = tid / 16;
    float kk[4][4], qk[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int l = 0; l < 4; l++) kk[i][l] = 0.f, qk[i][l] = 0.f;
    for (int a = 0; a < CD; a += 4) {
        float4 kt[4], qt[4], ks[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            kt[i] = ld4(Ks + (ty + 16 * i) * KP + a);
            qt[i] = ld4(Qs + (ty + 16 * i) * KP + a);
            ks[i] = ld4(Ks + (tx + 16 * i) * KP + a);
        }
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int l = 0; l < 4; l++) {
                kk[i][l] = fmaf(kt[i].x, ks[l].x, kk[i][l]);
                kk[i][l] = fmaf(kt[i].y, ks[l].y, kk[i][l]);
                kk[i][l] = fmaf(kt[i].z, ks[l].z, kk[i][l]);
                kk[i][l] = fmaf(kt[i].w, ks[l].w, kk[i][l]);
                qk[i][l] = fmaf(qt[i].x, ks[l].x, qk[i][l]);
                qk[i][l] = fmaf(qt[i].y, ks[l].y, qk[i][l]);
                qk[i][l] = fmaf(qt[i].z, ks[l].z, qk[i][l]);
                qk[i][l] = fmaf(qt[i].w, ks[l].w, qk[i][l]);
            }
    }
    __syncthreads();  // Gs complete
    const float scale = 1.0f / sqrtf((float)CD);
    float* pout = pm + unit * CH * CH;
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const int t = ty + 16 * i, s = tx + 16 * l;
            const float dec = s <= t ? expf(Gs[t] - Gs[s]) : 0.f;
            As[t * TP + s] = s < t ? Bs[t] * dec * kk[i][l] : 0.f;
            pout[t * CH + s] = dec * qk[i][l] * scale;
        }
    if (tid < CH) gc[unit * CH + tid] = Gs[tid];
    __syncthreads();
    // (I + A)^-1, one column per thread: T[t][c] = [t == c] - sum_{s<t} A[t][s] T[s][c]. Column c needs only
    // column c of the rows above, so the 64 threads run the whole substitution in registers.
    if (tid < CH) {
        float T[CH];
#pragma unroll
        for (int t = 0; t < CH; t++) {
            float acc = (t == tid) ? 1.f : 0.f;
#pragma unroll
            for (int s4 = 0; s4 < t; s4 += 4) {
                const float4 a4 = ld4(As + t * TP + s4);  // entries at s >= t are zero
                acc = fmaf(-a4.x, T[s4], acc);
                if (s4 + 1 < t) acc = fmaf(-a4.y, T[s4 + 1], acc);
                if (s4 + 2 < t) acc = fmaf(-a4.z, T[s4 + 2], acc);
                if (s4 + 3 < t) acc = fmaf(-a4.w, T[s4 + 3], acc);
            }
            T[t] = acc;
        }
        const float bc = Bs[tid];
        float* tout = tp + unit * CH * CH;
#pragma unroll
        for (int t = 0; t < CH; t++) tout[t * CH + tid] = T[t] * bc;  // T' = T diag(beta)
    }
}

// ---------------------------------------------------------------------------------------------- scan
// grid (v_heads, CD / SC), 512 threads: thread (tr, col) with col = tid % 16 one of the CTA's state columns.
__global__ void __launch_bounds__(SCAN_T, 1) delta_chunk_scan(PDeltaRule p, int chunks, const float* __restrict__ conv,
                                                             const float* __restrict__ tp, const float* __restrict__ pm,
                                                             const float* __restrict__ gc, float* __restrict__ state,
                                                             float* __restrict__ out) {
    extern __shared__ __align__(16) float sm[];
    float* Ks = sm;                  // [64][KP]
    float* Qs = Ks + CH * KP;        // [64][KP]
    float* Ts = Qs + CH * KP;        // [64][TP]  T'
    float* Ps = Ts + CH * TP;        // [64][TP]
    float* Ss = Ps + CH * TP;        // [128][16] the state slice
    float* Rs = Ss + CD * SC;        // [64][16]  V, then V - Gamma U
    float* Ys = Rs + CH * SC;        // [64][16]  Gamma Y / sqrt(d)
    float* Ds = Ys + CH * SC;        // [64][16]  Delta
    float* Dd = Ds + CH * SC;        // [64][16]  e^{G_C - G_s} Delta
    float* Gs = Dd + CH * SC;        // [64]
    const int tid = threadIdx.x, col = tid % SC, tr = tid / SC;  // tr in 0..31
    const int j = blockIdx.x, b0 = blockIdx.y * SC;
    const int kh = j % (int)p.k_heads, key_dim = (int)p.k_heads * CD;
    const size_t s0 = (size_t)j * CD * CD;
    const float scale = 1.0f / sqrtf((float)CD);
    for (int i = tid; i < CD * SC; i += SCAN_T) Ss[i] = state[s0 + (size_t)(i / SC) * CD + b0 + i % SC];

    for (int c = 0; c < chunks; c++) {
        const size_t tok0 = (size_t)c * CH, unit = (size_t)c * p.v_heads + j;
        for (int i = tid; i < CH * (CD / 4); i += SCAN_T) {
            const int t = i / (CD / 4), a4 = i % (CD / 4);
            const float* row = conv + (tok0 + t) * p.conv_stride + (size_t)kh * CD + 4 * a4;
            *reinterpret_cast<float4*>(Qs + t * KP + 4 * a4) = ld4(row);
            *reinterpret_cast<float4*>(Ks + t * KP + 4 * a4) = ld4(row + key_dim);
        }
        for (int i = tid; i < CH * (CH / 4); i += SCAN_T) {
            const int t = i / (CH / 4), s4 = i % (CH / 4);
            *reinterpret_cast<float4*>(Ts + t * TP + 4 * s4) = ld4(tp + unit * CH * CH + t * CH + 4 * s4);
            *reinterpret_cast<float4*>(Ps + t * TP + 4 * s4) = ld4(pm + unit * CH * CH + t * CH + 4 * s4);
        }
        for (int i = tid; i < CH * SC; i += SCAN_T)
            Rs[i] = conv[(tok0 + i / SC) * p.conv_stride + 2 * (size_t)key_dim + (size_t)j * CD + b0 + i % SC];
        if (tid < CH) Gs[tid] = gc[unit * CH + tid];
        __syncthreads();

        // 1. U = K S0 and Y = Q S0 for tokens tr and tr + 32 at this column
        {
            float u0 = 0.f, u1 = 0.f, y0 = 0.f, y1 = 0.f;
            const float *k0 = Ks + tr * KP, *k1 = Ks + (tr + 32) * KP, *q0 = Qs + tr * KP, *q1 = Qs + (tr + 32) * KP;
#pragma unroll 4
            for (int a = 0; a < CD; a += 4) {
                const float sa = Ss[a * SC + col], sb = Ss[(a + 1) * SC + col], sc = Ss[(a + 2) * SC + col], sd = Ss[(a + 3) * SC + col];
                const float4 ka = ld4(k0 + a), kb = ld4(k1 + a), qa = ld4(q0 + a), qb = ld4(q1 + a);
                u0 = fmaf(ka.x, sa, u0), u0 = fmaf(ka.y, sb, u0), u0 = fmaf(ka.z, sc, u0), u0 = fmaf(ka.w, sd, u0);
                u1 = fmaf(kb.x, sa, u1), u1 = fmaf(kb.y, sb, u1), u1 = fmaf(kb.z, sc, u1), u1 = fmaf(kb.w, sd, u1);
                y0 = fmaf(qa.x, sa, y0), y0 = fmaf(qa.y, sb, y0), y0 = fmaf(qa.z, sc, y0), y0 = fmaf(qa.w, sd, y0);
                y1 = fmaf(qb.x, sa, y1), y1 = fmaf(qb.y, sb, y1), y1 = fmaf(qb.z, sc, y1), y1 = fmaf(qb.w, sd, y1);
            }
            const float e0 = expf(Gs[tr]), e1 = expf(Gs[tr + 32]);
            Rs[tr * SC + col] = Rs[tr * SC + col] - e0 * u0;
            Rs[(tr + 32) * SC + col] = Rs[(tr + 32) * SC + col] - e1 * u1;
            Ys[tr * SC + col] = e0 * y0 * scale;
            Ys[(tr + 32) * SC + col] = e1 * y1 * scale;
        }
        __syncthreads();
        // 2. Delta = T' R (T' is lower triangular: s <= t)
        {
            const float gC = Gs[CH - 1];
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int t = tr + 32 * h;
                float acc = 0.f;
                const float* trow = Ts + t * TP;
                for (int s = 0; s <= t; s += 4) {  // entries past t are zero
                    const float4 w = ld4(trow + s);
                    acc = fmaf(w.x, Rs[s * SC + col], acc);
                    acc = fmaf(w.y, Rs[(s + 1) * SC + col], acc);
                    acc = fmaf(w.z, Rs[(s + 2) * SC + col], acc);
                    acc = fmaf(w.w, Rs[(s + 3) * SC + col], acc);
                }
                Ds[t * SC + col] = acc;
                Dd[t * SC + col] = acc * expf(gC - Gs[t]);
            }
        }
        __syncthreads();
        // 3. O = Gamma Y / sqrt(d) + P Delta
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const int t = tr + 32 * h;
            float acc = Ys[t * SC + col];
            const float* prow = Ps + t * TP;
            for (int s = 0; s <= t; s += 4) {
                const float4 w = ld4(prow + s);
                acc = fmaf(w.x, Ds[s * SC + col], acc);
                acc = fmaf(w.y, Ds[(s + 1) * SC + col], acc);
                acc = fmaf(w.z, Ds[(s + 2) * SC + col], acc);
                acc = fmaf(w.w, Ds[(s + 3) * SC + col], acc);
            }
            out[(tok0 + t) * p.v_heads * CD + (size_t)j * CD + b0 + col] = acc;
        }
        // 4. S <- e^{G_C} S + sum_s k_s (e^{G_C - G_s} delta_s)^T for key rows 4 tr .. 4 tr + 3
        {
            const float eC = expf(Gs[CH - 1]);
            const int a0 = 4 * tr;
            float n0 = eC * Ss[a0 * SC + col], n1 = eC * Ss[(a0 + 1) * SC + col], n2 = eC * Ss[(a0 + 2) * SC + col],
                  n3 = eC * Ss[(a0 + 3) * SC + col];
#pragma unroll 8
            for (int s = 0; s < CH; s++) {
                const float4 kv = ld4(Ks + s * KP + a0);
                const float dd = Dd[s * SC + col];
                n0 = fmaf(kv.x, dd, n0), n1 = fmaf(kv.y, dd, n1), n2 = fmaf(kv.z, dd, n2), n3 = fmaf(kv.w, dd, n3);
            }
            Ss[a0 * SC + col] = n0, Ss[(a0 + 1) * SC + col] = n1, Ss[(a0 + 2) * SC + col] = n2, Ss[(a0 + 3) * SC + col] = n3;
        }
        __syncthreads();  // the tiles are overwritten by the next chunk; the state rows by their own threads only
    }
    for (int i = tid; i < CD * SC; i += SCAN_T) state[s0 + (size_t)(i / SC) * CD + b0 + i % SC] = Ss[i];
}

constexpr int PREP_SMEM = (2 * CH * KP + CH * TP + 2 * CH) * 4;
constexpr int SCAN_SMEM = (2 * CH * KP + 2 * CH * TP + CD * SC + 4 * CH * SC + CH) * 4;

}  // namespace

// Same bindings as delta_rule: conv, g, beta, state (rw), out (rw), step[, proj, hist (rw), kept (rw)].
zcu_result launch_delta_chunked(const LaunchArgs& a) {
    PDeltaRule p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 6, "delta_rule (chunked): bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.dim == CD, "delta_rule (chunked): the chunked form is built for dim %d, got %u", CD, p.dim);
    ZCU_NEED(a, p.k_heads > 0 && p.v_heads > 0 && p.conv_stride % 4 == 0, "delta_rule (chunked): heads or row stride");
    ZCU_NEED(a, ((uintptr_t)a.b[0].ptr & 15) == 0, "delta_rule (chunked): conv must be 16-byte aligned");
    const uint32_t m = p._pad;  // the step's token count, known to the host
    const int chunks = (int)(m / CH);
    if (chunks > 0) {
        const size_t units = (size_t)chunks * p.v_heads;
        float* scratch = nullptr;
        const size_t bytes = units * (2 * CH * CH + CH) * sizeof(float);
        if (cudaMallocAsync((void**)&scratch, bytes, a.stream) != cudaSuccess) {
            cudaGetLastError();
            ZCU_NEED(a, false, "delta_rule (chunked): no memory for %zu bytes of chunk matrices", bytes);
        }
        float *tp = scratch, *pm = tp + units * CH * CH, *gc = pm + units * CH * CH;
        cudaFuncSetAttribute(delta_chunk_prep, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_SMEM);
        cudaFuncSetAttribute(delta_chunk_scan, cudaFuncAttributeMaxDynamicSharedMemorySize, SCAN_SMEM);
        delta_chunk_prep<<<dim3(chunks, p.v_heads), PREP_T, PREP_SMEM, a.stream>>>(p, (const float*)a.b[0].ptr, (const float*)a.b[1].ptr,
                                                                                  (const float*)a.b[2].ptr, tp, pm, gc);
        delta_chunk_scan<<<dim3(p.v_heads, CD / SC), SCAN_T, SCAN_SMEM, a.stream>>>(p, chunks, (const float*)a.b[0].ptr, tp, pm, gc,
                                                                                   (float*)a.b[3].ptr, (float*)a.b[4].ptr);
        const cudaError_t e = cudaGetLastError();
        cudaFreeAsync(scratch, a.stream);
        ZCU_NEED(a, e == cudaSuccess, "delta_rule (chunked): launch failed: %s", cudaGetErrorString(e));
    }
    // tokens past the last whole chunk, the conv history and the kept state
    return launch_delta_recurrent(a, (uint32_t)chunks * CH, m);
}
