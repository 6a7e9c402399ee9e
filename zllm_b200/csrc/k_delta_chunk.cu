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
//
// The default form runs the scan's five contractions on the 5th-generation tensor cores (tcgen05, accumulators in
// tensor memory); the all-f32 CUDA-core pair above stays as variant ZCU_VARIANT_DELTA_CHUNK64_F32. Transposed, with
// the state column b as the MMA's row (lane) and every operand K-major:
//   [U'^T | Y'^T][b][t] = sum_a S^T[b][a] [K' ; Q'][t][a]      K'_t = e^{G_t} k_t,  Q'_t = e^{G_t} q_t / sqrt(d)
//   Delta^T[b][t]       = sum_s R^T[b][s] T'[t][s]              R = V - U'
//   O^T[b][t]           = Y'^T[b][t] + sum_s Delta^T[b][s] P[t][s]
//   S^T[b][a]           = e^{G_C} S^T[b][a] + sum_s Delta^T[b][s] Kd^T[a][s]      Kd_s = e^{G_C - G_s} k_s
// Every f32 operand x goes in as two bf16 terms hi + lo (16 bits of mantissa) and a product as hi hi + lo hi + hi lo,
// summed in f32 by the tensor cores: errors of 2^-16 relative per term instead of bf16's 2^-8.
//   delta_chunk_prep_tc   as delta_chunk_prep, but it leaves per (chunk, head) the B operands ready for the copy
//                         engine: 1024 rows of 64 bf16 - [K';Q'] hi, lo (two halves of the key dimension each), T' hi,
//                         lo, P hi, lo, Kd^T hi, lo - and e^{G_C}
//   delta_chunk_scan_tc   one CTA per value head, serial over chunks. Warp 8 issues the TMA tile loads (128-byte
//                         swizzle, a chunk ahead) and the MMAs; warps 0-7 (thread = state column b x one half of the
//                         other index) hold S in registers, move accumulators out of tensor memory (tcgen05.ld),
//                         do the f32 algebra between the contractions and write the next A operand (S^T, R^T,
//                         Delta^T as bf16 pairs) straight back into tensor memory (tcgen05.st): the A side never
//                         crosses shared memory.

#include "tc_util.cuh"
#include "tma_util.cuh"
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


// ---------------------------------------------------------------------------------------------- tensor-core form
constexpr int UNIT_ROWS = 1024, UNIT_BYTES = UNIT_ROWS * 128;   // rows of 64 bf16 per (chunk, head)
constexpr int R_KQ_HI = 0, R_KQ_LO = 256, R_T_HI = 512, R_T_LO = 576, R_P_HI = 640, R_P_LO = 704, R_KD_HI = 768, R_KD_LO = 896;

__device__ __forceinline__ void split8(const float* x, uint4& hi, uint4& lo) {
    tcu::split_pair(x[0], x[1], hi.x, lo.x);
    tcu::split_pair(x[2], x[3], hi.y, lo.y);
    tcu::split_pair(x[4], x[5], hi.z, lo.z);
    tcu::split_pair(x[6], x[7], hi.w, lo.w);
}

// grid (chunks of this pass, v_heads). tiles[(c * v_heads + j)][1024][64] bf16, ec[(c * v_heads + j)].
__global__ void __launch_bounds__(PREP_T) delta_chunk_prep_tc(PDeltaRule p, size_t tok_base, const float* __restrict__ conv,
                                                             const float* __restrict__ g, const float* __restrict__ beta,
                                                             unsigned char* __restrict__ tiles, float* __restrict__ ec) {
    extern __shared__ __align__(16) float sm[];
    float* Ks = sm;                 // [64][KP]
    float* Qs = Ks + CH * KP;       // [64][KP]
    float* As = Qs + CH * KP;       // [64][TP]
    float* Ps = As + CH * TP;       // [64][TP]
    float* Gs = Ps + CH * TP;       // [64] cumulative log-decay
    float* Bs = Gs + CH;            // [64]
    float* Es = Bs + CH;            // [64] e^{G_t}
    float* Ed = Es + CH;            // [64] e^{G_C - G_t}
    const int tid = threadIdx.x, c = blockIdx.x, j = blockIdx.y;
    const int kh = j % (int)p.k_heads, key_dim = (int)p.k_heads * CD;
    const size_t tok0 = tok_base + (size_t)c * CH;
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
    if (tid == 0) {
        float run = 0.f;
        for (int t = 0; t < CH; t++) {
            run = __fadd_rn(run, Gs[t]);
            Gs[t] = run;
        }
    }
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
    if (tid < CH) {
        Es[tid] = expf(Gs[tid]);
        Ed[tid] = expf(Gs[CH - 1] - Gs[tid]);
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int l = 0; l < 4; l++) {
            const int t = ty + 16 * i, s = tx + 16 * l;
            const float dec = s <= t ? expf(Gs[t] - Gs[s]) : 0.f;
            As[t * TP + s] = s < t ? Bs[t] * dec * kk[i][l] : 0.f;
            Ps[t * TP + s] = dec * qk[i][l] * scale;
        }
    __syncthreads();
    unsigned char* ut = tiles + unit * (size_t)UNIT_BYTES;
    if (tid < CH) {
        // (I + A)^-1 diag(beta), one column per thread (see delta_chunk_prep), written as bf16 pairs of terms
        float T[CH];
#pragma unroll
        for (int t = 0; t < CH; t++) {
            float acc = (t == tid) ? 1.f : 0.f;
#pragma unroll
            for (int s4 = 0; s4 < t; s4 += 4) {
                const float4 a4 = ld4(As + t * TP + s4);
                acc = fmaf(-a4.x, T[s4], acc);
                if (s4 + 1 < t) acc = fmaf(-a4.y, T[s4 + 1], acc);
                if (s4 + 2 < t) acc = fmaf(-a4.z, T[s4 + 2], acc);
                if (s4 + 3 < t) acc = fmaf(-a4.w, T[s4 + 3], acc);
            }
            T[t] = acc;
        }
        const float bc = Bs[tid];
#pragma unroll
        for (int t = 0; t < CH; t++) {
            const float v = T[t] * bc;
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            reinterpret_cast<unsigned short*>(ut + (size_t)(R_T_HI + t) * 128)[tid] = __bfloat16_as_ushort(h);
            reinterpret_cast<unsigned short*>(ut + (size_t)(R_T_LO + t) * 128)[tid] =
                __bfloat16_as_ushort(__float2bfloat16_rn(v - __bfloat162float(h)));
        }
        if (tid == 0) ec[unit] = Es[CH - 1];
    } else {
        const int e = tid - CH, ne = PREP_T - CH;
        float x[8];
        uint4 hi, lo;
        // [K' ; Q']: 128 rows x 16 groups of 8 key dimensions (8 groups per half)
        for (int i = e; i < 2 * CH * 16; i += ne) {
            const int r = i / 16, g8 = i % 16, t = r & (CH - 1);
            const float* src = (r < CH ? Ks : Qs) + t * KP + 8 * g8;
            const float f = r < CH ? Es[t] : Es[t] * scale;
            const float4 a = ld4(src), b = ld4(src + 4);
            x[0] = a.x * f, x[1] = a.y * f, x[2] = a.z * f, x[3] = a.w * f, x[4] = b.x * f, x[5] = b.y * f, x[6] = b.z * f, x[7] = b.w * f;
            split8(x, hi, lo);
            const size_t row = (size_t)(g8 / 8) * 128 + r, off = (size_t)(g8 % 8) * 16;
            *reinterpret_cast<uint4*>(ut + (R_KQ_HI + row) * 128 + off) = hi;
            *reinterpret_cast<uint4*>(ut + (R_KQ_LO + row) * 128 + off) = lo;
        }
        // Kd^T: 128 rows (key dimension a) x 8 groups of 8 tokens
        for (int i = e; i < CD * 8; i += ne) {
            const int a = i % CD, g8 = i / CD;
#pragma unroll
            for (int q = 0; q < 8; q++) x[q] = Ks[(8 * g8 + q) * KP + a] * Ed[8 * g8 + q];
            split8(x, hi, lo);
            *reinterpret_cast<uint4*>(ut + (size_t)(R_KD_HI + a) * 128 + g8 * 16) = hi;
            *reinterpret_cast<uint4*>(ut + (size_t)(R_KD_LO + a) * 128 + g8 * 16) = lo;
        }
        // P: 64 rows x 8 groups of 8 tokens
        for (int i = e; i < CH * 8; i += ne) {
            const int t = i / 8, g8 = i % 8;
            const float4 a = ld4(Ps + t * TP + 8 * g8), b = ld4(Ps + t * TP + 8 * g8 + 4);
            x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
            split8(x, hi, lo);
            *reinterpret_cast<uint4*>(ut + (size_t)(R_P_HI + t) * 128 + g8 * 16) = hi;
            *reinterpret_cast<uint4*>(ut + (size_t)(R_P_LO + t) * 128 + g8 * 16) = lo;
        }
    }
}

constexpr int TCS_WORKERS = 256, TCS_THREADS = 288, TCS_TMEM = 512;
constexpr int TCS_TILE_BYTES = UNIT_BYTES;                 // one unit's operands, in the scratch's row order
constexpr int TCS_SMEM = TCS_TILE_BYTES + 1024 + 128;
// tensor-memory columns
constexpr uint32_t TC_D1 = 0, TC_D2 = 128, TC_A1_HI = 192, TC_A1_LO = 256, TC_A2_HI = 320, TC_A2_LO = 352;

// 32 values of one lane as bf16 pairs of terms -> 16 + 16 columns of tensor memory.
__device__ __forceinline__ void st_split32(uint32_t t_hi, uint32_t t_lo, const float* x) {
    uint32_t hi[16], lo[16];
#pragma unroll
    for (int i = 0; i < 16; i++) tcu::split_pair(x[2 * i], x[2 * i + 1], hi[i], lo[i]);
    tcu::tmem_st8(t_hi, hi);
    tcu::tmem_st8(t_hi + 8, hi + 8);
    tcu::tmem_st8(t_lo, lo);
    tcu::tmem_st8(t_lo + 8, lo + 8);
}

// grid (v_heads), 288 threads.
__global__ void __launch_bounds__(TCS_THREADS, 1)
    delta_chunk_scan_tc(const __grid_constant__ CUtensorMap map, PDeltaRule p, size_t tok_base, int chunks, const float* __restrict__ conv,
                        const float* __restrict__ ec, float* __restrict__ state, float* __restrict__ out, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + TCS_TILE_BYTES);
    const uint32_t bar_b1 = tcu::smem_u32(bars), bar_b2 = bar_b1 + 8, bar_a = bar_b1 + 16, bar_mma = bar_b1 + 24;
    uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 4);  // [0] tensor-memory base, [1] abort flag
    volatile uint32_t* abort_flag = holder + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x;

    if (threadIdx.x == 0) {
        tcu::mbar_init(bar_b1, 1);
        tcu::mbar_init(bar_b2, 1);
        tcu::mbar_init(bar_a, TCS_WORKERS);
        tcu::mbar_init(bar_mma, 1);
        holder[1] = 0;
        tcu::mbar_init_fence();
    }
    if (warp == 8) tcu::tmem_alloc(tcu::smem_u32(holder), TCS_TMEM);
    tcu::fence_before();
    __syncthreads();
    tcu::fence_after();
    const uint32_t tmem = holder[0];
    bool gave_up = false;

    if (warp == 8) {
        // ---- copies and MMA issue: the whole warp runs the loop, one elected lane issues
        const uint32_t sb = tcu::smem_u32(smem);
        const uint32_t i128 = tcu::idesc_bf16_m128(128), i64 = tcu::idesc_bf16_m128(64);
        uint32_t ph_a = 0, ph_mma = 0, ph_b1 = 0, ph_b2 = 0;
        auto load_b1 = [&](int c) {   // [K';Q'] hi (two halves), lo (two halves): rows 0..511
            const int row0 = (c * (int)p.v_heads + j) * UNIT_ROWS;
            tcu::mbar_expect_tx(bar_b1, 4 * 16384);
#pragma unroll
            for (int i = 0; i < 4; i++) tcu::tma_load_2d(sb + i * 16384, &map, 0, row0 + 128 * i, bar_b1);
        };
        auto load_b2 = [&](int c) {   // T' hi lo, P hi lo, Kd^T hi, Kd^T lo: rows 512..1023
            const int row0 = (c * (int)p.v_heads + j) * UNIT_ROWS;
            tcu::mbar_expect_tx(bar_b2, 4 * 16384);
#pragma unroll
            for (int i = 4; i < 8; i++) tcu::tma_load_2d(sb + i * 16384, &map, 0, row0 + 128 * i, bar_b2);
        };
        if (tcu::elect_one()) {
            load_b1(0);
            load_b2(0);
        }
        __syncwarp();
        for (int c = 0; c < chunks; c++) {
            // 1. [U'^T | Y'^T] = S^T [K';Q']^T
            bool ok = tcu::mbar_wait(bar_a, ph_a, abort_flag) && tcu::mbar_wait(bar_b1, ph_b1, abort_flag);
            ph_a ^= 1u, ph_b1 ^= 1u;
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            tcu::fence_after();
            if (tcu::elect_one()) {
#pragma unroll
                for (int sp = 0; sp < 3; sp++) {
                    const uint32_t ta = tmem + (sp == 1 ? TC_A1_LO : TC_A1_HI);
                    const uint32_t tb = sb + (sp == 2 ? 32768u : 0u);
#pragma unroll
                    for (int kq = 0; kq < 8; kq++)
                        tcu::mma_bf16_ts(tmem + TC_D1, ta + 8u * kq, tcu::desc_sw128(tb + (kq / 4) * 16384u) + (uint64_t)(2 * (kq % 4)), i128,
                                         (sp | kq) != 0);
                }
                tcu::mma_commit(bar_mma);
            }
            __syncwarp();
            ok = tcu::mbar_wait(bar_mma, ph_mma, abort_flag);
            ph_mma ^= 1u;
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            if (c + 1 < chunks && tcu::elect_one()) load_b1(c + 1);   // the [K';Q'] tiles are free again
            __syncwarp();
            // 2. Delta^T = R^T T'^T
            ok = tcu::mbar_wait(bar_a, ph_a, abort_flag) && tcu::mbar_wait(bar_b2, ph_b2, abort_flag);
            ph_a ^= 1u, ph_b2 ^= 1u;
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            tcu::fence_after();
            if (tcu::elect_one()) {
#pragma unroll
                for (int sp = 0; sp < 3; sp++) {
                    const uint32_t ta = tmem + (sp == 1 ? TC_A2_LO : TC_A2_HI);
                    const uint32_t tb = sb + 65536u + (sp == 2 ? 8192u : 0u);
#pragma unroll
                    for (int kq = 0; kq < 4; kq++)
                        tcu::mma_bf16_ts(tmem + TC_D2, ta + 8u * kq, tcu::desc_sw128(tb) + (uint64_t)(2 * kq), i64, (sp | kq) != 0);
                }
                tcu::mma_commit(bar_mma);
            }
            __syncwarp();
            ok = tcu::mbar_wait(bar_mma, ph_mma, abort_flag);
            ph_mma ^= 1u;
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            // 3. O^T = Delta^T P^T (over the accumulator Delta left) and S^T's increment = Delta^T Kd
            ok = tcu::mbar_wait(bar_a, ph_a, abort_flag);
            ph_a ^= 1u;
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            tcu::fence_after();
            if (tcu::elect_one()) {
#pragma unroll
                for (int sp = 0; sp < 3; sp++) {
                    const uint32_t ta = tmem + (sp == 1 ? TC_A2_LO : TC_A2_HI);
                    const uint32_t tp = sb + 65536u + 16384u + (sp == 2 ? 8192u : 0u);
                    const uint32_t tk = sb + 65536u + 32768u + (sp == 2 ? 16384u : 0u);
#pragma unroll
                    for (int kq = 0; kq < 4; kq++) {
                        tcu::mma_bf16_ts(tmem + TC_D2, ta + 8u * kq, tcu::desc_sw128(tp) + (uint64_t)(2 * kq), i64, (sp | kq) != 0);
                        tcu::mma_bf16_ts(tmem + TC_D1, ta + 8u * kq, tcu::desc_sw128(tk) + (uint64_t)(2 * kq), i128, (sp | kq) != 0);
                    }
                }
                tcu::mma_commit(bar_mma);
            }
            __syncwarp();
            ok = tcu::mbar_wait(bar_mma, ph_mma, abort_flag);
            ph_mma ^= 1u;
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            if (c + 1 < chunks && tcu::elect_one()) load_b2(c + 1);
            __syncwarp();
        }
        if (gave_up && lane == 0)  // copies still in flight must land before the CTA's shared memory is given back
            for (int i = 0; i < 200; i++) __nanosleep(1000);
    } else {
        // ---- the algebra between the contractions: thread = (state column b, half h)
        const int quad = warp & 3, h = warp >> 2, b = quad * 32 + lane;
        const uint32_t tl = tmem + ((uint32_t)(quad * 32) << 16);
        const int key_dim = (int)p.k_heads * CD;
        const size_t s0 = (size_t)j * CD * CD;
        const size_t out_row = (size_t)p.v_heads * CD;
        uint32_t ph_mma = 0;
        float S[64];   // S^T[b][a], a = 64 h + i
#pragma unroll
        for (int i = 0; i < 64; i++) S[i] = state[s0 + (size_t)(64 * h + i) * CD + b];
        st_split32(tl + TC_A1_HI + 32 * h, tl + TC_A1_LO + 32 * h, S);
        st_split32(tl + TC_A1_HI + 32 * h + 16, tl + TC_A1_LO + 32 * h + 16, S + 32);
        tcu::tmem_st_wait();
        tcu::fence_before();
        tcu::mbar_arrive(bar_a);
        for (int c = 0; c < chunks; c++) {
            const size_t tok0 = tok_base + (size_t)c * CH + 32 * h;
            float v[32], y[32];
            uint32_t r[32];
            const float* vp = conv + tok0 * p.conv_stride + 2 * (size_t)key_dim + (size_t)j * CD + b;
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = vp[(size_t)i * p.conv_stride];
            const float eC = ec[(size_t)c * p.v_heads + j];
            // 1 -> 2: R^T = V^T - U'^T; keep Y'^T
            if (!__all_sync(0xffffffffu, tcu::mbar_wait(bar_mma, ph_mma, abort_flag))) {
                gave_up = true;
                break;
            }
            ph_mma ^= 1u;
            tcu::fence_after();
            tcu::tmem_ld16(tl + TC_D1 + 32 * h, r);
            tcu::tmem_ld16(tl + TC_D1 + 32 * h + 16, r + 16);
            tcu::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] -= __uint_as_float(r[i]);
            st_split32(tl + TC_A2_HI + 16 * h, tl + TC_A2_LO + 16 * h, v);
            tcu::tmem_ld16(tl + TC_D1 + 64 + 32 * h, r);
            tcu::tmem_ld16(tl + TC_D1 + 64 + 32 * h + 16, r + 16);
            tcu::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) y[i] = __uint_as_float(r[i]);
            tcu::tmem_st_wait();
            tcu::fence_before();
            tcu::mbar_arrive(bar_a);
            // 2 -> 3: Delta^T as the next A operand
            if (!__all_sync(0xffffffffu, tcu::mbar_wait(bar_mma, ph_mma, abort_flag))) {
                gave_up = true;
                break;
            }
            ph_mma ^= 1u;
            tcu::fence_after();
            tcu::tmem_ld16(tl + TC_D2 + 32 * h, r);
            tcu::tmem_ld16(tl + TC_D2 + 32 * h + 16, r + 16);
            tcu::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
            st_split32(tl + TC_A2_HI + 16 * h, tl + TC_A2_LO + 16 * h, v);
            tcu::tmem_st_wait();
            tcu::fence_before();
            tcu::mbar_arrive(bar_a);
            // 3 -> next chunk: the outputs, and the state as the next chunk's A operand
            if (!__all_sync(0xffffffffu, tcu::mbar_wait(bar_mma, ph_mma, abort_flag))) {
                gave_up = true;
                break;
            }
            ph_mma ^= 1u;
            tcu::fence_after();
            tcu::tmem_ld16(tl + TC_D2 + 32 * h, r);
            tcu::tmem_ld16(tl + TC_D2 + 32 * h + 16, r + 16);
            tcu::tmem_ld_wait();
            float* op = out + tok0 * out_row + (size_t)j * CD + b;
#pragma unroll
            for (int i = 0; i < 32; i++) op[(size_t)i * out_row] = y[i] + __uint_as_float(r[i]);
#pragma unroll
            for (int q = 0; q < 2; q++) {
                tcu::tmem_ld16(tl + TC_D1 + 64 * h + 32 * q, r);
                tcu::tmem_ld16(tl + TC_D1 + 64 * h + 32 * q + 16, r + 16);
                tcu::tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i++) S[32 * q + i] = fmaf(eC, S[32 * q + i], __uint_as_float(r[i]));
            }
            st_split32(tl + TC_A1_HI + 32 * h, tl + TC_A1_LO + 32 * h, S);
            st_split32(tl + TC_A1_HI + 32 * h + 16, tl + TC_A1_LO + 32 * h + 16, S + 32);
            tcu::tmem_st_wait();
            tcu::fence_before();
            tcu::mbar_arrive(bar_a);
        }
        if (!gave_up) {
#pragma unroll
            for (int i = 0; i < 64; i++) state[s0 + (size_t)(64 * h + i) * CD + b] = S[i];
        }
    }
    if (gave_up && status) atomicExch(status, 2);
    tcu::fence_before();
    __syncthreads();
    if (warp == 8) {
        tcu::fence_after();
        tcu::tmem_free(tmem, TCS_TMEM);
    }
}

constexpr int PREP_TC_SMEM = (2 * CH * KP + 2 * CH * TP + 4 * CH) * 4;

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
    const float *conv = (const float*)a.b[0].ptr, *g = (const float*)a.b[1].ptr, *beta = (const float*)a.b[2].ptr;
    float *state = (float*)a.b[3].ptr, *out = (float*)a.b[4].ptr;
    if (chunks > 0 && a.variant == ZCU_VARIANT_DELTA_CHUNK64_F32) {
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
        delta_chunk_prep<<<dim3(chunks, p.v_heads), PREP_T, PREP_SMEM, a.stream>>>(p, conv, g, beta, tp, pm, gc);
        delta_chunk_scan<<<dim3(p.v_heads, CD / SC), SCAN_T, SCAN_SMEM, a.stream>>>(p, chunks, conv, tp, pm, gc, state, out);
        const cudaError_t e = cudaGetLastError();
        cudaFreeAsync(scratch, a.stream);
        ZCU_NEED(a, e == cudaSuccess, "delta_rule (chunked): launch failed: %s", cudaGetErrorString(e));
    } else if (chunks > 0) {
        // passes of at most 256 MB of prepared operands (128 KB per chunk and head)
        const size_t per_chunk = (size_t)p.v_heads * (UNIT_BYTES + 256);
        const int pass_max = (int)(((size_t)256 << 20) / per_chunk) > 0 ? (int)(((size_t)256 << 20) / per_chunk) : 1;
        const int pass_chunks = chunks < pass_max ? chunks : pass_max;
        const size_t pass_units = (size_t)pass_chunks * p.v_heads;
        unsigned char* scratch = nullptr;
        const size_t bytes = pass_units * UNIT_BYTES + pass_units * sizeof(float);
        if (cudaMallocAsync((void**)&scratch, bytes, a.stream) != cudaSuccess) {
            cudaGetLastError();
            ZCU_NEED(a, false, "delta_rule (chunked): no memory for %zu bytes of chunk operands", bytes);
        }
        float* ec = reinterpret_cast<float*>(scratch + pass_units * UNIT_BYTES);
        CUtensorMap map;
        const bool map_ok = tma::bf16_rows64_sw128(&map, scratch, pass_units * UNIT_ROWS, 128);
        cudaError_t e = cudaSuccess;
        if (map_ok) {
            cudaFuncSetAttribute(delta_chunk_prep_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_TC_SMEM);
            cudaFuncSetAttribute(delta_chunk_scan_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, TCS_SMEM);
            for (int c0 = 0; c0 < chunks && e == cudaSuccess; c0 += pass_chunks) {
                const int n = chunks - c0 < pass_chunks ? chunks - c0 : pass_chunks;
                delta_chunk_prep_tc<<<dim3(n, p.v_heads), PREP_T, PREP_TC_SMEM, a.stream>>>(p, (size_t)c0 * CH, conv, g, beta, scratch, ec);
                delta_chunk_scan_tc<<<p.v_heads, TCS_THREADS, TCS_SMEM, a.stream>>>(map, p, (size_t)c0 * CH, n, conv, ec, state, out, a.status);
                e = cudaGetLastError();
            }
        }
        cudaFreeAsync(scratch, a.stream);
        ZCU_NEED(a, map_ok, "delta_rule (chunked): the driver refused a tensor map over %zu rows", pass_units * UNIT_ROWS);
        ZCU_NEED(a, e == cudaSuccess, "delta_rule (chunked): launch failed: %s", cudaGetErrorString(e));
    }
    // tokens past the last whole chunk, the conv history and the kept state
    return launch_delta_recurrent(a, (uint32_t)chunks * CH, m);
}
