// The decode-attention fast path (f16 cache) and the merge of its partials, written for virtual blocks (vblock.cuh);
// the kernels of k_attn.cu map one CUDA block to each.
#pragma once

#include <cfloat>
#include <cuda_fp16.h>

#include "tma_util.cuh"
#include "vblock.cuh"
#include "zcu_internal.h"

#ifdef ZCU_TRACE
__device__ unsigned long long g_at_trace[1024 * 8];
#define ATRACE(i)                                                                   \
    do {                                                                            \
        const unsigned cta__ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x; \
        if (threadIdx.x == 0 && cta__ < 1024) {                                     \
            unsigned long long t__;                                                 \
            asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t__));                \
            g_at_trace[cta__ * 8 + (i)] = t__;                                      \
        }                                                                           \
    } while (0)
#else
#define ATRACE(i) do {} while (0)
#endif

namespace attn {

// ---- the fast path: f16 cache, GQA group <= 4, head_dim 64 or 128; 128 cache positions per CTA.
// The cache and the queries are read past L1 (ld.global.cg): the newest row of the cache and the queries were
// written by another SM just before (the kernel may overlap the end of its producer as a programmatic dependent).
// Scores: 8 threads per key, each with its hd/8 dims of the group's queries in registers, so K is read
// with 16-byte loads and no shared-memory traffic; the 8 partial dots meet by shuffles. Softmax: one warp
// per head. Sum of exp * v: 16 threads per key (8 dims each, 16-byte V loads), 16 key groups per CTA
// that meet in shared memory in group order.
constexpr int AF_KEYS = 128;
constexpr int AF_THREADS = 256;

// Shared memory of one virtual block: scores [GROUP_CAP][128], statistics, then one region that first holds the
// block's values (128 keys x hd halves, each thread's own 16-byte pieces, brought in by cp.async while the
// scores are computed) and afterwards the [8 warps][group][HD] partial sums.
__host__ __device__ constexpr size_t attn_fast_smem(int group_cap, int group, int hd) {
    const size_t pv = (size_t)(AF_THREADS / 32) * group * hd * sizeof(float), vals = (size_t)AF_KEYS * hd * 2;
    return ((size_t)group_cap * AF_KEYS + 2 * group_cap + 8) * sizeof(float) + (pv > vals ? pv : vals);
}

template <int HD, int GROUP_CAP>
__device__ __forceinline__ void attn_split_fast_body(const VBlock& vb, const PAttention& p, const float* __restrict__ qg,
                                                     const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                     float* __restrict__ part, const PStep* __restrict__ step,
                                                     const uint32_t* __restrict__ seq_pos) {
    constexpr int DPT = HD / 8;     // dims per thread in the score phase
    constexpr int KPP = AF_THREADS / 8;  // keys per pass
    constexpr int PASSES = AF_KEYS / KPP;
    float (*sc)[AF_KEYS] = reinterpret_cast<float (*)[AF_KEYS]>(vb.smem);
    float* stat = reinterpret_cast<float*>(vb.smem) + GROUP_CAP * AF_KEYS;
    float* pv = stat + 2 * GROUP_CAP + 8;  // [8 warps][group][HD]; the offset keeps it 16-byte aligned
    const int tid = vb.tid, lane = tid & 31, warp = tid >> 5;
    const int g = vb.x, b = vb.y, t = vb.z;
    const int group = (int)(p.heads / p.kv_heads);
    const int row = (int)p.row0 + t;
    const size_t seq_off = (size_t)row * p._pad[0];
    const int keys = (seq_pos ? (int)seq_pos[row] : (int)step->pos0 + row) + 1;
    const int k0 = b * AF_KEYS;
    const size_t kv_stride = (size_t)p.kv_heads * HD;
    const int q_head = p.gated ? 2 * HD : HD;
    const int n = min(AF_KEYS, keys - min(keys, k0));

    // ---- scores
    const int kl = tid >> 3, sl = tid & 7;
    float q[GROUP_CAP][DPT];
#pragma unroll
    for (int h = 0; h < GROUP_CAP; h++) {
        const float* qp = qg + (size_t)row * p.q_row + (size_t)(g * group + min(h, group - 1)) * q_head + sl * DPT;
#pragma unroll
        for (int d = 0; d < DPT; d += 4) {
            const float4 v = __ldcg(reinterpret_cast<const float4*>(qp + d));
            q[h][d] = v.x; q[h][d + 1] = v.y; q[h][d + 2] = v.z; q[h][d + 3] = v.w;
        }
    }
    uint4 kraw[PASSES][DPT / 8];
#pragma unroll
    for (int ps = 0; ps < PASSES; ps++) {
        const int key = k0 + ps * KPP + kl;
        const __half* kp = kc + seq_off + (size_t)min(key, keys - 1) * kv_stride + (size_t)g * HD + sl * DPT;
#pragma unroll
        for (int c = 0; c < DPT / 8; c++) kraw[ps][c] = __ldcg(reinterpret_cast<const uint4*>(kp) + c);
    }
    // the values do not depend on the scores: their loads are in flight while the scores are computed
    constexpr int TPK = HD / 8;            // threads per key in the value phase
    constexpr int KG = AF_THREADS / TPK;   // key groups
    constexpr int KPT = AF_KEYS / KG;      // keys per thread
    const int kg = tid / TPK, dl = tid % TPK;
    // piece i of this thread sits at (i * 256 + tid) * 16 bytes: only the thread that copied a piece reads it
    const uint32_t vslot = (uint32_t)__cvta_generic_to_shared(pv) + (uint32_t)tid * 16u;
#pragma unroll
    for (int i = 0; i < KPT; i++) {
        const int key = k0 + kg + KG * i;
        const __half* src = vc + seq_off + (size_t)min(key, keys - 1) * kv_stride + (size_t)g * HD + 8 * dl;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(vslot + (uint32_t)i * AF_THREADS * 16u), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
#pragma unroll
    for (int ps = 0; ps < PASSES; ps++) {
        const int key = k0 + ps * KPP + kl;
        float dot[GROUP_CAP];
#pragma unroll
        for (int h = 0; h < GROUP_CAP; h++) dot[h] = 0.f;
#pragma unroll
        for (int c = 0; c < DPT / 8; c++) {
            const __half2* hp = reinterpret_cast<const __half2*>(&kraw[ps][c]);
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 kk = __half22float2(hp[e]);
#pragma unroll
                for (int h = 0; h < GROUP_CAP; h++) {
                    dot[h] = __fmaf_rn(q[h][8 * c + 2 * e], kk.x, dot[h]);
                    dot[h] = __fmaf_rn(q[h][8 * c + 2 * e + 1], kk.y, dot[h]);
                }
            }
        }
#pragma unroll
        for (int h = 0; h < GROUP_CAP; h++) {
            float v = dot[h];
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 4));
            if (sl == 0 && h < group) sc[h][ps * KPP + kl] = key < keys ? v * p.scale : -FLT_MAX;
        }
    }
    vb.sync();

    // ---- block softmax: warp h takes head h, four keys per lane
    if (warp < group) {
        float s[4], mx = -FLT_MAX;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            s[i] = lane + 32 * i < n ? sc[warp][lane + 32 * i] : -FLT_MAX;
            mx = fmaxf(mx, s[i]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float e = (lane + 32 * i < n && s[i] != -FLT_MAX) ? expf(s[i] - mx) : 0.f;
            sc[warp][lane + 32 * i] = e;
            sum = __fadd_rn(sum, e);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
        if (lane == 0) {
            stat[2 * warp] = mx;
            stat[2 * warp + 1] = sum;
        }
    }
    vb.sync();

    // ---- sum exp * v: thread (key group kg of 16, dims 8 dl .. 8 dl + 7)
    float acc[GROUP_CAP][8];
#pragma unroll
    for (int h = 0; h < GROUP_CAP; h++)
#pragma unroll
        for (int d = 0; d < 8; d++) acc[h][d] = 0.f;
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < KPT; i++) {
        const int ki = kg + KG * i;
        if (ki < n) {
            uint4 vpiece;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                         : "=r"(vpiece.x), "=r"(vpiece.y), "=r"(vpiece.z), "=r"(vpiece.w)
                         : "r"(vslot + (uint32_t)i * AF_THREADS * 16u));
            const __half2* hp = reinterpret_cast<const __half2*>(&vpiece);
            float vv[8];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float2 f = __half22float2(hp[e]);
                vv[2 * e] = f.x;
                vv[2 * e + 1] = f.y;
            }
#pragma unroll
            for (int h = 0; h < GROUP_CAP; h++) {
                const float w = sc[h < group ? h : 0][ki];
#pragma unroll
                for (int d = 0; d < 8; d++) acc[h][d] = __fmaf_rn(w, vv[d], acc[h][d]);
            }
        }
    }
    // key groups of one warp first (shuffles, fixed order), then the warps through shared memory
    constexpr int GPW = 32 / TPK;  // key groups per warp
#pragma unroll
    for (int h = 0; h < GROUP_CAP; h++)
#pragma unroll
        for (int d = 0; d < 8; d++) {
            float v = acc[h][d];
#pragma unroll
            for (int o = TPK; o < 32; o <<= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
            acc[h][d] = v;
        }
    vb.sync();  // every thread is done with its values: the region now takes the warps' partial sums
    if (lane < TPK) {
#pragma unroll
        for (int h = 0; h < GROUP_CAP; h++)
            if (h < group) {
                float* dst = pv + ((size_t)warp * group + h) * HD + 8 * lane;
                *reinterpret_cast<float4*>(dst) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
            }
    }
    (void)GPW;
    vb.sync();
    for (int i = tid; i < group * HD; i += AF_THREADS) {
        const int h = i / HD, d = i % HD;
        float o = 0.f;
#pragma unroll
        for (int wv = 0; wv < AF_THREADS / 32; wv++) o = __fadd_rn(o, pv[((size_t)wv * group + h) * HD + d]);
        const int head = g * group + h;
        const size_t base = (((size_t)t * p.heads + head) * p.max_blocks + b) * (HD + 2);
        part[base + 2 + d] = o;
        if (d == 0) {
            part[base] = stat[2 * h];
            part[base + 1] = stat[2 * h + 1];
        }
    }
}

// ---- the block on the f16 tensor cores (mma.sync.m16n8k16, f32 accumulate). The cache holds f16 values, which the
// tensor cores multiply exactly; the f32 queries and probabilities are split into two f16 terms each
// (x = hi + lo, |x - hi - lo| <= 2^-22 |x|), which occupy rows 0-3 (hi of the group's heads) and 4-7 (lo) of the
// 16-row A operand; the two partial results are added afterwards.
//
// Each of the 8 warps owns 16 of the block's 128 keys from start to end and meets the others only once:
//   scores    A = Q [16 x dims] from fragments prepared once per CTA, B = K^T through ldmatrix.x4 (16 keys x 16 dims
//             per instruction) straight out of the staged tile;
//   softmax   over the warp's 16 keys, in registers (two shuffles per head for the maximum, two for the sum);
//   exp * v   A = the probabilities, taken from the score accumulators' registers (the C layout of the score MMA
//             is the A layout of this one), B = V through ldmatrix.x4.trans, 16 dims per instruction;
//   then the warp leaves {max, sum, o[dims]} of its keys in shared memory (in the place of its own K rows, which
//   nobody else reads) and, after the CTA's only barrier, the eight are merged the way attn_combine merges blocks.
// A warp waits only for its own rows of K and V (its threads copy exactly those), so the arithmetic of one warp
// overlaps the copies of another. K and V tiles: rows padded to head_dim * 2 + 16 bytes (conflict-free ldmatrix).
constexpr int AM_THREADS = 256;
__host__ __device__ constexpr size_t attn_mma_smem(int hd) {
    return (size_t)2 * AF_KEYS * (hd * 2 + 16) + (size_t)(hd / 16) * 32 * 8 + (8 * 4 * 2 + 8 * 4 + 4) * sizeof(float);
}

__device__ __forceinline__ void mma_f16_16816(float* c, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // rows 8-15 of A are zero (a1 = a3 = 0)
    asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
// (hi, hi) or (lo, lo) halves of two floats, as one A-operand register
__device__ __forceinline__ uint32_t split_pair(float x0, float x1, bool low) {
    __half h0 = __float2half_rn(x0), h1 = __float2half_rn(x1);
    if (low) {
        h0 = __float2half_rn(x0 - __half2float(h0));
        h1 = __float2half_rn(x1 - __half2float(h1));
    }
    return (uint32_t)__half_as_ushort(h0) | ((uint32_t)__half_as_ushort(h1) << 16);
}

template <int HD, bool PDL = false>
__device__ __forceinline__ void attn_split_mma_body(unsigned char* smem, const PAttention& p, const float* __restrict__ qg,
                                                    const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                    float* __restrict__ part, const PStep* __restrict__ step,
                                                    const uint32_t* __restrict__ seq_pos, int g_kv, int b, int t,
                                                    int* __restrict__ status = nullptr) {
    constexpr int RS = HD * 2 + 16;              // bytes between the rows of a staged tile
    constexpr int KSTEPS = HD / 16;              // k-steps of the score product
    constexpr int CPR = HD / 8;                  // 16-byte pieces per cache row
    constexpr int PIECES = 16 * CPR / 32;        // pieces of the warp's 16 rows per lane
    unsigned char* Kt = smem;
    unsigned char* Vt = smem + (size_t)AF_KEYS * RS;
    uint2* qf = reinterpret_cast<uint2*>(Vt + (size_t)AF_KEYS * RS);   // [KSTEPS][32]: the lanes' A registers per k-step
    float* ml = reinterpret_cast<float*>(qf + KSTEPS * 32);            // [8 warps][4 heads] {max, sum}
    const uint32_t kt_s = (uint32_t)__cvta_generic_to_shared(Kt), vt_s = (uint32_t)__cvta_generic_to_shared(Vt);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;      // fragment coordinates
    const int group = (int)(p.heads / p.kv_heads);
    const int row = (int)p.row0 + t;
    const size_t seq_off = (size_t)row * p._pad[0];
    int keys = (seq_pos ? (int)seq_pos[row] : (int)step->pos0 + row) + 1;
    // the launch covers gridDim.y blocks of the cache: a step past them is an error of the caller, reported, not followed
    if (keys > (int)gridDim.y * AF_KEYS) {
        keys = (int)gridDim.y * AF_KEYS;
        if (tid == 0 && status) atomicExch(status, 6);
    }
    const int k0 = b * AF_KEYS;
    const size_t kv_stride = (size_t)p.kv_heads * HD;
    const int q_head = p.gated ? 2 * HD : HD;
    const int r0 = 16 * warp;                    // this warp's rows of the tiles
    // Launched as a programmatic dependent: the queries and the step's new cache rows come from the kernel before.
    // The step's new rows start at the sequence's position (a sequence's own, or the step's first); a block that
    // ends before them holds only rows of earlier steps, and its copies may start while that kernel still runs.
    const int first_new = seq_pos ? (int)seq_pos[row] : (int)step->pos0;
    const bool early = PDL && k0 + AF_KEYS <= first_new;
    if (PDL) asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // (what follows waits for this kernel's end itself)
    if (PDL && !early) asm volatile("griddepcontrol.wait;\n" ::: "memory");

    // ---- this warp's rows of K, then of V, on their way (two groups: the scores need only the first)
    ATRACE(1);
    // (lane l copies piece l % CPR of rows r0 + l / CPR + (32 / CPR) i; a row past the sequence's last key repeats that
    // key: the offsets are clamped, not the addresses recomputed)
    {
        constexpr int RPI = 32 / CPR;   // rows a warp covers per instruction
        const int row0 = r0 + lane / CPR, piece = lane % CPR;
        const size_t col = seq_off + (size_t)g_kv * HD + 8 * piece;
        const int last = keys - 1 - k0;   // the block's last valid row
        const uint32_t dst0 = (uint32_t)row0 * RS + 16u * piece;
#pragma unroll
        for (int i = 0; i < PIECES; i++) {
            const size_t src = col + (size_t)(k0 + min(row0 + RPI * i, last)) * kv_stride;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(kt_s + dst0 + (uint32_t)(RPI * i) * RS), "l"(kc + src) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
#pragma unroll
        for (int i = 0; i < PIECES; i++) {
            const size_t src = col + (size_t)(k0 + min(row0 + RPI * i, last)) * kv_stride;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(vt_s + dst0 + (uint32_t)(RPI * i) * RS), "l"(vc + src) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    }
    if (early) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    // ---- the group's queries as A fragments: entry (k-step, lane) = {a0, a2} of that lane (head g & 3; hi for g < 4,
    //      lo for g >= 4; rows 8-15 of A stay zero). One entry per thread for head_dim 128.
    for (int e = tid; e < KSTEPS * 32; e += AM_THREADS) {
        const int ks = e >> 5, ln = e & 31, gg = ln >> 2, tt = ln & 3;
        const float* qp = qg + (size_t)row * p.q_row + (size_t)(g_kv * group + min(gg & 3, group - 1)) * q_head + 16 * ks + 2 * tt;
        const float2 qa = __ldcg(reinterpret_cast<const float2*>(qp)), qb = __ldcg(reinterpret_cast<const float2*>(qp + 8));
        qf[e] = make_uint2(split_pair(qa.x, qa.y, gg >= 4), split_pair(qb.x, qb.y, gg >= 4));
    }
    __syncthreads();   // the query fragments (the tiles are private to their warps)
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    __syncwarp();
    ATRACE(2);

    // ---- scores of the warp's 16 keys for the group's heads
    float c[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; nb++) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.f;
    {
        // ldmatrix.x4: lanes 0-7 name the rows of matrix 0 (keys 0-7, dims 16 ks ..+7), 8-15 matrix 1 (keys 0-7, dims
        // +8..+15), 16-23 matrix 2 (keys 8-15, low dims), 24-31 matrix 3: the four B registers of the two key blocks
        const uint32_t krow = kt_s + (uint32_t)(r0 + (lane & 7) + 8 * (lane >> 4)) * RS + 16u * ((lane >> 3) & 1);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            const uint2 a = qf[ks * 32 + lane];
            uint32_t b0, b1, b2, b3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(krow + 32u * ks));
            mma_f16_16816(c[0], a.x, a.y, b0, b1);
            mma_f16_16816(c[1], a.x, a.y, b2, b3);
        }
    }
    ATRACE(3);
    // hi rows (lanes g < 4) + lo rows (lanes g + 4 = lane + 16): both lanes then hold the head's scores of keys
    // r0 + 8 nb + 2 tq, + 1
    float s[4];
#pragma unroll
    for (int nb = 0; nb < 2; nb++)
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const float v = __fadd_rn(c[nb][i], __shfl_xor_sync(0xffffffffu, c[nb][i], 16));
            s[2 * nb + i] = k0 + r0 + 8 * nb + 2 * tq + i < keys ? v * p.scale : -FLT_MAX;
        }
    // ---- softmax over the warp's 16 keys (the four lanes tq of a head)
    float mx = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    float pr[4], sum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) pr[i] = s[i] != -FLT_MAX ? expf(s[i] - mx) : 0.f;
    sum = __fadd_rn(__fadd_rn(pr[0], pr[1]), __fadd_rn(pr[2], pr[3]));
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 1));
    sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 2));
    if (g < group && tq == 0) {
        ml[(warp * 4 + g) * 2] = mx;
        ml[(warp * 4 + g) * 2 + 1] = sum;
    }
    ATRACE(4);
    // ---- sum exp * v over the warp's 16 keys: one k-step; the probabilities go from the score accumulators'
    //      registers into the A operand (hi in lanes g < 4, lo in lanes g >= 4)
    const uint32_t pa0 = split_pair(pr[0], pr[1], g >= 4), pa2 = split_pair(pr[2], pr[3], g >= 4);
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncwarp();
    ATRACE(5);
    constexpr int PVS = HD + 8;   // floats between the heads' rows of a warp's result (the four heads' stores hit different banks)
    float* pv = reinterpret_cast<float*>(Kt + (size_t)r0 * RS);   // [4 heads][PVS], in the place of this warp's K rows
    __syncwarp();                                                  // every lane has read its K fragments
    {
        // ldmatrix.x4.trans: lanes 0-15 name the 16 key rows at dims d .. d+7, lanes 16-31 the same rows at d+8 .. d+15
        const uint32_t vrow = vt_s + (uint32_t)(r0 + (lane & 15)) * RS + 16u * (lane >> 4);
#pragma unroll
        for (int nb = 0; nb < HD / 16; nb++) {
            uint32_t b0, b1, b2, b3;
            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(b0), "=r"(b1), "=r"(b2), "=r"(b3) : "r"(vrow + 32u * nb));
            float o0[4] = {0.f, 0.f, 0.f, 0.f}, o1[4] = {0.f, 0.f, 0.f, 0.f};
            mma_f16_16816(o0, pa0, pa2, b0, b1);
            mma_f16_16816(o1, pa0, pa2, b2, b3);
            const float v00 = __fadd_rn(o0[0], __shfl_xor_sync(0xffffffffu, o0[0], 16)), v01 = __fadd_rn(o0[1], __shfl_xor_sync(0xffffffffu, o0[1], 16));
            const float v10 = __fadd_rn(o1[0], __shfl_xor_sync(0xffffffffu, o1[0], 16)), v11 = __fadd_rn(o1[1], __shfl_xor_sync(0xffffffffu, o1[1], 16));
            if (g < group) {
                *reinterpret_cast<float2*>(pv + g * PVS + 16 * nb + 2 * tq) = make_float2(v00, v01);
                *reinterpret_cast<float2*>(pv + g * PVS + 16 * nb + 8 + 2 * tq) = make_float2(v10, v11);
            }
        }
    }
    __syncthreads();
    // ---- the eight warps' results merged in warp order (attn_combine's arithmetic): the block's partial. The
    //      weight of a warp's result, exp(its maximum - the block's), is the same for every dim of a head: the
    //      first 32 threads compute the 8 x 4 weights once.
    float* wts = ml + 8 * 4 * 2;   // [8 warps][4 heads], then the heads' maxima [4]
    if (tid < 32) {
        const int w = tid >> 2, h = tid & 3;
        float M = -FLT_MAX;
#pragma unroll
        for (int ww = 0; ww < 8; ww++) M = fmaxf(M, ml[(ww * 4 + h) * 2]);
        const float mw = ml[(w * 4 + h) * 2];
        wts[w * 4 + h] = mw != -FLT_MAX ? expf(mw - M) : 0.f;
        if (w == 0) wts[32 + h] = M;
    }
    __syncthreads();
    for (int e = tid; e < group * HD; e += AM_THREADS) {
        const int h = e / HD, d = e % HD;
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) o = __fmaf_rn(reinterpret_cast<const float*>(Kt + (size_t)16 * w * RS)[h * PVS + d], wts[w * 4 + h], o);
        const int head = g_kv * group + h;
        const size_t base = (((size_t)t * p.heads + head) * p.max_blocks + b) * (HD + 2);
        part[base + 2 + d] = o;
        if (d == 0) {
            float L = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) L = __fmaf_rn(ml[(w * 4 + h) * 2 + 1], wts[w * 4 + h], L);
            part[base] = wts[32 + h];
            part[base + 1] = L;
        }
    }
    ATRACE(6);
}

// grid (heads, rows). Merges the blocks' partials (src/kernels/attn_combine.wgsl):
//   M = max m_b,  L = sum l_b e^(m_b - M),  o = sum o_b e^(m_b - M) / L,  times sigmoid(gate) when gated.
// Bindings: qg, part, out, step (+ per-row positions for batched sequences). `kb`: cache positions per block.
// AC_THREADS threads = AC_THREADS / 128 (or / 256) lanes of blocks per dim: thread (q, d) owns blocks q, q + Q, ...
// of dim d. Everything a thread needs from memory is asked for before anything is computed (the block maxima and
// sums by the first `blocks` threads, the thread's AC_KEEP first partial outputs into registers), so the kernel
// pays one round trip to L2, not one per phase. Sums run in a fixed order: a lane's blocks in block order, then
// the lanes in lane order.
constexpr int AC_MAX_BLOCKS = 4096;
constexpr int AC_THREADS = 512;
constexpr int AC_KEEP = 20;
__host__ __device__ constexpr size_t attn_combine_smem(int max_blocks) { return ((size_t)2 * max_blocks + 64 + 2 * AC_THREADS) * sizeof(float); }

__device__ __forceinline__ void attn_combine_body(const VBlock& vb, const PAttention& p, const float* __restrict__ qg,
                                                  const float* __restrict__ part, float* __restrict__ out,
                                                  const PStep* __restrict__ step, const uint32_t* __restrict__ seq_pos,
                                                  int kb, int* __restrict__ status, const PeerUse* __restrict__ pu = nullptr) {
    float* wsm = reinterpret_cast<float*>(vb.smem);  // [blocks] weights, [blocks] weighted sums, [64] scratch, [AC_THREADS] float2
    const int tid = vb.tid, lane = tid & 31, warp = tid >> 5, h = vb.x, t = vb.y;
    const int hd = (int)p.head_dim;
    const int row = (int)p.row0 + t;
    const int keys = (seq_pos ? (int)seq_pos[row] : (int)step->pos0 + row) + 1;
    int blocks = (keys + kb - 1) / kb;
    // the partials hold p.max_blocks blocks per head: a step past that is an error of the caller, reported, not followed
    const int cap = (int)p.max_blocks;
    if (blocks > cap) {
        blocks = cap;
        if (tid == 0 && status) atomicExch(status, 6);
    }
    float* lsm = wsm + cap;
    float* red = lsm + cap;
    float2* lanes_sm = reinterpret_cast<float2*>(red + 64);
    const size_t base0 = ((size_t)t * p.heads + h) * p.max_blocks * (hd + 2);
    const size_t bs = (size_t)hd + 2;
    const int dims = hd <= 128 ? 128 : 256;
    const int Q = AC_THREADS / dims;                 // lanes of blocks
    const int d = tid % dims, q = tid / dims;
    // ---- every load first
    float keep[AC_KEEP];
#pragma unroll
    for (int i = 0; i < AC_KEEP; i++) {
        const int b = q + Q * i;
        keep[i] = (b < blocks && d < hd) ? __ldcg(part + base0 + b * bs + 2 + d) : 0.f;
    }
    float mx = -FLT_MAX;
    for (int b = tid; b < blocks; b += AC_THREADS) {
        const float2 ml = __ldcg(reinterpret_cast<const float2*>(part + base0 + b * bs));
        wsm[b] = ml.x;
        lsm[b] = ml.y;
        mx = fmaxf(mx, ml.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) red[warp] = mx;
    vb.sync();
    mx = red[0];
#pragma unroll
    for (int wv = 1; wv < AC_THREADS / 32; wv++) mx = fmaxf(mx, red[wv]);
    vb.sync();
    for (int b = tid; b < blocks; b += AC_THREADS) {
        const float w = expf(wsm[b] - mx);
        wsm[b] = w;
        lsm[b] = __fmul_rn(lsm[b], w);
    }
    vb.sync();
    // ---- this thread's lane of blocks
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int i = 0; i < AC_KEEP; i++) {
        const int b = q + Q * i;
        if (b < blocks) {
            o = __fmaf_rn(keep[i], wsm[b], o);
            l = __fadd_rn(l, lsm[b]);
        }
    }
    if (d < hd)
        for (int b = q + Q * AC_KEEP; b < blocks; b += Q) {
            o = __fmaf_rn(__ldcg(part + base0 + b * bs + 2 + d), wsm[b], o);
            l = __fadd_rn(l, lsm[b]);
        }
    lanes_sm[tid] = make_float2(l, o);
    vb.sync();
    if (q != 0 || d >= hd) return;
    for (int qq = 1; qq < Q; qq++) {
        const float2 v = lanes_sm[qq * dims + d];
        l = __fadd_rn(l, v.x);
        o = __fadd_rn(o, v.y);
    }
    // _pad[1] != 0 (extension): floats between output rows, for writing a rank's head columns of a wider row.
    const size_t orow = p._pad[1] ? (size_t)p._pad[1] : (size_t)p.heads * hd;
    const size_t oi = (size_t)row * orow + (size_t)h * hd + d;
    float res = o / l;
    if (p.gated) {
        const float gate = __ldcg(qg + (size_t)row * p.q_row + (size_t)2 * h * hd + hd + d);
        res = o / l / (1.0f + expf(-gate));
    }
    out[oi] = res;
    if (pu != nullptr && pu->push_slot != PEER_NONE) peer::push(*pu, out + oi, res, peer::push_tag(*pu));  // this rank's heads, to every rank
}


}  // namespace attn
