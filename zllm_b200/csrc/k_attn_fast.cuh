// The decode-attention fast path (f16 cache) and the merge of its partials, written for virtual blocks (vblock.cuh);
// the kernels of k_attn.cu map one CUDA block to each.
#pragma once

#include <cfloat>
#include <cuda_fp16.h>

#include "tma_util.cuh"
#include "vblock.cuh"
#include "zcu_internal.h"

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
// 16-row A operand; the two partial results are added afterwards. Scores: A = Q [16 x dims], B = K^T [dims x keys]
// read straight out of the staged K tile; sum exp * v: A = P [16 x keys], B = V [keys x dims] through
// ldmatrix.trans, each warp owning head_dim / 8 output dims over all 128 keys, so no cross-warp reduction is
// left. About 350 warp instructions per warp and block instead of 1600 on the CUDA cores. K and V tiles (rows
// padded to head_dim * 2 + 16 bytes: conflict-free fragment reads) arrive by cp.async while the queries are split.
constexpr int AM_THREADS = 256;
__host__ __device__ constexpr size_t attn_mma_smem(int hd) {
    return (size_t)2 * AF_KEYS * (hd * 2 + 16) + (size_t)(4 * AF_KEYS + 8 + 4 * hd) * sizeof(float);
}

__device__ __forceinline__ void mma_f16_16816(float* c, uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1) {
    // rows 8-15 of A are zero (a1 = a3 = 0)
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
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

// One block's arithmetic once its K and V tiles (rows RS bytes apart) and the group's queries (qs) are in shared
// memory. Every thread of the 256 calls it; it ends with the partial written.
// Where 16 bytes (8 dims starting at `dim`, a multiple of 8) of key/value row r sit in a staged tile.
// SWZ = false: rows HD * 2 + 16 bytes apart (cp.async fills them). SWZ = true: the tile as TMA leaves it with the
// 128-byte swizzle: one 128-row x 128-byte panel per 64 dims, 16-byte chunks XORed with the row's low three bits.
template <int HD, bool SWZ>
__device__ __forceinline__ uint32_t tile_addr(uint32_t tile, int r, int dim) {
    if (!SWZ) return tile + (uint32_t)r * (HD * 2 + 16) + (uint32_t)dim * 2u;
    const int panel = dim >> 6, chunk = (dim & 63) >> 3;
    return tile + (uint32_t)panel * (AF_KEYS * 128) + (uint32_t)r * 128u + (uint32_t)((chunk ^ (r & 7)) << 4);
}

template <int HD, bool SWZ = false>
__device__ __forceinline__ void mma_block_compute(uint32_t kt_s, uint32_t vt_s, float (*sc)[AF_KEYS], float* stat, const float* qs,
                                                  const PAttention& p, float* __restrict__ part, int g_kv, int b, int t, int keys,
                                                  int k0, bool wait_values) {
    constexpr int KSTEPS = HD / 16;              // k-steps of the score product
    constexpr int NBLK = HD / 64;                // 8-dim output blocks per warp in the value product
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, tq = lane & 3;      // fragment coordinates
    const int group = (int)(p.heads / p.kv_heads);
    const int n = min(AF_KEYS, keys - min(keys, k0));
    // ---- scores: warp w takes keys 16 w .. 16 w + 15
    {
        const float* qrow = qs + (size_t)(g & 3) * HD;
        const bool low = g >= 4;
        float c[2][4];
#pragma unroll
        for (int nb = 0; nb < 2; nb++) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ks++) {
            const float2 qa = *reinterpret_cast<const float2*>(qrow + 16 * ks + 2 * tq);
            const float2 qb = *reinterpret_cast<const float2*>(qrow + 16 * ks + 8 + 2 * tq);
            const uint32_t a0 = split_pair(qa.x, qa.y, low), a2 = split_pair(qb.x, qb.y, low);
#pragma unroll
            for (int nb = 0; nb < 2; nb++) {
                const int kr = 16 * warp + 8 * nb + g;
                uint32_t b0, b1;
                asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(b0) : "r"(tile_addr<HD, SWZ>(kt_s, kr, 16 * ks) + 4u * tq));
                asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(b1) : "r"(tile_addr<HD, SWZ>(kt_s, kr, 16 * ks + 8) + 4u * tq));
                mma_f16_16816(c[nb], a0, a2, b0, b1);
            }
        }
#pragma unroll
        for (int nb = 0; nb < 2; nb++) {
            // hi rows (lanes g < 4) + lo rows (lanes g + 4 = lane + 16)
            const float s0 = __fadd_rn(c[nb][0], __shfl_xor_sync(0xffffffffu, c[nb][0], 16));
            const float s1 = __fadd_rn(c[nb][1], __shfl_xor_sync(0xffffffffu, c[nb][1], 16));
            if (g < group) {
                const int kl = 16 * warp + 8 * nb + 2 * tq;
                sc[g][kl] = k0 + kl < keys ? s0 * p.scale : -FLT_MAX;
                sc[g][kl + 1] = k0 + kl + 1 < keys ? s1 * p.scale : -FLT_MAX;
            }
        }
    }
    __syncthreads();
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
    if (wait_values) asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    __syncthreads();
    // ---- sum exp * v: warp w takes dims (HD / 8) w .. over all 128 keys
    {
        const float* prow = sc[min(g & 3, group - 1)];
        const bool low = g >= 4;
        float c[NBLK][4];
#pragma unroll
        for (int nb = 0; nb < NBLK; nb++) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.f;
        const int d0 = (HD / 8) * warp;
#pragma unroll
        for (int ks = 0; ks < AF_KEYS / 16; ks++) {
            const float2 pa = *reinterpret_cast<const float2*>(prow + 16 * ks + 2 * tq);
            const float2 pb = *reinterpret_cast<const float2*>(prow + 16 * ks + 8 + 2 * tq);
            const uint32_t a0 = split_pair(pa.x, pa.y, low), a2 = split_pair(pb.x, pb.y, low);
#pragma unroll
            for (int nb = 0; nb < NBLK; nb++) {
                // two 8 x 8 matrices of V (keys 16 ks .. +7 and +8 .. +15, dims d0 + 8 nb .. +7), transposed on the way
                const uint32_t vaddr = tile_addr<HD, SWZ>(vt_s, 16 * ks + (lane & 15), d0 + 8 * nb);
                uint32_t b0, b1;
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(vaddr));
                mma_f16_16816(c[nb], a0, a2, b0, b1);
            }
        }
#pragma unroll
        for (int nb = 0; nb < NBLK; nb++) {
            const float o0 = __fadd_rn(c[nb][0], __shfl_xor_sync(0xffffffffu, c[nb][0], 16));
            const float o1 = __fadd_rn(c[nb][1], __shfl_xor_sync(0xffffffffu, c[nb][1], 16));
            if (g < group) {
                const int head = g_kv * group + g, d = d0 + 8 * nb + 2 * tq;
                const size_t base = (((size_t)t * p.heads + head) * p.max_blocks + b) * (HD + 2);
                part[base + 2 + d] = o0;
                part[base + 2 + d + 1] = o1;
                if (d == 0) {
                    part[base] = stat[2 * g];
                    part[base + 1] = stat[2 * g + 1];
                }
            }
        }
    }
}

template <int HD>
__device__ __forceinline__ void attn_split_mma_body(unsigned char* smem, const PAttention& p, const float* __restrict__ qg,
                                                    const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                    float* __restrict__ part, const PStep* __restrict__ step,
                                                    const uint32_t* __restrict__ seq_pos, int g_kv, int b, int t,
                                                    int* __restrict__ status = nullptr) {
    constexpr int RS = HD * 2 + 16;              // bytes between the rows of a staged tile
    constexpr int PIECES = AF_KEYS * (HD / 8) / AM_THREADS;
    unsigned char* Kt = smem;
    unsigned char* Vt = smem + (size_t)AF_KEYS * RS;
    float (*sc)[AF_KEYS] = reinterpret_cast<float (*)[AF_KEYS]>(Vt + (size_t)AF_KEYS * RS);
    float* stat = reinterpret_cast<float*>(sc) + 4 * AF_KEYS;
    float* qs = stat + 8;                        // [4][HD]
    const uint32_t kt_s = (uint32_t)__cvta_generic_to_shared(Kt), vt_s = (uint32_t)__cvta_generic_to_shared(Vt);
    const int tid = threadIdx.x;
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

    // ---- tiles on their way
#pragma unroll
    for (int i = 0; i < PIECES; i++) {
        const int j = tid + AM_THREADS * i, key = j / (HD / 8), piece = j % (HD / 8);
        const size_t src = seq_off + (size_t)min(k0 + key, keys - 1) * kv_stride + (size_t)g_kv * HD + 8 * piece;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(kt_s + (uint32_t)key * RS + 16u * piece), "l"(kc + src) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < PIECES; i++) {
        const int j = tid + AM_THREADS * i, key = j / (HD / 8), piece = j % (HD / 8);
        const size_t src = seq_off + (size_t)min(k0 + key, keys - 1) * kv_stride + (size_t)g_kv * HD + 8 * piece;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(vt_s + (uint32_t)key * RS + 16u * piece), "l"(vc + src) : "memory");
    }
    asm volatile("cp.async.commit_group;\n" ::: "memory");
    // ---- the group's queries
    for (int i = tid; i < 4 * HD / 4; i += AM_THREADS) {
        const int h = i / (HD / 4), d4 = i % (HD / 4);
        const float* qp = qg + (size_t)row * p.q_row + (size_t)(g_kv * group + min(h, group - 1)) * q_head;
        reinterpret_cast<float4*>(qs)[i] = __ldcg(reinterpret_cast<const float4*>(qp) + d4);
    }
    asm volatile("cp.async.wait_group 1;\n" ::: "memory");
    __syncthreads();

    mma_block_compute<HD>(kt_s, vt_s, sc, stat, qs, p, part, g_kv, b, t, keys, k0, true);
}

// ---- the same block arithmetic as a persistent kernel: one CTA per SM walks a contiguous range of the
// (row, KV head, key block) space with its K and V tiles (128 keys x head_dim halves each) arriving through a
// 3-stage cp.async pipeline, so the loads of the next two blocks are in flight while a block is computed. With
// one block per CTA (the kernel above) each CTA pays an HBM round trip before its first multiply and a wave and a
// bit of CTAs pay it twice; here it is paid once per CTA. Every sum keeps the order of attn_split_fast_body, so
// the partials are the same bits.
constexpr int AP_STAGES = 3;
__host__ __device__ constexpr size_t attn_persist_smem(int group_cap, int group, int hd) {
    return (size_t)AP_STAGES * 2 * AF_KEYS * hd * 2 + ((size_t)group_cap * AF_KEYS + 2 * group_cap + 8) * sizeof(float) +
           (size_t)(AF_THREADS / 32) * group * hd * sizeof(float);
}

// The tensor-core block arithmetic as a persistent walk: one CTA per SM, the K/V tiles of the next two blocks in
// flight. A tile is TMA box copies (one per 64 dims: 128 rows x 128 bytes, 128-byte swizzle) issued by one thread
// and completing on the stage's mbarrier, so the arithmetic warps spend no instructions on loading. A block costs
// about a microsecond of arithmetic, so the walk is bound by the tiles' arrival, i.e. by HBM. Waits are bounded.
__host__ __device__ constexpr size_t attn_mma_persist_smem(int hd) {
    return 1024 + (size_t)AP_STAGES * 2 * AF_KEYS * hd * 2 + (size_t)(4 * AF_KEYS + 8 + 4 * hd) * sizeof(float) + 64;
}

template <int HD>
__device__ __forceinline__ void attn_split_mma_persistent_body(unsigned char* smem_raw, const PAttention& p, const float* __restrict__ qg,
                                                               const CUtensorMap* kmap, const CUtensorMap* vmap,
                                                               float* __restrict__ part, const PStep* __restrict__ step,
                                                               const uint32_t* __restrict__ seq_pos, int by, int rows,
                                                               int* __restrict__ status) {
    constexpr int TILE = AF_KEYS * HD * 2;       // bytes of a K (or V) tile: HD / 64 panels of 128 rows x 128 bytes
    constexpr int PANELS = HD / 64;
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);  // swizzled tiles
    float (*sc)[AF_KEYS] = reinterpret_cast<float (*)[AF_KEYS]>(smem + (size_t)AP_STAGES * 2 * TILE);
    float* stat = reinterpret_cast<float*>(sc) + 4 * AF_KEYS;
    float* qs = stat + 8;
    const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(smem);
    const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(qs + 4 * HD);
    const int tid = threadIdx.x;
    const int kvh = (int)p.kv_heads, group = (int)(p.heads / p.kv_heads);
    const int q_head = p.gated ? 2 * HD : HD;
    const int total = kvh * by * rows;
    const int lo = (int)((long long)blockIdx.x * total / gridDim.x), hi = (int)((long long)(blockIdx.x + 1) * total / gridDim.x);
    if (tid == 0) {
        for (int s = 0; s < AP_STAGES; s++) asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar0 + 8 * s), "r"(1) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    auto keys_of = [&](int t) {
        const int row = (int)p.row0 + t;
        return (seq_pos ? (int)seq_pos[row] : (int)step->pos0 + row) + 1;
    };
    // thread 0 asks for block idx's tiles into `stage` (nothing for a block past its row's keys or this CTA's range)
    auto issue = [&](int idx, int stage) {
        if (tid != 0 || idx >= hi) return;
        const int b = idx % by, g = (idx / by) % kvh, t = idx / (by * kvh);
        if (b * AF_KEYS >= keys_of(t)) return;
        const uint32_t bar = bar0 + 8 * stage, kt = stage0 + (uint32_t)stage * 2 * TILE;
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");  // the stage was read with ordinary loads
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(2 * TILE) : "memory");
#pragma unroll
        for (int pn = 0; pn < PANELS; pn++) {
            const int x = g * HD * 2 + 128 * pn, y = b * AF_KEYS, z = p._pad[0] ? (int)p.row0 + t : 0;  // one cache unless rows are sequences
            asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(kt + pn * (AF_KEYS * 128)),
                         "l"((uint64_t)kmap), "r"(bar), "r"(x), "r"(y), "r"(z)
                         : "memory");
            asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];\n" ::"r"(kt + TILE + pn * (AF_KEYS * 128)),
                         "l"((uint64_t)vmap), "r"(bar), "r"(x), "r"(y), "r"(z)
                         : "memory");
        }
    };
#pragma unroll
    for (int s = 0; s < AP_STAGES - 1; s++) issue(lo + s, s);
    int q_g = -1, q_t = -1, stage = 0;
    uint32_t phase_bits = 0;
    bool timed_out = false;
    for (int idx = lo; idx < hi; idx++) {
        issue(idx + AP_STAGES - 1, stage == 0 ? AP_STAGES - 1 : stage - 1);
        const int b = idx % by, g = (idx / by) % kvh, t = idx / (by * kvh);
        const int keys = keys_of(t), k0 = b * AF_KEYS;
        const uint32_t kt = stage0 + (uint32_t)stage * 2 * TILE, bar = bar0 + 8 * stage;
        const int this_stage = stage;
        stage = stage + 1 == AP_STAGES ? 0 : stage + 1;
        if (k0 >= keys) continue;  // nothing was asked for: the stage's barrier is untouched
        if (g != q_g || t != q_t) {  // consecutive blocks of a CTA mostly share their queries
            q_g = g, q_t = t;
            const int row = (int)p.row0 + t;
            for (int i = tid; i < 4 * HD / 4; i += AM_THREADS) {
                const int h = i / (HD / 4), d4 = i % (HD / 4);
                const float* qp = qg + (size_t)row * p.q_row + (size_t)(g * group + min(h, group - 1)) * q_head;
                reinterpret_cast<float4*>(qs)[i] = __ldcg(reinterpret_cast<const float4*>(qp) + d4);
            }
        }
        {   // the tiles of this block (at most 2^20 polls)
            bool ok = false;
            const uint32_t parity = (phase_bits >> this_stage) & 1u;
            for (int spin = 0; spin < (1 << 20) && !ok; spin++) {
                uint32_t done;
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                             : "=r"(done) : "r"(bar), "r"(parity) : "memory");
                ok = done != 0;
            }
            if (!ok) timed_out = true;
            phase_bits ^= 1u << this_stage;
        }
        __syncthreads();  // the queries are in place
        mma_block_compute<HD, true>(kt, kt + TILE, sc, stat, qs, p, part, g, b, t, keys, k0, false);
        __syncthreads();  // every warp is done with this block's tiles, probabilities and queries
    }
    if (timed_out && (tid & 31) == 0 && status) atomicExch(status, 1);
}

template <int HD, int GROUP_CAP>
__device__ __forceinline__ void attn_split_persistent_body(unsigned char* smem, const PAttention& p, const float* __restrict__ qg,
                                                           const __half* __restrict__ kc, const __half* __restrict__ vc,
                                                           float* __restrict__ part, const PStep* __restrict__ step,
                                                           const uint32_t* __restrict__ seq_pos, int by, int rows) {
    constexpr int DPT = HD / 8, KPP = AF_THREADS / 8, PASSES = AF_KEYS / KPP;
    constexpr int TPK = HD / 8, KG = AF_THREADS / TPK, KPT = AF_KEYS / KG;
    constexpr int TILE = AF_KEYS * HD * 2;        // bytes of one K (or V) tile
    constexpr int PIECES = TILE / 16 / AF_THREADS; // 16-byte pieces of a tile per thread
    float (*sc)[AF_KEYS] = reinterpret_cast<float (*)[AF_KEYS]>(smem + (size_t)AP_STAGES * 2 * TILE);
    float* stat = reinterpret_cast<float*>(sc) + GROUP_CAP * AF_KEYS;
    float* pv = stat + 2 * GROUP_CAP + 8;
    const uint32_t stage0 = (uint32_t)__cvta_generic_to_shared(smem);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kvh = (int)p.kv_heads, group = (int)(p.heads / p.kv_heads);
    const size_t kv_stride = (size_t)kvh * HD;
    const int q_head = p.gated ? 2 * HD : HD;
    const int total = kvh * by * rows;
    const int lo = (int)((long long)blockIdx.x * total / gridDim.x), hi = (int)((long long)(blockIdx.x + 1) * total / gridDim.x);
    const int kl = tid >> 3, sl = tid & 7, kg = tid / TPK, dl = tid % TPK;

    auto keys_of = [&](int t) {
        const int row = (int)p.row0 + t;
        return (seq_pos ? (int)seq_pos[row] : (int)step->pos0 + row) + 1;
    };
    // asks for block idx's tiles into `stage` (nothing for a block past its row's keys or past this CTA's range)
    auto issue = [&](int idx, int stage) {
        if (idx < hi) {
            const int b = idx % by, g = (idx / by) % kvh, t = idx / (by * kvh);
            const int keys = keys_of(t), k0 = b * AF_KEYS;
            if (k0 < keys) {
                const size_t seq_off = (size_t)((int)p.row0 + t) * p._pad[0];
#pragma unroll
                for (int i = 0; i < PIECES; i++) {
                    const int j = tid + AF_THREADS * i, key = j / (HD / 8), piece = j % (HD / 8);
                    const size_t src = seq_off + (size_t)min(k0 + key, keys - 1) * kv_stride + (size_t)g * HD + 8 * piece;
                    const uint32_t dst = stage0 + (uint32_t)stage * 2 * TILE + (uint32_t)j * 16u;
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(kc + src) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst + TILE), "l"(vc + src) : "memory");
                }
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");  // one group per call, empty or not
    };
#pragma unroll
    for (int s = 0; s < AP_STAGES - 1; s++) issue(lo + s, s);

    float q[GROUP_CAP][DPT];
    int q_g = -1, q_t = -1;
    int stage = 0;
    for (int idx = lo; idx < hi; idx++) {
        issue(idx + AP_STAGES - 1, stage == 0 ? AP_STAGES - 1 : stage - 1);
        asm volatile("cp.async.wait_group %0;\n" ::"n"(AP_STAGES - 1) : "memory");
        __syncthreads();  // every thread's pieces of this block have landed; the last block's scratch is free
        const int b = idx % by, g = (idx / by) % kvh, t = idx / (by * kvh);
        const int keys = keys_of(t), k0 = b * AF_KEYS;
        const uint32_t ktile = stage0 + (uint32_t)stage * 2 * TILE, vtile = ktile + TILE;
        stage = stage + 1 == AP_STAGES ? 0 : stage + 1;
        if (k0 >= keys) continue;
        const int n = min(AF_KEYS, keys - k0);
        const int row = (int)p.row0 + t;
        if (g != q_g || t != q_t) {  // consecutive blocks of a CTA mostly share their queries
            q_g = g, q_t = t;
#pragma unroll
            for (int h = 0; h < GROUP_CAP; h++) {
                const float* qp = qg + (size_t)row * p.q_row + (size_t)(g * group + min(h, group - 1)) * q_head + sl * DPT;
#pragma unroll
                for (int d = 0; d < DPT; d += 4) {
                    const float4 v = __ldcg(reinterpret_cast<const float4*>(qp + d));
                    q[h][d] = v.x; q[h][d + 1] = v.y; q[h][d + 2] = v.z; q[h][d + 3] = v.w;
                }
            }
        }
        // ---- scores: 8 threads per key, K from the tile
#pragma unroll
        for (int ps = 0; ps < PASSES; ps++) {
            const int key = k0 + ps * KPP + kl;
            float dot[GROUP_CAP];
#pragma unroll
            for (int h = 0; h < GROUP_CAP; h++) dot[h] = 0.f;
#pragma unroll
            for (int c = 0; c < DPT / 8; c++) {
                uint4 kraw;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(kraw.x), "=r"(kraw.y), "=r"(kraw.z), "=r"(kraw.w)
                             : "r"(ktile + (uint32_t)(ps * KPP + kl) * (HD * 2) + (uint32_t)sl * (DPT * 2) + 16u * c));
                const __half2* hp = reinterpret_cast<const __half2*>(&kraw);
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
        __syncthreads();
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
        __syncthreads();
        // ---- sum exp * v: thread (key group kg, dims 8 dl .. 8 dl + 7), V from the tile
        float acc[GROUP_CAP][8];
#pragma unroll
        for (int h = 0; h < GROUP_CAP; h++)
#pragma unroll
            for (int d = 0; d < 8; d++) acc[h][d] = 0.f;
#pragma unroll
        for (int i = 0; i < KPT; i++) {
            const int ki = kg + KG * i;
            if (ki < n) {
                uint4 vpiece;
                asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(vpiece.x), "=r"(vpiece.y), "=r"(vpiece.z), "=r"(vpiece.w)
                             : "r"(vtile + (uint32_t)ki * (HD * 2) + 16u * dl));
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
#pragma unroll
        for (int h = 0; h < GROUP_CAP; h++)
#pragma unroll
            for (int d = 0; d < 8; d++) {
                float v = acc[h][d];
#pragma unroll
                for (int o = TPK; o < 32; o <<= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
                acc[h][d] = v;
            }
        if (lane < TPK) {
#pragma unroll
            for (int h = 0; h < GROUP_CAP; h++)
                if (h < group) {
                    float* dst = pv + ((size_t)warp * group + h) * HD + 8 * lane;
                    *reinterpret_cast<float4*>(dst) = make_float4(acc[h][0], acc[h][1], acc[h][2], acc[h][3]);
                    *reinterpret_cast<float4*>(dst + 4) = make_float4(acc[h][4], acc[h][5], acc[h][6], acc[h][7]);
                }
        }
        __syncthreads();
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
    asm volatile("cp.async.wait_group 0;\n" ::: "memory");
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
