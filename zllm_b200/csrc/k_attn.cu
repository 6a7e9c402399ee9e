// GQA decode attention over the KV cache, split over blocks of 64 cache
// positions (flash-decoding) and merged by a second kernel. Replaces the
// reference's attn_split / attn_split_wide / attn_combine
// (src/kernels/attn_split.wgsl, src/kernels/attn_combine.wgsl) with the same
// parameter block (params.Attention), bindings and partials layout:
//   part[((t * heads + head) * max_blocks + b) * (head_dim + 2)] = {block max, block sum, o[0..head_dim)}
// Cache layout pos * (kv_heads * head_dim) + g * head_dim + d, f16 pairs per
// word (kv = 1) or f32 (kv = 0). Each K and V row is read once for the whole
// GQA group. A token's result depends only on its position and the fixed
// 64-key blocks, not on how the step was split.
//
// Extension for batches of independent sequences (the reference runs one sequence at a time): with
// params._pad[0] = S != 0, row r is sequence r: its cache starts S elements after row r-1's, and its
// position comes from one more binding (u32 per row) after `step`.

#include <cfloat>
#include <cuda_fp16.h>

#include <atomic>

#include "k_attn_fast.cuh"
#include "zcu_internal.h"

namespace {

constexpr int AT_THREADS = 256;
constexpr int AT_BLOCK = 64;       // cache positions per CTA (kernels.attn_block)
constexpr int AT_MAX_GROUP = 12;   // kernels.attn_max_group_wide
constexpr int AT_SPLIT = AT_THREADS / AT_BLOCK;  // threads per key

// FP8 E4M3FN (src/kernels/fp8.wgsl:59-64, src/ref/fp8.zig:37-42): 1 sign, 4 exponent (bias 7), 3 mantissa bits.
__device__ __forceinline__ float fp8_value(uint32_t b) {
    const uint32_t e = (b >> 3) & 15u, m = b & 7u;
    const float mag = e == 0 ? (float)m * 0.001953125f : __uint_as_float(((e + 120u) << 23) | (m << 20));
    return (b & 0x80u) ? -mag : mag;
}

// FMT: 0 f32, 1 f16, 2 FP8 bytes (the caller applies the row's scale).
template <int FMT>
__device__ __forceinline__ void load8(const void* base, size_t elem, float* out) {
    if (FMT == 2) {
        const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(base) + elem);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            out[i] = fp8_value((v.x >> (8 * i)) & 0xffu);
            out[4 + i] = fp8_value((v.y >> (8 * i)) & 0xffu);
        }
    } else if (FMT == 1) {
        const uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const __half*>(base) + elem);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(h[i]);
            out[2 * i] = f.x;
            out[2 * i + 1] = f.y;
        }
    } else {
        const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + elem);
        const float4 a = p[0], b = p[1];
        out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
        out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
    }
}

template <int FMT>
__device__ __forceinline__ float2 load2(const void* base, size_t elem) {
    if (FMT == 2) {
        const uint32_t v = *reinterpret_cast<const unsigned short*>(reinterpret_cast<const uint8_t*>(base) + elem);
        return make_float2(fp8_value(v & 0xffu), fp8_value(v >> 8));
    }
    if (FMT == 1) return __half22float2(*reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(base) + elem));
    return *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(base) + elem);
}

// grid (kv_heads, blocks, rows). Dynamic shared memory:
//   qs[group * hd] | sc[group * 64] | stat[2 * group] | pv[parts * group * hd]
template <int FMT, int GROUP_CAP>
__global__ void __launch_bounds__(AT_THREADS) attn_split_kernel(PAttention p, const float* __restrict__ qg,
                                                               const void* __restrict__ kc,
                                                               const void* __restrict__ vc, float* __restrict__ part,
                                                               const PStep* __restrict__ step,
                                                               const uint32_t* __restrict__ seq_pos) {
    extern __shared__ __align__(16) float sm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = blockIdx.x, b = blockIdx.y, t = blockIdx.z;
    const int hd = (int)p.head_dim;
    const int group = (int)(p.heads / p.kv_heads);
    const int row = (int)p.row0 + t;
    // Batched sequences (an extension for independent sequences in one step): row r reads its own
    // cache, seq_stride elements further on, at its own position.
    const size_t seq_off = (size_t)row * p._pad[0];
    const int keys = (seq_pos ? (int)seq_pos[row] : (int)step->pos0 + row) + 1;
    const int k0 = b * AT_BLOCK;
    const size_t kv_stride = (size_t)p.kv_heads * hd;
    const int q_head = p.gated ? 2 * hd : hd;
    const int dpairs = hd / 2;
    const int parts = AT_THREADS / dpairs > 0 ? min(AT_THREADS / dpairs, AT_BLOCK) : 1;

    float* qs = sm;
    float* sc = qs + group * hd;
    float* stat = sc + group * AT_BLOCK;
    float* pv = stat + 2 * AT_MAX_GROUP;

    for (int i = tid; i < group * hd; i += AT_THREADS) {
        const int h = g * group + i / hd;
        qs[i] = qg[(size_t)row * p.q_row + (size_t)h * q_head + i % hd];
    }
    __syncthreads();

    // Scores: thread (key j, quarter s) over dims [s*hd/4, (s+1)*hd/4).
    const int j = tid / AT_SPLIT, s = tid % AT_SPLIT;
    const int key = k0 + j;
    const bool live = key < keys;
    const int span = hd / AT_SPLIT;
    float dot[GROUP_CAP];
#pragma unroll
    for (int h = 0; h < GROUP_CAP; h++) dot[h] = 0.f;
    if (live) {
        const size_t kb = seq_off + (size_t)key * kv_stride + (size_t)g * hd + (size_t)s * span;
        // FP8: the (position, KV head) row's power-of-two scale, stored as f32 at word `scales` on; applying it to
        // each value is exact (src/kernels/attn_split.wgsl:71-78)
        const float ks = FMT == 2 ? reinterpret_cast<const float*>(kc)[p.scales + kb / hd] : 1.0f;
        for (int d = 0; d < span; d += 8) {
            float kk[8];
            load8<FMT>(kc, kb + d, kk);
            if (FMT == 2) {
#pragma unroll
                for (int q = 0; q < 8; q++) kk[q] *= ks;
            }
            const int e = s * span + d;
#pragma unroll
            for (int h = 0; h < GROUP_CAP; h++) {
                if (h < group) {
                    const float4 q0 = *reinterpret_cast<const float4*>(qs + h * hd + e);
                    const float4 q1 = *reinterpret_cast<const float4*>(qs + h * hd + e + 4);
                    float a = dot[h];
                    a = __fmaf_rn(q0.x, kk[0], a);
                    a = __fmaf_rn(q0.y, kk[1], a);
                    a = __fmaf_rn(q0.z, kk[2], a);
                    a = __fmaf_rn(q0.w, kk[3], a);
                    a = __fmaf_rn(q1.x, kk[4], a);
                    a = __fmaf_rn(q1.y, kk[5], a);
                    a = __fmaf_rn(q1.z, kk[6], a);
                    a = __fmaf_rn(q1.w, kk[7], a);
                    dot[h] = a;
                }
            }
        }
    }
#pragma unroll
    for (int h = 0; h < GROUP_CAP; h++) {
        if (h < group) {
            float v = dot[h];
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 1));
            v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, 2));
            if (s == 0) sc[h * AT_BLOCK + j] = live ? v * p.scale : -FLT_MAX;
        }
    }
    __syncthreads();

    // Block softmax per head: one warp per head, two keys per lane.
    const int n = min(AT_BLOCK, keys - min(keys, k0));
    for (int h = warp; h < group; h += AT_THREADS / 32) {
        const float s0 = lane < n ? sc[h * AT_BLOCK + lane] : -FLT_MAX;
        const float s1 = lane + 32 < n ? sc[h * AT_BLOCK + lane + 32] : -FLT_MAX;
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float e0 = (lane < n && s0 != -FLT_MAX) ? expf(s0 - mx) : 0.f;
        const float e1 = (lane + 32 < n && s1 != -FLT_MAX) ? expf(s1 - mx) : 0.f;
        sc[h * AT_BLOCK + lane] = e0;
        sc[h * AT_BLOCK + lane + 32] = e1;
        float sum = __fadd_rn(e0, e1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, o));
        if (lane == 0) {
            stat[2 * h] = mx;
            stat[2 * h + 1] = sum;
        }
    }
    __syncthreads();

    // sum exp * v: thread (key part kp, dim pair dp); each V pair is read once for the group.
    const int dp = tid % dpairs, kp = tid / dpairs;
    float acc[GROUP_CAP][2];
#pragma unroll
    for (int h = 0; h < GROUP_CAP; h++) acc[h][0] = acc[h][1] = 0.f;
    if (kp < parts) {
        for (int i = kp; i < n; i += parts) {
            const size_t vi = seq_off + (size_t)(k0 + i) * kv_stride + (size_t)g * hd + 2 * dp;
            float2 v = load2<FMT>(vc, vi);
            if (FMT == 2) {
                const float vs = reinterpret_cast<const float*>(vc)[p.scales + vi / hd];
                v.x *= vs, v.y *= vs;
            }
#pragma unroll
            for (int h = 0; h < GROUP_CAP; h++) {
                if (h < group) {
                    const float w = sc[h * AT_BLOCK + i];
                    acc[h][0] = __fmaf_rn(w, v.x, acc[h][0]);
                    acc[h][1] = __fmaf_rn(w, v.y, acc[h][1]);
                }
            }
        }
#pragma unroll
        for (int h = 0; h < GROUP_CAP; h++) {
            if (h < group) {
                pv[((size_t)kp * group + h) * hd + 2 * dp] = acc[h][0];
                pv[((size_t)kp * group + h) * hd + 2 * dp + 1] = acc[h][1];
            }
        }
    }
    __syncthreads();
    for (int i = tid; i < group * hd; i += AT_THREADS) {
        const int h = i / hd, d = i % hd;
        float o = 0.f;
        for (int q = 0; q < parts; q++) o = __fadd_rn(o, pv[((size_t)q * group + h) * hd + d]);
        const int head = g * group + h;
        const size_t base = (((size_t)t * p.heads + head) * p.max_blocks + b) * (hd + 2);
        part[base + 2 + d] = o;
        if (d == 0) {
            part[base] = stat[2 * h];
            part[base + 1] = stat[2 * h + 1];
        }
    }
}

template <int HD, int GROUP_CAP>
__global__ void __launch_bounds__(attn::AF_THREADS, 3) attn_split_fast(PAttention p, const float* __restrict__ qg,
                                                                   const __half* __restrict__ kc,
                                                                   const __half* __restrict__ vc, float* __restrict__ part,
                                                                   const PStep* __restrict__ step,
                                                                   const uint32_t* __restrict__ seq_pos) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    attn::attn_split_fast_body<HD, GROUP_CAP>(vblock_of_cta(dyn_smem), p, qg, kc, vc, part, step, seq_pos);
}

template <int HD>
__global__ void __launch_bounds__(attn::AM_THREADS, 3) attn_split_mma(PAttention p, const float* __restrict__ qg,
                                                                     const __half* __restrict__ kc,
                                                                     const __half* __restrict__ vc, float* __restrict__ part,
                                                                     const PStep* __restrict__ step,
                                                                     const uint32_t* __restrict__ seq_pos, int* __restrict__ status) {
    extern __shared__ __align__(128) unsigned char dyn_smem[];
    ATRACE(0);
    // (a programmatic dependent: the body waits for the kernel before - after its first copies where those read only
    // rows of earlier steps)
    attn::attn_split_mma_body<HD, true>(dyn_smem, p, qg, kc, vc, part, step, seq_pos, (int)blockIdx.x, (int)blockIdx.y, (int)blockIdx.z, status);
}

__global__ void __launch_bounds__(attn::AC_THREADS) attn_combine_kernel(PAttention p, const float* __restrict__ qg,
                                                                       const float* __restrict__ part, float* __restrict__ out,
                                                                       const PStep* __restrict__ step,
                                                                       const uint32_t* __restrict__ seq_pos, int kb, int* __restrict__ status,
                                                                       const __grid_constant__ PeerUse pu) {
    extern __shared__ __align__(16) unsigned char dyn_smem[];
    // launched as a programmatic dependent of attn_split; what follows it (a multiply) may move in and start its
    // weight copies at once
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    attn::attn_combine_body(vblock_of_cta(dyn_smem), p, qg, part, out, step, seq_pos, kb, status, &pu);
}

// Copies an exchanged vector out of its exchange slots into the plain floats beside them, waiting for every
// slice (ZCU_K_EXT_PEER_WAIT): what a host that is about to read a gathered vector puts at the end of its step.
__global__ void __launch_bounds__(256) peer_unpack_kernel(const __grid_constant__ PeerUse pu, float* __restrict__ v, uint32_t count,
                                                          int* __restrict__ status) {
    const uint32_t tag = peer::want_tag(pu);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < count; i += gridDim.x * blockDim.x)
        v[i] = peer::read1(pu, v + i, tag, status);
}

using attn::AF_KEYS;
using attn::AF_THREADS;
using attn::AC_MAX_BLOCKS;

}  // namespace

// Cache positions per partial block: 128 on the fast path, else the reference's 64.
int attn_keys_per_block(const PAttention& p) {
    const uint32_t group = p.kv_heads ? p.heads / p.kv_heads : 0;
    const bool fast = p.kv == KV_F16 && group >= 1 && group <= 4 && (p.head_dim == 64 || p.head_dim == 128);
    return fast ? attn::AF_KEYS : AT_BLOCK;
}

namespace {

template <int FMT>
zcu_result launch_split_fmt(const LaunchArgs& a, const PAttention& p, dim3 grid, size_t smem, int group) {
    const float* qg = (const float*)a.b[0].ptr;
    float* part = (float*)a.b[3].ptr;
    const PStep* step = (const PStep*)a.b[4].ptr;
    const uint32_t* seq_pos = (a.nb >= 6 && p._pad[0] != 0) ? (const uint32_t*)a.b[5].ptr : nullptr;
    if (group <= 4) {
        attn_split_kernel<FMT, 4><<<grid, AT_THREADS, smem, a.stream>>>(p, qg, a.b[1].ptr, a.b[2].ptr, part, step, seq_pos);
    } else if (group <= 8) {
        attn_split_kernel<FMT, 8><<<grid, AT_THREADS, smem, a.stream>>>(p, qg, a.b[1].ptr, a.b[2].ptr, part, step, seq_pos);
    } else {
        attn_split_kernel<FMT, AT_MAX_GROUP><<<grid, AT_THREADS, smem, a.stream>>>(p, qg, a.b[1].ptr, a.b[2].ptr, part, step, seq_pos);
    }
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

}  // namespace

zcu_result launch_attn_split(const LaunchArgs& a) {
    PAttention p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 5, "attn_split: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.kv_heads > 0 && p.heads % p.kv_heads == 0, "attn_split: heads %u over kv_heads %u", p.heads, p.kv_heads);
    const int group = (int)(p.heads / p.kv_heads);
    ZCU_NEED(a, group <= AT_MAX_GROUP, "attn_split: GQA group %d above %d", group, AT_MAX_GROUP);
    ZCU_NEED(a, p.head_dim % 32 == 0 && p.head_dim <= 256 && p.head_dim >= 32, "attn_split: head_dim %u", p.head_dim);
    ZCU_NEED(a, p.kv == KV_F32 || p.kv == KV_F16 || p.kv == KV_FP8, "attn_split: cache format %u is not built", p.kv);
    ZCU_NEED(a, p.kv != KV_FP8 || p.head_dim % 64 == 0, "attn_split: an FP8 cache needs head_dim %u in whole 64s (8-byte loads)", p.head_dim);
    ZCU_NEED(a, a.grid[1] <= p.max_blocks, "attn_split: %u key blocks above max_blocks %u", a.grid[1], p.max_blocks);
    if (a.grid[1] == 0 || a.grid[2] == 0) return ZCU_OK;
    const int hd = (int)p.head_dim;
    if (attn_keys_per_block(p) == AF_KEYS) {
        // the dispatch's grid counts 64-key blocks (kernels.attn_block); this path takes 128 keys per CTA
        const dim3 grid(p.kv_heads, (a.grid[1] * AT_BLOCK + AF_KEYS - 1) / AF_KEYS, a.grid[2]);
        const size_t smem = attn::attn_fast_smem(4, (int)group, (int)hd);
        const float* qg = (const float*)a.b[0].ptr;
        const __half* kc = (const __half*)a.b[1].ptr;
        const __half* vc = (const __half*)a.b[2].ptr;
        float* part = (float*)a.b[3].ptr;
        const PStep* step = (const PStep*)a.b[4].ptr;
        const uint32_t* seq_pos = (a.nb >= 6 && p._pad[0] != 0) ? (const uint32_t*)a.b[5].ptr : nullptr;
        // Variants: 0 (default) and 3 = tensor cores; 1 = CUDA cores (exact f32 products). One CTA per block.
        if (a.variant == 0 || a.variant == 3) {
            // one CTA per block on the f16 tensor cores (queries and probabilities as two f16 terms)
            const size_t msmem = attn::attn_mma_smem(hd);
            auto mk = hd == 128 ? attn_split_mma<128> : attn_split_mma<64>;
            if (cudaFuncSetAttribute(mk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)msmem) != cudaSuccess) {
                cudaGetLastError();
                return zcu_fail(a, ZCU_E_GPU, "attn_split: %zu bytes of shared memory refused", msmem);
            }
            cudaError_t e = launch_pdl(mk, grid, dim3(attn::AM_THREADS), msmem, a.stream, p, qg, kc, vc, part, step, seq_pos, a.status);
            if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "attn_split: launch failed: %s", cudaGetErrorString(e));
            return ZCU_OK;
        }
        if (a.variant == 1) {
            if (hd == 128) attn_split_fast<128, 4><<<grid, AF_THREADS, smem, a.stream>>>(p, qg, kc, vc, part, step, seq_pos);
            else attn_split_fast<64, 4><<<grid, AF_THREADS, smem, a.stream>>>(p, qg, kc, vc, part, step, seq_pos);
            ZCU_CHECK_LAUNCH(a);
            return ZCU_OK;
        }
        return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "attn_split: variant %u is not built", a.variant);
    }
    const int dpairs = hd / 2;
    const int parts = AT_THREADS / dpairs > AT_BLOCK ? AT_BLOCK : AT_THREADS / dpairs;
    const size_t smem = ((size_t)group * hd + (size_t)group * AT_BLOCK + 2 * AT_MAX_GROUP + (size_t)parts * group * hd) * sizeof(float);
    ZCU_NEED(a, smem <= 48 * 1024, "attn_split: %zu bytes of shared memory", smem);
    const dim3 grid(p.kv_heads, a.grid[1], a.grid[2]);
    if (p.kv == KV_FP8) return launch_split_fmt<2>(a, p, grid, smem, group);
    return p.kv == KV_F16 ? launch_split_fmt<1>(a, p, grid, smem, group) : launch_split_fmt<0>(a, p, grid, smem, group);
}

zcu_result launch_attn_combine(const LaunchArgs& a) {
    PAttention p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 4, "attn_combine: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.head_dim <= 256, "attn_combine: head_dim %u", p.head_dim);
    ZCU_NEED(a, p.max_blocks <= AC_MAX_BLOCKS, "attn_combine: max_blocks %u above %d", p.max_blocks, AC_MAX_BLOCKS);
    if (a.grid[0] == 0 || a.grid[1] == 0) return ZCU_OK;
    const uint32_t* seq_pos = (a.nb >= 5 && p._pad[0] != 0) ? (const uint32_t*)a.b[4].ptr : nullptr;
    const size_t smem = attn::attn_combine_smem((int)p.max_blocks);
    PeerUse pu;
    {
        // the columns this launch writes: heads * head_dim floats of each of its rows
        const size_t orow = p._pad[1] ? (size_t)p._pad[1] : (size_t)p.heads * p.head_dim;
        const float* lo = (const float*)a.b[2].ptr + (size_t)p.row0 * orow;
        const float* hi = lo + (size_t)(a.grid[1] - 1) * orow + (size_t)p.heads * p.head_dim;
        zcu_result pr = parse_peer(a, pu, lo, hi);
        if (pr != ZCU_OK) return pr;
    }
    if (smem > 48 * 1024 && cudaFuncSetAttribute(attn_combine_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "attn_combine: %zu bytes of shared memory refused", smem);
    }
    cudaError_t e = launch_pdl(attn_combine_kernel, dim3(p.heads, a.grid[1]), dim3(attn::AC_THREADS), smem, a.stream, p, (const float*)a.b[0].ptr,
                               (const float*)a.b[1].ptr, (float*)a.b[2].ptr, (const PStep*)a.b[3].ptr, seq_pos, attn_keys_per_block(p),
                               a.status, pu);
    if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "attn_combine: launch failed: %s", cudaGetErrorString(e));
    return ZCU_OK;
}

// ---------------------------------------------------------------------------------------------------
// Decode attention for callers that cannot allocate device memory.
//
// attn_split hands its per-block partials to attn_combine through a buffer the caller normally
// allocates. Some callers cannot do that: a host that runs inside somebody else's memory budget
// (a plugin that was given fixed input/output buffers and nothing more), or code on a path where
// cudaMalloc is forbidden because it would synchronise the device or break a latency guarantee.
// For them the partials live in the fixed array below, which is part of the library image: every GPU
// that loads the library holds these 4 MiB until the process exits.
//
// `g_attn_partials` is a device symbol. In host code its name is only a stand-in; the device address
// comes from cudaGetSymbolAddress, asked once per device with that device current.
constexpr size_t ATTN_STATIC_FLOATS = (size_t)1 << 20;  // 4 MiB
static __device__ __align__(256) float g_attn_partials[ATTN_STATIC_FLOATS];
static std::atomic<float*> g_attn_partials_ptr[64] = {};   // contexts on several threads may resolve it at once

// Bindings: qg, kc, vc, out, step (+ per-row positions for batched sequences). `max_keys`: the largest
// number of cache positions any row attends to (its position + 1). The partials are laid out as
// attn_split lays them out, max_blocks = ceil(max_keys / 64) blocks per (row, head).
zcu_result launch_attn_static(const LaunchArgs& a, uint32_t max_keys, uint32_t rows) {
    PAttention p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 5, "attention (static partials): bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.kv_heads > 0 && p.heads % p.kv_heads == 0 && max_keys > 0 && rows > 0,
             "attention (static partials): heads %u over kv_heads %u, %u keys, %u rows", p.heads, p.kv_heads, max_keys, rows);
    p.max_blocks = (max_keys + AT_BLOCK - 1) / AT_BLOCK;
    // everything either launch would refuse is refused here, before the first of them is enqueued
    ZCU_NEED(a, p.heads / p.kv_heads <= AT_MAX_GROUP && p.head_dim % 32 == 0 && p.head_dim >= 32 && p.head_dim <= 256 &&
                    (p.kv == KV_F32 || p.kv == KV_F16 || (p.kv == KV_FP8 && p.head_dim % 64 == 0)) && p.max_blocks <= AC_MAX_BLOCKS,
             "attention (static partials): group %u, head_dim %u, cache format %u or %u key blocks is not built", p.heads / p.kv_heads,
             p.head_dim, p.kv, p.max_blocks);
    const size_t need = (size_t)rows * p.heads * p.max_blocks * (p.head_dim + 2);
    if (need > ATTN_STATIC_FLOATS)
        return zcu_fail(a, ZCU_E_INVALID,
                        "attention (static partials): %u rows x %u heads x %u blocks x (%u + 2) = %zu floats exceed the fixed "
                        "%zu-float (4 MiB) array; use attn_split / attn_combine with a buffer of your own",
                        rows, p.heads, p.max_blocks, p.head_dim, need, ATTN_STATIC_FLOATS);
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return zcu_fail(a, ZCU_E_GPU, "attention (static partials): no current device");
    if (!g_attn_partials_ptr[dev].load()) {
        // First call on this device: resolve the symbol's device address. Not a stream operation, so it
        // should happen before any stream capture starts.
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_attn_partials);
        if (e != cudaSuccess || !ptr)
            return zcu_fail(a, ZCU_E_GPU, "attention (static partials): cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_attn_partials_ptr[dev].store(ptr);
    }
    const zcu_binding part = {g_attn_partials_ptr[dev].load(), need * sizeof(float)};
    const bool batched = a.nb >= 6 && p._pad[0] != 0;
    // attn_split: qg, kc, vc, part, step [, positions]; grid (kv_heads, 64-key blocks, rows)
    zcu_binding sb[6] = {a.b[0], a.b[1], a.b[2], part, a.b[4], {nullptr, 0}};
    if (batched) sb[5] = a.b[5];
    LaunchArgs s = a;
    s.params = &p;
    s.params_bytes = sizeof(p);
    s.b = sb;
    s.nb = batched ? 6 : 5;
    s.grid[0] = p.kv_heads;
    s.grid[1] = p.max_blocks;
    s.grid[2] = rows;
    zcu_result r = launch_attn_split(s);
    if (r != ZCU_OK) return r;
    // attn_combine: qg, part, out, step [, positions]; grid (heads, rows)
    zcu_binding cb[5] = {a.b[0], part, a.b[3], a.b[4], {nullptr, 0}};
    if (batched) cb[4] = a.b[5];
    LaunchArgs c = a;
    c.params = &p;
    c.params_bytes = sizeof(p);
    c.b = cb;
    c.nb = batched ? 5 : 4;
    c.grid[0] = p.heads;
    c.grid[1] = rows;
    c.grid[2] = 1;
    return launch_attn_combine(c);
}

// Parameter block: a PPeer naming the slot to wait for. Binding: the vector (inside the local arena).
zcu_result launch_peer_wait(const LaunchArgs& a) {
    PeerUse pu;
    zcu_result pr = parse_peer(a, pu, nullptr, nullptr);
    if (pr != ZCU_OK) return pr;
    ZCU_NEED(a, pu.wait_slot != PEER_NONE && pu.push_slot == PEER_NONE && a.nb >= 1, "peer_wait: needs a slot to wait for and the vector");
    const uint64_t lo = reinterpret_cast<uint64_t>(a.b[0].ptr), base = pu.t.base[pu.t.rank];
    ZCU_NEED(a, lo >= base && lo + a.b[0].size <= base + pu.t.ll_off && a.b[0].size % 4 == 0, "peer_wait: the vector is not inside the local arena");
    const uint32_t count = (uint32_t)(a.b[0].size / 4);
    if (count == 0) return ZCU_OK;
    const int blocks = (int)((count + 255) / 256 < (uint32_t)(a.sm_count * 4) ? (count + 255) / 256 : (uint32_t)(a.sm_count * 4));
    peer_unpack_kernel<<<blocks, 256, 0, a.stream>>>(pu, (float*)a.b[0].ptr, count, a.status);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

// Ends a run of the launch list (ZCU_K_EXT_PEER_NEXT; parameter block: a PPeer, its slots unused): the epoch that
// every exchange tag of the list derives from moves on. An ordinary launch: it starts after everything before it in
// the stream has ended, and what follows starts after it.
__global__ void peer_next_kernel(uint32_t* epoch) { epoch[0] += 1; }

zcu_result launch_peer_next(const LaunchArgs& a) {
    PeerUse pu;
    zcu_result pr = parse_peer(a, pu, nullptr, nullptr);
    if (pr != ZCU_OK) return pr;
    ZCU_NEED(a, pu.t.epoch != nullptr, "peer_next: the parameter block is not a peer block");
    peer_next_kernel<<<1, 1, 0, a.stream>>>(pu.t.epoch);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

#ifdef ZCU_TRACE
extern "C" __attribute__((visibility("default"))) int zcu_dbg_attn_trace_read(unsigned long long* out, size_t count) {
    return (int)cudaMemcpyFromSymbol(out, g_at_trace, count * sizeof(unsigned long long));
}
#endif
