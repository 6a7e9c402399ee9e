// rope_append and the embedding rows, written for virtual blocks (vblock.cuh); the kernels of k_glue.cu map one
// CUDA block to each.
#pragma once

#include <cuda_fp16.h>

#include "vblock.cuh"
#include "zcu_internal.h"

namespace glue {

// Sum of doubles over a virtual block; every thread gets the total. `red` holds 32 doubles.
__device__ __forceinline__ double vblock_sum_d(const VBlock& vb, double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    vb.sync();
    if ((vb.tid & 31) == 0) red[vb.tid >> 5] = v;
    vb.sync();
    double t = 0.0;
    for (int w = 0; w < (vb.nthreads >> 5); w++) t += red[w];
    return t;
}

// ---- embed_* (src/kernels/embed_quant.wgsl, embed_half.wgsl): bindings
// tokens, w, out. out[t] = table[tokens[t] - row0] decoded to f32 for tokens
// in this chunk; one CTA per token. Decoding is bit for bit the CPU
// reference's (src/ref/tensor.zig:50-53, 101-116): products and differences
// are rounded separately, never fused.
enum { E_Q4_K = 0, E_Q8_0 = 1, E_BF16 = 2, E_F16 = 3 };

template <int TYPE>
__device__ __forceinline__ void embed_body(const VBlock& vb, const PEmbed& p, const uint32_t* __restrict__ tokens,
                                           const uint8_t* __restrict__ w, float* __restrict__ out) {
    const uint32_t t = (uint32_t)vb.x;
    const uint32_t tok = tokens[t];
    if (tok < p.row0 || tok >= p.row0 + p.chunk_rows) return;
    const uint32_t r = tok - p.row0;
    float* o = out + (size_t)t * p.dim;
    if (TYPE == E_Q4_K) {
        const size_t stride = p.stride ? p.stride : (size_t)(p.dim / 256) * 144;
        const uint8_t* row = w + (size_t)r * stride;
        // one thread per (super-block, sub-block pair j, byte l)
        for (uint32_t i = (uint32_t)vb.tid; i < p.dim / 2; i += (uint32_t)vb.nthreads) {
            const uint32_t blk = i / 128, j = (i % 128) / 32, l = i % 32;
            const uint8_t* b = row + (size_t)blk * 144;
            const float d = __half2float(__ushort_as_half((unsigned short)(b[0] | (b[1] << 8))));
            const float mn = __half2float(__ushort_as_half((unsigned short)(b[2] | (b[3] << 8))));
            const uint8_t* s = b + 4;
            uint32_t sc1, m1, sc2, m2;
            const uint32_t j1 = 2 * j, j2 = 2 * j + 1;
            if (j1 < 4) { sc1 = s[j1] & 63; m1 = s[j1 + 4] & 63; }
            else { sc1 = (s[j1 + 4] & 0xF) | ((s[j1 - 4] >> 6) << 4); m1 = (s[j1 + 4] >> 4) | ((s[j1] >> 6) << 4); }
            if (j2 < 4) { sc2 = s[j2] & 63; m2 = s[j2 + 4] & 63; }
            else { sc2 = (s[j2 + 4] & 0xF) | ((s[j2 - 4] >> 6) << 4); m2 = (s[j2 + 4] >> 4) | ((s[j2] >> 6) << 4); }
            const float d1 = __fmul_rn(d, (float)sc1), mm1 = __fmul_rn(mn, (float)m1);
            const float d2 = __fmul_rn(d, (float)sc2), mm2 = __fmul_rn(mn, (float)m2);
            const uint8_t q = b[16 + 32 * j + l];
            o[blk * 256 + 64 * j + l] = __fsub_rn(__fmul_rn(d1, (float)(q & 0xF)), mm1);
            o[blk * 256 + 64 * j + 32 + l] = __fsub_rn(__fmul_rn(d2, (float)(q >> 4)), mm2);
        }
    } else if (TYPE == E_Q8_0) {
        if (p.stride) {
            // rows as in the file: 34-byte blocks
            const uint8_t* row = w + (size_t)r * p.stride;
            for (uint32_t i = (uint32_t)vb.tid; i < p.dim; i += (uint32_t)vb.nthreads) {
                const uint8_t* b = row + (size_t)(i / 32) * 34;
                const float d = __half2float(__ushort_as_half((unsigned short)(b[0] | (b[1] << 8))));
                o[i] = __fmul_rn((float)(int)(int8_t)b[2 + i % 32], d);
            }
        } else {
            // split rows (repack_q8_0)
            const size_t stride = ((size_t)p.dim + p.dim / 16 + 15) & ~(size_t)15;
            const uint8_t* row = w + (size_t)r * stride;
            for (uint32_t i = (uint32_t)vb.tid; i < p.dim; i += (uint32_t)vb.nthreads) {
                const uint8_t* sp = row + p.dim + 2 * (i / 32);
                const float d = __half2float(__ushort_as_half((unsigned short)(sp[0] | (sp[1] << 8))));
                o[i] = __fmul_rn((float)(int)(int8_t)row[i], d);
            }
        }
    } else {
        const uint16_t* row = reinterpret_cast<const uint16_t*>(w) + (size_t)r * p.dim;
        for (uint32_t i = (uint32_t)vb.tid; i < p.dim; i += (uint32_t)vb.nthreads) {
            const uint32_t bits = row[i];
            o[i] = TYPE == E_BF16 ? __uint_as_float(bits << 16) : __half2float(__ushort_as_half((unsigned short)bits));
        }
    }
}

// ---- rope_append (src/kernels/rope_append.wgsl): bindings qkv (rw), q_norm,
// k_norm, rope table, kc (rw), vc (rw), step. One CTA per (head x, token t)
// over heads + kv_heads; thread i owns dim i. K and V go to the cache at
// pos0 + t; the f16 cache rounds to nearest even (src/ref/qwen35.zig:32-42).
constexpr size_t ROPE_SMEM = 32 * sizeof(double) + 256 * sizeof(float);

// The exponent k of an FP8 row's scale 2^k: the smallest with m <= 448 * 2^k; 0 for a zero or subnormal maximum.
__device__ __forceinline__ int fp8_scale_exp(float m) {
    const uint32_t bits = __float_as_uint(m);
    const int e = (int)((bits >> 23) & 255u);
    if (e == 0) return 0;
    return e - 127 - 8 + ((bits & 0x7fffffu) > 0x600000u ? 1 : 0);
}
// |x| <= 448 (clamped) -> E4M3FN bits, round to nearest, ties to even (src/ref/fp8.zig:12-35).
__device__ __forceinline__ uint32_t fp8_bits(float x) {
    const uint32_t sign = (__float_as_uint(x) >> 24) & 0x80u;
    const float a = fminf(fabsf(x), 448.0f);
    if (a < 0.015625f) {
        const float s = a * 512.0f;   // exact
        uint32_t q = (uint32_t)floorf(s);
        const float r = s - (float)q;
        if (r > 0.5f || (r == 0.5f && (q & 1u) == 1u)) q += 1u;
        return sign | q;
    }
    const uint32_t ab = __float_as_uint(a);
    uint32_t e = (ab >> 23) - 120u;
    const uint32_t mant = ab & 0x7fffffu;
    uint32_t q = mant >> 20;
    const uint32_t rem = mant & 0xfffffu;
    if (rem > 0x80000u || (rem == 0x80000u && (q & 1u) == 1u)) q += 1u;
    if (q == 8u) q = 0u, e += 1u;
    const uint32_t code = (e << 3) | q;
    return sign | (code < 0x7eu ? code : 0x7eu);
}

__device__ __forceinline__ void rope_append_body(const VBlock& vb, const PRopeAppend& p, float* __restrict__ qkv,
                                                 const float* __restrict__ q_norm, const float* __restrict__ k_norm,
                                                 const float2* __restrict__ rope, uint32_t* __restrict__ kc,
                                                 uint32_t* __restrict__ vc, const PStep* __restrict__ step,
                                                 const uint32_t* __restrict__ seq_pos) {
    double* red = reinterpret_cast<double*>(vb.smem);
    float* vals = reinterpret_cast<float*>(vb.smem + 32 * sizeof(double));
    const uint32_t i = (uint32_t)vb.tid, xh = (uint32_t)vb.x, t = (uint32_t)vb.y;
    const uint32_t hd = p.head_dim;
    const bool is_q = xh < p.heads;
    const uint32_t g = xh - (is_q ? 0u : p.heads);
    const uint32_t q_head = p.gated ? 2 * hd : hd;
    const size_t base = (size_t)t * p.row + (is_q ? xh * q_head : p.k_off + g * hd);
    float v = 0.f;
    if (i < hd) v = __ldcg(qkv + base + i);
    const double ss = vblock_sum_d(vb, (double)__fmul_rn(v, v), red);
    if (i < hd) {
        if (p.qk_norm) {
            const float mean = (float)(ss / (double)hd);
            const float scale = 1.0f / sqrtf(mean + p.eps);
            vals[i] = __fmul_rn(__fmul_rn(v, scale), is_q ? q_norm[i] : k_norm[i]);
        } else {
            vals[i] = v;
        }
    }
    vb.sync();
    const uint32_t half = p.n_rot / 2;
    // Batched sequences (an extension): with _pad[0] = S != 0, row t is sequence t, with its own position
    // (one more binding, u32 per row) and its own cache, S elements after row t-1's.
    const uint32_t pos = seq_pos ? seq_pos[t] : step->pos0 + t;
    float r0 = 0.f, r1 = 0.f;
    uint32_t a = 0, b = 0;
    if (i < half) {
        const float2 cs = rope[(size_t)pos * half + i];
        a = p.normal ? 2 * i : i;
        b = p.normal ? 2 * i + 1 : i + half;
        const float x0 = vals[a], x1 = vals[b];
        // x0*cos - x1*sin and x0*sin + x1*cos with every product rounded (src/ref/ops.zig:64-86).
        r0 = __fsub_rn(__fmul_rn(x0, cs.x), __fmul_rn(x1, cs.y));
        r1 = __fadd_rn(__fmul_rn(x0, cs.y), __fmul_rn(x1, cs.x));
    }
    vb.sync();
    if (i < half) {
        vals[a] = r0;
        vals[b] = r1;
    }
    vb.sync();
    if (is_q) {
        if (i < hd) qkv[base + i] = vals[i];
        return;
    }
    const size_t width = (size_t)p.kv_heads * hd;
    const size_t e = (size_t)t * p._pad[0] + (size_t)pos * width + (size_t)g * hd;
    const size_t vo = (size_t)t * p.row + p.v_off + (size_t)g * hd;
    if (p.kv == KV_FP8) {
        // each row divided by its power-of-two scale (the smallest with amax / scale <= 448), four codes a word, the
        // scale as f32 at word `scales` + row (src/kernels/rope_append.wgsl:118-137, src/ref/fp8.zig:44-55)
        float* mx = reinterpret_cast<float*>(red);   // [2][warps]; the sums it held are consumed
        float ka = i < hd ? fabsf(vals[i]) : 0.f, va = i < hd ? fabsf(__ldcg(qkv + vo + i)) : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ka = fmaxf(ka, __shfl_xor_sync(0xffffffffu, ka, o));
            va = fmaxf(va, __shfl_xor_sync(0xffffffffu, va, o));
        }
        const int warps = vb.nthreads / 32;
        if ((i & 31u) == 0) mx[i / 32] = ka, mx[32 + i / 32] = va;
        vb.sync();
        ka = va = 0.f;
        for (int w = 0; w < warps; w++) ka = fmaxf(ka, mx[w]), va = fmaxf(va, mx[32 + w]);
        const int k_exp = fp8_scale_exp(ka), v_exp = fp8_scale_exp(va);
        const float k_inv = __uint_as_float((uint32_t)(127 - k_exp) << 23), v_inv = __uint_as_float((uint32_t)(127 - v_exp) << 23);
        if (i < hd / 4) {
            uint32_t kw = 0, vw = 0;
#pragma unroll
            for (uint32_t q = 0; q < 4; q++) {
                kw |= fp8_bits(vals[4 * i + q] * k_inv) << (8 * q);
                vw |= fp8_bits(__ldcg(qkv + vo + 4 * i + q) * v_inv) << (8 * q);
            }
            kc[e / 4 + i] = kw;
            vc[e / 4 + i] = vw;
        }
        if (i == 0) {
            kc[p.scales + e / hd] = (uint32_t)(127 + k_exp) << 23;
            vc[p.scales + e / hd] = (uint32_t)(127 + v_exp) << 23;
        }
        return;
    }
    if (i < hd / 2) {
        const float k0 = vals[2 * i], k1 = vals[2 * i + 1];
        const float v0 = __ldcg(qkv + vo + 2 * i), v1 = __ldcg(qkv + vo + 2 * i + 1);
        if (p.kv == KV_F16) {
            const uint32_t kw = (uint32_t)__half_as_ushort(__float2half_rn(k0)) | ((uint32_t)__half_as_ushort(__float2half_rn(k1)) << 16);
            const uint32_t vw = (uint32_t)__half_as_ushort(__float2half_rn(v0)) | ((uint32_t)__half_as_ushort(__float2half_rn(v1)) << 16);
            kc[e / 2 + i] = kw;
            vc[e / 2 + i] = vw;
        } else {
            kc[e + 2 * i] = __float_as_uint(k0);
            kc[e + 2 * i + 1] = __float_as_uint(k1);
            vc[e + 2 * i] = __float_as_uint(v0);
            vc[e + 2 * i + 1] = __float_as_uint(v1);
        }
    }
}

}  // namespace glue
