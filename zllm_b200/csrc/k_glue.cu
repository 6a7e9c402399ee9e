// The small kernels around the multiplies: row RMSNorm, SwiGLU, embedding
// gather (with bit-exact block dequantisation), the Q8_0 load-time row split,
// the attention prologue (per-head norm, RoPE, cache append with f16 RNE) and
// the DeltaNet front end and output gate. Each keeps the reference kernel's
// parameter block and binding order (cited per kernel).

#include <cuda_fp16.h>

#include "k_glue_body.cuh"
#include "zcu_internal.h"

namespace {

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// Block-wide sum of doubles; every thread gets the total. `red` holds 32 doubles.
__device__ double block_sum_d(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += red[w];
    return t;
}

// ---- rmsnorm (src/kernels/rmsnorm.wgsl): bindings x, w, y. One CTA per row.
// f32 squares summed in f64, f32 mean, f32 1/sqrt, x * scale * w
// (src/ref/ops.zig:30-41; the reference kernel emulates the f64 sum with
// two-float arithmetic, src/kernels/norm.wgsl:1-77).
__global__ void __launch_bounds__(256) rmsnorm_kernel(PRmsNorm p, const float* __restrict__ x,
                                                     const float* __restrict__ w, float* __restrict__ y) {
    __shared__ double red[32];
    const int r = blockIdx.x;
    const float* xr = x + (size_t)r * p.dim;
    double ss = 0.0;
    for (int i = threadIdx.x; i < (int)p.dim; i += blockDim.x) {
        const float v = xr[i];
        ss += (double)__fmul_rn(v, v);
    }
    ss = block_sum_d(ss, red);
    const float mean = (float)(ss / (double)p.dim);
    const float scale = 1.0f / sqrtf(mean + p.eps);
    const size_t wb = (size_t)(r % max(p.w_rows, 1u)) * p.dim;
    for (int i = threadIdx.x; i < (int)p.dim; i += blockDim.x)
        y[(size_t)r * p.dim + i] = __fmul_rn(__fmul_rn(xr[i], scale), w[wb + i]);
}

// ---- silu_mul (src/kernels/silu_mul.wgsl): bindings gu, act.
__global__ void silu_mul_kernel(PSiluMul p, const float* __restrict__ gu, float* __restrict__ act) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= p.count) return;
    const uint32_t t = i / p.width, j = i % p.width;
    const float g = gu[(size_t)t * 2 * p.width + j];
    act[i] = silu_f(g) * gu[(size_t)t * 2 * p.width + p.width + j];
}

// ---- repack_q8_0 (src/kernels/repack_q8_0.wgsl): bindings src, dst. File
// rows of 34-byte blocks become split rows: k int8, k/32 f16 scales, zero
// padding to 16 bytes. One thread per destination word.
__global__ void repack_q8_0_kernel(PRepackQ80 p, const uint8_t* __restrict__ src, uint32_t* __restrict__ dst) {
    const uint32_t stride = (p.k + p.k / 16 + 15) & ~15u;
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)p.rows * (stride / 4)) return;
    const uint32_t r = (uint32_t)(i / (stride / 4));
    const uint32_t o = 4 * (uint32_t)(i % (stride / 4));
    const size_t raw = (size_t)r * (p.k / 32) * 34;
    const uint32_t blocks = p.k / 32;
    uint32_t word = 0;
    if (o < p.k) {
        const uint8_t* b = src + raw + (size_t)(o / 32) * 34 + 2 + o % 32;
        word = b[0] | (b[1] << 8) | (b[2] << 16) | ((uint32_t)b[3] << 24);
    } else if (o < p.k + p.k / 16) {
        const uint32_t s = (o - p.k) / 2;
        const uint8_t* b = src + raw + (size_t)s * 34;
        word = b[0] | (b[1] << 8);
        if (s + 1 < blocks) word |= ((uint32_t)b[34] << 16) | ((uint32_t)b[35] << 24);
    }
    dst[i] = word;
}

using glue::E_Q4_K;
using glue::E_Q8_0;
using glue::E_BF16;
using glue::E_F16;

template <int TYPE>
__global__ void __launch_bounds__(256) embed_kernel(PEmbed p, const uint32_t* __restrict__ tokens,
                                                   const uint8_t* __restrict__ w, float* __restrict__ out) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // (the first multiply may start its weight copies)
    glue::embed_body<TYPE>(vblock_of_cta(nullptr), p, tokens, w, out);
}

__global__ void __launch_bounds__(256) rope_append_kernel(PRopeAppend p, float* __restrict__ qkv,
                                                         const float* __restrict__ q_norm,
                                                         const float* __restrict__ k_norm,
                                                         const float2* __restrict__ rope, uint32_t* __restrict__ kc,
                                                         uint32_t* __restrict__ vc, const PStep* __restrict__ step,
                                                         const uint32_t* __restrict__ seq_pos) {
    __shared__ __align__(16) unsigned char sm[glue::ROPE_SMEM];
    // (attn_split, a programmatic dependent, may be scheduled now: its blocks of earlier steps' rows start their copies,
    // the others wait for this kernel's end)
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
    glue::rope_append_body(vblock_of_cta(sm), p, qkv, q_norm, k_norm, rope, kc, vc, step, seq_pos);
}

// ---- gated_norm (src/kernels/gated_norm.wgsl): bindings o (rw), z, w. One
// CTA per (head, token): o <- rmsnorm(o) * w * silu(z) (or sigmoid(z)).
// In a tensor-parallel exchange the rank's heads are pushed to every rank (they are columns of the vector the
// output projection reads whole).
__global__ void __launch_bounds__(256) gated_norm_kernel(PGatedNorm p, float* __restrict__ o,
                                                        const float* __restrict__ z, const float* __restrict__ w,
                                                        const __grid_constant__ PeerUse pu) {
    __shared__ double red[32];
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // (the output projection may start its weight copies)
    const uint32_t b = threadIdx.x;
    const size_t base = ((size_t)blockIdx.y * p.v_heads + blockIdx.x) * p.dim;
    const bool in_head = b < p.dim;
    float v = 0.f;
    if (in_head) v = o[base + b];
    const double ss = block_sum_d((double)__fmul_rn(v, v), red);
    if (in_head) {
        const float zz = z[(size_t)blockIdx.y * p.z_row + p.z_off + (size_t)blockIdx.x * p.dim + b];
        const float mean = (float)(ss / (double)p.dim);
        const float r = 1.0f / sqrtf(mean + p.eps);
        const float gate = p.sigmoid ? 1.0f / (1.0f + expf(-zz)) : zz / (1.0f + expf(-zz));
        // rmsNorm then the gate (src/ref/qwen35.zig:543-545): ((v * r) * w) * gate
        const float res = __fmul_rn(__fmul_rn(__fmul_rn(v, r), w[b]), gate);
        o[base + b] = res;
        if (pu.push_slot != PEER_NONE) peer::push(pu, o + base + b, res, peer::push_tag(pu));
    }
}

// ---- delta_prep (src/kernels/delta_prep.wgsl): bindings proj, conv_w, hist,
// out (rw), dt_bias, a, g (rw), beta (rw). CTA (c, t): c < groups does the
// depthwise causal conv + SiLU over one head's channels and L2-normalises q/k
// heads; c == groups computes the gates.
__global__ void __launch_bounds__(256) delta_prep_kernel(PDeltaPrep p, const float* __restrict__ proj,
                                                        const float* __restrict__ conv_w,
                                                        const float* __restrict__ hist, float* __restrict__ out,
                                                        const float* __restrict__ dt_bias, const float* __restrict__ a,
                                                        float* __restrict__ g, float* __restrict__ beta) {
    __shared__ float red[256];
    const uint32_t i = threadIdx.x, c = blockIdx.x, t = blockIdx.y;
    const uint32_t groups = p.channels / p.head;
    if (c == groups) {
        if (i < p.v_heads) {
            const size_t k = (size_t)t * p.v_heads + i;
            beta[k] = 1.0f / (1.0f + expf(-proj[(size_t)t * p.row + p.beta_off + i]));
            const float x = proj[(size_t)t * p.row + p.alpha_off + i] + dt_bias[i];
            const float sp = x > 20.0f ? x : logf(1.0f + expf(x));
            g[k] = sp * a[i];
        }
        return;
    }
    const uint32_t ch = c * p.head + i;
    const bool on = i < p.head;
    float y = 0.f;
    if (on) {
        float sum = 0.f;
        for (uint32_t tap = 0; tap < p.taps; tap++) {
            const uint32_t back = p.taps - 1 - tap;
            float xv;
            if (t >= back) xv = proj[(size_t)(t - back) * p.row + ch];
            else xv = hist[(size_t)(p.taps - 1 - (back - t)) * p.channels + ch];
            sum = __fadd_rn(sum, __fmul_rn(conv_w[(size_t)ch * p.taps + tap], xv));
        }
        y = silu_f(sum);
    }
    if (c * p.head < p.key_channels) {
        // L2 norm over the head: sum of squares in a fixed tree.
        red[i] = on ? __fmul_rn(y, y) : 0.f;
        __syncthreads();
        for (uint32_t s = 128; s > 0; s >>= 1) {
            if (i < s) red[i] = __fadd_rn(red[i], red[i + s]);
            __syncthreads();
        }
        // x * (1 / sqrt(sum + eps)), as the CPU reference's l2Norm (src/ref/ops.zig:44-47)
        y = __fmul_rn(y, 1.0f / sqrtf(red[0] + p.eps));
    }
    if (on) out[(size_t)t * p.channels + ch] = y;
}

}  // namespace

zcu_result launch_rmsnorm(const LaunchArgs& a) {
    PRmsNorm p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "rmsnorm: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    if (p.rows == 0) return ZCU_OK;
    rmsnorm_kernel<<<p.rows, 256, 0, a.stream>>>(p, (const float*)a.b[0].ptr, (const float*)a.b[1].ptr, (float*)a.b[2].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_silu_mul(const LaunchArgs& a) {
    PSiluMul p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 2, "silu_mul: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    if (p.count == 0) return ZCU_OK;
    silu_mul_kernel<<<(p.count + 255) / 256, 256, 0, a.stream>>>(p, (const float*)a.b[0].ptr, (float*)a.b[1].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_repack_q8_0(const LaunchArgs& a) {
    PRepackQ80 p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 2, "repack_q8_0: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.k % 32 == 0, "repack_q8_0: k = %u is not a multiple of 32", p.k);
    const uint32_t stride = (p.k + p.k / 16 + 15) & ~15u;
    const size_t words = (size_t)p.rows * (stride / 4);
    if (words == 0) return ZCU_OK;
    repack_q8_0_kernel<<<(unsigned)((words + 255) / 256), 256, 0, a.stream>>>(p, (const uint8_t*)a.b[0].ptr, (uint32_t*)a.b[1].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_embed(const LaunchArgs& a, uint32_t kernel) {
    PEmbed p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "embed: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    const uint32_t m = a.grid[0];
    if (m == 0) return ZCU_OK;
    const uint32_t* tok = (const uint32_t*)a.b[0].ptr;
    const uint8_t* w = (const uint8_t*)a.b[1].ptr;
    float* out = (float*)a.b[2].ptr;
    switch (kernel) {
        case ZCU_K_EMBED_Q4_K:
            ZCU_NEED(a, p.dim % 256 == 0, "embed_q4_k: dim = %u is not a multiple of 256", p.dim);
            embed_kernel<E_Q4_K><<<m, 256, 0, a.stream>>>(p, tok, w, out);
            break;
        case ZCU_K_EMBED_Q8_0:
            ZCU_NEED(a, p.dim % 32 == 0, "embed_q8_0: dim = %u is not a multiple of 32", p.dim);
            embed_kernel<E_Q8_0><<<m, 256, 0, a.stream>>>(p, tok, w, out);
            break;
        case ZCU_K_EMBED_BF16: embed_kernel<E_BF16><<<m, 256, 0, a.stream>>>(p, tok, w, out); break;
        case ZCU_K_EMBED_F16: embed_kernel<E_F16><<<m, 256, 0, a.stream>>>(p, tok, w, out); break;
        default: return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "embed: kernel %u is not built", kernel);
    }
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_rope_append(const LaunchArgs& a) {
    PRopeAppend p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 7, "rope_append: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.head_dim <= 256 && p.head_dim % 2 == 0, "rope_append: head_dim %u", p.head_dim);
    ZCU_NEED(a, p.kv == KV_F32 || p.kv == KV_F16 || (p.kv == KV_FP8 && p.head_dim % 4 == 0), "rope_append: cache format %u is not built", p.kv);
    const uint32_t m = a.grid[1];
    if (m == 0) return ZCU_OK;
    rope_append_kernel<<<dim3(p.heads + p.kv_heads, m), 256, 0, a.stream>>>(
        p, (float*)a.b[0].ptr, (const float*)a.b[1].ptr, (const float*)a.b[2].ptr, (const float2*)a.b[3].ptr,
        (uint32_t*)a.b[4].ptr, (uint32_t*)a.b[5].ptr, (const PStep*)a.b[6].ptr,
        (a.nb >= 8 && p._pad[0] != 0) ? (const uint32_t*)a.b[7].ptr : nullptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_gated_norm(const LaunchArgs& a) {
    PGatedNorm p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "gated_norm: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.dim <= 256, "gated_norm: dim %u", p.dim);
    const uint32_t m = a.grid[1];
    if (m == 0 || p.v_heads == 0) return ZCU_OK;
    PeerUse pu;
    {
        const float* lo = (const float*)a.b[0].ptr;
        zcu_result pr = parse_peer(a, pu, lo, lo + (size_t)m * p.v_heads * p.dim);
        if (pr != ZCU_OK) return pr;
    }
    gated_norm_kernel<<<dim3(p.v_heads, m), 256, 0, a.stream>>>(p, (float*)a.b[0].ptr, (const float*)a.b[1].ptr, (const float*)a.b[2].ptr, pu);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_delta_prep(const LaunchArgs& a) {
    PDeltaPrep p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 8, "delta_prep: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.head > 0 && p.head <= 256 && p.channels % p.head == 0 && p.v_heads <= 256, "delta_prep: head %u channels %u", p.head, p.channels);
    const uint32_t m = a.grid[1];
    if (m == 0) return ZCU_OK;
    delta_prep_kernel<<<dim3(p.channels / p.head + 1, m), 256, 0, a.stream>>>(
        p, (const float*)a.b[0].ptr, (const float*)a.b[1].ptr, (const float*)a.b[2].ptr, (float*)a.b[3].ptr,
        (const float*)a.b[4].ptr, (const float*)a.b[5].ptr, (float*)a.b[6].ptr, (float*)a.b[7].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}
