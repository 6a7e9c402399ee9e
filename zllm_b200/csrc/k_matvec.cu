// Decode-path multiplies: out[t][col0 + j] (+)= sum_i x[t][i] * w[j][i], with
// the weights' dequantisation fused into the dot product. Replaces the
// reference's matvec_q4_k / matvec_q8_0 / matvec_bf16 / matvec_f16 identities
// (src/kernels/matvec_quant.wgsl.hbs, src/kernels/matvec_half.wgsl) with the
// same parameter block, bindings and fused flags:
//   NORM        x <- rmsnorm(x) * norm_w first
//   ACCUMULATE  out += result
//   SILU_PAIR   out[j] = silu(w[j].x) * (w[half + j].x)
//
// Two families per quantised type:
//   scalar  f32 activations from shared memory, f32 FMA on the CUDA cores,
//           warp-shuffle reduction in a fixed tree. The default identity.
//   mma     the weights' integer codes become exact f16 A-fragments (one LOP3
//           per two nibbles, one HFMA2 that removes the magic offset and
//           applies the 6-bit sub-block scale, exactly), activations are split
//           into two f16 terms (hi + lo * 2^-11, scaled per token by a power of
//           two), and mma.sync m16n8k16 accumulates in f32. Sixteen rows per
//           warp, 8-byte coalesced loads of the packed blocks, activations
//           staged once per CTA in shared memory in fragment order. The f16
//           super-block scales d/dmin multiply the f32 accumulators once per
//           super-block on the CUDA cores.
//
// Every reduction has a fixed order, so a token's result does not depend on
// how many tokens the step has (the reference's step-split invariance,
// src/kernels/check.zig:1019-1031).
//
// Weight layouts: Q4_K rows as in the GGUF file (144-byte super-blocks,
// src/ref/tensor.zig:100-116); Q8_0 rows split by repack_q8_0 (k int8 values,
// then k/32 f16 scales, padded to 16 bytes: src/kernels/quant/q8_0.wgsl:1-24);
// BF16/F16 two per word (src/kernels/half/bf16.wgsl:3-9).

#include <cuda_fp16.h>
#include <cuda_bf16.h>

#include "zcu_internal.h"

namespace {

enum { W_Q4_K = 0, W_Q8_0 = 1, W_BF16 = 2, W_F16 = 3 };

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = __fadd_rn(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }

// Sum of squares of token row `x` (k floats) over the whole CTA, in f64 as the
// reference's CPU norm sums (src/ref/ops.zig:30-41); also the largest
// |x * norm_w| (or |x|). `red` holds 2 * 32 doubles. Every thread calls it.
__device__ void cta_norm_stats(const float* __restrict__ x, const float* __restrict__ nw, int k, bool norm,
                               double* red, double& ss_out, float& amax_out) {
    const int tid = threadIdx.x, nt = blockDim.x;
    double ss = 0.0;
    float amax = 0.0f;
    for (int i = tid; i < k / 4; i += nt) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        ss += (double)__fmul_rn(v.x, v.x);
        ss += (double)__fmul_rn(v.y, v.y);
        ss += (double)__fmul_rn(v.z, v.z);
        ss += (double)__fmul_rn(v.w, v.w);
        float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
        if (norm) w = reinterpret_cast<const float4*>(nw)[i];
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x * w.x), fabsf(v.y * w.y)), fmaxf(fabsf(v.z * w.z), fabsf(v.w * w.w))));
    }
    ss = warp_sum_d(ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    __syncthreads();
    if ((tid & 31) == 0) {
        red[tid >> 5] = ss;
        red[32 + (tid >> 5)] = (double)amax;
    }
    __syncthreads();
    double tot = 0.0;
    float am = 0.0f;
    for (int w = 0; w < (nt >> 5); w++) {
        tot += red[w];
        am = fmaxf(am, (float)red[32 + w]);
    }
    ss_out = tot;
    amax_out = am;
}

// ------------------------------------------------------------------ scalar family

// Per-lane partial dot products of one (block, part) task for MT tokens.
// xs points at the task's block inside the staged tile; token t's tile is
// xs + t * xs_stride.
template <int TYPE, int MT>
struct BlockDot;

// Q4_K: 8 parts per 256-weight super-block; part p covers 16 bytes of qs:
// 16 weights of sub-block 2j (low nibbles) and 16 of sub-block 2j+1 (high
// nibbles), j = p/2, at elements 16*(p&1).. of each.
template <int MT>
struct BlockDot<W_Q4_K, MT> {
    static constexpr int BLOCK = 256, PARTS = 8;
    __device__ static size_t row_bytes(int k) { return (size_t)(k / 256) * 144; }
    __device__ static void run(const uint8_t* __restrict__ row, int /*k*/, int gblk, int part, const float* xs,
                               int xs_stride, float* acc) {
        const uint8_t* blk = row + (size_t)gblk * 144;
        const uint4 hdr = *reinterpret_cast<const uint4*>(blk);
        const uint4 q = *reinterpret_cast<const uint4*>(blk + 16 + 16 * part);
        const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
        const int j = part >> 1;
        // 6-bit scales and mins of sub-blocks 2j and 2j+1 (src/ref/tensor.zig:95-98).
        const uint32_t sc_lo4 = hdr.y & 0x3f3f3f3fu, m_lo4 = hdr.z & 0x3f3f3f3fu;
        const uint32_t sc_hi4 = (hdr.w & 0x0f0f0f0fu) | ((hdr.y >> 2) & 0x30303030u);
        const uint32_t m_hi4 = ((hdr.w >> 4) & 0x0f0f0f0fu) | ((hdr.z >> 2) & 0x30303030u);
        const int s1 = 2 * j, s2 = 2 * j + 1;
        const uint32_t scr = (s1 < 4) ? sc_lo4 : sc_hi4, mr = (s1 < 4) ? m_lo4 : m_hi4;
        const float d1 = __fmul_rn(d, (float)((scr >> (8 * (s1 & 3))) & 0xffu));
        const float m1 = __fmul_rn(dmin, (float)((mr >> (8 * (s1 & 3))) & 0xffu));
        const float d2 = __fmul_rn(d, (float)((scr >> (8 * (s2 & 3))) & 0xffu));
        const float m2 = __fmul_rn(dmin, (float)((mr >> (8 * (s2 & 3))) & 0xffu));
        const int e0 = 64 * j + 16 * (part & 1);
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int t = 0; t < MT; t++) {
            const float4* xl = reinterpret_cast<const float4*>(xs + (size_t)t * xs_stride + e0);
            const float4* xh = reinterpret_cast<const float4*>(xs + (size_t)t * xs_stride + e0 + 32);
            float sl = 0.f, sh = 0.f, xsl = 0.f, xsh = 0.f;
#pragma unroll
            for (int v = 0; v < 4; v++) {
                const float4 a = xl[v], b = xh[v];
                const uint32_t w = qw[v];
                sl = __fmaf_rn(a.x, (float)(w & 0xfu), sl);
                sl = __fmaf_rn(a.y, (float)((w >> 8) & 0xfu), sl);
                sl = __fmaf_rn(a.z, (float)((w >> 16) & 0xfu), sl);
                sl = __fmaf_rn(a.w, (float)((w >> 24) & 0xfu), sl);
                sh = __fmaf_rn(b.x, (float)((w >> 4) & 0xfu), sh);
                sh = __fmaf_rn(b.y, (float)((w >> 12) & 0xfu), sh);
                sh = __fmaf_rn(b.z, (float)((w >> 20) & 0xfu), sh);
                sh = __fmaf_rn(b.w, (float)(w >> 28), sh);
                xsl = __fadd_rn(xsl, __fadd_rn(__fadd_rn(a.x, a.y), __fadd_rn(a.z, a.w)));
                xsh = __fadd_rn(xsh, __fadd_rn(__fadd_rn(b.x, b.y), __fadd_rn(b.z, b.w)));
            }
            float r = __fmaf_rn(d1, sl, acc[t]);
            r = __fmaf_rn(-m1, xsl, r);
            r = __fmaf_rn(d2, sh, r);
            acc[t] = __fmaf_rn(-m2, xsh, r);
        }
    }
};

// Q8_0 on split rows: 2 parts per 32-weight block, 16 weights each.
template <int MT>
struct BlockDot<W_Q8_0, MT> {
    static constexpr int BLOCK = 32, PARTS = 2;
    __device__ static size_t row_bytes(int k) { return ((size_t)k + k / 16 + 15) & ~(size_t)15; }
    __device__ static void run(const uint8_t* __restrict__ row, int k, int gblk, int part, const float* xs,
                               int xs_stride, float* acc) {
        const uint4 q = *reinterpret_cast<const uint4*>(row + (size_t)gblk * 32 + 16 * part);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(row + k + 2 * gblk)));
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int t = 0; t < MT; t++) {
            const float4* xv = reinterpret_cast<const float4*>(xs + (size_t)t * xs_stride + 16 * part);
            float s = 0.f;
#pragma unroll
            for (int v = 0; v < 4; v++) {
                const float4 a = xv[v];
                const uint32_t w = qw[v];
                s = __fmaf_rn(a.x, (float)(int)(int8_t)(w & 0xffu), s);
                s = __fmaf_rn(a.y, (float)(int)(int8_t)((w >> 8) & 0xffu), s);
                s = __fmaf_rn(a.z, (float)(int)(int8_t)((w >> 16) & 0xffu), s);
                s = __fmaf_rn(a.w, (float)(int)(int8_t)(w >> 24), s);
            }
            acc[t] = __fmaf_rn(d, s, acc[t]);
        }
    }
};

// BF16 / F16: "blocks" of 8 weights, one 16-byte load.
template <int TYPE, int MT>
struct BlockDotHalf {
    static constexpr int BLOCK = 8, PARTS = 1;
    __device__ static size_t row_bytes(int k) { return (size_t)k * 2; }
    __device__ static float widen(uint32_t bits16) {
        if (TYPE == W_BF16) return __uint_as_float(bits16 << 16);
        return __half2float(__ushort_as_half((unsigned short)bits16));
    }
    __device__ static void run(const uint8_t* __restrict__ row, int /*k*/, int gblk, int /*part*/, const float* xs,
                               int xs_stride, float* acc) {
        const uint4 q = *reinterpret_cast<const uint4*>(row + (size_t)gblk * 16);
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int t = 0; t < MT; t++) {
            const float4* xv = reinterpret_cast<const float4*>(xs + (size_t)t * xs_stride);
            const float4 a = xv[0], b = xv[1];
            float s = acc[t];
            s = __fmaf_rn(a.x, widen(qw[0] & 0xffffu), s);
            s = __fmaf_rn(a.y, widen(qw[0] >> 16), s);
            s = __fmaf_rn(a.z, widen(qw[1] & 0xffffu), s);
            s = __fmaf_rn(a.w, widen(qw[1] >> 16), s);
            s = __fmaf_rn(b.x, widen(qw[2] & 0xffffu), s);
            s = __fmaf_rn(b.y, widen(qw[2] >> 16), s);
            s = __fmaf_rn(b.z, widen(qw[3] & 0xffffu), s);
            s = __fmaf_rn(b.w, widen(qw[3] >> 16), s);
            acc[t] = s;
        }
    }
};
template <int MT>
struct BlockDot<W_BF16, MT> : BlockDotHalf<W_BF16, MT> {};
template <int MT>
struct BlockDot<W_F16, MT> : BlockDotHalf<W_F16, MT> {};

constexpr int SC_THREADS = 256;
constexpr int SC_TILE = 2048;  // staged floats per token per tile (the reference's TILE_ONE)

// One CTA = 8 warps x ROWS rows; x staged in tiles of SC_TILE floats for MT
// tokens; lanes take (block, part) tasks in lane order.
template <int TYPE, int MT, int ROWS>
__global__ void __launch_bounds__(SC_THREADS) matvec_scalar(PMatvec p, const float* __restrict__ x,
                                                           const uint8_t* __restrict__ w, float* __restrict__ out,
                                                           const float* __restrict__ norm_w, int t0) {
    using BD = BlockDot<TYPE, MT>;
    __shared__ __align__(16) float xs[MT * SC_TILE];
    __shared__ double red[64];
    __shared__ float scales[MT];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int k = (int)p.k;
    const int xr = p.x_stride ? (int)p.x_stride * 4 : k;
    const bool norm = (p.flags & MV_NORM) != 0, pair = (p.flags & MV_SILU_PAIR) != 0;
    const size_t rb = BD::row_bytes(k);
    const int j0 = (blockIdx.x * (SC_THREADS / 32) + warp) * ROWS;

    if (norm) {
        for (int t = 0; t < MT; t++) {
            double ss;
            float am;
            cta_norm_stats(x + (size_t)(t0 + t) * xr, norm_w, k, false, red, ss, am);
            if (tid == 0) {
                const float mean = (float)(ss / (double)k);
                scales[t] = 1.0f / sqrtf(mean + p.eps);
            }
        }
        __syncthreads();
    }

    float acc[ROWS][MT], acc2[ROWS][MT];
#pragma unroll
    for (int r = 0; r < ROWS; r++)
#pragma unroll
        for (int t = 0; t < MT; t++) acc[r][t] = acc2[r][t] = 0.f;

    for (int k0 = 0; k0 < k; k0 += SC_TILE) {
        const int len = min(SC_TILE, k - k0);
        __syncthreads();
        for (int i = tid; i < MT * (len / 4); i += SC_THREADS) {
            const int t = i / (len / 4), v = i % (len / 4);
            float4 a = reinterpret_cast<const float4*>(x + (size_t)(t0 + t) * xr + k0)[v];
            if (norm) {
                const float4 nw = reinterpret_cast<const float4*>(norm_w + k0)[v];
                const float s = scales[t];
                a.x = __fmul_rn(__fmul_rn(a.x, s), nw.x);
                a.y = __fmul_rn(__fmul_rn(a.y, s), nw.y);
                a.z = __fmul_rn(__fmul_rn(a.z, s), nw.z);
                a.w = __fmul_rn(__fmul_rn(a.w, s), nw.w);
            }
            reinterpret_cast<float4*>(xs + t * SC_TILE)[v] = a;
        }
        __syncthreads();
        const int tasks = (len / BD::BLOCK) * BD::PARTS;
        for (int task = lane; task < tasks; task += 32) {
            const int blk = task / BD::PARTS, part = task % BD::PARTS;
            const int gblk = k0 / BD::BLOCK + blk;
            const float* xb = xs + blk * BD::BLOCK;
#pragma unroll
            for (int r = 0; r < ROWS; r++) {
                const int j = j0 + r;
                if (j >= (int)p.n) break;
                BD::run(w + (size_t)j * rb, k, gblk, part, xb, SC_TILE, acc[r]);
                if (pair) BD::run(w + (size_t)(p.half + j) * rb, k, gblk, part, xb, SC_TILE, acc2[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < ROWS; r++) {
        const int j = j0 + r;
#pragma unroll
        for (int t = 0; t < MT; t++) {
            float v = warp_sum(acc[r][t]);
            float u = pair ? warp_sum(acc2[r][t]) : 0.f;
            if (lane == 0 && j < (int)p.n) {
                if (pair) v = silu_f(v) * u;
                const size_t o = (size_t)(t0 + t) * p.out_stride + p.col0 + j;
                if (p.flags & MV_ACCUMULATE) v += out[o];
                out[o] = v;
            }
        }
    }
}

// ------------------------------------------------------------------ mma family

__device__ __forceinline__ void mma_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_1688(float* c, uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xea;\n" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t hfma2_u(uint32_t a, uint32_t b, uint32_t c) {
    return h2_as_u32(__hfma2(u32_as_h2(a), u32_as_h2(b), u32_as_h2(c)));
}
__device__ __forceinline__ uint32_t hsub2_u(uint32_t a, uint32_t b) {
    return h2_as_u32(__hsub2(u32_as_h2(a), u32_as_h2(b)));
}
__device__ __forceinline__ uint32_t hmul2_u(uint32_t a, uint32_t b) {
    return h2_as_u32(__hmul2(u32_as_h2(a), u32_as_h2(b)));
}

constexpr int MM_THREADS = 256;
constexpr int MM_WARPS = 8;
constexpr int MM_PAD = 32;            // halfs of padding per staged column (keeps LDS.128 conflict-free)
constexpr uint32_t H2_1024 = 0x64006400u, H2_64 = 0x54005400u, H2_1152 = 0x64806480u;
constexpr uint32_t H2_M1024 = 0xe400e400u, H2_M64 = 0xd400d400u;

// Position of element i of a staged column. Q4_K nibble pairs come out of a
// word as (byte0, byte2) and (byte1, byte3), so the middle two of every four
// elements swap places; Q8_0 keeps natural order.
template <int TYPE>
__device__ __forceinline__ int stage_pos(int i) {
    if (TYPE == W_Q4_K) return (i & ~3) | ((i & 1) << 1) | ((i >> 1) & 1);
    return i;
}

struct MmaShared {
    // byte offsets into dynamic shared memory
    int xs, sx, red, meta, total;
};

__host__ __device__ inline MmaShared mma_layout(int cols, int kt, bool q4k, int tr, int nb, bool pair) {
    MmaShared s;
    int off = 0;
    s.xs = off;
    off += cols * (kt + MM_PAD) * 2;
    s.sx = off;
    if (q4k) off += cols * (kt / 32 + 8) * 2;
    off = (off + 15) & ~15;
    s.red = off;
    off += MM_WARPS * 16 * 4 * nb * (pair ? 2 : 1) * 4;
    s.meta = off;
    off += 64 * 8 + 4 * nb * 2 * 4;  // reduction scratch (64 doubles) + per-token {norm scale, 1/s}
    s.total = off;
    (void)tr;
    return s;
}

// One CTA: 8 warps = TR row tiles (16 rows each) x KS k-splits. NB column
// blocks of 8 (4 tokens each, hi/lo).
template <int TYPE, int KS, int NB>
__global__ void __launch_bounds__(MM_THREADS) matvec_mma(PMatvec p, const float* __restrict__ x,
                                                        const uint8_t* __restrict__ w, float* __restrict__ out,
                                                        const float* __restrict__ norm_w, int t0, int mt, int kt) {
    constexpr int TR = MM_WARPS / KS;
    constexpr bool Q4 = TYPE == W_Q4_K;
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int k = (int)p.k;
    const int xr = p.x_stride ? (int)p.x_stride * 4 : k;
    const bool norm = (p.flags & MV_NORM) != 0, pair = (p.flags & MV_SILU_PAIR) != 0;
    const int cols = 2 * mt;  // staged columns: token c/2, hi (even) or lo (odd)
    const MmaShared L = mma_layout(cols, kt, Q4, TR, NB, pair);
    __half* xs = reinterpret_cast<__half*>(smem + L.xs);
    __half* sxs = reinterpret_cast<__half*>(smem + L.sx);
    float* red = reinterpret_cast<float*>(smem + L.red);
    double* dred = reinterpret_cast<double*>(smem + L.meta);
    float* tokmeta = reinterpret_cast<float*>(smem + L.meta + 64 * 8);  // [token][0: norm scale, 1: 1/s]
    const int xcol = kt + MM_PAD, sxcol = kt / 32 + 8;

    const int rt = warp / KS, ks = warp % KS;
    const int row_tile0 = (blockIdx.x * TR + rt) * 16;
    const size_t rb = Q4 ? (size_t)(k / 256) * 144 : (((size_t)k + k / 16 + 15) & ~(size_t)15);
    const int n = (int)p.n;
    const int nparts = pair ? 2 : 1;

    // ---- per-token statistics: RMSNorm scale and the power-of-two range scale
    for (int tk = 0; tk < mt; tk++) {
        double ss;
        float am;
        cta_norm_stats(x + (size_t)(t0 + tk) * xr, norm_w, k, norm, dred, ss, am);
        if (tid == 0) {
            float nscale = 1.0f;
            if (norm) {
                const float mean = (float)(ss / (double)k);
                nscale = 1.0f / sqrtf(mean + p.eps);
            }
            const float amax = am * nscale;
            int e = 0;
            float s = 1.0f;
            if (amax > 0.f && amax < 3.0e38f) {
                frexpf(amax, &e);            // amax = f * 2^e, f in [0.5, 1)
                int sh = 14 - e;             // amax * 2^sh in [2^13, 2^14)
                sh = max(-100, min(100, sh));
                s = ldexpf(1.0f, sh);
            }
            tokmeta[2 * tk] = nscale;
            tokmeta[2 * tk + 1] = s;
        }
        __syncthreads();
    }

    float run[2][NB][4], mrun[2][NB][4];
#pragma unroll
    for (int a = 0; a < 2; a++)
#pragma unroll
        for (int b = 0; b < NB; b++)
#pragma unroll
            for (int c = 0; c < 4; c++) run[a][b][c] = mrun[a][b][c] = 0.f;

    const int units_total = Q4 ? k / 256 : k / 32;  // super-blocks (Q4_K) or blocks (Q8_0)
    const int unit_elems = Q4 ? 256 : 32;

    for (int k0 = 0; k0 < k; k0 += kt) {
        const int len = min(kt, k - k0);
        __syncthreads();
        // ---- stage x[k0 .. k0+len) of every token as f16 hi/lo in fragment order
        const int vecs = len / 4;
        for (int i = tid; i < mt * vecs; i += MM_THREADS) {
            const int tk = i / vecs, v = i % vecs;
            float4 a = reinterpret_cast<const float4*>(x + (size_t)(t0 + tk) * xr + k0)[v];
            if (norm) {
                const float4 nw = reinterpret_cast<const float4*>(norm_w + k0)[v];
                const float sc = tokmeta[2 * tk];
                a.x = __fmul_rn(__fmul_rn(a.x, sc), nw.x);
                a.y = __fmul_rn(__fmul_rn(a.y, sc), nw.y);
                a.z = __fmul_rn(__fmul_rn(a.z, sc), nw.z);
                a.w = __fmul_rn(__fmul_rn(a.w, sc), nw.w);
            }
            const float s = tokmeta[2 * tk + 1];
            const float e[4] = {a.x * s, a.y * s, a.z * s, a.w * s};
            __half* ch = xs + (size_t)(2 * tk) * xcol;
            __half* cl = ch + xcol;
            float part = 0.f;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const __half hi = __float2half_rn(e[q]);
                const __half lo = __float2half_rn((e[q] - __half2float(hi)) * 2048.0f);
                const int pos = stage_pos<TYPE>(4 * v + q);
                ch[pos] = hi;
                cl[pos] = lo;
                part = __fadd_rn(part, e[q]);
            }
            if (Q4) {
                // Sum over the 32 elements of a sub-block: 8 consecutive threads.
                part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, 1));
                part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, 2));
                part = __fadd_rn(part, __shfl_xor_sync(0xffffffffu, part, 4));
                if ((v & 7) == 0) {
                    const float m = part * (1.0f / 32.0f);
                    const __half hi = __float2half_rn(m);
                    const __half lo = __float2half_rn((m - __half2float(hi)) * 2048.0f);
                    sxs[(size_t)(2 * tk) * sxcol + (v >> 3)] = hi;
                    sxs[(size_t)(2 * tk + 1) * sxcol + (v >> 3)] = lo;
                }
            }
        }
        __syncthreads();

        const int u0 = k0 / unit_elems, u1 = (k0 + len) / unit_elems;
#pragma unroll
        for (int part = 0; part < 2; part++) {
            if (part >= nparts) break;
            const int jbase = (part ? (int)p.half : 0) + row_tile0;
            const int lim = (part ? (int)p.half : 0) + n - 1;
            const uint8_t* r0 = w + (size_t)min(jbase + g, lim) * rb;
            const uint8_t* r1 = w + (size_t)min(jbase + g + 8, lim) * rb;
            if (Q4) {
#pragma unroll 1
                for (int sb = u0 + ks; sb < u1; sb += KS) {
                    const uint8_t* b0 = r0 + (size_t)sb * 144;
                    const uint8_t* b1 = r1 + (size_t)sb * 144;
                    const uint4 h0 = *reinterpret_cast<const uint4*>(b0);
                    const uint4 h1 = *reinterpret_cast<const uint4*>(b1);
                    uint2 q0[4], q1[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        q0[j] = *reinterpret_cast<const uint2*>(b0 + 16 + 32 * j + 8 * t);
                        q1[j] = *reinterpret_cast<const uint2*>(b1 + 16 + 32 * j + 8 * t);
                    }
                    // 6-bit scales/mins of the 8 sub-blocks, four per register.
                    const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u)};
                    const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u)};
                    const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u)};
                    const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u)};
                    float acc[NB][4];
#pragma unroll
                    for (int b = 0; b < NB; b++) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f;
                    const int ebase = (sb - u0) * 256;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
#pragma unroll
                        for (int hi = 0; hi < 2; hi++) {
                            const int s = 2 * j + hi;  // sub-block
                            // {sc, sc} as f16, exactly: bytes -> 1024 + sc -> minus 1024.
                            const uint32_t sel = 0x4040u | (uint32_t)(s & 3) | ((uint32_t)(s & 3) << 8);
                            const uint32_t s0 = hsub2_u(__byte_perm(sc0[s >> 2], 0x64646464u, sel), H2_1024);
                            const uint32_t s1 = hsub2_u(__byte_perm(sc1[s >> 2], 0x64646464u, sel), H2_1024);
                            const uint32_t off = hi ? H2_M64 : H2_M1024;
                            const uint32_t n0 = hmul2_u(s0, off), n1 = hmul2_u(s1, off);
                            const uint32_t mask = hi ? 0x00f000f0u : 0x000f000fu;
                            const uint32_t magic = hi ? H2_64 : H2_1024;
                            // B fragments of this sub-block's 32 elements: 16 bytes per lane.
                            uint4 bv[NB];
#pragma unroll
                            for (int b = 0; b < NB; b++) {
                                const int col = 8 * b + g;
                                bv[b] = make_uint4(0, 0, 0, 0);
                                if (col < cols)
                                    bv[b] = *reinterpret_cast<const uint4*>(xs + (size_t)col * xcol + ebase + 32 * s + 8 * t);
                            }
#pragma unroll
                            for (int wv = 0; wv < 2; wv++) {
                                const uint32_t w0 = wv ? q0[j].y : q0[j].x;
                                const uint32_t w1 = wv ? q1[j].y : q1[j].x;
                                // (q + magic) * sc - magic * sc = q * sc, exact in f16 (q*sc <= 945).
                                const uint32_t a0 = hfma2_u(lop3_and_or(w0, mask, magic), s0, n0);
                                const uint32_t a1 = hfma2_u(lop3_and_or(w1, mask, magic), s1, n1);
                                const uint32_t a2 = hfma2_u(lop3_and_or(w0 >> 8, mask, magic), s0, n0);
                                const uint32_t a3 = hfma2_u(lop3_and_or(w1 >> 8, mask, magic), s1, n1);
#pragma unroll
                                for (int b = 0; b < NB; b++)
                                    mma_16816(acc[b], a0, a1, a2, a3, wv ? bv[b].z : bv[b].x, wv ? bv[b].w : bv[b].y);
                            }
                        }
                    }
                    // mins: A = {m[2t], m[2t+1]} of rows g and g+8, B = sub-block sums of x.
                    const uint32_t mr0 = (t < 2 ? mn0[0] : mn0[1]) >> (16 * (t & 1));
                    const uint32_t mr1 = (t < 2 ? mn1[0] : mn1[1]) >> (16 * (t & 1));
                    const uint32_t ma0 = hsub2_u(__byte_perm(mr0, 0x64646464u, 0x4140u), H2_1024);
                    const uint32_t ma1 = hsub2_u(__byte_perm(mr1, 0x64646464u, 0x4140u), H2_1024);
                    const float d0 = __half2float(__ushort_as_half((unsigned short)(h0.x & 0xffffu)));
                    const float d1 = __half2float(__ushort_as_half((unsigned short)(h1.x & 0xffffu)));
                    const float dm0 = __half2float(__ushort_as_half((unsigned short)(h0.x >> 16)));
                    const float dm1 = __half2float(__ushort_as_half((unsigned short)(h1.x >> 16)));
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const int col = 8 * b + g;
                        uint32_t bs = 0;
                        if (col < cols) bs = *reinterpret_cast<const uint32_t*>(sxs + (size_t)col * sxcol + (sb - u0) * 8 + 2 * t);
                        float am[4] = {0.f, 0.f, 0.f, 0.f};
                        mma_1688(am, ma0, ma1, bs);
                        run[part][b][0] = __fmaf_rn(d0, acc[b][0], run[part][b][0]);
                        run[part][b][1] = __fmaf_rn(d0, acc[b][1], run[part][b][1]);
                        run[part][b][2] = __fmaf_rn(d1, acc[b][2], run[part][b][2]);
                        run[part][b][3] = __fmaf_rn(d1, acc[b][3], run[part][b][3]);
                        mrun[part][b][0] = __fmaf_rn(dm0, am[0], mrun[part][b][0]);
                        mrun[part][b][1] = __fmaf_rn(dm0, am[1], mrun[part][b][1]);
                        mrun[part][b][2] = __fmaf_rn(dm1, am[2], mrun[part][b][2]);
                        mrun[part][b][3] = __fmaf_rn(dm1, am[3], mrun[part][b][3]);
                    }
                }
            } else {
                // Q8_0 split rows: 32 int8 per block; lane t holds bytes 8t..8t+7.
                const unsigned short* sc0p = reinterpret_cast<const unsigned short*>(r0 + k);
                const unsigned short* sc1p = reinterpret_cast<const unsigned short*>(r1 + k);
#pragma unroll 2
                for (int blk = u0 + ks; blk < u1; blk += KS) {
                    const uint2 q0 = *reinterpret_cast<const uint2*>(r0 + (size_t)blk * 32 + 8 * t);
                    const uint2 q1 = *reinterpret_cast<const uint2*>(r1 + (size_t)blk * 32 + 8 * t);
                    const float d0 = __half2float(__ushort_as_half(sc0p[blk]));
                    const float d1 = __half2float(__ushort_as_half(sc1p[blk]));
                    float acc[NB][4];
#pragma unroll
                    for (int b = 0; b < NB; b++) acc[b][0] = acc[b][1] = acc[b][2] = acc[b][3] = 0.f;
                    uint4 bv[NB];
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const int col = 8 * b + g;
                        bv[b] = make_uint4(0, 0, 0, 0);
                        if (col < cols)
                            bv[b] = *reinterpret_cast<const uint4*>(xs + (size_t)col * xcol + (blk - u0) * 32 + 8 * t);
                    }
#pragma unroll
                    for (int wv = 0; wv < 2; wv++) {
                        // int8 -> f16 exactly: flip the sign bit (q + 128), put each byte under 0x64
                        // (1024 + 128 + q), subtract 1152.
                        const uint32_t w0 = (wv ? q0.y : q0.x) ^ 0x80808080u;
                        const uint32_t w1 = (wv ? q1.y : q1.x) ^ 0x80808080u;
                        const uint32_t a0 = hsub2_u(__byte_perm(w0, 0x64646464u, 0x4140u), H2_1152);
                        const uint32_t a1 = hsub2_u(__byte_perm(w1, 0x64646464u, 0x4140u), H2_1152);
                        const uint32_t a2 = hsub2_u(__byte_perm(w0, 0x64646464u, 0x4342u), H2_1152);
                        const uint32_t a3 = hsub2_u(__byte_perm(w1, 0x64646464u, 0x4342u), H2_1152);
#pragma unroll
                        for (int b = 0; b < NB; b++)
                            mma_16816(acc[b], a0, a1, a2, a3, wv ? bv[b].z : bv[b].x, wv ? bv[b].w : bv[b].y);
                    }
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        run[part][b][0] = __fmaf_rn(d0, acc[b][0], run[part][b][0]);
                        run[part][b][1] = __fmaf_rn(d0, acc[b][1], run[part][b][1]);
                        run[part][b][2] = __fmaf_rn(d1, acc[b][2], run[part][b][2]);
                        run[part][b][3] = __fmaf_rn(d1, acc[b][3], run[part][b][3]);
                    }
                }
            }
        }
    }

    // ---- combine hi/lo, undo the range scale, reduce the k-splits in order, epilogue
    // red[part][warp][row 16][token 4*NB]
    const int tokslots = 4 * NB;
#pragma unroll
    for (int part = 0; part < 2; part++) {
        if (part >= nparts) break;
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int tk = 4 * b + t;
            const float inv_s = tk < mt ? 1.0f / tokmeta[2 * tk + 1] : 0.f;
            float v0 = __fmaf_rn(run[part][b][1], 1.0f / 2048.0f, run[part][b][0]);
            float v1 = __fmaf_rn(run[part][b][3], 1.0f / 2048.0f, run[part][b][2]);
            if (Q4) {
                const float m0 = __fmaf_rn(mrun[part][b][1], 1.0f / 2048.0f, mrun[part][b][0]);
                const float m1 = __fmaf_rn(mrun[part][b][3], 1.0f / 2048.0f, mrun[part][b][2]);
                v0 = __fmaf_rn(-32.0f, m0, v0);
                v1 = __fmaf_rn(-32.0f, m1, v1);
            }
            float* rr = red + ((size_t)(part * MM_WARPS + warp) * 16) * tokslots;
            rr[g * tokslots + tk] = v0 * inv_s;
            rr[(g + 8) * tokslots + tk] = v1 * inv_s;
        }
    }
    __syncthreads();
    for (int i = tid; i < TR * 16 * mt; i += MM_THREADS) {
        const int tk = i % mt, row = (i / mt) % 16, tile = i / (mt * 16);
        const int j = (blockIdx.x * TR + tile) * 16 + row;
        if (j >= n) continue;
        float v = 0.f, u = 0.f;
        for (int s = 0; s < KS; s++) {
            v = __fadd_rn(v, red[((size_t)(tile * KS + s) * 16 + row) * tokslots + tk]);
            if (pair) u = __fadd_rn(u, red[((size_t)(MM_WARPS + tile * KS + s) * 16 + row) * tokslots + tk]);
        }
        if (pair) v = silu_f(v) * u;
        const size_t o = (size_t)(t0 + tk) * p.out_stride + p.col0 + j;
        if (p.flags & MV_ACCUMULATE) v += out[o];
        out[o] = v;
    }
}

// ------------------------------------------------------------------ host side

struct MvArgs {
    PMatvec p;
    const float* x;
    const uint8_t* w;
    float* out;
    const float* nw;
    int m;
};

template <int TYPE>
zcu_result launch_scalar(const LaunchArgs& a, const MvArgs& v) {
    constexpr int ROWS = 2;
    const int rows_per_cta = (SC_THREADS / 32) * ROWS;
    const dim3 grid((v.p.n + rows_per_cta - 1) / rows_per_cta);
    for (int t0 = 0; t0 < v.m;) {
        const int left = v.m - t0;
        if (left >= 4) {
            matvec_scalar<TYPE, 4, ROWS><<<grid, SC_THREADS, 0, a.stream>>>(v.p, v.x, v.w, v.out, v.nw, t0);
            t0 += 4;
        } else if (left >= 2) {
            matvec_scalar<TYPE, 2, ROWS><<<grid, SC_THREADS, 0, a.stream>>>(v.p, v.x, v.w, v.out, v.nw, t0);
            t0 += 2;
        } else {
            matvec_scalar<TYPE, 1, ROWS><<<grid, SC_THREADS, 0, a.stream>>>(v.p, v.x, v.w, v.out, v.nw, t0);
            t0 += 1;
        }
        ZCU_CHECK_LAUNCH(a);
    }
    return ZCU_OK;
}

constexpr int MM_SMEM_BUDGET = 100 * 1024;

template <int TYPE, int KS, int NB>
zcu_result launch_mma_one(const LaunchArgs& a, const MvArgs& v, int t0, int mt) {
    constexpr int TR = MM_WARPS / KS;
    const bool q4 = TYPE == W_Q4_K, pair = (v.p.flags & MV_SILU_PAIR) != 0;
    const int cols = 2 * mt, k = (int)v.p.k;
    // Largest k tile (a multiple of 256) whose staging fits the budget.
    int kt = k;
    while (mma_layout(cols, kt, q4, TR, NB, pair).total > MM_SMEM_BUDGET && kt > 256) {
        kt = ((kt / 2 + 255) / 256) * 256;
    }
    const MmaShared L = mma_layout(cols, kt, q4, TR, NB, pair);
    auto kern = matvec_mma<TYPE, KS, NB>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM_BUDGET + 4096);
        if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "matvec_mma: shared memory attribute: %s", cudaGetErrorString(e));
        configured[dev & 63] = true;
    }
    const dim3 grid((v.p.n + 16 * TR - 1) / (16 * TR));
    kern<<<grid, MM_THREADS, L.total, a.stream>>>(v.p, v.x, v.w, v.out, v.nw, t0, mt, kt);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

template <int TYPE, int KS>
zcu_result launch_mma_ks(const LaunchArgs& a, const MvArgs& v) {
    for (int t0 = 0; t0 < v.m;) {
        const int left = v.m - t0;
        zcu_result r;
        if (left > 4) {
            const int mt = left < 8 ? left : 8;
            r = launch_mma_one<TYPE, KS, 2>(a, v, t0, mt);
            t0 += mt;
        } else {
            r = launch_mma_one<TYPE, KS, 1>(a, v, t0, left);
            t0 += left;
        }
        if (r != ZCU_OK) return r;
    }
    return ZCU_OK;
}

template <int TYPE>
zcu_result launch_mma(const LaunchArgs& a, const MvArgs& v, int ks) {
    switch (ks) {
        case 1: return launch_mma_ks<TYPE, 1>(a, v);
        case 2: return launch_mma_ks<TYPE, 2>(a, v);
        case 4: return launch_mma_ks<TYPE, 4>(a, v);
        case 8: return launch_mma_ks<TYPE, 8>(a, v);
        default: return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: split-K %d is not built", ks);
    }
}

// Default in-CTA split-K: enough CTAs to fill the device a few times over.
int default_ks(uint32_t n, int sm_count) {
    const int tiles = (int)((n + 15) / 16);
    int ks = 1;
    while (ks < 8 && tiles / (MM_WARPS / ks) < 3 * sm_count) ks *= 2;
    return ks;
}

zcu_result parse_matvec(const LaunchArgs& a, MvArgs& v, uint32_t elem_block, bool needs_256) {
    ZCU_NEED(a, a.params_bytes >= sizeof(PMatvec), "matvec: parameter block of %u bytes, need %zu", a.params_bytes, sizeof(PMatvec));
    memcpy(&v.p, a.params, sizeof(PMatvec));
    ZCU_NEED(a, a.nb >= 3, "matvec: %u bindings, need x, w, out", a.nb);
    const bool norm = (v.p.flags & MV_NORM) != 0;
    ZCU_NEED(a, !norm || a.nb >= 4, "matvec: NORM without a norm weight binding");
    v.x = static_cast<const float*>(a.b[0].ptr);
    v.w = static_cast<const uint8_t*>(a.b[1].ptr);
    v.out = static_cast<float*>(a.b[2].ptr);
    v.nw = a.nb >= 4 ? static_cast<const float*>(a.b[3].ptr) : nullptr;
    v.m = (int)a.grid[1];
    ZCU_NEED(a, v.m >= 1, "matvec: zero tokens");
    ZCU_NEED(a, v.p.k % elem_block == 0 && v.p.k > 0, "matvec: k = %u is not a multiple of %u", v.p.k, elem_block);
    ZCU_NEED(a, v.p.k % 8 == 0, "matvec: k = %u is not a multiple of 8", v.p.k);
    ZCU_NEED(a, ((uintptr_t)v.x & 15) == 0 && ((uintptr_t)v.w & 15) == 0, "matvec: x and w must be 16-byte aligned");
    ZCU_NEED(a, v.p.x_stride == 0 || v.p.x_stride * 4 >= v.p.k, "matvec: x_stride shorter than k");
    (void)needs_256;
    return ZCU_OK;
}

template <int TYPE>
zcu_result launch_quant(const LaunchArgs& a, uint32_t block) {
    MvArgs v;
    zcu_result r = parse_matvec(a, v, block, true);
    if (r != ZCU_OK) return r;
    if (v.p.n == 0) return ZCU_OK;
    const uint32_t family = (a.variant >> 16) & 0xffu;
    int ks = (int)((a.variant >> 8) & 0xffu);
    if (a.variant == 0 || family == ZCU_FAMILY_MMA) {
        if (ks == 0) ks = default_ks(v.p.n, a.sm_count);
        return launch_mma<TYPE>(a, v, ks);
    }
    if (family == ZCU_FAMILY_SCALAR) return launch_scalar<TYPE>(a, v);
    return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: variant 0x%x is not built", a.variant);
}

}  // namespace

bool matvec_variant_ok(uint32_t kernel, uint32_t variant) {
    const uint32_t family = (variant >> 16) & 0xffu, ks = (variant >> 8) & 0xffu;
    if (variant == 0) return true;
    if (variant >> 24) return false;
    if (kernel == ZCU_K_MATVEC_BF16 || kernel == ZCU_K_MATVEC_F16) return family == ZCU_FAMILY_SCALAR && ks == 0;
    if (family == ZCU_FAMILY_SCALAR) return ks == 0;
    if (family == ZCU_FAMILY_MMA) return ks == 0 || ks == 1 || ks == 2 || ks == 4 || ks == 8;
    return false;
}

zcu_result launch_matvec_q4_k(const LaunchArgs& a) { return launch_quant<W_Q4_K>(a, 256); }
zcu_result launch_matvec_q8_0(const LaunchArgs& a) { return launch_quant<W_Q8_0>(a, 32); }

zcu_result launch_matvec_bf16(const LaunchArgs& a) {
    MvArgs v;
    zcu_result r = parse_matvec(a, v, 8, false);
    if (r != ZCU_OK) return r;
    if (v.p.n == 0) return ZCU_OK;
    return launch_scalar<W_BF16>(a, v);
}
zcu_result launch_matvec_f16(const LaunchArgs& a) {
    MvArgs v;
    zcu_result r = parse_matvec(a, v, 8, false);
    if (r != ZCU_OK) return r;
    if (v.p.n == 0) return ZCU_OK;
    return launch_scalar<W_F16>(a, v);
}
