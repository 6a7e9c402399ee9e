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
//   scalar  (this file) f32 activations from shared memory, f32 FMA on the CUDA
//           cores, warp-shuffle reduction in a fixed tree.
//   imma    (k_matvec_imma.cu) integer tensor-core fragments; the default.
//
// Every reduction has a fixed order, so a token's result does not depend on
// how many tokens the step has (the reference's step-split invariance,
// src/kernels/check.zig:1019-1031).
//
// Weight layouts: Q4_K rows as in the GGUF file (144-byte super-blocks,
// src/ref/tensor.zig:100-116); Q8_0 rows split by repack_q8_0 (k int8 values,
// then k/32 f16 scales, padded to 16 bytes: src/kernels/quant/q8_0.wgsl:1-24);
// BF16/F16 two per word (src/kernels/half/bf16.wgsl:3-9).

#include "k_matvec_common.cuh"

namespace {

using namespace mv;

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

// The other K-quants, in the layouts the reference's kernels read (kernels.blockStride, src/kernels/kernels.zig:
// 137-151): Q6_K blocks padded from 210 to 224 bytes by `repad`, Q5_K as in the file (176), Q3_K repacked by
// repack_q3_k into eight 16-byte units (128). Eight parts of 32 weights per 256-weight block; a weight is decoded
// with the CPU reference's roundings (src/ref/tensor.zig:54-160: the scale product first, then the value).
__device__ __forceinline__ void k4_scale_min(const uint8_t* s, int j, uint32_t& sc, uint32_t& m) {
    if (j < 4) {
        sc = s[j] & 63u, m = s[j + 4] & 63u;
    } else {
        sc = (s[j + 4] & 0xFu) | ((uint32_t)(s[j - 4] >> 6) << 4), m = (uint32_t)(s[j + 4] >> 4) | ((uint32_t)(s[j] >> 6) << 4);
    }
}

template <int MT>
struct BlockDot<W_Q6_K, MT> {
    static constexpr int BLOCK = 256, PARTS = 8;
    __device__ static size_t row_bytes(int k) { return (size_t)(k / 256) * 224; }
    __device__ static void run(const uint8_t* __restrict__ row, int /*k*/, int gblk, int part, const float* xs, int xs_stride, float* acc) {
        const uint8_t* b = row + (size_t)gblk * 224;
        const int n = part >> 2, c = part & 3;
        const uint4 l0 = *reinterpret_cast<const uint4*>(b + 64 * n + 32 * (c & 1)), l1 = *reinterpret_cast<const uint4*>(b + 64 * n + 32 * (c & 1) + 16);
        const uint4 h0 = *reinterpret_cast<const uint4*>(b + 128 + 32 * n), h1 = *reinterpret_cast<const uint4*>(b + 128 + 32 * n + 16);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(b + 208)));
        const int8_t* sc = reinterpret_cast<const int8_t*>(b + 192 + 8 * n + 2 * c);
        const float ds0 = __fmul_rn(d, (float)sc[0]), ds1 = __fmul_rn(d, (float)sc[1]);
        const uint32_t lw[8] = {l0.x, l0.y, l0.z, l0.w, l1.x, l1.y, l1.z, l1.w}, hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
        const int ls = 4 * (c >> 1), hs = 2 * c;
#pragma unroll
        for (int t = 0; t < MT; t++) {
            const float* xv = xs + (size_t)t * xs_stride + 32 * part;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int v = 0; v < 8; v++) {
                const float4 a = *reinterpret_cast<const float4*>(xv + 4 * v);
                const uint32_t q = ((lw[v] >> ls) & 0x0f0f0f0fu) | (((hw[v] >> hs) & 0x03030303u) << 4);
                float& s = v < 4 ? s0 : s1;
                s = __fmaf_rn(a.x, (float)((int)(q & 0xffu) - 32), s);
                s = __fmaf_rn(a.y, (float)((int)((q >> 8) & 0xffu) - 32), s);
                s = __fmaf_rn(a.z, (float)((int)((q >> 16) & 0xffu) - 32), s);
                s = __fmaf_rn(a.w, (float)((int)(q >> 24) - 32), s);
            }
            acc[t] = __fmaf_rn(ds1, s1, __fmaf_rn(ds0, s0, acc[t]));
        }
    }
};

template <int MT>
struct BlockDot<W_Q5_K, MT> {
    static constexpr int BLOCK = 256, PARTS = 8;
    __device__ static size_t row_bytes(int k) { return (size_t)(k / 256) * 176; }
    __device__ static void run(const uint8_t* __restrict__ row, int /*k*/, int gblk, int part, const float* xs, int xs_stride, float* acc) {
        const uint8_t* b = row + (size_t)gblk * 176;
        const int j = part >> 1, hi = part & 1;
        const uint4 q0 = *reinterpret_cast<const uint4*>(b + 48 + 32 * j), q1 = *reinterpret_cast<const uint4*>(b + 48 + 32 * j + 16);
        const uint4 h0 = *reinterpret_cast<const uint4*>(b + 16), h1 = *reinterpret_cast<const uint4*>(b + 32);
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(b)));
        const float dmin = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(b + 2)));
        uint32_t sc, mn;
        k4_scale_min(b + 4, part, sc, mn);
        const float d1 = __fmul_rn(d, (float)sc), m1 = __fmul_rn(dmin, (float)mn);
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w}, hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
#pragma unroll
        for (int t = 0; t < MT; t++) {
            const float* xv = xs + (size_t)t * xs_stride + 32 * part;
            float s = 0.f, xsum = 0.f;
#pragma unroll
            for (int v = 0; v < 8; v++) {
                const float4 a = *reinterpret_cast<const float4*>(xv + 4 * v);
                const uint32_t q = ((qw[v] >> (4 * hi)) & 0x0f0f0f0fu) | (((hw[v] >> part) & 0x01010101u) << 4);
                s = __fmaf_rn(a.x, (float)(q & 0xffu), s);
                s = __fmaf_rn(a.y, (float)((q >> 8) & 0xffu), s);
                s = __fmaf_rn(a.z, (float)((q >> 16) & 0xffu), s);
                s = __fmaf_rn(a.w, (float)(q >> 24), s);
                xsum = __fadd_rn(xsum, __fadd_rn(__fadd_rn(a.x, a.y), __fadd_rn(a.z, a.w)));
            }
            acc[t] = __fmaf_rn(-m1, xsum, __fmaf_rn(d1, s, acc[t]));
        }
    }
};

template <int MT>
struct BlockDot<W_Q3_K, MT> {
    static constexpr int BLOCK = 256, PARTS = 8;
    __device__ static size_t row_bytes(int k) { return (size_t)(k / 256) * 128; }
    __device__ static void run(const uint8_t* __restrict__ row, int /*k*/, int gblk, int part, const float* xs, int xs_stride, float* acc) {
        // one repacked unit (src/kernels/repack_q3_k.wgsl): two words of 2-bit values, one of high bits, two scales
        // minus 32 as signed bytes, d
        const uint4 u = *reinterpret_cast<const uint4*>(row + (size_t)gblk * 128 + 16 * part);
        const float d = __half2float(__ushort_as_half((unsigned short)(u.w >> 16)));
        const float dl0 = __fmul_rn(d, (float)(int)(int8_t)(u.w & 0xffu)), dl1 = __fmul_rn(d, (float)(int)(int8_t)((u.w >> 8) & 0xffu));
#pragma unroll
        for (int t = 0; t < MT; t++) {
            const float* xv = xs + (size_t)t * xs_stride + 32 * part;
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int e = 0; e < 8; e++) {   // weights 4e .. 4e + 3: byte b of the word holds position 4e + b
                const float4 a = *reinterpret_cast<const float4*>(xv + 4 * e);
                const uint32_t q = ((e < 4 ? u.x : u.y) >> (2 * (e & 3))) & 0x03030303u;
                const uint32_t h = (u.z >> e) & 0x01010101u;
                float& s = e < 4 ? s0 : s1;
                s = __fmaf_rn(a.x, (float)((int)(q & 0xffu) - ((h & 1u) ? 0 : 4)), s);
                s = __fmaf_rn(a.y, (float)((int)((q >> 8) & 0xffu) - (((h >> 8) & 1u) ? 0 : 4)), s);
                s = __fmaf_rn(a.z, (float)((int)((q >> 16) & 0xffu) - (((h >> 16) & 1u) ? 0 : 4)), s);
                s = __fmaf_rn(a.w, (float)((int)(q >> 24) - (((h >> 24) & 1u) ? 0 : 4)), s);
            }
            acc[t] = __fmaf_rn(dl1, s1, __fmaf_rn(dl0, s0, acc[t]));
        }
    }
};

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

// ------------------------------------------------------------------ host side

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
    {
        // the rows this launch writes: [col0, col0 + n) of m output rows
        const float* lo = v.out + v.p.col0;
        const float* hi = v.out + (size_t)(v.m - 1) * v.p.out_stride + v.p.col0 + v.p.n;
        zcu_result pr = parse_peer(a, v.peer, lo, hi);
        if (pr != ZCU_OK) return pr;
    }
    v.has_rope = (v.p.flags & MV_ROPE_APPEND) != 0;
    if (v.has_rope) {
        // an extension: rope_append fused into the multiply that produces the Q|K|V row. The parameter block is
        // PMatvec followed by params.RopeAppend; bindings 4.. are rope_append's table, kc, vc, step[, positions].
        ZCU_NEED(a, a.params_bytes >= sizeof(PMatvec) + sizeof(PRopeAppend) && a.nb >= 8, "matvec + rope_append: parameter block or bindings too short");
        memcpy(&v.rope.p, static_cast<const char*>(a.params) + sizeof(PMatvec), sizeof(PRopeAppend));
        const PRopeAppend& r = v.rope.p;
        ZCU_NEED(a, r.normal == 1 && r.qk_norm == 0, "matvec + rope_append: only adjacent-pair RoPE without q/k norms is fused");
        ZCU_NEED(a, r.head_dim % 2 == 0 && r.n_rot % 2 == 0 && r.n_rot <= r.head_dim && (r.kv == KV_F32 || r.kv == KV_F16), "matvec + rope_append: head_dim %u n_rot %u cache %u", r.head_dim, r.n_rot, r.kv);
        ZCU_NEED(a, v.m == 1 || v.m == 2 || v.m == 4, "matvec + rope_append: %d tokens (1, 2 or 4)", v.m);
        ZCU_NEED(a, v.p.col0 % 2 == 0 && v.p.n % 2 == 0 && !(v.p.flags & (MV_SILU_PAIR | MV_ACCUMULATE)), "matvec + rope_append: odd column range or conflicting flags");
        v.rope.table = static_cast<const float2*>(a.b[4].ptr);
        v.rope.kc = a.b[5].ptr;
        v.rope.vc = a.b[6].ptr;
        v.rope.step = static_cast<const PStep*>(a.b[7].ptr);
        v.rope.seq_pos = (a.nb >= 9 && r._pad[0] != 0) ? static_cast<const uint32_t*>(a.b[8].ptr) : nullptr;
    }
    memset(&v.combine, 0, sizeof(v.combine));
    if (v.p.flags & MV_ATTN_COMBINE) {
        // an extension: attn_combine as a first phase of the multiply that reads the attention output. The
        // parameter block is PMatvec followed by params.Attention; bindings 4.. are attn_combine's qg, part, out,
        // step[, positions]. The merged heads reach the multiply's other CTAs through the exchange slots of its own
        // wait_slot, so the dispatch must take its input from an exchange.
        ZCU_NEED(a, !v.has_rope && a.params_bytes >= sizeof(PMatvec) + sizeof(PAttention) && a.nb >= 8, "matvec + attn_combine: parameter block or bindings too short");
        ZCU_NEED(a, v.peer.wait_slot != PEER_NONE, "matvec + attn_combine: the multiply must read its input from an exchange (zcu_peer_ext.wait_slot)");
        MvCombine& c = v.combine;
        memcpy(&c.p, static_cast<const char*>(a.params) + sizeof(PMatvec), sizeof(PAttention));
        ZCU_NEED(a, c.p.head_dim <= 256 && c.p.heads > 0 && c.p.max_blocks > 0 && c.p.max_blocks <= 1024, "matvec + attn_combine: head_dim %u, %u heads, max_blocks %u", c.p.head_dim, c.p.heads, c.p.max_blocks);
        c.qg = static_cast<const float*>(a.b[4].ptr);
        c.part = static_cast<const float*>(a.b[5].ptr);
        c.out = static_cast<float*>(a.b[6].ptr);
        c.step = static_cast<const PStep*>(a.b[7].ptr);
        c.seq_pos = (a.nb >= 9 && c.p._pad[0] != 0) ? static_cast<const uint32_t*>(a.b[8].ptr) : nullptr;
        c.kb = attn_keys_per_block(c.p);
        c.blocks = (int)c.p.heads * v.m;
        {
            // the merged heads are pushed as the exchange the multiply waits for: they must lie inside the local arena
            const size_t orow = c.p._pad[1] ? (size_t)c.p._pad[1] : (size_t)c.p.heads * c.p.head_dim;
            const uint64_t lo = reinterpret_cast<uint64_t>(c.out + (size_t)c.p.row0 * orow);
            const uint64_t hi = lo + 4 * ((size_t)(v.m - 1) * orow + (size_t)c.p.heads * c.p.head_dim), base = v.peer.t.base[v.peer.t.rank];
            ZCU_NEED(a, lo >= base && hi <= base + v.peer.t.ll_off, "matvec + attn_combine: the attention output is not inside the local arena");
        }
    }
    return ZCU_OK;
}

template <int TYPE>
zcu_result launch_quant(const LaunchArgs& a, uint32_t block) {
    MvArgs v;
    zcu_result r = parse_matvec(a, v, block, true);
    if (r != ZCU_OK) return r;
    if (v.p.n == 0) return ZCU_OK;
    const uint32_t family = (a.variant >> 16) & 0xffu;
    if (family == ZCU_FAMILY_TCGEN05) {
        if (TYPE != W_Q4_K) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: the tcgen05 family is built for Q4_K only");
        return launch_matvec_q4_k_tc(a, v);
    }
    // Q8_0 rows that are not whole 256-weight pieces have ragged tiles: the scalar family takes them.
    const bool imma_ok = TYPE != W_Q8_0 || v.p.k % 256 == 0;
    // The default of Q4_K is what the sweep ends up choosing for every shape of a decode step: a ring of three tiles
    // and a CTA on every SM (a shorter ring means fewer requests in front of the activation staging, and the CTAs
    // that end a row tile early let the next kernel's CTAs in early).
    if (a.variant == 0 && imma_ok && TYPE == W_Q4_K) return launch_matvec_imma(a, v, TYPE, 3, 0x10);
    if ((a.variant == 0 && imma_ok) || family == ZCU_FAMILY_MMA)
        return launch_matvec_imma(a, v, TYPE, (int)(a.variant & 0xffu), (int)((a.variant >> 8) & 0xffu));
    if (v.has_rope) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec + rope_append: only the tensor-core family fuses it");
    if (v.combine.blocks) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec + attn_combine: only the tensor-core family fuses it");
    if (v.peer.wait_slot != PEER_NONE || v.peer.push_slot != PEER_NONE)
        return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec in a peer exchange: only the tensor-core family takes part");
    if (a.variant == 0) return launch_scalar<TYPE>(a, v);
    if (family == ZCU_FAMILY_SCALAR) return launch_scalar<TYPE>(a, v);
    return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: variant 0x%x is not built", a.variant);
}

}  // namespace

bool matvec_variant_ok(uint32_t kernel, uint32_t variant) {
    const uint32_t family = (variant >> 16) & 0xffu, ks = (variant >> 8) & 0xffu;
    if (variant == 0) return true;
    if (variant >> 24) return false;
    if (kernel == ZCU_K_MATVEC_BF16 || kernel == ZCU_K_MATVEC_F16 || kernel == ZCU_K_MATVEC_Q3_K || kernel == ZCU_K_MATVEC_Q5_K ||
        kernel == ZCU_K_MATVEC_Q6_K)
        return family == ZCU_FAMILY_SCALAR && ks == 0;
    if (family == ZCU_FAMILY_SCALAR) return ks == 0;
    if (family == ZCU_FAMILY_MMA) {
        const uint32_t stages = variant & 0xffu;
        return (ks & ~0x11u) == 0 && (stages == 0 || (stages >= 2 && stages <= 6));   // ks: CTA shape | every-SM bit
    }
    if (family == ZCU_FAMILY_TCGEN05) return kernel == ZCU_K_MATVEC_Q4_K && (variant & 0xffffu) == 0;
    return false;
}

zcu_result launch_matvec_q4_k(const LaunchArgs& a) { return launch_quant<W_Q4_K>(a, 256); }
zcu_result launch_matvec_q8_0(const LaunchArgs& a) { return launch_quant<W_Q8_0>(a, 32); }

// Q3_K (repacked), Q5_K and Q6_K (padded): the scalar family only.
template <int TYPE>
static zcu_result launch_kquant(const LaunchArgs& a) {
    MvArgs v;
    zcu_result r = parse_matvec(a, v, 256, true);
    if (r != ZCU_OK) return r;
    if (v.p.n == 0) return ZCU_OK;
    if (v.has_rope || v.combine.blocks || v.peer.wait_slot != PEER_NONE || v.peer.push_slot != PEER_NONE)
        return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: this weight type runs the scalar family, which takes no fused rope_append or peer exchange");
    return launch_scalar<TYPE>(a, v);
}
zcu_result launch_matvec_q3_k(const LaunchArgs& a) { return launch_kquant<W_Q3_K>(a); }
zcu_result launch_matvec_q5_k(const LaunchArgs& a) { return launch_kquant<W_Q5_K>(a); }
zcu_result launch_matvec_q6_k(const LaunchArgs& a) { return launch_kquant<W_Q6_K>(a); }

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
