// Prefill multiply on half-precision weights with f32 activations, exact f32
// accumulation: out[t][col0 + j] (+)= sum_i x[t][i] * w[j][i]. Replaces the
// reference's matmul_bf16 / matmul_f16 (src/kernels/matmul_half.wgsl) with the
// same parameter block (params.MatmulBf16) and bindings x, w, out. Each
// output accumulates in i order whatever the step's token count, so a token's
// result does not depend on how the prompt was split into steps.
//
// This is the scalar identity (the reference's contract takes f32
// activations). The tensor-core rung that rounds activations to bf16 is a
// separate variant (k_matmul_tc.cu), selected like the reference's
// lower-precision prefill rungs (src/kernels/kernels.zig:798-822).

#include <cuda_fp16.h>

#include "zcu_internal.h"

namespace {

constexpr int BM = 64, BN = 64, BK = 32, MM_T = 256;

// The same tiles for Q8_0 weights without rounding the activations (matmul_q8_0_float, src/kernels/
// matmul_q8_0_float.wgsl): rows are k int8 values, then k / 32 f16 scales (repack_q8_0); a weight is
// f32(q) * f32(d), one rounding, as the CPU reference decodes it. Workgroup z sums positions
// [z * k_slice, (z + 1) * k_slice) and writes at z * slice_stride (params.MatmulQuant).
struct PMatmulQ8F {
    uint32_t rows, n, k, col0, out_stride, accumulate, k_slice, slice_stride;
};

__global__ void __launch_bounds__(256) matmul_q8_0_float_kernel(PMatmulQ8F p, const float* __restrict__ x, const uint8_t* __restrict__ w,
                                                               float* __restrict__ out, int tokens) {
    constexpr int BM = 64, BN = 64, BK = 32, MM_T = 256;
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int j0 = blockIdx.x * BN, t0 = blockIdx.y * BM, z = blockIdx.z;
    const int k = (int)p.k, n = (int)p.n;
    const size_t rb = ((size_t)k + k / 16 + 15) & ~(size_t)15;
    const int kb = min(k, z * (int)p.k_slice), ke = min(k, kb + (int)p.k_slice);
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.f;
    for (int k0 = kb; k0 < ke; k0 += BK) {
        for (int i = tid; i < BM * BK / 4; i += MM_T) {
            const int tr = i / (BK / 4), c4 = i % (BK / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + tr < tokens) v = *reinterpret_cast<const float4*>(x + (size_t)(t0 + tr) * k + k0 + 4 * c4);
            xs[4 * c4 + 0][tr] = v.x;
            xs[4 * c4 + 1][tr] = v.y;
            xs[4 * c4 + 2][tr] = v.z;
            xs[4 * c4 + 3][tr] = v.w;
        }
        for (int i = tid; i < BN * BK / 4; i += MM_T) {  // four int8 values of one row per thread
            const int jr = i / (BK / 4), c4 = i % (BK / 4);
            float d = 0.f;
            uint32_t q4 = 0;
            if (j0 + jr < n) {
                const uint8_t* row = w + (size_t)(j0 + jr) * rb;
                q4 = *reinterpret_cast<const uint32_t*>(row + k0 + 4 * c4);
                d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short*>(row + k + 2 * (k0 / 32))));
            }
#pragma unroll
            for (int e = 0; e < 4; e++) ws[4 * c4 + e][jr] = __fmul_rn((float)(int)(int8_t)((q4 >> (8 * e)) & 0xffu), d);
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < BK; i++) {
            const float4 xv = *reinterpret_cast<const float4*>(&xs[i][ty * 4]);
            const float4 wv = *reinterpret_cast<const float4*>(&ws[i][tx * 4]);
            const float xa[4] = {xv.x, xv.y, xv.z, xv.w}, wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++) acc[a][b] = __fmaf_rn(xa[a], wa[b], acc[a][b]);
        }
        __syncthreads();
    }
    float* dst = out + (size_t)z * p.slice_stride;
#pragma unroll
    for (int a = 0; a < 4; a++) {
        const int t = t0 + ty * 4 + a;
        if (t >= tokens) continue;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int j = j0 + tx * 4 + b;
            if (j >= n) continue;
            const size_t o = (size_t)t * p.out_stride + p.col0 + j;
            dst[o] = p.accumulate ? dst[o] + acc[a][b] : acc[a][b];
        }
    }
}

template <bool BF16>
__device__ __forceinline__ float widen(uint32_t bits16) {
    if (BF16) return __uint_as_float(bits16 << 16);
    return __half2float(__ushort_as_half((unsigned short)bits16));
}

// grid (ceil(n / 64), ceil(rows / 64)); thread (ty, tx) owns tokens ty*4.. and outputs tx*4...
template <bool BF16>
__global__ void __launch_bounds__(MM_T) matmul_half_kernel(PMatmulBf16 p, const float* __restrict__ x,
                                                          const uint16_t* __restrict__ w, float* __restrict__ out) {
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const int j0 = blockIdx.x * BN, t0 = blockIdx.y * BM;
    const int k = (int)p.k, rows = (int)p.rows, n = (int)p.n;
    float acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; a++)
#pragma unroll
        for (int b = 0; b < 4; b++) acc[a][b] = 0.f;
    for (int k0 = 0; k0 < k; k0 += BK) {
        // x tile: 64 tokens x 32 floats; thread loads 8 floats (two float4)
        for (int i = tid; i < BM * BK / 4; i += MM_T) {
            const int tr = i / (BK / 4), c4 = i % (BK / 4);
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if (t0 + tr < rows) v = *reinterpret_cast<const float4*>(x + (size_t)(t0 + tr) * k + k0 + 4 * c4);
            xs[4 * c4 + 0][tr] = v.x;
            xs[4 * c4 + 1][tr] = v.y;
            xs[4 * c4 + 2][tr] = v.z;
            xs[4 * c4 + 3][tr] = v.w;
        }
        // w tile: 64 outputs x 32 halves; thread loads 8 halves (one uint4)
        for (int i = tid; i < BN * BK / 8; i += MM_T) {
            const int jr = i / (BK / 8), c8 = i % (BK / 8);
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j0 + jr < n) v = *reinterpret_cast<const uint4*>(w + (size_t)(j0 + jr) * k + k0 + 8 * c8);
            const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; e++) {
                ws[8 * c8 + 2 * e][jr] = widen<BF16>(q[e] & 0xffffu);
                ws[8 * c8 + 2 * e + 1][jr] = widen<BF16>(q[e] >> 16);
            }
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < BK; i++) {
            const float4 xv = *reinterpret_cast<const float4*>(&xs[i][ty * 4]);
            const float4 wv = *reinterpret_cast<const float4*>(&ws[i][tx * 4]);
            const float xa[4] = {xv.x, xv.y, xv.z, xv.w}, wa[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int b = 0; b < 4; b++) acc[a][b] = __fmaf_rn(xa[a], wa[b], acc[a][b]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int a = 0; a < 4; a++) {
        const int t = t0 + ty * 4 + a;
        if (t >= rows) continue;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const int j = j0 + tx * 4 + b;
            if (j >= n) continue;
            const size_t o = (size_t)t * p.out_stride + p.col0 + j;
            float v = acc[a][b];
            if (p.accumulate) v += out[o];
            out[o] = v;
        }
    }
}

template <bool BF16>
zcu_result launch_half(const LaunchArgs& a) {
    PMatmulBf16 p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "matmul: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.k % BK == 0 && p.k > 0, "matmul: k = %u is not a multiple of %d", p.k, BK);
    if (p.rows == 0 || p.n == 0) return ZCU_OK;
    const dim3 grid((p.n + BN - 1) / BN, (p.rows + BM - 1) / BM);
    matmul_half_kernel<BF16><<<grid, MM_T, 0, a.stream>>>(p, (const float*)a.b[0].ptr, (const uint16_t*)a.b[1].ptr, (float*)a.b[2].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

}  // namespace

// Bindings x, w, out. The reference dispatches token tiles of 16 (grid y): the step's tokens are at most that many.
zcu_result launch_matmul_q8_0_float(const LaunchArgs& a) {
    PMatmulQ8F p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "matmul_q8_0_float: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.k % 32 == 0 && p.k > 0 && p.k_slice % 32 == 0 && p.k_slice > 0, "matmul_q8_0_float: k = %u, k_slice = %u (multiples of 32)", p.k, p.k_slice);
    const uint32_t cap = a.grid[1] * 16u;
    const int tokens = (int)(p.rows < cap ? p.rows : cap);
    if (tokens == 0 || p.n == 0) return ZCU_OK;
    const uint32_t slices = (p.k + p.k_slice - 1) / p.k_slice;
    const dim3 grid((p.n + 63) / 64, (tokens + 63) / 64, slices);
    matmul_q8_0_float_kernel<<<grid, 256, 0, a.stream>>>(p, (const float*)a.b[0].ptr, (const uint8_t*)a.b[1].ptr, (float*)a.b[2].ptr, tokens);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_matmul_bf16(const LaunchArgs& a) { return launch_half<true>(a); }
zcu_result launch_matmul_f16(const LaunchArgs& a) { return launch_half<false>(a); }
