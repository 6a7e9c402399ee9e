// The quantised prefill family: quantize_q8, matmul_q4_k, matmul_q8_0, matmul_reduce.
//
// The reference's prefill for quantised models multiplies as llama.cpp's CPU backend does (src/kernels/
// quantize_q8.wgsl, matmul_quant.wgsl; oracle: roundLikeLlama + matmul, src/ref/matmul.zig:203-258): activations
// are rounded to 8-bit blocks (Q8_K: 256 values, d = 1 / (-127 / max); Q8_0: 32 values, d = f16(amax / 127)), each
// 32-weight unit's dot product is exact in integers, then scaled:
//   out[t][j] = sum over blocks of dx[t][blk] * (d_w * sum_s sc_s (q . qx)_s - dmin_w * sum_s m_s * (sum qx)_s).
// Same parameter blocks (params.QuantizeQ8, MatmulQuant, MatmulReduce) and bindings as the reference:
//   quantize_q8: x, qx (rw), dx (rw), nw      grid (k / 256, rows)
//   matmul_q*:   qx, w, out (rw), dx          grid (n tiles, token tiles of 32, k slices)
//   matmul_reduce: partials, out (rw)
//
// The multiplies run on the integer tensor cores (mma.sync.m16n8k32.s8): a CTA of 8 warps owns 128 output rows x
// 64 tokens; per 256-weight step its weight rows (one TMA box, as in the decode multiply) and the tokens' int8
// activations (cp.async, rows padded for conflict-free fragment reads) are double-buffered in shared memory; warp w
// multiplies rows 16 w .. 16 w + 15 by all 64 tokens: per 32-weight unit one IMMA per 8 tokens, the 6-bit unit
// scale applied to the exact s32 sums in integers, the Q4_K min term as two more IMMAs per 8 tokens (6-bit mins
// against the two balanced digits of each unit's sum of qx), and once per 256 weights the step's integers meet
// the f16 super-scales and the token's f32 block scale. Every wait is bounded.

#include <cuda_fp16.h>

#include "imma_util.cuh"
#include "k_matvec_common.cuh"
#include "tma_util.cuh"

namespace {

using namespace imma;
using namespace mv;

// ---------------------------------------------------------------------------------------------- quantize_q8
struct PQuantize {  // kernels.zig:495-501
    uint32_t k, block, mode;
    float eps;
};

__global__ void __launch_bounds__(64) quantize_q8_kernel(PQuantize p, const float* __restrict__ x, int8_t* __restrict__ qx,
                                                        float* __restrict__ dx, const float* __restrict__ nw) {
    __shared__ double red[2];
    __shared__ float best_v[64];
    __shared__ int best_i[64];
    __shared__ float vals[256];
    const int li = threadIdx.x, chunk = blockIdx.x, row = blockIdx.y, k = (int)p.k;
    float4 v;
    if (p.mode == 2) {  // silu(gate) * up over rows of gate | up
        const float4 g = reinterpret_cast<const float4*>(x + (size_t)row * 2 * k)[chunk * 64 + li];
        const float4 u = reinterpret_cast<const float4*>(x + (size_t)row * 2 * k + k)[chunk * 64 + li];
        v = make_float4(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y, g.z / (1.0f + expf(-g.z)) * u.z,
                        g.w / (1.0f + expf(-g.w)) * u.w);
    } else {
        v = reinterpret_cast<const float4*>(x + (size_t)row * k)[chunk * 64 + li];
    }
    if (p.mode == 1) {  // RMSNorm(x) * w: f32 squares summed in f64 (src/ref/ops.zig:30-41)
        double ss = 0.0;
        for (int i = li; i < k / 4; i += 64) {
            const float4 r = reinterpret_cast<const float4*>(x + (size_t)row * k)[i];
            ss += (double)__fmul_rn(r.x, r.x);
            ss += (double)__fmul_rn(r.y, r.y);
            ss += (double)__fmul_rn(r.z, r.z);
            ss += (double)__fmul_rn(r.w, r.w);
        }
        ss = warp_sum_d(ss);
        if ((li & 31) == 0) red[li >> 5] = ss;
        __syncthreads();
        const float mean = (float)((red[0] + red[1]) / (double)k);
        const float scale = 1.0f / sqrtf(mean + p.eps);
        const float4 w = reinterpret_cast<const float4*>(nw)[chunk * 64 + li];
        v.x = __fmul_rn(__fmul_rn(v.x, scale), w.x);
        v.y = __fmul_rn(__fmul_rn(v.y, scale), w.y);
        v.z = __fmul_rn(__fmul_rn(v.z, scale), w.z);
        v.w = __fmul_rn(__fmul_rn(v.w, scale), w.w);
    }
    vals[4 * li] = v.x, vals[4 * li + 1] = v.y, vals[4 * li + 2] = v.z, vals[4 * li + 3] = v.w;
    // the value of largest magnitude of each block, the first on ties
    float m = fabsf(v.x);
    int at = 4 * li;
    if (fabsf(v.y) > m) m = fabsf(v.y), at = 4 * li + 1;
    if (fabsf(v.z) > m) m = fabsf(v.z), at = 4 * li + 2;
    if (fabsf(v.w) > m) m = fabsf(v.w), at = 4 * li + 3;
    best_v[li] = m, best_i[li] = at;
    __syncthreads();
    const int span = (int)p.block / 4;  // threads per block: 64 (Q8_K) or 8 (Q8_0)
    for (int s = span / 2; s > 0; s /= 2) {
        if (li % span < s) {
            const float ov = best_v[li + s];
            const int oi = best_i[li + s];
            if (ov > best_v[li] || (ov == best_v[li] && oi < best_i[li])) best_v[li] = ov, best_i[li] = oi;
        }
        __syncthreads();
    }
    const int lead = li - li % span;
    const float amax = best_v[lead];
    int q[4] = {0, 0, 0, 0};
    float d = 0.f;
    if (amax != 0.f) {
        if (p.block == 256) {
            const float mx = vals[best_i[lead]];
            const float iscale = __fdiv_rn(-127.0f, mx);
            d = __fdiv_rn(1.0f, iscale);
            q[0] = min(127, __float2int_rn(__fmul_rn(iscale, v.x)));
            q[1] = min(127, __float2int_rn(__fmul_rn(iscale, v.y)));
            q[2] = min(127, __float2int_rn(__fmul_rn(iscale, v.z)));
            q[3] = min(127, __float2int_rn(__fmul_rn(iscale, v.w)));
        } else {
            const float id = __fdiv_rn(127.0f, amax);
            d = __half2float(__float2half_rn(__fdiv_rn(amax, 127.0f)));
            q[0] = __float2int_rn(__fmul_rn(v.x, id));
            q[1] = __float2int_rn(__fmul_rn(v.y, id));
            q[2] = __float2int_rn(__fmul_rn(v.z, id));
            q[3] = __float2int_rn(__fmul_rn(v.w, id));
        }
    }
    const uint32_t word = ((uint32_t)q[0] & 0xffu) | (((uint32_t)q[1] & 0xffu) << 8) | (((uint32_t)q[2] & 0xffu) << 16) | (((uint32_t)q[3] & 0xffu) << 24);
    reinterpret_cast<uint32_t*>(qx + (size_t)row * k)[chunk * 64 + li] = word;
    if (li % span == 0) dx[((size_t)row * k + (size_t)chunk * 256 + 4 * li) / p.block] = d;
}

// ---------------------------------------------------------------------------------------------- matmul_q4_k / q8_0
struct PMatmulQ {  // kernels.zig:452-461
    uint32_t rows, n, k, col0, out_stride, accumulate, k_slice, slice_stride;
};
struct PMatmulReduceQ {  // kernels.zig:462-471
    uint32_t rows, n, slices, col0, out_stride, accumulate, slice_stride, _pad;
};

constexpr int QM_ROWS = 128, QM_TOK = 64, QM_THREADS = 256;
constexpr int QM_WTILE = QM_ROWS * TILE_ROW;   // 128 rows x 160 bytes: a Q4_K super-block, or 128 Q8_0 values (+ spare)
constexpr int QM_WSCALES = QM_ROWS * 16;       // Q8_0: the 16 bytes that hold the step's four scales, per row

template <int TYPE>
struct QmShape {
    static constexpr bool Q4 = TYPE == W_Q4_K;
    static constexpr int KSTEP = Q4 ? 256 : 128;            // weights of a row per step
    static constexpr int XROW = KSTEP + 32;                 // bytes between the tokens' rows (conflict-free 8-byte reads)
    static constexpr int XTILE = QM_TOK * XROW;
    static constexpr int STAGE = QM_WTILE + QM_WSCALES + XTILE;
    static constexpr int SUMS = 2 * QM_TOK * 8;             // two balanced digits of each (token, unit) sum of qx
    static constexpr int DXS = QM_TOK * 4 * 4;              // f32 scales of the step's activation blocks, per token
    static constexpr int SMEM = 2 * (STAGE + SUMS + DXS) + 64;
};

// grid (ceil(n / 128), ceil(tokens / 64), k slices); 8 warps: warp w owns rows 16 w .. 16 w + 15 of the CTA's 128.
template <int TYPE>
__global__ void __launch_bounds__(QM_THREADS, 2) matmul_quant_kernel(PMatmulQ p, const __grid_constant__ CUtensorMap wmap,
                                                                    const __grid_constant__ CUtensorMap smap,
                                                                    const int8_t* __restrict__ qx, float* __restrict__ out,
                                                                    const float* __restrict__ dx, int tokens,
                                                                    int* __restrict__ status) {
    using S = QmShape<TYPE>;
    constexpr bool Q4 = S::Q4;
    constexpr int KSTEP = S::KSTEP, XROW = S::XROW;
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t = lane & 3;
    const int j0 = blockIdx.x * QM_ROWS, t0 = blockIdx.y * QM_TOK, z = (int)blockIdx.z;
    const int k = (int)p.k, n = (int)p.n;
    const int k_lo = (int)min((unsigned long long)k, (unsigned long long)z * p.k_slice);
    const int k_hi = (int)min((unsigned long long)k, ((unsigned long long)z + 1) * p.k_slice);
    const int step_lo = k_lo / KSTEP, step_hi = k_hi / KSTEP;
    const uint32_t s0 = (uint32_t)__cvta_generic_to_shared(smem);
    uint8_t* aux = smem + 2 * S::STAGE;                      // per stage: sums, then dx
    const uint32_t bar_s = s0 + 2 * (S::STAGE + S::SUMS + S::DXS);
    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_s + 8, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    // step `st` into stage `sg`: thread 0 asks for the weight boxes, every thread copies its pieces of the tokens'
    // activations, threads 0..63 fetch the tokens' block scales
    auto issue = [&](int st, int sg) {
        const uint32_t base = s0 + (uint32_t)sg * S::STAGE;
        if (tid == 0) {
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            if (Q4) {
                mbar_expect_tx(bar_s + 8 * sg, QM_WTILE);
                tma_tile(base, &wmap, st * 144, j0, bar_s + 8 * sg);
            } else {
                mbar_expect_tx(bar_s + 8 * sg, QM_WTILE + QM_WSCALES);
                tma_tile(base, &wmap, st * 128, j0, bar_s + 8 * sg);
                tma_tile(base + QM_WTILE, &smap, k + 2 * ((st * 4) & ~7), j0, bar_s + 8 * sg);
            }
        }
        constexpr int PIECES = KSTEP / 16;
        for (int i = tid; i < QM_TOK * PIECES; i += QM_THREADS) {
            const int tok = i / PIECES, piece = i % PIECES;
            const int8_t* src = qx + (size_t)min(t0 + tok, tokens - 1) * k + (size_t)st * KSTEP + 16 * piece;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(base + QM_WTILE + QM_WSCALES + (uint32_t)tok * XROW + 16u * piece), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        if (tid < QM_TOK) {
            float* dst = reinterpret_cast<float*>(aux + sg * (S::SUMS + S::DXS) + S::SUMS) + 4 * tid;
            const size_t row = (size_t)min(t0 + tid, tokens - 1);
            if (Q4) {
                dst[0] = dx[row * (k / 256) + st];
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) dst[i] = dx[row * (k / 32) + (size_t)st * 4 + i];
            }
        }
    };

    float accf[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; nb++) accf[nb][0] = accf[nb][1] = accf[nb][2] = accf[nb][3] = 0.f;
    bool timed_out = false;
    uint32_t phases = 0;
    if (step_lo < step_hi) issue(step_lo, 0);
    for (int st = step_lo; st < step_hi; st++) {
        const int sg = (st - step_lo) & 1;
        if (st + 1 < step_hi) {
            issue(st + 1, sg ^ 1);  // the other stage was released by the barrier that ended the step before
            asm volatile("cp.async.wait_group 1;\n" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        }
        if (!mbar_wait(bar_s + 8 * sg, (phases >> sg) & 1u)) timed_out = true;
        phases ^= 1u << sg;
        __syncthreads();
        const uint32_t wt = s0 + (uint32_t)sg * S::STAGE, xt = wt + QM_WTILE + QM_WSCALES;
        int8_t* sums = reinterpret_cast<int8_t*>(aux + sg * (S::SUMS + S::DXS));
        const float* dxs = reinterpret_cast<const float*>(aux + sg * (S::SUMS + S::DXS) + S::SUMS);
        const uint32_t wrow0 = wt + (uint32_t)(16 * warp + g) * TILE_ROW, wrow1 = wrow0 + 8 * TILE_ROW;
        if constexpr (Q4) {
            // the sum of each (token, unit)'s 32 activations as two balanced byte digits
            for (int i = tid; i < QM_TOK * 8; i += QM_THREADS) {
                const int tok = i >> 3, unit = i & 7;
                int sum = 0;
#pragma unroll
                for (int w4 = 0; w4 < 8; w4++) {
                    uint32_t word;
                    asm volatile("ld.shared.u32 %0, [%1];\n" : "=r"(word) : "r"(xt + (uint32_t)tok * XROW + 32u * unit + 4u * w4));
                    sum = __dp4a((int)word, 0x01010101, sum);
                }
                sums[tok * 8 + unit] = (int8_t)(sum & 0xff);
                sums[QM_TOK * 8 + tok * 8 + unit] = (int8_t)((sum + 128) >> 8);
            }
            __syncthreads();
            const uint4 h0 = lds128(wrow0), h1 = lds128(wrow1);
            const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u)};
            const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u)};
            const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u)};
            const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u)};
            int run[8][4];
#pragma unroll
            for (int nb = 0; nb < 8; nb++) run[nb][0] = run[nb][1] = run[nb][2] = run[nb][3] = 0;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 q0 = lds64(wrow0 + 16 + 8 * t + 32 * j), q1 = lds64(wrow1 + 16 + 8 * t + 32 * j);
#pragma unroll
                for (int hi_n = 0; hi_n < 2; hi_n++) {
                    const int s = 2 * j + hi_n, sh = hi_n ? 4 : 0;
                    // the lane's eight codes of unit s, rows g and g + 8: elements 8 t .. 8 t + 7 of the unit
                    const uint32_t a0 = (q0.x >> sh) & 0x0f0f0f0fu, a1 = (q1.x >> sh) & 0x0f0f0f0fu;
                    const uint32_t a2 = (q0.y >> sh) & 0x0f0f0f0fu, a3 = (q1.y >> sh) & 0x0f0f0f0fu;
                    const int u0 = (int)__byte_perm(sc0[s >> 2], 0u, 0x4440 | (s & 3));
                    const int u1 = (int)__byte_perm(sc1[s >> 2], 0u, 0x4440 | (s & 3));
#pragma unroll
                    for (int nb = 0; nb < 8; nb++) {
                        const uint2 b = lds64(xt + (uint32_t)(8 * nb + g) * XROW + 32u * s + 8u * t);  // the same eight elements
                        int acc[4];
                        imma_16832(acc, a0, a1, a2, a3, b.x, b.y);
                        run[nb][0] += acc[0] * u0;
                        run[nb][1] += acc[1] * u0;
                        run[nb][2] += acc[2] * u1;
                        run[nb][3] += acc[3] * u1;
                    }
                }
            }
            // mins: lanes t = 0, 1 carry the eight 6-bit mins of rows g and g + 8, against the sums' two digits
            const uint32_t ma0 = t == 0 ? mn0[0] : (t == 1 ? mn0[1] : 0u);
            const uint32_t ma1 = t == 0 ? mn1[0] : (t == 1 ? mn1[1] : 0u);
            const float d0 = __half2float(__ushort_as_half((unsigned short)(h0.x & 0xffffu)));
            const float d1 = __half2float(__ushort_as_half((unsigned short)(h1.x & 0xffffu)));
            const float dm0 = -__half2float(__ushort_as_half((unsigned short)(h0.x >> 16)));
            const float dm1 = -__half2float(__ushort_as_half((unsigned short)(h1.x >> 16)));
#pragma unroll
            for (int nb = 0; nb < 8; nb++) {
                uint32_t lo = 0, hi = 0;
                if (t < 2) {
                    lo = *reinterpret_cast<const uint32_t*>(sums + (8 * nb + g) * 8 + 4 * t);
                    hi = *reinterpret_cast<const uint32_t*>(sums + QM_TOK * 8 + (8 * nb + g) * 8 + 4 * t);
                }
                int ml[4], mh[4];
                imma_16832(ml, ma0, ma1, 0u, 0u, lo, 0u);
                imma_16832(mh, ma0, ma1, 0u, 0u, hi, 0u);
                const float x0 = dxs[4 * (8 * nb + 2 * t)], x1 = dxs[4 * (8 * nb + 2 * t + 1)];
                float* af = accf[nb];
                af[0] = __fmaf_rn(__fmaf_rn((float)run[nb][0], d0, (float)(ml[0] + 256 * mh[0]) * dm0), x0, af[0]);
                af[1] = __fmaf_rn(__fmaf_rn((float)run[nb][1], d0, (float)(ml[1] + 256 * mh[1]) * dm0), x1, af[1]);
                af[2] = __fmaf_rn(__fmaf_rn((float)run[nb][2], d1, (float)(ml[2] + 256 * mh[2]) * dm1), x0, af[2]);
                af[3] = __fmaf_rn(__fmaf_rn((float)run[nb][3], d1, (float)(ml[3] + 256 * mh[3]) * dm1), x1, af[3]);
            }
        } else {
            // the 16 bytes copied hold the scales of blocks (4 st & ~7) .. +7: this step's four are its low or high half
            const uint32_t soff = wt + QM_WTILE + 8u * (st & 1);
            const uint2 sw0 = lds64(soff + 16u * (16 * warp + g)), sw1 = lds64(soff + 16u * (16 * warp + g + 8));
            const uint32_t scw0[2] = {sw0.x, sw0.y}, scw1[2] = {sw1.x, sw1.y};
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint2 q0 = lds64(wrow0 + 8 * t + 32 * i), q1 = lds64(wrow1 + 8 * t + 32 * i);
                const float d0 = __half2float(__ushort_as_half((unsigned short)((scw0[i >> 1] >> (16 * (i & 1))) & 0xffffu)));
                const float d1 = __half2float(__ushort_as_half((unsigned short)((scw1[i >> 1] >> (16 * (i & 1))) & 0xffffu)));
#pragma unroll
                for (int nb = 0; nb < 8; nb++) {
                    const uint2 b = lds64(xt + (uint32_t)(8 * nb + g) * XROW + 32u * i + 8u * t);
                    int acc[4];
                    imma_16832(acc, q0.x, q1.x, q0.y, q1.y, b.x, b.y);
                    const float x0 = dxs[4 * (8 * nb + 2 * t) + i], x1 = dxs[4 * (8 * nb + 2 * t + 1) + i];
                    float* af = accf[nb];
                    af[0] = __fmaf_rn((float)acc[0], d0 * x0, af[0]);
                    af[1] = __fmaf_rn((float)acc[1], d0 * x1, af[1]);
                    af[2] = __fmaf_rn((float)acc[2], d1 * x0, af[2]);
                    af[3] = __fmaf_rn((float)acc[3], d1 * x1, af[3]);
                }
            }
        }
        __syncthreads();  // every warp is done with this stage before the next step's copies overwrite it
    }
    if (timed_out && lane == 0 && status) atomicExch(status, 1);
    // ---- out[token][col0 + row] (+)= sum, or the slice's partial at z * slice_stride
    float* dst = out + (size_t)z * p.slice_stride;
#pragma unroll
    for (int nb = 0; nb < 8; nb++)
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int row = j0 + 16 * warp + g + (i >= 2 ? 8 : 0), tok = t0 + 8 * nb + 2 * t + (i & 1);
            if (row < n && tok < tokens) {
                const size_t o = (size_t)tok * p.out_stride + p.col0 + row;
                dst[o] = p.accumulate ? dst[o] + accf[nb][i] : accf[nb][i];
            }
        }
}

__global__ void matmul_reduce_kernel(PMatmulReduceQ p, const float* __restrict__ partials, float* __restrict__ out, int tokens) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)tokens * p.n) return;
    const size_t tok = i / p.n, j = i % p.n;
    float v = 0.f;
    for (uint32_t s = 0; s < p.slices; s++) v = __fadd_rn(v, partials[(size_t)s * p.slice_stride + i]);  // slice order
    const size_t o = tok * p.out_stride + p.col0 + j;
    out[o] = p.accumulate ? out[o] + v : v;
}

template <int TYPE>
zcu_result launch_matmul_quant(const LaunchArgs& a) {
    using S = QmShape<TYPE>;
    constexpr bool Q4 = TYPE == W_Q4_K;
    PMatmulQ p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 4, "matmul (quantised): bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    // the reference dispatches token tiles of 32 (grid y): the step's token count is at most that many
    const uint32_t cap = a.grid[1] * 32u;
    const int tokens = (int)(p.rows < cap ? p.rows : cap);
    if (tokens == 0 || p.n == 0) return ZCU_OK;
    ZCU_NEED(a, p.k % 256 == 0 && p.k > 0, "matmul (quantised): k = %u is not a multiple of 256", p.k);
    ZCU_NEED(a, p.k_slice > 0 && p.k_slice % 256 == 0, "matmul (quantised): k_slice = %u is not a multiple of 256", p.k_slice);
    const uint32_t slices = (p.k + p.k_slice - 1) / p.k_slice;
    ZCU_NEED(a, a.grid[2] <= 1 || a.grid[2] == slices, "matmul (quantised): %u slices in the grid, %u by k_slice", a.grid[2], slices);
    ZCU_NEED(a, ((uintptr_t)a.b[0].ptr & 15) == 0 && ((uintptr_t)a.b[1].ptr & 15) == 0, "matmul (quantised): qx and w must be 16-byte aligned");
    CUtensorMap wmap, smap;
    const uint64_t rb = Q4 ? (uint64_t)(p.k / 256) * 144 : (((uint64_t)p.k + p.k / 16 + 15) & ~(uint64_t)15);
    if (!tma::bytes_2d(&wmap, a.b[1].ptr, p.n, rb, TILE_ROW, QM_ROWS) || !tma::bytes_2d(&smap, a.b[1].ptr, p.n, rb, 16, QM_ROWS))
        return zcu_fail(a, ZCU_E_GPU, "matmul (quantised): the driver refused a tensor map (n %u, k %u)", p.n, p.k);
    auto kern = matmul_quant_kernel<TYPE>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "matmul (quantised): %d bytes of shared memory refused", S::SMEM);
    }
    const dim3 grid((p.n + QM_ROWS - 1) / QM_ROWS, (tokens + QM_TOK - 1) / QM_TOK, slices);
    kern<<<grid, QM_THREADS, S::SMEM, a.stream>>>(p, wmap, smap, (const int8_t*)a.b[0].ptr, (float*)a.b[2].ptr, (const float*)a.b[3].ptr,
                                                  tokens, a.status);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

}  // namespace

zcu_result launch_quantize_q8(const LaunchArgs& a) {
    PQuantize p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "quantize_q8: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.k % 256 == 0 && p.k > 0, "quantize_q8: k = %u is not a multiple of 256", p.k);
    ZCU_NEED(a, p.block == 256 || p.block == 32, "quantize_q8: block %u (256 for the K-quants, 32 for Q8_0)", p.block);
    ZCU_NEED(a, p.mode <= 2 && (p.mode != 1 || a.nb >= 4), "quantize_q8: mode %u", p.mode);
    const uint32_t rows = a.grid[1];
    if (rows == 0) return ZCU_OK;
    quantize_q8_kernel<<<dim3(p.k / 256, rows), 64, 0, a.stream>>>(p, (const float*)a.b[0].ptr, (int8_t*)a.b[1].ptr, (float*)a.b[2].ptr,
                                                                 a.nb >= 4 ? (const float*)a.b[3].ptr : nullptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_matmul_q4_k(const LaunchArgs& a) { return launch_matmul_quant<mv::W_Q4_K>(a); }
zcu_result launch_matmul_q8_0(const LaunchArgs& a) { return launch_matmul_quant<mv::W_Q8_0>(a); }

zcu_result launch_matmul_reduce(const LaunchArgs& a) {
    PMatmulReduceQ p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 2, "matmul_reduce: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    // the reference dispatches one thread per (token, output) in workgroups of 256: the grid bounds the step's tokens
    const uint64_t cap = (uint64_t)a.grid[0] * 256u * (a.grid[1] ? a.grid[1] : 1u);
    const uint64_t want = (uint64_t)p.rows * p.n;
    const uint64_t count = want < cap ? want : cap;
    const int tokens = p.n ? (int)(count / p.n) : 0;
    if (tokens == 0) return ZCU_OK;
    const uint64_t elems = (uint64_t)tokens * p.n;
    matmul_reduce_kernel<<<(unsigned)((elems + 255) / 256), 256, 0, a.stream>>>(p, (const float*)a.b[0].ptr, (float*)a.b[1].ptr, tokens);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}
