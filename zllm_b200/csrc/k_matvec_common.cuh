// Helpers shared by the decode-multiply families (k_matvec.cu, k_matvec_imma.cu).
#pragma once

#include <cuda_fp16.h>

#include "zcu_internal.h"

namespace mv {

enum { W_Q4_K = 0, W_Q8_0 = 1, W_BF16 = 2, W_F16 = 3, W_Q3_K = 4, W_Q5_K = 5, W_Q6_K = 6 };

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
__device__ inline void cta_norm_stats(const float* __restrict__ x, const float* __restrict__ nw, int k, bool norm,
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


struct MvArgs {
    PMatvec p;
    const float* x;
    const uint8_t* w;
    float* out;
    const float* nw;
    int m;
    PeerUse peer;    // tensor-parallel exchange this launch waits for / publishes (slots PEER_NONE: none)
    bool has_rope;   // MV_ROPE_APPEND: the outputs are a Q|K|V row that is rotated and appended to the cache
    MvRope rope;
    MvCombine combine;   // MV_ATTN_COMBINE: combine.blocks != 0
};

}  // namespace mv

// The tensor-core family (k_matvec_imma.cu). stages = 0 picks the deepest ring that fits; shape 0 = CTAs of 16
// warps, 1 = CTAs of 8 warps (two per SM).
zcu_result launch_matvec_imma(const LaunchArgs& a, const mv::MvArgs& v, int type, int stages, int shape);
// The batched tcgen05 family of matvec_q4_k (k_quant_tc.cu): up to 64 tokens in one pass over the weights.
zcu_result launch_matvec_q4_k_tc(const LaunchArgs& a, const mv::MvArgs& v);
