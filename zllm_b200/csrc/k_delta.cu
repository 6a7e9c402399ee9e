// Gated delta rule (the recurrent form) over a step's m tokens. Replaces the
// reference's delta_rule (src/kernels/delta_rule.wgsl) with the same parameter
// block (params.DeltaRule), bindings and state layout
// state[j * dim^2 + a * dim + b] (a key row, b value column), f32.
// Per token, per value head j (key head j mod k_heads):
//   S <- e^g S;  delta = beta (v - S^T k);  S <- S + k delta^T;  o = S^T q / sqrt(dim)
// (src/ref/qwen35.zig:493-546). It also advances the conv history and, with
// step.keep = r + 1, saves the state and history as they stand after row r.
//
// Column b of S depends only on column b: CTA (j, c) owns COLS columns, and
// thread (row group r, column) keeps dim/RG rows of its column in registers
// for the whole step, so the state is read once and written once per step.
// The two dot products per token reduce over the row groups in a fixed order.

#include "zcu_internal.h"

namespace {

constexpr int DR_THREADS = 256;
constexpr int DR_MAX_DIM = 256;

// hist[i] <- the input K-1-i positions before the step's end, every channel
// (src/kernels/delta_rule.wgsl:67-95). The kept history is taken first.
__device__ void advance_history(const PDeltaRule& p, const PStep& st, const float* __restrict__ proj,
                                float* __restrict__ hist, float* __restrict__ kept, uint32_t id, uint32_t threads) {
    const uint32_t back = p.taps - 1;
    for (uint32_t c = id; c < p.conv_stride; c += threads) {
        if (st.keep != 0 && kept != nullptr) {
            for (uint32_t i = 0; i < back; i++) {
                const uint32_t j = st.keep + i;
                const float v = j < back ? hist[(size_t)j * p.conv_stride + c] : proj[(size_t)(j - back) * p.row + c];
                kept[p.kept_hist + (size_t)i * p.conv_stride + c] = v;
            }
        }
        for (uint32_t i = 0; i < back; i++) {
            const uint32_t j = st.m + i;
            hist[(size_t)i * p.conv_stride + c] =
                j < back ? hist[(size_t)j * p.conv_stride + c] : proj[(size_t)(j - back) * p.row + c];
        }
    }
}

// COLS columns per CTA, RG = 256 / COLS row groups, ROWS_CAP >= dim / RG.
template <int COLS, int ROWS_CAP>
__global__ void __launch_bounds__(DR_THREADS) delta_rule_kernel(PDeltaRule p, const float* __restrict__ conv,
                                                               const float* __restrict__ g,
                                                               const float* __restrict__ beta,
                                                               float* __restrict__ state, float* __restrict__ out,
                                                               const PStep* __restrict__ step,
                                                               const float* __restrict__ proj, float* __restrict__ hist,
                                                               float* __restrict__ kept, int with_hist,
                                                               uint32_t t_first, uint32_t m_expect, int* __restrict__ status) {
    constexpr int RG = DR_THREADS / COLS;
    __shared__ float qs[DR_MAX_DIM], ks[DR_MAX_DIM];
    __shared__ float red[DR_THREADS];
    __shared__ float delta[COLS];
    const PStep st = *step;
    const int lid = threadIdx.x;
    // After the chunked form has consumed tokens [0, t_first): the host-side token count must be the step's, and
    // a kept row inside the chunked part cannot be produced. Both are reported, not guessed around.
    if (m_expect != 0xffffffffu && (st.m != m_expect || (st.keep != 0 && st.keep <= t_first))) {
        if (lid == 0 && status) atomicExch(status, 3);
        return;
    }
    if (with_hist)
        advance_history(p, st, proj, hist, kept, (blockIdx.y * gridDim.x + blockIdx.x) * DR_THREADS + lid,
                        gridDim.x * gridDim.y * DR_THREADS);
    const int j = blockIdx.x;
    const int col = lid % COLS, r = lid / COLS;
    const int d = (int)p.dim;
    const int b = blockIdx.y * COLS + col;
    const bool in_head = b < d;
    const int rows = d / RG;
    const int a0 = r * rows;
    const int key_dim = (int)p.k_heads * d;
    const int kh = j % (int)p.k_heads;
    const size_t s0 = (size_t)j * d * d;
    const float scale = 1.0f / sqrtf((float)d);

    float s[ROWS_CAP];
#pragma unroll
    for (int i = 0; i < ROWS_CAP; i++) s[i] = (i < rows && in_head) ? state[s0 + (size_t)(a0 + i) * d + b] : 0.f;

    for (uint32_t t = t_first; t < st.m; t++) {
        const size_t row = (size_t)t * p.conv_stride;
        for (int i = lid; i < d; i += DR_THREADS) {
            qs[i] = conv[row + (size_t)kh * d + i];
            ks[i] = conv[row + key_dim + (size_t)kh * d + i];
        }
        __syncthreads();
        const float decay = expf(g[(size_t)t * p.v_heads + j]);
        float stk = 0.f;
#pragma unroll
        for (int i = 0; i < ROWS_CAP; i++) {
            if (i < rows) {
                s[i] = __fmul_rn(s[i], decay);
                stk = __fmaf_rn(s[i], ks[a0 + i], stk);
            }
        }
        red[lid] = stk;
        __syncthreads();
        if (r == 0) {
            float total = 0.f;
#pragma unroll
            for (int q = 0; q < RG; q++) total = __fadd_rn(total, red[q * COLS + col]);
            const float v = in_head ? conv[row + 2 * (size_t)key_dim + (size_t)j * d + b] : 0.f;
            delta[col] = __fmul_rn(__fsub_rn(v, total), beta[(size_t)t * p.v_heads + j]);
        }
        __syncthreads();
        const float dl = delta[col];
        float o = 0.f;
#pragma unroll
        for (int i = 0; i < ROWS_CAP; i++) {
            if (i < rows) {
                s[i] = __fmaf_rn(ks[a0 + i], dl, s[i]);
                o = __fmaf_rn(s[i], qs[a0 + i], o);
            }
        }
        red[lid] = o;
        __syncthreads();
        if (r == 0 && in_head) {
            float total = 0.f;
#pragma unroll
            for (int q = 0; q < RG; q++) total = __fadd_rn(total, red[q * COLS + col]);
            out[(size_t)t * p.v_heads * d + (size_t)j * d + b] = __fmul_rn(total, scale);
        }
        if (t + 1 == st.keep && in_head && kept != nullptr) {
#pragma unroll
            for (int i = 0; i < ROWS_CAP; i++)
                if (i < rows) kept[s0 + (size_t)(a0 + i) * d + b] = s[i];
        }
        __syncthreads();
    }
    if (in_head) {
#pragma unroll
        for (int i = 0; i < ROWS_CAP; i++)
            if (i < rows) state[s0 + (size_t)(a0 + i) * d + b] = s[i];
    }
}

}  // namespace

// Bindings: conv, g, beta, state (rw), out (rw), step, proj, hist (rw), kept (rw).
// proj/hist/kept may be absent (fewer bindings): the history is then left alone,
// which is what a caller that supplies q, k, v directly wants.
zcu_result launch_delta_rule(const LaunchArgs& a) {
    if (a.variant == ZCU_VARIANT_DELTA_CHUNK64 || a.variant == ZCU_VARIANT_DELTA_CHUNK64_F32) return launch_delta_chunked(a);
    return launch_delta_recurrent(a, 0, 0xffffffffu);
}

// The recurrent kernel over tokens [t_first, step.m). m_expect: the host's idea of step.m (checked on the
// device), or 0xffffffff for none.
zcu_result launch_delta_recurrent(const LaunchArgs& a, uint32_t t_first, uint32_t m_expect) {
    PDeltaRule p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 6, "delta_rule: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.dim >= 16 && p.dim <= DR_MAX_DIM && p.dim % 16 == 0, "delta_rule: dim %u", p.dim);
    ZCU_NEED(a, p.k_heads > 0 && p.v_heads > 0, "delta_rule: no heads");
    const int with_hist = a.nb >= 9 && p.taps > 1;
    const float* proj = with_hist ? (const float*)a.b[6].ptr : nullptr;
    float* hist = with_hist ? (float*)a.b[7].ptr : nullptr;
    float* kept = a.nb >= 9 ? (float*)a.b[8].ptr : nullptr;
    // 16 columns per CTA (16 row groups): more CTAs than the 32-column shape, which
    // leaves most of 148 SMs idle at 16 heads.
    constexpr int COLS = 16;
    const dim3 grid(p.v_heads, (p.dim + COLS - 1) / COLS);
    delta_rule_kernel<COLS, DR_MAX_DIM / (DR_THREADS / COLS)><<<grid, DR_THREADS, 0, a.stream>>>(
        p, (const float*)a.b[0].ptr, (const float*)a.b[1].ptr, (const float*)a.b[2].ptr, (float*)a.b[3].ptr,
        (float*)a.b[4].ptr, (const PStep*)a.b[5].ptr, proj, hist, kept, with_hist, t_first, m_expect, a.status);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}
