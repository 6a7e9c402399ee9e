// Shared between the host (zcu_host.cu) and the kernel translation units.
#pragma once

#include "peer.cuh"
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/zllm_cuda.h"

// ---- parameter blocks: the reference's `params.*` extern structs, bit for bit
// (src/kernels/kernels.zig:432-650). Binding 0 of every dispatch.

struct PStep {  // kernels.zig:436
    uint32_t m, pos0;
    float u;
    uint32_t keep;
};
struct PRmsNorm {  // kernels.zig:438
    uint32_t rows, dim;
    float eps;
    uint32_t w_rows;
};
struct PMatmulBf16 {  // kernels.zig:439-448
    uint32_t rows, n, k, col0, out_stride, accumulate, _pad[2];
};
struct PMatmulQuant {  // kernels.zig:452-461
    uint32_t rows, n, k, col0, out_stride, accumulate, k_slice, slice_stride;
};
struct PMatmulReduce {  // kernels.zig:462-471
    uint32_t rows, n, slices, col0, out_stride, accumulate, slice_stride, _pad;
};
struct PMatvec {  // kernels.zig:472-494 (MatvecBf16, shared by every matvec identity)
    uint32_t n, k, col0, out_stride;
    float eps;
    uint32_t flags, half, x_stride;
};
enum : uint32_t { MV_NORM = 1u, MV_ACCUMULATE = 2u, MV_SILU_PAIR = 4u, MV_ROPE_APPEND = 8u, MV_ATTN_COMBINE = 16u };
struct PQuantizeQ8 {  // kernels.zig:495-501
    uint32_t k, block, mode;
    float eps;
};
struct PRepackQ80 {  // kernels.zig:502
    uint32_t rows, k, _pad[2];
};
struct PSiluMul {  // kernels.zig:505
    uint32_t count, width, _pad[2];
};
struct PEmbed {  // kernels.zig:508 (EmbedBf16)
    uint32_t dim, row0, chunk_rows, stride;
};
struct PRopeAppend {  // kernels.zig:509-532
    uint32_t heads, kv_heads, head_dim, n_rot, row, k_off, v_off, kv;
    float eps;
    uint32_t gated, qk_norm, normal, scales, _pad[3];
};
struct PAttention {  // kernels.zig:548-564
    uint32_t heads, kv_heads, head_dim, kv;
    float scale;
    uint32_t max_blocks, q_row, row0, gated, scales, _pad[2];
};
struct PDeltaPrep {  // kernels.zig:565-576
    uint32_t channels, taps, key_channels, head, row, v_heads, beta_off, alpha_off;
    float eps;
    uint32_t _pad[3];
};
struct PDeltaRule {  // kernels.zig:577-588
    uint32_t k_heads, v_heads, dim, conv_stride, taps, row, kept_hist, _pad;
};
struct PGatedNorm {  // kernels.zig:624-633
    uint32_t v_heads, dim;
    float eps;
    uint32_t z_row, z_off, sigmoid, _pad[2];
};

// What a multiply with MV_ROPE_APPEND needs beyond its own block: the rope_append parameters (they follow
// PMatvec in the parameter block) and that kernel's other bindings.
struct MvRope {
    PRopeAppend p;
    const float2* table;
    void* kc;
    void* vc;
    const PStep* step;
    const uint32_t* seq_pos;
};

// What a multiply with MV_ATTN_COMBINE needs beyond its own block: it reads the attention output, and merges the
// attention's partials into it itself before it does (attn_combine's parameters follow PMatvec in the parameter
// block; attn_combine's bindings follow the multiply's).
struct MvCombine {
    PAttention p;
    const float* qg;
    const float* part;
    float* out;              // where attn_combine would write: this rank's head columns of the multiply's input
    const PStep* step;
    const uint32_t* seq_pos;
    int kb;                  // cache positions per partial block
    int blocks;              // heads * rows merges (0: none)
};

static_assert(sizeof(PStep) == 16, "Step");
static_assert(sizeof(PMatmulBf16) == 32, "MatmulBf16");
static_assert(sizeof(PMatvec) == 32, "MatvecBf16");
static_assert(sizeof(PRopeAppend) == 64, "RopeAppend");
static_assert(sizeof(PAttention) == 48, "Attention");
static_assert(sizeof(PDeltaPrep) == 48, "DeltaPrep");
static_assert(sizeof(PDeltaRule) == 32, "DeltaRule");
static_assert(sizeof(PGatedNorm) == 32, "GatedNorm");

// KV cache formats (plan.common.KvFormat, src/plan/common.zig:30-50).
enum : uint32_t { KV_F32 = 0, KV_F16 = 1, KV_FP8 = 2 };

// Attention block: cache positions per partial (kernels.attn_block, kernels.zig:397).
#define ZCU_ATTN_BLOCK 64u

// ---- one dispatch as the launchers see it
struct LaunchArgs {
    cudaStream_t stream;
    const void* params;            // host copy of binding 0
    uint32_t params_bytes;
    const zcu_binding* b;          // b[i] = binding i + 1
    uint32_t nb;
    uint32_t grid[3];              // the reference's workgroup grid
    uint32_t variant;
    int sm_count;
    int* status;                   // device-visible word a kernel sets when a bounded wait gives up
    const PeerTable* peers;        // the context's tensor-parallel exchange table (null: none configured)
    void* scratch;                 // the context's device scratch (null: none) for launches that stage inputs; one stream, in order
    size_t scratch_bytes;
    char* err;                     // message buffer on failure
    size_t err_cap;
};

// Each returns ZCU_OK or a negative result with a message in a.err.
zcu_result launch_matvec_q4_k(const LaunchArgs& a);
zcu_result launch_matvec_q8_0(const LaunchArgs& a);
zcu_result launch_matvec_q3_k(const LaunchArgs& a);   // repacked units (repack_q3_k)
zcu_result launch_matvec_q5_k(const LaunchArgs& a);
zcu_result launch_matvec_q6_k(const LaunchArgs& a);   // blocks padded to 224 bytes (repad)
zcu_result launch_repad(const LaunchArgs& a);
zcu_result launch_repack_q3_k(const LaunchArgs& a);
zcu_result launch_embed_kquant(const LaunchArgs& a, uint32_t kernel);
zcu_result launch_matvec_bf16(const LaunchArgs& a);
zcu_result launch_matvec_f16(const LaunchArgs& a);
zcu_result launch_matmul_bf16(const LaunchArgs& a);
zcu_result launch_matmul_f16(const LaunchArgs& a);
zcu_result launch_matmul_tc(const LaunchArgs& a, bool bf16);   // the tensor-core prefill rung of both
zcu_result launch_rmsnorm(const LaunchArgs& a);
zcu_result launch_silu_mul(const LaunchArgs& a);
zcu_result launch_embed(const LaunchArgs& a, uint32_t kernel);
zcu_result launch_repack_q8_0(const LaunchArgs& a);
zcu_result launch_rope_append(const LaunchArgs& a);
zcu_result launch_attn_split(const LaunchArgs& a);
zcu_result launch_attn_combine(const LaunchArgs& a);
zcu_result launch_delta_prep(const LaunchArgs& a);
zcu_result launch_sample(const LaunchArgs& a);        // the whole draw on the sequence's first phase (k_sample.cu)
zcu_result launch_mark_tokens(const LaunchArgs& a);
zcu_result launch_draft(const LaunchArgs& a);
zcu_result launch_delta_rule(const LaunchArgs& a);
zcu_result launch_delta_recurrent(const LaunchArgs& a, uint32_t t_first, uint32_t m_expect);
zcu_result launch_delta_chunked(const LaunchArgs& a);          // 64-token chunks, then the recurrent tail
zcu_result launch_gated_norm(const LaunchArgs& a);
zcu_result launch_attn_static(const LaunchArgs& a, uint32_t max_keys, uint32_t rows);
int attn_keys_per_block(const PAttention& p);   // cache positions per partial block of this attention (k_attn.cu)
zcu_result launch_peer_wait(const LaunchArgs& a);
zcu_result launch_peer_next(const LaunchArgs& a);
zcu_result launch_quantize_q8(const LaunchArgs& a);
zcu_result launch_matmul_q4_k(const LaunchArgs& a);
zcu_result launch_matmul_q8_0(const LaunchArgs& a);
zcu_result launch_matmul_reduce(const LaunchArgs& a);
zcu_result launch_matmul_q8_0_float(const LaunchArgs& a);
zcu_result launch_matmul_q4_k_tc(const LaunchArgs& a);       // the tcgen05 prefill rung of matmul_q4_k

// The exchange a dispatch takes part in: a PPeer block trailing its parameter block (see peer.cuh). `outs`: the
// ranges it stores to, which must lie in the local arena when it pushes. Fills `u` (both slots PEER_NONE without one).
zcu_result parse_peer(const LaunchArgs& a, PeerUse& u, const void* out_lo, const void* out_hi);

// Launches `kern` as a programmatic dependent of the kernel before it in the stream: its CTAs may be placed while
// that kernel drains; it orders itself with griddepcontrol.wait before it reads what that kernel wrote.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// Whether (kernel, variant) exists, and its artifact name.
bool matvec_variant_ok(uint32_t kernel, uint32_t variant);

zcu_result zcu_fail(const LaunchArgs& a, zcu_result r, const char* fmt, ...);

#define ZCU_CHECK_LAUNCH(a)                                                          \
    do {                                                                             \
        cudaError_t e__ = cudaGetLastError();                                        \
        if (e__ != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "%s: launch failed: %s", __func__, cudaGetErrorString(e__)); \
    } while (0)

#define ZCU_NEED(a, cond, ...)                                        \
    do {                                                              \
        if (!(cond)) return zcu_fail(a, ZCU_E_BAD_COMMAND, __VA_ARGS__); \
    } while (0)
