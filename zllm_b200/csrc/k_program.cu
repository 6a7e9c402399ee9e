// The step program: a recorded list of dispatches replayed by ONE persistent kernel, one CTA per SM.
//
// The reference submits a decode step as a few hundred dispatches (src/plan/qwen35.zig builds them once and
// replays them, src/gpu/cmd.zig carries them). At batch 1 each of those kernels lives for a few microseconds,
// and what a launch costs (the drain of the kernel before, the launch itself, the first trip to HBM) is as long
// as the work. Here the same list runs inside one cooperative kernel:
//   * every operation is the code of its standalone kernel (k_matvec_imma.cuh, k_attn_fast.cuh,
//     k_glue_body.cuh), so results are bit for bit those of the launch-by-launch path;
//   * operations are separated by a grid-wide barrier (one atomic counter in global memory);
//   * a warp's ring of weight tiles lives across operations: when a warp finishes its tiles of one multiply it
//     starts the copies of its first tiles of the NEXT multiply before it joins the barrier. Weights do not
//     depend on the step, so HBM keeps streaming through barriers, small operations and activation staging;
//   * the small kernels (embedding row, rope_append, attention) were written for 256 threads: two of their
//     blocks run side by side in each 512-thread CTA as virtual blocks (vblock.cuh).
// Data written by one operation and read by a later one crosses SMs inside one kernel, so those reads
// bypass L1 (ld.global.cg) and every CTA fences before it arrives at the barrier.
//
// Every spin is bounded: a CTA that gives up sets the abort word, the others leave at their next poll, and the
// context's status word reports it at the next sync.

#include <vector>

#include "k_attn_fast.cuh"
#include "k_glue_body.cuh"
#include "k_matvec_imma.cuh"

namespace {

using namespace imma;

constexpr int PROG_STAGES = 3;       // tiles per warp ring
constexpr int PROG_THREADS = IM_THREADS;
constexpr int VB_THREADS = 256;      // threads of a virtual block
constexpr int VB_PER_CTA = PROG_THREADS / VB_THREADS;
constexpr int VB_SMEM = 36 * 1024;   // shared memory of a virtual block
constexpr int PROG_SMEM_MAX = 227 * 1024;

enum : uint32_t { PK_MV_Q4_K = 1, PK_MV_Q8_0, PK_EMBED_Q4_K, PK_EMBED_Q8_0, PK_EMBED_BF16, PK_EMBED_F16, PK_ROPE_APPEND, PK_ATTN_SPLIT, PK_ATTN_COMBINE };

struct alignas(64) ProgOp {
    CUtensorMap map;         // multiply: the weight matrix as 16-row x 160-byte boxes (64-byte aligned)
    CUtensorMap smap;        // Q8_0 multiply: its scales as 16-row x 16-byte boxes
    uint32_t kind;
    uint32_t gx, gy, gz;     // grid of virtual blocks (the small kernels)
    uint32_t ncta;           // multiply: CTAs that take part (the standalone kernel's grid)
    uint32_t seg_max, mt, t0;
    int32_t next_mv;         // the next multiply in the list (-1: none): its first tiles are copied ahead
    uint32_t kb;             // attn_combine: cache positions per partial block
    uint32_t hd;             // attn_split: head_dim (64 or 128)
    uint32_t _pad;
    uint32_t params[24];     // the dispatch's parameter block (a multiply's may carry rope_append's after its own)
    const void* b[9];        // its bindings
};

// The shared memory every program kernel uses: the ring and its barriers first (im_layout puts them at offsets
// that depend on the stage count only), then a region that each operation lays out for itself.
__host__ __device__ inline int prog_scratch_offset() { return im_layout(4, 256, true, 2, 1, PROG_STAGES).xd; }

// All CTAs of the (cooperative, co-resident) grid meet here. bar[0] counts arrivals over the whole launch;
// bar[1] is the abort word. Returns false when the launch is being abandoned.
__device__ __forceinline__ bool grid_sync(unsigned* bar, unsigned target, int* status) {
    __syncthreads();
    int bad = 0;
    if (threadIdx.x == 0) {
        __threadfence();  // this CTA's writes are visible before its arrival is
        atomicAdd(&bar[0], 1u);
        unsigned spins = 0;
        for (;;) {
            unsigned seen;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(bar) : "memory");
            if (seen >= target) break;
            if ((++spins & 255u) == 0) {
                unsigned ab;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(ab) : "l"(bar + 1) : "memory");
                if (ab != 0) {
                    bad = 1;
                    break;
                }
                if (spins > (1u << 22)) {  // some CTA never arrived: give the launch up
                    atomicExch(&bar[1], 1u);
                    if (status) atomicExch(status, 4);
                    bad = 1;
                    break;
                }
            }
        }
        __threadfence();
    }
    return __syncthreads_or(bad) == 0;
}

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];\n" ::"l"(p)); }
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];\n" ::"l"(p)); }

// The constant inputs a multiply reads right after its barrier (the norm weights) are asked into L2 one
// multiply ahead, by one CTA.
__device__ __forceinline__ void prefetch_constants(const ProgOp* ops, int index) {
    if (index < 0) return;
    const ProgOp& op = ops[index];
    PMatvec p;
    memcpy(&p, op.params, sizeof(p));
    if (!(p.flags & MV_NORM) || op.b[3] == nullptr) return;
    const char* nw = static_cast<const char*>(op.b[3]);
    for (uint32_t off = threadIdx.x * 128u; off < p.k * 4u; off += PROG_THREADS * 128u) prefetch_l2(nw + off);
}

template <int TYPE>
__device__ __forceinline__ void prime_op(ImRing& rg, ImIssue& iss, const ProgOp& op, int index, int cta, int warp, int lane) {
    PMatvec p;
    memcpy(&p, op.params, sizeof(p));
    im_prime<TYPE, PROG_STAGES>(rg, iss, p, &op.map, &op.smap, cta, (int)op.ncta, warp, lane, index);
}

// Starts the copies of the multiply at `index` (if this CTA takes part in it) unless they were started already.
__device__ __forceinline__ void prime_ahead(ImRing& rg, ImIssue& iss, const ProgOp* ops, int index, int cta, int warp, int lane) {
    if (index < 0 || iss.op == index) return;
    const ProgOp& op = ops[index];
    if (cta >= (int)op.ncta) return;
    if (op.kind == PK_MV_Q4_K) prime_op<W_Q4_K>(rg, iss, op, index, cta, warp, lane);
    else prime_op<W_Q8_0>(rg, iss, op, index, cta, warp, lane);
}

// Not inlined: the multiply gets the register allocation of its standalone kernel; the ring and the copy
// iterator are copied into registers on entry and written back on exit.
template <int TYPE>
__device__ __noinline__ void run_multiply(uint8_t* smem, ImRing& rg_io, ImIssue& iss_io, const ProgOp* ops, int index, int cta,
                                          int* status) {
    const ProgOp& op = ops[index];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    ImRing rg = rg_io;
    ImIssue iss = iss_io;
    if (cta < (int)op.ncta) {
        PMatvec p;
        memcpy(&p, op.params, sizeof(p));
        prime_ahead(rg, iss, ops, index, cta, warp, lane);  // normally done one multiply ago
        MvRope rope;
        if (p.flags & MV_ROPE_APPEND) {
            memcpy(&rope.p, op.params + sizeof(PMatvec) / 4, sizeof(PRopeAppend));
            rope.table = static_cast<const float2*>(op.b[4]);
            rope.kc = const_cast<void*>(op.b[5]);
            rope.vc = const_cast<void*>(op.b[6]);
            rope.step = static_cast<const PStep*>(op.b[7]);
            rope.seq_pos = static_cast<const uint32_t*>(op.b[8]);
        }
        im_multiply<TYPE, 1, PROG_STAGES>(
            smem, rg, iss, cta, (int)op.ncta, p, static_cast<const float*>(op.b[0]), static_cast<float*>(const_cast<void*>(op.b[2])),
            static_cast<const float*>(op.b[3]), (int)op.t0, (int)op.mt, (int)op.seg_max, status,
            (p.flags & MV_ROPE_APPEND) ? &rope : nullptr, nullptr, [] {},
            [&] { prime_ahead(rg, iss, ops, op.next_mv, cta, warp, lane); });
    } else {
        prime_ahead(rg, iss, ops, op.next_mv, cta, warp, lane);
    }
    if (cta == index % (int)gridDim.x) prefetch_constants(ops, op.next_mv);
    rg_io = rg;
    iss_io = iss;
}

// Runs `body(vb)` for the virtual blocks of the operation's grid that fall to this half of this CTA.
template <class Body>
__device__ __forceinline__ void for_vblocks(const ProgOp& op, uint8_t* scratch, Body body) {
    const int half = threadIdx.x / VB_THREADS;
    VBlock vb;
    vb.tid = threadIdx.x % VB_THREADS;
    vb.nthreads = VB_THREADS;
    vb.bar = 1 + half;
    vb.smem = scratch + half * VB_SMEM;
    const unsigned total = op.gx * op.gy * op.gz;
    for (unsigned v = blockIdx.x * VB_PER_CTA + half; v < total; v += gridDim.x * VB_PER_CTA) {
        vb.x = (int)(v % op.gx);
        vb.y = (int)((v / op.gx) % op.gy);
        vb.z = (int)(v / (op.gx * op.gy));
        body(vb);
        vb.sync();  // the block's shared memory is reused by its next virtual block
    }
}

__device__ __noinline__ void run_embed(const ProgOp& op, uint8_t* scratch) {
    PEmbed p;
    memcpy(&p, op.params, sizeof(p));
    const uint32_t* tok = static_cast<const uint32_t*>(op.b[0]);
    const uint8_t* w = static_cast<const uint8_t*>(op.b[1]);
    float* out = static_cast<float*>(const_cast<void*>(op.b[2]));
    const uint32_t kind = op.kind;
    for_vblocks(op, scratch, [&](const VBlock& vb) {
        if (kind == PK_EMBED_Q4_K) glue::embed_body<glue::E_Q4_K>(vb, p, tok, w, out);
        else if (kind == PK_EMBED_Q8_0) glue::embed_body<glue::E_Q8_0>(vb, p, tok, w, out);
        else if (kind == PK_EMBED_BF16) glue::embed_body<glue::E_BF16>(vb, p, tok, w, out);
        else glue::embed_body<glue::E_F16>(vb, p, tok, w, out);
    });
}

__device__ __noinline__ void run_rope(const ProgOp& op, uint8_t* scratch) {
    PRopeAppend p;
    memcpy(&p, op.params, sizeof(p));
    for_vblocks(op, scratch, [&](const VBlock& vb) {
        glue::rope_append_body(vb, p, static_cast<float*>(const_cast<void*>(op.b[0])), static_cast<const float*>(op.b[1]),
                               static_cast<const float*>(op.b[2]), static_cast<const float2*>(op.b[3]),
                               static_cast<uint32_t*>(const_cast<void*>(op.b[4])), static_cast<uint32_t*>(const_cast<void*>(op.b[5])),
                               static_cast<const PStep*>(op.b[6]), static_cast<const uint32_t*>(op.b[7]));
    });
}

__device__ __noinline__ void run_split(const ProgOp& op, uint8_t* scratch) {
    PAttention p;
    memcpy(&p, op.params, sizeof(p));
    const uint32_t hd = op.hd;
    const float* qg = static_cast<const float*>(op.b[0]);
    const __half* kc = static_cast<const __half*>(op.b[1]);
    const __half* vc = static_cast<const __half*>(op.b[2]);
    float* part = static_cast<float*>(const_cast<void*>(op.b[3]));
    const PStep* st = static_cast<const PStep*>(op.b[4]);
    const uint32_t* sp = static_cast<const uint32_t*>(op.b[5]);
    for_vblocks(op, scratch, [&](const VBlock& vb) {
        if (hd == 128) attn::attn_split_fast_body<128, 4>(vb, p, qg, kc, vc, part, st, sp);
        else attn::attn_split_fast_body<64, 4>(vb, p, qg, kc, vc, part, st, sp);
    });
}

__device__ __noinline__ void run_combine(const ProgOp& op, uint8_t* scratch) {
    PAttention p;
    memcpy(&p, op.params, sizeof(p));
    for_vblocks(op, scratch, [&](const VBlock& vb) {
        attn::attn_combine_body(vb, p, static_cast<const float*>(op.b[0]), static_cast<const float*>(op.b[1]),
                                static_cast<float*>(const_cast<void*>(op.b[2])), static_cast<const PStep*>(op.b[3]),
                                static_cast<const uint32_t*>(op.b[4]), (int)op.kb);
    });
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}

// trace[2 i], trace[2 i + 1]: when CTA 0 entered operation i and when it finished its share of it (nanoseconds
// of the GPU's global timer). The gap to the next entry is the barrier.
__global__ void __launch_bounds__(PROG_THREADS, 1) program_kernel(const ProgOp* __restrict__ ops, int n_ops, unsigned* bar,
                                                                 int* __restrict__ status, unsigned long long* __restrict__ trace) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, cta = (int)blockIdx.x;
    uint8_t* scratch = smem + prog_scratch_offset();
    ImRing rg;
    ImIssue iss;
    iss.op = -1;
    iss.issued = iss.hi = iss.lo = 0;
    im_ring_init<PROG_STAGES>(rg, smem, im_layout(4, 256, true, 2, 1, PROG_STAGES), warp, lane);
    // the operation list is read once per launch: ask all of it into L2 now, and each operation's lines into
    // L1 one operation ahead
    for (size_t off = ((size_t)cta * PROG_THREADS + threadIdx.x) * 128; off < (size_t)n_ops * sizeof(ProgOp); off += (size_t)gridDim.x * PROG_THREADS * 128)
        prefetch_l2(reinterpret_cast<const char*>(ops) + off);
    __syncthreads();
    unsigned epoch = 0;
    for (int i = 0; i < n_ops; i++) {
        const ProgOp& op = ops[i];
        if (threadIdx.x < 8) {
            if (i + 1 < n_ops && threadIdx.x < 4) prefetch_l1(reinterpret_cast<const char*>(&ops[i + 1]) + 128 * (threadIdx.x & 3));
            if (op.next_mv >= 0 && threadIdx.x >= 4) prefetch_l1(reinterpret_cast<const char*>(&ops[op.next_mv]) + 128 * (threadIdx.x & 3));
        }
        const bool tracer = trace != nullptr && cta == 0 && threadIdx.x == 0;
        if (tracer) trace[2 * i] = global_ns();
        switch (op.kind) {
            case PK_MV_Q4_K: run_multiply<W_Q4_K>(smem, rg, iss, ops, i, cta, status); break;
            case PK_MV_Q8_0: run_multiply<W_Q8_0>(smem, rg, iss, ops, i, cta, status); break;
            case PK_EMBED_Q4_K:
            case PK_EMBED_Q8_0:
            case PK_EMBED_BF16:
            case PK_EMBED_F16: run_embed(op, scratch); break;
            case PK_ROPE_APPEND: run_rope(op, scratch); break;
            case PK_ATTN_SPLIT: run_split(op, scratch); break;
            case PK_ATTN_COMBINE: run_combine(op, scratch); break;
            default: break;
        }
        if (tracer) trace[2 * i + 1] = global_ns();
        if (i + 1 < n_ops && !grid_sync(bar, ++epoch * gridDim.x, status)) break;
    }
}

}  // namespace

// ---------------------------------------------------------------------------------------------- host side
struct zcu_program {
    std::vector<ProgOp> ops;
    ProgOp* d_ops = nullptr;
    unsigned* d_bar = nullptr;
    unsigned long long* d_trace = nullptr;
    int grid = 0;
    int smem = 0;
    uint64_t launches_equiv = 0;  // dispatches the program stands for
};

zcu_program* program_new() { return new zcu_program(); }

void program_free(zcu_program* pr) {
    if (!pr) return;
    if (pr->d_ops) cudaFree(pr->d_ops);
    if (pr->d_bar) cudaFree(pr->d_bar);
    if (pr->d_trace) cudaFree(pr->d_trace);
    delete pr;
}

uint64_t program_dispatches(const zcu_program* pr) { return pr ? pr->launches_equiv : 0; }

static void copy_common(ProgOp& op, const LaunchArgs& a) {
    memset(&op, 0, sizeof(op));
    op.next_mv = -1;
    memcpy(op.params, a.params, a.params_bytes < sizeof(op.params) ? a.params_bytes : sizeof(op.params));
    for (uint32_t i = 0; i < a.nb && i < 9; i++) op.b[i] = a.b[i].ptr;
}

// Records one dispatch. Only what the persistent kernel can run is accepted; anything else is an error (there is
// no silent second path): the caller keeps launch-by-launch replay for those steps.
zcu_result program_record(zcu_program* pr, uint32_t kernel, const LaunchArgs& a) {
    ProgOp op;
    copy_common(op, a);
    const int sms = a.sm_count > 0 ? a.sm_count : 148;
    switch (kernel) {
        case ZCU_K_MATVEC_Q4_K:
        case ZCU_K_MATVEC_Q8_0: {
            const bool q4 = kernel == ZCU_K_MATVEC_Q4_K;
            PMatvec p;
            ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "step program: matvec with a bad parameter block or bindings");
            memcpy(&p, a.params, sizeof(p));
            const uint32_t family = (a.variant >> 16) & 0xffu;
            if (a.variant != 0 && family != ZCU_FAMILY_MMA)
                return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: matvec variant 0x%x (only the tensor-core family runs inside it)", a.variant);
            const int m = (int)a.grid[1];
            if (p.n == 0 || m == 0) return ZCU_OK;
            if (m > 2) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: %d tokens per multiply (at most 2)", m);
            if (p.k % 256 != 0 || p.k == 0) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: k = %u is not a multiple of 256", p.k);
            ZCU_NEED(a, !(p.flags & MV_NORM) || a.nb >= 4, "step program: NORM without a norm weight binding");
            if (p.flags & MV_ROPE_APPEND) {
                PRopeAppend r;
                ZCU_NEED(a, a.params_bytes >= sizeof(PMatvec) + sizeof(PRopeAppend) && a.nb >= 8, "step program: matvec + rope_append with a short parameter block or bindings");
                memcpy(&r, static_cast<const char*>(a.params) + sizeof(PMatvec), sizeof(r));
                ZCU_NEED(a, r.normal == 1 && r.qk_norm == 0 && r.head_dim % 2 == 0 && r.n_rot % 2 == 0 && r.n_rot <= r.head_dim && (r.kv == KV_F32 || r.kv == KV_F16) &&
                                p.col0 % 2 == 0 && p.n % 2 == 0 && !(p.flags & (MV_SILU_PAIR | MV_ACCUMULATE)),
                         "step program: this matvec + rope_append is not fused (adjacent pairs, no q/k norm, f16 or f32 cache)");
                if (!(a.nb >= 9 && r._pad[0] != 0)) op.b[8] = nullptr;
            }
            ZCU_NEED(a, ((uintptr_t)a.b[0].ptr & 15) == 0 && ((uintptr_t)a.b[1].ptr & 15) == 0, "step program: x and w must be 16-byte aligned");
            const int row_tiles = ((int)p.n + 15) / 16;
            op.kind = q4 ? PK_MV_Q4_K : PK_MV_Q8_0;
            op.ncta = (uint32_t)(row_tiles < sms ? row_tiles : sms);
            op.seg_max = (uint32_t)segments_needed((int)p.n, (int)p.k, q4, (p.flags & MV_SILU_PAIR) != 0, (int)op.ncta);
            op.mt = (uint32_t)m;
            op.t0 = 0;
            const int need = im_layout(4 * m, (int)p.k, q4, 2, (int)op.seg_max, PROG_STAGES).total;
            if (need > PROG_SMEM_MAX)
                return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: k = %u with %d tokens needs %d bytes of shared memory", p.k, m, need);
            if (need > pr->smem) pr->smem = need;
            const size_t rows = (size_t)p.n + ((p.flags & MV_SILU_PAIR) ? p.half : 0);
            if (!im_weight_map(&op.map, a.b[1].ptr, q4, (int)p.k, rows, false) || !im_weight_map(&op.smap, a.b[1].ptr, q4, (int)p.k, rows, !q4))
                return zcu_fail(a, ZCU_E_GPU, "step program: the driver refused a tensor map (n %u, k %u)", p.n, p.k);
            break;
        }
        case ZCU_K_EMBED_Q4_K:
        case ZCU_K_EMBED_Q8_0:
        case ZCU_K_EMBED_BF16:
        case ZCU_K_EMBED_F16: {
            ZCU_NEED(a, a.params_bytes >= sizeof(PEmbed) && a.nb >= 3, "step program: embed with a bad parameter block or bindings");
            if (a.grid[0] == 0) return ZCU_OK;
            op.kind = kernel == ZCU_K_EMBED_Q4_K ? PK_EMBED_Q4_K : kernel == ZCU_K_EMBED_Q8_0 ? PK_EMBED_Q8_0 : kernel == ZCU_K_EMBED_BF16 ? PK_EMBED_BF16 : PK_EMBED_F16;
            op.gx = a.grid[0], op.gy = 1, op.gz = 1;
            break;
        }
        case ZCU_K_ROPE_APPEND: {
            PRopeAppend p;
            ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 7, "step program: rope_append with a bad parameter block or bindings");
            memcpy(&p, a.params, sizeof(p));
            ZCU_NEED(a, p.head_dim <= 256 && p.head_dim % 2 == 0 && (p.kv == KV_F32 || p.kv == KV_F16), "step program: rope_append head_dim %u cache %u", p.head_dim, p.kv);
            if (a.grid[1] == 0) return ZCU_OK;
            if (!(a.nb >= 8 && p._pad[0] != 0)) op.b[7] = nullptr;  // per-sequence positions only with the batched extension
            op.kind = PK_ROPE_APPEND;
            op.gx = p.heads + p.kv_heads, op.gy = a.grid[1], op.gz = 1;
            break;
        }
        case ZCU_K_ATTN_SPLIT: {
            PAttention p;
            ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 5, "step program: attn_split with a bad parameter block or bindings");
            memcpy(&p, a.params, sizeof(p));
            const uint32_t group = p.kv_heads ? p.heads / p.kv_heads : 0;
            const bool fast = p.kv == KV_F16 && p.kv_heads > 0 && p.heads % p.kv_heads == 0 && group >= 1 && group <= 4 && (p.head_dim == 64 || p.head_dim == 128);
            if (!fast) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: attention needs the f16 cache, a GQA group of at most 4 and head_dim 64 or 128");
            if (a.variant != 1) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: only attn_split's CUDA-core form (variant 1) runs inside it");
            ZCU_NEED(a, a.grid[1] <= p.max_blocks, "step program: %u key blocks above max_blocks %u", a.grid[1], p.max_blocks);
            if (a.grid[1] == 0 || a.grid[2] == 0) return ZCU_OK;
            if (!(a.nb >= 6 && p._pad[0] != 0)) op.b[5] = nullptr;
            op.kind = PK_ATTN_SPLIT;
            op.hd = p.head_dim;
            op.gx = p.kv_heads, op.gy = (a.grid[1] * 64 + attn::AF_KEYS - 1) / attn::AF_KEYS, op.gz = a.grid[2];
            if ((int)attn::attn_fast_smem(4, (int)group, (int)p.head_dim) > VB_SMEM) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: attention scratch does not fit");
            break;
        }
        case ZCU_K_ATTN_COMBINE: {
            PAttention p;
            ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 4, "step program: attn_combine with a bad parameter block or bindings");
            memcpy(&p, a.params, sizeof(p));
            const uint32_t group = p.kv_heads ? p.heads / p.kv_heads : 0;
            const bool fast = p.kv == KV_F16 && group >= 1 && group <= 4 && (p.head_dim == 64 || p.head_dim == 128);
            if (!fast) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: attention needs the f16 cache, a GQA group of at most 4 and head_dim 64 or 128");
            if ((int)attn::attn_combine_smem((int)p.max_blocks) > VB_SMEM) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: max_blocks %u does not fit the combine's scratch", p.max_blocks);
            if (a.grid[0] == 0 || a.grid[1] == 0) return ZCU_OK;
            if (!(a.nb >= 5 && p._pad[0] != 0)) op.b[4] = nullptr;
            op.kind = PK_ATTN_COMBINE;
            op.kb = attn::AF_KEYS;
            op.gx = p.heads, op.gy = a.grid[1], op.gz = 1;
            break;
        }
        default: return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "step program: kernel %u does not run inside the persistent kernel", kernel);
    }
    pr->ops.push_back(op);
    pr->launches_equiv++;
    return ZCU_OK;
}

// Uploads the list. `sm_count` CTAs must be co-resident (one per SM).
zcu_result program_finish(zcu_program* pr, const LaunchArgs& a) {
    ZCU_NEED(a, !pr->ops.empty(), "step program: nothing was recorded");
    int next = -1;
    for (int i = (int)pr->ops.size() - 1; i >= 0; i--) {  // link every op to the next multiply after it
        pr->ops[i].next_mv = next;
        if (pr->ops[i].kind == PK_MV_Q4_K || pr->ops[i].kind == PK_MV_Q8_0) next = i;
    }
    const int scratch_end = prog_scratch_offset() + VB_PER_CTA * VB_SMEM;
    if (scratch_end > pr->smem) pr->smem = scratch_end;
    if (cudaFuncSetAttribute(program_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pr->smem) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "step program: %d bytes of shared memory refused", pr->smem);
    }
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, program_kernel, PROG_THREADS, pr->smem) != cudaSuccess || per_sm < 1) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "step program: the persistent kernel does not fit an SM");
    }
    pr->grid = a.sm_count;
    const size_t bytes = pr->ops.size() * sizeof(ProgOp);
    if (cudaMalloc((void**)&pr->d_ops, bytes) != cudaSuccess || cudaMalloc((void**)&pr->d_bar, 64) != cudaSuccess ||
        cudaMalloc((void**)&pr->d_trace, pr->ops.size() * 16) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_OUT_OF_MEMORY, "step program: no memory for %zu bytes of operations", bytes);
    }
    if (cudaMemcpy(pr->d_ops, pr->ops.data(), bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "step program: upload failed");
    }
    return ZCU_OK;
}

zcu_result program_launch(zcu_program* pr, const LaunchArgs& a) {
    ZCU_NEED(a, pr && pr->d_ops, "step program: not finished");
    if (cudaMemsetAsync(pr->d_bar, 0, 64, a.stream) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "step program: barrier reset failed");
    }
    const ProgOp* ops = pr->d_ops;
    int n = (int)pr->ops.size();
    unsigned* bar = pr->d_bar;
    int* status = a.status;
    unsigned long long* trace = pr->d_trace;
    void* args[] = {(void*)&ops, (void*)&n, (void*)&bar, (void*)&status, (void*)&trace};
    const cudaError_t e = cudaLaunchCooperativeKernel((const void*)program_kernel, dim3(pr->grid), dim3(PROG_THREADS), args, (size_t)pr->smem, a.stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "step program: cooperative launch failed: %s", cudaGetErrorString(e));
    }
    return ZCU_OK;
}

// Per-operation times of the program's last completed launch, as CTA 0 saw them: out[3 i] = kind of operation i,
// out[3 i + 1] = nanoseconds in the operation, out[3 i + 2] = nanoseconds at the barrier after it.
zcu_result program_timings(zcu_program* pr, const LaunchArgs& a, uint64_t* out, size_t cap, size_t* n_out) {
    ZCU_NEED(a, pr && pr->d_trace, "step program: not finished");
    const size_t n = pr->ops.size();
    std::vector<unsigned long long> t(2 * n);
    if (cudaMemcpy(t.data(), pr->d_trace, 16 * n, cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "step program: reading the trace failed");
    }
    if (n_out) *n_out = n;
    for (size_t i = 0; i < n && 3 * i + 2 < cap; i++) {
        out[3 * i] = pr->ops[i].kind;
        out[3 * i + 1] = t[2 * i + 1] - t[2 * i];
        out[3 * i + 2] = i + 1 < n ? t[2 * i + 2] - t[2 * i + 1] : 0;
    }
    return ZCU_OK;
}
