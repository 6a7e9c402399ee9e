// The tensor-core family of the quantised decode multiplies (matvec_q4_k, matvec_q8_0):
//   out[t][col0 + j] (+)= sum_i x[t][i] * w[j][i]      (src/kernels/matvec_quant.wgsl.hbs:1-31)
// with the RMSNorm prologue (NORM), ACCUMULATE and the SwiGLU pair epilogue (SILU_PAIR) of the reference's
// kernel, for 1..4 tokens per pass over the weights.
//
// Why integer tensor cores: at B200's HBM rate a Q4_K multiply has about three issue slots per weight, and
// turning a 4-bit code into a float on the CUDA cores costs more than that. So the codes stay integers. The
// activations are turned once per CTA into 32-bit fixed point (one power-of-two scale per token and 256-weight
// block) and split into four balanced signed byte digits; mma.sync.m16n8k32 (u8 x s8 -> s32) accumulates
// exactly. Every sum up to the super-block level is exact integer arithmetic and all later sums have a fixed
// order, so a token's result does not depend on the step's token count.
//
// Q4_K, per token one 8-column block: a byte of the file holds the codes of weight l (low nibble, sub-block
// 2j) and weight l + 32 (high nibble, sub-block 2j + 1). Columns 0-3 of the B operand are the four digits of
// x[64 j + l], columns 4-7 those of x[64 j + 32 + l]. Two MMAs per 64 weights:
//     D1 = (byte & 0xf0) x B      cols 0-3: 16 sum hi * xa      cols 4-7: 16 sum hi * xb
//     D2 =  byte         x B      cols 0-3: sum lo * xa + 16 sum hi * xa
// so lanes that hold columns 0-3 get the low sub-block's sum as D2 - D1 and lanes that hold columns 4-7 the
// high sub-block's as D1 / 16: one mask per four bytes instead of a mask and a shift-and-mask, and all eight
// columns do work. The 6-bit sub-block scales multiply in integers (the sign and the lane's choice between the
// two sub-blocks are in the scale the lane picks), once per super-block the sum becomes a float and meets d;
// the "min" term is one more small MMA of the 6-bit mins against the sub-block sums of the activations.
// Q8_0 needs no decoding: the file's int8 bytes are the A operand, two tokens share a column block.
//
// Shape: one CTA per SM stages the activations and owns a contiguous set of 16-row tiles; its warps split the
// (row tile, k) tiles of those rows into contiguous ranges. A tile is ONE TMA box copy (16 rows x 160 bytes)
// into the warp's private ring of stages, several tiles ahead of the multiply; every warp issues its own copies
// (an issuing lane waits about 170 cycles for the copy engine to take a box: sixteen warps issue in parallel, a
// warp that only copied for the others could not keep up), the first before the kernel boundary, the rest of the
// ring between the steps of the activation staging. A warp takes two tiles per round of its loop where the next
// one continues the row tile (both waited for first; the round's requests, waits and warp barrier paid once).
// The kernel is launched as a programmatic dependent: ring and first copies start while the kernel before it drains.
// Optional phases: attn_combine's merge in front (MV_ATTN_COMBINE), rope_append in the epilogue (MV_ROPE_APPEND).
//
// Fragment layout of mma.m16n8k32 (lane = 4 g + t): A regs {row g, k 4t..4t+3}, {row g+8, same},
// {row g, k 16+4t..}, {row g+8, same}; B regs {k 4t..4t+3, col g}, {k 16+4t.., col g}; C regs
// {row g, cols 2t, 2t+1}, {row g+8, same}. A lane's 8 consecutive weight bytes fill its two k groups, so a
// lane's B registers are 8 consecutive activation bytes too.

#include "imma_util.cuh"
#include "k_attn_fast.cuh"
#include "k_matvec_common.cuh"
#include "tma_util.cuh"

namespace {

using namespace mv;
using namespace imma;

constexpr int FIX_BITS = 25;   // |X| <= 2^25, so a 32-element sub-block sum fits 32 bits
constexpr int XPAD = 32;       // bytes of padding per digit plane: the four planes a half-warp reads hit different banks
constexpr int Q8_UNIT = 4;     // blocks per Q8_0 tile
constexpr int TILE_SCALES = 16 * TILE_ROW;       // where a Q8_0 tile's [16 rows][16 bytes] of scales sit
// a stage of the ring (a multiple of 128 bytes): 16 rows of 160 bytes, and for Q8_0 the 256 bytes of scales
__host__ __device__ constexpr int tile_bytes(bool q4) { return 16 * TILE_ROW + (q4 ? 0 : 256); }
constexpr int SMEM_MAX = 220 * 1024;   // (a fifth stage at k = 4096 would fit in 227 KB; measured: no gain)

#ifdef ZCU_TRACE
// Debug build only: per-CTA timestamps of the kernel's phases (globaltimer, ns).
__device__ unsigned long long g_mv_trace[256 * 12];
__device__ int g_mv_dbg;   // bit 0: the tile stream without its arithmetic; bit 1: the arithmetic without copies or waits
#define MV_DBG g_mv_dbg
#define TRACE(i)                                                                    \
    do {                                                                            \
        if (threadIdx.x == 0 && blockIdx.x < 256) {                                 \
            unsigned long long t__;                                                 \
            asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t__));                \
            g_mv_trace[blockIdx.x * 12 + (i)] = t__;                                 \
        }                                                                           \
    } while (0)
#else
#define TRACE(i) do {} while (0)
#define MV_DBG 0
#endif

// Tensor map of a weight matrix for these tiles: the matrix as bytes, boxes of 16 rows x 160 bytes (or x 16
// bytes for the scales of Q8_0 rows). The box is 160 bytes wide so that rows sit 160 bytes apart in shared
// memory and the 8-byte fragment loads of a half-warp cover 128 distinct bytes; the 16 (Q4_K) or 32 (Q8_0)
// extra bytes of a row are the start of the next tile's (sectors that are fetched anyway) or zeros past the
// row's end. `rows`: every row the multiply may touch (both halves of a SILU_PAIR matrix).
bool weight_map(CUtensorMap* map, const void* w, bool q4, int k, size_t rows, bool scales) {
    const uint64_t rb = q4 ? (uint64_t)(k / 256) * 144 : (((uint64_t)k + k / 16 + 15) & ~(uint64_t)15);
    return tma::bytes_2d(map, w, rows, rb, scales ? 16u : (uint32_t)TILE_ROW, 16u);
}

struct Layout {
    int ring, mbar, xd, sxd, inv, red, ss, tab, total;
};
// Shared memory of a CTA of `warps` warps that stages `tokens` tokens: the ring and its barriers, the digit
// planes xd[4 * tokens][k + XPAD], (Q4_K) the digits of the sub-block sums sxd[4 * tokens][k / 32 + 16], the
// inverse block scales inv[tokens][k / 256], the warps' parked sums red[warps][seg_max][16][slots], the warps'
// partial sums of squares ss[tokens][warps], and the epilogue's tables tab[]: where each warp's range of tiles
// starts (warps + 1), the first (row tile, part) of each warp (warps), then the tokens' RMS scales.
// (`xd_min`: bytes the digit planes' region must hold at least: attn_combine's shared memory, when it runs first)
__host__ __device__ inline Layout layout(int warps, int tokens, int k, bool q4, int slots, int seg_max, int stages, int xd_min = 0) {
    Layout L;
    int off = 0;
    L.ring = off;
    off += warps * stages * tile_bytes(q4);
    L.mbar = off;
    off += warps * stages * 8;
    off = (off + 127) & ~127;
    L.xd = off;
    off += max(4 * tokens * (k + XPAD), (xd_min + 15) & ~15);
    L.sxd = off;
    if (q4) off += 4 * tokens * (k / 32 + 16);
    off = (off + 15) & ~15;
    L.inv = off;
    off += tokens * (k / 256) * 4;
    off = (off + 15) & ~15;
    L.red = off;
    off += warps * seg_max * 16 * slots * 4;
    off = (off + 15) & ~15;
    L.ss = off;
    off += tokens * warps * 8;
    L.tab = off;
    off += (2 * warps + 2 + tokens) * 4;
    L.total = off;
    return L;
}

// Segments a warp may need: its range of ceil(nt / warps) tiles crosses a (row tile, part) boundary every
// `units` tiles.
inline int segments_needed(int n, int k, bool q4, bool pair, int grid, int warps) {
    const int units = q4 ? k / 256 : (k / 32 + Q8_UNIT - 1) / Q8_UNIT;
    const int row_tiles = (n + 15) / 16;
    const int per_cta = (row_tiles + grid - 1) / grid;
    const int nt = per_cta * (pair ? 2 : 1) * units;
    const int len = (nt + warps - 1) / warps;
    return len / units + 2;
}

// CTAs of a launch: every CTA owns floor or ceil(row_tiles / grid) row tiles and the slowest sets the time, so the
// count is the one (from 3/4 of the SMs up) that wastes the least of grid * ceil(row_tiles / grid); ties go to
// the larger count. 896 row tiles on 148 SMs: 128 CTAs of 7 instead of 140 of 6 and 8 of 7.
inline int balanced_grid(int row_tiles, int sms) {
    if (row_tiles <= sms) return row_tiles;
    int best = sms;
    double best_eff = 0.0;
    for (int gsz = sms; gsz >= (3 * sms + 3) / 4; gsz--) {
        const int per = (row_tiles + gsz - 1) / gsz;
        const double eff = (double)row_tiles / ((double)gsz * per) * (0.5 + 0.5 * (double)gsz / sms);  // fewer SMs: fewer tiles in flight
        if (eff > best_eff + 1e-9) {
            best_eff = eff;
            best = gsz;
        }
    }
    return best;
}

// Balanced byte digits of four 32-bit integers, transposed: dg[d] holds digit d of X[0..3] (one byte each).
// X + 0x80808080 biases every byte by 128 with the carries a balanced representation needs; flipping the top
// bit of each byte takes the bias out again: X = sum_d (int8)byte_d * 256^d.
__device__ __forceinline__ void digits4(const int* X, uint32_t* dg) {
    uint32_t y[4];
#pragma unroll
    for (int q = 0; q < 4; q++) y[q] = ((uint32_t)X[q] + 0x80808080u) ^ 0x80808080u;
    const uint32_t t0 = __byte_perm(y[0], y[1], 0x5140), t1 = __byte_perm(y[2], y[3], 0x5140);
    const uint32_t t2 = __byte_perm(y[0], y[1], 0x7362), t3 = __byte_perm(y[2], y[3], 0x7362);
    dg[0] = __byte_perm(t0, t1, 0x5410);
    dg[1] = __byte_perm(t0, t1, 0x7632);
    dg[2] = __byte_perm(t2, t3, 0x5410);
    dg[3] = __byte_perm(t2, t3, 0x7632);
}

// attn_combine's merge for the multiply's MV_ATTN_COMBINE phase, out of line: the multiplies that do not use it
// (all but one per layer) keep its code out of their instruction stream.
__device__ __noinline__ void combine_phase(const MvCombine& comb, const PeerUse& cpu, unsigned char* smem, int cta, int ncta, int tid,
                                           int nthreads, int* status) {
    for (int c = cta; c < comb.blocks; c += ncta) {
        VBlock vb;
        vb.x = c % (int)comb.p.heads, vb.y = c / (int)comb.p.heads, vb.z = 0;
        vb.tid = tid, vb.nthreads = nthreads, vb.bar = 1;
        vb.smem = smem;
        attn::attn_combine_body(vb, comb.p, comb.qg, comb.part, comb.out, comb.step, comb.seq_pos, comb.kb, status, &cpu);
        vb.sync();   // the next merge, or the staging, reuses the shared memory
    }
}

// TYPE: W_Q4_K or W_Q8_0. NT: tokens of the pass (1..4). STAGES: tiles in flight per warp. W: warps per CTA.
template <int TYPE, int NT, int STAGES, int W>
__global__ void __launch_bounds__(W * 32, 16 / W) matvec_imma(PMatvec p, const float* __restrict__ x,
                                                             const __grid_constant__ CUtensorMap wmap,
                                                             const __grid_constant__ CUtensorMap smap, float* __restrict__ out,
                                                             const float* __restrict__ norm_w, int t0, int seg_max,
                                                             int* __restrict__ status, const __grid_constant__ MvRope rope_arg,
                                                             const __grid_constant__ PeerUse pu_arg, const __grid_constant__ MvCombine comb) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    constexpr int NB = Q4 ? NT : (NT + 1) / 2;   // 8-column blocks: one per token (Q4_K), one per two tokens (Q8_0)
    constexpr int SLOTS = Q4 ? NT : 2 * NB;       // token slots of a parked segment
    constexpr int THREADS = W * 32;
    extern __shared__ __align__(128) uint8_t smem[];
    // (broadcast from lane 0: the compiler then knows the warp index, and what derives from it - ring addresses, tile
    // coordinates - to be the same in every lane, and feeds the copy instructions from uniform registers)
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    const int g = lane >> 2, t = lane & 3;
    const int k = (int)p.k, n = (int)p.n;
    const int cta = (int)blockIdx.x, ncta = (int)gridDim.x;
    const bool norm = (p.flags & MV_NORM) != 0, pair = (p.flags & MV_SILU_PAIR) != 0;
    const MvRope* rope = (p.flags & MV_ROPE_APPEND) ? &rope_arg : nullptr;
    const PeerUse* pu = &pu_arg;
    const Layout L = layout(W, NT, k, Q4, SLOTS, seg_max, STAGES, comb.blocks ? (int)attn::attn_combine_smem((int)comb.p.max_blocks) : 0);
    const int xcol = k + XPAD, sxcol = k / 32 + 16, nblk = k / 256;
    const int nparts = pair ? 2 : 1;
    const int units = Q4 ? k / 256 : (k / 32 + Q8_UNIT - 1) / Q8_UNIT;  // tiles along k
    const int row_tiles = (n + 15) / 16;
    // CTA `cta` owns the contiguous row tiles [rt_lo, rt_hi); its tiles, ordered (row tile, part, k), are cut
    // into W contiguous ranges, one per warp.
    const int rt_lo = (int)((unsigned)cta * (unsigned)row_tiles / (unsigned)ncta);   // cta * row_tiles < 2^31
    const int rt_hi = (int)((unsigned)(cta + 1) * (unsigned)row_tiles / (unsigned)ncta);
    const int per_rt = nparts * units;
    const int nt = (rt_hi - rt_lo) * per_rt;
    const int lo = (int)(((unsigned)warp * (unsigned)nt) / W), hi = (int)(((unsigned)(warp + 1) * (unsigned)nt) / W);
    TRACE(0);
    // (the kernel after this one may be scheduled as soon as every CTA of this one has started: it waits for this
    // one's end itself, before it reads what this one writes)
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

    // ---- the ring: this warp's stages and their barriers; the first STAGES - 1 tiles are asked for at once
    constexpr int TILE_BYTES = tile_bytes(Q4);
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem + L.ring) + (uint32_t)warp * STAGES * TILE_BYTES;
    const uint32_t mbar = (uint32_t)__cvta_generic_to_shared(smem + L.mbar) + (uint32_t)warp * STAGES * 8;
    if (lane == 0) {
        if (warp == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"((uint64_t)&wmap));
            if (!Q4) asm volatile("prefetch.tensormap [%0];\n" ::"l"((uint64_t)&smap));
        }
#pragma unroll
        for (int st = 0; st < STAGES; st++) mbar_init(mbar + 8 * st, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    TRACE(8);
    int is_stage = 0, issued = lo;
    int is_rp = lo / units, is_unit = lo % units;   // (row tile, part) index and k tile of the next copy
    auto issue = [&]() {
        if (issued >= hi) return;
        // (the stage's last reader was this warp's tile STAGES - 1 iterations ago: its loads have long returned,
        // the multiplies that used them have been issued, and the __syncwarp after them has passed)
        if (lane == 0) {
            const uint32_t mb = mbar + 8 * is_stage;
            const uint32_t dst = ring + (uint32_t)is_stage * TILE_BYTES;
            const int rtl = pair ? is_rp >> 1 : is_rp;
            const int y = ((pair && (is_rp & 1)) ? (int)p.half : 0) + (rt_lo + rtl) * 16;
            if constexpr (Q4) {
                mbar_expect_tx(mb, 16u * TILE_ROW);
                tma_tile(dst, &wmap, is_unit * 144, y, mb);
            } else {
                // four blocks of values, and the 16 bytes that hold the scales of blocks (b0 & ~7) .. +7 (k is a
                // multiple of 256 here, so both boxes start on 16-byte boundaries)
                const int b0 = is_unit * Q8_UNIT;
                mbar_expect_tx(mb, 16u * TILE_ROW + 256u);
                tma_tile(dst, &wmap, b0 * 32, y, mb);
                tma_tile(dst + TILE_SCALES, &smap, k + 2 * (b0 & ~7), y, mb);
            }
        }
        issued++;
        is_stage = is_stage + 1 == STAGES ? 0 : is_stage + 1;
        if (++is_unit == units) {
            is_unit = 0;
            is_rp++;
        }
    };
    const int dbg = MV_DBG;
    // The copy engine takes a box every few tens of cycles, and an issuing lane waits while its queue is full:
    // 16 warps x (STAGES - 1) boxes keep it busy for more than a microsecond. Each warp asks for its first tile
    // here and for the rest of its ring between the steps of the activation staging below.
    int fill = (dbg & 2) ? 0 : STAGES - 2;
    if (!(dbg & 2)) issue();
    auto fill_one = [&]() {
        if (fill > 0) {
            issue();
            fill--;
        }
    };

    int8_t* xd = reinterpret_cast<int8_t*>(smem + L.xd);
    int8_t* sxd = reinterpret_cast<int8_t*>(smem + L.sxd);
    float* inv = reinterpret_cast<float*>(smem + L.inv);
    float* red = reinterpret_cast<float*>(smem + L.red);
    double* ssw = reinterpret_cast<double*>(smem + L.ss);
    int* tab_lo = reinterpret_cast<int*>(smem + L.tab);          // [W + 1]: first tile of each warp's range
    int* tab_rp = tab_lo + W + 1;                                // [W]: first (row tile, part) of each warp
    float* nsc = reinterpret_cast<float*>(tab_rp + W + 1);       // [NT]: the tokens' RMS scales
    if (lane == 0) {
        tab_lo[warp] = lo;
        tab_rp[warp] = lo / units;
        if (warp == W - 1) tab_lo[W] = nt;
    }

    // the norm weights are constants: this lane's share for the warp's first two blocks is loaded now, while the
    // kernel before this one is still running
    float4 nwr[2][2];
#pragma unroll
    for (int u = 0; u < 2; u++) {
        nwr[u][0] = nwr[u][1] = make_float4(1.f, 1.f, 1.f, 1.f);
        const int blk = warp + u * W;
        if (norm && blk < nblk) {
            // (volatile: the loads must be issued here, ahead of the wait, not where their values are used)
            const float4* src = reinterpret_cast<const float4*>(norm_w) + blk * 64 + lane;
            asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(nwr[u][0].x), "=f"(nwr[u][0].y), "=f"(nwr[u][0].z), "=f"(nwr[u][0].w) : "l"(src));
            asm volatile("ld.global.nc.v4.f32 {%0,%1,%2,%3}, [%4];\n" : "=f"(nwr[u][1].x), "=f"(nwr[u][1].y), "=f"(nwr[u][1].z), "=f"(nwr[u][1].w) : "l"(src + 32));
        }
    }
    TRACE(1);
    // everything before touched only the weights, which no kernel writes; from here on the activations are
    // read, so the kernels before this one must have finished on this GPU (in a tensor-parallel exchange the
    // reads themselves wait for the other ranks' slices)
    // the exchange tags of this run of the launch list
    const bool x_exchanged = pu->wait_slot != PEER_NONE, pushing = pu->push_slot != PEER_NONE;
    const uint32_t x_tag = x_exchanged ? peer::want_tag(*pu) : 0u, out_tag = pushing ? peer::push_tag(*pu) : 0u;
    if (!(dbg & 8)) asm volatile("griddepcontrol.wait;\n" ::: "memory");
    TRACE(2);
    // MV_ATTN_COMBINE: the input is the attention output, and nobody has merged the attention's partials into it yet.
    // The first CTAs do (one head of one row each, attn_combine's own code on this CTA's 512 threads, its shared
    // memory where the digit planes will be); they push the heads under the tag this multiply's staging waits for,
    // so every CTA - on this rank and on the others - sees them arrive element by element.
    if (comb.blocks != 0) {
        if constexpr (W * 32 == attn::AC_THREADS) {
            PeerUse cpu = *pu;
            cpu.push_slot = pu->wait_slot;
            cpu.wait_slot = PEER_NONE;
            if (comb.p.heads != 0) combine_phase(comb, cpu, smem + L.xd, cta, ncta, tid, W * 32, status);
        }
    }
    // the value this thread's first output accumulates onto: asked for now, needed after the tile stream
    float first_old = 0.f;
    const int ep = tid >> 2;   // the first output this thread's quad writes in the epilogue
    if ((p.flags & MV_ACCUMULATE) && ep < (rt_hi - rt_lo) * 16 * NT) {
        const int j0 = (rt_lo + ep / (NT * 16)) * 16 + (ep / NT) % 16;
        if (j0 < n) first_old = __ldcg(out + (size_t)(t0 + ep % NT) * p.out_stride + p.col0 + j0);
    }

    // MV_ROPE_APPEND: the position and the (cos, sin) pair of this thread's first output, asked for now too
    uint32_t rope_pos = 0;
    float2 rope_cs = make_float2(1.f, 0.f);
    if (rope != nullptr && ep < (rt_hi - rt_lo) * 16 * NT) {
        const int tok = t0 + ep % NT;
        rope_pos = rope->seq_pos ? __ldcg(rope->seq_pos + tok) : __ldcg(&rope->step->pos0) + (uint32_t)tok;
        const PRopeAppend& r = rope->p;
        const uint32_t col = p.col0 + (uint32_t)((rt_lo + ep / (NT * 16)) * 16 + (ep / NT) % 16), hd = r.head_dim;
        const bool is_q = col < r.k_off, is_k = !is_q && col < r.v_off;
        const uint32_t d = is_q ? col % (r.gated ? 2 * hd : hd) : (col - (is_k ? r.k_off : r.v_off)) % hd;
        if ((is_q || is_k) && d < r.n_rot) rope_cs = __ldg(rope->table + (size_t)rope_pos * (r.n_rot / 2) + d / 2);
    }

    // ---- activations -> fixed point. Each warp takes whole 256-element blocks of a token: the block's largest
    //      magnitude (of x, or of x * norm_w) gives a power-of-two scale s with |x s| <= 2^25, X = rint(x s) is
    //      split into four balanced byte digits (planes of xd), and the exact sums of X over each 32 elements
    //      into four digits too (sxd, the Q4_K min term). 1 / s goes to inv[]. With NORM the RMS scale is a
    //      factor of every output and is applied in the epilogue; the warps leave their sums of squares in ss[].
    if (!(dbg & 4)) {
        const int xr = p.x_stride ? (int)p.x_stride * 4 : k;
        constexpr int UBX = 2;   // blocks per round of an exchanged vector (a slot is twice a float)
        const int ub = x_exchanged ? UBX : 4;   // blocks per round
#pragma unroll 1
        for (int tk = 0; tk < NT; tk++) {
            const float* xt = x + (size_t)(t0 + tk) * xr;
            double ss = 0.0;
#pragma unroll 1
            for (int b0 = warp; b0 < nblk; b0 += ub * W) {
                // up to four blocks per round: their loads are in flight together
                float4 a[4][2];
#pragma unroll
                for (int u = 0; u < 4; u++) a[u][0] = a[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (x_exchanged) {
                    uint4 raw[UBX][2][2];
#pragma unroll
                    for (int u = 0; u < UBX; u++)
#pragma unroll
                        for (int h = 0; h < 2; h++)
                            if (b0 + u * W < nblk) peer::look4(*pu, xt + 4 * ((b0 + u * W) * 64 + 32 * h + lane), raw[u][h][0], raw[u][h][1]);
#pragma unroll
                    for (int u = 0; u < UBX; u++)
#pragma unroll
                        for (int h = 0; h < 2; h++)
                            if (b0 + u * W < nblk)
                                a[u][h] = peer::take4(*pu, xt + 4 * ((b0 + u * W) * 64 + 32 * h + lane), x_tag, raw[u][h][0], raw[u][h][1], status);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        const int blk = b0 + u * W;
                        if (blk < nblk) {
                            a[u][0] = __ldcg(reinterpret_cast<const float4*>(xt) + blk * 64 + lane);
                            a[u][1] = __ldcg(reinterpret_cast<const float4*>(xt) + blk * 64 + 32 + lane);
                        }
                    }
                }
                fill_one();
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int blk = b0 + u * W;
                    if (blk >= nblk || u >= ub) break;   // warp-uniform
                    float amax = 0.f;
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        float4& v = a[u][h];
                        if (norm) {
                            ss += ((double)__fmul_rn(v.x, v.x) + (double)__fmul_rn(v.y, v.y)) +
                                  ((double)__fmul_rn(v.z, v.z) + (double)__fmul_rn(v.w, v.w));
                            float4 nw;
                            if (u < 2 && b0 == warp) nw = nwr[u][h];
                            else nw = __ldg(reinterpret_cast<const float4*>(norm_w) + blk * 64 + 32 * h + lane);
                            v.x = __fmul_rn(v.x, nw.x);
                            v.y = __fmul_rn(v.y, nw.y);
                            v.z = __fmul_rn(v.z, nw.z);
                            v.w = __fmul_rn(v.w, nw.w);
                        }
                        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
                    fill_one();
                    TRACE(9);
                    float sc = 1.0f, is = 1.0f;
                    if (amax > 0.f && amax < 3.0e38f) {
                        // amax = f * 2^e with f in [1, 2): scale 2^(24 - e), so |x * scale| < 2^25
                        const int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
                        const int se = max(-100, min(100, FIX_BITS - 1 - e));
                        sc = __uint_as_float((uint32_t)(se + 127) << 23);
                        is = __uint_as_float((uint32_t)(127 - se) << 23);
                    }
                    if (lane == 0) inv[tk * nblk + blk] = is;
#pragma unroll
                    for (int h = 0; h < 2; h++) {
                        const float4 v = a[u][h];
                        int X[4] = {__float2int_rn(v.x * sc), __float2int_rn(v.y * sc), __float2int_rn(v.z * sc), __float2int_rn(v.w * sc)};
                        uint32_t dg[4];
                        digits4(X, dg);
                        const int e0 = blk * 256 + 128 * h + 4 * lane;
#pragma unroll
                        for (int d = 0; d < 4; d++) *reinterpret_cast<uint32_t*>(xd + (size_t)(4 * tk + d) * xcol + e0) = dg[d];
                        if (Q4) {
                            // exact sum over the 32 elements of a sub-block: 8 consecutive lanes
                            int sum = X[0] + X[1] + X[2] + X[3];
                            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                            if ((lane & 7) == 0) {
                                const uint32_t y = ((uint32_t)sum + 0x80808080u) ^ 0x80808080u;
                                const int sb = blk * 8 + 4 * h + (lane >> 3);
#pragma unroll
                                for (int d = 0; d < 4; d++) sxd[(size_t)(4 * tk + d) * sxcol + sb] = (int8_t)((y >> (8 * d)) & 0xffu);
                            }
                        }
                    }
                }
            }
            if (norm) {
                ss = warp_sum_d(ss);
                if (lane == 0) ssw[tk * W + warp] = ss;
            }
        }
    }
    TRACE(10);
    while (fill > 0) fill_one();
    TRACE(11);
    __syncthreads();  // every warp reads every block of xd
    TRACE(3);
    if (norm && warp < NT && lane == 0) {
        // the token's RMS scale: squares in f32, their sum in f64 (src/ref/ops.zig:30-41), the warps' sums in order
        double tot = 0.0;
#pragma unroll
        for (int wv = 0; wv < W; wv++) tot += ssw[warp * W + wv];
        const float mean = (k & (k - 1)) == 0 ? (float)(tot * (1.0 / (double)k)) : (float)(tot / (double)k);
        nsc[warp] = 1.0f / sqrtf(mean + p.eps);
    }

    // ---- the tile stream
    float accf[NB][4];
#pragma unroll
    for (int b = 0; b < NB; b++) accf[b][0] = accf[b][1] = accf[b][2] = accf[b][3] = 0.f;
    // digits -> value: this lane's columns 2t, 2t+1 are digits 2(t&1), 2(t&1)+1
    const float w0 = (t & 1) ? 65536.0f : 1.0f, w1 = w0 * 256.0f;
    int seg = 0;
    int cur_rp = lo / units, cur_unit = lo % units;
    int cs_stage = 0;
    uint32_t phase_bits = 0;   // bit st: the parity to wait for on stage st

    auto park = [&]() {
        // parks this warp's sums for (row tile, part) cur_rp in segment `seg`
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v0 = __fmaf_rn(accf[b][1], w1, accf[b][0] * w0);
            float v1 = __fmaf_rn(accf[b][3], w1, accf[b][2] * w0);
            v0 = __fadd_rn(v0, __shfl_xor_sync(0xffffffffu, v0, 1));  // low digits + high digits
            v1 = __fadd_rn(v1, __shfl_xor_sync(0xffffffffu, v1, 1));
            float* rr = red + ((size_t)(warp * seg_max + seg) * 16) * SLOTS;
            if constexpr (Q4) {
                v0 = __fadd_rn(v0, __shfl_xor_sync(0xffffffffu, v0, 2));  // low sub-blocks + high sub-blocks
                v1 = __fadd_rn(v1, __shfl_xor_sync(0xffffffffu, v1, 2));
                if (t == 0 && seg < seg_max) {
                    rr[g * SLOTS + b] = v0;
                    rr[(g + 8) * SLOTS + b] = v1;
                }
            } else {
                const int slot = 2 * b + (t >> 1);
                if ((t & 1) == 0 && seg < seg_max && slot < SLOTS) {
                    rr[g * SLOTS + slot] = v0;
                    rr[(g + 8) * SLOTS + slot] = v1;
                }
            }
            accf[b][0] = accf[b][1] = accf[b][2] = accf[b][3] = 0.f;
        }
        seg++;
    };

    // lane-constant offsets into a tile: header of row g; bytes 16 + 8 t (Q4_K) or 8 t (Q8_0) of row g
    const uint32_t hoff = (uint32_t)g * TILE_ROW;
    const uint32_t qoff = hoff + (Q4 ? 16u : 0u) + 8u * (uint32_t)t;
    const uint32_t xd_s = (uint32_t)__cvta_generic_to_shared(xd), sxd_s = (uint32_t)__cvta_generic_to_shared(sxd);
    // Q4_K lane constants. Lanes t < 2 hold columns 0-3 (the low-nibble sub-block 2j), lanes t >= 2 columns 4-7
    // (the high-nibble sub-block 2j + 1). Scale selectors for PRMT (byte jb or jb + 1 of the register that holds
    // four sub-block scales; selector 4 reads the zero operand):
    //   sA multiplies D2: the low sub-block's scale for t < 2, zero otherwise
    //   sB multiplies D1: minus the low sub-block's scale for t < 2, the high sub-block's otherwise
    const bool hi_lane = t >= 2;
    const uint32_t selA[2] = {hi_lane ? 0x4444u : 0x4440u, hi_lane ? 0x4444u : 0x4442u};
    const uint32_t selB[2] = {hi_lane ? 0x4441u : 0x4440u, hi_lane ? 0x4443u : 0x4442u};
    const int sgnB = hi_lane ? 1 : -1;
    const float dfac = hi_lane ? 0.0625f : 1.0f;
    // this lane's B bytes: plane (4 b + (g & 3)), the group's second half for g >= 4, bytes 8t..8t+7
    const uint32_t xb_lane = xd_s + (uint32_t)(g & 3) * (uint32_t)xcol + 32u * (uint32_t)(g >> 2) + 8u * (uint32_t)t;
    bool timed_out = false;
#ifdef ZCU_TRACE
    long long tr_wait = 0, tr_comp = 0;
#endif
    int freed = 1;   // stages without a tile on its way (all but one were asked for before the loop)
    // the arithmetic of one tile (its sums join accf)
    auto tile_math = [&](const uint32_t tile, const int unit) {
        if (dbg & 1) {
        } else if constexpr (Q4) {
            const uint4 h0 = lds128(tile + hoff), h1 = lds128(tile + hoff + 8 * TILE_ROW);
            // 6-bit scales and mins of the eight sub-blocks, four per register (src/ref/tensor.zig:95-98)
            const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u)};
            const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u)};
            const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u)};
            const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u)};
            int run[NB][4];
#pragma unroll
            for (int b = 0; b < NB; b++) run[b][0] = run[b][1] = run[b][2] = run[b][3] = 0;
            const uint32_t xb = xb_lane + (uint32_t)unit * 256u;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 q0 = lds64(tile + qoff + 32 * j), q1 = lds64(tile + qoff + 8 * TILE_ROW + 32 * j);
                const uint32_t a0 = q0.x & 0xf0f0f0f0u, a1 = q1.x & 0xf0f0f0f0u, a2 = q0.y & 0xf0f0f0f0u, a3 = q1.y & 0xf0f0f0f0u;
                const int sA0 = (int)__byte_perm(sc0[j >> 1], 0u, selA[j & 1]), sA1 = (int)__byte_perm(sc1[j >> 1], 0u, selA[j & 1]);
                const int sB0 = (int)__byte_perm(sc0[j >> 1], 0u, selB[j & 1]) * sgnB, sB1 = (int)__byte_perm(sc1[j >> 1], 0u, selB[j & 1]) * sgnB;
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const uint2 bv = lds64(xb + (uint32_t)(4 * b) * (uint32_t)xcol + 64u * j);
                    int d1[4], d2[4];
                    imma_u8(d1, a0, a1, a2, a3, bv.x, bv.y);
                    imma_u8(d2, q0.x, q1.x, q0.y, q1.y, bv.x, bv.y);
                    run[b][0] += d2[0] * sA0 + d1[0] * sB0;
                    run[b][1] += d2[1] * sA0 + d1[1] * sB0;
                    run[b][2] += d2[2] * sA1 + d1[2] * sB1;
                    run[b][3] += d2[3] * sA1 + d1[3] * sB1;
                }
            }
            // mins: lanes t = 0, 1 carry the eight 6-bit mins of rows g and g+8 (four per register); their B
            // operand is the digits of the eight sub-block sums, in columns 0-3 only
            const uint32_t ma0 = t == 0 ? mn0[0] : (t == 1 ? mn0[1] : 0u);
            const uint32_t ma1 = t == 0 ? mn1[0] : (t == 1 ? mn1[1] : 0u);
            const float d0 = __half2float(__ushort_as_half((unsigned short)(h0.x & 0xffffu))) * dfac;
            const float d1f = __half2float(__ushort_as_half((unsigned short)(h1.x & 0xffffu))) * dfac;
            const float dm0 = -__half2float(__ushort_as_half((unsigned short)(h0.x >> 16)));
            const float dm1 = -__half2float(__ushort_as_half((unsigned short)(h1.x >> 16)));
#pragma unroll
            for (int b = 0; b < NB; b++) {
                uint32_t bs = 0;
                if (g < 4 && t < 2) bs = lds32(sxd_s + (uint32_t)(4 * b + g) * (uint32_t)sxcol + (uint32_t)unit * 8u + 4u * (uint32_t)t);
                int am[4];
                imma_16832(am, ma0, ma1, 0u, 0u, bs, 0u);
                const float is = inv[b * nblk + unit];
                float* af = accf[b];
                af[0] = __fmaf_rn((float)run[b][0], d0 * is, af[0]);
                af[1] = __fmaf_rn((float)run[b][1], d0 * is, af[1]);
                af[2] = __fmaf_rn((float)run[b][2], d1f * is, af[2]);
                af[3] = __fmaf_rn((float)run[b][3], d1f * is, af[3]);
                af[0] = __fmaf_rn((float)am[0], dm0 * is, af[0]);
                af[1] = __fmaf_rn((float)am[1], dm0 * is, af[1]);
                af[2] = __fmaf_rn((float)am[2], dm1 * is, af[2]);
                af[3] = __fmaf_rn((float)am[3], dm1 * is, af[3]);
            }
        } else {
            const int b0 = unit * Q8_UNIT;
            const int nb32 = k / 32;
            // the 16 bytes copied hold the scales of blocks (b0 & ~7) .. +7: this tile's four are its low or high half
            const uint2 s0 = lds64(tile + TILE_SCALES + 16 * g + 8 * (unit & 1)), s1 = lds64(tile + TILE_SCALES + 16 * (g + 8) + 8 * (unit & 1));
            const uint32_t scw0[2] = {s0.x, s0.y}, scw1[2] = {s1.x, s1.y};
            float is[NB];
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int slot = 2 * b + (t >> 1);
                is[b] = slot < NT ? inv[slot * nblk + (unit >> 1)] : 0.f;
            }
#pragma unroll
            for (int i = 0; i < Q8_UNIT; i++) {
                const int blk = b0 + i;
                if (blk < nb32) {
                    const uint2 q0 = lds64(tile + qoff + 32 * i), q1 = lds64(tile + qoff + 8 * TILE_ROW + 32 * i);
                    const float d0 = __half2float(__ushort_as_half((unsigned short)((scw0[i >> 1] >> (16 * (i & 1))) & 0xffffu)));
                    const float d1f = __half2float(__ushort_as_half((unsigned short)((scw1[i >> 1] >> (16 * (i & 1))) & 0xffffu)));
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        // column 8 b + g = digit (g & 3) of token 2 b + (g >> 2)
                        uint2 bv = make_uint2(0, 0);
                        if (2 * b + (g >> 2) < NT) bv = lds64(xd_s + (uint32_t)(8 * b + g) * (uint32_t)xcol + (uint32_t)blk * 32u + 8u * (uint32_t)t);
                        int acc[4];
                        imma_16832(acc, q0.x, q1.x, q0.y, q1.y, bv.x, bv.y);
                        float* af = accf[b];
                        af[0] = __fmaf_rn((float)acc[0], d0 * is[b], af[0]);
                        af[1] = __fmaf_rn((float)acc[1], d0 * is[b], af[1]);
                        af[2] = __fmaf_rn((float)acc[2], d1f * is[b], af[2]);
                        af[3] = __fmaf_rn((float)acc[3], d1f * is[b], af[3]);
                    }
                }
            }
        }
    };
#pragma unroll 1
    for (int tau = lo; tau < hi;) {
#ifdef ZCU_TRACE
        const long long tr0 = clock64();
#endif
        // two tiles a round where the next one belongs to the same (row tile, part): both are waited for before either
        // is touched, so that the arithmetic of the second fills the latencies at the end of the first (the sums keep
        // their order: the first tile's join accf before the second's)
        const bool two = STAGES >= 4 && tau + 1 < hi && cur_unit + 1 < units;
        const int sa = cs_stage, sb = cs_stage + 1 == STAGES ? 0 : cs_stage + 1;
        if (!(dbg & 2)) {
            for (int f = 0; f < freed; f++) issue();  // a tile into every stage that the round before left
            if (!mbar_wait(mbar + 8 * sa, (phase_bits >> sa) & 1u)) timed_out = true;
            if (two && !mbar_wait(mbar + 8 * sb, (phase_bits >> sb) & 1u)) timed_out = true;
        }
#ifdef ZCU_TRACE
        const long long tr1 = clock64();
        tr_wait += tr1 - tr0;
#endif
        phase_bits ^= 1u << sa;
        if (two) phase_bits ^= 1u << sb;
        cs_stage = two ? (sb + 1 == STAGES ? 0 : sb + 1) : sb;
        tile_math(ring + (uint32_t)sa * TILE_BYTES, cur_unit);
        if (two) tile_math(ring + (uint32_t)sb * TILE_BYTES, cur_unit + 1);
        __syncwarp();  // every lane is done with these stages before a later copy overwrites them
        // step to the next tile; on leaving this (row tile, part), park the sums
        freed = two ? 2 : 1;
        tau += freed;
        cur_unit += freed;
        if (cur_unit == units || tau == hi) {
            park();
            if (cur_unit == units) {
                cur_unit = 0;
                cur_rp++;
            }
        }
#ifdef ZCU_TRACE
        tr_comp += clock64() - tr1;
#endif
    }
#ifdef ZCU_TRACE
    if (tid == 0 && blockIdx.x < 256) g_mv_trace[blockIdx.x * 12 + 7] = ((unsigned long long)tr_wait << 32) | (unsigned long long)(tr_comp & 0xffffffffll);
#endif
    if (timed_out && lane == 0 && status) atomicExch(status, 1);
    TRACE(4);
    __syncthreads();
    TRACE(5);

    // ---- add each output's segments in warp order and write it. The warps that hold tiles of (row tile, part)
    //      rp are consecutive, and rp is segment rp - (first rp of the warp) of each. With MV_ROPE_APPEND the row
    //      is Q|K|V: adjacent outputs (2i, 2i+1) of a q or k head are a RoPE pair held by quads NT apart; q is
    //      written rotated, k and v go to the cache at the token's position (rope_append's arithmetic,
    //      src/kernels/rope_append.wgsl; every product rounded, src/ref/ops.zig:64-86).
    const int local_rts = rt_hi - rt_lo;
    const int total = local_rts * 16 * NT;
    // Four adjacent lanes (a quad) work on one output: lane q loads the candidates of warps q W/4 .. (a warp that
    // holds no tile of rp contributes zero) and adds them pairwise; two shuffles add the quads' sums. Together this
    // is one fixed pairwise tree over the W warps: the order does not depend on the step's token count.
    constexpr int CPT = W / 4;
    const int q4 = tid & 3;
    auto seg_sum = [&](int rp, int row, int tk) {
        const int T0 = rp * units, T1 = T0 + units;
        float c[CPT];
#pragma unroll
        for (int e = 0; e < CPT; e++) {
            const int w = q4 * CPT + e;
            const int wlo = tab_lo[w], whi = tab_lo[w + 1];
            const bool has = wlo < T1 && whi > T0 && whi > wlo;   // (an empty range holds nothing)
            const int sg = has ? rp - tab_rp[w] : 0;
            const float r = red[((size_t)(w * seg_max + sg) * 16 + row) * SLOTS + tk];
            c[e] = has ? r : 0.f;
        }
#pragma unroll
        for (int span = 1; span < CPT; span *= 2)
#pragma unroll
            for (int e = 0; e < CPT; e += 2 * span) c[e] = __fadd_rn(c[e], c[e + span]);
        float sum = c[0];
        sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 1));
        sum = __fadd_rn(sum, __shfl_xor_sync(0xffffffffu, sum, 2));
        return sum;
    };
    for (int i0 = 0; i0 < total; i0 += THREADS / 4) {
        const int i = i0 + ep;
        const bool in_range = i < total;
        const int ic = in_range ? i : total - 1;   // (whole warps take part in the shuffles)
        const int tk = ic % NT, row = (ic / NT) % 16, rtl = ic / (NT * 16);
        const int j = (rt_lo + rtl) * 16 + row;
        const bool valid = in_range && j < n;
        float v = seg_sum(rtl * nparts, row, tk), u = 0.f;
        if (pair) u = seg_sum(rtl * nparts + 1, row, tk);
        if (norm) {
            // (explicitly rounded: a product that the compiler fused with the accumulation below in one
            // instantiation and not in another would change a token's bits with the step's token count)
            v = __fmul_rn(v, nsc[tk]);
            u = __fmul_rn(u, nsc[tk]);
        }
        if (!valid) v = u = 0.f;
        if (pair) v = __fmul_rn(silu_f(v), u);
        const size_t o = (size_t)(t0 + tk) * p.out_stride + p.col0 + j;
        if (rope != nullptr) {
            const float other = __shfl_xor_sync(0xffffffffu, v, 4 * NT);  // the pair's other element (whole warps run this loop)
            if (!valid || q4 != 0) continue;
            const PRopeAppend& r = rope->p;
            const int tok = t0 + tk;
            const uint32_t pos = i0 == 0 ? rope_pos : (rope->seq_pos ? rope->seq_pos[tok] : rope->step->pos0 + (uint32_t)tok);
            const uint32_t col = p.col0 + (uint32_t)j, hd = r.head_dim, q_head = r.gated ? 2 * hd : hd;
            const bool is_q = col < r.k_off, is_k = !is_q && col < r.v_off;
            const uint32_t d = is_q ? col % q_head : (col - (is_k ? r.k_off : r.v_off)) % hd;
            float val = v;
            if ((is_q || is_k) && d < r.n_rot) {
                const float2 cs = i0 == 0 ? rope_cs : rope->table[(size_t)pos * (r.n_rot / 2) + d / 2];
                val = (d & 1) ? __fadd_rn(__fmul_rn(other, cs.y), __fmul_rn(v, cs.x)) : __fsub_rn(__fmul_rn(v, cs.x), __fmul_rn(other, cs.y));
            }
            out[o] = is_q ? val : v;  // the row keeps rotated q and, like rope_append, unrotated k and v
            if (!is_q) {
                const uint32_t gh = (col - (is_k ? r.k_off : r.v_off)) / hd;
                const size_t e = (size_t)tok * r._pad[0] + (size_t)pos * r.kv_heads * hd + (size_t)gh * hd + d;
                void* cache = is_k ? rope->kc : rope->vc;
                if (r.kv == KV_F16) reinterpret_cast<__half*>(cache)[e] = __float2half_rn(val);
                else reinterpret_cast<float*>(cache)[e] = val;
            }
            continue;
        }
        if (!valid || q4 != 0) continue;
        if (p.flags & MV_ACCUMULATE) v = __fadd_rn(v, i0 == 0 ? first_old : __ldcg(out + o));
        out[o] = v;
        if (pushing) peer::push(*pu, out + o, v, out_tag);  // this rank's slice, to every rank's exchange slots
    }
    TRACE(6);
}

template <int TYPE, int NT, int STAGES, int W>
zcu_result launch_staged(const LaunchArgs& a, const MvArgs& v, int t0, int grid, int seg_max) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    constexpr int SLOTS = Q4 ? NT : 2 * ((NT + 1) / 2);
    // (every pass of a dispatch with MV_ATTN_COMBINE reserves the merge's shared memory: one layout per dispatch)
    const int xd_min = v.combine.blocks ? (int)attn::attn_combine_smem((int)v.combine.p.max_blocks) : 0;
    const Layout L = layout(W, NT, (int)v.p.k, Q4, SLOTS, seg_max, STAGES, xd_min);
    auto kern = matvec_imma<TYPE, NT, STAGES, W>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_MAX);
        if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "matvec_imma: shared memory attribute: %s", cudaGetErrorString(e));
        configured[dev & 63] = true;
    }
    // Programmatic dependent launch: this kernel may start while the one before it drains; it prefetches
    // weights, then waits (griddepcontrol.wait) before it reads activations.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(W * 32);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // the weights as a byte matrix of 16-row boxes (both halves of a SILU_PAIR matrix are rows of one matrix)
    const size_t rows = (size_t)v.p.n + ((v.p.flags & MV_SILU_PAIR) ? v.p.half : 0);
    CUtensorMap wmap, smap;
    if (!weight_map(&wmap, v.w, Q4, (int)v.p.k, rows, false) || !weight_map(&smap, v.w, Q4, (int)v.p.k, rows, !Q4))
        return zcu_fail(a, ZCU_E_GPU, "matvec_imma: the driver refused a tensor map (n %u, k %u)", v.p.n, v.p.k);
    if (v.combine.blocks != 0) {
        if (W * 32 != attn::AC_THREADS) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec + attn_combine: needs CTAs of 16 warps");
    }
    MvCombine comb = v.combine;
    if (t0 != 0) comb.p.heads = 0;   // (the dispatch's first pass merges every row; blocks != 0 keeps the layout)
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, v.p, v.x, wmap, smap, v.out, v.nw, t0, seg_max, a.status, v.rope, v.peer, comb);
    if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "matvec_imma: launch failed: %s", cudaGetErrorString(e));
    return ZCU_OK;
}

// The deepest ring (at most `want`, 0 = 6) that fits beside the staged activations; 0 when not even two stages fit.
template <int TYPE, int NT, int W>
int stages_that_fit(int k, int seg_max, int want, int smem_cap, int xd_min) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    constexpr int SLOTS = Q4 ? NT : 2 * ((NT + 1) / 2);
    int stages = want ? want : 6;
    while (stages > 2 && layout(W, NT, k, Q4, SLOTS, seg_max, stages, xd_min).total > smem_cap) stages--;
    return layout(W, NT, k, Q4, SLOTS, seg_max, stages, xd_min).total > smem_cap ? 0 : stages;
}

template <int TYPE, int NT, int W>
zcu_result launch_one(const LaunchArgs& a, const MvArgs& v, int t0, int want_stages, bool every_sm) {
    const bool q4 = TYPE == W_Q4_K, pair = (v.p.flags & MV_SILU_PAIR) != 0;
    const int row_tiles = ((int)v.p.n + 15) / 16;
    const int grid = every_sm ? (row_tiles < a.sm_count ? row_tiles : a.sm_count) : balanced_grid(row_tiles, a.sm_count);
    const int seg_max = segments_needed((int)v.p.n, (int)v.p.k, q4, pair, grid, W);
    // two CTAs of eight warps share an SM (this kernel's and its neighbour's in the stream): half the memory each
    const int cap = W == 16 ? SMEM_MAX : 110 * 1024;
    const int stages = stages_that_fit<TYPE, NT, W>((int)v.p.k, seg_max, want_stages, cap,
                                                    v.combine.blocks ? (int)attn::attn_combine_smem((int)v.combine.p.max_blocks) : 0);
    switch (stages) {
        case 2: return launch_staged<TYPE, NT, 2, W>(a, v, t0, grid, seg_max);
        case 3: return launch_staged<TYPE, NT, 3, W>(a, v, t0, grid, seg_max);
        case 4: return launch_staged<TYPE, NT, 4, W>(a, v, t0, grid, seg_max);
        case 5: return launch_staged<TYPE, NT, 5, W>(a, v, t0, grid, seg_max);
        case 6: return launch_staged<TYPE, NT, 6, W>(a, v, t0, grid, seg_max);
        default: return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: k = %u with %d tokens does not fit shared memory", v.p.k, NT);
    }
}

// Tokens one pass can stage beside a two-stage ring.
template <int TYPE, int W>
int tokens_per_pass(int k, int cap) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    int mt = 4;
    while (mt > 1 && layout(W, mt, k, Q4, 4, 8, 2).total > cap) mt--;
    return mt;
}

template <int TYPE, int W>
zcu_result launch_type(const LaunchArgs& a, const MvArgs& v, int stages, bool every_sm) {
    const int cap = tokens_per_pass<TYPE, W>((int)v.p.k, W == 16 ? SMEM_MAX : 110 * 1024);
    MvArgs pass = v;
    for (int t0 = 0; t0 < v.m;) {
        const int mt = (v.m - t0) < cap ? (v.m - t0) : cap;
        zcu_result r;
        switch (mt) {
            case 1: r = launch_one<TYPE, 1, W>(a, pass, t0, stages, every_sm); break;
            case 2: r = launch_one<TYPE, 2, W>(a, pass, t0, stages, every_sm); break;
            case 3: r = launch_one<TYPE, 3, W>(a, pass, t0, stages, every_sm); break;
            default: r = launch_one<TYPE, 4, W>(a, pass, t0, stages, every_sm); break;
        }
        if (r != ZCU_OK) return r;
        t0 += mt;
    }
    return ZCU_OK;
}

}  // namespace

// `stages`: tiles in flight per warp (2..6; 0 = as deep as fits). `shape`, low nibble: 0 = CTAs of 16 warps, one per
// SM; 1 = CTAs of 8 warps with at most half an SM's shared memory, so that the next kernel's CTAs can move in and
// fill their rings while this one still computes. `shape` bit 4: a CTA on every SM (the last ones with a row tile
// fewer) instead of the CTA count that divides the row tiles most evenly. Q8_0 needs k % 256 == 0.
zcu_result launch_matvec_imma(const LaunchArgs& a, const mv::MvArgs& v, int type, int stages, int shape) {
    if (type == mv::W_Q8_0 && v.p.k % 256 != 0) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec_q8_0: k = %u is not a multiple of 256", v.p.k);
    if (type == mv::W_Q4_K && v.p.k % 256 != 0) return zcu_fail(a, ZCU_E_BAD_COMMAND, "matvec_q4_k: k = %u is not a multiple of 256", v.p.k);
    if (stages != 0 && (stages < 2 || stages > 6))
        return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: %d stages is not built", stages);
    const bool every_sm = (shape & 0x10) != 0;
    const int warps = shape & 0x0f;
    if ((shape & ~0x1f) != 0 || warps > 1) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: CTA shape 0x%x is not built", shape);
    if (warps == 1) return type == mv::W_Q4_K ? launch_type<mv::W_Q4_K, 8>(a, v, stages, every_sm) : launch_type<mv::W_Q8_0, 8>(a, v, stages, every_sm);
    return type == mv::W_Q4_K ? launch_type<mv::W_Q4_K, 16>(a, v, stages, every_sm) : launch_type<mv::W_Q8_0, 16>(a, v, stages, every_sm);
}

#ifdef ZCU_TRACE
extern "C" __attribute__((visibility("default"))) int zcu_dbg_trace_read(unsigned long long* out, size_t count) {
    return (int)cudaMemcpyFromSymbol(out, g_mv_trace, count * sizeof(unsigned long long));
}
extern "C" __attribute__((visibility("default"))) int zcu_dbg_mode(int mode) {
    return (int)cudaMemcpyToSymbol(g_mv_dbg, &mode, sizeof(int));
}
extern "C" __attribute__((visibility("default"))) int zcu_dbg_trace_clear() {
    void* ptr = nullptr;
    cudaGetSymbolAddress(&ptr, g_mv_trace);
    return (int)cudaMemset(ptr, 0, sizeof(g_mv_trace));
}
#endif
