// The tensor-core family of the quantised decode multiplies (matvec_q4_k, matvec_q8_0).
//
// Why integer tensor cores: at B200's HBM rate a Q4_K multiply has about three issue slots per
// weight, and turning a 4-bit code into a float on the CUDA cores costs more than that (the integer
// ALU pipe runs at half rate). So the codes stay integers: one mask gives four of them as an s8x4
// A-fragment register, the activations are turned ONCE per CTA into 32-bit fixed point (scaled per
// token by a power of two) and split into four balanced signed bytes, and
// mma.sync.m16n8k32.s32.s8.s8 accumulates exactly. Per 32-weight sub-block the s32 sums are multiplied
// by the 6-bit sub-block scale in integers (IMAD); once per 256-weight super-block they become floats
// and meet the f16 super-block scales d and dmin. The Q4_K "min" term is a second small integer MMA
// of the 6-bit mins against the per-sub-block sums of the fixed-point activations. Q8_0 needs no
// decoding at all: the file's int8 bytes are the A fragment.
//
// Every sum up to the super-block level is exact integer arithmetic, and all later sums have a
// fixed order, so a token's result does not depend on the step's token count.
//
// Shape: one CTA of 16 warps per SM stages the activations once and owns a contiguous set of row
// tiles (16 rows each); its warps split the tiles of those rows along k (see matvec_imma). Each warp
// brings its tiles global -> shared memory with bulk copies (cp.async.bulk on an mbarrier) into a
// private ring, several tiles ahead of the multiply, so HBM latency is covered without holding tiles
// in registers. The kernel is launched as a programmatic dependent: it starts its weight copies while
// the kernel before it drains, and waits (griddepcontrol.wait) only before it reads activations.
//
// Fragment layout of mma.m16n8k32 (lane = 4 g + t): A regs {row g, k 4t..4t+3}, {row g+8, same},
// {row g, k 16+4t..}, {row g+8, same}; B regs {k 4t..4t+3, col g}, {k 16+4t.., col g}; C regs
// {row g, cols 2t, 2t+1}, {row g+8, same}. Columns are (token, digit): col = 4 * token + digit.

#pragma once

#include "k_matvec_common.cuh"
#include "tma_util.cuh"

namespace imma {

using namespace mv;

constexpr int IM_THREADS = 512;
constexpr int IM_WARPS = 16;
// bytes of padding per staged column: fragment loads of neighbouring columns then hit different banks
// (16-byte loads, two columns per phase: 64; 8-byte loads, four columns per phase: 32)
__host__ __device__ constexpr int im_xpad(bool q4) { return q4 ? 64 : 32; }
constexpr int IM_FIX_BITS = 25;   // |X| <= 2^25, so a 32-element sub-block sum fits 32 bits

// D = A * B with a zero accumulator (each sub-block starts a fresh sum: its scale differs).
__device__ __forceinline__ void imma_16832(int* d, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                           uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(0));
}

// ---- bulk copies (the TMA engine, no tensor map) completing on a shared-memory mbarrier
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(mbar)
                 : "memory");
}
// Waits for phase `parity` of the barrier, at most 2^20 polls: a copy that never lands must not hang
// the GPU. Returns false when it gave up (the caller flags the error and carries on).
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity) {
    for (int spin = 0; spin < (1 << 20); spin++) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Where element e of a staged column lives. Q4_K: within each 64-element group the two sub-blocks'
// bytes for a lane sit side by side, so one 16-byte load gives a lane its B registers for both.
template <int TYPE>
__device__ __forceinline__ int stage_pos(int e) {
    if (TYPE == W_Q4_K) return (e & ~63) | (((e >> 3) & 3) << 4) | (((e >> 5) & 1) << 3) | (e & 7);
    return e;
}

// One warp's tile of weights: 16 rows x one super-block (Q4_K, 144 bytes a row) or x four blocks (Q8_0: 128
// value bytes a row, and the 16 bytes that hold the rows' scales). A tile is ONE TMA copy of a 16-row x 160-byte
// box of the weight matrix (seen as a byte matrix through a tensor map), completing on an mbarrier, into a ring
// of stages per warp, several tiles ahead of the one being multiplied; Q8_0 adds a 16 x 16-byte box for the
// scales. One request per tile matters: the TMA unit takes requests at a limited rate, and 16 row copies per
// tile made that rate the bound. The box is 160 bytes wide so that rows sit 160 bytes apart in shared memory
// and the 8-byte fragment loads of a half-warp (four rows) cover 128 distinct bytes; the 16 (Q4_K) or 32
// (Q8_0) extra bytes of a row are the start of the next tile's (sectors that are fetched anyway) or zeros past
// the row's end.
constexpr int Q8_UNIT = 4;        // blocks per Q8_0 tile
constexpr int TILE_ROW = 160;
constexpr int TILE_SCALES = 16 * TILE_ROW;         // where a Q8_0 tile's [16 rows][16 bytes] of scales sit
constexpr int TILE_BYTES = 16 * TILE_ROW + 256;    // a stage: a multiple of 128 bytes

// Tensor map of a weight matrix for these tiles. `rows`: every row the multiply may touch (both halves of a
// SILU_PAIR matrix).
inline bool im_weight_map(CUtensorMap* map, const void* w, bool q4, int k, size_t rows, bool scales) {
    const uint64_t rb = q4 ? (uint64_t)(k / 256) * 144 : (((uint64_t)k + k / 16 + 15) & ~(uint64_t)15);
    return tma::bytes_2d(map, w, rows, rb, scales ? 16u : (uint32_t)TILE_ROW, 16u);
}

__device__ __forceinline__ void tma_tile(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
                 "l"((uint64_t)map), "r"(mbar), "r"(x), "r"(y)
                 : "memory");
}

struct ImLayout {
    int ring, mbar, xd, sxd, red, segkey, meta, total;
};
// The ring and its barriers come first, at offsets that depend on `stages` only, so a persistent kernel can
// keep them across multiplies of different shapes.
__host__ __device__ inline ImLayout im_layout(int cols, int k, bool q4, int slots, int seg_max, int stages) {
    ImLayout L;
    int off = 0;
    L.ring = off;
    off += IM_WARPS * stages * TILE_BYTES;
    L.mbar = off;
    off += IM_WARPS * stages * 8;
    off = (off + 127) & ~127;
    L.xd = off;
    off += cols * (k + im_xpad(q4));
    L.sxd = off;
    if (q4) off += cols * (k / 32 + 16);
    off = (off + 15) & ~15;
    L.red = off;
    off += IM_WARPS * seg_max * 16 * slots * 4;
    L.segkey = off;
    off += IM_WARPS * seg_max * 4;
    off = (off + 15) & ~15;
    L.meta = off;
    off += 64 * 8 + slots * 2 * 4;
    L.total = off;
    return L;
}

// Segments a warp may need: its range of ceil(nt / 16) tiles crosses a (row tile, part) boundary every
// `units` tiles.
__host__ __device__ inline int segments_needed(int n, int k, bool q4, bool pair, int grid) {
    const int units = q4 ? k / 256 : (k / 32 + Q8_UNIT - 1) / Q8_UNIT;
    const int row_tiles = (n + 15) / 16;
    const int per_cta = (row_tiles + grid - 1) / grid;
    const int nt = per_cta * (pair ? 2 : 1) * units;
    const int len = (nt + IM_WARPS - 1) / IM_WARPS;
    return len / units + 2;
}

// A warp's ring of tile stages and where its producer and consumer stand. Lives as long as the kernel.
struct ImRing {
    uint32_t base, mbar;   // shared-memory addresses of this warp's stages and their barriers
    int is_stage, cs_stage;
    uint32_t phase_bits;   // bit st: the parity to wait for on stage st
};

template <int STAGES>
__device__ __forceinline__ void im_ring_init(ImRing& rg, uint8_t* smem, const ImLayout& L, int warp, int lane) {
    rg.base = (uint32_t)__cvta_generic_to_shared(smem + L.ring) + (uint32_t)warp * STAGES * TILE_BYTES;
    rg.mbar = (uint32_t)__cvta_generic_to_shared(smem + L.mbar) + (uint32_t)warp * STAGES * 8;
    rg.is_stage = rg.cs_stage = 0;
    rg.phase_bits = 0;
    if (lane == 0) {
#pragma unroll
        for (int st = 0; st < STAGES; st++) mbar_init(rg.mbar + 8 * st, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
}

// The copy side of one multiply for one warp: which tile comes next and where its rows start.
struct ImIssue {
    const CUtensorMap* map;   // the weight matrix as 160-byte-wide boxes
    const CUtensorMap* smap;  // Q8_0: its scales as 16-byte-wide boxes
    int n, half, k, units, nparts, rt_lo;
    int is_rtl, is_part, is_unit, issued, lo, hi;
    int op;                // which operation of a program this iterator belongs to (-1: none)
};

// CTA `cta` of `ncta` owns the contiguous row tiles [cta*RT/ncta, (cta+1)*RT/ncta); its tiles, ordered (row
// tile, part, k), are cut into 16 contiguous ranges, one per warp.
template <int TYPE>
__device__ __forceinline__ void im_issue_setup(ImIssue& s, const PMatvec& p, const CUtensorMap* map, const CUtensorMap* smap, int cta,
                                               int ncta, int warp) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    const int k = (int)p.k, n = (int)p.n;
    s.map = map;
    s.smap = smap;
    s.k = k;
    s.n = n;
    s.half = (int)p.half;
    s.nparts = (p.flags & MV_SILU_PAIR) ? 2 : 1;
    s.units = Q4 ? k / 256 : (k / 32 + Q8_UNIT - 1) / Q8_UNIT;
    const int row_tiles = (n + 15) / 16;
    s.rt_lo = (int)((unsigned)cta * (unsigned)row_tiles / (unsigned)ncta);   // cta * row_tiles < 2^31
    const int rt_hi = (int)((unsigned)(cta + 1) * (unsigned)row_tiles / (unsigned)ncta);
    const int per_rt = s.nparts * s.units;
    const int nt = (rt_hi - s.rt_lo) * per_rt;
    s.lo = (int)(((unsigned)warp * (unsigned)nt) / IM_WARPS);
    s.hi = (int)(((unsigned)(warp + 1) * (unsigned)nt) / IM_WARPS);
    s.is_rtl = s.lo / per_rt;
    s.is_part = (s.lo % per_rt) / s.units;
    s.is_unit = s.lo % s.units;
    s.issued = s.lo;
}

// Copies tile `issued` into the ring's next stage (one lane asks the TMA unit for the whole box), then steps the
// iterator. Does nothing once the warp's range is exhausted.
template <int TYPE, int STAGES>
__device__ __forceinline__ void im_issue(ImRing& rg, ImIssue& s, int lane) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    if (s.issued >= s.hi) return;
    const uint32_t mb = rg.mbar + 8 * rg.is_stage;
    // the stage was read with ordinary loads; the copy writes it through the async proxy
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    __syncwarp();
    if (lane == 0) {
        const uint32_t dst = rg.base + (uint32_t)rg.is_stage * TILE_BYTES;
        const int y = (s.is_part ? s.half : 0) + (s.rt_lo + s.is_rtl) * 16;
        if constexpr (Q4) {
            mbar_expect_tx(mb, 16u * TILE_ROW);
            tma_tile(dst, s.map, s.is_unit * 144, y, mb);
        } else {
            // four blocks of values, and the 16 bytes that hold the scales of blocks (b0 & ~7) .. +7 (k is a
            // multiple of 256 here, so both boxes start on 16-byte boundaries)
            const int b0 = s.is_unit * Q8_UNIT;
            mbar_expect_tx(mb, 16u * TILE_ROW + 256u);
            tma_tile(dst, s.map, b0 * 32, y, mb);
            tma_tile(dst + TILE_SCALES, s.smap, s.k + 2 * (b0 & ~7), y, mb);
        }
    }
    s.issued++;
    rg.is_stage = rg.is_stage + 1 == STAGES ? 0 : rg.is_stage + 1;
    s.is_unit++;
    if (s.is_unit == s.units) {
        s.is_unit = 0;
        s.is_part++;
        if (s.is_part == s.nparts) {
            s.is_part = 0;
            s.is_rtl++;
        }
    }
}

// Starts a multiply's copies: the first STAGES - 1 tiles of this warp's range. Weights do not depend on
// the activations, so this may run long before the multiply itself.
template <int TYPE, int STAGES>
__device__ __forceinline__ void im_prime(ImRing& rg, ImIssue& s, const PMatvec& p, const CUtensorMap* map, const CUtensorMap* smap,
                                         int cta, int ncta, int warp, int lane, int op) {
    im_issue_setup<TYPE>(s, p, map, smap, cta, ncta, warp);
    s.op = op;
#pragma unroll
    for (int i = 0; i < STAGES - 1; i++) im_issue<TYPE, STAGES>(rg, s, lane);
}

// One multiply on CTA `cta` of `ncta`. NB column blocks of 8 = 2 tokens each; STAGES tiles in flight per warp.
// `iss` must have been primed for this multiply (im_prime). `between()` runs after this warp's last tile and
// before the CTA-wide reduction: a persistent kernel primes its next multiply there. `wait_inputs()` runs
// before the activations are read.
//
// When a warp's range crosses into another (row tile, part) it parks its sums in a shared-memory segment;
// after one barrier the segments of each row are added in (warp, segment) order.
template <int TYPE, int NB, int STAGES, class WaitInputs, class Between>
__device__ __forceinline__ void im_multiply(uint8_t* smem, ImRing& rg, ImIssue& iss, int cta, int ncta, const PMatvec& p,
                                            const float* __restrict__ x, float* __restrict__ out,
                                            const float* __restrict__ norm_w, int t0, int mt, int seg_max,
                                            int* __restrict__ status, const MvRope* __restrict__ rope, const PeerUse* __restrict__ pu, WaitInputs wait_inputs,
                                            Between between) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    constexpr int SLOTS = 2 * NB;  // token slots of a pass
    const int tid = threadIdx.x, lane = tid & 31, warp = __shfl_sync(0xffffffffu, tid >> 5, 0);   // warp-uniform to the compiler
    const int g = lane >> 2, t = lane & 3;
    const int k = (int)p.k, n = (int)p.n;
    const int xr = p.x_stride ? (int)p.x_stride * 4 : k;
    const bool norm = (p.flags & MV_NORM) != 0, pair = (p.flags & MV_SILU_PAIR) != 0;
    const int cols = 4 * mt;
    const ImLayout L = im_layout(cols, k, Q4, SLOTS, seg_max, STAGES);
    int8_t* xd = reinterpret_cast<int8_t*>(smem + L.xd);
    int8_t* sxd = reinterpret_cast<int8_t*>(smem + L.sxd);
    float* red = reinterpret_cast<float*>(smem + L.red);
    int* segkey = reinterpret_cast<int*>(smem + L.segkey);
    double* dred = reinterpret_cast<double*>(smem + L.meta);
    float* tokmeta = reinterpret_cast<float*>(smem + L.meta + 64 * 8);  // [slot][0: norm scale, 1: fixed-point scale]
    const int xcol = k + im_xpad(Q4), sxcol = k / 32 + 16;
    const int nparts = pair ? 2 : 1;
    const int units = Q4 ? k / 256 : (k / 32 + Q8_UNIT - 1) / Q8_UNIT;  // tiles along k
    const int nblk = k / 32;
    const int row_tiles = (n + 15) / 16;
    const int rt_lo = (int)((unsigned)cta * (unsigned)row_tiles / (unsigned)ncta);
    const int rt_hi = (int)((unsigned)(cta + 1) * (unsigned)row_tiles / (unsigned)ncta);
    const int per_rt = nparts * units;
    const int lo = iss.lo, hi = iss.hi;

    for (int i = tid; i < IM_WARPS * seg_max; i += IM_THREADS) segkey[i] = -1;
    // the norm weights are constants read once per step: ask for them now, while the kernel before this one
    // is still running, so the staging below finds them on chip
    if (norm)
        for (int off = tid * 128; off < k * 4; off += IM_THREADS * 128)
            asm volatile("prefetch.global.L1 [%0];\n" ::"l"(reinterpret_cast<const char*>(norm_w) + off));
    wait_inputs();
    // the value this thread's first output accumulates onto: asked for now, needed after the tile stream
    float first_old = 0.f;
    if ((p.flags & MV_ACCUMULATE) && tid < (rt_hi - rt_lo) * 16 * mt) {
        const int j0 = (rt_lo + tid / (mt * 16)) * 16 + (tid / mt) % 16;
        if (j0 < n) first_old = __ldcg(out + (size_t)(t0 + tid % mt) * p.out_stride + p.col0 + j0);
    }

    // the activations: local memory, or the slots of a tensor-parallel exchange (each read waits for its tag)
    const bool x_exchanged = pu != nullptr && pu->wait_slot != PEER_NONE;
    const uint32_t x_tag = x_exchanged ? peer::want_tag(*pu) : 0u;
    auto ldx = [&](const float* row, int i) {
        return x_exchanged ? peer::read4(*pu, row + 4 * i, x_tag, status) : __ldcg(reinterpret_cast<const float4*>(row) + i);
    };
    // ---- activations -> fixed point. Per token: sum of squares (RMSNorm) and largest magnitude over
    //      the CTA, a power-of-two scale s with |x * s| <= 2^25, then four balanced signed byte digits of
    //      X = rint(x * s):  X = D0 + 2^8 D1 + 2^16 D2 + 2^24 D3, each D in [-128, 127].
    {
        const int vecs = k / 4;
        constexpr int KEEP = 8;  // float4 of a token a thread keeps between the two passes
        const float lim = (float)(1 << IM_FIX_BITS);
        for (int tk = 0; tk < mt; tk++) {
            const float* xt = x + (size_t)(t0 + tk) * xr;
            float4 keep[KEEP];
            double ss = 0.0;
            float amax = 0.f;
            auto stat = [&](const float4& a, int i) {
                if (norm) {
                    ss += (double)__fmul_rn(a.x, a.x);
                    ss += (double)__fmul_rn(a.y, a.y);
                    ss += (double)__fmul_rn(a.z, a.z);
                    ss += (double)__fmul_rn(a.w, a.w);
                    const float4 nw = reinterpret_cast<const float4*>(norm_w)[i];
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x * nw.x), fabsf(a.y * nw.y)), fmaxf(fabsf(a.z * nw.z), fabsf(a.w * nw.w))));
                } else {
                    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
                }
            };
#pragma unroll
            for (int c = 0; c < KEEP; c++) {
                const int i = tid + c * IM_THREADS;
                keep[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (i < vecs) {
                    keep[c] = ldx(xt, i);
                    stat(keep[c], i);
                }
            }
            for (int i = tid + KEEP * IM_THREADS; i < vecs; i += IM_THREADS) stat(ldx(xt, i), i);
            if (norm) ss = warp_sum_d(ss);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0) {
                dred[warp] = ss;
                dred[32 + warp] = (double)amax;
            }
            __syncthreads();
            // every thread finishes the reduction itself (fixed order), so no second barrier is needed
            // (a pairwise tree: four dependent f64 additions instead of sixteen)
            double part[IM_WARPS];
            float am = 0.f;
#pragma unroll
            for (int wv = 0; wv < IM_WARPS; wv++) {
                part[wv] = dred[wv];
                am = fmaxf(am, (float)dred[32 + wv]);
            }
#pragma unroll
            for (int span = 1; span < IM_WARPS; span *= 2)
#pragma unroll
                for (int wv = 0; wv < IM_WARPS; wv += 2 * span) part[wv] += part[wv + span];
            const double tot = part[0];
            float nscale = 1.0f;
            if (norm) {
                // (a power-of-two k divides exactly either way; the multiply skips the slow f64 division)
                const float mean = (k & (k - 1)) == 0 ? (float)(tot * (1.0 / (double)k)) : (float)(tot / (double)k);
                nscale = 1.0f / sqrtf(mean + p.eps);
            }
            am = am * nscale * 1.0001f;  // the staged products round separately
            float s = 1.0f;
            if (am > 0.f && am < 3.0e38f) {
                // am = f * 2^e with f in [1, 2): s = 2^(24 - e), so am * s < 2^25
                const int e = (int)((__float_as_uint(am) >> 23) & 0xffu) - 127;
                s = __uint_as_float((uint32_t)(max(-100, min(100, IM_FIX_BITS - 1 - e)) + 127) << 23);
            }
            if (tid == 0) tokmeta[2 * tk + 1] = s;
            auto stage = [&](float4 a, int i) {
                if (norm) {
                    const float4 nw = reinterpret_cast<const float4*>(norm_w)[i];
                    a.x = __fmul_rn(__fmul_rn(a.x, nscale), nw.x);
                    a.y = __fmul_rn(__fmul_rn(a.y, nscale), nw.y);
                    a.z = __fmul_rn(__fmul_rn(a.z, nscale), nw.z);
                    a.w = __fmul_rn(__fmul_rn(a.w, nscale), nw.w);
                }
                int X[4];
                X[0] = __float2int_rn(fminf(fmaxf(a.x * s, -lim), lim));
                X[1] = __float2int_rn(fminf(fmaxf(a.y * s, -lim), lim));
                X[2] = __float2int_rn(fminf(fmaxf(a.z * s, -lim), lim));
                X[3] = __float2int_rn(fminf(fmaxf(a.w * s, -lim), lim));
                uint32_t dg[4];
                int sum = X[0] + X[1] + X[2] + X[3];
#pragma unroll
                for (int dgt = 0; dgt < 4; dgt++) {
                    // byte 0 of each X is its digit; then carry: X <- (X + 128) >> 8
                    dg[dgt] = __byte_perm(__byte_perm((uint32_t)X[0], (uint32_t)X[1], 0x0040),
                                          __byte_perm((uint32_t)X[2], (uint32_t)X[3], 0x0040), 0x5410);
#pragma unroll
                    for (int q = 0; q < 4; q++) X[q] = (X[q] + 128) >> 8;
                }
                const int pos = stage_pos<TYPE>(4 * i);
#pragma unroll
                for (int dgt = 0; dgt < 4; dgt++)
                    *reinterpret_cast<uint32_t*>(xd + (size_t)(4 * tk + dgt) * xcol + pos) = dg[dgt];
                if (Q4) {
                    // exact sum over the 32 elements of a sub-block: 8 consecutive threads (k / 4 is a multiple
                    // of 64, so a warp is in or out of the loop as a whole)
                    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
                    if ((i & 7) == 0) {
                        int v0 = sum;
#pragma unroll
                        for (int dgt = 0; dgt < 4; dgt++) {
                            sxd[(size_t)(4 * tk + dgt) * sxcol + (i >> 3)] = (int8_t)(v0 & 0xff);
                            v0 = (v0 + 128) >> 8;
                        }
                    }
                }
            };
#pragma unroll
            for (int c = 0; c < KEEP; c++) {
                const int i = tid + c * IM_THREADS;
                if (i < vecs) stage(keep[c], i);
            }
            for (int i = tid + KEEP * IM_THREADS; i < vecs; i += IM_THREADS) stage(ldx(xt, i), i);
            __syncthreads();  // dred is reused by the next token; xd is read after the last one
        }
    }

    // ---- the tile stream
    float accf[NB][4];
#pragma unroll
    for (int b = 0; b < NB; b++) accf[b][0] = accf[b][1] = accf[b][2] = accf[b][3] = 0.f;
    // digits -> value: cols 2t, 2t+1 are digits 2(t&1), 2(t&1)+1 of token slot 2b + (t>>1)
    const float w0 = (t & 1) ? 65536.0f : 1.0f, w1 = w0 * 256.0f;
    int seg = 0;
    int cur_rtl = lo / per_rt, cur_part = (lo % per_rt) / units, cur_unit = lo % units;

    auto park = [&]() {
        // parks this warp's sums for (cur_rtl, cur_part) in segment `seg`
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v0 = __fmaf_rn(accf[b][1], w1, accf[b][0] * w0);
            float v1 = __fmaf_rn(accf[b][3], w1, accf[b][2] * w0);
            v0 = __fadd_rn(v0, __shfl_xor_sync(0xffffffffu, v0, 1));  // low digits + high digits
            v1 = __fadd_rn(v1, __shfl_xor_sync(0xffffffffu, v1, 1));
            const int slot = 2 * b + (t >> 1);
            if ((t & 1) == 0 && seg < seg_max) {
                const float inv_s = slot < mt ? 1.0f / tokmeta[2 * slot + 1] : 0.f;
                float* rr = red + ((size_t)(warp * seg_max + seg) * 16) * SLOTS;
                rr[g * SLOTS + slot] = v0 * inv_s;
                rr[(g + 8) * SLOTS + slot] = v1 * inv_s;
            }
            accf[b][0] = accf[b][1] = accf[b][2] = accf[b][3] = 0.f;
        }
        if (lane == 0 && seg < seg_max) segkey[warp * seg_max + seg] = cur_rtl * 2 + cur_part;
        seg++;
    };

    // lane-constant offsets into a tile: header of row g; bytes 16 + 8 t (Q4_K) or 8 t (Q8_0) of row g
    const uint32_t hoff = (uint32_t)g * TILE_ROW;
    const uint32_t qoff = hoff + (Q4 ? 16u : 0u) + 8u * (uint32_t)t;
    bool timed_out = false;
    for (int tau = lo; tau < hi; tau++) {
        im_issue<TYPE, STAGES>(rg, iss, lane);  // tile tau + STAGES - 1
        if (!mbar_wait(rg.mbar + 8 * rg.cs_stage, (rg.phase_bits >> rg.cs_stage) & 1u)) timed_out = true;
        rg.phase_bits ^= 1u << rg.cs_stage;
        const uint32_t tile = rg.base + (uint32_t)rg.cs_stage * TILE_BYTES;
        rg.cs_stage = rg.cs_stage + 1 == STAGES ? 0 : rg.cs_stage + 1;
        const int unit = cur_unit;
        if constexpr (Q4) {
            const uint4 h0 = lds128(tile + hoff), h1 = lds128(tile + hoff + 8 * TILE_ROW);
            const uint32_t sc0[2] = {h0.y & 0x3f3f3f3fu, (h0.w & 0x0f0f0f0fu) | ((h0.y >> 2) & 0x30303030u)};
            const uint32_t sc1[2] = {h1.y & 0x3f3f3f3fu, (h1.w & 0x0f0f0f0fu) | ((h1.y >> 2) & 0x30303030u)};
            const uint32_t mn0[2] = {h0.z & 0x3f3f3f3fu, ((h0.w >> 4) & 0x0f0f0f0fu) | ((h0.z >> 2) & 0x30303030u)};
            const uint32_t mn1[2] = {h1.z & 0x3f3f3f3fu, ((h1.w >> 4) & 0x0f0f0f0fu) | ((h1.z >> 2) & 0x30303030u)};
            int run[NB][4];
#pragma unroll
            for (int b = 0; b < NB; b++) run[b][0] = run[b][1] = run[b][2] = run[b][3] = 0;
            const int8_t* xb = xd + unit * 256 + 16 * t;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const uint2 q0 = lds64(tile + qoff + 32 * j), q1 = lds64(tile + qoff + 8 * TILE_ROW + 32 * j);
                uint4 bv[NB];
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const int col = 8 * b + g;
                    bv[b] = make_uint4(0, 0, 0, 0);
                    if (col < cols) bv[b] = *reinterpret_cast<const uint4*>(xb + (size_t)col * xcol + 64 * j);
                }
#pragma unroll
                for (int hi_n = 0; hi_n < 2; hi_n++) {
                    const int s = 2 * j + hi_n;
                    const int sh = hi_n ? 4 : 0;
                    const uint32_t a0 = (q0.x >> sh) & 0x0f0f0f0fu, a1 = (q1.x >> sh) & 0x0f0f0f0fu;
                    const uint32_t a2 = (q0.y >> sh) & 0x0f0f0f0fu, a3 = (q1.y >> sh) & 0x0f0f0f0fu;
                    const int s0 = (int)__byte_perm(sc0[s >> 2], 0u, 0x4440 | (s & 3));
                    const int s1 = (int)__byte_perm(sc1[s >> 2], 0u, 0x4440 | (s & 3));
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        int acc[4];
                        imma_16832(acc, a0, a1, a2, a3, hi_n ? bv[b].z : bv[b].x, hi_n ? bv[b].w : bv[b].y);
                        run[b][0] += acc[0] * s0;
                        run[b][1] += acc[1] * s0;
                        run[b][2] += acc[2] * s1;
                        run[b][3] += acc[3] * s1;
                    }
                }
            }
            // mins: lanes t = 0, 1 carry the eight 6-bit mins of rows g and g+8 (four per register)
            const uint32_t ma0 = t == 0 ? mn0[0] : (t == 1 ? mn0[1] : 0u);
            const uint32_t ma1 = t == 0 ? mn1[0] : (t == 1 ? mn1[1] : 0u);
            const float d0 = __half2float(__ushort_as_half((unsigned short)(h0.x & 0xffffu)));
            const float d1 = __half2float(__ushort_as_half((unsigned short)(h1.x & 0xffffu)));
            const float dm0 = -__half2float(__ushort_as_half((unsigned short)(h0.x >> 16)));
            const float dm1 = -__half2float(__ushort_as_half((unsigned short)(h1.x >> 16)));
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int col = 8 * b + g;
                uint32_t bs = 0;
                if (col < cols && t < 2) bs = *reinterpret_cast<const uint32_t*>(sxd + (size_t)col * sxcol + unit * 8 + 4 * t);
                int am[4];
                imma_16832(am, ma0, ma1, 0u, 0u, bs, 0u);
                float* af = accf[b];
                af[0] = __fmaf_rn((float)run[b][0], d0, af[0]);
                af[1] = __fmaf_rn((float)run[b][1], d0, af[1]);
                af[2] = __fmaf_rn((float)run[b][2], d1, af[2]);
                af[3] = __fmaf_rn((float)run[b][3], d1, af[3]);
                af[0] = __fmaf_rn((float)am[0], dm0, af[0]);
                af[1] = __fmaf_rn((float)am[1], dm0, af[1]);
                af[2] = __fmaf_rn((float)am[2], dm1, af[2]);
                af[3] = __fmaf_rn((float)am[3], dm1, af[3]);
            }
        } else {
            const int b0 = unit * Q8_UNIT;
            // the 16 bytes copied hold the scales of blocks (b0 & ~7) .. +7: this tile's four are its low or high half
            const uint2 sc0 = lds64(tile + TILE_SCALES + 16 * g + 8 * (unit & 1)), sc1 = lds64(tile + TILE_SCALES + 16 * (g + 8) + 8 * (unit & 1));
            const uint32_t scw0[2] = {sc0.x, sc0.y}, scw1[2] = {sc1.x, sc1.y};
#pragma unroll
            for (int i = 0; i < Q8_UNIT; i++) {
                const int blk = b0 + i;
                if (blk < nblk) {
                    const uint2 q0 = lds64(tile + qoff + 32 * i), q1 = lds64(tile + qoff + 8 * TILE_ROW + 32 * i);
                    const float d0 = __half2float(__ushort_as_half((unsigned short)((scw0[i >> 1] >> (16 * (i & 1))) & 0xffffu)));
                    const float d1 = __half2float(__ushort_as_half((unsigned short)((scw1[i >> 1] >> (16 * (i & 1))) & 0xffffu)));
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const int col = 8 * b + g;
                        uint2 bv = make_uint2(0, 0);
                        if (col < cols) bv = *reinterpret_cast<const uint2*>(xd + (size_t)col * xcol + blk * 32 + 8 * t);
                        int acc[4];
                        imma_16832(acc, q0.x, q1.x, q0.y, q1.y, bv.x, bv.y);
                        float* af = accf[b];
                        af[0] = __fmaf_rn((float)acc[0], d0, af[0]);
                        af[1] = __fmaf_rn((float)acc[1], d0, af[1]);
                        af[2] = __fmaf_rn((float)acc[2], d1, af[2]);
                        af[3] = __fmaf_rn((float)acc[3], d1, af[3]);
                    }
                }
            }
        }
        __syncwarp();  // every lane is done with this stage before a later copy overwrites it
        // step to the next tile; on leaving this (row tile, part), park the sums
        int nx_rtl = cur_rtl, nx_part = cur_part, nx_unit = cur_unit + 1;
        if (nx_unit == units) {
            nx_unit = 0;
            nx_part++;
            if (nx_part == nparts) {
                nx_part = 0;
                nx_rtl++;
            }
        }
        if (tau + 1 == hi || nx_rtl != cur_rtl || nx_part != cur_part) park();
        cur_rtl = nx_rtl;
        cur_part = nx_part;
        cur_unit = nx_unit;
    }
    if (timed_out && lane == 0 && status) atomicExch(status, 1);
    between();
    __syncthreads();

    // ---- add each row's segments in (warp, segment) order and write it. With MV_ROPE_APPEND the row is
    //      Q|K|V: adjacent outputs (2i, 2i+1) of a q or k head are a RoPE pair held by lanes `mt` apart; q is
    //      written rotated, k and v go to the cache at the token's position (rope_append's arithmetic,
    //      src/kernels/rope_append.wgsl; every product rounded, src/ref/ops.zig:64-86).
    const int local_rts = rt_hi - rt_lo;
    const bool fused_rope = rope != nullptr && (p.flags & MV_ROPE_APPEND);
    const bool pushing = pu != nullptr && pu->push_slot != PEER_NONE;
    const uint32_t out_tag = pushing ? peer::push_tag(*pu) : 0u;
    const int total = local_rts * 16 * mt;
    for (int i0 = 0; i0 < total; i0 += IM_THREADS) {
        const int i = i0 + tid;
        const int tk = i % mt, row = (i / mt) % 16, rtl = i / (mt * 16);
        const int j = (rt_lo + rtl) * 16 + row;
        const bool valid = i < total && j < n;
        float v = 0.f, u = 0.f;
        if (valid) {
            // every segment is loaded (eight at a time, no dependent branches) and added only where its key
            // matches, in (warp, segment) order
            const float* rbase = red + (size_t)row * SLOTS + tk;
#pragma unroll 8
            for (int sgi = 0; sgi < IM_WARPS * seg_max; sgi++) {
                const int key = segkey[sgi];
                const float r = rbase[(size_t)sgi * 16 * SLOTS];
                v = __fadd_rn(v, key == rtl * 2 ? r : 0.f);
                u = __fadd_rn(u, key == rtl * 2 + 1 ? r : 0.f);
            }
        }
        if (pair) v = silu_f(v) * u;
        const size_t o = (size_t)(t0 + tk) * p.out_stride + p.col0 + j;
        if (fused_rope) {
            const float other = __shfl_xor_sync(0xffffffffu, v, mt);  // the pair's other element (whole warps run this loop)
            if (!valid) continue;
            const PRopeAppend& r = rope->p;
            const int tok = t0 + tk;
            const uint32_t pos = rope->seq_pos ? rope->seq_pos[tok] : rope->step->pos0 + (uint32_t)tok;
            const uint32_t col = p.col0 + (uint32_t)j, hd = r.head_dim, q_head = r.gated ? 2 * hd : hd;
            const bool is_q = col < r.k_off, is_k = !is_q && col < r.v_off;
            const uint32_t d = is_q ? col % q_head : (col - (is_k ? r.k_off : r.v_off)) % hd;
            float val = v;
            if ((is_q || is_k) && d < r.n_rot) {
                const float2 cs = rope->table[(size_t)pos * (r.n_rot / 2) + d / 2];
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
        if (!valid) continue;
        if (p.flags & MV_ACCUMULATE) v += i == tid ? first_old : __ldcg(out + o);
        out[o] = v;
        if (pushing) peer::push(*pu, out + o, v, out_tag);  // this rank's slice, to every rank's exchange slots
    }
    if (pu != nullptr) peer::finish(*pu, (unsigned)ncta);
}

}  // namespace imma
