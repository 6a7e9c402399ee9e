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

#include "k_matvec_common.cuh"

namespace {

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

struct ImLayout {
    int xd, sxd, red, segkey, meta, ring, mbar, total;
};
__host__ __device__ inline ImLayout im_layout(int cols, int k, bool q4, int slots, int seg_max, int stages) {
    ImLayout L;
    int off = 0;
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
    off = (off + 127) & ~127;
    L.ring = off;
    off += IM_WARPS * stages * 16 * 160;
    L.mbar = off;
    off += IM_WARPS * stages * 8;
    L.total = off;
    return L;
}

// One warp's tile of weights: 16 rows x one super-block (Q4_K, 144 bytes a row) or x four blocks
// (Q8_0: 128 value bytes a row, then its 4 f16 scales). Each row of a tile is one bulk copy
// (cp.async.bulk, global -> shared, completing on an mbarrier) into a ring of stages per warp, several
// tiles ahead of the one being multiplied. Rows sit 160 bytes apart in shared memory, so the 8-byte
// fragment loads of a half-warp (four rows) cover 128 distinct bytes.
constexpr int Q8_UNIT = 4;        // blocks per Q8_0 tile
constexpr int TILE_ROW = 160;
constexpr int TILE_BYTES = 16 * TILE_ROW;

// NB column blocks of 8 = 2 tokens each. STAGES tiles in flight per warp.
//
// Work split: CTA c owns the contiguous row tiles [c*RT/G, (c+1)*RT/G). Its tiles, ordered (row tile,
// part, k), are cut into 16 contiguous ranges, one per warp, so a warp streams consecutive super-blocks
// of the same 16 rows. When a warp's range crosses into another (row tile, part) it parks its sums in a
// shared-memory segment; after one barrier the segments of each row are added in (warp, segment) order.
template <int TYPE, int NB, int STAGES>
__global__ void __launch_bounds__(IM_THREADS, 1) matvec_imma(PMatvec p, const float* __restrict__ x,
                                                            const uint8_t* __restrict__ w, float* __restrict__ out,
                                                            const float* __restrict__ norm_w, int t0, int mt,
                                                            int seg_max, int* __restrict__ status) {
    constexpr bool Q4 = TYPE == W_Q4_K;
    constexpr int SLOTS = 2 * NB;  // token slots of a pass
    extern __shared__ __align__(16) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
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
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem + L.ring) + (uint32_t)warp * STAGES * TILE_BYTES;
    const uint32_t mbar0 = (uint32_t)__cvta_generic_to_shared(smem + L.mbar) + (uint32_t)warp * STAGES * 8;
    const int xcol = k + im_xpad(Q4), sxcol = k / 32 + 16;
    const size_t rb = Q4 ? (size_t)(k / 256) * 144 : (((size_t)k + k / 16 + 15) & ~(size_t)15);
    const int nparts = pair ? 2 : 1;
    const int units = Q4 ? k / 256 : (k / 32 + Q8_UNIT - 1) / Q8_UNIT;  // tiles along k
    const int nblk = k / 32;

    // ---- this CTA's row tiles and this warp's tile range
    const int row_tiles = (n + 15) / 16;
    const int rt_lo = (int)(((long long)blockIdx.x * row_tiles) / gridDim.x);
    const int rt_hi = (int)(((long long)(blockIdx.x + 1) * row_tiles) / gridDim.x);
    const int per_rt = nparts * units;
    const int nt = (rt_hi - rt_lo) * per_rt;
    const int lo = (int)(((long long)warp * nt) / IM_WARPS), hi = (int)(((long long)(warp + 1) * nt) / IM_WARPS);

    // ---- the copy side: lane l < 16 copies row l of a tile with one bulk copy
    if (lane == 0) {
#pragma unroll
        for (int st = 0; st < STAGES; st++) mbar_init(mbar0 + 8 * st, 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncwarp();
    int is_rtl = lo / per_rt, is_part = (lo % per_rt) / units, is_unit = lo % units;  // next tile to issue
    const uint8_t* is_row = w;
    auto set_issue_row = [&]() {
        const int j = (is_part ? (int)p.half : 0) + (rt_lo + is_rtl) * 16 + (lane & 15);
        const int lim = (is_part ? (int)p.half : 0) + n - 1;
        is_row = w + (size_t)min(j, lim) * rb;
    };
    set_issue_row();
    int issued = lo, is_stage = 0;
    constexpr uint32_t ROW_COPY = Q4 ? 144u : 128u;
    auto issue = [&]() {
        // copies tile `issued` into stage `is_stage`, then steps the issue iterator
        if (issued < hi) {
            const uint32_t mb = mbar0 + 8 * is_stage;
            // the stage was read with ordinary loads; the bulk copy writes it through the async proxy
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            if (lane == 0) mbar_expect_tx(mb, Q4 ? 16u * 144u : 16u * (128u + 16u));
            __syncwarp();
            if (lane < 16) {
                const uint32_t dst = ring + (uint32_t)is_stage * TILE_BYTES + (uint32_t)lane * TILE_ROW;
                if constexpr (Q4) {
                    bulk_g2s(dst, is_row + (size_t)is_unit * 144, ROW_COPY, mb);
                } else {
                    // four blocks of values, and the 16 bytes that hold their four scales (k is a multiple of
                    // 256 here, so both copies are 16-byte aligned and never run past the row)
                    const int b0 = is_unit * Q8_UNIT;
                    bulk_g2s(dst, is_row + (size_t)b0 * 32, ROW_COPY, mb);
                    bulk_g2s(dst + 128, is_row + k + 2 * (b0 & ~7), 16u, mb);
                }
            }
            issued++;
            is_stage = is_stage + 1 == STAGES ? 0 : is_stage + 1;
            is_unit++;
            if (is_unit == units) {
                is_unit = 0;
                is_part++;
                if (is_part == nparts) {
                    is_part = 0;
                    is_rtl++;
                }
                if (issued < hi) set_issue_row();
            }
        }
    };
#pragma unroll
    for (int i = 0; i < STAGES - 1; i++) issue();  // weights do not depend on the activations: start them first
    for (int i = tid; i < IM_WARPS * seg_max; i += IM_THREADS) segkey[i] = -1;

    // Programmatic dependent launch: everything above touched only the weights, which no kernel writes.
    // From here on the activations are read, so the kernels before this one must have finished.
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");

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
                    keep[c] = reinterpret_cast<const float4*>(xt)[i];
                    stat(keep[c], i);
                }
            }
            for (int i = tid + KEEP * IM_THREADS; i < vecs; i += IM_THREADS) stat(reinterpret_cast<const float4*>(xt)[i], i);
            if (norm) ss = warp_sum_d(ss);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
            if (lane == 0) {
                dred[warp] = ss;
                dred[32 + warp] = (double)amax;
            }
            __syncthreads();
            // every thread finishes the reduction itself (fixed order), so no second barrier is needed
            double tot = 0.0;
            float am = 0.f;
#pragma unroll
            for (int wv = 0; wv < IM_WARPS; wv++) {
                tot += dred[wv];
                am = fmaxf(am, (float)dred[32 + wv]);
            }
            float nscale = 1.0f;
            if (norm) {
                const float mean = (float)(tot / (double)k);
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
            for (int i = tid + KEEP * IM_THREADS; i < vecs; i += IM_THREADS) stage(reinterpret_cast<const float4*>(xt)[i], i);
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
    int cs_stage = 0;
    uint32_t phase_bits = 0;  // bit st: the parity to wait for on stage st
    bool timed_out = false;
    for (int tau = lo; tau < hi; tau++) {
        issue();  // tile tau + STAGES - 1
        if (!mbar_wait(mbar0 + 8 * cs_stage, (phase_bits >> cs_stage) & 1u)) timed_out = true;
        phase_bits ^= 1u << cs_stage;
        const uint32_t tile = ring + (uint32_t)cs_stage * TILE_BYTES;
        cs_stage = cs_stage + 1 == STAGES ? 0 : cs_stage + 1;
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
            const uint2 sc0 = lds64(tile + hoff + 128 + 8 * (unit & 1)), sc1 = lds64(tile + hoff + 8 * TILE_ROW + 128 + 8 * (unit & 1));
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
    __syncthreads();

    // ---- add each row's segments in (warp, segment) order and write it
    const int local_rts = rt_hi - rt_lo;
    for (int i = tid; i < local_rts * 16 * mt; i += IM_THREADS) {
        const int tk = i % mt, row = (i / mt) % 16, rtl = i / (mt * 16);
        const int j = (rt_lo + rtl) * 16 + row;
        if (j >= n) continue;
        float v = 0.f, u = 0.f;
        for (int sgi = 0; sgi < IM_WARPS * seg_max; sgi++) {
            const int key = segkey[sgi];
            if (key == rtl * 2) v = __fadd_rn(v, red[((size_t)sgi * 16 + row) * SLOTS + tk]);
            else if (key == rtl * 2 + 1) u = __fadd_rn(u, red[((size_t)sgi * 16 + row) * SLOTS + tk]);
        }
        if (pair) v = silu_f(v) * u;
        const size_t o = (size_t)(t0 + tk) * p.out_stride + p.col0 + j;
        if (p.flags & MV_ACCUMULATE) v += out[o];
        out[o] = v;
    }
}

constexpr int IM_SMEM_MAX = 220 * 1024;

// Segments a warp may need: its range of ceil(nt / 16) tiles crosses a (row tile, part) boundary every
// `units` tiles.
int segments_needed(int n, int k, bool q4, bool pair, int grid) {
    const int units = q4 ? k / 256 : (k / 32 + Q8_UNIT - 1) / Q8_UNIT;
    const int row_tiles = (n + 15) / 16;
    const int per_cta = (row_tiles + grid - 1) / grid;
    const int nt = per_cta * (pair ? 2 : 1) * units;
    const int len = (nt + IM_WARPS - 1) / IM_WARPS;
    return len / units + 2;
}

template <int TYPE, int NB, int STAGES>
zcu_result launch_staged(const LaunchArgs& a, const MvArgs& v, int t0, int mt, int grid, int seg_max) {
    const ImLayout L = im_layout(4 * mt, (int)v.p.k, TYPE == W_Q4_K, 2 * NB, seg_max, STAGES);
    auto kern = matvec_imma<TYPE, NB, STAGES>;
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!configured[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, IM_SMEM_MAX);
        if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "matvec_imma: shared memory attribute: %s", cudaGetErrorString(e));
        configured[dev & 63] = true;
    }
    // Programmatic dependent launch: this kernel may start while the one before it drains; it prefetches
    // weights, then waits (griddepcontrol.wait) before it reads activations.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(IM_THREADS);
    cfg.dynamicSmemBytes = L.total;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, v.p, v.x, v.w, v.out, v.nw, t0, mt, seg_max, a.status);
    if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "matvec_imma: launch failed: %s", cudaGetErrorString(e));
    return ZCU_OK;
}

template <int TYPE, int NB>
zcu_result launch_one(const LaunchArgs& a, const MvArgs& v, int t0, int mt, int want_stages) {
    const bool q4 = TYPE == W_Q4_K, pair = (v.p.flags & MV_SILU_PAIR) != 0;
    const int row_tiles = ((int)v.p.n + 15) / 16;
    const int grid = row_tiles < a.sm_count ? row_tiles : a.sm_count;
    const int seg_max = segments_needed((int)v.p.n, (int)v.p.k, q4, pair, grid);
    // the deepest ring that fits beside the staged activations
    int stages = want_stages ? want_stages : 6;
    while (stages > 2 && im_layout(4 * mt, (int)v.p.k, q4, 2 * NB, seg_max, stages).total > IM_SMEM_MAX) stages--;
    if (im_layout(4 * mt, (int)v.p.k, q4, 2 * NB, seg_max, stages).total > IM_SMEM_MAX)
        return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: k = %u with %d tokens does not fit shared memory", v.p.k, mt);
    switch (stages) {
        case 2: return launch_staged<TYPE, NB, 2>(a, v, t0, mt, grid, seg_max);
        case 3: return launch_staged<TYPE, NB, 3>(a, v, t0, mt, grid, seg_max);
        case 4: return launch_staged<TYPE, NB, 4>(a, v, t0, mt, grid, seg_max);
        case 5: return launch_staged<TYPE, NB, 5>(a, v, t0, mt, grid, seg_max);
        default: return launch_staged<TYPE, NB, 6>(a, v, t0, mt, grid, seg_max);
    }
}

// Tokens one pass can stage: four byte columns of k (+ padding) per token beside a two-stage ring.
int tokens_per_pass(int k, bool q4) {
    int mt = 4;
    while (mt > 1 && im_layout(4 * mt, k, q4, 4, 8, 2).total > IM_SMEM_MAX) mt--;
    return mt;
}

template <int TYPE>
zcu_result launch_type(const LaunchArgs& a, const MvArgs& v, int stages) {
    const bool q4 = TYPE == W_Q4_K;
    const int cap = tokens_per_pass((int)v.p.k, q4);
    for (int t0 = 0; t0 < v.m;) {
        const int mt = (v.m - t0) < cap ? (v.m - t0) : cap;
        zcu_result r = mt > 2 ? launch_one<TYPE, 2>(a, v, t0, mt, stages) : launch_one<TYPE, 1>(a, v, t0, mt, stages);
        if (r != ZCU_OK) return r;
        t0 += mt;
    }
    return ZCU_OK;
}

}  // namespace

// `stages`: tiles in flight per warp (2..6; 0 = as deep as fits). Q8_0 needs k % 128 == 0.
zcu_result launch_matvec_imma(const LaunchArgs& a, const mv::MvArgs& v, int type, int stages, int unused) {
    (void)unused;
    if (type == mv::W_Q8_0 && v.p.k % 256 != 0) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec_q8_0: k = %u is not a multiple of 256", v.p.k);
    if (stages != 0 && (stages < 2 || stages > 6))
        return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec: %d stages is not built", stages);
    return type == mv::W_Q4_K ? launch_type<mv::W_Q4_K>(a, v, stages) : launch_type<mv::W_Q8_0>(a, v, stages);
}
