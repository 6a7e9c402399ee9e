// Q4_K multiplies on the 5th-generation tensor cores (tcgen05, accumulators in tensor memory), for steps with
// enough columns to share a weight tile: the prefill rung of matmul_q4_k (variant 0xfffc0000) and the batched
// form of matvec_q4_k (family 3: 1..64 tokens in ONE pass over the weights).
//
// The arithmetic stays the reference's integer one (src/kernels/matmul_quant.wgsl:1-16, quant/q4_k.wgsl:1-35):
//   out[c][j] = sum over 256-weight super-blocks b of
//               s[c][b] * ( d[j][b] * sum_i (sc_u(i) q_i) X[c][i]  -  dmin[j][b] * sum_u m_u S[c][u] )
// with q the 4-bit codes, sc_u / m_u the 6-bit scale and min of 32-weight unit u, X the column's values and
// S[c][u] the sum of X over unit u. What changes is where the products run: the CUDA cores only turn a weight
// tile into the f16 INTEGERS sc_u q_i (at most 63 * 15 = 945, exact in f16: one mask, one fused multiply-add per
// two weights) and hand them to the tensor cores as the A operand - in tensor memory (tcgen05.st; up to 64 columns)
// or in shared memory in the K-major 128-byte-swizzled layout (128 columns, whose accumulators fill tensor memory);
// tcgen05.mma (kind::f16, M 128 weight rows, N columns, K 16) accumulates them against the columns in f32. The
// min term is one more K = 16 instruction per super-block (each m_u twice, against S[c][u] as two f16 terms).
// Once per super-block the two sums leave tensor memory and meet the f16 super-scales and the column's scale in
// registers. A column is
//   prefill: a token's Q8_K block values (integers, exact in f16), s = the block's f32 scale (quantize_q8's dx);
//   decode:  one of the TWO f16 terms of a token's f32 activations (x 2^e per block = hi + lo, 22 bits), s = 2^-e;
//            the token's result is the sum of its two columns.
// Products are exact (10 x 11 bits), sums are f32 over at most 256 terms per drain: within 1e-6 of the integer
// arithmetic, against the 1e-5 bar of the reference's kernel checks.
//
// One CTA owns 128 weight rows x BN columns (16, 32, 64 or 128) x a slice of k. Roles (20 or 24 warps):
//   warp 0          TMA: the raw weight tiles (128 rows x 144 bytes per super-block), several super-blocks ahead
//   warp 1          TMA: the columns' tiles (BN x 64 values, 128-byte swizzle), the unit sums, the column scales
//   warp 2          allocates tensor memory; issues the MMAs and commits stages / accumulators
//   decoders        two (BN > 32) or four groups of four warps take alternate 64-weight chunks, thread = weight row
//   drain           eight (BN > 32) or four warps: thread (quadrant, lane) owns a weight row's accumulators
// Warps 0-2 run their loops as WHOLE warps with one elected lane issuing: addresses and descriptors then stay
// warp-uniform and feed the TMA / MMA instructions from uniform registers (issued from a single-lane branch the same
// loops took five times longer). Two accumulator sets alternate, so a super-block's products run while the one
// before it drains; up to 32 columns tensor memory also holds two or three whole decoded super-blocks, and decoders,
// issuing warp and drain meet once per super-block (17 MMAs) instead of once per 64 weights. Every wait suspends the
// thread (mbarrier.try_wait with a time hint) and is bounded in time; one that gives up raises the CTA's abort
// flag, every role leaves, tensor memory is freed and the context's status word reports it.

#include <cuda.h>
#include <cuda_fp16.h>

#include "k_matvec_common.cuh"
#include "tma_util.cuh"

namespace {

constexpr int QT_ROWS = 128, QT_CHUNK = 64;
// Warps: 4 for the copy / issue roles (one idle), 4 per decoder group, 4 or 8 for the drain. Narrow tiles (<= 32
// columns) drain little and are bound by the decoders: four groups there, two otherwise.
__host__ __device__ constexpr int decode_groups(int bn) { return bn <= 32 ? 4 : 2; }
__host__ __device__ constexpr int drain_warps(int bn) { return bn <= 32 ? 4 : 8; }
__host__ __device__ constexpr int qt_threads(int bn) { return 32 * (4 + 4 * decode_groups(bn) + drain_warps(bn)); }
constexpr int RAW_ROW = 144, RAW_BYTES = QT_ROWS * RAW_ROW;   // a super-block of 128 rows as stored
constexpr int A_BYTES = QT_ROWS * 128;                        // 128 rows x 64 f16
constexpr int HDR_SLOTS = 4, CSC_SLOTS = 8;   // super-blocks whose row scales / column scales are in flight

// Ring depths. The decoded tiles are made on the SM (short latency: few stages); the columns' tiles and the raw
// weights cross the chip (about a microsecond each): their rings must hold what the SM consumes in that time.
// Up to 64 columns the decoded tiles live in TENSOR memory (the accumulators leave room: 4 BN <= 256 of the 512
// columns), written there by tcgen05.st and read by the MMA as its A operand: the tile then crosses shared memory
// neither on its way in nor out (16 KB each way per 64 weights of 128 rows).
__host__ __device__ constexpr bool a_in_tmem(int bn) { return bn <= 64; }
constexpr int A_COL0 = 256, A_COLS = 32;   // tensor-memory columns of the A ring: 8 stages x 32 (64 f16 per row)
__host__ __device__ constexpr int a_stages(int bn) { return bn > 64 ? 3 : 8; }
__host__ __device__ constexpr int b_stages(int bn) { return bn > 64 ? 8 : bn > 32 ? 10 : bn > 16 ? 15 : 20; }
__host__ __device__ constexpr int raw_stages(int bn) { return bn > 64 ? 2 : 6; }
__host__ __device__ constexpr int qt_smem(int bn) {
    return 1024 + (a_in_tmem(bn) ? 0 : a_stages(bn) * A_BYTES) + b_stages(bn) * bn * 128 + raw_stages(bn) * RAW_BYTES + HDR_SLOTS * QT_ROWS * 8 +
           CSC_SLOTS * bn * 4 + 1024;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t mbar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(mbar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(mbar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(mbar) : "memory");
}
// Waits for phase `parity`. A waiting thread is SUSPENDED by the hardware (try_wait with a time hint) and resumes
// when the phase completes, so the many waiting warps of this kernel leave the issue slots to the working ones; a
// plain polling loop here took about half of them. The wait is bounded in time (about two seconds of SM clocks)
// and ends early when another role raised the abort flag. Returns false (flag raised) when it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity, volatile uint32_t* abort_flag) {
    {   // the phase is usually complete already: test_wait answers at once
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(mbar), "r"(parity), "r"(100000u)   // suspend for up to 100 microseconds at a time
            : "memory");
        if (ok) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > 4000000000ll) break;
    }
    *abort_flag = 1;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
                 "l"((uint64_t)map), "r"(mbar), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t mbar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst), "l"(src),
                 "r"(bytes), "r"(mbar)
                 : "memory");
}
// K-major rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// The same with A read from tensor memory (lane = row, one 32-bit column = two consecutive K values).
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "r"(a_tmem), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3, uint32_t r4, uint32_t r5, uint32_t r6,
                                         uint32_t r7) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};\n" ::"r"(taddr), "r"(r0), "r"(r1), "r"(r2), "r"(r3),
                 "r"(r4), "r"(r5), "r"(r6), "r"(r7)
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
// One lane of the (converged) warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n.reg .pred p;\nelect.sync _|p, 0xffffffff;\nselp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, uint32_t* r) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// Build with -DQT_TRACE to collect, for CTA (0, 0, 0), the clocks each role spends in its waits and in its work
// (a profiling aid for this file alone; nothing reads it otherwise).
#ifdef QT_TRACE
__device__ unsigned long long qt_trace[32];
#define QT_DECL() long long trace_acc__[20] = {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0}
#define QT_MARK(slot, tprev) do { const long long now__ = clock64(); trace_acc__[slot] += now__ - tprev; tprev = now__; } while (0)
#define QT_T0() const long long t0__ = clock64()
#define QT_ADD(slot, cond) trace_acc__[slot] += clock64() - t0__
#define QT_FLUSH(slot, cond)                                                                                      \
    do {                                                                                                          \
        if ((cond) && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) qt_trace[slot] += (unsigned long long)trace_acc__[slot]; \
    } while (0)
#else
#define QT_DECL()
#define QT_MARK(slot, tprev)
#define QT_T0()
#define QT_ADD(slot, cond)
#define QT_FLUSH(slot, cond)
#endif

struct QtArgs {
    int seg_rows, nseg, seg1_y, tiles_per_seg;   // weight-row segments (two for a SILU_PAIR matrix: gate rows, up rows)
    int cols, cols_pad;                          // columns, and the padded width of the scale table
    int nsb, sb_per_slice;                       // super-blocks of a row, and per k slice
    float* out;                                  // out[z * slice_stride + c * out_stride + col0 + seg * seg_out + row]
    size_t slice_stride;
    uint32_t out_stride, col0, seg_out, accumulate;
    const float* scales;                         // [nsb][cols_pad]
    int* status;
};

// Two f16 in one register from an int pair held in 16-bit lanes: 0x6400 | v is the f16 1024 + v.
__device__ __forceinline__ uint32_t scaled_pair(uint32_t bits, __half2 sc, __half2 off) {
    const uint32_t h = bits | 0x64006400u;
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&h), sc, off);
    return *reinterpret_cast<const uint32_t*>(&r);
}

template <int BN>
__global__ void __launch_bounds__(qt_threads(BN), 1)
    qgemm_q4k_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap bmap,
                     const __grid_constant__ CUtensorMap smap, QtArgs q) {
    constexpr int RS = raw_stages(BN), NA = a_stages(BN), NB = b_stages(BN), B_BYTES = BN * 128, TCOLS = 512;
    constexpr int NG = decode_groups(BN), ND = drain_warps(BN), CPT = BN / (ND / 4), DRAIN0 = 4 + 4 * NG;
    constexpr bool ATM = a_in_tmem(BN);
    static_assert(!ATM || (4 * BN <= A_COL0 && A_COL0 + NA * A_COLS <= TCOLS), "accumulators and the A ring share tensor memory");
    // The columns' tiles of a super-block share one barrier pair where the ring holds whole super-blocks (narrow
    // tiles): the issuing thread then waits and commits once per super-block instead of once per tile.
    constexpr int G = BN <= 64 ? 5 : 1;
    static_assert(NB % G == 0, "the column ring holds whole groups");
    // Up to 32 columns tensor memory has room for whole decoded super-blocks (4 x 32 columns and 8 for the mins),
    // two or three of them: the issuing warp then waits, issues (17 MMAs) and commits once per super-block, and
    // the decoders run a super-block ahead. (Wider tiles keep the 64-weight stages.)
    constexpr bool SBM = BN <= 32;
    constexpr int SB_COLS = 136, SB_COL0 = 4 * BN, SLOTS = (TCOLS - SB_COL0) / SB_COLS;
    static_assert(!SBM || (SLOTS >= 2 && SLOTS <= NA), "super-block slots and their barriers");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* a_ring = smem;
    unsigned char* b_ring = a_ring + (ATM ? 0 : NA * A_BYTES);
    unsigned char* raw_ring = b_ring + NB * B_BYTES;
    float2* hdr = reinterpret_cast<float2*>(raw_ring + RS * RAW_BYTES);          // [slot][row]: d, dmin
    float* csc = reinterpret_cast<float*>(hdr + HDR_SLOTS * QT_ROWS);            // [slot][BN]: the columns' scales
    uint64_t* bars = reinterpret_cast<uint64_t*>(csc + CSC_SLOTS * BN);
    const uint32_t full_a0 = smem_u32(bars), empty_a0 = full_a0 + 8 * NA, full_b0 = empty_a0 + 8 * NA, empty_b0 = full_b0 + 8 * NB,
                   raw_full0 = empty_b0 + 8 * NB, raw_empty0 = raw_full0 + 8 * RS, tfull0 = raw_empty0 + 8 * RS, tempty0 = tfull0 + 16;
    uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 2 * NA + 2 * NB + 2 * RS + 4);
    volatile uint32_t* abort_flag = holder + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NA; s++) {
            mbar_init(full_a0 + 8 * s, BN <= 32 ? 4 * NG : 4);
            mbar_init(empty_a0 + 8 * s, 1);
        }
        for (int s = 0; s < NB; s++) {
            mbar_init(full_b0 + 8 * s, 1);
            mbar_init(empty_b0 + 8 * s, 1);
        }
        for (int s = 0; s < RS; s++) {
            mbar_init(raw_full0 + 8 * s, 1);
            mbar_init(raw_empty0 + 8 * s, 4 * NG);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull0 + 8 * a, 1);
            mbar_init(tempty0 + 8 * a, 32 * ND);
        }
        holder[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(holder)), "r"(TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = holder[0];
    // a dependent kernel after this one (the reduction) may be scheduled once every CTA of this grid is running
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
#ifdef QT_TRACE
    const long long kernel_t0 = clock64();
#endif

    const int seg = (int)blockIdx.x / q.tiles_per_seg, tile = (int)blockIdx.x % q.tiles_per_seg;
    const int row0 = tile * QT_ROWS;                          // within the segment
    const int y0 = (seg ? q.seg1_y : 0) + row0;               // in the weight matrix
    const int c0 = (int)blockIdx.y * BN, z = (int)blockIdx.z;
    const int sb_lo = min(q.nsb, z * q.sb_per_slice), sb_hi = min(q.nsb, sb_lo + q.sb_per_slice);
    bool gave_up = false;
    QT_DECL();

    // (The two copy warps run their loops as whole warps too, one elected lane issuing: addresses stay warp-uniform.)
    if (warp == 0) {
        int rs = 0;
        uint32_t rphase = 0;
        for (int sb = sb_lo; sb < sb_hi; sb++) {
            bool ok;
            {
                QT_T0();
                ok = mbar_wait(raw_empty0 + 8 * rs, rphase ^ 1u, abort_flag);
                QT_ADD(0, true);
            }
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            if (elect_one()) {
                mbar_expect_tx(raw_full0 + 8 * rs, RAW_BYTES);
                tma_load_2d(smem_u32(raw_ring + rs * RAW_BYTES), &wmap, sb * RAW_ROW, y0, raw_full0 + 8 * rs);
            }
            __syncwarp();
            if (++rs == RS) rs = 0, rphase ^= 1u;
        }
        QT_FLUSH(0, lane == 0);
        if (gave_up)
            for (int i = 0; i < 200; i++) __nanosleep(1000);
    } else if (warp == 1) {
        // Launched as a programmatic dependent of the kernel that writes the columns: everything else in this CTA
        // (the weight copies, the decoders) may run while that kernel finishes; the columns are read after it.
        asm volatile("griddepcontrol.wait;\n" ::: "memory");
        int s = 0;
        uint32_t phase = 0;
        for (int sb = sb_lo; sb < sb_hi && !gave_up; sb++) {
            if constexpr (G == 5) {
                // the super-block's five tiles and its column scales complete one barrier
                bool ok;
                {
                    QT_T0();
                    ok = mbar_wait(empty_b0 + 8 * (s / G), phase ^ 1u, abort_flag);
                    QT_ADD(1, true);
                }
                if (!__all_sync(0xffffffffu, ok)) {
                    gave_up = true;
                    break;
                }
                if (elect_one()) {
                    const uint32_t fb = full_b0 + 8 * (s / G), dst = smem_u32(b_ring + s * B_BYTES);
                    mbar_expect_tx(fb, 5 * B_BYTES + BN * 4);
#pragma unroll
                    for (int c = 0; c < 4; c++) tma_load_2d(dst + c * B_BYTES, &bmap, (sb * 256 + c * QT_CHUNK) * 2, c0, fb);
                    tma_load_2d(dst + 4 * B_BYTES, &smap, sb * 128, c0, fb);
                    bulk_load(smem_u32(csc + ((sb - sb_lo) & (CSC_SLOTS - 1)) * BN), q.scales + (size_t)sb * q.cols_pad + c0, BN * 4, fb);
                }
                __syncwarp();
                s += 5;
                if (s == NB) s = 0, phase ^= 1u;
            } else {
                for (int c = 0; c < 5; c++) {
                    bool ok;
                    {
                        QT_T0();
                        ok = mbar_wait(empty_b0 + 8 * s, phase ^ 1u, abort_flag);
                        QT_ADD(1, true);
                    }
                    if (!__all_sync(0xffffffffu, ok)) {
                        gave_up = true;
                        break;
                    }
                    if (elect_one()) {
                        const uint32_t fb = full_b0 + 8 * s, dst = smem_u32(b_ring + s * B_BYTES);
                        if (c < 4) {
                            mbar_expect_tx(fb, B_BYTES);
                            tma_load_2d(dst, &bmap, (sb * 256 + c * QT_CHUNK) * 2, c0, fb);
                        } else {
                            // the unit sums of this super-block, and the columns' scales for it
                            mbar_expect_tx(fb, B_BYTES + BN * 4);
                            tma_load_2d(dst, &smap, sb * 128, c0, fb);
                            bulk_load(smem_u32(csc + ((sb - sb_lo) & (CSC_SLOTS - 1)) * BN), q.scales + (size_t)sb * q.cols_pad + c0, BN * 4, fb);
                        }
                    }
                    __syncwarp();
                    if (++s == NB) s = 0, phase ^= 1u;
                }
            }
        }
        QT_FLUSH(1, lane == 0);
        if (gave_up)
            for (int i = 0; i < 200; i++) __nanosleep(1000);
    } else if (warp == 2) {
        // The whole warp runs this loop, so that its addresses and descriptors stay warp-uniform (they feed the
        // instructions from uniform registers); one elected lane issues the MMAs and the commits.
        const uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(QT_ROWS >> 4) << 24);
        const uint64_t a_desc0 = umma_desc_sw128(smem_u32(a_ring)), b_desc0 = umma_desc_sw128(smem_u32(b_ring));
        int s = 0, t = 0, acc = 0;
        uint32_t phase = 0, bphase = 0, acc_phase = 0;
        for (int sb = sb_lo; sb < sb_hi && !gave_up; sb++) {
            bool ok;
            {
                QT_T0();
                ok = mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag);
                QT_ADD(2, true);
            }
            if (!__all_sync(0xffffffffu, ok)) {
                gave_up = true;
                break;
            }
            tc_fence_after();
            const uint32_t d1 = tmem_base + (uint32_t)acc * 2 * BN, d2 = d1 + BN;
            if constexpr (SBM) {
                const int sbi = sb - sb_lo, slot = sbi % SLOTS;
                const uint32_t sphase = (uint32_t)(sbi / SLOTS) & 1u;
                {
                    QT_T0();
                    ok = mbar_wait(full_a0 + 8 * slot, sphase, abort_flag);
                    QT_ADD(3, true);
                }
                {
                    QT_T0();
                    ok = ok && mbar_wait(full_b0 + 8 * (t / G), bphase, abort_flag);
                    QT_ADD(4, true);
                }
                if (!__all_sync(0xffffffffu, ok)) {
                    gave_up = true;
                    break;
                }
                QT_T0();
                tc_fence_after();
                const uint32_t ta = tmem_base + (uint32_t)(SB_COL0 + slot * SB_COLS);
                const uint64_t db = b_desc0 + (uint64_t)(t * (B_BYTES >> 4));
                if (elect_one()) {
#pragma unroll
                    for (int c = 0; c < 4; c++)
#pragma unroll
                        for (int kk = 0; kk < 4; kk++)
                            umma_f16_ts(d1, ta + (uint32_t)(32 * c + 8 * kk), db + (uint64_t)(c * (B_BYTES >> 4) + 2 * kk), idesc, (c | kk) != 0);
                    umma_f16_ts(d2, ta + 128u, db + (uint64_t)(4 * (B_BYTES >> 4)), idesc, 0u);
                    umma_commit(empty_a0 + 8 * slot);
                    umma_commit(empty_b0 + 8 * (t / G));
                    umma_commit(tfull0 + 8 * acc);
                }
                __syncwarp();
                QT_ADD(11, true);
                t += 5;
                if (t == NB) t = 0, bphase ^= 1u;
                if (++acc == 2) acc = 0, acc_phase ^= 1u;
                continue;
            }
            for (int c = 0; c < 5; c++) {
                {
                    QT_T0();
                    ok = mbar_wait(full_a0 + 8 * s, phase, abort_flag);
                    QT_ADD(3, true);
                }
                if (t % G == 0) {
                    QT_T0();
                    ok = ok && mbar_wait(full_b0 + 8 * (t / G), bphase, abort_flag);
                    QT_ADD(4, true);
                }
                if (!__all_sync(0xffffffffu, ok)) {
                    gave_up = true;
                    break;
                }
                QT_T0();
                tc_fence_after();
                const uint64_t da = a_desc0 + (uint64_t)(s * (A_BYTES >> 4)), db = b_desc0 + (uint64_t)(t * (B_BYTES >> 4));
                const uint32_t ta = tmem_base + (uint32_t)(A_COL0 + s * A_COLS);
                if (elect_one()) {
                    if (c < 4) {
#pragma unroll
                        for (int kk = 0; kk < 4; kk++) {
                            if (ATM) umma_f16_ts(d1, ta + 8u * kk, db + (uint64_t)(2 * kk), idesc, (c | kk) != 0);
                            else umma_f16(d1, da + (uint64_t)(2 * kk), db + (uint64_t)(2 * kk), idesc, (c | kk) != 0);
                        }
                    } else {
                        if (ATM) umma_f16_ts(d2, ta, db, idesc, 0u);
                        else umma_f16(d2, da, db, idesc, 0u);
                    }
                    umma_commit(empty_a0 + 8 * s);
                    if (t % G == G - 1) umma_commit(empty_b0 + 8 * (t / G));
                    if (c == 4) umma_commit(tfull0 + 8 * acc);
                }
                __syncwarp();
                QT_ADD(11, true);
                if (++s == NA) s = 0, phase ^= 1u;
                if (++t == NB) t = 0, bphase ^= 1u;
            }
            if (gave_up) break;
            if (++acc == 2) acc = 0, acc_phase ^= 1u;
        }
        QT_FLUSH(2, lane == 0);
        QT_FLUSH(3, lane == 0);
        QT_FLUSH(4, lane == 0);
        QT_FLUSH(11, lane == 0);
    } else if (warp >= 4 && warp < DRAIN0) {
        // ---- raw tile -> the tensor cores' A operand. Two groups of four warps take alternate 64-weight chunks
        //      (so two chunks are in flight per scheduler); in a group, thread r owns weight row r.
        const int r = ((int)threadIdx.x - 128) & 127, grp = ((int)threadIdx.x - 128) >> 7;
        const uint32_t swz = (uint32_t)(r & 7);
        const int total = 5 * (sb_hi - sb_lo);
        int cur = -1;                       // the super-block (index within the slice) whose raw tile this thread holds
        const unsigned char* raw = nullptr;
        uint32_t scw[2] = {0, 0}, mnw[2] = {0, 0}, dword = 0;
        for (int ci = grp; ci < total && !gave_up; ci += NG) {
            const int sbi = ci / 5, c = ci - 5 * sbi, s = SBM ? sbi % SLOTS : ci % NA;
            const uint32_t phase = (uint32_t)(SBM ? sbi / SLOTS : ci / NA) & 1u;
            const bool first_of_sb = sbi != cur, last_of_sb = (ci + NG) / 5 != sbi || ci + NG >= total;
            if (sbi != cur) {
                if (cur >= 0) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(raw_empty0 + 8 * (cur % RS));
                }
                cur = sbi;
                bool ok;
                {
                    QT_T0();
                    ok = mbar_wait(raw_full0 + 8 * (sbi % RS), (uint32_t)(sbi / RS) & 1u, abort_flag);
                    QT_ADD(5, threadIdx.x == 128);
                }
                if (!ok) {
                    gave_up = true;
                    break;
                }
                raw = raw_ring + (sbi % RS) * RAW_BYTES + r * RAW_ROW;
                const uint4 h = *reinterpret_cast<const uint4*>(raw);
                // 6-bit scales and mins of the eight units (src/ref/tensor.zig:95-104)
                scw[0] = h.y & 0x3f3f3f3fu, scw[1] = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
                mnw[0] = h.z & 0x3f3f3f3fu, mnw[1] = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
                dword = h.x;
            }
            bool oka = true;
            if (!SBM || first_of_sb) {
                QT_T0();
                oka = mbar_wait(empty_a0 + 8 * s, phase ^ 1u, abort_flag);
                QT_ADD(6, threadIdx.x == 128);
            }
            if (!oka) {
                gave_up = true;
                break;
            }
            QT_T0();
#ifdef QT_TRACE
            long long td__ = clock64();
#endif
            unsigned char* arow = a_ring + s * A_BYTES + r * 128;
            const uint32_t ta = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) +
                                (uint32_t)(SBM ? SB_COL0 + s * SB_COLS + (c < 4 ? 32 * c : 128) : A_COL0 + s * A_COLS);
            if (ATM) tc_fence_after();  // the wait above ordered this stage's last reads (the MMAs) before these writes
            if (c < 4) {
                const uint4 qa = *reinterpret_cast<const uint4*>(raw + 16 + 32 * c), qb = *reinterpret_cast<const uint4*>(raw + 32 + 32 * c);
                const uint32_t qw[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
                // units 2c (low nibbles) and 2c + 1 (high nibbles): bytes 2c & 3 and (2c + 1) & 3 of word c >> 1
                const uint32_t sw = c < 2 ? scw[0] : scw[1];
                const __half2 scl = __half2half2(__int2half_rn((int)((sw >> (16 * (c & 1))) & 0xffu)));
                const __half2 sch = __half2half2(__int2half_rn((int)((sw >> (16 * (c & 1) + 8)) & 0xffu)));
                // Codes in bits 0-3 of a 16-bit lane: 0x6400 | q is the f16 1024 + q, and (1024 + q) sc - 1024 sc = q sc;
                // codes in bits 4-7: 0x6400 | (q << 4) is 1024 + 16 q, and (1024 + 16 q) (sc / 16) - 64 sc = q sc. Both
                // exact (one rounding of an exactly representable result), and only the upper bytes need a shift.
                const __half2 offl = __hmul2(scl, __half2half2(__int2half_rn(-1024)));
                const __half2 sch16 = __hmul2(sch, __float2half2_rn(0.0625f)), offh = __hmul2(sch, __half2half2(__int2half_rn(-64)));
                uint4 lo[4], hi[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    // 16 bytes = positions 8i .. 8i+7 of the unit: values (0,2,1,3 | 4,6,5,7) of two code words
                    const uint32_t w0 = qw[2 * i], w1 = qw[2 * i + 1], v0 = w0 >> 8, v1 = w1 >> 8;
                    lo[i].x = scaled_pair(w0 & 0x000f000fu, scl, offl);
                    lo[i].y = scaled_pair(v0 & 0x000f000fu, scl, offl);
                    lo[i].z = scaled_pair(w1 & 0x000f000fu, scl, offl);
                    lo[i].w = scaled_pair(v1 & 0x000f000fu, scl, offl);
                    hi[i].x = scaled_pair(w0 & 0x00f000f0u, sch16, offh);
                    hi[i].y = scaled_pair(v0 & 0x00f000f0u, sch16, offh);
                    hi[i].z = scaled_pair(w1 & 0x00f000f0u, sch16, offh);
                    hi[i].w = scaled_pair(v1 & 0x00f000f0u, sch16, offh);
                }
                if (ATM) {
                    // columns 0..15: the low unit (two values a column), 16..31: the high unit
                    tmem_st8(ta, lo[0].x, lo[0].y, lo[0].z, lo[0].w, lo[1].x, lo[1].y, lo[1].z, lo[1].w);
                    tmem_st8(ta + 8u, lo[2].x, lo[2].y, lo[2].z, lo[2].w, lo[3].x, lo[3].y, lo[3].z, lo[3].w);
                    tmem_st8(ta + 16u, hi[0].x, hi[0].y, hi[0].z, hi[0].w, hi[1].x, hi[1].y, hi[1].z, hi[1].w);
                    tmem_st8(ta + 24u, hi[2].x, hi[2].y, hi[2].z, hi[2].w, hi[3].x, hi[3].y, hi[3].z, hi[3].w);
                } else {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        *reinterpret_cast<uint4*>(arow + (((uint32_t)i ^ swz) << 4)) = lo[i];
                        *reinterpret_cast<uint4*>(arow + (((uint32_t)(i + 4) ^ swz) << 4)) = hi[i];
                    }
                }
            } else {
                // the mins, each twice: K positions 2u, 2u + 1 meet the two terms of unit u's column sum
                uint4 m0, m1;
                auto dup = [](uint32_t byte) {
                    const __half2 v = __half2half2(__int2half_rn((int)byte));
                    return *reinterpret_cast<const uint32_t*>(&v);
                };
                m0.x = dup(mnw[0] & 0xffu), m0.y = dup((mnw[0] >> 8) & 0xffu), m0.z = dup((mnw[0] >> 16) & 0xffu), m0.w = dup(mnw[0] >> 24);
                m1.x = dup(mnw[1] & 0xffu), m1.y = dup((mnw[1] >> 8) & 0xffu), m1.z = dup((mnw[1] >> 16) & 0xffu), m1.w = dup(mnw[1] >> 24);
                if (ATM) {
                    tmem_st8(ta, m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w);
                } else {
                    *reinterpret_cast<uint4*>(arow + ((0u ^ swz) << 4)) = m0;
                    *reinterpret_cast<uint4*>(arow + ((1u ^ swz) << 4)) = m1;
                }
                // the row's super-scales, for the drain of this super-block (it starts after this chunk's MMA)
                hdr[(sbi & (HDR_SLOTS - 1)) * QT_ROWS + r] = make_float2(__half2float(__ushort_as_half((unsigned short)(dword & 0xffffu))),
                                                                        __half2float(__ushort_as_half((unsigned short)(dword >> 16))));
            }
            QT_MARK(15, td__);
            if (SBM) {
                if (last_of_sb) {   // this group's chunks of the super-block are written: publish them
                    tmem_st_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(full_a0 + 8 * s);
                }
            } else {
                if (ATM) {
                    tmem_st_wait();
                    tc_fence_before();
                } else {
                    // these stores are read through the async proxy (the tensor cores)
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(full_a0 + 8 * s);
            }
            QT_MARK(17, td__);
            QT_ADD(7, threadIdx.x == 128);
        }
        if (cur >= 0 && !gave_up) {
            __syncwarp();
            if (lane == 0) mbar_arrive(raw_empty0 + 8 * (cur % RS));
        }
        QT_FLUSH(5, threadIdx.x == 128);
        QT_FLUSH(6, threadIdx.x == 128);
        QT_FLUSH(7, threadIdx.x == 128);
        QT_FLUSH(15, threadIdx.x == 128);
        QT_FLUSH(16, threadIdx.x == 128);
        QT_FLUSH(17, threadIdx.x == 128);
    } else if (warp >= DRAIN0) {
        // ---- drain. Thread (quad, lane) owns weight row quad * 32 + lane and CPT of the CTA's columns.
        const int quad = warp & 3, chalf = (warp - DRAIN0) >> 2;
        const int r = quad * 32 + lane;
        float accv[CPT];
#pragma unroll
        for (int i = 0; i < CPT; i++) accv[i] = 0.f;
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int sb = sb_lo; sb < sb_hi; sb++) {
            bool ok;
            {
                QT_T0();
                ok = __all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag));
                QT_ADD(8, threadIdx.x == 32 * DRAIN0);
            }
            if (!ok) {
                gave_up = true;
                break;
            }
            QT_T0();
            tc_fence_after();
            const float2 dd = hdr[((sb - sb_lo) & (HDR_SLOTS - 1)) * QT_ROWS + r];
            const float* cs = csc + ((sb - sb_lo) & (CSC_SLOTS - 1)) * BN + chalf * CPT;
            const uint32_t t1 = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * 2 * BN + (uint32_t)(chalf * CPT), t2 = t1 + BN;
#pragma unroll
            for (int i0 = 0; i0 < CPT; i0 += 8) {
                uint32_t v1[8], v2[8];
                tmem_ld8(t1 + i0, v1);
                tmem_ld8(t2 + i0, v2);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 8; i++)
                    accv[i0 + i] = __fmaf_rn(cs[i0 + i], __fmaf_rn(dd.x, __uint_as_float(v1[i]), -(dd.y * __uint_as_float(v2[i]))), accv[i0 + i]);
            }
            tc_fence_before();
            mbar_arrive(tempty0 + 8 * acc);
            QT_ADD(9, threadIdx.x == 32 * DRAIN0);
            if (++acc == 2) acc = 0, acc_phase ^= 1u;
        }
        QT_FLUSH(8, threadIdx.x == 32 * DRAIN0);
        QT_FLUSH(9, threadIdx.x == 32 * DRAIN0);
        asm volatile("griddepcontrol.wait;\n" ::: "memory");   // (long past: the MMAs needed the columns)
        if (!gave_up && row0 + r < q.seg_rows) {
            float* dst = q.out + (size_t)z * q.slice_stride + q.col0 + (size_t)seg * q.seg_out + row0 + r;
#pragma unroll
            for (int i = 0; i < CPT; i++) {
                const int c = c0 + chalf * CPT + i;
                if (c < q.cols) {
                    float* o = dst + (size_t)c * q.out_stride;
                    *o = q.accumulate ? *o + accv[i] : accv[i];
                }
            }
        }
    }
    if (gave_up && q.status) atomicExch(q.status, 2);
    tc_fence_before();
    __syncthreads();
#ifdef QT_TRACE
    if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) qt_trace[10] += (unsigned long long)(clock64() - kernel_t0);
#endif
    if (warp == 2) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TCOLS) : "memory");
    }
}


// ---------------------------------------------------------------------------------------------- the columns
// Position of value e inside its group of four: the decoder leaves a code word's values as (0, 2, 1, 3).
__device__ __forceinline__ uint2 perm_pack(__half a, __half b, __half c, __half d) {
    const __half2 lo = __halves2half2(a, c), hi = __halves2half2(b, d);
    return make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}

// Prefill: the Q8_K values of quantize_q8 -> f16 columns, their unit sums as two exact f16 terms (even part, low
// bit), and the block scales transposed. grid (k / 256, tokens), 64 threads, thread = four values.
__global__ void __launch_bounds__(64) cols_from_q8_kernel(const int8_t* __restrict__ qx, const float* __restrict__ dx, __half* __restrict__ bcol,
                                                         __half* __restrict__ bsum, float* __restrict__ scales, int k, int cols_pad) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // the multiply may start its weight copies now
    const int li = threadIdx.x, sb = blockIdx.x, tok = blockIdx.y, nsb = k / 256;
    const char4 v = reinterpret_cast<const char4*>(qx + (size_t)tok * k + (size_t)sb * 256)[li];
    reinterpret_cast<uint2*>(bcol + (size_t)tok * k + (size_t)sb * 256)[li] =
        perm_pack(__int2half_rn(v.x), __int2half_rn(v.y), __int2half_rn(v.z), __int2half_rn(v.w));
    int s = (int)v.x + v.y + v.z + v.w;
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    s += __shfl_xor_sync(0xffffffffu, s, 4);
    if ((li & 7) == 0) {
        const __half2 two = __halves2half2(__int2half_rn(s & ~1), __int2half_rn(s & 1));  // |s| <= 4064: both exact
        reinterpret_cast<__half2*>(bsum + (size_t)tok * nsb * 64 + (size_t)sb * 64)[li >> 3] = two;
    }
    if (li == 0) scales[(size_t)sb * cols_pad + tok] = dx[(size_t)tok * nsb + sb];
}

// Decode: f32 activations (RMSNorm or SiLU-pair fused, as quantize_q8 fuses them) -> two f16 columns per token.
// Per 256-value block: e with amax * 2^e in [2^9, 2^10); hi = f16(x 2^e), lo = f16(x 2^e - hi); the block's
// scale is 2^-e for both columns. grid (k / 256, tokens), 64 threads.
__global__ void __launch_bounds__(64) cols_from_f32_kernel(const float* __restrict__ x, const float* __restrict__ nw, __half* __restrict__ bcol,
                                                          __half* __restrict__ bsum, float* __restrict__ scales, int k, int x_stride, int mode,
                                                          float eps, int cols_pad, const __grid_constant__ PeerUse pu, int* __restrict__ status) {
    __shared__ double red[2];
    __shared__ float amax_s[2];
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // the multiply may start its weight copies now (it waits for this kernel itself)
    asm volatile("griddepcontrol.wait;\n" ::: "memory");                // the kernels before this one are done (inputs, and the scratch's last readers)
    const int li = threadIdx.x, sb = blockIdx.x, tok = blockIdx.y, nsb = k / 256;
    const float* xt = x + (size_t)tok * x_stride;
    // the activations: local memory, or the slots of a tensor-parallel exchange (each read waits for its tag)
    const bool exchanged = pu.wait_slot != PEER_NONE;
    const uint32_t x_tag = exchanged ? peer::want_tag(pu) : 0u;
    auto ldx = [&](int i) { return exchanged ? peer::read4(pu, xt + 4 * i, x_tag, status) : reinterpret_cast<const float4*>(xt)[i]; };
    float4 v;
    if (mode == 2) {  // silu(gate) * up over rows of gate | up (src/kernels/quantize_q8.wgsl)
        const float4 g = reinterpret_cast<const float4*>(xt)[sb * 64 + li], u = reinterpret_cast<const float4*>(xt + k)[sb * 64 + li];
        v = make_float4(mv::silu_f(g.x) * u.x, mv::silu_f(g.y) * u.y, mv::silu_f(g.z) * u.z, mv::silu_f(g.w) * u.w);
    } else {
        v = ldx(sb * 64 + li);
    }
    if (mode == 1) {  // RMSNorm(x) * w: f32 squares summed in f64 (src/ref/ops.zig:30-41)
        double ss = 0.0;
        for (int i = li; i < k / 4; i += 64) {
            const float4 r = ldx(i);
            ss += (double)__fmul_rn(r.x, r.x);
            ss += (double)__fmul_rn(r.y, r.y);
            ss += (double)__fmul_rn(r.z, r.z);
            ss += (double)__fmul_rn(r.w, r.w);
        }
        ss = mv::warp_sum_d(ss);
        if ((li & 31) == 0) red[li >> 5] = ss;
        __syncthreads();
        const float mean = (float)((red[0] + red[1]) / (double)k);
        const float scale = 1.0f / sqrtf(mean + eps);
        const float4 w = reinterpret_cast<const float4*>(nw)[sb * 64 + li];
        v.x = __fmul_rn(__fmul_rn(v.x, scale), w.x);
        v.y = __fmul_rn(__fmul_rn(v.y, scale), w.y);
        v.z = __fmul_rn(__fmul_rn(v.z, scale), w.z);
        v.w = __fmul_rn(__fmul_rn(v.w, scale), w.w);
    }
    float am = fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w)));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
    if ((li & 31) == 0) amax_s[li >> 5] = am;
    __syncthreads();
    am = fmaxf(amax_s[0], amax_s[1]);
    float up = 1.0f, down = 1.0f;
    if (am > 0.f && am < 3.0e38f) {
        const int e = (int)((__float_as_uint(am) >> 23) & 0xffu) - 127;   // am = f 2^e, f in [1, 2)
        const int sh = max(-110, min(110, 9 - e));
        up = __uint_as_float((uint32_t)(sh + 127) << 23);
        down = __uint_as_float((uint32_t)(127 - sh) << 23);
    }
    const float y[4] = {v.x * up, v.y * up, v.z * up, v.w * up};
    __half hi[4], lo[4];
    float sh_ = 0.f, sl_ = 0.f;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        hi[i] = __float2half_rn(y[i]);
        lo[i] = __float2half_rn(y[i] - __half2float(hi[i]));
        sh_ += __half2float(hi[i]);
        sl_ += __half2float(lo[i]);
    }
    __half* b0 = bcol + (size_t)(2 * tok) * k + (size_t)sb * 256;
    reinterpret_cast<uint2*>(b0)[li] = perm_pack(hi[0], hi[1], hi[2], hi[3]);
    reinterpret_cast<uint2*>(b0 + k)[li] = perm_pack(lo[0], lo[1], lo[2], lo[3]);
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
        sh_ += __shfl_xor_sync(0xffffffffu, sh_, o);
        sl_ += __shfl_xor_sync(0xffffffffu, sl_, o);
    }
    if ((li & 7) == 0) {
        const __half a = __float2half_rn(sh_), c = __float2half_rn(sl_);
        __half* s0 = bsum + (size_t)(2 * tok) * nsb * 64 + (size_t)sb * 64 + 2 * (li >> 3);
        *reinterpret_cast<__half2*>(s0) = __halves2half2(a, __float2half_rn(sh_ - __half2float(a)));
        *reinterpret_cast<__half2*>(s0 + (size_t)nsb * 64) = __halves2half2(c, __float2half_rn(sl_ - __half2float(c)));
    }
    if (li == 0) {
        scales[(size_t)sb * cols_pad + 2 * tok] = down;
        scales[(size_t)sb * cols_pad + 2 * tok + 1] = down;
    }
}

// Decode: the k slices and the two columns of a token, added in a fixed order; SILU_PAIR and ACCUMULATE as the
// multiply's epilogue applies them. part[z][column][seg * n + j].
__global__ void __launch_bounds__(256) cols_reduce_kernel(const float* __restrict__ part, float* __restrict__ out, int n, int m, int slices,
                                                         int cols, int pair, int accumulate, uint32_t out_stride, uint32_t col0,
                                                         const __grid_constant__ PeerUse pu) {
    asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");   // a dependent kernel after this one may be scheduled
    asm volatile("griddepcontrol.wait;\n" ::: "memory");                // the multiply is done
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < (size_t)n * m) {
        const int tok = (int)(i / n), j = (int)(i % n);
        const size_t width = (size_t)n * (pair ? 2 : 1), zs = (size_t)cols * width;
        float v = 0.f, u = 0.f;
        for (int z = 0; z < slices; z++) {
            const float* p = part + z * zs + (size_t)(2 * tok) * width + j;
            v = __fadd_rn(v, __fadd_rn(p[0], p[width]));
            if (pair) u = __fadd_rn(u, __fadd_rn(p[n], p[width + n]));
        }
        if (pair) v = mv::silu_f(v) * u;
        const size_t o = (size_t)tok * out_stride + col0 + j;
        if (accumulate) v += out[o];
        out[o] = v;
        // this rank's slice of an exchanged vector: to every rank's exchange slots
        if (pu.push_slot != PEER_NONE) peer::push(pu, out + o, v, peer::push_tag(pu));
    }
}

// ---------------------------------------------------------------------------------------------- host side
inline bool cols_map(CUtensorMap* map, const void* base, uint64_t cols, uint64_t row_bytes, uint32_t bn) {
    tma::EncodeTiledFn enc = tma::encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[2] = {row_bytes, cols}, strides[1] = {row_bytes};
    const cuuint32_t box[2] = {128, bn}, elem[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

struct QtPlan {
    const void* w;
    uint64_t w_rows;     // every row the weight map may touch
    int k, cols, bn;
    const void* bcol;
    const void* bsum;
    QtArgs q;
    int slices;
};

template <int BN>
zcu_result launch_qgemm_bn(const LaunchArgs& a, const QtPlan& pl) {
    CUtensorMap wmap, bmap, smap;
    const uint64_t rb = (uint64_t)(pl.k / 256) * 144;
    const bool ok = tma::bytes_2d(&wmap, pl.w, pl.w_rows, rb, RAW_ROW, QT_ROWS) && cols_map(&bmap, pl.bcol, (uint64_t)pl.cols, (uint64_t)pl.k * 2, BN) &&
                    cols_map(&smap, pl.bsum, (uint64_t)pl.cols, (uint64_t)(pl.k / 256) * 128, BN);
    if (!ok) return zcu_fail(a, ZCU_E_GPU, "q4_k multiply (tcgen05): the driver refused a tensor map (k %d, columns %d)", pl.k, pl.cols);
    auto kern = qgemm_q4k_kernel<BN>;
    constexpr int SMEM = qt_smem(BN);
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) {
        cudaGetLastError();
        return zcu_fail(a, ZCU_E_GPU, "q4_k multiply (tcgen05): %d bytes of shared memory refused", SMEM);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(pl.q.tiles_per_seg * pl.q.nseg), (unsigned)((pl.cols + BN - 1) / BN), (unsigned)pl.slices);
    cfg.blockDim = dim3(qt_threads(BN));
    cfg.dynamicSmemBytes = SMEM;
    cfg.stream = a.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;   // see the wait in the kernel's column warp
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, wmap, bmap, smap, pl.q);
    if (e != cudaSuccess) return zcu_fail(a, ZCU_E_GPU, "q4_k multiply (tcgen05): launch failed: %s", cudaGetErrorString(e));
    return ZCU_OK;
}

zcu_result launch_qgemm(const LaunchArgs& a, const QtPlan& pl) {
    switch (pl.bn) {
        case 16: return launch_qgemm_bn<16>(a, pl);
        case 32: return launch_qgemm_bn<32>(a, pl);
        case 64: return launch_qgemm_bn<64>(a, pl);
        default: return launch_qgemm_bn<128>(a, pl);
    }
}

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Staging memory of one multiply: the context's scratch when it is large enough (launches of a context run in
// stream order, so the next multiply reuses it), else a stream-ordered allocation freed after the last kernel.
struct Scratch {
    unsigned char* p = nullptr;
    bool owned = false;
};
inline bool scratch_get(const LaunchArgs& a, size_t bytes, Scratch& s) {
    if (a.scratch && bytes <= a.scratch_bytes) {
        s.p = static_cast<unsigned char*>(a.scratch);
        return true;
    }
    if (cudaMallocAsync((void**)&s.p, bytes, a.stream) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    s.owned = true;
    return true;
}
inline void scratch_put(const LaunchArgs& a, Scratch& s) {
    if (s.owned) cudaFreeAsync(s.p, a.stream);
}

// A launch that may start while the kernel before it in the stream finishes (programmatic dependent launch): the
// kernel orders itself with griddepcontrol.wait before it touches what that kernel wrote or still reads.
template <class... KArgs, class... Args>
cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
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
    return cudaLaunchKernelEx(&cfg, kern, args...);
}

}  // namespace

// matmul_q4_k, the tensor-core rung: params.MatmulQuant and the bindings qx, w, out, dx of the integer-dot identity.
zcu_result launch_matmul_q4_k_tc(const LaunchArgs& a) {
    PMatmulQuant p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 4, "matmul_q4_k (tcgen05): bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    const uint32_t cap = a.grid[1] * 32u;   // the reference dispatches token tiles of 32 (grid y)
    const int tokens = (int)(p.rows < cap ? p.rows : cap);
    if (tokens == 0 || p.n == 0) return ZCU_OK;
    ZCU_NEED(a, p.k % 256 == 0 && p.k > 0, "matmul_q4_k (tcgen05): k = %u is not a multiple of 256", p.k);
    ZCU_NEED(a, p.k_slice > 0 && p.k_slice % 256 == 0, "matmul_q4_k (tcgen05): k_slice = %u is not a multiple of 256", p.k_slice);
    const uint32_t slices = (p.k + p.k_slice - 1) / p.k_slice;
    ZCU_NEED(a, a.grid[2] <= 1 || a.grid[2] == slices, "matmul_q4_k (tcgen05): %u slices in the grid, %u by k_slice", a.grid[2], slices);
    ZCU_NEED(a, ((uintptr_t)a.b[0].ptr & 15) == 0 && ((uintptr_t)a.b[1].ptr & 15) == 0, "matmul_q4_k (tcgen05): qx and w must be 16-byte aligned");
    const int k = (int)p.k, nsb = k / 256;
    const int bn = tokens > 64 ? 128 : tokens > 32 ? 64 : tokens > 16 ? 32 : 16;
    const int cols_pad = (int)align_up((size_t)tokens, (size_t)bn);
    const size_t b_bytes = align_up((size_t)tokens * k * 2, 1024), s_bytes = align_up((size_t)tokens * nsb * 128, 1024),
                 c_bytes = align_up((size_t)nsb * cols_pad * 4, 1024);
    Scratch sc;
    if (!scratch_get(a, b_bytes + s_bytes + c_bytes, sc))
        return zcu_fail(a, ZCU_E_GPU, "matmul_q4_k (tcgen05): no memory for %zu bytes of columns", b_bytes + s_bytes + c_bytes);
    unsigned char* scratch = sc.p;
    __half* bcol = reinterpret_cast<__half*>(scratch);
    __half* bsum = reinterpret_cast<__half*>(scratch + b_bytes);
    float* scales = reinterpret_cast<float*>(scratch + b_bytes + s_bytes);
    cudaMemsetAsync(scales, 0, c_bytes, a.stream);
    cols_from_q8_kernel<<<dim3((unsigned)nsb, (unsigned)tokens), 64, 0, a.stream>>>((const int8_t*)a.b[0].ptr, (const float*)a.b[3].ptr, bcol, bsum, scales,
                                                                                 k, cols_pad);
    QtPlan pl{};
    pl.w = a.b[1].ptr;
    pl.w_rows = p.n;
    pl.k = k;
    pl.cols = tokens;
    pl.bn = bn;
    pl.bcol = bcol;
    pl.bsum = bsum;
    pl.slices = (int)slices;
    pl.q.seg_rows = (int)p.n;
    pl.q.nseg = 1;
    pl.q.seg1_y = 0;
    pl.q.tiles_per_seg = ((int)p.n + QT_ROWS - 1) / QT_ROWS;
    pl.q.cols = tokens;
    pl.q.cols_pad = cols_pad;
    pl.q.nsb = nsb;
    pl.q.sb_per_slice = (int)p.k_slice / 256;
    pl.q.out = (float*)a.b[2].ptr;
    pl.q.slice_stride = p.slice_stride;
    pl.q.out_stride = p.out_stride;
    pl.q.col0 = p.col0;
    pl.q.seg_out = 0;
    pl.q.accumulate = p.accumulate;
    pl.q.scales = scales;
    pl.q.status = a.status;
    const zcu_result r = launch_qgemm(a, pl);
    scratch_put(a, sc);
    return r;
}

// matvec_q4_k, the batched family: one pass over the weights for up to 64 tokens.
zcu_result launch_matvec_q4_k_tc(const LaunchArgs& a, const mv::MvArgs& v) {
    if (v.combine.blocks) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec_q4_k (tcgen05): attn_combine is not fused into this family");
    const PMatvec& p = v.p;
    const int m = v.m, k = (int)p.k, n = (int)p.n, nsb = k / 256;
    ZCU_NEED(a, m <= 64, "matvec_q4_k (tcgen05): %d tokens in one step (at most 64)", m);
    ZCU_NEED(a, k % 256 == 0, "matvec_q4_k (tcgen05): k = %d is not a multiple of 256", k);
    if (v.has_rope) return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "matvec + rope_append: only the mma.sync family fuses it");
    const bool pair = (p.flags & MV_SILU_PAIR) != 0, norm = (p.flags & MV_NORM) != 0;
    const int cols = 2 * m;
    const int bn = cols > 64 ? 128 : cols > 32 ? 64 : cols > 16 ? 32 : 16;
    const int cols_pad = (int)align_up((size_t)cols, (size_t)bn);
    const int tiles_per_seg = (n + QT_ROWS - 1) / QT_ROWS, nseg = pair ? 2 : 1;
    const int tiles = tiles_per_seg * nseg, sms = a.sm_count > 0 ? a.sm_count : 148;
    // k slices: fill the SMs once, but keep at least four super-blocks per CTA
    int slices = sms / tiles;
    if (slices < 1) slices = 1;
    if (slices > nsb / 4) slices = nsb / 4 > 0 ? nsb / 4 : 1;
    const int sb_per_slice = (nsb + slices - 1) / slices;
    slices = (nsb + sb_per_slice - 1) / sb_per_slice;
    const size_t width = (size_t)n * nseg;
    const size_t b_bytes = align_up((size_t)cols * k * 2, 1024), s_bytes = align_up((size_t)cols * nsb * 128, 1024),
                 c_bytes = align_up((size_t)nsb * cols_pad * 4, 1024), p_bytes = align_up((size_t)slices * cols * width * 4, 1024);
    Scratch sc;
    if (!scratch_get(a, b_bytes + s_bytes + c_bytes + p_bytes, sc))
        return zcu_fail(a, ZCU_E_GPU, "matvec_q4_k (tcgen05): no memory for %zu bytes of scratch", b_bytes + s_bytes + c_bytes + p_bytes);
    unsigned char* scratch = sc.p;
    __half* bcol = reinterpret_cast<__half*>(scratch);
    __half* bsum = reinterpret_cast<__half*>(scratch + b_bytes);
    float* scales = reinterpret_cast<float*>(scratch + b_bytes + s_bytes);
    float* part = reinterpret_cast<float*>(scratch + b_bytes + s_bytes + c_bytes);
    if (cols_pad != cols) cudaMemsetAsync(scales, 0, c_bytes, a.stream);
    const int xr = p.x_stride ? (int)p.x_stride * 4 : k;
    // (the column kernel, the multiply and the reduction are programmatic dependents of one another and of the kernel
    // before them: each may be scheduled while its predecessor finishes, and waits before it touches memory)
    if (launch_dependent(cols_from_f32_kernel, dim3((unsigned)nsb, (unsigned)m), dim3(64), 0, a.stream, v.x, v.nw, bcol, bsum, scales, k, xr,
                         norm ? 1 : 0, p.eps, cols_pad, v.peer, a.status) != cudaSuccess) {
        scratch_put(a, sc);
        return zcu_fail(a, ZCU_E_GPU, "matvec_q4_k (tcgen05): launch failed: %s", cudaGetErrorString(cudaGetLastError()));
    }
    QtPlan pl{};
    pl.w = v.w;
    pl.w_rows = pair ? (uint64_t)p.half + n : (uint64_t)n;
    pl.k = k;
    pl.cols = cols;
    pl.bn = bn;
    pl.bcol = bcol;
    pl.bsum = bsum;
    pl.slices = slices;
    pl.q.seg_rows = n;
    pl.q.nseg = nseg;
    pl.q.seg1_y = (int)p.half;
    pl.q.tiles_per_seg = tiles_per_seg;
    pl.q.cols = cols;
    pl.q.cols_pad = cols_pad;
    pl.q.nsb = nsb;
    pl.q.sb_per_slice = sb_per_slice;
    pl.q.out = part;
    pl.q.slice_stride = (size_t)cols * width;
    pl.q.out_stride = (uint32_t)width;
    pl.q.col0 = 0;
    pl.q.seg_out = (uint32_t)n;
    pl.q.accumulate = 0;
    pl.q.scales = scales;
    pl.q.status = a.status;
    zcu_result r = launch_qgemm(a, pl);
    if (r == ZCU_OK) {
        const size_t elems = (size_t)n * m;
        const cudaError_t e = launch_dependent(cols_reduce_kernel, dim3((unsigned)((elems + 255) / 256)), dim3(256), 0, a.stream, (const float*)part,
                                               v.out, n, m, slices, cols, pair ? 1 : 0, (p.flags & MV_ACCUMULATE) ? 1 : 0, p.out_stride, p.col0, v.peer);
        if (e != cudaSuccess) r = zcu_fail(a, ZCU_E_GPU, "matvec_q4_k (tcgen05): launch failed: %s", cudaGetErrorString(e));
    }
    scratch_put(a, sc);
    return r;
}
