// Prefill multiply on the 5th-generation tensor cores: out[t][col0 + j] (+)= sum_i x[t][i] * w[j][i] with
// bf16 (or f16) operands and f32 accumulation in tensor memory. This is the lower-precision prefill rung of
// matmul_bf16 / matmul_f16 (the reference selects such rungs per device with the reserved variant 0xfffc0000,
// src/kernels/kernels.zig:798-822, src/agility/kernels.zig:112-157: activations rounded to the half type, one
// product per element pair). Same parameter block (params.MatmulBf16) and bindings x, w, out as the scalar
// identity in k_matmul.cu; _pad[0] carries two layout bits the reference zero-fills:
//   bit 0: x already holds the half type ([rows, k], 2 bytes per element) instead of f32
//   bit 1: out holds the half type (rounded to nearest even) instead of f32
//
// One persistent CTA per SM, three roles:
//   warp 0    one lane issues TMA tile loads (x tile 128 x 64, w tile bn x 64, 128-byte swizzle) into a
//             4-stage shared-memory ring; each stage completes on an mbarrier
//   warp 1    allocates the 512 tensor-memory columns; one lane issues tcgen05.mma (M 128, N bn, K 16) four
//             times per stage and commits the stage back to the loader; two accumulators alternate so the
//             next tile's products start while the previous tile drains
//   warps 2-5 read the finished accumulator with tcgen05.ld (each warp its own 32 lanes = 32 token rows),
//             convert, and store
// bn (the tile's output columns, a multiple of 16 up to 256) is chosen per launch so that the last wave of
// tiles wastes the fewest SMs. Every wait is bounded: a wait that gives up raises the CTA's abort flag, all
// roles leave their loops, tensor memory is freed, and the context's status word reports it.

#include <cuda.h>  // CUtensorMap and its enums; cuTensorMapEncodeTiled is looked up at run time, nothing links libcuda
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "zcu_internal.h"

namespace {

constexpr int BM = 128, BN_MAX = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES_MAX = BN_MAX * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES_MAX;
constexpr int TC_THREADS = 192, TMEM_COLS = 512;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr uint32_t X_HALF = 1u, OUT_HALF = 2u;

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
// Waits for phase `parity`, at most 2^20 polls, and gives up early when another role has raised the abort
// flag. Returns false (with the flag raised) when it gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t mbar, uint32_t parity, volatile uint32_t* abort_flag) {
    for (int spin = 0; spin < (1 << 20); spin++) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
            : "=r"(ok)
            : "r"(mbar), "r"(parity)
            : "memory");
        if (ok) return true;
        if ((spin & 63) == 63 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// One 2-D tile, global -> shared, completing on the stage's mbarrier. x (the innermost coordinate) is a
// multiple of 64 two-byte elements, so the copy starts on a 128-byte boundary.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t mbar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n" ::"r"(dst),
                 "l"((uint64_t)map), "r"(mbar), "r"(x), "r"(y)
                 : "memory");
}
// Shared-memory operand descriptor: K-major rows of 128 bytes, 128-byte swizzle, groups of 8 rows 1024 bytes
// apart (the layout a TMA tile load with CU_TENSOR_MAP_SWIZZLE_128B leaves behind).
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t saddr) {
    uint64_t d = (uint64_t)((saddr >> 4) & 0x3FFFu);  // start address / 16
    d |= (uint64_t)1 << 16;                           // leading byte offset / 16 (not used by swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                 // stride byte offset / 16
    d |= (uint64_t)1 << 46;                           // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                           // 128-byte swizzle
    return d;
}
// D[tmem] (+)= A[smem] * B[smem]^T, issued by one thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\ntcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
                 "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
                 : "memory");
}
// The mbarrier gets one arrival when every tcgen05.mma this thread issued so far has completed.
__device__ __forceinline__ void umma_commit(uint32_t mbar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(mbar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
// 16 consecutive f32 columns of this thread's tensor-memory lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

template <bool BF16>
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    if (BF16) {
        const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    const __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}
template <bool BF16>
__device__ __forceinline__ float widen_half(unsigned short bits) {
    if (BF16) return __uint_as_float((uint32_t)bits << 16);
    return __half2float(__ushort_as_half(bits));
}
template <bool BF16>
__device__ __forceinline__ unsigned short narrow_half(float v) {
    if (BF16) return __bfloat16_as_ushort(__float2bfloat16_rn(v));
    return __half_as_ushort(__float2half_rn(v));
}

// 16 accumulator columns of one token row -> out. `vec`: 16-byte stores are legal for this launch.
template <bool BF16>
__device__ __forceinline__ void store16(const PMatmulBf16& p, void* out, uint32_t flags, bool vec, int t, int j0, const uint32_t* r) {
    if (t >= (int)p.rows || j0 >= (int)p.n) return;
    const size_t o = (size_t)t * p.out_stride + p.col0 + j0;
    const bool whole = j0 + 16 <= (int)p.n;
    if (flags & OUT_HALF) {
        unsigned short* dst = reinterpret_cast<unsigned short*>(out) + o;
        if (vec && whole && !p.accumulate) {
#pragma unroll
            for (int i = 0; i < 2; i++) {
                uint4 v;
                v.x = pack_half2<BF16>(__uint_as_float(r[8 * i + 0]), __uint_as_float(r[8 * i + 1]));
                v.y = pack_half2<BF16>(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
                v.z = pack_half2<BF16>(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]));
                v.w = pack_half2<BF16>(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
                reinterpret_cast<uint4*>(dst)[i] = v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                if (j0 + i < (int)p.n) {
                    float v = __uint_as_float(r[i]);
                    if (p.accumulate) v += widen_half<BF16>(dst[i]);
                    dst[i] = narrow_half<BF16>(v);
                }
            }
        }
    } else {
        float* dst = reinterpret_cast<float*>(out) + o;
        if (vec && whole) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                float4 v = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]),
                                       __uint_as_float(r[4 * i + 3]));
                if (p.accumulate) {
                    const float4 old = reinterpret_cast<const float4*>(dst)[i];
                    v.x += old.x, v.y += old.y, v.z += old.z, v.w += old.w;
                }
                reinterpret_cast<float4*>(dst)[i] = v;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; i++) {
                if (j0 + i < (int)p.n) {
                    float v = __uint_as_float(r[i]);
                    if (p.accumulate) v += dst[i];
                    dst[i] = v;
                }
            }
        }
    }
}

template <bool BF16>
__global__ void __launch_bounds__(TC_THREADS, 1)
    matmul_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w, PMatmulBf16 p, void* out,
                     uint32_t flags, int bn, int vec, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    // the swizzled tiles need 1024-byte alignment
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8 * STAGES, tfull0 = empty0 + 8 * STAGES, tempty0 = tfull0 + 16;
    uint32_t* holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);  // [0] tensor-memory base, [1] abort flag
    volatile uint32_t* abort_flag = holder + 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(tfull0 + 8 * a, 1);
            mbar_init(tempty0 + 8 * a, 128);
        }
        holder[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {  // the whole warp allocates; the base address lands in shared memory
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(holder)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = holder[0];

    const int tiles_m = ((int)p.rows + BM - 1) / BM, tiles_n = ((int)p.n + bn - 1) / bn;
    const int tiles = tiles_m * tiles_n, kblocks = ((int)p.k + BK - 1) / BK;
    const uint32_t stage_tx = (uint32_t)(A_BYTES + bn * BK * 2);
    bool gave_up = false;

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int tile = blockIdx.x; tile < tiles && !gave_up; tile += gridDim.x) {
                const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * bn;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(empty0 + 8 * stage, phase ^ 1u, abort_flag)) {
                        gave_up = true;
                        break;
                    }
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES), fb = full0 + 8 * stage;
                    mbar_expect_tx(fb, stage_tx);
                    tma_load_2d(sa, &map_x, kb * BK, m0, fb);
                    tma_load_2d(sa + A_BYTES, &map_w, kb * BK, n0, fb);
                    if (++stage == STAGES) stage = 0, phase ^= 1u;
                }
            }
            if (gave_up)  // copies still in flight must land before the CTA's shared memory is given back
                for (int i = 0; i < 200; i++) __nanosleep(1000);
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: f32 accumulate, A and B in the half type, both K-major, N = bn, M = 128
            const uint32_t fmt = BF16 ? 1u : 0u;
            const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            for (int tile = blockIdx.x; tile < tiles && !gave_up; tile += gridDim.x) {
                if (!mbar_wait(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag)) {
                    gave_up = true;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)acc * BN_MAX;
                for (int kb = 0; kb < kblocks; kb++) {
                    if (!mbar_wait(full0 + 8 * stage, phase, abort_flag)) {
                        gave_up = true;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
                    const uint64_t da = umma_desc_sw128(sa), db = umma_desc_sw128(sa + A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; kk++)  // 32 bytes further along K inside the swizzled row: +2 in the address field
                        umma_f16(d_tmem, da + (uint64_t)(2 * kk), db + (uint64_t)(2 * kk), idesc, (kb | kk) != 0);
                    umma_commit(empty0 + 8 * stage);
                    if (++stage == STAGES) stage = 0, phase ^= 1u;
                }
                if (gave_up) break;
                umma_commit(tfull0 + 8 * acc);
                if (++acc == 2) acc = 0, acc_phase ^= 1u;
            }
        }
    } else {
        const int quad = warp & 3;  // a warp reads the 32 tensor-memory lanes of its quadrant
        int acc = 0;
        uint32_t acc_phase = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * bn;
            // every lane waits (each needs the barrier's ordering); the verdict is made warp-uniform because
            // tcgen05.ld below must be executed by the whole warp
            if (!__all_sync(0xffffffffu, mbar_wait(tfull0 + 8 * acc, acc_phase, abort_flag))) {
                gave_up = true;
                break;
            }
            tc_fence_after();
            const uint32_t ta = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * BN_MAX;
            const int t = m0 + quad * 32 + lane;
            for (int c = 0; c < bn; c += 32) {
                uint32_t r[32];
                const bool two = c + 16 < bn;  // bn is a multiple of 16: the same for the whole warp
                tmem_ld16(ta + c, r);
                if (two) tmem_ld16(ta + c + 16, r + 16);
                tmem_ld_wait();
                store16<BF16>(p, out, flags, vec != 0, t, n0 + c, r);
                if (two) store16<BF16>(p, out, flags, vec != 0, t, n0 + c + 16, r + 16);
            }
            tc_fence_before();
            mbar_arrive(tempty0 + 8 * acc);
            if (++acc == 2) acc = 0, acc_phase ^= 1u;
        }
    }
    if (gave_up && status) atomicExch(status, 2);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// x f32 -> the half type, round to nearest even (the rounding the oracle's roundLikeLlama applies).
template <bool BF16>
__global__ void __launch_bounds__(256) narrow_rows_kernel(const float* __restrict__ x, unsigned short* __restrict__ y, size_t count4) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += (size_t)gridDim.x * blockDim.x) {
        const float4 v = reinterpret_cast<const float4*>(x)[i];
        uint2 o;
        o.x = pack_half2<BF16>(v.x, v.y);
        o.y = pack_half2<BF16>(v.z, v.w);
        reinterpret_cast<uint2*>(y)[i] = o;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            sym = nullptr;
        return (EncodeTiledFn)sym;
    }();
    return fn;
}

// [rows, k] two-byte elements, row-major; tiles of box_rows x 64 elements with the 128-byte swizzle;
// out-of-range rows and the K tail read as zero.
bool make_map(CUtensorMap* map, bool bf16, const void* base, uint64_t rows, uint64_t k, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled();
    if (!enc) return false;
    const cuuint64_t dims[2] = {k, rows}, strides[1] = {k * 2};
    const cuuint32_t box[2] = {(cuuint32_t)BK, box_rows}, elem[2] = {1, 1};
    return enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides,
               box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The tile width (multiple of 16, 128..256) that costs the fewest (waves x width) on `sms` SMs.
int pick_bn(int rows, int n, int sms) {
    const int tiles_m = (rows + BM - 1) / BM;
    int best = BN_MAX;
    long best_cost = -1;
    for (int bn = BN_MAX; bn >= 128; bn -= 16) {
        const long tiles = (long)tiles_m * ((n + bn - 1) / bn);
        const long waves = (tiles + sms - 1) / sms;
        const long cost = waves * bn;
        if (best_cost < 0 || cost < best_cost) best = bn, best_cost = cost;
    }
    return best;
}

template <bool BF16>
zcu_result launch_tc(const LaunchArgs& a) {
    PMatmulBf16 p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "matmul (tensor-core rung): bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    const uint32_t flags = p._pad[0];
    ZCU_NEED(a, (flags & ~(X_HALF | OUT_HALF)) == 0, "matmul (tensor-core rung): unknown layout bits %#x", flags);
    ZCU_NEED(a, p.k > 0 && p.k % 8 == 0, "matmul (tensor-core rung): k = %u is not a multiple of 8 (16-byte rows)", p.k);
    if (p.rows == 0 || p.n == 0) return ZCU_OK;
    const void* x = a.b[0].ptr;
    const void* w = a.b[1].ptr;
    void* out = a.b[2].ptr;
    ZCU_NEED(a, ((uintptr_t)w & 15) == 0 && ((uintptr_t)x & 15) == 0, "matmul (tensor-core rung): x and w must be 16-byte aligned");
    auto kern = matmul_tc_kernel<BF16>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES) != cudaSuccess) {  // per device
        cudaGetLastError();
        ZCU_NEED(a, false, "matmul (tensor-core rung): %d bytes of shared memory refused", SMEM_BYTES);
    }
    void* scratch = nullptr;
    if (!(flags & X_HALF)) {  // round the f32 activations once, into stream-ordered scratch
        const size_t count = (size_t)p.rows * p.k;
        if (cudaMallocAsync(&scratch, count * 2, a.stream) != cudaSuccess) {
            cudaGetLastError();
            ZCU_NEED(a, false, "matmul (tensor-core rung): no memory for %zu bytes of rounded activations", count * 2);
        }
        const size_t count4 = count / 4;  // k % 8 == 0
        const size_t want = (count4 + 255) / 256, cap = (size_t)(a.sm_count > 0 ? a.sm_count : 148) * 8;
        const int blocks = (int)(want < cap ? want : cap);
        narrow_rows_kernel<BF16><<<blocks, 256, 0, a.stream>>>((const float*)x, (unsigned short*)scratch, count4);
        x = scratch;
    }
    const int sms = a.sm_count > 0 ? a.sm_count : 148;
    const int bn = pick_bn((int)p.rows, (int)p.n, sms);
    CUtensorMap map_x, map_w;
    const bool maps_ok = make_map(&map_x, BF16, x, p.rows, p.k, BM) && make_map(&map_w, BF16, w, p.n, p.k, (uint32_t)bn);
    if (!maps_ok) {
        if (scratch) cudaFreeAsync(scratch, a.stream);
        ZCU_NEED(a, false, "matmul (tensor-core rung): the driver refused a tensor map (rows %u, n %u, k %u)", p.rows, p.n, p.k);
    }
    const int tiles = (int)(((p.rows + BM - 1) / BM) * ((p.n + bn - 1) / bn));
    const uint32_t esz = (flags & OUT_HALF) ? 2u : 4u, per16 = 16u / esz;
    const int vec = ((uintptr_t)out & 15) == 0 && p.out_stride % per16 == 0 && p.col0 % per16 == 0;
    kern<<<tiles < sms ? tiles : sms, TC_THREADS, SMEM_BYTES, a.stream>>>(map_x, map_w, p, out, flags, bn, vec, a.status);
    const cudaError_t e = cudaGetLastError();
    if (scratch) cudaFreeAsync(scratch, a.stream);
    ZCU_NEED(a, e == cudaSuccess, "matmul (tensor-core rung): launch failed: %s", cudaGetErrorString(e));
    return ZCU_OK;
}

}  // namespace

zcu_result launch_matmul_tc(const LaunchArgs& a, bool bf16) { return bf16 ? launch_tc<true>(a) : launch_tc<false>(a); }
