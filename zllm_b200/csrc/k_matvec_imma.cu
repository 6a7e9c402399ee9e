// The standalone kernel of the tensor-core decode multiplies (see k_matvec_imma.cuh for the method).

#include "k_matvec_imma.cuh"

namespace {

using namespace imma;

// Launched as a programmatic dependent: its weight copies start while the kernel before it drains; it waits
// (griddepcontrol.wait) only before it reads activations.
template <int TYPE, int NB, int STAGES>
__global__ void __launch_bounds__(IM_THREADS, 1) matvec_imma(PMatvec p, const float* __restrict__ x,
                                                            const __grid_constant__ CUtensorMap wmap,
                                                            const __grid_constant__ CUtensorMap smap, float* __restrict__ out,
                                                            const float* __restrict__ norm_w, int t0, int mt,
                                                            int seg_max, int* __restrict__ status, const __grid_constant__ MvRope rope,
                                                            const __grid_constant__ PeerUse pu) {
    extern __shared__ __align__(128) uint8_t smem[];
    // (broadcast from lane 0: the compiler then knows the warp index, and what derives from it - ring addresses, tile
    // coordinates - to be the same in every lane, and feeds the copy instructions from uniform registers)
    const int lane = threadIdx.x & 31, warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const ImLayout L = im_layout(4 * mt, (int)p.k, TYPE == W_Q4_K, 2 * NB, seg_max, STAGES);
    ImRing rg;
    ImIssue iss;
    im_ring_init<STAGES>(rg, smem, L, warp, lane);
    im_prime<TYPE, STAGES>(rg, iss, p, &wmap, &smap, (int)blockIdx.x, (int)gridDim.x, warp, lane, 0);
    im_multiply<TYPE, NB, STAGES>(
        smem, rg, iss, (int)blockIdx.x, (int)gridDim.x, p, x, out, norm_w, t0, mt, seg_max, status,
        (p.flags & MV_ROPE_APPEND) ? &rope : nullptr, &pu,
        [&] {
            // everything before touched only the weights, which no kernel writes; from here on the
            // activations are read, so the kernels before this one must have finished on this GPU (in a
            // tensor-parallel exchange the reads themselves wait for the other ranks' slices)
            asm volatile("griddepcontrol.wait;\n" ::: "memory");
            asm volatile("griddepcontrol.launch_dependents;\n" ::: "memory");
        },
        [] {});
}

constexpr int IM_SMEM_MAX = 220 * 1024;

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
    // the weights as a byte matrix of 16-row boxes (both halves of a SILU_PAIR matrix are rows of one matrix)
    const size_t rows = (size_t)v.p.n + ((v.p.flags & MV_SILU_PAIR) ? v.p.half : 0);
    CUtensorMap wmap, smap;
    if (!im_weight_map(&wmap, v.w, TYPE == W_Q4_K, (int)v.p.k, rows, false) ||
        !im_weight_map(&smap, v.w, TYPE == W_Q4_K, (int)v.p.k, rows, TYPE != W_Q4_K))
        return zcu_fail(a, ZCU_E_GPU, "matvec_imma: the driver refused a tensor map (n %u, k %u)", v.p.n, v.p.k);
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, v.p, v.x, wmap, smap, v.out, v.nw, t0, mt, seg_max, a.status, v.rope, v.peer);
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
    MvArgs pass = v;
    for (int t0 = 0; t0 < v.m;) {
        const int mt = (v.m - t0) < cap ? (v.m - t0) : cap;
        // every pass of one dispatch pushes under the same exchange tag: only the last one advances the slot's count
        pass.peer.hold = t0 + mt < v.m ? 1u : 0u;
        zcu_result r = mt > 2 ? launch_one<TYPE, 2>(a, pass, t0, mt, stages) : launch_one<TYPE, 1>(a, pass, t0, mt, stages);
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
