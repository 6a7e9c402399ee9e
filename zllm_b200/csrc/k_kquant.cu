// The loader path of the block types beside Q4_K and Q8_0: repad and repack_q3_k lay file blocks out for 16-byte
// loads (src/kernels/repad.wgsl, repack_q3_k.wgsl; layouts kernels.blockStride, src/kernels/kernels.zig:137-151),
// and embed_q3_k / q5_k / q6_k / iq4_xs decode table rows to f32 (src/kernels/embed_quant.wgsl), bit for bit as
// the CPU reference does (src/ref/tensor.zig:54-181: every product rounded on its own, scale products first).

#include <cuda_fp16.h>

#include "zcu_internal.h"

namespace {

struct PRepad {  // kernels.zig params.Repad
    uint32_t blocks, src_bytes, dst_bytes, _pad;
};
struct PRepackQ3K {
    uint32_t blocks, _pad[3];
};

// One thread per destination word; the padding is zero. src_bytes is even, so a source word takes at most two loads.
__global__ void repad_kernel(PRepad p, const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const uint32_t words = p.dst_bytes / 4;
    const size_t blk = i / words;
    const uint32_t off = 4u * (uint32_t)(i % words);
    if (off >= p.src_bytes) {
        dst[i] = 0u;
        return;
    }
    const size_t s = blk * p.src_bytes + off, q = s >> 2;
    uint32_t v = src[q];
    const uint32_t own = p.src_bytes - off < 4u ? p.src_bytes - off : 4u;
    if ((s & 2u) != 0u) {
        v >>= 16;
        if (own > 2u) v |= src[q + 1] << 16;   // never reads past the last block's end
    }
    if (own < 4u) v &= (1u << (8u * own)) - 1u;
    dst[i] = v;
}

__device__ __forceinline__ uint32_t byte_at(const uint8_t* src, size_t i) { return src[i]; }
// Scale i (0..16) of a Q3_K block: low 4 bits from scale bytes 0..8, high 2 bits from 8..12.
__device__ __forceinline__ uint32_t scale3(const uint8_t* sb, uint32_t i) {
    const uint32_t k = i % 4, g = i / 4;
    const uint32_t low = (sb[4 * (g % 2) + k] >> (4 * (g / 2))) & 0xfu;
    const uint32_t high = (sb[8 + k] >> (2 * g)) & 3u;
    return low | (high << 4);
}
// One thread per 16-byte unit (32 weights): two words of 2-bit values, a word of high bits, the unit's two scales
// minus 32 as signed bytes, d.
__global__ void repack_q3_k_kernel(PRepackQ3K p, const uint8_t* __restrict__ src, uint4* __restrict__ dst) {
    const size_t unit = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (unit >= (size_t)p.blocks * 8) return;
    const uint8_t* b = src + (unit / 8) * 110;
    const uint32_t s = (uint32_t)(unit % 8), half = s / 4, j = s % 4;
    uint32_t l0 = 0, l1 = 0, hw = 0;
    for (uint32_t l = 0; l < 32; l++) {
        const uint32_t q = (b[32 + 32 * half + l] >> (2 * j)) & 3u;
        const uint32_t h = (b[l] >> (4 * half + j)) & 1u;
        const uint32_t e = l / 4, byte = l % 4;
        if (e < 4) l0 |= q << (8 * byte + 2 * e);
        else l1 |= q << (8 * byte + 2 * (e - 4));
        hw |= h << (8 * byte + e);
    }
    const uint32_t sc0 = (scale3(b + 96, 8 * half + 2 * j) + 224u) & 0xffu;
    const uint32_t sc1 = (scale3(b + 96, 8 * half + 2 * j + 1) + 224u) & 0xffu;
    const uint32_t d = b[108] | ((uint32_t)b[109] << 8);
    dst[unit] = make_uint4(l0, l1, hw, sc0 | (sc1 << 8) | (d << 16));
}

__device__ __forceinline__ float half_at(const uint8_t* p) { return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8)))); }

enum { E_Q3_K = 0, E_Q5_K = 1, E_Q6_K = 2, E_IQ4_XS = 3 };

// Element i (0..255) of one block. `b` points at the block: the file layout (and its padded form, which only adds
// bytes after it); Q3_K blocks may also be the repacked 128-byte form (`packed`).
template <int TYPE>
__device__ __forceinline__ float decode_elem(const uint8_t* b, uint32_t i, bool packed) {
    if (TYPE == E_Q6_K) {
        const uint32_t n = i / 128, r = i % 128, c = r / 32, l = r % 32;
        const float d = half_at(b + 208);
        const int sc = (int)(int8_t)b[192 + 8 * n + 2 * c + l / 16];
        const uint32_t lo = (b[64 * n + 32 * (c & 1) + l] >> (4 * (c >> 1))) & 0xFu;
        const uint32_t hi = (b[128 + 32 * n + l] >> (2 * c)) & 3u;
        return __fmul_rn(__fmul_rn(d, (float)sc), (float)((int)(lo | (hi << 4)) - 32));
    }
    if (TYPE == E_Q5_K) {
        const uint32_t j = i / 64, hi = (i % 64) / 32, l = i % 32, sidx = 2 * j + hi;
        const float d = half_at(b), mn = half_at(b + 2);
        const uint8_t* s = b + 4;
        uint32_t sc, m;
        if (sidx < 4) sc = s[sidx] & 63u, m = s[sidx + 4] & 63u;
        else sc = (s[sidx + 4] & 0xFu) | ((uint32_t)(s[sidx - 4] >> 6) << 4), m = (uint32_t)(s[sidx + 4] >> 4) | ((uint32_t)(s[sidx] >> 6) << 4);
        const uint32_t q = ((b[48 + 32 * j + l] >> (4 * hi)) & 0xFu) + (((b[16 + l] >> sidx) & 1u) ? 16u : 0u);
        return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(mn, (float)m));
    }
    if (TYPE == E_IQ4_XS) {
        const int values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
        const uint32_t group = i / 32, r = i % 32, jx = r % 16, hi = r / 16;
        const float d = half_at(b);
        const uint32_t scales_h = b[2] | ((uint32_t)b[3] << 8);
        const uint32_t low = (b[4 + group / 2] >> (4 * (group % 2))) & 15u, high = (scales_h >> (2 * group)) & 3u;
        const float dl = __fmul_rn(d, (float)((int)(low | (high << 4)) - 32));
        const uint32_t q = b[8 + 16 * group + jx];
        return __fmul_rn(dl, (float)values[hi ? (q >> 4) : (q & 15u)]);
    }
    // Q3_K
    const uint32_t s = i / 32, l = i % 32;
    if (packed) {
        const uint32_t* u = reinterpret_cast<const uint32_t*>(b + 16 * s);
        const uint32_t e = l / 4, byte = l % 4;
        const uint32_t q = ((e < 4 ? u[0] : u[1]) >> (8 * byte + 2 * (e & 3))) & 3u;
        const uint32_t h = (u[2] >> (8 * byte + e)) & 1u;
        const float d = __half2float(__ushort_as_half((unsigned short)(u[3] >> 16)));
        const int sc = (int)(int8_t)((u[3] >> (l < 16 ? 0 : 8)) & 0xffu);
        return __fmul_rn(__fmul_rn(d, (float)sc), (float)((int)q - (h ? 0 : 4)));
    }
    const uint32_t half = s / 4, j = s % 4;
    const uint32_t q = (b[32 + 32 * half + l] >> (2 * j)) & 3u;
    const uint32_t h = (b[l] >> (4 * half + j)) & 1u;
    const int sc = (int)scale3(b + 96, 8 * half + 2 * j + l / 16) - 32;
    return __fmul_rn(__fmul_rn(half_at(b + 108), (float)sc), (float)((int)q - (h ? 0 : 4)));
}

// grid (tokens), 256 threads: out[t] = table[tokens[t] - row0]. stride == 0: rows packed in the layout the multiplies
// read (block stride `gpu_block`); else rows `stride` bytes apart, as in the file (block stride `file_block`).
template <int TYPE>
__global__ void __launch_bounds__(256) embed_kquant_kernel(PEmbed p, const uint32_t* __restrict__ tokens, const uint8_t* __restrict__ w,
                                                          float* __restrict__ out, uint32_t gpu_block, uint32_t file_block) {
    const uint32_t t = blockIdx.x, tok = tokens[t];
    if (tok < p.row0 || tok >= p.row0 + p.chunk_rows) return;
    const bool file = p.stride != 0;
    const uint32_t bb = file ? file_block : gpu_block;
    const size_t row_bytes = file ? p.stride : (size_t)(p.dim / 256) * gpu_block;
    const uint8_t* row = w + (size_t)(tok - p.row0) * row_bytes;
    for (uint32_t i = threadIdx.x; i < p.dim; i += 256) out[(size_t)t * p.dim + i] = decode_elem<TYPE>(row + (size_t)(i / 256) * bb, i % 256, !file);
}

}  // namespace

// Bindings: src, dst (rw).
zcu_result launch_repad(const LaunchArgs& a) {
    PRepad p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 2, "repad: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.dst_bytes >= p.src_bytes && p.dst_bytes % 16 == 0 && p.src_bytes % 2 == 0 && p.src_bytes > 0, "repad: %u -> %u bytes per block",
             p.src_bytes, p.dst_bytes);
    ZCU_NEED(a, (uint64_t)p.blocks * p.src_bytes <= a.b[0].size && (uint64_t)p.blocks * p.dst_bytes <= a.b[1].size, "repad: %u blocks do not fit the bindings", p.blocks);
    const size_t total = (size_t)p.blocks * (p.dst_bytes / 4);
    if (total == 0) return ZCU_OK;
    repad_kernel<<<(unsigned)((total + 255) / 256), 256, 0, a.stream>>>(p, (const uint32_t*)a.b[0].ptr, (uint32_t*)a.b[1].ptr, total);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

zcu_result launch_repack_q3_k(const LaunchArgs& a) {
    PRepackQ3K p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 2, "repack_q3_k: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, (uint64_t)p.blocks * 110 <= a.b[0].size && (uint64_t)p.blocks * 128 <= a.b[1].size, "repack_q3_k: %u blocks do not fit the bindings", p.blocks);
    if (p.blocks == 0) return ZCU_OK;
    const size_t units = (size_t)p.blocks * 8;
    repack_q3_k_kernel<<<(unsigned)((units + 255) / 256), 256, 0, a.stream>>>(p, (const uint8_t*)a.b[0].ptr, (uint4*)a.b[1].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

// Bindings: tokens, w, out (rw).
zcu_result launch_embed_kquant(const LaunchArgs& a, uint32_t kernel) {
    PEmbed p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 3, "embed: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, p.dim % 256 == 0, "embed: dim = %u is not a multiple of 256", p.dim);
    const uint32_t m = a.grid[0];
    if (m == 0) return ZCU_OK;
    const uint32_t* tok = (const uint32_t*)a.b[0].ptr;
    const uint8_t* w = (const uint8_t*)a.b[1].ptr;
    float* out = (float*)a.b[2].ptr;
    switch (kernel) {
        case ZCU_K_EMBED_Q3_K: embed_kquant_kernel<E_Q3_K><<<m, 256, 0, a.stream>>>(p, tok, w, out, 128, 110); break;
        case ZCU_K_EMBED_Q5_K: embed_kquant_kernel<E_Q5_K><<<m, 256, 0, a.stream>>>(p, tok, w, out, 176, 176); break;
        case ZCU_K_EMBED_Q6_K: embed_kquant_kernel<E_Q6_K><<<m, 256, 0, a.stream>>>(p, tok, w, out, 224, 210); break;
        case ZCU_K_EMBED_IQ4_XS: embed_kquant_kernel<E_IQ4_XS><<<m, 256, 0, a.stream>>>(p, tok, w, out, 144, 136); break;
        default: return zcu_fail(a, ZCU_E_UNSUPPORTED_KERNEL, "embed: kernel %u is not built", kernel);
    }
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}
