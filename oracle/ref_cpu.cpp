// TEST INFRASTRUCTURE, NOT PRODUCT CODE.
//
// CPU restatement of zllm's own CPU reference (its src/ref directory) for the
// decode/prefill hot path: GGUF block dequantisation, the panel matmul, the
// scalar operators, GQA attention over an f16-rounded cache, the Gated
// DeltaNet recurrence and a Llama-shaped decode layer built from them.
// The reference is Zig and cannot be compiled where this runs, so every
// function below follows the cited reference lines operation by operation.
//
// Only the parity tests, the smoke check and the bench's CPU-baseline leg may
// load this library. The CUDA library never links or calls it.
//
// Parity pins: the RMSNorm bit fixture (ref/ops.zig:139-168), the f16 RNE
// vectors (ref/qwen35.zig:565-578), the bf16/f16 decode values
// (ref/tensor.zig:192-209), the roundLikeLlama cases (ref/matmul.zig:382-419),
// the matmul-vs-naive cases (ref/matmul.zig:296-380) and the tiny attention
// cases (ref/dense.zig:282-382) are all checked in tests/. Q8_0/Q4_K block
// decoding has no known-answer vector in the reference tree (it is pinned
// there against ggml through a build that is not available); it is checked
// against fixtures made with the independent numpy decoders of the `gguf`
// Python package, bit for bit.
//
// Build: see oracle/Makefile (-ffp-contract=off: the reference's float mode
// is strict, a multiply and an add are never fused unless it says so).

#include <algorithm>
#include <atomic>
#include <cmath>
#include <condition_variable>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <mutex>
#include <thread>
#include <type_traits>
#include <vector>

#define REF_API extern "C" __attribute__((visibility("default")))

// GGUF tensor type ids (src/gguf/gguf.zig TensorType).
enum : int { T_F32 = 0, T_F16 = 1, T_Q8_0 = 8, T_Q3_K = 11, T_Q4_K = 12, T_Q5_K = 13, T_Q6_K = 14, T_IQ4_XS = 23, T_BF16 = 30 };

// ---------------------------------------------------------------- f16 / bf16

// IEEE binary16 -> binary32, exact (what Zig's `@as(f32, f16)` does).
static inline float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {
            // Subnormal: normalise.
            int shift = 0;
            while (!(man & 0x400u)) { man <<= 1; shift++; }
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - shift + 1) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

// binary32 -> binary16, round to nearest even (Zig's `@as(f16, @floatCast(v))`).
static inline uint16_t f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u | ((ax >> 13) & 0x3ffu) : 0));
    }
    if (ax >= 0x477ff000u) {  // >= 65520 rounds to inf
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) {  // <= 2^-25 rounds to zero (exactly 2^-25 ties to even = 0)
        return (uint16_t)sign;
    }
    int32_t e = (int32_t)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) {  // subnormal result
        shift = 13 + (-14 - e);
        base = 0;
    } else {
        shift = 13;
        base = (uint32_t)(e + 15) << 10;
        man &= 0x7fffffu;
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) q++;
    return (uint16_t)(sign | (base + q));  // a carry out of the mantissa bumps the exponent
}

REF_API float ref_f16_to_f32(uint16_t h) { return f16_to_f32(h); }
REF_API uint16_t ref_f32_to_f16(float f) { return f32_to_f16(f); }

static inline uint16_t rd16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

// ---------------------------------------------------------------- dequantise

// ref/tensor.zig:50-53 — block_q8_0: d (f16), qs[32] (i8); y = f32(q) * d.
static void q8_0_block(const uint8_t* b, float* y) {
    const float d = f16_to_f32(rd16(b));
    for (int i = 0; i < 32; i++) y[i] = (float)(int8_t)b[2 + i] * d;
}

// ref/tensor.zig:95-98 — 6-bit scale and min of sub-block j.
static inline void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* m) {
    if (j < 4) {
        *sc = q[j] & 63;
        *m = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        *m = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

// ref/tensor.zig:101-116 — block_q4_K: d, dmin (f16), scales[12], qs[128].
// d1 = d*sc and m1 = dmin*m are rounded to f32 first; each value is then a
// separate multiply and subtract.
static void q4_k_block(const uint8_t* b, float* y) {
    const float d = f16_to_f32(rd16(b));
    const float mn = f16_to_f32(rd16(b + 2));
    const uint8_t* scales = b + 4;
    for (int j = 0; j < 4; j++) {
        const uint8_t* q = b + 16 + 32 * j;
        uint8_t sc1, mm1, sc2, mm2;
        scale_min_k4(2 * j, scales, &sc1, &mm1);
        scale_min_k4(2 * j + 1, scales, &sc2, &mm2);
        const float d1 = d * (float)sc1;
        const float m1 = mn * (float)mm1;
        const float d2 = d * (float)sc2;
        const float m2 = mn * (float)mm2;
        for (int l = 0; l < 32; l++) y[64 * j + l] = d1 * (float)(q[l] & 0xF) - m1;
        for (int l = 0; l < 32; l++) y[64 * j + 32 + l] = d2 * (float)(q[l] >> 4) - m2;
    }
}

// ref/tensor.zig:54-93 — block_q3_K: hmask[32], qs[64], scales[12] (16 six-bit scales, packed), d (f16);
// y = (d * (scale - 32)) * (two bits - (4 unless the mask bit is set)).
static void q3_k_block(const uint8_t* b, float* y) {
    const uint8_t* hm = b;
    const float d_all = f16_to_f32(rd16(b + 108));
    uint32_t aux[4];
    for (int i = 0; i < 4; i++) aux[i] = i < 3 ? (uint32_t)(b[96 + 4 * i] | (b[97 + 4 * i] << 8) | (b[98 + 4 * i] << 16) | ((uint32_t)b[99 + 4 * i] << 24)) : 0;
    const uint32_t kmask1 = 0x03030303u, kmask2 = 0x0f0f0f0fu, tmp = aux[2];
    aux[2] = ((aux[0] >> 4) & kmask2) | (((tmp >> 4) & kmask1) << 4);
    aux[3] = ((aux[1] >> 4) & kmask2) | (((tmp >> 6) & kmask1) << 4);
    aux[0] = (aux[0] & kmask2) | (((tmp >> 0) & kmask1) << 4);
    aux[1] = (aux[1] & kmask2) | (((tmp >> 2) & kmask1) << 4);
    int8_t scales[16];
    memcpy(scales, aux, 16);
    size_t out = 0, is = 0;
    uint8_t m = 1;
    for (int n = 0; n < 2; n++) {
        const uint8_t* q = b + 32 + n * 32;
        int shift = 0;
        for (int r = 0; r < 4; r++) {
            for (int h = 0; h < 2; h++) {
                const float dl = d_all * (float)((int)scales[is++] - 32);
                for (int l = 0; l < 16; l++) {
                    const int lo = (q[l + 16 * h] >> shift) & 3;
                    const int v = lo - ((hm[l + 16 * h] & m) ? 0 : 4);
                    y[out++] = dl * (float)v;
                }
            }
            shift += 2;
            m = (uint8_t)(m << 1);
        }
    }
}

// ref/tensor.zig:118-137 — block_q5_K: d, dmin (f16), scales[12], qh[32] (fifth bits), qs[128].
static void q5_k_block(const uint8_t* b, float* y) {
    const float d = f16_to_f32(rd16(b));
    const float mn = f16_to_f32(rd16(b + 2));
    const uint8_t* scales = b + 4;
    const uint8_t* qh = b + 16;
    for (int j = 0; j < 4; j++) {
        const uint8_t* ql = b + 48 + 32 * j;
        const uint8_t bit_lo = (uint8_t)(1u << (2 * j)), bit_hi = (uint8_t)(2u << (2 * j));
        uint8_t sc1, mm1, sc2, mm2;
        scale_min_k4(2 * j, scales, &sc1, &mm1);
        scale_min_k4(2 * j + 1, scales, &sc2, &mm2);
        const float d1 = d * (float)sc1, m1 = mn * (float)mm1, d2 = d * (float)sc2, m2 = mn * (float)mm2;
        for (int l = 0; l < 32; l++) y[64 * j + l] = d1 * (float)((ql[l] & 0xF) + ((qh[l] & bit_lo) ? 16 : 0)) - m1;
        for (int l = 0; l < 32; l++) y[64 * j + 32 + l] = d2 * (float)((ql[l] >> 4) + ((qh[l] & bit_hi) ? 16 : 0)) - m2;
    }
}

// ref/tensor.zig:139-160 — block_q6_K: ql[128], qh[64], scales[16] (i8), d (f16); y = (d * sc) * (q - 32).
static void q6_k_block(const uint8_t* b, float* y) {
    const float d = f16_to_f32(rd16(b + 208));
    for (int n = 0; n < 2; n++) {
        const uint8_t* ql = b + 64 * n;
        const uint8_t* qh = b + 128 + 32 * n;
        const int8_t* sc = (const int8_t*)(b + 192 + 8 * n);
        float* out = y + 128 * n;
        for (int l = 0; l < 32; l++) {
            const int is = l / 16;
            const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
            const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            out[l] = d * (float)sc[is] * (float)q1;
            out[l + 32] = d * (float)sc[is + 2] * (float)q2;
            out[l + 64] = d * (float)sc[is + 4] * (float)q3;
            out[l + 96] = d * (float)sc[is + 6] * (float)q4;
        }
    }
}

// ref/tensor.zig:162-181 — block_iq4_xs: d (f16), scales_h (u16), scales_l[4], qs[128]; signed six-bit group
// scales biased by 32, nonlinear four-bit values (low nibbles precede high nibbles).
static void iq4_xs_block(const uint8_t* b, float* y) {
    static const int8_t values[16] = {-127, -104, -83, -65, -49, -35, -22, -10, 1, 13, 25, 38, 53, 69, 89, 113};
    const float d = f16_to_f32(rd16(b));
    const uint32_t scales_h = rd16(b + 2);
    for (int group = 0; group < 8; group++) {
        const uint32_t low = (b[4 + group / 2] >> (4 * (group % 2))) & 15u;
        const uint32_t high = (scales_h >> (2 * group)) & 3u;
        const float dl = d * (float)((int)(low | (high << 4)) - 32);
        const uint8_t* qs = b + 8 + 16 * group;
        for (int j = 0; j < 16; j++) {
            y[32 * group + j] = dl * (float)values[qs[j] & 15];
            y[32 * group + 16 + j] = dl * (float)values[qs[j] >> 4];
        }
    }
}

struct Layout { size_t block_elems, block_bytes; };
static bool layout_of(int t, Layout* l) {
    switch (t) {
        case T_F32: *l = {1, 4}; return true;
        case T_F16: *l = {1, 2}; return true;
        case T_BF16: *l = {1, 2}; return true;
        case T_Q8_0: *l = {32, 34}; return true;
        case T_Q4_K: *l = {256, 144}; return true;
        case T_Q3_K: *l = {256, 110}; return true;
        case T_Q5_K: *l = {256, 176}; return true;
        case T_Q6_K: *l = {256, 210}; return true;
        case T_IQ4_XS: *l = {256, 136}; return true;
        default: return false;
    }
}

// ref/tensor.zig:21-43 — one f32 per element; returns 0, or -1 for a type
// outside this path (error.UnsupportedTensorType).
REF_API int ref_dequantize(int type, const uint8_t* bytes, float* out, size_t n) {
    switch (type) {
        case T_Q8_0:
            for (size_t i = 0; i < n / 32; i++) q8_0_block(bytes + i * 34, out + i * 32);
            return 0;
        case T_Q4_K:
            for (size_t i = 0; i < n / 256; i++) q4_k_block(bytes + i * 144, out + i * 256);
            return 0;
        case T_Q3_K:
            for (size_t i = 0; i < n / 256; i++) q3_k_block(bytes + i * 110, out + i * 256);
            return 0;
        case T_Q5_K:
            for (size_t i = 0; i < n / 256; i++) q5_k_block(bytes + i * 176, out + i * 256);
            return 0;
        case T_Q6_K:
            for (size_t i = 0; i < n / 256; i++) q6_k_block(bytes + i * 210, out + i * 256);
            return 0;
        case T_IQ4_XS:
            for (size_t i = 0; i < n / 256; i++) iq4_xs_block(bytes + i * 136, out + i * 256);
            return 0;
        case T_F32:
            memcpy(out, bytes, n * 4);
            return 0;
        case T_F16:
            for (size_t i = 0; i < n; i++) out[i] = f16_to_f32(rd16(bytes + 2 * i));
            return 0;
        case T_BF16:
            for (size_t i = 0; i < n; i++) {
                uint32_t b = (uint32_t)rd16(bytes + 2 * i) << 16;
                memcpy(out + i, &b, 4);
            }
            return 0;
        default:
            return -1;
    }
}

// ---------------------------------------------------------------- operators

static const int VEC = 16;  // ref/ops.zig:8 — the reference's vector length

// ref/ops.zig:11-23 — 16 partial sums, reduced lane by lane, then the tail.
static float dot(const float* a, const float* b, size_t n) {
    float acc[VEC] = {0};
    size_t i = 0;
    for (; i + VEC <= n; i += VEC)
        for (int l = 0; l < VEC; l++) acc[l] += a[i + l] * b[i + l];
    float sum = acc[0];
    for (int l = 1; l < VEC; l++) sum += acc[l];
    for (; i < n; i++) sum += a[i] * b[i];
    return sum;
}
REF_API float ref_dot(const float* a, const float* b, size_t n) { return dot(a, b, n); }

// ref/ops.zig:30-41 — f32 squares summed in f64, f32 mean, f32 1/sqrt,
// x * scale * w left to right.
static void rms_norm(float* x, const float* w, size_t n, float eps) {
    double sum = 0;
    for (size_t i = 0; i < n; i++) {
        const float sq = x[i] * x[i];
        sum += sq;
    }
    const float mean = (float)(sum / (double)n);
    const float scale = 1.0f / sqrtf(mean + eps);
    for (size_t i = 0; i < n; i++) x[i] = x[i] * scale * w[i];
}
REF_API void ref_rms_norm(float* x, const float* w, size_t n, float eps) { rms_norm(x, w, n, eps); }

// ref/ops.zig:44-47
static void l2_norm(float* x, size_t n, float eps) {
    const float scale = 1.0f / sqrtf(dot(x, x, n) + eps);
    for (size_t i = 0; i < n; i++) x[i] *= scale;
}
REF_API void ref_l2_norm(float* x, size_t n, float eps) { l2_norm(x, n, eps); }

// ref/ops.zig:49-60
static inline float silu(float x) { return x / (1.0f + expf(-x)); }
static inline float sigmoid(float x) { return 1.0f / (1.0f + expf(-x)); }
static inline float softplus(float x) { return x > 20 ? x : logf(1.0f + expf(x)); }
REF_API float ref_silu(float x) { return silu(x); }
REF_API float ref_sigmoid(float x) { return sigmoid(x); }
REF_API float ref_softplus(float x) { return softplus(x); }

// ref/ops.zig:95-99 — theta = pos * base^(-2i/n_rot) / factor, all f32.
static inline void rope_cos_sin(uint32_t pos, size_t i, size_t n_rot, float base, float factor, float* cs) {
    const float exponent = -2.0f * (float)i / (float)n_rot;
    const float theta = (float)pos * powf(base, exponent) / factor;
    cs[0] = cosf(theta);
    cs[1] = sinf(theta);
}
REF_API void ref_rope_cos_sin(uint32_t pos, size_t i, size_t n_rot, float base, float factor, float* cs) {
    rope_cos_sin(pos, i, n_rot, base, factor, cs);
}

// ref/ops.zig:64-73 — NeoX pairs (i, i + n_rot/2).
static void rope_neox(float* x, uint32_t pos, size_t n_rot, float base) {
    const size_t half = n_rot / 2;
    for (size_t i = 0; i < half; i++) {
        float cs[2];
        rope_cos_sin(pos, i, n_rot, base, 1.0f, cs);
        const float x0 = x[i], x1 = x[i + half];
        x[i] = x0 * cs[0] - x1 * cs[1];
        x[i + half] = x0 * cs[1] + x1 * cs[0];
    }
}
REF_API void ref_rope(float* x, uint32_t pos, size_t n_rot, float base) { rope_neox(x, pos, n_rot, base); }

// ref/ops.zig:78-86 — normal pairs (2i, 2i+1), optional per-pair divisors.
static void rope_normal(float* x, uint32_t pos, size_t n_rot, float base, const float* factors) {
    for (size_t i = 0; i < n_rot / 2; i++) {
        float cs[2];
        rope_cos_sin(pos, i, n_rot, base, factors ? factors[i] : 1.0f, cs);
        const float x0 = x[2 * i], x1 = x[2 * i + 1];
        x[2 * i] = x0 * cs[0] - x1 * cs[1];
        x[2 * i + 1] = x0 * cs[1] + x1 * cs[0];
    }
}
REF_API void ref_rope_normal(float* x, uint32_t pos, size_t n_rot, float base, const float* factors) {
    rope_normal(x, pos, n_rot, base, factors);
}

// src/kernels/kernels.zig:730-744 — (cos, sin) at (pos * n_rot/2 + i) * 2.
REF_API void ref_rope_table(float* table, size_t positions, size_t n_rot, float base, const float* factors) {
    const size_t half = n_rot / 2;
    for (size_t pos = 0; pos < positions; pos++)
        for (size_t i = 0; i < half; i++)
            rope_cos_sin((uint32_t)pos, i, n_rot, base, factors ? factors[i] : 1.0f, table + (pos * half + i) * 2);
}

// ref/ops.zig:102-111
REF_API void ref_softmax(float* x, size_t n) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; i++) mx = std::max(mx, x[i]);
    float sum = 0;
    for (size_t i = 0; i < n; i++) {
        x[i] = expf(x[i] - mx);
        sum += x[i];
    }
    for (size_t i = 0; i < n; i++) x[i] /= sum;
}

// ---------------------------------------------------------------- rounding

// ref/matmul.zig:203-258 — activations as ggml's x86 CPU backend rounds them
// for a dot product with weights of type `type`, back to f32.
REF_API void ref_round_like_llama(int type, float* x, size_t n) {
    switch (type) {
        case T_Q8_0:
            for (size_t b = 0; b + 32 <= n; b += 32) {
                float* blk = x + b;
                float amax = 0;
                for (int i = 0; i < 32; i++) amax = std::max(amax, fabsf(blk[i]));
                const float d = amax / 127;
                const float id = amax != 0 ? 127 / amax : 0;
                const float d16 = f16_to_f32(f32_to_f16(d));
                for (int i = 0; i < 32; i++) {
                    const float t = blk[i] * id + 12582912.0f;
                    int32_t bits;
                    memcpy(&bits, &t, 4);
                    const int8_t q = (int8_t)(bits - 0x4b400000);
                    blk[i] = (float)q * d16;
                }
            }
            break;
        case T_Q4_K:
            for (size_t b = 0; b + 256 <= n; b += 256) {
                float* blk = x + b;
                float amax = 0, mx = 0;
                for (int i = 0; i < 256; i++)
                    if (fabsf(blk[i]) > amax) {
                        amax = fabsf(blk[i]);
                        mx = blk[i];
                    }
                if (amax == 0) {
                    memset(blk, 0, 256 * 4);
                    continue;
                }
                const float iscale = -127.0f / mx;
                const float d = 1 / iscale;
                for (int i = 0; i < 256; i++) {
                    const float t = iscale * blk[i] + 12582912.0f;
                    int32_t bits;
                    memcpy(&bits, &t, 4);
                    blk[i] = (float)std::min(127, bits - 0x4b400000) * d;
                }
            }
            break;
        case T_F16:
            for (size_t i = 0; i < n; i++) x[i] = f16_to_f32(f32_to_f16(x[i]));
            break;
        case T_BF16:
            for (size_t i = 0; i < n; i++) {
                uint32_t bits;
                memcpy(&bits, x + i, 4);
                uint32_t r = bits + (0x7fffu + ((bits >> 16) & 1u));
                r &= 0xffff0000u;
                memcpy(x + i, &r, 4);
            }
            break;
        default:
            break;
    }
}

// ---------------------------------------------------------------- pool

// ref/pool.zig:76-122 — a persistent fork-join pool: contiguous ranges, the
// caller runs the range after the workers'. (Workers here sleep on a condition
// variable after a short spin; the reference spins then waits on a futex.)
struct Pool {
    std::vector<std::thread> workers;
    std::mutex mu;
    std::condition_variable cv;
    std::atomic<uint32_t> generation{0};
    std::atomic<int> pending{0};
    bool stop = false;
    std::function<void(size_t, size_t)> func;
    size_t n = 0, chunk = 0;

    explicit Pool(size_t threads) {
        for (size_t i = 0; i + 1 < threads; i++) workers.emplace_back([this, i] { worker(i); });
    }
    ~Pool() {
        {
            std::lock_guard<std::mutex> g(mu);
            stop = true;
            generation.fetch_add(1);
        }
        cv.notify_all();
        for (auto& t : workers) t.join();
    }
    size_t thread_count() const { return workers.size() + 1; }

    void run_range(size_t index) {
        const size_t first = index * chunk;
        if (first >= n) return;
        func(first, std::min(n, first + chunk));
    }
    void worker(size_t index) {
        uint32_t seen = 0;
        for (;;) {
            int spins = 0;
            while (generation.load(std::memory_order_acquire) == seen && spins < 20000) spins++;
            if (generation.load(std::memory_order_acquire) == seen) {
                std::unique_lock<std::mutex> lk(mu);
                cv.wait(lk, [&] { return generation.load() != seen; });
            }
            seen = generation.load(std::memory_order_acquire);
            if (stop) return;
            run_range(index);
            pending.fetch_sub(1, std::memory_order_acq_rel);
        }
    }
    // parts = max(1, min(threads, n / max(1, min_chunk))); chunk = ceil(n / parts)
    // rounded up to align_to (ref/pool.zig:94-95).
    void parallel_for(size_t count, size_t align_to, size_t min_chunk, std::function<void(size_t, size_t)> f) {
        const size_t parts = std::max<size_t>(1, std::min(thread_count(), count / std::max<size_t>(1, min_chunk)));
        size_t ch = (count + parts - 1) / parts;
        ch = (ch + align_to - 1) / align_to * align_to;
        if (parts == 1 || workers.empty()) {
            f(0, count);
            return;
        }
        func = std::move(f);
        n = count;
        chunk = ch;
        pending.store((int)workers.size());
        {
            std::lock_guard<std::mutex> g(mu);
            generation.fetch_add(1);
        }
        cv.notify_all();
        run_range(workers.size());
        while (pending.load(std::memory_order_acquire) != 0) std::this_thread::yield();
    }
};

REF_API Pool* ref_pool_create(size_t threads) { return new Pool(std::max<size_t>(1, threads)); }
REF_API void ref_pool_destroy(Pool* p) { delete p; }
REF_API size_t ref_pool_threads(const Pool* p) { return p->thread_count(); }

// ---------------------------------------------------------------- matmul

static const size_t PANEL = 32;      // ref/matmul.zig:28 — output rows per panel
static const size_t BLOCK_ROWS = 8;  // ref/matmul.zig:30 — tokens per microkernel call

// ref/matmul.zig:111-133 — rows [p*32, p*32+32) decoded k-major, rows past n zero.
static void pack_panel(int type, const uint8_t* bytes, size_t n, size_t k, size_t p, float* dst) {
    Layout l;
    layout_of(type, &l);
    const size_t row_bytes = k / l.block_elems * l.block_bytes;
    const size_t chunk = 256;
    float buf[256];
    for (size_t col = 0; col < PANEL; col++) {
        const size_t j = p * PANEL + col;
        if (j >= n) {
            for (size_t i = 0; i < k; i++) dst[i * PANEL + col] = 0;
            continue;
        }
        const uint8_t* src = bytes + j * row_bytes;
        for (size_t start = 0; start < k; start += chunk) {
            const size_t len = std::min(chunk, k - start);
            const size_t b0 = start / l.block_elems * l.block_bytes;
            ref_dequantize(type, src + b0, buf, len);
            for (size_t i = 0; i < len; i++) dst[(start + i) * PANEL + col] = buf[i];
        }
    }
}

// ref/matmul.zig:37-107 — f32/f16/bf16 matrices are packed into panels once;
// quantised ones keep their bytes and decode a panel on every use.
struct Matrix {
    std::vector<float> data;
    size_t n = 0, k = 0;
    int type = T_F32;
    const uint8_t* quant = nullptr;
    size_t panels() const { return (n + PANEL - 1) / PANEL; }
};

REF_API Matrix* ref_matrix_create(Pool* pool, int type, const uint8_t* bytes, size_t n, size_t k) {
    Layout l;
    if (!layout_of(type, &l) || k % l.block_elems != 0) return nullptr;
    Matrix* m = new Matrix();
    m->n = n;
    m->k = k;
    m->type = type;
    if (l.block_elems > 1) {  // every block-quantised type is decoded panel by panel as it is used
        m->quant = bytes;  // must outlive the matrix
        return m;
    }
    m->data.resize(m->panels() * PANEL * k);
    pool->parallel_for(m->panels(), 1, 1, [&](size_t first, size_t last) {
        for (size_t p = first; p < last; p++) pack_panel(type, bytes, n, k, p, m->data.data() + p * PANEL * k);
    });
    return m;
}
REF_API void ref_matrix_destroy(Matrix* m) { delete m; }

// ref/matmul.zig:93-106 — row j of the matrix as f32.
REF_API void ref_matrix_row(const Matrix* m, size_t j, float* out) {
    if (m->quant) {
        Layout l;
        layout_of(m->type, &l);
        const size_t row_bytes = m->k / l.block_elems * l.block_bytes;
        ref_dequantize(m->type, m->quant + j * row_bytes, out, m->k);
        return;
    }
    const float* base = m->data.data() + (j / PANEL) * PANEL * m->k + j % PANEL;
    for (size_t i = 0; i < m->k; i++) out[i] = base[i * PANEL];
}

// Accumulation modes. 0 is the reference's: every output is one f32
// accumulator that takes x*w (rounded) then an add (rounded), in i order
// (ref/matmul.zig:270-280). 1 fuses them (in case the published binaries
// were built with contraction). 2 accumulates in f64: the "truth" the
// reference's GPU kernel check compares against (src/kernels/check.zig:1033-1046).
enum : int { ACC_MUL_ADD = 0, ACC_FMA = 1, ACC_F64 = 2 };

template <int MODE>
static void microkernel(size_t R, const float* const* xp, const float* wp, size_t k, float* const* outp, size_t cols) {
    if (MODE == ACC_F64) {
        double acc[BLOCK_ROWS][PANEL] = {};
        for (size_t i = 0; i < k; i++) {
            const float* w = wp + i * PANEL;
            for (size_t a = 0; a < R; a++) {
                const double xb = xp[a][i];
                for (size_t c = 0; c < PANEL; c++) acc[a][c] += xb * (double)w[c];
            }
        }
        for (size_t a = 0; a < R; a++)
            for (size_t c = 0; c < cols; c++) outp[a][c] = (float)acc[a][c];
        return;
    }
    float acc[BLOCK_ROWS][PANEL] = {};
    for (size_t i = 0; i < k; i++) {
        const float* w = wp + i * PANEL;
        for (size_t a = 0; a < R; a++) {
            const float xb = xp[a][i];
            if (MODE == ACC_FMA) {
                for (size_t c = 0; c < PANEL; c++) acc[a][c] = __builtin_fmaf(xb, w[c], acc[a][c]);
            } else {
                for (size_t c = 0; c < PANEL; c++) acc[a][c] += xb * w[c];
            }
        }
    }
    for (size_t a = 0; a < R; a++)
        for (size_t c = 0; c < cols; c++) outp[a][c] = acc[a][c];
}

// ref/matmul.zig:160-195 — out[t][j] = sum_i x[t][i] * w[j][i]; panels split
// over the pool, each thread decoding quantised panels into its own buffer,
// tokens in blocks of 8. `act` != 0 rounds the input like llama.cpp first.
REF_API void ref_matmul(Pool* pool, float* out, const float* x_in, const Matrix* w, size_t rows, int act, int mode) {
    const size_t k = w->k, n = w->n;
    std::vector<float> rounded;
    const float* x = x_in;
    if (act) {
        rounded.assign(x_in, x_in + rows * k);
        for (size_t r = 0; r < rows; r++) ref_round_like_llama(w->type, rounded.data() + r * k, k);
        x = rounded.data();
    }
    pool->parallel_for(w->panels(), 1, 1, [&](size_t first, size_t last) {
        static thread_local std::vector<float> panel_buf;
        for (size_t p = first; p < last; p++) {
            const float* wp;
            if (w->quant) {
                if (panel_buf.size() < PANEL * k) panel_buf.resize(PANEL * k);
                pack_panel(w->type, w->quant, n, k, p, panel_buf.data());
                wp = panel_buf.data();
            } else {
                wp = w->data.data() + p * PANEL * k;
            }
            const size_t j0 = p * PANEL;
            const size_t cols = std::min(PANEL, n - j0);
            for (size_t t = 0; t < rows; t += BLOCK_ROWS) {
                const size_t R = std::min(BLOCK_ROWS, rows - t);
                const float* xp[BLOCK_ROWS];
                float* op[BLOCK_ROWS];
                for (size_t a = 0; a < R; a++) {
                    xp[a] = x + (t + a) * k;
                    op[a] = out + (t + a) * n + j0;
                }
                if (mode == ACC_FMA) microkernel<ACC_FMA>(R, xp, wp, k, op, cols);
                else if (mode == ACC_F64) microkernel<ACC_F64>(R, xp, wp, k, op, cols);
                else microkernel<ACC_MUL_ADD>(R, xp, wp, k, op, cols);
            }
        }
    });
}

// ---------------------------------------------------------------- attention

// ref/dense.zig:252-274 (`attend`) for ONE query token at position
// `keys - 1` over a cache of `keys` positions: per head, pass 1 takes the max
// of q.k*scale, pass 2 sums p = exp(s - max) and o += p*v, then o /= sum.
// The cache holds binary16 bits laid out pos*(kv_heads*hd) + g*hd + d, i.e.
// values already rounded at the cache boundary (ref/qwen35.zig:32-42).
// `gate` (or null): per-head sigmoid output gate, ref/qwen35.zig:413.
REF_API void ref_attend_decode(Pool* pool, float* out, const float* q, size_t q_head_stride, const uint16_t* kc,
                               const uint16_t* vc, size_t keys, size_t heads, size_t kv_heads, size_t hd, float scale,
                               const float* gate, size_t gate_stride) {
    const size_t group = heads / kv_heads;
    const size_t kv_stride = kv_heads * hd;
    pool->parallel_for(heads, 1, 1, [&](size_t first, size_t last) {
        std::vector<float> kf(hd), vf(hd);
        for (size_t hh = first; hh < last; hh++) {
            const size_t kvh = hh / group;
            const float* qh = q + hh * q_head_stride;
            float mx = -INFINITY;
            for (size_t j = 0; j < keys; j++) {
                const uint16_t* kr = kc + j * kv_stride + kvh * hd;
                for (size_t d = 0; d < hd; d++) kf[d] = f16_to_f32(kr[d]);
                mx = std::max(mx, dot(qh, kf.data(), hd) * scale);
            }
            float* o = out + hh * hd;
            for (size_t d = 0; d < hd; d++) o[d] = 0;
            float sum = 0;
            for (size_t j = 0; j < keys; j++) {
                const uint16_t* kr = kc + j * kv_stride + kvh * hd;
                const uint16_t* vr = vc + j * kv_stride + kvh * hd;
                for (size_t d = 0; d < hd; d++) kf[d] = f16_to_f32(kr[d]);
                const float p = expf(dot(qh, kf.data(), hd) * scale - mx);
                sum += p;
                for (size_t d = 0; d < hd; d++) o[d] += p * f16_to_f32(vr[d]);
            }
            if (gate) {
                const float* g = gate + hh * gate_stride;
                for (size_t d = 0; d < hd; d++) o[d] = o[d] / sum * sigmoid(g[d]);
            } else {
                for (size_t d = 0; d < hd; d++) o[d] /= sum;
            }
        }
    });
}

// ---------------------------------------------------------------- DeltaNet

// ref/qwen35.zig:464-481 (`convNorm`) — causal depthwise conv over the fused
// q|k|v projection (taps per channel, zero history before token 0) + SiLU,
// then L2-normalise each q and k head.
REF_API void ref_conv_norm(float* conv, const float* qkv, const float* taps_w, size_t n, size_t k_heads, size_t inner,
                           size_t d, size_t kernel, float eps) {
    const size_t key_dim = d * k_heads;
    const size_t cd = 2 * key_dim + inner;
    for (size_t t = 0; t < n; t++) {
        float* row = conv + t * cd;
        for (size_t ch = 0; ch < cd; ch++) {
            float sum = 0;
            for (size_t tap = 0; tap < kernel; tap++) {
                const size_t back = kernel - 1 - tap;
                if (t >= back) sum += taps_w[ch * kernel + tap] * qkv[(t - back) * cd + ch];
            }
            row[ch] = silu(sum);
        }
        for (size_t i = 0; i < 2 * k_heads; i++) l2_norm(row + i * d, d, eps);
    }
}

// ref/qwen35.zig:493-546 (`recurHead`) without the trailing norm/gate: for
// value head j over n tokens, on state s[a*D + b] (a key row, b value column):
//   x = s*decay (stored), stk += x*k[a]        (first pass, a ascending)
//   delta = (v - stk) * beta
//   x = s + k[a]*delta (stored), o += x*q[a]   (second pass)
//   out = o * (1/sqrt(D))
// Each product and each sum is rounded on its own, as the reference's vector
// code does. mode 2 keeps the state and sums in f64 (the check's truth,
// src/kernels/check.zig:2018-2050).
template <typename F>
static void recur_head(float* state_f32, float* out, const float* conv, const float* g, const float* beta, size_t n,
                       size_t j, size_t hk, size_t hv, size_t D) {
    const size_t key_dim = D * hk;
    const size_t cd = 2 * key_dim + hv * D;
    const float scale = 1.0f / sqrtf((float)D);
    std::vector<F> s(D * D);
    for (size_t i = 0; i < D * D; i++) s[i] = state_f32[i];
    std::vector<F> stk(D), delta(D), o(D);
    for (size_t t = 0; t < n; t++) {
        const float* row = conv + t * cd;
        const float* q = row + (j % hk) * D;
        const float* kk = row + key_dim + (j % hk) * D;
        const float* v = row + 2 * key_dim + j * D;
        const F decay = std::is_same<F, float>::value ? (F)expf(g[t * hv + j]) : (F)exp((double)g[t * hv + j]);
        const F b = beta[t * hv + j];
        std::fill(stk.begin(), stk.end(), (F)0);
        for (size_t a = 0; a < D; a++) {
            const F ka = kk[a];
            F* p = s.data() + a * D;
            for (size_t i = 0; i < D; i++) {
                const F x = p[i] * decay;
                p[i] = x;
                stk[i] += x * ka;
            }
        }
        for (size_t i = 0; i < D; i++) delta[i] = ((F)v[i] - stk[i]) * b;
        std::fill(o.begin(), o.end(), (F)0);
        for (size_t a = 0; a < D; a++) {
            const F ka = kk[a], qa = q[a];
            F* p = s.data() + a * D;
            for (size_t i = 0; i < D; i++) {
                const F x = p[i] + ka * delta[i];
                p[i] = x;
                o[i] += x * qa;
            }
        }
        float* oh = out + t * hv * D + j * D;
        for (size_t i = 0; i < D; i++) oh[i] = (float)(o[i] * (F)scale);
    }
    for (size_t i = 0; i < D * D; i++) state_f32[i] = (float)s[i];
}

// All value heads, split over the pool as the reference does (one head per task).
REF_API void ref_delta_rule(Pool* pool, float* state, float* out, const float* conv, const float* g, const float* beta,
                            size_t n, size_t k_heads, size_t v_heads, size_t d, int mode) {
    pool->parallel_for(v_heads, 1, 1, [&](size_t first, size_t last) {
        for (size_t j = first; j < last; j++) {
            if (mode == ACC_F64) recur_head<double>(state + j * d * d, out, conv, g, beta, n, j, k_heads, v_heads, d);
            else recur_head<float>(state + j * d * d, out, conv, g, beta, n, j, k_heads, v_heads, d);
        }
    });
}

// ref/qwen35.zig:543-545 — per head: rmsNorm(o, norm_w) then o *= silu(z).
REF_API void ref_gated_norm(float* o, const float* z, const float* norm_w, size_t n, size_t v_heads, size_t d,
                            float eps) {
    for (size_t t = 0; t < n; t++)
        for (size_t j = 0; j < v_heads; j++) {
            float* oh = o + (t * v_heads + j) * d;
            const float* zz = z + (t * v_heads + j) * d;
            rms_norm(oh, norm_w, d, eps);
            for (size_t i = 0; i < d; i++) oh[i] *= silu(zz[i]);
        }
}

// ---------------------------------------------------------------- dense layer

// One Llama-shaped layer for ONE new token at position `pos` of one sequence,
// restating ref/dense.zig:134-146 (layer body), :201-280 (attention with
// normal RoPE, K/V rounded to f16 at the cache boundary) and :179-197 (SwiGLU
// FFN) on an existing cache instead of teacher-forcing from an empty state.
struct DenseLayer {
    const float* attn_norm;
    const Matrix *wq, *wk, *wv, *wo;
    const float* ffn_norm;
    const Matrix *gate, *up, *down;
};

REF_API void ref_dense_decode_layer(Pool* pool, const DenseLayer* L, float* x, uint16_t* kc, uint16_t* vc,
                                    uint32_t pos, size_t e, size_t heads, size_t kv_heads, size_t hd, size_t ff,
                                    float eps, float rope_base, float attn_scale, int mode) {
    std::vector<float> h(e), q(heads * hd), k(kv_heads * hd), v(kv_heads * hd), attn(heads * hd), mix(e);
    // normRows: h = rmsnorm(x) * attn_norm
    h.assign(x, x + e);
    rms_norm(h.data(), L->attn_norm, e, eps);
    ref_matmul(pool, q.data(), h.data(), L->wq, 1, 0, mode);
    ref_matmul(pool, k.data(), h.data(), L->wk, 1, 0, mode);
    ref_matmul(pool, v.data(), h.data(), L->wv, 1, 0, mode);
    for (size_t hh = 0; hh < heads; hh++) rope_normal(q.data() + hh * hd, pos, hd, rope_base, nullptr);
    const size_t kv_stride = kv_heads * hd;
    for (size_t g = 0; g < kv_heads; g++) {
        rope_normal(k.data() + g * hd, pos, hd, rope_base, nullptr);
        for (size_t d = 0; d < hd; d++) {
            kc[pos * kv_stride + g * hd + d] = f32_to_f16(k[g * hd + d]);
            vc[pos * kv_stride + g * hd + d] = f32_to_f16(v[g * hd + d]);
        }
    }
    ref_attend_decode(pool, attn.data(), q.data(), hd, kc, vc, (size_t)pos + 1, heads, kv_heads, hd, attn_scale, nullptr, 0);
    ref_matmul(pool, mix.data(), attn.data(), L->wo, 1, 0, mode);
    for (size_t i = 0; i < e; i++) x[i] += mix[i];
    // FFN
    h.assign(x, x + e);
    rms_norm(h.data(), L->ffn_norm, e, eps);
    std::vector<float> gt(ff), upv(ff);
    ref_matmul(pool, gt.data(), h.data(), L->gate, 1, 0, mode);
    ref_matmul(pool, upv.data(), h.data(), L->up, 1, 0, mode);
    for (size_t i = 0; i < ff; i++) gt[i] = silu(gt[i]) * upv[i];
    ref_matmul(pool, mix.data(), gt.data(), L->down, 1, 0, mode);
    for (size_t i = 0; i < e; i++) x[i] += mix[i];
}

// ref/dense.zig:148-156 — final norm then the LM head.
REF_API void ref_dense_head(Pool* pool, float* logits, const float* x, const float* out_norm, const Matrix* head,
                            size_t e, float eps, int mode) {
    std::vector<float> h(x, x + e);
    rms_norm(h.data(), out_norm, e, eps);
    ref_matmul(pool, logits, h.data(), head, 1, 0, mode);
}

REF_API const char* ref_build_info() {
    return
#if defined(__AVX512F__)
        "avx512"
#elif defined(__AVX2__)
        "avx2"
#else
        "baseline"
#endif
        ;
}
