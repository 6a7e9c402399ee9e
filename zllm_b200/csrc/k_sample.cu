// The sampler (src/kernels/sample.wgsl, semantics src/sampler/sampler.zig:1-16): one token from a row of logits
// with vLLM's order of operations - logit bias; repetition, frequency and presence penalties; greedy argmax (first
// index on ties); else temperature, min-p, top-k, top-p (ties at a threshold all kept) and an inverse-CDF draw in
// token order at the step's u. Plus its two small companions, mark_tokens and draft.
//
// The reference runs a draw as a sequence of up to 78 dispatches (kernels.sampleSteps: prep, reduce, four
// histogram/digit rounds, gather/final or 32 bisection rounds, mass, pick), passing values through the state
// buffer. Here the whole draw is ONE cooperative launch, issued for the sequence's first phase (prep); the other
// phases of the sequence are accepted and launch nothing, so a host that dispatches the reference's sequence gets
// the same results in the same places: the token in st[0], its stop flag in st[1], next[0] = token, counts[token]
// bumped, and `work` holding the processed logits. Phase unbump undoes the count as in the reference.
//
// One CTA per SM (at most one per 1024 tokens), 512 threads; every thread keeps its tokens' processed logits in
// registers for the whole draw, so the vocabulary is read once. The CTAs meet at a grid barrier (bounded; a
// cooperative launch makes them co-resident) after each global reduction:
//   1        the maximum and its first index: one 64-bit atomicMax of (key << 32 | ~index)
//   top-k    radix select on the order-preserving key, 8 bits a round: counts per digit (shared-memory histogram,
//            then integer atomics into the round's own global histogram), 4 barriers; skipped when min-p leaves
//            at most k tokens
//   top-p    the same select on MASS: a token stays while the mass ranked above it is < p, so the threshold is the
//            lowest key whose mass above is < p z; found digit by digit from per-digit masses, 4 barriers
//   draw     each CTA's kept mass, a barrier, then the CTA that holds u z scans its tokens in order
// A token's mass is exp(l - max) in 64-bit fixed point (43 fractional bits): integer sums do not depend on the
// order of the additions, so every CTA computes the same thresholds from the same histograms and a draw is
// reproducible bit for bit, and the CDF is finer than an f32 accumulation (the reference's check allows 1e-6 of
// the mass for that, src/kernels/check.zig:2123-2127).

#include "zcu_internal.h"

namespace {

constexpr int ST = 512;                  // threads per CTA
constexpr int PER_MAX = 8;               // tokens per thread
constexpr int GROUP = 1024;              // tokens per group of the reference's dispatch (kernels.sample_span)
constexpr uint32_t NONE = 0xffffffffu;
constexpr float LOWEST = -3.402823466e+38f;
constexpr float MASS_ONE = 8796093022208.f;   // 2^43

enum : uint32_t { PH_PREP = 0, PH_UNBUMP = 11, PH_COUNT = 12 };

struct PSample {  // kernels.zig:635-650
    uint32_t vocab, n_bias, n_stop, greedy;
    float temperature;
    uint32_t top_k;
    float top_p, min_p, repetition, presence, frequency;
    uint32_t n_prompt;
    uint32_t stops[16];
};
static_assert(sizeof(PSample) == 112, "Sample");
struct PSamplePhase {
    uint32_t phase, round, _pad[2];
};
struct PDraft {
    uint32_t vocab, row, slot, _pad;
};

// The draw's global scratch (zeroed before the launch): the barrier, the abort flag, the maximum, one histogram
// per select round, every CTA's kept mass.
constexpr int ROUNDS = 8, MAX_CTAS = 256;
struct Scratch {
    unsigned int arrived;
    unsigned int abort_flag;
    unsigned long long top;                       // key << 32 | ~index of the maximum
    unsigned int count[ROUNDS][256];
    unsigned long long mass[ROUNDS][256];
    unsigned long long part[MAX_CTAS];
};

__device__ __forceinline__ uint32_t key_of(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b >> 31) ? ~b : (b ^ 0x80000000u);
}
__device__ __forceinline__ float unkey(uint32_t k) { return __uint_as_float((k >> 31) ? (k ^ 0x80000000u) : ~k); }

// (found, bias) of token i in the list sorted by token.
__device__ __forceinline__ bool bias_of(const uint2* __restrict__ bias, uint32_t n, uint32_t i, float& out) {
    uint32_t lo = 0, hi = n;
    while (lo < hi) {
        const uint32_t mid = (lo + hi) / 2;
        const uint2 b = bias[mid];
        if (b.x == i) {
            out = __uint_as_float(b.y);
            return true;
        }
        if (b.x < i) lo = mid + 1;
        else hi = mid;
    }
    return false;
}

// Every CTA arrives, then waits until all `k` * gridDim.x arrivals of the draw's first k barriers are in. False
// when the wait ran out (two seconds) or another CTA gave up.
__device__ __forceinline__ bool grid_barrier(Scratch* s, unsigned k, bool* sh_ok) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(&s->arrived, 1u);
        const unsigned want = k * gridDim.x;
        const long long t0 = clock64();
        bool ok = true;
        unsigned spins = 0;
        for (;;) {
            unsigned got;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];\n" : "=r"(got) : "l"(&s->arrived) : "memory");
            if (got >= want) break;
            if ((++spins & 255u) == 0) {
                unsigned ab;
                asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];\n" : "=r"(ab) : "l"(&s->abort_flag) : "memory");
                if (ab != 0 || clock64() - t0 > 4000000000ll) {
                    atomicExch(&s->abort_flag, 1u);
                    ok = false;
                    break;
                }
            }
        }
        *sh_ok = ok;
    }
    __syncthreads();
    return *sh_ok;
}

struct Shared {
    unsigned int cnt[256];
    unsigned long long mass[256];
    unsigned long long warp_sum[32];
    unsigned long long pk[32];
    unsigned int prefix, left, skip, dstar;
    unsigned long long above;
    unsigned long long zq;
    bool ok;
};

__device__ __forceinline__ unsigned long long warp_sum_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ unsigned long long warp_max_u64(unsigned long long v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const unsigned long long w = __shfl_xor_sync(0xffffffffu, v, o);
        v = w > v ? w : v;
    }
    return v;
}

__device__ void finish(const PSample& p, uint32_t token, uint32_t* st, uint32_t* next, uint32_t* counts) {
    uint32_t stop = 0;
    for (uint32_t i = 0; i < p.n_stop && i < 16; i++)
        if (p.stops[i] == token) stop = 1;
    st[0] = token;
    st[1] = stop;
    next[0] = token;
    counts[token] += 1u;
}

// Adds the CTA's shared histogram of one round into the round's global one (nonzero bins only).
__device__ __forceinline__ void publish(Shared& sh, Scratch* s, int round, bool with_mass) {
    __syncthreads();
    const int t = threadIdx.x;
    if (t < 256) {
        if (sh.cnt[t]) atomicAdd(&s->count[round][t], sh.cnt[t]);
        if (with_mass && sh.mass[t]) atomicAdd(&s->mass[round][t], sh.mass[t]);
    }
}
__device__ __forceinline__ void fetch(Shared& sh, Scratch* s, int round, bool with_mass) {
    const int t = threadIdx.x;
    if (t < 256) {
        sh.cnt[t] = __ldcg(&s->count[round][t]);
        if (with_mass) sh.mass[t] = __ldcg(&s->mass[round][t]);
    }
    __syncthreads();
}

__global__ void __launch_bounds__(ST, 1)
    sample_kernel(const float* __restrict__ logits, const uint2* __restrict__ bias, const uint32_t* __restrict__ prompt_mask,
                  uint32_t* __restrict__ counts, float* __restrict__ work, uint32_t* __restrict__ st, uint32_t* __restrict__ next,
                  const PStep* __restrict__ step, const PSample* __restrict__ params, Scratch* __restrict__ s, int per,
                  uint32_t vocab_cap, int* __restrict__ status) {
    __shared__ Shared sh;
    __shared__ PSample p;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid < (int)(sizeof(PSample) / 4)) reinterpret_cast<uint32_t*>(&p)[tid] = reinterpret_cast<const uint32_t*>(params)[tid];
    __syncthreads();
    const uint32_t vocab = p.vocab < vocab_cap ? p.vocab : vocab_cap;   // never past what the launch covers
    const uint32_t base = blockIdx.x * (uint32_t)per * ST;
    unsigned nbar = 0;

    // ---- bias, penalties, temperature; the maximum and its first index
    float v[PER_MAX];
    unsigned long long best = 0;
#pragma unroll
    for (int j = 0; j < PER_MAX; j++) {
        v[j] = LOWEST;
        const uint32_t i = base + (uint32_t)j * ST + tid;
        if (j < per && i < vocab) {
            float x = logits[i];
            float b;
            if (p.n_bias > 0 && bias_of(bias, p.n_bias, i, b)) x = __fadd_rn(x, b);
            const uint32_t n = counts[i];
            if (prompt_mask[i] != 0u || n != 0u) x = x > 0.0f ? __fdiv_rn(x, p.repetition) : __fmul_rn(x, p.repetition);
            x = __fsub_rn(x, __fmul_rn(p.frequency, (float)n));
            x = __fsub_rn(x, __fmul_rn(p.presence, n != 0u ? 1.0f : 0.0f));
            if (p.greedy == 0u) x = __fdiv_rn(x, p.temperature);
            work[i] = x;
            v[j] = x;
            const unsigned long long pk = ((unsigned long long)key_of(x) << 32) | (unsigned long long)(NONE - i);
            best = pk > best ? pk : best;
        }
    }
    best = warp_max_u64(best);
    if (lane == 0) sh.pk[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = warp_max_u64(lane < ST / 32 ? sh.pk[lane] : 0ull);
        if (lane == 0) atomicMax(&s->top, best);
    }
    if (!grid_barrier(s, ++nbar, &sh.ok)) {
        if (tid == 0 && status) atomicExch(status, 1);
        return;
    }
    const unsigned long long top_pk = __ldcg(&s->top);
    const float t = unkey((uint32_t)(top_pk >> 32));
    const uint32_t argmax = NONE - (uint32_t)(top_pk & 0xffffffffu);
    if (p.greedy != 0u) {
        if (blockIdx.x == 0 && tid == 0) finish(p, argmax, st, next, counts);
        return;
    }

    // ---- min-p; every token's key and mass
    uint32_t key[PER_MAX];
    unsigned long long q[PER_MAX];
    bool kept[PER_MAX];
#pragma unroll
    for (int j = 0; j < PER_MAX; j++) {
        const uint32_t i = base + (uint32_t)j * ST + tid;
        const bool valid = j < per && i < vocab;
        const float e = valid ? expf(v[j] - t) : 0.0f;
        key[j] = key_of(v[j]);
        kept[j] = valid && (p.min_p <= 0.0f || e >= p.min_p);
        q[j] = kept[j] ? __float2ull_rz(e * MASS_ONE) : 0ull;
    }
    int round = 0;
    bool failed = false;

    // ---- top-k: the k-th largest key among the survivors, 8 bits a round
    if (p.top_k > 0u) {
        uint32_t prefix = 0, left = p.top_k;
        bool skip = false;
        for (int r = 0; r < 4 && !skip; r++, round++) {
            if (tid < 256) sh.cnt[tid] = 0;
            __syncthreads();
#pragma unroll
            for (int j = 0; j < PER_MAX; j++)
                if (kept[j] && (r == 0 || (key[j] >> (32 - 8 * r)) == prefix)) atomicAdd(&sh.cnt[(key[j] >> (24 - 8 * r)) & 255u], 1u);
            publish(sh, s, round, false);
            if (!grid_barrier(s, ++nbar, &sh.ok)) {
                failed = true;
                break;
            }
            fetch(sh, s, round, false);
            if (tid == 0) {
                uint32_t total = 0;
                if (r == 0)
                    for (int d = 0; d < 256; d++) total += sh.cnt[d];
                if (r == 0 && total <= left) {
                    sh.skip = 1;   // at most k tokens survive min-p: top-k removes nothing
                } else {
                    uint32_t above = 0;
                    int d = 255;
                    for (;;) {
                        const uint32_t c = sh.cnt[d];
                        if (above + c >= left || d == 0) break;
                        above += c;
                        d--;
                    }
                    sh.skip = 0;
                    sh.prefix = (prefix << 8) | (uint32_t)d;
                    sh.left = left - above;
                }
            }
            __syncthreads();
            skip = sh.skip != 0;
            if (!skip) prefix = sh.prefix, left = sh.left;
            __syncthreads();
        }
        if (!failed) {
            if (skip) round = 4;   // the rounds not run keep their slots
            else {
#pragma unroll
                for (int j = 0; j < PER_MAX; j++)
                    if (key[j] < prefix) kept[j] = false, q[j] = 0ull;
            }
        }
        round = 4;
    }

    // ---- top-p: the lowest key whose mass ranked above is < p z
    if (!failed && p.top_p < 1.0f) {
        uint32_t prefix = 0;
        unsigned long long above0 = 0;
        round = 4;
        for (int r = 0; r < 4; r++, round++) {
            if (tid < 256) sh.cnt[tid] = 0, sh.mass[tid] = 0ull;
            __syncthreads();
#pragma unroll
            for (int j = 0; j < PER_MAX; j++)
                if (kept[j] && (r == 0 || (key[j] >> (32 - 8 * r)) == prefix)) {
                    const uint32_t d = (key[j] >> (24 - 8 * r)) & 255u;
                    atomicAdd(&sh.cnt[d], 1u);
                    if (q[j]) atomicAdd(&sh.mass[d], q[j]);
                }
            publish(sh, s, round, true);
            if (!grid_barrier(s, ++nbar, &sh.ok)) {
                failed = true;
                break;
            }
            fetch(sh, s, round, true);
            if (tid == 0) {
                if (r == 0) {
                    unsigned long long z = 0;
                    for (int d = 0; d < 256; d++) z += sh.mass[d];
                    sh.zq = z;
                }
                const double g = (double)p.top_p * (double)sh.zq;
                unsigned long long above = above0, at_star = above0;
                uint32_t dstar = 0;
                for (int d = 255; d >= 0; d--) {
                    if (sh.cnt[d] == 0) continue;
                    if ((double)above >= g) break;
                    dstar = (uint32_t)d;
                    at_star = above;
                    above += sh.mass[d];
                }
                sh.dstar = dstar;
                sh.above = at_star;
            }
            __syncthreads();
            prefix = (prefix << 8) | sh.dstar;
            above0 = sh.above;
            __syncthreads();
        }
        if (!failed) {
#pragma unroll
            for (int j = 0; j < PER_MAX; j++)
                if (key[j] < prefix) kept[j] = false, q[j] = 0ull;
        }
    }
    if (failed) {
        if (tid == 0 && status) atomicExch(status, 1);
        return;
    }

    // ---- the draw: every CTA's kept mass, then the CTA that holds u z walks its tokens in order
    unsigned long long mine = 0;
#pragma unroll
    for (int j = 0; j < PER_MAX; j++) mine += q[j];
    mine = warp_sum_u64(mine);
    if (lane == 0) sh.warp_sum[warp] = mine;
    __syncthreads();
    if (tid == 0) {
        unsigned long long tot = 0;
        for (int w = 0; w < ST / 32; w++) tot += sh.warp_sum[w];
        s->part[blockIdx.x] = tot;
    }
    if (!grid_barrier(s, ++nbar, &sh.ok)) {
        if (tid == 0 && status) atomicExch(status, 1);
        return;
    }
    if (tid == 0) {
        unsigned long long z = 0;
        for (unsigned g = 0; g < gridDim.x; g++) z += __ldcg(&s->part[g]);
        unsigned long long at = (unsigned long long)((double)step->u * (double)z);
        if (at >= z) at = z - 1;                    // u < 1, z > 0 (the maximum's own mass)
        unsigned long long before = 0;
        unsigned target = 0;
        for (unsigned g = 0; g < gridDim.x; g++) {
            const unsigned long long m = __ldcg(&s->part[g]);
            if (before + m > at) {
                target = g;
                break;
            }
            before += m;
        }
        sh.dstar = target;
        sh.above = at - before;                    // the position inside the target CTA's mass
    }
    __syncthreads();
    if (sh.dstar != blockIdx.x) return;
    unsigned long long rel = sh.above;
    __syncthreads();
    for (int j = 0; j < per; j++) {   // token order: slab j holds tokens base + j * 1024 + tid
        unsigned long long mq = 0;
#pragma unroll
        for (int jj = 0; jj < PER_MAX; jj++)
            if (jj == j) mq = q[jj];
        // inclusive scan over the slab
        unsigned long long inc = mq;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long n = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += n;
        }
        if (lane == 31) sh.warp_sum[warp] = inc;
        __syncthreads();
        unsigned long long before = 0, slab = 0;
        for (int w = 0; w < ST / 32; w++) {
            const unsigned long long ws = sh.warp_sum[w];
            if (w < warp) before += ws;
            slab += ws;
        }
        inc += before;
        if (rel < slab) {
            if (mq != 0 && inc - mq <= rel && rel < inc) finish(p, base + (uint32_t)j * ST + tid, st, next, counts);
            return;
        }
        rel -= slab;
        __syncthreads();
    }
}

__global__ void unbump_kernel(const uint32_t* __restrict__ st, uint32_t* __restrict__ counts, const PSample* __restrict__ params) {
    const uint32_t token = st[0];
    if (token < params->vocab && counts[token] > 0) counts[token] -= 1u;
}

// mark_tokens (src/kernels/mark_tokens.wgsl): mask[tokens[i]] = 1 for i < n_prompt.
__global__ void mark_tokens_kernel(PSample p, const uint32_t* __restrict__ tokens, uint32_t* __restrict__ mask) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < p.n_prompt) {
        const uint32_t t = tokens[i];
        if (t < p.vocab) mask[t] = 1u;
    }
}

// draft (src/kernels/draft.wgsl): the first index of the maximum of one row of logits, to out[slot].
__global__ void __launch_bounds__(1024) draft_kernel(PDraft p, const float* __restrict__ logits, uint32_t* __restrict__ out) {
    __shared__ unsigned long long pk[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    unsigned long long best = 0;
    for (uint32_t i = tid; i < p.vocab; i += 1024) {
        const unsigned long long k = ((unsigned long long)key_of(logits[(size_t)p.row + i]) << 32) | (unsigned long long)(NONE - i);
        best = k > best ? k : best;
    }
    best = warp_max_u64(best);
    if (lane == 0) pk[warp] = best;
    __syncthreads();
    if (warp == 0) {
        best = warp_max_u64(pk[lane]);
        if (lane == 0) out[p.slot] = p.vocab ? NONE - (uint32_t)(best & 0xffffffffu) : NONE;
    }
}

}  // namespace

// Bindings: logits, bias, prompt_mask, counts (rw), work (rw), st (rw), next (rw), step, params (the Sample block).
zcu_result launch_sample(const LaunchArgs& a) {
    PSamplePhase ph;
    ZCU_NEED(a, a.params_bytes >= sizeof(ph) && a.nb >= 9, "sample: bad parameter block or bindings");
    memcpy(&ph, a.params, sizeof(ph));
    ZCU_NEED(a, ph.phase < PH_COUNT, "sample: phase %u", ph.phase);
    ZCU_NEED(a, a.b[8].size >= sizeof(PSample) && a.b[7].size >= sizeof(PStep) && a.b[5].size >= 8 && a.b[6].size >= 4,
             "sample: a binding is too small");
    const PSample* params = (const PSample*)a.b[8].ptr;
    if (ph.phase == PH_UNBUMP) {
        unbump_kernel<<<1, 1, 0, a.stream>>>((const uint32_t*)a.b[5].ptr, (uint32_t*)a.b[3].ptr, params);
        ZCU_CHECK_LAUNCH(a);
        return ZCU_OK;
    }
    if (ph.phase != PH_PREP) return ZCU_OK;   // the draw was made by the sequence's first dispatch
    // prep runs one group per 1024 tokens (kernels.sampleGroups): that bounds the vocabulary
    const uint64_t cover = (uint64_t)a.grid[0] * GROUP;
    const uint64_t in_bytes = a.b[0].size < a.b[4].size ? a.b[0].size : a.b[4].size;
    ZCU_NEED(a, a.grid[0] > 0 && cover / 4 <= in_bytes && in_bytes / 4 >= 1, "sample: %u groups for %llu bytes of logits", a.grid[0],
             (unsigned long long)in_bytes);
    uint32_t vocab_cap = (uint32_t)(cover < in_bytes / 4 ? cover : in_bytes / 4);
    const uint64_t small = a.b[2].size < a.b[3].size ? a.b[2].size : a.b[3].size;
    if (small / 4 < vocab_cap) vocab_cap = (uint32_t)(small / 4);
    const int sms = a.sm_count > 0 ? a.sm_count : 148;
    const int ctas = (int)a.grid[0] < sms ? (int)a.grid[0] : (sms < MAX_CTAS ? sms : MAX_CTAS);
    int per = (((int)a.grid[0] + ctas - 1) / ctas) * (GROUP / ST);   // slabs of ST tokens per CTA
    ZCU_NEED(a, per <= PER_MAX, "sample: a vocabulary of %u x 1024 tokens is past this kernel's %d per thread on %d CTAs", a.grid[0], PER_MAX, ctas);
    ZCU_NEED(a, a.scratch != nullptr && a.scratch_bytes >= sizeof(Scratch), "sample: the context has no scratch");
    Scratch* s = (Scratch*)a.scratch;
    if (cudaMemsetAsync(s, 0, sizeof(Scratch), a.stream) != cudaSuccess) {
        cudaGetLastError();
        ZCU_NEED(a, false, "sample: could not clear the draw's scratch");
    }
    const float* logits = (const float*)a.b[0].ptr;
    const uint2* bias = (const uint2*)a.b[1].ptr;
    const uint32_t* mask = (const uint32_t*)a.b[2].ptr;
    uint32_t* counts = (uint32_t*)a.b[3].ptr;
    float* work = (float*)a.b[4].ptr;
    uint32_t* st = (uint32_t*)a.b[5].ptr;
    uint32_t* next = (uint32_t*)a.b[6].ptr;
    const PStep* step = (const PStep*)a.b[7].ptr;
    int* status = a.status;
    void* args[] = {&logits, &bias, &mask, &counts, &work, &st, &next, &step, &params, &s, &per, &vocab_cap, &status};
    // cooperative: every CTA is resident before any starts, which the grid barrier needs
    const cudaError_t e = cudaLaunchCooperativeKernel((const void*)sample_kernel, dim3(ctas), dim3(ST), args, 0, a.stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        ZCU_NEED(a, false, "sample: cooperative launch of %d CTAs failed: %s", ctas, cudaGetErrorString(e));
    }
    return ZCU_OK;
}

// Bindings: tokens, mask (rw). Parameter block: the Sample block.
zcu_result launch_mark_tokens(const LaunchArgs& a) {
    PSample p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 2, "mark_tokens: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, (uint64_t)p.n_prompt * 4 <= a.b[0].size, "mark_tokens: %u tokens in %llu bytes", p.n_prompt, (unsigned long long)a.b[0].size);
    if ((uint64_t)p.vocab * 4 > a.b[1].size) p.vocab = (uint32_t)(a.b[1].size / 4);
    if (p.n_prompt == 0) return ZCU_OK;
    mark_tokens_kernel<<<(p.n_prompt + 255) / 256, 256, 0, a.stream>>>(p, (const uint32_t*)a.b[0].ptr, (uint32_t*)a.b[1].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}

// Bindings: logits, out (rw).
zcu_result launch_draft(const LaunchArgs& a) {
    PDraft p;
    ZCU_NEED(a, a.params_bytes >= sizeof(p) && a.nb >= 2, "draft: bad parameter block or bindings");
    memcpy(&p, a.params, sizeof(p));
    ZCU_NEED(a, ((uint64_t)p.row + p.vocab) * 4 <= a.b[0].size && ((uint64_t)p.slot + 1) * 4 <= a.b[1].size, "draft: row %u + %u or slot %u out of range",
             p.row, p.vocab, p.slot);
    draft_kernel<<<1, 1024, 0, a.stream>>>(p, (const float*)a.b[0].ptr, (uint32_t*)a.b[1].ptr);
    ZCU_CHECK_LAUNCH(a);
    return ZCU_OK;
}
