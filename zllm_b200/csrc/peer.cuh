// Tensor-parallel exchange without a collective library and without fences: every rank keeps the vectors that
// all ranks read whole (the residual stream, the attention output, the FFN activations, the logits) in one
// "arena" that its peers have mapped (CUDA IPC over NVLink). Beside each float of the arena's data region there is
// an 8-byte slot {value bits, tag} in its exchange region (at ll_off + 2 * offset). A kernel that produces a slice
// of such a vector stores {value, tag} into the slot of EVERY rank (its own included) with one 8-byte store; a
// kernel that reads the vector reads the slots and waits, element by element, until the tag is the one it
// expects. An 8-byte store arrives whole, so a matching tag proves its value: no flag, no fence, no round trip -
// the data is its own signal (the idea of NCCL's low-latency protocol). No multicast: plain stores and loads.
//
// Tags: a run of the launch list is an epoch; exchange `slot` uses tag epoch * slots + slot + 1 in it. A buffer that
// several exchanges of a step write in turn (the residual stream) therefore never shows the same tag twice, and
// tags are never 0 (the arena starts zeroed). The epoch is one local word that every kernel of the list reads
// at its start and that only the list's closing dispatch (ZCU_K_EXT_PEER_NEXT, ordered after everything before it)
// advances: producer and consumer of a slot agree on its tag without telling each other anything, and there is no
// per-kernel counting. Every
// rank runs the same list, so the epochs of all ranks agree. A slot is written at most once per epoch.
// A fast rank cannot overwrite a slot that a slow rank still has to read: to reach the next write of a buffer it
// must have read, through the exchanges in between, data that the slow rank produces only after that read.
// Every wait is bounded in time (2 s unless the host sets another limit); a rank that gives up sets the context's
// status word and an abort word that ends every later wait at once.
#pragma once

#include <cstdint>

constexpr int PEER_MAX = 8;
constexpr uint32_t PEER_MAGIC = 0x52454550u;  // "PEER"
constexpr uint32_t PEER_NONE = 0xffffffffu;

// Trails a kernel's own parameter block when the dispatch takes part in an exchange.
struct PPeer {
    uint32_t magic;      // PEER_MAGIC
    uint32_t wait_slot;  // the input vector comes from this exchange (PEER_NONE: it is local)
    uint32_t push_slot;  // outputs go to every rank as this exchange (PEER_NONE: local only)
    uint32_t _pad;
};

struct PeerTable {
    int32_t rank, world;
    uint32_t slots;
    uint32_t wait_ms;          // how long a wait for a slot may last before it gives up (0: 2000)
    uint64_t base[PEER_MAX];   // every rank's arena as mapped here (base[rank] is the local one)
    uint64_t arena_bytes;
    uint64_t ll_off;           // arena offset of the exchange region: the float at offset q has its slot at ll_off + 2 q
    uint32_t* epoch;           // local: epoch[0] = runs of the launch list so far; epoch[1] = the abort word
};

struct PeerUse {  // what one launch does with the table
    PeerTable t;
    uint32_t wait_slot, push_slot;
    uint32_t _pad[2];
};

#ifdef __CUDACC__
namespace peer {

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}

// The tag of `slot` in this run of the list (read once, at the kernel's start).
__device__ __forceinline__ uint32_t tag_of(const PeerUse& u, uint32_t slot) { return __ldcg(u.t.epoch) * u.t.slots + slot + 1; }
__device__ __forceinline__ uint32_t want_tag(const PeerUse& u) { return tag_of(u, u.wait_slot); }
__device__ __forceinline__ uint32_t push_tag(const PeerUse& u) { return tag_of(u, u.push_slot); }

// The exchange slot of the float at `local` (an address inside the local arena's data region), in rank r's arena.
__device__ __forceinline__ uint2* slot_of(const PeerUse& u, const float* local, int r) {
    const uint64_t q = reinterpret_cast<uint64_t>(local) - u.t.base[u.t.rank];
    return reinterpret_cast<uint2*>(u.t.base[r] + u.t.ll_off + 2 * q);
}

// One output of an exchange: its slot on every rank.
__device__ __forceinline__ void push(const PeerUse& u, const float* local, float v, uint32_t tag) {
    for (int r = 0; r < u.t.world; r++) {
        uint2* s = slot_of(u, local, r);
        if (r == u.t.rank) asm volatile("st.relaxed.gpu.global.v2.u32 [%0], {%1, %2};\n" ::"l"(s), "r"(__float_as_uint(v)), "r"(tag) : "memory");
        else asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};\n" ::"l"(s), "r"(__float_as_uint(v)), "r"(tag) : "memory");
    }
}

__device__ __forceinline__ bool gave_up(const PeerUse& u, unsigned long long t0, unsigned spins, int* status) {
    if ((spins & 1023u) != 1023u) return false;
    if (__ldcg(u.t.epoch + 1) != 0) return true;  // another wait of this context gave up
    if (now_ns() - t0 > (unsigned long long)(u.t.wait_ms ? u.t.wait_ms : 2000u) * 1000000ull) {
        if (status) atomicExch(status, 5);
        atomicExch(u.t.epoch + 1, 1u);
        return true;
    }
    return false;
}

// Four consecutive floats of an exchanged vector (`local` is 16-byte aligned): waits until all four slots carry `tag`.
// (out of line: a kernel that reads many pieces calls it only for a piece whose tags were not there at first look)
static __device__ __noinline__ float4 read4(const PeerUse& u, const float* local, uint32_t tag, int* status) {
    const uint2* s = slot_of(u, local, u.t.rank);
    uint4 a, b;
    unsigned long long t0 = 0;   // the clock is read only once a first look has failed
    for (unsigned spins = 0;; spins++) {
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(s) : "memory");
        asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(s + 2) : "memory");
        if (a.y == tag && a.w == tag && b.y == tag && b.w == tag) break;
        if (spins == 0) t0 = now_ns();
        if (gave_up(u, t0, spins, status)) break;
        if (spins >= 32) __nanosleep(64u);   // (a long wait does not poll back to back)
    }
    return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
}

// The same in two steps, for a reader that wants several pieces in flight at once: look4 only issues the two loads;
// take4 checks the tags and, where one is missing, falls back to read4's loop.
__device__ __forceinline__ void look4(const PeerUse& u, const float* local, uint4& a, uint4& b) {
    const uint2* s = slot_of(u, local, u.t.rank);
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(a.x), "=r"(a.y), "=r"(a.z), "=r"(a.w) : "l"(s) : "memory");
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(b.x), "=r"(b.y), "=r"(b.z), "=r"(b.w) : "l"(s + 2) : "memory");
}
__device__ __forceinline__ float4 take4(const PeerUse& u, const float* local, uint32_t tag, const uint4& a, const uint4& b, int* status) {
    if (a.y == tag && a.w == tag && b.y == tag && b.w == tag)
        return make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
    return read4(u, local, tag, status);
}

__device__ __forceinline__ float read1(const PeerUse& u, const float* local, uint32_t tag, int* status) {
    const uint2* s = slot_of(u, local, u.t.rank);
    uint2 a;
    unsigned long long t0 = 0;
    for (unsigned spins = 0;; spins++) {
        asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];\n" : "=r"(a.x), "=r"(a.y) : "l"(s) : "memory");
        if (a.y == tag) break;
        if (spins == 0) t0 = now_ns();
        if (gave_up(u, t0, spins, status)) break;
        if (spins >= 32) __nanosleep(64u);
    }
    return __uint_as_float(a.x);
}

}  // namespace peer
#endif
