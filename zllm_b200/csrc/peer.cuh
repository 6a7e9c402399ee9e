// Tensor-parallel exchange without a collective library: every rank keeps the vectors that all ranks read
// whole (the residual stream, the attention output, the FFN activations, the logits) in one "arena" that its
// peers have mapped (CUDA IPC over NVLink). A kernel that produces a slice of such a vector stores it into the
// arena of EVERY rank (its own included), and the last CTA of that kernel then publishes, on every rank, that
// rank's count for the exchange ("slot"). A kernel that reads the vector first waits until every rank's count for
// the slot has reached its own. No multicast: plain stores and loads on peer memory.
//
// Counts only grow (one per execution of the slot's producer on each rank, and all ranks run the same list),
// so nothing is reset between steps. Every wait is bounded in time; a rank that gives up sets the status word.
#pragma once

#include <cstdint>

constexpr int PEER_MAX = 8;
constexpr uint32_t PEER_MAGIC = 0x52454550u;  // "PEER"
constexpr uint32_t PEER_NONE = 0xffffffffu;

// Trails a kernel's own parameter block when the dispatch takes part in an exchange.
struct PPeer {
    uint32_t magic;      // PEER_MAGIC
    uint32_t wait_slot;  // wait for this exchange before reading inputs (PEER_NONE: none)
    uint32_t push_slot;  // store outputs to every rank and publish this exchange (PEER_NONE: none)
    uint32_t _pad;
};

struct PeerTable {
    int32_t rank, world;
    uint32_t slots, _pad;
    uint64_t base[PEER_MAX];   // every rank's arena as mapped here (base[rank] is the local one)
    uint64_t arena_bytes;
    uint64_t flags_off;        // arena offset of flags[slots][PEER_MAX] (u32): flags[s][r] = rank r's count
    uint32_t* counts;          // local: this rank's count per slot
    uint32_t* tickets;         // local: CTAs of the producing kernel that have finished, per slot; tickets[slots] is
                               // the abort word: set by the first wait that gives up, it ends every later wait at once
};

struct PeerUse {  // what one launch does with the table
    PeerTable t;
    uint32_t wait_slot, push_slot;
};

#ifdef __CUDACC__
namespace peer {

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;\n" : "=l"(t));
    return t;
}

// Every thread of the CTA calls it. Returns false (and sets *status) if a rank did not publish within 2 s.
__device__ __forceinline__ bool wait_slot(const PeerUse& u, int* status) {
    __shared__ int ok_flag;
    if (u.wait_slot == PEER_NONE) return true;
    if (threadIdx.x == 0) {
        int ok = 1;
        const uint32_t want = __ldcg(u.t.counts + u.wait_slot);  // this rank's own count: its producer ran before us
        const uint32_t* flags = reinterpret_cast<const uint32_t*>(u.t.base[u.t.rank] + u.t.flags_off) + (size_t)u.wait_slot * PEER_MAX;
        const unsigned long long t0 = now_ns();
        if (__ldcg(u.t.tickets + u.t.slots) != 0) ok = 0;  // an earlier wait of this context gave up
        for (int r = 0; r < u.t.world && ok; r++) {
            for (unsigned spins = 0;; spins++) {
                uint32_t seen;
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];\n" : "=r"(seen) : "l"(flags + r) : "memory");
                if ((int32_t)(seen - want) >= 0) break;
                if ((spins & 1023u) == 1023u && now_ns() - t0 > 2000000000ull) {
                    if (status) atomicExch(status, 5);
                    atomicExch(u.t.tickets + u.t.slots, 1u);
                    ok = 0;
                    break;
                }
            }
        }
        ok_flag = ok;
    }
    __syncthreads();
    return ok_flag != 0;
}

// Where element `offset_bytes` of the local arena lives in rank r's arena.
__device__ __forceinline__ float* remote(const PeerUse& u, const float* local, int r) {
    return reinterpret_cast<float*>(u.t.base[r] + (reinterpret_cast<uint64_t>(local) - u.t.base[u.t.rank]));
}

// Every thread of the CTA calls it after its last store of the exchange. The last CTA of the grid publishes.
__device__ __forceinline__ void publish(const PeerUse& u, unsigned ncta) {
    if (u.push_slot == PEER_NONE) return;
    __syncthreads();  // the CTA's peer stores happen before thread 0's fence (cumulative), which precedes the ticket
    if (threadIdx.x == 0) {
        __threadfence_system();
        const unsigned t = atomicAdd(u.t.tickets + u.push_slot, 1u);
        if (t == ncta - 1) {
            u.t.tickets[u.push_slot] = 0;
            __threadfence_system();
            const uint32_t count = u.t.counts[u.push_slot] + 1;
            u.t.counts[u.push_slot] = count;
            for (int r = 0; r < u.t.world; r++) {
                uint32_t* flag = reinterpret_cast<uint32_t*>(u.t.base[r] + u.t.flags_off) + (size_t)u.push_slot * PEER_MAX + u.t.rank;
                asm volatile("st.release.sys.global.u32 [%0], %1;\n" ::"l"(flag), "r"(count) : "memory");
            }
        }
    }
}

}  // namespace peer
#endif
