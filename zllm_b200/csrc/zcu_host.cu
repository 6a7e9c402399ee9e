// The host side of libzllm_cuda: contexts, buffers, the command-stream
// interpreter and the dispatch table. Semantics follow the reference's native
// host (src/agility/host.zig:293-607): write_buffer / write_file are staged
// and land before all work of the next submit; ops between submits run in
// recorded order (one in-order CUDA stream gives that without hazard
// tracking); submit blocks until the device has finished, then fills the
// read destinations and reports one completion per read and one for itself;
// a dispatch of a pipeline created with an empty artifact fails the batch
// with UnsupportedKernel and drops the submission in progress.

#include <chrono>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <thread>
#include <vector>

#include "zcu_internal.h"

#define ZCU_EXPORT extern "C" __attribute__((visibility("default")))

namespace {

constexpr uint32_t USAGE_UNIFORM = 1u << 6;  // cmd.Usage.uniform (src/gpu/cmd.zig:62-75)

struct Buffer {
    uint8_t* ptr = nullptr;  // device memory, or host memory in a dry run
    uint64_t size = 0;
    uint32_t usage = 0;
    std::vector<uint8_t> shadow;  // host copy of uniform buffers (parameter pages, Step)
    bool shadow_stale = false;
    bool live = false;
};
struct Pipeline {
    uint32_t kernel = 0, variant = 0, writes = 0;
    bool missing = false, live = false;
};
struct GroupEntry {
    uint32_t binding, buffer;
    uint64_t offset, size;
};
struct Group {
    uint32_t pipeline = 0;
    std::vector<GroupEntry> entries;
    bool live = false;
};
struct Write {
    uint32_t buffer;
    uint64_t offset;
    size_t start, len;        // write_buffer: a copy of the caller's bytes in write_data (they may be gone by the submit)
    const uint8_t* file_src;  // write_file: the bytes where they lie in the mapped file (nothing is copied until the submit)
};
enum OpKind { OP_DISPATCH, OP_COPY, OP_FILL, OP_READ };
struct Op {
    OpKind kind;
    uint32_t pipeline = 0, group = 0, has_group = 0;
    uint32_t grid[3] = {0, 0, 0};
    uint32_t src = 0, dst = 0;
    uint64_t src_off = 0, dst_off = 0, size = 0;
    void* host_dst = nullptr;
};
struct Read {
    uint32_t token;
};
struct TimingKey {
    uint32_t kernel, variant, grid[3];
    bool operator<(const TimingKey& o) const { return memcmp(this, &o, sizeof(*this)) < 0; }
};
struct TimingVal {
    uint32_t count = 0;
    double total_us = 0;
};

}  // namespace

struct zcu_context {
    int device = 0;
    bool dry = false, lost = false, own_stream = false;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    char err[1024] = {0};
    std::vector<Buffer> buffers;
    std::vector<Pipeline> pipelines;
    std::vector<Group> groups;
    std::vector<Write> writes;
    std::vector<uint8_t> write_data;
    std::vector<Op> ops;
    std::vector<Read> reads;
    std::vector<uint32_t> released;
    const uint8_t* file = nullptr;
    uint64_t file_len = 0;
    bool profiling = false;
    std::map<TimingKey, TimingVal> timings;
    uint64_t launches = 0;
    bool capturing = false;
    std::vector<cudaGraphExec_t> graphs;
    PeerTable peers = {};                 // tensor-parallel exchange (world == 0: not configured)
    std::vector<void*> ipc_open;          // peer arenas this context mapped
    std::vector<void*> retired;           // epoch words of earlier peer configurations
    uint8_t* pinned = nullptr;  // staging for readbacks
    // uploads go through a small ring of pinned chunks: the payload is copied once (mapping or write_data -> chunk)
    // and the chunk is handed to the copy engine; a chunk is reused once its copy has finished
    static constexpr int UP_CHUNKS = 2;
    static constexpr size_t UP_CHUNK_BYTES = (size_t)32 << 20;
    uint8_t* up_chunk[UP_CHUNKS] = {nullptr, nullptr};
    cudaEvent_t up_done[UP_CHUNKS] = {nullptr, nullptr};
    int up_next = 0;
    bool unfinished = false;    // a wait timed out: work may still be in flight and may still read the pinned memory
    int* status = nullptr;      // mapped host word kernels set when a bounded wait gives up
    void* scratch = nullptr;    // device scratch of the multiplies that stage their inputs (k_quant_tc.cu): work of one stream, used in order
    size_t scratch_bytes = 0;
    size_t pinned_cap = 0;
};

namespace {

zcu_result fail(zcu_context* c, zcu_result r, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(c->err, sizeof(c->err), fmt, ap);
    va_end(ap);
    return r;
}

#define CU(c, call)                                                                               \
    do {                                                                                          \
        cudaError_t e__ = (call);                                                                 \
        if (e__ != cudaSuccess) return fail(c, ZCU_E_GPU, "%s: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

inline uint64_t join64(uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; }

template <typename T>
zcu_result put(zcu_context* c, std::vector<T>& v, uint32_t id, T&& item) {
    if (id > (1u << 24)) return fail(c, ZCU_E_BAD_ID, "id %u is out of range", id);
    if (id >= v.size()) v.resize(id + 1);
    if (v[id].live) return fail(c, ZCU_E_BAD_ID, "id %u is already in use", id);
    v[id] = std::move(item);
    v[id].live = true;
    return ZCU_OK;
}
template <typename T>
T* get(std::vector<T>& v, uint32_t id) {
    if (id >= v.size() || !v[id].live) return nullptr;
    return &v[id];
}

// One upload of `len` bytes from host memory `src` to device memory `dst`, through the chunk ring.
zcu_result upload_streamed(zcu_context* c, uint8_t* dst, const uint8_t* src, size_t len) {
    for (size_t done = 0; done < len;) {
        const int i = c->up_next;
        if (!c->up_chunk[i]) {
            CU(c, cudaMallocHost((void**)&c->up_chunk[i], zcu_context::UP_CHUNK_BYTES));
            CU(c, cudaEventCreateWithFlags(&c->up_done[i], cudaEventDisableTiming));
        } else {
            CU(c, cudaEventSynchronize(c->up_done[i]));   // the chunk's last copy (a bounded, short transfer)
        }
        const size_t n = len - done < zcu_context::UP_CHUNK_BYTES ? len - done : zcu_context::UP_CHUNK_BYTES;
        memcpy(c->up_chunk[i], src + done, n);
        CU(c, cudaMemcpyAsync(dst + done, c->up_chunk[i], n, cudaMemcpyHostToDevice, c->stream));
        CU(c, cudaEventRecord(c->up_done[i], c->stream));
        c->up_next = (i + 1) % zcu_context::UP_CHUNKS;
        done += n;
    }
    return ZCU_OK;
}

zcu_result ensure_pinned(zcu_context* c, size_t bytes) {
    if (c->dry || bytes <= c->pinned_cap) return ZCU_OK;
    if (c->pinned) cudaFreeHost(c->pinned);
    c->pinned = nullptr;
    c->pinned_cap = 0;
    size_t cap = 1 << 20;
    while (cap < bytes) cap <<= 1;
    CU(c, cudaMallocHost((void**)&c->pinned, cap));
    c->pinned_cap = cap;
    return ZCU_OK;
}

// Waits for everything on the stream, polling so that a deadline can end the wait.
zcu_result wait_stream(zcu_context* c, uint32_t timeout_ms) {
    if (c->dry) return ZCU_OK;
    cudaEvent_t ev;
    CU(c, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, c->stream);
    if (e != cudaSuccess) {
        cudaEventDestroy(ev);
        return fail(c, ZCU_E_GPU, "cudaEventRecord: %s", cudaGetErrorString(e));
    }
    const auto start = std::chrono::steady_clock::now();
    int spins = 0;
    for (;;) {
        e = cudaEventQuery(ev);
        if (e == cudaSuccess) break;
        if (e != cudaErrorNotReady) {
            cudaEventDestroy(ev);
            c->lost = true;
            return fail(c, ZCU_E_GPU, "device error while waiting: %s", cudaGetErrorString(e));
        }
        if (++spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - start).count();
        if (timeout_ms != 0 && ms > (long long)timeout_ms) {
            cudaEventDestroy(ev);
            c->unfinished = true;
            return fail(c, ZCU_E_TIMEOUT, "the device did not finish within %u ms", timeout_ms);
        }
    }
    cudaEventDestroy(ev);
    c->unfinished = false;
    if (c->status && *(volatile int*)c->status != 0) {
        const int what = *(volatile int*)c->status;
        *c->status = 0;
        if (what == 3)
            return fail(c, ZCU_E_GPU, "delta_rule (chunked): the token count in the parameter block is not the step's, or a kept row "
                                      "lies inside the chunked part; the step was not applied past its whole chunks");
        if (what == 5)
            return fail(c, ZCU_E_GPU, "a slice of a tensor-parallel exchange did not arrive within the wait limit; every later wait of this context "
                                      "gives up at once (configure the peers again to clear it)");
        if (what == 6)
            return fail(c, ZCU_E_GPU, "attention: the step's position lies past the key blocks the dispatch covers (or past max_blocks); "
                                      "the keys beyond were left out");
        return fail(c, ZCU_E_GPU, "a kernel gave up a bounded wait (a copy or a peer never arrived); its results are invalid");
    }
    return ZCU_OK;
}

zcu_result dispatch_kernel(zcu_context* c, uint32_t kernel, uint32_t variant, const void* params, uint32_t params_bytes,
                           const zcu_binding* b, uint32_t nb, const uint32_t grid[3]) {
    LaunchArgs a;
    a.stream = c->stream;
    a.params = params;
    a.params_bytes = params_bytes;
    a.b = b;
    a.nb = nb;
    a.grid[0] = grid[0];
    a.grid[1] = grid[1];
    a.grid[2] = grid[2];
    a.variant = variant;
    a.sm_count = c->dry ? 148 : c->prop.multiProcessorCount;
    a.status = c->status;
    a.peers = c->peers.world > 0 ? &c->peers : nullptr;
    a.scratch = c->scratch;
    a.scratch_bytes = c->scratch_bytes;
    a.err = c->err;
    a.err_cap = sizeof(c->err);
    char name[64];
    if (zcu_artifact(kernel, variant, name, sizeof(name)) == 0)
        return fail(c, ZCU_E_UNSUPPORTED_KERNEL, "kernel %u variant 0x%x is not implemented by the cuda backend", kernel, variant);
    c->launches++;
    if (c->dry) return ZCU_OK;
    switch (kernel) {
        case ZCU_K_RMSNORM: return launch_rmsnorm(a);
        case ZCU_K_MATMUL_BF16: return variant == ZCU_VARIANT_PREFILL_BF16_TC ? launch_matmul_tc(a, true) : launch_matmul_bf16(a);
        case ZCU_K_MATMUL_F16: return variant == ZCU_VARIANT_PREFILL_BF16_TC ? launch_matmul_tc(a, false) : launch_matmul_f16(a);
        case ZCU_K_MATVEC_BF16: return launch_matvec_bf16(a);
        case ZCU_K_MATVEC_F16: return launch_matvec_f16(a);
        case ZCU_K_SILU_MUL: return launch_silu_mul(a);
        case ZCU_K_EMBED_BF16:
        case ZCU_K_EMBED_F16:
        case ZCU_K_EMBED_Q8_0:
        case ZCU_K_EMBED_Q4_K: return launch_embed(a, kernel);
        case ZCU_K_ROPE_APPEND: return launch_rope_append(a);
        case ZCU_K_ATTN_SPLIT:
        case ZCU_K_ATTN_SPLIT_WIDE: return launch_attn_split(a);
        case ZCU_K_ATTN_COMBINE: return launch_attn_combine(a);
        case ZCU_K_DELTA_PREP: return launch_delta_prep(a);
        case ZCU_K_DELTA_RULE: return launch_delta_rule(a);
        case ZCU_K_MARK_TOKENS: return launch_mark_tokens(a);
        case ZCU_K_SAMPLE: return launch_sample(a);
        case ZCU_K_DRAFT: return launch_draft(a);
        case ZCU_K_EXT_PEER_WAIT: return launch_peer_wait(a);
        case ZCU_K_EXT_PEER_NEXT: return launch_peer_next(a);
        case ZCU_K_QUANTIZE_Q8: return launch_quantize_q8(a);
        case ZCU_K_MATMUL_Q4_K: return variant == ZCU_VARIANT_PREFILL_BF16_TC ? launch_matmul_q4_k_tc(a) : launch_matmul_q4_k(a);
        case ZCU_K_MATMUL_Q8_0: return launch_matmul_q8_0(a);
        case ZCU_K_MATMUL_REDUCE: return launch_matmul_reduce(a);
        case ZCU_K_MATMUL_Q8_0_FLOAT: return launch_matmul_q8_0_float(a);
        case ZCU_K_GATED_NORM: return launch_gated_norm(a);
        case ZCU_K_REPACK_Q8_0: return launch_repack_q8_0(a);
        case ZCU_K_MATVEC_Q8_0: return launch_matvec_q8_0(a);
        case ZCU_K_MATVEC_Q4_K: return launch_matvec_q4_k(a);
        case ZCU_K_MATVEC_Q3_K: return launch_matvec_q3_k(a);
        case ZCU_K_MATVEC_Q5_K: return launch_matvec_q5_k(a);
        case ZCU_K_MATVEC_Q6_K: return launch_matvec_q6_k(a);
        case ZCU_K_REPAD: return launch_repad(a);
        case ZCU_K_REPACK_Q3_K: return launch_repack_q3_k(a);
        case ZCU_K_EMBED_Q3_K:
        case ZCU_K_EMBED_Q5_K:
        case ZCU_K_EMBED_Q6_K:
        case ZCU_K_EMBED_IQ4_XS: return launch_embed_kquant(a, kernel);
        default: return fail(c, ZCU_E_UNSUPPORTED_KERNEL, "kernel %u is not implemented by the cuda backend", kernel);
    }
}

void drop_submission(zcu_context* c) {
    c->writes.clear();
    c->write_data.clear();
    c->ops.clear();
    c->reads.clear();
}

zcu_result release_buffer(zcu_context* c, uint32_t id) {
    Buffer* b = get(c->buffers, id);
    if (!b) return fail(c, ZCU_E_BAD_ID, "destroy: no buffer %u", id);
    if (b->ptr) {
        if (c->dry) free(b->ptr);
        else CU(c, cudaFree(b->ptr));
    }
    *b = Buffer();
    return ZCU_OK;
}

// The parameter block of a dispatch: binding 0 of its bind group, read from
// the uniform buffer's host shadow (refreshed from the device if a copy or a
// kernel may have changed it).
zcu_result resolve_params(zcu_context* c, const GroupEntry& e, std::vector<uint8_t>& out) {
    Buffer* b = get(c->buffers, e.buffer);
    if (!b) return fail(c, ZCU_E_BAD_ID, "dispatch: no buffer %u", e.buffer);
    if (e.offset + e.size > b->size || e.size > 4096) return fail(c, ZCU_E_BAD_COMMAND, "dispatch: parameter range outside buffer %u", e.buffer);
    out.resize(e.size);
    if (c->dry) {
        memcpy(out.data(), b->ptr + e.offset, e.size);
        return ZCU_OK;
    }
    if (b->shadow.empty() || b->shadow_stale) {
        b->shadow.resize(b->size);
        CU(c, cudaMemcpyAsync(b->shadow.data(), b->ptr, b->size, cudaMemcpyDeviceToHost, c->stream));
        CU(c, cudaStreamSynchronize(c->stream));
        b->shadow_stale = false;
    }
    memcpy(out.data(), b->shadow.data() + e.offset, e.size);
    return ZCU_OK;
}

zcu_result run_submit(zcu_context* c, uint32_t timeout_ms) {
    // 1. staged writes, in order, before any work of this submission
    size_t read_bytes = 0;
    for (const Op& op : c->ops)
        if (op.kind == OP_READ) read_bytes += (op.size + 255) & ~(uint64_t)255;
    if (!c->dry) {
        if (c->unfinished) {
            // an earlier wait gave up: its work may still read the pinned memory that is about to be reused
            zcu_result w = wait_stream(c, timeout_ms);
            if (w != ZCU_OK) return w;
        }
        zcu_result r = ensure_pinned(c, read_bytes + 256);
        if (r != ZCU_OK) return r;
    }
    for (const Write& w : c->writes) {
        Buffer* b = get(c->buffers, w.buffer);
        if (!b) return fail(c, ZCU_E_BAD_ID, "write: buffer %u was destroyed", w.buffer);
        const uint8_t* src = w.file_src ? w.file_src : c->write_data.data() + w.start;
        if (c->dry) {
            memcpy(b->ptr + w.offset, src, w.len);
        } else {
            zcu_result r = upload_streamed(c, b->ptr + w.offset, src, w.len);
            if (r != ZCU_OK) return r;
            if (b->usage & USAGE_UNIFORM) {
                if (b->shadow.size() != b->size) {
                    b->shadow.assign(b->size, 0);
                    b->shadow_stale = b->shadow_stale || false;
                }
                memcpy(b->shadow.data() + w.offset, src, w.len);
            }
        }
    }
    // 2. ops in recorded order
    size_t read_at = 0;
    struct PendingRead { void* dst; size_t at, size; };
    std::vector<PendingRead> pending;
    std::vector<uint8_t> params;
    std::vector<zcu_binding> binds;
    struct Timed { TimingKey key; cudaEvent_t a, b; };
    std::vector<Timed> timed;
    for (const Op& op : c->ops) {
        switch (op.kind) {
            case OP_DISPATCH: {
                Pipeline* p = get(c->pipelines, op.pipeline);
                if (!p) return fail(c, ZCU_E_BAD_ID, "dispatch: no pipeline %u", op.pipeline);
                Group* g = op.has_group ? get(c->groups, op.group) : nullptr;
                if (op.has_group && !g) return fail(c, ZCU_E_BAD_ID, "dispatch: no bind group %u", op.group);
                params.clear();
                binds.clear();
                if (g) {
                    uint32_t maxb = 0;
                    for (const GroupEntry& e : g->entries) maxb = e.binding > maxb ? e.binding : maxb;
                    binds.assign(maxb, zcu_binding{nullptr, 0});
                    for (const GroupEntry& e : g->entries) {
                        if (e.binding == 0) {
                            zcu_result r = resolve_params(c, e, params);
                            if (r != ZCU_OK) return r;
                            continue;
                        }
                        Buffer* b = get(c->buffers, e.buffer);
                        if (!b) return fail(c, ZCU_E_BAD_ID, "dispatch: no buffer %u", e.buffer);
                        if (e.offset + e.size > b->size) return fail(c, ZCU_E_BAD_COMMAND, "dispatch: binding %u outside buffer %u", e.binding, e.buffer);
                        binds[e.binding - 1] = zcu_binding{b->ptr + e.offset, e.size};
                        if ((p->writes >> e.binding) & 1u) {
                            if (b->usage & USAGE_UNIFORM) b->shadow_stale = true;
                        }
                    }
                }
                Timed tm{};
                if (c->profiling && !c->dry) {
                    tm.key = TimingKey{p->kernel, p->variant, {op.grid[0], op.grid[1], op.grid[2]}};
                    cudaEventCreate(&tm.a);
                    cudaEventCreate(&tm.b);
                    cudaEventRecord(tm.a, c->stream);
                }
                zcu_result r = dispatch_kernel(c, p->kernel, p->variant, params.data(), (uint32_t)params.size(), binds.data(),
                                               (uint32_t)binds.size(), op.grid);
                if (c->profiling && !c->dry) {
                    cudaEventRecord(tm.b, c->stream);
                    timed.push_back(tm);
                } else if (c->profiling) {
                    TimingVal& v = c->timings[TimingKey{p->kernel, p->variant, {op.grid[0], op.grid[1], op.grid[2]}}];
                    v.count++;
                }
                if (r != ZCU_OK) return r;
                break;
            }
            case OP_COPY: {
                Buffer *s = get(c->buffers, op.src), *d = get(c->buffers, op.dst);
                if (!s || !d) return fail(c, ZCU_E_BAD_ID, "copy: buffer was destroyed");
                if (c->dry) memmove(d->ptr + op.dst_off, s->ptr + op.src_off, op.size);
                else CU(c, cudaMemcpyAsync(d->ptr + op.dst_off, s->ptr + op.src_off, op.size, cudaMemcpyDeviceToDevice, c->stream));
                if (d->usage & USAGE_UNIFORM) d->shadow_stale = true;
                break;
            }
            case OP_FILL: {
                Buffer* d = get(c->buffers, op.dst);
                if (!d) return fail(c, ZCU_E_BAD_ID, "clear: buffer was destroyed");
                if (c->dry) memset(d->ptr + op.dst_off, 0, op.size);
                else CU(c, cudaMemsetAsync(d->ptr + op.dst_off, 0, op.size, c->stream));
                if (d->usage & USAGE_UNIFORM) d->shadow_stale = true;
                break;
            }
            case OP_READ: {
                Buffer* s = get(c->buffers, op.src);
                if (!s) return fail(c, ZCU_E_BAD_ID, "read: buffer was destroyed");
                if (op.size == 0) break;
                if (c->dry) {
                    memcpy(op.host_dst, s->ptr + op.src_off, op.size);
                } else {
                    CU(c, cudaMemcpyAsync(c->pinned + read_at, s->ptr + op.src_off, op.size, cudaMemcpyDeviceToHost, c->stream));
                    pending.push_back({op.host_dst, read_at, (size_t)op.size});
                    read_at += (op.size + 255) & ~(uint64_t)255;
                }
                break;
            }
        }
    }
    // 3. block until the device is done, then hand the reads over
    zcu_result r = wait_stream(c, timeout_ms);
    if (r != ZCU_OK) return r;
    for (const PendingRead& pr : pending) memcpy(pr.dst, c->pinned + pr.at, pr.size);
    for (Timed& tm : timed) {
        float ms = 0;
        if (cudaEventElapsedTime(&ms, tm.a, tm.b) == cudaSuccess) {
            TimingVal& v = c->timings[tm.key];
            v.count++;
            v.total_us += (double)ms * 1000.0;
        }
        cudaEventDestroy(tm.a);
        cudaEventDestroy(tm.b);
    }
    c->writes.clear();
    c->write_data.clear();
    c->ops.clear();
    // 4. buffers destroyed while work was pending
    for (uint32_t id : c->released) {
        r = release_buffer(c, id);
        if (r != ZCU_OK) return r;
    }
    c->released.clear();
    return ZCU_OK;
}

#define NEED_ARGS(n_)                                                                                  \
    do {                                                                                               \
        if (na < (n_)) return fail(c, ZCU_E_BAD_COMMAND, "opcode %u with %zu argument words, need %d", op, na, (int)(n_)); \
    } while (0)

zcu_result run_command(zcu_context* c, uint32_t op, const uint32_t* a, size_t na, zcu_completion* out, size_t cap,
                       size_t* n_out, uint32_t timeout_ms) {
    switch (op) {
        case 1: {  // create_buffer: id, size u64, usage
            NEED_ARGS(4);
            Buffer b;
            b.size = join64(a[1], a[2]);
            b.usage = a[3];
            const uint64_t alloc = b.size < 4 ? 4 : b.size;
            if (c->dry) {
                b.ptr = (uint8_t*)calloc(1, alloc);
                if (!b.ptr) return fail(c, ZCU_E_OUT_OF_MEMORY, "create_buffer: %llu bytes", (unsigned long long)alloc);
            } else {
                cudaError_t e = cudaMalloc((void**)&b.ptr, alloc);
                if (e != cudaSuccess) {
                    cudaGetLastError();
                    return fail(c, e == cudaErrorMemoryAllocation ? ZCU_E_OUT_OF_MEMORY : ZCU_E_GPU, "create_buffer: %llu bytes: %s",
                                (unsigned long long)alloc, cudaGetErrorString(e));
                }
                CU(c, cudaMemsetAsync(b.ptr, 0, alloc, c->stream));  // WebGPU buffers start zeroed
            }
            zcu_result r = put(c, c->buffers, a[0], std::move(b));
            if (r != ZCU_OK) return r;
            return ZCU_OK;
        }
        case 2: {  // write_buffer: buffer, offset u64, data ptr, len u64
            NEED_ARGS(7);
            Buffer* b = get(c->buffers, a[0]);
            if (!b) return fail(c, ZCU_E_BAD_ID, "write_buffer: no buffer %u", a[0]);
            const uint64_t off = join64(a[1], a[2]), len = join64(a[5], a[6]);
            if (len % 4 != 0 || off % 4 != 0 || off + len > b->size) return fail(c, ZCU_E_BAD_COMMAND, "write_buffer: range %llu+%llu in %llu", (unsigned long long)off, (unsigned long long)len, (unsigned long long)b->size);
            if (len == 0) return ZCU_OK;
            const uint8_t* data = (const uint8_t*)(uintptr_t)join64(a[3], a[4]);
            const size_t start = (c->write_data.size() + 15) & ~(size_t)15;
            c->write_data.resize(start + len);
            memcpy(c->write_data.data() + start, data, len);
            c->writes.push_back(Write{a[0], off, start, (size_t)len, nullptr});
            return ZCU_OK;
        }
        case 12: {  // write_file: buffer, offset u64, file_offset u64, size u64
            NEED_ARGS(7);
            Buffer* b = get(c->buffers, a[0]);
            if (!b) return fail(c, ZCU_E_BAD_ID, "write_file: no buffer %u", a[0]);
            const uint64_t off = join64(a[1], a[2]), foff = join64(a[3], a[4]), len = join64(a[5], a[6]);
            if (!c->file) return fail(c, ZCU_E_BAD_COMMAND, "write_file: no file set");
            if (foff + len > c->file_len || off + len > b->size || (off | len) % 4 != 0) return fail(c, ZCU_E_BAD_COMMAND, "write_file: range outside the file or the buffer");
            if (len == 0) return ZCU_OK;
            // only the range is recorded: the bytes go from the mapping to the device at the submit, a chunk at a time
            // (the mapping belongs to the caller and stays valid while it is the context's file: zcu_set_file)
            c->writes.push_back(Write{a[0], off, 0, (size_t)len, c->file + foff});
            return ZCU_OK;
        }
        case 3: {  // create_kernel: id, kernel, variant, writes, artifact ptr, len
            NEED_ARGS(7);
            Pipeline p;
            p.kernel = a[1];
            p.variant = a[2];
            p.writes = a[3];
            p.missing = a[6] == 0;
            if (!p.missing) {
                if (p.kernel >= ZCU_K_COUNT) return fail(c, ZCU_E_BAD_COMMAND, "create_kernel: unknown kernel %u", p.kernel);
                char name[64];
                if (zcu_artifact(p.kernel, p.variant, name, sizeof(name)) == 0)
                    return fail(c, ZCU_E_UNSUPPORTED_KERNEL, "create_kernel: kernel %u variant 0x%x is not implemented by the cuda backend", p.kernel, p.variant);
            }
            return put(c, c->pipelines, a[0], std::move(p));
        }
        case 5: {  // create_bind_group: id, pipeline, group, count, entries
            NEED_ARGS(4);
            const uint32_t count = a[3];
            if (na != 4 + (size_t)count * 6 || a[2] != 0) return fail(c, ZCU_E_BAD_COMMAND, "create_bind_group: malformed");
            Group g;
            g.pipeline = a[1];
            for (uint32_t i = 0; i < count; i++) {
                const uint32_t* e = a + 4 + i * 6;
                if (e[0] > 15) return fail(c, ZCU_E_BAD_COMMAND, "create_bind_group: binding %u", e[0]);
                Buffer* b = get(c->buffers, e[1]);
                if (!b) return fail(c, ZCU_E_BAD_ID, "create_bind_group: no buffer %u", e[1]);
                g.entries.push_back(GroupEntry{e[0], e[1], join64(e[2], e[3]), join64(e[4], e[5])});
            }
            return put(c, c->groups, a[0], std::move(g));
        }
        case 6: {  // dispatch: pipeline, x, y, z, count, groups
            NEED_ARGS(5);
            if (na != 5 + (size_t)a[4] || a[4] > 1) return fail(c, ZCU_E_BAD_COMMAND, "dispatch: malformed");
            Pipeline* p = get(c->pipelines, a[0]);
            if (!p) return fail(c, ZCU_E_BAD_ID, "dispatch: no pipeline %u", a[0]);
            if (a[4] == 1 && !get(c->groups, a[5])) return fail(c, ZCU_E_BAD_ID, "dispatch: no bind group %u", a[5]);
            if (p->missing) return fail(c, ZCU_E_UNSUPPORTED_KERNEL, "kernel %u is not implemented by this backend", p->kernel);
            Op o;
            o.kind = OP_DISPATCH;
            o.pipeline = a[0];
            o.grid[0] = a[1];
            o.grid[1] = a[2];
            o.grid[2] = a[3];
            o.has_group = a[4];
            o.group = a[4] ? a[5] : 0;
            c->ops.push_back(o);
            return ZCU_OK;
        }
        case 7: {  // copy_buffer: src, src_offset u64, dst, dst_offset u64, size u64
            NEED_ARGS(8);
            Buffer *s = get(c->buffers, a[0]), *d = get(c->buffers, a[3]);
            if (!s || !d) return fail(c, ZCU_E_BAD_ID, "copy_buffer: no such buffer");
            Op o;
            o.kind = OP_COPY;
            o.src = a[0];
            o.src_off = join64(a[1], a[2]);
            o.dst = a[3];
            o.dst_off = join64(a[4], a[5]);
            o.size = join64(a[6], a[7]);
            if ((o.src_off | o.dst_off | o.size) % 4 != 0 || o.src_off + o.size > s->size || o.dst_off + o.size > d->size)
                return fail(c, ZCU_E_BAD_COMMAND, "copy_buffer: range outside a buffer");
            if (o.size > 0) c->ops.push_back(o);
            return ZCU_OK;
        }
        case 11: {  // clear_buffer: buffer, offset u64, size u64
            NEED_ARGS(5);
            Buffer* d = get(c->buffers, a[0]);
            if (!d) return fail(c, ZCU_E_BAD_ID, "clear_buffer: no buffer %u", a[0]);
            Op o;
            o.kind = OP_FILL;
            o.dst = a[0];
            o.dst_off = join64(a[1], a[2]);
            o.size = join64(a[3], a[4]);
            if ((o.dst_off | o.size) % 4 != 0 || o.dst_off + o.size > d->size) return fail(c, ZCU_E_BAD_COMMAND, "clear_buffer: range outside the buffer");
            if (o.size > 0) c->ops.push_back(o);
            return ZCU_OK;
        }
        case 8: {  // read_buffer: token, buffer, offset u64, size u64, dst ptr
            NEED_ARGS(8);
            Buffer* s = get(c->buffers, a[1]);
            if (!s) return fail(c, ZCU_E_BAD_ID, "read_buffer: no buffer %u", a[1]);
            Op o;
            o.kind = OP_READ;
            o.src = a[1];
            o.src_off = join64(a[2], a[3]);
            o.size = join64(a[4], a[5]);
            o.host_dst = (void*)(uintptr_t)join64(a[6], a[7]);
            if ((o.src_off | o.size) % 4 != 0 || o.src_off + o.size > s->size) return fail(c, ZCU_E_BAD_COMMAND, "read_buffer: range outside the buffer");
            c->reads.push_back(Read{a[0]});
            c->ops.push_back(o);
            return ZCU_OK;
        }
        case 9: {  // submit: token
            NEED_ARGS(1);
            zcu_result r = run_submit(c, timeout_ms);
            if (r != ZCU_OK) return r;
            for (const Read& rd : c->reads) {
                if (*n_out < cap) out[*n_out] = zcu_completion{rd.token, 0};
                (*n_out)++;
            }
            c->reads.clear();
            if (*n_out < cap) out[*n_out] = zcu_completion{a[0], 0};
            (*n_out)++;
            return ZCU_OK;
        }
        case 10: {  // destroy: kind, id
            NEED_ARGS(2);
            switch (a[0]) {
                case 0: {
                    if (!get(c->buffers, a[1])) return fail(c, ZCU_E_BAD_ID, "destroy: no buffer %u", a[1]);
                    if (!c->ops.empty() || !c->writes.empty()) {
                        c->released.push_back(a[1]);
                        return ZCU_OK;
                    }
                    return release_buffer(c, a[1]);
                }
                case 1: {
                    Pipeline* p = get(c->pipelines, a[1]);
                    if (!p) return fail(c, ZCU_E_BAD_ID, "destroy: no pipeline %u", a[1]);
                    *p = Pipeline();
                    return ZCU_OK;
                }
                case 2: {
                    Group* g = get(c->groups, a[1]);
                    if (!g) return fail(c, ZCU_E_BAD_ID, "destroy: no bind group %u", a[1]);
                    *g = Group();
                    return ZCU_OK;
                }
                default: return fail(c, ZCU_E_BAD_COMMAND, "destroy: kind %u", a[0]);
            }
        }
        default: return fail(c, ZCU_E_BAD_COMMAND, "unknown opcode %u", op);
    }
}

const char* kernel_name(uint32_t k) {
    switch (k) {
        case ZCU_K_RMSNORM: return "rmsnorm";
        case ZCU_K_MATMUL_BF16: return "matmul_bf16";
        case ZCU_K_MATMUL_F16: return "matmul_f16";
        case ZCU_K_MATMUL_REDUCE: return "matmul_reduce";
        case ZCU_K_QUANTIZE_Q8: return "quantize_q8";
        case ZCU_K_MATMUL_Q8_0: return "matmul_q8_0";
        case ZCU_K_MATMUL_Q4_K: return "matmul_q4_k";
        case ZCU_K_MATMUL_Q8_0_FLOAT: return "matmul_q8_0_float";
        case ZCU_K_MATVEC_BF16: return "matvec_bf16";
        case ZCU_K_MATVEC_F16: return "matvec_f16";
        case ZCU_K_SILU_MUL: return "silu_mul";
        case ZCU_K_EMBED_BF16: return "embed_bf16";
        case ZCU_K_EMBED_F16: return "embed_f16";
        case ZCU_K_ROPE_APPEND: return "rope_append";
        case ZCU_K_ATTN_SPLIT: return "attn_split";
        case ZCU_K_ATTN_SPLIT_WIDE: return "attn_split_wide";
        case ZCU_K_ATTN_COMBINE: return "attn_combine";
        case ZCU_K_DELTA_PREP: return "delta_prep";
        case ZCU_K_DELTA_RULE: return "delta_rule";
        case ZCU_K_MARK_TOKENS: return "mark_tokens";
        case ZCU_K_SAMPLE: return "sample";
        case ZCU_K_DRAFT: return "draft";
        case ZCU_K_EXT_PEER_WAIT: return "ext_peer_wait";
        case ZCU_K_EXT_PEER_NEXT: return "ext_peer_next";
        case ZCU_K_GATED_NORM: return "gated_norm";
        case ZCU_K_REPACK_Q8_0: return "repack_q8_0";
        case ZCU_K_MATVEC_Q8_0: return "matvec_q8_0";
        case ZCU_K_MATVEC_Q4_K: return "matvec_q4_k";
        case ZCU_K_EMBED_Q8_0: return "embed_q8_0";
        case ZCU_K_EMBED_Q4_K: return "embed_q4_k";
        case ZCU_K_REPAD: return "repad";
        case ZCU_K_REPACK_Q3_K: return "repack_q3_k";
        case ZCU_K_MATVEC_Q3_K: return "matvec_q3_k";
        case ZCU_K_MATVEC_Q5_K: return "matvec_q5_k";
        case ZCU_K_MATVEC_Q6_K: return "matvec_q6_k";
        case ZCU_K_EMBED_Q3_K: return "embed_q3_k";
        case ZCU_K_EMBED_Q5_K: return "embed_q5_k";
        case ZCU_K_EMBED_Q6_K: return "embed_q6_k";
        case ZCU_K_EMBED_IQ4_XS: return "embed_iq4_xs";
        default: return nullptr;
    }
}

}  // namespace

zcu_result zcu_fail(const LaunchArgs& a, zcu_result r, const char* fmt, ...) {
    if (a.err && a.err_cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(a.err, a.err_cap, fmt, ap);
        va_end(ap);
    }
    return r;
}

zcu_result parse_peer(const LaunchArgs& a, PeerUse& u, const void* out_lo, const void* out_hi) {
    memset(&u, 0, sizeof(u));
    u.wait_slot = u.push_slot = PEER_NONE;
    if (a.params_bytes < sizeof(PPeer)) return ZCU_OK;
    PPeer pp;
    memcpy(&pp, static_cast<const char*>(a.params) + a.params_bytes - sizeof(PPeer), sizeof(pp));
    if (pp.magic != PEER_MAGIC) return ZCU_OK;
    ZCU_NEED(a, a.peers != nullptr, "this dispatch takes part in a peer exchange, but zcu_peer_config was not called");
    u.t = *a.peers;
    ZCU_NEED(a, (pp.wait_slot == PEER_NONE || pp.wait_slot < u.t.slots) && (pp.push_slot == PEER_NONE || pp.push_slot < u.t.slots),
             "peer exchange: slot out of range (%u, %u of %u)", pp.wait_slot, pp.push_slot, u.t.slots);
    u.wait_slot = pp.wait_slot;
    u.push_slot = pp.push_slot;
    if (u.push_slot != PEER_NONE) {
        const uint64_t lo = reinterpret_cast<uint64_t>(out_lo), hi = reinterpret_cast<uint64_t>(out_hi), base = u.t.base[u.t.rank];
        ZCU_NEED(a, lo >= base && hi <= base + u.t.ll_off && lo <= hi, "peer exchange: the output is not inside the local arena");
    }
    return ZCU_OK;
}

// ------------------------------------------------------------------ exports

ZCU_EXPORT const char* zcu_backend_source(void) {
    // Changes with every build of any kernel: the plan cache keys on it.
    return "zllm-cuda sm_100a abi1 " __DATE__ " " __TIME__;
}

ZCU_EXPORT size_t zcu_artifact(uint32_t kernel, uint32_t variant, char* out, size_t capacity) {
    const char* name = kernel_name(kernel);
    bool ok = name != nullptr;
    if (ok) {
        const bool is_matvec = kernel == ZCU_K_MATVEC_Q4_K || kernel == ZCU_K_MATVEC_Q8_0 || kernel == ZCU_K_MATVEC_BF16 || kernel == ZCU_K_MATVEC_F16 ||
                               kernel == ZCU_K_MATVEC_Q3_K || kernel == ZCU_K_MATVEC_Q5_K || kernel == ZCU_K_MATVEC_Q6_K;
        const bool has_rung = kernel == ZCU_K_MATMUL_BF16 || kernel == ZCU_K_MATMUL_F16 || kernel == ZCU_K_MATMUL_Q4_K;  // tensor-core prefill rung
        if (is_matvec) ok = matvec_variant_ok(kernel, variant);
        else ok = variant == 0 || (has_rung && variant == ZCU_VARIANT_PREFILL_BF16_TC) ||
                  (kernel == ZCU_K_DELTA_RULE && (variant == ZCU_VARIANT_DELTA_CHUNK64 || variant == ZCU_VARIANT_DELTA_CHUNK64_F32)) ||
                  (kernel == ZCU_K_ATTN_SPLIT && (variant == 1 || variant == 3));  // the forms of the fast path (k_attn.cu)
    }
    if (!ok) {
        if (out && capacity) out[0] = 0;
        return 0;
    }
    char buf[64];
    int n = variant ? snprintf(buf, sizeof(buf), "cuda:%s:%x", name, variant) : snprintf(buf, sizeof(buf), "cuda:%s", name);
    if (out && capacity) {
        snprintf(out, capacity, "%s", buf);
    }
    return (size_t)n;
}

ZCU_EXPORT zcu_result zcu_create(const zcu_options* options, zcu_context** out_context) {
    if (!options || !out_context || options->abi_version != ZCU_ABI_VERSION) return ZCU_E_INVALID;
    zcu_context* c = new zcu_context();
    c->dry = options->dry_run != 0;
    c->device = (int)options->device_index;
    if (!c->dry) {
        int count = 0;
        cudaError_t e = cudaGetDeviceCount(&count);
        if (e != cudaSuccess || (int)options->device_index >= count) {
            fprintf(stderr, "zllm_cuda: no CUDA device %u (%s); this backend has no CPU path\n", options->device_index,
                    e != cudaSuccess ? cudaGetErrorString(e) : "ordinal out of range");
            delete c;
            return ZCU_E_GPU;
        }
        if (cudaSetDevice(c->device) != cudaSuccess || cudaGetDeviceProperties(&c->prop, c->device) != cudaSuccess) {
            delete c;
            return ZCU_E_GPU;
        }
        if (c->prop.major != 10) {   // sm_100a code runs on sm_10x only (not on sm_9x, nor on sm_12x)
            fprintf(stderr, "zllm_cuda: device %d is sm_%d%d; the kernels are built for sm_100a only\n", c->device, c->prop.major, c->prop.minor);
            delete c;
            return ZCU_E_GPU;
        }
        if (options->stream) {
            c->stream = (cudaStream_t)options->stream;
        } else {
            if (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess) {
                delete c;
                return ZCU_E_GPU;
            }
            c->own_stream = true;
        }
        if (cudaHostAlloc((void**)&c->status, 64, cudaHostAllocMapped) != cudaSuccess) {
            cudaGetLastError();
            c->status = nullptr;
        } else {
            *c->status = 0;
        }
        // Stream-ordered scratch (the prefill rungs' rounded activations, the chunked delta rule's operands) stays in
        // the device's pool between steps: by default a pool gives its memory back at every synchronisation, and the
        // next step's allocation maps it again (2.5 ms for the 128 MB of a 4096-token DeltaNet step).
        {
            cudaMemPool_t pool;
            unsigned long long keep = ~0ull;
            if (cudaDeviceGetDefaultMemPool(&pool, c->device) != cudaSuccess ||
                cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) != cudaSuccess)
                cudaGetLastError();
        }
        // 64 MiB for the staged multiplies: allocated here so that no launch allocates (larger needs fall back to
        // stream-ordered allocation)
        if (cudaMalloc(&c->scratch, (size_t)64 << 20) == cudaSuccess) c->scratch_bytes = (size_t)64 << 20;
        else cudaGetLastError(), c->scratch = nullptr;
    }
    *out_context = c;
    return ZCU_OK;
}

ZCU_EXPORT zcu_result zcu_destroy(zcu_context* c, uint32_t timeout_ms) {
    if (!c) return ZCU_E_INVALID;
    if (!c->dry && !c->lost) {
        cudaSetDevice(c->device);
        zcu_result r = wait_stream(c, timeout_ms);
        if (r == ZCU_E_TIMEOUT) return r;  // the handle stays valid for a retry
    }
    for (void* m : c->ipc_open) cudaIpcCloseMemHandle(m);
    if (c->peers.epoch) cudaFree(c->peers.epoch);
    for (void* w : c->retired) cudaFree(w);
    for (cudaGraphExec_t g : c->graphs)
        if (g) cudaGraphExecDestroy(g);
    for (size_t i = 0; i < c->buffers.size(); i++)
        if (c->buffers[i].live && c->buffers[i].ptr) {
            if (c->dry) free(c->buffers[i].ptr);
            else cudaFree(c->buffers[i].ptr);
        }
    if (c->pinned) cudaFreeHost(c->pinned);
    for (int i = 0; i < zcu_context::UP_CHUNKS; i++) {
        if (c->up_chunk[i]) cudaFreeHost(c->up_chunk[i]);
        if (c->up_done[i]) cudaEventDestroy(c->up_done[i]);
    }
    if (c->status) cudaFreeHost(c->status);
    if (c->scratch) cudaFree(c->scratch);
    if (c->own_stream) cudaStreamDestroy(c->stream);
    delete c;
    return ZCU_OK;
}

ZCU_EXPORT zcu_result zcu_get_caps(zcu_context* c, zcu_caps* caps) {
    if (!c || !caps) return ZCU_E_INVALID;
    memset(caps, 0, sizeof(*caps));
    caps->abi_version = ZCU_ABI_VERSION;
    caps->dry_run = c->dry;
    caps->offset_align = 256;
    const uint64_t max_binding = c->dry ? (1ull << 40) : (uint64_t)c->prop.totalGlobalMem;
    caps->max_binding_lo = (uint32_t)max_binding;
    caps->max_binding_hi = (uint32_t)(max_binding >> 32);
    if (c->dry) {
        snprintf(caps->device_name, sizeof(caps->device_name), "dry run (no device)");
        return ZCU_OK;
    }
    caps->sm_major = c->prop.major;
    caps->sm_minor = c->prop.minor;
    caps->sm_count = c->prop.multiProcessorCount;
    caps->max_shared_per_block = (uint32_t)c->prop.sharedMemPerBlockOptin;
    caps->l2_bytes = (uint32_t)c->prop.l2CacheSize;
    size_t fr = 0, tot = 0;
    cudaSetDevice(c->device);
    if (cudaMemGetInfo(&fr, &tot) == cudaSuccess) {
        caps->free_bytes = fr;
        caps->total_bytes = tot;
    }
    snprintf(caps->device_name, sizeof(caps->device_name), "%s", c->prop.name);
    return ZCU_OK;
}

ZCU_EXPORT size_t zcu_last_error(zcu_context* c, char* out, size_t capacity) {
    if (!c) return 0;
    const size_t n = strlen(c->err);
    if (out && capacity) snprintf(out, capacity, "%s", c->err);
    return n;
}

ZCU_EXPORT zcu_result zcu_force_loss(zcu_context* c) {
    if (!c) return ZCU_E_INVALID;
    c->lost = true;
    snprintf(c->err, sizeof(c->err), "device loss forced by the host");
    return ZCU_OK;
}

ZCU_EXPORT zcu_result zcu_memory_budget(zcu_context* c, uint64_t* out_bytes) {
    if (!c || !out_bytes) return ZCU_E_INVALID;
    if (c->lost) return ZCU_E_DEVICE_LOST;
    if (c->dry) {
        *out_bytes = 180ull << 30;
        return ZCU_OK;
    }
    size_t fr = 0, tot = 0;
    cudaSetDevice(c->device);
    CU(c, cudaMemGetInfo(&fr, &tot));
    *out_bytes = fr;
    return ZCU_OK;
}

ZCU_EXPORT int32_t zcu_supports_prefill(zcu_context* c, uint32_t rung_variant) {
    if (!c || c->lost) return 0;
    // 0 = the scalar f32 identities; the single-product half rung runs on the tensor cores; the
    // compensated rung (0xffff0000) does not exist here
    return rung_variant == 0 || rung_variant == ZCU_VARIANT_PREFILL_BF16_TC;
}

ZCU_EXPORT zcu_result zcu_rope_table(float* out, uint32_t positions, uint32_t n_rot, float base, const float* factors) {
    if (!out || n_rot == 0 || (n_rot & 1)) return ZCU_E_INVALID;
    const uint32_t half = n_rot / 2;
    for (uint32_t pos = 0; pos < positions; pos++)
        for (uint32_t i = 0; i < half; i++) {
            const float exponent = -2.0f * (float)i / (float)n_rot;
            const float theta = (float)pos * powf(base, exponent) / (factors ? factors[i] : 1.0f);
            out[((size_t)pos * half + i) * 2] = cosf(theta);
            out[((size_t)pos * half + i) * 2 + 1] = sinf(theta);
        }
    return ZCU_OK;
}

ZCU_EXPORT zcu_result zcu_set_file(zcu_context* c, const void* mapped, uint64_t length, const char* path) {
    if (!c) return ZCU_E_INVALID;
    (void)path;
    c->file = (const uint8_t*)mapped;
    c->file_len = length;
    return ZCU_OK;
}

ZCU_EXPORT zcu_result zcu_execute(zcu_context* c, const uint32_t* words, size_t n_words, zcu_completion* out, size_t cap,
                                  size_t* n_out, uint32_t timeout_ms) {
    if (!c || (!words && n_words) || !n_out) return ZCU_E_INVALID;
    *n_out = 0;
    if (c->lost) return fail(c, ZCU_E_DEVICE_LOST, "the device is lost");
    if (!c->dry) cudaSetDevice(c->device);
    size_t pos = 0;
    while (pos < n_words) {
        const uint32_t word = words[pos];
        const size_t n = word >> 8;
        if (n == 0) return fail(c, ZCU_E_BAD_LENGTH, "command at word %zu has length 0", pos);
        if (n > n_words - pos) return fail(c, ZCU_E_TRUNCATED, "command at word %zu runs past the batch", pos);
        zcu_result r = run_command(c, word & 0xffu, words + pos + 1, n - 1, out, cap, n_out, timeout_ms ? timeout_ms : 60000u);
        if (r != ZCU_OK) {
            if (r == ZCU_E_UNSUPPORTED_KERNEL) drop_submission(c);
            return r;
        }
        pos += n;
    }
    return ZCU_OK;
}

ZCU_EXPORT zcu_result zcu_start_profile(zcu_context* c) {
    if (!c) return ZCU_E_INVALID;
    c->profiling = true;
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_stop_profile(zcu_context* c) {
    if (!c) return ZCU_E_INVALID;
    c->profiling = false;
    c->timings.clear();
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_read_timings(zcu_context* c, zcu_timing* out, size_t cap, size_t* n_out) {
    if (!c || !n_out) return ZCU_E_INVALID;
    if (!c->profiling) return fail(c, ZCU_E_NO_TIMESTAMPS, "profiling is off");
    size_t i = 0;
    for (const auto& kv : c->timings) {
        if (out && i < cap) {
            out[i].kernel = kv.first.kernel;
            out[i].variant = kv.first.variant;
            memcpy(out[i].grid, kv.first.grid, sizeof(out[i].grid));
            out[i].count = kv.second.count;
            out[i].total_us = kv.second.total_us;
        }
        i++;
    }
    *n_out = i;
    return ZCU_OK;
}

#define LIVE(c)                                                         \
    do {                                                                \
        if (!(c)) return ZCU_E_INVALID;                                 \
        if ((c)->lost) return fail(c, ZCU_E_DEVICE_LOST, "the device is lost"); \
        if (!(c)->dry) cudaSetDevice((c)->device);                      \
    } while (0)

ZCU_EXPORT zcu_result zcu_alloc(zcu_context* c, uint64_t bytes, void** out_ptr) {
    LIVE(c);
    if (!out_ptr) return ZCU_E_INVALID;
    const uint64_t alloc = bytes < 256 ? 256 : bytes;
    if (c->dry) {
        *out_ptr = calloc(1, alloc);
        return *out_ptr ? ZCU_OK : fail(c, ZCU_E_OUT_OF_MEMORY, "alloc: %llu bytes", (unsigned long long)alloc);
    }
    cudaError_t e = cudaMalloc(out_ptr, alloc);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(c, e == cudaErrorMemoryAllocation ? ZCU_E_OUT_OF_MEMORY : ZCU_E_GPU, "alloc: %llu bytes: %s", (unsigned long long)alloc, cudaGetErrorString(e));
    }
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_free(zcu_context* c, void* ptr) {
    if (!c) return ZCU_E_INVALID;
    if (!ptr) return ZCU_OK;
    if (c->dry) {
        free(ptr);
        return ZCU_OK;
    }
    cudaSetDevice(c->device);
    CU(c, cudaFree(ptr));
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_upload(zcu_context* c, void* dst, const void* src, uint64_t bytes) {
    LIVE(c);
    if (bytes == 0) return ZCU_OK;
    if (c->dry) {
        memcpy(dst, src, bytes);
        return ZCU_OK;
    }
    CU(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, c->stream));
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_download(zcu_context* c, void* dst, const void* src, uint64_t bytes) {
    LIVE(c);
    if (bytes == 0) return ZCU_OK;
    if (c->dry) {
        memcpy(dst, src, bytes);
        return ZCU_OK;
    }
    CU(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    return wait_stream(c, 60000);
}
ZCU_EXPORT zcu_result zcu_memset(zcu_context* c, void* dst, int value, uint64_t bytes) {
    LIVE(c);
    if (bytes == 0) return ZCU_OK;
    if (c->dry) {
        memset(dst, value, bytes);
        return ZCU_OK;
    }
    CU(c, cudaMemsetAsync(dst, value, bytes, c->stream));
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_launch(zcu_context* c, uint32_t kernel, uint32_t variant, const void* params, uint32_t params_bytes,
                                 const zcu_binding* bindings, uint32_t n_bindings, const uint32_t grid[3]) {
    LIVE(c);
    if (!params || !grid || (!bindings && n_bindings)) return fail(c, ZCU_E_INVALID, "launch: null argument");
    return dispatch_kernel(c, kernel, variant, params, params_bytes, bindings, n_bindings, grid);
}
// Decode attention with the partials in the library's fixed array: no allocation on this path, for
// callers that cannot allocate (see the header). Not available in a dry run (there is no device array).
ZCU_EXPORT zcu_result zcu_attention_decode_static(zcu_context* c, const void* params, uint32_t params_bytes,
                                                  const zcu_binding* bindings, uint32_t n_bindings, uint32_t max_keys,
                                                  uint32_t rows) {
    LIVE(c);
    if (!params || !bindings) return fail(c, ZCU_E_INVALID, "attention (static partials): null argument");
    if (c->dry) return fail(c, ZCU_E_INVALID, "attention (static partials): needs a device");
    LaunchArgs a;
    a.stream = c->stream;
    a.params = params;
    a.params_bytes = params_bytes;
    a.b = bindings;
    a.nb = n_bindings;
    a.grid[0] = a.grid[1] = a.grid[2] = 0;
    a.variant = 0;
    a.sm_count = c->prop.multiProcessorCount;
    a.status = c->status;
    a.peers = nullptr;
    a.scratch = nullptr;
    a.scratch_bytes = 0;
    a.err = c->err;
    a.err_cap = sizeof(c->err);
    const zcu_result r = launch_attn_static(a, max_keys, rows);
    if (r == ZCU_OK) c->launches += 2;
    return r;
}

ZCU_EXPORT zcu_result zcu_sync(zcu_context* c, uint32_t timeout_ms) {
    LIVE(c);
    return wait_stream(c, timeout_ms ? timeout_ms : 60000u);
}
ZCU_EXPORT uint64_t zcu_launch_count(zcu_context* c) { return c ? c->launches : 0; }

ZCU_EXPORT zcu_result zcu_capture_begin(zcu_context* c) {
    LIVE(c);
    if (c->dry) return fail(c, ZCU_E_INVALID, "capture needs a device");
    if (c->capturing) return fail(c, ZCU_E_INVALID, "a capture is already open");
    CU(c, cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    c->capturing = true;
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_capture_end(zcu_context* c, uint32_t* out_graph) {
    LIVE(c);
    if (!c->capturing || !out_graph) return fail(c, ZCU_E_INVALID, "no capture is open");
    c->capturing = false;
    cudaGraph_t g = nullptr;
    CU(c, cudaStreamEndCapture(c->stream, &g));
    cudaGraphExec_t ex = nullptr;
    cudaError_t e = cudaGraphInstantiate(&ex, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) return fail(c, ZCU_E_GPU, "cudaGraphInstantiate: %s", cudaGetErrorString(e));
    c->graphs.push_back(ex);
    *out_graph = (uint32_t)c->graphs.size() - 1;
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_graph_launch(zcu_context* c, uint32_t graph) {
    LIVE(c);
    if (graph >= c->graphs.size() || !c->graphs[graph]) return fail(c, ZCU_E_BAD_ID, "no graph %u", graph);
    CU(c, cudaGraphLaunch(c->graphs[graph], c->stream));
    return ZCU_OK;
}
static void fill_args(zcu_context* c, LaunchArgs& a) {
    memset(&a, 0, sizeof(a));
    a.stream = c->stream;
    a.sm_count = c->dry ? 148 : c->prop.multiProcessorCount;
    a.status = c->status;
    a.peers = c->peers.world > 0 ? &c->peers : nullptr;
    a.err = c->err;
    a.err_cap = sizeof(c->err);
}

// ---- tensor-parallel exchange over peer memory (peer.cuh)
ZCU_EXPORT zcu_result zcu_ipc_export(zcu_context* c, void* ptr, void* out_handle64) {
    LIVE(c);
    if (c->dry || !ptr || !out_handle64) return fail(c, ZCU_E_INVALID, "ipc_export: needs a device allocation");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
    CU(c, cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(out_handle64), ptr));
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_ipc_open(zcu_context* c, const void* handle64, void** out_ptr) {
    LIVE(c);
    if (c->dry || !handle64 || !out_ptr) return fail(c, ZCU_E_INVALID, "ipc_open: needs a device and a handle");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    CU(c, cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    c->ipc_open.push_back(*out_ptr);
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_peer_config(zcu_context* c, uint32_t rank, uint32_t world, const uint64_t* bases, uint64_t arena_bytes,
                                      uint64_t exchange_offset, uint32_t slots) {
    LIVE(c);
    if (c->dry) return fail(c, ZCU_E_INVALID, "peer_config: needs a device");
    if (!bases || world == 0 || world > PEER_MAX || rank >= world || slots == 0)
        return fail(c, ZCU_E_INVALID, "peer_config: rank %u of %u, %u slots", rank, world, slots);
    if (exchange_offset % 16 != 0 || exchange_offset * 3 > arena_bytes)
        return fail(c, ZCU_E_INVALID, "peer_config: the exchange region (twice the data region) does not fit the arena");
    PeerTable t = {};
    t.rank = (int32_t)rank;
    t.world = (int32_t)world;
    t.slots = slots;
    for (uint32_t r = 0; r < world; r++) t.base[r] = bases[r];
    t.arena_bytes = arena_bytes;
    t.ll_off = exchange_offset;
    uint32_t* words = nullptr;
    CU(c, cudaMalloc((void**)&words, 2 * sizeof(uint32_t)));
    CU(c, cudaMemset(words, 0, 2 * sizeof(uint32_t)));
    CU(c, cudaMemset(reinterpret_cast<void*>(t.base[rank] + exchange_offset), 0, (size_t)exchange_offset * 2));  // tag 0: nothing yet
    t.epoch = words;
    // (the old epoch words stay allocated until the context goes: graphs captured under the old configuration hold
    // their address)
    if (c->peers.epoch) c->retired.push_back(c->peers.epoch);
    t.wait_ms = c->peers.wait_ms;
    c->peers = t;
    return ZCU_OK;
}

ZCU_EXPORT zcu_result zcu_peer_wait_limit(zcu_context* c, uint32_t milliseconds) {
    LIVE(c);
    if (c->peers.world == 0) return fail(c, ZCU_E_INVALID, "peer_wait_limit: zcu_peer_config was not called");
    c->peers.wait_ms = milliseconds;   // launches from now on carry it
    return ZCU_OK;
}
ZCU_EXPORT zcu_result zcu_graph_destroy(zcu_context* c, uint32_t graph) {
    if (!c) return ZCU_E_INVALID;
    if (graph >= c->graphs.size() || !c->graphs[graph]) return fail(c, ZCU_E_BAD_ID, "no graph %u", graph);
    cudaGraphExecDestroy(c->graphs[graph]);
    c->graphs[graph] = nullptr;
    return ZCU_OK;
}
